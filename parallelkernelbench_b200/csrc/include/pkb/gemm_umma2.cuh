// CTA-pair variant of the persistent tcgen05 GEMM: two CTAs of a cluster share one 256 x 256
// output tile (tcgen05.mma.cta_group::2, M = 256). Each CTA loads its own 128 rows of A and its own
// 128 rows (output features) of B, so every operand byte crosses L2 -> shared memory once per pair
// instead of once per CTA, and the smaller per-CTA stage (32 KiB) leaves room for a six-deep ring.
//   warp 0 (both CTAs): TMA producer; completion bytes of both CTAs land on the leader's barrier
//   warp 1 (leader)   : MMA issuer; commits arrive on both CTAs' barriers
//   warps 2-5 (both)  : epilogue of the CTA's own 128 accumulator rows
// Hooks (a_ready flags, row-block scatter) and bounded waits are the same as in gemm_umma.cuh.
#pragma once
#include "pkb/gemm_umma.cuh"

namespace pkb {

constexpr int kGemm2TileM = 256;
constexpr int kGemm2TileN = 256;
constexpr int kGemm2Stages = 6;
constexpr int kGemm2ABytes = 128 * kGemmBlockK * 2;   // this CTA's half of A
constexpr int kGemm2BBytes = 128 * kGemmBlockK * 2;   // this CTA's half of B
constexpr int kGemm2StageBytes = kGemm2ABytes + kGemm2BBytes;
constexpr int kGemm2StoreBytes = 4 * 2 * 4096;      // per epilogue warp: two 32 x 128-byte buffers
constexpr int kGemm2SmemTotal = kGemm2Stages * kGemm2StageBytes + kGemm2StoreBytes + 256 + 1024;

// Tensor maps of the output for the TMA-store epilogue: one map for a local C, or one per
// destination rank for the reduce-scatter form (box = 64 bf16 columns x 32 rows, 128-byte swizzle).
struct alignas(64) GemmOutMaps {
  CUtensorMap m[kGemmMaxWorld];
};

// BCAST (with TMA_STORE): every output tile is stored into the result of EVERY rank (maps m[0 .. world)), at column
// p.bcast_col0 + its own column: the all-gather along N of a column-parallel GEMM happens in the epilogue.
// A_MN / B_MN: the operand is given MN-major ([K, M] resp. [K, N] row-major, the layouts of dX = dY W and dW = dY^T X): a CTA's
// 128 rows (columns) of it arrive as two 64 x 64 boxes (one 128-byte-swizzle atom each, 8 KiB apart) and are described to the
// tensor core as MN-major; 16 along K is then 16 shared-memory rows = 2048 bytes.
// GROUPED: A is a stack of row groups (p.grp_offsets, device memory) and group e multiplies with rows [e * N, (e + 1) * N) of B
// (one weight matrix per group, e.g. the experts of a MoE layer): tiles are (group, 256-row block of the group, n block), rows
// of a tile beyond the group's end are computed and not stored. Register epilogue only.
template <int EPI, bool OUT_F32, bool A_READY, bool RS_SCATTER, bool TMA_STORE = false, bool BCAST = false, bool A_MN = false,
          bool B_MN = false, bool GROUPED = false>
__device__ __forceinline__ void gemm_umma2_cta(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b,
                                               const GemmParams& p, const int pair,
                                               const int num_pairs,
                                               const GemmOutMaps* out_maps = nullptr,
                                               const CUtensorMap* tmap_a_local = nullptr) {
  static_assert(!(TMA_STORE && OUT_F32), "the TMA-store epilogue writes bf16");
  static_assert(!BCAST || (TMA_STORE && !RS_SCATTER), "the broadcast epilogue is a TMA-store epilogue");
  static_assert(!(A_MN && A_READY), "the gathered-A hook loads A K-major");
  static_assert(!GROUPED || (!TMA_STORE && !RS_SCATTER && !A_READY && !A_MN && !B_MN && !OUT_F32), "the grouped form is K-major, bf16, register epilogue");
  constexpr int kStages = kGemm2Stages;
  constexpr int BN = kGemm2TileN;
  constexpr uint32_t kTmemCols = 512;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t store_base = smem_base + kStages * kGemm2StageBytes;
  const uint32_t bar_base = store_base + kGemm2StoreBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(
      smem_gen + kStages * kGemm2StageBytes + kGemm2StoreBytes + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;

  const int num_m = (p.M + kGemm2TileM - 1) / kGemm2TileM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_k = (p.K + kGemmBlockK - 1) / kGemmBlockK;
  // grouped form: prefix sums of the groups' 256-row tile counts, built once per CTA from the device-side offsets
  __shared__ int s_tile_prefix[GROUPED ? kGemmMaxGroups + 1 : 1];
  if constexpr (GROUPED) {
    for (int e = threadIdx.x; e < p.grp_count; e += blockDim.x) {
      const int cnt = p.grp_offsets[e + 1] - p.grp_offsets[e];
      s_tile_prefix[e + 1] = (cnt + kGemm2TileM - 1) / kGemm2TileM;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      s_tile_prefix[0] = 0;
      for (int e = 0; e < p.grp_count; ++e) s_tile_prefix[e + 1] += s_tile_prefix[e];
    }
    __syncthreads();
  }
  const int num_tiles = GROUPED ? s_tile_prefix[p.grp_count] * num_n : num_m * num_n;
  // grouped: tile -> first row of the pair's 256-row block, the group's row limit, first row of B, n block (n fastest)
  auto tile_rows = [&](int tile, int& row0, int& row_end, int& b_row0, int& n_blk) {
    const int mi = tile / num_n;
    n_blk = tile - mi * num_n;
    int lo = 0, hi = p.grp_count;  // find e with prefix[e] <= mi < prefix[e+1]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_tile_prefix[mid] <= mi) lo = mid; else hi = mid;
    }
    row0 = p.grp_offsets[lo] + (mi - s_tile_prefix[lo]) * kGemm2TileM;
    row_end = p.grp_offsets[lo + 1];
    b_row0 = lo * p.N + n_blk * BN;
  };
  const int group_m = p.group_m > 0 ? p.group_m : 8;

  auto tile_coords = [&](int tile, int& m_blk, int& n_blk) {
    const int tiles_per_group = group_m * num_n;
    const int g = tile / tiles_per_group;
    const int first_m = g * group_m;
    const int gm = min(group_m, num_m - first_m);
    const int local = tile - g * tiles_per_group;
    n_blk = local / gm;
    m_blk = first_m + (local - n_blk * gm) + p.m_block_rotation;
    if (m_blk >= num_m) m_blk -= num_m;
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);   // leader's producer arrives (expect_tx of both CTAs' bytes)
      mbar_init(empty_bar(s), 1);  // one commit arrival, delivered to both CTAs
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);  // four epilogue warps of each CTA
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_holder), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    {
      // warp-uniform loop: one elected lane's copies take effect (see umma_f16_ss_p)
      const uint32_t lead = elect_one() ? 1u : 0u;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long waited = 0;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int m_blk = 0, n_blk = 0, g_row0 = 0, g_row_end = 0, g_b_row0 = 0;
        if constexpr (GROUPED) tile_rows(tile, g_row0, g_row_end, g_b_row0, n_blk);
        else tile_coords(tile, m_blk, n_blk);
        const int row0 = (GROUPED ? g_row0 : m_blk * kGemm2TileM) + (int)cta_rank * 128;
        const int col0 = (GROUPED ? g_b_row0 : n_blk * BN) + (int)cta_rank * 128;   // this CTA's 128 rows of B
        const CUtensorMap* map_a = &tmap_a;
        int a_row = row0;
        bool a_is_local = false;
        if constexpr (A_READY) {
          if (tmap_a_local != nullptr && row0 >= p.a_local_row0 &&
              row0 < p.a_local_row0 + p.a_local_rows) {
            map_a = tmap_a_local;
            a_row = row0 - p.a_local_row0;
            a_is_local = true;
          }
        }
        if (A_READY && !a_is_local) {
          int chunk = row0 / p.a_chunk_rows;
          const int last_chunk = (p.M - 1) / p.a_chunk_rows;
          if (chunk > last_chunk) chunk = last_chunk;
          const long long w0 = p.a_wait_cycles != nullptr ? clock64() : 0;
          const bool arrived = wait_flag_ge(p.a_ready + chunk, p.a_ready_epoch, p.wait_budget_ns);
          if (p.a_wait_cycles != nullptr) waited += clock64() - w0;
          if (!arrived) {
            *abort_flag = 1;
            if (lane == 0) record_status(p.status, kStatusPeerTimeout, p.kernel_id, p.rank, chunk, 10, tile);
            ok = false;
            break;
          }
          fence_proxy_async_all();
        }
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_budget_ns)) {
            if (lane == 0) record_status(p.status, kStatusMbarTimeout, p.kernel_id, p.rank, stage, 11, tile);
            ok = false;
            break;
          }
          mbar_expect_tx_p(full_bar(stage), 2 * kGemm2StageBytes, leader ? lead : 0u);
          const uint32_t sa = smem_base + stage * kGemm2StageBytes;
          if constexpr (A_MN) {
            tma_load_2d_pair_p(sa, map_a, full_bar(stage), a_row, kb * kGemmBlockK, lead);
            tma_load_2d_pair_p(sa + 8192, map_a, full_bar(stage), a_row + 64, kb * kGemmBlockK, lead);
          } else {
            tma_load_2d_pair_p(sa, map_a, full_bar(stage), kb * kGemmBlockK, a_row, lead);
          }
          if constexpr (B_MN) {
            tma_load_2d_pair_p(sa + kGemm2ABytes, &tmap_b, full_bar(stage), col0, kb * kGemmBlockK, lead);
            tma_load_2d_pair_p(sa + kGemm2ABytes + 8192, &tmap_b, full_bar(stage), col0 + 64, kb * kGemmBlockK, lead);
          } else {
            tma_load_2d_pair_p(sa + kGemm2ABytes, &tmap_b, full_bar(stage), kb * kGemmBlockK, col0, lead);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if constexpr (A_READY) {
        if (p.a_wait_cycles != nullptr && lane == 0) p.a_wait_cycles[blockIdx.x] += (unsigned long long)waited;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    // The whole warp walks the loop and waits on the barriers; one elected lane's tcgen05 instructions take effect. Under
    // `if (lane == 0)` the loop would run in divergent code, where addresses and descriptors cannot live in uniform
    // registers and every tcgen05 instruction drags register-to-uniform moves behind it (see umma_f16_ss_p).
    if (leader) {
      const uint32_t lead = elect_one() ? 1u : 0u;
      constexpr uint32_t idesc = make_idesc(kGemm2TileM, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      // low descriptor words of stage 0; a stage adds kGemm2StageBytes >> 4, a K step of 16 adds 2 (K-major) or 128 (MN-major)
      const uint32_t a_lo0 = A_MN ? smem_desc_lo_mnmajor(smem_base, 8192u) : smem_desc_lo_kmajor(smem_base);
      const uint32_t b_lo0 = B_MN ? smem_desc_lo_mnmajor(smem_base + kGemm2ABytes, 8192u) : smem_desc_lo_kmajor(smem_base + kGemm2ABytes);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.wait_budget_ns)) {
          if (lane == 0) record_status(p.status, kStatusMbarTimeout, p.kernel_id, p.rank, acc, 20, tile);
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.wait_budget_ns)) {
            if (lane == 0) record_status(p.status, kStatusMbarTimeout, p.kernel_id, p.rank, stage, 21, tile);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_lo = a_lo0 + stage * (kGemm2StageBytes >> 4), b_lo = b_lo0 + stage * (kGemm2StageBytes >> 4);
#pragma unroll
          for (int k = 0; k < kGemmBlockK / 16; ++k)
            umma_f16_ss_pair_p(tmem_d, smem_desc_join(a_lo + (A_MN ? 128u : 2u) * k), smem_desc_join(b_lo + (B_MN ? 128u : 2u) * k), idesc,
                               (kb | k) != 0 ? 1u : 0u, lead);
          umma_commit_pair_p(empty_bar(stage), 0x3, lead);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_pair_p(tfull_bar(acc), 0x3, lead);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue (warps 2..5, both CTAs) ------------------------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t leader_tempty0 = mapa_shared(tempty_bar(0), 0);
    const uint32_t leader_tempty1 = mapa_shared(tempty_bar(1), 0);
    for (int tile = pair; tile < num_tiles; tile += num_pairs) {
      int m_blk = 0, n_blk = 0, g_row0 = 0, g_row_end = 0, g_b_row0 = 0;
      if constexpr (GROUPED) tile_rows(tile, g_row0, g_row_end, g_b_row0, n_blk);
      else tile_coords(tile, m_blk, n_blk);
      bool ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.wait_budget_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0)
          record_status(p.status, kStatusMbarTimeout, p.kernel_id, p.rank, acc, 30, tile);
        break;
      }
      tc_fence_after_sync();
      const int row_blk0 = (GROUPED ? g_row0 : m_blk * kGemm2TileM) + (int)cta_rank * 128;
      const int row = row_blk0 + q * 32 + lane;
      const int n0 = n_blk * BN;
      uint8_t* out_row;
      constexpr int kOutBytes = OUT_F32 ? 4 : 2;
      if constexpr (RS_SCATTER) {
        const int owner = row / p.rs_rows_per_rank;
        const int r_in = row - owner * p.rs_rows_per_rank;
        out_row = static_cast<uint8_t*>(p.rs_out[owner < p.world ? owner : 0]) +
                  static_cast<long long>(r_in) * p.ldc * kOutBytes;
      } else {
        out_row = static_cast<uint8_t*>(p.C) + static_cast<long long>(row) * p.ldc * kOutBytes;
      }
      if constexpr (TMA_STORE) {
        // ---- staged epilogue: registers -> swizzled shared memory -> TMA store (128-byte rows,
        // issued by one lane, so the destination sees full-line bursts even over NVLink) ----
        const uint32_t stg = store_base + static_cast<uint32_t>(warp - 2) * 8192u;
        int map_idx = 0;
        int row_coord = row_blk0 + q * 32;
        if constexpr (RS_SCATTER) {
          const int owner = row_blk0 / p.rs_rows_per_rank;
          map_idx = owner < p.world ? owner : 0;
          row_coord -= owner * p.rs_rows_per_rank;
        }
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const uint32_t buf = stg + static_cast<uint32_t>(c & 1) * 4096u;
          if (lane == 0) tma_store_wait_read<1>();  // the store that last used this buffer was read
          __syncwarp();
          uint32_t r0[32], r1[32];
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                 static_cast<uint32_t>(acc * BN + c * 64);
          tmem_ld_32x32(taddr, r0);
          tmem_ld_32x32(taddr + 32, r1);
          tmem_ld_wait();
          const int col0 = n0 + c * 64;
          uint32_t w[32];
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float a0 = __uint_as_float(r0[j]) * p.alpha, a1 = __uint_as_float(r0[j + 1]) * p.alpha;
            float b0 = __uint_as_float(r1[j]) * p.alpha, b1 = __uint_as_float(r1[j + 1]) * p.alpha;
            if constexpr (EPI == kEpiBias || EPI == kEpiBiasSilu) {
              if (col0 + j + 1 < p.N) {
                a0 += __bfloat162float(p.bias[col0 + j]);
                a1 += __bfloat162float(p.bias[col0 + j + 1]);
              }
              if (col0 + 32 + j + 1 < p.N) {
                b0 += __bfloat162float(p.bias[col0 + 32 + j]);
                b1 += __bfloat162float(p.bias[col0 + 32 + j + 1]);
              }
            }
            if constexpr (EPI == kEpiSilu || EPI == kEpiBiasSilu) {
              a0 = silu_f(a0); a1 = silu_f(a1); b0 = silu_f(b0); b1 = silu_f(b1);
            }
            w[j >> 1] = pack_bf16x2(a0, a1);
            w[16 + (j >> 1)] = pack_bf16x2(b0, b1);
          }
          // row `lane` of the 32 x 128-byte buffer; 16-byte chunk j lands at chunk (j ^ (row & 7))
          const uint32_t row_addr = buf + static_cast<uint32_t>(lane) * 128u;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t dst = row_addr + (static_cast<uint32_t>(j ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[4 * j]),
                         "r"(w[4 * j + 1]), "r"(w[4 * j + 2]), "r"(w[4 * j + 3])
                         : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && col0 < p.N && row_blk0 + q * 32 < p.M) {
            if constexpr (BCAST) {
              for (int k = 0; k < p.world; ++k) {
                int g = p.rank_in_group + k;  // own copy first, the peers spread over time
                if (g >= p.world) g -= p.world;
                tma_store_2d(&out_maps->m[g], buf, p.bcast_col0 + col0, row_coord);
              }
            } else {
              tma_store_2d(&out_maps->m[map_idx], buf, col0, row_coord);
            }
            tma_store_commit();
          }
        }
        if constexpr (RS_SCATTER) {
          // the owner may only be told once the stores have been performed, not merely read
          if (lane == 0) {
            tma_store_wait_all<0>();
            fence_proxy_async_all();
          }
        }
      } else {
      const bool row_ok = row < (GROUPED ? g_row_end : p.M);
  #pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                 static_cast<uint32_t>(acc * BN + c * 32);
          tmem_ld_32x32(taddr, r);
          tmem_ld_wait();
          const int col0 = n0 + c * 32;
          if (row_ok && col0 < p.N) {
            float v[32];
  #pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
            if constexpr (EPI == kEpiBias || EPI == kEpiBiasSilu) {
  #pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
            }
            if constexpr (EPI == kEpiSilu || EPI == kEpiBiasSilu) {
  #pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = silu_f(v[j]);
            }
            if constexpr (EPI == kEpiSwiGLU) {
              // accumulator columns come in (gate, up) pairs: 32 of them give 16 outputs at column col0 / 2
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out_row) + (col0 >> 1);
              float h[16];
  #pragma unroll
              for (int j = 0; j < 16; ++j) h[j] = silu_f(v[2 * j]) * v[2 * j + 1];
              if (col0 + 32 <= p.N && (p.ldc & 7) == 0) {
                st_global_v4(o, U4{pack_bf16x2(h[0], h[1]), pack_bf16x2(h[2], h[3]), pack_bf16x2(h[4], h[5]), pack_bf16x2(h[6], h[7])});
                st_global_v4(o + 8, U4{pack_bf16x2(h[8], h[9]), pack_bf16x2(h[10], h[11]), pack_bf16x2(h[12], h[13]), pack_bf16x2(h[14], h[15])});
              } else {
                for (int j = 0; j < 16; ++j)
                  if (col0 + 2 * j + 1 < p.N) o[j] = __float2bfloat16_rn(h[j]);
              }
            } else if constexpr (OUT_F32) {
              float* o = reinterpret_cast<float*>(out_row) + col0;
              if (col0 + 32 <= p.N && (p.ldc & 3) == 0) {
  #pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  U4 u{__float_as_uint(v[j]), __float_as_uint(v[j + 1]), __float_as_uint(v[j + 2]),
                       __float_as_uint(v[j + 3])};
                  st_global_v4(o + j, u);
                }
              } else {
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < p.N) o[j] = v[j];
              }
            } else {
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out_row) + col0;
              if (col0 + 32 <= p.N && (p.ldc & 7) == 0) {
  #pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  U4 u{pack_bf16x2(v[j], v[j + 1]), pack_bf16x2(v[j + 2], v[j + 3]),
                       pack_bf16x2(v[j + 4], v[j + 5]), pack_bf16x2(v[j + 6], v[j + 7])};
                  st_global_v4(o + j, u);
                }
              } else {
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < p.N) o[j] = __float2bfloat16_rn(v[j]);
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc == 0 ? leader_tempty0 : leader_tempty1);

      if constexpr (RS_SCATTER) {
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          const int owner = row_blk0 / p.rs_rows_per_rank;
          if (owner < p.world && row_blk0 < p.M) {
            const int blk_in_rank = (row_blk0 - owner * p.rs_rows_per_rank) / kGemmBlockM;
            red_release_sys_add(p.rs_done[owner] + blk_in_rank, 1u);
          }
        }
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if constexpr (TMA_STORE) {
      if (lane == 0) {
        tma_store_wait_all<0>();  // staging memory and stores are done before exit
        if constexpr (BCAST) fence_proxy_async_all();  // ... and ordered before the barrier that publishes them
      }
      __syncwarp();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  // neither CTA may leave (or free TMEM) while the other can still signal its barriers
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <int EPI, bool OUT_F32, bool A_READY, bool RS_SCATTER>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_umma2_kernel(const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  gemm_umma2_cta<EPI, OUT_F32, A_READY, RS_SCATTER>(tmap_a, tmap_b, p, blockIdx.x >> 1,
                                                    gridDim.x >> 1);
}

// MN-major operands (see gemm_umma2_cta), register epilogue (bf16 or fp32 output)
template <int EPI, bool OUT_F32, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_umma2_mn_kernel(const __grid_constant__ CUtensorMap tmap_a,
                     const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  gemm_umma2_cta<EPI, OUT_F32, false, false, false, false, A_MN, B_MN>(tmap_a, tmap_b, p, blockIdx.x >> 1, gridDim.x >> 1);
}

// grouped form (see gemm_umma2_cta): one weight matrix per row group, register epilogue
template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_umma2_grouped_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  gemm_umma2_cta<EPI, false, false, false, false, false, false, false, true>(tmap_a, tmap_b, p, blockIdx.x >> 1, gridDim.x >> 1);
}

// bf16 output through the TMA-store epilogue
template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_umma2_tma_kernel(const __grid_constant__ CUtensorMap tmap_a,
                      const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ GemmOutMaps out_maps, const GemmParams p) {
  gemm_umma2_cta<EPI, false, false, false, true>(tmap_a, tmap_b, p, blockIdx.x >> 1,
                                                 gridDim.x >> 1, &out_maps);
}

}  // namespace pkb
