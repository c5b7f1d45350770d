// Persistent warp-specialised tcgen05 GEMM:  C[M,N] = epilogue( A[M,K] * B[N,K]^T ).
//
// Both operands are K-major (row-major A, row-major "weight" B with one output feature per row,
// the torch.nn.Linear layout). One CTA per SM walks output tiles of 128 x BN:
//   warp 0   : TMA producer  - fills a ring of (A 128x64, B BNx64) bf16 stages, 128-byte swizzle
//   warp 1   : MMA issuer    - one thread issues tcgen05.mma (128 x BN x 16), accumulators in TMEM,
//                              two accumulator buffers so tile i+1 computes while tile i drains
//   warps 2-5: epilogue      - tcgen05.ld 32x32 chunks, apply the epilogue functor, 16-byte stores
// The optional hooks turn the same kernel into the fused tensor-parallel forms:
//   * a_ready flags: the producer waits (bounded) until the row chunk of A it is about to read
//     has been gathered into local memory by the communication CTAs (all-gather -> GEMM);
//   * row-block scatter: the epilogue stores each 128-row block into the buffer of the rank that
//     owns it, then bumps a counter there (GEMM -> reduce-scatter).
// Every wait is bounded; on a time-out the CTA records a status word, drains and frees its TMEM.
#pragma once
#include "pkb/ptx.cuh"

namespace pkb {

constexpr int kGemmBlockM = 128;
constexpr int kGemmBlockK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int kGemmThreads = 192;
constexpr int kGemmMaxWorld = 8;

enum GemmEpilogue : int {
  kEpiNone = 0,
  kEpiSilu = 1,
  kEpiBias = 2,
  kEpiBiasSilu = 3,
  kEpiSwiGLU = 4,  // columns come in (gate, up) pairs: out[:, j] = silu(acc[:, 2j]) * acc[:, 2j+1]
  kEpiRowScatter = 5,  // row m goes to row row_meta[m].y of the buffer rs_out[row_meta[m].x] (possibly on another rank)
};
constexpr int kGemmMaxGroups = 256;

struct GemmParams {
  int M, N, K;
  void* C;          // bf16 or fp32, row-major with leading dimension ldc (elements)
  long long ldc;
  const __nv_bfloat16* bias;  // [N] or nullptr
  float alpha;
  uint32_t* status;
  uint64_t wait_budget_ns;
  int group_m;  // m-blocks per rasterisation group (L2 reuse)
  int kernel_id;

  // ---- all-gather -> GEMM hook --------------------------------------------------------------
  // Rows [c*a_chunk_rows, (c+1)*a_chunk_rows) of A are readable once a_ready[c] >= a_ready_epoch.
  const uint32_t* a_ready;
  uint32_t a_ready_epoch;
  int a_chunk_rows;
  // Rows [a_local_row0, a_local_row0 + a_local_rows) of A are this rank's own shard: they are read
  // through a second tensor map straight from the caller's tensor, with no flag to wait for.
  int a_local_row0;
  int a_local_rows;
  // Optional instrumentation: when not null, every CTA's producer adds the SM cycles it spent waiting for a_ready
  // flags to a_wait_cycles[blockIdx.x] (one word per CTA of the launch; the caller zeroes it).
  unsigned long long* a_wait_cycles;
  // ---- GEMM -> reduce-scatter hook ----------------------------------------------------------
  // Output row m belongs to rank m / rs_rows_per_rank; it is stored at
  // rs_out[rank_of_m] + (m % rs_rows_per_rank) * ldc, and when a tile of that row block is done
  // the counter rs_done[rank_of_m][m_block_in_rank] (on the owner) is incremented by one.
  void* rs_out[kGemmMaxWorld];
  uint32_t* rs_done[kGemmMaxWorld];
  int rs_rows_per_rank;
  // ---- rank / schedule ----------------------------------------------------------------------
  int rank, world;
  int m_block_rotation;  // logical m-block i is physical (i + rotation) % num_m_blocks
  // ---- GEMM -> all-gather along N (broadcast epilogue of the CTA-pair kernel) ------------------
  int rank_in_group;     // index of this rank among the `world` destination maps
  int bcast_col0;        // first column of this rank's block in the gathered result
  // ---- grouped (ragged) form ------------------------------------------------------------------
  // A holds the rows of `grp_count` groups back to back: group e owns rows
  // [grp_offsets[e], grp_offsets[e+1]) (device memory, so the host never learns the counts) and
  // multiplies them with its own weight block B[e*N .. e*N+N, :].
  const int* grp_offsets;
  int grp_count;
  // ---- row-scatter epilogue (expert outputs pushed to the ranks their tokens came from) --------
  const int2* row_meta;  // per row of A: (index into rs_out, destination row)
};

template <int BN>
struct GemmSmem {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = kGemmBlockM * kGemmBlockK * 2;
  static constexpr int kBBytes = BN * kGemmBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + 1024;  // + align slack
};

// Body of one GEMM CTA. `cta` / `num_ctas` are this CTA's index and the number of CTAs that share
// the tile loop (a fused kernel may reserve some of its grid for communication roles).
// B_MN: B is given as [K, N] row-major (N contiguous) instead of [N, K]; its tiles are loaded as
// BN/64 boxes of 64 x 64 and described to the tensor core as MN-major.
// A_MN: A is given as [K, M] row-major (M contiguous), i.e. the kernel computes A^T B.
template <int BN, int EPI, bool OUT_F32, bool A_READY, bool RS_SCATTER, bool GROUPED = false,
          bool B_MN = false, bool A_MN = false>
__device__ __forceinline__ void gemm_umma_cta(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b,
                                              const GemmParams& p, const int cta,
                                              const int num_ctas) {
  using S = GemmSmem<BN>;
  constexpr int kStages = S::kStages;
  constexpr uint32_t kTmemCols = 2 * BN;  // two accumulator buffers (power of two: 256 or 512)

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t bar_base = smem_base + kStages * S::kStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  uint32_t* tmem_holder =
      reinterpret_cast<uint32_t*>(smem_gen + kStages * S::kStageBytes + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_m = (p.M + kGemmBlockM - 1) / kGemmBlockM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_k = (p.K + kGemmBlockK - 1) / kGemmBlockK;
  const int group_m = p.group_m > 0 ? p.group_m : 16;

  // grouped form: prefix sums of the groups' m-tile counts, built once per CTA from device counts
  __shared__ int s_tile_prefix[GROUPED ? kGemmMaxGroups + 1 : 1];
  if constexpr (GROUPED) {
    for (int e = threadIdx.x; e < p.grp_count; e += blockDim.x) {
      const int cnt = p.grp_offsets[e + 1] - p.grp_offsets[e];
      s_tile_prefix[e + 1] = (cnt + kGemmBlockM - 1) / kGemmBlockM;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      s_tile_prefix[0] = 0;
      for (int e = 0; e < p.grp_count; ++e) s_tile_prefix[e + 1] += s_tile_prefix[e];
    }
    __syncthreads();
  }
  const int num_tiles = GROUPED ? s_tile_prefix[p.grp_count] * num_n : num_m * num_n;

  // tile -> first row of A / C, row limit, n block, first row of B.
  // dense: groups of `group_m` m-blocks, n outer / m inner inside a group, so one wave of CTAs
  // touches a near-square set of A and B panels that stays in L2.
  // grouped: group-major, then m-tile, n fastest (the 128 x K row panel is shared by a wave).
  auto tile_coords = [&](int tile, int& row0, int& row_end, int& n_blk, int& b_row0) {
    if constexpr (GROUPED) {
      const int mi = tile / num_n;
      n_blk = tile - mi * num_n;
      int lo = 0, hi = p.grp_count;  // find e with prefix[e] <= mi < prefix[e+1]
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_tile_prefix[mid] <= mi) lo = mid; else hi = mid;
      }
      row0 = p.grp_offsets[lo] + (mi - s_tile_prefix[lo]) * kGemmBlockM;
      row_end = p.grp_offsets[lo + 1];
      b_row0 = lo * p.N + n_blk * BN;
    } else {
      const int tiles_per_group = group_m * num_n;
      const int g = tile / tiles_per_group;
      const int first_m = g * group_m;
      const int gm = min(group_m, num_m - first_m);
      const int local = tile - g * tiles_per_group;
      n_blk = local / gm;
      int m_blk = first_m + (local - n_blk * gm) + p.m_block_rotation;
      if (m_blk >= num_m) m_blk -= num_m;
      row0 = m_blk * kGemmBlockM;
      row_end = p.M;
      b_row0 = n_blk * BN;
    }
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);  // one arrival per epilogue warp
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    {
      // warp-uniform loop: one elected lane's copies take effect (see umma_f16_ss_p)
      const uint32_t lead = elect_one() ? 1u : 0u;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += num_ctas) {
        int row0, row_end, n_blk, b_row0;
        tile_coords(tile, row0, row_end, n_blk, b_row0);
        if constexpr (A_READY) {
          const int chunk = row0 / p.a_chunk_rows;
          if (!wait_flag_ge(p.a_ready + chunk, p.a_ready_epoch, p.wait_budget_ns)) {
            *abort_flag = 1;
            if (lane == 0) record_status(p.status, kStatusPeerTimeout, p.kernel_id, p.rank, chunk, 10, tile);
            ok = false;
            break;
          }
          // the gathered rows were written through the generic proxy (possibly by another CTA);
          // order them before this thread's async-proxy (TMA) reads
          fence_proxy_async_all();
        }
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_budget_ns)) {
            if (lane == 0) record_status(p.status, kStatusMbarTimeout, p.kernel_id, p.rank, stage, 11, tile);
            ok = false;
            break;
          }
          mbar_expect_tx_p(full_bar(stage), S::kStageBytes, lead);
          const uint32_t sa = smem_base + stage * S::kStageBytes;
          if constexpr (A_MN) {
#pragma unroll
            for (int j = 0; j < kGemmBlockM / 64; ++j)
              tma_load_2d_p(sa + j * 8192, &tmap_a, full_bar(stage), row0 + j * 64, kb * kGemmBlockK, lead);
          } else {
            tma_load_2d_p(sa, &tmap_a, full_bar(stage), kb * kGemmBlockK, row0, lead);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d_p(sa + S::kABytes + j * 8192, &tmap_b, full_bar(stage), b_row0 + j * 64,
                          kb * kGemmBlockK, lead);
          } else {
            tma_load_2d_p(sa + S::kABytes, &tmap_b, full_bar(stage), kb * kGemmBlockK, b_row0, lead);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // warp-uniform loop, one elected lane's tcgen05 instructions take effect (see umma_f16_ss_p)
    {
      const uint32_t lead = elect_one() ? 1u : 0u;
      constexpr uint32_t idesc = make_idesc(kGemmBlockM, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      // low descriptor words of stage 0; a stage adds kStageBytes >> 4, a K step of 16 adds 2 (K-major: 32 bytes inside the
      // swizzled row) or 128 (MN-major: 16 rows of 128 bytes)
      const uint32_t a_lo0 = A_MN ? smem_desc_lo_mnmajor(smem_base, 8192u) : smem_desc_lo_kmajor(smem_base);
      const uint32_t b_lo0 = B_MN ? smem_desc_lo_mnmajor(smem_base + S::kABytes, 8192u) : smem_desc_lo_kmajor(smem_base + S::kABytes);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += num_ctas) {
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
          const uint32_t a_lo = a_lo0 + stage * (S::kStageBytes >> 4), b_lo = b_lo0 + stage * (S::kStageBytes >> 4);
#pragma unroll
          for (int k = 0; k < kGemmBlockK / 16; ++k)
            umma_f16_ss_p(tmem_d, smem_desc_join(a_lo + (A_MN ? 128u : 2u) * k), smem_desc_join(b_lo + (B_MN ? 128u : 2u) * k), idesc,
                          (kb | k) != 0 ? 1u : 0u, lead);
          umma_commit_p(empty_bar(stage), lead);  // smem stage reusable once these MMAs have read it
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_p(tfull_bar(acc), lead);  // accumulator complete
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue (warps 2..5) ------------------------------
    const int q = warp & 3;  // TMEM lane quadrant this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = cta; tile < num_tiles; tile += num_ctas) {
      int tile_row0, row_end, n_blk, b_row0;
      tile_coords(tile, tile_row0, row_end, n_blk, b_row0);
      bool ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.wait_budget_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0)
          record_status(p.status, kStatusMbarTimeout, p.kernel_id, p.rank, acc, 30, tile);
        break;
      }
      tc_fence_after_sync();
      const int row = tile_row0 + q * 32 + lane;
      const int n0 = n_blk * BN;

      // destination row pointer (local, or the owner's buffer for the reduce-scatter form)
      uint8_t* out_row;
      constexpr int kOutBytes = OUT_F32 ? 4 : 2;
      if constexpr (RS_SCATTER) {
        const int owner = row / p.rs_rows_per_rank;
        const int r_in = row - owner * p.rs_rows_per_rank;
        out_row = static_cast<uint8_t*>(p.rs_out[owner < p.world ? owner : 0]) +
                  static_cast<long long>(r_in) * p.ldc * kOutBytes;
      } else if constexpr (EPI == kEpiRowScatter) {
        const int2 meta = row < row_end ? p.row_meta[row] : make_int2(0, 0);
        out_row = static_cast<uint8_t*>(p.rs_out[meta.x]) + static_cast<long long>(meta.y) * p.ldc * kOutBytes;
      } else {
        out_row = static_cast<uint8_t*>(p.C) + static_cast<long long>(row) * p.ldc * kOutBytes;
      }
      const bool row_ok = row < row_end;

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
          if constexpr (OUT_F32) {
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
          } else if constexpr (EPI == kEpiSwiGLU) {
            // 32 accumulator columns = 16 (gate, up) pairs -> 16 outputs at column col0 / 2
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out_row) + (col0 >> 1);
            float g[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) g[j] = silu_f(v[2 * j]) * v[2 * j + 1];
            if (col0 + 32 <= p.N && (p.ldc & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 16; j += 8) {
                U4 u{pack_bf16x2(g[j], g[j + 1]), pack_bf16x2(g[j + 2], g[j + 3]),
                     pack_bf16x2(g[j + 4], g[j + 5]), pack_bf16x2(g[j + 6], g[j + 7])};
                st_global_v4(o + j, u);
              }
            } else {
              for (int j = 0; j < 16; ++j)
                if (col0 + 2 * j + 1 < p.N) o[j] = __float2bfloat16_rn(g[j]);
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
      // accumulator buffer drained: hand it back to the MMA warp
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));

      if constexpr (RS_SCATTER) {
        // publish this warp's 32 rows x BN columns to the owner of the row block
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          const int row0 = tile_row0;
          const int owner = row0 / p.rs_rows_per_rank;
          if (owner < p.world) {
            const int blk_in_rank = (row0 - owner * p.rs_rows_per_rank) / kGemmBlockM;
            red_release_sys_add(p.rs_done[owner] + blk_in_rank, 1u);
          }
        }
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // give copies that are still in flight time to land before the shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int BN, int EPI, bool OUT_F32, bool A_READY, bool RS_SCATTER>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  gemm_umma_cta<BN, EPI, OUT_F32, A_READY, RS_SCATTER>(tmap_a, tmap_b, p, blockIdx.x, gridDim.x);
}

// B given as [K, N] row-major
template <int BN, int EPI, bool OUT_F32>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_umma_bkn_kernel(const __grid_constant__ CUtensorMap tmap_a,
                     const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  gemm_umma_cta<BN, EPI, OUT_F32, false, false, false, true>(tmap_a, tmap_b, p, blockIdx.x, gridDim.x);
}

// C = A^T B with A [K, M] and B [K, N], both row-major (weight gradients: dW = dY^T X)
template <int BN, bool OUT_F32>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_umma_tn_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  gemm_umma_cta<BN, kEpiNone, OUT_F32, false, false, false, true, true>(tmap_a, tmap_b, p, blockIdx.x, gridDim.x);
}

// ragged groups (MoE experts): A rows grouped by expert, B = [groups * N, K]
template <int BN, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_umma_grouped_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  gemm_umma_cta<BN, EPI, false, false, false, true>(tmap_a, tmap_b, p, blockIdx.x, gridDim.x);
}

}  // namespace pkb
