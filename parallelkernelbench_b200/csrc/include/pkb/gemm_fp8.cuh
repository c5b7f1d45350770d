// Block-scaled fp8 (e4m3) GEMM on tcgen05:  C = epilogue( sum_kb sa[m, kb] * sb[n/128, kb] * A8[m, kb] . B8[n, kb] ).
//
// A8 [M, K] and B8 [N, K] are e4m3, both K-major. A carries one fp32 scale per row and 128 consecutive
// K elements (the 1x128 form a row quantiser produces); B carries one fp32 scale per 128 x 128 block
// (weights quantised once). The scales are arbitrary fp32 numbers, so the tensor core cannot apply
// them: every 128-deep K block is multiplied on its own into one of two TMEM partial buffers
// (`tcgen05.mma.kind::f8f6f4`, 128 x 256 x 32 per instruction) and eight promotion warps fold the
// finished partial into fp32 register accumulators with acc += (sa * sb) * partial while the
// tensor core already works on the next K block in the other buffer.
//
//   warp 0     : TMA producer - ring of (A 128 x 128 B, B 256 x 128 B) stages, 128-byte swizzle
//   warp 1     : MMA issuer   - four K=32 instructions per stage, commit -> stage free + partial full
//   warps 2-9  : promotion + epilogue - warp w owns TMEM lanes 32*(w%4).. and the 128 accumulator
//                columns of half (w-2)/4; 128 fp32 accumulators per thread
//
// Epilogues: bf16 store; SwiGLU over interleaved (gate, up) columns -> bf16; SwiGLU followed by
// 1x128 re-quantisation to e4m3 + fp32 scales, so a second block-scaled GEMM can consume the result
// without a pass through bf16 (one output scale group = the 128 outputs of one 256-column tile; the
// two column halves exchange their maxima through shared memory and an mbarrier).
// The grouped (ragged) form multiplies row group e of A with weight block e, groups given by a
// device-resident offsets array. Every wait is bounded; on expiry the CTA records a status word,
// drains and frees its TMEM.
#pragma once
#include <cuda_fp8.h>

#include "pkb/gemm_umma.cuh"

namespace pkb {

constexpr int kFp8BlockM = 128;
constexpr int kFp8BlockN = 256;
constexpr int kFp8BlockK = 128;   // e4m3 elements = bytes = one 128-byte swizzle row = one scale block
constexpr int kFp8Threads = 320;  // producer warp, MMA warp, eight promotion warps
constexpr int kFp8Stages = 4;

enum GemmFp8Epilogue : int {
  kFp8EpiNone = 0,         // bf16 out [M, N]
  kFp8EpiSwiGLU = 1,       // bf16 out [M, N/2]
  kFp8EpiSwiGLUQuant = 2,  // e4m3 out [M, N/2] + fp32 scales [M, N/256]
  kFp8EpiRowScatter = 3,   // bf16 row m -> row row_meta[m].y of the buffer scatter_out[row_meta[m].x] (maybe on a peer)
};

struct GemmFp8Params {
  int M, N, K;               // M = rows of A the tensor map covers (grouped: upper bound of offsets[groups])
  void* C;                   // bf16 or e4m3
  long long ldc;             // elements between output rows
  const float* sa;           // A scales: sa[row * sa_stride + kb]
  long long sa_stride;
  const float* sb;           // B scales: sb[(b_row / 128) * sb_stride + kb], b_row counts rows of the whole B
  long long sb_stride;
  float* out_scales;         // re-quantising epilogue: out_scales[row * os_stride + n_blk]
  long long os_stride;
  float alpha;
  uint32_t* status;
  uint64_t wait_budget_ns;
  int kernel_id;
  const int* grp_offsets;    // grouped form: [grp_count + 1] row offsets in device memory
  int grp_count;
  const int2* row_meta;      // row-scatter epilogue: per row of A (index into scatter_out, destination row)
  void* scatter_out[kGemmMaxWorld];
};

struct GemmFp8Smem {
  static constexpr int kABytes = kFp8BlockM * kFp8BlockK;
  static constexpr int kBBytes = kFp8BlockN * kFp8BlockK;
  static constexpr int kStageBytes = kABytes + kBBytes;  // 48 KiB
  static constexpr int kBarrierBytes = 256;
  static constexpr int kXchgBytes = 2 * 2 * kFp8BlockM * 4;  // [tile parity][column half][row] maxima
  static constexpr int kTotal = kFp8Stages * kStageBytes + kBarrierBytes + kXchgBytes + 1024;
};

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

template <int EPI, bool GROUPED>
__device__ __forceinline__ void gemm_fp8_cta(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b,
                                             const GemmFp8Params& p, const int cta, const int num_ctas) {
  using S = GemmFp8Smem;
  constexpr int BN = kFp8BlockN;
  constexpr int kStages = kFp8Stages;
  constexpr uint32_t kTmemCols = 2 * BN;  // two partial-sum buffers

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t bar_base = smem_base + kStages * S::kStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto pfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
  auto pempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
  const uint32_t xchg_bar = bar_base + 8u * (2 * kStages + 4);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem_gen + kStages * S::kStageBytes + 8 * (2 * kStages + 5));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* xchg = reinterpret_cast<float*>(smem_gen + kStages * S::kStageBytes + S::kBarrierBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_m = (p.M + kFp8BlockM - 1) / kFp8BlockM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_k = p.K / kFp8BlockK;

  __shared__ int s_tile_prefix[GROUPED ? kGemmMaxGroups + 1 : 1];
  if constexpr (GROUPED) {
    for (int e = threadIdx.x; e < p.grp_count; e += blockDim.x) {
      const int cnt = p.grp_offsets[e + 1] - p.grp_offsets[e];
      s_tile_prefix[e + 1] = (cnt + kFp8BlockM - 1) / kFp8BlockM;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      s_tile_prefix[0] = 0;
      for (int e = 0; e < p.grp_count; ++e) s_tile_prefix[e + 1] += s_tile_prefix[e];
    }
    __syncthreads();
  }
  const int num_tiles = GROUPED ? s_tile_prefix[p.grp_count] * num_n : num_m * num_n;

  // tile -> first row of A / C, row limit, n block, first row of B (n fastest: the 128 x K row panel of A is
  // shared by the CTAs of a wave through L2)
  auto tile_coords = [&](int tile, int& row0, int& row_end, int& n_blk, int& b_row0) {
    const int mi = tile / num_n;
    n_blk = tile - mi * num_n;
    if constexpr (GROUPED) {
      int lo = 0, hi = p.grp_count;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_tile_prefix[mid] <= mi) lo = mid; else hi = mid;
      }
      row0 = p.grp_offsets[lo] + (mi - s_tile_prefix[lo]) * kFp8BlockM;
      row_end = min(p.grp_offsets[lo + 1], p.M);
      b_row0 = lo * p.N + n_blk * BN;
    } else {
      row0 = mi * kFp8BlockM;
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
    for (int b = 0; b < 2; ++b) {
      mbar_init(pfull_bar(b), 1);
      mbar_init(pempty_bar(b), 8);  // one arrival per promotion warp
    }
    mbar_init(xchg_bar, 256);       // one arrival per promotion thread
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
    // warp-uniform loop: one elected lane's copies take effect (see umma_f16_ss_p)
    {
      const uint32_t lead = elect_one() ? 1u : 0u;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += num_ctas) {
        int row0, row_end, n_blk, b_row0;
        tile_coords(tile, row0, row_end, n_blk, b_row0);
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.wait_budget_ns)) {
            if (lane == 0) record_status(p.status, kStatusMbarTimeout, p.kernel_id, 0, stage, 11, tile);
            ok = false;
            break;
          }
          mbar_expect_tx_p(full_bar(stage), S::kStageBytes, lead);
          const uint32_t sa = smem_base + stage * S::kStageBytes;
          tma_load_2d_p(sa, &tmap_a, full_bar(stage), kb * kFp8BlockK, row0, lead);
          tma_load_2d_p(sa + S::kABytes, &tmap_b, full_bar(stage), kb * kFp8BlockK, b_row0, lead);
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
      constexpr uint32_t idesc = make_idesc(kFp8BlockM, BN, 0, 0);  // e4m3 x e4m3, fp32 accumulate
      const uint32_t a_lo0 = smem_desc_lo_kmajor(smem_base), b_lo0 = smem_desc_lo_kmajor(smem_base + S::kABytes);
      int stage = 0;
      uint32_t phase = 0;
      int pb = 0;
      uint32_t pb_phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += num_ctas) {
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(pempty_bar(pb), pb_phase ^ 1u, abort_flag, p.wait_budget_ns)) {
            if (lane == 0) record_status(p.status, kStatusMbarTimeout, p.kernel_id, 0, pb, 20, tile);
            ok = false;
            break;
          }
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.wait_budget_ns)) {
            if (lane == 0) record_status(p.status, kStatusMbarTimeout, p.kernel_id, 0, stage, 21, tile);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_lo = a_lo0 + stage * (S::kStageBytes >> 4), b_lo = b_lo0 + stage * (S::kStageBytes >> 4);
          const uint32_t tmem_d = tmem_base + pb * BN;
#pragma unroll
          for (int k = 0; k < kFp8BlockK / 32; ++k)   // 32 e4m3 = 32 bytes along K inside the swizzled row: +2 in the address field
            umma_f8_ss_p(tmem_d, smem_desc_join(a_lo + 2u * k), smem_desc_join(b_lo + 2u * k), idesc, k != 0 ? 1u : 0u, lead);
          umma_commit_p(empty_bar(stage), lead);  // stage reusable once these MMAs have read it
          umma_commit_p(pfull_bar(pb), lead);     // partial sum of this K block complete
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
          if (++pb == 2) {
            pb = 0;
            pb_phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ promotion + epilogue (warps 2..9) ------------------------------
    const int q = warp & 3;          // TMEM lane quadrant this warp may access
    const int half = (warp - 2) >> 2;  // which 128 accumulator columns of the tile
    const int r_in_tile = q * 32 + lane;
    int pb = 0;
    uint32_t pb_phase = 0;
    uint32_t xchg_phase = 0;
    int tile_parity = 0;
    bool ok = true;
    for (int tile = cta; tile < num_tiles && ok; tile += num_ctas) {
      int tile_row0, row_end, n_blk, b_row0;
      tile_coords(tile, tile_row0, row_end, n_blk, b_row0);
      const int row = tile_row0 + r_in_tile;
      const bool row_ok = row < row_end;
      const int col0 = n_blk * BN + half * 128;        // first accumulator column of this thread
      const bool half_ok = col0 < p.N;
      const float* sa_row = p.sa + (long long)(row_ok ? row : min(tile_row0, p.M - 1)) * p.sa_stride;
      const float* sb_row = p.sb + (long long)((b_row0 + (half_ok ? half * 128 : 0)) >> 7) * p.sb_stride;

      float acc[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) acc[j] = 0.f;
      float s_next = sa_row[0] * sb_row[0];
      for (int kb = 0; kb < num_k; ++kb) {
        const float s = row_ok ? s_next : 0.f;
        if (kb + 1 < num_k) s_next = sa_row[kb + 1] * sb_row[kb + 1];
        bool got = mbar_wait(pfull_bar(pb), pb_phase, abort_flag, p.wait_budget_ns);
        got = __all_sync(0xffffffffu, got);
        if (!got) {
          if (lane == 0) record_status(p.status, kStatusMbarTimeout, p.kernel_id, 0, pb, 30, tile);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                               static_cast<uint32_t>(pb * BN + half * 128);
#pragma unroll
        for (int c = 0; c < 8; c += 2) {
          uint32_t r0[16], r1[16];      // two reads in flight per wait
          tmem_ld_32x16(taddr + c * 16, r0);
          tmem_ld_32x16(taddr + c * 16 + 16, r1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c * 16 + j] = fmaf(s, __uint_as_float(r0[j]), acc[c * 16 + j]);
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c * 16 + 16 + j] = fmaf(s, __uint_as_float(r1[j]), acc[c * 16 + 16 + j]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(pempty_bar(pb));
        if (++pb == 2) {
          pb = 0;
          pb_phase ^= 1u;
        }
      }
      if (!ok) break;

      // ---- epilogue from registers ----
      if constexpr (EPI == kFp8EpiNone || EPI == kFp8EpiRowScatter) {
        if (row_ok && half_ok) {
          __nv_bfloat16* o;
          if constexpr (EPI == kFp8EpiRowScatter) {
            const int2 meta = p.row_meta[row];
            o = static_cast<__nv_bfloat16*>(p.scatter_out[meta.x]) + (long long)meta.y * p.ldc + col0;
          } else {
            o = static_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
          }
          if (col0 + 128 <= p.N && (p.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 128; j += 8) {
              U4 u{pack_bf16x2(acc[j] * p.alpha, acc[j + 1] * p.alpha), pack_bf16x2(acc[j + 2] * p.alpha, acc[j + 3] * p.alpha),
                   pack_bf16x2(acc[j + 4] * p.alpha, acc[j + 5] * p.alpha), pack_bf16x2(acc[j + 6] * p.alpha, acc[j + 7] * p.alpha)};
              st_global_v4(o + j, u);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 128; ++j)
              if (col0 + j < p.N) o[j] = __float2bfloat16_rn(acc[j] * p.alpha);
          }
        }
      } else {
        // 128 accumulator columns = 64 (gate, up) pairs -> 64 outputs starting at output column col0 / 2
        float g[64];
#pragma unroll
        for (int j = 0; j < 64; ++j) g[j] = silu_f(acc[2 * j] * p.alpha) * (acc[2 * j + 1] * p.alpha);
        const int ocol0 = col0 >> 1;
        const int n_out = p.N >> 1;
        if constexpr (EPI == kFp8EpiSwiGLU) {
          if (row_ok && half_ok) {
            __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + ocol0;
            if (ocol0 + 64 <= n_out && (p.ldc & 7) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 64; j += 8) {
                U4 u{pack_bf16x2(g[j], g[j + 1]), pack_bf16x2(g[j + 2], g[j + 3]), pack_bf16x2(g[j + 4], g[j + 5]),
                     pack_bf16x2(g[j + 6], g[j + 7])};
                st_global_v4(o + j, u);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 64; ++j)
                if (ocol0 + j < n_out) o[j] = __float2bfloat16_rn(g[j]);
            }
          }
        } else {
          // re-quantise: the 128 outputs of this tile row form one scale group; this thread holds 64 of them.
          // The values are rounded to bf16 first so that the result equals quantising a bf16 activation tensor.
          float amax = 0.f;
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            g[j] = __bfloat162float(__float2bfloat16_rn(g[j]));
            amax = fmaxf(amax, fabsf(g[j]));
          }
          if (!(row_ok && half_ok)) amax = 0.f;
          float* slot = xchg + (tile_parity * 2) * kFp8BlockM;
          slot[half * kFp8BlockM + r_in_tile] = amax;
          mbar_arrive(xchg_bar);
          bool got = mbar_wait(xchg_bar, xchg_phase, abort_flag, p.wait_budget_ns);
          got = __all_sync(0xffffffffu, got);
          if (!got) {
            if (lane == 0) record_status(p.status, kStatusMbarTimeout, p.kernel_id, 0, 0, 31, tile);
            ok = false;
            break;
          }
          xchg_phase ^= 1u;
          amax = fmaxf(amax, slot[(half ^ 1) * kFp8BlockM + r_in_tile]);
          tile_parity ^= 1;
          float sc = amax / 448.0f;
          if (sc == 0.f) sc = 1.0f;
          const float inv = 1.0f / sc;
          if (row_ok && half_ok) {
            uint8_t* o = static_cast<uint8_t*>(p.C) + (long long)row * p.ldc + ocol0;
            if (ocol0 + 64 <= n_out && (p.ldc & 15) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 64; j += 16) {
                U4 u{pack_e4m3x4(g[j] * inv, g[j + 1] * inv, g[j + 2] * inv, g[j + 3] * inv),
                     pack_e4m3x4(g[j + 4] * inv, g[j + 5] * inv, g[j + 6] * inv, g[j + 7] * inv),
                     pack_e4m3x4(g[j + 8] * inv, g[j + 9] * inv, g[j + 10] * inv, g[j + 11] * inv),
                     pack_e4m3x4(g[j + 12] * inv, g[j + 13] * inv, g[j + 14] * inv, g[j + 15] * inv)};
                st_global_v4(o + j, u);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 64; ++j)
                if (ocol0 + j < n_out)
                  o[j] = (uint8_t)__nv_cvt_float_to_fp8(g[j] * inv, __NV_SATFINITE, __NV_E4M3);
            }
            if (half == 0) p.out_scales[(long long)row * p.os_stride + n_blk] = sc;
          }
        }
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

template <int EPI, bool GROUPED>
__global__ void __launch_bounds__(kFp8Threads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const GemmFp8Params p) {
  gemm_fp8_cta<EPI, GROUPED>(tmap_a, tmap_b, p, blockIdx.x, gridDim.x);
}

}  // namespace pkb
