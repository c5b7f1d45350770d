// RMSNorm kernels (memory bound: 16-byte accesses, fp32 statistics, one CTA per row).
//  * rmsnorm_bf16: y = x * rsqrt(mean(x^2) + eps) * gamma
//  * sum_rmsnorm: the tail of a reduce-scatter: sums `nsrc` partial buffers of the same shape in
//    a fixed order (deterministic), scales, normalises and writes bf16 - the reduced tensor never
//    goes to memory un-normalised.
#include "pkb/api.h"
#include "pkb/host.h"
#include "pkb/ptx.cuh"

namespace pkb {

constexpr int kNormThreads = 256;
constexpr int kNormRowChunks = 4;   // bf16 rows of up to 4 * 8 * 256 = 8192 elements stay in registers between the two passes
constexpr int kNormMaxSrc = 8;      // ... when at most this many source buffers are summed

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (blockDim.x >> 5)) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// Row lives in dynamic shared memory as fp32 between the two passes.
// MAXSRC: upper bound of nsrc the register path is compiled for (1: plain RMSNorm, more CTAs per SM; kNormMaxSrc: sums)
template <bool SRC_F32, int MAXSRC>
__global__ void __launch_bounds__(kNormThreads, MAXSRC == 1 ? 4 : 2)
sum_rmsnorm_kernel(const void* __restrict__ src, long long src_stride, int nsrc,
                   const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ y, int rows,
                   int cols, float scale, float eps) {
  extern __shared__ float rowbuf[];
  __shared__ float red[32];
  if constexpr (!SRC_F32 && MAXSRC == 1) {
    if (cols <= kNormRowChunks * 8 * kNormThreads && nsrc == 1) {
      // plain RMSNorm of a row that fits in registers: the loads of the CTA's NEXT row are issued before the reduction of
      // the current one, so a CTA always has a row in flight (two block-wide synchronisations per row otherwise leave the
      // memory system idle: 4.2 TB/s without the prefetch)
      const __nv_bfloat16* s0 = static_cast<const __nv_bfloat16*>(src);
      U4 cur[kNormRowChunks];
      int row = blockIdx.x;
      if (row < rows) {
#pragma unroll
        for (int ch = 0; ch < kNormRowChunks; ++ch) {
          const int i = (ch * kNormThreads + (int)threadIdx.x) * 8;
          if (i < cols) cur[ch] = ld_global_nc_v4(s0 + (long long)row * cols + i);
        }
      }
      for (; row < rows; row += gridDim.x) {
        const int nrow = row + (int)gridDim.x;
        U4 nxt[kNormRowChunks];
        if (nrow < rows) {
#pragma unroll
          for (int ch = 0; ch < kNormRowChunks; ++ch) {
            const int i = (ch * kNormThreads + (int)threadIdx.x) * 8;
            if (i < cols) nxt[ch] = ld_global_nc_v4(s0 + (long long)nrow * cols + i);
          }
        }
        float vals[kNormRowChunks][8];
        float ss = 0.f;
#pragma unroll
        for (int ch = 0; ch < kNormRowChunks; ++ch) {
          const int i = (ch * kNormThreads + (int)threadIdx.x) * 8;
          if (i < cols) {
            const float2 f0 = unpack_bf16x2(cur[ch].x), f1 = unpack_bf16x2(cur[ch].y), f2 = unpack_bf16x2(cur[ch].z),
                         f3 = unpack_bf16x2(cur[ch].w);
            vals[ch][0] = f0.x * scale; vals[ch][1] = f0.y * scale; vals[ch][2] = f1.x * scale; vals[ch][3] = f1.y * scale;
            vals[ch][4] = f2.x * scale; vals[ch][5] = f2.y * scale; vals[ch][6] = f3.x * scale; vals[ch][7] = f3.y * scale;
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += vals[ch][j] * vals[ch][j];
          }
        }
        const float total = block_sum(ss, red);
        const float rstd = rsqrtf(total / (float)cols + eps);
        __nv_bfloat16* yrow = y + (long long)row * cols;
#pragma unroll
        for (int ch = 0; ch < kNormRowChunks; ++ch) {
          const int i = (ch * kNormThreads + (int)threadIdx.x) * 8;
          if (i < cols) {
            const U4 g = ld_global_v4(gamma + i);
            const float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z), g3 = unpack_bf16x2(g.w);
            U4 o;
            o.x = pack_bf16x2(vals[ch][0] * rstd * g0.x, vals[ch][1] * rstd * g0.y);
            o.y = pack_bf16x2(vals[ch][2] * rstd * g1.x, vals[ch][3] * rstd * g1.y);
            o.z = pack_bf16x2(vals[ch][4] * rstd * g2.x, vals[ch][5] * rstd * g2.y);
            o.w = pack_bf16x2(vals[ch][6] * rstd * g3.x, vals[ch][7] * rstd * g3.y);
            st_global_v4(yrow + i, o);
          }
        }
#pragma unroll
        for (int ch = 0; ch < kNormRowChunks; ++ch) cur[ch] = nxt[ch];
      }
      return;
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    __nv_bfloat16* yrow = y + (long long)row * cols;
    if constexpr (!SRC_F32) {
      if (cols <= kNormRowChunks * 8 * kNormThreads && nsrc <= MAXSRC) {
        // bf16 sources, row short enough for registers: thread t owns the 16-byte chunks t, t + 256, ...; the loads of all
        // sources of a chunk are issued before the first addition (memory bound: what counts is loads in flight)
        const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(src) + (long long)row * cols;
        float vals[kNormRowChunks][8];
        float ss = 0.f;
#pragma unroll
        for (int ch = 0; ch < kNormRowChunks; ++ch) {
          const int i = (ch * kNormThreads + (int)threadIdx.x) * 8;
          if (i < cols) {
            U4 u[MAXSRC];
#pragma unroll
            for (int sidx = 0; sidx < MAXSRC; ++sidx)
              if (sidx < nsrc) u[sidx] = ld_global_nc_v4(base + (long long)sidx * src_stride + i);
#pragma unroll
            for (int j = 0; j < 8; ++j) vals[ch][j] = 0.f;
#pragma unroll
            for (int sidx = 0; sidx < MAXSRC; ++sidx) {
              if (sidx < nsrc) {
                const float2 f0 = unpack_bf16x2(u[sidx].x), f1 = unpack_bf16x2(u[sidx].y), f2 = unpack_bf16x2(u[sidx].z),
                             f3 = unpack_bf16x2(u[sidx].w);
                vals[ch][0] += f0.x; vals[ch][1] += f0.y; vals[ch][2] += f1.x; vals[ch][3] += f1.y;
                vals[ch][4] += f2.x; vals[ch][5] += f2.y; vals[ch][6] += f3.x; vals[ch][7] += f3.y;
              }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              vals[ch][j] *= scale;
              ss += vals[ch][j] * vals[ch][j];
            }
          }
        }
        const float total = block_sum(ss, red);
        const float rstd = rsqrtf(total / (float)cols + eps);
#pragma unroll
        for (int ch = 0; ch < kNormRowChunks; ++ch) {
          const int i = (ch * kNormThreads + (int)threadIdx.x) * 8;
          if (i < cols) {
            const U4 g = ld_global_v4(gamma + i);
            const float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z), g3 = unpack_bf16x2(g.w);
            U4 o;
            o.x = pack_bf16x2(vals[ch][0] * rstd * g0.x, vals[ch][1] * rstd * g0.y);
            o.y = pack_bf16x2(vals[ch][2] * rstd * g1.x, vals[ch][3] * rstd * g1.y);
            o.z = pack_bf16x2(vals[ch][4] * rstd * g2.x, vals[ch][5] * rstd * g2.y);
            o.w = pack_bf16x2(vals[ch][6] * rstd * g3.x, vals[ch][7] * rstd * g3.y);
            st_global_v4(yrow + i, o);
          }
        }
        continue;
      }
    }
    float ss = 0.f;
    if constexpr (SRC_F32) {
      const float* base = static_cast<const float*>(src) + (long long)row * cols;
      for (int i = threadIdx.x * 4; i < cols; i += kNormThreads * 4) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        for (int s = 0; s < nsrc; ++s) {
          U4 u = ld_global_nc_v4(base + (long long)s * src_stride + i);
          a0 += __uint_as_float(u.x); a1 += __uint_as_float(u.y);
          a2 += __uint_as_float(u.z); a3 += __uint_as_float(u.w);
        }
        a0 *= scale; a1 *= scale; a2 *= scale; a3 *= scale;
        rowbuf[i] = a0; rowbuf[i + 1] = a1; rowbuf[i + 2] = a2; rowbuf[i + 3] = a3;
        ss += a0 * a0 + a1 * a1 + a2 * a2 + a3 * a3;
      }
    } else {
      const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(src) + (long long)row * cols;
      for (int i = threadIdx.x * 8; i < cols; i += kNormThreads * 8) {
        float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < nsrc; ++s) {
          U4 u = ld_global_nc_v4(base + (long long)s * src_stride + i);
          float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z),
                 f3 = unpack_bf16x2(u.w);
          a[0] += f0.x; a[1] += f0.y; a[2] += f1.x; a[3] += f1.y;
          a[4] += f2.x; a[5] += f2.y; a[6] += f3.x; a[7] += f3.y;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          a[j] *= scale;
          rowbuf[i + j] = a[j];
          ss += a[j] * a[j];
        }
      }
    }
    const float total = block_sum(ss, red);
    const float rstd = rsqrtf(total / (float)cols + eps);
    for (int i = threadIdx.x * 8; i < cols; i += kNormThreads * 8) {
      U4 g = ld_global_v4(gamma + i);
      float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z),
             g3 = unpack_bf16x2(g.w);
      U4 o;
      o.x = pack_bf16x2(rowbuf[i] * rstd * g0.x, rowbuf[i + 1] * rstd * g0.y);
      o.y = pack_bf16x2(rowbuf[i + 2] * rstd * g1.x, rowbuf[i + 3] * rstd * g1.y);
      o.z = pack_bf16x2(rowbuf[i + 4] * rstd * g2.x, rowbuf[i + 5] * rstd * g2.y);
      o.w = pack_bf16x2(rowbuf[i + 6] * rstd * g3.x, rowbuf[i + 7] * rstd * g3.y);
      st_global_v4(yrow + i, o);
    }
    __syncthreads();
  }
}

static int launch_sum_rmsnorm(const void* src, long long src_stride, int nsrc, int src_is_f32,
                              const void* gamma, void* y, int rows, int cols, float scale,
                              float eps, cudaStream_t stream) {
  PKB_CHECK_ARG(rows > 0 && cols > 0 && cols % 8 == 0, "cols must be a positive multiple of 8");
  PKB_CHECK_ARG(nsrc >= 1, "need at least one source");
  const bool in_regs = !src_is_f32 && cols <= kNormRowChunks * 8 * kNormThreads && nsrc <= kNormMaxSrc;
  const int smem = in_regs ? 0 : cols * (int)sizeof(float);
  PKB_CHECK_ARG(smem <= 200 * 1024, "row too long for the shared-memory row buffer");
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
#define PKB_NORM_LAUNCH(F32, MS)                                                                        \
  {                                                                                                    \
    auto k = sum_rmsnorm_kernel<F32, MS>;                                                              \
    if (smem > 48 * 1024)                                                                              \
      PKB_CHECK_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));      \
    k<<<grid, kNormThreads, smem, stream>>>(src, src_stride, nsrc, static_cast<const __nv_bfloat16*>(gamma), \
                                            static_cast<__nv_bfloat16*>(y), rows, cols, scale, eps);   \
  }
  if (src_is_f32) PKB_NORM_LAUNCH(true, 1)
  else if (nsrc == 1) PKB_NORM_LAUNCH(false, 1)
  else PKB_NORM_LAUNCH(false, kNormMaxSrc)
#undef PKB_NORM_LAUNCH
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

}  // namespace pkb

using namespace pkb;

extern "C" int pkb_rmsnorm_bf16(const void* x, const void* gamma, void* y, int rows, int cols,
                                float eps, void* stream) {
  return launch_sum_rmsnorm(x, 0, 1, 0, gamma, y, rows, cols, 1.0f, eps,
                            static_cast<cudaStream_t>(stream));
}

extern "C" int pkb_sum_rmsnorm(const void* src, long long src_stride_elems, int nsrc,
                               int src_is_f32, const void* gamma, void* y, int rows, int cols,
                               float scale, float eps, void* stream) {
  return launch_sum_rmsnorm(src, src_stride_elems, nsrc, src_is_f32, gamma, y, rows, cols, scale,
                            eps, static_cast<cudaStream_t>(stream));
}
