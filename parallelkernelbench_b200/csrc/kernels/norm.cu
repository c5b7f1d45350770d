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
template <bool SRC_F32>
__global__ void __launch_bounds__(kNormThreads)
sum_rmsnorm_kernel(const void* __restrict__ src, long long src_stride, int nsrc,
                   const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ y, int rows,
                   int cols, float scale, float eps) {
  extern __shared__ float rowbuf[];
  __shared__ float red[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
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
    __nv_bfloat16* yrow = y + (long long)row * cols;
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
  const int smem = cols * (int)sizeof(float);
  PKB_CHECK_ARG(smem <= 200 * 1024, "row too long for the shared-memory row buffer");
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  if (src_is_f32) {
    auto k = sum_rmsnorm_kernel<true>;
    if (smem > 48 * 1024)
      PKB_CHECK_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    k<<<grid, kNormThreads, smem, stream>>>(src, src_stride, nsrc,
                                            static_cast<const __nv_bfloat16*>(gamma),
                                            static_cast<__nv_bfloat16*>(y), rows, cols, scale, eps);
  } else {
    auto k = sum_rmsnorm_kernel<false>;
    if (smem > 48 * 1024)
      PKB_CHECK_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    k<<<grid, kNormThreads, smem, stream>>>(src, src_stride, nsrc,
                                            static_cast<const __nv_bfloat16*>(gamma),
                                            static_cast<__nv_bfloat16*>(y), rows, cols, scale, eps);
  }
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
