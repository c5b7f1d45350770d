// Quantised-wire helpers: the payload that crosses NVLink is 1 byte per element (fp8 e4m3 or int8)
// plus scales; the receiver dequantises and accumulates in fp32 on arrival.
//   fp8_quant_scaled   per-tensor scale read from device memory (delayed-scaling recipes)
//   int8_quant_block   per-block scale = max(amax, 1e-8) / 127, round to nearest, clamp to +-127
//   dequant_sum        out = out_scale * sum_w dequant(payload[w]) for per-tensor, 1x128 or int8 block scales
// Reference behaviour: reference/44_quantized_grad_allreduce.py:10-39,
// reference/52_fp8_reduce_scatter_grads.py:17-41, reference/53_fp8_allgather_params.py:17-39.
#include <cuda_fp8.h>

#include "pkb/api.h"
#include "pkb/host.h"
#include "pkb/ptx.cuh"

namespace pkb {

template <typename T>
__global__ void fp8_quant_scaled_kernel(const T* __restrict__ x, const float* __restrict__ scale_ptr,
                                        uint8_t* __restrict__ y, long long n) {
  const float inv = 1.0f / *scale_ptr;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4) {
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = (i + j < n) ? (float)x[i + j] * inv : 0.f;
    __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[0], v[1]), __NV_SATFINITE, __NV_E4M3);
    __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[2], v[3]), __NV_SATFINITE, __NV_E4M3);
    if (i + 3 < n) {
      *reinterpret_cast<uint32_t*>(y + i) = (uint32_t)lo | ((uint32_t)hi << 16);
    } else {
      const uint32_t p = (uint32_t)lo | ((uint32_t)hi << 16);
      for (int j = 0; j < 4 && i + j < n; ++j) y[i + j] = (uint8_t)(p >> (8 * j));
    }
  }
}

template <typename T>
__global__ void int8_quant_block_kernel(const T* __restrict__ x, int8_t* __restrict__ y, float* __restrict__ scales,
                                        long long n, int block) {
  // one warp per block of `block` elements (block <= 1024)
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long nb = (n + block - 1) / block;
  for (long long b = warp; b < nb; b += nwarps) {
    const long long base = b * block;
    float amax = 0.f;
    for (int j = lane; j < block; j += 32)
      if (base + j < n) amax = fmaxf(amax, fabsf((float)x[base + j]));
    amax = warp_max(amax);
    const float s = fmaxf(amax, 1e-8f) / 127.0f;
    for (int j = lane; j < block; j += 32)
      if (base + j < n) {
        float q = rintf((float)x[base + j] / s);
        q = fminf(fmaxf(q, -127.f), 127.f);
        y[base + j] = (int8_t)q;
      }
    if (lane == 0) scales[b] = s;
  }
}

__device__ __forceinline__ float fp8_to_float(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// mode 0: fp8, scales[w]; mode 1: fp8, scales[w * nb + i / block]; mode 2: int8, scales[w * nb + i / block]
template <typename T>
__global__ void dequant_sum_kernel(const uint8_t* __restrict__ payload, const float* __restrict__ scales,
                                   T* __restrict__ out, int W, long long n, long long slice_stride, int mode,
                                   int block, float out_scale) {
  const long long nb = (n + block - 1) / block;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int w = 0; w < W; ++w) {
      const uint8_t b = payload[w * slice_stride + i];
      const float s = (mode == 0) ? scales[w] : scales[w * nb + i / block];
      acc += ((mode == 2) ? (float)(int8_t)b : fp8_to_float(b)) * s;
    }
    out[i] = (T)(acc * out_scale);
  }
}

static int grid_for(long long items, int threads) {
  long long b = (items + threads - 1) / threads;
  if (b < 1) b = 1;
  return (int)(b > 148 * 16 ? 148 * 16 : b);
}

}  // namespace pkb

using namespace pkb;

extern "C" {

int pkb_fp8_quant_scaled(const void* x, const void* scale_dev, void* y, long long n, int dtype, void* stream) {
  if (n == 0) return kApiOk;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = grid_for((n + 3) / 4, 256);
  if (dtype == 0)
    fp8_quant_scaled_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                               static_cast<const float*>(scale_dev),
                                                               static_cast<uint8_t*>(y), n);
  else
    fp8_quant_scaled_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), static_cast<const float*>(scale_dev),
                                                       static_cast<uint8_t*>(y), n);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_int8_quant_block(const void* x, void* y, void* scales, long long n, int block, int dtype, void* stream) {
  PKB_CHECK_ARG(block >= 1, "block must be positive");
  if (n == 0) return kApiOk;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long nb = (n + block - 1) / block;
  const int grid = grid_for(nb * 32, 256);
  if (dtype == 0)
    int8_quant_block_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                               static_cast<int8_t*>(y), static_cast<float*>(scales), n, block);
  else
    int8_quant_block_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), static_cast<int8_t*>(y),
                                                       static_cast<float*>(scales), n, block);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_dequant_sum(const void* payload, const void* scales, void* out, int W, long long n, long long slice_stride,
                    int mode, int block, float out_scale, int out_dtype, void* stream) {
  PKB_CHECK_ARG(mode >= 0 && mode <= 2 && block >= 1 && W >= 1, "bad dequant_sum arguments");
  if (n == 0) return kApiOk;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n, 256);
  if (out_dtype == 0)
    dequant_sum_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(payload), static_cast<const float*>(scales),
                                                          static_cast<__nv_bfloat16*>(out), W, n, slice_stride, mode, block, out_scale);
  else
    dequant_sum_kernel<float><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(payload), static_cast<const float*>(scales),
                                                  static_cast<float*>(out), W, n, slice_stride, mode, block, out_scale);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

}  // extern "C"
