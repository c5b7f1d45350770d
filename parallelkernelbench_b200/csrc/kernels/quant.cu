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

// ------------------------------------------------------------------------------------------------
// Gradient clipping by global norm without a host round trip: (1) sum of squares of up to eight tensors in one launch,
// (2) [the all-reduce of that scalar], (3) every tensor scaled in place by min(1, max_norm / sqrt(total)) read from device
// memory. The reference computes a norm per tensor, all-reduces, and branches on the host
// (reference: reference/21_clip_grad_norm_no_ep.py:25-50).
// ------------------------------------------------------------------------------------------------
namespace pkb {

constexpr int kClipMaxTensors = 8;
struct ClipArgs {
  void* ptr[kClipMaxTensors];
  long long n[kClipMaxTensors];
  float pre_scale[kClipMaxTensors];   // each tensor is multiplied by this before it is measured (and stays scaled)
  int slot[kClipMaxTensors];          // which accumulator the tensor's sum of squares goes to
  int count;
};

template <typename T>
__global__ void __launch_bounds__(256) clip_sumsq_kernel(const ClipArgs a, float* __restrict__ acc) {
  __shared__ float red[8];
  for (int t = 0; t < a.count; ++t) {
    const T* p = static_cast<const T*>(a.ptr[t]);
    const float ps = a.pre_scale[t];
    float s = 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n[t]; i += (long long)gridDim.x * blockDim.x) {
      const float v = (float)p[i] * ps;
      s += v * v;
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int w = 0; w < 8; ++w) tot += red[w];
      if (tot != 0.f) atomicAdd(acc + a.slot[t], tot);
    }
    __syncthreads();
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
clip_scale_kernel(const ClipArgs a, const float* __restrict__ total_sq, int n_slots, float max_norm, float* __restrict__ total_norm_out) {
  float tot = 0.f;
  for (int s = 0; s < n_slots; ++s) tot += total_sq[s];
  const float norm = sqrtf(tot);
  const float coef = fminf(max_norm / norm, 1.0f);
  if (blockIdx.x == 0 && threadIdx.x == 0 && total_norm_out != nullptr) *total_norm_out = norm;
  for (int t = 0; t < a.count; ++t) {
    T* p = static_cast<T*>(a.ptr[t]);
    const float f = coef * a.pre_scale[t];
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n[t]; i += (long long)gridDim.x * blockDim.x)
      p[i] = (T)((float)p[i] * f);
  }
}

static int fill_clip_args(ClipArgs& a, void* const* ptrs, const long long* ns, const float* pre_scale, const int* slots, int count) {
  PKB_CHECK_ARG(count >= 1 && count <= kClipMaxTensors, "1..8 tensors per call");
  a.count = count;
  for (int i = 0; i < count; ++i) {
    a.ptr[i] = ptrs[i];
    a.n[i] = ns[i];
    a.pre_scale[i] = pre_scale ? pre_scale[i] : 1.0f;
    a.slot[i] = slots ? slots[i] : 0;
  }
  return kApiOk;
}

}  // namespace pkb

// acc (fp32, zero-filled by the caller) receives sum((x * pre_scale)^2) per slot. dtype: 0 bf16, 1 fp32.
extern "C" int pkb_clip_sumsq(void* const* ptrs, const long long* ns, const float* pre_scale, const int* slots, int count, int dtype,
                              void* acc, void* stream) {
  pkb::ClipArgs a;
  if (int rc = pkb::fill_clip_args(a, ptrs, ns, pre_scale, slots, count)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0) pkb::clip_sumsq_kernel<__nv_bfloat16><<<148 * 4, 256, 0, s>>>(a, static_cast<float*>(acc));
  else pkb::clip_sumsq_kernel<float><<<148 * 4, 256, 0, s>>>(a, static_cast<float*>(acc));
  PKB_CHECK_CUDA(cudaGetLastError());
  return pkb::kApiOk;
}

// Every tensor is multiplied in place by pre_scale * min(1, max_norm / sqrt(sum of the n_slots totals)).
extern "C" int pkb_clip_scale(void* const* ptrs, const long long* ns, const float* pre_scale, int count, int dtype, const void* total_sq,
                              int n_slots, float max_norm, void* total_norm_out, void* stream) {
  pkb::ClipArgs a;
  if (int rc = pkb::fill_clip_args(a, ptrs, ns, pre_scale, nullptr, count)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    pkb::clip_scale_kernel<__nv_bfloat16><<<148 * 4, 256, 0, s>>>(a, static_cast<const float*>(total_sq), n_slots, max_norm,
                                                                 static_cast<float*>(total_norm_out));
  else
    pkb::clip_scale_kernel<float><<<148 * 4, 256, 0, s>>>(a, static_cast<const float*>(total_sq), n_slots, max_norm,
                                                         static_cast<float*>(total_norm_out));
  PKB_CHECK_CUDA(cudaGetLastError());
  return pkb::kApiOk;
}
