// Sharded optimiser step fused with the fp8 gradient exchange of an FSDP step.
//
// After the all-to-all of fp8 gradient slices, the owner of a shard holds W payload slices
// ([W, n] e4m3 bytes) and their 1x128 block scales ([W, n/128] fp32). One warp per 128-element
// block then does, without touching memory in between:
//   g = (sum_w dequant(slice_w)) * grad_scale          (the reduce half of the reduce-scatter)
//   AdamW on the fp32 master weights and moments
//   re-quantise the new weights to e4m3 with a fresh 1x128 scale  (what the next all-gather ships)
// In-switch (NVLS) reduction cannot be used for this exchange because every rank's blocks carry
// their own scales. Reference behaviour: reduce_scatter + AdamW on the shard as separate steps, with
// per-tensor delayed scaling (reference: reference/47_fsdp_step_e2e.py:49-65,
// reference/52_fp8_reduce_scatter_grads.py:26-41, reference/53_fp8_allgather_params.py:26-39).
#include <cuda_fp8.h>

#include "pkb/api.h"
#include "pkb/host.h"
#include "pkb/ptx.cuh"

namespace pkb {

struct FsdpAdamArgs {
  const uint8_t* payload;  // [W, n]
  const float* scales;     // [W, n / 128]
  int W;
  long long n;             // shard elements, multiple of 128
  float* p; float* m; float* v;
  uint8_t* q_out;          // [n] new weights as e4m3
  float* s_out;            // [n / 128]
  __nv_bfloat16* p_bf16;   // optional bf16 copy of the new weights
  float lr, beta1, beta2, eps, weight_decay, grad_scale, bias_c1, bias_c2;
};

__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)byte, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

__global__ void __launch_bounds__(256) fsdp_adamw_fp8_kernel(const FsdpAdamArgs a) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long nb = a.n / 128;
  for (long long b = warp; b < nb; b += nwarps) {
    const long long i0 = b * 128 + lane * 4;
    float g[4] = {0.f, 0.f, 0.f, 0.f};
    for (int w = 0; w < a.W; ++w) {
      const uint32_t packed = *reinterpret_cast<const uint32_t*>(a.payload + (long long)w * a.n + i0);
      const float s = a.scales[(long long)w * nb + b];
#pragma unroll
      for (int j = 0; j < 4; ++j) g[j] += e4m3_to_float((packed >> (8 * j)) & 0xffu) * s;
    }
    float wnew[4];
    float amax = 0.f;
    // master weights and moments move as 16-byte vectors (i0 is a multiple of 4 elements)
    const float4 p4 = *reinterpret_cast<const float4*>(a.p + i0);
    const float4 m4 = *reinterpret_cast<const float4*>(a.m + i0);
    const float4 v4 = *reinterpret_cast<const float4*>(a.v + i0);
    const float pin[4] = {p4.x, p4.y, p4.z, p4.w}, min_[4] = {m4.x, m4.y, m4.z, m4.w}, vin[4] = {v4.x, v4.y, v4.z, v4.w};
    float mo[4], vo[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float grad = g[j] * a.grad_scale;
      float w = pin[j] * (1.0f - a.lr * a.weight_decay);
      const float mi = a.beta1 * min_[j] + (1.0f - a.beta1) * grad;
      const float vi = a.beta2 * vin[j] + (1.0f - a.beta2) * grad * grad;
      w -= a.lr * (mi / a.bias_c1) / (sqrtf(vi / a.bias_c2) + a.eps);
      mo[j] = mi; vo[j] = vi;
      wnew[j] = w;
      amax = fmaxf(amax, fabsf(w));
    }
    *reinterpret_cast<float4*>(a.p + i0) = make_float4(wnew[0], wnew[1], wnew[2], wnew[3]);
    *reinterpret_cast<float4*>(a.m + i0) = make_float4(mo[0], mo[1], mo[2], mo[3]);
    *reinterpret_cast<float4*>(a.v + i0) = make_float4(vo[0], vo[1], vo[2], vo[3]);
    if (a.p_bf16) {
      *reinterpret_cast<uint2*>(a.p_bf16 + i0) = make_uint2(pack_bf16x2(wnew[0], wnew[1]), pack_bf16x2(wnew[2], wnew[3]));
    }
    amax = warp_max(amax);
    float s = amax / 448.0f;
    if (s == 0.f) s = 1.0f;
    const float inv = 1.0f / s;
    __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(wnew[0] * inv, wnew[1] * inv), __NV_SATFINITE, __NV_E4M3);
    __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(wnew[2] * inv, wnew[3] * inv), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint32_t*>(a.q_out + i0) = (uint32_t)lo | ((uint32_t)hi << 16);
    if (lane == 0) a.s_out[b] = s;
  }
}

}  // namespace pkb

using namespace pkb;

extern "C" int pkb_fsdp_adamw_fp8(const void* payload, const void* scales, int W, long long n, void* p, void* m,
                                  void* v, void* q_out, void* s_out, void* p_bf16, float lr, float beta1, float beta2,
                                  float eps, float weight_decay, float grad_scale, int step, void* stream) {
  PKB_CHECK_ARG(n % 128 == 0 && W >= 1 && step >= 1, "n must be a multiple of 128, W and step positive");
  if (n == 0) return kApiOk;
  FsdpAdamArgs a{static_cast<const uint8_t*>(payload), static_cast<const float*>(scales), W, n,
                 static_cast<float*>(p), static_cast<float*>(m), static_cast<float*>(v), static_cast<uint8_t*>(q_out),
                 static_cast<float*>(s_out), static_cast<__nv_bfloat16*>(p_bf16), lr, beta1, beta2, eps, weight_decay,
                 grad_scale, 1.0f - powf(beta1, (float)step), 1.0f - powf(beta2, (float)step)};
  long long blocks = (n / 128 * 32 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  fsdp_adamw_fp8_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}
