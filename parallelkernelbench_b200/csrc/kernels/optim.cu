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
#include "pkb/symm.cuh"
#include "pkb/symm_host.h"

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

// One 128-element block per warp iteration, four elements per lane: every access of a warp is coalesced and the kernel runs
// at full occupancy (40 registers). Two wider forms were measured and dropped: 16 consecutive elements per thread (strided
// warp accesses, 307 us against 292 us on the 8-rank profile case) and four blocks per warp iteration with all loads issued
// first (128 registers, a quarter of the occupancy, 585 us).
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
  PKB_CHECK_ARG((((uintptr_t)payload | (uintptr_t)p | (uintptr_t)m | (uintptr_t)v | (uintptr_t)q_out | (uintptr_t)p_bf16) & 15) == 0,
                "buffers must be 16-byte aligned");
  long long blocks = (n / 128 * 32 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  fsdp_adamw_fp8_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// ================================================================================================
// Sharded Adam(W) step with both of its collectives inside: reduce-scatter -> Adam -> all-gather in ONE kernel.
//
// Every rank has written its full gradient (bf16, [gsize * part]) into the symmetric heap. After the entry barrier the
// owner of shard g reads the sum of slice g over all ranks - one `multimem.ld_reduce` per 16 bytes when the group is the
// whole job and the heap has a multicast mapping (the switch adds, fp32 accumulation), else one peer load per member -
// updates its parameters and moments in registers, and stores the new bf16 parameters into the gathered parameter buffer
// of EVERY rank (`multimem.st`, or one peer store per member). The reduced gradient and the updated shard never exist in
// memory as separate tensors, and nothing is launched between the three steps. A closing barrier tells each rank that all
// shards have landed. This is the data-parallel optimiser step of the reference's DDP / ZeRO-1 / ZeRO-2 / fused
// Adam + all-gather workloads (reference: reference/40_ddp_step.py, reference/41_zero1_optimizer_shard.py:50-68,
// reference/42_zero2_optimizer_shard_grad.py:50-67, reference/43_fused_adam_grad_unshard_allgather.py:28-43), which run
// them as reduce-scatter / all-reduce, an optimiser loop and an all-gather.
// ================================================================================================
namespace pkb {

struct ZeroAdamArgs {
  SymmCtx ctx;
  uint64_t grad_off;          // heap offset of the gradient: [gsize * part] bf16 (reduce = 1) or [part] bf16 (reduce = 0)
  int reduce;                 // 1: this rank's slice summed over all members; 0: the local shard gradient as it is
  void* p; void* m; void* v;  // shard state [part], bf16 (state_f32 = 0) or fp32 (state_f32 = 1); updated in place
  int state_f32;
  uint64_t out_off;           // heap offset of the gathered parameters [gsize * part] bf16 on every rank
  int gather;                 // 0: no gather (only the shard state is updated)
  long long part;             // elements per shard, a multiple of 8
  float lr, beta1, beta2, eps, weight_decay, grad_scale, bias_c1, bias_c2;
  int use_mc;
};

__device__ __forceinline__ void load8(const void* base, long long i, int f32, float (&x)[8]) {
  if (f32) {
    const U4 a = ld_global_v4(static_cast<const float*>(base) + i), b = ld_global_v4(static_cast<const float*>(base) + i + 4);
    x[0] = __uint_as_float(a.x); x[1] = __uint_as_float(a.y); x[2] = __uint_as_float(a.z); x[3] = __uint_as_float(a.w);
    x[4] = __uint_as_float(b.x); x[5] = __uint_as_float(b.y); x[6] = __uint_as_float(b.z); x[7] = __uint_as_float(b.w);
  } else {
    const U4 u = ld_global_v4(static_cast<const __nv_bfloat16*>(base) + i);
    const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
    x[0] = f0.x; x[1] = f0.y; x[2] = f1.x; x[3] = f1.y; x[4] = f2.x; x[5] = f2.y; x[6] = f3.x; x[7] = f3.y;
  }
}
__device__ __forceinline__ U4 pack8(const float (&x)[8]) {
  return U4{pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7])};
}
__device__ __forceinline__ void store8(void* base, long long i, int f32, const float (&x)[8]) {
  if (f32) {
    st_global_v4(static_cast<float*>(base) + i, U4{__float_as_uint(x[0]), __float_as_uint(x[1]), __float_as_uint(x[2]), __float_as_uint(x[3])});
    st_global_v4(static_cast<float*>(base) + i + 4, U4{__float_as_uint(x[4]), __float_as_uint(x[5]), __float_as_uint(x[6]), __float_as_uint(x[7])});
  } else {
    st_global_v4(static_cast<__nv_bfloat16*>(base) + i, pack8(x));
  }
}

__global__ void __launch_bounds__(256) zero_adam_allgather_kernel(const ZeroAdamArgs a) {
  const SymmCtx& c = a.ctx;
  // all members have entered this call: their gradients are in the heap and nobody still reads the previous gathered result
  if (!symm_block_barrier(c, 700, 1)) return;
  const long long nvec = a.part >> 3;
  const long long shard0 = (long long)c.grank * a.part;
  for (long long vi = (long long)blockIdx.x * blockDim.x + threadIdx.x; vi < nvec; vi += (long long)gridDim.x * blockDim.x) {
    const long long i = vi << 3;
    float g[8];
    if (!a.reduce) {
      load8(symm_local<__nv_bfloat16>(c, a.grad_off), i, 0, g);
    } else if (a.use_mc) {
      const U4 u = multimem_ld_reduce_bf16x8(symm_mc<__nv_bfloat16>(c, a.grad_off) + shard0 + i);
      const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
      g[0] = f0.x; g[1] = f0.y; g[2] = f1.x; g[3] = f1.y; g[4] = f2.x; g[5] = f2.y; g[6] = f3.x; g[7] = f3.y;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = 0.f;
      for (int k = 0; k < c.gsize; ++k) {       // member order: the sum does not depend on arrival order
        float t[8];
        load8(symm_ptr<__nv_bfloat16>(c, c.members[k], a.grad_off), shard0 + i, 0, t);
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] += t[j];
      }
    }
    float p[8], m[8], v[8];
    load8(a.p, i, a.state_f32, p);
    load8(a.m, i, a.state_f32, m);
    load8(a.v, i, a.state_f32, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float grad = g[j] * a.grad_scale;
      m[j] = a.beta1 * m[j] + (1.0f - a.beta1) * grad;
      v[j] = a.beta2 * v[j] + (1.0f - a.beta2) * grad * grad;
      const float upd = (m[j] / a.bias_c1) / (sqrtf(v[j] / a.bias_c2) + a.eps);
      p[j] = p[j] - a.lr * upd - a.lr * a.weight_decay * p[j];
    }
    store8(a.p, i, a.state_f32, p);
    store8(a.m, i, a.state_f32, m);
    store8(a.v, i, a.state_f32, v);
    if (a.gather) {
      const U4 o = pack8(p);
      if (a.use_mc) {
        multimem_st_v4(symm_mc<__nv_bfloat16>(c, a.out_off) + shard0 + i, o);
      } else {
        for (int k = 0; k < c.gsize; ++k) {
          int gk = c.grank + k;                  // own copy first, peers spread over time
          if (gk >= c.gsize) gk -= c.gsize;
          st_global_v4(symm_ptr<__nv_bfloat16>(c, c.members[gk], a.out_off) + shard0 + i, o);
        }
      }
    }
  }
  // same-index blocks of all members have stored their part of every shard (and finished reading the peers' gradients) once
  // this barrier passes; the kernel ends on a rank only after all of its blocks passed, i.e. after every shard has landed
  // here and no peer still reads this rank's gradient buffer
  if (a.gather || a.reduce) symm_block_barrier(c, 700, 2);
}

}  // namespace pkb

// One optimiser step on this rank's shard of `part` elements (a multiple of 8) with the gradient reduction and the parameter
// gather inside the kernel (see above). grad_off: heap offset of the bf16 gradient ([gsize * part] when reduce != 0, this
// rank's [part] otherwise); p, m, v: local shard state, bf16 or fp32 (state_f32), updated in place; out_off: heap offset of the
// gathered bf16 parameters [gsize * part] (ignored when gather == 0). Decoupled weight decay; `step` counts from 1.
extern "C" int pkb_zero_adam_allgather(const pkb_symm_ctx* h, unsigned long long grad_off, int reduce, void* p, void* m, void* v,
                                       int state_f32, unsigned long long out_off, int gather, long long part, float lr,
                                       float beta1, float beta2, float eps, float weight_decay, float grad_scale, int step,
                                       int allow_multicast, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(part > 0 && part % 8 == 0 && step >= 1, "part must be a positive multiple of 8, step positive");
  PKB_CHECK_ARG((grad_off & 15) == 0 && (out_off & 15) == 0, "heap offsets must be 16-byte aligned");
  PKB_CHECK_ARG(((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15) == 0,
                "shard state must be 16-byte aligned");
  ZeroAdamArgs a;
  a.ctx = symm_ctx_from_api(h);
  a.grad_off = grad_off; a.reduce = reduce ? 1 : 0;
  a.p = p; a.m = m; a.v = v; a.state_f32 = state_f32 ? 1 : 0;
  a.out_off = out_off; a.gather = gather ? 1 : 0; a.part = part;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay; a.grad_scale = grad_scale;
  a.bias_c1 = 1.0f - powf(beta1, (float)step);
  a.bias_c2 = 1.0f - powf(beta2, (float)step);
  a.use_mc = (allow_multicast && h->mc_base != 0 && h->gsize == h->world && h->gsize > 1) ? 1 : 0;
  long long blocks = (part / 8 + 255) / 256;
  int cap = sm_count();                     // the barriers pair blocks by index: every block must be resident
  if (cap > kSymmMaxBlocks) cap = kSymmMaxBlocks;
  if (blocks > cap) blocks = cap;
  zero_adam_allgather_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}
