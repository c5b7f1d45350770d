// Memory-bound kernels around the GEMMs: RoPE, fp8 1x128 block quantise / dequantise, fused
// Adam / AdamW, vocab-parallel cross-entropy statistics, column reductions for the LayerNorm
// backward, and a tensor-parallel RMSNorm whose cross-rank sum runs inside the kernel.
// All use 16-byte global accesses and fp32 arithmetic.
//
// Reference behaviour: reference/17_rope_allgather.py:10-37, reference/19_blocked_fp8_quantize.py:7-23,
// reference/20_blocked_fp8_dequantize.py:6-16, reference/43_fused_adam_grad_unshard_allgather.py:28-40,
// reference/47_fsdp_step_e2e.py:52-65, reference/73_vocab_parallel_cross_entropy_loss.py:21-42,
// reference/9_layernorm_backward.py:6-11, reference/18_tp_rms_norm.py:9-19.
#include <cuda_fp8.h>

#include "pkb/api.h"
#include "pkb/collectives_api.h"
#include "pkb/host.h"
#include "pkb/symm.cuh"

namespace pkb {

constexpr float kInv448 = 1.0f / 448.0f;

// ================================================================================================
// RoPE (rotate-half): x is [tokens, heads, dim]; cos/sin are [tokens, dim] (the two halves of a row
// of cos/sin normally repeat). out[.., :d/2] = x1*cos1 - x2*sin1 ; out[.., d/2:] = x2*cos2 + x1*sin2
// ================================================================================================
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, const T* __restrict__ cs, const T* __restrict__ sn,
                            T* __restrict__ out, long long tokens, int heads, int dim) {
  const int half = dim >> 1;
  const long long total = tokens * heads * half;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(i % half);
    const long long th = i / half;
    const long long t = th / heads;
    const T* xr = x + th * dim;
    const float x1 = (float)xr[j], x2 = (float)xr[j + half];
    const float c1 = (float)cs[t * dim + j], c2 = (float)cs[t * dim + j + half];
    const float s1 = (float)sn[t * dim + j], s2 = (float)sn[t * dim + j + half];
    out[th * dim + j] = (T)(x1 * c1 - x2 * s1);
    out[th * dim + j + half] = (T)(x2 * c2 + x1 * s2);
  }
}

// ================================================================================================
// fp8 e4m3 quantise with one fp32 scale per 128 consecutive elements: s = amax/448 (1 if amax = 0),
// y = sat(x / s). One warp handles one block: 4 elements per lane.
// ================================================================================================
template <typename T>
__device__ __forceinline__ void load16(const T* p, float (&v)[16]);
template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[16]) {
  const U4 u0 = ld_global_nc_v4(p), u1 = ld_global_nc_v4(p + 8);
  const uint32_t w[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float2 f = unpack_bf16x2(w[j]);
    v[2 * j] = f.x; v[2 * j + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load16<float>(const float* p, float (&v)[16]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const U4 u = ld_global_nc_v4(p + 4 * q);
    v[4 * q] = __uint_as_float(u.x); v[4 * q + 1] = __uint_as_float(u.y);
    v[4 * q + 2] = __uint_as_float(u.z); v[4 * q + 3] = __uint_as_float(u.w);
  }
}

// A thread owns 16 consecutive elements (32 or 64 bytes in, one 16-byte store out); the 8 lanes of a 128-element block share
// its maximum through three shuffles. Memory bound: what counts is bytes in flight per thread, not arithmetic.
template <typename T>
__global__ void __launch_bounds__(256) fp8_quant_kernel(const T* __restrict__ x, uint8_t* __restrict__ y, float* __restrict__ scales,
                                                        long long nblocks, int pow2_scales) {
  const long long nthr = nblocks * 8;
  for (long long t0 = (long long)blockIdx.x * blockDim.x; t0 < nthr; t0 += (long long)gridDim.x * blockDim.x) {
    const long long t = t0 + threadIdx.x;      // nthr is a multiple of 8: a group of 8 lanes is active or idle as a whole
    float v[16];
    float amax = 0.f;
    if (t < nthr) {
      load16<T>(x + (t << 4), v);
#pragma unroll
      for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    if (t >= nthr) continue;
    float s = amax * kInv448;   // amax / 448 the way PyTorch evaluates a tensor divided by a Python scalar on the GPU: times the rounded reciprocal
    if (pow2_scales && s > 0.f) s = exp2f(ceilf(log2f(s)));  // power-of-two scale (exact to undo)
    if (s == 0.f) s = 1.0f;
    // the correctly rounded quotient x / s, not x * (1 / s): the quotient decides the e4m3 code at rounding boundaries, and
    // x / s is what the PyTorch formulation computes. One reciprocal per block, then per element a product, its residual
    // and one correction (three FMA-pipe instructions instead of a division each).
    const float inv = __frcp_rn(s);
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(div_rn_by(v[4 * j], s, inv), div_rn_by(v[4 * j + 1], s, inv)), __NV_SATFINITE, __NV_E4M3);
      const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(div_rn_by(v[4 * j + 2], s, inv), div_rn_by(v[4 * j + 3], s, inv)), __NV_SATFINITE, __NV_E4M3);
      o[j] = (uint32_t)lo | ((uint32_t)hi << 16);
    }
    st_global_v4(y + (t << 4), U4{o[0], o[1], o[2], o[3]});
    if ((t & 7) == 0) scales[t >> 3] = s;
  }
}

// A thread owns 16 consecutive e4m3 values (one 16-byte load, 32 or 64 bytes out as 16-byte stores); 8 threads share a block's
// scale. `valid_rows` (device, may be null): rows at and beyond *valid_rows of a [rows, blocks_per_row * 128] buffer are left
// alone - a receive buffer sized for the worst case is only dequantised as far as it was filled.
template <typename T>
__global__ void __launch_bounds__(256) fp8_dequant_kernel(const uint8_t* __restrict__ y, const float* __restrict__ scales,
                                                          T* __restrict__ x, long long nblocks, const int* __restrict__ valid_rows,
                                                          long long blocks_per_row) {
  long long nb = nblocks;
  if (valid_rows != nullptr) {
    const long long lim = (long long)(*valid_rows) * blocks_per_row;
    if (lim < nb) nb = lim;
  }
  const long long nthr = nb * 8;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < nthr; t += (long long)gridDim.x * blockDim.x) {
    const U4 u = ld_global_nc_v4(y + (t << 4));
    const float sc = scales[t >> 3];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    float v[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __half2_raw h0 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[j] & 0xffffu), __NV_E4M3);
      __half2_raw h1 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[j] >> 16), __NV_E4M3);
      const float2 f0 = __half22float2(*reinterpret_cast<__half2*>(&h0));
      const float2 f1 = __half22float2(*reinterpret_cast<__half2*>(&h1));
      v[4 * j] = f0.x * sc; v[4 * j + 1] = f0.y * sc; v[4 * j + 2] = f1.x * sc; v[4 * j + 3] = f1.y * sc;
    }
    T* o = x + (t << 4);
    if constexpr (sizeof(T) == 2) {
      st_global_v4(o, U4{pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7])});
      st_global_v4(o + 8, U4{pack_bf16x2(v[8], v[9]), pack_bf16x2(v[10], v[11]), pack_bf16x2(v[12], v[13]), pack_bf16x2(v[14], v[15])});
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        st_global_v4(o + 4 * q, U4{__float_as_uint(v[4 * q]), __float_as_uint(v[4 * q + 1]), __float_as_uint(v[4 * q + 2]),
                                   __float_as_uint(v[4 * q + 3])});
    }
  }
}

// ================================================================================================
// Adam / AdamW on fp32 master weights. grad is fp32 or bf16 and is multiplied by grad_scale first.
// decoupled = 1: AdamW (p *= 1 - lr*wd before the update); 0: L2 folded into the gradient.
// Optionally writes a bf16 copy of the new parameters (what the next forward consumes).
// ================================================================================================
struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, grad_scale, bias_c1, bias_c2;
  int decoupled;
};

template <typename G>
__global__ void adam_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                            const G* __restrict__ g, __nv_bfloat16* __restrict__ p_bf16, long long n, AdamArgs a) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float grad = (float)g[i] * a.grad_scale;
    float w = p[i];
    if (a.decoupled) w *= (1.0f - a.lr * a.weight_decay);
    else grad += a.weight_decay * w;
    const float mi = a.beta1 * m[i] + (1.0f - a.beta1) * grad;
    const float vi = a.beta2 * v[i] + (1.0f - a.beta2) * grad * grad;
    const float mhat = mi / a.bias_c1;
    const float vhat = vi / a.bias_c2;
    w -= a.lr * mhat / (sqrtf(vhat) + a.eps);
    p[i] = w; m[i] = mi; v[i] = vi;
    if (p_bf16) p_bf16[i] = __float2bfloat16_rn(w);
  }
}

// ================================================================================================
// Vocab-parallel cross-entropy, local pass: per row of this rank's logit shard emit
// {local max, sum exp(x - local max), target logit (0 if the target lives on another rank)}.
// The three values of all ranks are then combined (tiny all-gather) by ce_finalize_kernel.
// ================================================================================================
template <typename T>
__global__ void ce_stats_kernel(const T* __restrict__ logits, const long long* __restrict__ target,
                                float* __restrict__ stats, int rows, int vocab_local, long long vocab_start) {
  __shared__ float red[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* lr = logits + (long long)row * vocab_local;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < vocab_local; i += blockDim.x) mx = fmaxf(mx, (float)lr[i]);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = -INFINITY;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float se = 0.f;
    for (int i = threadIdx.x; i < vocab_local; i += blockDim.x) se += __expf((float)lr[i] - mx);
    se = warp_sum(se);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = se;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
      const long long t = target[row] - vocab_start;
      stats[row * 3 + 0] = mx;
      stats[row * 3 + 1] = tot;
      stats[row * 3 + 2] = (t >= 0 && t < vocab_local) ? (float)lr[t] : 0.f;
    }
    __syncthreads();
  }
}

// stats_all is [W, rows, 3]; loss[row] = log(sum_w se_w * exp(mx_w - gmax)) + gmax - sum_w tgt_w
__global__ void ce_finalize_kernel(const float* __restrict__ stats_all, float* __restrict__ loss, int rows, int world) {
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < rows; row += gridDim.x * blockDim.x) {
    float gmax = -INFINITY;
    for (int w = 0; w < world; ++w) gmax = fmaxf(gmax, stats_all[((long long)w * rows + row) * 3]);
    float se = 0.f, tgt = 0.f;
    for (int w = 0; w < world; ++w) {
      const float* s = stats_all + ((long long)w * rows + row) * 3;
      se += s[1] * __expf(s[0] - gmax);
      tgt += s[2];
    }
    loss[row] = logf(se) + gmax - tgt;
  }
}

// ================================================================================================
// Column reductions of the LayerNorm backward: dgamma[c] = sum_r dY[r,c] * Xhat[r,c], dbeta[c] = sum_r dY[r,c]
// One block per 32-column strip; 32 x 8 threads walk the rows, shared-memory finish. fp32 output.
// ================================================================================================
template <typename T>
__global__ void ln_bwd_colreduce_kernel(const T* __restrict__ xhat, const T* __restrict__ dy,
                                        float* __restrict__ dgamma, float* __restrict__ dbeta, int rows, int cols) {
  __shared__ float sg[8][33], sb[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float g = 0.f, b = 0.f;
  if (c < cols) {
    for (int r = threadIdx.y; r < rows; r += 8) {
      const float d = (float)dy[(long long)r * cols + c];
      g += d * (float)xhat[(long long)r * cols + c];
      b += d;
    }
  }
  sg[threadIdx.y][threadIdx.x] = g;
  sb[threadIdx.y][threadIdx.x] = b;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    for (int k = 1; k < 8; ++k) { g += sg[k][threadIdx.x]; b += sb[k][threadIdx.x]; }
    dgamma[c] = g;
    dbeta[c] = b;
  }
}

// ================================================================================================
// Tensor-parallel RMSNorm (hidden dimension sharded): every block owns a set of rows on every rank,
// publishes their local sums of squares in the symmetric heap, crosses ONE in-kernel barrier with the
// same-index blocks of the peers, adds the peers' partial sums and normalises. One launch, no NCCL.
// ================================================================================================
struct TpRmsArgs {
  const __nv_bfloat16* x;
  const __nv_bfloat16* gamma;
  __nv_bfloat16* y;
  int rows, cols_local;
  long long cols_total;
  float eps;
  uint64_t sums_off;  // heap offset of fp32 [rows] partial sums
};

__global__ void __launch_bounds__(256) tp_rmsnorm_kernel(const SymmCtx c, const TpRmsArgs a) {
  __shared__ float red[8];
  float* my_sums = symm_local<float>(c, a.sums_off);
  const int rows_per_block = (a.rows + gridDim.x - 1) / gridDim.x;
  const int r0 = blockIdx.x * rows_per_block;
  const int r1 = min(a.rows, r0 + rows_per_block);
  for (int row = r0; row < r1; ++row) {
    const __nv_bfloat16* xr = a.x + (long long)row * a.cols_local;
    float ss = 0.f;
    for (int i = threadIdx.x * 8; i < a.cols_local; i += blockDim.x * 8) {
      U4 u = ld_global_v4(xr + i);
      float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
      ss += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y + f2.x * f2.x + f2.y * f2.y + f3.x * f3.x + f3.y * f3.y;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
      my_sums[row] = t;
    }
    __syncthreads();
  }
  if (!symm_block_barrier(c, 400, 1)) return;
  for (int row = r0; row < r1; ++row) {
    float tot = 0.f;
    for (int g = 0; g < c.gsize; ++g) tot += symm_ptr<float>(c, c.members[g], a.sums_off)[row];
    const float rstd = rsqrtf(tot / (float)a.cols_total + a.eps);
    const __nv_bfloat16* xr = a.x + (long long)row * a.cols_local;
    __nv_bfloat16* yr = a.y + (long long)row * a.cols_local;
    for (int i = threadIdx.x * 8; i < a.cols_local; i += blockDim.x * 8) {
      U4 u = ld_global_v4(xr + i), g = ld_global_v4(a.gamma + i);
      float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
      float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z), g3 = unpack_bf16x2(g.w);
      U4 o{pack_bf16x2(f0.x * rstd * g0.x, f0.y * rstd * g0.y), pack_bf16x2(f1.x * rstd * g1.x, f1.y * rstd * g1.y),
           pack_bf16x2(f2.x * rstd * g2.x, f2.y * rstd * g2.y), pack_bf16x2(f3.x * rstd * g3.x, f3.y * rstd * g3.y)};
      st_global_v4(yr + i, o);
    }
  }
  // the sums buffer is rewritten by the next call: peers must have read it first
  symm_block_barrier(c, 400, 2);
}

static int grid_1d(long long work_items, int threads, int max_blocks = 148 * 8) {
  long long b = (work_items + threads - 1) / threads;
  if (b < 1) b = 1;
  return (int)(b > max_blocks ? max_blocks : b);
}

static SymmCtx ctx_of(const pkb_symm_ctx* h) {
  SymmCtx c;
  c.base = h->base; c.stride = h->stride; c.mc_base = h->mc_base;
  c.rank = h->rank; c.world = h->world; c.gsize = h->gsize; c.grank = h->grank;
  for (int i = 0; i < kSymmMaxWorld; ++i) c.members[i] = h->members[i];
  c.channel = h->channel;
  c.status = status_block_device_ptr();
  c.budget_ns = h->budget_ns ? h->budget_ns : kDefaultWaitBudgetNs;
  return c;
}

}  // namespace pkb

using namespace pkb;

extern "C" {

// dtype: 0 bf16, 1 fp32
int pkb_rope(const void* x, const void* cos_t, const void* sin_t, void* out, long long tokens, int heads,
             int dim, int dtype, void* stream) {
  PKB_CHECK_ARG(dim % 2 == 0 && tokens >= 0 && heads > 0, "bad RoPE shape");
  if (tokens == 0) return kApiOk;
  const long long total = tokens * heads * (dim / 2);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    rope_kernel<__nv_bfloat16><<<grid_1d(total, 256), 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(cos_t),
        static_cast<const __nv_bfloat16*>(sin_t), static_cast<__nv_bfloat16*>(out), tokens, heads, dim);
  else
    rope_kernel<float><<<grid_1d(total, 256), 256, 0, s>>>(static_cast<const float*>(x), static_cast<const float*>(cos_t),
                                                        static_cast<const float*>(sin_t), static_cast<float*>(out),
                                                        tokens, heads, dim);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_fp8_quant_1x128(const void* x, void* y, void* scales, long long n, int dtype, int pow2_scales, void* stream) {
  PKB_CHECK_ARG(n % 128 == 0, "element count must be a multiple of 128");
  if (n == 0) return kApiOk;
  const long long nb = n / 128;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  PKB_CHECK_ARG(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0, "input and payload must be 16-byte aligned");
  const int grid = grid_1d(nb * 8, 256);
  if (dtype == 0)
    fp8_quant_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(y),
                                                        static_cast<float*>(scales), nb, pow2_scales);
  else
    fp8_quant_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), static_cast<uint8_t*>(y),
                                                static_cast<float*>(scales), nb, pow2_scales);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

static int launch_fp8_dequant(const void* y, const void* scales, void* x, long long n, int dtype, const int* valid_rows,
                              long long blocks_per_row, void* stream) {
  PKB_CHECK_ARG(n % 128 == 0, "element count must be a multiple of 128");
  PKB_CHECK_ARG((((uintptr_t)y | (uintptr_t)x) & 15) == 0, "buffers must be 16-byte aligned");
  if (n == 0) return kApiOk;
  const long long nb = n / 128;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = grid_1d(nb * 8, 256);
  if (dtype == 0)
    fp8_dequant_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(y), static_cast<const float*>(scales),
                                                          static_cast<__nv_bfloat16*>(x), nb, valid_rows, blocks_per_row);
  else
    fp8_dequant_kernel<float><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(y), static_cast<const float*>(scales),
                                                  static_cast<float*>(x), nb, valid_rows, blocks_per_row);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_fp8_dequant_1x128(const void* y, const void* scales, void* x, long long n, int dtype, void* stream) {
  return launch_fp8_dequant(y, scales, x, n, dtype, nullptr, 0, stream);
}

// The same for a [rows, cols] buffer of which only the first *valid_rows rows (an int32 in device memory) hold data.
int pkb_fp8_dequant_1x128_rows(const void* y, const void* scales, void* x, long long rows, long long cols, int dtype,
                               const void* valid_rows, void* stream) {
  PKB_CHECK_ARG(cols % 128 == 0 && valid_rows != nullptr, "cols must be a multiple of 128 and valid_rows given");
  return launch_fp8_dequant(y, scales, x, rows * cols, dtype, static_cast<const int*>(valid_rows), cols / 128, stream);
}

int pkb_adam(void* p, void* m, void* v, const void* g, void* p_bf16, long long n, int grad_dtype, float lr,
             float beta1, float beta2, float eps, float weight_decay, float grad_scale, int step, int decoupled,
             void* stream) {
  PKB_CHECK_ARG(step >= 1, "step counts from 1");
  if (n == 0) return kApiOk;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, grad_scale, 1.0f - powf(beta1, (float)step),
             1.0f - powf(beta2, (float)step), decoupled};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = grid_1d(n, 256);
  if (grad_dtype == 0)
    adam_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<float*>(p), static_cast<float*>(m), static_cast<float*>(v),
                                                   static_cast<const __nv_bfloat16*>(g),
                                                   static_cast<__nv_bfloat16*>(p_bf16), n, a);
  else
    adam_kernel<float><<<grid, 256, 0, s>>>(static_cast<float*>(p), static_cast<float*>(m), static_cast<float*>(v),
                                           static_cast<const float*>(g), static_cast<__nv_bfloat16*>(p_bf16), n, a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_ce_stats(const void* logits, const void* target, void* stats, int rows, int vocab_local,
                 long long vocab_start, int dtype, void* stream) {
  if (rows == 0) return kApiOk;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  if (dtype == 0)
    ce_stats_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(logits),
                                                       static_cast<const long long*>(target),
                                                       static_cast<float*>(stats), rows, vocab_local, vocab_start);
  else
    ce_stats_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(logits), static_cast<const long long*>(target),
                                               static_cast<float*>(stats), rows, vocab_local, vocab_start);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_ce_finalize(const void* stats_all, void* loss, int rows, int world, void* stream) {
  if (rows == 0) return kApiOk;
  ce_finalize_kernel<<<grid_1d(rows, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(stats_all), static_cast<float*>(loss), rows, world);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_ln_bwd_colreduce(const void* xhat, const void* dy, void* dgamma, void* dbeta, int rows, int cols,
                         int dtype, void* stream) {
  if (cols == 0) return kApiOk;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 block(32, 8);
  const int grid = (cols + 31) / 32;
  if (dtype == 0)
    ln_bwd_colreduce_kernel<__nv_bfloat16><<<grid, block, 0, s>>>(static_cast<const __nv_bfloat16*>(xhat),
                                                                 static_cast<const __nv_bfloat16*>(dy),
                                                                 static_cast<float*>(dgamma), static_cast<float*>(dbeta),
                                                                 rows, cols);
  else
    ln_bwd_colreduce_kernel<float><<<grid, block, 0, s>>>(static_cast<const float*>(xhat), static_cast<const float*>(dy),
                                                         static_cast<float*>(dgamma), static_cast<float*>(dbeta), rows, cols);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_tp_rmsnorm(const pkb_symm_ctx* h, const void* x, const void* gamma, void* y, int rows, int cols_local,
                   long long cols_total, float eps, unsigned long long sums_off, void* stream) {
  PKB_CHECK_ARG(h && h->base, "symmetric heap not initialised");
  PKB_CHECK_ARG(cols_local % 8 == 0 && rows > 0, "cols_local must be a multiple of 8");
  TpRmsArgs a{static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gamma),
              static_cast<__nv_bfloat16*>(y), rows, cols_local, cols_total, eps, sums_off};
  int grid = rows < 148 ? rows : 148;
  tp_rmsnorm_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(ctx_of(h), a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

}  // extern "C"
