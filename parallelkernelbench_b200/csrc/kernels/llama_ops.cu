// Elementwise and row-wise kernels of the decoder layer that are not GEMMs: SwiGLU forward / backward and the RMSNorm
// backward. Each is one pass over its tensors with 16-byte accesses (the framework's autograd would run five to eight
// passes over the [tokens, 2 * ffn] activation). Used by the FSDP Llama step.
#include "pkb/api.h"
#include "pkb/host.h"
#include "pkb/ptx.cuh"

namespace pkb {

// gu: [rows, 2F] bf16 (gate | up); a: [rows, F] = silu(gate) * up
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ a, long long rows, int F) {
  const long long vec_per_row = F / 8;
  const long long total = rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const long long c = (i - r * vec_per_row) * 8;
    const U4 g4 = ld_global_v4(gu + r * 2 * F + c), u4 = ld_global_v4(gu + r * 2 * F + F + c);
    const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = unpack_bf16x2(gw[j]), u = unpack_bf16x2(uw[j]);
      o[j] = pack_bf16x2(silu_f(g.x) * u.x, silu_f(g.y) * u.y);
    }
    st_global_v4(a + r * F + c, U4{o[0], o[1], o[2], o[3]});
  }
}

// dgate = da * up * s * (1 + gate * (1 - s)), dup = da * gate * s, with s = sigmoid(gate)
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ da,
                  __nv_bfloat16* __restrict__ dgu, long long rows, int F) {
  const long long vec_per_row = F / 8;
  const long long total = rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const long long c = (i - r * vec_per_row) * 8;
    const U4 g4 = ld_global_v4(gu + r * 2 * F + c), u4 = ld_global_v4(gu + r * 2 * F + F + c), d4 = ld_global_v4(da + r * F + c);
    const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w}, dw[4] = {d4.x, d4.y, d4.z, d4.w};
    uint32_t og[4], ou[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = unpack_bf16x2(gw[j]), u = unpack_bf16x2(uw[j]), d = unpack_bf16x2(dw[j]);
      const float s0 = 1.f / (1.f + __expf(-g.x)), s1 = 1.f / (1.f + __expf(-g.y));
      og[j] = pack_bf16x2(d.x * u.x * s0 * (1.f + g.x * (1.f - s0)), d.y * u.y * s1 * (1.f + g.y * (1.f - s1)));
      ou[j] = pack_bf16x2(d.x * g.x * s0, d.y * g.y * s1);
    }
    st_global_v4(dgu + r * 2 * F + c, U4{og[0], og[1], og[2], og[3]});
    st_global_v4(dgu + r * 2 * F + F + c, U4{ou[0], ou[1], ou[2], ou[3]});
  }
}

// RMSNorm backward. y = x * rstd * gamma:  dxhat = dy * gamma ;  dx = rstd * (dxhat - xhat * mean(dxhat * xhat)) ;
// dgamma = sum_rows dy * xhat. One block walks several rows and keeps its dgamma partial sums in registers (each thread
// owns fixed columns), then adds them to the fp32 result with one atomic per column.
template <int COLS_PER_THREAD>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                   const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx, float* __restrict__ dgamma,
                   int rows, int H, float eps) {
  __shared__ float red[2][8];
  float gam[COLS_PER_THREAD], dg[COLS_PER_THREAD];
#pragma unroll
  for (int j = 0; j < COLS_PER_THREAD; ++j) {
    const int c = threadIdx.x + j * 256;
    gam[j] = c < H ? __bfloat162float(gamma[c]) : 0.f;
    dg[j] = 0.f;
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + (long long)row * H;
    const __nv_bfloat16* dyr = dy + (long long)row * H;
    float xv[COLS_PER_THREAD], dv[COLS_PER_THREAD];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int j = 0; j < COLS_PER_THREAD; ++j) {
      const int c = threadIdx.x + j * 256;
      xv[j] = c < H ? __bfloat162float(xr[c]) : 0.f;
      dv[j] = c < H ? __bfloat162float(dyr[c]) : 0.f;
      ss += xv[j] * xv[j];
      dot += dv[j] * gam[j] * xv[j];
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = ss; red[1][threadIdx.x >> 5] = dot; }
    __syncthreads();
    float tss = 0.f, tdot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { tss += red[0][w]; tdot += red[1][w]; }
    __syncthreads();
    const float rstd = rsqrtf(tss / (float)H + eps);
    const float mean_term = tdot * rstd / (float)H;      // mean(dxhat * xhat), xhat = x * rstd
#pragma unroll
    for (int j = 0; j < COLS_PER_THREAD; ++j) {
      const int c = threadIdx.x + j * 256;
      if (c < H) {
        const float xhat = xv[j] * rstd;
        dx[(long long)row * H + c] = __float2bfloat16_rn(rstd * (dv[j] * gam[j] - xhat * mean_term));
        dg[j] += dv[j] * xhat;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < COLS_PER_THREAD; ++j) {
    const int c = threadIdx.x + j * 256;
    if (c < H) atomicAdd(dgamma + c, dg[j]);
  }
}

// d logits of the mean cross-entropy over a vocabulary shard: (exp(logit - lse) - [col == target - vocab_start]) * scale,
// written as bf16 in one pass (lse is the GLOBAL log-sum-exp of the row, natural log).
__global__ void __launch_bounds__(256)
ce_bwd_kernel(const __nv_bfloat16* __restrict__ logits, const float* __restrict__ lse, const long long* __restrict__ target,
              __nv_bfloat16* __restrict__ dlog, long long rows, int V, long long vocab_start, float scale,
              const float* __restrict__ upstream) {
  if (upstream != nullptr) scale *= *upstream;     // gradient of the loss itself, kept on the device
  const long long vec_per_row = V / 8;
  const long long total = rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = (int)(i - r * vec_per_row) * 8;
    const float l = lse[r];
    const long long t = target[r] - vocab_start;
    const U4 v = ld_global_v4(logits + r * V + c);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(w[j]);
      const float a = (__expf(f.x - l) - ((long long)(c + 2 * j) == t ? 1.f : 0.f)) * scale;
      const float b = (__expf(f.y - l) - ((long long)(c + 2 * j + 1) == t ? 1.f : 0.f)) * scale;
      o[j] = pack_bf16x2(a, b);
    }
    st_global_v4(dlog + r * V + c, U4{o[0], o[1], o[2], o[3]});
  }
}

}  // namespace pkb

using namespace pkb;

extern "C" int pkb_ce_bwd(const void* logits, const void* lse, const void* target, void* dlog, long long rows, int V,
                          long long vocab_start, float scale, const void* upstream, void* stream) {
  PKB_CHECK_ARG(rows >= 0 && V > 0 && V % 8 == 0, "the vocabulary shard must be a positive multiple of 8");
  if (rows == 0) return kApiOk;
  long long blocks = (rows * (V / 8) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  ce_bwd_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), static_cast<const float*>(lse), static_cast<const long long*>(target),
      static_cast<__nv_bfloat16*>(dlog), rows, V, vocab_start, scale, static_cast<const float*>(upstream));
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

extern "C" int pkb_swiglu_fwd(const void* gu, void* a, long long rows, int F, void* stream) {
  PKB_CHECK_ARG(rows >= 0 && F > 0 && F % 8 == 0, "F must be a positive multiple of 8");
  if (rows == 0) return kApiOk;
  long long blocks = (rows * (F / 8) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  swiglu_fwd_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(gu),
                                                                                static_cast<__nv_bfloat16*>(a), rows, F);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

extern "C" int pkb_swiglu_bwd(const void* gu, const void* da, void* dgu, long long rows, int F, void* stream) {
  PKB_CHECK_ARG(rows >= 0 && F > 0 && F % 8 == 0, "F must be a positive multiple of 8");
  if (rows == 0) return kApiOk;
  long long blocks = (rows * (F / 8) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  swiglu_bwd_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(da), static_cast<__nv_bfloat16*>(dgu), rows, F);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// dgamma (fp32 [H]) must be zero-filled by the caller.
extern "C" int pkb_rmsnorm_bwd(const void* x, const void* gamma, const void* dy, void* dx, void* dgamma, int rows, int H,
                               float eps, void* stream) {
  PKB_CHECK_ARG(rows >= 0 && H > 0 && H <= 256 * 32, "hidden size must be at most 8192");
  if (rows == 0) return kApiOk;
  int blocks = rows < 148 * 4 ? rows : 148 * 4;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16 *xp = static_cast<const __nv_bfloat16*>(x), *gp = static_cast<const __nv_bfloat16*>(gamma),
                      *dyp = static_cast<const __nv_bfloat16*>(dy);
  __nv_bfloat16* dxp = static_cast<__nv_bfloat16*>(dx);
  float* dgp = static_cast<float*>(dgamma);
  if (H <= 256 * 4) rmsnorm_bwd_kernel<4><<<blocks, 256, 0, s>>>(xp, gp, dyp, dxp, dgp, rows, H, eps);
  else if (H <= 256 * 16) rmsnorm_bwd_kernel<16><<<blocks, 256, 0, s>>>(xp, gp, dyp, dxp, dgp, rows, H, eps);
  else rmsnorm_bwd_kernel<32><<<blocks, 256, 0, s>>>(xp, gp, dyp, dxp, dgp, rows, H, eps);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}
