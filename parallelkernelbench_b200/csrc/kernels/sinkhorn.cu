// Sinkhorn-Knopp normalisation of exp(t / temp), t [B, P] fp32 with the batch B sharded over the ranks
// (reference: reference/80_dinov2_distributed_sinkhorn_knopp.py:16-35).
//
// The reference rewrites the whole P x B matrix four times per iteration (divide by the row sums, by P, by the column sums,
// by the batch size). The iterations only ever scale rows and columns, so the matrix itself never has to exist: a scale
// r[p] per prototype and a scale c[b] per sample carry the state, every pass recomputes exp(t / temp) from t on the fly, and
// the result is written once at the end:
//   sinkhorn_rowdot_kernel   v[b] = sum_p exp(t[b,p] / temp) r[p]          one block per sample, fixed summation order
//   sinkhorn_coldot_kernel   u[s][p] = sum_{b in split s} exp(t[b,p] / temp) c[b]   partial sums per row split; the caller
//                            adds the splits (a fixed order again) and all-reduces the P-vector across ranks
//   sinkhorn_scale_kernel    out[b,p] = exp(t[b,p] / temp) r[p] c[b]
// Each pass streams t once (16-byte loads when P is a multiple of four); the exponentials are a small fraction of the time a
// pass spends on memory.
#include "pkb/api.h"
#include "pkb/host.h"

namespace pkb {

constexpr int kSkThreads = 256;

template <bool VEC4>
__global__ void __launch_bounds__(kSkThreads)
sinkhorn_rowdot_kernel(const float* __restrict__ t, const float* __restrict__ r, float* __restrict__ v, int B, int P, float inv_temp) {
  __shared__ float part[kSkThreads / 32];
  for (int b = blockIdx.x; b < B; b += gridDim.x) {
    const float* row = t + (long long)b * P;
    float acc = 0.f;
    if constexpr (VEC4) {
      for (int p = threadIdx.x * 4; p < P; p += kSkThreads * 4) {
        const float4 x = *reinterpret_cast<const float4*>(row + p);
        const float4 s = *reinterpret_cast<const float4*>(r + p);
        acc += expf(x.x * inv_temp) * s.x + expf(x.y * inv_temp) * s.y + expf(x.z * inv_temp) * s.z + expf(x.w * inv_temp) * s.w;
      }
    } else {
      for (int p = threadIdx.x; p < P; p += kSkThreads) acc += expf(row[p] * inv_temp) * r[p];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < kSkThreads / 32; ++i) s += part[i];
      v[b] = s;
    }
    __syncthreads();   // part is reused by the block's next row
  }
}

// grid = (column groups, row splits); partial [splits, P]
template <bool VEC4>
__global__ void __launch_bounds__(kSkThreads)
sinkhorn_coldot_kernel(const float* __restrict__ t, const float* __restrict__ c, float* __restrict__ partial, int B, int P,
                       int rows_per_split, float inv_temp) {
  constexpr int kCols = VEC4 ? 4 : 1;
  const int p = (blockIdx.x * kSkThreads + threadIdx.x) * kCols;
  if (p >= P) return;
  const int b0 = blockIdx.y * rows_per_split;
  const int b1 = min(B, b0 + rows_per_split);
  if constexpr (VEC4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int b = b0; b < b1; ++b) {
      const float4 x = *reinterpret_cast<const float4*>(t + (long long)b * P + p);
      const float cb = c[b];
      acc.x += expf(x.x * inv_temp) * cb;
      acc.y += expf(x.y * inv_temp) * cb;
      acc.z += expf(x.z * inv_temp) * cb;
      acc.w += expf(x.w * inv_temp) * cb;
    }
    *reinterpret_cast<float4*>(partial + (long long)blockIdx.y * P + p) = acc;
  } else {
    float acc = 0.f;
    for (int b = b0; b < b1; ++b) acc += expf(t[(long long)b * P + p] * inv_temp) * c[b];
    partial[(long long)blockIdx.y * P + p] = acc;
  }
}

template <bool VEC4>
__global__ void __launch_bounds__(kSkThreads)
sinkhorn_scale_kernel(const float* __restrict__ t, const float* __restrict__ r, const float* __restrict__ c, float* __restrict__ out,
                      long long total, int P, float inv_temp) {
  constexpr int kCols = VEC4 ? 4 : 1;
  const long long stride = (long long)gridDim.x * kSkThreads * kCols;
  for (long long e = ((long long)blockIdx.x * kSkThreads + threadIdx.x) * kCols; e < total; e += stride) {
    const long long b = e / P;
    const int p = (int)(e - b * P);
    const float cb = c[b];
    if constexpr (VEC4) {
      const float4 x = *reinterpret_cast<const float4*>(t + e);
      const float4 s = *reinterpret_cast<const float4*>(r + p);
      float4 o;
      o.x = expf(x.x * inv_temp) * s.x * cb;
      o.y = expf(x.y * inv_temp) * s.y * cb;
      o.z = expf(x.z * inv_temp) * s.z * cb;
      o.w = expf(x.w * inv_temp) * s.w * cb;
      *reinterpret_cast<float4*>(out + e) = o;
    } else {
      out[e] = expf(t[e] * inv_temp) * r[p] * cb;
    }
  }
}

static bool sk_aligned16(const void* a, const void* b = nullptr, const void* c = nullptr) {
  return reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(b) % 16 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0;
}

}  // namespace pkb

using namespace pkb;

#define PKB_SK_SHAPE_CHECK()                                                                                              \
  PKB_CHECK_ARG(B >= 1 && P >= 1 && (long long)B * P <= (1ll << 40), "need 1 <= B, 1 <= P");                              \
  PKB_CHECK_ARG(temp > 0.0, "the temperature must be positive")

extern "C" int pkb_sinkhorn_rowdot(const void* t, const void* r, void* v, int B, int P, double temp, void* stream) {
  PKB_SK_SHAPE_CHECK();
  PKB_CHECK_ARG(t != nullptr && r != nullptr && v != nullptr, "null tensor");
  const float inv = (float)(1.0 / temp);
  const int grid = B < sm_count() * 8 ? B : sm_count() * 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float *tp = static_cast<const float*>(t), *rp = static_cast<const float*>(r);
  if (P % 4 == 0 && sk_aligned16(t, r)) sinkhorn_rowdot_kernel<true><<<grid, kSkThreads, 0, st>>>(tp, rp, static_cast<float*>(v), B, P, inv);
  else sinkhorn_rowdot_kernel<false><<<grid, kSkThreads, 0, st>>>(tp, rp, static_cast<float*>(v), B, P, inv);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// partial is [splits, P]; rows_per_split * splits >= B
extern "C" int pkb_sinkhorn_coldot(const void* t, const void* c, void* partial, int B, int P, int splits, double temp, void* stream) {
  PKB_SK_SHAPE_CHECK();
  PKB_CHECK_ARG(t != nullptr && c != nullptr && partial != nullptr, "null tensor");
  PKB_CHECK_ARG(splits >= 1 && splits <= 65535 && splits <= B, "need 1 <= splits <= min(B, 65535)");
  const float inv = (float)(1.0 / temp);
  const int rows_per_split = (B + splits - 1) / splits;
  PKB_CHECK_ARG((long long)(splits - 1) * rows_per_split < B, "a split would be empty: choose fewer splits");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float *tp = static_cast<const float*>(t), *cp = static_cast<const float*>(c);
  if (P % 4 == 0 && sk_aligned16(t, partial)) {
    const dim3 grid((P / 4 + kSkThreads - 1) / kSkThreads, splits);
    sinkhorn_coldot_kernel<true><<<grid, kSkThreads, 0, st>>>(tp, cp, static_cast<float*>(partial), B, P, rows_per_split, inv);
  } else {
    const dim3 grid((P + kSkThreads - 1) / kSkThreads, splits);
    sinkhorn_coldot_kernel<false><<<grid, kSkThreads, 0, st>>>(tp, cp, static_cast<float*>(partial), B, P, rows_per_split, inv);
  }
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

extern "C" int pkb_sinkhorn_scale(const void* t, const void* r, const void* c, void* out, int B, int P, double temp, void* stream) {
  PKB_SK_SHAPE_CHECK();
  PKB_CHECK_ARG(t != nullptr && r != nullptr && c != nullptr && out != nullptr, "null tensor");
  const float inv = (float)(1.0 / temp);
  const long long total = (long long)B * P;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float *tp = static_cast<const float*>(t), *rp = static_cast<const float*>(r), *cp = static_cast<const float*>(c);
  const bool vec = P % 4 == 0 && sk_aligned16(t, r, out);
  long long blocks = (total / (vec ? 4 : 1) + kSkThreads - 1) / kSkThreads;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (vec) sinkhorn_scale_kernel<true><<<(int)blocks, kSkThreads, 0, st>>>(tp, rp, cp, static_cast<float*>(out), total, P, inv);
  else sinkhorn_scale_kernel<false><<<(int)blocks, kSkThreads, 0, st>>>(tp, rp, cp, static_cast<float*>(out), total, P, inv);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}
