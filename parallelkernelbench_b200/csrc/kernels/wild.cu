// Small compute kernels of the project-derived workloads (each is the local half of a fused exchange + compute op).
#include "pkb/api.h"
#include "pkb/symm_host.h"

namespace pkb {

// ------------------------------------------------------------------------------------------------
// DISCO contraction on the sphere: y[bc, row, p] = sum_e val[e] * x[bc, lat[e], (lon[e] + p * pscale) mod nlon_in]
// for the entries e of sparse row `row` = (kernel index, output latitude). One thread per (bc, row, p); the
// reference loops over p with a sparse bmm and a roll of the whole input per step
// (reference: reference/62_torchharmonics_spherical_convolution.py:42-69).
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
disco_contract_kernel(const float* __restrict__ x, const int* __restrict__ row_ptr, const int* __restrict__ col,
                      const float* __restrict__ val, float* __restrict__ y, long long bc, int rows, int nlat_in,
                      int nlon_in, int nlon_out, int pscale) {
  const long long total = bc * rows * nlon_out;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int p = (int)(i % nlon_out);
    const long long t = i / nlon_out;
    const int row = (int)(t % rows);
    const long long b = t / rows;
    const float* xb = x + b * nlat_in * nlon_in;
    float acc = 0.f;
    for (int e = row_ptr[row]; e < row_ptr[row + 1]; ++e) {
      const int c = col[e];
      const int lat = c / nlon_in;
      int lon = c - lat * nlon_in + p * pscale;
      lon %= nlon_in;
      acc += val[e] * xb[lat * nlon_in + lon];
    }
    y[i] = acc;
  }
}

// ------------------------------------------------------------------------------------------------
// Gated delta-rule recurrence. Per (batch*head) a state S[K][V] evolves over time:
//   S <- diag(decay_t) S ;  u = (v_t - k_t^T S) * beta_t ;  S <- S + k_t u^T ;  o_t = q_t^T S
// The columns of S are independent, so one warp owns one value column: lane l keeps rows l, l+32, ... of that column
// in registers, the two dot products are warp reductions, and q_t, k_t, decay_t are read once per step from L2.
// `decay` is [BH, T, KD] with KD = K (a decay per key channel) or 1 (one per step). The reference steps through time
// with three batched matrix products per step launched from Python
// (reference: reference/74_fla_kimi_delta_attention_cp_tp.py:73-81, reference/75_fla_gated_deltanet_cp.py:96-104).
// ------------------------------------------------------------------------------------------------
template <int KPL>  // key rows per lane = K / 32
__global__ void __launch_bounds__(256)
delta_rule_scan_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                       const float* __restrict__ decay, const float* __restrict__ beta, float* __restrict__ out,
                       int T, int V, int KD) {
  constexpr int K = KPL * 32;
  const int lane = threadIdx.x & 31;
  const int col = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long bh = blockIdx.y;
  if (col >= V) return;
  float S[KPL];
#pragma unroll
  for (int i = 0; i < KPL; ++i) S[i] = 0.f;
  const float* qb = q + bh * T * K;
  const float* kb = k + bh * T * K;
  const float* db = decay + bh * T * KD;
  for (int t = 0; t < T; ++t) {
    float kt[KPL], proj = 0.f;
    const float dscalar = KD == 1 ? db[t] : 0.f;
#pragma unroll
    for (int i = 0; i < KPL; ++i) {
      kt[i] = kb[(long long)t * K + lane + 32 * i];
      const float d = KD == 1 ? dscalar : db[(long long)t * K + lane + 32 * i];
      S[i] *= d;
      proj += kt[i] * S[i];
    }
    proj = warp_sum(proj);
    const float u = (v[(bh * T + t) * V + col] - proj) * beta[bh * T + t];
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < KPL; ++i) {
      S[i] += kt[i] * u;
      o += qb[(long long)t * K + lane + 32 * i] * S[i];
    }
    o = warp_sum(o);
    if (lane == 0) out[(bh * T + t) * V + col] = o;
  }
}

// ------------------------------------------------------------------------------------------------
// Depthwise causal conv1d over a sequence sharded in the load-balanced ("zigzag") layout: every rank holds global
// chunks r and 2W-1-r. The left halo of a chunk is the tail of the previous global chunk, which lives on a neighbour:
// every rank publishes the tails of its two chunks in its symmetric heap, and after one grid-wide barrier the
// convolution reads its halos straight from the neighbours' tails (zeros left of the sequence start; the last rank's
// second chunk continues its own first chunk). One launch replaces four point-to-point transfers, the concatenation
// with the padding and the library convolution (reference: reference/71_hyena_conv1d_boundary_exchange.py:24-95).
// ------------------------------------------------------------------------------------------------
struct HaloConvArgs {
  const void* x;       // [B, C, 2 * L]
  const void* w;       // [C, KS]
  void* y;             // [B, C, 2 * L]
  uint64_t tails_off;  // heap: [2][B * C][KS - 1] elements
  int B, C, L, KS;
};

template <typename T>
__global__ void __launch_bounds__(256) halo_conv1d_kernel(const SymmCtx c, const HaloConvArgs a) {
  const T* x = static_cast<const T*>(a.x);
  const T* w = static_cast<const T*>(a.w);
  T* y = static_cast<T*>(a.y);
  const int P = a.KS - 1;
  const long long BC = (long long)a.B * a.C;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
  T* tails = symm_local<T>(c, a.tails_off);
  for (long long i = tid; i < 2 * BC * P; i += nth) {
    const int j = (int)(i % P);
    const long long bc = (i / P) % BC;
    const int ch = (int)(i / (P * BC));
    tails[i] = x[bc * 2 * a.L + (long long)ch * a.L + a.L - P + j];
  }
  if (!symm_grid_barrier(c, 620, 1)) return;
  const int r = c.grank, W = c.gsize;
  // chunk 0 (global r) continues chunk 0 of rank r-1; chunk 1 (global 2W-1-r) continues chunk 1 of rank r+1,
  // or this rank's own chunk 0 on the last rank
  const T* halo0 = r > 0 ? symm_ptr<T>(c, c.members[r - 1], a.tails_off) : nullptr;
  const T* halo1 = r < W - 1 ? symm_ptr<T>(c, c.members[r + 1], a.tails_off) + BC * P : tails;
  for (long long i = tid; i < 2 * BC * a.L; i += nth) {
    const int t = (int)(i % a.L);
    const int ch = (int)((i / a.L) & 1);
    const long long bc = i / (2 * a.L);
    const int chan = (int)(bc % a.C);
    const T* xr = x + bc * 2 * a.L + (long long)ch * a.L;
    const T* hl = ch == 0 ? halo0 : halo1;
    float acc = 0.f;
    for (int j = 0; j < a.KS; ++j) {
      const int src = t + j - P;
      float xv;
      if (src >= 0) xv = (float)xr[src];
      else xv = hl ? (float)hl[bc * P + (src + P)] : 0.f;
      acc += (float)w[chan * a.KS + j] * xv;
    }
    y[i] = (T)acc;
  }
  // the tails are rewritten by the next call: the neighbours must have read them first
  symm_block_barrier(c, 620, 2);
}

}  // namespace pkb

using namespace pkb;

extern "C" int pkb_disco_contract(const void* x, const void* row_ptr, const void* col, const void* val, void* y,
                                  long long bc, int rows, int nlat_in, int nlon_in, int nlon_out, void* stream) {
  PKB_CHECK_ARG(bc >= 1 && rows >= 1 && nlat_in >= 1 && nlon_in >= 1 && nlon_out >= 1 && nlon_in % nlon_out == 0,
                "bad DISCO shape (nlon_in must be a multiple of nlon_out)");
  const long long total = bc * rows * nlon_out;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  disco_contract_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(x), static_cast<const int*>(row_ptr), static_cast<const int*>(col),
      static_cast<const float*>(val), static_cast<float*>(y), bc, rows, nlat_in, nlon_in, nlon_out, nlon_in / nlon_out);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

extern "C" int pkb_delta_rule_scan(const void* q, const void* k, const void* v, const void* decay, const void* beta,
                                   void* out, long long BH, int T, int K, int V, int KD, void* stream) {
  PKB_CHECK_ARG(BH >= 1 && BH <= 65535 && T >= 1 && V >= 1, "bad shape");
  PKB_CHECK_ARG(K == 32 || K == 64 || K == 128 || K == 256, "key dimension must be 32, 64, 128 or 256");
  PKB_CHECK_ARG(KD == 1 || KD == K, "decay is per step (1) or per key channel (K)");
  const dim3 grid((V + 7) / 8, (unsigned)BH);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float *qf = static_cast<const float*>(q), *kf = static_cast<const float*>(k), *vf = static_cast<const float*>(v);
  const float *df = static_cast<const float*>(decay), *bf = static_cast<const float*>(beta);
  float* of = static_cast<float*>(out);
  switch (K) {
    case 32: delta_rule_scan_kernel<1><<<grid, 256, 0, s>>>(qf, kf, vf, df, bf, of, T, V, KD); break;
    case 64: delta_rule_scan_kernel<2><<<grid, 256, 0, s>>>(qf, kf, vf, df, bf, of, T, V, KD); break;
    case 128: delta_rule_scan_kernel<4><<<grid, 256, 0, s>>>(qf, kf, vf, df, bf, of, T, V, KD); break;
    default: delta_rule_scan_kernel<8><<<grid, 256, 0, s>>>(qf, kf, vf, df, bf, of, T, V, KD); break;
  }
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

extern "C" int pkb_halo_conv1d_zigzag(const pkb_symm_ctx* h, const void* x, const void* w, void* y,
                                      unsigned long long tails_off, int B, int C, int L, int KS, int dtype, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(B >= 1 && C >= 1 && KS >= 2 && L >= KS - 1, "need a chunk at least as long as the halo");
  PKB_CHECK_ARG(dtype == 0 || dtype == 1, "dtype must be 0 (bf16) or 1 (fp32)");
  HaloConvArgs a{x, w, y, tails_off, B, C, L, KS};
  long long blocks = (2ll * B * C * L + 255) / 256;
  const int cap = sm_count() < kSymmMaxBlocks ? sm_count() : kSymmMaxBlocks;   // grid-wide barrier: one block per SM
  if (blocks > cap) blocks = cap;
  const SymmCtx c = symm_ctx_from_api(h);
  if (dtype == 0) halo_conv1d_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(c, a);
  else halo_conv1d_kernel<float><<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(c, a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}
