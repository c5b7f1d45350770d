// Block Kalman-filter optimiser step in fp64 (reference: reference/63_deepmd_kalman_filter_optimizer.py:20-32).
//
// Per block b with covariance P_b [n, n], gradient H_b [n] and weights w_b [n]:
//     K_b = P_b H_b ;  s = sum_b (lambda + H_b^T K_b)   (summed over all ranks by the caller) ;  A = 1 / s
//     w_b <- w_b + (A err) K_b ;  P_b <- (1 / lambda) (P_b - A K_b K_b^T)
// The reference spells this out as library products: H^T P, (H^T P) H, P H, K K^T (an n x n temporary), a subtraction and a
// scaling, about eight passes over n^2 doubles per block. Here P is read twice and written once:
//   kalman_gain_kernel    K = P H, one warp per row of P, 16-byte loads, a shuffle reduction in a fixed order
//   kalman_dot_kernel     s_local = nb lambda + sum H K, one block, fixed summation order (the result is bit-reproducible)
//   kalman_update_kernel  reads A's denominator and err from device memory (no value comes back to the host), forms the
//                         rank-one term on the fly and writes the new P and the new weights
// Everything is memory-bound fp64; no tensor-core work is involved.
#include "pkb/api.h"
#include "pkb/host.h"

namespace pkb {

constexpr int kKalmanThreads = 256;
constexpr int kKalmanDotThreads = 1024;

__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <bool VEC2>  // VEC2: n is even, so every row of P starts on a 16-byte boundary
__global__ void __launch_bounds__(kKalmanThreads)
kalman_gain_kernel(const double* __restrict__ P, const double* __restrict__ H, double* __restrict__ K, long long rows, int n) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * kKalmanThreads + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * kKalmanThreads) >> 5;
  for (long long row = warp; row < rows; row += nwarps) {
    const double* p = P + row * n;
    const double* h = H + (row / n) * n;
    double acc0 = 0.0, acc1 = 0.0;
    if constexpr (VEC2) {
      for (int j = lane * 2; j < n; j += 64) {
        const double2 pv = *reinterpret_cast<const double2*>(p + j);
        const double2 hv = *reinterpret_cast<const double2*>(h + j);
        acc0 = fma(pv.x, hv.x, acc0);
        acc1 = fma(pv.y, hv.y, acc1);
      }
    } else {
      for (int j = lane; j < n; j += 32) acc0 = fma(p[j], h[j], acc0);
    }
    const double k = warp_sum_f64(acc0 + acc1);
    if (lane == 0) K[row] = k;
  }
}

__global__ void __launch_bounds__(kKalmanDotThreads)
kalman_dot_kernel(const double* __restrict__ H, const double* __restrict__ K, double* __restrict__ s_out, long long total,
                  double lambda_times_blocks) {
  __shared__ double part[kKalmanDotThreads / 32];
  double acc = 0.0;
  for (long long i = threadIdx.x; i < total; i += kKalmanDotThreads) acc = fma(H[i], K[i], acc);
  acc = warp_sum_f64(acc);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    double v = part[threadIdx.x];          // kKalmanDotThreads / 32 == 32 partial sums
    v = warp_sum_f64(v);
    if (threadIdx.x == 0) s_out[0] = lambda_times_blocks + v;
  }
}

// One block per row of P at a time (no index division in the inner loop); thread 0 of the row also writes the new weight.
template <bool VEC2>
__global__ void __launch_bounds__(kKalmanThreads)
kalman_update_kernel(const double* __restrict__ P, const double* __restrict__ K, const double* __restrict__ w,
                     const double* __restrict__ err, const double* __restrict__ s, double* __restrict__ P_new,
                     double* __restrict__ w_new, long long rows, int n, double inv_lambda) {
  const double A = 1.0 / s[0];
  const double a_err = A * err[0];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const double* kb = K + (row / n) * n;   // the block's gain vector
    const double ki = K[row];
    const double a_ki = A * ki;
    const double* p = P + row * n;
    double* o = P_new + row * n;
    if constexpr (VEC2) {
      for (int j = threadIdx.x * 2; j < n; j += kKalmanThreads * 2) {
        const double2 pv = *reinterpret_cast<const double2*>(p + j);
        const double2 kj = *reinterpret_cast<const double2*>(kb + j);
        double2 r;
        r.x = inv_lambda * (pv.x - a_ki * kj.x);
        r.y = inv_lambda * (pv.y - a_ki * kj.y);
        *reinterpret_cast<double2*>(o + j) = r;
      }
    } else {
      for (int j = threadIdx.x; j < n; j += kKalmanThreads) o[j] = inv_lambda * (p[j] - a_ki * kb[j]);
    }
    if (threadIdx.x == 0) w_new[row] = w[row] + a_err * ki;
  }
}

static int kalman_grid(long long work_items, int per_block) {
  long long blocks = (work_items + per_block - 1) / per_block;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : (int)blocks;
}

}  // namespace pkb

using namespace pkb;

// K [nb * n] and s_local [1] are outputs. `lambda` enters s_local once per block, as in the reference's loop.
extern "C" int pkb_kalman_gain(const void* P, const void* H, void* K, void* s_local, long long nb, int n, double lambda, void* stream) {
  PKB_CHECK_ARG(nb >= 1 && n >= 1 && nb * (long long)n <= (1ll << 31), "need 1 <= blocks, 1 <= n and blocks * n <= 2^31");
  PKB_CHECK_ARG(P != nullptr && H != nullptr && K != nullptr && s_local != nullptr, "null tensor");
  PKB_CHECK_ARG(reinterpret_cast<uintptr_t>(P) % 16 == 0 && reinterpret_cast<uintptr_t>(H) % 16 == 0, "P and H must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long rows = nb * n;
  const int grid = kalman_grid(rows, kKalmanThreads / 32);
  const double *p = static_cast<const double*>(P), *h = static_cast<const double*>(H);
  double* k = static_cast<double*>(K);
  if (n % 2 == 0) kalman_gain_kernel<true><<<grid, kKalmanThreads, 0, st>>>(p, h, k, rows, n);
  else kalman_gain_kernel<false><<<grid, kKalmanThreads, 0, st>>>(p, h, k, rows, n);
  PKB_CHECK_CUDA(cudaGetLastError());
  kalman_dot_kernel<<<1, kKalmanDotThreads, 0, st>>>(h, k, static_cast<double*>(s_local), rows, lambda * (double)nb);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// `s` [1] is the denominator summed over all ranks, `err` [1] the scalar error; both stay on the device.
extern "C" int pkb_kalman_update(const void* P, const void* K, const void* w, const void* err, const void* s, void* P_new,
                                 void* w_new, long long nb, int n, double lambda, void* stream) {
  PKB_CHECK_ARG(nb >= 1 && n >= 1 && nb * (long long)n <= (1ll << 31), "need 1 <= blocks, 1 <= n and blocks * n <= 2^31");
  PKB_CHECK_ARG(lambda != 0.0, "lambda must not be zero");
  PKB_CHECK_ARG(P != nullptr && K != nullptr && w != nullptr && err != nullptr && s != nullptr && P_new != nullptr && w_new != nullptr,
                "null tensor");
  PKB_CHECK_ARG(reinterpret_cast<uintptr_t>(P) % 16 == 0 && reinterpret_cast<uintptr_t>(K) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(P_new) % 16 == 0,
                "P, K and the new P must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long rows = nb * n;
  const double *p = static_cast<const double*>(P), *k = static_cast<const double*>(K), *wv = static_cast<const double*>(w);
  const double *e = static_cast<const double*>(err), *sv = static_cast<const double*>(s);
  double *pn = static_cast<double*>(P_new), *wn = static_cast<double*>(w_new);
  const long long cap = (long long)sm_count() * 16;
  const int grid = (int)(rows < cap ? rows : cap);
  if (n % 2 == 0) kalman_update_kernel<true><<<grid, kKalmanThreads, 0, st>>>(p, k, wv, e, sv, pn, wn, rows, n, 1.0 / lambda);
  else kalman_update_kernel<false><<<grid, kKalmanThreads, 0, st>>>(p, k, wv, e, sv, pn, wn, rows, n, 1.0 / lambda);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}
