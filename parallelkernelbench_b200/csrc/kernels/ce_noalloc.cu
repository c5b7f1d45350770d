// Cross-entropy loss without any allocation at call time (declaration and contract: pkb/noalloc_api.h).
//
// Same two phases as the vocab-parallel cross-entropy (row statistics, then the loss), but the
// statistics go to a file-scope device array instead of a buffer the caller would have to allocate.
#include <mutex>

#include "pkb/host.h"
#include "pkb/noalloc_api.h"
#include "pkb/ptx.cuh"

namespace pkb {

// {row max, sum exp(x - max), target logit} per row. Lives in the library image on every GPU.
static __device__ __align__(256) float g_ce_scratch[PKB_CE_NOALLOC_MAX_ROWS * 3];

template <typename T>
__global__ void ce_noalloc_stats_kernel(const T* __restrict__ logits, const long long* __restrict__ target,
                                        float* __restrict__ stats, int rows, int vocab) {
  __shared__ float red[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* lr = logits + (long long)row * vocab;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, (float)lr[i]);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = -INFINITY;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float se = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) se += __expf((float)lr[i] - mx);
    se = warp_sum(se);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = se;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
      const long long t = target[row];
      stats[row * 3 + 0] = mx;
      stats[row * 3 + 1] = tot;
      stats[row * 3 + 2] = (t >= 0 && t < vocab) ? (float)lr[t] : 0.f;
    }
    __syncthreads();
  }
}

__global__ void ce_noalloc_loss_kernel(const float* __restrict__ stats, float* __restrict__ loss, int rows) {
  for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < rows; row += gridDim.x * blockDim.x)
    loss[row] = logf(stats[row * 3 + 1]) + stats[row * 3] - stats[row * 3 + 2];
}

// Device address of the scratch array, looked up once per device. In host code the array's name
// is only a handle for the runtime, not an address a kernel could use.
static float* scratch_ptr_for_current_device(int* rc_out) {
  constexpr int kMaxDev = 16;
  static float* ptrs[kMaxDev] = {nullptr};
  static std::mutex mu;
  *rc_out = kApiOk;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) {
    set_last_error("pkb_ce_loss_noalloc: cannot identify the current device");
    *rc_out = kApiCudaError;
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(mu);
  if (ptrs[dev] == nullptr) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_ce_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_last_error(std::string("pkb_ce_loss_noalloc: cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
      *rc_out = kApiCudaError;
      return nullptr;
    }
    ptrs[dev] = p;
  }
  return ptrs[dev];
}

}  // namespace pkb

using namespace pkb;

extern "C" int pkb_ce_loss_noalloc(const void* logits, const void* target, void* loss, int rows, int vocab,
                                   int dtype, void* stream) {
  PKB_CHECK_ARG(rows >= 0 && vocab >= 1, "rows must be non-negative and vocab positive");
  if (rows > PKB_CE_NOALLOC_MAX_ROWS) {
    char buf[160];
    snprintf(buf, sizeof(buf), "pkb_ce_loss_noalloc: %d rows exceed the fixed scratch capacity of %d rows", rows,
             PKB_CE_NOALLOC_MAX_ROWS);
    set_last_error(buf);
    return kApiBadArgument;
  }
  PKB_CHECK_ARG(dtype == 0 || dtype == 1, "dtype must be 0 (bf16) or 1 (fp32)");
  PKB_CHECK_ARG(logits != nullptr && target != nullptr && loss != nullptr, "null pointer");
  if (rows == 0) return kApiOk;
  int rc = kApiOk;
  float* scratch = scratch_ptr_for_current_device(&rc);
  if (scratch == nullptr) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  if (dtype == 0)
    ce_noalloc_stats_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(logits),
                                                               static_cast<const long long*>(target), scratch, rows, vocab);
  else
    ce_noalloc_stats_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(logits),
                                                       static_cast<const long long*>(target), scratch, rows, vocab);
  PKB_CHECK_CUDA(cudaGetLastError());
  ce_noalloc_loss_kernel<<<(rows + 255) / 256, 256, 0, s>>>(scratch, static_cast<float*>(loss), rows);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}
