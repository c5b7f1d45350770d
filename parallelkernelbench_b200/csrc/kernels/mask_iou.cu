// Pairwise mask IoU and occlusion-order suppression on bit-packed masks
// (reference: reference/81_sam3_allgather_iou_suppression.py:9-16 IoU, 30-48 suppression rule).
//
// The reference binarises the gathered mask logits to fp32, multiplies the n x HW matrix with its transpose for the
// intersections, and derives the suppression flags through half a dozen n x n temporaries. Here:
//   mask_pack_kernel      logits > 0 -> one bit per pixel (warp ballots) and the area of every mask
//   mask_suppress_kernel  one block per pair i < j: intersection = popcount of the AND of the two bit rows, IoU in fp32 with
//                         the reference's rounding (integers below 2^24 are exact, the division is IEEE), and the flags
//                         suppress[i] / suppress[j] set by plain stores of 1 (idempotent, so no atomics and no ordering issue)
// The masks shrink 32-fold before the pairwise pass, which then reads bits instead of floats.
#include "pkb/api.h"
#include "pkb/host.h"

namespace pkb {

constexpr int kMaskThreads = 256;

// grid = n masks; hw is a multiple of 32
__global__ void __launch_bounds__(kMaskThreads)
mask_pack_kernel(const float* __restrict__ logits, unsigned* __restrict__ bits, int* __restrict__ area, int hw) {
  __shared__ int part[kMaskThreads / 32];
  const long long m = blockIdx.x;
  const float* row = logits + m * hw;
  unsigned* brow = bits + m * (hw / 32);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int count = 0;                                        // meaningful on lane 0 of each warp
  for (int base = warp * 32; base < hw; base += kMaskThreads) {
    const unsigned word = __ballot_sync(0xffffffffu, row[base + lane] > 0.f);
    if (lane == 0) {
      brow[base >> 5] = word;
      count += __popc(word);
    }
  }
  if (lane == 0) part[warp] = count;
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
#pragma unroll
    for (int i = 0; i < kMaskThreads / 32; ++i) s += part[i];
    area[m] = s;
  }
}

// grid = (n, n); only blocks with i < j work. reverse: the reference's `reverse` flag (compare with < instead of >).
__global__ void __launch_bounds__(kMaskThreads)
mask_suppress_kernel(const unsigned* __restrict__ bits, const int* __restrict__ area, const long long* __restrict__ last,
                     int* __restrict__ suppress, int words, float threshold, int reverse) {
  const int i = blockIdx.y, j = blockIdx.x;
  if (i >= j) return;
  __shared__ int part[kMaskThreads / 32];
  const unsigned* bi = bits + (long long)i * words;
  const unsigned* bj = bits + (long long)j * words;
  int acc = 0;
  for (int w = threadIdx.x; w < words; w += kMaskThreads) acc += __popc(bi[w] & bj[w]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    int inter = 0;
#pragma unroll
    for (int k = 0; k < kMaskThreads / 32; ++k) inter += part[k];
    const float fi = (float)inter;
    const float uni = fmaxf(((float)area[i] + (float)area[j]) - fi, 1.0f);
    if (__fdiv_rn(fi, uni) >= threshold) {
      const long long li = last[i], lj = last[j];
      const bool i_after_j = reverse ? (li < lj) : (li > lj);
      const bool j_after_i = reverse ? (lj < li) : (lj > li);
      if (i_after_j && lj > -1) suppress[i] = 1;
      if (j_after_i && li > -1) suppress[j] = 1;
    }
  }
}

}  // namespace pkb

using namespace pkb;

// logits [n, hw] fp32; bits [n, hw / 32] uint32 and area [n] int32 are scratch; suppress [n] int32 must be zeroed by the caller.
extern "C" int pkb_mask_iou_suppress(const void* logits, const void* last, void* bits, void* area, void* suppress, int n, int hw,
                                     double threshold, int reverse, void* stream) {
  PKB_CHECK_ARG(n >= 1 && n <= 65535 && hw >= 32 && hw % 32 == 0, "need 1 <= n <= 65535 masks of a multiple of 32 pixels");
  PKB_CHECK_ARG(logits != nullptr && last != nullptr && bits != nullptr && area != nullptr && suppress != nullptr, "null tensor");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  mask_pack_kernel<<<n, kMaskThreads, 0, st>>>(static_cast<const float*>(logits), static_cast<unsigned*>(bits), static_cast<int*>(area), hw);
  PKB_CHECK_CUDA(cudaGetLastError());
  if (n > 1) {
    mask_suppress_kernel<<<dim3(n, n), kMaskThreads, 0, st>>>(static_cast<const unsigned*>(bits), static_cast<const int*>(area),
                                                             static_cast<const long long*>(last), static_cast<int*>(suppress), hw / 32,
                                                             (float)threshold, reverse);
    PKB_CHECK_CUDA(cudaGetLastError());
  }
  return kApiOk;
}
