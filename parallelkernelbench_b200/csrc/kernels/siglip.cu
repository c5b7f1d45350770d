// Sigmoid contrastive loss over a block of image-text products
// (reference: reference/58_openclip_contrastive_loss.py; the per-block formula is -sum logsigmoid(label * (scale * x + bias)) / B
// with label +1 on the matching pair and -1 elsewhere).
//
// The products of this rank's images with the text features of ALL ranks come from one GEMM (fp32 out). This kernel is the
// rest of the loss in one pass over that matrix: scale and bias, the sign of the matching pair (column = rank * B + row), a
// numerically safe softplus, and a two-level sum with a fixed order (per block here, the handful of block results by the
// caller). The reference walks the text blocks around a ring and, per block, runs a GEMM and five elementwise / reduction
// launches over the block's logits.
#include "pkb/api.h"
#include "pkb/host.h"

namespace pkb {

constexpr int kSiglipThreads = 256;

__global__ void __launch_bounds__(kSiglipThreads)
siglip_loss_kernel(const float* __restrict__ prod, float* __restrict__ partial, int rows, int cols, int diag_offset, float scale,
                   float bias, float inv_rows) {
  __shared__ float part[kSiglipThreads / 32];
  float acc = 0.f;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* p = prod + (long long)r * cols;
    const int match = diag_offset + r;
    for (int c = threadIdx.x; c < cols; c += kSiglipThreads) {
      const float logit = fmaf(scale, p[c], bias);
      const float z = c == match ? logit : -logit;
      acc += fmaxf(-z, 0.f) + log1pf(expf(-fabsf(z)));     // -logsigmoid(z)
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kSiglipThreads / 32; ++i) s += part[i];
    partial[blockIdx.x] = s * inv_rows;
  }
}

}  // namespace pkb

using namespace pkb;

// prod [rows, cols] fp32; partial [blocks] fp32 receives one partial loss per block (already divided by rows); the caller adds them.
extern "C" int pkb_siglip_loss_partials(const void* prod, void* partial, int rows, int cols, int diag_offset, double scale, double bias,
                                        int blocks, void* stream) {
  PKB_CHECK_ARG(prod != nullptr && partial != nullptr && rows >= 1 && cols >= 1, "need a non-empty matrix");
  PKB_CHECK_ARG(blocks >= 1 && blocks <= rows && blocks <= 65535, "need 1 <= blocks <= rows");
  PKB_CHECK_ARG(diag_offset >= 0 && (long long)diag_offset + rows <= cols, "the matching pairs must lie inside the matrix");
  siglip_loss_kernel<<<blocks, kSiglipThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(prod), static_cast<float*>(partial), rows, cols, diag_offset, (float)scale, (float)bias, 1.0f / (float)rows);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}
