// Host launcher of the block-scaled fp8 GEMM (kernel template in pkb/gemm_fp8.cuh).
#include "pkb/gemm_fp8.cuh"
#include "pkb/host.h"

using namespace pkb;

template <int EPI, bool GROUPED>
static int launch_fp8(const CUtensorMap& ta, const CUtensorMap& tb, const GemmFp8Params& p, int ctas, cudaStream_t s) {
  auto kern = gemm_fp8_kernel<EPI, GROUPED>;
  PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmFp8Smem::kTotal));
  kern<<<ctas, kFp8Threads, GemmFp8Smem::kTotal, s>>>(ta, tb, p);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// C = epi(alpha * dequant(A) @ dequant(B)^T) with e4m3 operands and fp32 block scales.
//   a8 [M, K] e4m3, lda bytes between rows; sa fp32, sa[row * sa_stride + k / 128]
//   b8 [N, K] (dense) or [groups * N, K] (grouped) e4m3; sb fp32, sb[(row of b8 / 128) * sb_stride + k / 128]
//   epilogue 0: c bf16 [M, N];  1: SwiGLU over interleaved (gate, up) columns, c bf16 [M, N / 2];
//            2: SwiGLU, then 1x128 re-quantisation: c e4m3 [M, N / 2], out_scales[row * os_stride + n / 256]
//            3: row scatter: bf16 row m is stored as row row_meta[m].y (ldc elements per row) of the buffer
//               dest_ptrs[row_meta[m].x], which may live on another rank (c is unused); row_meta is an int2 device array
//               with one entry per row of A, dest_ptrs a HOST array of ndest <= 8 device addresses
//   groups 0: dense. groups >= 1: rows [offsets[e], offsets[e + 1]) of A use weight block e; offsets is an
//   int32 device array of groups + 1 entries that only the device reads, M bounds offsets[groups].
// K % 128 == 0, N % 128 == 0 (N % 256 == 0 for epilogue 2), lda % 16 == 0, ldb % 16 == 0.
extern "C" int pkb_gemm_fp8_blockscaled(const void* a8, long long lda, const void* sa, long long sa_stride,
                                        const void* b8, long long ldb, const void* sb, long long sb_stride, void* c,
                                        long long ldc, void* out_scales, long long os_stride, const void* offsets,
                                        int groups, int M, int N, int K, float alpha, int epilogue, int num_ctas,
                                        const void* row_meta, const unsigned long long* dest_ptrs, int ndest, void* stream) {
  PKB_CHECK_ARG(M > 0 && N > 0 && K > 0, "empty problem");
  PKB_CHECK_ARG(K % kFp8BlockK == 0 && N % 128 == 0, "K and N must be multiples of 128");
  PKB_CHECK_ARG(lda % 16 == 0 && ldb % 16 == 0, "lda and ldb must be multiples of 16");
  PKB_CHECK_ARG(epilogue >= kFp8EpiNone && epilogue <= kFp8EpiRowScatter, "unknown epilogue");
  PKB_CHECK_ARG(epilogue != kFp8EpiRowScatter || (row_meta != nullptr && dest_ptrs != nullptr && ndest >= 1 && ndest <= kGemmMaxWorld),
                "the row-scatter epilogue needs row_meta and 1..8 destination buffers");
  PKB_CHECK_ARG(epilogue != kFp8EpiSwiGLUQuant || (out_scales != nullptr && N % 256 == 0),
                "the re-quantising epilogue needs out_scales and N % 256 == 0");
  PKB_CHECK_ARG(groups >= 0 && groups <= kGemmMaxGroups, "0..256 groups");
  PKB_CHECK_ARG(groups == 0 || offsets != nullptr, "grouped form without offsets");
  PKB_CHECK_ARG(sa != nullptr && sb != nullptr && sa_stride >= K / kFp8BlockK && sb_stride >= K / kFp8BlockK,
                "scale tensors missing or too narrow");
  const long long b_rows = (long long)(groups > 0 ? groups : 1) * N;
  CUtensorMap ta, tb;
  int rc = encode_tmap_2d(&ta, kTmapFp8, a8, (uint64_t)K, (uint64_t)M, (uint64_t)lda, kFp8BlockK, kFp8BlockM, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_2d(&tb, kTmapFp8, b8, (uint64_t)K, (uint64_t)b_rows, (uint64_t)ldb, kFp8BlockK, kFp8BlockN, kSwizzle128);
  if (rc) return rc;
  GemmFp8Params p = {};
  p.M = M; p.N = N; p.K = K;
  p.C = c; p.ldc = ldc;
  p.sa = static_cast<const float*>(sa); p.sa_stride = sa_stride;
  p.sb = static_cast<const float*>(sb); p.sb_stride = sb_stride;
  p.out_scales = static_cast<float*>(out_scales); p.os_stride = os_stride;
  p.alpha = alpha;
  p.status = status_block_device_ptr();
  p.wait_budget_ns = kDefaultWaitBudgetNs;
  p.kernel_id = 105;
  p.grp_offsets = static_cast<const int*>(offsets);
  p.grp_count = groups;
  if (epilogue == kFp8EpiRowScatter) {
    p.row_meta = static_cast<const int2*>(row_meta);
    for (int g = 0; g < kGemmMaxWorld; ++g)
      p.scatter_out[g] = reinterpret_cast<void*>(static_cast<uintptr_t>(dest_ptrs[g < ndest ? g : 0]));
  }
  int ctas = num_ctas > 0 ? num_ctas : sm_count();
  if (groups == 0) {
    const int tiles = ((M + kFp8BlockM - 1) / kFp8BlockM) * ((N + kFp8BlockN - 1) / kFp8BlockN);
    if (ctas > tiles) ctas = tiles;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (groups > 0) {
    switch (epilogue) {
      case kFp8EpiNone: return launch_fp8<kFp8EpiNone, true>(ta, tb, p, ctas, s);
      case kFp8EpiSwiGLU: return launch_fp8<kFp8EpiSwiGLU, true>(ta, tb, p, ctas, s);
      case kFp8EpiRowScatter: return launch_fp8<kFp8EpiRowScatter, true>(ta, tb, p, ctas, s);
      default: return launch_fp8<kFp8EpiSwiGLUQuant, true>(ta, tb, p, ctas, s);
    }
  }
  switch (epilogue) {
    case kFp8EpiNone: return launch_fp8<kFp8EpiNone, false>(ta, tb, p, ctas, s);
    case kFp8EpiSwiGLU: return launch_fp8<kFp8EpiSwiGLU, false>(ta, tb, p, ctas, s);
    case kFp8EpiRowScatter: return launch_fp8<kFp8EpiRowScatter, false>(ta, tb, p, ctas, s);
    default: return launch_fp8<kFp8EpiSwiGLUQuant, false>(ta, tb, p, ctas, s);
  }
}
