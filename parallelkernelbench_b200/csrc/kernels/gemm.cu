// Host launchers of the tcgen05 GEMM (kernel template in pkb/gemm_umma.cuh).
#include <cstdlib>

#include "pkb/api.h"
#include "pkb/gemm_umma2.cuh"
#include "pkb/host.h"

namespace pkb {

template <int BN, int EPI, bool OUT_F32>
static int launch_plain(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                        int num_ctas, cudaStream_t stream) {
  auto kern = gemm_umma_kernel<BN, EPI, OUT_F32, false, false>;
  constexpr int smem = GemmSmem<BN>::kTotal;
  static bool configured = false;  // per instantiation; attribute is per device but idempotent
  if (!configured) {
    PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  kern<<<num_ctas, kGemmThreads, smem, stream>>>(ta, tb, p);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

template <int BN, bool OUT_F32>
static int dispatch_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                        int num_ctas, cudaStream_t stream) {
  switch (epi) {
    case kEpiNone: return launch_plain<BN, kEpiNone, OUT_F32>(ta, tb, p, num_ctas, stream);
    case kEpiSilu: return launch_plain<BN, kEpiSilu, OUT_F32>(ta, tb, p, num_ctas, stream);
    case kEpiBias: return launch_plain<BN, kEpiBias, OUT_F32>(ta, tb, p, num_ctas, stream);
    case kEpiBiasSilu: return launch_plain<BN, kEpiBiasSilu, OUT_F32>(ta, tb, p, num_ctas, stream);
  }
  set_last_error("unknown epilogue");
  return kApiBadArgument;
}

template <int EPI, bool OUT_F32>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                       int num_ctas, cudaStream_t stream) {
  auto kern = gemm_umma2_kernel<EPI, OUT_F32, false, false>;
  PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kGemm2SmemTotal));
  kern<<<num_ctas, kGemmThreads, kGemm2SmemTotal, stream>>>(ta, tb, p);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

template <int EPI>
static int launch_pair_tma(const CUtensorMap& ta, const CUtensorMap& tb, const GemmOutMaps& om,
                           const GemmParams& p, int num_ctas, cudaStream_t stream) {
  auto kern = gemm_umma2_tma_kernel<EPI>;
  PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kGemm2SmemTotal));
  kern<<<num_ctas, kGemmThreads, kGemm2SmemTotal, stream>>>(ta, tb, om, p);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

static int dispatch_pair_tma(int epi, const CUtensorMap& ta, const CUtensorMap& tb,
                             const GemmOutMaps& om, const GemmParams& p, int num_ctas,
                             cudaStream_t stream) {
  switch (epi) {
    case kEpiNone: return launch_pair_tma<kEpiNone>(ta, tb, om, p, num_ctas, stream);
    case kEpiSilu: return launch_pair_tma<kEpiSilu>(ta, tb, om, p, num_ctas, stream);
    case kEpiBias: return launch_pair_tma<kEpiBias>(ta, tb, om, p, num_ctas, stream);
    case kEpiBiasSilu: return launch_pair_tma<kEpiBiasSilu>(ta, tb, om, p, num_ctas, stream);
  }
  set_last_error("unknown epilogue");
  return kApiBadArgument;
}

template <bool OUT_F32>
static int dispatch_pair(int epi, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                         int num_ctas, cudaStream_t stream) {
  switch (epi) {
    case kEpiNone: return launch_pair<kEpiNone, OUT_F32>(ta, tb, p, num_ctas, stream);
    case kEpiSilu: return launch_pair<kEpiSilu, OUT_F32>(ta, tb, p, num_ctas, stream);
    case kEpiBias: return launch_pair<kEpiBias, OUT_F32>(ta, tb, p, num_ctas, stream);
    case kEpiBiasSilu: return launch_pair<kEpiBiasSilu, OUT_F32>(ta, tb, p, num_ctas, stream);
  }
  set_last_error("unknown epilogue");
  return kApiBadArgument;
}

// The backward layouts on CTA pairs: PKB_GEMM_PAIR_MN=0 keeps the one-CTA-per-tile kernels.
static bool pair_mn_enabled() {
  static const bool on = [] { const char* e = getenv("PKB_GEMM_PAIR_MN"); return !(e != nullptr && e[0] == '0'); }();
  return on;
}

template <int EPI, bool OUT_F32, bool A_MN, bool B_MN>
static int launch_pair_mn(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams p, int M, int N, cudaStream_t stream) {
  auto kern = gemm_umma2_mn_kernel<EPI, OUT_F32, A_MN, B_MN>;
  PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemm2SmemTotal));
  p.group_m = 8;
  const int tiles = ((M + 255) / 256) * ((N + 255) / 256);
  int ctas = sm_count() & ~1;
  if (ctas > 2 * tiles) ctas = 2 * tiles;
  kern<<<ctas, kGemmThreads, kGemm2SmemTotal, stream>>>(ta, tb, p);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

}  // namespace pkb

using namespace pkb;

// CTA-pair form: 256 x 256 tiles on clusters of two CTAs (see pkb/gemm_umma2.cuh).
extern "C" int pkb_gemm_bf16_pair(const void* a, long long lda, const void* b, long long ldb,
                                  void* c, long long ldc, int M, int N, int K, const void* bias,
                                  float alpha, int epilogue, int out_f32, int num_ctas,
                                  void* stream) {
  PKB_CHECK_ARG(M > 0 && N > 0 && K > 0, "empty problem");
  PKB_CHECK_ARG(lda % 8 == 0 && ldb % 8 == 0 && K % 8 == 0, "lda, ldb, K must be multiples of 8");
  PKB_CHECK_ARG((epilogue & 2) == 0 || bias != nullptr, "bias epilogue without bias");
  CUtensorMap ta, tb;
  int rc = encode_tmap_2d(&ta, kTmapBf16, a, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2,
                          kGemmBlockK, 128, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_2d(&tb, kTmapBf16, b, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, kGemmBlockK,
                      128, kSwizzle128);
  if (rc) return rc;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.C = c; p.ldc = ldc;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.alpha = alpha;
  p.status = status_block_device_ptr();
  p.wait_budget_ns = kDefaultWaitBudgetNs;
  p.group_m = 8;
  p.kernel_id = 101;
  p.world = 1;
  const int tiles = ((M + 255) / 256) * ((N + 255) / 256);
  int ctas = num_ctas > 0 ? num_ctas : sm_count();
  ctas &= ~1;
  if (ctas > 2 * tiles) ctas = 2 * tiles;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!out_f32 && ldc % 8 == 0 && (reinterpret_cast<uintptr_t>(c) & 15) == 0) {
    GemmOutMaps om;
    rc = encode_tmap_2d(&om.m[0], kTmapBf16, c, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 2, 64, 32,
                        kSwizzle128);
    if (rc) return rc;
    return dispatch_pair_tma(epilogue, ta, tb, om, p, ctas, s);
  }
  return out_f32 ? dispatch_pair<true>(epilogue, ta, tb, p, ctas, s)
                 : dispatch_pair<false>(epilogue, ta, tb, p, ctas, s);
}

extern "C" int pkb_gemm_bf16(const void* a, long long lda, const void* b, long long ldb, void* c,
                             long long ldc, int M, int N, int K, const void* bias, float alpha,
                             int epilogue, int out_f32, int block_n, int num_ctas, void* stream) {
  PKB_CHECK_ARG(M > 0 && N > 0 && K > 0, "empty problem");
  PKB_CHECK_ARG(lda % 8 == 0 && ldb % 8 == 0 && K % 8 == 0, "lda, ldb, K must be multiples of 8");
  PKB_CHECK_ARG((epilogue & 2) == 0 || bias != nullptr, "bias epilogue without bias");
  if (block_n == 0) block_n = (N >= 256 && (long long)M * N >= 128ll * 256 * 64) ? 256 : 128;
  PKB_CHECK_ARG(block_n == 128 || block_n == 256, "block_n must be 128 or 256");

  CUtensorMap ta, tb;
  int rc = encode_tmap_2d(&ta, kTmapBf16, a, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2,
                          kGemmBlockK, kGemmBlockM, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_2d(&tb, kTmapBf16, b, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, kGemmBlockK,
                      (uint32_t)block_n, kSwizzle128);
  if (rc) return rc;

  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.C = c; p.ldc = ldc;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.alpha = alpha;
  p.status = status_block_device_ptr();
  p.wait_budget_ns = kDefaultWaitBudgetNs;
  p.group_m = 16;
  p.kernel_id = 100;
  p.world = 1;

  const int num_m = (M + kGemmBlockM - 1) / kGemmBlockM;
  const int num_n = (N + block_n - 1) / block_n;
  const int tiles = num_m * num_n;
  int ctas = num_ctas > 0 ? num_ctas : sm_count();
  if (ctas > tiles) ctas = tiles;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (block_n == 256)
    return out_f32 ? dispatch_epi<256, true>(epilogue, ta, tb, p, ctas, s)
                   : dispatch_epi<256, false>(epilogue, ta, tb, p, ctas, s);
  return out_f32 ? dispatch_epi<128, true>(epilogue, ta, tb, p, ctas, s)
                 : dispatch_epi<128, false>(epilogue, ta, tb, p, ctas, s);
}

// Grouped (ragged) GEMM: rows of A are grouped back to back, group e = rows
// [offsets[e], offsets[e+1]) (int32 device array of groups + 1 entries, read on the device only) and
// uses the weight block b[e*N : (e+1)*N, :]. C[total_rows, N] (or N/2 columns for the SwiGLU
// epilogue). max_rows bounds offsets[groups]; rows at or beyond it are never touched.
// epilogue: 0 none, 1 SiLU, 4 SwiGLU over interleaved (gate, up) weight rows.
extern "C" int pkb_gemm_bf16_grouped(const void* a, long long lda, const void* b, long long ldb,
                                     void* c, long long ldc, const void* offsets, int groups,
                                     int max_rows, int N, int K, int epilogue, int block_n,
                                     void* stream) {
  PKB_CHECK_ARG(groups >= 1 && groups <= kGemmMaxGroups, "1..256 groups");
  PKB_CHECK_ARG(max_rows > 0 && N > 0 && K > 0, "empty problem");
  PKB_CHECK_ARG(lda % 8 == 0 && ldb % 8 == 0 && K % 8 == 0, "lda, ldb, K must be multiples of 8");
  PKB_CHECK_ARG(epilogue == kEpiNone || epilogue == kEpiSilu || epilogue == kEpiSwiGLU, "unsupported epilogue");
  if (block_n == 0) block_n = N >= 256 ? 256 : 128;
  PKB_CHECK_ARG(block_n == 128 || block_n == 256, "block_n must be 128 or 256");
  CUtensorMap ta, tb;
  int rc = encode_tmap_2d(&ta, kTmapBf16, a, (uint64_t)K, (uint64_t)max_rows, (uint64_t)lda * 2,
                          kGemmBlockK, kGemmBlockM, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_2d(&tb, kTmapBf16, b, (uint64_t)K, (uint64_t)groups * N, (uint64_t)ldb * 2,
                      kGemmBlockK, (uint32_t)block_n, kSwizzle128);
  if (rc) return rc;
  GemmParams p = {};
  p.M = max_rows; p.N = N; p.K = K;
  p.C = c; p.ldc = ldc; p.alpha = 1.0f;
  p.status = status_block_device_ptr();
  p.wait_budget_ns = kDefaultWaitBudgetNs;
  p.kernel_id = 102;
  p.world = 1;
  p.grp_offsets = static_cast<const int*>(offsets);
  p.grp_count = groups;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // CTA pairs (256 x 256 tiles over two SMs, half of the B traffic per SM) when the shape allows; PKB_GROUPED_PAIR=0 keeps
  // the one-CTA-per-tile kernel
  static const bool pair_on = [] { const char* e = getenv("PKB_GROUPED_PAIR"); return !(e != nullptr && e[0] == '0'); }();
  if (pair_on && block_n == 256 && N % 256 == 0 && K % kGemmBlockK == 0 && sm_count() >= 2) {
    CUtensorMap tb2;
    rc = encode_tmap_2d(&tb2, kTmapBf16, b, (uint64_t)K, (uint64_t)groups * N, (uint64_t)ldb * 2, kGemmBlockK, 128, kSwizzle128);
    if (rc) return rc;
    p.kernel_id = 107;
    const int num_ctas = sm_count() & ~1;
#define PKB_GROUPED_PAIR_LAUNCH(EPI)                                                                             \
    {                                                                                                             \
      auto kern = gemm_umma2_grouped_kernel<EPI>;                                                                 \
      PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemm2SmemTotal));   \
      kern<<<num_ctas, kGemmThreads, kGemm2SmemTotal, s>>>(ta, tb2, p);                                           \
    }
    if (epilogue == kEpiNone) PKB_GROUPED_PAIR_LAUNCH(kEpiNone)
    else if (epilogue == kEpiSilu) PKB_GROUPED_PAIR_LAUNCH(kEpiSilu)
    else PKB_GROUPED_PAIR_LAUNCH(kEpiSwiGLU)
#undef PKB_GROUPED_PAIR_LAUNCH
    PKB_CHECK_CUDA(cudaGetLastError());
    return kApiOk;
  }
  const int ctas = sm_count();
#define PKB_GROUPED(BN, EPI)                                                                        \
  {                                                                                                 \
    auto kern = gemm_umma_grouped_kernel<BN, EPI>;                                                  \
    PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                                        GemmSmem<BN>::kTotal));                                     \
    kern<<<ctas, kGemmThreads, GemmSmem<BN>::kTotal, s>>>(ta, tb, p);                               \
  }
  if (block_n == 256) {
    if (epilogue == kEpiNone) PKB_GROUPED(256, kEpiNone)
    else if (epilogue == kEpiSilu) PKB_GROUPED(256, kEpiSilu)
    else PKB_GROUPED(256, kEpiSwiGLU)
  } else {
    if (epilogue == kEpiNone) PKB_GROUPED(128, kEpiNone)
    else if (epilogue == kEpiSilu) PKB_GROUPED(128, kEpiSilu)
    else PKB_GROUPED(128, kEpiSwiGLU)
  }
#undef PKB_GROUPED
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// Grouped GEMM whose output rows are scattered: row m of the product is stored as row row_meta[m].y (ldc elements per
// row, bf16) of the buffer dest_ptrs[row_meta[m].x], which may live on another rank. row_meta is an int2 device array with
// one entry per row of A; dest_ptrs is a HOST array of ndest <= 8 device addresses (16-byte aligned).
extern "C" int pkb_gemm_bf16_grouped_scatter(const void* a, long long lda, const void* b, long long ldb, long long ldc,
                                             const void* offsets, int groups, int max_rows, int N, int K, int block_n,
                                             const void* row_meta, const unsigned long long* dest_ptrs, int ndest,
                                             void* stream) {
  PKB_CHECK_ARG(groups >= 1 && groups <= kGemmMaxGroups, "1..256 groups");
  PKB_CHECK_ARG(max_rows > 0 && N > 0 && K > 0, "empty problem");
  PKB_CHECK_ARG(lda % 8 == 0 && ldb % 8 == 0 && K % 8 == 0 && ldc % 8 == 0, "lda, ldb, ldc, K must be multiples of 8");
  PKB_CHECK_ARG(row_meta != nullptr && dest_ptrs != nullptr && ndest >= 1 && ndest <= kGemmMaxWorld,
                "row_meta and 1..8 destination buffers are required");
  if (block_n == 0) block_n = N >= 256 ? 256 : 128;
  PKB_CHECK_ARG(block_n == 128 || block_n == 256, "block_n must be 128 or 256");
  CUtensorMap ta, tb;
  int rc = encode_tmap_2d(&ta, kTmapBf16, a, (uint64_t)K, (uint64_t)max_rows, (uint64_t)lda * 2, kGemmBlockK, kGemmBlockM,
                          kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_2d(&tb, kTmapBf16, b, (uint64_t)K, (uint64_t)groups * N, (uint64_t)ldb * 2, kGemmBlockK, (uint32_t)block_n,
                      kSwizzle128);
  if (rc) return rc;
  GemmParams p = {};
  p.M = max_rows; p.N = N; p.K = K;
  p.C = nullptr; p.ldc = ldc; p.alpha = 1.0f;
  p.status = status_block_device_ptr();
  p.wait_budget_ns = kDefaultWaitBudgetNs;
  p.kernel_id = 106;
  p.world = 1;
  p.grp_offsets = static_cast<const int*>(offsets);
  p.grp_count = groups;
  p.row_meta = static_cast<const int2*>(row_meta);
  for (int g = 0; g < kGemmMaxWorld; ++g) {
    PKB_CHECK_ARG((dest_ptrs[g < ndest ? g : 0] & 15) == 0, "destination buffers must be 16-byte aligned");
    p.rs_out[g] = reinterpret_cast<void*>(static_cast<uintptr_t>(dest_ptrs[g < ndest ? g : 0]));
  }
  const int ctas = sm_count();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (block_n == 256) {
    auto kern = gemm_umma_grouped_kernel<256, kEpiRowScatter>;
    PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<256>::kTotal));
    kern<<<ctas, kGemmThreads, GemmSmem<256>::kTotal, s>>>(ta, tb, p);
  } else {
    auto kern = gemm_umma_grouped_kernel<128, kEpiRowScatter>;
    PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<128>::kTotal));
    kern<<<ctas, kGemmThreads, GemmSmem<128>::kTotal, s>>>(ta, tb, p);
  }
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// C[M,N] = epi(A[M,K] @ B[K,N]) with B row-major [K, N] (ldb elements between K rows, N % 8 == 0).
// epilogue: 0 none, 1 SiLU. out_f32 selects fp32 output.
extern "C" int pkb_gemm_bf16_bkn(const void* a, long long lda, const void* b, long long ldb, void* c,
                                 long long ldc, int M, int N, int K, float alpha, int epilogue,
                                 int out_f32, void* stream) {
  PKB_CHECK_ARG(M > 0 && N > 0 && K > 0, "empty problem");
  PKB_CHECK_ARG(lda % 8 == 0 && ldb % 8 == 0 && K % 8 == 0 && N % 8 == 0, "lda, ldb, K, N must be multiples of 8");
  PKB_CHECK_ARG(epilogue == kEpiNone || epilogue == kEpiSilu, "epilogue must be none or silu");
  CUtensorMap ta, tb;
  int rc = encode_tmap_2d(&ta, kTmapBf16, a, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, kGemmBlockK,
                          kGemmBlockM, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_2d(&tb, kTmapBf16, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, kGemmBlockK,
                      kSwizzle128);
  if (rc) return rc;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K; p.C = c; p.ldc = ldc; p.alpha = alpha;
  p.status = status_block_device_ptr();
  p.wait_budget_ns = kDefaultWaitBudgetNs;
  p.group_m = 16; p.kernel_id = 103; p.world = 1;
  const int tiles = ((M + 127) / 128) * ((N + 127) / 128);
  int ctas = sm_count();
  if (ctas > tiles) ctas = tiles;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (pair_mn_enabled() && M >= 256 && N >= 256) {
    // large problems: 256 x 256 tiles on CTA pairs (every operand byte crosses L2 -> shared memory once per pair)
    if (epilogue == kEpiSilu)
      return out_f32 ? launch_pair_mn<kEpiSilu, true, false, true>(ta, tb, p, M, N, s) : launch_pair_mn<kEpiSilu, false, false, true>(ta, tb, p, M, N, s);
    return out_f32 ? launch_pair_mn<kEpiNone, true, false, true>(ta, tb, p, M, N, s) : launch_pair_mn<kEpiNone, false, false, true>(ta, tb, p, M, N, s);
  }
  constexpr int smem = GemmSmem<128>::kTotal;
#define PKB_BKN(EPI, F32)                                                                          \
  {                                                                                                \
    auto kern = gemm_umma_bkn_kernel<128, EPI, F32>;                                               \
    PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
    kern<<<ctas, kGemmThreads, smem, s>>>(ta, tb, p);                                              \
  }
  if (epilogue == kEpiSilu) { if (out_f32) PKB_BKN(kEpiSilu, true) else PKB_BKN(kEpiSilu, false) }
  else { if (out_f32) PKB_BKN(kEpiNone, true) else PKB_BKN(kEpiNone, false) }
#undef PKB_BKN
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// C[M,N] = alpha * A^T B with A [K, M] and B [K, N] row-major (lda, ldb in elements; M, N, K % 8 == 0).
// The natural form of a weight gradient (dW = dY^T X): no transposed copy of either operand.
extern "C" int pkb_gemm_bf16_tn(const void* a, long long lda, const void* b, long long ldb, void* c,
                                long long ldc, int M, int N, int K, float alpha, int out_f32, void* stream) {
  PKB_CHECK_ARG(M > 0 && N > 0 && K > 0, "empty problem");
  PKB_CHECK_ARG(lda % 8 == 0 && ldb % 8 == 0 && M % 8 == 0 && N % 8 == 0, "lda, ldb, M, N must be multiples of 8");
  CUtensorMap ta, tb;
  int rc = encode_tmap_2d(&ta, kTmapBf16, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, kGemmBlockK, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_2d(&tb, kTmapBf16, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, kGemmBlockK, kSwizzle128);
  if (rc) return rc;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K; p.C = c; p.ldc = ldc; p.alpha = alpha;
  p.status = status_block_device_ptr();
  p.wait_budget_ns = kDefaultWaitBudgetNs;
  p.group_m = 16; p.kernel_id = 104; p.world = 1;
  const int tiles = ((M + 127) / 128) * ((N + 255) / 256);
  int ctas = sm_count();
  if (ctas > tiles) ctas = tiles;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (pair_mn_enabled() && M >= 256 && N >= 256)
    return out_f32 ? launch_pair_mn<kEpiNone, true, true, true>(ta, tb, p, M, N, s) : launch_pair_mn<kEpiNone, false, true, true>(ta, tb, p, M, N, s);
  constexpr int smem = GemmSmem<256>::kTotal;
  if (out_f32) {
    auto kern = gemm_umma_tn_kernel<256, true>;
    PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<ctas, kGemmThreads, smem, s>>>(ta, tb, p);
  } else {
    auto kern = gemm_umma_tn_kernel<256, false>;
    PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<ctas, kGemmThreads, smem, s>>>(ta, tb, p);
  }
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}
