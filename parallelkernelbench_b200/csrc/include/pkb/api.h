// C API of libpkb200_cuda.so. Every function returns 0 on success or a pkb::ApiCode; the message
// of the last failure on the calling thread is available from pkb_last_error(). Pointers are raw
// device pointers, `stream` is a cudaStream_t passed as void*. Nothing here allocates device
// memory unless its comment says so.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* pkb_last_error();
int pkb_version();

// Per-device status block (16 uint32 words): word 0 is the first error code a kernel recorded.
int pkb_status_read(uint32_t* out_words);
int pkb_status_clear();
// Launch a one-thread kernel that waits (at most budget_ns) for *flag >= target.
int pkb_wait_selftest(const void* flag, uint32_t target, uint64_t budget_ns, void* out_elapsed_us,
                      void* stream);

// ---- dense GEMM (tcgen05): C[M,N] = epi(alpha * A[M,K] @ B[N,K]^T + bias) -------------------
// a, b: bf16 row-major with leading dimensions lda, ldb (elements, multiples of 8).
// out_f32: 0 -> C is bf16, 1 -> C is fp32. epilogue: 0 none, 1 SiLU, 2 bias, 3 bias + SiLU.
// block_n: 128 or 256 (0 = choose). num_ctas: 0 = one per SM.
int pkb_gemm_bf16(const void* a, long long lda, const void* b, long long ldb, void* c,
                  long long ldc, int M, int N, int K, const void* bias, float alpha, int epilogue,
                  int out_f32, int block_n, int num_ctas, void* stream);

// ---- normalisation / elementwise ------------------------------------------------------------
// y = x * rsqrt(mean(x^2) + eps) * gamma; x, y, gamma bf16; rows x cols (cols % 8 == 0).
int pkb_rmsnorm_bf16(const void* x, const void* gamma, void* y, int rows, int cols, float eps,
                     void* stream);
// sums `nsrc` row-major bf16 (or fp32) partial buffers (src + i*src_stride_elems), optionally
// scales by `scale`, applies RMSNorm with gamma, writes bf16.
int pkb_sum_rmsnorm(const void* src, long long src_stride_elems, int nsrc, int src_is_f32,
                    const void* gamma, void* y, int rows, int cols, float scale, float eps,
                    void* stream);

#ifdef __cplusplus
}
#endif
