// Allocation-free entry point. It has no counterpart in the reference benchmark: it exists for
// callers of this library that are not allowed to allocate device memory at the point of the call -
// code running inside a memory pool that has been frozen for the step, a plugin called from a host
// runtime that owns every byte of the GPU, or a latency-critical serving loop where an allocator
// call (and the implicit synchronisation it can cause) is not acceptable.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest number of rows one call may process (the scratch holds three floats per row).
#define PKB_CE_NOALLOC_MAX_ROWS 65536

// Per-row cross-entropy loss of `rows` rows of `vocab` logits against int64 targets:
//     loss[r] = logsumexp(logits[r, :]) - logits[r, target[r]]
// logits: [rows, vocab] bf16 (dtype 0) or fp32 (dtype 1), row-major; target: [rows] int64;
// loss: [rows] fp32. All three are device pointers supplied by the caller; `stream` is a
// cudaStream_t. Returns 0 on success, a non-zero pkb::ApiCode otherwise (pkb_last_error() has the
// text); rows > PKB_CE_NOALLOC_MAX_ROWS is rejected with a bad-argument error.
//
// The per-row statistics that the two-kernel form keeps in a caller-allocated buffer live here in a
// fixed array inside the library image (768 KiB of every GPU that loads the library, until the
// process exits). The call itself allocates and frees nothing: no cudaMalloc, no cudaFree, no
// library routine that allocates.
//
// * The first call on a device looks up the device address of that array (once per device, with
//   that device current). With lazy module loading that lookup can also be what makes the driver
//   load the library's device code and back the array with memory, so "allocates nothing" holds
//   from the second call on each device: make the first call during warm-up, before the region in
//   which allocation is forbidden and before any stream capture begins.
// * Every call uses the same array. Two calls whose kernels may overlap on the GPU (different
//   streams, or different host threads without ordering) race on it: serialise them.
// * Nothing in the array has to start at zero; each call overwrites the entries it reads.
int pkb_ce_loss_noalloc(const void* logits, const void* target, void* loss, int rows, int vocab,
                        int dtype, void* stream);

#ifdef __cplusplus
}
#endif
