// Host-side helpers shared by every translation unit of the CUDA library: error capture (the C
// API returns int codes and keeps the last message in a thread-local string; it never throws
// across the C boundary), the per-device status block, and CUtensorMap encoding.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <string>

namespace pkb {

enum ApiCode : int {
  kApiOk = 0,
  kApiCudaError = 1,
  kApiBadArgument = 2,
  kApiUnsupported = 3,
  kApiDeviceStatus = 4,  // a kernel recorded a non-zero status word (time-out, ...)
};

void set_last_error(const std::string& msg);
const char* last_error_cstr();

#define PKB_CHECK_CUDA(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess) {                                                              \
      char _buf[512];                                                                     \
      snprintf(_buf, sizeof(_buf), "%s:%d: %s failed: %s", __FILE__, __LINE__, #expr,      \
               cudaGetErrorString(_e));                                                   \
      ::pkb::set_last_error(_buf);                                                        \
      return ::pkb::kApiCudaError;                                                        \
    }                                                                                     \
  } while (0)

#define PKB_CHECK_ARG(cond, msg)                                                          \
  do {                                                                                    \
    if (!(cond)) {                                                                        \
      char _buf[512];                                                                     \
      snprintf(_buf, sizeof(_buf), "%s:%d: bad argument: %s (%s)", __FILE__, __LINE__, msg, \
               #cond);                                                                    \
      ::pkb::set_last_error(_buf);                                                        \
      return ::pkb::kApiBadArgument;                                                      \
    }                                                                                     \
  } while (0)

// Device pointer of the current device's status block (kStatusWords uint32 in mapped pinned host
// memory, so the host can read it after any synchronisation without a copy). nullptr on failure.
uint32_t* status_block_device_ptr();

enum TmapDtype : int { kTmapBf16 = 0, kTmapFp8 = 1, kTmapFp32 = 2, kTmapU8 = 3, kTmapFp16 = 4 };
enum TmapSwizzle : int { kSwizzleNone = 0, kSwizzle32 = 1, kSwizzle64 = 2, kSwizzle128 = 3 };

// Encode a 2-D row-major tensor map: `inner` contiguous elements per row, `outer` rows,
// `row_stride_bytes` between rows (multiple of 16), box = box_inner x box_outer elements.
// Out-of-range parts of a box read as zero. Returns an ApiCode.
int encode_tmap_2d(CUtensorMap* out, int dtype, const void* base, uint64_t inner, uint64_t outer,
                   uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle);
// 3-D variant: dims (inner, mid, outer) with byte strides for mid and outer.
int encode_tmap_3d(CUtensorMap* out, int dtype, const void* base, uint64_t inner, uint64_t mid,
                   uint64_t outer, uint64_t mid_stride_bytes, uint64_t outer_stride_bytes,
                   uint32_t box_inner, uint32_t box_mid, uint32_t box_outer, int swizzle);

int sm_count();

}  // namespace pkb
