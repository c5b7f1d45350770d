// Runtime plumbing of the CUDA library: last-error string, per-device status block in mapped
// pinned memory, CUtensorMap encoding through the driver entry point (so the library links
// against nothing but the CUDA runtime), and a bounded-wait self test.
#include <mutex>
#include <string>

#include "pkb/api.h"
#include "pkb/host.h"
#include "pkb/ptx.cuh"

namespace pkb {

static thread_local std::string g_last_error;

void set_last_error(const std::string& msg) { g_last_error = msg; }
const char* last_error_cstr() { return g_last_error.c_str(); }

constexpr int kMaxDevices = 16;
static uint32_t* g_status_host[kMaxDevices] = {nullptr};
static uint32_t* g_status_dev[kMaxDevices] = {nullptr};
static int g_sm_count[kMaxDevices] = {0};
static std::mutex g_mu;

static int current_device() {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess) return -1;
  return d;
}

uint32_t* status_block_device_ptr() {
  int d = current_device();
  if (d < 0 || d >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status_dev[d] == nullptr) {
    void* h = nullptr;
    if (cudaHostAlloc(&h, kStatusWords * sizeof(uint32_t), cudaHostAllocMapped) != cudaSuccess)
      return nullptr;
    for (int i = 0; i < kStatusWords; ++i) static_cast<uint32_t*>(h)[i] = 0;
    void* dptr = nullptr;
    if (cudaHostGetDevicePointer(&dptr, h, 0) != cudaSuccess) {
      cudaFreeHost(h);
      return nullptr;
    }
    g_status_host[d] = static_cast<uint32_t*>(h);
    g_status_dev[d] = static_cast<uint32_t*>(dptr);
  }
  return g_status_dev[d];
}

int sm_count() {
  int d = current_device();
  if (d < 0 || d >= kMaxDevices) return 148;
  if (g_sm_count[d] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0)
      n = 148;
    g_sm_count[d] = n;
  }
  return g_sm_count[d];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

static bool tmap_types(int dtype, CUtensorMapDataType* t, uint32_t* esize) {
  switch (dtype) {
    case kTmapBf16: *t = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; *esize = 2; return true;
    case kTmapFp16: *t = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; *esize = 2; return true;
    case kTmapFp8:
    case kTmapU8: *t = CU_TENSOR_MAP_DATA_TYPE_UINT8; *esize = 1; return true;
    case kTmapFp32: *t = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; *esize = 4; return true;
  }
  return false;
}

static CUtensorMapSwizzle tmap_swizzle(int s) {
  switch (s) {
    case kSwizzle32: return CU_TENSOR_MAP_SWIZZLE_32B;
    case kSwizzle64: return CU_TENSOR_MAP_SWIZZLE_64B;
    case kSwizzle128: return CU_TENSOR_MAP_SWIZZLE_128B;
    default: return CU_TENSOR_MAP_SWIZZLE_NONE;
  }
}

int encode_tmap_2d(CUtensorMap* out, int dtype, const void* base, uint64_t inner, uint64_t outer,
                   uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                   int swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled entry point unavailable");
    return kApiCudaError;
  }
  CUtensorMapDataType t;
  uint32_t es;
  PKB_CHECK_ARG(tmap_types(dtype, &t, &es), "unknown tensor-map dtype");
  PKB_CHECK_ARG((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor base must be 16-byte aligned");
  PKB_CHECK_ARG((row_stride_bytes & 15) == 0, "row stride must be a multiple of 16 bytes");
  PKB_CHECK_ARG(box_inner * es % 16 == 0, "box inner extent must be a multiple of 16 bytes");
  PKB_CHECK_ARG(box_outer >= 1 && box_outer <= 256 && box_inner <= 256, "box extents out of range");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, t, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, tmap_swizzle(swizzle),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    snprintf(buf, sizeof(buf),
             "cuTensorMapEncodeTiled(2d) failed with %d (inner=%llu outer=%llu stride=%llu box=%ux%u)",
             (int)r, (unsigned long long)inner, (unsigned long long)outer,
             (unsigned long long)row_stride_bytes, box_inner, box_outer);
    set_last_error(buf);
    return kApiCudaError;
  }
  return kApiOk;
}

int encode_tmap_3d(CUtensorMap* out, int dtype, const void* base, uint64_t inner, uint64_t mid,
                   uint64_t outer, uint64_t mid_stride_bytes, uint64_t outer_stride_bytes,
                   uint32_t box_inner, uint32_t box_mid, uint32_t box_outer, int swizzle) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled entry point unavailable");
    return kApiCudaError;
  }
  CUtensorMapDataType t;
  uint32_t es;
  PKB_CHECK_ARG(tmap_types(dtype, &t, &es), "unknown tensor-map dtype");
  PKB_CHECK_ARG((reinterpret_cast<uintptr_t>(base) & 15) == 0, "tensor base must be 16-byte aligned");
  PKB_CHECK_ARG((mid_stride_bytes & 15) == 0 && (outer_stride_bytes & 15) == 0,
                "strides must be multiples of 16 bytes");
  PKB_CHECK_ARG(box_inner * es % 16 == 0, "box inner extent must be a multiple of 16 bytes");
  cuuint64_t dims[3] = {inner, mid, outer};
  cuuint64_t strides[2] = {mid_stride_bytes, outer_stride_bytes};
  cuuint32_t box[3] = {box_inner, box_mid, box_outer};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, t, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, tmap_swizzle(swizzle),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[256];
    snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled(3d) failed with %d", (int)r);
    set_last_error(buf);
    return kApiCudaError;
  }
  return kApiOk;
}

// A kernel that waits on a flag nobody sets: exercises the bounded-wait path end to end.
__global__ void stamp_globaltimer_kernel(unsigned long long* out) { *out = globaltimer_ns(); }

__global__ void wait_selftest_kernel(const uint32_t* flag, uint32_t target, uint64_t budget_ns,
                                     uint32_t* status, uint32_t* out_elapsed_us) {
  const uint64_t t0 = globaltimer_ns();
  bool ok = wait_flag_ge(flag, target, budget_ns);
  if (!ok) record_status(status, kStatusPeerTimeout, /*kernel_id=*/900, 0, 0, /*site=*/1, 0);
  *out_elapsed_us = static_cast<uint32_t>((globaltimer_ns() - t0) / 1000);
}

}  // namespace pkb

using namespace pkb;

extern "C" {

const char* pkb_last_error() { return last_error_cstr(); }

int pkb_version() { return 1; }

int pkb_status_read(uint32_t* out_words) {
  uint32_t* dptr = status_block_device_ptr();
  if (!dptr) {
    set_last_error("status block unavailable");
    return kApiCudaError;
  }
  int d = current_device();
  for (int i = 0; i < kStatusWords; ++i) out_words[i] = g_status_host[d][i];
  return kApiOk;
}

int pkb_status_clear() {
  uint32_t* dptr = status_block_device_ptr();
  if (!dptr) return kApiCudaError;
  int d = current_device();
  for (int i = 0; i < kStatusWords; ++i) g_status_host[d][i] = 0;
  return kApiOk;
}

// One thread writes the GPU's nanosecond timer to *out_ns (uint64, device memory) when the stream reaches this point:
// a device-side clock for cross-checking event timings.
int pkb_stamp_globaltimer(void* out_ns, void* stream) {
  PKB_CHECK_ARG(out_ns != nullptr && (reinterpret_cast<uintptr_t>(out_ns) & 7) == 0, "out_ns must be an 8-byte aligned device pointer");
  stamp_globaltimer_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<unsigned long long*>(out_ns));
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_wait_selftest(const void* flag, uint32_t target, uint64_t budget_ns, void* out_elapsed_us,
                      void* stream) {
  uint32_t* status = status_block_device_ptr();
  PKB_CHECK_ARG(status != nullptr, "status block unavailable");
  wait_selftest_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(flag), target, budget_ns, status,
      static_cast<uint32_t*>(out_elapsed_us));
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

}  // extern "C"
