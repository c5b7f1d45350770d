// Symmetric heap over CUDA virtual memory management.
//
// Every rank creates one physical allocation of `bytes` on its GPU (cuMemCreate, shareable as a
// POSIX file descriptor), hands the descriptor to its peers (the Python side passes descriptors
// over unix sockets), imports the peers' allocations and maps all of them into one contiguous
// virtual range:   va_base + p * stride  is rank p's memory, for p = 0..world-1, on every rank.
// A kernel therefore reaches the same offset on any peer with one multiply-add, and P2P loads and
// stores travel over NVLink/NVSwitch.
//
// Optionally the ranks bind their allocations to one NVSwitch multicast object (cuMulticast*):
// a store to mc_base + offset lands in every rank's memory at that offset and multimem.ld_reduce
// reads the in-switch sum. Multicast mappings are only ever the target of multimem instructions
// and plain stores, never of TMA loads.
//
// The driver API is reached through cudaGetDriverEntryPoint, so this library has no link-time
// dependency on libcuda and still loads on a machine without a GPU driver.
#include <string.h>
#include <unistd.h>

#include <vector>

#include "pkb/api.h"
#include "pkb/host.h"

namespace pkb {

struct DriverApi {
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*,
                                          CUmemAllocationGranularity_flags);
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*,
                        unsigned long long);
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle,
                                         CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*,
                                           CUmemAllocationHandleType);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle,
                     unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle,
                               size_t, size_t, unsigned long long);
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*,
                                      CUmulticastGranularity_flags);
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  CUresult (*GetErrorString)(CUresult, const char**);
  bool ok = false;
};

static bool load_sym(const char* name, void** out) {
  cudaDriverEntryPointQueryResult q;
  return cudaGetDriverEntryPoint(name, out, cudaEnableDefault, &q) == cudaSuccess &&
         q == cudaDriverEntryPointSuccess && *out != nullptr;
}

static DriverApi& driver() {
  static DriverApi d;
  static bool tried = false;
  if (!tried) {
    tried = true;
    bool ok = true;
#define PKB_LOAD(field, name) ok = load_sym(name, reinterpret_cast<void**>(&d.field)) && ok
    PKB_LOAD(MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
    PKB_LOAD(MemCreate, "cuMemCreate");
    PKB_LOAD(MemExportToShareableHandle, "cuMemExportToShareableHandle");
    PKB_LOAD(MemImportFromShareableHandle, "cuMemImportFromShareableHandle");
    PKB_LOAD(MemAddressReserve, "cuMemAddressReserve");
    PKB_LOAD(MemAddressFree, "cuMemAddressFree");
    PKB_LOAD(MemMap, "cuMemMap");
    PKB_LOAD(MemUnmap, "cuMemUnmap");
    PKB_LOAD(MemSetAccess, "cuMemSetAccess");
    PKB_LOAD(MemRelease, "cuMemRelease");
    PKB_LOAD(MulticastCreate, "cuMulticastCreate");
    PKB_LOAD(MulticastAddDevice, "cuMulticastAddDevice");
    PKB_LOAD(MulticastBindMem, "cuMulticastBindMem");
    PKB_LOAD(MulticastUnbind, "cuMulticastUnbind");
    PKB_LOAD(MulticastGetGranularity, "cuMulticastGetGranularity");
    PKB_LOAD(DeviceGetAttribute, "cuDeviceGetAttribute");
    PKB_LOAD(GetErrorString, "cuGetErrorString");
#undef PKB_LOAD
    d.ok = ok;
  }
  return d;
}

#define PKB_CHECK_DRV(expr)                                                                 \
  do {                                                                                      \
    CUresult _r = (expr);                                                                   \
    if (_r != CUDA_SUCCESS) {                                                               \
      const char* _s = nullptr;                                                             \
      driver().GetErrorString(_r, &_s);                                                     \
      char _buf[512];                                                                       \
      snprintf(_buf, sizeof(_buf), "%s:%d: %s failed: %d (%s)", __FILE__, __LINE__, #expr,   \
               (int)_r, _s ? _s : "?");                                                     \
      set_last_error(_buf);                                                                 \
      return kApiCudaError;                                                                 \
    }                                                                                       \
  } while (0)

constexpr int kMaxWorld = 16;

struct Heap {
  int rank = 0, world = 1, device = 0;
  size_t bytes = 0;   // per-rank size (multiple of the granularity)
  size_t stride = 0;  // distance between consecutive ranks in the virtual range (== bytes)
  CUdeviceptr va_base = 0;
  CUmemGenericAllocationHandle local = 0;
  CUmemGenericAllocationHandle peers[kMaxWorld] = {0};
  bool mapped[kMaxWorld] = {false};
  int local_fd = -1;
  // multicast
  CUmemGenericAllocationHandle mc = 0;
  CUdeviceptr mc_va = 0;
  bool mc_bound = false, mc_mapped = false, mc_device_added = false;
  int mc_fd = -1;
};

static std::vector<Heap*> g_heaps;

static Heap* get_heap(int h) {
  if (h < 0 || h >= (int)g_heaps.size() || g_heaps[h] == nullptr) return nullptr;
  return g_heaps[h];
}

static CUmemAllocationProp alloc_prop(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

static int set_access(CUdeviceptr va, size_t bytes, int device) {
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  PKB_CHECK_DRV(driver().MemSetAccess(va, bytes, &acc, 1));
  return kApiOk;
}

}  // namespace pkb

using namespace pkb;

extern "C" {

// Whether this device supports NVSwitch multicast objects (1/0), or <0 on error.
int pkb_heap_multicast_supported() {
  if (!driver().ok) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  int v = 0;
  if (driver().DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS)
    return 0;
  return v;
}

// Round `bytes` up to what both the allocation and (if requested) the multicast granularity need.
long long pkb_heap_round_size(long long bytes, int world, int with_multicast) {
  if (!driver().ok) return -1;
  int dev = 0;
  cudaGetDevice(&dev);
  CUmemAllocationProp prop = alloc_prop(dev);
  size_t gran = 0;
  if (driver().MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) !=
      CUDA_SUCCESS)
    return -1;
  if (with_multicast) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = world;
    mp.size = (size_t)bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (driver().MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) ==
            CUDA_SUCCESS &&
        mg > gran)
      gran = mg;
  }
  size_t b = ((size_t)bytes + gran - 1) / gran * gran;
  return (long long)b;
}

// Create the local allocation (ALLOCATES device memory: `bytes`, already rounded) and reserve the
// world-wide virtual range. Returns a heap handle >= 0, or -1. *out_fd receives the shareable fd.
int pkb_heap_create(long long bytes, int rank, int world, int* out_fd) {
  if (!driver().ok) {
    set_last_error("CUDA driver entry points unavailable");
    return -1;
  }
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || bytes <= 0) {
    set_last_error("pkb_heap_create: bad rank/world/bytes");
    return -1;
  }
  cudaFree(0);  // make sure the primary context exists
  Heap* h = new Heap();
  h->rank = rank;
  h->world = world;
  cudaGetDevice(&h->device);
  h->bytes = (size_t)bytes;
  h->stride = (size_t)bytes;
  CUmemAllocationProp prop = alloc_prop(h->device);
  auto fail = [&](const char* what, CUresult r) {
    const char* s = nullptr;
    driver().GetErrorString(r, &s);
    char buf[256];
    snprintf(buf, sizeof(buf), "pkb_heap_create: %s failed: %d (%s)", what, (int)r, s ? s : "?");
    set_last_error(buf);
    delete h;
    return -1;
  };
  CUresult r = driver().MemCreate(&h->local, h->bytes, &prop, 0);
  if (r != CUDA_SUCCESS) return fail("cuMemCreate", r);
  r = driver().MemExportToShareableHandle(&h->local_fd, h->local,
                                          CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) return fail("cuMemExportToShareableHandle", r);
  r = driver().MemAddressReserve(&h->va_base, h->stride * world, 0, 0, 0);
  if (r != CUDA_SUCCESS) return fail("cuMemAddressReserve", r);
  r = driver().MemMap(h->va_base + h->stride * rank, h->bytes, 0, h->local, 0);
  if (r != CUDA_SUCCESS) return fail("cuMemMap(local)", r);
  h->mapped[rank] = true;
  if (set_access(h->va_base + h->stride * rank, h->bytes, h->device) != kApiOk) {
    delete h;
    return -1;
  }
  if (cudaMemset(reinterpret_cast<void*>(h->va_base + h->stride * rank), 0, h->bytes) !=
          cudaSuccess ||
      cudaDeviceSynchronize() != cudaSuccess) {
    set_last_error("pkb_heap_create: clearing the local allocation failed");
    delete h;
    return -1;
  }
  *out_fd = h->local_fd;
  g_heaps.push_back(h);
  return (int)g_heaps.size() - 1;
}

// Import the allocation of `peer` from a file descriptor received from that rank and map it.
int pkb_heap_import_peer(int heap, int peer, int fd) {
  Heap* h = get_heap(heap);
  PKB_CHECK_ARG(h != nullptr, "bad heap handle");
  PKB_CHECK_ARG(peer >= 0 && peer < h->world && peer != h->rank, "bad peer");
  PKB_CHECK_DRV(driver().MemImportFromShareableHandle(
      &h->peers[peer], reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
      CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  PKB_CHECK_DRV(driver().MemMap(h->va_base + h->stride * peer, h->bytes, 0, h->peers[peer], 0));
  h->mapped[peer] = true;
  return set_access(h->va_base + h->stride * peer, h->bytes, h->device);
}

unsigned long long pkb_heap_base(int heap) {
  Heap* h = get_heap(heap);
  return h ? (unsigned long long)h->va_base : 0ull;
}
unsigned long long pkb_heap_stride(int heap) {
  Heap* h = get_heap(heap);
  return h ? (unsigned long long)h->stride : 0ull;
}
unsigned long long pkb_heap_mc_base(int heap) {
  Heap* h = get_heap(heap);
  return (h && h->mc_mapped) ? (unsigned long long)h->mc_va : 0ull;
}

// ---- multicast (NVLS) -------------------------------------------------------------------------
// Rank 0: create the multicast object and export it; *out_fd receives the fd to send to peers.
int pkb_heap_mc_create(int heap, int* out_fd) {
  Heap* h = get_heap(heap);
  PKB_CHECK_ARG(h != nullptr, "bad heap handle");
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = h->world;
  mp.size = h->bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  PKB_CHECK_DRV(driver().MulticastCreate(&h->mc, &mp));
  PKB_CHECK_DRV(driver().MemExportToShareableHandle(&h->mc_fd, h->mc,
                                                    CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *out_fd = h->mc_fd;
  return kApiOk;
}
// Other ranks: import the multicast object from rank 0's descriptor.
int pkb_heap_mc_import(int heap, int fd) {
  Heap* h = get_heap(heap);
  PKB_CHECK_ARG(h != nullptr, "bad heap handle");
  PKB_CHECK_DRV(driver().MemImportFromShareableHandle(
      &h->mc, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
      CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  return kApiOk;
}
// Every rank: add its device. All ranks must have done this before anyone binds memory.
int pkb_heap_mc_add_device(int heap) {
  Heap* h = get_heap(heap);
  PKB_CHECK_ARG(h != nullptr && h->mc != 0, "no multicast object");
  PKB_CHECK_DRV(driver().MulticastAddDevice(h->mc, h->device));
  h->mc_device_added = true;
  return kApiOk;
}
// Every rank (after a barrier): bind the local allocation and map the multicast range.
int pkb_heap_mc_bind(int heap) {
  Heap* h = get_heap(heap);
  PKB_CHECK_ARG(h != nullptr && h->mc != 0, "no multicast object");
  PKB_CHECK_DRV(driver().MulticastBindMem(h->mc, 0, h->local, 0, h->bytes, 0));
  h->mc_bound = true;
  PKB_CHECK_DRV(driver().MemAddressReserve(&h->mc_va, h->bytes, 0, 0, 0));
  PKB_CHECK_DRV(driver().MemMap(h->mc_va, h->bytes, 0, h->mc, 0));
  h->mc_mapped = true;
  return set_access(h->mc_va, h->bytes, h->device);
}

// Tear down in the safe order: multicast mapping, multicast binding, peer mappings, local memory.
// The caller synchronises the device and all ranks (host barrier) before calling this.
int pkb_heap_destroy(int heap) {
  Heap* h = get_heap(heap);
  PKB_CHECK_ARG(h != nullptr, "bad heap handle");
  cudaDeviceSynchronize();
  if (h->mc_mapped) {
    driver().MemUnmap(h->mc_va, h->bytes);
    driver().MemAddressFree(h->mc_va, h->bytes);
  }
  if (h->mc_bound) driver().MulticastUnbind(h->mc, h->device, 0, h->bytes);
  if (h->mc) driver().MemRelease(h->mc);
  if (h->mc_fd >= 0) close(h->mc_fd);
  for (int p = 0; p < h->world; ++p) {
    if (h->mapped[p]) driver().MemUnmap(h->va_base + h->stride * p, h->bytes);
    if (p != h->rank && h->peers[p]) driver().MemRelease(h->peers[p]);
  }
  if (h->va_base) driver().MemAddressFree(h->va_base, h->stride * h->world);
  if (h->local) driver().MemRelease(h->local);
  if (h->local_fd >= 0) close(h->local_fd);
  delete h;
  g_heaps[heap] = nullptr;
  return kApiOk;
}

}  // extern "C"
