// CPU twin of the symmetric heap: ranks are processes on one host, the "heap" is a POSIX shared
// memory segment mapped by all of them (slab p at base + p * stride, same control-space layout as
// the GPU heap), flags are std::atomic<uint32_t> with acquire/release ordering, and the collectives
// run the same algorithms as the CUDA kernels (stage -> barrier -> read peers -> barrier).
//
// Purpose: (1) the no-GPU plumbing configuration (all-reduce, all-gather, reduce-scatter at world
// size 2 against gloo); (2) a place where the epoch/flag protocol can be stress-tested and where
// failures can be injected - a dropped signal, a late rank, a rank that never arrives - without
// touching a GPU. Every wait is bounded and reports which peer was missing.
#include <errno.h>
#include <sched.h>
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <string>
#include <vector>

namespace {

constexpr int kMaxWorld = 16;
constexpr int kMaxBlocks = 256;
constexpr int kChannels = 32;
constexpr uint64_t kFlagBytes = (uint64_t)kMaxBlocks * kMaxWorld * 4;
constexpr uint64_t kEpochBytes = (uint64_t)kMaxBlocks * 4;
constexpr uint64_t kChannelBytes = kFlagBytes + kEpochBytes;
constexpr uint64_t kCtrlBytes = 1ull << 20;

enum Code : int { kOk = 0, kError = 1, kTimeout = 2, kBadArgument = 3 };
enum Dtype : int { kBf16 = 0, kF32 = 1, kF64 = 2, kF16 = 3, kI32 = 4, kI64 = 5 };
enum Op : int { kSum = 0, kMax = 1, kMin = 2 };

struct Heap {
  std::string name;
  int rank = 0, world = 1;
  uint64_t stride = 0;
  uint8_t* base = nullptr;
  int fd = -1;
  // fault injection (host side only)
  int drop_signals = 0;  // number of upcoming barrier signals this rank silently skips
  int delay_ms = 0;      // sleep before every signal
  int last_missing_peer = -1;
};

thread_local std::string g_err;
std::vector<Heap*> g_heaps;

Heap* get(int h) { return (h >= 0 && h < (int)g_heaps.size()) ? g_heaps[h] : nullptr; }

uint64_t now_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + ts.tv_nsec;
}

void sleep_ms(int ms) {
  timespec ts{ms / 1000, (ms % 1000) * 1000000L};
  nanosleep(&ts, nullptr);
}

inline uint8_t* slab(Heap* h, int r) { return h->base + (uint64_t)r * h->stride; }

inline std::atomic<uint32_t>* flag(Heap* h, int owner, int channel, int block, int from) {
  return reinterpret_cast<std::atomic<uint32_t>*>(slab(h, owner) + (uint64_t)channel * kChannelBytes) +
         block * kMaxWorld + from;
}
inline uint32_t* epoch(Heap* h, int channel, int block) {
  return reinterpret_cast<uint32_t*>(slab(h, h->rank) + (uint64_t)channel * kChannelBytes + kFlagBytes) + block;
}

int barrier(Heap* h, const int* members, int gsize, int channel, int timeout_ms) {
  const uint32_t e = ++(*epoch(h, channel, 0));
  if (h->delay_ms > 0) sleep_ms(h->delay_ms);
  if (h->drop_signals > 0) {
    --h->drop_signals;  // injected fault: this rank "forgets" to signal
  } else {
    for (int g = 0; g < gsize; ++g) flag(h, members[g], channel, 0, h->rank)->store(e, std::memory_order_release);
  }
  const uint64_t t0 = now_ns();
  for (int g = 0; g < gsize; ++g) {
    std::atomic<uint32_t>* f = flag(h, h->rank, channel, 0, members[g]);
    uint32_t spins = 0;
    while ((int32_t)(f->load(std::memory_order_acquire) - e) < 0) {
      if ((++spins & 0xff) == 0) {
        if (now_ns() - t0 > (uint64_t)timeout_ms * 1000000ull) {
          h->last_missing_peer = members[g];
          char buf[128];
          snprintf(buf, sizeof(buf), "barrier time-out: rank %d waited %d ms for rank %d (epoch %u)", h->rank,
                   timeout_ms, members[g], e);
          g_err = buf;
          return kTimeout;
        }
        sched_yield();
      }
    }
  }
  return kOk;
}

float bf16_to_f(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
uint16_t f_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // NaN
  u += 0x7fffu + ((u >> 16) & 1u);                                             // round to nearest even
  return (uint16_t)(u >> 16);
}

int esize(int dt) {
  switch (dt) {
    case kBf16: case kF16: return 2;
    case kF32: case kI32: return 4;
    case kF64: case kI64: return 8;
  }
  return 0;
}

template <typename T>
T comb(T a, T b, int op) { return op == kSum ? a + b : (op == kMax ? (a > b ? a : b) : (a < b ? a : b)); }

template <typename T>
void reduce_typed(Heap* h, const int* members, int gsize, uint64_t off, long long n, T* out, int op, double scale) {
  for (long long i = 0; i < n; ++i) {
    T acc = reinterpret_cast<const T*>(slab(h, members[0]) + off)[i];
    for (int g = 1; g < gsize; ++g) acc = comb<T>(acc, reinterpret_cast<const T*>(slab(h, members[g]) + off)[i], op);
    if (scale != 1.0) acc = (T)(acc * scale);
    out[i] = acc;
  }
}

void reduce_bf16(Heap* h, const int* members, int gsize, uint64_t off, long long n, uint16_t* out, int op, double scale) {
  for (long long i = 0; i < n; ++i) {
    float acc = bf16_to_f(reinterpret_cast<const uint16_t*>(slab(h, members[0]) + off)[i]);
    for (int g = 1; g < gsize; ++g)
      acc = comb<float>(acc, bf16_to_f(reinterpret_cast<const uint16_t*>(slab(h, members[g]) + off)[i]), op);
    if (scale != 1.0) acc = (float)(acc * scale);
    out[i] = f_to_bf16(acc);
  }
}

}  // namespace

extern "C" {

const char* pkbh_last_error() { return g_err.c_str(); }
int pkbh_last_missing_peer(int heap) { Heap* h = get(heap); return h ? h->last_missing_peer : -1; }
unsigned long long pkbh_ctrl_bytes() { return kCtrlBytes; }

// Map (rank 0: create) the shared segment `name` of world * bytes. Returns a handle >= 0 or -1.
int pkbh_heap_create(const char* name, int rank, int world, long long bytes, int timeout_ms) {
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || bytes < (long long)kCtrlBytes) {
    g_err = "pkbh_heap_create: bad arguments";
    return -1;
  }
  Heap* h = new Heap();
  h->name = name;
  h->rank = rank;
  h->world = world;
  h->stride = (uint64_t)bytes;
  const uint64_t total = (uint64_t)bytes * world;
  if (rank == 0) {
    shm_unlink(name);
    h->fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
    if (h->fd < 0 || ftruncate(h->fd, (off_t)total) != 0) {
      g_err = std::string("shm_open/ftruncate failed: ") + strerror(errno);
      delete h;
      return -1;
    }
  } else {
    const uint64_t t0 = now_ns();
    for (;;) {
      h->fd = shm_open(name, O_RDWR, 0600);
      if (h->fd >= 0) {
        struct stat st;
        if (fstat(h->fd, &st) == 0 && (uint64_t)st.st_size >= total) break;
        close(h->fd);
        h->fd = -1;
      }
      if (now_ns() - t0 > (uint64_t)timeout_ms * 1000000ull) {
        g_err = "pkbh_heap_create: timed out waiting for rank 0 to create the segment";
        delete h;
        return -1;
      }
      sleep_ms(2);
    }
  }
  void* p = mmap(nullptr, total, PROT_READ | PROT_WRITE, MAP_SHARED, h->fd, 0);
  if (p == MAP_FAILED) {
    g_err = std::string("mmap failed: ") + strerror(errno);
    delete h;
    return -1;
  }
  h->base = static_cast<uint8_t*>(p);
  g_heaps.push_back(h);
  return (int)g_heaps.size() - 1;
}

void* pkbh_heap_local(int heap) { Heap* h = get(heap); return h ? slab(h, h->rank) : nullptr; }
void* pkbh_heap_peer(int heap, int r) { Heap* h = get(heap); return (h && r >= 0 && r < h->world) ? slab(h, r) : nullptr; }

int pkbh_heap_close(int heap, int unlink_segment) {
  Heap* h = get(heap);
  if (!h) return kBadArgument;
  munmap(h->base, h->stride * h->world);
  close(h->fd);
  if (unlink_segment) shm_unlink(h->name.c_str());
  delete h;
  g_heaps[heap] = nullptr;
  return kOk;
}

// fault injection, host side only
int pkbh_debug_drop_signals(int heap, int count) { Heap* h = get(heap); if (!h) return kBadArgument; h->drop_signals = count; return kOk; }
int pkbh_debug_delay_ms(int heap, int ms) { Heap* h = get(heap); if (!h) return kBadArgument; h->delay_ms = ms; return kOk; }

int pkbh_barrier(int heap, const int* members, int gsize, int channel, int timeout_ms) {
  Heap* h = get(heap);
  if (!h || gsize < 1 || gsize > kMaxWorld || channel < 0 || channel >= kChannels) return kBadArgument;
  return barrier(h, members, gsize, channel, timeout_ms);
}

// stage `stage_elems` from src into the heap at stage_off, barrier, reduce n elements starting at
// in_base from every member into out (if active), barrier.
int pkbh_reduce(int heap, const int* members, int gsize, int channel, int dtype, int op, const void* src,
                long long stage_elems, unsigned long long stage_off, long long in_base, long long n, void* out,
                int active, double scale, int timeout_ms) {
  Heap* h = get(heap);
  const int es = esize(dtype);
  if (!h || es == 0 || stage_off < kCtrlBytes || stage_off + (uint64_t)stage_elems * es > h->stride) {
    g_err = "pkbh_reduce: bad arguments";
    return kBadArgument;
  }
  if (stage_elems > 0) memcpy(slab(h, h->rank) + stage_off, src, (size_t)stage_elems * es);
  if (int rc = barrier(h, members, gsize, channel, timeout_ms)) return rc;
  if (active) {
    const uint64_t off = stage_off + (uint64_t)in_base * es;
    switch (dtype) {
      case kBf16: reduce_bf16(h, members, gsize, off, n, static_cast<uint16_t*>(out), op, scale); break;
      case kF32: reduce_typed<float>(h, members, gsize, off, n, static_cast<float*>(out), op, scale); break;
      case kF64: reduce_typed<double>(h, members, gsize, off, n, static_cast<double*>(out), op, scale); break;
      case kI32: reduce_typed<int32_t>(h, members, gsize, off, n, static_cast<int32_t*>(out), op, scale); break;
      case kI64: reduce_typed<int64_t>(h, members, gsize, off, n, static_cast<int64_t*>(out), op, scale); break;
      default: g_err = "pkbh_reduce: dtype not supported on the host"; return kBadArgument;
    }
  }
  return barrier(h, members, gsize, channel, timeout_ms);
}

// stage, barrier, copy seg_bytes from each member selected by src_mask (at in_base +
// in_member_stride * my group index) to out + k * out_stride, barrier.
int pkbh_gather(int heap, const int* members, int gsize, int grank, int channel, const void* src,
                long long stage_bytes, unsigned long long stage_off, unsigned int src_mask, long long in_base,
                long long in_member_stride, long long seg_bytes, void* out, long long out_stride, int active,
                int timeout_ms) {
  Heap* h = get(heap);
  if (!h || stage_off < kCtrlBytes || stage_off + (uint64_t)stage_bytes > h->stride) {
    g_err = "pkbh_gather: bad arguments";
    return kBadArgument;
  }
  if (stage_bytes > 0) memcpy(slab(h, h->rank) + stage_off, src, (size_t)stage_bytes);
  if (int rc = barrier(h, members, gsize, channel, timeout_ms)) return rc;
  if (active) {
    int k = 0;
    for (int g = 0; g < gsize; ++g) {
      if (!((src_mask >> g) & 1u)) continue;
      memcpy(static_cast<uint8_t*>(out) + (long long)k * out_stride,
             slab(h, members[g]) + stage_off + in_base + in_member_stride * grank, (size_t)seg_bytes);
      ++k;
    }
  }
  return barrier(h, members, gsize, channel, timeout_ms);
}

}  // extern "C"
