// Collectives over the symmetric heap: every kernel stages its input into this rank's heap
// (unless it already lives there), crosses one in-kernel barrier, and then reads its peers'
// memory directly over NVLink with 16-byte loads. There are no rings: NVSwitch gives every pair
// full bandwidth, so each rank talks to all peers at once.
//
//   reduce family  (all-reduce one-shot, reduce-scatter, reduce-to-root): sum/max/min in fp32/fp64
//                  in a fixed member order, so every rank computes bit-identical results
//   gather family  (all-gather, all-to-all, broadcast, scatter, gather-to-root): byte copies
//   two-shot all-reduce: reduce own slice, publish it, gather the other slices
//   NVLS all-reduce: multimem.ld_reduce of the own slice, multimem.st of the result to everyone
//   all-to-all-v: per-destination counts and offsets travel through the heap; nothing returns
//                 to the host
// They replace the NCCL calls of the reference's collective problems
// (reference: reference/1_allreduce.py:8 ... reference/8_alltoall.py:8) and the example kernels
// (reference: kernelgen/solution_new_add_cuda.py:16-26,
//  kernelgen/solutions_new_allreduce_parallelkittens.py:31-69).
#include "pkb/api.h"
#include "pkb/collectives_api.h"
#include "pkb/host.h"
#include "pkb/bulk_copy.cuh"
#include "pkb/symm_host.h"

namespace pkb {

constexpr int kCollThreads = 512;

enum CollDtype : int { kCollBf16 = 0, kCollF32 = 1, kCollF64 = 2, kCollF16 = 3, kCollI32 = 4, kCollI64 = 5 };
enum CollOp : int { kCollSum = 0, kCollMax = 1, kCollMin = 2 };

template <int OP, typename A>
__device__ __forceinline__ A combine(A a, A b) {
  if constexpr (OP == kCollSum) return a + b;
  else if constexpr (OP == kCollMax) return a > b ? a : b;
  else return a < b ? a : b;
}

// ---- 16-byte packs per dtype: unpack to an accumulator array, combine, pack ------------------
template <int DT> struct Pack;
template <> struct Pack<kCollBf16> {
  using Acc = float; static constexpr int kN = 8; static constexpr int kElem = 2;
  static __device__ __forceinline__ void unpack(const U4& u, Acc* a) {
    float2 f;
    f = unpack_bf16x2(u.x); a[0] = f.x; a[1] = f.y;
    f = unpack_bf16x2(u.y); a[2] = f.x; a[3] = f.y;
    f = unpack_bf16x2(u.z); a[4] = f.x; a[5] = f.y;
    f = unpack_bf16x2(u.w); a[6] = f.x; a[7] = f.y;
  }
  static __device__ __forceinline__ U4 pack(const Acc* a) {
    return U4{pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]),
              pack_bf16x2(a[6], a[7])};
  }
  static __device__ __forceinline__ Acc load1(const void* p, long long i) {
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  }
  static __device__ __forceinline__ void store1(void* p, long long i, Acc v) {
    static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  }
};
template <> struct Pack<kCollF16> {
  using Acc = float; static constexpr int kN = 8; static constexpr int kElem = 2;
  static __device__ __forceinline__ void unpack(const U4& u, Acc* a) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); a[2 * i] = f.x; a[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ U4 pack(const Acc* a) {
    U4 u; __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(a[2 * i], a[2 * i + 1]);
    return u;
  }
  static __device__ __forceinline__ Acc load1(const void* p, long long i) {
    return __half2float(static_cast<const __half*>(p)[i]);
  }
  static __device__ __forceinline__ void store1(void* p, long long i, Acc v) {
    static_cast<__half*>(p)[i] = __float2half_rn(v);
  }
};
template <> struct Pack<kCollF32> {
  using Acc = float; static constexpr int kN = 4; static constexpr int kElem = 4;
  static __device__ __forceinline__ void unpack(const U4& u, Acc* a) {
    a[0] = __uint_as_float(u.x); a[1] = __uint_as_float(u.y);
    a[2] = __uint_as_float(u.z); a[3] = __uint_as_float(u.w);
  }
  static __device__ __forceinline__ U4 pack(const Acc* a) {
    return U4{__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]), __float_as_uint(a[3])};
  }
  static __device__ __forceinline__ Acc load1(const void* p, long long i) { return static_cast<const float*>(p)[i]; }
  static __device__ __forceinline__ void store1(void* p, long long i, Acc v) { static_cast<float*>(p)[i] = v; }
};
template <> struct Pack<kCollF64> {
  using Acc = double; static constexpr int kN = 2; static constexpr int kElem = 8;
  static __device__ __forceinline__ void unpack(const U4& u, Acc* a) {
    a[0] = __hiloint2double((int)u.y, (int)u.x); a[1] = __hiloint2double((int)u.w, (int)u.z);
  }
  static __device__ __forceinline__ U4 pack(const Acc* a) {
    return U4{(uint32_t)__double2loint(a[0]), (uint32_t)__double2hiint(a[0]),
              (uint32_t)__double2loint(a[1]), (uint32_t)__double2hiint(a[1])};
  }
  static __device__ __forceinline__ Acc load1(const void* p, long long i) { return static_cast<const double*>(p)[i]; }
  static __device__ __forceinline__ void store1(void* p, long long i, Acc v) { static_cast<double*>(p)[i] = v; }
};
template <> struct Pack<kCollI32> {
  using Acc = int; static constexpr int kN = 4; static constexpr int kElem = 4;
  static __device__ __forceinline__ void unpack(const U4& u, Acc* a) { a[0] = u.x; a[1] = u.y; a[2] = u.z; a[3] = u.w; }
  static __device__ __forceinline__ U4 pack(const Acc* a) { return U4{(uint32_t)a[0], (uint32_t)a[1], (uint32_t)a[2], (uint32_t)a[3]}; }
  static __device__ __forceinline__ Acc load1(const void* p, long long i) { return static_cast<const int*>(p)[i]; }
  static __device__ __forceinline__ void store1(void* p, long long i, Acc v) { static_cast<int*>(p)[i] = v; }
};
template <> struct Pack<kCollI64> {
  using Acc = long long; static constexpr int kN = 2; static constexpr int kElem = 8;
  static __device__ __forceinline__ void unpack(const U4& u, Acc* a) {
    a[0] = (long long)(((unsigned long long)u.y << 32) | u.x); a[1] = (long long)(((unsigned long long)u.w << 32) | u.z);
  }
  static __device__ __forceinline__ U4 pack(const Acc* a) {
    return U4{(uint32_t)a[0], (uint32_t)((unsigned long long)a[0] >> 32), (uint32_t)a[1], (uint32_t)((unsigned long long)a[1] >> 32)};
  }
  static __device__ __forceinline__ Acc load1(const void* p, long long i) { return static_cast<const long long*>(p)[i]; }
  static __device__ __forceinline__ void store1(void* p, long long i, Acc v) { static_cast<long long*>(p)[i] = v; }
};

// Copy `bytes` from src to dst with the whole grid (16-byte body, byte tail). Both 16-aligned or not.
__device__ __forceinline__ void grid_copy_bytes(void* dst, const void* src, long long bytes) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  if ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
    const long long nvec = bytes >> 4;
    const uint8_t* s8 = static_cast<const uint8_t*>(src);
    uint8_t* d8 = static_cast<uint8_t*>(dst);
    // four independent 16-byte loads in flight per thread: a peer load takes microseconds, so bandwidth over NVLink
    // is bytes in flight divided by that latency
    long long i = tid;
    for (; i + 3 * nthreads < nvec; i += 4 * nthreads) {
      const U4 a = ld_global_v4(s8 + (i << 4));
      const U4 b = ld_global_v4(s8 + ((i + nthreads) << 4));
      const U4 c = ld_global_v4(s8 + ((i + 2 * nthreads) << 4));
      const U4 e = ld_global_v4(s8 + ((i + 3 * nthreads) << 4));
      st_global_v4(d8 + (i << 4), a);
      st_global_v4(d8 + ((i + nthreads) << 4), b);
      st_global_v4(d8 + ((i + 2 * nthreads) << 4), c);
      st_global_v4(d8 + ((i + 3 * nthreads) << 4), e);
    }
    for (; i < nvec; i += nthreads) st_global_v4(d8 + (i << 4), ld_global_v4(s8 + (i << 4)));
    for (long long j = (nvec << 4) + tid; j < bytes; j += nthreads) d8[j] = s8[j];
  } else {
    for (long long i = tid; i < bytes; i += nthreads)
      static_cast<uint8_t*>(dst)[i] = static_cast<const uint8_t*>(src)[i];
  }
}

// Large aligned copies go through the TMA bulk ring (dynamic shared memory of kBulkSmemBytes), the rest through 16-byte
// loads. Every thread of every block calls init() once and copy() for each piece.
struct GridCopier {
  BulkRing ring;
  volatile int* abort_flag;
  uint64_t budget_ns;
  bool ok;
  __device__ __forceinline__ void init(uint8_t* smem, volatile int* abort_slot, uint64_t budget) {
    abort_flag = abort_slot;
    budget_ns = budget;
    ok = true;
    if (threadIdx.x == 0) {
      *abort_slot = 0;
      bulk_ring_init(ring, smem_u32(smem));
    }
    __syncthreads();
  }
  __device__ __forceinline__ void copy(void* dst, const void* src, long long bytes) {
    if (bulk_copy_eligible(dst, src, bytes)) {
      if (!grid_bulk_copy(ring, dst, src, bytes, abort_flag, budget_ns)) ok = false;
    } else {
      grid_copy_bytes(dst, src, bytes);
    }
  }
  // after copies whose result other ranks read behind a barrier / before bulk loads of data others wrote
  __device__ __forceinline__ void proxy_fence() {
    if (threadIdx.x == 0) fence_proxy_async_all();
  }
};

// ================================================================================================
// reduce family
// ================================================================================================
struct ReduceArgs {
  const void* src;        // local input (any device memory); staged into the heap if stage_elems > 0
  long long stage_elems;  // elements to copy from src to heap[stage_off]; 0: input already in heap
  uint64_t stage_off;     // heap offset of the (staged) input on every rank
  long long in_base;      // first element (in the peers' staged input) this rank reduces
  long long n;            // elements this rank reduces
  void* out;              // local output
  int active;             // 0: take part in the barriers only (non-root of a reduce-to-root)
  double scale;           // applied after the reduction (1/W for a mean)
};

template <int DT, int OP>
__global__ void __launch_bounds__(kCollThreads)
coll_reduce_kernel(const SymmCtx c, const ReduceArgs a) {
  using P = Pack<DT>;
  using Acc = typename P::Acc;
  if (a.stage_elems > 0)
    grid_copy_bytes(symm_local<uint8_t>(c, a.stage_off), a.src, a.stage_elems * P::kElem);
  if (!symm_grid_barrier(c, 200, 1)) return;
  if (a.active) {
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long nthreads = (long long)gridDim.x * blockDim.x;
    const uint64_t in_off = a.stage_off + (uint64_t)a.in_base * P::kElem;
    const bool vec_ok = ((in_off | (uintptr_t)a.out) & 15) == 0;
    const long long nvec = vec_ok ? a.n / P::kN : 0;
    for (long long i = tid; i < nvec; i += nthreads) {
      Acc acc[P::kN];
      P::unpack(ld_global_v4(symm_ptr<uint8_t>(c, c.members[0], in_off) + (i << 4)), acc);
      for (int g = 1; g < c.gsize; ++g) {
        Acc v[P::kN];
        P::unpack(ld_global_v4(symm_ptr<uint8_t>(c, c.members[g], in_off) + (i << 4)), v);
#pragma unroll
        for (int j = 0; j < P::kN; ++j) acc[j] = combine<OP>(acc[j], v[j]);
      }
      if (a.scale != 1.0) {
#pragma unroll
        for (int j = 0; j < P::kN; ++j) acc[j] = (Acc)(acc[j] * (Acc)a.scale);
      }
      st_global_v4(static_cast<uint8_t*>(a.out) + (i << 4), P::pack(acc));
    }
    for (long long i = nvec * P::kN + tid; i < a.n; i += nthreads) {
      Acc acc = P::load1(symm_ptr<uint8_t>(c, c.members[0], in_off), i);
      for (int g = 1; g < c.gsize; ++g)
        acc = combine<OP>(acc, P::load1(symm_ptr<uint8_t>(c, c.members[g], in_off), i));
      if (a.scale != 1.0) acc = (Acc)(acc * (Acc)a.scale);
      P::store1(a.out, i, acc);
    }
  }
  symm_block_barrier(c, 200, 2);
}

// ================================================================================================
// gather family
// ================================================================================================
struct GatherArgs {
  const void* src;
  long long stage_bytes;  // bytes to stage from src; 0: already in heap
  uint64_t stage_off;
  uint32_t src_mask;      // bit g set: read from group member g
  long long in_base;      // byte offset inside the member's staged buffer
  long long in_member_stride;  // extra byte offset per *reading* rank (all-to-all: chunk index = my grank)
  long long seg_bytes;    // bytes read from each selected member
  void* out;              // local output; segment k (k-th selected member) goes to out + k*out_stride
  long long out_stride;
  int active;
};

__global__ void __launch_bounds__(kCollThreads)
coll_gather_kernel(const SymmCtx c, const GatherArgs a) {
  // large, aligned pieces move through the TMA bulk ring (one request carries 16 KiB, so a few requests per SM fill
  // NVLink); everything else with 16-byte loads
  extern __shared__ __align__(128) uint8_t bulk_smem[];
  __shared__ int s_abort;
  BulkRing ring;
  if (threadIdx.x == 0) {
    s_abort = 0;
    bulk_ring_init(ring, smem_u32(bulk_smem));
  }
  __syncthreads();
  bool ok = true;
  auto copy = [&](void* dst, const void* src, long long bytes) {
    if (bulk_copy_eligible(dst, src, bytes)) {
      if (!grid_bulk_copy(ring, dst, src, bytes, &s_abort, c.budget_ns)) ok = false;
    } else {
      grid_copy_bytes(dst, src, bytes);
    }
  };
  if (a.stage_bytes > 0) copy(symm_local<uint8_t>(c, a.stage_off), a.src, a.stage_bytes);
  if (threadIdx.x == 0) fence_proxy_async_all();   // bulk stores of the staging are visible before the release below
  if (!symm_grid_barrier(c, 201, 1)) return;
  if (threadIdx.x == 0) fence_proxy_async_all();   // peers' writes are visible to the bulk loads issued below
  if (a.active) {
    int k = 0;
    for (int g = 0; g < c.gsize; ++g) {
      if (!((a.src_mask >> g) & 1u)) continue;
      const uint8_t* from = symm_ptr<uint8_t>(c, c.members[g], a.stage_off) + a.in_base +
                            a.in_member_stride * c.grank;
      copy(static_cast<uint8_t*>(a.out) + (long long)k * a.out_stride, from, a.seg_bytes);
      ++k;
    }
  }
  if (threadIdx.x == 0 && !ok) record_status(c.status, kStatusMbarTimeout, 201, c.rank, c.rank, 3, 0);
  symm_block_barrier(c, 201, 2);
}

// ================================================================================================
// remote row gather: out[i] = row (ids[i] % rows_per_member) of member (ids[i] / rows_per_member)
// ================================================================================================
struct RowGatherArgs {
  const void* src;          // local table shard, staged into the heap when stage_bytes > 0
  long long stage_bytes;
  uint64_t table_off;       // heap offset of every member's shard
  const long long* ids;     // [n] global row ids
  long long n;
  long long rows_per_member;
  long long row_bytes;
  void* out;                // [n, row_bytes]
  int sync;                 // 0: the table is resident and unchanged, no barrier needed
};

__global__ void __launch_bounds__(kCollThreads)
coll_row_gather_kernel(const SymmCtx c, const RowGatherArgs a) {
  if (a.stage_bytes > 0) grid_copy_bytes(symm_local<uint8_t>(c, a.table_off), a.src, a.stage_bytes);
  if (a.sync && !symm_grid_barrier(c, 207, 1)) return;
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const bool vec = ((a.row_bytes | a.table_off | (uintptr_t)a.out) & 15) == 0;
  for (long long i = warp; i < a.n; i += nwarps) {
    const long long id = a.ids[i];
    long long g = id / a.rows_per_member;
    uint8_t* dst = static_cast<uint8_t*>(a.out) + i * a.row_bytes;
    if (id < 0 || g >= c.gsize) {                       // out-of-range id: a row of zeros, never a wild load
      for (long long b = lane; b < a.row_bytes; b += 32) dst[b] = 0;
      continue;
    }
    const uint8_t* from = symm_ptr<uint8_t>(c, c.members[g], a.table_off) + (id - g * a.rows_per_member) * a.row_bytes;
    if (vec) {
      for (long long b = (long long)lane << 4; b < a.row_bytes; b += 32 << 4) st_global_v4(dst + b, ld_global_v4(from + b));
    } else {
      for (long long b = lane; b < a.row_bytes; b += 32) dst[b] = from[b];
    }
  }
  if (a.sync) symm_block_barrier(c, 207, 2);
}

// ================================================================================================
// all-to-all with a layout change: member g's block for me is a strided box of its staged tensor, and it
// lands as a strided box of my output (sequence <-> head exchanges, distributed transposes)
// ================================================================================================
struct A2APermArgs {
  const void* src;
  long long stage_bytes;
  uint64_t stage_off;
  long long in_rank_off;     // byte offset of the box addressed to member index r: r * in_rank_off
  long long n0, n1, n2;      // outer extents of the box
  long long in_s0, in_s1, in_s2;     // byte strides inside the sender's tensor
  long long out_member_off;  // byte offset of the box received from member index g: g * out_member_off
  long long out_s0, out_s1, out_s2;  // byte strides inside the output
  long long inner_bytes;     // contiguous bytes per (i0, i1, i2)
  void* out;
};

__global__ void __launch_bounds__(kCollThreads)
coll_a2a_perm_kernel(const SymmCtx c, const A2APermArgs a) {
  if (a.stage_bytes > 0) grid_copy_bytes(symm_local<uint8_t>(c, a.stage_off), a.src, a.stage_bytes);
  if (!symm_grid_barrier(c, 206, 1)) return;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long rows = a.n0 * a.n1 * a.n2;
  const bool vec = ((a.inner_bytes | a.in_rank_off | a.in_s0 | a.in_s1 | a.in_s2 | a.out_member_off | a.out_s0 | a.out_s1 |
                     a.out_s2 | (long long)a.stage_off | (long long)(uintptr_t)a.out) & 15) == 0;
  const long long unit = vec ? 16 : 1;
  const long long upr = a.inner_bytes / unit;   // units per row
  for (int k = 0; k < c.gsize; ++k) {
    const int g = (c.grank + k) % c.gsize;      // start with my own box, spread the peers over time
    const uint8_t* from = symm_ptr<uint8_t>(c, c.members[g], a.stage_off) + (long long)c.grank * a.in_rank_off;
    uint8_t* to = static_cast<uint8_t*>(a.out) + (long long)g * a.out_member_off;
    for (long long idx = tid; idx < rows * upr; idx += nthreads) {
      const long long row = idx / upr, u = idx - row * upr;
      const long long i2 = row % a.n2, t = row / a.n2, i1 = t % a.n1, i0 = t / a.n1;
      const long long so = i0 * a.in_s0 + i1 * a.in_s1 + i2 * a.in_s2 + u * unit;
      const long long dof = i0 * a.out_s0 + i1 * a.out_s1 + i2 * a.out_s2 + u * unit;
      if (vec) st_global_v4(to + dof, ld_global_v4(from + so));
      else to[dof] = from[so];
    }
  }
  symm_block_barrier(c, 206, 2);
}

// ================================================================================================
// all-to-all as a push: every block moves one slice of each outgoing chunk with the TMA unit, local memory -> shared-memory
// ring -> the receiver's buffer (cp.async.bulk loads of this GPU's memory, cp.async.bulk stores into the peer's). Stores over
// NVLink are posted, so the sender never waits a round trip, and the input needs no staging copy. The project's example
// all-to-all is built the same way from TMA loads and TMA stores into the destination device
// (reference: kernelgen/solutions_new_alltoall_parallelkittens.py:36-122).
// Slice b of a chunk is written by block b of the sender and copied out by block b of the receiver, so barriers between
// same-index blocks are enough: one before the first store (the receiver has finished reading its buffer in its previous
// call) and one after the last.
// ================================================================================================
struct A2APushArgs {
  const void* src;      // [gsize, chunk] local input, any device memory
  long long chunk;      // bytes per destination (multiple of 16)
  uint64_t recv_off;    // heap offset of the [gsize, chunk] receive buffer of every member
  void* out;            // local output; null when the receive buffer is the output
};

__global__ void __launch_bounds__(kCollThreads)
coll_a2a_push_kernel(const SymmCtx c, const A2APushArgs a) {
  extern __shared__ __align__(128) uint8_t bulk_smem[];
  __shared__ int s_abort;
  BulkRing ring;
  if (threadIdx.x == 0) {
    s_abort = 0;
    bulk_ring_init(ring, smem_u32(bulk_smem));
  }
  __syncthreads();
  if (!symm_block_barrier(c, 211, 1)) return;
  long long per = (a.chunk + gridDim.x - 1) / gridDim.x;
  per = (per + 1023) & ~1023ll;
  const long long b0 = per * blockIdx.x;
  const long long nb = b0 >= a.chunk ? 0 : (b0 + per <= a.chunk ? per : a.chunk - b0);
  const uint8_t* src = static_cast<const uint8_t*>(a.src);
  uint8_t* out = static_cast<uint8_t*>(a.out);
  if (threadIdx.x == 0 && nb > 0) {
    bool ok = true;
    for (int k = 0; k < c.gsize && ok; ++k) {
      const int g = (c.grank + k) % c.gsize;      // every member starts with its own chunk, then a different peer each
      uint8_t* to = (g == c.grank && out) ? out + (long long)g * a.chunk
                                          : symm_ptr<uint8_t>(c, c.members[g], a.recv_off) + (long long)c.grank * a.chunk;
      ok = bulk_copy(ring, to + b0, src + (long long)g * a.chunk + b0, nb, &s_abort, c.budget_ns);
    }
    fence_proxy_async_all();                      // the bulk stores are ordered before the release in the barrier
    if (!ok) record_status(c.status, kStatusMbarTimeout, 211, c.rank, c.rank, 3, 0);
  }
  if (!symm_block_barrier(c, 211, 2)) return;
  if (out && threadIdx.x == 0 && nb > 0) {
    fence_proxy_async_all();                      // the peers' stores are visible to the bulk loads below
    const uint8_t* recv = symm_local<uint8_t>(c, a.recv_off);
    for (int g = 0; g < c.gsize; ++g) {
      if (g == c.grank) continue;
      if (!bulk_copy(ring, out + (long long)g * a.chunk + b0, recv + (long long)g * a.chunk + b0, nb, &s_abort, c.budget_ns)) {
        record_status(c.status, kStatusMbarTimeout, 211, c.rank, c.rank, 4, 0);
        break;
      }
    }
  }
}

// ================================================================================================
// latency-optimised all-reduce for small messages: every 4 bytes of data travel with a 4-byte epoch word in ONE 8-byte
// store straight into the receiver's slot for this sender, and the receiver polls the words it is about to reduce.
// There is no barrier at all: the cost is one kernel launch plus one one-way NVLink store. Two slots alternate by the
// parity of the epoch, which is enough because a rank can run at most one call ahead of any peer (it needs the peer's
// data of the current call to finish it). The epoch lives in the heap and is advanced by the last block of each call.
// Layout at ll_off: header {uint32 epoch, uint32 done_blocks, pad to 16 B}, then [2 parities][gsize sources][cap units] x 8 B.
// ================================================================================================
struct LLArgs {
  const void* src;
  long long n;          // elements
  uint64_t ll_off;
  long long cap_units;  // 4-byte data words per (parity, source) slot
  void* out;
  float scale;
};

__device__ __forceinline__ void st_volatile_v2(void* p, uint32_t a, uint32_t b) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_volatile_v2(const void* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

template <int DT, int OP>
__global__ void __launch_bounds__(kCollThreads)
coll_allreduce_ll_kernel(const SymmCtx c, const LLArgs a) {
  uint32_t* hdr = symm_local<uint32_t>(c, a.ll_off);
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(hdr) + 1u;   // advanced only after every block has read it
  const uint32_t parity = epoch & 1u;
  const long long elems_per_word = DT == kCollF32 ? 1 : 2;
  const long long units = (a.n + elems_per_word - 1) / elems_per_word;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const uint64_t slots = a.ll_off + 16;
  const uint64_t my_slot = slots + (((uint64_t)parity * c.gsize + c.grank) * a.cap_units) * 8;
  // send: my words into slot [parity][me] of every member (my own copy included: one code path, one rounding order)
  for (long long i = tid; i < units; i += nthreads) {
    uint32_t w;
    if (DT == kCollF32) {
      w = static_cast<const uint32_t*>(a.src)[i];
    } else {
      const uint16_t* s16 = static_cast<const uint16_t*>(a.src);
      const uint32_t lo = s16[2 * i], hi = (2 * i + 1 < a.n) ? s16[2 * i + 1] : 0u;
      w = lo | (hi << 16);
    }
    for (int g = 0; g < c.gsize; ++g) st_volatile_v2(symm_ptr<uint8_t>(c, c.members[g], my_slot) + i * 8, w, epoch);
  }
  // receive + reduce: poll the (data, epoch) pairs of every source in member order
  bool ok = true;
  for (long long i = tid; i < units && ok; i += nthreads) {
    float acc0 = 0.f, acc1 = 0.f;
    for (int g = 0; g < c.gsize && ok; ++g) {
      const uint8_t* p = symm_local<uint8_t>(c, slots + (((uint64_t)parity * c.gsize + g) * a.cap_units) * 8) + i * 8;
      uint2 v = ld_volatile_v2(p);
      if (v.y != epoch) {
        const long long t0 = clock64();
        while ((v = ld_volatile_v2(p)).y != epoch) {
          if (clock64() - t0 > budget_cycles(c.budget_ns)) {
            record_status(c.status, kStatusPeerTimeout, 208, c.rank, c.members[g], 1, epoch);
            ok = false;
            break;
          }
        }
      }
      float x0, x1 = 0.f;
      if (DT == kCollF32) {
        x0 = __uint_as_float(v.x);
      } else {
        const float2 f = unpack_bf16x2(v.x);
        x0 = f.x; x1 = f.y;
      }
      if (g == 0) { acc0 = x0; acc1 = x1; }
      else { acc0 = combine<OP>(acc0, x0); acc1 = combine<OP>(acc1, x1); }
    }
    if (!ok) break;
    acc0 *= a.scale; acc1 *= a.scale;
    if (DT == kCollF32) {
      static_cast<float*>(a.out)[i] = acc0;
    } else {
      __nv_bfloat16* o = static_cast<__nv_bfloat16*>(a.out);
      o[2 * i] = __float2bfloat16_rn(acc0);
      if (2 * i + 1 < a.n) o[2 * i + 1] = __float2bfloat16_rn(acc1);
    }
  }
  // the last block to finish advances the epoch for the next call (kernels of one stream do not overlap)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(hdr + 1, 1u) + 1u;
    if (done == gridDim.x) {
      hdr[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(hdr) = epoch;
    }
  }
}

// The same exchange without the reduction: out[g] = the words of member g (small all-gathers: counts, row statistics).
__global__ void __launch_bounds__(kCollThreads)
coll_allgather_ll_kernel(const SymmCtx c, const LLArgs a) {
  uint32_t* hdr = symm_local<uint32_t>(c, a.ll_off);
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(hdr) + 1u;
  const uint32_t parity = epoch & 1u;
  const long long units = a.n;       // 4-byte words per member
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const uint64_t slots = a.ll_off + 16;
  const uint64_t my_slot = slots + (((uint64_t)parity * c.gsize + c.grank) * a.cap_units) * 8;
  for (long long i = tid; i < units; i += nthreads) {
    const uint32_t w = static_cast<const uint32_t*>(a.src)[i];
    for (int g = 0; g < c.gsize; ++g) st_volatile_v2(symm_ptr<uint8_t>(c, c.members[g], my_slot) + i * 8, w, epoch);
  }
  bool ok = true;
  for (long long i = tid; i < units * c.gsize && ok; i += nthreads) {
    const int g = (int)(i / units);
    const long long u = i - (long long)g * units;
    const uint8_t* p = symm_local<uint8_t>(c, slots + (((uint64_t)parity * c.gsize + g) * a.cap_units) * 8) + u * 8;
    uint2 v = ld_volatile_v2(p);
    if (v.y != epoch) {
      const long long t0 = clock64();
      while ((v = ld_volatile_v2(p)).y != epoch) {
        if (clock64() - t0 > budget_cycles(c.budget_ns)) {
          record_status(c.status, kStatusPeerTimeout, 209, c.rank, c.members[g], 1, epoch);
          ok = false;
          break;
        }
      }
    }
    if (ok) static_cast<uint32_t*>(a.out)[i] = v.x;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(hdr + 1, 1u) + 1u;
    if (done == gridDim.x) {
      hdr[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(hdr) = epoch;
    }
  }
}

// ================================================================================================
// two-shot all-reduce: reduce own slice -> publish -> gather all slices
// ================================================================================================
struct TwoShotArgs {
  const void* src;
  long long n;          // total elements (every rank holds n)
  uint64_t stage_off;   // staged inputs
  uint64_t result_off;  // n elements: slice g is produced by member g in its own heap
  void* out;
  int src_in_heap;
  double scale;
};

template <int DT, int OP>
__global__ void __launch_bounds__(kCollThreads)
coll_allreduce_twoshot_kernel(const SymmCtx c, const TwoShotArgs a) {
  using P = Pack<DT>;
  using Acc = typename P::Acc;
  extern __shared__ __align__(128) uint8_t bulk_smem[];
  __shared__ int s_abort;
  GridCopier cp;
  cp.init(bulk_smem, &s_abort, c.budget_ns);
  if (!a.src_in_heap) cp.copy(symm_local<uint8_t>(c, a.stage_off), a.src, a.n * P::kElem);
  cp.proxy_fence();
  if (!symm_grid_barrier(c, 202, 1)) return;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  // slices in units of 16-byte vectors; the last member also takes the ragged tail
  const long long nvec_total = a.n / P::kN;
  const long long per = (nvec_total + c.gsize - 1) / c.gsize;
  const long long v0 = min(per * c.grank, nvec_total), v1 = min(v0 + per, nvec_total);
  long long i0 = v0 + tid;
  // four vectors per thread and iteration: 4 x gsize independent loads in flight
  for (; i0 + 3 * nthreads < v1; i0 += 4 * nthreads) {
    Acc acc[4][P::kN];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      P::unpack(ld_global_v4(symm_ptr<uint8_t>(c, c.members[0], a.stage_off) + ((i0 + u * nthreads) << 4)), acc[u]);
    for (int g = 1; g < c.gsize; ++g) {
      U4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) raw[u] = ld_global_v4(symm_ptr<uint8_t>(c, c.members[g], a.stage_off) + ((i0 + u * nthreads) << 4));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        Acc v[P::kN];
        P::unpack(raw[u], v);
#pragma unroll
        for (int j = 0; j < P::kN; ++j) acc[u][j] = combine<OP>(acc[u][j], v[j]);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (a.scale != 1.0) {
#pragma unroll
        for (int j = 0; j < P::kN; ++j) acc[u][j] = (Acc)(acc[u][j] * (Acc)a.scale);
      }
      st_global_v4(symm_local<uint8_t>(c, a.result_off) + ((i0 + u * nthreads) << 4), P::pack(acc[u]));
    }
  }
  for (long long i = i0; i < v1; i += nthreads) {
    Acc acc[P::kN];
    P::unpack(ld_global_v4(symm_ptr<uint8_t>(c, c.members[0], a.stage_off) + (i << 4)), acc);
    for (int g = 1; g < c.gsize; ++g) {
      Acc v[P::kN];
      P::unpack(ld_global_v4(symm_ptr<uint8_t>(c, c.members[g], a.stage_off) + (i << 4)), v);
#pragma unroll
      for (int j = 0; j < P::kN; ++j) acc[j] = combine<OP>(acc[j], v[j]);
    }
    if (a.scale != 1.0) {
#pragma unroll
      for (int j = 0; j < P::kN; ++j) acc[j] = (Acc)(acc[j] * (Acc)a.scale);
    }
    st_global_v4(symm_local<uint8_t>(c, a.result_off) + (i << 4), P::pack(acc));
  }
  if (c.grank == c.gsize - 1) {
    for (long long i = nvec_total * P::kN + tid; i < a.n; i += nthreads) {
      Acc acc = P::load1(symm_ptr<uint8_t>(c, c.members[0], a.stage_off), i);
      for (int g = 1; g < c.gsize; ++g)
        acc = combine<OP>(acc, P::load1(symm_ptr<uint8_t>(c, c.members[g], a.stage_off), i));
      if (a.scale != 1.0) acc = (Acc)(acc * (Acc)a.scale);
      P::store1(symm_local<uint8_t>(c, a.result_off), i, acc);
    }
  }
  if (!symm_grid_barrier(c, 202, 2)) return;
  cp.proxy_fence();
  for (int k = 0; k < c.gsize; ++k) {
    const int g = (c.grank + k) % c.gsize;      // own slice first, then the peers in a rotated order
    const long long s0 = min(per * g, nvec_total), s1 = min(s0 + per, nvec_total);
    const uint8_t* from = symm_ptr<uint8_t>(c, c.members[g], a.result_off);
    cp.copy(static_cast<uint8_t*>(a.out) + (s0 << 4), from + (s0 << 4), (s1 - s0) << 4);
    if (g == c.gsize - 1)
      for (long long i = nvec_total * P::kN + tid; i < a.n; i += nthreads)
        P::store1(a.out, i, P::load1(from, i));
  }
  symm_block_barrier(c, 202, 3);
}

// ================================================================================================
// NVLS all-reduce (bf16 / fp32 sum): in-switch reduction through the multicast mapping
// ================================================================================================
template <int DT>
__global__ void __launch_bounds__(kCollThreads)
coll_allreduce_nvls_kernel(const SymmCtx c, const TwoShotArgs a) {
  using P = Pack<DT>;
  extern __shared__ __align__(128) uint8_t bulk_smem[];
  __shared__ int s_abort;
  GridCopier cp;
  cp.init(bulk_smem, &s_abort, c.budget_ns);
  if (!a.src_in_heap) cp.copy(symm_local<uint8_t>(c, a.stage_off), a.src, a.n * P::kElem);
  cp.proxy_fence();
  if (!symm_grid_barrier(c, 203, 1)) return;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long nvec_total = (a.n + P::kN - 1) / P::kN;  // staging buffers are padded to 16 bytes
  const long long per = (nvec_total + c.gsize - 1) / c.gsize;
  const long long v0 = min(per * c.grank, nvec_total), v1 = min(v0 + per, nvec_total);
  auto ldr = [&](long long i) {
    if constexpr (DT == kCollBf16) return multimem_ld_reduce_bf16x8(symm_mc<uint8_t>(c, a.stage_off) + (i << 4));
    else return multimem_ld_reduce_f32x4(symm_mc<uint8_t>(c, a.stage_off) + (i << 4));
  };
  long long i = v0 + tid;
  for (; i + 7 * nthreads < v1; i += 8 * nthreads) {   // eight in-switch reductions in flight per thread
    U4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = ldr(i + u * nthreads);
#pragma unroll
    for (int u = 0; u < 8; ++u) multimem_st_v4(symm_mc<uint8_t>(c, a.result_off) + ((i + u * nthreads) << 4), v[u]);
  }
  for (; i < v1; i += nthreads) multimem_st_v4(symm_mc<uint8_t>(c, a.result_off) + (i << 4), ldr(i));
  if (!symm_grid_barrier(c, 203, 2)) return;
  cp.proxy_fence();
  if (a.out != nullptr) cp.copy(a.out, symm_local<uint8_t>(c, a.result_off), a.n * P::kElem);
  symm_block_barrier(c, 203, 3);
}

// ================================================================================================
// NVLS push all-gather: every rank reads its own shard once and stores it through the multicast mapping, the switch
// replicates each 16-byte store into the gathered buffer of every rank. A sender's link carries its shard once (a pull
// all-gather serves it W-1 times), stores are posted (no round trip to hide), and the local loads come from HBM.
// NVLS reduce-scatter: every rank reads the sum of its slice over all ranks with multimem.ld_reduce (the switch adds) and
// writes it to its local output - the first half of the NVLS all-reduce on its own.
// ================================================================================================
struct NvlsAgArgs {
  const void* src;         // this rank's shard, `bytes` bytes (16-byte aligned, any device memory)
  long long bytes;         // multiple of 16
  uint64_t gather_off;     // heap offset of the gathered buffer [gsize][bytes]
  void* out;               // optional local output that receives a copy of the gathered buffer (null: caller reads the heap)
  int root;                // -1: all-gather (member g stores slot g); >= 0: broadcast - only member `root` stores, into slot 0
};

__global__ void __launch_bounds__(kCollThreads)
coll_allgather_nvls_kernel(const SymmCtx c, const NvlsAgArgs a) {
  extern __shared__ __align__(128) uint8_t bulk_smem[];
  __shared__ int s_abort;
  GridCopier cp;
  cp.init(bulk_smem, &s_abort, c.budget_ns);
  // all ranks have entered: the previous gathered result has been consumed everywhere
  if (!symm_grid_barrier(c, 206, 1)) return;
  const long long nvec = a.bytes >> 4;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const uint8_t* src = static_cast<const uint8_t*>(a.src);
  uint8_t* dst = symm_mc<uint8_t>(c, a.gather_off) + (a.root < 0 ? (long long)c.grank * a.bytes : 0ll);
  long long i = (a.root < 0 || a.root == c.grank) ? tid : nvec;      // broadcast: only the root has something to store
  for (; i + 7 * nthreads < nvec; i += 8 * nthreads) {   // eight local loads in flight per thread, then eight posted stores
    U4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = ld_global_nc_v4(src + ((i + u * nthreads) << 4));
#pragma unroll
    for (int u = 0; u < 8; ++u) multimem_st_v4(dst + ((i + u * nthreads) << 4), v[u]);
  }
  for (; i < nvec; i += nthreads) multimem_st_v4(dst + (i << 4), ld_global_nc_v4(src + (i << 4)));
  // every block of every rank has issued its stores once this barrier passes
  if (!symm_grid_barrier(c, 206, 2)) return;
  if (a.out != nullptr) {
    cp.proxy_fence();
    cp.copy(a.out, symm_local<uint8_t>(c, a.gather_off), a.root < 0 ? a.bytes * c.gsize : a.bytes);
  }
}

struct NvlsRsArgs {
  const void* src;       // this rank's full input [gsize * n] (staged into the heap unless it already lives there)
  long long n;           // elements per slice
  uint64_t stage_off;
  void* out;             // local output, n elements
  int src_in_heap;
};

template <int DT>
__global__ void __launch_bounds__(kCollThreads)
coll_reduce_scatter_nvls_kernel(const SymmCtx c, const NvlsRsArgs a) {
  using P = Pack<DT>;
  extern __shared__ __align__(128) uint8_t bulk_smem[];
  __shared__ int s_abort;
  GridCopier cp;
  cp.init(bulk_smem, &s_abort, c.budget_ns);
  if (!a.src_in_heap) cp.copy(symm_local<uint8_t>(c, a.stage_off), a.src, a.n * c.gsize * P::kElem);
  cp.proxy_fence();
  if (!symm_grid_barrier(c, 207, 1)) return;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long nvec = a.n / P::kN;                       // the host checks that n is a multiple of the vector width
  const uint8_t* mc = symm_mc<uint8_t>(c, a.stage_off) + (long long)c.grank * a.n * P::kElem;
  uint8_t* out = static_cast<uint8_t*>(a.out);
  auto ldr = [&](long long i) {
    if constexpr (DT == kCollBf16) return multimem_ld_reduce_bf16x8(mc + (i << 4));
    else return multimem_ld_reduce_f32x4(mc + (i << 4));
  };
  long long i = tid;
  for (; i + 7 * nthreads < nvec; i += 8 * nthreads) {   // eight in-switch reductions in flight per thread (a round trip through the switch each)
    U4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = ldr(i + u * nthreads);
#pragma unroll
    for (int u = 0; u < 8; ++u) st_global_v4(out + ((i + u * nthreads) << 4), v[u]);
  }
  for (; i < nvec; i += nthreads) st_global_v4(out + (i << 4), ldr(i));
  // nobody may overwrite its staged input (the next call) while a peer still reads it through the switch
  symm_grid_barrier(c, 207, 2);
}

// ================================================================================================
// all-to-all-v: rows of row_bytes; send_counts/send_offsets (in rows, int64, device) per destination
// ================================================================================================
struct A2AVArgs {
  const void* src;            // local rows, already grouped by destination
  long long src_rows;         // rows to stage
  long long row_bytes;
  const long long* send_counts;   // [gsize] rows for each destination (device memory)
  const long long* send_offsets;  // [gsize] first row for each destination
  uint64_t stage_off;         // staged rows
  uint64_t meta_off;          // 2*kSymmMaxWorld int64: counts then offsets, as seen by the sender
  void* out;                  // received rows, grouped by source in member order
  long long out_capacity_rows;
  long long* recv_counts;     // [gsize] rows received from each source (device memory, may be null)
  long long* recv_total;      // [1]
};

__global__ void __launch_bounds__(kCollThreads)
coll_a2av_kernel(const SymmCtx c, const A2AVArgs a) {
  grid_copy_bytes(symm_local<uint8_t>(c, a.stage_off), a.src, a.src_rows * a.row_bytes);
  if (blockIdx.x == 0 && (int)threadIdx.x < c.gsize) {
    long long* meta = symm_local<long long>(c, a.meta_off);
    meta[threadIdx.x] = a.send_counts[threadIdx.x];
    meta[kSymmMaxWorld + threadIdx.x] = a.send_offsets[threadIdx.x];
  }
  if (!symm_grid_barrier(c, 204, 1)) return;
  long long out_row = 0;
  for (int g = 0; g < c.gsize; ++g) {
    const long long* meta = symm_ptr<long long>(c, c.members[g], a.meta_off);
    const long long cnt = meta[c.grank];
    const long long off = meta[kSymmMaxWorld + c.grank];
    long long take = cnt;
    if (out_row + take > a.out_capacity_rows) take = max(0ll, a.out_capacity_rows - out_row);
    grid_copy_bytes(static_cast<uint8_t*>(a.out) + out_row * a.row_bytes,
                    symm_ptr<uint8_t>(c, c.members[g], a.stage_off) + off * a.row_bytes,
                    take * a.row_bytes);
    if (blockIdx.x == 0 && threadIdx.x == 0 && a.recv_counts) a.recv_counts[g] = cnt;
    out_row += cnt;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0 && a.recv_total) *a.recv_total = out_row;
  symm_block_barrier(c, 204, 2);
}

// A barrier and nothing else (used by tests and to fence phases of composite ops).
__global__ void coll_barrier_kernel(const SymmCtx c) { symm_block_barrier(c, 205, 1); }



// Launch of a kernel that carries the bulk-copy ring in dynamic shared memory.
template <typename K, typename A>
static void launch_with_ring(K kernel, int grid, cudaStream_t s, const SymmCtx& c, const A& a) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkSmemBytes);
  kernel<<<grid, kCollThreads, kBulkSmemBytes, s>>>(c, a);
}

static int grid_for(long long bytes, int max_blocks) {
  long long per_block = (long long)kCollThreads * 16 * 4;
  long long b = (bytes + per_block - 1) / per_block;
  if (b < 1) b = 1;
  int cap = sm_count();                       // the grid-wide barrier needs every block resident: one block per SM
  if (max_blocks > 0 && max_blocks < cap) cap = max_blocks;
  if (cap > kSymmMaxBlocks) cap = kSymmMaxBlocks;
  return (int)(b > cap ? cap : b);
}

template <int DT>
static int launch_reduce_op(int op, const SymmCtx& c, const ReduceArgs& a, int grid, cudaStream_t s) {
  switch (op) {
    case kCollSum: coll_reduce_kernel<DT, kCollSum><<<grid, kCollThreads, 0, s>>>(c, a); break;
    case kCollMax: coll_reduce_kernel<DT, kCollMax><<<grid, kCollThreads, 0, s>>>(c, a); break;
    case kCollMin: coll_reduce_kernel<DT, kCollMin><<<grid, kCollThreads, 0, s>>>(c, a); break;
    default: set_last_error("unknown reduce op"); return kApiBadArgument;
  }
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

static int elem_size(int dt) {
  switch (dt) {
    case kCollBf16: case kCollF16: return 2;
    case kCollF32: case kCollI32: return 4;
    case kCollF64: case kCollI64: return 8;
  }
  return 0;
}

}  // namespace pkb

using namespace pkb;

extern "C" {

int pkb_coll_barrier(const pkb_symm_ctx* h, int blocks, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(blocks >= 1 && blocks <= kSymmMaxBlocks, "blocks out of range");
  coll_barrier_kernel<<<blocks, 32, 0, static_cast<cudaStream_t>(stream)>>>(symm_ctx_from_api(h));
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_coll_reduce(const pkb_symm_ctx* h, int dtype, int op, const void* src, long long stage_elems,
                    unsigned long long stage_off, long long in_base, long long n, void* out, int active,
                    double scale, int max_blocks, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(elem_size(dtype) > 0, "unknown dtype");
  PKB_CHECK_ARG((stage_off & 15) == 0, "stage offset must be 16-byte aligned");
  ReduceArgs a{src, stage_elems, stage_off, in_base, n, out, active, scale};
  const long long work = (stage_elems > n * h->gsize ? stage_elems : n * h->gsize) * elem_size(dtype);
  const int grid = grid_for(work, max_blocks);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  SymmCtx c = symm_ctx_from_api(h);
  switch (dtype) {
    case kCollBf16: return launch_reduce_op<kCollBf16>(op, c, a, grid, s);
    case kCollF16: return launch_reduce_op<kCollF16>(op, c, a, grid, s);
    case kCollF32: return launch_reduce_op<kCollF32>(op, c, a, grid, s);
    case kCollF64: return launch_reduce_op<kCollF64>(op, c, a, grid, s);
    case kCollI32: return launch_reduce_op<kCollI32>(op, c, a, grid, s);
    case kCollI64: return launch_reduce_op<kCollI64>(op, c, a, grid, s);
  }
  return kApiBadArgument;
}

int pkb_coll_gather(const pkb_symm_ctx* h, const void* src, long long stage_bytes,
                    unsigned long long stage_off, unsigned int src_mask, long long in_base,
                    long long in_member_stride, long long seg_bytes, void* out, long long out_stride,
                    int active, int max_blocks, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG((stage_off & 15) == 0, "stage offset must be 16-byte aligned");
  GatherArgs a{src, stage_bytes, stage_off, src_mask, in_base, in_member_stride, seg_bytes, out, out_stride, active};
  const long long work = stage_bytes > seg_bytes * h->gsize ? stage_bytes : seg_bytes * h->gsize;
  const int grid = grid_for(work, max_blocks);
  static bool attr_set = false;
  if (!attr_set) {
    PKB_CHECK_CUDA(cudaFuncSetAttribute(coll_gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkSmemBytes));
    attr_set = true;
  }
  coll_gather_kernel<<<grid, kCollThreads, kBulkSmemBytes, static_cast<cudaStream_t>(stream)>>>(symm_ctx_from_api(h), a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_coll_row_gather(const pkb_symm_ctx* h, const void* src, long long stage_bytes, unsigned long long table_off,
                        const void* ids, long long n, long long rows_per_member, long long row_bytes, void* out,
                        int sync, int max_blocks, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(rows_per_member > 0 && row_bytes > 0 && n >= 0, "rows_per_member and row_bytes must be positive");
  PKB_CHECK_ARG(stage_bytes == 0 || sync, "a staged table needs the barriers");
  RowGatherArgs a{src, stage_bytes, table_off, static_cast<const long long*>(ids), n, rows_per_member, row_bytes, out, sync};
  const long long work = stage_bytes > n * row_bytes ? stage_bytes : n * row_bytes;
  const int grid = grid_for(work, max_blocks);
  coll_row_gather_kernel<<<grid, kCollThreads, 0, static_cast<cudaStream_t>(stream)>>>(symm_ctx_from_api(h), a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_coll_a2a_permute(const pkb_symm_ctx* h, const void* src, long long stage_bytes, unsigned long long stage_off,
                         long long in_rank_off, const long long* extents, const long long* in_strides,
                         long long out_member_off, const long long* out_strides, long long inner_bytes, void* out,
                         int max_blocks, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(extents && in_strides && out_strides && inner_bytes > 0, "extents, strides and inner_bytes are required");
  PKB_CHECK_ARG(extents[0] > 0 && extents[1] > 0 && extents[2] > 0, "extents must be positive");
  A2APermArgs a{src, stage_bytes, stage_off, in_rank_off, extents[0], extents[1], extents[2], in_strides[0], in_strides[1],
                in_strides[2], out_member_off, out_strides[0], out_strides[1], out_strides[2], inner_bytes, out};
  const long long moved = extents[0] * extents[1] * extents[2] * inner_bytes * h->gsize;
  const int grid = grid_for(moved > stage_bytes ? moved : stage_bytes, max_blocks);
  coll_a2a_perm_kernel<<<grid, kCollThreads, 0, static_cast<cudaStream_t>(stream)>>>(symm_ctx_from_api(h), a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_coll_all_to_all_push(const pkb_symm_ctx* h, const void* src, long long chunk_bytes, unsigned long long recv_off,
                             void* out, int max_blocks, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(chunk_bytes > 0 && (chunk_bytes & 15) == 0, "chunk_bytes must be a positive multiple of 16");
  PKB_CHECK_ARG((((uintptr_t)src | (uintptr_t)out | recv_off) & 15) == 0, "buffers must be 16-byte aligned");
  A2APushArgs a{src, chunk_bytes, recv_off, out};
  // one ring thread per block: blocks beyond the point where each holds a few ring-fulls only add barrier traffic
  int grid = grid_for(chunk_bytes / 8, max_blocks);
  launch_with_ring(coll_a2a_push_kernel, grid, static_cast<cudaStream_t>(stream), symm_ctx_from_api(h), a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_coll_allreduce_ll(const pkb_symm_ctx* h, int dtype, int op, const void* src, long long n, unsigned long long ll_off,
                          long long cap_units, void* out, double scale, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(dtype == kCollBf16 || dtype == kCollF32, "the latency-optimised all-reduce takes bf16 or fp32");
  PKB_CHECK_ARG((ll_off & 15) == 0 && n >= 1, "heap offset misaligned or empty input");
  const long long units = dtype == kCollF32 ? n : (n + 1) / 2;
  PKB_CHECK_ARG(units <= cap_units, "message larger than the slot");
  LLArgs a{src, n, ll_off, cap_units, out, (float)scale};
  int grid = (int)((units + 4 * kCollThreads - 1) / (4 * kCollThreads));
  if (grid < 1) grid = 1;
  if (grid > 32) grid = 32;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  SymmCtx c = symm_ctx_from_api(h);
#define PKB_LL(DT)                                                                              \
  switch (op) {                                                                                 \
    case kCollSum: coll_allreduce_ll_kernel<DT, kCollSum><<<grid, kCollThreads, 0, s>>>(c, a); break; \
    case kCollMax: coll_allreduce_ll_kernel<DT, kCollMax><<<grid, kCollThreads, 0, s>>>(c, a); break; \
    case kCollMin: coll_allreduce_ll_kernel<DT, kCollMin><<<grid, kCollThreads, 0, s>>>(c, a); break; \
    default: set_last_error("unknown reduce op"); return kApiBadArgument;                       \
  }
  if (dtype == kCollBf16) { PKB_LL(kCollBf16); } else { PKB_LL(kCollF32); }
#undef PKB_LL
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_coll_allgather_ll(const pkb_symm_ctx* h, const void* src, long long words, unsigned long long ll_off,
                          long long cap_units, void* out, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG((ll_off & 15) == 0 && words >= 1 && words <= cap_units, "heap offset misaligned or message larger than the slot");
  LLArgs a{src, words, ll_off, cap_units, out, 1.0f};
  int grid = (int)((words * h->gsize + 4 * kCollThreads - 1) / (4 * kCollThreads));
  if (grid < 1) grid = 1;
  if (grid > 32) grid = 32;
  coll_allgather_ll_kernel<<<grid, kCollThreads, 0, static_cast<cudaStream_t>(stream)>>>(symm_ctx_from_api(h), a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_coll_allreduce_twoshot(const pkb_symm_ctx* h, int dtype, int op, const void* src, long long n,
                               unsigned long long stage_off, unsigned long long result_off, void* out,
                               int src_in_heap, double scale, int max_blocks, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(((stage_off | result_off) & 15) == 0, "heap offsets must be 16-byte aligned");
  PKB_CHECK_ARG(((uintptr_t)out & 15) == 0, "output must be 16-byte aligned");
  TwoShotArgs a{src, n, stage_off, result_off, out, src_in_heap, scale};
  const int grid = grid_for(n * elem_size(dtype) * 2, max_blocks);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  SymmCtx c = symm_ctx_from_api(h);
#define PKB_TWOSHOT(DT)                                                                         \
  switch (op) {                                                                                 \
    case kCollSum: launch_with_ring(coll_allreduce_twoshot_kernel<DT, kCollSum>, grid, s, c, a); break; \
    case kCollMax: launch_with_ring(coll_allreduce_twoshot_kernel<DT, kCollMax>, grid, s, c, a); break; \
    case kCollMin: launch_with_ring(coll_allreduce_twoshot_kernel<DT, kCollMin>, grid, s, c, a); break; \
    default: set_last_error("unknown reduce op"); return kApiBadArgument;                       \
  }
  switch (dtype) {
    case kCollBf16: PKB_TWOSHOT(kCollBf16); break;
    case kCollF16: PKB_TWOSHOT(kCollF16); break;
    case kCollF32: PKB_TWOSHOT(kCollF32); break;
    case kCollF64: PKB_TWOSHOT(kCollF64); break;
    case kCollI32: PKB_TWOSHOT(kCollI32); break;
    case kCollI64: PKB_TWOSHOT(kCollI64); break;
    default: set_last_error("unknown dtype"); return kApiBadArgument;
  }
#undef PKB_TWOSHOT
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_coll_allreduce_nvls(const pkb_symm_ctx* h, int dtype, const void* src, long long n,
                            unsigned long long stage_off, unsigned long long result_off, void* out,
                            int src_in_heap, int max_blocks, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(h->mc_base != 0, "NVLS multicast mapping not available");
  PKB_CHECK_ARG(h->gsize == h->world, "NVLS all-reduce runs on the whole heap group only");
  PKB_CHECK_ARG(((stage_off | result_off) & 15) == 0, "heap offsets must be 16-byte aligned");
  TwoShotArgs a{src, n, stage_off, result_off, out, src_in_heap, 1.0};
  const int grid = grid_for(n * elem_size(dtype), max_blocks);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  SymmCtx c = symm_ctx_from_api(h);
  if (dtype == kCollBf16) launch_with_ring(coll_allreduce_nvls_kernel<kCollBf16>, grid, s, c, a);
  else if (dtype == kCollF32) launch_with_ring(coll_allreduce_nvls_kernel<kCollF32>, grid, s, c, a);
  else { set_last_error("NVLS all-reduce supports bf16 and fp32"); return kApiUnsupported; }
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// Gathered buffer [gsize][bytes] at heap offset gather_off on every rank (and a local copy in `out` when it is not null);
// bytes % 16 == 0, src 16-byte aligned; needs the multicast mapping and the whole-job group.
int pkb_coll_allgather_nvls(const pkb_symm_ctx* h, const void* src, long long bytes, unsigned long long gather_off, void* out,
                            int max_blocks, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(h->mc_base != 0 && h->gsize == h->world, "NVLS all-gather needs the multicast mapping and the whole-job group");
  PKB_CHECK_ARG(bytes > 0 && bytes % 16 == 0 && (gather_off & 15) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
                (reinterpret_cast<uintptr_t>(out) & 15) == 0, "16-byte alignment and a size that is a multiple of 16");
  NvlsAgArgs a{src, bytes, gather_off, out, -1};
  launch_with_ring(coll_allgather_nvls_kernel, grid_for(bytes, max_blocks), static_cast<cudaStream_t>(stream), symm_ctx_from_api(h), a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// Broadcast through the switch: member `root` stores its `bytes` once through the multicast mapping and they land in the buffer
// at heap offset bcast_off of every rank (and in `out` when it is not null). Same constraints as the all-gather above.
int pkb_coll_broadcast_nvls(const pkb_symm_ctx* h, const void* src, long long bytes, int root, unsigned long long bcast_off, void* out,
                            int max_blocks, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(h->mc_base != 0 && h->gsize == h->world, "NVLS broadcast needs the multicast mapping and the whole-job group");
  PKB_CHECK_ARG(root >= 0 && root < h->gsize, "root out of range");
  PKB_CHECK_ARG(bytes > 0 && bytes % 16 == 0 && (bcast_off & 15) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
                (reinterpret_cast<uintptr_t>(out) & 15) == 0, "16-byte alignment and a size that is a multiple of 16");
  NvlsAgArgs a{src, bytes, bcast_off, out, root};
  launch_with_ring(coll_allgather_nvls_kernel, grid_for(bytes, max_blocks), static_cast<cudaStream_t>(stream), symm_ctx_from_api(h), a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// out[n] = sum over ranks of slice grank of every rank's [gsize * n] input (bf16 or fp32, n a multiple of 8 resp. 4).
int pkb_coll_reduce_scatter_nvls(const pkb_symm_ctx* h, int dtype, const void* src, long long n, unsigned long long stage_off,
                                 void* out, int src_in_heap, int max_blocks, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(h->mc_base != 0 && h->gsize == h->world, "NVLS reduce-scatter needs the multicast mapping and the whole-job group");
  PKB_CHECK_ARG(dtype == kCollBf16 || dtype == kCollF32, "NVLS reduce-scatter supports bf16 and fp32");
  PKB_CHECK_ARG(n > 0 && n % (dtype == kCollBf16 ? 8 : 4) == 0, "slice length must be a multiple of 16 bytes");
  PKB_CHECK_ARG((stage_off & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0, "16-byte alignment");
  NvlsRsArgs a{src, n, stage_off, out, src_in_heap};
  const int grid = grid_for(n * elem_size(dtype), max_blocks);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  SymmCtx c = symm_ctx_from_api(h);
  if (dtype == kCollBf16) launch_with_ring(coll_reduce_scatter_nvls_kernel<kCollBf16>, grid, s, c, a);
  else launch_with_ring(coll_reduce_scatter_nvls_kernel<kCollF32>, grid, s, c, a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_coll_all_to_all_v(const pkb_symm_ctx* h, const void* src, long long src_rows, long long row_bytes,
                          const void* send_counts, const void* send_offsets, unsigned long long stage_off,
                          unsigned long long meta_off, void* out, long long out_capacity_rows,
                          void* recv_counts, void* recv_total, int max_blocks, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(row_bytes > 0, "row_bytes must be positive");
  PKB_CHECK_ARG(((stage_off | meta_off) & 15) == 0, "heap offsets must be 16-byte aligned");
  A2AVArgs a{src, src_rows, row_bytes, static_cast<const long long*>(send_counts),
             static_cast<const long long*>(send_offsets), stage_off, meta_off, out, out_capacity_rows,
             static_cast<long long*>(recv_counts), static_cast<long long*>(recv_total)};
  int cap = sm_count();
  if (max_blocks > 0 && max_blocks < cap) cap = max_blocks;
  if (cap > kSymmMaxBlocks) cap = kSymmMaxBlocks;
  coll_a2av_kernel<<<cap, kCollThreads, 0, static_cast<cudaStream_t>(stream)>>>(symm_ctx_from_api(h), a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

}  // extern "C"
