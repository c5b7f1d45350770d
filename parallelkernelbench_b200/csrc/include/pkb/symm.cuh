// Device view of the symmetric heap and the cross-GPU barrier built on it.
//
// Address of byte `off` of rank p's heap:  base + p * stride + off  (same on every rank).
// The first kSymmCtrlBytes of every rank's heap are control space: per channel, a table of
// barrier flags [kSymmMaxBlocks][kSymmMaxWorld] written by peers and a table of per-block epoch
// counters written only locally. A channel belongs to one process group, so groups with
// different members never share counters.
//
// Barrier protocol (per block index b, all ranks launch the same grid): thread p < world does
//   fence.acq_rel.sys; st.release.sys  flags_of_peer_p[b][my_rank] = epoch
//   wait (bounded) until ld.acquire.sys my_flags[b][p] >= epoch
// Epochs only grow, so flags never need resetting and a late reader cannot miss a signal.
// This is the bounded-wait counterpart of the CAS hand-shake the reference offers to kernel
// authors (reference: utils/triton_utils.py:75-221), fused into the kernel that needs it instead of
// being separate one-thread launches (reference: kernelgen/solutions_new_allreduce_parallelkittens.py:71-113).
#pragma once
#include "pkb/ptx.cuh"

namespace pkb {

constexpr int kSymmMaxWorld = 16;
constexpr int kSymmTableBlocks = 256;  // rows of the per-channel tables
constexpr int kSymmMaxBlocks = 240;    // largest block index that may take part in a barrier; the last epoch words
                                       // of a channel hold the state of the grid-wide barrier
constexpr int kSymmChannels = 32;
constexpr uint64_t kSymmFlagBytes = (uint64_t)kSymmTableBlocks * kSymmMaxWorld * 4;  // 16 KiB
constexpr uint64_t kSymmEpochBytes = (uint64_t)kSymmTableBlocks * 4;                 // 1 KiB
constexpr uint64_t kSymmChannelBytes = kSymmFlagBytes + kSymmEpochBytes;
constexpr uint64_t kSymmCtrlBytes = 1ull << 20;  // user allocations start at 1 MiB
static_assert(kSymmChannels * kSymmChannelBytes <= kSymmCtrlBytes, "control space too small");

struct SymmCtx {
  uint64_t base;     // virtual address of rank 0's heap
  uint64_t stride;   // bytes between consecutive ranks
  uint64_t mc_base;  // multicast mapping of the heap, 0 if NVLS is not set up
  int rank;          // global rank of this process
  int world;         // ranks in the heap
  int gsize;         // members of the process group this call runs on
  int grank;         // index of this rank inside the group
  int members[kSymmMaxWorld];  // global ranks of the group members
  int channel;       // control channel owned by the group
  uint32_t* status;
  uint64_t budget_ns;
};

// Checked build (-DPKB_DEBUG_BOUNDS, `python -m parallelkernelbench_b200.build --debug-bounds`): a rank outside the heap or an
// offset beyond one rank's slab is recorded in the status block (BOUNDS_VIOLATION with this rank, the bad rank and the
// offset in 4 KiB units) and the access is redirected to a scratch line at the end of this rank's control space, so
// nothing outside the heap is touched and nothing traps. Only the base of an access is checked, not the index added to it.
constexpr uint64_t kSymmBoundsScratch = kSymmCtrlBytes - 4096;
static_assert(kSymmChannels * kSymmChannelBytes <= kSymmBoundsScratch, "the scratch line overlaps the channel tables");

template <typename T>
__device__ __forceinline__ T* symm_ptr(const SymmCtx& c, int global_rank, uint64_t off) {
#ifdef PKB_DEBUG_BOUNDS
  if (static_cast<unsigned>(global_rank) >= static_cast<unsigned>(c.world) || off >= c.stride) {
    record_status(c.status, kStatusBoundsViolation, 0, c.rank, static_cast<uint32_t>(global_rank), 0,
                  static_cast<uint32_t>(off >> 12));
    return reinterpret_cast<T*>(c.base + (uint64_t)c.rank * c.stride + kSymmBoundsScratch);
  }
#endif
  return reinterpret_cast<T*>(c.base + (uint64_t)global_rank * c.stride + off);
}
template <typename T>
__device__ __forceinline__ T* symm_local(const SymmCtx& c, uint64_t off) {
  return symm_ptr<T>(c, c.rank, off);
}
template <typename T>
__device__ __forceinline__ T* symm_mc(const SymmCtx& c, uint64_t off) {
  return reinterpret_cast<T*>(c.mc_base + off);
}

// Barrier between the same-index blocks of all group members. Every thread of the block calls it.
// Returns false (on every thread) if a peer did not arrive within the budget; the status block
// then names the kernel, this rank and the peer that was missing.
// `s_epoch_slot` is one uint32 of shared memory used to broadcast the epoch inside the block.
__device__ __forceinline__ bool symm_block_barrier_at(const SymmCtx& c, int kernel_id, int site,
                                                      volatile uint32_t* s_epoch_slot) {
  volatile uint32_t& s_epoch = *s_epoch_slot;
  const int b = blockIdx.x;
  const uint64_t chan_off = (uint64_t)c.channel * kSymmChannelBytes;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* epochs = symm_local<uint32_t>(c, chan_off + kSymmFlagBytes);
    const uint32_t e = epochs[b] + 1u;
    epochs[b] = e;
    s_epoch = e;
  }
  __syncthreads();
  const uint32_t e = s_epoch;
  int ok = 1;
  if ((int)threadIdx.x < c.gsize) {
    const int peer = c.members[threadIdx.x];
    fence_acq_rel_sys();
    st_release_sys(symm_ptr<uint32_t>(c, peer, chan_off) + b * kSymmMaxWorld + c.rank, e);
    const uint32_t* mine = symm_local<uint32_t>(c, chan_off) + b * kSymmMaxWorld + peer;
    if (!wait_flag_ge(mine, e, c.budget_ns)) {
      ok = 0;
      record_status(c.status, kStatusPeerTimeout, kernel_id, c.rank, peer, site, e);
    }
  }
  return __syncthreads_and(ok) != 0;
}

__device__ __forceinline__ bool symm_block_barrier(const SymmCtx& c, int kernel_id, int site) {
  __shared__ uint32_t s_epoch_static;
  return symm_block_barrier_at(c, kernel_id, site, &s_epoch_static);
}

// Barrier between ALL blocks of ALL group members: use it when a block reads data that a different block index of a
// peer wrote in the same launch (stage with a grid-stride loop, then read the peers' staged bytes with another mapping).
// Every block arrives on a local counter; block 0 waits for the whole grid, does the cross-rank flag exchange of the
// block barrier (row 0 of the flag table) and then advances a local release word that the other blocks wait on.
// The whole grid must be resident at once (launch at most one block per SM). Three words at the end of the channel's
// epoch table hold the state, so grids that use this barrier have at most kSymmGridMaxBlocks blocks.
constexpr int kSymmGridMaxBlocks = kSymmMaxBlocks;
constexpr int kSymmGridArriveSlot = 253, kSymmGridErrSlot = 254, kSymmGridReleaseSlot = 255;

__device__ __forceinline__ bool symm_grid_barrier(const SymmCtx& c, int kernel_id, int site) {
  __shared__ uint32_t s_word;
  __shared__ int s_ok;
  const uint64_t chan_off = (uint64_t)c.channel * kSymmChannelBytes;
  uint32_t* epochs = symm_local<uint32_t>(c, chan_off + kSymmFlagBytes);
  uint32_t* arrive = epochs + kSymmGridArriveSlot;
  uint32_t* err = epochs + kSymmGridErrSlot;
  uint32_t* release = epochs + kSymmGridReleaseSlot;
  __syncthreads();
  if (threadIdx.x == 0) {
    s_word = ld_acquire_sys(release);     // cannot advance before this block has arrived
    s_ok = 1;
    __threadfence();
    atomicAdd(arrive, 1u);
  }
  __syncthreads();
  const uint32_t target = s_word + 1u;
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) {
      if (!wait_flag_ge(arrive, gridDim.x, c.budget_ns)) {
        s_ok = 0;
        record_status(c.status, kStatusPeerTimeout, kernel_id, c.rank, c.rank, site, gridDim.x);
      }
      *reinterpret_cast<volatile uint32_t*>(arrive) = 0u;
      const uint32_t e = epochs[0] + 1u;
      epochs[0] = e;
      s_word = e;
    }
    __syncthreads();
    const uint32_t e = s_word;
    if ((int)threadIdx.x < c.gsize && s_ok) {
      const int peer = c.members[threadIdx.x];
      fence_acq_rel_sys();
      st_release_sys(symm_ptr<uint32_t>(c, peer, chan_off) + c.rank, e);
      const uint32_t* mine = symm_local<uint32_t>(c, chan_off) + peer;
      if (!wait_flag_ge(mine, e, c.budget_ns)) {
        s_ok = 0;
        record_status(c.status, kStatusPeerTimeout, kernel_id, c.rank, peer, site, e);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      if (!s_ok) *reinterpret_cast<volatile uint32_t*>(err) = target;
      fence_acq_rel_sys();
      st_release_sys(release, target);
    }
  } else if (threadIdx.x == 0) {
    if (!wait_flag_ge(release, target, 2 * c.budget_ns)) {
      s_ok = 0;
      record_status(c.status, kStatusPeerTimeout, kernel_id, c.rank, c.rank, site + 100, target);
    } else if (ld_acquire_sys(err) == target) {
      s_ok = 0;
    }
  }
  __syncthreads();
  return s_ok != 0;
}

}  // namespace pkb
