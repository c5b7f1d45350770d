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
constexpr int kSymmMaxBlocks = 256;
constexpr int kSymmChannels = 32;
constexpr uint64_t kSymmFlagBytes = (uint64_t)kSymmMaxBlocks * kSymmMaxWorld * 4;  // 16 KiB
constexpr uint64_t kSymmEpochBytes = (uint64_t)kSymmMaxBlocks * 4;                 // 1 KiB
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

template <typename T>
__device__ __forceinline__ T* symm_ptr(const SymmCtx& c, int global_rank, uint64_t off) {
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

}  // namespace pkb
