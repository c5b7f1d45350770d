// Block-wide bulk copy driven by the TMA unit (untiled cp.async.bulk, no multicast).
//
// A thread that copies with 16-byte loads has one small request in flight per load, and the number of outstanding
// requests per SM is limited - over NVLink (microseconds of latency) that caps an SM-driven copy well below the link.
// One bulk request moves kilobytes, so a handful of requests in flight per CTA is enough to fill the link: data goes
// global (local or peer) -> shared-memory ring -> global (local or peer), one elected thread issues everything.
// Both pointers must be 16-byte aligned and `bytes` a multiple of 16.
#pragma once
#include "pkb/ptx.cuh"

namespace pkb {

constexpr int kBulkStageBytes = 16 * 1024;
constexpr int kBulkStages = 6;
constexpr int kBulkSmemBytes = kBulkStages * kBulkStageBytes + kBulkStages * 8;   // ring + one mbarrier per stage

__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst),
               "l"(gsrc), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src), "r"(bytes) : "memory");
}

// State of one CTA's ring; lives in registers of the issuing thread. `phase` holds one parity bit per stage.
struct BulkRing {
  uint32_t smem;     // shared-memory address of the ring (16-byte aligned), followed by the mbarriers
  uint32_t phase;
  int stages;        // depth of the ring: `stages` buffers of kBulkStageBytes, then `stages` mbarriers (at most 32)
};

constexpr int bulk_ring_bytes(int stages) { return stages * (kBulkStageBytes + 8); }

// Call once per kernel by thread 0 of the block (then __syncthreads before the first copy).
__device__ __forceinline__ void bulk_ring_init(BulkRing& r, uint32_t smem_addr, int stages = kBulkStages) {
  r.smem = smem_addr;
  r.phase = 0;
  r.stages = stages;
  for (int s = 0; s < stages; ++s) mbar_init(smem_addr + stages * kBulkStageBytes + 8 * s, 1);
  fence_mbar_init();
}

// Copies [src, src + bytes) to dst. Executed by ONE thread (the one that owns the ring). Returns false if a load did
// not complete within the budget (the caller records the status). On return all stores have been performed.
__device__ __forceinline__ bool bulk_copy(BulkRing& r, void* dst, const void* src, long long bytes, volatile int* abort_flag,
                                          uint64_t budget_ns) {
  const long long n = (bytes + kBulkStageBytes - 1) / kBulkStageBytes;
  auto chunk_bytes = [&](long long c) { return (uint32_t)((c + 1 < n) ? kBulkStageBytes : (bytes - c * kBulkStageBytes)); };
  const int stages = r.stages;
  auto bar = [&](int s) { return r.smem + stages * kBulkStageBytes + 8u * s; };
  auto issue_load = [&](long long c) {
    const int s = (int)(c % stages);
    mbar_expect_tx(bar(s), chunk_bytes(c));
    bulk_load(r.smem + s * kBulkStageBytes, static_cast<const uint8_t*>(src) + c * kBulkStageBytes, chunk_bytes(c), bar(s));
  };
  const int kAhead = stages - 2;              // loads in flight; two stages may still be read by stores
  for (long long c = 0; c < n && c < kAhead; ++c) issue_load(c);
  bool ok = true;
  for (long long c = 0; c < n; ++c) {
    if (c + kAhead < n) {
      // chunk c + kAhead reuses the stage of chunk c - 2, whose store was committed two iterations ago
      tma_store_wait_read<1>();
      issue_load(c + kAhead);
    }
    const int s = (int)(c % stages);
    if (!mbar_wait(bar(s), (r.phase >> s) & 1u, abort_flag, budget_ns)) { ok = false; break; }
    r.phase ^= 1u << s;
    bulk_store(static_cast<uint8_t*>(dst) + c * kBulkStageBytes, r.smem + s * kBulkStageBytes, chunk_bytes(c));
    tma_store_commit();
  }
  tma_store_wait_all<0>();
  return ok;
}

}  // namespace pkb

namespace pkb {

// Grid-wide copy: every block takes one contiguous slice and its thread 0 moves it with the bulk ring. All threads of all
// blocks call it. Falls back to nothing - the caller checks `bulk_copy_eligible` first.
__device__ __forceinline__ bool bulk_copy_eligible(const void* dst, const void* src, long long bytes) {
  return bytes >= (1ll << 20) && ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) && (bytes & 15) == 0;
}

__device__ __forceinline__ bool grid_bulk_copy(BulkRing& r, void* dst, const void* src, long long bytes, volatile int* abort_flag,
                                               uint64_t budget_ns) {
  bool ok = true;
  if (threadIdx.x == 0) {
    long long per = (bytes + gridDim.x - 1) / gridDim.x;
    per = (per + 1023) & ~1023ll;
    const long long b0 = per * blockIdx.x;
    if (b0 < bytes) {
      const long long nb = (b0 + per <= bytes) ? per : (bytes - b0);
      ok = bulk_copy(r, static_cast<uint8_t*>(dst) + b0, static_cast<const uint8_t*>(src) + b0, nb, abort_flag, budget_ns);
    }
  }
  return ok;
}

}  // namespace pkb
