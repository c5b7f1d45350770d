// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (tiled bulk tensor copies, one CTA as the
// destination), tcgen05 (TMEM allocation, MMA, commit, load), system-scope acquire/release
// accesses for cross-GPU flags, and NVLS multimem loads/stores.
//
// Every blocking primitive here is bounded: a wait returns false once its time budget is spent
// (or once another role of the CTA has raised the abort flag) instead of spinning forever.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pkb {

// ----------------------------------------------------------------------------------------------
// status words (see runtime/status.cu): a kernel that gives up a wait records why.
// ----------------------------------------------------------------------------------------------
enum StatusCode : uint32_t {
  kStatusOk = 0,
  kStatusMbarTimeout = 1,     // an intra-CTA mbarrier wait ran out of budget
  kStatusPeerTimeout = 2,     // a wait on a flag written by another GPU ran out of budget
  kStatusBadArgument = 3,
  kStatusBoundsViolation = 4, // a checked accessor saw an out-of-range index (debug builds)
};

// Layout of the status block (uint32 words): [0] code (first error wins), [1] kernel id,
// [2] rank, [3] peer / barrier index, [4] phase / site, [5] tile, [6] blockIdx.x, [7] count.
constexpr int kStatusWords = 16;

__device__ __forceinline__ void record_status(uint32_t* status, uint32_t code, uint32_t kernel_id,
                                              uint32_t rank, uint32_t who, uint32_t site,
                                              uint32_t tile) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0u, code) == 0u) {
    status[1] = kernel_id;
    status[2] = rank;
    status[3] = who;
    status[4] = site;
    status[5] = tile;
    status[6] = blockIdx.x;
    __threadfence_system();
  }
  atomicAdd(status + 7, 1u);
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// predicated forms for a producer WARP whose lanes walk the loop together (see umma_f16_ss_p)
__device__ __forceinline__ void mbar_expect_tx_p(uint32_t bar, uint32_t bytes, uint32_t lead) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %2, 0;\n\t@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}\n" ::"r"(bar),
               "r"(bytes), "r"(lead)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// The same test with a suspend-time hint: the thread may sleep in hardware for up to `hint_ns` and is woken as soon as the
// phase completes, so a waiting warp polls (and takes issue slots from the warps that compute) far less often.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}

// Default budget of a device-side wait. Generous for production kernels (a healthy wait is
// microseconds); tests that exercise the time-out path pass a few milliseconds instead.
constexpr uint64_t kDefaultWaitBudgetNs = 4000000000ull;

// Budgets are given in nanoseconds but measured with the SM-local cycle counter (reading the
// global timer costs on the order of a microsecond, far too much for a wait that normally succeeds
// within a few polls). 2 cycles per nanosecond over-estimates the clock a little, so a wait gives
// up slightly late rather than early.
__device__ __forceinline__ long long budget_cycles(uint64_t budget_ns) {
  return static_cast<long long>(budget_ns) * 2;
}

constexpr uint32_t kMbarSuspendHintNs = 4000;

// Bounded mbarrier wait. `abort_flag` lives in shared memory and is shared by all roles of the
// CTA: the first role whose budget expires raises it, every other wait sees it within 64 polls (a poll sleeps up to kMbarSuspendHintNs).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint64_t budget_ns = kDefaultWaitBudgetNs) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = 0;
  uint32_t spins = 0;
  while (!mbar_try_wait_hint(bar, parity, kMbarSuspendHintNs)) {
    if ((++spins & 0x3fu) == 0u) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > budget_cycles(budget_ns)) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

// The same bounded wait for roles that are NOT on a kernel's critical path (a producer that runs steps ahead, a warp that only
// reacts to rare events): between two tests the warp sleeps `sleep_ns`, so it takes far fewer issue slots from the warps of
// its scheduler that compute, at the price of waking up to `sleep_ns` late.
__device__ __forceinline__ bool mbar_wait_backoff(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint64_t budget_ns,
                                                  uint32_t sleep_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = 0;
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    __nanosleep(sleep_ns);
    if ((++spins & 0x3fu) == 0u) {
      if (*abort_flag) return false;
      const long long now = clock64();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > budget_cycles(budget_ns)) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

// The same wait for a warp whose lanes walk a loop together: one lane polls (32 lanes testing the same barrier are 32
// barrier operations), the result is shared by a vote. `lead` is non-zero in exactly one lane.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint64_t budget_ns,
                                               uint32_t lead) {
  bool ok = true;
  if (lead) ok = mbar_wait(bar, parity, abort_flag, budget_ns);
  return __all_sync(0xffffffffu, ok);
}

// ----------------------------------------------------------------------------------------------
// TMA: tiled bulk tensor copies. Loads complete on an mbarrier of this CTA; stores use bulk groups.
// The innermost coordinate times the element size must be a multiple of 16 bytes.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* desc) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(desc)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* desc,
                                            uint32_t bar, int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_p(uint32_t smem_dst, const CUtensorMap* desc, uint32_t bar, int32_t c0, int32_t c1,
                                              uint32_t lead) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n\t}\n"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "r"(lead)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_p(uint32_t smem_dst, const CUtensorMap* desc, uint32_t bar, int32_t c0, int32_t c1,
                                              int32_t c2, uint32_t lead) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %6, 0;\n\t"
      "@q cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n\t}\n"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(lead)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* desc,
                                            uint32_t bar, int32_t c0, int32_t c1, int32_t c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* desc, uint32_t smem_src,
                                             int32_t c0, int32_t c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_src), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Adds `bytes` of fp32 from shared memory into global memory (16-byte aligned on both sides, a multiple of 16 bytes): one
// request to the TMA unit instead of bytes / 16 vector reductions issued by threads. Joins the thread's bulk group.
__device__ __forceinline__ void bulk_reduce_add_f32(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src), "r"(bytes)
               : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------------------------
// tcgen05: tensor memory + 5th-generation tensor-core MMA (single-CTA group)
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_holder, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_holder),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by ONE thread.
__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A operand from tensor memory (used by attention: P stays on chip).
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Predicated forms for an issuing WARP: all 32 lanes walk the issue loop together and `lead` (non-zero in one lane, see
// elect_one) selects the lane whose instruction takes effect. With the loop wrapped in `if (lane == 0)` instead, the code
// runs under a divergent branch, the compiler cannot keep descriptors and addresses in uniform registers, and every
// tcgen05 instruction is preceded by register-to-uniform-register moves whose latency, not the tensor pipe, then sets the
// pace of a kernel that issues a product every 64 cycles.
__device__ __forceinline__ void umma_f16_ss_p(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate, uint32_t lead) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(lead)
      : "memory");
}
__device__ __forceinline__ void umma_f16_ts_p(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate, uint32_t lead) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(lead)
      : "memory");
}
__device__ __forceinline__ void umma_commit_p(uint32_t bar, uint32_t lead) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}\n" ::"r"(bar), "r"(lead)
      : "memory");
}
__device__ __forceinline__ void umma_f8_ss_p(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate,
                                             uint32_t lead) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(lead)
      : "memory");
}
// fp8 (e4m3/e5m2) operands, fp32 accumulate.
__device__ __forceinline__ void umma_f8_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Make the mbarrier track completion of all MMAs issued so far by this thread.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp gets row (lane base + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Per-warpgroup register budget: data-movement warps give registers back, math warps take them. Every warp of a
// warpgroup (four consecutive warps) must execute the same instruction; `inc` waits until the registers are free.
template <int N>
__device__ __forceinline__ void warpgroup_reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void warpgroup_reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------------------------
// UMMA descriptors
// ----------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the 128-byte
// swizzle (what a TMA box of 64 bf16 / 128 fp8 columns with SWIZZLE_128B produces). Groups of
// eight rows are 1024 bytes apart; the tile base must be 1024-byte aligned. Stepping along K
// inside the 128-byte row is done by adding (bytes >> 4) to the low word.
__device__ __forceinline__ uint64_t make_smem_desc_sw128_kmajor(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);   // start address, bits [0,14)
  d |= static_cast<uint64_t>(0) << 16;                        // leading byte offset (unused here)
  d |= static_cast<uint64_t>(1024u >> 4) << 32;               // stride byte offset, bits [32,46)
  d |= static_cast<uint64_t>(1) << 46;                        // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                        // layout type: SWIZZLE_128B
  return d;
}

// Shared-memory descriptor of an MN-major tile (the MN index is contiguous in memory, e.g. a weight
// stored [K, N] row-major or V stored [kv, d]): the tile is a sequence of "atoms" of 64 bf16 along
// MN (one 128-byte swizzled row per K index). Inside an atom, groups of eight K rows are 1024 bytes
// apart (stride byte offset); consecutive atoms along MN are `atom_stride_bytes` apart (leading
// byte offset). Stepping 16 along K moves the start address by 16 rows = 2048 bytes.
__device__ __forceinline__ uint64_t make_smem_desc_sw128_mnmajor(uint32_t smem_addr,
                                                                 uint32_t atom_stride_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((atom_stride_bytes >> 4) & 0x3FFFu) << 16;  // leading byte offset
  d |= static_cast<uint64_t>(1024u >> 4) << 32;                            // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// The two words of the 128-byte-swizzle descriptors above, for issue loops that must stay short: the high word is a constant,
// and stepping the start address by `bytes` adds bytes >> 4 to the low word (the address field holds (addr & 0x3FFFF) >> 4 and
// cannot carry into the next field while the operand stays inside the 256 KiB window). One thread issues every product of a
// CTA; if it rebuilds a descriptor from the address for each product its own instruction latency, not the tensor pipe, sets
// the pace (measured: 115 cycles per 128 x 128 x 16 product against 65 with the words prepared).
constexpr uint32_t kSmemDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t smem_desc_lo_kmajor(uint32_t smem_addr) { return (smem_addr & 0x3FFFFu) >> 4; }
__device__ __forceinline__ uint32_t smem_desc_lo_mnmajor(uint32_t smem_addr, uint32_t atom_stride_bytes) {
  return ((smem_addr & 0x3FFFFu) >> 4) | (((atom_stride_bytes >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ uint64_t smem_desc_join(uint32_t lo) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(kSmemDescHiSw128));
  return d;
}

// Instruction descriptor for kind::f16 / kind::f8f6f4, fp32 accumulate, both operands K-major.
// a_fmt/b_fmt: f16 kinds 0 = fp16, 1 = bf16; f8f6f4 kinds 0 = e4m3, 1 = e5m2.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t m, uint32_t n, uint32_t a_fmt,
                                                  uint32_t b_fmt, uint32_t a_mn_major = 0,
                                                  uint32_t b_mn_major = 0) {
  return (1u << 4)               // accumulator format: fp32
         | (a_fmt << 7)          // A format
         | (b_fmt << 10)         // B format
         | (a_mn_major << 15)    // A: 0 K-major, 1 MN-major
         | (b_mn_major << 16)    // B: 0 K-major, 1 MN-major
         | ((n >> 3) << 17)      // N / 8
         | ((m >> 4) << 24);     // M / 16
}

// ----------------------------------------------------------------------------------------------
// system-scope flag accesses (flags written by another GPU over NVLink)
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Timing-perturbation build (-DPKB_JITTER, `python -m parallelkernelbench_b200.build --jitter`): a pseudo-random pause of up
// to ~4 us before every system-scope signal and after every successful wait shifts the ranks against each other from call to
// call, so an ordering that only holds by luck (a missing fence, a flag published before its data) shows up as a wrong
// result in the ordinary tests instead of once in a long run. The release build compiles the pause away.
#ifdef PKB_JITTER
__device__ __forceinline__ void jitter_pause() {
  uint32_t h = static_cast<uint32_t>(clock64()) * 2654435761u;
  h ^= threadIdx.x * 40503u + blockIdx.x * 9176u;
  __nanosleep((h >> 19) & 0xfffu);
}
#else
__device__ __forceinline__ void jitter_pause() {}
#endif

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  jitter_pause();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  jitter_pause();
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_relaxed_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}

// Bounded wait until *flag >= target (flags are monotonically increasing epoch counters).
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t target,
                                             uint64_t budget_ns = kDefaultWaitBudgetNs) {
  if (static_cast<int32_t>(ld_acquire_sys(flag) - target) >= 0) {
    jitter_pause();
    return true;
  }
  long long t0 = 0;
  uint32_t spins = 0;
  while (static_cast<int32_t>(ld_acquire_sys(flag) - target) < 0) {
    if ((++spins & 0x3fu) == 0u) {
      const long long now = clock64();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_cycles(budget_ns)) return false;
      __nanosleep(32);
    }
  }
  jitter_pause();
  return true;
}

// 16-byte global accesses
struct __align__(16) U4 {
  uint32_t x, y, z, w;
};
__device__ __forceinline__ U4 ld_global_v4(const void* p) {
  U4 v;
  asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// streaming (no L1 allocate) read, used for peer memory and one-pass inputs
__device__ __forceinline__ U4 ld_global_nc_v4(const void* p) {
  U4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// volatile-style read that always observes peer writes published by a release flag
__device__ __forceinline__ U4 ld_global_relaxed_v4(const void* p) {
  U4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_global_v4(void* p, const U4& v) {
  asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// ----------------------------------------------------------------------------------------------
// NVLS multimem (addresses inside a multicast mapping of symmetric memory)
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ U4 multimem_ld_reduce_bf16x8(const void* mc_ptr) {
  U4 v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc_ptr)
      : "memory");
  return v;
}
__device__ __forceinline__ U4 multimem_ld_reduce_f32x4(const void* mc_ptr) {
  U4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_ptr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_v4(void* mc_ptr, const U4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_ptr),
               "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void multimem_red_add_u32(uint32_t* mc_ptr, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_ptr), "r"(v)
               : "memory");
}

// ----------------------------------------------------------------------------------------------
// small numeric helpers
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// The same packing for non-negative finite inputs on the integer pipe: add half an ulp of bf16 to each word and take the upper
// halves with one byte permute (round to nearest, ties away from zero). cvt.rn.bf16x2.f32 executes on the special-function
// pipe, which a softmax already saturates with its exponentials; this form leaves that pipe to them.
__device__ __forceinline__ uint32_t pack_bf16x2_alu(float lo, float hi) {
  return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}
// x / s rounded to nearest, given inv = 1 / s rounded to nearest: q0 = x * inv is within an ulp, the residual x - q0 * s is
// exact in an FMA, and one correction step lands on the correctly rounded quotient (x and s normal, no overflow).
__device__ __forceinline__ float div_rn_by(float x, float s, float inv) {
  const float q0 = x * inv;
  const float r = fmaf(-q0, s, x);
  return fmaf(r, inv, q0);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }
// 2^x on the special-function unit (one MUFU instruction; -inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x on the FMA and integer pipes (no MUFU): floor(x) through a round-down add of 1.5 * 2^23, a degree-3 minimax polynomial of
// 2^f on [0, 1), and the integer part added to the exponent field. Relative error below 1e-4; x is clamped at -126, so
// minus infinity gives 2^-126, not 0 (callers that need an exact zero for masked entries use fast_exp2 there).
__device__ __forceinline__ float poly_exp2(float x) {
  x = fmaxf(x, -126.f);
  float xr;
  asm("add.rm.ftz.f32 %0, %1, %2;" : "=f"(xr) : "f"(x), "f"(12582912.f));
  const float n = xr - 12582912.f;
  const float f = x - n;
  const float pl = fmaf(fmaf(fmaf(0.077119089663028717f, f, 0.227564394474029541f), f, 0.695146143436431884f), f, 1.0f);
  return __int_as_float(__float_as_int(pl) + (__float_as_int(xr) << 23));
}
// Two 2^x at once on the FMA and integer pipes, packed fp32 arithmetic for the range reduction and the polynomial (see
// poly_exp2 for the method): 2 clamps, 6 packed operations and 2 integer multiply-adds per pair, against 2 special-function
// instructions of about 12 pipe cycles each.
__device__ __forceinline__ void poly_exp2_x2(float& e0, float& e1, float x0, float x1) {
  x0 = fmaxf(x0, -126.f);
  x1 = fmaxf(x1, -126.f);
  uint32_t p0, p1, r0, r1;
  asm("{\n\t.reg .b64 x, xr, n, f, p, magic, nmagic, mone, c1, c2, c3, one;\n\t"
      "mov.b64 x, {%4, %5};\n\t"
      "mov.b64 magic, {0f4B400000, 0f4B400000};\n\t"      // 1.5 * 2^23
      "mov.b64 nmagic, {0fCB400000, 0fCB400000};\n\t"
      "mov.b64 mone, {0fBF800000, 0fBF800000};\n\t"
      "mov.b64 one, {0f3F800000, 0f3F800000};\n\t"
      "mov.b64 c3, {0f3D9DF09D, 0f3D9DF09D};\n\t"         // 0.0771190897
      "mov.b64 c2, {0f3E6906A4, 0f3E6906A4};\n\t"         // 0.2275643945
      "mov.b64 c1, {0f3F31F519, 0f3F31F519};\n\t"         // 0.6951461434
      "add.rm.ftz.f32x2 xr, x, magic;\n\t"                 // low mantissa bits of xr = floor(x)
      "add.rn.ftz.f32x2 n, xr, nmagic;\n\t"                // floor(x) as a float
      "fma.rn.ftz.f32x2 f, n, mone, x;\n\t"                // fraction in [0, 1)
      "fma.rn.ftz.f32x2 p, c3, f, c2;\n\t"
      "fma.rn.ftz.f32x2 p, p, f, c1;\n\t"
      "fma.rn.ftz.f32x2 p, p, f, one;\n\t"
      "mov.b64 {%0, %1}, p;\n\t"
      "mov.b64 {%2, %3}, xr;\n\t}"
      : "=r"(p0), "=r"(p1), "=r"(r0), "=r"(r1)
      : "f"(x0), "f"(x1));
  e0 = __uint_as_float(p0 + (r0 << 23));                  // the integer part goes into the exponent field
  e1 = __uint_as_float(p1 + (r1 << 23));
}
// Packed fp32 arithmetic of sm_100 (two lanes per instruction) and the three-input maximum: they halve the issue slots of the
// scale / subtract, row-sum and row-maximum steps of a softmax.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// (d0, d1) = (a0, a1) * b + c
__device__ __forceinline__ void fma2_bcast(float& d0, float& d1, float a0, float a1, float b, float c) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
      "fma.rn.ftz.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
// (d0, d1) = (a0, a1) * (b0, b1)
__device__ __forceinline__ void mul2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.ftz.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
// (d0, d1) += (a0, a1)
__device__ __forceinline__ void add2_acc(float& d0, float& d1, float a0, float a1) {
  asm("{\n\t.reg .b64 ra, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rd, {%0, %1};\n\tadd.rn.ftz.f32x2 rd, rd, ra;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "+f"(d0), "+f"(d1)
      : "f"(a0), "f"(a1));
}

}  // namespace pkb

// ----------------------------------------------------------------------------------------------
// CTA-pair (cta_group::2) forms: two CTAs of a cluster drive one 256-row MMA. The leader CTA
// (cluster rank 0) issues the MMAs; both CTAs load their own halves of the operands, and the
// loads of both complete on the leader's mbarrier (bit 24 of a shared-window address selects the
// CTA inside the pair, clearing it addresses the leader).
// ----------------------------------------------------------------------------------------------
namespace pkb {

constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  cluster_arrive();
  cluster_wait();
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t local_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(cta_rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// tiled load into THIS CTA's shared memory; completion bytes go to the pair leader's mbarrier
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* desc,
                                                 uint32_t bar, int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar & kPeerBitMask), "r"(c0),
        "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair_p(uint32_t smem_dst, const CUtensorMap* desc, uint32_t bar, int32_t c0, int32_t c1,
                                                   uint32_t lead) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n\t}\n"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar & kPeerBitMask), "r"(c0), "r"(c1), "r"(lead)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_holder, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_holder),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the mbarrier at the same shared-memory offset in every CTA selected by cta_mask
// predicated forms for an issuing warp whose lanes walk the loop together (see umma_f16_ss_p)
__device__ __forceinline__ void umma_f16_ss_pair_p(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                   uint32_t accumulate, uint32_t lead) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(lead)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair_p(uint32_t bar, uint16_t cta_mask, uint32_t lead) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %2, 0;\n\t"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t"
      "}\n"
      :
      : "r"(bar), "h"(cta_mask), "r"(lead)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;"
      :
      : "r"(bar), "h"(cta_mask)
      : "memory");
}

}  // namespace pkb
