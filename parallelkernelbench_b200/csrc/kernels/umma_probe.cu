// Rate of tcgen05.mma by operand form, measured on the device: one thread issues a run of M = 128, K = 16 bf16 products into
// one accumulator, commits, waits for the commit and reports the SM cycles per product. The attention kernels pick their
// tile shapes and operand placements (P in tensor memory as the A operand, V as an MN-major B operand, steps of 64 or 128
// keys) from these numbers; a trace of the forward kernel showed its P V products taking about twice as long as its S
// products, which a FLOP count does not predict. Operand contents do not matter (shared memory is zeroed).
// No counterpart in the reference (its attention is PyTorch SDPA: reference/54_ring_attention.py).
#include "pkb/api.h"
#include "pkb/host.h"
#include "pkb/ptx.cuh"

namespace pkb {

constexpr int kProbeThreads = 128;
constexpr int kProbeA = 0;                     // 128 rows x 128 bytes, one 64-column atom, K-major
constexpr int kProbeB = 16384;                 // up to 256 rows x 128 bytes K-major, or two MN-major atoms of 16 KiB
constexpr int kProbeBars = kProbeB + 32768;
constexpr int kProbeSmem = kProbeBars + 64;

// FORM: 0 SS N=128 | 1 SS N=64 | 2 SS N=256 | 3 TS (A in tensor memory), B MN-major N=128 | 4 SS, B MN-major N=128 |
//       5 TS, B K-major N=128 | 6 TS, B MN-major N=64 | 7 SS, A and B as 0 but the accumulator alternates between two buffers
// The descriptors of the four K steps are built before the clock starts and the issue loop is unrolled by four, so that the
// issuing thread's own instruction latency (about 115 cycles per product with the descriptors built in the loop) does not
// hide the rate of the tensor pipe.
template <int FORM>
__global__ void __launch_bounds__(kProbeThreads, 1)
umma_probe_kernel(int mmas, long long* __restrict__ out_cycles, uint32_t* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sb = smem_u32(smem);
  const uint32_t bar = sb + kProbeBars;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + kProbeBars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kProbeBars + 24);
  for (int i = threadIdx.x; i < kProbeBars / 16; i += kProbeThreads) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar, 1);
    fence_mbar_init();
  }
  if (threadIdx.x < 32) {
    tmem_alloc(smem_u32(tmem_holder), 512);
    tmem_relinquish();
  }
  fence_proxy_async_all();            // the zeroes are visible to the tensor core's shared-memory reads
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  if (threadIdx.x == 32) {
    constexpr int n = (FORM == 1 || FORM == 6) ? 64 : (FORM == 2 ? 256 : 128);
    constexpr bool b_mn = FORM == 3 || FORM == 4 || FORM == 6;
    constexpr bool a_tmem = FORM == 3 || FORM == 5 || FORM == 6;
    constexpr uint32_t idesc = make_idesc(128, n, 1, 1, 0, b_mn ? 1 : 0);
    uint64_t da[4], db[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {     // four K steps inside one 128-byte row / eight-row group
      da[k] = make_smem_desc_sw128_kmajor(sb + kProbeA + k * 32);
      db[k] = b_mn ? make_smem_desc_sw128_mnmajor(sb + kProbeB + k * 2048, 16384) : make_smem_desc_sw128_kmajor(sb + kProbeB + k * 32);
    }
    long long t0;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t0)::"memory");
    for (int i = 0; i < mmas; i += 4) {
      const uint32_t d_addr = tmem_base + ((FORM == 7 && (i & 8)) ? 128 : 0);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if constexpr (a_tmem) umma_f16_ts(d_addr, tmem_base + 256 + k * 8, db[k], idesc, 1u);
        else umma_f16_ss(d_addr, da[k], db[k], idesc, 1u);
      }
    }
    umma_commit(bar);
    const bool ok = mbar_wait(bar, 0, abort_flag, 100000000ull);
    long long t1;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t1)::"memory");
    out_cycles[blockIdx.x] = ok ? (t1 - t0) : -1;
    if (!ok) record_status(status, kStatusMbarTimeout, 900, 0, 0, 1, FORM);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int FORM>
static int launch_probe(int mmas, int ctas, long long* out, cudaStream_t s) {
  PKB_CHECK_CUDA(cudaFuncSetAttribute(umma_probe_kernel<FORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, kProbeSmem));
  umma_probe_kernel<FORM><<<ctas, kProbeThreads, kProbeSmem, s>>>(mmas, out, status_block_device_ptr());
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

}  // namespace pkb

extern "C" int pkb_umma_rate(int form, int mmas, int ctas, void* out_cycles, void* stream) {
  using namespace pkb;
  PKB_CHECK_ARG(form >= 0 && form <= 7 && mmas >= 1 && mmas <= (1 << 20) && ctas >= 1 && ctas <= 1024, "form 0..7, 1 <= mmas <= 2^20, 1 <= ctas <= 1024");
  PKB_CHECK_ARG(out_cycles != nullptr, "out_cycles (int64[ctas], device) is required");
  PKB_CHECK_ARG(mmas % 4 == 0, "mmas must be a multiple of four");
  long long* out = static_cast<long long*>(out_cycles);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (form) {
    case 0: return launch_probe<0>(mmas, ctas, out, s);
    case 1: return launch_probe<1>(mmas, ctas, out, s);
    case 2: return launch_probe<2>(mmas, ctas, out, s);
    case 3: return launch_probe<3>(mmas, ctas, out, s);
    case 4: return launch_probe<4>(mmas, ctas, out, s);
    case 5: return launch_probe<5>(mmas, ctas, out, s);
    case 6: return launch_probe<6>(mmas, ctas, out, s);
    default: return launch_probe<7>(mmas, ctas, out, s);
  }
}

