// Expert-parallel MoE data movement over peer memory. No host round trip anywhere: counts, offsets
// and slots stay on the device (the reference pays three host syncs per layer call,
// reference: reference/31_fused_moe_fwd.py:60-101).
//
//  moe_route       one warp per token: router logits (+ bias) -> softmax -> top-k (descending, ties to the lower
//                  expert index) -> gates, expert indices and the per-expert histogram, in one pass over the row
//  moe_histogram   per-expert assignment counts of this rank's tokens
//  moe_plan        from the all-gathered count matrix [W, E]: where each (source, expert) segment starts
//                  in its destination's receive buffer (expert-major, source-minor), this rank's own
//                  expert row offsets for the grouped GEMM, and its total of received rows
//  moe_dispatch    one warp per (token, k) assignment: claim a slot in the (expert, me) segment and
//                  write the token's payload row (fp8 e4m3 bytes, or any 16-byte-multiple row) and its
//                  scale row STRAIGHT into the destination rank's receive buffers with 16-byte P2P
//                  stores; ends with the in-kernel cross-rank barrier so that, when the kernel is
//                  complete everywhere, every rank holds all of its tokens
//  moe_combine     one warp per token: after a barrier, pull the k expert-output rows from the ranks that
//                  computed them (P2P loads), weight by the gates, add in a fixed order (deterministic)
//                  and store bf16
// Reference behaviour replaced: permute + all_to_all_single + chunk sort, and the inverse path with
// scatter_add_ (reference: reference/28_moe_pre_all2all.py, reference/29_moe_post_all2all.py).
#include "pkb/api.h"
#include "pkb/collectives_api.h"
#include "pkb/host.h"
#include "pkb/symm_host.h"

namespace pkb {

__global__ void moe_histogram_kernel(const int* __restrict__ expert_idx, long long n, int num_experts,
                                     int* __restrict__ counts) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int e = expert_idx[i];
    if (e >= 0 && e < num_experts) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x)
    if (hist[e]) atomicAdd(&counts[e], hist[e]);
}

// Softmax over up to 256 experts and top-k selection, one warp per token. Lane l holds experts l, l + 32, ...
// Selection = k rounds of a warp-wide arg-max on (probability, lower index wins ties), so the output is sorted by
// descending probability like torch.topk. The histogram is accumulated per block in shared memory first.
constexpr int kRouteMaxPerLane = 8;

__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ bias, int num_tokens,
                 int num_experts, int top_k, float* __restrict__ gates, int* __restrict__ idx, int* __restrict__ counts) {
  extern __shared__ int hist[];
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  for (long long t = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < num_tokens;
       t += (long long)gridDim.x * warps_per_block) {
    const float* row = logits + t * ld;
    float v[kRouteMaxPerLane];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < kRouteMaxPerLane; ++j) {
      const int e = j * 32 + lane;
      v[j] = e < num_experts ? row[e] + (bias ? bias[e] : 0.f) : -INFINITY;
      m = fmaxf(m, v[j]);
    }
    m = warp_max(m);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kRouteMaxPerLane; ++j) {
      v[j] = (j * 32 + lane) < num_experts ? expf(v[j] - m) : -1.f;   // probabilities are >= 0: -1 marks "absent / taken"
      sum += fmaxf(v[j], 0.f);
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int r = 0; r < top_k; ++r) {
      float best = -1.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < kRouteMaxPerLane; ++j)
        if (v[j] > best) { best = v[j]; best_e = j * 32 + lane; }   // ascending j: the lower index wins ties
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
        if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
      }
      if ((best_e & 31) == lane) {
#pragma unroll
        for (int j = 0; j < kRouteMaxPerLane; ++j)
          if (j == (best_e >> 5)) v[j] = -1.f;
      }
      if (lane == 0) {
        gates[t * top_k + r] = best * inv;
        idx[t * top_k + r] = best_e;
        atomicAdd(&hist[best_e], 1);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x)
    if (hist[e]) atomicAdd(&counts[e], hist[e]);
}

// One block. all_counts[s * E + e] = rows source rank s sends to expert e.
// seg_base[e]   : first slot, in the receive buffer of the rank that owns expert e, of MY segment
// my_offsets[le]: row offsets of my local experts (E_local + 1 entries), my_total = my_offsets[E_local]
__global__ void moe_plan_kernel(const int* __restrict__ all_counts, int world, int num_experts, int experts_per_rank,
                                int my_grank, int* __restrict__ seg_base, int* __restrict__ my_offsets,
                                int* __restrict__ cursor) {
  extern __shared__ int total[];  // [E] rows per expert over all sources
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    int t = 0;
    for (int s = 0; s < world; ++s) t += all_counts[s * num_experts + e];
    total[e] = t;
    cursor[e] = 0;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    const int first = (e / experts_per_rank) * experts_per_rank;  // first expert of the owning rank
    int base = 0;
    for (int e2 = first; e2 < e; ++e2) base += total[e2];
    for (int s = 0; s < my_grank; ++s) base += all_counts[s * num_experts + e];
    seg_base[e] = base;
  }
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int le = 0; le < experts_per_rank; ++le) {
      my_offsets[le] = acc;
      acc += total[my_grank * experts_per_rank + le];
    }
    my_offsets[experts_per_rank] = acc;
  }
}

struct MoeDispatchArgs {
  const uint8_t* payload;   // [T, payload_bytes] rows to send (already quantised if fp8)
  const uint8_t* scales;    // [T, scale_bytes] or nullptr
  int payload_bytes, scale_bytes;   // multiples of 16
  const int* expert_idx;    // [T * k] global expert per assignment
  long long num_assign;     // T * k
  int top_k;
  int experts_per_rank;
  const int* seg_base;      // [E]
  int* cursor;              // [E] zeroed by the plan kernel
  int* slots;               // [T * k] out: slot on the destination (or -1 if it did not fit)
  uint64_t recv_payload_off, recv_scale_off;   // heap offsets of the receive buffers
  int capacity;             // rows of the receive buffers
  int* overflow;            // incremented when a row does not fit
  uint64_t recv_meta_off;   // 0, or heap offset of int2 [capacity]: (sender's index in the group, assignment index) per row
};

// 512 threads per block, two blocks per SM: the cross-GPU block barrier caps the grid at kSymmMaxBlocks blocks, so the warps
// that keep copies in flight have to come from the block size.
constexpr int kMoeXchgThreads = 512;

__global__ void __launch_bounds__(kMoeXchgThreads, 2) moe_dispatch_kernel(const SymmCtx c, const MoeDispatchArgs a) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = warp; i < a.num_assign; i += nwarps) {
    const int e = a.expert_idx[i];
    int slot = 0;
    if (lane == 0) slot = a.seg_base[e] + atomicAdd(&a.cursor[e], 1);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    const long long t = i / a.top_k;
    if (slot >= a.capacity) {
      if (lane == 0) {
        a.slots[i] = -1;
        atomicAdd(a.overflow, 1);
      }
      continue;
    }
    const int dest = c.members[e / a.experts_per_rank];
    const uint8_t* src = a.payload + t * a.payload_bytes;
    uint8_t* dst = symm_ptr<uint8_t>(c, dest, a.recv_payload_off) + (long long)slot * a.payload_bytes;
    // four 16-byte loads in flight per lane before the first store
    int b = lane * 16;
    for (; b + 3 * 512 < a.payload_bytes; b += 4 * 512) {
      const U4 u0 = ld_global_v4(src + b), u1 = ld_global_v4(src + b + 512), u2 = ld_global_v4(src + b + 1024), u3 = ld_global_v4(src + b + 1536);
      st_global_v4(dst + b, u0); st_global_v4(dst + b + 512, u1); st_global_v4(dst + b + 1024, u2); st_global_v4(dst + b + 1536, u3);
    }
    for (; b < a.payload_bytes; b += 512) st_global_v4(dst + b, ld_global_v4(src + b));
    if (a.scales != nullptr) {
      const uint8_t* ss = a.scales + t * a.scale_bytes;
      uint8_t* sd = symm_ptr<uint8_t>(c, dest, a.recv_scale_off) + (long long)slot * a.scale_bytes;
      for (int b = lane * 16; b < a.scale_bytes; b += 32 * 16) st_global_v4(sd + b, ld_global_v4(ss + b));
    }
    if (lane == 0) {
      a.slots[i] = slot;
      if (a.recv_meta_off != 0) symm_ptr<int2>(c, dest, a.recv_meta_off)[slot] = make_int2(c.grank, (int)i);
    }
  }
  // when this barrier has been crossed by every block of every rank, all rows have landed everywhere
  symm_block_barrier(c, 500, 1);
}

struct MoeCombineArgs {
  uint64_t y_off;            // heap offset of the expert outputs [capacity, hidden] bf16 on every rank
  const int* expert_idx;     // [T * k]
  const int* slots;          // [T * k]
  const float* gates;        // [T * k]
  __nv_bfloat16* out;        // [T, hidden]
  long long num_tokens;
  int top_k, hidden, experts_per_rank;
  int local_rows;            // 1: row (t, j) sits at row t * k + j of THIS rank's buffer (the experts pushed it there)
};

template <int MAXK>
__global__ void __launch_bounds__(kMoeXchgThreads, 2) moe_combine_kernel(const SymmCtx c, const MoeCombineArgs a) {
  // every rank's expert outputs are complete once all ranks have entered this kernel
  if (!symm_block_barrier(c, 501, 1)) return;
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long t = warp; t < a.num_tokens; t += nwarps) {
    const __nv_bfloat16* rows[MAXK];
    float w[MAXK];
#pragma unroll
    for (int j = 0; j < MAXK; ++j) {
      rows[j] = nullptr;
      w[j] = 0.f;
      if (j < a.top_k) {
        const int e = a.expert_idx[t * a.top_k + j];
        const int slot = a.slots[t * a.top_k + j];
        if (slot >= 0) {
          rows[j] = a.local_rows
                        ? symm_local<__nv_bfloat16>(c, a.y_off) + (t * a.top_k + j) * a.hidden
                        : symm_ptr<__nv_bfloat16>(c, c.members[e / a.experts_per_rank], a.y_off) + (long long)slot * a.hidden;
          w[j] = a.gates[t * a.top_k + j];
        }
      }
    }
    for (int col = lane * 8; col < a.hidden; col += 256) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < MAXK; ++j) {
        if (rows[j] != nullptr) {
          U4 u = ld_global_relaxed_v4(rows[j] + col);
          float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
          acc[0] += w[j] * f0.x; acc[1] += w[j] * f0.y; acc[2] += w[j] * f1.x; acc[3] += w[j] * f1.y;
          acc[4] += w[j] * f2.x; acc[5] += w[j] * f2.y; acc[6] += w[j] * f3.x; acc[7] += w[j] * f3.y;
        }
      }
      U4 o{pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7])};
      st_global_v4(a.out + t * a.hidden + col, o);
    }
  }
  // peers may still be reading my expert outputs: nobody overwrites them before everyone is done
  symm_block_barrier(c, 501, 2);
}


}  // namespace pkb

using namespace pkb;

extern "C" {

int pkb_moe_histogram(const void* expert_idx, long long n, int num_experts, void* counts, void* stream) {
  PKB_CHECK_ARG(num_experts >= 1 && num_experts <= 4096, "1..4096 experts");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  PKB_CHECK_CUDA(cudaMemsetAsync(counts, 0, sizeof(int) * num_experts, s));
  if (n == 0) return kApiOk;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  moe_histogram_kernel<<<(int)blocks, 256, num_experts * sizeof(int), s>>>(static_cast<const int*>(expert_idx), n,
                                                                          num_experts, static_cast<int*>(counts));
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// logits [T, E] fp32 (row pitch ld elements) + optional fp32 bias [E] -> gates [T, k] fp32 (softmax probabilities of the
// chosen experts, descending), idx [T, k] int32, counts [E] int32 (zeroed here, then accumulated). E <= 256, k <= E.
int pkb_moe_route(const void* logits, long long ld, const void* bias, int num_tokens, int num_experts, int top_k,
                  void* gates, void* idx, void* counts, void* stream) {
  PKB_CHECK_ARG(num_experts >= 1 && num_experts <= 32 * kRouteMaxPerLane, "1..256 experts");
  PKB_CHECK_ARG(top_k >= 1 && top_k <= num_experts, "top_k must be in 1..experts");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  PKB_CHECK_CUDA(cudaMemsetAsync(counts, 0, sizeof(int) * num_experts, s));
  if (num_tokens == 0) return kApiOk;
  long long blocks = ((long long)num_tokens + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  moe_route_kernel<<<(int)blocks, 256, num_experts * sizeof(int), s>>>(
      static_cast<const float*>(logits), ld, static_cast<const float*>(bias), num_tokens, num_experts, top_k,
      static_cast<float*>(gates), static_cast<int*>(idx), static_cast<int*>(counts));
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_moe_plan(const void* all_counts, int world, int num_experts, int experts_per_rank, int my_grank,
                 void* seg_base, void* my_offsets, void* cursor, void* stream) {
  PKB_CHECK_ARG(num_experts == world * experts_per_rank, "experts must divide evenly over the group");
  PKB_CHECK_ARG(num_experts <= 4096, "at most 4096 experts");
  moe_plan_kernel<<<1, 256, num_experts * sizeof(int), static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int*>(all_counts), world, num_experts, experts_per_rank, my_grank, static_cast<int*>(seg_base),
      static_cast<int*>(my_offsets), static_cast<int*>(cursor));
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// recv_meta_off: 0, or the heap offset of an int2 [capacity] array that receives, for every row written, the sender's
// index in the group and the assignment index (token * k + j) - what an expert needs to send the row's result home.
int pkb_moe_dispatch_meta(const pkb_symm_ctx* h, const void* payload, const void* scales, int payload_bytes,
                          int scale_bytes, const void* expert_idx, long long num_assign, int top_k, int experts_per_rank,
                          const void* seg_base, void* cursor, void* slots, unsigned long long recv_payload_off,
                          unsigned long long recv_scale_off, int capacity, void* overflow,
                          unsigned long long recv_meta_off, void* stream) {
  PKB_CHECK_ARG(h && h->base, "symmetric heap not initialised");
  PKB_CHECK_ARG(payload_bytes % 16 == 0 && scale_bytes % 16 == 0, "row sizes must be multiples of 16 bytes");
  PKB_CHECK_ARG((recv_payload_off & 15) == 0 && (recv_scale_off & 15) == 0, "heap offsets misaligned");
  MoeDispatchArgs a{static_cast<const uint8_t*>(payload), static_cast<const uint8_t*>(scales), payload_bytes, scale_bytes,
                    static_cast<const int*>(expert_idx), num_assign, top_k, experts_per_rank,
                    static_cast<const int*>(seg_base), static_cast<int*>(cursor), static_cast<int*>(slots),
                    recv_payload_off, recv_scale_off, capacity, static_cast<int*>(overflow), recv_meta_off};
  PKB_CHECK_ARG((recv_meta_off & 7) == 0, "heap offsets misaligned");
  int grid = sm_count() * 2;   // fixed: the same on every rank, the barrier pairs blocks by index
  if (grid > kSymmMaxBlocks) grid = kSymmMaxBlocks;
  moe_dispatch_kernel<<<grid, kMoeXchgThreads, 0, static_cast<cudaStream_t>(stream)>>>(symm_ctx_from_api(h), a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_moe_dispatch(const pkb_symm_ctx* h, const void* payload, const void* scales, int payload_bytes,
                     int scale_bytes, const void* expert_idx, long long num_assign, int top_k, int experts_per_rank,
                     const void* seg_base, void* cursor, void* slots, unsigned long long recv_payload_off,
                     unsigned long long recv_scale_off, int capacity, void* overflow, void* stream) {
  return pkb_moe_dispatch_meta(h, payload, scales, payload_bytes, scale_bytes, expert_idx, num_assign, top_k, experts_per_rank,
                               seg_base, cursor, slots, recv_payload_off, recv_scale_off, capacity, overflow, 0ull, stream);
}

// local_rows = 0: pull row `slots[t, j]` of the expert outputs at y_off from the rank that owns expert idx[t, j].
// local_rows = 1: the experts already pushed the result of assignment (t, j) to row t * k + j of THIS rank's buffer at y_off.
int pkb_moe_combine_from(const pkb_symm_ctx* h, unsigned long long y_off, const void* expert_idx, const void* slots,
                         const void* gates, void* out, long long num_tokens, int top_k, int hidden, int experts_per_rank,
                         int local_rows, void* stream) {
  PKB_CHECK_ARG(h && h->base, "symmetric heap not initialised");
  PKB_CHECK_ARG(hidden % 8 == 0 && top_k >= 1 && top_k <= 8, "hidden % 8 == 0 and top_k <= 8");
  MoeCombineArgs a{y_off, static_cast<const int*>(expert_idx), static_cast<const int*>(slots),
                   static_cast<const float*>(gates), static_cast<__nv_bfloat16*>(out), num_tokens, top_k, hidden,
                   experts_per_rank, local_rows};
  int grid = sm_count() * 2;
  if (grid > kSymmMaxBlocks) grid = kSymmMaxBlocks;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (top_k <= 2) moe_combine_kernel<2><<<grid, kMoeXchgThreads, 0, s>>>(symm_ctx_from_api(h), a);
  else if (top_k <= 4) moe_combine_kernel<4><<<grid, kMoeXchgThreads, 0, s>>>(symm_ctx_from_api(h), a);
  else moe_combine_kernel<8><<<grid, kMoeXchgThreads, 0, s>>>(symm_ctx_from_api(h), a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

int pkb_moe_combine(const pkb_symm_ctx* h, unsigned long long y_off, const void* expert_idx, const void* slots,
                    const void* gates, void* out, long long num_tokens, int top_k, int hidden, int experts_per_rank,
                    void* stream) {
  return pkb_moe_combine_from(h, y_off, expert_idx, slots, gates, out, num_tokens, top_k, hidden, experts_per_rank, 0, stream);
}

}  // extern "C"
