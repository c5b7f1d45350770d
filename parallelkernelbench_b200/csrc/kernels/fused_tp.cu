// Fused tensor-parallel kernels: the collective runs inside the GEMM kernel, over peer memory.
//
//  tp_ag_gemm       all-gather -> GEMM (+SiLU). A few CTAs of the persistent grid are communication
//                   CTAs: they push this rank's activation shard into every peer's gather buffer
//                   with 16-byte P2P stores, sub-block by sub-block, and publish one flag per
//                   sub-block with a system-scope release. The other CTAs are the tcgen05 GEMM; its
//                   TMA producer waits (bounded) for the flag of the rows it is about to load and
//                   starts with the local shard, so the transfer hides behind the math.
//  tp_gemm_rs_rmsnorm  GEMM -> reduce-scatter -> RMSNorm. The GEMM walks row blocks in destination
//                   order (rank+1 first, own rows last); its epilogue stores each partial tile
//                   straight into the owner's receive slot and bumps a per-row-block counter there.
//                   After its tiles, every CTA turns into a consumer: it waits for the counters of
//                   its rows, adds the W partial slots in rank order in fp32, applies RMSNorm and
//                   writes bf16 - the reduced tensor never exists un-normalised in memory.
//  tp_gemm_allreduce  GEMM -> all-reduce (row-parallel linear). The same scatter epilogue as above sends every partial
//                   tile to the rank that owns its rows; the consumer phase adds the W partial slots of its rows in
//                   rank order and stores the sum into the result buffer of EVERY rank: one `multimem.st` through
//                   the switch when the group is the whole job and the heap has a multicast mapping, else one
//                   16-byte P2P store per member. A closing barrier tells each rank that all rows have landed.
//  tp_gemm_allgather  GEMM -> all-gather along N (column-parallel linear). The TMA-store epilogue stores every output
//                   tile into the gathered result of every rank at this rank's column block; a closing barrier
//                   tells each rank that all column blocks have landed.
//  tp_gemv_allgather  decode-time LM head: logits of this rank's vocabulary block for 1..4 tokens (memory bound: one warp
//                   per 8 weight rows, 16-byte loads, fp32 accumulation), bias, and the all-gather along the vocabulary
//                   in the same kernel - each group of 8 logits leaves as one 16-byte `multimem.st` (or one P2P store
//                   per member) into every rank's result; results alternate between two buffers so that one closing
//                   barrier per call is enough.
//
// Reference behaviour being replaced: all_gather + matmul + silu, matmul + reduce_scatter,
// reduce_scatter + RMSNorm and matmul + all_reduce as separate NCCL / cuBLAS / elementwise launches
// (reference: reference/15_combined_sharded_gemms.py:17-31, reference/16_gemm_reducescatter.py:19-22,
//  reference/45_reducescatter_fused_rmsnorm.py:23-29, reference/13_gemm_allreduce.py:17-20, reference/14_gemm_allgather.py:17-22,
//  reference/46_gemv_decode.py:13-18).
#include <stdlib.h>

#include "pkb/api.h"
#include "pkb/bulk_copy.cuh"
#include "pkb/collectives_api.h"
#include "pkb/gemm_umma2.cuh"
#include "pkb/host.h"
#include "pkb/symm_host.h"

namespace pkb {

struct TpAgArgs {
  SymmCtx ctx;
  const uint8_t* x_local;  // this rank's shard, rows x K bf16, contiguous
  uint64_t gather_off;     // heap offset of the gather buffer [gsize * rows, K]
  uint64_t flags_off;      // heap offset of the readiness flags [gsize * sub_per_shard] (uint32)
  long long sub_bytes;     // bytes of one sub-block (a_chunk_rows * K * 2)
  int sub_per_shard;
  uint32_t epoch;
  int local_in_place;      // x_local already is the local slice of the gather buffer
  int comm_ctas;
  int bulk_push;           // 1: sub-blocks travel as 16 KiB TMA bulk requests through a shared-memory ring (one issuing thread)
};

// Depth of the push ring: a communication CTA owns the whole dynamic shared memory of the GEMM configuration, and the
// bytes in flight per CTA (ring depth - 2 requests of 16 KiB) decide how few CTAs can keep the link busy.
constexpr int kTpPushStages = 12;
static_assert(bulk_ring_bytes(kTpPushStages) + 128 <= kGemm2SmemTotal, "push ring does not fit the kernel's shared memory");

// Both CTAs of a pair must take the same branch after a cross-GPU barrier: the pair GEMM that follows allocates tensor
// memory for the pair and meets at cluster barriers, so one CTA leaving alone would strand its partner. Every thread of
// both CTAs calls this; it returns true only if `ok` was true in both CTAs.
__device__ __forceinline__ bool cluster_pair_all(bool ok) {
  __shared__ int s_vote;
  if (threadIdx.x == 0) s_vote = ok ? 1 : 0;
  cluster_sync_all();
  int peer;
  const uint32_t peer_addr = mapa_shared(smem_u32(&s_vote), cluster_ctarank() ^ 1u);
  asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(peer) : "r"(peer_addr) : "memory");
  cluster_sync_all();  // the partner has read this CTA's vote before the CTA can exit or vote again
  return ok && peer != 0;
}

__device__ __forceinline__ void ag_push_role(const TpAgArgs& a) {
  const SymmCtx& c = a.ctx;
  // every rank has entered this call, so every rank has finished reading the previous gather
  // bulk form: a communication CTA does no GEMM work, so the kernel's dynamic shared memory is free for the copy ring
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_bulk_abort;
  BulkRing ring;
  if (a.bulk_push && threadIdx.x == 0) {
    s_bulk_abort = 0;
    bulk_ring_init(ring, (smem_u32(smem_raw) + 127u) & ~127u, kTpPushStages);
  }
  if (!symm_block_barrier(c, 300, 1)) return;
  const int W = c.gsize;
  const int total_items = W * a.sub_per_shard;
  // the local shard is read in place by the GEMM (its own tensor map): only remote pushes here
  for (int item = a.sub_per_shard + blockIdx.x; item < total_items; item += a.comm_ctas) {
    const int step = item / a.sub_per_shard;
    const int sb = item - step * a.sub_per_shard;
    int dest_g = c.grank - step;
    if (dest_g < 0) dest_g += W;
    const int dest = c.members[dest_g];
    const int chunk = c.grank * a.sub_per_shard + sb;
    if (a.bulk_push) {
      if (threadIdx.x == 0) {
        const uint8_t* src = a.x_local + (long long)sb * a.sub_bytes;
        uint8_t* dst = symm_ptr<uint8_t>(c, dest, a.gather_off) + (long long)chunk * a.sub_bytes;
        if (!bulk_copy(ring, dst, src, a.sub_bytes, &s_bulk_abort, c.budget_ns))
          record_status(c.status, kStatusMbarTimeout, 300, c.rank, dest, 3, item);
        fence_proxy_async_all();
      }
    } else {
      const uint8_t* src = a.x_local + (long long)sb * a.sub_bytes;
      uint8_t* dst = symm_ptr<uint8_t>(c, dest, a.gather_off) + (long long)chunk * a.sub_bytes;
      const long long nvec = a.sub_bytes >> 4;
      long long i = threadIdx.x;
      // four independent 16-byte loads in flight per thread
      for (; i + 3ll * blockDim.x < nvec; i += 4ll * blockDim.x) {
        U4 v0 = ld_global_nc_v4(src + (i << 4));
        U4 v1 = ld_global_nc_v4(src + ((i + blockDim.x) << 4));
        U4 v2 = ld_global_nc_v4(src + ((i + 2ll * blockDim.x) << 4));
        U4 v3 = ld_global_nc_v4(src + ((i + 3ll * blockDim.x) << 4));
        st_global_v4(dst + (i << 4), v0);
        st_global_v4(dst + ((i + blockDim.x) << 4), v1);
        st_global_v4(dst + ((i + 2ll * blockDim.x) << 4), v2);
        st_global_v4(dst + ((i + 3ll * blockDim.x) << 4), v3);
      }
      for (; i < nvec; i += blockDim.x) st_global_v4(dst + (i << 4), ld_global_nc_v4(src + (i << 4)));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      fence_acq_rel_sys();
      st_release_sys(symm_ptr<uint32_t>(c, dest, a.flags_off) + chunk, a.epoch);
    }
  }
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
tp_ag_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_a_local,
                  const __grid_constant__ GemmOutMaps out_maps, const GemmParams p,
                  const TpAgArgs a) {
  if ((int)blockIdx.x < a.comm_ctas) {
    ag_push_role(a);
    return;
  }
  gemm_umma2_cta<EPI, false, true, false, true>(tmap_a, tmap_b, p, (blockIdx.x - a.comm_ctas) >> 1,
                                                (gridDim.x - a.comm_ctas) >> 1, &out_maps,
                                                &tmap_a_local);
}

// Sum of the partial slots of one output row, kept in registers. Thread t owns the 16-byte chunks t, t + T, t + 2T, ... of
// the row (T = threads of the CTA), at most kRowChunks of them; for every chunk the loads of ALL slots are issued before the
// first addition, so a thread has up to kGemmMaxWorld independent 16-byte loads in flight instead of one (the slots were
// written by peers over NVLink and are read once, from HBM: this phase is bound by loads in flight, not by arithmetic).
// The slots are added in rank order in fp32, so the result does not depend on arrival order.
constexpr int kRowChunks = 8;   // rows of up to 8 * 8 * 192 = 12288 elements stay in registers

__device__ __forceinline__ void sum_slots_chunk(const __nv_bfloat16* p0, long long slot_stride, int gsize, float scale, float (&v)[8]) {
  U4 u[kGemmMaxWorld];
#pragma unroll
  for (int g = 0; g < kGemmMaxWorld; ++g)
    if (g < gsize) u[g] = ld_global_relaxed_v4(p0 + g * slot_stride);   // peers wrote these rows: read them coherently
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = 0.f;
#pragma unroll
  for (int g = 0; g < kGemmMaxWorld; ++g) {
    if (g < gsize) {
      const float2 f0 = unpack_bf16x2(u[g].x), f1 = unpack_bf16x2(u[g].y), f2 = unpack_bf16x2(u[g].z), f3 = unpack_bf16x2(u[g].w);
      v[0] += f0.x; v[1] += f0.y; v[2] += f1.x; v[3] += f1.y;
      v[4] += f2.x; v[5] += f2.y; v[6] += f3.x; v[7] += f3.y;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] *= scale;
}

struct TpRsArgs {
  SymmCtx ctx;
  uint64_t recv_off;     // heap offset of the receive slots [gsize][rows_per_rank, N] bf16
  uint64_t done_off;     // heap offset of the per-row-block arrival counters (uint32)
  uint32_t done_target;  // cumulative arrivals expected per row block once this call is complete
  const __nv_bfloat16* gamma;
  __nv_bfloat16* out;    // [rows_per_rank, N]
  float eps;
  float scale;
  int N;
  int rows_per_rank;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
tp_gemm_rs_rmsnorm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                          const __grid_constant__ CUtensorMap tmap_b,
                          const __grid_constant__ GemmOutMaps out_maps, const GemmParams p,
                          const TpRsArgs a) {
  const SymmCtx& c = a.ctx;
  // all ranks have entered this call => all ranks have consumed the previous call's receive slots
  if (!cluster_pair_all(symm_block_barrier(c, 301, 1))) return;
  gemm_umma2_cta<kEpiNone, false, false, true, true>(tmap_a, tmap_b, p, blockIdx.x >> 1,
                                                     gridDim.x >> 1, &out_maps);
  __syncthreads();

  // ---- consumer phase: reduce the W partial slots of my rows and normalise --------------------
  extern __shared__ uint8_t smem_raw[];
  float* rowbuf = reinterpret_cast<float*>(smem_raw);
  __shared__ float red[8];
  __shared__ int s_ok;
  const uint32_t* done = symm_local<uint32_t>(c, a.done_off);
  const __nv_bfloat16* slots = symm_local<__nv_bfloat16>(c, a.recv_off);
  const long long slot_stride = (long long)a.rows_per_rank * a.N;
  int waited_blk = -1;
  const int nthreads = blockDim.x;
  for (int row = blockIdx.x; row < a.rows_per_rank; row += gridDim.x) {
    const int blk = row / kGemmBlockM;
    if (blk != waited_blk) {
      if (threadIdx.x == 0) {
        s_ok = wait_flag_ge(done + blk, a.done_target, c.budget_ns) ? 1 : 0;
        if (!s_ok) record_status(c.status, kStatusPeerTimeout, 301, c.rank, blk, 2, row);
      }
      __syncthreads();
      if (!s_ok) return;
      waited_blk = blk;
    }
    const __nv_bfloat16* row_slots = slots + (long long)row * a.N;
    __nv_bfloat16* yrow = a.out + (long long)row * a.N;
    if (a.N <= kRowChunks * 8 * nthreads) {
      // the row stays in registers between the sum and the normalisation
      float vals[kRowChunks][8];
      float ss = 0.f;
#pragma unroll
      for (int ch = 0; ch < kRowChunks; ++ch) {
        const int i = (ch * nthreads + (int)threadIdx.x) * 8;
        if (i < a.N) {
          sum_slots_chunk(row_slots + i, slot_stride, c.gsize, a.scale, vals[ch]);
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += vals[ch][j] * vals[ch][j];
        }
      }
      ss = warp_sum(ss);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      float total = 0.f;
      for (int w = 0; w < (nthreads >> 5); ++w) total += red[w];
      const float rstd = rsqrtf(total / (float)a.N + a.eps);
#pragma unroll
      for (int ch = 0; ch < kRowChunks; ++ch) {
        const int i = (ch * nthreads + (int)threadIdx.x) * 8;
        if (i < a.N) {
          const U4 g = ld_global_v4(a.gamma + i);
          const float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z), g3 = unpack_bf16x2(g.w);
          U4 o;
          o.x = pack_bf16x2(vals[ch][0] * rstd * g0.x, vals[ch][1] * rstd * g0.y);
          o.y = pack_bf16x2(vals[ch][2] * rstd * g1.x, vals[ch][3] * rstd * g1.y);
          o.z = pack_bf16x2(vals[ch][4] * rstd * g2.x, vals[ch][5] * rstd * g2.y);
          o.w = pack_bf16x2(vals[ch][6] * rstd * g3.x, vals[ch][7] * rstd * g3.y);
          st_global_v4(yrow + i, o);
        }
      }
      __syncthreads();        // red[] is reused by the next row
      continue;
    }
    // rows too long for registers: fp32 row buffer in shared memory
    float ss = 0.f;
    for (int i = threadIdx.x * 8; i < a.N; i += nthreads * 8) {
      float v[8];
      sum_slots_chunk(row_slots + i, slot_stride, c.gsize, a.scale, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        rowbuf[i + j] = v[j];
        ss += v[j] * v[j];
      }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < (nthreads >> 5); ++w) total += red[w];
    const float rstd = rsqrtf(total / (float)a.N + a.eps);
    for (int i = threadIdx.x * 8; i < a.N; i += nthreads * 8) {
      U4 g = ld_global_v4(a.gamma + i);
      float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z),
             g3 = unpack_bf16x2(g.w);
      U4 o;
      o.x = pack_bf16x2(rowbuf[i] * rstd * g0.x, rowbuf[i + 1] * rstd * g0.y);
      o.y = pack_bf16x2(rowbuf[i + 2] * rstd * g1.x, rowbuf[i + 3] * rstd * g1.y);
      o.z = pack_bf16x2(rowbuf[i + 4] * rstd * g2.x, rowbuf[i + 5] * rstd * g2.y);
      o.w = pack_bf16x2(rowbuf[i + 6] * rstd * g3.x, rowbuf[i + 7] * rstd * g3.y);
      st_global_v4(yrow + i, o);
    }
    __syncthreads();
  }
}

struct TpArArgs {
  SymmCtx ctx;
  uint64_t recv_off;     // heap offset of the receive slots [gsize][rows_per_rank, N] bf16
  uint64_t done_off;     // heap offset of the per-row-block arrival counters (uint32)
  uint32_t done_target;  // cumulative arrivals expected per row block once this call is complete
  uint64_t out_off;      // heap offset of the all-reduced result [gsize * rows_per_rank, N] bf16 (same on every rank)
  float scale;
  int N;
  int rows_per_rank;
  int use_mc;            // 1: broadcast the reduced rows with multimem.st (whole-job group with a multicast mapping)
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
tp_gemm_allreduce_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ GemmOutMaps out_maps, const GemmParams p,
                         const TpArArgs a) {
  const SymmCtx& c = a.ctx;
  // all ranks have entered this call => all ranks have consumed the previous call's receive slots and result
  if (!cluster_pair_all(symm_block_barrier(c, 302, 1))) return;
  gemm_umma2_cta<kEpiNone, false, false, true, true>(tmap_a, tmap_b, p, blockIdx.x >> 1,
                                                     gridDim.x >> 1, &out_maps);
  __syncthreads();

  // ---- consumer phase: reduce the W partial slots of my rows, store the sums on every rank ----
  __shared__ int s_ok;
  const uint32_t* done = symm_local<uint32_t>(c, a.done_off);
  const __nv_bfloat16* slots = symm_local<__nv_bfloat16>(c, a.recv_off);
  const long long slot_stride = (long long)a.rows_per_rank * a.N;
  const long long my_row0 = (long long)c.grank * a.rows_per_rank;
  int waited_blk = -1;
  const int nthreads = blockDim.x;
  for (int row = blockIdx.x; row < a.rows_per_rank; row += gridDim.x) {
    const int blk = row / kGemmBlockM;
    if (blk != waited_blk) {
      if (threadIdx.x == 0) {
        s_ok = wait_flag_ge(done + blk, a.done_target, c.budget_ns) ? 1 : 0;
        if (!s_ok) record_status(c.status, kStatusPeerTimeout, 302, c.rank, blk, 2, row);
      }
      __syncthreads();
      if (!s_ok) return;
      waited_blk = blk;
    }
    for (int i = threadIdx.x * 8; i < a.N; i += nthreads * 8) {
      float acc[8];
      sum_slots_chunk(slots + (long long)row * a.N + i, slot_stride, c.gsize, a.scale, acc);
      U4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      const long long eoff = (my_row0 + row) * a.N + i;
      if (a.use_mc) {
        multimem_st_v4(symm_mc<__nv_bfloat16>(c, a.out_off) + eoff, o);
      } else {
        for (int k = 0; k < c.gsize; ++k) {
          int g = c.grank + k;       // own copy first, peers spread over time
          if (g >= c.gsize) g -= c.gsize;
          st_global_v4(symm_ptr<__nv_bfloat16>(c, c.members[g], a.out_off) + eoff, o);
        }
      }
    }
  }
  // every same-index block of every rank has stored its rows once this barrier passes; the kernel ends on a rank
  // only after all its blocks passed, i.e. after all rows of all ranks have landed here
  symm_block_barrier(c, 302, 3);
}


template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
tp_gemm_allgather_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ GemmOutMaps out_maps, const GemmParams p,
                         const __grid_constant__ SymmCtx c) {
  // all ranks have entered this call => all ranks have consumed the previous call's gathered result
  if (!cluster_pair_all(symm_block_barrier(c, 303, 1))) return;
  gemm_umma2_cta<EPI, false, false, false, true, true>(tmap_a, tmap_b, p, blockIdx.x >> 1, gridDim.x >> 1, &out_maps);
  // the same-index blocks of every rank have completed their stores once this barrier passes
  symm_block_barrier(c, 303, 2);
}

struct TpGemvArgs {
  SymmCtx ctx;
  const __nv_bfloat16* h;     // [M, K] activations (the same on every rank)
  const __nv_bfloat16* w;     // [n_local, K] this rank's rows of the weight
  const __nv_bfloat16* bias;  // [n_local] or nullptr
  uint64_t out_off;           // heap offset of the result buffer of this call: [M, gsize * n_local] bf16
  int K, n_local;
  long long ldw;              // elements between rows of w
  int use_mc;
};

// One warp computes 8 consecutive logits for all M tokens: per 16-byte chunk of K it loads the chunk of the M activation
// rows once and of 8 weight rows (8 independent loads in flight), accumulates in fp32, reduces across the warp.
template <int M>
__global__ void __launch_bounds__(256) tp_gemv_allgather_kernel(const TpGemvArgs a) {
  const SymmCtx& c = a.ctx;
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int groups = a.n_local >> 3;
  const long long n_total = (long long)c.gsize * a.n_local;
  for (int grp = blockIdx.x * warps_per_block + (threadIdx.x >> 5); grp < groups; grp += gridDim.x * warps_per_block) {
    const int n0 = grp << 3;
    float acc[8][M];
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
    for (int k = lane * 8; k < a.K; k += 256) {
      float hv[M][8];
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const U4 u = ld_global_nc_v4(a.h + (long long)m * a.K + k);
        const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
        hv[m][0] = f0.x; hv[m][1] = f0.y; hv[m][2] = f1.x; hv[m][3] = f1.y;
        hv[m][4] = f2.x; hv[m][5] = f2.y; hv[m][6] = f3.x; hv[m][7] = f3.y;
      }
      U4 wv[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) wv[r] = ld_global_nc_v4(a.w + (long long)(n0 + r) * a.ldw + k);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float2 f0 = unpack_bf16x2(wv[r].x), f1 = unpack_bf16x2(wv[r].y), f2 = unpack_bf16x2(wv[r].z),
                     f3 = unpack_bf16x2(wv[r].w);
        const float wf[8] = {f0.x, f0.y, f1.x, f1.y, f2.x, f2.y, f3.x, f3.y};
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[r][m] = fmaf(wf[j], hv[m][j], acc[r][m]);
      }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = warp_sum(acc[r][m]);
    if (lane == 0) {
      float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (a.bias != nullptr) {
#pragma unroll
        for (int r = 0; r < 8; ++r) b[r] = __bfloat162float(a.bias[n0 + r]);
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        U4 o{pack_bf16x2(acc[0][m] + b[0], acc[1][m] + b[1]), pack_bf16x2(acc[2][m] + b[2], acc[3][m] + b[3]),
             pack_bf16x2(acc[4][m] + b[4], acc[5][m] + b[5]), pack_bf16x2(acc[6][m] + b[6], acc[7][m] + b[7])};
        const long long eoff = (long long)m * n_total + (long long)c.grank * a.n_local + n0;
        if (a.use_mc) {
          multimem_st_v4(symm_mc<__nv_bfloat16>(c, a.out_off) + eoff, o);
        } else {
          for (int g = 0; g < c.gsize; ++g) st_global_v4(symm_ptr<__nv_bfloat16>(c, c.members[g], a.out_off) + eoff, o);
        }
      }
    }
  }
  // all same-index blocks of all ranks have stored their logits once this barrier passes
  symm_block_barrier(c, 304, 1);
}

}  // namespace pkb

using namespace pkb;

// device buffer that receives, per CTA of pkb_tp_ag_gemm, the cycles its producer waited for gathered rows (null: off)
static unsigned long long* g_ag_wait_stats = nullptr;

extern "C" {

// Instrumentation of pkb_tp_ag_gemm: `dev_words` points to at least 148 zeroed 64-bit words of device memory (or null to
// switch it off). Every later call adds, per CTA, the SM cycles its TMA producer spent waiting for rows from the peers.
int pkb_tp_ag_gemm_set_wait_stats(void* dev_words) {
  g_ag_wait_stats = static_cast<unsigned long long*>(dev_words);
  return kApiOk;
}

// Default number of communication CTAs of the all-gather -> GEMM kernel for a group of `world` ranks (bulk_push: the TMA bulk
// ring; otherwise the thread-copy push). Exposed so that the rule can be checked without a GPU.
extern "C" int pkb_tp_default_comm_ctas(int world, int bulk_push) {
  if (world <= 1) return 2;
  if (bulk_push) return world >= 8 ? 16 : (world > 4 ? 12 : 8);
  return world >= 8 ? 16 : 8;
}

// C[gsize*rows, N] = epi( allgather(x_local)[gsize*rows, K] @ w[N, K]^T ), C local bf16.
// gather_off / flags_off: heap offsets of the gather buffer (gsize*rows*K bf16) and of
// gsize * (rows / a_chunk_rows) uint32 flags. `epoch` must grow by one on every call (same value
// on all ranks). comm_ctas CTAs of the grid push the shard to the peers.
int pkb_tp_ag_gemm(const pkb_symm_ctx* h, const void* x_local, int rows, int K,
                   unsigned long long gather_off, unsigned long long flags_off, int a_chunk_rows,
                   unsigned int epoch, const void* w, long long ldb, void* c, long long ldc, int N,
                   int epilogue, int comm_ctas, void* stream) {
  PKB_CHECK_ARG(h && h->base, "symmetric heap not initialised");
  PKB_CHECK_ARG(h->gsize >= 1 && h->gsize <= kGemmMaxWorld, "group size must be 1..8");
  PKB_CHECK_ARG(rows > 0 && K % 8 == 0 && N > 0, "bad shapes");
  PKB_CHECK_ARG(a_chunk_rows % kGemmBlockM == 0 && rows % a_chunk_rows == 0,
                "a_chunk_rows must be a multiple of 128 that divides rows");
  PKB_CHECK_ARG(rows % kGemm2TileM == 0, "rows per rank must be a multiple of 256");
  PKB_CHECK_ARG(epilogue == kEpiNone || epilogue == kEpiSilu, "epilogue must be none or silu");
  PKB_CHECK_ARG((gather_off & 1023) == 0 && (flags_off & 15) == 0, "heap offsets misaligned");
  const int W = h->gsize;
  const int M = W * rows;
  SymmCtx ctx = symm_ctx_from_api(h);
  uint8_t* g_local = reinterpret_cast<uint8_t*>(h->base + (uint64_t)h->rank * h->stride + gather_off);

  CUtensorMap ta, tb;
  int rc = encode_tmap_2d(&ta, kTmapBf16, g_local, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2,
                          kGemmBlockK, kGemmBlockM, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_2d(&tb, kTmapBf16, w, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, kGemmBlockK, 128,
                      kSwizzle128);
  if (rc) return rc;
  PKB_CHECK_ARG((reinterpret_cast<uintptr_t>(x_local) & 15) == 0, "x_local must be 16-byte aligned");
  CUtensorMap tal;
  rc = encode_tmap_2d(&tal, kTmapBf16, x_local, (uint64_t)K, (uint64_t)rows, (uint64_t)K * 2, kGemmBlockK,
                      kGemmBlockM, kSwizzle128);
  if (rc) return rc;

  PKB_CHECK_ARG(ldc % 8 == 0 && (reinterpret_cast<uintptr_t>(c) & 15) == 0,
                "output must be 16-byte aligned with ldc a multiple of 8");
  GemmOutMaps om;
  rc = encode_tmap_2d(&om.m[0], kTmapBf16, c, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 2, 64, 32,
                      kSwizzle128);
  if (rc) return rc;

  GemmParams p = {};
  p.M = M; p.N = N; p.K = K; p.C = c; p.ldc = ldc; p.alpha = 1.0f;
  p.status = ctx.status; p.wait_budget_ns = ctx.budget_ns;
  p.kernel_id = 300;
  p.rank = h->rank; p.world = W;
  p.a_ready = reinterpret_cast<const uint32_t*>(h->base + (uint64_t)h->rank * h->stride + flags_off);
  p.a_ready_epoch = epoch;
  p.a_chunk_rows = a_chunk_rows;
  p.a_local_row0 = h->grank * rows;
  p.a_local_rows = rows;
  p.a_wait_cycles = g_ag_wait_stats;
  const int blocks_per_shard = rows / kGemm2TileM;
  p.group_m = blocks_per_shard < 8 ? blocks_per_shard : 8;
  // keep whole shards inside rasterisation groups when possible
  while (blocks_per_shard % p.group_m != 0) --p.group_m;
  p.m_block_rotation = h->grank * blocks_per_shard;  // local rows first, then rank+1, ...

  TpAgArgs a;
  a.ctx = ctx;
  a.x_local = static_cast<const uint8_t*>(x_local);
  a.gather_off = gather_off; a.flags_off = flags_off;
  a.sub_bytes = (long long)a_chunk_rows * K * 2;
  a.sub_per_shard = rows / a_chunk_rows;
  a.epoch = epoch;
  a.local_in_place = (x_local == g_local + (long long)h->grank * rows * K * 2) ? 1 : 0;
  // The shard travels as 16 KiB TMA bulk requests through a shared-memory ring, one issuing thread per communication CTA
  // (PKB_TP_BULK_PUSH=0 selects the older form: 16-byte loads and stores by all threads of the CTA). With thread copies
  // the rate is bound by the loads a CTA can keep in flight, so many CTAs are needed and the step time follows their
  // number (8 ranks, 2048 x 8192 rows per rank, ms per TP-MLP block: 8 CTAs 2.24, 16 CTAs 1.95, 24 CTAs 2.03); a bulk ring
  // keeps 160 KiB in flight per CTA, so a few CTAs fill the link and the rest of the SMs stay with the GEMM.
  static const bool bulk_off = [] { const char* e = getenv("PKB_TP_BULK_PUSH"); return e != nullptr && e[0] == '0'; }();
  a.bulk_push = (!bulk_off && a.sub_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(x_local) & 15) == 0) ? 1 : 0;
  // Number of communication CTAs: a bulk-push CTA sustains about 36 GB/s (measured at 4 ranks: 4 CTAs made the GEMM's
  // producers wait 169 us per call for 96 MiB of remote rows, 8 CTAs 2 us), and the GEMM consumes one remote shard per
  // 1/W of its run time, so the rate the push needs grows with W while the shard size stays: 8 CTAs cover a 32 MiB shard in
  // 115 us, which is enough up to 4 ranks (175 us per shard of GEMM time) and not at 8 ranks (87 us), where 16 are used.
  if (comm_ctas <= 0) comm_ctas = pkb_tp_default_comm_ctas(W, a.bulk_push);
  comm_ctas = (comm_ctas + 1) & ~1;  // whole clusters
  const int sms = sm_count() & ~1;
  PKB_CHECK_ARG(comm_ctas < sms && comm_ctas <= kSymmMaxBlocks, "too many communication CTAs");
  a.comm_ctas = comm_ctas;

  constexpr int smem = kGemm2SmemTotal;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (epilogue == kEpiSilu) {
    auto k = tp_ag_gemm_kernel<kEpiSilu>;
    PKB_CHECK_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    k<<<sms, kGemmThreads, smem, s>>>(ta, tb, tal, om, p, a);
  } else {
    auto k = tp_ag_gemm_kernel<kEpiNone>;
    PKB_CHECK_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    k<<<sms, kGemmThreads, smem, s>>>(ta, tb, tal, om, p, a);
  }
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// out[rows_per_rank, N] = RMSNorm( reduce_scatter( a[gsize*rows_per_rank, K] @ w[N, K]^T ) * scale )
// recv_off: heap offset of gsize receive slots of rows_per_rank*N bf16; done_off: heap offset of
// rows_per_rank/128 uint32 counters; call_index counts calls on these buffers starting at 1.
int pkb_tp_gemm_rs_rmsnorm(const pkb_symm_ctx* h, const void* a_mat, long long lda, const void* w,
                           long long ldb, int rows_per_rank, int N, int K,
                           unsigned long long recv_off, unsigned long long done_off,
                           unsigned int call_index, const void* gamma, void* out, float eps,
                           float scale, void* stream) {
  PKB_CHECK_ARG(h && h->base, "symmetric heap not initialised");
  PKB_CHECK_ARG(h->gsize >= 1 && h->gsize <= kGemmMaxWorld, "group size must be 1..8");
  PKB_CHECK_ARG(rows_per_rank % kGemm2TileM == 0, "rows_per_rank must be a multiple of 256");
  PKB_CHECK_ARG(N % 8 == 0 && K % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0, "N, K, lda, ldb must be multiples of 8");
  PKB_CHECK_ARG(N * 4 <= kGemm2SmemTotal, "row too long for the shared-memory row buffer");
  PKB_CHECK_ARG((recv_off & 15) == 0 && (done_off & 15) == 0, "heap offsets misaligned");
  const int W = h->gsize;
  const int M = W * rows_per_rank;
  SymmCtx ctx = symm_ctx_from_api(h);

  CUtensorMap ta, tb;
  int rc = encode_tmap_2d(&ta, kTmapBf16, a_mat, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2,
                          kGemmBlockK, kGemmBlockM, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_2d(&tb, kTmapBf16, w, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, kGemmBlockK, 128,
                      kSwizzle128);
  if (rc) return rc;

  GemmOutMaps om;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K; p.C = nullptr; p.ldc = N; p.alpha = 1.0f;
  p.status = ctx.status; p.wait_budget_ns = ctx.budget_ns;
  p.kernel_id = 301;
  p.rank = h->rank; p.world = W;
  p.rs_rows_per_rank = rows_per_rank;
  const long long slot_bytes = (long long)rows_per_rank * N * 2;
  for (int g = 0; g < W; ++g) {
    const uint64_t peer = h->base + (uint64_t)h->members[g] * h->stride;
    p.rs_out[g] = reinterpret_cast<void*>(peer + recv_off + (uint64_t)h->grank * slot_bytes);
    p.rs_done[g] = reinterpret_cast<uint32_t*>(peer + done_off);
    rc = encode_tmap_2d(&om.m[g], kTmapBf16, p.rs_out[g], (uint64_t)N, (uint64_t)rows_per_rank,
                        (uint64_t)N * 2, 64, 32, kSwizzle128);
    if (rc) return rc;
  }
  const int blocks_per_rank = rows_per_rank / kGemm2TileM;
  p.group_m = blocks_per_rank < 8 ? blocks_per_rank : 8;
  while (blocks_per_rank % p.group_m != 0) --p.group_m;
  p.m_block_rotation = ((h->grank + 1) % W) * blocks_per_rank;  // rank+1's rows first, own rows last

  const int num_n = (N + 255) / 256;
  TpRsArgs a;
  a.ctx = ctx;
  a.recv_off = recv_off; a.done_off = done_off;
  a.done_target = call_index * (uint32_t)(W * num_n * 4);
  a.gamma = static_cast<const __nv_bfloat16*>(gamma);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.eps = eps; a.scale = scale; a.N = N; a.rows_per_rank = rows_per_rank;

  constexpr int smem = kGemm2SmemTotal;
  auto k = tp_gemm_rs_rmsnorm_kernel;
  PKB_CHECK_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  int grid = sm_count() & ~1;
  if (grid > kSymmMaxBlocks) grid = kSymmMaxBlocks;
  k<<<grid, kGemmThreads, smem, static_cast<cudaStream_t>(stream)>>>(ta, tb, om, p, a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// result[gsize * rows_per_rank, N] (bf16, at heap offset out_off on every rank) = scale * all_reduce( a @ w^T ), with
// a [gsize * rows_per_rank, K] and w [N, K] this rank's K-shard of a row-parallel linear layer. recv_off / done_off /
// call_index as for pkb_tp_gemm_rs_rmsnorm. N % 8 == 0. The result is valid on this rank when the kernel has finished.
int pkb_tp_gemm_allreduce(const pkb_symm_ctx* h, const void* a_mat, long long lda, const void* w, long long ldb,
                          int rows_per_rank, int N, int K, unsigned long long recv_off, unsigned long long done_off,
                          unsigned int call_index, unsigned long long out_off, float scale, int allow_multicast,
                          void* stream) {
  PKB_CHECK_ARG(h && h->base, "symmetric heap not initialised");
  PKB_CHECK_ARG(h->gsize >= 1 && h->gsize <= kGemmMaxWorld, "group size must be 1..8");
  PKB_CHECK_ARG(rows_per_rank % kGemm2TileM == 0, "rows_per_rank must be a multiple of 256");
  PKB_CHECK_ARG(N % 8 == 0 && K % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0, "N, K, lda, ldb must be multiples of 8");
  PKB_CHECK_ARG((recv_off & 15) == 0 && (done_off & 15) == 0 && (out_off & 15) == 0, "heap offsets misaligned");
  const int W = h->gsize;
  const int M = W * rows_per_rank;
  SymmCtx ctx = symm_ctx_from_api(h);

  CUtensorMap ta, tb;
  int rc = encode_tmap_2d(&ta, kTmapBf16, a_mat, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2,
                          kGemmBlockK, kGemmBlockM, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_2d(&tb, kTmapBf16, w, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, kGemmBlockK, 128,
                      kSwizzle128);
  if (rc) return rc;

  GemmOutMaps om;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K; p.C = nullptr; p.ldc = N; p.alpha = 1.0f;
  p.status = ctx.status; p.wait_budget_ns = ctx.budget_ns;
  p.kernel_id = 302;
  p.rank = h->rank; p.world = W;
  p.rs_rows_per_rank = rows_per_rank;
  const long long slot_bytes = (long long)rows_per_rank * N * 2;
  for (int g = 0; g < W; ++g) {
    const uint64_t peer = h->base + (uint64_t)h->members[g] * h->stride;
    p.rs_out[g] = reinterpret_cast<void*>(peer + recv_off + (uint64_t)h->grank * slot_bytes);
    p.rs_done[g] = reinterpret_cast<uint32_t*>(peer + done_off);
    rc = encode_tmap_2d(&om.m[g], kTmapBf16, p.rs_out[g], (uint64_t)N, (uint64_t)rows_per_rank,
                        (uint64_t)N * 2, 64, 32, kSwizzle128);
    if (rc) return rc;
  }
  const int blocks_per_rank = rows_per_rank / kGemm2TileM;
  p.group_m = blocks_per_rank < 8 ? blocks_per_rank : 8;
  while (blocks_per_rank % p.group_m != 0) --p.group_m;
  p.m_block_rotation = ((h->grank + 1) % W) * blocks_per_rank;  // rank+1's rows first, own rows last

  const int num_n = (N + 255) / 256;
  TpArArgs a;
  a.ctx = ctx;
  a.recv_off = recv_off; a.done_off = done_off; a.out_off = out_off;
  a.done_target = call_index * (uint32_t)(W * num_n * 4);
  a.scale = scale; a.N = N; a.rows_per_rank = rows_per_rank;
  a.use_mc = (allow_multicast && h->mc_base != 0 && h->gsize == h->world && W > 1) ? 1 : 0;

  constexpr int smem = kGemm2SmemTotal;
  auto k = tp_gemm_allreduce_kernel;
  PKB_CHECK_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  int grid = sm_count() & ~1;
  if (grid > kSymmMaxBlocks) grid = kSymmMaxBlocks;
  k<<<grid, kGemmThreads, smem, static_cast<cudaStream_t>(stream)>>>(ta, tb, om, p, a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// result[M, gsize * n_local] (bf16, at heap offset out_off on every rank) = all_gather along N of epi(a @ w^T + bias), with
// a [M, K] (the same on every rank) and w [n_local, K] this rank's block of output features. n_local % 64 == 0.
// epilogue: 0 none, 1 SiLU, 2 bias, 3 bias + SiLU. The result is valid on this rank when the kernel has finished.
int pkb_tp_gemm_allgather(const pkb_symm_ctx* h, const void* a_mat, long long lda, const void* w, long long ldb, int M,
                          int n_local, int K, const void* bias, int epilogue, unsigned long long out_off, void* stream) {
  PKB_CHECK_ARG(h && h->base, "symmetric heap not initialised");
  PKB_CHECK_ARG(h->gsize >= 1 && h->gsize <= kGemmMaxWorld, "group size must be 1..8");
  PKB_CHECK_ARG(M > 0 && n_local > 0 && n_local % 64 == 0, "n_local must be a positive multiple of 64");
  PKB_CHECK_ARG(K % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0, "K, lda, ldb must be multiples of 8");
  PKB_CHECK_ARG((out_off & 1023) == 0, "heap offset misaligned");
  PKB_CHECK_ARG(epilogue >= kEpiNone && epilogue <= kEpiBiasSilu, "unknown epilogue");
  PKB_CHECK_ARG((epilogue & 2) == 0 || bias != nullptr, "bias epilogue without bias");
  const int W = h->gsize;
  SymmCtx ctx = symm_ctx_from_api(h);
  CUtensorMap ta, tb;
  int rc = encode_tmap_2d(&ta, kTmapBf16, a_mat, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, kGemmBlockK, kGemmBlockM,
                          kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_2d(&tb, kTmapBf16, w, (uint64_t)K, (uint64_t)n_local, (uint64_t)ldb * 2, kGemmBlockK, 128, kSwizzle128);
  if (rc) return rc;
  GemmOutMaps om;
  const long long n_total = (long long)W * n_local;
  for (int g = 0; g < W; ++g) {
    void* dst = reinterpret_cast<void*>(h->base + (uint64_t)h->members[g] * h->stride + out_off);
    rc = encode_tmap_2d(&om.m[g], kTmapBf16, dst, (uint64_t)n_total, (uint64_t)M, (uint64_t)n_total * 2, 64, 32, kSwizzle128);
    if (rc) return rc;
  }
  GemmParams p = {};
  p.M = M; p.N = n_local; p.K = K; p.C = nullptr; p.ldc = n_total; p.alpha = 1.0f;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.status = ctx.status; p.wait_budget_ns = ctx.budget_ns;
  p.kernel_id = 303;
  p.rank = h->rank; p.world = W;
  p.rank_in_group = h->grank;
  p.bcast_col0 = h->grank * n_local;
  p.group_m = 8;
  int grid = sm_count() & ~1;
  if (grid > kSymmMaxBlocks) grid = kSymmMaxBlocks;
  constexpr int smem = kGemm2SmemTotal;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define PKB_GAG(EPI)                                                                             \
  {                                                                                              \
    auto k = tp_gemm_allgather_kernel<EPI>;                                                      \
    PKB_CHECK_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
    k<<<grid, kGemmThreads, smem, s>>>(ta, tb, om, p, ctx);                                      \
  }
  switch (epilogue) {
    case kEpiNone: PKB_GAG(kEpiNone) break;
    case kEpiSilu: PKB_GAG(kEpiSilu) break;
    case kEpiBias: PKB_GAG(kEpiBias) break;
    default: PKB_GAG(kEpiBiasSilu) break;
  }
#undef PKB_GAG
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// logits[M, gsize * n_local] (bf16, at heap offset out_off on every rank) = all_gather along the vocabulary of h @ w^T + bias
// for M in {1, 2, 4} tokens: h [M, K] the same on every rank, w [n_local, K] this rank's rows. K % 8 == 0, n_local % 8 == 0,
// all pointers 16-byte aligned. Consecutive calls must alternate between two result buffers (there is no entry barrier);
// the result is valid on this rank when the kernel has finished.
int pkb_tp_gemv_allgather(const pkb_symm_ctx* h, const void* act, const void* w, long long ldw, const void* bias, int M,
                          int n_local, int K, unsigned long long out_off, int allow_multicast, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(M == 1 || M == 2 || M == 4, "1, 2 or 4 tokens");
  PKB_CHECK_ARG(K > 0 && K % 8 == 0 && n_local > 0 && n_local % 8 == 0 && ldw % 8 == 0, "K, n_local, ldw must be multiples of 8");
  PKB_CHECK_ARG(((reinterpret_cast<uintptr_t>(act) | reinterpret_cast<uintptr_t>(w) | out_off) & 15) == 0, "16-byte alignment");
  PKB_CHECK_ARG((((long long)h->gsize * n_local) & 7) == 0, "row pitch of the result must be a multiple of 8");
  TpGemvArgs a;
  a.ctx = symm_ctx_from_api(h);
  a.h = static_cast<const __nv_bfloat16*>(act);
  a.w = static_cast<const __nv_bfloat16*>(w);
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.out_off = out_off; a.K = K; a.n_local = n_local; a.ldw = ldw;
  a.use_mc = (allow_multicast && h->mc_base != 0 && h->gsize == h->world && h->gsize > 1) ? 1 : 0;
  int grid = sm_count();           // the same on every rank: the closing barrier pairs blocks by index
  if (grid > kSymmMaxBlocks) grid = kSymmMaxBlocks;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (M == 1) tp_gemv_allgather_kernel<1><<<grid, 256, 0, s>>>(a);
  else if (M == 2) tp_gemv_allgather_kernel<2><<<grid, 256, 0, s>>>(a);
  else tp_gemv_allgather_kernel<4><<<grid, 256, 0, s>>>(a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

}  // extern "C"
