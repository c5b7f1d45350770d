// Flash-attention backward on tcgen05 / TMEM.
//
// One CTA owns one 128-row KV tile of one KV head and walks every (query head of the group, 128-row Q tile) pair
// that can see it. Per pair, from the saved forward (O, log-sum-exp):
//     S  = Q K^T                         (tensor core, TMEM)
//     dP = dO V^T                        (tensor core, TMEM)
//     P  = exp2(S * scale * log2e - lse2)            dS = P * (dP - delta) * scale     (softmax warps, thread = q row)
//     dV += P^T dO     dK += dS^T Q      (tensor core, accumulate in TMEM over the whole walk - no atomics, GQA summed)
//     dQ_partial = dS K                  (tensor core, into the TMEM columns S has just left) -> fp32 vector `red` into dQ
// delta = rowsum(dO * O) and lse2 = lse * log2e come from a small pre-kernel.
//
//   warp 0      TMA producer: K_j, V_j once; Q_i and dO_i per step
//   warp 1      MMA issuer
//   warps 4-11  softmax / dS (thread = q row; warps 4-7 take KV columns 0-63, warps 8-11 columns 64-127): read S and dP
//               from TMEM, write P and dS as bf16 into 128-byte-swizzled shared memory; the same [q][kv] tiles serve
//               as K-major A (dS for dQ) and as MN-major A (P^T, dS^T)
//   warps 12-15 dQ drain (thread = q row), and at the end dV, dK
// K_j ([kv][d]) is the K-major B operand of S and the MN-major B operand of dQ; Q_i and dO_i are K-major A operands of
// S / dP and MN-major B operands of dK / dV: every tile is loaded once and read through two descriptors.
//
// Positions follow the forward kernel's segment description, so causal masks in context-parallel (zigzag) layouts are
// exact. Reference behaviour replaced: materialised fp32 scores and their softmax per ring step
// (reference: reference/57_ring_attention_backward_dp.py:39-69).
#include "pkb/api.h"
#include "pkb/attention_api.h"
#include "pkb/host.h"
#include "pkb/ptx.cuh"

namespace pkb {

constexpr int kFbThreads = 512;
constexpr int kFbTile = 128;
constexpr float kFbLog2e = 1.4426950408889634f;

struct FaBwdParams {
  pkb_attn_desc d;
  const float* lse2;    // [batch, hq, sq]  log-sum-exp in base-2 units
  const float* delta;   // [batch, hq, sq]  rowsum(dO * O)
  float* dq;            // [batch * sq, hq, D] fp32, zero-initialised by the caller
  float* dk;            // [batch * skv, hkv, D] fp32
  float* dv;            // [batch * skv, hkv, D] fp32
  // Context-parallel form: when seg_scatter != 0 the dK / dV rows of KV segment s are ADDED (fp32 vector reductions) into
  // dk_seg[s] / dv_seg[s], which point at row 0 of that segment inside the accumulator of the rank that owns the rows -
  // peer memory for remote segments, so the partial sums go home from the epilogue instead of through a reduce-scatter.
  int seg_scatter;
  float* dk_seg[16];
  float* dv_seg[16];
  uint32_t* status;
  uint64_t budget_ns;
  long long* trace;     // optional: CTA (0,0,0) stamps clock64 at its hand-overs (see fb_trace)
};

// Device-side trace: a plain store into the slot of (role, step, event); roles 0 issuing warp, 1 P / dS warps (first warp),
// 2 dQ drain warps (first warp). Layout: [3 roles][kFbTraceSteps][8 events] int64.
constexpr int kFbTraceSteps = 160;
__device__ __forceinline__ void fb_trace(const FaBwdParams& p, int role, int event, int step) {
  if (p.trace == nullptr || blockIdx.x != 0 || blockIdx.y != 0 || blockIdx.z != 0 || step >= kFbTraceSteps) return;
  long long t;
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)::"memory");
  p.trace[(role * kFbTraceSteps + step) * 8 + event] = t;
}

template <int D>
struct FbSmem {
  static constexpr int kTileBytes = kFbTile * D * 2;
  static constexpr int kPBytes = kFbTile * kFbTile * 2;
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTileBytes;
  static constexpr int kQ = kV + kTileBytes;
  static constexpr int kDO = kQ + kTileBytes;
  static constexpr int kP = kDO + kTileBytes;
  static constexpr int kDS = kP + kPBytes;
  // dQ staging: half of a step's fp32 partial at a time ([128 rows][D / 2] with a row pitch of D * 2 + 16 bytes, which is
  // conflict-free for threads that each write their own row). A buffer of its own, so that the reductions of step s run
  // under the products and the P / dS computation of step s+1.
  static constexpr int kDqPitch = D * 2 + 16;
  static constexpr int kDqStage = kDS + kPBytes;
  static constexpr int kBars = kDqStage + kFbTile * kDqPitch;
  static constexpr int kTotal = kBars + 256;
  static_assert(kTotal <= 232448, "shared-memory plan exceeds the 227 KiB a CTA may use");
};

// delta[b,h,s] = sum_d dO * O ; lse2 = lse * log2(e). One warp per (token, head).
__global__ void __launch_bounds__(256)
fa_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout, const float* __restrict__ lse,
                   float* __restrict__ delta, float* __restrict__ lse2, int batch, int sq, int hq, int D) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long total = (long long)batch * sq * hq;
  for (long long i = warp; i < total; i += nwarps) {
    const int h = (int)(i % hq);
    const long long tok = i / hq;                 // batch * sq + s
    const __nv_bfloat16* op = o + (tok * hq + h) * D;
    const __nv_bfloat16* dp = dout + (tok * hq + h) * D;
    float acc = 0.f;
    for (int c = lane; c < D; c += 32) acc += __bfloat162float(op[c]) * __bfloat162float(dp[c]);
    acc = warp_sum(acc);
    if (lane == 0) {
      const int b = (int)(tok / sq), s = (int)(tok % sq);
      const long long idx = ((long long)b * hq + h) * sq + s;
      delta[idx] = acc;
      lse2[idx] = lse[idx] * kFbLog2e;
    }
  }
}

__device__ __forceinline__ void red_add_v4_f32(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Position of Q row `row` (inside one batch entry) and whether the 128-row tile starting there can see kv position kp0.
__device__ __forceinline__ int fb_q_pos(const pkb_attn_desc& d, int row) {
  const int seg = row / d.q_seg_rows;
  return d.q_seg_pos[seg] + (row - seg * d.q_seg_rows);
}

template <int D, bool TRACE = false>
__global__ void __launch_bounds__(kFbThreads, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
              const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
              const FaBwdParams p) {
  using S = FbSmem<D>;
  constexpr int kAtoms = D / 64;
  constexpr int kAtomBytes = kFbTile * 128;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sb = smem_u32(smem);
  const pkb_attn_desc& d = p.d;

  const uint32_t bar0 = sb + S::kBars;
  const uint32_t kv_full = bar0;
  const uint32_t qdo_full = bar0 + 8;
  const uint32_t qdo_empty = bar0 + 16;
  const uint32_t sdp_full = bar0 + 24;    // S and dP in TMEM
  const uint32_t pds_full = bar0 + 32;    // P and dS in shared memory (and S, dP read out of TMEM)
  const uint32_t pds_empty = bar0 + 40;   // the MMAs that read P and dS are complete
  const uint32_t dq_full = bar0 + 48;     // dQ partial in TMEM
  const uint32_t dq_empty = bar0 + 56;    // dQ partial drained: the S columns may be overwritten
  const uint32_t acc_full = bar0 + 64;    // dV and dK final
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + S::kBars + 8 * 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rep = d.hq / d.hkv;
  const int kv_head = blockIdx.y;
  const int batch = blockIdx.z;

  // which KV tile: heavy tiles (early positions see the most queries under a causal mask) come first in launch order
  int kv_row0 = 0, kv_pos0 = 0, kv_valid = 0, kv_seg = 0, kv_row_in_seg = 0;
  {
    int t = blockIdx.x;
    bool found = false;
    for (int seg = 0; seg < d.num_kv_segs && !found; ++seg) {
      const int nt = (d.kv_seg_len[seg] + kFbTile - 1) / kFbTile;
      if (t < nt) {
        kv_seg = seg;
        kv_row_in_seg = t * kFbTile;
        kv_row0 = d.kv_seg_row0[seg] + t * kFbTile;
        kv_pos0 = d.kv_seg_pos0[seg] + t * kFbTile;
        kv_valid = min(kFbTile, d.kv_seg_len[seg] - t * kFbTile);
        found = true;
      }
      t -= nt;
    }
    if (!found) return;   // uniform over the CTA: nothing allocated yet
  }
  // Active Q tiles: inside a segment positions grow, so under a causal mask the tiles that can see this KV tile are a
  // suffix of every segment. seg_first / seg_cnt (shared memory, filled below) turn a step index into a tile in O(segments).
  int* seg_first = reinterpret_cast<int*>(smem + S::kBars + 8 * 12);
  int* seg_cnt = seg_first + 16;
  int* n_active_s = seg_cnt + 16;
  const int tiles_per_seg = d.num_q_segs == 1 ? (d.sq + kFbTile - 1) / kFbTile : d.q_seg_rows / kFbTile;
  const int rows_per_seg = d.num_q_segs == 1 ? d.sq : d.q_seg_rows;
  if (threadIdx.x == 0) {
    int total = 0;
    for (int sg = 0; sg < d.num_q_segs; ++sg) {
      int first = 0;
      if (d.causal) {
        while (first < tiles_per_seg && d.q_seg_pos[sg] + min(first * kFbTile + kFbTile, rows_per_seg) - 1 < kv_pos0) ++first;
      }
      seg_first[sg] = first;
      seg_cnt[sg] = tiles_per_seg - first;
      total += tiles_per_seg - first;
    }
    *n_active_s = total;
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    if ((sb & 1023u) != 0) {
      *abort_flag = 1;
      record_status(p.status, kStatusBadArgument, 650, 0, 0, 1, 0);
    }
    mbar_init(kv_full, 1);
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 8);
    mbar_init(pds_empty, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 4);
    mbar_init(acc_full, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_do);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const int n_active = *n_active_s;
  const int n_steps = n_active * rep;
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_s = tmem_base;          // S, then the dQ partial (128 / D columns)
  const uint32_t tmem_dp = tmem_base + 128;
  const uint32_t tmem_dv = tmem_base + 256;
  const uint32_t tmem_dk = tmem_base + 256 + D;
  const bool bad = *abort_flag != 0;
  const int kv_tok0 = batch * d.skv + kv_row0;

  // step -> (query head, q tile): heads outer, active tiles inner
  auto step_coords = [&](int step, int& head, int& qt) {
    head = kv_head * rep + step / n_active;
    int k = step % n_active;
    qt = 0;
    for (int sg = 0; sg < d.num_q_segs; ++sg) {
      if (k < seg_cnt[sg]) {
        qt = sg * tiles_per_seg + seg_first[sg] + k;
        break;
      }
      k -= seg_cnt[sg];
    }
  };

  if (bad || n_steps == 0) {
    // nothing to accumulate for this tile: its dK / dV rows keep the zeros the caller put there
  } else if (warp == 0) {
    // producer: the whole warp walks the loop, one elected lane's copies take effect. Under `if (lane == 0)` the loop would
    // run in divergent code, where addresses cannot live in uniform registers (see umma_f16_ss_p).
    {
      const uint32_t lead = elect_one() ? 1u : 0u;
      mbar_expect_tx_p(kv_full, 2 * S::kTileBytes, lead);
#pragma unroll
      for (int a = 0; a < kAtoms; ++a) {
        tma_load_3d_p(sb + S::kK + a * kAtomBytes, &tmap_k, kv_full, a * 64, kv_head, kv_tok0, lead);
        tma_load_3d_p(sb + S::kV + a * kAtomBytes, &tmap_v, kv_full, a * 64, kv_head, kv_tok0, lead);
      }
      bool ok = true;
      for (int step = 0; step < n_steps && ok; ++step) {
        int head, qt;
        step_coords(step, head, qt);
        if (!mbar_wait(qdo_empty, (step & 1) ^ 1u, abort_flag, p.budget_ns)) { ok = false; break; }
        const int q_tok0 = batch * d.sq + qt * kFbTile;
        mbar_expect_tx_p(qdo_full, 2 * S::kTileBytes, lead);
#pragma unroll
        for (int a = 0; a < kAtoms; ++a) {
          tma_load_3d_p(sb + S::kQ + a * kAtomBytes, &tmap_q, qdo_full, a * 64, head, q_tok0, lead);
          tma_load_3d_p(sb + S::kDO + a * kAtomBytes, &tmap_do, qdo_full, a * 64, head, q_tok0, lead);
        }
      }
      if (!ok && lane == 0) record_status(p.status, kStatusMbarTimeout, 650, 0, 0, 11, 0);
    }
    __syncwarp();
  } else if (warp == 1) {
    // issuer: warp-uniform loop with prepared descriptor words; one elected lane's tcgen05 instructions take effect
    {
      const uint32_t lead = elect_one() ? 1u : 0u;
      constexpr uint32_t idesc_s = make_idesc(kFbTile, kFbTile, 1, 1, 0, 0);   // S, dP: both operands K-major
      constexpr uint32_t idesc_acc = make_idesc(kFbTile, D, 1, 1, 1, 1);       // dV, dK: A and B MN-major
      constexpr uint32_t idesc_dq = make_idesc(kFbTile, D, 1, 1, 0, 1);        // dQ: A K-major, B MN-major
      // K-major views step 16 along K by 32 bytes inside a 64-column atom (atoms kAtomBytes apart); MN-major views step 16
      // along K by 16 rows of 128 bytes
      const uint32_t q_k = smem_desc_lo_kmajor(sb + S::kQ), k_k = smem_desc_lo_kmajor(sb + S::kK);
      const uint32_t do_k = smem_desc_lo_kmajor(sb + S::kDO), v_k = smem_desc_lo_kmajor(sb + S::kV);
      const uint32_t ds_k = smem_desc_lo_kmajor(sb + S::kDS);
      const uint32_t k_mn = smem_desc_lo_mnmajor(sb + S::kK, kAtomBytes), p_mn = smem_desc_lo_mnmajor(sb + S::kP, kAtomBytes);
      const uint32_t do_mn = smem_desc_lo_mnmajor(sb + S::kDO, kAtomBytes), ds_mn = smem_desc_lo_mnmajor(sb + S::kDS, kAtomBytes);
      const uint32_t q_mn = smem_desc_lo_mnmajor(sb + S::kQ, kAtomBytes);
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.budget_ns);
      for (int step = 0; step < n_steps && ok; ++step) {
        const uint32_t ph = step & 1;
        if constexpr (TRACE) { if (lane == 0) fb_trace(p, 0, 0, step); }
        if (!mbar_wait(qdo_full, ph, abort_flag, p.budget_ns)) { ok = false; break; }
        if constexpr (TRACE) { if (lane == 0) fb_trace(p, 0, 1, step); }
        if (!mbar_wait(dq_empty, ph ^ 1u, abort_flag, p.budget_ns)) { ok = false; break; }
        if constexpr (TRACE) { if (lane == 0) fb_trace(p, 0, 2, step); }
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = ((k >> 2) * kAtomBytes + (k & 3) * 32) >> 4;
          umma_f16_ss_p(tmem_s, smem_desc_join(q_k + off), smem_desc_join(k_k + off), idesc_s, k != 0, lead);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = ((k >> 2) * kAtomBytes + (k & 3) * 32) >> 4;
          umma_f16_ss_p(tmem_dp, smem_desc_join(do_k + off), smem_desc_join(v_k + off), idesc_s, k != 0, lead);
        }
        umma_commit_p(sdp_full, lead);
        if constexpr (TRACE) { if (lane == 0) fb_trace(p, 0, 3, step); }
        if (!mbar_wait(pds_full, ph, abort_flag, p.budget_ns)) { ok = false; break; }
        if constexpr (TRACE) { if (lane == 0) fb_trace(p, 0, 4, step); }
        tc_fence_after_sync();
        // dV += P^T dO ; dK += dS^T Q   (K dimension = the 128 q rows, 16 per instruction = 2048 bytes of a [row][128 B] atom)
        // These are the last readers of the Q and dO tiles, so they go first: the load of the next step's Q and dO (one
        // buffer each - shared memory is full) then runs under the dQ product and its drain instead of after them.
        const uint32_t acc0 = step != 0;
#pragma unroll
        for (int k = 0; k < kFbTile / 16; ++k)
          umma_f16_ss_p(tmem_dv, smem_desc_join(p_mn + k * (2048 >> 4)), smem_desc_join(do_mn + k * (2048 >> 4)), idesc_acc,
                        k != 0 ? 1u : acc0, lead);
#pragma unroll
        for (int k = 0; k < kFbTile / 16; ++k)
          umma_f16_ss_p(tmem_dk, smem_desc_join(ds_mn + k * (2048 >> 4)), smem_desc_join(q_mn + k * (2048 >> 4)), idesc_acc,
                        k != 0 ? 1u : acc0, lead);
        umma_commit_p(qdo_empty, lead);
        if constexpr (TRACE) { if (lane == 0) fb_trace(p, 0, 5, step); }
        // dQ partial = dS K_j  (K dimension = the 128 kv rows), into the columns that held S
#pragma unroll
        for (int k = 0; k < kFbTile / 16; ++k) {
          const uint32_t aoff = ((k >> 2) * kAtomBytes + (k & 3) * 32) >> 4;
          umma_f16_ss_p(tmem_s, smem_desc_join(ds_k + aoff), smem_desc_join(k_mn + k * (2048 >> 4)), idesc_dq, k != 0, lead);
        }
        umma_commit_p(dq_full, lead);
        umma_commit_p(pds_empty, lead);
        if constexpr (TRACE) { if (lane == 0) fb_trace(p, 0, 6, step); }
      }
      if (ok) umma_commit_p(acc_full, lead);
      else if (lane == 0) record_status(p.status, kStatusMbarTimeout, 650, 0, 0, 20, 0);
    }
    __syncwarp();
  } else if (warp < 4) {
    // idle
  } else if (warp < 12) {
    // ------------------------------ P and dS (thread = q row, half of the KV columns) ------------------------------
    const int q4 = warp & 3;
    const int c_begin = (warp >= 8) ? 2 : 0;      // 32-column chunks handled by this warpgroup
    const int row = q4 * 32 + lane;
    const float scale2 = d.scale * kFbLog2e;
    bool ok = true;
    for (int step = 0; step < n_steps && ok; ++step) {
      int head, qt;
      step_coords(step, head, qt);
      const uint32_t ph = step & 1;
      const int q_row = qt * kFbTile + row;
      const bool row_ok = q_row < d.sq;
      const int my_pos = row_ok ? fb_q_pos(d, q_row) : -1;
      const long long sidx = ((long long)batch * d.hq + head) * d.sq + q_row;
      const float lse2 = row_ok ? p.lse2[sidx] : 0.f;
      const float delta = row_ok ? p.delta[sidx] : 0.f;
      const bool row_dead = !row_ok || lse2 == -INFINITY;
      const bool need_mask = row_dead || kv_valid < kFbTile || (d.causal && kv_pos0 + kFbTile - 1 > my_pos);
      if constexpr (TRACE) { if (warp == 4 && lane == 0) fb_trace(p, 1, 0, step); }
      ok = mbar_wait(sdp_full, ph, abort_flag, p.budget_ns);
      if constexpr (TRACE) { if (warp == 4 && lane == 0) fb_trace(p, 1, 1, step); }
      if (ok && step > 0) ok = mbar_wait(pds_empty, ph ^ 1u, abort_flag, p.budget_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if constexpr (TRACE) { if (warp == 4 && lane == 0) fb_trace(p, 1, 2, step); }
      tc_fence_after_sync();
      const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
      const uint32_t prow = sb + S::kP + static_cast<uint32_t>(row) * 128u;
      const uint32_t dsrow = sb + S::kDS + static_cast<uint32_t>(row) * 128u;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = c_begin + cc;
        uint32_t rs[32], rd[32];
        tmem_ld_32x32(tmem_s + lane_off + c * 32, rs);
        tmem_ld_32x32(tmem_dp + lane_off + c * 32, rd);
        tmem_ld_wait();
        float pv[32], dsv[32];
        if (!need_mask) {                 // the whole row of this tile is visible: no per-element tests, packed fp32 pairs
          const float neg_lse2 = -lse2, neg_ds = -delta * d.scale;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float x0, x1, t0, t1;
            fma2_bcast(x0, x1, __uint_as_float(rs[i]), __uint_as_float(rs[i + 1]), scale2, neg_lse2);
            fma2_bcast(t0, t1, __uint_as_float(rd[i]), __uint_as_float(rd[i + 1]), d.scale, neg_ds);   // (dP - delta) * scale
            pv[i] = fast_exp2(x0);
            pv[i + 1] = fast_exp2(x1);
            mul2(dsv[i], dsv[i + 1], pv[i], pv[i + 1], t0, t1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = c * 32 + i;
            const bool masked = row_dead || col >= kv_valid || (d.causal && kv_pos0 + col > my_pos);
            const float pe = masked ? 0.f : fast_exp2(fmaf(__uint_as_float(rs[i]), scale2, -lse2));
            pv[i] = pe;
            dsv[i] = pe * (__uint_as_float(rd[i]) - delta) * d.scale;
          }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = c * 4 + g;
          const uint32_t atom = (chunk >> 3) * kAtomBytes;
          const uint32_t sw = (static_cast<uint32_t>((chunk & 7) ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(prow + atom + sw), "r"(pack_bf16x2(pv[8 * g], pv[8 * g + 1])),
                       "r"(pack_bf16x2(pv[8 * g + 2], pv[8 * g + 3])), "r"(pack_bf16x2(pv[8 * g + 4], pv[8 * g + 5])),
                       "r"(pack_bf16x2(pv[8 * g + 6], pv[8 * g + 7]))
                       : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dsrow + atom + sw), "r"(pack_bf16x2(dsv[8 * g], dsv[8 * g + 1])),
                       "r"(pack_bf16x2(dsv[8 * g + 2], dsv[8 * g + 3])), "r"(pack_bf16x2(dsv[8 * g + 4], dsv[8 * g + 5])),
                       "r"(pack_bf16x2(dsv[8 * g + 6], dsv[8 * g + 7]))
                       : "memory");
        }
      }
      if constexpr (TRACE) { if (warp == 4 && lane == 0) fb_trace(p, 1, 3, step); }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      if constexpr (TRACE) { if (warp == 4 && lane == 0) fb_trace(p, 1, 4, step); }
    }
    if (!ok && lane == 0) record_status(p.status, kStatusMbarTimeout, 650, 0, 0, 30, 0);
  } else {
    // ------------------------------ dQ drain, then dV / dK (thread = row) ------------------------------
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    constexpr int DH = D;
    const int col0 = 0;
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    bool ok = !bad;
    for (int step = 0; step < n_steps && ok; ++step) {
      int head, qt;
      step_coords(step, head, qt);
      if constexpr (TRACE) { if (warp == 12 && lane == 0) fb_trace(p, 2, 0, step); }
      ok = mbar_wait(dq_full, step & 1, abort_flag, p.budget_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if constexpr (TRACE) { if (warp == 12 && lane == 0) fb_trace(p, 2, 1, step); }
      tc_fence_after_sync();
      const int q_row = qt * kFbTile + row;
      float* dst = p.dq + ((static_cast<long long>(batch) * d.sq + q_row) * d.hq + head) * D + col0;
      // The partial goes to the fp32 dQ in global memory as two bulk reductions per row (one per half of the head dimension,
      // staged in shared memory) instead of 32 vector reductions per thread, which took 4100 of a step's 11000 cycles and sat
      // between two steps' products. Tensor memory is released as soon as both halves have been read: the second half waits
      // in registers while the TMA unit reads the first out of the staging buffer.
      const uint32_t stage_row = sb + S::kDqStage + static_cast<uint32_t>(row) * S::kDqPitch;
      constexpr int HC = DH / 2;             // columns per half
      auto stage_half = [&](const uint32_t (&r)[HC]) {
#pragma unroll
        for (int i = 0; i < HC; i += 4)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage_row + i * 4), "r"(r[i]), "r"(r[i + 1]), "r"(r[i + 2]), "r"(r[i + 3])
                       : "memory");
        fence_proxy_async_smem();            // this thread's row is visible to the TMA unit
        return 0;
      };
      uint32_t r0[HC], r1[HC];
#pragma unroll
      for (int c = 0; c < HC / 32; ++c) tmem_ld_32x32(tmem_s + lane_off + c * 32, *reinterpret_cast<uint32_t (*)[32]>(&r0[c * 32]));
      tmem_ld_wait();
      tma_store_wait_read<0>();              // the previous step's second half has left the staging buffer
      stage_half(r0);
#pragma unroll
      for (int c = 0; c < HC / 32; ++c) tmem_ld_32x32(tmem_s + lane_off + HC + c * 32, *reinterpret_cast<uint32_t (*)[32]>(&r1[c * 32]));
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_empty);
      if (q_row < d.sq) bulk_reduce_add_f32(dst, stage_row, HC * 4);
      tma_store_commit();
      tma_store_wait_read<0>();
      stage_half(r1);
      if (q_row < d.sq) bulk_reduce_add_f32(dst + HC, stage_row, HC * 4);
      tma_store_commit();
      if constexpr (TRACE) { if (warp == 12 && lane == 0) fb_trace(p, 2, 2, step); }
    }
    tma_store_wait_all<0>();               // every bulk reduction of this thread has been performed
    if (ok && n_steps > 0) {
      ok = mbar_wait(acc_full, 0, abort_flag, p.budget_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) tc_fence_after_sync();
    }
    if (ok) {
      // rows of dV / dK are the KV rows of this tile
      const bool row_ok = row < kv_valid && !(p.seg_scatter && n_steps == 0);   // nothing to add for a tile no query saw
      float* dvp = p.dv + ((static_cast<long long>(kv_tok0) + row) * d.hkv + kv_head) * D + col0;
      float* dkp = p.dk + ((static_cast<long long>(kv_tok0) + row) * d.hkv + kv_head) * D + col0;
      if (p.seg_scatter) {
        const long long off = (static_cast<long long>(kv_row_in_seg + row) * d.hkv + kv_head) * D + col0;
        dvp = p.dv_seg[kv_seg] + off;
        dkp = p.dk_seg[kv_seg] + off;
      }
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t rv[32], rk[32];
        if (n_steps > 0) {
          tmem_ld_32x32(tmem_dv + lane_off + col0 + c * 32, rv);
          tmem_ld_32x32(tmem_dk + lane_off + col0 + c * 32, rk);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { rv[i] = 0u; rk[i] = 0u; }
        }
        if (row_ok && p.seg_scatter) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            red_add_v4_f32(dvp + c * 32 + i, __uint_as_float(rv[i]), __uint_as_float(rv[i + 1]), __uint_as_float(rv[i + 2]),
                           __uint_as_float(rv[i + 3]));
            red_add_v4_f32(dkp + c * 32 + i, __uint_as_float(rk[i]), __uint_as_float(rk[i + 1]), __uint_as_float(rk[i + 2]),
                           __uint_as_float(rk[i + 3]));
          }
        } else if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            st_global_v4(dvp + c * 32 + i, U4{rv[i], rv[i + 1], rv[i + 2], rv[i + 3]});
            st_global_v4(dkp + c * 32 + i, U4{rk[i], rk[i + 1], rk[i + 2], rk[i + 3]});
          }
        }
      }
      // remote additions must have been performed before this rank tells its peers (the barrier launch that follows) that it is done
      if (p.seg_scatter) __threadfence_system();
    } else if (lane == 0 && !bad) {
      record_status(p.status, kStatusMbarTimeout, 650, 0, 0, 40, 0);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// Trace buffer of the next backward launches (device memory, 3 * kFbTraceSteps * 8 int64, zeroed by the caller); null = off.
static long long* g_fb_trace = nullptr;

template <int D>
static int launch_fa_bwd(const pkb_attn_desc& d, const void* q, const void* k, const void* v, const void* o, const void* dout,
                         const void* lse, void* delta, void* lse2, void* dq, void* dk, void* dv, cudaStream_t stream,
                         const unsigned long long* dk_seg = nullptr, const unsigned long long* dv_seg = nullptr) {
  CUtensorMap tq, tk, tv, tdo;
  int rc = encode_tmap_3d(&tq, kTmapBf16, q, D, d.hq, (uint64_t)d.batch * d.sq, (uint64_t)D * 2, (uint64_t)d.hq * D * 2, 64, 1,
                          kFbTile, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_3d(&tdo, kTmapBf16, dout, D, d.hq, (uint64_t)d.batch * d.sq, (uint64_t)D * 2, (uint64_t)d.hq * D * 2, 64, 1,
                      kFbTile, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_3d(&tk, kTmapBf16, k, D, d.hkv, (uint64_t)d.batch * d.skv, (uint64_t)D * 2, (uint64_t)d.hkv * D * 2, 64, 1,
                      kFbTile, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_3d(&tv, kTmapBf16, v, D, d.hkv, (uint64_t)d.batch * d.skv, (uint64_t)D * 2, (uint64_t)d.hkv * D * 2, 64, 1,
                      kFbTile, kSwizzle128);
  if (rc) return rc;
  const long long rows = (long long)d.batch * d.sq * d.hq;
  long long pblocks = (rows * 32 + 255) / 256;
  if (pblocks > 148 * 16) pblocks = 148 * 16;
  fa_bwd_prep_kernel<<<(int)pblocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dout),
                                                       static_cast<const float*>(lse), static_cast<float*>(delta),
                                                       static_cast<float*>(lse2), d.batch, d.sq, d.hq, D);
  PKB_CHECK_CUDA(cudaGetLastError());
  FaBwdParams p;
  p.d = d;
  p.lse2 = static_cast<const float*>(lse2);
  p.delta = static_cast<const float*>(delta);
  p.dq = static_cast<float*>(dq);
  p.dk = static_cast<float*>(dk);
  p.dv = static_cast<float*>(dv);
  p.seg_scatter = (dk_seg != nullptr && dv_seg != nullptr) ? 1 : 0;
  for (int sg = 0; sg < 16; ++sg) {
    p.dk_seg[sg] = p.seg_scatter && sg < d.num_kv_segs ? reinterpret_cast<float*>(dk_seg[sg]) : nullptr;
    p.dv_seg[sg] = p.seg_scatter && sg < d.num_kv_segs ? reinterpret_cast<float*>(dv_seg[sg]) : nullptr;
  }
  p.status = status_block_device_ptr();
  p.trace = g_fb_trace;
  p.budget_ns = d.budget_ns ? d.budget_ns : kDefaultWaitBudgetNs;
  auto kern = g_fb_trace != nullptr ? fa_bwd_kernel<D, true> : fa_bwd_kernel<D, false>;
  constexpr int smem = FbSmem<D>::kTotal;
  PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  int kv_tiles = 0;
  for (int s = 0; s < d.num_kv_segs; ++s) kv_tiles += (d.kv_seg_len[s] + kFbTile - 1) / kFbTile;
  dim3 grid(kv_tiles, d.hkv, d.batch);
  kern<<<grid, kFbThreads, smem, stream>>>(tq, tk, tv, tdo, p);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

}  // namespace pkb

using namespace pkb;

// dq, dk and dv must be zero-filled by the caller (dq is accumulated into; KV tiles that no query can see are skipped).
extern "C" int pkb_flash_attn_bwd(const pkb_attn_desc* desc, const void* q, const void* k, const void* v, const void* o,
                                  const void* dout, const void* lse, void* delta_scratch, void* lse2_scratch, void* dq,
                                  void* dk, void* dv, void* stream) {
  PKB_CHECK_ARG(desc != nullptr, "null descriptor");
  const pkb_attn_desc& d = *desc;
  PKB_CHECK_ARG(d.head_dim == 64 || d.head_dim == 128, "head_dim must be 64 or 128");
  PKB_CHECK_ARG(d.hq % d.hkv == 0 && d.batch >= 1 && d.sq >= 1 && d.skv >= 1, "bad attention shape");
  PKB_CHECK_ARG(d.num_q_segs >= 1 && d.num_q_segs <= 16 && d.num_kv_segs >= 1 && d.num_kv_segs <= 16, "1..16 segments");
  PKB_CHECK_ARG(d.q_seg_rows % kFbTile == 0 || d.num_q_segs == 1, "q segments must be multiples of 128 rows");
  PKB_CHECK_ARG(d.q_seg_rows >= 1, "q_seg_rows must be positive");
  for (int s = 0; s < d.num_kv_segs; ++s)
    PKB_CHECK_ARG(d.kv_seg_row0[s] >= 0 && d.kv_seg_len[s] >= 0 && d.kv_seg_row0[s] + d.kv_seg_len[s] <= d.skv,
                  "kv segment outside the buffer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (d.head_dim == 128) return launch_fa_bwd<128>(d, q, k, v, o, dout, lse, delta_scratch, lse2_scratch, dq, dk, dv, s);
  return launch_fa_bwd<64>(d, q, k, v, o, dout, lse, delta_scratch, lse2_scratch, dq, dk, dv, s);
}

// Context-parallel backward: like pkb_flash_attn_bwd, but the dK / dV rows of KV segment s are added into the fp32 buffers at
// addresses dk_seg[s] / dv_seg[s] ([kv_seg_len[s], hkv, d] each, row 0 of the segment first), which may be peers' symmetric
// memory. The caller zero-fills every accumulator and makes all ranks meet (a barrier launch) before this call, and makes
// them meet again after it before anyone reads its accumulator. dq as in pkb_flash_attn_bwd.
extern "C" int pkb_flash_attn_bwd_scatter(const pkb_attn_desc* desc, const void* q, const void* k, const void* v, const void* o,
                                          const void* dout, const void* lse, void* delta_scratch, void* lse2_scratch, void* dq,
                                          const unsigned long long* dk_seg, const unsigned long long* dv_seg, void* stream) {
  PKB_CHECK_ARG(desc != nullptr && dk_seg != nullptr && dv_seg != nullptr, "null descriptor or destination table");
  const pkb_attn_desc& d = *desc;
  PKB_CHECK_ARG(d.head_dim == 64 || d.head_dim == 128, "head_dim must be 64 or 128");
  PKB_CHECK_ARG(d.hq % d.hkv == 0 && d.batch == 1 && d.sq >= 1 && d.skv >= 1, "bad attention shape (one sequence)");
  PKB_CHECK_ARG(d.num_q_segs >= 1 && d.num_q_segs <= 16 && d.num_kv_segs >= 1 && d.num_kv_segs <= 16, "1..16 segments");
  PKB_CHECK_ARG(d.q_seg_rows % kFbTile == 0 || d.num_q_segs == 1, "q segments must be multiples of 128 rows");
  PKB_CHECK_ARG(d.q_seg_rows >= 1, "q_seg_rows must be positive");
  for (int s = 0; s < d.num_kv_segs; ++s) {
    PKB_CHECK_ARG(d.kv_seg_row0[s] >= 0 && d.kv_seg_len[s] >= 0 && d.kv_seg_row0[s] + d.kv_seg_len[s] <= d.skv,
                  "kv segment outside the buffer");
    PKB_CHECK_ARG(dk_seg[s] != 0 && dv_seg[s] != 0 && ((dk_seg[s] | dv_seg[s]) & 15) == 0, "segment destinations must be 16-byte aligned");
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (d.head_dim == 128)
    return launch_fa_bwd<128>(d, q, k, v, o, dout, lse, delta_scratch, lse2_scratch, dq, nullptr, nullptr, s, dk_seg, dv_seg);
  return launch_fa_bwd<64>(d, q, k, v, o, dout, lse, delta_scratch, lse2_scratch, dq, nullptr, nullptr, s, dk_seg, dv_seg);
}

extern "C" int pkb_flash_attn_bwd_set_trace(void* dev_words) {
  pkb::g_fb_trace = static_cast<long long*>(dev_words);
  return pkb::kApiOk;
}
