// Flash-attention forward on tcgen05 / TMEM (never materialises the score matrix).
//
// One CTA owns one 128-row Q tile of one head and walks the KV tiles it is allowed to see:
//   warp 0      TMA producer: Q once, then K and V tiles through two-stage rings
//   warp 1      MMA issuer:   S = Q K^T (128 x 128 x D) into a TMEM S buffer, and O_j = P V
//                             (128 x D x 128) into a TMEM O buffer; S of tile j+1 is issued before
//                             P V of tile j so the tensor core works while the softmax runs
//   warps 4-7   softmax:      thread = row. Two passes over the S row in TMEM (maximum, then
//                             base-2 exponentials and row sum), mask, write P as bf16 into
//                             128-byte-swizzled shared memory (the A operand of the P V MMA),
//                             publish the rescale factor alpha
//   warps 8-15  accumulate:   thread = row, two warpgroups take half of the D columns each.
//                             o = o * alpha + O_j read back from TMEM; at the end divide by the row
//                             sum and store bf16
// K is the K-major B operand of the first MMA; V, stored [kv, d], is the MN-major B operand of the
// second one - both arrive through the same TMA tile shape.
//
// Sequence layout is described by segments, so the same kernel serves plain attention, GQA, causal
// masks and context-parallel layouts: Q rows come in `num_q_segs` runs of `q_seg_rows` rows whose
// global positions start at q_seg_pos[i] (a zigzag rank owns two runs); the KV buffer is a list of
// segments (buffer row, global position, length), and a segment may carry a readiness flag that the
// producer waits for (bounded) - that is how the ring / all-gather of KV blocks from other ranks
// overlaps with the math. The mask compares GLOBAL positions, and tiles that lie entirely in the
// masked future are skipped.
//
// Reference behaviour replaced: materialised fp32 scores + logsumexp merge per ring step
// (reference: reference/54_ring_attention.py:61-100) and SDPA calls (reference/77_magi1_cso_async_attention.py:108).
#include <cstdlib>

#include "pkb/api.h"
#include "pkb/attention_api.h"
#include "pkb/host.h"
#include "pkb/collectives_api.h"
#include "pkb/bulk_copy.cuh"
#include "pkb/symm_host.h"

namespace pkb {

constexpr int kFaThreads = 512;  // four warpgroups: {producer, MMA, 2 idle}, softmax, accumulate x 2
constexpr int kFaTile = 128;  // q rows per CTA and kv rows per step
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct FaParams {
  pkb_attn_desc d;
  __nv_bfloat16* out;  // [batch * sq, hq, D]
  float* lse;          // [batch, hq, sq] natural-log LSE (may be null)
  uint32_t* status;
  uint64_t budget_ns;
  // optional device-side trace: CTA (0,0,0) records (role, event, tile, clock64) as four int64 per
  // record, so the overlap of the roles can be plotted without a profiler
  long long* trace;
  int trace_capacity;  // records
};

__device__ __forceinline__ void fa_trace(const FaParams& p, int role, int event, int tile) {
  if (p.trace == nullptr || blockIdx.x != 0 || blockIdx.y != 0 || blockIdx.z != 0) return;
  const unsigned long long slot = atomicAdd(reinterpret_cast<unsigned long long*>(p.trace), 1ull);
  if (slot < (unsigned long long)p.trace_capacity) {
    long long* r = p.trace + 4 + slot * 4;
    r[0] = role; r[1] = event; r[2] = tile; r[3] = clock64();
  }
}

// Trace of the P-in-TMEM kernel: a plain store into the slot of (role, tile, event) - no atomic, nothing to wait for, so the
// stamps do not stretch the chain they measure. Layout after the four header words: [4 roles][kFaTraceTiles][8 events].
constexpr int kFaTraceTiles = 160;
__device__ __forceinline__ void fa_trace_slot(const FaParams& p, int role, int event, int tile, bool flag = false) {
  if (p.trace == nullptr || blockIdx.x != 0 || blockIdx.y != 0 || blockIdx.z != 0 || tile >= kFaTraceTiles) return;
  if (p.trace_capacity * 4 < 4 * kFaTraceTiles * 8) return;
  long long t;
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(t)::"memory");
  p.trace[4 + (role * kFaTraceTiles + tile) * 8 + event] = t | (flag ? (1ll << 62) : 0ll);   // bit 62: a caller-defined flag
}

template <int D>
struct FaSmem {
  static constexpr int kTileBytes = kFaTile * D * 2;       // Q, K, V tile
  static constexpr int kPBytes = kFaTile * kFaTile * 2;    // P tile
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTileBytes;               // 2 stages
  static constexpr int kV = kK + 2 * kTileBytes;           // 2 stages
  static constexpr int kP = kV + 2 * kTileBytes;           // 2 buffers
  static constexpr int kAlpha = kP + 2 * kPBytes;          // [2][128] fp32
  static constexpr int kStats = kAlpha + 2 * kFaTile * 4;  // l[128], m[128] fp32
  static constexpr int kBars = kStats + 2 * kFaTile * 4;
  static constexpr int kTotal = kBars + 256;
};

// Calls body(j, buffer_row, global_pos, valid_rows, segment) for every KV tile this Q tile touches.
template <typename F>
__device__ __forceinline__ int for_each_kv_tile(const pkb_attn_desc& d, int q_pos_last, F&& body) {
  int j = 0;
  for (int seg = 0; seg < d.num_kv_segs; ++seg) {
    const int len = d.kv_seg_len[seg];
    for (int t0 = 0; t0 < len; t0 += kFaTile) {
      const int kp = d.kv_seg_pos0[seg] + t0;
      if (d.causal && kp > q_pos_last) break;  // positions only grow inside a segment
      body(j, d.kv_seg_row0[seg] + t0, kp, min(kFaTile, len - t0), seg);
      ++j;
    }
  }
  return j;
}

template <int D>
__device__ __forceinline__ void fa_fwd_cta(const CUtensorMap& tmap_q, const CUtensorMap& tmap_k,
                                           const CUtensorMap& tmap_v, const FaParams& p, const int q_tile,
                                           const int head, const int batch) {
  using S = FaSmem<D>;
  constexpr int kAtoms = D / 64;          // 64-column (128-byte) swizzle atoms per tile row
  constexpr int kAtomBytes = kFaTile * 128;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sb = smem_u32(smem);
  const pkb_attn_desc& d = p.d;

  const uint32_t bar0 = sb + S::kBars;
  const uint32_t q_full = bar0;
  auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar0 + 8u * (3 + s); };
  auto v_full = [&](int s) { return bar0 + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bar0 + 8u * (7 + s); };
  auto s_full = [&](int b) { return bar0 + 8u * (9 + b); };
  auto s_empty = [&](int b) { return bar0 + 8u * (11 + b); };
  auto p_full = [&](int b) { return bar0 + 8u * (13 + b); };
  auto p_empty = [&](int b) { return bar0 + 8u * (15 + b); };
  auto o_full = [&](int b) { return bar0 + 8u * (17 + b); };
  auto o_empty = [&](int b) { return bar0 + 8u * (19 + b); };
  auto a_empty = [&](int b) { return bar0 + 8u * (21 + b); };
  const uint32_t stats_full = bar0 + 8u * 23;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + S::kBars + 8 * 24);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* alpha_s = reinterpret_cast<float*>(smem + S::kAlpha);
  float* stats_s = reinterpret_cast<float*>(smem + S::kStats);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kv_head = head / (d.hq / d.hkv);
  const int q_row0 = q_tile * kFaTile;  // row inside this batch's sequence
  const int q_seg = q_row0 / d.q_seg_rows;
  const int q_pos0 = d.q_seg_pos[q_seg] + (q_row0 - q_seg * d.q_seg_rows);
  const int q_pos_last = q_pos0 + kFaTile - 1;
  const int q_tok0 = batch * d.sq + q_row0;       // token coordinate in the Q / O tensors
  const int kv_tok_base = batch * d.skv;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    if ((sb & 1023u) != 0) {
      *abort_flag = 1;
      record_status(p.status, kStatusBadArgument, 600, 0, 0, 1, 0);
    }
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1); mbar_init(k_empty(s), 1);
      mbar_init(v_full(s), 1); mbar_init(v_empty(s), 1);
      mbar_init(s_full(s), 1); mbar_init(s_empty(s), 4);
      mbar_init(p_full(s), 4); mbar_init(p_empty(s), 1);
      mbar_init(o_full(s), 1); mbar_init(o_empty(s), 8);
      mbar_init(a_empty(s), 8);
    }
    mbar_init(stats_full, 4);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_s = tmem_base;        // two S buffers of 128 columns
  const uint32_t tmem_o = tmem_base + 256;  // two O buffers of D columns
  const bool bad = *abort_flag != 0;

  if (bad) {
    // fall through to the common exit
  } else if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_expect_tx(q_full, S::kTileBytes);
#pragma unroll
      for (int a = 0; a < kAtoms; ++a)
        tma_load_3d(sb + S::kQ + a * kAtomBytes, &tmap_q, q_full, a * 64, head, q_tok0);
      bool ok = true;
      int last_seg = -1;
      for_each_kv_tile(d, q_pos_last, [&](int j, int row, int /*kp*/, int /*valid*/, int seg) {
        if (!ok) return;
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (seg != last_seg) {
          last_seg = seg;
          if (d.kv_seg_ready != nullptr && d.kv_seg_flag[seg] >= 0) {
            if (!wait_flag_ge(d.kv_seg_ready + d.kv_seg_flag[seg], d.ready_epoch, p.budget_ns)) {
              *abort_flag = 1;
              record_status(p.status, kStatusPeerTimeout, 600, 0, seg, 10, j);
              ok = false;
              return;
            }
            fence_proxy_async_all();
          }
        }
        if (!mbar_wait(k_empty(st), ph ^ 1u, abort_flag, p.budget_ns)) { ok = false; return; }
        fa_trace(p, 0, 0, j);  // K(j) load issue
        mbar_expect_tx(k_full(st), S::kTileBytes);
#pragma unroll
        for (int a = 0; a < kAtoms; ++a)
          tma_load_3d(sb + S::kK + st * S::kTileBytes + a * kAtomBytes, &tmap_k, k_full(st), a * 64, kv_head,
                      kv_tok_base + row);
        if (!mbar_wait(v_empty(st), ph ^ 1u, abort_flag, p.budget_ns)) { ok = false; return; }
        mbar_expect_tx(v_full(st), S::kTileBytes);
#pragma unroll
        for (int a = 0; a < kAtoms; ++a)
          tma_load_3d(sb + S::kV + st * S::kTileBytes + a * kAtomBytes, &tmap_v, v_full(st), a * 64, kv_head,
                      kv_tok_base + row);
      });
      if (!ok) record_status(p.status, kStatusMbarTimeout, 600, 0, 0, 11, 0);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const int n = for_each_kv_tile(d, q_pos_last, [](int, int, int, int, int) {});
      constexpr uint32_t idesc_s = make_idesc(kFaTile, kFaTile, 1, 1, 0, 0);
      constexpr uint32_t idesc_o = make_idesc(kFaTile, D, 1, 1, 0, 1);  // V is MN-major
      bool ok = mbar_wait(q_full, 0, abort_flag, p.budget_ns);
      auto issue_s = [&](int j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(k_full(st), ph, abort_flag, p.budget_ns)) return false;
        if (!mbar_wait(s_empty(st), ph ^ 1u, abort_flag, p.budget_ns)) return false;
        tc_fence_after_sync();
        fa_trace(p, 1, 0, j);  // S(j) issue
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * kAtomBytes + (k & 3) * 32;
          umma_f16_ss(tmem_s + st * 128, make_smem_desc_sw128_kmajor(sb + S::kQ + off),
                      make_smem_desc_sw128_kmajor(sb + S::kK + st * S::kTileBytes + off), idesc_s, k != 0);
        }
        umma_commit(k_empty(st));
        umma_commit(s_full(st));
        return true;
      };
      if (ok && n > 0) ok = issue_s(0);
      for (int j = 0; j < n && ok; ++j) {
        if (j + 1 < n) ok = issue_s(j + 1);
        if (!ok) break;
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(p_full(st), ph, abort_flag, p.budget_ns) || !mbar_wait(v_full(st), ph, abort_flag, p.budget_ns) ||
            !mbar_wait(o_empty(st), ph ^ 1u, abort_flag, p.budget_ns)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        fa_trace(p, 1, 1, j);  // PV(j) issue
#pragma unroll
        for (int k = 0; k < kFaTile / 16; ++k) {
          const uint32_t poff = (k >> 2) * kAtomBytes + (k & 3) * 32;  // P: K-major, two 64-kv atoms
          const uint64_t dv = make_smem_desc_sw128_mnmajor(sb + S::kV + st * S::kTileBytes + k * 2048, kAtomBytes);
          umma_f16_ss(tmem_o + st * D, make_smem_desc_sw128_kmajor(sb + S::kP + st * S::kPBytes + poff), dv, idesc_o,
                      k != 0);
        }
        umma_commit(v_empty(st));
        umma_commit(p_empty(st));
        umma_commit(o_full(st));
      }
      if (!ok) record_status(p.status, kStatusMbarTimeout, 600, 0, 0, 20, 0);
    }
    __syncwarp();
  } else if (warp < 4) {
    // idle warps of the first warpgroup
  } else if (warp < 8) {
    // ------------------------------ softmax (thread = row) ------------------------------
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const int my_pos = q_pos0 + row;
    const float scale2 = d.scale * kLog2e;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for_each_kv_tile(d, q_pos_last, [&](int j, int /*rowbuf*/, int kp, int valid, int /*seg*/) {
      if (!ok) return;
      const int b = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      ok = mbar_wait(s_full(b), ph, abort_flag, p.budget_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) return;
      tc_fence_after_sync();
      if (row == 0) fa_trace(p, 2, 0, j);  // S(j) visible to the softmax
      // pass 1: row maximum (32 columns at a time; the row stays in TMEM, not in registers)
      const uint32_t s_row = tmem_s + (static_cast<uint32_t>(q4 * 32) << 16) + b * 128;
      const bool need_mask = (d.causal && kp + kFaTile - 1 > my_pos) || valid < kFaTile;
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(s_row + c * 32, r);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = c * 32 + i;
            if (!(col >= valid || (d.causal && kp + col > my_pos))) mx = fmaxf(mx, __uint_as_float(r[i]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
        }
      }
      mx *= scale2;  // scale2 > 0, so the maximum commutes with the scaling
      const float m_new = fmaxf(m_run, mx);
      const bool dead = m_new == -INFINITY;  // nothing visible yet for this row
      const float alpha = dead ? 1.f : fast_exp2(m_run - m_new);
      const float m_use = dead ? 0.f : m_new;
      // P[b] and alpha[b] are free once P V of tile j-2 has read P and the accumulators read alpha
      ok = mbar_wait(p_empty(b), ph ^ 1u, abort_flag, p.budget_ns) && mbar_wait(a_empty(b), ph ^ 1u, abort_flag, p.budget_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) return;
      if (row == 0) fa_trace(p, 2, 1, j);  // pass 1 done, P buffer free
      // pass 2: exponentials, row sum, P as bf16 into the swizzled A-operand tile
      const uint32_t prow = sb + S::kP + b * S::kPBytes + static_cast<uint32_t>(row) * 128u;
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(s_row + c * 32, r);
        tmem_ld_wait();
        float pv[32];
        if (need_mask || dead) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = c * 32 + i;
            const bool masked = dead || col >= valid || (d.causal && kp + col > my_pos);
            pv[i] = masked ? 0.f : fast_exp2(fmaf(__uint_as_float(r[i]), scale2, -m_use));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) pv[i] = fast_exp2(fmaf(__uint_as_float(r[i]), scale2, -m_use));
        }
        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 32; ++i) part[i & 3] += pv[i];
        sum += (part[0] + part[1]) + (part[2] + part[3]);
#pragma unroll
        for (int g = 0; g < 4; ++g) {  // 16-byte chunk = kv columns 32c + 8g .. + 7
          const int chunk = c * 4 + g;
          const uint32_t atom = (chunk >> 3) * kAtomBytes;
          const uint32_t dst = prow + atom + (static_cast<uint32_t>((chunk & 7) ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pack_bf16x2(pv[8 * g], pv[8 * g + 1])),
                       "r"(pack_bf16x2(pv[8 * g + 2], pv[8 * g + 3])), "r"(pack_bf16x2(pv[8 * g + 4], pv[8 * g + 5])),
                       "r"(pack_bf16x2(pv[8 * g + 6], pv[8 * g + 7]))
                       : "memory");
        }
      }
      if (row == 0) fa_trace(p, 2, 3, j);  // pass 2 loop done
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty(b));
      l_run = l_run * alpha + sum;
      m_run = m_new;
      alpha_s[b * kFaTile + row] = alpha;
      if (row == 0) fa_trace(p, 2, 4, j);  // before the proxy fence
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(b));
      if (row == 0) fa_trace(p, 2, 2, j);  // P(j) published
    });
    if (ok) {
      stats_s[row] = l_run;
      stats_s[kFaTile + row] = m_run;
      if (p.lse != nullptr && q_row0 + row < d.sq)
        p.lse[(static_cast<long long>(batch) * d.hq + head) * d.sq + q_row0 + row] =
            (l_run > 0.f) ? (m_run + log2f(l_run)) * kLn2 : -INFINITY;
      __syncwarp();
      if (lane == 0) mbar_arrive(stats_full);
    } else if (lane == 0) {
      record_status(p.status, kStatusMbarTimeout, 600, 0, 0, 30, 0);
    }
  } else {
    // ------------------------------ accumulate (thread = row) ------------------------------
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    constexpr int DH = D / 2;                 // columns per accumulate warpgroup
    const int col0 = (warp >= 12) ? DH : 0;   // warps 8-11: first half, warps 12-15: second half
    float o[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i) o[i] = 0.f;
    const int n = for_each_kv_tile(d, q_pos_last, [](int, int, int, int, int) {});
    bool ok = true;
    for (int j = 0; j < n && ok; ++j) {
      const int b = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      ok = mbar_wait(p_full(b), ph, abort_flag, p.budget_ns) && mbar_wait(o_full(b), ph, abort_flag, p.budget_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      if (row == 0 && col0 == 0) fa_trace(p, 3, 0, j);  // O(j) visible to the accumulators
      const float alpha = alpha_s[b * kFaTile + row];
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_o + (static_cast<uint32_t>(q4 * 32) << 16) + b * D + col0 + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * alpha + __uint_as_float(r[i]);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(o_empty(b));
        mbar_arrive(a_empty(b));
      }
    }
    if (ok) ok = mbar_wait(stats_full, 0, abort_flag, p.budget_ns);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      const float l = stats_s[row];
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      if (q_row0 + row < d.sq) {
        __nv_bfloat16* dst = p.out + (static_cast<long long>(q_tok0 + row) * d.hq + head) * D + col0;
#pragma unroll
        for (int i = 0; i < DH; i += 8) {
          U4 u{pack_bf16x2(o[i] * inv, o[i + 1] * inv), pack_bf16x2(o[i + 2] * inv, o[i + 3] * inv),
               pack_bf16x2(o[i + 4] * inv, o[i + 5] * inv), pack_bf16x2(o[i + 6] * inv, o[i + 7] * inv)};
          st_global_v4(dst + i, u);
        }
      }
    } else if (lane == 0) {
      record_status(p.status, kStatusMbarTimeout, 600, 0, 0, 40, 0);
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

// ================================================================================================
// Two Q tiles per CTA. The softmax, not the tensor core, bounds the one-tile kernel above (ncu: tensor pipe busy
// ~18 % of active cycles), so this form gives the tensor core two independent softmax warpgroups to wait for:
//   warp 0       TMA producer: Q0, Q1 once; K and V tiles one at a time (a K tile is free again as soon as both S
//                products are issued, a V tile as soon as both P V products are - the softmax in between hides the loads)
//   warp 1       MMA issuer: S_t = Q_t K^T into TMEM, O_t += P_t V accumulated IN TMEM over all KV tiles
//   warps 4-7    softmax of tile 0, warps 8-11 softmax of tile 1 (thread = row, two passes over S in TMEM as above)
//   warps 12-15  correction: before P_t V of step j is issued, scale the TMEM accumulator O_t by alpha_t(j) (tcgen05.ld,
//                multiply, tcgen05.st) - skipped for a warp whose 32 rows all kept their maximum
// At the end each softmax warpgroup reads its O from TMEM, divides by the row sums and stores bf16.
// K and V tiles are shared by the two Q tiles, so L2 -> shared-memory traffic per Q row halves as well.
// ================================================================================================
template <int D>
struct Fa2Smem {
  static constexpr int kTileBytes = kFaTile * D * 2;
  static constexpr int kPBytes = kFaTile * kFaTile * 2;
  static constexpr int kQ = 0;                              // two tiles
  static constexpr int kK = kQ + 2 * kTileBytes;
  static constexpr int kV = kK + kTileBytes;
  static constexpr int kP = kV + kTileBytes;                // two tiles
  static constexpr int kAlpha = kP + 2 * kPBytes;           // [2][128] fp32
  static constexpr int kBars = kAlpha + 2 * kFaTile * 4;
  static constexpr int kTotal = kBars + 256;
};

// SPEC (speculative single pass, PKB_FA_SPEC=1): from the second KV tile on, a softmax warp whose rows all have a finite
// offset computes the exponentials with the CURRENT offset in the same pass that finds the tile's row maximum - one read of
// S from TMEM instead of two - and tells the correction warps "no rescale" up front. Only if some row's maximum has grown by
// more than the lazy threshold does the warp repeat the pass with the new offset and rescale its own accumulator rows
// (after the previous P V product has landed). The pass reads S in 16-column pieces through a two-buffer software pipeline,
// so the TMEM read of the next piece overlaps the arithmetic on the current one. The offset moves under exactly the same rule as in the two-pass form, so
// the results are bit-identical to it.
template <int D, bool SPEC = false>
__device__ __forceinline__ void fa_fwd2_cta(const CUtensorMap& tmap_q, const CUtensorMap& tmap_k,
                                            const CUtensorMap& tmap_v, const FaParams& p, const int q_pair,
                                            const int head, const int batch) {
  using S = Fa2Smem<D>;
  constexpr int kAtoms = D / 64;
  constexpr int kAtomBytes = kFaTile * 128;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sb = smem_u32(smem);
  const pkb_attn_desc& d = p.d;

  const uint32_t bar0 = sb + S::kBars;
  const uint32_t q_full = bar0;
  const uint32_t k_full = bar0 + 8, k_empty = bar0 + 16, v_full = bar0 + 24, v_empty = bar0 + 32;
  auto s_full = [&](int t) { return bar0 + 8u * (5 + t); };
  auto p_full = [&](int t) { return bar0 + 8u * (7 + t); };
  auto p_empty = [&](int t) { return bar0 + 8u * (9 + t); };
  auto a_full = [&](int t) { return bar0 + 8u * (11 + t); };
  auto a_empty = [&](int t) { return bar0 + 8u * (13 + t); };
  auto o_scaled = [&](int t) { return bar0 + 8u * (15 + t); };
  auto pv_done = [&](int t) { return bar0 + 8u * (17 + t); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + S::kBars + 8 * 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* alpha_s = reinterpret_cast<float*>(smem + S::kAlpha);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kv_head = head / (d.hq / d.hkv);
  const int n_q_tiles = (d.sq + kFaTile - 1) / kFaTile;
  const int qt0 = q_pair * 2;
  const bool has1 = qt0 + 1 < n_q_tiles;
  const int q_row0 = qt0 * kFaTile;
  const int q_seg = q_row0 / d.q_seg_rows;
  const int q_pos0 = d.q_seg_pos[q_seg] + (q_row0 - q_seg * d.q_seg_rows);   // both tiles lie in one segment
  const int q_pos_last0 = q_pos0 + kFaTile - 1;
  const int q_pos_last = q_pos_last0 + (has1 ? kFaTile : 0);                  // last position of the pair
  const int q_tok0 = batch * d.sq + q_row0;
  const int kv_tok_base = batch * d.skv;
  // tile 1 sees every KV tile of the pair's walk; tile 0 only those that start at or before its last row
  auto need0 = [&](int kp) { return !(d.causal && kp > q_pos_last0); };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    if ((sb & 1023u) != 0) {
      *abort_flag = 1;
      record_status(p.status, kStatusBadArgument, 602, 0, 0, 1, 0);
    }
    mbar_init(q_full, 1);
    mbar_init(k_full, 1); mbar_init(k_empty, 1); mbar_init(v_full, 1); mbar_init(v_empty, 1);
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full(t), 1);
      mbar_init(p_full(t), 4); mbar_init(p_empty(t), 1);
      mbar_init(a_full(t), 4); mbar_init(a_empty(t), 4);
      mbar_init(o_scaled(t), 4); mbar_init(pv_done(t), 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  auto tmem_s = [&](int t) { return tmem_base + t * 128; };
  auto tmem_o = [&](int t) { return tmem_base + 256 + t * D; };
  const bool bad = *abort_flag != 0;

  if (bad) {
    // common exit
  } else if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_expect_tx(q_full, (has1 ? 2 : 1) * S::kTileBytes);
      for (int t = 0; t < (has1 ? 2 : 1); ++t)
#pragma unroll
        for (int a = 0; a < kAtoms; ++a)
          tma_load_3d(sb + S::kQ + t * S::kTileBytes + a * kAtomBytes, &tmap_q, q_full, a * 64, head, q_tok0 + t * kFaTile);
      bool ok = true;
      int last_seg = -1;
      for_each_kv_tile(d, q_pos_last, [&](int j, int row, int /*kp*/, int /*valid*/, int seg) {
        if (!ok) return;
        const uint32_t ph = j & 1;
        if (seg != last_seg) {
          last_seg = seg;
          if (d.kv_seg_ready != nullptr && d.kv_seg_flag[seg] >= 0) {
            if (!wait_flag_ge(d.kv_seg_ready + d.kv_seg_flag[seg], d.ready_epoch, p.budget_ns)) {
              *abort_flag = 1;
              record_status(p.status, kStatusPeerTimeout, 602, 0, seg, 10, j);
              ok = false;
              return;
            }
            fence_proxy_async_all();
          }
        }
        if (!mbar_wait(k_empty, ph ^ 1u, abort_flag, p.budget_ns)) { ok = false; return; }
        mbar_expect_tx(k_full, S::kTileBytes);
#pragma unroll
        for (int a = 0; a < kAtoms; ++a)
          tma_load_3d(sb + S::kK + a * kAtomBytes, &tmap_k, k_full, a * 64, kv_head, kv_tok_base + row);
        if (!mbar_wait(v_empty, ph ^ 1u, abort_flag, p.budget_ns)) { ok = false; return; }
        mbar_expect_tx(v_full, S::kTileBytes);
#pragma unroll
        for (int a = 0; a < kAtoms; ++a)
          tma_load_3d(sb + S::kV + a * kAtomBytes, &tmap_v, v_full, a * 64, kv_head, kv_tok_base + row);
      });
      if (!ok) record_status(p.status, kStatusMbarTimeout, 602, 0, 0, 11, 0);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(kFaTile, kFaTile, 1, 1, 0, 0);
      constexpr uint32_t idesc_o = make_idesc(kFaTile, D, 1, 1, 0, 1);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.budget_ns);
      int pv[2] = {0, 0};         // P V products issued per tile
      auto issue_s = [&](int t) {
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * kAtomBytes + (k & 3) * 32;
          umma_f16_ss(tmem_s(t), make_smem_desc_sw128_kmajor(sb + S::kQ + t * S::kTileBytes + off),
                      make_smem_desc_sw128_kmajor(sb + S::kK + off), idesc_s, k != 0);
        }
        umma_commit(s_full(t));
      };
      // P_t of step pv[t] is in shared memory, so S_t in TMEM has been read for the last time
      auto wait_p = [&](int t) { return mbar_wait(p_full(t), pv[t] & 1, abort_flag, p.budget_ns); };
      auto issue_pv = [&](int t) {
        if (!mbar_wait(o_scaled(t), pv[t] & 1, abort_flag, p.budget_ns)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < kFaTile / 16; ++k) {
          const uint32_t poff = (k >> 2) * kAtomBytes + (k & 3) * 32;
          const uint64_t dv = make_smem_desc_sw128_mnmajor(sb + S::kV + k * 2048, kAtomBytes);
          umma_f16_ss(tmem_o(t), make_smem_desc_sw128_kmajor(sb + S::kP + t * S::kPBytes + poff), dv, idesc_o,
                      (k != 0) || (pv[t] != 0));
        }
        umma_commit(p_empty(t));
        umma_commit(pv_done(t));
        ++pv[t];
        return true;
      };
      // One walk over the KV tiles with a one-tile lookahead: when tile j is visited, the S products of tile j and the
      // P V products of tile j-1 are issued. Per Q tile the next S goes out FIRST (its TMEM columns are free as soon as
      // P is written), so a softmax warpgroup waits for one product, not two, before its next tile; the other Q tile's
      // products fill the tensor core meanwhile.
      int prev_kp = 0;
      const int n = for_each_kv_tile(d, q_pos_last, [&](int j, int /*row*/, int kp, int /*valid*/, int /*seg*/) {
        if (!ok) return;
        if (!mbar_wait(k_full, j & 1, abort_flag, p.budget_ns)) { ok = false; return; }
        if (j == 0) {
          if (need0(kp)) issue_s(0);
          if (has1) issue_s(1);
          umma_commit(k_empty);
          prev_kp = kp;
          return;
        }
        const bool pv0 = need0(prev_kp);
        if (pv0 && !wait_p(0)) { ok = false; return; }
        if (need0(kp)) issue_s(0);
        if (!has1) umma_commit(k_empty);
        if (!mbar_wait(v_full, (j - 1) & 1, abort_flag, p.budget_ns)) { ok = false; return; }
        if (pv0 && !issue_pv(0)) { ok = false; return; }
        if (has1) {
          if (!wait_p(1)) { ok = false; return; }
          issue_s(1);
          umma_commit(k_empty);
          if (!issue_pv(1)) { ok = false; return; }
        }
        umma_commit(v_empty);
        prev_kp = kp;
      });
      if (ok && n > 0) {
        ok = mbar_wait(v_full, (n - 1) & 1, abort_flag, p.budget_ns);
        if (ok && need0(prev_kp)) ok = wait_p(0) && issue_pv(0);
        if (ok && has1) ok = wait_p(1) && issue_pv(1);
      }
      if (!ok) record_status(p.status, kStatusMbarTimeout, 602, 0, 0, 20, 0);
    }
    __syncwarp();
  } else if (warp < 4) {
    // idle
  } else if (warp < 12) {
    // ------------------------------ softmax of tile t (thread = row) ------------------------------
    const int t = (warp >= 8) ? 1 : 0;
    if (t == 0 || has1) {
      const int q4 = warp & 3;
      const int row = q4 * 32 + lane;
      const int my_pos = q_pos0 + t * kFaTile + row;
      const int tile_row0 = q_row0 + t * kFaTile;
      const float scale2 = d.scale * kLog2e;
      float m_run = -INFINITY, l_run = 0.f;
      bool ok = true;
      int cnt = 0;
      const uint32_t s_row = tmem_s(t) + (static_cast<uint32_t>(q4 * 32) << 16);
      for_each_kv_tile(d, q_pos_last, [&](int /*j*/, int /*rowbuf*/, int kp, int valid, int /*seg*/) {
        if (!ok) return;
        if (t == 0 && !need0(kp)) return;
        const uint32_t ph = cnt & 1;
        ok = mbar_wait(s_full(t), ph, abort_flag, p.budget_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return;
        tc_fence_after_sync();
        const bool need_mask = (d.causal && kp + kFaTile - 1 > my_pos) || valid < kFaTile;
        if constexpr (SPEC) {
          if (cnt > 0 && __all_sync(0xffffffffu, m_run != -INFINITY)) {
            // exponentials of S with offset `off`, written to shared memory as bf16 P; returns the row sum and, through
            // `mx_out`, the largest unmasked raw score of the row
            auto exp_pass = [&](const float off, float& mx_out) {
              const uint32_t prow = sb + S::kP + t * S::kPBytes + static_cast<uint32_t>(row) * 128u;
              float sum = 0.f, mxl = -INFINITY;
              float part[4] = {0.f, 0.f, 0.f, 0.f};
              // 16 columns: exponentials, running maximum, partial sums in the same order as the two-pass form (four
              // interleaved partials per 32 columns, folded after the second half), two 16-byte chunks of P
              auto half = [&](const uint32_t (&r)[16], const int c16) {
                float pvv[16];
                if (need_mask) {
#pragma unroll
                  for (int i = 0; i < 16; ++i) {
                    const int col = c16 * 16 + i;
                    const bool masked = col >= valid || (d.causal && kp + col > my_pos);
                    const float sv = __uint_as_float(r[i]);
                    if (!masked) mxl = fmaxf(mxl, sv);
                    pvv[i] = masked ? 0.f : fast_exp2(fmaf(sv, scale2, -off));
                  }
                } else {
#pragma unroll
                  for (int i = 0; i < 16; ++i) {
                    const float sv = __uint_as_float(r[i]);
                    mxl = fmaxf(mxl, sv);
                    pvv[i] = fast_exp2(fmaf(sv, scale2, -off));
                  }
                }
                if ((c16 & 1) == 0) part[0] = part[1] = part[2] = part[3] = 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) part[i & 3] += pvv[i];
                if (c16 & 1) sum += (part[0] + part[1]) + (part[2] + part[3]);
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                  const int chunk = c16 * 2 + g;
                  const uint32_t atom = (chunk >> 3) * kAtomBytes;
                  const uint32_t dst = prow + atom + (static_cast<uint32_t>((chunk & 7) ^ (row & 7)) << 4);
                  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pack_bf16x2(pvv[8 * g], pvv[8 * g + 1])),
                               "r"(pack_bf16x2(pvv[8 * g + 2], pvv[8 * g + 3])), "r"(pack_bf16x2(pvv[8 * g + 4], pvv[8 * g + 5])),
                               "r"(pack_bf16x2(pvv[8 * g + 6], pvv[8 * g + 7]))
                               : "memory");
                }
              };
              // software pipeline over eight 16-column reads with two register buffers: the read of the next piece is in
              // flight while the current one is processed (tcgen05.wait::ld waits for every outstanding read, so the next
              // read is issued right after a wait and before the arithmetic on the piece that wait delivered)
              uint32_t ra[16], rb[16];
              tmem_ld_32x16(s_row, ra);
              tmem_ld_wait();
#pragma unroll
              for (int c = 0; c < 8; c += 2) {
                tmem_ld_32x16(s_row + (c + 1) * 16, rb);
                half(ra, c);
                tmem_ld_wait();
                if (c + 2 < 8) tmem_ld_32x16(s_row + (c + 2) * 16, ra);
                half(rb, c + 1);
                if (c + 2 < 8) tmem_ld_wait();
              }
              mx_out = mxl;
              return sum;
            };
            // the guess "no rescale" goes to the correction warps before the pass
            ok = mbar_wait(a_empty(t), ph ^ 1u, abort_flag, p.budget_ns);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return;
            alpha_s[t * kFaTile + row] = 1.f;
            __syncwarp();
            if (lane == 0) mbar_arrive(a_full(t));
            ok = mbar_wait(p_empty(t), ph ^ 1u, abort_flag, p.budget_ns);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return;
            float mxs;
            float sum = exp_pass(m_run, mxs);
            mxs *= scale2;
            const bool grow = mxs > m_run + 8.f;
            if (!__any_sync(0xffffffffu, grow)) {
              l_run += sum;
            } else {
              // the guess was wrong for some row of this warp: repeat with the new offsets and rescale the accumulator here
              const float m_new = grow ? mxs : m_run;
              const float alpha = grow ? fast_exp2(m_run - m_new) : 1.f;
              float unused;
              sum = exp_pass(m_new, unused);
              l_run = l_run * alpha + sum;
              m_run = m_new;
              ok = mbar_wait(pv_done(t), (cnt - 1) & 1, abort_flag, p.budget_ns);   // cnt > 0 on this path
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) return;
              tc_fence_after_sync();
              const uint32_t o_row = tmem_o(t) + (static_cast<uint32_t>(q4 * 32) << 16);
#pragma unroll
              for (int cc = 0; cc < D / 32; ++cc) {
                uint32_t r[32];
                tmem_ld_32x32(o_row + cc * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                tmem_st_32x32(o_row + cc * 32, r);
              }
              tmem_st_wait();
            }
            tc_fence_before_sync();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(t));
            ++cnt;
            return;
          }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t r[32];
          tmem_ld_32x32(s_row + cc * 32, r);
          tmem_ld_wait();
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int col = cc * 32 + i;
              if (!(col >= valid || (d.causal && kp + col > my_pos))) mx = fmaxf(mx, __uint_as_float(r[i]));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
          }
        }
        mx *= scale2;
        // The offset used for the exponentials follows the row maximum lazily: it moves only when the maximum has grown
        // by more than 8 (a factor 256 in the exponentials, harmless in fp32 sums and bf16 P), so rescaling the
        // accumulator becomes rare; the row sum carries the same offset, which keeps O / l and the log-sum-exp exact.
        const float m_new = (mx > m_run + 8.f) ? mx : m_run;
        const bool dead = m_new == -INFINITY;
        const float alpha = (dead || m_new == m_run) ? 1.f : fast_exp2(m_run - m_new);
        const float m_use = dead ? 0.f : m_new;
        // publish alpha for the correction warps as early as possible
        ok = mbar_wait(a_empty(t), ph ^ 1u, abort_flag, p.budget_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return;
        alpha_s[t * kFaTile + row] = alpha;
        __syncwarp();
        if (lane == 0) mbar_arrive(a_full(t));
        ok = mbar_wait(p_empty(t), ph ^ 1u, abort_flag, p.budget_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return;
        const uint32_t prow = sb + S::kP + t * S::kPBytes + static_cast<uint32_t>(row) * 128u;
        float sum = 0.f;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t r[32];
          tmem_ld_32x32(s_row + cc * 32, r);
          tmem_ld_wait();
          float pvv[32];
          if (need_mask || dead) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int col = cc * 32 + i;
              const bool masked = dead || col >= valid || (d.causal && kp + col > my_pos);
              pvv[i] = masked ? 0.f : fast_exp2(fmaf(__uint_as_float(r[i]), scale2, -m_use));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) pvv[i] = fast_exp2(fmaf(__uint_as_float(r[i]), scale2, -m_use));
          }
          float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int i = 0; i < 32; ++i) part[i & 3] += pvv[i];
          sum += (part[0] + part[1]) + (part[2] + part[3]);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int chunk = cc * 4 + g;
            const uint32_t atom = (chunk >> 3) * kAtomBytes;
            const uint32_t dst = prow + atom + (static_cast<uint32_t>((chunk & 7) ^ (row & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pack_bf16x2(pvv[8 * g], pvv[8 * g + 1])),
                         "r"(pack_bf16x2(pvv[8 * g + 2], pvv[8 * g + 3])), "r"(pack_bf16x2(pvv[8 * g + 4], pvv[8 * g + 5])),
                         "r"(pack_bf16x2(pvv[8 * g + 6], pvv[8 * g + 7]))
                         : "memory");
          }
        }
        l_run = l_run * alpha + sum;
        m_run = m_new;
        tc_fence_before_sync();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full(t));
        ++cnt;
      });
      // epilogue: O_t / l -> bf16
      const bool row_ok = tile_row0 + row < d.sq;
      if (ok && cnt > 0) {
        ok = mbar_wait(pv_done(t), (cnt - 1) & 1, abort_flag, p.budget_ns);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        if (cnt > 0) tc_fence_after_sync();
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
        if (p.lse != nullptr && row_ok)
          p.lse[(static_cast<long long>(batch) * d.hq + head) * d.sq + tile_row0 + row] =
              (l_run > 0.f) ? (m_run + log2f(l_run)) * kLn2 : -INFINITY;
        __nv_bfloat16* dst = p.out + (static_cast<long long>(q_tok0 + t * kFaTile + row) * d.hq + head) * D;
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t r[32];
          if (cnt > 0) {
            tmem_ld_32x32(tmem_o(t) + (static_cast<uint32_t>(q4 * 32) << 16) + cc * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              U4 u{pack_bf16x2(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv),
                   pack_bf16x2(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv),
                   pack_bf16x2(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv),
                   pack_bf16x2(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv)};
              st_global_v4(dst + cc * 32 + i, u);
            }
          }
        }
      } else if (lane == 0) {
        record_status(p.status, kStatusMbarTimeout, 602, 0, 0, 30 + t, 0);
      }
    }
  } else {
    // ------------------------------ correction (thread = row, both tiles) ------------------------------
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    int cnt[2] = {0, 0};
    bool ok = true;
    for_each_kv_tile(d, q_pos_last, [&](int /*j*/, int /*rowbuf*/, int kp, int /*valid*/, int /*seg*/) {
      for (int t = 0; t < 2 && ok; ++t) {
        if (t == 0 ? !need0(kp) : !has1) continue;
        const uint32_t ph = cnt[t] & 1;
        ok = mbar_wait(a_full(t), ph, abort_flag, p.budget_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const float alpha = alpha_s[t * kFaTile + row];
        __syncwarp();
        if (lane == 0) mbar_arrive(a_empty(t));
        if (cnt[t] > 0) {
          // the accumulator may only be touched once the previous P V product has landed in it
          ok = mbar_wait(pv_done(t), (cnt[t] - 1) & 1, abort_flag, p.budget_ns);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (__any_sync(0xffffffffu, alpha != 1.f)) {
            tc_fence_after_sync();
#pragma unroll
            for (int cc = 0; cc < D / 32; ++cc) {
              uint32_t r[32];
              tmem_ld_32x32(tmem_o(t) + lane_off + cc * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st_32x32(tmem_o(t) + lane_off + cc * 32, r);
            }
            tmem_st_wait();
            tc_fence_before_sync();
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(o_scaled(t));
        ++cnt[t];
      }
    });
    if (!ok && lane == 0) record_status(p.status, kStatusMbarTimeout, 602, 0, 0, 40, 0);
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

// ================================================================================================
// Two Q tiles per CTA, P kept in tensor memory.
// The S = Q K^T and O += P V products of a 128 x 128 x 128 step each read 64 KiB of operands from shared memory in the
// 512 cycles they take, which is the whole shared-memory bandwidth of the SM: with P also written to and read from shared
// memory the tensor core cannot be kept busy. Here the softmax thread of a row reads its 128 scores with ONE round of
// tcgen05.ld (the row stays in registers, so S is read once, not twice), and writes the bf16 probabilities back into the
// first 64 columns of the same TMEM buffer with tcgen05.st; the P V product takes its A operand from there
// (tcgen05.mma with A in tensor memory). Shared memory then only feeds K, V and Q, and the 64 KiB that P occupied hold a
// second stage of K and V, so the loads of tile j+1 run under the products of tile j.
//   warp 0       TMA producer: Q0, Q1 once; K and V through two-stage rings
//   warp 1       MMA issuer, per KV tile j:  O_0 += P_0(j-1) V(j-1);  S_0 = Q_0 K(j)^T;  O_1 += P_1(j-1) V(j-1);  S_1 = Q_1 K(j)^T
//                (S_t(j) overwrites P_t(j-1); products of one thread execute in issue order, so no extra wait is needed)
//   warps 4-7    softmax of tile 0, warps 8-11 softmax of tile 1 (thread = row; more registers via setmaxnreg)
//   warps 12-15  correction: scale O_t in TMEM by alpha when a row's offset moved (rare: the offset follows the maximum lazily)
// ================================================================================================
template <int D>
struct Fa3Smem {
  static constexpr int kTileBytes = kFaTile * D * 2;
  static constexpr int kStagesK = 3;                         // K(j+1) is wanted earlier than V(j+1): one stage more
  static constexpr int kStagesV = 2;
  static constexpr int kQ = 0;                               // two tiles
  static constexpr int kK = kQ + 2 * kTileBytes;
  static constexpr int kV = kK + kStagesK * kTileBytes;
  static constexpr int kAlpha = kV + kStagesV * kTileBytes;  // [2 tiles][2 step parities][128] fp32
  static constexpr int kBars = kAlpha + 2 * 2 * kFaTile * 4;
  static constexpr int kTotal = kBars + 512;
};
static_assert(Fa3Smem<128>::kTotal <= 232448, "shared-memory plan exceeds the 227 KiB a CTA may use");

// Softmax arithmetic variant of the P-in-TMEM kernel used by default (see fa_fwd3_cta). Measured at S = 16384 causal, 32 / 8
// heads, d = 128: 0 (scalar) 876 TFLOP/s, 1 (packed pairs, three-input maxima) 916, 2 (polynomial for a quarter of the
// exponentials) 644, 3 (both) 676 - the polynomial costs more issue slots than the special-function unit it relieves.
constexpr int kFa3DefaultOpt = 1;

// register budgets per warpgroup after the prologue (the kernel is compiled for 128 per thread: 512 x 128 = the whole file)
constexpr int kFa3RegsIo = 80, kFa3RegsSoftmax = 168, kFa3RegsCorr = 80;
static_assert(128 * kFa3RegsIo + 256 * kFa3RegsSoftmax + 128 * kFa3RegsCorr <= 65536, "register budgets exceed the register file");

// OPT bit 0: three-input maxima and packed fp32 pairs for scale / subtract and the row sum; bit 1: every fourth pair of
// exponentials of an unmasked tile on the FMA pipe (packed polynomial, poly_exp2_x2) instead of the special-function unit,
// bit 3: every second pair; bit 2: P packed to
// bf16 on the integer pipe (pack_bf16x2_alu) - the conversion instruction shares the special-function pipe with the
// exponentials, and the trace of a softmax step showed that pipe saturated: (128 ex2 + 64 conversions) x 8 cycles = the
// 1540 cycles the exponential loop took.
// TRACE: CTA (0,0,0) records clock64 at the hand-over points of every role (see fa_trace) - a separate instantiation, so the
// production kernel carries none of it.
template <int D, int OPT, bool TRACE = false>
__device__ __forceinline__ void fa_fwd3_cta(const CUtensorMap& tmap_q, const CUtensorMap& tmap_k,
                                            const CUtensorMap& tmap_v, const FaParams& p, const int q_pair,
                                            const int head, const int batch) {
  using S = Fa3Smem<D>;
  constexpr int kAtoms = D / 64;
  constexpr int kAtomBytes = kFaTile * 128;
  constexpr int kStagesK = S::kStagesK, kStagesV = S::kStagesV;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sb = smem_u32(smem);
  const pkb_attn_desc& d = p.d;

  const uint32_t bar0 = sb + S::kBars;
  const uint32_t q_full = bar0;
  // kv_full(j % 3): K of tile j and V of tile j-1 arrive together (the issuing warp needs both for step j and every barrier
  // operation it executes sits on the chain between two products). Three of them, because the producer can be two steps ahead.
  auto kv_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar0 + 8u * (4 + s); };
  auto v_empty = [&](int s) { return bar0 + 8u * (7 + s); };
  auto s_full = [&](int t) { return bar0 + 8u * (9 + t); };
  // p_full(t): P of the step is in tensor memory (four softmax warps) AND the accumulator has been rescaled where a row's
  // offset moved (four correction warps): one wait for the issuing warp before the P V product
  auto p_full = [&](int t) { return bar0 + 8u * (11 + t); };
  auto a_full = [&](int t) { return bar0 + 8u * (13 + t); };
  auto pv_done = [&](int t) { return bar0 + 8u * (15 + t); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + S::kBars + 8 * 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* alpha_s = reinterpret_cast<float*>(smem + S::kAlpha);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kv_head = head / (d.hq / d.hkv);
  const int n_q_tiles = (d.sq + kFaTile - 1) / kFaTile;
  const int qt0 = q_pair * 2;
  const bool has1 = qt0 + 1 < n_q_tiles;
  const int q_row0 = qt0 * kFaTile;
  const int q_seg = q_row0 / d.q_seg_rows;
  const int q_pos0 = d.q_seg_pos[q_seg] + (q_row0 - q_seg * d.q_seg_rows);   // both tiles lie in one segment
  const int q_pos_last0 = q_pos0 + kFaTile - 1;
  const int q_pos_last = q_pos_last0 + (has1 ? kFaTile : 0);
  const int q_tok0 = batch * d.sq + q_row0;
  const int kv_tok_base = batch * d.skv;
  auto need0 = [&](int kp) { return !(d.causal && kp > q_pos_last0); };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    if ((sb & 1023u) != 0) {
      *abort_flag = 1;
      record_status(p.status, kStatusBadArgument, 603, 0, 0, 1, 0);
    }
    mbar_init(q_full, 1);
    for (int s = 0; s < kStagesK; ++s) { mbar_init(kv_full(s), 1); mbar_init(k_empty(s), 1); }
    for (int s = 0; s < kStagesV; ++s) mbar_init(v_empty(s), 1);
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full(t), 1);
      mbar_init(p_full(t), 8);
      mbar_init(a_full(t), 4);
      mbar_init(pv_done(t), 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  auto tmem_s = [&](int t) { return tmem_base + t * 128; };      // S_t: 128 fp32 columns; P_t (bf16 pairs) reuses the first 64
  auto tmem_o = [&](int t) { return tmem_base + 256 + t * D; };
  const bool bad = *abort_flag != 0;

  if (warp < 4) {
    warpgroup_reg_dec<kFa3RegsIo>();
    if (bad) {
      // common exit
    } else if (warp == 0) {
      // ------------------------------ TMA producer ------------------------------
      // warp-uniform loop, one elected lane's copies take effect (see umma_f16_ss_p)
      {
        const uint32_t lead = elect_one() ? 1u : 0u;
        mbar_expect_tx_p(q_full, (has1 ? 2 : 1) * S::kTileBytes, lead);
        for (int t = 0; t < (has1 ? 2 : 1); ++t)
#pragma unroll
          for (int a = 0; a < kAtoms; ++a)
            tma_load_3d_p(sb + S::kQ + t * S::kTileBytes + a * kAtomBytes, &tmap_q, q_full, a * 64, head, q_tok0 + t * kFaTile, lead);
        bool ok = true;
        int last_seg = -1;
        // step j's barrier carries K(j) and V(j-1): the K slot was freed at the end of step j-3, the V slot at the end of
        // step j-2, so both are requested about two steps before the issuing warp asks for them
        auto load_v = [&](int j, int row, uint32_t bar) {
          const int sv = j % kStagesV;
          if (!mbar_wait_backoff(v_empty(sv), ((j / kStagesV) & 1) ^ 1u, abort_flag, p.budget_ns, 256)) { ok = false; return; }
#pragma unroll
          for (int a = 0; a < kAtoms; ++a)
            tma_load_3d_p(sb + S::kV + sv * S::kTileBytes + a * kAtomBytes, &tmap_v, bar, a * 64, kv_head, kv_tok_base + row, lead);
        };
        int prev_row = 0;
        const int n = for_each_kv_tile(d, q_pos_last, [&](int j, int row, int /*kp*/, int /*valid*/, int seg) {
          if (!ok) return;
          const int sk = j % kStagesK;
          if (seg != last_seg) {
            last_seg = seg;
            if (d.kv_seg_ready != nullptr && d.kv_seg_flag[seg] >= 0) {
              if (!wait_flag_ge(d.kv_seg_ready + d.kv_seg_flag[seg], d.ready_epoch, p.budget_ns)) {
                *abort_flag = 1;
                if (lane == 0) record_status(p.status, kStatusPeerTimeout, 603, 0, seg, 10, j);
                ok = false;
                return;
              }
              fence_proxy_async_all();
            }
          }
          if (!mbar_wait_backoff(k_empty(sk), ((j / kStagesK) & 1) ^ 1u, abort_flag, p.budget_ns, 256)) { ok = false; return; }
          mbar_expect_tx_p(kv_full(sk), (j > 0 ? 2 : 1) * S::kTileBytes, lead);
#pragma unroll
          for (int a = 0; a < kAtoms; ++a)
            tma_load_3d_p(sb + S::kK + sk * S::kTileBytes + a * kAtomBytes, &tmap_k, kv_full(sk), a * 64, kv_head, kv_tok_base + row, lead);
          if (j > 0) load_v(j - 1, prev_row, kv_full(sk));
          prev_row = row;
        });
        if (ok && n > 0) {                     // the last V tile alone, on the barrier step n would have used
          if (mbar_wait_backoff(k_empty(n % kStagesK), ((n / kStagesK) & 1) ^ 1u, abort_flag, p.budget_ns, 256)) {
            mbar_expect_tx_p(kv_full(n % kStagesK), S::kTileBytes, lead);
            load_v(n - 1, prev_row, kv_full(n % kStagesK));
          } else {
            ok = false;
          }
        }
        if (!ok && lane == 0) record_status(p.status, kStatusMbarTimeout, 603, 0, 0, 11, 0);
      }
      __syncwarp();
    } else if (warp == 1) {
      // ------------------------------ MMA issuer ------------------------------
      // The whole warp walks the loop and waits on the barriers; one elected lane's tcgen05 instructions take effect
      // (see umma_f16_ss_p): addresses and descriptors then live in uniform registers.
      {
        const uint32_t lead = elect_one() ? 1u : 0u;
        constexpr uint32_t idesc_s = make_idesc(kFaTile, kFaTile, 1, 1, 0, 0);
        constexpr uint32_t idesc_o = make_idesc(kFaTile, D, 1, 1, 0, 1);
        bool ok = mbar_wait(q_full, 0, abort_flag, p.budget_ns);
        int pv[2] = {0, 0};         // P V products issued per tile
        const uint32_t q_lo0 = smem_desc_lo_kmajor(sb + S::kQ);
        const uint32_t k_lo0 = smem_desc_lo_kmajor(sb + S::kK);
        const uint32_t v_lo0 = smem_desc_lo_mnmajor(sb + S::kV, kAtomBytes);
        const uint32_t tmem_s0 = tmem_base, tmem_o0 = tmem_base + 256;
        auto issue_s = [&](int t, int st) {            // st: K stage
          tc_fence_after_sync();
          const uint32_t ql = q_lo0 + t * (S::kTileBytes >> 4), kl = k_lo0 + st * (S::kTileBytes >> 4), ds = tmem_s0 + t * 128;
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t off = ((k >> 2) * kAtomBytes + (k & 3) * 32) >> 4;
            umma_f16_ss_p(ds, smem_desc_join(ql + off), smem_desc_join(kl + off), idesc_s, k != 0, lead);
          }
          umma_commit_p(s_full(t), lead);
        };
        // O_t += P_t V: A = P_t from tensor memory (16 bf16 of K per step = 8 columns), B = V tile, MN-major
        auto issue_pv = [&](int t, int st) {
          const uint32_t ph = pv[t] & 1;
          const uint32_t vl = v_lo0 + st * (S::kTileBytes >> 4), ds = tmem_s0 + t * 128, dout = tmem_o0 + t * D;
          const uint32_t acc0 = pv[t] != 0;
          if (!mbar_wait(p_full(t), ph, abort_flag, p.budget_ns)) return false;
          if constexpr (TRACE) { if (t == 0 && lane == 0) fa_trace_slot(p, 0, 7, pv[0] + 1); }
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < kFaTile / 16; ++k)
            umma_f16_ts_p(dout, ds + k * 8, smem_desc_join(vl + k * (2048 >> 4)), idesc_o, k != 0 ? 1u : acc0, lead);
          umma_commit_p(pv_done(t), lead);
          ++pv[t];
          return true;
        };
        int prev_kp = 0, prev_st = 0;                   // prev_st: V stage of the previous tile
        const int n = for_each_kv_tile(d, q_pos_last, [&](int j, int /*row*/, int kp, int /*valid*/, int /*seg*/) {
          if (!ok) return;
          const int st = j % kStagesK;
          if constexpr (TRACE) { if (lane == 0 && j > 0) fa_trace_slot(p, 0, 6, j - 1); }
          if (!mbar_wait(kv_full(st), (j / kStagesK) & 1, abort_flag, p.budget_ns)) { ok = false; return; }
          if constexpr (TRACE) { if (lane == 0) fa_trace_slot(p, 0, 0, j); }
          if (j == 0) {
            if (need0(kp)) issue_s(0, st);
            if (has1) issue_s(1, st);
            umma_commit_p(k_empty(st), lead);
            prev_kp = kp; prev_st = j % kStagesV;
            return;
          }
          if (need0(prev_kp) && !issue_pv(0, prev_st)) { ok = false; return; }
          if constexpr (TRACE) { if (lane == 0) fa_trace_slot(p, 0, 2, j); }
          if (need0(kp)) issue_s(0, st);
          if constexpr (TRACE) { if (lane == 0) fa_trace_slot(p, 0, 3, j); }
          if (has1) {
            if (!issue_pv(1, prev_st)) { ok = false; return; }
            if constexpr (TRACE) { if (lane == 0) fa_trace_slot(p, 0, 4, j); }
            issue_s(1, st);
            if constexpr (TRACE) { if (lane == 0) fa_trace_slot(p, 0, 5, j); }
          }
          umma_commit_p(v_empty(prev_st), lead);
          umma_commit_p(k_empty(st), lead);
          prev_kp = kp; prev_st = j % kStagesV;
        });
        if (ok && n > 0) {
          ok = mbar_wait(kv_full(n % kStagesK), (n / kStagesK) & 1, abort_flag, p.budget_ns);
          umma_commit_p(k_empty(n % kStagesK), lead);          // no K tile was read in this step; the commit keeps the ring's phases in step
          if (ok && need0(prev_kp)) ok = issue_pv(0, prev_st);
          if (ok && has1) ok = issue_pv(1, prev_st);
        }
        if (!ok && lane == 0) record_status(p.status, kStatusMbarTimeout, 603, 0, 0, 20, 0);
      }
      __syncwarp();
    }
  } else if (warp < 12) {
    warpgroup_reg_inc<kFa3RegsSoftmax>();
    // ------------------------------ softmax of tile t (thread = row) ------------------------------
    const int t = (warp >= 8) ? 1 : 0;
    if (!bad && (t == 0 || has1)) {
      const int q4 = warp & 3;
      const int row = q4 * 32 + lane;
      const int my_pos = q_pos0 + t * kFaTile + row;
      const int tile_row0 = q_row0 + t * kFaTile;
      const float scale2 = d.scale * kLog2e;
      float m_run = -INFINITY, l_run = 0.f;
      bool ok = true;
      int cnt = 0;
      const uint32_t s_row = tmem_s(t) + (static_cast<uint32_t>(q4 * 32) << 16);
      for_each_kv_tile(d, q_pos_last, [&](int /*j*/, int /*rowbuf*/, int kp, int valid, int /*seg*/) {
        if (!ok) return;
        if (t == 0 && !need0(kp)) return;
        const uint32_t ph = cnt & 1;
        ok = mbar_wait(s_full(t), ph, abort_flag, p.budget_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return;
        if constexpr (TRACE) { if (q4 == 0 && lane == 0) fa_trace_slot(p, 1 + t, 0, cnt); }
        tc_fence_after_sync();
        // the whole row of scores in registers, read in four chunks of 32 columns: the read of the next chunk is in flight
        // while the maximum of the current one is taken (masking first where the tile crosses the diagonal or the end)
        uint32_t r[128];
        const bool need_mask = (d.causal && kp + kFaTile - 1 > my_pos) || valid < kFaTile;
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        tmem_ld_32x32(s_row, *reinterpret_cast<uint32_t (*)[32]>(&r[0]));
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tmem_ld_wait();
          if (c < 3) tmem_ld_32x32(s_row + (c + 1) * 32, *reinterpret_cast<uint32_t (*)[32]>(&r[(c + 1) * 32]));
          if (need_mask) {
#pragma unroll
            for (int i = c * 32; i < c * 32 + 32; ++i)
              if (i >= valid || (d.causal && kp + i > my_pos)) r[i] = 0xff800000u;    // -inf: exp2 gives 0
          }
          if constexpr (OPT & 1) {
#pragma unroll
            for (int i = c * 32; i < c * 32 + 32; i += 8) {
              mx4[0] = max3(mx4[0], __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
              mx4[1] = max3(mx4[1], __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
              mx4[2] = max3(mx4[2], __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
              mx4[3] = max3(mx4[3], __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
            }
          } else {
#pragma unroll
            for (int i = c * 32; i < c * 32 + 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[i]));
          }
        }
        if constexpr (TRACE) { if (q4 == 0 && lane == 0) fa_trace_slot(p, 1 + t, 1, cnt); }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale2;
        // the offset follows the row maximum lazily: it moves only when the maximum has grown by more than 8 (a factor
        // 256 in the exponentials, harmless in fp32 sums and bf16 P), which makes rescaling the accumulator rare
        const float m_new = (mx > m_run + 8.f) ? mx : m_run;
        const bool dead = m_new == -INFINITY;
        const float alpha = (dead || m_new == m_run) ? 1.f : fast_exp2(m_run - m_new);
        const float neg_m = dead ? 0.f : -m_new;
        if constexpr (TRACE) { if (q4 == 0 && lane == 0) fa_trace_slot(p, 1 + t, 2, cnt); }
        // one alpha slot per step parity: the slot is rewritten two steps later, and the scores of step j+2 only exist
        // after the P V product of step j, which waited for the correction warp's arrival on p_full (it read the slot first)
        alpha_s[(t * 2 + ph) * kFaTile + row] = alpha;
        __syncwarp();
        if (lane == 0) mbar_arrive(a_full(t));
        if constexpr (TRACE) { if (q4 == 0 && lane == 0) fa_trace_slot(p, 1 + t, 3, cnt); }
        // exponentials, packed to bf16 pairs and written over the first 64 score columns, 64 keys at a time (the packed words
        // of one half are stored while the next half is computed, and fewer registers are live than with the whole row)
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        const bool poly_ok = (OPT & 10) && !need_mask && !dead;      // masked tiles need the exact zero of ex2(-inf)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t w[32];
#pragma unroll
          for (int ii = 0; ii < 32; ++ii) {
            const int i = half * 32 + ii;
            float x0, x1;
            if constexpr (OPT & 1) {
              fma2_bcast(x0, x1, __uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]), scale2, neg_m);
            } else {
              x0 = fmaf(__uint_as_float(r[2 * i]), scale2, neg_m);
              x1 = fmaf(__uint_as_float(r[2 * i + 1]), scale2, neg_m);
            }
            float e0, e1;
            if ((((OPT & 2) && (i & 3) == 3) || ((OPT & 8) && (i & 1) == 1)) && poly_ok) {
              poly_exp2_x2(e0, e1, x0, x1);
            } else {
              e0 = fast_exp2(x0);
              e1 = fast_exp2(x1);
            }
            if constexpr (OPT & 1) {
              if (i & 1) add2_acc(sum4[2], sum4[3], e0, e1);
              else add2_acc(sum4[0], sum4[1], e0, e1);
            } else {
              sum4[(2 * i) & 3] += e0;
              sum4[(2 * i + 1) & 3] += e1;
            }
            w[ii] = (OPT & 4) ? pack_bf16x2_alu(e0, e1) : pack_bf16x2(e0, e1);
          }
          tmem_st_32x32(s_row + half * 32, w);
        }
        if constexpr (TRACE) { if (q4 == 0 && lane == 0) fa_trace_slot(p, 1 + t, 4, cnt); }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full(t));
        if constexpr (TRACE) { if (q4 == 0 && lane == 0) fa_trace_slot(p, 1 + t, 5, cnt); }
        l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        m_run = m_new;
        ++cnt;
      });
      // epilogue: O_t / l -> bf16
      const bool row_ok = tile_row0 + row < d.sq;
      if (ok && cnt > 0) {
        ok = mbar_wait(pv_done(t), (cnt - 1) & 1, abort_flag, p.budget_ns);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        if (cnt > 0) tc_fence_after_sync();
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
        if (p.lse != nullptr && row_ok)
          p.lse[(static_cast<long long>(batch) * d.hq + head) * d.sq + tile_row0 + row] =
              (l_run > 0.f) ? (m_run + log2f(l_run)) * kLn2 : -INFINITY;
        __nv_bfloat16* dst = p.out + (static_cast<long long>(q_tok0 + t * kFaTile + row) * d.hq + head) * D;
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t o[32];
          if (cnt > 0) {
            tmem_ld_32x32(tmem_o(t) + (static_cast<uint32_t>(q4 * 32) << 16) + cc * 32, o);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0u;
          }
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              U4 u{pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv),
                   pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv),
                   pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv),
                   pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv)};
              st_global_v4(dst + cc * 32 + i, u);
            }
          }
        }
      } else if (lane == 0) {
        record_status(p.status, kStatusMbarTimeout, 603, 0, 0, 30 + t, 0);
      }
    }
  } else {
    warpgroup_reg_dec<kFa3RegsCorr>();
    // ------------------------------ correction (thread = row, both tiles) ------------------------------
    if (!bad) {
      const int q4 = warp & 3;
      const int row = q4 * 32 + lane;
      const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
      int cnt[2] = {0, 0};
      bool ok = true;
      for_each_kv_tile(d, q_pos_last, [&](int /*j*/, int /*rowbuf*/, int kp, int /*valid*/, int /*seg*/) {
        for (int t = 0; t < 2 && ok; ++t) {
          if (t == 0 ? !need0(kp) : !has1) continue;
          const uint32_t ph = cnt[t] & 1;
          // the rescale factors arrive long before the step's P: this warp may wake a little late and polls sparingly
          ok = mbar_wait_backoff(a_full(t), ph, abort_flag, p.budget_ns, 128);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if constexpr (TRACE) { if (q4 == 0 && lane == 0) fa_trace_slot(p, 3, 2 * t, cnt[t]); }
          const float alpha = alpha_s[(t * 2 + ph) * kFaTile + row];
          if (cnt[t] > 0) {
            // the accumulator may only be touched once the previous P V product has landed in it
            ok = mbar_wait(pv_done(t), (cnt[t] - 1) & 1, abort_flag, p.budget_ns);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (__any_sync(0xffffffffu, alpha != 1.f)) {
              tc_fence_after_sync();
#pragma unroll
              for (int cc = 0; cc < D / 32; ++cc) {
                uint32_t o[32];
                tmem_ld_32x32(tmem_o(t) + lane_off + cc * 32, o);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                tmem_st_32x32(tmem_o(t) + lane_off + cc * 32, o);
              }
              tmem_st_wait();
              tc_fence_before_sync();
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(p_full(t));
          if constexpr (TRACE) { if (q4 == 0 && lane == 0) fa_trace_slot(p, 3, 2 * t + 1, cnt[t]); }
          ++cnt[t];
        }
      });
      if (!ok && lane == 0) record_status(p.status, kStatusMbarTimeout, 603, 0, 0, 40, 0);
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

template <int D, int OPT, bool TRACE = false>
__global__ void __launch_bounds__(kFaThreads, 1)
fa_fwd3_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  fa_fwd3_cta<D, OPT, TRACE>(tmap_q, tmap_k, tmap_v, p, gridDim.x - 1 - blockIdx.x, blockIdx.y, blockIdx.z);
}

// ================================================================================================
// Two Q tiles per CTA, P in tensor memory, TWO threads per row.
// With one thread per row a softmax step costs its warp at least 128 ex2 x 8 cycles of the special-function pipe plus the
// TMEM read and the maximum, about 1500 cycles, while the other Q tile's two products cover only 1024: the chain
// S product -> softmax -> P V product -> next S product (S and P share TMEM columns) sets the pace, not a pipe. Here a row
// is split between two threads of two warps that sit on the same TMEM lane quadrant (columns 0-63 and 64-127): each reads 64
// scores, the two exchange their maxima through shared memory and an mbarrier (a bounded wait), each computes 64 exponentials
// and stores its 32 packed columns of P. Row sums stay per half until the end. There is no correction warpgroup: the offset
// of the exponentials follows the maximum lazily, so a rescale is rare, and when a row does need one the two threads of the
// row scale their halves of the accumulator themselves once the previous P V product has landed.
//   warp 0        TMA producer (Q0, Q1 once; K, V through two-stage rings)      warp 1   MMA issuer (as above)
//   warps 4-7 / 8-11     softmax of tile 0, column half 0 / 1
//   warps 12-15 / 16-19  softmax of tile 1, column half 0 / 1
// ================================================================================================
constexpr int kFa4Threads = 640;
constexpr int kFa4RegsIo = 56, kFa4RegsSoftmax = 104;   // compiled for 96 per thread (640 x 96 = 61440 registers at launch)
static_assert(128 * kFa4RegsIo + 512 * kFa4RegsSoftmax <= 640 * 96, "register budgets exceed the register file");

template <int D>
struct Fa4Smem {
  static constexpr int kTileBytes = kFaTile * D * 2;
  static constexpr int kStages = 2;
  static constexpr int kQ = 0;                               // two tiles
  static constexpr int kK = kQ + 2 * kTileBytes;
  static constexpr int kV = kK + kStages * kTileBytes;
  static constexpr int kXch = kV + kStages * kTileBytes;     // [parity][tile][half][128] fp32: maxima / row sums of the halves
  static constexpr int kBars = kXch + 2 * 2 * 2 * kFaTile * 4;
  static constexpr int kTotal = kBars + 512;
};

template <int D, bool POLY, bool TRACE = false>
__device__ __forceinline__ void fa_fwd4_cta(const CUtensorMap& tmap_q, const CUtensorMap& tmap_k,
                                            const CUtensorMap& tmap_v, const FaParams& p, const int q_pair,
                                            const int head, const int batch) {
  using S = Fa4Smem<D>;
  constexpr int kAtoms = D / 64;
  constexpr int kAtomBytes = kFaTile * 128;
  constexpr int kStages = S::kStages;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sb = smem_u32(smem);
  const pkb_attn_desc& d = p.d;

  const uint32_t bar0 = sb + S::kBars;
  const uint32_t q_full = bar0;
  auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar0 + 8u * (3 + s); };
  auto v_full = [&](int s) { return bar0 + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bar0 + 8u * (7 + s); };
  auto s_full = [&](int t) { return bar0 + 8u * (9 + t); };
  auto p_full = [&](int t) { return bar0 + 8u * (11 + t); };
  auto pv_done = [&](int t) { return bar0 + 8u * (13 + t); };
  auto x_bar = [&](int t, int q) { return bar0 + 8u * (15 + t * 4 + q); };   // the two warps of (tile, lane quadrant) meet here
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + S::kBars + 8 * 24);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* xch = reinterpret_cast<float*>(smem + S::kXch);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kv_head = head / (d.hq / d.hkv);
  const int n_q_tiles = (d.sq + kFaTile - 1) / kFaTile;
  const int qt0 = q_pair * 2;
  const bool has1 = qt0 + 1 < n_q_tiles;
  const int q_row0 = qt0 * kFaTile;
  const int q_seg = q_row0 / d.q_seg_rows;
  const int q_pos0 = d.q_seg_pos[q_seg] + (q_row0 - q_seg * d.q_seg_rows);   // both tiles lie in one segment
  const int q_pos_last0 = q_pos0 + kFaTile - 1;
  const int q_pos_last = q_pos_last0 + (has1 ? kFaTile : 0);
  const int q_tok0 = batch * d.sq + q_row0;
  const int kv_tok_base = batch * d.skv;
  auto need0 = [&](int kp) { return !(d.causal && kp > q_pos_last0); };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    if ((sb & 1023u) != 0) {
      *abort_flag = 1;
      record_status(p.status, kStatusBadArgument, 604, 0, 0, 1, 0);
    }
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(k_full(s), 1); mbar_init(k_empty(s), 1); mbar_init(v_full(s), 1); mbar_init(v_empty(s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full(t), 1);
      mbar_init(p_full(t), 8);          // lane 0 of the eight softmax warps of the tile
      mbar_init(pv_done(t), 1);
      for (int q = 0; q < 4; ++q) mbar_init(x_bar(t, q), 2);   // lane 0 of the warp of either column half
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  auto tmem_s = [&](int t) { return tmem_base + t * 128; };      // S_t: 128 fp32 columns; P_t (bf16 pairs) reuses the first 64
  auto tmem_o = [&](int t) { return tmem_base + 256 + t * D; };
  const bool bad = *abort_flag != 0;

  if (warp < 4) {
    warpgroup_reg_dec<kFa4RegsIo>();
    if (bad) {
      // common exit
    } else if (warp == 0) {
      // ------------------------------ TMA producer ------------------------------
      if (lane == 0) {
        mbar_expect_tx(q_full, (has1 ? 2 : 1) * S::kTileBytes);
        for (int t = 0; t < (has1 ? 2 : 1); ++t)
#pragma unroll
          for (int a = 0; a < kAtoms; ++a)
            tma_load_3d(sb + S::kQ + t * S::kTileBytes + a * kAtomBytes, &tmap_q, q_full, a * 64, head, q_tok0 + t * kFaTile);
        bool ok = true;
        int last_seg = -1;
        for_each_kv_tile(d, q_pos_last, [&](int j, int row, int /*kp*/, int /*valid*/, int seg) {
          if (!ok) return;
          const int st = j % kStages;
          const uint32_t ph = (j / kStages) & 1;
          if (seg != last_seg) {
            last_seg = seg;
            if (d.kv_seg_ready != nullptr && d.kv_seg_flag[seg] >= 0) {
              if (!wait_flag_ge(d.kv_seg_ready + d.kv_seg_flag[seg], d.ready_epoch, p.budget_ns)) {
                *abort_flag = 1;
                record_status(p.status, kStatusPeerTimeout, 604, 0, seg, 10, j);
                ok = false;
                return;
              }
              fence_proxy_async_all();
            }
          }
          if (!mbar_wait(k_empty(st), ph ^ 1u, abort_flag, p.budget_ns)) { ok = false; return; }
          mbar_expect_tx(k_full(st), S::kTileBytes);
#pragma unroll
          for (int a = 0; a < kAtoms; ++a)
            tma_load_3d(sb + S::kK + st * S::kTileBytes + a * kAtomBytes, &tmap_k, k_full(st), a * 64, kv_head, kv_tok_base + row);
          if (!mbar_wait(v_empty(st), ph ^ 1u, abort_flag, p.budget_ns)) { ok = false; return; }
          mbar_expect_tx(v_full(st), S::kTileBytes);
#pragma unroll
          for (int a = 0; a < kAtoms; ++a)
            tma_load_3d(sb + S::kV + st * S::kTileBytes + a * kAtomBytes, &tmap_v, v_full(st), a * 64, kv_head, kv_tok_base + row);
        });
        if (!ok) record_status(p.status, kStatusMbarTimeout, 604, 0, 0, 11, 0);
      }
      __syncwarp();
    } else if (warp == 1) {
      // ------------------------------ MMA issuer ------------------------------
      if (lane == 0) {
        constexpr uint32_t idesc_s = make_idesc(kFaTile, kFaTile, 1, 1, 0, 0);
        constexpr uint32_t idesc_o = make_idesc(kFaTile, D, 1, 1, 0, 1);
        bool ok = mbar_wait(q_full, 0, abort_flag, p.budget_ns);
        int pv[2] = {0, 0};
        auto issue_s = [&](int t, int st) {
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t off = (k >> 2) * kAtomBytes + (k & 3) * 32;
            umma_f16_ss(tmem_s(t), make_smem_desc_sw128_kmajor(sb + S::kQ + t * S::kTileBytes + off),
                        make_smem_desc_sw128_kmajor(sb + S::kK + st * S::kTileBytes + off), idesc_s, k != 0);
          }
          umma_commit(s_full(t));
        };
        // O_t += P_t V: A = P_t from tensor memory (16 bf16 of K per step = 8 columns), B = V tile, MN-major. P_t is complete -
        // and, if rows had to be rescaled, O_t already scaled - when all eight softmax warps of the tile have arrived.
        auto issue_pv = [&](int t, int st) {
          if (!mbar_wait(p_full(t), pv[t] & 1, abort_flag, p.budget_ns)) return false;
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < kFaTile / 16; ++k) {
            const uint64_t dv = make_smem_desc_sw128_mnmajor(sb + S::kV + st * S::kTileBytes + k * 2048, kAtomBytes);
            umma_f16_ts(tmem_o(t), tmem_s(t) + k * 8, dv, idesc_o, (k != 0) || (pv[t] != 0));
          }
          umma_commit(pv_done(t));
          ++pv[t];
          return true;
        };
        int prev_kp = 0, prev_st = 0;
        const int n = for_each_kv_tile(d, q_pos_last, [&](int j, int /*row*/, int kp, int /*valid*/, int /*seg*/) {
          if (!ok) return;
          const int st = j % kStages;
          if (!mbar_wait(k_full(st), (j / kStages) & 1, abort_flag, p.budget_ns)) { ok = false; return; }
          if constexpr (TRACE) fa_trace_slot(p, 0, 0, j);
          if (j == 0) {
            if (need0(kp)) issue_s(0, st);
            if (has1) issue_s(1, st);
            umma_commit(k_empty(st));
            prev_kp = kp; prev_st = st;
            return;
          }
          if (!mbar_wait(v_full(prev_st), ((j - 1) / kStages) & 1, abort_flag, p.budget_ns)) { ok = false; return; }
          if constexpr (TRACE) fa_trace_slot(p, 0, 1, j);
          if (need0(prev_kp) && !issue_pv(0, prev_st)) { ok = false; return; }
          if constexpr (TRACE) fa_trace_slot(p, 0, 2, j);
          if (need0(kp)) issue_s(0, st);
          if constexpr (TRACE) fa_trace_slot(p, 0, 3, j);
          if (has1) {
            if (!issue_pv(1, prev_st)) { ok = false; return; }
            if constexpr (TRACE) fa_trace_slot(p, 0, 4, j);
            issue_s(1, st);
            if constexpr (TRACE) fa_trace_slot(p, 0, 5, j);
          }
          umma_commit(v_empty(prev_st));
          umma_commit(k_empty(st));
          prev_kp = kp; prev_st = st;
        });
        if (ok && n > 0) {
          ok = mbar_wait(v_full(prev_st), ((n - 1) / kStages) & 1, abort_flag, p.budget_ns);
          if (ok && need0(prev_kp)) ok = issue_pv(0, prev_st);
          if (ok && has1) ok = issue_pv(1, prev_st);
        }
        if (!ok) record_status(p.status, kStatusMbarTimeout, 604, 0, 0, 20, 0);
      }
      __syncwarp();
    }
  } else {
    warpgroup_reg_inc<kFa4RegsSoftmax>();
    // ------------------------------ softmax: tile t, column half `half`, thread = row ------------------------------
    const int wg = (warp >> 2) - 1;            // 0..3
    const int t = wg >> 1;
    const int half = wg & 1;
    if (!bad && (t == 0 || has1)) {
      const int q4 = warp & 3;
      const int row = q4 * 32 + lane;
      const uint32_t xb = x_bar(t, q4);
      uint32_t xph = 0;
      // bounded meeting of the two warps that share this tile's rows (an mbarrier, not bar.sync, so that a failed wait
      // elsewhere can never leave a warp parked at a barrier its partner will not reach)
      auto meet = [&]() {
        __syncwarp();
        if (lane == 0) mbar_arrive(xb);
        bool got = mbar_wait(xb, xph, abort_flag, p.budget_ns);
        got = __all_sync(0xffffffffu, got);
        xph ^= 1u;
        return got;
      };
      const int my_pos = q_pos0 + t * kFaTile + row;
      const int tile_row0 = q_row0 + t * kFaTile;
      const float scale2 = d.scale * kLog2e;
      float m_run = -INFINITY, l_run = 0.f;      // l_run: sum over this thread's 64 columns only
      bool ok = true;
      int cnt = 0;
      const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
      const uint32_t s_cols = tmem_s(t) + lane_off + half * 64;     // this thread's 64 score columns
      const uint32_t p_cols = tmem_s(t) + lane_off + half * 32;     // ... and where its 32 packed P columns go
      const uint32_t o_cols = tmem_o(t) + lane_off + half * (D / 2);
      for_each_kv_tile(d, q_pos_last, [&](int /*j*/, int /*rowbuf*/, int kp, int valid, int /*seg*/) {
        if (!ok) return;
        if (t == 0 && !need0(kp)) return;
        const uint32_t ph = cnt & 1;
        ok = mbar_wait(s_full(t), ph, abort_flag, p.budget_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return;
        if constexpr (TRACE) { if (q4 == 0 && lane == 0 && half == 0) fa_trace_slot(p, 1 + t, 0, cnt); }
        tc_fence_after_sync();
        uint32_t r[64];
        {
          uint32_t (&r0)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[0]);
          uint32_t (&r1)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[32]);
          tmem_ld_32x32(s_cols, r0);
          tmem_ld_32x32(s_cols + 32, r1);
          tmem_ld_wait();
        }
        if constexpr (TRACE) { if (q4 == 0 && lane == 0 && half == 0) fa_trace_slot(p, 1 + t, 1, cnt); }
        const bool need_mask = (d.causal && kp + kFaTile - 1 > my_pos) || valid < kFaTile;
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const int col = half * 64 + i;
            if (col >= valid || (d.causal && kp + col > my_pos)) r[i] = 0xff800000u;    // -inf: exp2 gives 0
          }
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 64; i += 8) {        // three-input maxima: half the issue slots of a chain of two-input ones
          mx4[0] = max3(mx4[0], __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
          mx4[1] = max3(mx4[1], __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
          mx4[2] = max3(mx4[2], __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
          mx4[3] = max3(mx4[3], __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // exchange with the thread that holds the other half of the row (it has finished READING its scores by then, so the
        // P columns that overlap its score columns may be written after this point)
        float* slot = xch + ((ph * 2 + t) * 2) * kFaTile;
        slot[half * kFaTile + row] = mx;
        if constexpr (TRACE) { if (q4 == 0 && lane == 0 && half == 0) fa_trace_slot(p, 1 + t, 2, cnt); }
        ok = meet();
        if (!ok) return;
        if constexpr (TRACE) { if (q4 == 0 && lane == 0 && half == 0) fa_trace_slot(p, 1 + t, 3, cnt); }
        mx = fmaxf(mx, slot[(half ^ 1) * kFaTile + row]) * scale2;
        // the offset follows the row maximum lazily: it moves only when the maximum has grown by more than 8
        const float m_new = (mx > m_run + 8.f) ? mx : m_run;
        const bool dead = m_new == -INFINITY;
        const float alpha = (dead || m_new == m_run) ? 1.f : fast_exp2(m_run - m_new);
        const float neg_m = dead ? 0.f : -m_new;
        if (cnt > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
          // rare: rows of this warp moved their offset - scale this thread's half of the accumulator row once the previous
          // P V product has landed (the next one is not issued before this warp has arrived on p_full)
          ok = mbar_wait(pv_done(t), (cnt - 1) & 1, abort_flag, p.budget_ns);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) return;
          tc_fence_after_sync();
#pragma unroll
          for (int cc = 0; cc < D / 2 / 16; ++cc) {
            uint32_t o[16];
            tmem_ld_32x16(o_cols + cc * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x16(o_cols + cc * 16, o);
          }
          tmem_st_wait();
        }
        // exponentials: scale / subtract and the row sum as packed fp32 pairs; every fourth pair of an unmasked tile takes the
        // polynomial on the FMA pipe instead of the special-function unit (masked tiles need the exact zero of ex2(-inf))
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t w[32];
        const bool poly_ok = POLY && !need_mask && !dead;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x0, x1;
          fma2_bcast(x0, x1, __uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]), scale2, neg_m);
          float e0, e1;
          if (POLY && (i & 3) == 3 && poly_ok) {
            e0 = poly_exp2(x0);
            e1 = poly_exp2(x1);
          } else {
            e0 = fast_exp2(x0);
            e1 = fast_exp2(x1);
          }
          if (i & 1) add2_acc(sum4[2], sum4[3], e0, e1);
          else add2_acc(sum4[0], sum4[1], e0, e1);
          w[i] = pack_bf16x2(e0, e1);
        }
        if constexpr (TRACE) { if (q4 == 0 && lane == 0 && half == 0) fa_trace_slot(p, 1 + t, 4, cnt); }
        tmem_st_32x32(p_cols, w);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full(t));
        if constexpr (TRACE) { if (q4 == 0 && lane == 0 && half == 0) fa_trace_slot(p, 1 + t, 5, cnt); }
        l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        m_run = m_new;
        ++cnt;
      });
      // epilogue: the two halves add their row sums, then each normalises and stores its half of the output row
      float* slot = xch + ((cnt & 1) * 2 + t) * 2 * kFaTile;
      slot[half * kFaTile + row] = l_run;
      if (ok) ok = meet();
      const float l_tot = ok ? l_run + slot[(half ^ 1) * kFaTile + row] : 0.f;
      const bool row_ok = tile_row0 + row < d.sq;
      if (ok && cnt > 0) {
        ok = mbar_wait(pv_done(t), (cnt - 1) & 1, abort_flag, p.budget_ns);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        if (cnt > 0) tc_fence_after_sync();
        const float inv = l_tot > 0.f ? 1.0f / l_tot : 0.f;
        if (p.lse != nullptr && row_ok && half == 0)
          p.lse[(static_cast<long long>(batch) * d.hq + head) * d.sq + tile_row0 + row] =
              (l_tot > 0.f) ? (m_run + log2f(l_tot)) * kLn2 : -INFINITY;
        __nv_bfloat16* dst = p.out + (static_cast<long long>(q_tok0 + t * kFaTile + row) * d.hq + head) * D + half * (D / 2);
#pragma unroll
        for (int cc = 0; cc < D / 2 / 32; ++cc) {
          uint32_t o[32];
          if (cnt > 0) {
            tmem_ld_32x32(o_cols + cc * 32, o);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0u;
          }
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              U4 u{pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv),
                   pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv),
                   pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv),
                   pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv)};
              st_global_v4(dst + cc * 32 + i, u);
            }
          }
        }
      } else if (lane == 0) {
        record_status(p.status, kStatusMbarTimeout, 604, 0, 0, 30 + t, 0);
      }
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

template <int D, bool POLY, bool TRACE = false>
__global__ void __launch_bounds__(kFa4Threads, 1)
fa_fwd4_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  fa_fwd4_cta<D, POLY, TRACE>(tmap_q, tmap_k, tmap_v, p, gridDim.x - 1 - blockIdx.x, blockIdx.y, blockIdx.z);
}

template <int D, bool SPEC = false>
__global__ void __launch_bounds__(kFaThreads, 1)
fa_fwd2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  fa_fwd2_cta<D, SPEC>(tmap_q, tmap_k, tmap_v, p, gridDim.x - 1 - blockIdx.x, blockIdx.y, blockIdx.z);
}

template <int D>
__global__ void __launch_bounds__(kFaThreads, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
              const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  // heavy (late, causal) tiles first
  fa_fwd_cta<D>(tmap_q, tmap_k, tmap_v, p, gridDim.x - 1 - blockIdx.x, blockIdx.y, blockIdx.z);
}

// ---- context-parallel form: the KV exchange runs inside the attention kernel -------------------
// The first `comm_blocks` CTAs push this rank's K and V chunks into every peer's gather buffer
// (16-byte P2P stores) and count each finished piece on the peer's per-segment counter; the other
// CTAs are attention CTAs whose TMA producer waits for the counter of a segment before loading it.
// With NVSwitch every peer is one hop away, so the "ring" is only the order of the pushes.
struct FaCommArgs {
  SymmCtx ctx;
  const uint8_t* k_local;     // [rows_local, hkv, D] bf16, rows_local = segs_per_rank * seg_rows
  const uint8_t* v_local;
  uint64_t k_gather_off;      // heap offsets of the gather buffers [gsize * rows_local, hkv, D]
  uint64_t v_gather_off;
  uint64_t flags_off;         // heap offset of gsize * segs_per_rank uint32 counters
  long long seg_bytes;        // bytes of one segment of K (or V)
  long long piece_bytes;      // a segment is pushed in pieces of this size
  int segs_per_rank;
  int comm_blocks;
  int local_in_place;         // k_local / v_local already are this rank's slots of the gather buffers
  int num_q_tiles, hq;
};

__device__ __forceinline__ void fa_push_role(const FaCommArgs& a) {
  const SymmCtx& c = a.ctx;
  // all ranks have entered this call => nobody still reads the previous call's gathered KV
  // (the epoch slot lives in dynamic shared memory: this kernel has no room for static shared memory)
  extern __shared__ __align__(1024) uint8_t smem_comm[];
  BulkRing ring;
  if (threadIdx.x == 0) {
    *reinterpret_cast<volatile int*>(smem_comm + 8) = 0;        // abort flag of the ring's waits
    bulk_ring_init(ring, smem_u32(smem_comm) + 128);
  }
  if (!symm_block_barrier_at(c, 601, 1, reinterpret_cast<volatile uint32_t*>(smem_comm))) return;
  const int W = c.gsize;
  const int pieces = static_cast<int>((a.seg_bytes + a.piece_bytes - 1) / a.piece_bytes);
  const int per_dest = a.segs_per_rank * 2 * pieces;  // (segment, K|V, piece)
  const int first = a.local_in_place ? per_dest : 0;
  for (int item = first + blockIdx.x; item < W * per_dest; item += a.comm_blocks) {
    const int step = item / per_dest;          // 0 = local copy, then rank+1, rank+2, ...
    int rem = item - step * per_dest;
    const int seg = rem / (2 * pieces);
    rem -= seg * 2 * pieces;
    const int is_v = rem / pieces;
    const int piece = rem - is_v * pieces;
    int dest_g = c.grank + step;
    if (dest_g >= W) dest_g -= W;
    const int dest = c.members[dest_g];
    const long long off = (long long)seg * a.seg_bytes + (long long)piece * a.piece_bytes;
    const long long n = min(a.piece_bytes, a.seg_bytes - (long long)piece * a.piece_bytes);
    const uint8_t* src = (is_v ? a.v_local : a.k_local) + off;
    uint8_t* dst = symm_ptr<uint8_t>(c, dest, is_v ? a.v_gather_off : a.k_gather_off) +
                   (long long)c.grank * a.segs_per_rank * a.seg_bytes + off;
    if (threadIdx.x == 0) {
      // the piece moves as 16 KiB TMA requests through a shared-memory ring (this CTA does no attention work, so the
      // kernel's dynamic shared memory is free for it)
      if (!bulk_copy(ring, dst, src, n, reinterpret_cast<volatile int*>(smem_comm + 8), c.budget_ns)) {
        record_status(c.status, kStatusMbarTimeout, 601, c.rank, dest, 2, item);
        return;
      }
      fence_proxy_async_all();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      fence_acq_rel_sys();
      red_release_sys_add(symm_ptr<uint32_t>(c, dest, a.flags_off) + c.grank * a.segs_per_rank + seg, 1u);
    }
  }
}

template <int D>
__global__ void __launch_bounds__(kFaThreads, 1)
fa_fwd_ring_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const FaParams p, const FaCommArgs a) {
  if ((int)blockIdx.x < a.comm_blocks) {
    fa_push_role(a);
    return;
  }
  const int id = blockIdx.x - a.comm_blocks;
  const int qt = a.num_q_tiles - 1 - id % a.num_q_tiles;
  const int hb = id / a.num_q_tiles;
  fa_fwd_cta<D>(tmap_q, tmap_k, tmap_v, p, qt, hb % a.hq, hb / a.hq);
}

template <int D, bool SPEC = false>
__global__ void __launch_bounds__(kFaThreads, 1)
fa_fwd2_ring_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const FaParams p, const FaCommArgs a) {
  if ((int)blockIdx.x < a.comm_blocks) {
    fa_push_role(a);
    return;
  }
  const int pairs = (a.num_q_tiles + 1) / 2;
  const int id = blockIdx.x - a.comm_blocks;
  const int qp = pairs - 1 - id % pairs;
  const int hb = id / pairs;
  fa_fwd2_cta<D, SPEC>(tmap_q, tmap_k, tmap_v, p, qp, hb % a.hq, hb / a.hq);
}

template <int D>
__global__ void __launch_bounds__(kFaThreads, 1)
fa_fwd3_ring_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const FaParams p, const FaCommArgs a) {
  if ((int)blockIdx.x < a.comm_blocks) {
    fa_push_role(a);
    return;
  }
  const int pairs = (a.num_q_tiles + 1) / 2;
  const int id = blockIdx.x - a.comm_blocks;
  const int qp = pairs - 1 - id % pairs;
  const int hb = id / pairs;
  fa_fwd3_cta<D, kFa3DefaultOpt>(tmap_q, tmap_k, tmap_v, p, qp, hb % a.hq, hb / a.hq);
}

// The two-tile kernel that keeps P in tensor memory is the default (880 against 670 TFLOP/s at S = 16384 causal, 32 / 8 heads,
// d = 128); PKB_FA_V3=0 selects the older form with P in shared memory.
static bool fa_use_v3() {
  static const bool on = [] { const char* e = getenv("PKB_FA_V3"); return !(e != nullptr && e[0] == '0'); }();
  return on;
}

// PKB_FA_V4=1 selects the P-in-TMEM kernel with two threads per row.
static bool fa_use_v4() {
  static const bool on = [] { const char* e = getenv("PKB_FA_V4"); return e != nullptr && e[0] == '1'; }();
  return on;
}

// PKB_FA_SPEC=1 selects the speculative single-pass softmax of the two-tile kernel (off by default).
static bool fa_use_spec() {
  static const bool on = [] { const char* e = getenv("PKB_FA_SPEC"); return e != nullptr && e[0] == '1'; }();
  return on;
}

// The two-tile form needs both tiles of a pair in one position run; PKB_FA_ONE_TILE=1 forces the one-tile kernel.
static bool fa_use_pairs(const pkb_attn_desc& d) {
  static const bool forced_off = [] { const char* e = getenv("PKB_FA_ONE_TILE"); return e != nullptr && e[0] == '1'; }();
  if (forced_off) return false;
  return d.num_q_segs == 1 || d.q_seg_rows % (2 * kFaTile) == 0;
}

template <int D>
static int launch_fa(const pkb_attn_desc* desc, const void* q, const void* k, const void* v, void* out, void* lse,
                     cudaStream_t stream) {
  const pkb_attn_desc& d = *desc;
  CUtensorMap tq, tk, tv;
  // (d, head, token) views: d contiguous, head stride D*2 bytes, token stride heads*D*2 bytes
  int rc = encode_tmap_3d(&tq, kTmapBf16, q, D, d.hq, (uint64_t)d.batch * d.sq, (uint64_t)D * 2, (uint64_t)d.hq * D * 2, 64,
                          1, kFaTile, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_3d(&tk, kTmapBf16, k, D, d.hkv, (uint64_t)d.batch * d.skv, (uint64_t)D * 2, (uint64_t)d.hkv * D * 2, 64, 1,
                      kFaTile, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_3d(&tv, kTmapBf16, v, D, d.hkv, (uint64_t)d.batch * d.skv, (uint64_t)D * 2, (uint64_t)d.hkv * D * 2, 64, 1,
                      kFaTile, kSwizzle128);
  if (rc) return rc;
  FaParams p;
  p.d = d;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.lse = static_cast<float*>(lse);
  p.status = status_block_device_ptr();
  p.budget_ns = d.budget_ns ? d.budget_ns : kDefaultWaitBudgetNs;
  p.trace = reinterpret_cast<long long*>(d.trace);
  p.trace_capacity = d.trace_capacity;
  const int n_tiles = (d.sq + kFaTile - 1) / kFaTile;
  if (fa_use_pairs(d) && p.trace != nullptr && fa_use_v4()) {
    constexpr int smem = Fa4Smem<D>::kTotal;
    dim3 grid((n_tiles + 1) / 2, d.hq, d.batch);
    auto kern = fa_fwd4_kernel<D, false, true>;
    PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<grid, kFa4Threads, smem, stream>>>(tq, tk, tv, p);
  } else if (fa_use_pairs(d) && p.trace == nullptr && fa_use_v4()) {
    constexpr int smem = Fa4Smem<D>::kTotal;
    dim3 grid((n_tiles + 1) / 2, d.hq, d.batch);
    // PKB_FA_POLY=0: all exponentials on the special-function unit
    static const bool poly = [] { const char* e = getenv("PKB_FA_POLY"); return !(e != nullptr && e[0] == '0'); }();
    if (poly) {
      auto kern = fa_fwd4_kernel<D, true>;
      PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      kern<<<grid, kFa4Threads, smem, stream>>>(tq, tk, tv, p);
    } else {
      auto kern = fa_fwd4_kernel<D, false>;
      PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      kern<<<grid, kFa4Threads, smem, stream>>>(tq, tk, tv, p);
    }
  } else if (fa_use_pairs(d) && p.trace != nullptr && fa_use_v3()) {
    constexpr int smem = Fa3Smem<D>::kTotal;
    dim3 grid((n_tiles + 1) / 2, d.hq, d.batch);
    auto kern = fa_fwd3_kernel<D, kFa3DefaultOpt, true>;
    PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<grid, kFaThreads, smem, stream>>>(tq, tk, tv, p);
  } else if (fa_use_pairs(d) && p.trace == nullptr && fa_use_v3()) {
    constexpr int smem = Fa3Smem<D>::kTotal;
    dim3 grid((n_tiles + 1) / 2, d.hq, d.batch);
    // PKB_FA_OPT=0..3 selects the softmax arithmetic variant (bit 0: packed pairs and three-input maxima, bit 1: polynomial)
    static const int opt = [] { const char* e = getenv("PKB_FA_OPT"); return (e != nullptr && e[0] >= '0' && e[0] <= '9') ? atoi(e) : kFa3DefaultOpt; }();
#define PKB_FA3(O)                                                                                   \
    {                                                                                                \
      auto kern = fa_fwd3_kernel<D, O>;                                                              \
      PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
      kern<<<grid, kFaThreads, smem, stream>>>(tq, tk, tv, p);                                       \
    }
    switch (opt) {
      case 1: PKB_FA3(1) break;
      case 2: PKB_FA3(2) break;
      case 3: PKB_FA3(3) break;
      case 5: PKB_FA3(5) break;
      case 7: PKB_FA3(7) break;
      case 9: PKB_FA3(9) break;
      default: PKB_FA3(0) break;
    }
#undef PKB_FA3
  } else if (fa_use_pairs(d) && p.trace == nullptr) {
    constexpr int smem = Fa2Smem<D>::kTotal;
    dim3 grid((n_tiles + 1) / 2, d.hq, d.batch);
    if (fa_use_spec()) {
      auto kern = fa_fwd2_kernel<D, true>;
      PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      kern<<<grid, kFaThreads, smem, stream>>>(tq, tk, tv, p);
    } else {
      auto kern = fa_fwd2_kernel<D, false>;
      PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      kern<<<grid, kFaThreads, smem, stream>>>(tq, tk, tv, p);
    }
  } else {
    auto kern = fa_fwd_kernel<D>;
    constexpr int smem = FaSmem<D>::kTotal;
    PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    dim3 grid(n_tiles, d.hq, d.batch);
    kern<<<grid, kFaThreads, smem, stream>>>(tq, tk, tv, p);
  }
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

}  // namespace pkb

using namespace pkb;

extern "C" int pkb_flash_attn_fwd(const pkb_attn_desc* desc, const void* q, const void* k, const void* v, void* out,
                                  void* lse, void* stream) {
  PKB_CHECK_ARG(desc != nullptr, "null descriptor");
  const pkb_attn_desc& d = *desc;
  PKB_CHECK_ARG(d.head_dim == 64 || d.head_dim == 128, "head_dim must be 64 or 128");
  PKB_CHECK_ARG(d.hq % d.hkv == 0 && d.batch >= 1 && d.sq >= 1 && d.skv >= 1, "bad attention shape");
  PKB_CHECK_ARG(d.num_q_segs >= 1 && d.num_q_segs <= 16 && d.num_kv_segs >= 1 && d.num_kv_segs <= 16, "1..16 segments");
  PKB_CHECK_ARG(d.q_seg_rows % kFaTile == 0 || d.num_q_segs == 1, "q segments must be multiples of 128 rows");
  for (int s = 0; s < d.num_kv_segs; ++s)
    PKB_CHECK_ARG(d.kv_seg_row0[s] >= 0 && d.kv_seg_len[s] >= 0 && d.kv_seg_row0[s] + d.kv_seg_len[s] <= d.skv,
                  "kv segment outside the buffer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (d.head_dim == 128) return launch_fa<128>(desc, q, k, v, out, lse, s);
  return launch_fa<64>(desc, q, k, v, out, lse, s);
}

namespace pkb {

template <int D>
static int launch_fa_ring(const pkb_attn_desc* desc, const pkb_symm_ctx* h, const void* q, const void* k_local,
                          const void* v_local, unsigned long long k_off, unsigned long long v_off,
                          unsigned long long flags_off, int segs_per_rank, int seg_rows, int comm_blocks, void* out,
                          void* lse, cudaStream_t stream) {
  pkb_attn_desc d = *desc;
  const uint64_t local_base = h->base + (uint64_t)h->rank * h->stride;
  const void* kg = reinterpret_cast<const void*>(local_base + k_off);
  const void* vg = reinterpret_cast<const void*>(local_base + v_off);
  CUtensorMap tq, tk, tv;
  int rc = encode_tmap_3d(&tq, kTmapBf16, q, D, d.hq, (uint64_t)d.batch * d.sq, (uint64_t)D * 2, (uint64_t)d.hq * D * 2, 64,
                          1, kFaTile, kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_3d(&tk, kTmapBf16, kg, D, d.hkv, (uint64_t)d.skv, (uint64_t)D * 2, (uint64_t)d.hkv * D * 2, 64, 1, kFaTile,
                      kSwizzle128);
  if (rc) return rc;
  rc = encode_tmap_3d(&tv, kTmapBf16, vg, D, d.hkv, (uint64_t)d.skv, (uint64_t)D * 2, (uint64_t)d.hkv * D * 2, 64, 1, kFaTile,
                      kSwizzle128);
  if (rc) return rc;

  FaCommArgs a;
  a.ctx = symm_ctx_from_api(h);
  a.k_local = static_cast<const uint8_t*>(k_local);
  a.v_local = static_cast<const uint8_t*>(v_local);
  a.k_gather_off = k_off; a.v_gather_off = v_off; a.flags_off = flags_off;
  a.seg_bytes = (long long)seg_rows * d.hkv * D * 2;
  a.piece_bytes = 1ll << 20;
  if (a.piece_bytes > a.seg_bytes) a.piece_bytes = a.seg_bytes;
  a.segs_per_rank = segs_per_rank;
  a.comm_blocks = comm_blocks;
  const long long rank_bytes = a.seg_bytes * segs_per_rank;
  a.local_in_place = (k_local == static_cast<const uint8_t*>(kg) + (long long)h->grank * rank_bytes &&
                      v_local == static_cast<const uint8_t*>(vg) + (long long)h->grank * rank_bytes) ? 1 : 0;
  a.num_q_tiles = (d.sq + kFaTile - 1) / kFaTile;
  a.hq = d.hq;
  const int pieces = (int)((a.seg_bytes + a.piece_bytes - 1) / a.piece_bytes);
  d.kv_seg_ready = reinterpret_cast<const uint32_t*>(local_base + flags_off);
  d.ready_epoch = desc->ready_epoch * (uint32_t)(2 * pieces);
  if (!a.local_in_place) {
    // the local rows are copied by the communication CTAs as well: they get a counter like the rest
  }

  FaParams p;
  p.d = d;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.lse = static_cast<float*>(lse);
  p.status = a.ctx.status;
  p.budget_ns = d.budget_ns ? d.budget_ns : kDefaultWaitBudgetNs;
  p.trace = nullptr;
  p.trace_capacity = 0;
  if (fa_use_pairs(d) && fa_use_v3()) {
    constexpr int smem = Fa3Smem<D>::kTotal;
    const int grid = comm_blocks + ((a.num_q_tiles + 1) / 2) * d.hq * d.batch;
    auto kern = fa_fwd3_ring_kernel<D>;
    PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<grid, kFaThreads, smem, stream>>>(tq, tk, tv, p, a);
  } else if (fa_use_pairs(d)) {
    constexpr int smem = Fa2Smem<D>::kTotal;
    const int grid = comm_blocks + ((a.num_q_tiles + 1) / 2) * d.hq * d.batch;
    if (fa_use_spec()) {
      auto kern = fa_fwd2_ring_kernel<D, true>;
      PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      kern<<<grid, kFaThreads, smem, stream>>>(tq, tk, tv, p, a);
    } else {
      auto kern = fa_fwd2_ring_kernel<D, false>;
      PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      kern<<<grid, kFaThreads, smem, stream>>>(tq, tk, tv, p, a);
    }
  } else {
    auto kern = fa_fwd_ring_kernel<D>;
    constexpr int smem = FaSmem<D>::kTotal;
    PKB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int grid = comm_blocks + a.num_q_tiles * d.hq * d.batch;
    kern<<<grid, kFaThreads, smem, stream>>>(tq, tk, tv, p, a);
  }
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

}  // namespace pkb

extern "C" int pkb_flash_attn_fwd_ring(const pkb_attn_desc* desc, const pkb_symm_ctx* h, const void* q,
                                       const void* k_local, const void* v_local, unsigned long long k_gather_off,
                                       unsigned long long v_gather_off, unsigned long long flags_off,
                                       int segs_per_rank, int seg_rows, int comm_blocks, void* out, void* lse,
                                       void* stream) {
  PKB_CHECK_ARG(desc != nullptr && h != nullptr && h->base != 0, "null descriptor or heap");
  const pkb_attn_desc& d = *desc;
  PKB_CHECK_ARG(d.head_dim == 64 || d.head_dim == 128, "head_dim must be 64 or 128");
  PKB_CHECK_ARG(d.batch == 1, "the context-parallel form takes one sequence");
  PKB_CHECK_ARG(d.hq % d.hkv == 0 && d.sq >= 1, "bad attention shape");
  PKB_CHECK_ARG(segs_per_rank >= 1 && seg_rows >= 1 && h->gsize * segs_per_rank <= 16, "at most 16 KV segments");
  PKB_CHECK_ARG(d.skv == h->gsize * segs_per_rank * seg_rows, "desc.skv must cover the gather buffer");
  PKB_CHECK_ARG(comm_blocks >= 1 && comm_blocks <= kSymmMaxBlocks, "1..240 communication blocks");
  PKB_CHECK_ARG((k_gather_off & 1023) == 0 && (v_gather_off & 1023) == 0 && (flags_off & 15) == 0, "heap offsets misaligned");
  PKB_CHECK_ARG(((long long)seg_rows * d.hkv * d.head_dim * 2) % 16 == 0, "segment size must be a multiple of 16 bytes");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (d.head_dim == 128)
    return pkb::launch_fa_ring<128>(desc, h, q, k_local, v_local, k_gather_off, v_gather_off, flags_off, segs_per_rank,
                                    seg_rows, comm_blocks, out, lse, s);
  return pkb::launch_fa_ring<64>(desc, h, q, k_local, v_local, k_gather_off, v_gather_off, flags_off, segs_per_rank, seg_rows,
                                 comm_blocks, out, lse, s);
}
