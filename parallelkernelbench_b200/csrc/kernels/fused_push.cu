// Elementwise producers fused with the all-gather that follows them: the result is never written locally and gathered
// afterwards, every 16-byte piece leaves the producing thread straight for the gathered buffer of EVERY rank - one
// `multimem.st` through the switch when the group is the whole job and the heap has a multicast mapping, else one
// peer store per member. One launch: entry barrier (the previous gathered result has been consumed everywhere),
// produce + push, closing barrier (all pieces of all ranks have landed here).
//
//  fp8_quant_allgather   x -> e4m3 payload + one fp32 scale per 128 elements (amax / 448, 1 for an all-zero block), gathered
//                        as [W, n] bytes and [W, n / 128] scales   (reference: reference/19_blocked_fp8_quantize.py:7-47
//                        quantises, then calls all_gather twice)
//  rope_allgather        rotate-half RoPE of q and k, gathered along the sequence: [b, t, h, d] per rank ->
//                        [b, W * t, h, d] on every rank            (reference: reference/17_rope_allgather.py:10-35)
#include <cuda_fp8.h>

#include "pkb/api.h"
#include "pkb/host.h"
#include "pkb/ptx.cuh"
#include "pkb/symm.cuh"
#include "pkb/symm_host.h"

namespace pkb {

constexpr float kInv448 = 1.0f / 448.0f;

__device__ __forceinline__ void multimem_st_f32(void* mc_ptr, float v) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc_ptr), "f"(v) : "memory");
}

// store 16 bytes at byte offset `off` of the buffer at heap offset `buf_off` on every member
__device__ __forceinline__ void push_v4(const SymmCtx& c, int use_mc, uint64_t buf_off, long long off, const U4& v) {
  if (use_mc) {
    multimem_st_v4(symm_mc<uint8_t>(c, buf_off) + off, v);
  } else {
    for (int k = 0; k < c.gsize; ++k) {
      int g = c.grank + k;                       // own copy first, the peers spread over time
      if (g >= c.gsize) g -= c.gsize;
      st_global_v4(symm_ptr<uint8_t>(c, c.members[g], buf_off) + off, v);
    }
  }
}

struct QuantAgArgs {
  SymmCtx ctx;
  const __nv_bfloat16* x;   // [n] local input
  long long n;              // multiple of 128
  uint64_t payload_off;     // heap offset of the gathered payload [gsize, n] bytes
  uint64_t scales_off;      // heap offset of the gathered scales [gsize, n / 128] fp32
  int use_mc;
};

// A thread owns 16 consecutive elements (32 bytes in, 16 bytes out); the 8 lanes of a 128-element block share its maximum.
__global__ void __launch_bounds__(256) fp8_quant_allgather_kernel(const QuantAgArgs a) {
  const SymmCtx& c = a.ctx;
  if (!symm_block_barrier(c, 710, 1)) return;
  const long long nthr = a.n >> 4;
  const long long nb = a.n >> 7;
  for (long long t0 = (long long)blockIdx.x * blockDim.x; t0 < nthr; t0 += (long long)gridDim.x * blockDim.x) {
    const long long t = t0 + threadIdx.x;      // nthr is a multiple of 8, so a group of 8 lanes is active or idle as a whole
    float v[16];
    float amax = 0.f;
    if (t < nthr) {
      const U4 u0 = ld_global_nc_v4(a.x + (t << 4)), u1 = ld_global_nc_v4(a.x + (t << 4) + 8);
      const uint32_t w[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        v[2 * j] = f.x; v[2 * j + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    if (t >= nthr) continue;
    float s = amax * kInv448;   // amax / 448 the way PyTorch evaluates a tensor divided by a Python scalar on the GPU: times the rounded reciprocal
    if (s == 0.f) s = 1.0f;
    const float inv = __frcp_rn(s);
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // correctly rounded x / s (the quotient decides the code at rounding boundaries, as in the PyTorch formulation)
      const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(div_rn_by(v[4 * j], s, inv), div_rn_by(v[4 * j + 1], s, inv)), __NV_SATFINITE, __NV_E4M3);
      const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(div_rn_by(v[4 * j + 2], s, inv), div_rn_by(v[4 * j + 3], s, inv)), __NV_SATFINITE, __NV_E4M3);
      o[j] = (uint32_t)lo | ((uint32_t)hi << 16);
    }
    push_v4(c, a.use_mc, a.payload_off, (long long)c.grank * a.n + (t << 4), U4{o[0], o[1], o[2], o[3]});
    if ((t & 7) == 0) {
      const long long soff = ((long long)c.grank * nb + (t >> 3)) * 4;
      if (a.use_mc) {
        multimem_st_f32(symm_mc<uint8_t>(c, a.scales_off) + soff, s);
      } else {
        for (int k = 0; k < c.gsize; ++k) *reinterpret_cast<float*>(symm_ptr<uint8_t>(c, c.members[k], a.scales_off) + soff) = s;
      }
    }
  }
  symm_block_barrier(c, 710, 2);
}

struct RopeAgArgs {
  SymmCtx ctx;
  const __nv_bfloat16* x[2];    // q and k: [batch, t, heads, dim] local
  const __nv_bfloat16* cs;      // [batch, t, dim]
  const __nv_bfloat16* sn;
  int heads[2];
  int batch, t, dim;
  uint64_t out_off[2];          // heap offsets of the gathered results [batch, gsize * t, heads, dim]
  int use_mc;
};

// A thread owns 8 consecutive elements of the first half of one head row and the 8 partners in the second half.
__global__ void __launch_bounds__(256) rope_allgather_kernel(const RopeAgArgs a) {
  const SymmCtx& c = a.ctx;
  if (!symm_block_barrier(c, 711, 1)) return;
  const int half = a.dim >> 1;
  const int vec_per_row = half >> 3;                       // 16-byte pieces of one half row
  const long long tokens = (long long)a.batch * a.t;
  const long long nvec0 = tokens * a.heads[0] * vec_per_row;
  const long long nvec = nvec0 + tokens * a.heads[1] * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const int which = i >= nvec0 ? 1 : 0;
    long long r = which ? i - nvec0 : i;
    const int heads = a.heads[which];
    const int j = (int)(r % vec_per_row) << 3;
    r /= vec_per_row;
    const int h = (int)(r % heads);
    const long long tok = r / heads;                       // b * t + tt
    const long long bb = tok / a.t, tt = tok - bb * a.t;
    const __nv_bfloat16* xr = a.x[which] + (tok * heads + h) * a.dim;
    const U4 x1 = ld_global_nc_v4(xr + j), x2 = ld_global_nc_v4(xr + j + half);
    const U4 c1 = ld_global_nc_v4(a.cs + tok * a.dim + j), c2 = ld_global_nc_v4(a.cs + tok * a.dim + j + half);
    const U4 s1 = ld_global_nc_v4(a.sn + tok * a.dim + j), s2 = ld_global_nc_v4(a.sn + tok * a.dim + j + half);
    const uint32_t xa[4] = {x1.x, x1.y, x1.z, x1.w}, xb[4] = {x2.x, x2.y, x2.z, x2.w};
    const uint32_t ca[4] = {c1.x, c1.y, c1.z, c1.w}, cb[4] = {c2.x, c2.y, c2.z, c2.w};
    const uint32_t sa[4] = {s1.x, s1.y, s1.z, s1.w}, sb2[4] = {s2.x, s2.y, s2.z, s2.w};
    uint32_t o1[4], o2[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 fa = unpack_bf16x2(xa[q]), fb = unpack_bf16x2(xb[q]);
      const float2 c_a = unpack_bf16x2(ca[q]), c_b = unpack_bf16x2(cb[q]), s_a = unpack_bf16x2(sa[q]), s_b = unpack_bf16x2(sb2[q]);
      o1[q] = pack_bf16x2(fa.x * c_a.x - fb.x * s_a.x, fa.y * c_a.y - fb.y * s_a.y);
      o2[q] = pack_bf16x2(fb.x * c_b.x + fa.x * s_b.x, fb.y * c_b.y + fa.y * s_b.y);
    }
    // row (bb, grank * t + tt) of the gathered [batch, gsize * t, heads, dim] tensor
    const long long drow = (bb * c.gsize + c.grank) * a.t + tt;
    const long long doff = ((drow * heads + h) * a.dim + j) * 2;
    push_v4(c, a.use_mc, a.out_off[which], doff, U4{o1[0], o1[1], o1[2], o1[3]});
    push_v4(c, a.use_mc, a.out_off[which], doff + (long long)half * 2, U4{o2[0], o2[1], o2[2], o2[3]});
  }
  symm_block_barrier(c, 711, 2);
}

static int resident_grid(long long work_items) {
  long long blocks = (work_items + 255) / 256;
  int cap = sm_count();                     // the barriers pair blocks by index: every block must be resident
  if (cap > kSymmMaxBlocks) cap = kSymmMaxBlocks;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : (int)blocks;
}

}  // namespace pkb

using namespace pkb;

extern "C" {

// Gathered e4m3 payload [gsize, n] (bytes, heap offset payload_off) and fp32 scales [gsize, n / 128] (heap offset scales_off)
// of every rank's bf16 x [n], n % 128 == 0; valid on this rank when the kernel has finished.
int pkb_fp8_quant_allgather(const pkb_symm_ctx* h, const void* x, long long n, unsigned long long payload_off,
                            unsigned long long scales_off, int allow_multicast, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(n > 0 && n % 128 == 0, "element count must be a positive multiple of 128");
  PKB_CHECK_ARG((payload_off & 15) == 0 && (scales_off & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0, "16-byte alignment");
  QuantAgArgs a;
  a.ctx = symm_ctx_from_api(h);
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.n = n; a.payload_off = payload_off; a.scales_off = scales_off;
  a.use_mc = (allow_multicast && h->mc_base != 0 && h->gsize == h->world && h->gsize > 1) ? 1 : 0;
  fp8_quant_allgather_kernel<<<resident_grid(n / 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

// Rotate-half RoPE of q [batch, t, heads_q, dim] and k [batch, t, heads_k, dim] (bf16, cos / sin [batch, t, dim]) gathered along
// the sequence into [batch, gsize * t, heads, dim] at heap offsets q_out_off / k_out_off on every rank. dim % 16 == 0.
int pkb_rope_allgather(const pkb_symm_ctx* h, const void* q, const void* k, const void* cos_t, const void* sin_t, int batch, int t,
                       int heads_q, int heads_k, int dim, unsigned long long q_out_off, unsigned long long k_out_off,
                       int allow_multicast, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(batch > 0 && t > 0 && heads_q > 0 && heads_k > 0 && dim > 0 && dim % 16 == 0, "bad shape (dim must be a multiple of 16)");
  PKB_CHECK_ARG((q_out_off & 15) == 0 && (k_out_off & 15) == 0, "heap offsets must be 16-byte aligned");
  PKB_CHECK_ARG(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(cos_t) |
                  reinterpret_cast<uintptr_t>(sin_t)) & 15) == 0, "inputs must be 16-byte aligned");
  RopeAgArgs a;
  a.ctx = symm_ctx_from_api(h);
  a.x[0] = static_cast<const __nv_bfloat16*>(q); a.x[1] = static_cast<const __nv_bfloat16*>(k);
  a.cs = static_cast<const __nv_bfloat16*>(cos_t); a.sn = static_cast<const __nv_bfloat16*>(sin_t);
  a.heads[0] = heads_q; a.heads[1] = heads_k;
  a.batch = batch; a.t = t; a.dim = dim;
  a.out_off[0] = q_out_off; a.out_off[1] = k_out_off;
  a.use_mc = (allow_multicast && h->mc_base != 0 && h->gsize == h->world && h->gsize > 1) ? 1 : 0;
  const long long nvec = (long long)batch * t * (heads_q + heads_k) * (dim / 16);
  rope_allgather_kernel<<<resident_grid(nvec), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}

}  // extern "C"
