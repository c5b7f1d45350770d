// Gaussian-splat projection stage with the redistribution to the camera owners fused in.
//
// Every rank holds N Gaussians and C_local cameras. Each Gaussian is projected into EVERY camera of
// the job (quaternion -> rotation, covariance R S^2 R^T, world -> camera, perspective Jacobian, 2-D
// covariance, conic, radius, near/far and frustum culling) and the survivors are written straight into
// the receive buffer of the rank that owns the camera, in the order (source rank, camera, Gaussian id).
// Three launches, nothing returns to the host in between:
//   gsplat_count   survivors per (camera, block of 256 Gaussians)
//   gsplat_scan    one block: offsets of every (camera, block) inside its destination segment, and this rank's
//                  per-destination totals published in its symmetric heap
//   gsplat_emit    barrier (totals visible) -> base of my segment in every destination = sum of the lower ranks'
//                  totals -> recompute the projection, ordered in-block compaction, 4-byte peer stores of the
//                  records -> barrier (records visible)
// The arithmetic is written with explicitly rounded single operations (no fused multiply-add) in a fixed
// order, so that an fp32 elementwise restatement in PyTorch gives bit-identical radii and culling decisions.
// Reference behaviour replaced: projection as a chain of einsum/elementwise kernels, torch.where packing, two
// count exchanges with host round trips and three list all-to-alls
// (reference: reference/61_gsplat_3d_gaussian_splatting.py:128-450). No graphics API is involved.
#include "pkb/api.h"
#include "pkb/symm_host.h"

namespace pkb {

constexpr int kGsThreads = 256;
constexpr int kGsMaxColor = 8;
constexpr int kGsHeader = 11;   // cam, gid, rx, ry, m2x, m2y, depth, con0, con1, con2, opacity

struct GsArgs {
  const float* means;      // [N,3]
  const float* quats;      // [N,4] (w,x,y,z)
  const float* scales;     // [N,3]
  const float* opac;       // [N]
  const float* colors;     // [N,D]
  const float* viewmats;   // [C,16] row-major
  const float* Ks;         // [C,9]
  int N, C, C_local, D;
  float width, height, eps2d, near_plane, far_plane;
  int gid_offset;          // global id of this rank's Gaussian 0
  int nblk;                // blocks per camera
  int* blk_counts;         // [C, nblk] survivors, then exclusive offsets inside the destination segment
  uint64_t cnt_off;        // heap: int32 [gsize] rows I send to each member
  uint64_t recv_off;       // heap: records [cap, kGsHeader + D] 32-bit words
  long long cap_rows;
  int* recv_count;         // out: rows received by this rank
};

struct GsProj { int rx, ry; float m2x, m2y, depth, c0, c1, c2; bool valid; };

#define M_(a, b) __fmul_rn((a), (b))
#define A_(a, b) __fadd_rn((a), (b))
#define S_(a, b) __fsub_rn((a), (b))
#define D_(a, b) __fdiv_rn((a), (b))

__device__ __forceinline__ float dot3(float a0, float b0, float a1, float b1, float a2, float b2) {
  return A_(A_(M_(a0, b0), M_(a1, b1)), M_(a2, b2));
}

__device__ GsProj gs_project(const GsArgs& a, int n, int c) {
  GsProj r;
  const float mx = a.means[n * 3], my = a.means[n * 3 + 1], mz = a.means[n * 3 + 2];
  float qw = a.quats[n * 4], qx = a.quats[n * 4 + 1], qy = a.quats[n * 4 + 2], qz = a.quats[n * 4 + 3];
  float nq = __fsqrt_rn(A_(A_(A_(M_(qw, qw), M_(qx, qx)), M_(qy, qy)), M_(qz, qz)));
  nq = fmaxf(nq, 1e-12f);
  qw = D_(qw, nq); qx = D_(qx, nq); qy = D_(qy, nq); qz = D_(qz, nq);
  float R[3][3];
  R[0][0] = S_(1.f, M_(2.f, A_(M_(qy, qy), M_(qz, qz))));
  R[0][1] = M_(2.f, S_(M_(qx, qy), M_(qw, qz)));
  R[0][2] = M_(2.f, A_(M_(qx, qz), M_(qw, qy)));
  R[1][0] = M_(2.f, A_(M_(qx, qy), M_(qw, qz)));
  R[1][1] = S_(1.f, M_(2.f, A_(M_(qx, qx), M_(qz, qz))));
  R[1][2] = M_(2.f, S_(M_(qy, qz), M_(qw, qx)));
  R[2][0] = M_(2.f, S_(M_(qx, qz), M_(qw, qy)));
  R[2][1] = M_(2.f, A_(M_(qy, qz), M_(qw, qx)));
  R[2][2] = S_(1.f, M_(2.f, A_(M_(qx, qx), M_(qy, qy))));
  float Mm[3][3], Sg[3][3];
#pragma unroll
  for (int i = 0; i < 3; ++i)
#pragma unroll
    for (int j = 0; j < 3; ++j) Mm[i][j] = M_(R[i][j], a.scales[n * 3 + j]);
#pragma unroll
  for (int i = 0; i < 3; ++i)
#pragma unroll
    for (int k = 0; k < 3; ++k) Sg[i][k] = dot3(Mm[i][0], Mm[k][0], Mm[i][1], Mm[k][1], Mm[i][2], Mm[k][2]);
  const float* V = a.viewmats + c * 16;
  const float* K = a.Ks + c * 9;
  float t[3];
#pragma unroll
  for (int i = 0; i < 3; ++i) t[i] = A_(dot3(V[i * 4], mx, V[i * 4 + 1], my, V[i * 4 + 2], mz), V[i * 4 + 3]);
  float T[3][3], Cc[3][3];
#pragma unroll
  for (int i = 0; i < 3; ++i)
#pragma unroll
    for (int j = 0; j < 3; ++j) T[i][j] = dot3(V[i * 4], Sg[0][j], V[i * 4 + 1], Sg[1][j], V[i * 4 + 2], Sg[2][j]);
#pragma unroll
  for (int i = 0; i < 3; ++i)
#pragma unroll
    for (int l = 0; l < 3; ++l) Cc[i][l] = dot3(T[i][0], V[l * 4], T[i][1], V[l * 4 + 1], T[i][2], V[l * 4 + 2]);
  const float fx = K[0], fy = K[4], cx = K[2], cy = K[5];
  const float tz = t[2], tz2 = M_(tz, tz);
  const float tanx = D_(M_(0.5f, a.width), fx), tany = D_(M_(0.5f, a.height), fy);
  const float lxp = A_(D_(S_(a.width, cx), fx), M_(0.3f, tanx)), lxn = A_(D_(cx, fx), M_(0.3f, tanx));
  const float lyp = A_(D_(S_(a.height, cy), fy), M_(0.3f, tany)), lyn = A_(D_(cy, fy), M_(0.3f, tany));
  const float txc = M_(tz, fminf(fmaxf(D_(t[0], tz), -lxn), lxp));
  const float tyc = M_(tz, fminf(fmaxf(D_(t[1], tz), -lyn), lyp));
  const float J00 = D_(fx, tz), J02 = D_(M_(-fx, txc), tz2), J11 = D_(fy, tz), J12 = D_(M_(-fy, tyc), tz2);
  const float U00 = A_(M_(J00, Cc[0][0]), M_(J02, Cc[2][0])), U01 = A_(M_(J00, Cc[0][1]), M_(J02, Cc[2][1])),
              U02 = A_(M_(J00, Cc[0][2]), M_(J02, Cc[2][2]));
  const float U10 = A_(M_(J11, Cc[1][0]), M_(J12, Cc[2][0])), U11 = A_(M_(J11, Cc[1][1]), M_(J12, Cc[2][1])),
              U12 = A_(M_(J11, Cc[1][2]), M_(J12, Cc[2][2]));
  const float c00 = A_(M_(U00, J00), M_(U02, J02)), c01 = A_(M_(U01, J11), M_(U02, J12));
  const float c10 = A_(M_(U10, J00), M_(U12, J02)), c11 = A_(M_(U11, J11), M_(U12, J12));
  r.m2x = D_(dot3(K[0], t[0], K[1], t[1], K[2], tz), tz);
  r.m2y = D_(dot3(K[3], t[0], K[4], t[1], K[5], tz), tz);
  const float aa = A_(c00, a.eps2d), dd = A_(c11, a.eps2d);
  float det = S_(M_(aa, dd), M_(c01, c10));
  det = fmaxf(det, 1e-10f);
  r.c0 = D_(dd, det);
  r.c1 = D_(D_(-A_(c01, c10), 2.f), det);
  r.c2 = D_(aa, det);
  r.depth = tz;
  float rx = ceilf(M_(3.33f, __fsqrt_rn(aa))), ry = ceilf(M_(3.33f, __fsqrt_rn(dd)));
  const bool depth_ok = tz > a.near_plane && tz < a.far_plane;
  if (!depth_ok) { rx = 0.f; ry = 0.f; }
  const bool inside = A_(r.m2x, rx) > 0.f && S_(r.m2x, rx) < a.width && A_(r.m2y, ry) > 0.f && S_(r.m2y, ry) < a.height;
  if (!inside) { rx = 0.f; ry = 0.f; }
  r.rx = (int)rx; r.ry = (int)ry;
  r.valid = r.rx > 0 && r.ry > 0;
  return r;
}

__global__ void __launch_bounds__(kGsThreads) gsplat_count_kernel(const GsArgs a) {
  const int c = blockIdx.y, n = blockIdx.x * kGsThreads + threadIdx.x;
  const bool v = n < a.N && gs_project(a, n, c).valid;
  const int cnt = __syncthreads_count(v);
  if (threadIdx.x == 0) a.blk_counts[c * a.nblk + blockIdx.x] = cnt;
}

// One block. Cameras are grouped by owner: member d owns cameras [d*C_local, (d+1)*C_local).
__global__ void gsplat_scan_kernel(const SymmCtx c, const GsArgs a) {
  int* to = symm_local<int>(c, a.cnt_off);
  for (int d = threadIdx.x; d < c.gsize; d += blockDim.x) {
    int run = 0;
    for (int cam = d * a.C_local; cam < (d + 1) * a.C_local; ++cam)
      for (int b = 0; b < a.nblk; ++b) {
        const int v = a.blk_counts[cam * a.nblk + b];
        a.blk_counts[cam * a.nblk + b] = run;
        run += v;
      }
    to[d] = run;
  }
}

__global__ void __launch_bounds__(kGsThreads) gsplat_emit_kernel(const SymmCtx c, const GsArgs a) {
  __shared__ int warp_cnt[kGsThreads / 32];
  __shared__ int s_base;
  // the barrier needs every block index < kSymmMaxBlocks: blocks walk (camera, chunk) pairs in a grid-stride loop
  if (!symm_block_barrier(c, 610, 1)) return;
  const int total_items = a.C * a.nblk;
  for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
    const int cam = item / a.nblk, blk = item - cam * a.nblk;
    const int d = cam / a.C_local;
    if (threadIdx.x == 0) {
      int base = 0;
      for (int s = 0; s < c.grank; ++s) base += symm_ptr<int>(c, c.members[s], a.cnt_off)[d];
      s_base = base + a.blk_counts[cam * a.nblk + blk];
    }
    const int n = blk * kGsThreads + threadIdx.x;
    GsProj p;
    p.valid = false;
    if (n < a.N) p = gs_project(a, n, cam);
    const unsigned m = __ballot_sync(0xffffffffu, p.valid);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) warp_cnt[wid] = __popc(m);
    __syncthreads();
    int pos = s_base + __popc(m & ((1u << lane) - 1));
    for (int w = 0; w < wid; ++w) pos += warp_cnt[w];
    if (p.valid && pos < a.cap_rows) {
      const int words = kGsHeader + a.D;
      uint32_t* rec = symm_ptr<uint32_t>(c, c.members[d], a.recv_off) + (long long)pos * words;
      rec[0] = (uint32_t)(cam - d * a.C_local);
      rec[1] = (uint32_t)(a.gid_offset + n);
      rec[2] = (uint32_t)p.rx; rec[3] = (uint32_t)p.ry;
      rec[4] = __float_as_uint(p.m2x); rec[5] = __float_as_uint(p.m2y); rec[6] = __float_as_uint(p.depth);
      rec[7] = __float_as_uint(p.c0); rec[8] = __float_as_uint(p.c1); rec[9] = __float_as_uint(p.c2);
      rec[10] = __float_as_uint(a.opac[n]);
      for (int j = 0; j < a.D; ++j) rec[kGsHeader + j] = __float_as_uint(a.colors[n * a.D + j]);
    }
    __syncthreads();
  }
  if (!symm_block_barrier(c, 610, 2)) return;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    int tot = 0;
    for (int s = 0; s < c.gsize; ++s) tot += symm_ptr<int>(c, c.members[s], a.cnt_off)[c.grank];
    *a.recv_count = tot;
  }
  // the count words are read above by peers of the NEXT call only after its first barrier; keep them stable until
  // every member has read them
  symm_block_barrier(c, 610, 3);
}

}  // namespace pkb

using namespace pkb;

extern "C" int pkb_gsplat_project_exchange(const pkb_symm_ctx* h, const void* means, const void* quats, const void* scales,
                                           const void* opac, const void* colors, const void* viewmats, const void* Ks,
                                           int N, int C_local, int D, float width, float height, float eps2d,
                                           float near_plane, float far_plane, int gid_offset, void* blk_counts,
                                           unsigned long long cnt_off, unsigned long long recv_off, long long cap_rows,
                                           void* recv_count, void* stream) {
  if (int rc = symm_ctx_check(h)) return rc;
  PKB_CHECK_ARG(N >= 1 && C_local >= 1 && D >= 0 && D <= kGsMaxColor, "need N, C_local >= 1 and at most 8 colour channels");
  PKB_CHECK_ARG((cnt_off & 3) == 0 && (recv_off & 15) == 0 && cap_rows >= 0, "heap offsets misaligned");
  const SymmCtx c = symm_ctx_from_api(h);
  GsArgs a;
  a.means = static_cast<const float*>(means); a.quats = static_cast<const float*>(quats);
  a.scales = static_cast<const float*>(scales); a.opac = static_cast<const float*>(opac);
  a.colors = static_cast<const float*>(colors); a.viewmats = static_cast<const float*>(viewmats);
  a.Ks = static_cast<const float*>(Ks);
  a.N = N; a.C = C_local * h->gsize; a.C_local = C_local; a.D = D;
  a.width = width; a.height = height; a.eps2d = eps2d; a.near_plane = near_plane; a.far_plane = far_plane;
  a.gid_offset = gid_offset;
  a.nblk = (N + kGsThreads - 1) / kGsThreads;
  a.blk_counts = static_cast<int*>(blk_counts);
  a.cnt_off = cnt_off; a.recv_off = recv_off; a.cap_rows = cap_rows;
  a.recv_count = static_cast<int*>(recv_count);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  gsplat_count_kernel<<<dim3(a.nblk, a.C), kGsThreads, 0, s>>>(a);
  PKB_CHECK_CUDA(cudaGetLastError());
  gsplat_scan_kernel<<<1, 32, 0, s>>>(c, a);
  PKB_CHECK_CUDA(cudaGetLastError());
  int grid = a.C * a.nblk;
  if (grid > kSymmMaxBlocks) grid = kSymmMaxBlocks;
  gsplat_emit_kernel<<<grid, kGsThreads, 0, s>>>(c, a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}
