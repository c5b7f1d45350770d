// Top-k selection with labels for the distributed nearest-neighbour search
// (reference: reference/79_dinov2_distributed_knn.py:7-14 local candidates, 43-65 merge on the owner).
//
// One block per query row sorts the row's candidates in shared memory (a bitonic network over (similarity, label) pairs,
// largest first, padded to a power of two with -inf) and writes the k best. The same kernel serves both stages:
//   local stage   candidates = one dense row of the similarity matrix, labels = the shard's label vector; the k best go out as
//                 (similarity, label) pairs, already in the layout of the exchange that hands every owner its candidate lists
//   merge stage   candidates = W lists of k pairs (one per source rank, strided as the exchange delivered them); the k best
//                 similarities go out together with the class votes (a shared-memory histogram divided by k)
// On one rank the local stage writes similarities and votes directly. The reference does each stage with a library top-k, a
// gather of the labels and, for the votes, a scatter-add into a zeroed matrix.
#include "pkb/api.h"
#include "pkb/host.h"

#include <cmath>

namespace pkb {

constexpr int kKnnThreads = 256;
constexpr int kKnnMaxCandidates = 4096;   // 32 KiB of shared memory for the pairs

struct KnnArgs {
  const float* vals;         // candidate similarities
  const long long* labels;   // dense form: label of candidate i (shared by all rows); nullptr in the packed form
  long long row_stride;      // elements between the rows of two queries
  long long seg_stride;      // elements between the segments of one query
  int nseg, seg_len;         // candidates of a row = nseg segments of seg_len
  int elem_stride;           // 1 dense, 2 packed (the label is the float after the similarity)
  int k, classes, np;        // np = candidates padded to a power of two
  float* out_pairs;          // [rows, k, 2] or nullptr
  float* out_sims;           // [rows, k] or nullptr
  float* out_votes;          // [rows, classes] or nullptr
};

__global__ void __launch_bounds__(kKnnThreads) knn_topk_kernel(const KnnArgs a) {
  extern __shared__ __align__(16) unsigned char knn_smem[];
  float* v = reinterpret_cast<float*>(knn_smem);
  int* l = reinterpret_cast<int*>(knn_smem + (size_t)a.np * 4);
  int* hist = reinterpret_cast<int*>(knn_smem + (size_t)a.np * 8);
  const long long row = blockIdx.x;
  const int total = a.nseg * a.seg_len;
  for (int i = threadIdx.x; i < a.np; i += kKnnThreads) {
    float val = -INFINITY;
    int lab = 0;
    if (i < total) {
      const int seg = i / a.seg_len, off = i - seg * a.seg_len;
      const float* p = a.vals + row * a.row_stride + seg * a.seg_stride + (long long)off * a.elem_stride;
      val = p[0];
      lab = a.labels ? (int)a.labels[i] : (int)p[1];
    }
    v[i] = val;
    l[i] = lab;
  }
  if (a.out_votes)
    for (int c = threadIdx.x; c < a.classes; c += kKnnThreads) hist[c] = 0;
  __syncthreads();
  for (int size = 2; size <= a.np; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < a.np; i += kKnnThreads) {
        const int j = i ^ stride;
        if (j > i) {
          const float x = v[i], y = v[j];
          const bool swap = ((i & size) == 0) ? (x < y) : (x > y);   // largest first in the final pass
          if (swap) {
            v[i] = y;
            v[j] = x;
            const int t = l[i];
            l[i] = l[j];
            l[j] = t;
          }
        }
      }
      __syncthreads();
    }
  }
  for (int i = threadIdx.x; i < a.k; i += kKnnThreads) {
    if (a.out_pairs) {
      a.out_pairs[(row * a.k + i) * 2] = v[i];
      a.out_pairs[(row * a.k + i) * 2 + 1] = (float)l[i];
    }
    if (a.out_sims) a.out_sims[row * a.k + i] = v[i];
    if (a.out_votes && l[i] >= 0 && l[i] < a.classes) atomicAdd(&hist[l[i]], 1);
  }
  if (a.out_votes) {
    __syncthreads();
    for (int c = threadIdx.x; c < a.classes; c += kKnnThreads) a.out_votes[row * a.classes + c] = (float)hist[c] / (float)a.k;
  }
}

}  // namespace pkb

using namespace pkb;

// vals: dense [rows, n] with labels int64 [n] (nseg = 1, seg_len = n, elem_stride = 1), or packed pairs
// [nseg, rows, seg_len, 2] with labels = nullptr (elem_stride = 2, row_stride = seg_len * 2, seg_stride = rows * seg_len * 2).
extern "C" int pkb_knn_topk(const void* vals, const void* labels, long long rows, long long row_stride, long long seg_stride, int nseg,
                            int seg_len, int elem_stride, int k, int classes, void* out_pairs, void* out_sims, void* out_votes,
                            void* stream) {
  PKB_CHECK_ARG(vals != nullptr && rows >= 1 && rows <= 0x7fffffffll && nseg >= 1 && seg_len >= 1, "need 1 <= rows, 1 <= segments, 1 <= length");
  PKB_CHECK_ARG((long long)nseg * seg_len <= kKnnMaxCandidates, "at most 4096 candidates per row");
  PKB_CHECK_ARG(elem_stride == 1 || elem_stride == 2, "candidates are dense (1) or (similarity, label) pairs (2)");
  PKB_CHECK_ARG((elem_stride == 1) == (labels != nullptr), "dense candidates need the label vector, packed ones carry their labels");
  PKB_CHECK_ARG(k >= 1 && k <= nseg * seg_len, "need 1 <= k <= candidates per row");
  PKB_CHECK_ARG(out_pairs != nullptr || out_sims != nullptr, "no output requested");
  PKB_CHECK_ARG(out_votes == nullptr || (classes >= 1 && classes <= 4096), "votes need 1 <= classes <= 4096");
  int np = 2;
  while (np < nseg * seg_len) np <<= 1;
  KnnArgs a{static_cast<const float*>(vals), static_cast<const long long*>(labels), row_stride, seg_stride, nseg, seg_len, elem_stride,
            k, classes, np, static_cast<float*>(out_pairs), static_cast<float*>(out_sims), static_cast<float*>(out_votes)};
  const size_t smem = (size_t)np * 8 + (out_votes ? (size_t)classes * 4 : 0);   // at most 32 KiB + 16 KiB
  knn_topk_kernel<<<(unsigned)rows, kKnnThreads, smem, static_cast<cudaStream_t>(stream)>>>(a);
  PKB_CHECK_CUDA(cudaGetLastError());
  return kApiOk;
}
