// C view of the symmetric-heap context and the collective entry points (collectives.cu).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Mirrors pkb::SymmCtx minus the device-only fields. Filled by the Python side (ctypes.Structure).
typedef struct pkb_symm_ctx {
  uint64_t base;
  uint64_t stride;
  uint64_t mc_base;
  int32_t rank;
  int32_t world;
  int32_t gsize;
  int32_t grank;
  int32_t members[16];
  int32_t channel;
  int32_t _pad;
  uint64_t budget_ns;  // 0 = library default
} pkb_symm_ctx;

// dtype: 0 bf16, 1 fp32, 2 fp64, 3 fp16, 4 int32, 5 int64. op: 0 sum, 1 max, 2 min.
int pkb_coll_barrier(const pkb_symm_ctx* h, int blocks, void* stream);
int pkb_coll_reduce(const pkb_symm_ctx* h, int dtype, int op, const void* src, long long stage_elems,
                    unsigned long long stage_off, long long in_base, long long n, void* out, int active,
                    double scale, int max_blocks, void* stream);
int pkb_coll_gather(const pkb_symm_ctx* h, const void* src, long long stage_bytes,
                    unsigned long long stage_off, unsigned int src_mask, long long in_base,
                    long long in_member_stride, long long seg_bytes, void* out, long long out_stride,
                    int active, int max_blocks, void* stream);
// All-to-all of gsize chunks of chunk_bytes as a push with the TMA unit (bulk loads of local memory, bulk stores into the
// receivers' [gsize, chunk_bytes] buffer at heap offset recv_off). out: local result, or null when the receive buffer itself
// is the result (it then has to be free on every member when the call starts).
int pkb_coll_all_to_all_push(const pkb_symm_ctx* h, const void* src, long long chunk_bytes, unsigned long long recv_off,
                             void* out, int max_blocks, void* stream);
// Latency-optimised all-reduce (bf16 / fp32, at most cap_units 4-byte words): data and an epoch word travel in one
// 8-byte store, no barrier. ll_off: header (16 bytes, zero at first use) + 2 * gsize * cap_units * 8 bytes in the heap.
int pkb_coll_allreduce_ll(const pkb_symm_ctx* h, int dtype, int op, const void* src, long long n, unsigned long long ll_off,
                          long long cap_units, void* out, double scale, void* stream);
// All-gather of `words` 4-byte words per member with the same no-barrier exchange; out is [gsize, words].
int pkb_coll_allgather_ll(const pkb_symm_ctx* h, const void* src, long long words, unsigned long long ll_off,
                          long long cap_units, void* out, void* stream);
int pkb_coll_allreduce_twoshot(const pkb_symm_ctx* h, int dtype, int op, const void* src, long long n,
                               unsigned long long stage_off, unsigned long long result_off, void* out,
                               int src_in_heap, double scale, int max_blocks, void* stream);
// NVLS push all-gather / NVLS reduce-scatter (see collectives.cu); both need the multicast mapping and the whole-job group.
int pkb_coll_allgather_nvls(const pkb_symm_ctx* h, const void* src, long long bytes, unsigned long long gather_off, void* out,
                            int max_blocks, void* stream);
// Broadcast of member `root`'s bytes through the switch (multimem.st by the root only) into heap offset bcast_off of every rank.
int pkb_coll_broadcast_nvls(const pkb_symm_ctx* h, const void* src, long long bytes, int root, unsigned long long bcast_off, void* out,
                            int max_blocks, void* stream);
int pkb_coll_reduce_scatter_nvls(const pkb_symm_ctx* h, int dtype, const void* src, long long n, unsigned long long stage_off,
                                 void* out, int src_in_heap, int max_blocks, void* stream);
int pkb_coll_allreduce_nvls(const pkb_symm_ctx* h, int dtype, const void* src, long long n,
                            unsigned long long stage_off, unsigned long long result_off, void* out,
                            int src_in_heap, int max_blocks, void* stream);
// Remote row gather over a table sharded by rows: out[i] = table_of_member(ids[i] / rows_per_member)[ids[i] % rows_per_member].
// ids are int64; ids outside [0, gsize * rows_per_member) produce rows of zeros. With sync = 0 the shards must already
// be resident at table_off on every member and unchanged since the last barrier.
int pkb_coll_row_gather(const pkb_symm_ctx* h, const void* src, long long stage_bytes, unsigned long long table_off,
                        const void* ids, long long n, long long rows_per_member, long long row_bytes, void* out,
                        int sync, int max_blocks, void* stream);
// All-to-all with a layout change. Every member stages its whole tensor; member r then copies, from each member g,
// the box  base_g + r * in_rank_off + i0*in_strides[0] + i1*in_strides[1] + i2*in_strides[2]  (inner_bytes contiguous
// bytes per index triple, extents[3] triples) to  out + g * out_member_off + i0*out_strides[0] + ... . All in bytes.
int pkb_coll_a2a_permute(const pkb_symm_ctx* h, const void* src, long long stage_bytes, unsigned long long stage_off,
                         long long in_rank_off, const long long* extents, const long long* in_strides,
                         long long out_member_off, const long long* out_strides, long long inner_bytes, void* out,
                         int max_blocks, void* stream);
int pkb_coll_all_to_all_v(const pkb_symm_ctx* h, const void* src, long long src_rows, long long row_bytes,
                          const void* send_counts, const void* send_offsets, unsigned long long stage_off,
                          unsigned long long meta_off, void* out, long long out_capacity_rows,
                          void* recv_counts, void* recv_total, int max_blocks, void* stream);

// symmetric heap (symm_heap.cu)
int pkb_heap_multicast_supported();
long long pkb_heap_round_size(long long bytes, int world, int with_multicast);
int pkb_heap_create(long long bytes, int rank, int world, int* out_fd);
int pkb_heap_import_peer(int heap, int peer, int fd);
unsigned long long pkb_heap_base(int heap);
unsigned long long pkb_heap_stride(int heap);
unsigned long long pkb_heap_mc_base(int heap);
int pkb_heap_mc_create(int heap, int* out_fd);
int pkb_heap_mc_import(int heap, int fd);
int pkb_heap_mc_add_device(int heap);
int pkb_heap_mc_bind(int heap);
int pkb_heap_destroy(int heap);

#ifdef __cplusplus
}
#endif
