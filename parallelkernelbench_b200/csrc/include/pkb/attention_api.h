// C view of the attention problem description (attention.cu).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct pkb_attn_desc {
  int32_t batch, sq, skv;       // sequences, Q rows per sequence, rows of the KV buffer per sequence
  int32_t hq, hkv, head_dim;    // query heads, KV heads (hq % hkv == 0), 64 or 128
  int32_t causal;
  float scale;                  // softmax scale (1/sqrt(d) usually)
  // Q rows come in runs of q_seg_rows rows; run i starts at global position q_seg_pos[i]
  int32_t q_seg_rows, num_q_segs;
  int32_t q_seg_pos[16];
  // KV buffer segments: rows [row0, row0 + len) hold global positions [pos0, pos0 + len)
  int32_t num_kv_segs;
  int32_t kv_seg_row0[16], kv_seg_pos0[16], kv_seg_len[16];
  // optional: segment s may be read once kv_seg_ready[kv_seg_flag[s]] >= ready_epoch (device
  // memory); kv_seg_flag[s] < 0 means the segment needs no wait (local data)
  int32_t kv_seg_flag[16];
  const uint32_t* kv_seg_ready;
  uint32_t ready_epoch;
  uint32_t _pad;
  uint64_t budget_ns;           // bound of device-side waits, 0 = default
  // optional trace buffer (int64): word 0 = record count, records of 4 words start at word 4
  void* trace;
  int32_t trace_capacity;
  int32_t _pad2;
} pkb_attn_desc;

// q: [batch*sq, hq, d], k/v: [batch*skv, hkv, d] bf16; out like q; lse: [batch, hq, sq] fp32 or NULL
int pkb_flash_attn_fwd(const pkb_attn_desc* desc, const void* q, const void* k, const void* v, void* out,
                       void* lse, void* stream);

struct pkb_symm_ctx;
// Context-parallel form. k_local / v_local: this rank's [segs_per_rank * seg_rows, hkv, d] rows. The
// gather buffers (heap offsets, [gsize * segs_per_rank * seg_rows, hkv, d]) receive every rank's rows
// in group order; desc->skv must equal that row count and desc->kv_seg_* must describe it.
// flags_off: gsize * segs_per_rank uint32 counters in the heap; desc->ready_epoch = call index
// (1, 2, ...) - it is scaled by the pieces per segment inside. comm_blocks CTAs do the pushes.
int pkb_flash_attn_fwd_ring(const pkb_attn_desc* desc, const struct pkb_symm_ctx* h, const void* q,
                            const void* k_local, const void* v_local, unsigned long long k_gather_off,
                            unsigned long long v_gather_off, unsigned long long flags_off, int segs_per_rank,
                            int seg_rows, int comm_blocks, void* out, void* lse, void* stream);

#ifdef __cplusplus
}
#endif
