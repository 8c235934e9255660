// Parameters shared by the attention kernels (decode, mma.sync prefill, tcgen05 prefill).
#pragma once

#include "common.cuh"
#include "tc5.cuh"

struct AttnParams {
  CUtensorMap tmap_q;   // [batch, nq, heads, D], box 64 x 1 x 128 x 1 (prefill only)
  CUtensorMap tmap_k;   // [batch, keys, kv_heads, D], box 64 x 1 x 64 x 1
  CUtensorMap tmap_v;
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  // decode only: f32 queries / f32 output instead of the bf16 ones when non-null (the reference's
  // flash_attention_launch takes and returns f32); queries are rounded to bf16 (f16 for NVFP4 rows) on load
  const float* q_f32;
  float* out_f32;
  float* part;          // decode partials [batch, kv_heads, slots, 16 rows, D + 2]
  int* flags;
  // keys: live rows of the key/value buffer as this launch sees it (row 0 = the first live row);
  // q0: position of the first query relative to row 0 (two's complement when the queries start before it)
  uint32_t batch, nq, keys, heads, kv_heads, q0, splits, keys_per_split;
  // a launch may be one of several over the key runs of a paged cache: its splits are slots
  // [slot0, slot0 + splits) of `slots` partials per (sequence, kv head); slots == 1 writes the output itself
  uint32_t slots, slot0;
  uint32_t cap;         // NVFP4 rows: rows per sequence of the buffers (the batch stride); the dense readers' is in the tensor map
  float scale_log2;     // scale * log2(e)
  int causal;
  // sliding window (0 = none): query at position q sees keys in (q - window, q]; k_lo = first key any query of
  // the call can see, rounded down to a tile (the decode splits start there)
  uint32_t window, k_lo;
  // NVFP4 key/value rows (decode only): codes [batch, keys, kv_heads * D / 2] bytes, E4M3 scales
  // [batch, keys, kv_heads * D / 16] bytes, blocks of 16 along the features of a row
  const uint8_t* k_codes;
  const uint8_t* k_scales;
  const uint8_t* v_codes;
  const uint8_t* v_scales;
  // decode only: relative bias rel[batch, nq, heads, eff] added to the scaled score of a visible key at
  // distance q_abs - k_abs < eff, and eviction gaps: the key in cache row r sits at position
  // r + gap_cums[g] for the last g with gap_rows[g] <= r (rows ascending; no gap before it: r)
  const float* rel;
  const uint32_t* gap_rows;
  const uint32_t* gap_cums;
  uint32_t eff, ngaps;
  // the same instantiation works in absolute terms: position of row 0 without gaps, logical row of row 0 (what
  // the gap table is indexed by), position of the first query
  uint32_t pos0, row0, q0_abs;
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}


// tcgen05 prefill (attention_tc5.cu). MB_ATTN_PREFILL=legacy in the environment keeps the
// mma.sync kernel, for comparison runs.
int mb_attention_prefill_tc5(mb_ctx* ctx, cudaStream_t stream, const AttnParams& p);
inline bool mb_attention_prefill_legacy() {
  static const bool legacy = [] { const char* e = getenv("MB_ATTN_PREFILL"); return e && e[0] == 'l'; }();
  return legacy;
}
