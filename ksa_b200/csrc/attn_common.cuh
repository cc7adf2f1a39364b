// Closed-form tile enumeration and masking for Kwai Summary Attention in the
// two-stream layout (text keys and summary keys are separate tensors).
//
// For a tile of 128 text queries the visible keys are
//   * summary keys  s  with  s / S  <  q_chunk - W          (older than the window),
//   * text keys     u  with  u <= t  and  q_chunk - u / C <= W  (window + own chunk, causal),
// so for every query row the allowed keys of a key tile form one interval
// [lo, hi] of columns.  No block list and no mask tensor is ever built; the
// reference evaluates a mask_mod per element to build O(M*N) block lists
// (flash_attn/cute/compute_block_sparsity.py:277 in its flash_attn_cute wheel, summary_attn/mask.py:19-59 in its
// summary_attn wheel).
// Plain causal attention is the case W = "infinite", no summary keys; a token
// sliding window adds t - u < tok_window.
#pragma once
#include "common.cuh"

namespace ksa {

struct AttnShape {
  int B, Hq, Hkv;
  int Lq;          // query rows held locally
  int Lk;          // text key rows held locally
  int Ns;          // summary key rows held locally
  int q_off;       // global text index of local query row 0
  int k_off;       // global text index of local text key row 0
  int s_off;       // global summary index of local summary key row 0
  int chunk;       // C
  int n_sum;       // S
  int window;      // W in chunks (>= 1<<29 means unbounded)
  int tok_window;  // > 0: additionally t - u < tok_window
  // Packed documents (both null: one document per sequence).  A query only sees keys of its own document:
  // q_doc_start[b * Lq + i] = global text index of the first token of local query row i's document,
  // k_doc_end[b * Lk + j]   = global text index one past the last token of local text key row j's document
  // (the replacement for flash_attn_varlen_func with cu_seqlens, muse/layers/attention_utils.py:222-246).
  const int* q_doc_start;
  const int* k_doc_end;
};

struct TileRange {
  int n_sum_tiles;  // summary key tiles [0, n_sum_tiles)
  int text_first;   // first text key tile
  int text_last;    // last text key tile (inclusive, the diagonal)
  __device__ __forceinline__ int total() const { return n_sum_tiles + (text_last - text_first + 1); }
};

__device__ __forceinline__ TileRange key_tiles_for_query_tile(const AttnShape& s, int q_tile, int b = 0) {
  TileRange r;
  const int t0 = s.q_off + q_tile * 128;
  const int t1 = min(s.q_off + s.Lq, t0 + 128) - 1;
  const int qc_lo = t0 / s.chunk, qc_hi = t1 / s.chunk;
  const int s_end = max(0, qc_hi - s.window) * s.n_sum;  // exclusive, global
  const int s_end_l = min(max(s_end - s.s_off, 0), s.Ns);
  r.n_sum_tiles = (s_end_l + 127) / 128;
  int u_min = max(0, qc_lo - s.window) * s.chunk;
  if (s.tok_window > 0) u_min = max(u_min, t0 - s.tok_window + 1);
  if (s.q_doc_start) u_min = max(u_min, s.q_doc_start[(long long)b * s.Lq + q_tile * 128]);   // non-decreasing in the row
  r.text_first = max(0, u_min - s.k_off) / 128;
  r.text_last = max(0, min(t1 - s.k_off, s.Lk - 1)) / 128;
  return r;
}

// Allowed column interval [lo, hi] (inclusive, in-tile columns 0..127) of key tile `kt` for global query index t.
// `doc_start`: global text index of the first token of the query's document (0 without packing).
__device__ __forceinline__ void allowed_columns(const AttnShape& s, int t, bool is_summary, int kt, int& lo, int& hi,
                                                int doc_start = 0) {
  const int qc = t / s.chunk;
  if (is_summary) {
    lo = 0;
    const int end_g = max(0, qc - s.window) * s.n_sum;            // exclusive, global
    hi = min(end_g - s.s_off, s.Ns) - kt * 128 - 1;
  } else {
    int lo_g = max(0, qc - s.window) * s.chunk;
    if (s.tok_window > 0) lo_g = max(lo_g, t - s.tok_window + 1);
    lo_g = max(lo_g, doc_start);
    lo = lo_g - s.k_off - kt * 128;
    hi = min(t - s.k_off, s.Lk - 1) - kt * 128;
  }
}

// Key tiles -> the query tiles that see them (used by the key-stationary backward pass).
struct QueryRange {
  int first, last;  // inclusive query tiles; empty when first > last
};
__device__ __forceinline__ QueryRange query_tiles_for_text_key_tile(const AttnShape& s, int k_tile, int b = 0) {
  QueryRange r;
  const int u0 = s.k_off + k_tile * 128;
  const int u1 = min(s.k_off + s.Lk, u0 + 128) - 1;
  // earliest query: t >= u0 ; latest query: chunk(t) <= chunk(u1) + W and (tok window) t <= u1 + tok_window - 1
  long long t_max = (s.window >= (1 << 29)) ? (long long)s.q_off + s.Lq - 1
                                            : (long long)(u1 / s.chunk + s.window + 1) * s.chunk - 1;
  if (s.tok_window > 0) t_max = min(t_max, (long long)u1 + s.tok_window - 1);
  if (s.k_doc_end) t_max = min(t_max, (long long)s.k_doc_end[(long long)b * s.Lk + (u1 - s.k_off)] - 1);   // non-decreasing
  t_max = min(t_max, (long long)s.q_off + s.Lq - 1);
  const int t_min = max(u0, s.q_off);
  if (t_max < t_min) { r.first = 1; r.last = 0; return r; }
  r.first = (t_min - s.q_off) / 128;
  r.last = (int)((t_max - s.q_off) / 128);
  return r;
}
__device__ __forceinline__ QueryRange query_tiles_for_summary_key_tile(const AttnShape& s, int s_tile) {
  QueryRange r;
  const int s0 = s.s_off + s_tile * 128;
  if (s.window >= (1 << 29) || s_tile * 128 >= s.Ns) { r.first = 1; r.last = 0; return r; }
  // summary key s is visible to text queries of chunk qc > s / S + W
  const long long t_min = max((long long)(s0 / s.n_sum + s.window + 1) * s.chunk, (long long)s.q_off);
  const long long t_max = (long long)s.q_off + s.Lq - 1;
  if (t_max < t_min) { r.first = 1; r.last = 0; return r; }
  r.first = (int)((t_min - s.q_off) / 128);
  r.last = (int)((t_max - s.q_off) / 128);
  return r;
}

// Key / value sources of a context-parallel shard: the tiles of the halo (the last text keys of the previous rank)
// and of older chunks' summaries are read by TMA straight from the owners' exchange slots, which are mapped into this
// process (peer memory; plain TMA loads, no multicast), while this rank's own tiles come from its own slot.
//   text tile kt : kt * 128 < halo ? (source 0, row kt*128) : (source 1, row kt*128 - halo)
//   summary tile j : source (j*128) / nsl, row (j*128) % nsl          (nsl is a multiple of 128 or the only source)
// flags[s] (null for this rank's own slot): a flag in THIS rank's memory that the owner of source s raises to
// `flag_target` once its keys and values are in its slot; the producer waits for it (bounded) before the first load.
constexpr int kCpMaxSum = 8;
struct CpSources {
  CUtensorMap kt[2], vt[2];
  CUtensorMap ks[kCpMaxSum], vs[kCpMaxSum];
  const uint32_t* text_flag[2];
  const uint32_t* sum_flag[kCpMaxSum];
  uint32_t flag_target;
  int halo, nsl;
};

}  // namespace ksa
