// Shared declarations of the flash-attention kernels (forward, dQ, dK/dV).
#pragma once
#include "host_common.h"

namespace ctb {
namespace attn {

// Visibility metadata, built once per step and shared by all layers:
//   seg    [B,S]      canonical run ids, 0 = padding
//   lim    [B,S]      inclusive last visible key index = max(i, attention_end[i]); null => i
//   row_start [B,S]   first token of the run that holds token i (the keys a query sees are the
//                     contiguous interval [row_start[i], lim[i]])
//   kv_lo  [B,S/128]  first key index any row of the 128-row query block can see
//   kv_hi  [B,S/128]  one past the last such key index (kv_hi <= kv_lo: nothing visible)
//   q_lo/q_hi [B,S/128] per 128-key block: range of query indices that can see it
// MoBA block-sparse routing (all null / zero for dense attention).  Keys are cut into blocks of
// `block` tokens counted from the start of their document; query i of head h may see key j of its
// own document iff j <= lim[i] and bit ((j - doc_start[i]) / block) of its selection mask is set
// (the query's own block is always selected).  Each CTA walks a list of key tiles (forward) or of
// (64-row block, head) pairs (backward) that the work-list kernels of moba.cu derived from the union
// of its rows' selections, instead of a contiguous range.
struct SparseArgs {
  const int* it_off;       // [work items + 1] offsets into it_list, work items in blockIdx order; or, when
                           // it_cnt is set, unused: item i owns it_list[i * it_stride ..] with it_cnt[i] entries
  const int* it_cnt;
  int it_stride;
  const int* it_list;      // forward: 128-key tile index; backward: 64-row block | head_in_group << 24
  const unsigned* sel;     // [B][Hq][S][words]
  const int* doc_start;    // [B][S]
  const unsigned* allsel;  // [B][Hq][S/64][words] AND of sel over each 64-query block (backward dK/dV fast path)
  int block;               // >= 128
  int words;
};

// Grouped MoBA: the query rows that selected a key block were gathered into one contiguous
// tensor (rows of a group adjacent, groups padded with zero rows to a multiple of 256), so the
// history part of MoBA is dense attention of each group against its key block and its cost follows
// the routing budget, not the sequence length.  Q / O / dO / dQ and the per-row statistics are then
// indexed by the gathered row (one batch, one head), K / V / dK / dV by (batch, kv head, token).
// One descriptor per CTA:
//   x  batch | kv head << 16
//   y  forward, dQ: first key of the group's block;  dK/dV: first key of the CTA's 128-key tile
//   z  dK/dV: first gathered row of the group
//   w  forward: rows of the CTA's 256-row tile that are real (0: nothing to do);  dQ: same for its
//      128-row tile;  dK/dV: rows of the group including padding (a multiple of 64; 0: nothing to do)
// No masks apply: every real row sees the whole block, padding rows are zero and contribute zero.
struct GroupArgs {
  const int4* desc;
  int block;          // keys per group, a multiple of 128
};

// Sequence parallelism: a rank may hold only the queries [q_off, q_off + Sq) of every row while
// keys and values cover the whole sequence of S tokens.  Q / O / dQ / dO / LSE / delta are then
// indexed by the local query position, the visibility metadata by the global one.
// Keys and values that an all-gather pull is still filling (sequence parallelism): K and V are the
// two halves of one gathered [S, row_elems] buffer whose chunks of `chunk` elements each have a flag;
// the producer warp acquires the flags of a 128-row tile before it issues the tile's copies, so the
// transfer overlaps the attention over the rows that are already there.
struct KvFlags {
  const unsigned* flags;   // null: K / V are plain memory
  long chunk;              // elements per flag
  long row_elems;          // elements per gathered row (K and V widths together)
  unsigned epoch;
};

struct FwdArgs {
  int B, S, Hq, Hkv;
  int Sq, q_off;
  float scale_log2;
  const int* seg;
  const int* lim;
  const int* row_start;
  const int* kv_lo;
  const int* kv_hi;
  float* lse;
  DeviceStatus* status;
  long long spin_budget;
  SparseArgs sp;
  GroupArgs grp;
  KvFlags kvf;
};

struct FwdCall {
  const void* q; const void* k; const void* v; void* o; float* lse;
  const int* seg; const int* lim; const int* row_start; const int* kv_lo; const int* kv_hi;
  int B, S, Hq, Hkv;
  int Sq = 0, q_off = 0;     // Sq == 0: all S queries
  long q_row_stride, k_row_stride, v_row_stride, o_row_stride;
  float scale;
  long long spin_budget;
  void* stream;
  SparseArgs sp{};
  GroupArgs grp{};
  int gathered_rows = 0;     // grouped: capacity of the gathered row space (a multiple of 256)
  KvFlags kvf{};
};

enum : int { MODE_DKV = 0, MODE_DQ = 1 };

// Extra metadata of the backward kernels, per token [B,S]:
//   run_start / run_end   first / last token of the token's run
//   first_q               first query that sees the token as a key
// so the keys query i sees are [run_start[i], lim[i]] and the queries that see key j are
// [first_q[j], run_end[j]].
struct BwdArgs {
  int B, S, Hq, Hkv;
  int Sq, q_off;
  float scale, scale_log2;
  const int* seg;
  const int* lim;
  const int* kv_lo;
  const int* kv_hi;
  const int* q_lo;
  const int* q_hi;
  const int* run_start;
  const int* run_end;
  const int* first_q;
  const float* neg_lse2;    // [B,Hq,Sq]  -lse * log2(e)
  const float* neg_delta;   // [B,Hq,Sq]  -sum_d O dO      (both from ctb_attn_bwd_stats)
  DeviceStatus* status;
  long long spin_budget;
  SparseArgs sp;
  GroupArgs grp;
};

struct BwdCall {
  const void* q; const void* k; const void* v; const void* dout;
  void* dq; void* dk; void* dv;
  const float* neg_lse2; const float* neg_delta;
  const int* seg; const int* lim; const int* kv_lo; const int* kv_hi; const int* q_lo; const int* q_hi;
  const int* run_start; const int* run_end; const int* first_q;
  int B, S, Hq, Hkv;
  int Sq = 0, q_off = 0;
  long q_row_stride, k_row_stride, v_row_stride, do_row_stride, dq_row_stride, dk_row_stride, dv_row_stride;
  float scale;
  long long spin_budget;
  void* stream;
  SparseArgs sp{};
  GroupArgs grp{};
  int gathered_rows = 0;     // grouped: capacity of the gathered row space
  int ctas = 0;              // grouped: CTAs to launch (one per descriptor)
};

// First entry and length of the work list of CTA `item`.
__device__ __forceinline__ void sparse_list(const SparseArgs& sp, int item, int& base, int& count) {
  if (sp.it_cnt != nullptr) {
    base = item * sp.it_stride;
    count = sp.it_cnt[item];
  } else {
    base = sp.it_off[item];
    count = sp.it_off[item + 1] - base;
  }
}

// Selection bit of document-relative block `blk` for (batch b, head h, query qi).
__device__ __forceinline__ bool sparse_bit(const SparseArgs& sp, int b, int h, int Hq, int S, int qi, int blk) {
  if (blk < 0 || (blk >> 5) >= sp.words) return false;
  const unsigned w = __ldg(sp.sel + ((static_cast<size_t>(b) * Hq + h) * S + qi) * sp.words + (blk >> 5));
  return (w >> (blk & 31)) & 1u;
}

// For a query row and the keys [k0, k0 + width): the keys before `bound` are visible iff `v0`,
// the keys from `bound` on iff `v1` (a tile no wider than a block holds at most one boundary).
struct SparseRow {
  int bound;
  bool v0, v1;
};
__device__ __forceinline__ SparseRow sparse_row(const SparseArgs& sp, int b, int h, int Hq, int S, int qi,
                                                int my_start, int k0, int width) {
  SparseRow r;
  const int rel = k0 - my_start;
  const int b0 = rel >= 0 ? rel / sp.block : -1;
  r.bound = my_start + (b0 + 1) * sp.block;
  r.v0 = sparse_bit(sp, b, h, Hq, S, qi, b0);
  r.v1 = (r.bound < k0 + width) ? sparse_bit(sp, b, h, Hq, S, qi, b0 + 1) : r.v0;
  return r;
}

}  // namespace attn
}  // namespace ctb
