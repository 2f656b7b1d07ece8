// Attention metadata of one micro-batch in a single launch: canonical segment ids, positions that
// restart per segment, the inclusive visibility limit of every query (MaskGIT image blocks), and
// the per-block summaries that let the flash kernels skip tiles.
//
// One CTA per batch row.  The row is cut into one contiguous chunk per thread; every prefix
// quantity (run counter, start of the current run, end of the current run, first query that sees
// a key) is a chunk-local pass, a block-wide scan of the chunk totals in shared memory, and a
// second chunk-local pass seeded with the scanned carry.
//
//   seg[i]       one-based id of the contiguous valid run that holds token i (0: padding); a run
//                ends where the mask drops or the caller's label changes
//   pos[i]       i - first token of the run
//   lim[i]       last key token i may see: max(i, attention_end[i]) clipped to its run
//   start[i], end[i]   first / last token of the run; first_q[i] first query that sees key i.  The
//                keys visible to query i are the interval [start[i], lim[i]], the queries that see
//                key j the interval [first_q[j], end[j]]: the flash kernels mask by interval
//   kv_lo/kv_hi  [S/128] key range [lo, hi) needed by the query block
//   q_lo/q_hi    [S/128] query range [lo, hi) that can see the key block
//
// Reference counterparts: run-based segment ids and restart positions
// (src/causal_trainer/modeling/rotary.py:13-50,82-110) and the per-block (min, max, max_end)
// summaries of the Pallas attention (src/causal_trainer/kernels/efficient_attention.py:313-374).
#include "host_common.h"

namespace ctb {
namespace meta {

constexpr int THREADS = 1024;
constexpr int BIG = 0x7fffffff;

enum Op { OP_SUM = 0, OP_MAX = 1, OP_MIN = 2 };

template <int OP>
__device__ __forceinline__ int combine(int a, int b) {
  return OP == OP_SUM ? a + b : (OP == OP_MAX ? max(a, b) : min(a, b));
}

// Exclusive scan of one value per thread (thread order, or reversed thread order).
template <int OP, bool REVERSE>
__device__ int block_scan_exclusive(int v, int identity, int* sh) {
  const int t = REVERSE ? THREADS - 1 - static_cast<int>(threadIdx.x) : static_cast<int>(threadIdx.x);
  sh[t] = v;
  __syncthreads();
  for (int off = 1; off < THREADS; off <<= 1) {
    const int other = t >= off ? sh[t - off] : identity;
    __syncthreads();
    sh[t] = combine<OP>(sh[t], other);
    __syncthreads();
  }
  const int excl = t > 0 ? sh[t - 1] : identity;
  __syncthreads();
  return excl;
}

struct Args {
  const int* mask;      // [B,S] non-zero: token exists
  const int* label;     // [B,S] caller's segment labels or nullptr
  const int* att_end;   // [B,S] MaskGIT block ends or nullptr
  int* seg;             // [B,S]
  int* pos;             // [B,S]
  int* lim;             // [B,S]
  int* rows;            // [4,B,S]: run start, run end (inclusive), first query that sees the key, scatter scratch
  int *kv_lo, *kv_hi, *q_lo, *q_hi;                         // [B,S/128]
  int S;
};

__global__ void __launch_bounds__(THREADS) attention_meta_kernel(const Args a) {
  __shared__ int sh[THREADS];
  const int S = a.S;
  const int row = blockIdx.x;
  const int* mask = a.mask + static_cast<size_t>(row) * S;
  const int* label = a.label ? a.label + static_cast<size_t>(row) * S : nullptr;
  const int* att_end = a.att_end ? a.att_end + static_cast<size_t>(row) * S : nullptr;
  int* seg = a.seg + static_cast<size_t>(row) * S;
  int* pos = a.pos + static_cast<size_t>(row) * S;
  int* lim = a.lim + static_cast<size_t>(row) * S;
  const size_t plane = static_cast<size_t>(gridDim.x) * S;
  int* run_start = a.rows + static_cast<size_t>(row) * S;
  int* run_end = run_start + plane;
  int* first_q = run_end + plane;
  int* first_at = first_q + plane;

  const int per = (S + THREADS - 1) / THREADS;
  const int lo = min(S, static_cast<int>(threadIdx.x) * per);
  const int hi = min(S, lo + per);

  auto starts = [&](int i) -> bool {
    if (mask[i] == 0) return false;
    if (i == 0 || mask[i - 1] == 0) return true;
    return label != nullptr && label[i] != label[i - 1];
  };
  auto ends = [&](int i) -> bool {
    if (mask[i] == 0) return false;
    return i == S - 1 || mask[i + 1] == 0 || starts(i + 1);
  };

  // ---- forward: run counter and start of the current run
  int n_starts = 0, last_start = 0;
  for (int i = lo; i < hi; ++i)
    if (starts(i)) {
      ++n_starts;
      last_start = i;
    }
  int run = block_scan_exclusive<OP_SUM, false>(n_starts, 0, sh);
  int start = block_scan_exclusive<OP_MAX, false>(last_start, 0, sh);
  for (int i = lo; i < hi; ++i) {
    if (starts(i)) {
      ++run;
      start = i;
    }
    const bool valid = mask[i] != 0;
    seg[i] = valid ? run : 0;
    pos[i] = valid ? i - start : 0;
    run_start[i] = start;
  }

  // ---- backward: end of the current run, visibility limit
  int first_end = BIG;
  for (int i = hi - 1; i >= lo; --i)
    if (ends(i)) first_end = i;
  int end = block_scan_exclusive<OP_MIN, true>(first_end, BIG, sh);
  for (int i = hi - 1; i >= lo; --i) {
    if (ends(i)) end = i;
    run_end[i] = end;
    int l = i;
    if (att_end != nullptr) l = min(max(i, att_end[i]), mask[i] != 0 ? end : i);
    lim[i] = l;
    first_at[i] = BIG;
  }
  __syncthreads();

  // ---- first query that sees key j: min(j, min over p >= j of the first query whose limit is p)
  if (att_end != nullptr) {
    for (int i = lo; i < hi; ++i)
      if (mask[i] != 0) atomicMin(&first_at[lim[i]], i);
    __syncthreads();
    int chunk_min = BIG;
    for (int i = lo; i < hi; ++i) chunk_min = min(chunk_min, first_at[i]);
    int carry = block_scan_exclusive<OP_MIN, true>(chunk_min, BIG, sh);
    for (int i = hi - 1; i >= lo; --i) {
      carry = min(carry, first_at[i]);
      first_q[i] = min(carry, i);
    }
  } else {
    for (int i = lo; i < hi; ++i) first_q[i] = i;
  }
  __syncthreads();

  // ---- block summaries: one warp per 128-token block, four tokens per lane
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb128 = S / 128;
  for (int blk = warp; blk < nb128; blk += THREADS / 32) {
    int v_kv_lo = BIG, v_kv_hi = 0, v_q_lo = BIG, v_q_hi = 0;
    for (int e = 0; e < 4; ++e) {
      const int i = blk * 128 + lane * 4 + e;
      if (seg[i] != 0) {
        v_kv_lo = min(v_kv_lo, run_start[i]);
        v_kv_hi = max(v_kv_hi, lim[i] + 1);
        v_q_lo = min(v_q_lo, first_q[i]);
        v_q_hi = max(v_q_hi, run_end[i] + 1);
      }
    }
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      v_kv_lo = min(v_kv_lo, __shfl_xor_sync(0xffffffffu, v_kv_lo, off));
      v_kv_hi = max(v_kv_hi, __shfl_xor_sync(0xffffffffu, v_kv_hi, off));
      v_q_lo = min(v_q_lo, __shfl_xor_sync(0xffffffffu, v_q_lo, off));
      v_q_hi = max(v_q_hi, __shfl_xor_sync(0xffffffffu, v_q_hi, off));
    }
    if (lane == 0) {
      const size_t o = static_cast<size_t>(row) * nb128 + blk;
      a.kv_lo[o] = v_kv_hi > 0 ? v_kv_lo : 0;
      a.kv_hi[o] = v_kv_hi;
      a.q_lo[o] = v_q_hi > 0 ? v_q_lo : 0;
      a.q_hi[o] = v_q_hi;
    }
  }
}

}  // namespace meta
}  // namespace ctb

// All tensors int32.  `label` and `att_end` may be null.  `rows` is [4][B][S]: per token the first
// and last token of its run, the first query that sees it as a key, and one plane of scratch.
// `summaries` is [4][B][S/128]: kv_lo, kv_hi, q_lo, q_hi.
CTB_API int ctb_attention_meta(const int* mask, const int* label, const int* att_end, int B, int S, int* seg, int* pos,
                               int* lim, int* rows, int* summaries, void* stream) {
  using namespace ctb;
  if (B <= 0 || S <= 0 || S % 128) return fail("attention_meta: S must be a positive multiple of 128");
  meta::Args a;
  a.mask = mask;
  a.label = label;
  a.att_end = att_end;
  a.seg = seg;
  a.pos = pos;
  a.lim = lim;
  a.rows = rows;
  const size_t n128 = static_cast<size_t>(B) * (S / 128);
  a.kv_lo = summaries;
  a.kv_hi = summaries + n128;
  a.q_lo = summaries + 2 * n128;
  a.q_hi = summaries + 3 * n128;
  a.S = S;
  meta::attention_meta_kernel<<<B, meta::THREADS, 0, static_cast<cudaStream_t>(stream)>>>(a);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}
