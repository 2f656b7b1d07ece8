// MoBA routing kernels for sm_100a: block mean-pool of the keys and the top-k block router.
//
// Keys are cut into blocks of `block` tokens counted from the start of their document.  A block
// is *complete* when all of its tokens exist inside the document.  Complete blocks are at least
// 128 tokens long and cannot overlap, so no two of them start inside the same 128-token tile:
// the pooled key of the block that starts at token p is stored at tile p / 128.
//
//   moba_pool    pooled[b][tile][hkv][:] = mean over the block's tokens of K (fp32), and
//                pool_start[b][tile] = p (or -1 when no complete block starts in the tile).
//   moba_route   for every (token i, query head h): scores q_i . pooled(block c) for the blocks
//                c < current(i) of i's document, keeps the top_k - 1 best (ties: lower block
//                first), and writes the selection bit mask (bit c; the query's own block is
//                always set) that the block-sparse flash kernels consume.
//
// Reference counterparts: moba_block_pool (src/causal_trainer/kernels/grouped_moba.py:275-324)
// and the router (grouped_moba.py:346-371, modeling/approximate_attention.py:46-73).
#include <cuda_bf16.h>

#include "host_common.h"

namespace ctb {
namespace moba {

constexpr int POOL_THREADS = 256;

// grid: (S/128, Hkv, B).  seg holds canonical run ids (0 = padding), doc_start the first token of
// each token's document.
template <int D>
__global__ void __launch_bounds__(POOL_THREADS)
moba_pool_kernel(const __nv_bfloat16* __restrict__ k, long k_row_stride, const int* __restrict__ seg,
                 const int* __restrict__ doc_start, int S, int Hkv, int block, float* __restrict__ pooled,
                 int* __restrict__ pool_start) {
  constexpr int VEC = D / 8;                    // 16-byte vectors per row
  constexpr int ROWS = POOL_THREADS / VEC;      // rows summed per pass
  __shared__ int s_p;
  __shared__ float red[ROWS][D];
  const int tile = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int ntile = S / 128;
  if (threadIdx.x == 0) s_p = -1;
  __syncthreads();
  if (threadIdx.x < 128) {
    const int p = tile * 128 + threadIdx.x;
    const int sg = seg[b * S + p];
    if (sg != 0 && (p - doc_start[b * S + p]) % block == 0 && p + block - 1 < S &&
        seg[b * S + p + block - 1] == sg)
      s_p = p;                                  // at most one thread qualifies
  }
  __syncthreads();
  const int p = s_p;
  if (hkv == 0 && threadIdx.x == 0) pool_start[b * ntile + tile] = p;
  float* out = pooled + ((static_cast<size_t>(b) * ntile + tile) * Hkv + hkv) * D;
  if (p < 0) {
    for (int c = threadIdx.x; c < D; c += POOL_THREADS) out[c] = 0.f;
    return;
  }
  const int v = threadIdx.x % VEC, rg = threadIdx.x / VEC;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  const __nv_bfloat16* base = k + (static_cast<size_t>(b) * S + p) * k_row_stride + static_cast<size_t>(hkv) * D + v * 8;
  for (int r = rg; r < block; r += ROWS) {
    const uint4 raw = *reinterpret_cast<const uint4*>(base + static_cast<size_t>(r) * k_row_stride);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h2[e]);
      acc[2 * e] += f.x;
      acc[2 * e + 1] += f.y;
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red[rg][v * 8 + e] = acc[e];
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += POOL_THREADS) {
    float t = 0.f;
    for (int g = 0; g < ROWS; ++g) t += red[g][c];   // fixed order: deterministic
    out[c] = t / static_cast<float>(block);
  }
}

// One warp per (token, query head).  sel is [B][Hq][S][words].
template <int D>
__global__ void __launch_bounds__(256)
moba_route_kernel(const __nv_bfloat16* __restrict__ q, long q_row_stride, const float* __restrict__ pooled,
                  const int* __restrict__ pool_start, const int* __restrict__ seg,
                  const int* __restrict__ doc_start, int B, int S, int Hq, int Hkv, int block, int top_k, int words,
                  unsigned* __restrict__ sel) {
  const long warp_id = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long total = static_cast<long>(B) * S * Hq;
  if (warp_id >= total) return;
  const int h = static_cast<int>(warp_id % Hq);
  const long t = warp_id / Hq;
  const int b = static_cast<int>(t / S), i = static_cast<int>(t % S);
  unsigned* out = sel + ((static_cast<size_t>(b) * Hq + h) * S + i) * words;
  const int sg = seg[b * S + i];
  if (sg == 0) {
    for (int w = lane; w < words; w += 32) out[w] = 0u;
    return;
  }
  const int start = doc_start[b * S + i];
  const int cur = (i - start) / block;
  const int hkv = h / (Hq / Hkv);
  const int ntile = S / 128;
  constexpr int PER = D / 32;                    // elements of the head dimension per lane
  float qv[PER];
  const __nv_bfloat16* qp = q + (static_cast<size_t>(b) * S + i) * q_row_stride + static_cast<size_t>(h) * D + lane * PER;
#pragma unroll
  for (int e = 0; e < PER; ++e) qv[e] = __bfloat162float(qp[e]);
  // lane r < top_k - 1 holds the r-th best (score, block) seen so far
  float held = -INFINITY;
  int held_id = -1;
  const int keep = top_k - 1;
  for (int c = 0; c < cur && keep > 0; ++c) {
    const int p = start + c * block;
    const int tile = p >> 7;
    float s = 0.f;
    if (pool_start[b * ntile + tile] == p) {
      const float* pk = pooled + ((static_cast<size_t>(b) * ntile + tile) * Hkv + hkv) * D + lane * PER;
#pragma unroll
      for (int e = 0; e < PER; ++e) s += qv[e] * pk[e];
    }
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    // insert: position = number of held scores that rank ahead (>= keeps earlier blocks first on ties)
    const unsigned ahead = __ballot_sync(0xffffffffu, lane < keep && held >= s);
    const int pos = __popc(ahead);
    const float up = __shfl_up_sync(0xffffffffu, held, 1);
    const int up_id = __shfl_up_sync(0xffffffffu, held_id, 1);
    if (lane > pos) {
      held = up;
      held_id = up_id;
    } else if (lane == pos) {
      held = s;
      held_id = c;
    }
  }
  // bit mask: own block + kept blocks
  for (int w = 0; w < words; ++w) {
    unsigned bits = 0u;
    if (lane < keep && held_id >= 0 && (held_id >> 5) == w) bits = 1u << (held_id & 31);
    for (int o = 16; o > 0; o >>= 1) bits |= __shfl_xor_sync(0xffffffffu, bits, o);
    if ((cur >> 5) == w) bits |= 1u << (cur & 31);
    if (lane == 0) out[w] = bits;
  }
}

}  // namespace moba
}  // namespace ctb

using namespace ctb;

// k: [B,S,Hkv,D] view with row stride (elements per token); pooled: [B,S/128,Hkv,D] fp32;
// pool_start: [B,S/128] int32.
CTB_API int ctb_moba_pool(const void* k, long k_row_stride, const int* seg, const int* doc_start, int B, int S,
                          int Hkv, int D, int block, float* pooled, int* pool_start, void* stream) {
  if (S % 128 || block < 128) return fail("moba_pool: S must be a multiple of 128 and block >= 128");
  dim3 grid(S / 128, Hkv, B);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* kp = static_cast<const __nv_bfloat16*>(k);
  if (D == 128)
    moba::moba_pool_kernel<128><<<grid, moba::POOL_THREADS, 0, s>>>(kp, k_row_stride, seg, doc_start, S, Hkv, block,
                                                                    pooled, pool_start);
  else if (D == 64)
    moba::moba_pool_kernel<64><<<grid, moba::POOL_THREADS, 0, s>>>(kp, k_row_stride, seg, doc_start, S, Hkv, block,
                                                                   pooled, pool_start);
  else
    return fail("moba_pool: head_dim must be 64 or 128");
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// q: [B,S,Hq,D] view with row stride; sel: [B,Hq,S,words] uint32 (every word is written).
CTB_API int ctb_moba_route(const void* q, long q_row_stride, const float* pooled, const int* pool_start,
                           const int* seg, const int* doc_start, int B, int S, int Hq, int Hkv, int D, int block,
                           int top_k, int words, unsigned* sel, void* stream) {
  if (top_k < 1 || top_k > 32) return fail("moba_route: top_k must be in [1, 32]");
  if (words * 32 * static_cast<long>(block) < S) return fail("moba_route: selection mask too narrow for S / block");
  const long warps = static_cast<long>(B) * S * Hq;
  const long blocks = (warps * 32 + 255) / 256;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* qp = static_cast<const __nv_bfloat16*>(q);
  if (D == 128)
    moba::moba_route_kernel<128><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        qp, q_row_stride, pooled, pool_start, seg, doc_start, B, S, Hq, Hkv, block, top_k, words, sel);
  else if (D == 64)
    moba::moba_route_kernel<64><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        qp, q_row_stride, pooled, pool_start, seg, doc_start, B, S, Hq, Hkv, block, top_k, words, sel);
  else
    return fail("moba_route: head_dim must be 64 or 128");
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------
// Work lists of the block-sparse flash kernels, built on the GPU without a host round trip.
//
//   moba_touch    per (batch, head, 64-query block): a bitmap over the 64-key blocks that at least
//                 one of its rows selected (own block up to the diagonal included), and the AND of
//                 the rows' selection masks (padding rows count as all ones).
//   moba_lists    per CTA of the flash kernels (a warp per work item): the ascending list of
//                 candidates whose bit is set, at a fixed stride, plus its length:
//                   mode 0  forward      item (query pair descending, batch, head)      -> 128-key tiles
//                   mode 1  dQ           item (query tile descending, batch, head)      -> 64-key blocks
//                   mode 2  dK/dV        item (key tile ascending, batch, kv head)      -> (head in group << 24) | 64-query block
//
// Reference counterpart: the query grouping of the Pallas path (stable argsort by block id,
// padded groups, src/causal_trainer/kernels/grouped_moba.py:25-57).
// ------------------------------------------------------------------------------------------
namespace ctb {
namespace moba {

constexpr int MAX_TOUCH_WORDS = 128;   // 64-key blocks per row / 32: sequences up to 262144 tokens
constexpr int MAX_SEL_WORDS = 64;      // selection words per row: up to 2048 blocks per document

// grid (S/64, Hq, B), 64 threads.  touch: [B][Hq][S/64][tw] words, tw = S/64/32 rounded up.
__global__ void __launch_bounds__(64)
moba_touch_kernel(const unsigned* __restrict__ sel, const int* __restrict__ seg, const int* __restrict__ doc_start,
                  int S, int Hq, int block, int words, int tw, unsigned* __restrict__ touch,
                  unsigned* __restrict__ allsel) {
  __shared__ unsigned bits[MAX_TOUCH_WORDS];
  __shared__ unsigned all_and[MAX_SEL_WORDS];
  const int q64 = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  for (int w = threadIdx.x; w < tw; w += 64) bits[w] = 0u;
  if (threadIdx.x < words) all_and[threadIdx.x] = 0xffffffffu;
  __syncthreads();
  const int i = q64 * 64 + threadIdx.x;
  const int sg = seg[b * S + i];
  const unsigned* my = sel + ((static_cast<size_t>(b) * Hq + h) * S + i) * words;
  if (sg != 0) {
    const int start = doc_start[b * S + i];
    for (int w = 0; w < words; ++w) {
      unsigned m = my[w];
      atomicAnd(&all_and[w], m);
      while (m) {
        const int c = w * 32 + __ffs(m) - 1;
        m &= m - 1;
        const int lo = start + c * block;
        if (lo > i) continue;
        const int hi = min(lo + block - 1, i);
        int k0 = lo >> 6;
        const int k1 = hi >> 6;
        while (k0 <= k1) {                         // set bits k0..k1, one word at a time
          const int word = k0 >> 5;
          const int last = min(k1, word * 32 + 31);
          const unsigned from = 0xffffffffu << (k0 & 31);
          const unsigned upto = 0xffffffffu >> (31 - (last & 31));
          atomicOr(&bits[word], from & upto);
          k0 = last + 1;
        }
      }
    }
  }
  __syncthreads();
  unsigned* out = touch + ((static_cast<size_t>(b) * Hq + h) * (S / 64) + q64) * tw;
  for (int w = threadIdx.x; w < tw; w += 64) out[w] = bits[w];
  if (threadIdx.x < words)
    allsel[((static_cast<size_t>(b) * Hq + h) * (S / 64) + q64) * words + threadIdx.x] =
        all_and[threadIdx.x];
}

// One warp per work item; 8 warps per CTA.
__global__ void __launch_bounds__(256)
moba_lists_kernel(int mode, const unsigned* __restrict__ touch, int B, int S, int Hq, int Hkv, int tw, int items,
                  int stride, int* __restrict__ list, int* __restrict__ count) {
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const int nb64 = S / 64, nb128 = S / 128;
  int* out = list + static_cast<size_t>(item) * stride;
  int n = 0;
  auto row = [&](int b, int h, int q64) -> const unsigned* {
    return touch + ((static_cast<size_t>(b) * Hq + h) * nb64 + q64) * tw;
  };
  if (mode == 0 || mode == 1) {
    const int per = mode == 0 ? (S + 255) / 256 : nb128;          // query groups per (b, h)
    const int h = item % Hq;
    const int b = (item / Hq) % B;
    const int grp = per - 1 - item / (Hq * B);
    const int rows = mode == 0 ? 4 : 2;                            // 64-query blocks per group
    const int cand = mode == 0 ? nb128 : nb64;
    for (int c0 = 0; c0 < cand; c0 += 32) {
      const int c = c0 + lane;
      bool hit = false;
      if (c < cand) {
        for (int r = 0; r < rows; ++r) {
          const int q64 = grp * rows + r;
          if (q64 >= nb64) break;
          const unsigned* t = row(b, h, q64);
          if (mode == 0) {
            const int k64 = 2 * c;                                  // two 64-key blocks per 128-key tile
            hit = hit || ((t[k64 >> 5] >> (k64 & 31)) & 3u);
          } else {
            hit = hit || ((t[c >> 5] >> (c & 31)) & 1u);
          }
        }
      }
      const unsigned mask = __ballot_sync(0xffffffffu, hit);
      if (hit) out[n + __popc(mask & ((1u << lane) - 1u))] = c;
      n += __popc(mask);
    }
  } else {
    const int g = Hq / Hkv;
    const int hkv = item % Hkv;
    const int b = (item / Hkv) % B;
    const int kt = item / (Hkv * B);
    const int k64 = 2 * kt;
    const int cand = g * nb64;
    for (int c0 = 0; c0 < cand; c0 += 32) {
      const int c = c0 + lane;
      bool hit = false;
      if (c < cand) {
        const int gi = c / nb64, q64 = c % nb64;
        const unsigned* t = row(b, hkv * g + gi, q64);
        hit = ((t[k64 >> 5] >> (k64 & 31)) & 3u) != 0u;
      }
      const unsigned mask = __ballot_sync(0xffffffffu, hit);
      if (hit) out[n + __popc(mask & ((1u << lane) - 1u))] = ((c / nb64) << 24) | (c % nb64);
      n += __popc(mask);
    }
  }
  if (lane == 0) count[item] = n;
}

}  // namespace moba
}  // namespace ctb

// touch: [B][Hq][S/64][tw] words with tw = ceil(S/64/32); allsel: [B][Hq][S/64][words].
CTB_API int ctb_moba_touch(const unsigned* sel, const int* seg, const int* doc_start, int B, int S, int Hq, int block,
                           int words, int tw, unsigned* touch, unsigned* allsel, void* stream) {
  if (S % 128 || block < 128) return fail("moba_touch: S must be a multiple of 128 and block >= 128");
  if (tw > moba::MAX_TOUCH_WORDS || tw * 32 < S / 64) return fail("moba_touch: sequence too long for the touch bitmap");
  if (words > moba::MAX_SEL_WORDS) return fail("moba_touch: at most 2048 blocks per document");
  dim3 grid(S / 64, Hq, B);
  moba::moba_touch_kernel<<<grid, 64, 0, static_cast<cudaStream_t>(stream)>>>(sel, seg, doc_start, S, Hq, block, words,
                                                                            tw, touch, allsel);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// list: [items][stride] int32, count: [items].  Items and strides per mode: see moba_lists above.
CTB_API int ctb_moba_lists(int mode, const unsigned* touch, int B, int S, int Hq, int Hkv, int tw, int items,
                           int stride, int* list, int* count, void* stream) {
  if (mode < 0 || mode > 2) return fail("moba_lists: mode must be 0, 1 or 2");
  if (items <= 0) return 0;
  moba::moba_lists_kernel<<<(items + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(mode, touch, B, S, Hq, Hkv, tw,
                                                                                       items, stride, list, count);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------
// Query grouping: cost proportional to the routing budget.
//
// A *group* is one complete key block of one (batch, kv head): (b, hkv, first key ks).  Every
// (token, query head) row that selected the block joins the group; the rows of a group are laid
// out next to each other in a gathered row space, groups one after another, each padded with zero
// rows to a multiple of 256.  The history part of MoBA is then dense, unmasked attention of each
// group's rows against its block (attention_fwd.cu / attention_bwd.cu, GroupArgs), and the own
// block of every query is a separate causal pass; moba_merge combines the partial softmaxes by
// their log-sum-exp.  The placement is a stable counting sort written without atomics, so that the
// order of the rows inside a group (and with it every floating-point sum over a group) is a pure
// function of the routing:
//
//   moba_rank    gives every row that selected block c of its document its rank among such rows of
//                the same (document, head) and leaves the count in cnt[group][head in group]:
//                moba_rank_scan_kernel, one CTA per (batch, head, c), a segmented scan over the
//                sequence (default); moba_rank_kernel, one warp per (batch, head, c) walking the
//                sequence (CTB_MOBA_RANK=walk; same result, kept for comparison).
//   moba_groups  one CTA: exclusive scan of the padded group sizes -> first row of every group,
//                offsets of the heads inside a group, the compact list of non-empty groups.
//   moba_desc    descriptors of the CTAs of the grouped flash kernels.
//   moba_fill    gathered position of every (row, pick) and its inverse.
//
// Reference counterpart: group_queries and its inverse permutation
// (src/causal_trainer/kernels/grouped_moba.py:25-57).
// ------------------------------------------------------------------------------------------
namespace ctb {
namespace moba {

__global__ void __launch_bounds__(256)
moba_rank_kernel(const unsigned* __restrict__ sel, const int* __restrict__ seg, const int* __restrict__ doc_start,
                 int B, int S, int Hq, int Hkv, int block, int words, int nblk, int picks,
                 int* __restrict__ rank, int* __restrict__ cnt) {
  const long warp_id = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long total = static_cast<long>(B) * Hq * nblk;
  if (warp_id >= total) return;
  const int c = static_cast<int>(warp_id % nblk);
  const int h = static_cast<int>((warp_id / nblk) % Hq);
  const int b = static_cast<int>(warp_id / nblk / Hq);
  const int gsize = Hq / Hkv;
  const int hkv = h / gsize, hg = h % gsize;
  const int nt128 = S / 128;
  const int word = c >> 5;
  const unsigned below = (1u << (c & 31)) - 1u;
  int carry_start = -1, carry_count = 0;
  for (int i0 = 0; i0 < S; i0 += 32) {
    const int i = i0 + lane;
    const int sg = seg[b * S + i];
    const int st = doc_start[b * S + i];
    const int cur = (i - st) / block;
    const unsigned* mine = sel + ((static_cast<size_t>(b) * Hq + h) * S + i) * words;
    const unsigned w = (sg != 0 && word < words) ? __ldg(mine + word) : 0u;
    const bool picked = sg != 0 && c < cur && ((w >> (c & 31)) & 1u);
    const unsigned peers = __match_any_sync(0xffffffffu, st);
    const unsigned pk = __ballot_sync(0xffffffffu, picked);
    const unsigned mates = peers & pk;
    const int my_rank = __popc(mates & ((1u << lane) - 1u)) + (st == carry_start ? carry_count : 0);
    if (picked) {
      int j = __popc(w & below);                       // earlier picks of this row: its slot for block c
      for (int x = 0; x < word; ++x) j += __popc(__ldg(mine + x));
      if (j < picks) rank[((static_cast<size_t>(b) * Hq + h) * S + i) * picks + j] = my_rank;
      if ((mates >> lane) == 1u) {                     // last picked row of this document in the chunk
        const int g = (b * Hkv + hkv) * nt128 + ((st + c * block) >> 7);
        cnt[g * gsize + hg] = my_rank + 1;             // later chunks overwrite with the larger count
      }
    }
    const int last_start = __shfl_sync(0xffffffffu, st, 31);
    const unsigned last_mates = __shfl_sync(0xffffffffu, mates, 31);
    const int add = __popc(last_mates);
    carry_count = (last_start == carry_start ? carry_count : 0) + add;
    carry_start = last_start;
  }
}

// The same ranks computed by one CTA per (batch, head, block index): every thread owns a contiguous
// span of the sequence and the spans are joined by a segmented scan keyed by the document, so the
// depth is S / 1024 + log(1024) steps instead of S / 32.  The result is identical to the walk above
// (ranks count earlier picked rows of the same document and head), so the grouping stays a pure
// function of the routing; the group counts are left by atomicMax (cnt is zero before the launch).
struct RankSpan {
  int head;    // document key of the span's first token
  int tail;    // document key of its last token
  int cnt;     // picked rows among the trailing tokens that share `tail`
  int flags;   // bit 0: every token of the span has the same key; bit 1: empty span
};
__device__ __forceinline__ RankSpan join_spans(const RankSpan& a, const RankSpan& b) {
  if (b.flags & 2) return a;
  if (a.flags & 2) return b;
  RankSpan r;
  r.head = a.head;
  r.tail = b.tail;
  if ((b.flags & 1) && b.head == a.tail) {
    r.cnt = a.cnt + b.cnt;
    r.flags = a.flags & 1;
  } else {
    r.cnt = b.cnt;
    r.flags = 0;
  }
  return r;
}
__device__ __forceinline__ RankSpan shfl_up_span(const RankSpan& v, int delta) {
  RankSpan r;
  r.head = __shfl_up_sync(0xffffffffu, v.head, delta);
  r.tail = __shfl_up_sync(0xffffffffu, v.tail, delta);
  r.cnt = __shfl_up_sync(0xffffffffu, v.cnt, delta);
  r.flags = __shfl_up_sync(0xffffffffu, v.flags, delta);
  return r;
}

__global__ void __launch_bounds__(1024)
moba_rank_scan_kernel(const unsigned* __restrict__ sel, const int* __restrict__ seg, const int* __restrict__ doc_start,
                      int B, int S, int Hq, int Hkv, int block, int words, int nblk, int picks,
                      int* __restrict__ rank, int* __restrict__ cnt) {
  __shared__ RankSpan s_warp[32];
  const int c = static_cast<int>(blockIdx.x % nblk);
  const int h = static_cast<int>((blockIdx.x / nblk) % Hq);
  const int b = static_cast<int>(blockIdx.x / nblk / Hq);
  if (b >= B) return;
  const int gsize = Hq / Hkv;
  const int hkv = h / gsize, hg = h % gsize;
  const int nt128 = S / 128;
  const int word = c >> 5;
  const unsigned bit = 1u << (c & 31);
  const unsigned below = bit - 1u;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int per = (S + 1023) / 1024;
  const int i0 = min(S, t * per), i1 = min(S, i0 + per);
  const size_t row_base = (static_cast<size_t>(b) * Hq + h) * S;
  auto key_of = [&](int i) { return seg[b * S + i] != 0 ? doc_start[b * S + i] : -1; };
  auto picked_at = [&](int i, int key, unsigned* w_out) {
    if (key < 0 || word >= words) return false;
    const unsigned w = __ldg(sel + (row_base + i) * words + word);
    *w_out = w;
    return c < (i - key) / block && (w & bit) != 0u;
  };

  // pass 1: the span's summary
  RankSpan mine;
  mine.head = mine.tail = -2;
  mine.cnt = 0;
  mine.flags = 2;
  if (i0 < i1) {
    mine.head = key_of(i0);
    mine.tail = mine.head;
    mine.flags = 1;
    for (int i = i0; i < i1; ++i) {
      const int key = key_of(i);
      if (key != mine.tail) {
        mine.tail = key;
        mine.cnt = 0;
        mine.flags = 0;
      }
      unsigned w;
      if (picked_at(i, key, &w)) ++mine.cnt;
    }
  }
  // inclusive scan over the CTA's spans: lanes, then warps
  RankSpan incl = mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const RankSpan up = shfl_up_span(incl, d);
    if (lane >= d) incl = join_spans(up, incl);
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    RankSpan w = s_warp[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const RankSpan up = shfl_up_span(w, d);
      if (lane >= d) w = join_spans(up, w);
    }
    s_warp[lane] = w;
  }
  __syncthreads();
  RankSpan before;                                  // everything left of this thread's span
  before.head = before.tail = -2;
  before.cnt = 0;
  before.flags = 2;
  if (warp > 0) before = s_warp[warp - 1];
  {
    const RankSpan left = shfl_up_span(incl, 1);    // lanes before this one, within the warp
    if (lane > 0) before = join_spans(before, left);
  }
  if (i0 >= i1) return;

  // pass 2: ranks of this span's picked rows
  int run_key = mine.head;
  int run = (!(before.flags & 2) && before.tail == run_key) ? before.cnt : 0;
  int last_rank = -1;
  auto close_run = [&]() {
    if (last_rank >= 0) {
      const int g = (b * Hkv + hkv) * nt128 + ((run_key + c * block) >> 7);
      atomicMax(cnt + g * gsize + hg, last_rank + 1);
    }
    last_rank = -1;
  };
  for (int i = i0; i < i1; ++i) {
    const int key = key_of(i);
    if (key != run_key) {
      close_run();
      run_key = key;
      run = 0;
    }
    unsigned w = 0u;
    if (picked_at(i, key, &w)) {
      const unsigned* row_words = sel + (row_base + i) * words;
      int j = __popc(w & below);                       // earlier picks of this row: its slot for block c
      for (int x = 0; x < word; ++x) j += __popc(__ldg(row_words + x));
      if (j < picks) rank[(row_base + i) * picks + j] = run;
      last_rank = run;
      ++run;
    }
  }
  close_run();
}

// ginfo[slot] = (batch | hkv << 16, first key, first gathered row, rows incl. padding); greal[slot] = real rows;
// totals[0] = gathered rows in use, totals[1] = non-empty groups.
__global__ void __launch_bounds__(1024)
moba_groups_kernel(const int* __restrict__ cnt, const int* __restrict__ pool_start, int G, int gsize, int Hkv,
                   int nt128, int* __restrict__ row0, int* __restrict__ hoff, int4* __restrict__ ginfo,
                   int* __restrict__ greal, int* __restrict__ totals, int slot_cap) {
  __shared__ int s_rows[1024];
  __shared__ int s_slots[1024];
  const int t = threadIdx.x;
  const int per = (G + 1023) / 1024;
  const int g_lo = t * per, g_hi = min(G, g_lo + per);
  int rows = 0, slots = 0;
  for (int g = g_lo; g < g_hi; ++g) {
    int r = 0;
    for (int x = 0; x < gsize; ++x) r += cnt[g * gsize + x];
    if (r > 0) {
      rows += (r + 255) & ~255;
      ++slots;
    }
  }
  s_rows[t] = rows;
  s_slots[t] = slots;
  __syncthreads();
  // inclusive scan over the 1024 partial sums (Hillis-Steele, two values)
  for (int off = 1; off < 1024; off <<= 1) {
    const int a = t >= off ? s_rows[t - off] : 0;
    const int c = t >= off ? s_slots[t - off] : 0;
    __syncthreads();
    s_rows[t] += a;
    s_slots[t] += c;
    __syncthreads();
  }
  int row = s_rows[t] - rows, slot = s_slots[t] - slots;
  for (int g = g_lo; g < g_hi; ++g) {
    int r = 0;
    for (int x = 0; x < gsize; ++x) {
      hoff[g * gsize + x] = r;
      r += cnt[g * gsize + x];
    }
    row0[g] = row;
    if (r > 0) {
      const int padded = (r + 255) & ~255;
      if (slot < slot_cap) {
        const int tile = g % nt128, hkv = (g / nt128) % Hkv, b = g / nt128 / Hkv;
        ginfo[slot] = make_int4(b | (hkv << 16), pool_start[b * nt128 + tile], row, padded);
        greal[slot] = r;
      }
      row += padded;
      ++slot;
    }
  }
  if (t == 1023) {
    totals[0] = s_rows[1023];
    totals[1] = min(s_slots[1023], slot_cap);
  }
}

__global__ void moba_desc_kernel(const int4* __restrict__ ginfo, const int* __restrict__ greal,
                                 const int* __restrict__ totals, int tiles128_cap, int slot_cap, int block_tiles,
                                 int4* __restrict__ fwd_desc, int4* __restrict__ dq_desc, int4* __restrict__ dkv_desc) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int total_rows = totals[0], n_slots = totals[1];
  if (idx < tiles128_cap) {
    const int row = idx * 128;
    int4 d = make_int4(0, 0, 0, 0);
    int real_left = 0;
    if (row < total_rows) {
      int lo = 0, hi = n_slots - 1;                 // last slot whose first row is <= row
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (ginfo[mid].z <= row) lo = mid; else hi = mid - 1;
      }
      const int4 gi = ginfo[lo];
      real_left = greal[lo] - (row - gi.z);
      d = make_int4(gi.x, gi.y, 0, max(0, min(128, real_left)));
    }
    dq_desc[idx] = d;
    if ((idx & 1) == 0) {
      d.w = max(0, min(256, real_left));
      fwd_desc[idx >> 1] = d;
    }
  }
  const int k = idx - tiles128_cap;
  if (k >= 0 && k < slot_cap * block_tiles) {
    const int slot = k / block_tiles, t = k % block_tiles;
    int4 d = make_int4(0, 0, 0, 0);
    if (slot < n_slots) {
      const int4 gi = ginfo[slot];
      d = make_int4(gi.x, gi.y + t * 128, gi.z, gi.w);
    }
    dkv_desc[k] = d;
  }
}

// One thread per (batch, head, token): gathered position of each of its picks.
__global__ void moba_fill_kernel(const unsigned* __restrict__ sel, const int* __restrict__ seg,
                                 const int* __restrict__ doc_start, const int* __restrict__ rank,
                                 const int* __restrict__ row0, const int* __restrict__ hoff, int B, int S, int Hq,
                                 int Hkv, int block, int words, int picks, int rows_cap, DeviceStatus* status,
                                 int* __restrict__ row_of, int* __restrict__ pos_of) {
  const long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x;
  const long total = static_cast<long>(B) * Hq * S;
  if (idx >= total) return;
  const int i = static_cast<int>(idx % S);
  const int h = static_cast<int>((idx / S) % Hq);
  const int b = static_cast<int>(idx / S / Hq);
  const int gsize = Hq / Hkv;
  const int hkv = h / gsize, hg = h % gsize;
  const int nt128 = S / 128;
  int* out = pos_of + idx * picks;
  int j = 0;
  const int sg = seg[b * S + i];
  if (sg != 0) {
    const int st = doc_start[b * S + i];
    const int cur = (i - st) / block;
    for (int w = 0; w < words && j < picks; ++w) {
      unsigned bits = sel[idx * words + w];
      while (bits != 0u && j < picks) {
        const int c = w * 32 + (__ffs(bits) - 1);
        bits &= bits - 1u;
        if (c >= cur) continue;
        const int g = (b * Hkv + hkv) * nt128 + ((st + c * block) >> 7);
        const int pos = row0[g] + hoff[g * gsize + hg] + rank[idx * picks + j];
        if (pos < 0 || pos >= rows_cap) {
          // cannot happen when the capacities match the routing; recorded instead of written out of bounds
          report_failure(status, 0x0603u, static_cast<unsigned>(idx), static_cast<unsigned>(pos));
          out[j] = -1;
          ++j;
          continue;
        }
        out[j] = pos;
        row_of[pos] = (b * S + i) * Hq + h;
        ++j;
      }
    }
  }
  for (; j < picks; ++j) out[j] = -1;
}

// Copies the rows named by row_of (token * Hq + head, -1 = padding -> zeros) into the gathered
// space: bf16 rows of D elements from a [B,S,Hq,D] view, and optionally two per-row fp32 statistics
// stored [B,Hq,S].  D / 8 threads per row; only the rows in use (totals[0]) are written.
template <int D>
__global__ void __launch_bounds__(256)
moba_gather_kernel(const int* __restrict__ row_of, const int* __restrict__ totals, const __nv_bfloat16* __restrict__ src,
                   long row_stride, int S, int Hq, __nv_bfloat16* __restrict__ dst, const float* __restrict__ stat_a,
                   const float* __restrict__ stat_b, float* __restrict__ out_a, float* __restrict__ out_b) {
  constexpr int TPR = D / 8;
  const int total_rows = totals[0];
  const long stride = static_cast<long>(gridDim.x) * blockDim.x / TPR;
  const int v = threadIdx.x % TPR;
  for (long pos = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) / TPR; pos < total_rows; pos += stride) {
    const int id = row_of[pos];
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    float a = 0.f, bb = 0.f;
    if (id >= 0) {
      const int h = id % Hq;
      const long tok = id / Hq;
      if (src != nullptr)
        val = *reinterpret_cast<const uint4*>(src + tok * row_stride + static_cast<long>(h) * D + v * 8);
      if (v == 0 && stat_a != nullptr) {
        const long at = (tok / S * Hq + h) * S + tok % S;
        a = stat_a[at];
        bb = stat_b[at];
      }
    }
    if (dst != nullptr) reinterpret_cast<uint4*>(dst + pos * D)[v] = val;
    if (v == 0 && out_a != nullptr) {
      out_a[pos] = a;
      out_b[pos] = bb;
    }
  }
}

// Combines the own-block partial softmax (o, lse: in place) with the partials of the picks.
template <int D>
__global__ void __launch_bounds__(256)
moba_merge_fwd_kernel(__nv_bfloat16* __restrict__ o, long o_row_stride, float* __restrict__ lse,
                      const __nv_bfloat16* __restrict__ og, const float* __restrict__ lse_g,
                      const int* __restrict__ pos_of, int B, int S, int Hq, int picks) {
  constexpr int TPR = D / 8;
  const long row = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) / TPR;   // (b, h, i) order of pos_of
  const int v = threadIdx.x % TPR;
  if (row >= static_cast<long>(B) * Hq * S) return;
  const int* mine = pos_of + row * picks;
  if (mine[0] < 0) return;                             // no history: the own-block result is final
  const int i = static_cast<int>(row % S);
  const int h = static_cast<int>((row / S) % Hq);
  const long tok = row / S / Hq * S + i;
  __nv_bfloat16* op = o + tok * o_row_stride + static_cast<long>(h) * D + v * 8;
  const float l0 = lse[row];
  float m = l0;
  for (int j = 0; j < picks; ++j) {
    const int p = mine[j];
    if (p >= 0) m = fmaxf(m, lse_g[p]);
  }
  float acc[8];
  float wsum = __expf(l0 - m);
  {
    const uint4 raw = *reinterpret_cast<const uint4*>(op);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h2[e]);
      acc[2 * e] = f.x * wsum;
      acc[2 * e + 1] = f.y * wsum;
    }
  }
  for (int j = 0; j < picks; ++j) {
    const int p = mine[j];
    if (p < 0) continue;
    const float w = __expf(lse_g[p] - m);
    wsum += w;
    const uint4 raw = reinterpret_cast<const uint4*>(og + static_cast<long>(p) * D)[v];
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h2[e]);
      acc[2 * e] += f.x * w;
      acc[2 * e + 1] += f.y * w;
    }
  }
  const float inv = 1.f / wsum;
  uint4 out;
  __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e] * inv, acc[2 * e + 1] * inv);
  *reinterpret_cast<uint4*>(op) = out;
  if (v == 0) lse[row] = m + __logf(wsum);
}

// dq[b, i, h, :] += sum over the row's picks of dqg[pos].
template <int D>
__global__ void __launch_bounds__(256)
moba_merge_dq_kernel(__nv_bfloat16* __restrict__ dq, long dq_row_stride, const __nv_bfloat16* __restrict__ dqg,
                     const int* __restrict__ pos_of, int B, int S, int Hq, int picks) {
  constexpr int TPR = D / 8;
  const long row = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) / TPR;
  const int v = threadIdx.x % TPR;
  if (row >= static_cast<long>(B) * Hq * S) return;
  const int* mine = pos_of + row * picks;
  if (mine[0] < 0) return;
  const int i = static_cast<int>(row % S);
  const int h = static_cast<int>((row / S) % Hq);
  const long tok = row / S / Hq * S + i;
  __nv_bfloat16* dp = dq + tok * dq_row_stride + static_cast<long>(h) * D + v * 8;
  float acc[8];
  {
    const uint4 raw = *reinterpret_cast<const uint4*>(dp);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h2[e]);
      acc[2 * e] = f.x;
      acc[2 * e + 1] = f.y;
    }
  }
  for (int j = 0; j < picks; ++j) {
    const int p = mine[j];
    if (p < 0) continue;
    const uint4 raw = reinterpret_cast<const uint4*>(dqg + static_cast<long>(p) * D)[v];
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h2[e]);
      acc[2 * e] += f.x;
      acc[2 * e + 1] += f.y;
    }
  }
  uint4 out;
  __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
  *reinterpret_cast<uint4*>(dp) = out;
}

}  // namespace moba
}  // namespace ctb

// Grouping of the routed (token, head) rows by selected key block.  Sizes: G = B * Hkv * S / 128
// potential groups, slot_cap = B * Hkv * ceil(S / block) non-empty ones at most, rows_cap gathered
// rows (a multiple of 256, >= B * Hq * S * picks + 256 * slot_cap).  Buffers (all device, int32):
//   rank [B,Hq,S,picks]  cnt [G, Hq/Hkv]  row0 [G]  hoff [G, Hq/Hkv]  ginfo [slot_cap] int4  greal [slot_cap]
//   totals [2]  fwd_desc [rows_cap/256] int4  dq_desc [rows_cap/128] int4  dkv_desc [slot_cap * block/128] int4
//   row_of [rows_cap]  pos_of [B,Hq,S,picks]
CTB_API int ctb_moba_group(const unsigned* sel, const int* seg, const int* doc_start, const int* pool_start, int B,
                           int S, int Hq, int Hkv, int block, int words, int picks, int rows_cap, int slot_cap,
                           int* rank, int* cnt, int* row0, int* hoff, void* ginfo, int* greal, int* totals,
                           void* fwd_desc, void* dq_desc, void* dkv_desc, int* row_of, int* pos_of, void* stream) {
  if (S % 128 || block % 128 || block < 128) return fail("moba_group: S and the block must be multiples of 128");
  if (picks < 1 || Hq % Hkv) return fail("moba_group: needs at least one pick per row and Hq a multiple of Hkv");
  if (rows_cap % 256 || B > 0xffff || Hkv > 0x7fff) return fail("moba_group: sizes out of range");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int gsize = Hq / Hkv, nt128 = S / 128, G = B * Hkv * nt128;
  const int nblk = (S + block - 1) / block;
  CTB_CUDA_OK(cudaMemsetAsync(cnt, 0, sizeof(int) * static_cast<size_t>(G) * gsize, s));
  CTB_CUDA_OK(cudaMemsetAsync(row_of, 0xff, sizeof(int) * static_cast<size_t>(rows_cap), s));
  const long warps = static_cast<long>(B) * Hq * nblk;
  // CTB_MOBA_RANK=walk selects the one-warp-per-(head, block) walk; the default is the CTA-wide scan
  static const bool walk = [] {
    const char* e = std::getenv("CTB_MOBA_RANK");
    return e != nullptr && e[0] == 'w';
  }();
  if (walk || warps > 0x7fffffffL)
    moba::moba_rank_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, s>>>(
        sel, seg, doc_start, B, S, Hq, Hkv, block, words, nblk, picks, rank, cnt);
  else
    moba::moba_rank_scan_kernel<<<static_cast<unsigned>(warps), 1024, 0, s>>>(
        sel, seg, doc_start, B, S, Hq, Hkv, block, words, nblk, picks, rank, cnt);
  CTB_CUDA_OK(cudaGetLastError());
  moba::moba_groups_kernel<<<1, 1024, 0, s>>>(cnt, pool_start, G, gsize, Hkv, nt128, row0, hoff,
                                              static_cast<int4*>(ginfo), greal, totals, slot_cap);
  CTB_CUDA_OK(cudaGetLastError());
  const int tiles128 = rows_cap / 128, block_tiles = block / 128;
  const int work = tiles128 + slot_cap * block_tiles;
  moba::moba_desc_kernel<<<(work + 255) / 256, 256, 0, s>>>(static_cast<const int4*>(ginfo), greal, totals, tiles128,
                                                           slot_cap, block_tiles, static_cast<int4*>(fwd_desc),
                                                           static_cast<int4*>(dq_desc), static_cast<int4*>(dkv_desc));
  CTB_CUDA_OK(cudaGetLastError());
  const long rows = static_cast<long>(B) * Hq * S;
  moba::moba_fill_kernel<<<static_cast<unsigned>((rows + 255) / 256), 256, 0, s>>>(
      sel, seg, doc_start, rank, row0, hoff, B, S, Hq, Hkv, block, words, picks, rows_cap, device_status(), row_of, pos_of);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// dst[pos] = src[row_of[pos]] (bf16 rows of a [B,S,Hq,D] view; may be null) and, when stat_a is
// given, out_a / out_b [pos] = stat_a / stat_b [B,Hq,S]; padding rows become zero.
CTB_API int ctb_moba_gather(const int* row_of, const int* totals, const void* src, long row_stride, int S, int Hq,
                            int D, void* dst, const float* stat_a, const float* stat_b, float* out_a, float* out_b,
                            int rows_cap, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = ctb::sm_count() * 8;
  const __nv_bfloat16* sp = static_cast<const __nv_bfloat16*>(src);
  __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(dst);
  if (D == 128)
    moba::moba_gather_kernel<128><<<grid, 256, 0, s>>>(row_of, totals, sp, row_stride, S, Hq, dp, stat_a, stat_b, out_a, out_b);
  else if (D == 64)
    moba::moba_gather_kernel<64><<<grid, 256, 0, s>>>(row_of, totals, sp, row_stride, S, Hq, dp, stat_a, stat_b, out_a, out_b);
  else
    return fail("moba_gather: head_dim must be 64 or 128");
  (void)rows_cap;
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_moba_merge_fwd(void* o, long o_row_stride, float* lse, const void* og, const float* lse_g,
                               const int* pos_of, int B, int S, int Hq, int D, int picks, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long threads = static_cast<long>(B) * Hq * S * (D / 8);
  const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
  if (D == 128)
    moba::moba_merge_fwd_kernel<128><<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(o), o_row_stride, lse,
                                                          static_cast<const __nv_bfloat16*>(og), lse_g, pos_of, B, S, Hq, picks);
  else if (D == 64)
    moba::moba_merge_fwd_kernel<64><<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(o), o_row_stride, lse,
                                                         static_cast<const __nv_bfloat16*>(og), lse_g, pos_of, B, S, Hq, picks);
  else
    return fail("moba_merge: head_dim must be 64 or 128");
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_moba_merge_dq(void* dq, long dq_row_stride, const void* dqg, const int* pos_of, int B, int S, int Hq,
                              int D, int picks, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long threads = static_cast<long>(B) * Hq * S * (D / 8);
  const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
  if (D == 128)
    moba::moba_merge_dq_kernel<128><<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(dq), dq_row_stride,
                                                         static_cast<const __nv_bfloat16*>(dqg), pos_of, B, S, Hq, picks);
  else if (D == 64)
    moba::moba_merge_dq_kernel<64><<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(dq), dq_row_stride,
                                                        static_cast<const __nv_bfloat16*>(dqg), pos_of, B, S, Hq, picks);
  else
    return fail("moba_merge: head_dim must be 64 or 128");
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}
