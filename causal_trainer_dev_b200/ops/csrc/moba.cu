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
