// In-kernel NVLink collectives of the tensor-parallel path (sm_100a, peer-mapped symmetric memory).
//
// Activations between the projections are sharded by token rows over the tp ranks (rank t owns
// rows [t*Rl, (t+1)*Rl) of every [R, d] activation).  The collectives around the projections are
// therefore an all-gather of rows in front of a column-parallel GEMM and a reduce-scatter of rows
// behind a row-parallel GEMM:
//
//   tp_ag_pull     all-gather by pull.  Every rank keeps a *symmetric* [R, d] buffer and writes
//                  its own rows in place (the producing RMSNorm does); this kernel waits (bounded)
//                  for each peer's "rows ready" flag, copies that peer's rows out of the peer's
//                  buffer with 16-byte loads over NVLink and publishes one flag per chunk.  The
//                  tcgen05 GEMM acquires the chunk flags of exactly the A rows a tile reads
//                  (gemm.cu, a_flags) and starts on the rows this rank already owns, so transfer
//                  and math overlap tile by tile: together they are the fused all-gather -> GEMM.
//   (GEMM push)    the reduce-scatter half lives in the GEMM epilogue (gemm.cu, GemmPush): each
//                  partial-sum tile is stored straight into the owner's receive buffer.
//   tp_reduce      waits (bounded) for the push flags of all sources and sums the world slabs of
//                  this rank's rows in fp32, in rank order (deterministic).
//   ce_exchange    cross-rank half of the vocab-parallel cut cross-entropy: folds this rank's
//                  per-slab (max, sum-exp) and target logit, stores the three per-row numbers
//                  into every peer's statistics buffer, publishes a flag, waits (bounded) for the
//                  peers and combines them into the global log-sum-exp, the weighted NLL and the
//                  backward coefficient -- one launch, no host round trip.
//   embed_push     vocab-parallel embedding lookup: the rank that owns a token's embedding row
//                  stores it into the residual-stream buffer of the rank that owns the token.
//
// Peer memory is only ever touched with plain ld/st.  Every wait has a clock64() budget; on
// expiry the kernel records the site in the status word and returns.
//
// Reference counterpart: token_tiling.py:60,126,244 (all_gather / psum_scatter over tp),
// cut_cross_entropy.py:503-511 (pmax/psum over tp), runtime.py:334-338 (tp shardings).
#include <cuda_bf16.h>

#include "host_common.h"

namespace ctb {
namespace tpc {

constexpr int MAX_RANKS = 16;
constexpr int THREADS = 256;

struct Ptrs {
  void* p[MAX_RANKS];
};

enum : unsigned {
  SITE_TP_AG_READY = 0x0501,
  SITE_TP_REDUCE = 0x0502,
  SITE_TP_CE = 0x0503,
};

__device__ __forceinline__ uint4 ld_peer(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait on one flag by thread 0 of the CTA; the verdict reaches every thread through the
// barrier itself.  No shared memory: a CTA of the pull kernel has to fit beside a resident
// tcgen05 GEMM CTA that owns nearly all of the SM's shared memory, or the GEMM would spin on
// flags that the pull can never get on the machine to publish.
__device__ __forceinline__ bool cta_wait_flag(const unsigned* f, unsigned epoch, long long budget, DeviceStatus* st,
                                              unsigned site, unsigned info) {
  int ok = 1;
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    while (ld_acquire_sys(f) < epoch) {
      if (clock64() - t0 > budget) {
        report_failure(st, site, info, epoch);
        ok = 0;
        break;
      }
      __nanosleep(64);
    }
  }
  return __syncthreads_and(ok) != 0;
}

// ------------------------------------------------------------------------------------------
// all-gather of token rows by pull, per-chunk flags for the consuming GEMM
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS, 4)
tp_ag_pull_kernel(Ptrs bufs, long slab_elems, int rank, int world, int chunk_elems, unsigned* __restrict__ flags,
                  unsigned epoch, const unsigned* __restrict__ ready, unsigned ready_epoch, long long budget,
                  DeviceStatus* st) {
  const int cps = static_cast<int>(slab_elems / chunk_elems);
  // own rows were written in place by the kernel before this one in stream order
  if (blockIdx.x == 0) {
    for (int c = threadIdx.x; c < cps; c += THREADS) st_release_gpu(flags + rank * cps + c, epoch);
  }
  const int total = cps * (world - 1);
  const int vec_per_chunk = chunk_elems / 8;
  __nv_bfloat16* mine = static_cast<__nv_bfloat16*>(bufs.p[rank]);
  int waited_src = -1;
  for (int pos = blockIdx.x; pos < total; pos += gridDim.x) {
    const int src = (rank + 1 + pos / cps) % world;
    const int c = pos % cps;
    if (src != waited_src) {
      if (!cta_wait_flag(ready + src, ready_epoch, budget, st, SITE_TP_AG_READY, static_cast<unsigned>(src)))
        return;
      waited_src = src;
    }
    const long off = static_cast<long>(src) * slab_elems + static_cast<long>(c) * chunk_elems;
    const uint4* from = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(bufs.p[src]) + off);
    uint4* to = reinterpret_cast<uint4*>(mine + off);
    for (int v = threadIdx.x; v < vec_per_chunk; v += THREADS * 8) {
      uint4 r[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = v + u * THREADS;
        if (i < vec_per_chunk) r[u] = ld_peer(from + i);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = v + u * THREADS;
        if (i < vec_per_chunk) to[i] = r[u];
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      st_release_gpu(flags + src * cps + c, epoch);
    }
  }
}

// ------------------------------------------------------------------------------------------
// sum of the pushed partial slabs: out[r][c] = sum_src recv[src][r][c]   (+ optional residual)
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS, 4)
tp_reduce_kernel(const __nv_bfloat16* __restrict__ recv, long slab_elems, int world,
                 const unsigned* __restrict__ flags, unsigned epoch, __nv_bfloat16* __restrict__ out,
                 long long budget, DeviceStatus* st) {
  int bad = 0;
  if (threadIdx.x < world) {
    const long long t0 = clock64();
    while (ld_acquire_sys(flags + threadIdx.x) < epoch) {
      if (clock64() - t0 > budget) {
        report_failure(st, SITE_TP_REDUCE, static_cast<unsigned>(threadIdx.x), epoch);
        bad = 1;
        break;
      }
      __nanosleep(64);
    }
  }
  if (__syncthreads_or(bad)) return;
  const long nvec = slab_elems / 8;
  const long stride = static_cast<long>(gridDim.x) * THREADS;
  for (long v = blockIdx.x * static_cast<long>(THREADS) + threadIdx.x; v < nvec; v += stride) {
    float s[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) s[e] = 0.f;
    for (int p = 0; p < world; ++p) {
      const uint4 raw = reinterpret_cast<const uint4*>(recv + static_cast<long>(p) * slab_elems)[v];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f2 = __bfloat1622float2(h[e]);
        s[2 * e] += f2.x;
        s[2 * e + 1] += f2.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(s[2 * e], s[2 * e + 1]);
    reinterpret_cast<uint4*>(out)[v] = o;
  }
}

// ------------------------------------------------------------------------------------------
// vocab-parallel cut-CE: local slab fold -> exchange over peer memory -> global combine
// stats buffer of every rank: [world sources][3][rows_cap] fp32
// ------------------------------------------------------------------------------------------
struct CeExchangeArgs {
  const float* pmax;
  const float* psum;
  int slabs;
  const float* target_logit;      // zero where the target lies in another rank's vocabulary slice
  const float* weights;
  float grad_scale;
  float* lse;
  float* coef;
  float* block_nll;
  float* block_w;
  int rows;
  int rows_cap;
  int rank, world;
  Ptrs stats;                     // every rank's statistics buffer
  Ptrs flag;                      // &pads_of_rank_p[base + rank]
  const unsigned* my_flags;       // &my_pads[base]
  unsigned epoch;
  unsigned* counter;
  long long budget;
  DeviceStatus* status;
};

__device__ __forceinline__ float block_sum_256(float v, float* scratch) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  if (threadIdx.x < 32) {
    t = threadIdx.x < THREADS / 32 ? scratch[threadIdx.x] : 0.f;
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  return t;  // valid in thread 0
}

__global__ void __launch_bounds__(THREADS, 2)
ce_exchange_kernel(const CeExchangeArgs a) {
  __shared__ float scratch[33];
  __shared__ int give_up;
  if (threadIdx.x == 0) give_up = 0;
  const long cap = a.rows_cap;
  // phase 1: fold this rank's slabs and store the row statistics into every rank's buffer
  for (int row = blockIdx.x * THREADS + threadIdx.x; row < a.rows; row += gridDim.x * THREADS) {
    float m = -INFINITY;
    for (int s = 0; s < a.slabs; ++s) m = fmaxf(m, a.pmax[static_cast<size_t>(s) * a.rows + row]);
    float acc = 0.f;
    for (int s = 0; s < a.slabs; ++s) {
      const size_t i = static_cast<size_t>(s) * a.rows + row;
      acc += a.psum[i] * __expf(a.pmax[i] - m);
    }
    const float tl = a.target_logit[row];
    for (int p = 0; p < a.world; ++p) {
      float* dst = static_cast<float*>(a.stats.p[p]) + static_cast<long>(a.rank) * 3 * cap;
      dst[row] = m;
      dst[cap + row] = acc;
      dst[2 * cap + row] = tl;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(a.counter, 1u) + 1u;
    if (done == gridDim.x) {
      *a.counter = 0u;
      __threadfence_system();
      for (int p = 0; p < a.world; ++p) st_release_sys(static_cast<unsigned*>(a.flag.p[p]), a.epoch);
    }
  }
  // phase 2: wait for every source, combine
  if (threadIdx.x < a.world) {
    const long long t0 = clock64();
    while (ld_acquire_sys(a.my_flags + threadIdx.x) < a.epoch) {
      if (clock64() - t0 > a.budget) {
        report_failure(a.status, SITE_TP_CE, static_cast<unsigned>(threadIdx.x), a.epoch);
        give_up = 1;
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  float nll = 0.f, w = 0.f;
  if (!give_up) {
    const float* mine = static_cast<const float*>(a.stats.p[a.rank]);
    for (int row = blockIdx.x * THREADS + threadIdx.x; row < a.rows; row += gridDim.x * THREADS) {
      float m = -INFINITY;
      for (int p = 0; p < a.world; ++p) m = fmaxf(m, mine[static_cast<long>(p) * 3 * cap + row]);
      float acc = 0.f, tl = 0.f;
      for (int p = 0; p < a.world; ++p) {
        const float* src = mine + static_cast<long>(p) * 3 * cap;
        acc += src[cap + row] * __expf(src[row] - m);
        tl += src[2 * cap + row];
      }
      const float l = m + logf(acc);
      a.lse[row] = l;
      const float wt = a.weights[row];
      a.coef[row] = wt * a.grad_scale;
      w += wt;
      nll += (wt != 0.f) ? (l - tl) * wt : 0.f;
    }
  }
  const float bn = block_sum_256(nll, scratch);
  const float bw = block_sum_256(w, scratch);
  if (threadIdx.x == 0) {
    a.block_nll[blockIdx.x] = bn;
    a.block_w[blockIdx.x] = bw;
  }
}

// ------------------------------------------------------------------------------------------
// vocab-parallel embedding lookup: the owner of the embedding row stores it at the owner of the token
// ------------------------------------------------------------------------------------------
__global__ void embed_push_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table, Ptrs out,
                                  long tokens, int d, int vocab, int vocab_lo, int vocab_rows, int rows_per_rank) {
  const int nvec = d / 8;
  const long total = tokens * nvec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = i / nvec;
    const int v = static_cast<int>(i % nvec);
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const int local = id - vocab_lo;
    if (local < 0 || local >= vocab_rows) continue;
    const int dest = static_cast<int>(t / rows_per_rank);
    const long row = t - static_cast<long>(dest) * rows_per_rank;
    reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(out.p[dest]) + row * d)[v] =
        reinterpret_cast<const uint4*>(table + static_cast<long>(local) * d)[v];
  }
}

// ------------------------------------------------------------------------------------------
// Embedding backward, deterministic: token gradients are summed per embedding row over runs of a
// stable sort of the ids (one CTA per run, fixed order, fp32) and added to the gradient table.
// Rows outside [vocab_lo, vocab_lo + vocab_rows) and the padding row are skipped.
// ------------------------------------------------------------------------------------------
template <typename G>
__global__ void embedding_backward_kernel(const int* __restrict__ sorted_ids, const int* __restrict__ perm,
                                          const int* __restrict__ run_start, int n_runs, long tokens,
                                          const __nv_bfloat16* __restrict__ dout, G* __restrict__ grad, int d,
                                          int vocab_lo, int vocab_rows, int pad_id) {
  for (int run = blockIdx.x; run < n_runs; run += gridDim.x) {
    const long s0 = run_start[run];
    const long s1 = (run + 1 < n_runs) ? run_start[run + 1] : tokens;
    const int id = sorted_ids[s0];
    const int local = id - vocab_lo;
    if (id == pad_id || local < 0 || local >= vocab_rows) continue;
    for (int c = threadIdx.x * 2; c < d; c += blockDim.x * 2) {
      float a0 = 0.f, a1 = 0.f;
      for (long s = s0; s < s1; ++s) {
        const float2 f = __bfloat1622float2(
            *reinterpret_cast<const __nv_bfloat162*>(dout + static_cast<long>(perm[s]) * d + c));
        a0 += f.x;
        a1 += f.y;
      }
      G* g = grad + static_cast<long>(local) * d + c;
      g[0] = static_cast<G>(static_cast<float>(g[0]) + a0);
      g[1] = static_cast<G>(static_cast<float>(g[1]) + a1);
    }
  }
}

}  // namespace tpc
}  // namespace ctb

using namespace ctb;
using namespace ctb::tpc;

CTB_API int ctb_tp_ag_pull(void* const* buf_ptrs, long slab_elems, int rank, int world, int chunk_elems,
                           unsigned* flags, unsigned epoch, const unsigned* ready, unsigned ready_epoch, int ctas,
                           long long budget, void* stream) {
  if (world > MAX_RANKS) return fail("tp_ag_pull: too many ranks");
  if (chunk_elems % 8 || slab_elems % chunk_elems) return fail("tp_ag_pull: slab must be a whole number of chunks");
  Ptrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = buf_ptrs[i];
  tp_ag_pull_kernel<<<ctas, THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      pp, slab_elems, rank, world, chunk_elems, flags, epoch, ready, ready_epoch, budget > 0 ? budget : CTB_SPIN_BUDGET,
      device_status());
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_tp_reduce(const void* recv, long slab_elems, int world, const unsigned* flags, unsigned epoch,
                          void* out, int ctas, long long budget, void* stream) {
  if (world > MAX_RANKS) return fail("tp_reduce: too many ranks");
  if (slab_elems % 8) return fail("tp_reduce: slab must be 16-byte aligned");
  tp_reduce_kernel<<<ctas, THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(recv), slab_elems, world, flags, epoch, static_cast<__nv_bfloat16*>(out),
      budget > 0 ? budget : CTB_SPIN_BUDGET, device_status());
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_ce_exchange_blocks(int rows) {
  const int want = (rows + THREADS - 1) / THREADS;
  const int cap = sm_count();
  return want < cap ? want : cap;
}

// block_nll / block_w must hold ctb_ce_exchange_blocks(rows) floats each.
CTB_API int ctb_ce_exchange(const float* pmax, const float* psum, int slabs, const float* target_logit,
                            const float* weights, float grad_scale, float* lse, float* coef, float* block_nll,
                            float* block_w, int rows, int rows_cap, int rank, int world, void* const* stats_ptrs,
                            unsigned* const* flag_ptrs, const unsigned* my_flags, unsigned epoch, unsigned* counter,
                            long long budget, void* stream) {
  if (world > MAX_RANKS) return fail("ce_exchange: too many ranks");
  if (rows > rows_cap) return fail("ce_exchange: more rows than the statistics buffers hold");
  CeExchangeArgs a{};
  a.pmax = pmax; a.psum = psum; a.slabs = slabs; a.target_logit = target_logit; a.weights = weights;
  a.grad_scale = grad_scale; a.lse = lse; a.coef = coef; a.block_nll = block_nll; a.block_w = block_w;
  a.rows = rows; a.rows_cap = rows_cap; a.rank = rank; a.world = world;
  for (int i = 0; i < world; ++i) {
    a.stats.p[i] = stats_ptrs[i];
    a.flag.p[i] = flag_ptrs[i];
  }
  a.my_flags = my_flags; a.epoch = epoch; a.counter = counter;
  a.budget = budget > 0 ? budget : CTB_SPIN_BUDGET; a.status = device_status();
  ce_exchange_kernel<<<ctb_ce_exchange_blocks(rows), THREADS, 0, static_cast<cudaStream_t>(stream)>>>(a);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_embed_push(const int* ids, const void* table, void* const* out_ptrs, int world, long tokens, int d,
                           int vocab, int vocab_lo, int vocab_rows, int rows_per_rank, void* stream) {
  if (world > MAX_RANKS) return fail("embed_push: too many ranks");
  if (d % 8) return fail("embed_push: hidden size must be a multiple of 8");
  Ptrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = out_ptrs[i];
  const long work = tokens * (d / 8);
  long blocks = (work + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  embed_push_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, static_cast<const __nv_bfloat16*>(table), pp, tokens, d, vocab, vocab_lo, vocab_rows, rows_per_rank);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_embedding_backward(const int* sorted_ids, const int* perm, const int* run_start, int n_runs,
                                   long tokens, const void* dout, void* grad, int grad_f32, int d, int vocab_lo,
                                   int vocab_rows, int pad_id, void* stream) {
  if (n_runs <= 0) return 0;
  if (d % 2) return fail("embedding_backward: hidden size must be even");
  const int grid = n_runs < 148 * 8 ? n_runs : 148 * 8;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (grad_f32)
    embedding_backward_kernel<float><<<grid, 256, 0, s>>>(sorted_ids, perm, run_start, n_runs, tokens,
                                                         static_cast<const __nv_bfloat16*>(dout),
                                                         static_cast<float*>(grad), d, vocab_lo, vocab_rows, pad_id);
  else
    embedding_backward_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(
        sorted_ids, perm, run_start, n_runs, tokens, static_cast<const __nv_bfloat16*>(dout),
        static_cast<__nv_bfloat16*>(grad), d, vocab_lo, vocab_rows, pad_id);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}
