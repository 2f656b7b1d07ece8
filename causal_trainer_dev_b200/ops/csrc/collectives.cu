// In-kernel NVLink collectives of the FSDP runtime (sm_100a, peer-mapped symmetric memory).
//
//   ag_pull         all-gather by pull: a few CTAs copy every peer's parameter shard into this
//                   GPU's gathered buffer with 16-byte peer loads over NVLink and publish one
//                   flag per 128 KiB chunk (st.release).  The consuming tcgen05 GEMM (gemm.cu)
//                   acquires the flags of exactly the B rows a tile needs, so the transfer and
//                   the math overlap tile by tile with no stream-level dependency: together they
//                   are the fused all-gather -> GEMM.  Chunks are visited in an order rotated by
//                   rank (own shard first, then rank+1, ...) so every link is busy and the first
//                   tiles can start at once.
//   signal_peers    publishes "my gradient slot s holds epoch e" on every peer (st.release.sys).
//   rs_reduce       reduce-scatter by pull, fused with what follows it: waits (bounded) for the
//                   slot flags of all ranks, sums this rank's shard slice from every peer in fp32
//                   in a fixed order, adds the fp32 micro-batch accumulator, and on the last
//                   micro-batch rounds to the parameter dtype, emits per-CTA sums of squares for
//                   the global norm and -- when clipping is off -- applies AdamW in the same pass.
//   wait_flags      bounded device-side wait used where a stream must not run ahead of peers
//                   (slot reuse) or of the pull (vector parameters).
//
// Peer memory is only ever touched with plain ld/st (never TMA, never a library kernel).
// Every wait has a clock64() budget; on expiry the kernel records the site in the status
// word and returns.
//
// Reference counterpart: the collectives GSPMD inserts for FSDP weights and gradients
// (src/causal_trainer/distributed/runtime.py:334-360, src/causal_trainer/training/steps.py:200-208).
#include <cuda_bf16.h>

#include "host_common.h"

namespace ctb {
namespace coll {

constexpr int MAX_RANKS = 16;
// 256 threads and a register cap keep these CTAs small enough to share an SM with a
// resident tcgen05 GEMM CTA (256 threads x 168 registers, ~225 KiB shared memory), which is
// what lets the transfer overlap the math instead of queueing behind it.
constexpr int PULL_THREADS = 256;

struct PeerPtrs {
  const void* p[MAX_RANKS];
};
struct PeerFlagPtrs {
  unsigned* p[MAX_RANKS];
};

enum : unsigned {
  SITE_RS_WAIT = 0x0401,
  SITE_WAIT_FLAGS = 0x0402,
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

// ------------------------------------------------------------------------------------------
// all-gather by pull with per-chunk flags
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(PULL_THREADS, 4)
ag_pull_kernel(PeerPtrs shards, __nv_bfloat16* __restrict__ gathered, long shard_elems, int rank, int world,
               int chunk_elems, unsigned* __restrict__ flags, unsigned epoch) {
  const int chunks_per_shard = static_cast<int>(shard_elems / chunk_elems);
  const int total = chunks_per_shard * world;
  const int vec_per_chunk = chunk_elems / 8;
  // position -1 (CTA 0 only): the first chunk of shard 0 holds the norm scales and biases,
  // which the layer needs before any GEMM tile.
  for (int pos = (blockIdx.x == 0 ? -1 : static_cast<int>(blockIdx.x)); pos < total;
       pos = (pos < 0 ? 0 : pos + static_cast<int>(gridDim.x))) {
    int src, c;
    if (pos < 0) {
      src = 0;
      c = 0;
    } else {
      src = (rank + pos / chunks_per_shard) % world;
      c = pos % chunks_per_shard;
    }
    const uint4* from = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(shards.p[src]) +
                                                       static_cast<long>(c) * chunk_elems);
    uint4* to = reinterpret_cast<uint4*>(gathered + static_cast<long>(src) * shard_elems +
                                         static_cast<long>(c) * chunk_elems);
    // 8 x 16 B per thread in flight: a CTA keeps 64 KiB outstanding across the NVLink latency
    for (int v = threadIdx.x; v < vec_per_chunk; v += PULL_THREADS * 8) {
      uint4 r[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = v + u * PULL_THREADS;
        if (i < vec_per_chunk) r[u] = ld_peer(from + i);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = v + u * PULL_THREADS;
        if (i < vec_per_chunk) to[i] = r[u];
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      st_release_gpu(flags + src * chunks_per_shard + c, epoch);
    }
  }
}

// ------------------------------------------------------------------------------------------
// embedding rows straight from the shards that own them (all-gather + gather in one kernel)
// ------------------------------------------------------------------------------------------
// The embedding unit is a flat buffer cut into `world` equal shards; element e of the unit lives
// on rank e / shard_elems.  Each thread moves one 16-byte vector of one token's row with a plain
// peer load, so a step moves tokens x d elements over NVLink instead of the whole table.
__global__ void __launch_bounds__(PULL_THREADS)
embed_gather_peer_kernel(const int* __restrict__ ids, PeerPtrs shards, long shard_elems, long table_offset,
                         __nv_bfloat16* __restrict__ out, long T, int d, int vocab) {
  const int nvec = d / 8;
  const long total = T * nvec;
  constexpr int UNR = 4;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  for (long i0 = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i0 < total; i0 += stride * UNR) {
    uint4 r[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long i = i0 + u * stride;
      if (i < total) {
        const long t = i / nvec;
        const int v = static_cast<int>(i % nvec);
        int id = ids[t];
        id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
        const long e = table_offset + static_cast<long>(id) * d + static_cast<long>(v) * 8;
        const int src = static_cast<int>(e / shard_elems);
        r[u] = ld_peer(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(shards.p[src]) +
                                                      (e - static_cast<long>(src) * shard_elems)));
      }
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long i = i0 + u * stride;
      if (i < total) reinterpret_cast<uint4*>(out)[i] = r[u];
    }
  }
}

// ------------------------------------------------------------------------------------------
// flags: publish to peers / wait locally
// ------------------------------------------------------------------------------------------
__global__ void signal_peers_kernel(PeerFlagPtrs pads, int world, int index, unsigned epoch) {
  const int p = threadIdx.x;
  if (p < world) {
    __threadfence_system();
    st_release_sys(pads.p[p] + index, epoch);
  }
}

// Waits until flags[first + i*stride] >= epoch for i in [0, count).  Bounded.
__global__ void wait_flags_kernel(const unsigned* __restrict__ flags, int first, int stride, int count,
                                  unsigned epoch, long long budget, DeviceStatus* st) {
  const int i = threadIdx.x;
  if (i >= count) return;
  const unsigned* f = flags + first + static_cast<long>(i) * stride;
  const long long t0 = clock64();
  while (ld_acquire_sys(f) < epoch) {
    if (clock64() - t0 > budget) {
      report_failure(st, SITE_WAIT_FLAGS, static_cast<unsigned>(first + i * stride), epoch);
      return;
    }
    __nanosleep(100);
  }
}

// ------------------------------------------------------------------------------------------
// reduce-scatter by pull, fused with accumulate / cast / sum of squares / AdamW
// ------------------------------------------------------------------------------------------
struct RsArgs {
  PeerPtrs staging;            // every rank's gradient slot (bf16, full unit)
  long shard_offset;           // element offset of this rank's shard inside the unit
  long shard_elems;
  int world;
  const unsigned* ready;       // ready[slot_base + p] >= epoch: rank p's slot is complete
  int ready_base;
  unsigned epoch;
  float* accum;                // fp32 shard accumulator (may be null when one micro-batch per step)
  int accumulate_in;           // add the previous contents of accum
  int last;                    // last micro-batch: produce the final gradient
  __nv_bfloat16* grad_out;     // final gradient, parameter dtype (last only; may be null with adam)
  float* sumsq_partial;        // [gridDim.x * 8] per-warp sums of squares of the rounded gradient (last only)
  // fused AdamW (last && apply_adam)
  int apply_adam;
  __nv_bfloat16* param;
  __nv_bfloat16* m;
  __nv_bfloat16* v;
  long decay_from;             // elements at shard-local index >= decay_from get weight decay
  float lr, b1, b2, eps, decay, bc1, bc2;
  PeerFlagPtrs done_pads;      // where to publish "I have consumed slot" (may be all null)
  int done_index;
  unsigned* finish_counter;    // device counter to find the last CTA
  long long budget;
  DeviceStatus* status;
};

// Per-vector tail of the reduce: accumulate / cast / sum of squares / optional AdamW.
__device__ __forceinline__ void rs_finish_vector(const RsArgs& a, long v, float (&s)[8], float& sq) {
  if (a.accum != nullptr) {
    float4* acc = reinterpret_cast<float4*>(a.accum + v * 8);
    if (a.accumulate_in) {
      const float4 a0 = acc[0], a1 = acc[1];
      s[0] += a0.x; s[1] += a0.y; s[2] += a0.z; s[3] += a0.w;
      s[4] += a1.x; s[5] += a1.y; s[6] += a1.z; s[7] += a1.w;
    }
    if (!a.last) {
      acc[0] = make_float4(s[0], s[1], s[2], s[3]);
      acc[1] = make_float4(s[4], s[5], s[6], s[7]);
    }
  }
  if (!a.last) return;
  uint4 out;
  __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&out);
  float g[8];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    oh[e] = __floats2bfloat162_rn(s[2 * e], s[2 * e + 1]);
    const float2 back = __bfloat1622float2(oh[e]);
    g[2 * e] = back.x;
    g[2 * e + 1] = back.y;
    sq += back.x * back.x + back.y * back.y;
  }
  if (a.grad_out != nullptr) reinterpret_cast<uint4*>(a.grad_out)[v] = out;
  if (a.apply_adam) {
    uint4 pr = reinterpret_cast<const uint4*>(a.param)[v];
    uint4 mr = reinterpret_cast<const uint4*>(a.m)[v];
    uint4 vr = reinterpret_cast<const uint4*>(a.v)[v];
    __nv_bfloat16* pe = reinterpret_cast<__nv_bfloat16*>(&pr);
    __nv_bfloat16* me = reinterpret_cast<__nv_bfloat16*>(&mr);
    __nv_bfloat16* ve = reinterpret_cast<__nv_bfloat16*>(&vr);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float dec = (v * 8 + e >= a.decay_from) ? a.decay : 0.f;
      const float mi = a.b1 * __bfloat162float(me[e]) + (1.f - a.b1) * g[e];
      const float vi = a.b2 * __bfloat162float(ve[e]) + (1.f - a.b2) * g[e] * g[e];
      const float pi = __bfloat162float(pe[e]);
      const float upd = -a.lr * ((mi / a.bc1) / (sqrtf(vi / a.bc2) + a.eps) + dec * pi);
      me[e] = __float2bfloat16(mi);
      ve[e] = __float2bfloat16(vi);
      pe[e] = __float2bfloat16(pi + __bfloat162float(__float2bfloat16(upd)));
    }
    reinterpret_cast<uint4*>(a.param)[v] = pr;
    reinterpret_cast<uint4*>(a.m)[v] = mr;
    reinterpret_cast<uint4*>(a.v)[v] = vr;
  }
}

__global__ void __launch_bounds__(PULL_THREADS, 3)
rs_reduce_kernel(const RsArgs a) {
  // No shared memory (see PULL_THREADS): the verdict of the wait travels through the barrier and
  // the sums of squares leave the CTA as one partial per warp.
  int bad = 0;
  if (threadIdx.x < a.world) {
    const unsigned* f = a.ready + a.ready_base + threadIdx.x;
    const long long t0 = clock64();
    while (ld_acquire_sys(f) < a.epoch) {
      if (clock64() - t0 > a.budget) {
        report_failure(a.status, SITE_RS_WAIT, static_cast<unsigned>(threadIdx.x), a.epoch);
        bad = 1;
        break;
      }
      __nanosleep(100);
    }
  }
  const int give_up = __syncthreads_or(bad);
  float sq = 0.f;
  if (!give_up) {
    const long nvec = a.shard_elems / 8;
    constexpr int UNR = 4;  // vectors per thread per round: UNR * world peer loads in flight
    const long stride = static_cast<long>(gridDim.x) * PULL_THREADS;
    for (long v0 = blockIdx.x * static_cast<long>(PULL_THREADS) + threadIdx.x; v0 < nvec; v0 += stride * UNR) {
      float s[UNR][8];
#pragma unroll
      for (int u = 0; u < UNR; ++u)
#pragma unroll
        for (int e = 0; e < 8; ++e) s[u][e] = 0.f;
      for (int p = 0; p < a.world; ++p) {
        const uint4* base = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.staging.p[p]) +
                                                           a.shard_offset);
        uint4 raw[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const long v = v0 + u * stride;
          if (v < nvec) raw[u] = ld_peer(base + v);
          else raw[u] = make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f2 = __bfloat1622float2(h[e]);
            s[u][2 * e] += f2.x;
            s[u][2 * e + 1] += f2.y;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const long v = v0 + u * stride;
        if (v >= nvec) continue;
        rs_finish_vector(a, v, s[u], sq);
      }
    }
  }
  // per-warp sums of squares (the host adds the partials in a fixed order)
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  if ((threadIdx.x & 31) == 0 && a.sumsq_partial != nullptr)
    a.sumsq_partial[blockIdx.x * (PULL_THREADS / 32) + (threadIdx.x >> 5)] = a.last ? sq : 0.f;
  __syncthreads();
  if (threadIdx.x == 0) {
    // the last CTA to finish tells every peer that this rank no longer reads their slot
    __threadfence();
    const unsigned done = atomicAdd(a.finish_counter, 1u) + 1u;
    if (done == gridDim.x) {
      *a.finish_counter = 0u;
      __threadfence_system();
      for (int p = 0; p < a.world; ++p)
        if (a.done_pads.p[p] != nullptr) st_release_sys(a.done_pads.p[p] + a.done_index, a.epoch);
    }
  }
}

}  // namespace coll
}  // namespace ctb

using namespace ctb;
using namespace ctb::coll;

CTB_API int ctb_max_ranks() { return MAX_RANKS; }

CTB_API int ctb_ag_pull(const void* const* shard_ptrs, void* gathered, long shard_elems, int rank, int world,
                        int chunk_elems, unsigned* flags, unsigned epoch, int ctas, void* stream) {
  if (world > MAX_RANKS) return fail("ag_pull: too many ranks");
  if (chunk_elems % 8 || shard_elems % chunk_elems) return fail("ag_pull: shard must be a whole number of chunks");
  PeerPtrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = shard_ptrs[i];
  ag_pull_kernel<<<ctas, PULL_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      pp, static_cast<__nv_bfloat16*>(gathered), shard_elems, rank, world, chunk_elems, flags, epoch);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_signal_peers(unsigned* const* pad_ptrs, int world, int index, unsigned epoch, void* stream) {
  if (world > MAX_RANKS) return fail("signal_peers: too many ranks");
  PeerFlagPtrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = pad_ptrs[i];
  signal_peers_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pp, world, index, epoch);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_wait_flags(const unsigned* flags, int first, int stride, int count, unsigned epoch,
                           long long budget, void* stream) {
  if (count > 1024) return fail("wait_flags: at most 1024 flags per call");
  if (count <= 0) return 0;
  wait_flags_kernel<<<1, count < 32 ? 32 : ((count + 31) / 32) * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      flags, first, stride, count, epoch, budget > 0 ? budget : CTB_SPIN_BUDGET, device_status());
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// One call = the fused reduce-scatter step of one unit.  Pointers documented at RsArgs.
CTB_API int ctb_rs_reduce(const void* const* staging_ptrs, long shard_offset, long shard_elems, int world,
                          const unsigned* ready, int ready_base, unsigned epoch, float* accum, int accumulate_in,
                          int last, void* grad_out, float* sumsq_partial, int apply_adam, void* param, void* m,
                          void* v, long decay_from, float lr, float b1, float b2, float eps, float decay, float bc1,
                          float bc2, unsigned* const* done_pads, int done_index, unsigned* finish_counter, int ctas,
                          long long budget, void* stream) {
  if (world > MAX_RANKS) return fail("rs_reduce: too many ranks");
  if (shard_elems % 8 || shard_offset % 8) return fail("rs_reduce: shard must be 16-byte aligned");
  RsArgs a{};
  for (int i = 0; i < world; ++i) {
    a.staging.p[i] = staging_ptrs[i];
    a.done_pads.p[i] = done_pads ? done_pads[i] : nullptr;
  }
  a.shard_offset = shard_offset; a.shard_elems = shard_elems; a.world = world;
  a.ready = ready; a.ready_base = ready_base; a.epoch = epoch;
  a.accum = accum; a.accumulate_in = accumulate_in; a.last = last;
  a.grad_out = static_cast<__nv_bfloat16*>(grad_out); a.sumsq_partial = sumsq_partial;
  a.apply_adam = apply_adam; a.param = static_cast<__nv_bfloat16*>(param);
  a.m = static_cast<__nv_bfloat16*>(m); a.v = static_cast<__nv_bfloat16*>(v);
  a.decay_from = decay_from; a.lr = lr; a.b1 = b1; a.b2 = b2; a.eps = eps; a.decay = decay; a.bc1 = bc1; a.bc2 = bc2;
  a.done_index = done_index; a.finish_counter = finish_counter;
  a.budget = budget > 0 ? budget : CTB_SPIN_BUDGET; a.status = device_status();
  rs_reduce_kernel<<<ctas, PULL_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(a);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// out[t] = table[ids[t]] where the table starts `table_offset` elements into a unit that is split
// into `world` shards of `shard_elems` elements (shard_ptrs[r] = rank r's shard).
CTB_API int ctb_embed_gather_peer(const int* ids, const void* const* shard_ptrs, int world, long shard_elems,
                                  long table_offset, void* out, long T, int d, int vocab, void* stream) {
  if (world > MAX_RANKS) return fail("embed_gather_peer: too many ranks");
  if (d % 8 || shard_elems % 8 || table_offset % 8) return fail("embed_gather_peer: rows and shards must be 16-byte multiples");
  if (table_offset + static_cast<long>(vocab) * d > shard_elems * world) return fail("embed_gather_peer: table exceeds the unit");
  if (T <= 0) return 0;
  PeerPtrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = shard_ptrs[i];
  const long work = T * (d / 8);
  long blocks = (work + PULL_THREADS * 4 - 1) / (PULL_THREADS * 4);
  const long cap = static_cast<long>(sm_count()) * 4;
  if (blocks > cap) blocks = cap;
  embed_gather_peer_kernel<<<static_cast<unsigned>(blocks), PULL_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, pp, shard_elems, table_offset, static_cast<__nv_bfloat16*>(out), T, d, vocab);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}
