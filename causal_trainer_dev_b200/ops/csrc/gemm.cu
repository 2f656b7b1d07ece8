// Persistent, warp-specialised bf16 GEMM for sm_100a:  C[M,N] (+)= A[M,K] * B[N,K]^T.
//
//   * 128x256 output tile per CTA, K step 64, UMMA 128x256x16 (tcgen05.mma, cta_group::1)
//   * operands staged by TMA (tiled, 128-byte swizzle) through a 4-stage mbarrier ring
//   * fp32 accumulators in TMEM, double buffered (2 x 256 columns) so the epilogue of
//     tile i overlaps the main loop of tile i+1
//   * epilogue: tcgen05.ld -> registers -> swizzled smem staging -> TMA store / reduce-add
//
// Operand layouts (row-major storage, `ld` in elements):
//   A "K-major":  A[M][K]  (activations in the forward pass)       a_mn = 0
//   A "MN-major": A[K][M]  (dY^T in the weight gradient)           a_mn = 1
//   B "K-major":  B[N][K]  (nn.Linear weight [out,in] forward)     b_mn = 0
//   B "MN-major": B[K][N]  (weight [out,in] in dX = dY W, X in dW) b_mn = 1
//
// Epilogues: plain store (bf16 / fp32, optional bias, optional accumulate through TMA
// reduce-add), cut-cross-entropy statistics (online max / sum-exp / target logit per row,
// logits never leave the SM), and cut-cross-entropy dlogits ((softmax - onehot) * coef).
//
// The B operand may be a buffer that other CTAs (the all-gather pull of the FSDP path)
// are still filling: with `b_flags` set, the producer acquires one flag per `b_flag_rows`
// rows of B before issuing the TMA load of a tile (bounded wait).
//
// Counterpart in the reference: XLA dot_general behind `linear`
// (src/causal_trainer/modeling/architecture.py:186-202) and the Pallas cut-CE kernels
// (src/causal_trainer/kernels/cut_cross_entropy.py:85-156, 225-278).
#include "gemm.h"

#include <algorithm>
#include <cstdlib>

#ifndef CTB_TAIL_SPLIT_DEFAULT
#define CTB_TAIL_SPLIT_DEFAULT 0
#endif

namespace ctb {
namespace gemm {

constexpr int BM = 128;            // rows of one UMMA accumulator (one TMEM slot)
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int B_STAGE = BN * BK * 2;   // 32 KiB
constexpr int EPI_BUF = 128 * 128;     // 128 rows x 128 B
constexpr int TQ = 4;                  // depth of the tile-index queue

// Cycles producer warps spent waiting for chunk flags of gathered operands, summed over CTAs
// since the last read (ctb_gemm_flag_wait_cycles): the exposed part of an all-gather -> GEMM.
__device__ unsigned long long g_flag_wait_cycles = 0ull;

// A CTA tile is TM row sub-tiles of 128 rows that share one B tile:
//   TM = 1: 128 x 256 tiles, 4 pipeline stages of 48 KiB, the two 256-column TMEM slots double-
//           buffer the accumulator (the epilogue of tile i overlaps the main loop of tile i+1);
//   TM = 2: 256 x 256 tiles, 3 stages of 64 KiB.  Each B k-block feeds two UMMAs, so a CTA reads a
//           third fewer operand bytes per FLOP from L2 and the same 192 KiB of stages cover 1.5x
//           as many tensor-core cycles of load latency; both TMEM slots belong to one tile and two
//           epilogue warpgroups drain them at the tile's end.
template <int TM>
struct Cfg {
  static constexpr int BMT = BM * TM;
  static constexpr int NSTAGE = TM == 1 ? 4 : 3;
  static constexpr int A_STAGE = BMT * BK * 2;
  static constexpr int OFF_B = NSTAGE * A_STAGE;
  static constexpr int OFF_EPI = OFF_B + NSTAGE * B_STAGE;
  static constexpr int OFF_BAR = OFF_EPI + 2 * EPI_BUF;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;  // + barrier block + alignment slack
  static constexpr int THREADS = 128 + 128 * TM;           // 4 service warps + TM epilogue warpgroups
  static constexpr int GROUP_M = 16 / TM;                  // tiles per band: 2048 rows either way
  static constexpr int EPI_BUFS = 2 / TM;                  // staging buffers per epilogue warpgroup
  // Declared thread capacity: caps registers (168 / 128 per thread) so that a 256-thread, 64-register
  // pull or reduce CTA always fits beside a resident GEMM CTA (a GEMM that waits on flags would
  // otherwise starve the kernel that publishes them).
  static constexpr int BOUND = TM == 1 ? 384 : 512;
};

enum : unsigned {
  SITE_PRODUCER_EMPTY = 0x0101,
  SITE_MMA_FULL = 0x0102,
  SITE_MMA_TEMPTY = 0x0103,
  SITE_EPI_TFULL = 0x0104,
  SITE_PRODUCER_FLAG = 0x0105,
  SITE_DRAIN = 0x0106,
  SITE_TILE_QUEUE = 0x0107,
};

struct TileCoord {
  int m0, n0;
};

// Tiles are walked in bands of GROUP_M row tiles; inside a band the column tile advances
// slowly so the B tile stays hot in L2.  `n_rotate` shifts the column order so that a rank
// starts on the weight rows it already owns while the all-gather pull brings the rest.
// `m_rotate` does the same for row tiles when the A operand is being gathered.
// A work unit is a whole output tile, or one K slice of a tile whose slices reduce-add into C.
//   split_k > 1   every tile is cut into split_k slices (unit = slice * tiles + tile);
//   tail_splits   only the tiles [tail_first, tiles) -- the ones a last, mostly empty wave of CTAs
//                 would compute -- are cut, into tail_splits slices each, so that the last wave
//                 is as full as the others and only those few tiles pay reduce traffic.
struct UnitMap {
  int tile;      // output tile index
  int kb0, kb1;  // k-block range of this unit
  bool reduce;   // the unit adds into C instead of storing
};
__device__ __forceinline__ UnitMap map_unit(int unit, int total, int num_k, int splits, int k_per, int tail_first,
                                            int tail_splits, int tail_k_per) {
  UnitMap u;
  if (tail_splits > 1) {
    if (unit < tail_first) {
      u.tile = unit;
      u.kb0 = 0;
      u.kb1 = num_k;
      u.reduce = false;
    } else {
      const int v = unit - tail_first;
      u.tile = tail_first + v / tail_splits;
      u.kb0 = (v % tail_splits) * tail_k_per;
      u.kb1 = min(num_k, u.kb0 + tail_k_per);
      u.reduce = true;
    }
  } else {
    u.tile = unit % total;
    u.kb0 = (unit / total) * k_per;
    u.kb1 = min(num_k, u.kb0 + k_per);
    u.reduce = splits > 1;
  }
  return u;
}

template <int TM>
__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int num_n, int n_rotate, int m_rotate) {
  constexpr int GROUP_M = Cfg<TM>::GROUP_M;
  const int per_group = GROUP_M * num_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int rows = min(GROUP_M, num_m - first_m);
  const int local = tile - group * per_group;
  int n = local / rows + n_rotate;
  if (n >= num_n) n -= num_n;
  int m = first_m + local % rows + m_rotate;
  if (m >= num_m) m -= num_m;
  TileCoord c;
  c.m0 = m * Cfg<TM>::BMT;
  c.n0 = n * BN;
  return c;
}

// Copies a staged 128 x 128 B block (128-byte swizzle) to `out` (row stride `ld` elements) with
// 16-byte stores: thread -> (row etid/8 + 16*i, 16-byte column etid%8), so a warp writes four
// full 128 B rows per step.  Kept out of line so its address arithmetic does not raise the
// register count of the whole kernel.
__device__ __noinline__ void push_block(const uint8_t* buf, __nv_bfloat16* out, long ld, int etid, int rows_left,
                                        int cols_left) {
  const int j = etid & 7;
  if (j * 8 >= cols_left) return;
  out += static_cast<long>(etid >> 3) * ld + j * 8;
#pragma unroll 4
  for (int i = 0; i < 8; ++i) {
    const int r = (etid >> 3) + i * 16;
    if (r < rows_left)
      *reinterpret_cast<uint4*>(out + static_cast<long>(i) * 16 * ld) =
          *reinterpret_cast<const uint4*>(buf + sw128_offset(r, j));
  }
}

template <int TM, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(Cfg<TM>::BOUND, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const __grid_constant__ CUtensorMap map_c, const GemmArgs args) {
  using C = Cfg<TM>;
  constexpr int NSTAGE = C::NSTAGE;
  constexpr int A_STAGE = C::A_STAGE;
  constexpr int BMT = C::BMT;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* empty = full + NSTAGE;
  uint64_t* tfull = empty + NSTAGE;      // [2] TMEM slot s holds a finished accumulator
  uint64_t* tempty = tfull + 2;          // [2] TMEM slot s has been drained
  uint64_t* tq_full = tempty + 2;        // tile queue: the producer hands tile indices
  uint64_t* tq_empty = tq_full + TQ;     // to the MMA and epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tq_empty + TQ);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile int* tile_ring = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (args.M + BMT - 1) / BMT;
  const int num_n = (args.N + BN - 1) / BN;
  const int num_k = (args.K + BK - 1) / BK;
  const int total = num_m * num_n;
  // Split-K: a work unit is (tile, K slice); every slice adds its partial product into C with a
  // TMA reduce, so a problem with few output tiles still fills all SMs in whole waves.
  const int splits = args.split_k > 1 ? args.split_k : 1;
  const int k_per = (num_k + splits - 1) / splits;
  const int tail_splits = (splits == 1 && args.tail_splits > 1) ? args.tail_splits : 1;
  const int tail_first = tail_splits > 1 ? args.tail_first : total;
  const int tail_k_per = (num_k + tail_splits - 1) / tail_splits;
  const int units = tail_splits > 1 ? tail_first + (total - tail_first) * tail_splits : total * splits;
  const int m_rot = args.m_rotate / TM < num_m ? args.m_rotate / TM : 0;   // given in 128-row units
  DeviceStatus* st = args.status;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    for (int t = 0; t < TQ; ++t) {
      mbar_init(&tq_full[t], 1);
      mbar_init(&tq_empty[t], 1 + 4 * TM);    // MMA thread + one lane of each epilogue warp
    }
    *abort_flag = 0u;
    mbar_fence_init();
  }
  if (warp == 3 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if (EPI != EPI_CE_STATS && EPI != EPI_PUSH) tma_prefetch_desc(&map_c);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // All 32 lanes take part in the flag acquisition (one chunk flag per lane per round);
    // lane 0 alone arms the barriers and issues the copies.
    uint32_t stage = 0, phase = 0;
    uint32_t armed = 0;      // bit s set: full[s] was armed by this thread at least once
    uint32_t armed_par = 0;  // bit s: parity of the phase last armed on full[s]
    bool ok = true;
    bool b_all_seen = false, a_all_seen = false;
    // Acquires every chunk flag covering elements [e0, e1) of a gathered buffer (warp-wide).
    auto acquire_range = [&](const unsigned* flags, long chunk, long e0, long e1, unsigned epoch) -> bool {
      const int first = static_cast<int>(e0 / chunk);
      const int last = static_cast<int>((e1 - 1) / chunk);
      bool mine = true;
      for (int f = first + lane; mine && f <= last; f += 32) {
        const long long t0 = clock64();
        while (true) {
          unsigned v;
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + f) : "memory");
          if (v >= epoch) break;
          if (*abort_flag || clock64() - t0 > args.spin_budget) {
            *abort_flag = 1u;
            report_failure(st, SITE_PRODUCER_FLAG, static_cast<unsigned>(f), epoch);
            mine = false;
            break;
          }
          __nanosleep(64);
        }
      }
      return __all_sync(0xffffffffu, mine);
    };
    uint32_t tq = 0, tq_phase = 0;
    // Tile order: static round-robin (tile = blockIdx.x + i * gridDim.x), or, with
    // args.dynamic_tiles, claimed from a global counter one claim ahead (the atomic for tile i+1
    // is in flight while the loads of tile i are issued, so its latency never drains the TMA
    // ring).  Either way the producer hands the index to the other warps through the tile queue.
    auto claim = [&](int previous) -> int {
      if (args.dynamic_tiles) return atomicAdd(args.tile_counter, 1);
      return previous < 0 ? static_cast<int>(blockIdx.x) : previous + static_cast<int>(gridDim.x);
    };
    int pending = (lane == 0) ? claim(-1) : 0;
    while (ok) {
      int tile = -1;
      if (lane == 0) {
        if (mbar_wait(&tq_empty[tq], tq_phase ^ 1u, abort_flag, st, SITE_TILE_QUEUE, args.spin_budget)) {
          tile = pending < units ? pending : -1;
          if (tile >= 0) pending = claim(pending);
          tile_ring[tq] = tile;
          mbar_arrive(&tq_full[tq]);
        } else {
          tile = -2;
        }
      }
      tile = __shfl_sync(0xffffffffu, tile, 0);
      if (++tq == TQ) {
        tq = 0;
        tq_phase ^= 1u;
      }
      if (tile < 0) {
        ok = (tile == -1);
        break;
      }
      const UnitMap um = map_unit(tile, total, num_k, splits, k_per, tail_first, tail_splits, tail_k_per);
      const int kb0 = um.kb0, kb1 = um.kb1;
      const TileCoord tc = tile_coord<TM>(um.tile, num_m, num_n, args.n_rotate, m_rot);
      if (args.b_flags != nullptr && !b_all_seen) {
        // The elements of B this tile reads must have landed in this GPU's memory.  A
        // K-major B tile is rows [n0, n0+BN) of the weight; an MN-major B (dgrad) strides
        // over the whole matrix, so it waits for all of it once.
        long e0, e1;
        if (B_MN || args.b_wait_all) {
          e0 = args.b_flag_base;
          e1 = args.b_flag_base + static_cast<long>(B_MN ? args.K : args.N) * args.ldb;
          b_all_seen = true;
        } else {
          const int nend = min(tc.n0 + BN, args.N);
          e0 = args.b_flag_base + static_cast<long>(tc.n0) * args.ldb;
          e1 = args.b_flag_base + static_cast<long>(nend - 1) * args.ldb + args.K;
        }
        const long long w0 = clock64();
        ok = acquire_range(args.b_flags, args.b_flag_chunk, e0, e1, args.b_flag_epoch);
        if (lane == 0) atomicAdd(&g_flag_wait_cycles, static_cast<unsigned long long>(clock64() - w0));
        if (!ok) break;
        fence_proxy_async_all();  // generic-proxy writes of the pull CTAs -> async-proxy reads below
      }
      if (args.a_flags != nullptr && !a_all_seen) {
        // Same for a gathered A operand (tensor-parallel all-gather of activation rows): a
        // K-major A tile is rows [m0, m0+BMT); an MN-major A waits for the whole matrix once.
        long e0, e1;
        if (A_MN) {
          e0 = args.a_flag_base;
          e1 = args.a_flag_base + static_cast<long>(args.K) * args.lda;
          a_all_seen = true;
        } else {
          const int mend = min(tc.m0 + BMT, args.M);
          e0 = args.a_flag_base + static_cast<long>(tc.m0) * args.lda;
          e1 = args.a_flag_base + static_cast<long>(mend - 1) * args.lda + args.K;
        }
        const long long w0 = clock64();
        ok = acquire_range(args.a_flags, args.a_flag_chunk, e0, e1, args.a_flag_epoch);
        if (lane == 0) atomicAdd(&g_flag_wait_cycles, static_cast<unsigned long long>(clock64() - w0));
        if (!ok) break;
        fence_proxy_async_all();
      }
      if (lane == 0) {
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, st, SITE_PRODUCER_EMPTY, args.spin_budget)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], A_STAGE + B_STAGE);
          armed |= 1u << stage;
          armed_par = (armed_par & ~(1u << stage)) | (phase << stage);
          uint8_t* sa = smem + stage * A_STAGE;
          uint8_t* sb = smem + C::OFF_B + stage * B_STAGE;
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int a = 0; a < BMT / 64; ++a) tma_load_2d(sa + a * 8192, &map_a, &full[stage], tc.m0 + a * 64, k0);
          } else {
#pragma unroll
            for (int h = 0; h < TM; ++h) tma_load_2d(sa + h * 16384, &map_a, &full[stage], k0, tc.m0 + h * BM);
          }
          if (B_MN) {
#pragma unroll
            for (int a = 0; a < BN / 64; ++a) tma_load_2d(sb + a * 8192, &map_b, &full[stage], tc.n0 + a * 64, k0);
          } else {
            tma_load_2d(sb, &map_b, &full[stage], k0, tc.n0);
          }
          if (++stage == NSTAGE) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }
    if (lane == 0 && (!ok || *abort_flag)) {
      // Leave no copy of ours in flight: wait (bounded) until the last phase armed on
      // each stage has completed, i.e. its TMA bytes have landed.
      for (int s = 0; s < NSTAGE; ++s) {
        if (!(armed & (1u << s))) continue;
        const uint32_t par = (armed_par >> s) & 1u;
        const long long t0 = clock64();
        while (!mbar_try_wait(&full[s], par)) {
          if (clock64() - t0 > 20000000ll) {
            report_failure(st, SITE_DRAIN, static_cast<unsigned>(s), par);
            break;
          }
        }
      }
    }
    if (lane == 0 && args.dynamic_tiles) {
      // the last CTA to stop claiming re-arms the counter pair for the next launch that uses it
      __threadfence();
      const int done = atomicAdd(args.tile_counter + 1, 1) + 1;
      if (done == static_cast<int>(gridDim.x)) {
        args.tile_counter[0] = 0;
        args.tile_counter[1] = 0;
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      uint32_t stage = 0, phase = 0;
      uint32_t uses[2] = {0, 0};     // completed uses of each TMEM slot
      uint32_t next_slot = 0;        // TM == 1: slots alternate from tile to tile
      bool ok = true;
      uint32_t tq = 0, tq_phase = 0;
      while (ok) {
        if (!mbar_wait(&tq_full[tq], tq_phase, abort_flag, st, SITE_TILE_QUEUE, args.spin_budget)) break;
        const int tile = tile_ring[tq];
        mbar_arrive(&tq_empty[tq]);
        if (++tq == TQ) {
          tq = 0;
          tq_phase ^= 1u;
        }
        if (tile < 0) break;
        const UnitMap um = map_unit(tile, total, num_k, splits, k_per, tail_first, tail_splits, tail_k_per);
        const int kb0 = um.kb0, kb1 = um.kb1;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, st, SITE_MMA_FULL, args.spin_budget)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * A_STAGE);
          const uint32_t sb = smem_u32(smem + C::OFF_B + stage * B_STAGE);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t db = B_MN ? desc_mnmajor(sb, k, 8192) : desc_kmajor(sb, k);
#pragma unroll
            for (int h = 0; h < TM; ++h) {
              const uint32_t slot = TM == 1 ? next_slot : static_cast<uint32_t>(h);
              if (kb == kb0 && k == 0) {
                // the slot must have been drained by the epilogue of the tile that used it last
                if (!mbar_wait(&tempty[slot], (uses[slot] & 1u) ^ 1u, abort_flag, st, SITE_MMA_TEMPTY,
                               args.spin_budget)) {
                  ok = false;
                  break;
                }
                tc_fence_after();
              }
              const uint64_t da = A_MN ? desc_mnmajor(sa + h * 16384, k, 8192) : desc_kmajor(sa + h * 16384, k);
              umma_bf16(tmem_base + slot * BN, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
            }
            if (!ok) break;
          }
          if (!ok) break;
          umma_commit(&empty[stage]);
          if (++stage == NSTAGE) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
#pragma unroll
        for (int h = 0; h < TM; ++h) {
          const uint32_t slot = TM == 1 ? next_slot : static_cast<uint32_t>(h);
          umma_commit(&tfull[slot]);
          ++uses[slot];
        }
        if (TM == 1) next_slot ^= 1u;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue (TM warpgroups of 4 warps, 128 TMEM lanes each) ------------
    const int wg = (warp - 4) >> 2;          // TM == 2: warpgroup wg drains slot wg = rows [128 wg, 128 wg + 128)
    const int q = warp & 3;                  // TMEM lane quadrant of this warp
    const int row = q * 32 + lane;           // row of the 128-row sub-tile owned by this thread
    const int etid = threadIdx.x - 128 - wg * 128;
    const uint32_t bar_stage = 1 + wg;       // named barriers of this warpgroup
    const uint32_t bar_vote = 3 + wg;
    uint32_t uses[2] = {0, 0};
    uint32_t next_slot = 0, buf_idx = 0;
    uint8_t* epi = smem + C::OFF_EPI + wg * EPI_BUF;
    uint32_t tq = 0, tq_phase = 0;
    while (true) {
      // The four warps of a warpgroup decide together: a thread that gave up must not leave
      // the others waiting at the staging barriers below.
      const bool queued = mbar_wait(&tq_full[tq], tq_phase, abort_flag, st, SITE_TILE_QUEUE, args.spin_budget);
      if (named_bar_or(bar_vote, 128, !queued)) break;
      const int tile = tile_ring[tq];
      __syncwarp();
      if (lane == 0) mbar_arrive(&tq_empty[tq]);
      if (++tq == TQ) {
        tq = 0;
        tq_phase ^= 1u;
      }
      if (tile < 0) break;
      const UnitMap um = map_unit(tile, total, num_k, splits, k_per, tail_first, tail_splits, tail_k_per);
      const bool add_into_c = args.accumulate || um.reduce;
      const TileCoord tc = tile_coord<TM>(um.tile, num_m, num_n, args.n_rotate, m_rot);
      const uint32_t slot = TM == 1 ? next_slot : static_cast<uint32_t>(wg);
      const bool got = mbar_wait(&tfull[slot], uses[slot] & 1u, abort_flag, st, SITE_EPI_TFULL, args.spin_budget);
      if (named_bar_or(bar_vote, 128, !got)) break;
      ++uses[slot];
      if (TM == 1) next_slot ^= 1u;
      tc_fence_after();
      const uint32_t taddr = tmem_base + slot * BN + (static_cast<uint32_t>(q * 32) << 16);
      const int m_sub = tc.m0 + wg * BM;     // first row of this warpgroup's sub-tile
      const int grow = m_sub + row;

      if (EPI == EPI_CE_STATS) {
        // Online softmax statistics of this 256-column slab for one row per thread.
        const int target = (grow < args.M) ? args.ce_targets[grow] : -1;
        float vmax = -INFINITY, vsum = 0.f, tlogit = 0.f;
        bool has_target = false;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = tc.n0 + c * 32;
          if (col0 >= args.N) break;
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          float cmax = -INFINITY;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float v = (col0 + j < args.N) ? __uint_as_float(r[j]) : -INFINITY;
            r[j] = __float_as_uint(v);
            cmax = fmaxf(cmax, v);
            if (col0 + j == target) {
              tlogit = v;
              has_target = true;
            }
          }
          const float nmax = fmaxf(vmax, cmax);
          float s = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) s += __expf(__uint_as_float(r[j]) - nmax);
          vsum = vsum * __expf(vmax - nmax) + s;
          vmax = nmax;
        }
        if (grow < args.M) {
          const int slab = tc.n0 / BN;
          args.ce_max[static_cast<size_t>(slab) * args.M + grow] = vmax;
          args.ce_sum[static_cast<size_t>(slab) * args.M + grow] = vsum;
          if (has_target) args.ce_target_logit[grow] = tlogit;
        }
      } else if (args.out_f32) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = tc.n0 + c * 32;
          if (col0 >= args.N) break;
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          uint8_t* buf = epi + (C::EPI_BUFS == 2 ? (buf_idx & 1u) * EPI_BUF : 0u);
          if (etid == 0) tma_wait_group_read<C::EPI_BUFS - 1>();
          named_bar_sync(bar_stage, 128);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 v;
            v.x = __uint_as_float(r[4 * j + 0]) * args.alpha;
            v.y = __uint_as_float(r[4 * j + 1]) * args.alpha;
            v.z = __uint_as_float(r[4 * j + 2]) * args.alpha;
            v.w = __uint_as_float(r[4 * j + 3]) * args.alpha;
            *reinterpret_cast<float4*>(buf + sw128_offset(row, j)) = v;
          }
          fence_proxy_async_smem();
          named_bar_sync(bar_stage, 128);
          if (etid == 0 && m_sub < args.M) {
            if (add_into_c) tma_reduce_add_2d(&map_c, buf, col0, m_sub);
            else tma_store_2d(&map_c, buf, col0, m_sub);
            tma_commit_group();
          }
          ++buf_idx;
        }
      } else {
        float lse = 0.f, coef = 0.f;
        int target = -1;
        if (EPI == EPI_CE_DLOGITS && grow < args.M) {
          lse = args.ce_lse[grow];
          coef = args.ce_coef[grow];
          target = args.ce_targets[grow];
        }
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col0 = tc.n0 + c * 64;
          if (col0 >= args.N) break;
          uint8_t* buf = epi + (C::EPI_BUFS == 2 ? (buf_idx & 1u) * EPI_BUF : 0u);
          // 64 output columns per staged block, converted 32 at a time to keep registers low
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t r[32];
            tmem_ld32(taddr + c * 64 + hh * 32, r);
            tmem_ld_wait();
            const int cb = col0 + hh * 32;
            if (EPI == EPI_CE_DLOGITS) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                float pv = __expf(__uint_as_float(r[j]) - lse);
                if (cb + j == target) pv -= 1.f;
                r[j] = __float_as_uint(pv * coef);
              }
            } else if (args.bias != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float bv = (cb + j < args.N) ? __bfloat162float(args.bias[cb + j]) : 0.f;
                r[j] = __float_as_uint(__uint_as_float(r[j]) + bv);
              }
            }
            if (args.alpha != 1.f) {
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * args.alpha);
            }
            if (hh == 0) {
              // the staging block may still be read by the store that used it last
              if (etid == 0) tma_wait_group_read<C::EPI_BUFS - 1>();
              named_bar_sync(bar_stage, 128);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
              v.y = pack_bf16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
              v.z = pack_bf16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
              v.w = pack_bf16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
              *reinterpret_cast<uint4*>(buf + sw128_offset(row, hh * 4 + j)) = v;
            }
          }
          if (EPI == EPI_PUSH) {
            // reduce-scatter by push: 128 threads copy the staged 128 x 128 B block into the
            // owner's receive buffer with 16-byte stores (peer memory: plain st.global only)
            named_bar_sync(bar_stage, 128);
            if (m_sub < args.M) {
              const int grow0 = args.push.row_offset + m_sub;
              const int dest = grow0 / args.push.rows_per_rank;
              const long drow0 = static_cast<long>(args.push.src_rank) * args.push.rows_per_rank +
                                 (grow0 - dest * args.push.rows_per_rank);
              push_block(buf, args.push.dest[dest] + drow0 * args.push.ld + col0, args.push.ld, etid,
                         args.M - m_sub, args.N - col0);
            }
            if (C::EPI_BUFS == 1) named_bar_sync(bar_stage, 128);   // one block: all copies out before it is refilled
          } else {
            fence_proxy_async_smem();
            named_bar_sync(bar_stage, 128);
            if (etid == 0 && m_sub < args.M) {
              if (add_into_c) tma_reduce_add_2d(&map_c, buf, col0, m_sub);
              else tma_store_2d(&map_c, buf, col0, m_sub);
              tma_commit_group();
            }
          }
          ++buf_idx;
        }
        if (EPI == EPI_PUSH && m_sub < args.M) {
          // this 128-row piece is on its way: count it, and publish the flag with the last one
          __threadfence_system();
          named_bar_sync(bar_stage, 128);
          if (etid == 0) {
            const int dest = (args.push.row_offset + m_sub) / args.push.rows_per_rank;
            const unsigned done = atomicAdd(args.push.counters + dest, 1u) + 1u;
            if (done == static_cast<unsigned>(args.push.tiles_per_dest)) {
              args.push.counters[dest] = 0u;
              __threadfence_system();
              asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(args.push.flag[dest]), "r"(args.push.epoch)
                           : "memory");
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[slot]);
    }
    if (etid == 0) tma_wait_group<0>();
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Pairs of (next tile, CTAs finished) counters, zero between launches (the kernel re-arms the pair
// it used).  Launches rotate through the pool so kernels that overlap on different streams never
// share a pair.
inline int& split_k_mode() {
  static int mode = [] {
    const char* e = std::getenv("CTB_GEMM_SPLITK");
    return (e != nullptr && e[0] == '1') ? 1 : 0;
  }();
  return mode;
}

// Tail split (see UnitMap): -1 = not decided yet (environment CTB_GEMM_TAIL_SPLIT, default on).
inline int& tail_split_mode() {
  static int mode = [] {
    const char* e = std::getenv("CTB_GEMM_TAIL_SPLIT");
    return (e != nullptr && e[0] == '0') ? 0 : ((e != nullptr && e[0] == '1') ? 1 : CTB_TAIL_SPLIT_DEFAULT);
  }();
  return mode;
}

// Host copy of tile_coord: first row / column of output tile `tile`.
template <int TM>
inline void host_tile_origin(int tile, int num_m, int num_n, int n_rotate, int m_rotate, int* m0, int* n0) {
  constexpr int GROUP_M = Cfg<TM>::GROUP_M;
  const int per_group = GROUP_M * num_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int rows = std::min(GROUP_M, num_m - first_m);
  const int local = tile - group * per_group;
  int n = local / rows + n_rotate;
  if (n >= num_n) n -= num_n;
  int m = first_m + local % rows + m_rotate;
  if (m >= num_m) m -= num_m;
  *m0 = m * Cfg<TM>::BMT;
  *n0 = n * BN;
}

inline int* next_tile_counter() {
  constexpr int POOL = 256;
  static int* pool[64] = {};
  static unsigned turn[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (pool[dev] == nullptr) {
    if (cudaMalloc(&pool[dev], POOL * 2 * sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(pool[dev], 0, POOL * 2 * sizeof(int));
  }
  return pool[dev] + 2 * (turn[dev]++ % POOL);
}

template <int TM, bool A_MN, bool B_MN, int EPI>
int launch(const CUtensorMap* ma, const CUtensorMap* mb, const CUtensorMap* mc, const GemmArgs& args, int grid,
           cudaStream_t stream) {
  using C = Cfg<TM>;
  auto kern = gemm_kernel<TM, A_MN, B_MN, EPI>;
  static int configured_dev = -1;  // per instantiation; the attribute is per function and device
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    CTB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    configured_dev = dev;
  }
  kern<<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(*ma, *mb, *mc, args);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace gemm

int run_gemm(const GemmCall& c) {
  using namespace gemm;
  if (c.M <= 0 || c.N <= 0 || c.K <= 0) return fail("gemm: M, N, K must be positive");
  if ((c.lda % 8) || (c.ldb % 8)) return fail("gemm: lda and ldb must be multiples of 8 elements (16 bytes)");
  const bool needs_c = (c.epi != EPI_CE_STATS) && !c.push.enabled;
  if (needs_c && (c.ldc % (c.out_f32 ? 4 : 8))) return fail("gemm: ldc must be a multiple of 16 bytes");
  if (gemm_pair_eligible(c)) return launch_gemm_pair(c);       // two-CTA 256 x 256 tiles (gemm_pair.cu)
  const CUtensorMap* ma = c.a_mn ? get_tensor_map_2d(c.A, Elt::BF16, c.M, c.K, c.lda, 64, 64, true)
                                 : get_tensor_map_2d(c.A, Elt::BF16, c.K, c.M, c.lda, 64, BM, true);
  if (!ma) return 1;
  const CUtensorMap* mb = c.b_mn ? get_tensor_map_2d(c.B, Elt::BF16, c.N, c.K, c.ldb, 64, 64, true)
                                 : get_tensor_map_2d(c.B, Elt::BF16, c.K, c.N, c.ldb, 64, BN, true);
  if (!mb) return 1;
  const CUtensorMap* mc = ma;  // placeholder when no C tensor is written
  if (needs_c) {
    mc = c.out_f32 ? get_tensor_map_2d(c.C, Elt::F32, c.N, c.M, c.ldc, 32, 128, true)
                   : get_tensor_map_2d(c.C, Elt::BF16, c.N, c.M, c.ldc, 64, 128, true);
    if (!mc) return 1;
  }
  GemmArgs a{};
  a.M = c.M;
  a.N = c.N;
  a.K = c.K;
  a.out_f32 = c.out_f32;
  a.accumulate = c.accumulate;
  a.alpha = c.alpha;
  a.bias = static_cast<const __nv_bfloat16*>(c.bias);
  a.status = device_status();
  a.spin_budget = c.spin_budget > 0 ? c.spin_budget : CTB_SPIN_BUDGET;
  a.b_flags = c.b_flags;
  a.b_flag_chunk = c.b_flag_chunk > 0 ? c.b_flag_chunk : 1;
  a.b_flag_base = c.b_flag_base;
  a.b_flag_epoch = c.b_flag_epoch;
  a.b_wait_all = c.b_wait_all;
  a.ldb = c.ldb;
  {
    const int num_n = (c.N + gemm::BN - 1) / gemm::BN;
    a.n_rotate = (c.n_rotate > 0 && c.n_rotate < num_n) ? c.n_rotate : 0;
    const int num_m = (c.M + gemm::BM - 1) / gemm::BM;
    a.m_rotate = (c.m_rotate > 0 && c.m_rotate < num_m) ? c.m_rotate : 0;
  }
  a.a_flags = c.a_flags;
  a.a_flag_chunk = c.a_flag_chunk > 0 ? c.a_flag_chunk : 1;
  a.a_flag_base = c.a_flag_base;
  a.a_flag_epoch = c.a_flag_epoch;
  a.lda = c.lda;
  a.ce_targets = c.ce_targets;
  a.ce_max = c.ce_max;
  a.ce_sum = c.ce_sum;
  a.ce_target_logit = c.ce_target_logit;
  a.ce_lse = c.ce_lse;
  a.ce_coef = c.ce_coef;
  a.push = c.push;
  // Dynamic tile claiming measured slightly slower than the static walk on B200 (0-4 % on the
  // projection shapes, alone and under communication), so it is opt-in.
  static const bool dynamic_tiles = [] {
    const char* e = std::getenv("CTB_GEMM_DYNAMIC_TILES");
    return e != nullptr && e[0] == '1';
  }();
  a.dynamic_tiles = dynamic_tiles ? 1 : 0;
  a.tile_counter = nullptr;
  if (dynamic_tiles) {
    a.tile_counter = gemm::next_tile_counter();
    if (a.tile_counter == nullptr) return fail("gemm: cannot allocate the tile counters");
  }
  if (c.push.enabled) {
    if (c.out_f32 || c.accumulate || c.epi != EPI_PUSH) return fail("gemm: the push epilogue writes plain bf16 tiles");
    if (c.push.rows_per_rank % BM || c.push.row_offset % BM || c.push.ld % 8 || c.N % 8)
      return fail("gemm: push needs 128-row aligned rank slabs and 16-byte aligned rows");
  }
  // Tile shape: 256 x 256 when there are enough of them to fill the machine a few times over,
  // 128 x 256 for small problems (CTB_GEMM_TM=1|2 forces one).
  static const int forced_tm = [] {
    const char* e = std::getenv("CTB_GEMM_TM");
    return (e != nullptr && (e[0] == '1' || e[0] == '2')) ? e[0] - '0' : 0;
  }();
  const int num_n = (c.N + BN - 1) / BN;
  const int tiles2 = ((c.M + 2 * BM - 1) / (2 * BM)) * num_n;
  // (the push epilogue copies every block out with the epilogue threads themselves and keeps its
  // two staging blocks: it measured faster on the smaller tile)
  int tm = forced_tm ? forced_tm : ((tiles2 >= 2 * sm_count() && c.epi != EPI_PUSH) ? 2 : 1);
  int tiles = tm == 2 ? tiles2 : ((c.M + BM - 1) / BM) * num_n;
  cudaStream_t s = static_cast<cudaStream_t>(c.stream);
  // Split-K for plain products whose tile count leaves the last wave of CTAs mostly empty (weight
  // gradients: few output tiles, K = tokens).  Candidates are scored by the fraction of SM-waves
  // that do work, with a small charge per extra slice (its prologue, epilogue and reduce traffic)
  // and for the smaller tile.  Off by default: alone the weight-gradient shapes of an 8B model run
  // 4-17 % faster with it, but inside a power-capped training step the extra reduce traffic costs
  // more clock than the idle SMs of the last wave did (measured -2.5 % tokens/s).
  // CTB_GEMM_SPLITK=1 or ctb_gemm_set_split_k(1) turns it on.
  const bool split_enabled = gemm::split_k_mode() != 0;
  a.split_k = 1;
  if (split_enabled && c.epi == EPI_STORE && c.bias == nullptr && c.a_flags == nullptr && c.b_flags == nullptr &&
      c.max_ctas <= 0 && c.K >= 4096) {
    const int sms = sm_count();
    const int num_k = (c.K + gemm::BK - 1) / gemm::BK;
    const int tiles1 = ((c.M + BM - 1) / BM) * num_n;
    double best = 0.0;
    int best_tm = tm, best_s = 1;
    for (int cand_tm = 1; cand_tm <= 2; ++cand_tm) {
      if (forced_tm && cand_tm != forced_tm) continue;
      const int t = cand_tm == 2 ? tiles2 : tiles1;
      for (int sp = 1; sp <= 8; ++sp) {
        if (num_k < 32 * sp) break;
        if (cand_tm == 2 && t * sp < 2 * sms) continue;          // the large tile wants a few waves
        const long u = static_cast<long>(t) * sp;
        const long waves = (u + sms - 1) / sms;
        double score = static_cast<double>(u) / static_cast<double>(waves * sms);
        score *= (cand_tm == 2 ? 1.0 : 0.93) * (1.0 - 0.012 * (sp - 1));
        if (score > best + 1e-9) {
          best = score;
          best_tm = cand_tm;
          best_s = sp;
        }
      }
    }
    if (best_s > 1) {
      tm = best_tm;
      tiles = (tm == 2 ? tiles2 : tiles1) * best_s;
      a.split_k = best_s;
      if (!c.accumulate) {
        const size_t es = c.out_f32 ? 4 : 2;
        CTB_CUDA_OK(cudaMemset2DAsync(c.C, static_cast<size_t>(c.ldc) * es, 0, static_cast<size_t>(c.N) * es,
                                      static_cast<size_t>(c.M), s));
      }
    }
  }
  // Tail split for fp32 outputs (weight gradients accumulated over micro-batches): when the tiles
  // do not fill a whole number of waves and the last wave would be less than half full, its tiles
  // are cut into K slices that reduce-add into C, one slice per otherwise idle CTA.  Only those
  // few tiles pay reduce traffic (and, on a first write, a memset), so unlike split-K over all
  // tiles this does not cost clock inside a power-capped step.
  a.tail_first = 0;
  a.tail_splits = 1;
  if (gemm::tail_split_mode() != 0 && a.split_k == 1 && c.epi == EPI_STORE && c.bias == nullptr && c.out_f32 &&
      c.a_flags == nullptr && c.b_flags == nullptr && c.max_ctas <= 0 && !dynamic_tiles) {
    const int sms = sm_count();
    const int num_k = (c.K + gemm::BK - 1) / gemm::BK;
    const int full = (tiles / sms) * sms;
    const int tail = tiles - full;
    if (full > 0 && tail > 0 && 2 * tail <= sms) {
      int ts = std::min(sms / tail, 16);
      // every slice must be non-empty and long enough to amortise its prologue and epilogue
      while (ts > 1 && (num_k / ts < 16 || (ts - 1) * ((num_k + ts - 1) / ts) >= num_k)) --ts;
      if (ts > 1) {
        if (!c.accumulate) {
          const int num_m_t = tm == 2 ? (c.M + 2 * BM - 1) / (2 * BM) : (c.M + BM - 1) / BM;
          const int m_rot = a.m_rotate / tm < num_m_t ? a.m_rotate / tm : 0;
          for (int t = full; t < tiles; ++t) {
            int m0 = 0, n0 = 0;
            if (tm == 2) gemm::host_tile_origin<2>(t, num_m_t, num_n, a.n_rotate, m_rot, &m0, &n0);
            else gemm::host_tile_origin<1>(t, num_m_t, num_n, a.n_rotate, m_rot, &m0, &n0);
            const int rows = std::min(tm * BM, c.M - m0), cols = std::min(static_cast<int>(BN), c.N - n0);
            float* origin = static_cast<float*>(c.C) + static_cast<size_t>(m0) * c.ldc + n0;
            CTB_CUDA_OK(cudaMemset2DAsync(origin, static_cast<size_t>(c.ldc) * 4, 0, static_cast<size_t>(cols) * 4,
                                          static_cast<size_t>(rows), s));
          }
        }
        a.tail_first = full;
        a.tail_splits = ts;
        tiles = full + tail * ts;
      }
    }
  }
  int grid = std::min(tiles, c.max_ctas > 0 ? c.max_ctas : sm_count());
#define CTB_DISPATCH_TM(TMV, AM, BMN)                                                       \
  switch (c.epi) {                                                                          \
    case EPI_STORE: return launch<TMV, AM, BMN, EPI_STORE>(ma, mb, mc, a, grid, s);         \
    case EPI_CE_STATS: return launch<TMV, AM, BMN, EPI_CE_STATS>(ma, mb, mc, a, grid, s);   \
    case EPI_CE_DLOGITS: return launch<TMV, AM, BMN, EPI_CE_DLOGITS>(ma, mb, mc, a, grid, s); \
    case EPI_PUSH: return launch<TMV, AM, BMN, EPI_PUSH>(ma, mb, mc, a, grid, s);           \
    default: return fail("gemm: unknown epilogue");                                         \
  }
#define CTB_DISPATCH(AM, BMN)                 \
  if (tm == 2) { CTB_DISPATCH_TM(2, AM, BMN) } \
  CTB_DISPATCH_TM(1, AM, BMN)
  if (!c.a_mn && !c.b_mn) { CTB_DISPATCH(false, false) }
  if (!c.a_mn && c.b_mn) { CTB_DISPATCH(false, true) }
  if (c.a_mn && c.b_mn) { CTB_DISPATCH(true, true) }
  CTB_DISPATCH(true, false)
#undef CTB_DISPATCH_TM
#undef CTB_DISPATCH
}

}  // namespace ctb

// C ABI ------------------------------------------------------------------------------------
// C[M,N] = alpha * A*B^T (+ bias) ; see the layout table at the top of this file.
CTB_API int ctb_gemm(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb, long ldc,
                     int a_mn, int b_mn, int out_f32, int accumulate, float alpha, const void* bias, int max_ctas,
                     void* stream) {
  ctb::GemmCall c{};
  c.A = A; c.B = B; c.C = C; c.M = M; c.N = N; c.K = K; c.lda = lda; c.ldb = ldb; c.ldc = ldc;
  c.a_mn = a_mn; c.b_mn = b_mn; c.out_f32 = out_f32; c.accumulate = accumulate; c.alpha = alpha; c.bias = bias;
  c.epi = ctb::EPI_STORE; c.max_ctas = max_ctas; c.stream = stream;
  return ctb::run_gemm(c);
}

// Same GEMM family whose B operand lives in a buffer that another kernel (the all-gather
// pull) is still filling: flags[i] >= epoch means elements [i*chunk, (i+1)*chunk) of that
// buffer are complete; `flag_base` is the element offset of B inside the buffer.
CTB_API int ctb_gemm_flagged(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb, long ldc,
                             int a_mn, int b_mn, int out_f32, int accumulate, float alpha, const void* bias,
                             const unsigned* flags, long flag_chunk, long flag_base, unsigned epoch, int wait_all,
                             int n_rotate, const unsigned* a_flags, long a_flag_chunk, long a_flag_base,
                             unsigned a_epoch, int m_rotate, long long spin_budget, int max_ctas, void* stream) {
  ctb::GemmCall c{};
  c.A = A; c.B = B; c.C = C; c.M = M; c.N = N; c.K = K; c.lda = lda; c.ldb = ldb; c.ldc = ldc;
  c.a_mn = a_mn; c.b_mn = b_mn; c.out_f32 = out_f32; c.accumulate = accumulate; c.alpha = alpha; c.bias = bias;
  c.epi = ctb::EPI_STORE; c.max_ctas = max_ctas; c.stream = stream;
  c.b_flags = flags; c.b_flag_chunk = flag_chunk; c.b_flag_base = flag_base; c.b_flag_epoch = epoch;
  c.b_wait_all = wait_all; c.spin_budget = spin_budget; c.n_rotate = n_rotate;
  c.a_flags = a_flags; c.a_flag_chunk = a_flag_chunk; c.a_flag_base = a_flag_base; c.a_flag_epoch = a_epoch;
  c.m_rotate = m_rotate;
  return ctb::run_gemm(c);
}

// Row-parallel projection with the reduce-scatter fused into the epilogue (see GemmPush).
// `dest_table[p]` (device memory) is rank p's receive buffer, `flag_table[p]` the address of this
// rank's flag on rank p.  A may be a gathered buffer (a_flags) exactly as in ctb_gemm_flagged.
CTB_API int ctb_gemm_push(const void* A, const void* B, int M, int N, int K, long lda, long ldb, int a_mn, int b_mn,
                          float alpha, const void* dest_table, const void* flag_table, unsigned* counters, int rows_per_rank, int row_offset, int src_rank, int tiles_per_dest,
                          long ld, unsigned epoch, const unsigned* b_flags, long b_flag_chunk, long b_flag_base,
                          unsigned b_epoch, int b_wait_all, int n_rotate, int m_rotate, long long spin_budget,
                          int max_ctas, void* stream) {
  ctb::GemmCall c{};
  c.A = A; c.B = B; c.C = nullptr; c.M = M; c.N = N; c.K = K; c.lda = lda; c.ldb = ldb; c.ldc = ld;
  c.a_mn = a_mn; c.b_mn = b_mn; c.alpha = alpha; c.epi = ctb::EPI_PUSH; c.max_ctas = max_ctas; c.stream = stream;
  c.b_flags = b_flags; c.b_flag_chunk = b_flag_chunk; c.b_flag_base = b_flag_base; c.b_flag_epoch = b_epoch;
  c.b_wait_all = b_wait_all; c.n_rotate = n_rotate; c.m_rotate = m_rotate; c.spin_budget = spin_budget;
  c.push.dest = static_cast<__nv_bfloat16* const*>(dest_table);
  c.push.flag = static_cast<unsigned* const*>(flag_table);
  c.push.counters = counters; c.push.rows_per_rank = rows_per_rank; c.push.row_offset = row_offset;
  c.push.src_rank = src_rank; c.push.tiles_per_dest = tiles_per_dest; c.push.ld = ld; c.push.epoch = epoch;
  c.push.enabled = 1;
  return ctb::run_gemm(c);
}

// Cut cross-entropy statistics: logits = hidden[rows,d] * head[vocab,d]^T are reduced per
// 256-column slab to pmax/psum[slab][row]; target_logit[row] is written by the slab that
// holds the row's target (rows with target < 0 are never written).
CTB_API int ctb_ce_stats(const void* hidden, const void* head, int rows, int vocab, int d, long ldh, long ldw,
                         const int* targets, float* pmax, float* psum, float* target_logit, const unsigned* flags,
                         long flag_chunk, long flag_base, unsigned epoch, const unsigned* a_flags, long a_flag_chunk,
                         long a_flag_base, unsigned a_epoch, int m_rotate, void* stream) {
  ctb::GemmCall c{};
  c.b_flags = flags; c.b_flag_chunk = flag_chunk; c.b_flag_base = flag_base; c.b_flag_epoch = epoch;
  c.a_flags = a_flags; c.a_flag_chunk = a_flag_chunk; c.a_flag_base = a_flag_base; c.a_flag_epoch = a_epoch;
  c.m_rotate = m_rotate;
  c.A = hidden; c.B = head; c.M = rows; c.N = vocab; c.K = d; c.lda = ldh; c.ldb = ldw;
  c.epi = ctb::EPI_CE_STATS; c.stream = stream;
  c.ce_targets = targets; c.ce_max = pmax; c.ce_sum = psum; c.ce_target_logit = target_logit;
  return ctb::run_gemm(c);
}

// Cut cross-entropy backward slab: G[rows,vocab] = (exp(logits - lse[row]) - onehot) * coef[row], bf16.
CTB_API int ctb_ce_dlogits(const void* hidden, const void* head, void* g, int rows, int vocab, int d, long ldh,
                           long ldw, long ldg, const int* targets, const float* lse, const float* coef,
                           void* stream) {
  ctb::GemmCall c{};
  c.A = hidden; c.B = head; c.C = g; c.M = rows; c.N = vocab; c.K = d; c.lda = ldh; c.ldb = ldw; c.ldc = ldg;
  c.epi = ctb::EPI_CE_DLOGITS; c.stream = stream;
  c.ce_targets = targets; c.ce_lse = lse; c.ce_coef = coef;
  return ctb::run_gemm(c);
}

// 0: never split K; 1: split K when it fills the last wave (see launch_gemm).  Returns the previous mode.
CTB_API int ctb_gemm_set_split_k(int mode) {
  int& m = ctb::gemm::split_k_mode();
  const int before = m;
  m = mode != 0 ? 1 : 0;
  return before;
}

// 0: never; 1: cut the tiles of a mostly empty last wave into K slices (fp32 outputs only, see
// launch_gemm).  Returns the previous mode.
CTB_API int ctb_gemm_set_tail_split(int mode) {
  int& m = ctb::gemm::tail_split_mode();
  const int before = m;
  m = mode != 0 ? 1 : 0;
  return before;
}

// Sum over CTAs of the cycles GEMM producer warps waited for gathered-operand flags since the
// previous call (the counter is cleared).  Synchronises the device; a diagnostic, not a hot path.
CTB_API int ctb_gemm_flag_wait_cycles(unsigned long long* out) {
  unsigned long long zero = 0ull;
  CTB_CUDA_OK(cudaDeviceSynchronize());
  CTB_CUDA_OK(cudaMemcpyFromSymbol(out, ctb::gemm::g_flag_wait_cycles, sizeof(*out)));
  CTB_CUDA_OK(cudaMemcpyToSymbol(ctb::gemm::g_flag_wait_cycles, &zero, sizeof(zero)));
  return 0;
}
