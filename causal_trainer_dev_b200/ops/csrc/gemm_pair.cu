// Two-CTA tcgen05 GEMM: a cluster of two CTAs on two SMs computes one 256 x 256 output tile with
// `tcgen05.mma.cta_group::2`.  Each CTA stages its own 128 rows of A and its own 128 columns of B;
// the tensor cores of both SMs read both halves of B, so a CTA moves a third fewer operand bytes
// per FLOP through its shared memory than the one-CTA 128 x 256 tile and the same 192 KiB of
// stages hold six k-blocks instead of four.
//
//   C[M,N] = alpha * A * B^T   (bf16 in, fp32 accumulate in TMEM, bf16 or fp32 out, store or
//                               TMA reduce-add), the four operand layouts of gemm.cu
//
// Roles per CTA (256 threads): warp 0 TMA producer (each CTA loads its own operands; the bytes of
// both are credited to the full barrier of the leader CTA), warp 1 of the leader issues the MMAs
// for the pair and releases stages / publishes accumulators with multicast commits to both CTAs,
// warp 2 owns the TMEM allocation, warps 4-7 drain this CTA's 128 accumulator rows.  The two
// 256-column TMEM slots double-buffer the accumulator.  Every wait is bounded; the two CTAs meet
// at a cluster barrier before they tear down, so neither leaves while the other can still signal it.
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>

#include "gemm.h"

namespace ctb {
namespace gemm2 {

constexpr int BM = 128;        // rows of A per CTA
constexpr int BN = 256;        // columns of the pair's tile
constexpr int BNH = 128;       // columns of B staged per CTA
constexpr int BK = 64;
constexpr int NSTAGE = 6;
constexpr int A_STAGE = BM * BK * 2;     // 16 KiB
constexpr int B_STAGE = BNH * BK * 2;    // 16 KiB
constexpr int EPI_BUF = 128 * 128;
constexpr int OFF_B = NSTAGE * A_STAGE;
constexpr int OFF_EPI = OFF_B + NSTAGE * B_STAGE;
constexpr int OFF_BAR = OFF_EPI + 2 * EPI_BUF;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
constexpr int THREADS = 256;
constexpr int GROUP_M = 8;     // 256-row tiles per band

enum : unsigned {
  SITE_P_EMPTY = 0x0801,
  SITE_P_FULL = 0x0802,
  SITE_P_TEMPTY = 0x0803,
  SITE_P_TFULL = 0x0804,
};

struct PairArgs {
  int M, N, K;
  int out_f32;
  int accumulate;
  float alpha;
  DeviceStatus* status;
  long long spin_budget;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory object in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Tensor copy into this CTA's shared memory whose bytes are credited to a barrier of the pair
// (`bar_cluster_addr` is a shared::cluster address, here always the leader's).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this offset in both CTAs once all MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

struct TileCoord {
  int m0, n0;
};
// Bands of GROUP_M row tiles; inside a band the column advances slowly (B stays hot in L2).
__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m, int num_n) {
  const int per_group = GROUP_M * num_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int rows = min(GROUP_M, num_m - first_m);
  const int local = tile - group * per_group;
  TileCoord c;
  c.m0 = (first_m + local % rows) * 2 * BM;
  c.n0 = (local / rows) * BN;
  return c;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, const PairArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + OFF_BAR);   // used in the leader only
  uint64_t* empty = full + NSTAGE;
  uint64_t* tfull = empty + NSTAGE;      // [2]
  uint64_t* tempty = tfull + 2;          // [2] used in the leader only: both CTAs' epilogue warps arrive
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  DeviceStatus* st = args.status;
  const long long budget = args.spin_budget;
  const int num_m = (args.M + 2 * BM - 1) / (2 * BM);
  const int num_n = (args.N + BN - 1) / BN;
  const int num_k = (args.K + BK - 1) / BK;
  const int total = num_m * num_n;
  const int pair = blockIdx.x >> 1;
  const int pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);      // four epilogue warps of each CTA
    }
    *abort_flag = 0u;
    mbar_fence_init();
  }
  if (warp == 3 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    tma_prefetch_desc(&map_c);
  }
  if (warp == 2) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();                    // both CTAs' barriers exist before either signals the other
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < total; tile += pairs) {
        const TileCoord tc = tile_coord(tile, num_m, num_n);
        const int m0 = tc.m0 + static_cast<int>(rank) * BM;       // this CTA's rows of A
        const int n0 = tc.n0 + static_cast<int>(rank) * BNH;      // this CTA's columns of B
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, st, SITE_P_EMPTY, budget)) {
            ok = false;
            break;
          }
          // the leader arms its barrier with the bytes of both CTAs
          if (leader) mbar_expect_tx(&full[stage], 2 * (A_STAGE + B_STAGE));
          const uint32_t bar = map_to_rank(smem_u32(&full[stage]), 0);
          uint8_t* sa = smem + stage * A_STAGE;
          uint8_t* sb = smem + OFF_B + stage * B_STAGE;
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int a = 0; a < BM / 64; ++a) tma_load_2d_pair(sa + a * 8192, &map_a, bar, m0 + a * 64, k0);
          } else {
            tma_load_2d_pair(sa, &map_a, bar, k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int a = 0; a < BNH / 64; ++a) tma_load_2d_pair(sb + a * 8192, &map_b, bar, n0 + a * 64, k0);
          } else {
            tma_load_2d_pair(sb, &map_b, bar, k0, n0);
          }
          if (++stage == NSTAGE) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA, for the pair) ------------------------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      uint32_t stage = 0, phase = 0;
      uint32_t uses[2] = {0, 0};
      uint32_t slot = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < total; tile += pairs) {
        // the slot must have been drained by both CTAs' epilogues of the tile that used it last
        if (!mbar_wait(&tempty[slot], (uses[slot] & 1u) ^ 1u, abort_flag, st, SITE_P_TEMPTY, budget)) break;
        tc_fence_after();
        for (int kb = 0; kb < num_k; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, st, SITE_P_FULL, budget)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * A_STAGE);
          const uint32_t sb = smem_u32(smem + OFF_B + stage * B_STAGE);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN ? desc_mnmajor(sa, k, 8192) : desc_kmajor(sa, k);
            const uint64_t db = B_MN ? desc_mnmajor(sb, k, 8192) : desc_kmajor(sb, k);
            umma_bf16_pair(tmem_base + slot * BN, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty[stage]);       // both producers may refill the stage
          if (++stage == NSTAGE) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_pair(&tfull[slot]);          // both epilogues may drain the slot
        ++uses[slot];
        slot ^= 1u;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ epilogue: this CTA's 128 accumulator rows ------------------------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int etid = threadIdx.x - 128;
    uint32_t uses[2] = {0, 0};
    uint32_t slot = 0, buf_idx = 0;
    uint8_t* epi = smem + OFF_EPI;
    for (int tile = pair; tile < total; tile += pairs) {
      const TileCoord tc = tile_coord(tile, num_m, num_n);
      const bool ready = mbar_wait(&tfull[slot], uses[slot] & 1u, abort_flag, st, SITE_P_TFULL, budget);
      if (named_bar_or(3, 128, !ready)) break;      // the four warps decide together
      tc_fence_after();
      const uint32_t taddr = tmem_base + slot * BN + (static_cast<uint32_t>(q * 32) << 16);
      const int m_sub = tc.m0 + static_cast<int>(rank) * BM;
      if (args.out_f32) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = tc.n0 + c * 32;
          if (col0 >= args.N) break;
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          uint8_t* buf = epi + (buf_idx & 1u) * EPI_BUF;
          if (etid == 0) tma_wait_group_read<1>();
          named_bar_sync(1, 128);
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
          named_bar_sync(1, 128);
          if (etid == 0 && m_sub < args.M) {
            if (args.accumulate) tma_reduce_add_2d(&map_c, buf, col0, m_sub);
            else tma_store_2d(&map_c, buf, col0, m_sub);
            tma_commit_group();
          }
          ++buf_idx;
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col0 = tc.n0 + c * 64;
          if (col0 >= args.N) break;
          uint8_t* buf = epi + (buf_idx & 1u) * EPI_BUF;
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t r[32];
            tmem_ld32(taddr + c * 64 + hh * 32, r);
            tmem_ld_wait();
            if (args.alpha != 1.f) {
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * args.alpha);
            }
            if (hh == 0) {
              if (etid == 0) tma_wait_group_read<1>();     // the block may still be read by its last store
              named_bar_sync(1, 128);
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
          fence_proxy_async_smem();
          named_bar_sync(1, 128);
          if (etid == 0 && m_sub < args.M) {
            if (args.accumulate) tma_reduce_add_2d(&map_c, buf, col0, m_sub);
            else tma_store_2d(&map_c, buf, col0, m_sub);
            tma_commit_group();
          }
          ++buf_idx;
        }
      }
      tc_fence_before();
      __syncwarp();
      // the leader's MMA thread counts the eight epilogue warps of the pair
      if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&tempty[slot]), 0));
      ++uses[slot];
      slot ^= 1u;
    }
    if (etid == 0) tma_wait_group<0>();
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  cluster_sync();                    // nobody leaves while its peer may still signal it
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

inline int& pair_mode() {
  static int mode = [] {
    const char* e = std::getenv("CTB_GEMM_PAIR");
    return (e != nullptr && e[0] == '1') ? 1 : 0;
  }();
  return mode;
}

template <bool A_MN, bool B_MN>
int launch(const CUtensorMap* ma, const CUtensorMap* mb, const CUtensorMap* mc, const PairArgs& a, int grid,
           cudaStream_t s) {
  auto kern = gemm_pair_kernel<A_MN, B_MN>;
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    CTB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    configured_dev = dev;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CTB_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, *ma, *mb, *mc, a));
  return 0;
}

}  // namespace gemm2

// True when the call is a plain product the two-CTA kernel covers (no gathered operands, no fused
// epilogue, no bias) and the mode is on.
bool gemm_pair_eligible(const GemmCall& c) {
  if (gemm2::pair_mode() == 0) return false;
  if (c.epi != EPI_STORE || c.bias != nullptr || c.a_flags != nullptr || c.b_flags != nullptr || c.push.enabled ||
      c.max_ctas > 0)
    return false;
  const int tiles = ((c.M + 255) / 256) * ((c.N + 255) / 256);
  return tiles >= sm_count() / 2 && c.K >= 512;
}

int launch_gemm_pair(const GemmCall& c) {
  using namespace gemm2;
  const CUtensorMap* ma = c.a_mn ? get_tensor_map_2d(c.A, Elt::BF16, c.M, c.K, c.lda, 64, 64, true)
                                 : get_tensor_map_2d(c.A, Elt::BF16, c.K, c.M, c.lda, 64, 128, true);
  const CUtensorMap* mb = c.b_mn ? get_tensor_map_2d(c.B, Elt::BF16, c.N, c.K, c.ldb, 64, 64, true)
                                 : get_tensor_map_2d(c.B, Elt::BF16, c.K, c.N, c.ldb, 64, 128, true);
  const CUtensorMap* mc = c.out_f32 ? get_tensor_map_2d(c.C, Elt::F32, c.N, c.M, c.ldc, 32, 128, true)
                                    : get_tensor_map_2d(c.C, Elt::BF16, c.N, c.M, c.ldc, 64, 128, true);
  if (!ma || !mb || !mc) return 1;
  PairArgs a{};
  a.M = c.M;
  a.N = c.N;
  a.K = c.K;
  a.out_f32 = c.out_f32;
  a.accumulate = c.accumulate;
  a.alpha = c.alpha;
  a.status = device_status();
  a.spin_budget = c.spin_budget > 0 ? c.spin_budget : CTB_SPIN_BUDGET;
  const int tiles = ((c.M + 255) / 256) * ((c.N + 255) / 256);
  const int pairs = std::min(tiles, sm_count() / 2);
  cudaStream_t s = static_cast<cudaStream_t>(c.stream);
  if (!c.a_mn && !c.b_mn) return launch<false, false>(ma, mb, mc, a, 2 * pairs, s);
  if (!c.a_mn && c.b_mn) return launch<false, true>(ma, mb, mc, a, 2 * pairs, s);
  if (c.a_mn && c.b_mn) return launch<true, true>(ma, mb, mc, a, 2 * pairs, s);
  return launch<true, false>(ma, mb, mc, a, 2 * pairs, s);
}

}  // namespace ctb

// 0: one-CTA kernels only; 1: plain products with enough tiles run on CTA pairs.  Returns the previous mode.
CTB_API int ctb_gemm_set_pair(int mode) {
  int& m = ctb::gemm2::pair_mode();
  const int before = m;
  m = mode != 0 ? 1 : 0;
  return before;
}
