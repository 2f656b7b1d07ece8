// Flash attention forward for sm_100a: segment-isolated causal attention with an optional
// per-query inclusive visibility end (MaskGIT block-local bidirectional attention), GQA.
//
//   key j is visible to query i  <=>  seg[j] == seg[i] != 0  and  j <= max(i, attention_end[i])
//
// One CTA owns 256 consecutive query rows of one (batch, query head): two 128-row tiles
// that ping-pong so the tensor core computes one tile's S = Q K^T / O += P V while the
// other tile's softmax runs.
//   warp 0      TMA producer (Q tiles once, then K(j), V(j) through a 5-slot ring)
//   warp 1      TMEM allocation + single-thread tcgen05.mma issue   (warps 2-3 idle)
//   warps 4-7   softmax of tile 0 (one query row per thread, TMEM lane = row)
//   warps 8-11  softmax of tile 1
// The softmax holds a whole score row (128 fp32) in registers: one TMEM round trip per tile.
// S (fp32) and O (fp32) live in TMEM.  P is written back into TMEM as bf16 pairs over the first
// half of its score row and is the TMEM A operand of the second MMA, so it never crosses shared
// memory and the shared memory it would need holds two more K/V slots; V is consumed in place as
// an MN-major operand.  The service warpgroup (warps 0-3) gives most of its registers to the two
// softmax warpgroups (setmaxnreg).
// The running maximum is only raised when it grows by more than 2^8 (the O rescale in TMEM
// is rare), the final O / l and LSE are written by the softmax warps.
// KV blocks outside [kv_lo, kv_hi) of a query block are never visited (block skipping from
// segment summaries); rows without any visible key produce O = 0 and LSE = 0.
//
// Reference counterpart: causal_trainer_attention_fwd
// (src/causal_trainer/kernels/efficient_attention.py:560-771, 931-978).
#include "attention.h"

namespace ctb {
namespace attn {

constexpr int FWD_THREADS = 384;
constexpr int KV_SLOTS = 5;

enum : unsigned {
  SITE_F_PROD = 0x0201,
  SITE_F_MMA_Q = 0x0202,
  SITE_F_MMA_KV = 0x0203,
  SITE_F_MMA_P = 0x0204,
  SITE_F_SM_S = 0x0205,
  SITE_F_SM_PV = 0x0206,
  SITE_F_KV_FLAG = 0x0207,
};

template <int D>
struct FwdSmem {
  static constexpr int HALVES = D / 64;
  static constexpr int QT = HALVES * 16384;        // one 128-row Q / K / V tile
  static constexpr int OFF_Q = 0;                  // two Q tiles; each doubles as the staging tile of its O
  static constexpr int OFF_KV = 2 * QT;
  static constexpr int OFF_BAR = OFF_KV + KV_SLOTS * QT;
  static constexpr int BYTES = OFF_BAR + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                const FwdArgs args) {
  using L = FwdSmem<D>;
  constexpr int HALVES = L::HALVES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* q_full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* kv_full = q_full + 1;
  uint64_t* kv_empty = kv_full + KV_SLOTS;
  uint64_t* s_full = kv_empty + KV_SLOTS;
  uint64_t* p_full = s_full + 2;
  uint64_t* pv_done = p_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  DeviceStatus* st = args.status;
  const long long budget = args.spin_budget;

  // ---- work item ----
  // grouped MoBA: this CTA's 256 gathered rows against one key block (see GroupArgs)
  const bool grouped = args.grp.desc != nullptr;
  int4 gd = make_int4(0, 0, 0, 0);
  if (grouped) {
    gd = __ldg(args.grp.desc + blockIdx.x);
    if (gd.w <= 0) return;                       // capacity beyond the rows in use: the whole CTA leaves
  }
  const int nqp = (args.Sq + 255) / 256;
  int idx = blockIdx.x;
  const int h = grouped ? 0 : idx % args.Hq;
  idx /= args.Hq;
  const int b = grouped ? 0 : idx % args.B;
  const int pair = grouped ? static_cast<int>(blockIdx.x) : nqp - 1 - idx / args.B;
  const int q0 = pair * 256;
  const int hkv = grouped ? (gd.x >> 16) : h / (args.Hq / args.Hkv);
  const int kb = grouped ? (gd.x & 0xffff) : b;  // batch of the keys
  const int nqb = args.S / 128;
  bool tile_valid[2];
  int lo_t[2], hi_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    tile_valid[t] = grouped ? (t * 128 < gd.w) : (q0 + t * 128) < args.Sq;
    lo_t[t] = 0;
    hi_t[t] = 0;
    if (tile_valid[t] && !grouped) {
      const int qb = (args.q_off + q0) / 128 + t;      // query block in the whole sequence
      const int lo_tok = args.kv_lo[b * nqb + qb];
      const int hi_tok = args.kv_hi[b * nqb + qb];
      if (hi_tok > lo_tok) {
        lo_t[t] = lo_tok / 128;
        hi_t[t] = (hi_tok + 127) / 128;
      }
    }
  }
  int lo = 0;
  if (hi_t[0] > lo_t[0] && hi_t[1] > lo_t[1]) lo = min(lo_t[0], lo_t[1]);
  else if (hi_t[0] > lo_t[0]) lo = lo_t[0];
  else if (hi_t[1] > lo_t[1]) lo = lo_t[1];
  int n0 = (hi_t[0] > lo_t[0]) ? hi_t[0] - lo : 0;
  int n1 = (hi_t[1] > lo_t[1]) ? hi_t[1] - lo : 0;
  // Block-sparse routing: both query tiles walk the listed key tiles (rows that selected nothing in
  // a tile see it fully masked).
  const bool sparse = args.sp.it_list != nullptr;
  const int* kv_list = nullptr;
  if (sparse) {
    int base, cnt;
    sparse_list(args.sp, blockIdx.x, base, cnt);
    kv_list = args.sp.it_list + base;
    n0 = tile_valid[0] ? cnt : 0;
    n1 = tile_valid[1] ? cnt : 0;
  }
  if (grouped) {
    n0 = args.grp.block / 128;
    n1 = tile_valid[1] ? n0 : 0;
  }
  const int nmax = max(n0, n1);
  // first key of the i-th key tile this CTA visits
  auto kv_pos = [&](int i) -> int {
    return grouped ? gd.y + i * 128 : (sparse ? __ldg(kv_list + i) : lo + i) * 128;
  };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_SLOTS; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 128);
      mbar_init(&pv_done[t], 1);
    }
    *abort_flag = 0u;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto tmem_s_of = [&](int t) -> uint32_t { return tmem_base + static_cast<uint32_t>(t) * 128u; };
  auto tmem_o_of = [&](int t) -> uint32_t { return tmem_base + 256u + static_cast<uint32_t>(t) * D; };

  if (warp < 4) {
  // the service warpgroup hands most of its registers to the two softmax warpgroups, which hold a
  // whole 128-column score row per thread
  asm volatile("setmaxnreg.dec.sync.aligned.u32 72;" ::: "memory");
  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0 && nmax > 0) {
      uint32_t bytes = 0;
      for (int t = 0; t < 2; ++t)
        if (tile_valid[t]) bytes += L::QT;
      mbar_expect_tx(q_full, bytes);
      for (int t = 0; t < 2; ++t) {
        if (!tile_valid[t]) continue;
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf)
          tma_load_4d(smem + L::OFF_Q + t * L::QT + hf * 16384, &map_q, q_full, hf * 64, h, q0 + t * 128, b);
      }
      uint32_t slot = 0, phase = 0;
      bool ok = true;
      for (int i = 0; ok && i < nmax; ++i) {
        const int k0 = kv_pos(i);
        if (args.kvf.flags != nullptr) {
          // gathered K / V (see KvFlags): the rows [k0, k0 + 128) of batch kb must have landed
          const long e0 = (static_cast<long>(kb) * args.S + k0) * args.kvf.row_elems;
          const long e1 = e0 + 128 * args.kvf.row_elems - 1;
          for (long f = e0 / args.kvf.chunk; ok && f <= e1 / args.kvf.chunk; ++f) {
            const long long t0 = clock64();
            while (true) {
              unsigned got;
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(got) : "l"(args.kvf.flags + f) : "memory");
              if (got >= args.kvf.epoch) break;
              if (*abort_flag || clock64() - t0 > budget) {
                *abort_flag = 1u;
                report_failure(st, SITE_F_KV_FLAG, static_cast<unsigned>(f), args.kvf.epoch);
                ok = false;
                break;
              }
              __nanosleep(64);
            }
          }
          if (!ok) break;
          fence_proxy_async_all();   // generic-proxy writes of the pull CTAs -> async-proxy reads below
        }
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          if (!mbar_wait(&kv_empty[slot], phase ^ 1u, abort_flag, st, SITE_F_PROD, budget)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&kv_full[slot], L::QT);
          uint8_t* dst = smem + L::OFF_KV + slot * L::QT;
          const CUtensorMap* m = which == 0 ? &map_k : &map_v;
#pragma unroll
          for (int hf = 0; hf < HALVES; ++hf) tma_load_4d(dst + hf * 16384, m, &kv_full[slot], hf * 64, hkv, k0, kb);
          if (++slot == KV_SLOTS) {
            slot = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && nmax > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, D, false, true);
      const int n_t[2] = {n0, n1};
      uint32_t slot = 0, phase = 0;
      uint32_t pph[2] = {0, 0};
      bool ok = mbar_wait(q_full, 0, abort_flag, st, SITE_F_MMA_Q, budget);
      auto issue_s = [&](int t, uint32_t kslot) {
        const uint32_t qa = smem_u32(smem + L::OFF_Q + t * L::QT);
        const uint32_t ka = smem_u32(smem + L::OFF_KV + kslot * L::QT);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t da = desc_kmajor(qa + (k / 4) * 16384, k % 4);
          const uint64_t db = desc_kmajor(ka + (k / 4) * 16384, k % 4);
          umma_bf16(tmem_s_of(t), da, db, idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      };
      uint32_t kslot = 0;
      if (ok) {
        ok = mbar_wait(&kv_full[slot], phase, abort_flag, st, SITE_F_MMA_KV, budget);
        if (ok) {
          tc_fence_after();
          kslot = slot;
          if (++slot == KV_SLOTS) { slot = 0; phase ^= 1u; }
          for (int t = 0; t < 2; ++t)
            if (n_t[t] > 0) issue_s(t, kslot);
          umma_commit(&kv_empty[kslot]);
        }
      }
      for (int i = 0; ok && i < nmax; ++i) {
        if (!mbar_wait(&kv_full[slot], phase, abort_flag, st, SITE_F_MMA_KV, budget)) break;
        const uint32_t vslot = slot;
        if (++slot == KV_SLOTS) { slot = 0; phase ^= 1u; }
        const bool has_next = (i + 1 < nmax);
        if (has_next) {
          if (!mbar_wait(&kv_full[slot], phase, abort_flag, st, SITE_F_MMA_KV, budget)) break;
          kslot = slot;
          if (++slot == KV_SLOTS) { slot = 0; phase ^= 1u; }
        }
        tc_fence_after();
        const uint32_t va = smem_u32(smem + L::OFF_KV + vslot * L::QT);
        for (int t = 0; t < 2; ++t) {
          if (i >= n_t[t]) continue;
          if (!mbar_wait(&p_full[t], pph[t], abort_flag, st, SITE_F_MMA_P, budget)) {
            ok = false;
            break;
          }
          pph[t] ^= 1u;
          tc_fence_after();
          // P is read from TMEM (bf16 pairs in the first 64 columns of the tile's score region):
          // it never crosses shared memory, whose bandwidth the operand fetches of the MMAs saturate
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint64_t db = desc_mnmajor(va, k, 16384);
            umma_bf16_ts(tmem_o_of(t), tmem_s_of(t) + k * 8, db, idesc_o, (i | k) != 0 ? 1u : 0u);
          }
          umma_commit(&pv_done[t]);
          if (i + 1 < n_t[t]) issue_s(t, kslot);
        }
        if (!ok) break;
        umma_commit(&kv_empty[vslot]);
        if (has_next) umma_commit(&kv_empty[kslot]);
      }
    }
  }
  } else {
    // ------------------------------ softmax warpgroups ------------------------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;" ::: "memory");
    const int t = (warp - 4) >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int n_mine = t == 0 ? n0 : n1;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    uint8_t* obuf = smem + L::OFF_Q + t * L::QT;       // staging of O: the Q tile is dead after the last S MMA
    bool ok = true;
    float m_ref = -INFINITY, l_sum = 0.f;
    const int qi_local = q0 + t * 128 + r;             // row of Q / O / LSE held by this rank
    const int qi = args.q_off + qi_local;              // its position in the whole sequence
    int my_seg = 0, my_lim = qi, my_start = 0, my_first = 0;
    if (tile_valid[t] && grouped) {
      // a real gathered row sees every key of the block; a padding row sees none
      my_seg = (t * 128 + r < gd.w) ? 1 : 0;
      my_first = -(1 << 30);
      my_lim = 1 << 30;
    } else if (tile_valid[t]) {
      my_seg = args.seg[b * args.S + qi];
      my_first = args.row_start[b * args.S + qi];
      if (args.lim != nullptr) my_lim = args.lim[b * args.S + qi];
      if (sparse) my_start = args.sp.doc_start[b * args.S + qi];
    }
    uint32_t sph = 0;
    const uint64_t scale2 = pack_f32x2(args.scale_log2, args.scale_log2);
    for (int i = 0; i < n_mine; ++i) {
      const int k0 = kv_pos(i);
      // ---- visible columns of this row inside the key tile: the keys of a row's run are
      // contiguous, so they form one interval [c_lo, c_hi] (tile-relative, may lie outside) ----
      const int c_lo = my_first - k0;
      const int c_hi = my_lim - k0;
      bool none = (my_seg == 0) || (c_hi < 0) || (c_lo > 127);
      int bound = 0x7fffffff;     // keys below it need v0, keys from it on need v1
      bool v0 = true, v1 = true;
      if (sparse && !none) {
        const SparseRow sr = sparse_row(args.sp, b, h, args.Hq, args.S, qi, my_start, k0, 128);
        bound = sr.bound; v0 = sr.v0; v1 = sr.v1;
        none = !v0 && !v1;
      }
      const bool all = !none && (c_lo <= 0) && (c_hi >= 127) && v0 && v1;
      if (!mbar_wait(&s_full[t], sph, abort_flag, st, SITE_F_SM_S, budget)) {
        ok = false;
        break;
      }
      sph ^= 1u;
      tc_fence_after();
      // ---- the whole score row in registers: one TMEM round trip ----
      uint32_t sc[128];
      tmem_ld32x4(tmem_s_of(t) + lane_off, sc);
      tmem_ld_wait();
      if (!all) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          unsigned vis = none ? 0u : (bits_from(c_lo - 32 * c) & bits_upto(c_hi - 32 * c));
          if (sparse) {
            const unsigned above = bits_from(bound - k0 - 32 * c);      // keys >= bound
            vis &= (v0 ? ~above : 0u) | (v1 ? above : 0u);
          }
          if (vis != 0xffffffffu) {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (!((vis >> e) & 1u)) sc[c * 32 + e] = 0xff800000u;     // -inf
          }
        }
      }
      // ---- row maximum of the raw scores (the scale is positive), four independent chains ----
      float mq[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        mq[c] = __uint_as_float(sc[c * 32]);
#pragma unroll
        for (int e = 1; e < 31; e += 2)
          mq[c] = fmax3(mq[c], __uint_as_float(sc[c * 32 + e]), __uint_as_float(sc[c * 32 + e + 1]));
        mq[c] = fmaxf(mq[c], __uint_as_float(sc[c * 32 + 31]));
      }
      const float mx = fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3])) * args.scale_log2;
      // ---- lazy running maximum ----
      const bool need = (mx > m_ref + 8.f) || (m_ref == -INFINITY && mx > -INFINITY);
      float alpha = 1.f;
      if (need) {
        alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - mx);
        m_ref = mx;
        l_sum *= alpha;
      }
      // PV(i-1) was issued before S(i) and the tensor core completes MMAs in issue order, so the
      // scores of this tile being ready means O holds every earlier tile: no separate wait.
      if (i > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
        for (int c = 0; c < D / 8; ++c) {      // narrow chunks: the score row stays in registers
          uint32_t rr[8];
          tmem_ld8(tmem_o_of(t) + lane_off + c * 8, rr);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 8; ++e) rr[e] = __float_as_uint(__uint_as_float(rr[e]) * alpha);
          tmem_st8(tmem_o_of(t) + lane_off + c * 8, rr);
        }
        tmem_st_wait();
      }
      // ---- P = exp2(s * scale - m): packed fma / add on pairs; P goes back into TMEM as bf16 pairs
      // over the first 64 columns of the score row this thread already holds in registers ----
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      const uint64_t neg_m2 = pack_f32x2(-m_use, -m_use);
      uint64_t rs2 = pack_f32x2(0.f, 0.f);
#pragma unroll
      for (int qt = 0; qt < 8; ++qt) {           // 16 scores -> 8 packed columns per store
        uint32_t pw[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const int e = qt * 16 + jj * 2;
          const uint64_t x2 = fma_f32x2(pack_f32x2(__uint_as_float(sc[e]), __uint_as_float(sc[e + 1])), scale2, neg_m2);
          float xa, xb;
          unpack_f32x2(x2, xa, xb);
          const float pa = fast_exp2(xa), pb = fast_exp2(xb);
          rs2 = add_f32x2(rs2, pack_f32x2(pa, pb));
          pw[jj] = pack_bf16(pa, pb);
        }
        tmem_st8(tmem_s_of(t) + lane_off + qt * 8, pw);
      }
      tmem_st_wait();
      float rs_a, rs_b;
      unpack_f32x2(rs2, rs_a, rs_b);
      l_sum += rs_a + rs_b;
      tc_fence_before();
      mbar_arrive(&p_full[t]);
    }
    // ---- finalize ----
    if (ok && n_mine > 0) {
      ok = mbar_wait(&pv_done[t], static_cast<uint32_t>(n_mine - 1) & 1u, abort_flag, st, SITE_F_SM_PV, budget);
      tc_fence_after();
    }
    const bool any_bad = named_bar_or(2 + t, 128, !ok);
    if (!any_bad && tile_valid[t]) {
      const float inv = (l_sum > 0.f) ? 1.f / l_sum : 0.f;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t rr[32];
        if (n_mine > 0) {
          tmem_ld32(tmem_o_of(t) + lane_off + c * 32, rr);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) rr[e] = 0u;
        }
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(rr[jj * 8 + 0]) * inv, __uint_as_float(rr[jj * 8 + 1]) * inv);
          v.y = pack_bf16(__uint_as_float(rr[jj * 8 + 2]) * inv, __uint_as_float(rr[jj * 8 + 3]) * inv);
          v.z = pack_bf16(__uint_as_float(rr[jj * 8 + 4]) * inv, __uint_as_float(rr[jj * 8 + 5]) * inv);
          v.w = pack_bf16(__uint_as_float(rr[jj * 8 + 6]) * inv, __uint_as_float(rr[jj * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(obuf + (c / 2) * 16384 + sw128_offset(r, (c % 2) * 4 + jj)) = v;
        }
      }
      fence_proxy_async_smem();
      named_bar_sync(4 + t, 128);
      if (r == 0) {
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) tma_store_4d(&map_o, obuf + hf * 16384, hf * 64, h, q0 + t * 128, b);
        tma_commit_group();
        tma_wait_group<0>();
      }
      const float lse = (l_sum > 0.f) ? (m_ref + log2f(l_sum)) * 0.6931471805599453f : 0.f;
      args.lse[(static_cast<size_t>(b) * args.Hq + h) * args.Sq + qi_local] = lse;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D>
int launch_fwd(const FwdCall& c) {
  using L = FwdSmem<D>;
  const bool grouped = c.grp.desc != nullptr;
  const int Sq = grouped ? c.gathered_rows : (c.Sq > 0 ? c.Sq : c.S);
  // grouped: Q / O are the gathered rows, one batch and one head
  const uint64_t dq[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(grouped ? 1 : c.Hq), static_cast<uint64_t>(Sq),
                          static_cast<uint64_t>(grouped ? 1 : c.B)};
  const uint64_t dk[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(c.Hkv), static_cast<uint64_t>(c.S),
                          static_cast<uint64_t>(c.B)};
  const uint32_t box[4] = {64, 1, 128, 1};
  const uint64_t sq[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(c.q_row_stride),
                          static_cast<uint64_t>(c.q_row_stride) * Sq};
  const uint64_t sk[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(c.k_row_stride),
                          static_cast<uint64_t>(c.k_row_stride) * c.S};
  const uint64_t sv[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(c.v_row_stride),
                          static_cast<uint64_t>(c.v_row_stride) * c.S};
  const uint64_t so[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(c.o_row_stride),
                          static_cast<uint64_t>(c.o_row_stride) * Sq};
  const CUtensorMap* mq = get_tensor_map_4d(c.q, Elt::BF16, dq, sq, box, true);
  const CUtensorMap* mk = get_tensor_map_4d(c.k, Elt::BF16, dk, sk, box, true);
  const CUtensorMap* mv = get_tensor_map_4d(c.v, Elt::BF16, dk, sv, box, true);
  const CUtensorMap* mo = get_tensor_map_4d(c.o, Elt::BF16, dq, so, box, true);
  if (!mq || !mk || !mv || !mo) return 1;
  FwdArgs a{};
  a.B = c.B; a.S = c.S; a.Hq = grouped ? 1 : c.Hq; a.Hkv = grouped ? 1 : c.Hkv;
  a.Sq = Sq; a.q_off = c.q_off;
  a.scale_log2 = c.scale * 1.4426950408889634f;
  a.seg = c.seg; a.lim = c.lim; a.row_start = c.row_start; a.kv_lo = c.kv_lo; a.kv_hi = c.kv_hi;
  a.lse = c.lse;
  a.sp = c.sp;
  a.grp = c.grp;
  a.kvf = c.kvf;
  a.status = device_status();
  a.spin_budget = c.spin_budget > 0 ? c.spin_budget : CTB_SPIN_BUDGET;
  auto kern = attn_fwd_kernel<D>;
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    CTB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES));
    configured_dev = dev;
  }
  const int grid = grouped ? Sq / 256 : c.B * c.Hq * ((Sq + 255) / 256);
  kern<<<grid, FWD_THREADS, L::BYTES, static_cast<cudaStream_t>(c.stream)>>>(*mq, *mk, *mv, *mo, a);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace attn
}  // namespace ctb

// q/k/v/o are [B, S, H, D] views with arbitrary row stride (elements between consecutive
// tokens), so the packed QKV projection output is read in place.  lse is [B, Hq, S] fp32.
CTB_API int ctb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* seg,
                         const int* lim, const int* row_start, const int* kv_lo, const int* kv_hi, int B,
                         int S, int Hq, int Hkv, int D, long q_row_stride, long k_row_stride, long v_row_stride,
                         long o_row_stride, float scale, long long spin_budget, void* stream) {
  if (S % 128) return ctb::fail("attention: sequence length must be a multiple of 128");
  if (Hq % Hkv) return ctb::fail("attention: Hq must be a multiple of Hkv");
  ctb::attn::FwdCall c{};
  c.q = q; c.k = k; c.v = v; c.o = o; c.lse = lse; c.seg = seg; c.lim = lim; c.row_start = row_start; c.kv_lo = kv_lo; c.kv_hi = kv_hi;
  c.B = B; c.S = S; c.Hq = Hq; c.Hkv = Hkv;
  c.q_row_stride = q_row_stride; c.k_row_stride = k_row_stride; c.v_row_stride = v_row_stride;
  c.o_row_stride = o_row_stride; c.scale = scale; c.spin_budget = spin_budget; c.stream = stream;
  if (D == 128) return ctb::attn::launch_fwd<128>(c);
  if (D == 64) return ctb::attn::launch_fwd<64>(c);
  return ctb::fail("attention: head_dim must be 64 or 128");
}

// Sequence-parallel forward: q / o hold the Sq queries [q_off, q_off + Sq) of every row, k / v all
// S keys; lse is [B, Hq, Sq].  q_off and Sq must be multiples of 128.
CTB_API int ctb_attn_fwd_range(const void* q, const void* k, const void* v, void* o, float* lse, const int* seg,
                               const int* lim, const int* row_start, const int* kv_lo, const int* kv_hi,
                               int B, int S, int Sq, int q_off, int Hq, int Hkv, int D, long q_row_stride,
                               long k_row_stride, long v_row_stride, long o_row_stride, float scale,
                               long long spin_budget, void* stream) {
  if (S % 128 || Sq % 128 || q_off % 128 || q_off < 0 || q_off + Sq > S)
    return ctb::fail("attention: S, Sq and q_off must be multiples of 128 with q_off + Sq <= S");
  if (Hq % Hkv) return ctb::fail("attention: Hq must be a multiple of Hkv");
  ctb::attn::FwdCall c{};
  c.q = q; c.k = k; c.v = v; c.o = o; c.lse = lse; c.seg = seg; c.lim = lim; c.row_start = row_start; c.kv_lo = kv_lo; c.kv_hi = kv_hi;
  c.B = B; c.S = S; c.Sq = Sq; c.q_off = q_off; c.Hq = Hq; c.Hkv = Hkv;
  c.q_row_stride = q_row_stride; c.k_row_stride = k_row_stride; c.v_row_stride = v_row_stride;
  c.o_row_stride = o_row_stride; c.scale = scale; c.spin_budget = spin_budget; c.stream = stream;
  if (D == 128) return ctb::attn::launch_fwd<128>(c);
  if (D == 64) return ctb::attn::launch_fwd<64>(c);
  return ctb::fail("attention: head_dim must be 64 or 128");
}

// Block-sparse (MoBA) forward: same operands plus the routing described at SparseArgs.  `it_off`
// has B * Hq * ceil(S / 256) + 1 entries in the order (query pair descending, batch, head) of the grid.
CTB_API int ctb_attn_fwd_sparse(const void* q, const void* k, const void* v, void* o, float* lse, const int* seg,
                                const int* lim, const int* row_start, const int* kv_lo, const int* kv_hi,
                                const int* it_off, const int* it_cnt, int it_stride, const int* it_list,
                                const unsigned* sel, const int* doc_start, int block, int words, int B, int S, int Hq,
                                int Hkv, int D, long q_row_stride,
                                long k_row_stride, long v_row_stride, long o_row_stride, float scale,
                                long long spin_budget, void* stream) {
  if (S % 128) return ctb::fail("attention: sequence length must be a multiple of 128");
  if (Hq % Hkv) return ctb::fail("attention: Hq must be a multiple of Hkv");
  if (block < 128) return ctb::fail("sparse attention: the routing block must hold at least 128 tokens");
  ctb::attn::FwdCall c{};
  c.q = q; c.k = k; c.v = v; c.o = o; c.lse = lse; c.seg = seg; c.lim = lim; c.row_start = row_start; c.kv_lo = kv_lo; c.kv_hi = kv_hi;
  c.B = B; c.S = S; c.Hq = Hq; c.Hkv = Hkv;
  c.q_row_stride = q_row_stride; c.k_row_stride = k_row_stride; c.v_row_stride = v_row_stride;
  c.o_row_stride = o_row_stride; c.scale = scale; c.spin_budget = spin_budget; c.stream = stream;
  c.sp.it_off = it_off; c.sp.it_cnt = it_cnt; c.sp.it_stride = it_stride; c.sp.it_list = it_list; c.sp.sel = sel;
  c.sp.doc_start = doc_start; c.sp.block = block; c.sp.words = words;
  if (D == 128) return ctb::attn::launch_fwd<128>(c);
  if (D == 64) return ctb::attn::launch_fwd<64>(c);
  return ctb::fail("attention: head_dim must be 64 or 128");
}

// Grouped MoBA forward (see GroupArgs): qg / og are [gathered_rows, D] contiguous, lse_g
// [gathered_rows]; k / v are the usual [B,S,Hkv,D] views; desc has gathered_rows / 256 entries.
CTB_API int ctb_attn_fwd_grouped(const void* qg, const void* k, const void* v, void* og, float* lse_g, const void* desc,
                                 int gathered_rows, int block, int B, int S, int Hkv, int D, long k_row_stride,
                                 long v_row_stride, float scale, long long spin_budget, void* stream) {
  if (S % 128 || block % 128 || block < 128) return ctb::fail("grouped attention: S and the block must be multiples of 128");
  if (gathered_rows <= 0 || gathered_rows % 256) return ctb::fail("grouped attention: gathered rows must be a positive multiple of 256");
  if (B > 0xffff || Hkv > 0x7fff) return ctb::fail("grouped attention: batch or head count too large for the descriptor");
  ctb::attn::FwdCall c{};
  c.q = qg; c.k = k; c.v = v; c.o = og; c.lse = lse_g;
  c.B = B; c.S = S; c.Hq = Hkv; c.Hkv = Hkv;
  c.q_row_stride = D; c.k_row_stride = k_row_stride; c.v_row_stride = v_row_stride; c.o_row_stride = D;
  c.scale = scale; c.spin_budget = spin_budget; c.stream = stream;
  c.grp.desc = static_cast<const int4*>(desc); c.grp.block = block; c.gathered_rows = gathered_rows;
  if (D == 128) return ctb::attn::launch_fwd<128>(c);
  if (D == 64) return ctb::attn::launch_fwd<64>(c);
  return ctb::fail("attention: head_dim must be 64 or 128");
}

// Sequence-parallel forward over gathered K / V whose all-gather may still be in flight: k and v are
// the halves of one [B, S, row_elems] buffer (k at its start); flags / chunk / epoch as in KvFlags.
CTB_API int ctb_attn_fwd_gathered(const void* q, const void* k, const void* v, void* o, float* lse, const int* seg,
                                  const int* lim, const int* row_start, const int* kv_lo, const int* kv_hi,
                                  int B, int S, int Sq, int q_off, int Hq, int Hkv, int D, long q_row_stride,
                                  long k_row_stride, long v_row_stride, long o_row_stride, float scale,
                                  const unsigned* kv_flags, long kv_chunk, long kv_row_elems, unsigned kv_epoch,
                                  long long spin_budget, void* stream) {
  if (S % 128 || Sq % 128 || q_off % 128 || q_off < 0 || q_off + Sq > S)
    return ctb::fail("attention: S, Sq and q_off must be multiples of 128 with q_off + Sq <= S");
  if (Hq % Hkv) return ctb::fail("attention: Hq must be a multiple of Hkv");
  if (kv_flags != nullptr && (kv_chunk <= 0 || kv_row_elems <= 0)) return ctb::fail("attention: bad K/V flag geometry");
  ctb::attn::FwdCall c{};
  c.q = q; c.k = k; c.v = v; c.o = o; c.lse = lse; c.seg = seg; c.lim = lim; c.row_start = row_start; c.kv_lo = kv_lo; c.kv_hi = kv_hi;
  c.B = B; c.S = S; c.Sq = Sq; c.q_off = q_off; c.Hq = Hq; c.Hkv = Hkv;
  c.q_row_stride = q_row_stride; c.k_row_stride = k_row_stride; c.v_row_stride = v_row_stride;
  c.o_row_stride = o_row_stride; c.scale = scale; c.spin_budget = spin_budget; c.stream = stream;
  c.kvf.flags = kv_flags; c.kvf.chunk = kv_chunk; c.kvf.row_elems = kv_row_elems; c.kvf.epoch = kv_epoch;
  if (D == 128) return ctb::attn::launch_fwd<128>(c);
  if (D == 64) return ctb::attn::launch_fwd<64>(c);
  return ctb::fail("attention: head_dim must be 64 or 128");
}
