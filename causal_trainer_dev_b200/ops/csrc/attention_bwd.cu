// Flash attention backward for sm_100a, two kernels from one template, no atomics:
//
//   MODE_DKV  KV-tile-owned: a CTA owns 128 keys of one KV head and walks every query
//             block (64 rows) of every query head of the GQA group that can see them.
//                 S^T = K Q^T          dP^T = V dO^T            (tcgen05, TMEM)
//                 P^T = exp2(S^T c - lse),  dS^T = P^T (dP^T - delta)   (registers; the per-query
//                 statistics arrive negated and in log2 units, ready for packed fma / add)
//                 dV += P^T dO         dK += dS^T Q             (tcgen05, TMEM accumulators)
//             The reduction over the group's query heads happens in the TMEM accumulators.
//   MODE_DQ   Q-tile-owned: a CTA owns 128 query rows of one query head and walks the
//             64-key blocks it can see:  S = Q K^T, dP = dO V^T, dS = P (dP - delta),
//             dQ += dS K.
//
// Structure of both: resident operand pair X (K,V or Q,dO), streamed pair Y (Q,dO or K,V)
// through a 4-stage TMA ring, four compute warpgroups that share every Y block (16 of its 64
// columns each) over two alternating S / dP buffers, so the tensor core works on block i+1 and
// on the accumulate MMAs of block i-1 while block i is exponentiated.  P^T / dS go back into TMEM
// as bf16 pairs over the scores they were computed from and are the TMEM A operands of the
// accumulate MMAs (they never cross shared memory); the Y tiles are reused in place as MN-major
// B operands.
//
// Reference counterparts: causal_trainer_attention_dq / _dkv
// (src/causal_trainer/kernels/efficient_attention.py:985-1173, 1270-1436); the psum that
// follows the reference's dK/dV kernel is not needed on one GPU because the group is reduced
// in TMEM.
#include <type_traits>

#include "attention.h"

namespace ctb {
namespace attn {

constexpr int BWD_THREADS = 640;   // 4 service warps + 4 compute warpgroups
constexpr int Y_STAGES = 4;

enum : unsigned {
  SITE_B_PROD = 0x0301,
  SITE_B_MMA_X = 0x0302,
  SITE_B_MMA_Y = 0x0303,
  SITE_B_MMA_T = 0x0304,
  SITE_B_CW_S = 0x0305,
  SITE_B_CW_ACC = 0x0307,
};

template <int D>
struct BwdSmem {
  static constexpr int HALVES = D / 64;
  static constexpr int XT = HALVES * 16384;   // 128-row resident tile
  static constexpr int YT = HALVES * 8192;    // 64-row streamed tile
  static constexpr int OFF_X = 0;             // X1, X2
  static constexpr int OFF_Y = 2 * XT;        // stages of (Y1, Y2)
  static constexpr int OFF_BAR = OFF_Y + Y_STAGES * 2 * YT;
  static constexpr int OFF_STAT = OFF_BAR + 256;   // per Y stage: 64 x -lse*log2(e), 64 x -delta of the block's queries (DKV)
  static constexpr int BYTES = OFF_STAT + Y_STAGES * 512 + 1024;
};

template <int D, int MODE>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                const __grid_constant__ CUtensorMap map_out1, const __grid_constant__ CUtensorMap map_out2,
                const BwdArgs args) {
  using L = BwdSmem<D>;
  constexpr int HALVES = L::HALVES;
  constexpr bool DKV = (MODE == MODE_DKV);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* x_full = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* y_full = x_full + 1;
  uint64_t* y_empty = y_full + Y_STAGES;
  uint64_t* s_full = y_empty + Y_STAGES;   // [2] S and dP of buffer u ready
  uint64_t* t_full = s_full + 2;           // [2] P^T / dS tiles of buffer u written
  uint64_t* acc_full = t_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  DeviceStatus* st = args.status;
  const long long budget = args.spin_budget;
  const int group = args.Hq / args.Hkv;
  const int nb128 = args.S / 128;
  const int nb64 = args.S / 64;

  // ---- work item ----
  // grouped MoBA (see GroupArgs): gathered rows of one group against the keys of its block, no masks
  const bool grouped = args.grp.desc != nullptr;
  int4 gd = make_int4(0, 0, 0, 0);
  if (grouped) {
    gd = __ldg(args.grp.desc + blockIdx.x);
    if (gd.w <= 0) return;                       // unused capacity: the whole CTA leaves
  }
  int idx = blockIdx.x;
  int b, head, x0, y_lo64, y_n64, heads_in_loop;
  if (grouped) {
    // X = this CTA's resident tile: 128 keys of the block (dK/dV) or 128 gathered rows (dQ);
    // Y = 64-row blocks of the group's gathered rows (dK/dV) or of the block's keys (dQ).
    b = DKV ? (gd.x & 0xffff) : 0;
    head = DKV ? (gd.x >> 16) : 0;
    x0 = DKV ? gd.y : static_cast<int>(blockIdx.x) * 128;
    y_lo64 = 0;
    y_n64 = DKV ? gd.w / 64 : args.grp.block / 64;
    heads_in_loop = 1;
  } else if (DKV) {
    head = idx % args.Hkv;      // kv head
    idx /= args.Hkv;
    b = idx % args.B;
    const int kb = idx / args.B;  // ascending: key blocks near the start see the most queries
    x0 = kb * 128;
    // only the queries this rank holds, [q_off, q_off + Sq), are walked
    const int qlo = max(args.q_lo[b * nb128 + kb], args.q_off);
    const int qhi = min(args.q_hi[b * nb128 + kb], args.q_off + args.Sq);
    y_lo64 = qlo / 64;
    y_n64 = qhi > qlo ? (qhi + 63) / 64 - y_lo64 : 0;
    heads_in_loop = group;
  } else {
    head = idx % args.Hq;       // query head
    idx /= args.Hq;
    b = idx % args.B;
    const int qb = args.Sq / 128 - 1 - idx / args.B;  // descending: late query blocks see the most keys
    x0 = qb * 128;                                    // row of the local Q / dO / dQ
    const int klo = args.kv_lo[b * nb128 + args.q_off / 128 + qb];
    const int khi = args.kv_hi[b * nb128 + args.q_off / 128 + qb];
    y_lo64 = klo / 64;
    y_n64 = khi > klo ? (khi + 63) / 64 - y_lo64 : 0;
    heads_in_loop = 1;
  }
  int n_iter = y_n64 * heads_in_loop;
  const int hkv = grouped ? (gd.x >> 16) : (DKV ? head : head / group);
  const int kbatch = grouped ? (gd.x & 0xffff) : b;     // batch of the K / V / dK / dV tensors
  const int y_base = grouped ? (DKV ? gd.z : gd.y) : 0; // first row (dK/dV) or key (dQ) of the streamed operand
  // Block-sparse routing: the (64-row block, head) pairs come from a list instead of a range.
  const bool sparse = args.sp.it_list != nullptr;
  const int* it_list = nullptr;
  if (sparse) {
    int base;
    sparse_list(args.sp, blockIdx.x, base, n_iter);
    it_list = args.sp.it_list + base;
  }
  // iteration -> (64-row block of the streamed operand, query head)
  auto y_block = [&](int it) -> int { return sparse ? (__ldg(it_list + it) & 0xffffff) : y_lo64 + it % y_n64; };
  auto y_head = [&](int it) -> int {
    if (grouped) return 0;
    if (!DKV) return head;
    return hkv * group + (sparse ? (__ldg(it_list + it) >> 24) : it / y_n64);
  };

  if (threadIdx.x == 0) {
    mbar_init(x_full, 1);
    for (int s = 0; s < Y_STAGES; ++s) {
      mbar_init(&y_full[s], 1);
      mbar_init(&y_empty[s], 1);
    }
    for (int u = 0; u < 2; ++u) {
      mbar_init(&s_full[u], 1);
      mbar_init(&t_full[u], 512);
    }
    mbar_init(acc_full, 1);
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
  // S^T / dP^T (or S / dP) of block buffer u: 64 columns each (address arithmetic, not arrays: a
  // runtime index into a local array would go through local memory)
  auto tmem_s = [&](int u) -> uint32_t { return tmem_base + static_cast<uint32_t>(u) * 64u; };
  auto tmem_dp = [&](int u) -> uint32_t { return tmem_base + 128u + static_cast<uint32_t>(u) * 64u; };
  const uint32_t tmem_acc1 = tmem_base + 256;       // dV (DKV) or dQ (DQ)
  const uint32_t tmem_acc2 = tmem_base + 256 + D;   // dK (DKV)

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0 && n_iter > 0) {
      mbar_expect_tx(x_full, 2 * L::XT);
      const CUtensorMap* mx1 = DKV ? &map_k : &map_q;
      const CUtensorMap* mx2 = DKV ? &map_v : &map_do;
      const int xh = DKV ? hkv : head;
      const int xb = DKV ? kbatch : b;
#pragma unroll
      for (int hf = 0; hf < HALVES; ++hf) {
        tma_load_4d(smem + L::OFF_X + hf * 16384, mx1, x_full, hf * 64, xh, x0, xb);
        tma_load_4d(smem + L::OFF_X + L::XT + hf * 16384, mx2, x_full, hf * 64, xh, x0, xb);
      }
      const CUtensorMap* my1 = DKV ? &map_q : &map_k;
      const CUtensorMap* my2 = DKV ? &map_do : &map_v;
      uint32_t stage = 0, phase = 0;
      for (int it = 0; it < n_iter; ++it) {
        const int yh = DKV ? y_head(it) : hkv;
        const int ybatch = DKV ? b * (grouped ? 0 : 1) : kbatch;
        const int y0 = y_base + y_block(it) * 64 - (DKV ? args.q_off : 0);   // streamed queries are stored locally
        if (!mbar_wait(&y_empty[stage], phase ^ 1u, abort_flag, st, SITE_B_PROD, budget)) break;
        mbar_expect_tx(&y_full[stage], 2 * L::YT + (DKV ? 512 : 0));
        uint8_t* dst = smem + L::OFF_Y + stage * 2 * L::YT;
        if (DKV) {
          // the per-query statistics of the block travel with it (256 B each, 256 B aligned)
          const size_t stat = grouped ? static_cast<size_t>(y0) : (static_cast<size_t>(b) * args.Hq + yh) * args.Sq + y0;
          tma_load_1d(smem + L::OFF_STAT + stage * 512, args.neg_lse2 + stat, 256, &y_full[stage]);
          tma_load_1d(smem + L::OFF_STAT + stage * 512 + 256, args.neg_delta + stat, 256, &y_full[stage]);
        }
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) {
          tma_load_4d(dst + hf * 8192, my1, &y_full[stage], hf * 64, yh, y0, ybatch);
          tma_load_4d(dst + L::YT + hf * 8192, my2, &y_full[stage], hf * 64, yh, y0, ybatch);
        }
        if (++stage == Y_STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, false, false);
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, false, true);
      const uint32_t x1 = smem_u32(smem + L::OFF_X);
      const uint32_t x2 = smem_u32(smem + L::OFF_X + L::XT);
      bool ok = mbar_wait(x_full, 0, abort_flag, st, SITE_B_MMA_X, budget);
      uint32_t stage = 0, phase = 0;       // stage of the block whose S/dP is issued next
      uint32_t astage = 0;                 // stage of the block whose accumulate MMAs come next
      uint32_t tph[2] = {0, 0};
      auto accumulate_block = [&](int k) -> bool {
        const int u = k & 1;
        if (!mbar_wait(&t_full[u], tph[u], abort_flag, st, SITE_B_MMA_T, budget)) return false;
        tph[u] ^= 1u;
        tc_fence_after();
        const uint32_t y1 = smem_u32(smem + L::OFF_Y + astage * 2 * L::YT);
        const uint32_t y2 = y1 + L::YT;
        // P^T / dS are bf16 pairs in TMEM: the 16 columns of group kk sit in the first 8 columns of
        // the group's own 16-column slice of the S / dP buffer (written over the scores it read)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          if (DKV) {
            umma_bf16_ts(tmem_acc1, tmem_s(u) + 16 * kk, desc_mnmajor(y2, kk, 8192), idesc_acc, (k | kk) != 0 ? 1u : 0u);
            umma_bf16_ts(tmem_acc2, tmem_dp(u) + 16 * kk, desc_mnmajor(y1, kk, 8192), idesc_acc, (k | kk) != 0 ? 1u : 0u);
          } else {
            umma_bf16_ts(tmem_acc1, tmem_dp(u) + 16 * kk, desc_mnmajor(y1, kk, 8192), idesc_acc, (k | kk) != 0 ? 1u : 0u);
          }
        }
        umma_commit(&y_empty[astage]);
        if (++astage == Y_STAGES) astage = 0;
        return true;
      };
      for (int it = 0; ok && it < n_iter; ++it) {
        const int u = it & 1;
        if (!mbar_wait(&y_full[stage], phase, abort_flag, st, SITE_B_MMA_Y, budget)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t y1 = smem_u32(smem + L::OFF_Y + stage * 2 * L::YT);
        const uint32_t y2 = y1 + L::YT;
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16(tmem_s(u), desc_kmajor(x1 + (k / 4) * 16384, k % 4), desc_kmajor(y1 + (k / 4) * 8192, k % 4),
                    idesc_s, k != 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16(tmem_dp(u), desc_kmajor(x2 + (k / 4) * 16384, k % 4), desc_kmajor(y2 + (k / 4) * 8192, k % 4),
                    idesc_s, k != 0 ? 1u : 0u);
        umma_commit(&s_full[u]);
        if (++stage == Y_STAGES) {
          stage = 0;
          phase ^= 1u;
        }
        if (it > 0) ok = accumulate_block(it - 1);
      }
      if (ok) ok = accumulate_block(n_iter - 1);
      if (ok) umma_commit(acc_full);
    }
  } else if (warp >= 4) {
    // ------------------------------ compute warpgroups ------------------------------
    // Four compute warpgroups work on every block together: warpgroup wg takes columns
    // [16 wg, 16 wg + 16) of the 64-column block, so one block costs a single short pass (one TMEM
    // round trip, 16 exponentials per thread).  The S / dP buffers alternate from block to block:
    // the tensor core fills buffer 1 - u and runs the accumulate MMAs of the previous block while
    // buffer u is exponentiated.
    const int wg = (warp - 4) >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    // position in the whole sequence of this thread's row: a key (DKV) or a local query (DQ)
    const int xi = x0 + r + (DKV ? 0 : args.q_off);
    const int xi_local = x0 + r;
    const int row_seg = grouped ? 1 : args.seg[b * args.S + xi];
    // interval of visible columns (whole-sequence positions): see the mask below
    int row_a, row_b;
    if (grouped) {
      row_a = -(1 << 30);       // everything is visible: padding rows hold zeros and contribute zero
      row_b = 1 << 30;
    } else if (DKV) {
      row_a = args.first_q[b * args.S + xi];
      row_b = args.run_end[b * args.S + xi];
    } else {
      row_a = args.run_start[b * args.S + xi];
      row_b = (args.lim != nullptr) ? args.lim[b * args.S + xi] : xi;
    }
    const int row_start = sparse ? args.sp.doc_start[b * args.S + xi] : 0;
    // DKV: the document-relative block of this key is the bit every query column is tested for
    const int row_blk = (sparse && DKV) ? (xi - row_start) / args.sp.block : 0;
    float neg_lse2 = 0.f, neg_delta = 0.f;      // DQ: per-row statistics (stored negated, lse in log2 units)
    if (!DKV) {
      const size_t at = grouped ? static_cast<size_t>(xi_local) : (static_cast<size_t>(b) * args.Hq + head) * args.Sq + xi_local;
      neg_lse2 = args.neg_lse2[at];
      neg_delta = args.neg_delta[at];
    }
    bool ok = true;
    uint32_t sph = 0;                      // bit u: phase parity of s_full[u]
    const uint64_t scale2 = pack_f32x2(args.scale_log2, args.scale_log2);
    // dense walk: (block, head) advance without a division per iteration
    int walk_block = 0, walk_head = 0;
    uint32_t ystage = 0, yphase = 0;        // stage of the Y ring that holds block `it` (and its statistics)
    for (int it = 0; it < n_iter; ++it) {
      const int u = it & 1;
      int yb, hq;
      if (sparse) {
        const int entry = __ldg(it_list + it);
        yb = entry & 0xffffff;
        hq = DKV ? hkv * group + (entry >> 24) : head;
      } else {
        yb = y_lo64 + walk_block;
        hq = DKV ? hkv * group + walk_head : head;
        if (++walk_block == y_n64) {
          walk_block = 0;
          ++walk_head;
        }
      }
      const int y0 = yb * 64;                   // (grouped: relative to the group, and nothing is masked)
      const int base = y0 + 16 * wg;            // first column of this thread
      // ---- visibility of this row against its 16 columns, as a bit mask.  The keys a query sees
      // and the queries that see a key are both contiguous intervals (runs are contiguous):
      //   DQ   row = query xi,  columns = keys     [start[xi], lim[xi]]
      //   DKV  row = key xi,    columns = queries  [first_q[xi], end[xi]]
      unsigned vis = (row_seg == 0) ? 0u : (bits_from(row_a - base) & bits_upto(row_b - base) & 0xffffu);
      if (sparse && vis != 0u) {
        if (DKV) {
          if ((row_blk >> 5) >= args.sp.words) {
            vis = 0u;
          } else {
            // when every query of the block selected this key's block the selection adds nothing
            const unsigned aw = __ldg(args.sp.allsel + ((static_cast<size_t>(b) * args.Hq + hq) * nb64 + yb) * args.sp.words +
                                      (row_blk >> 5));
            if (!((aw >> (row_blk & 31)) & 1u)) {
              // per-query selection bit of this key's block, for the 16 columns of this thread
              const unsigned* col_sel = args.sp.sel + ((static_cast<size_t>(b) * args.Hq + hq) * args.S + base) * args.sp.words +
                                        (row_blk >> 5);
              const int bit = row_blk & 31;
              unsigned selbits = 0u;
#pragma unroll 4
              for (int e = 0; e < 16; ++e)
                selbits |= ((__ldg(col_sel + static_cast<size_t>(e) * args.sp.words) >> bit) & 1u) << e;
              vis &= selbits;
            }
          }
        } else {
          const SparseRow sr = sparse_row(args.sp, b, head, args.Hq, args.S, xi, row_start, y0, 64);
          const unsigned above = bits_from(sr.bound - base);               // keys >= bound
          vis &= (sr.v0 ? ~above : 0u) | (sr.v1 ? above : 0u);
        }
      }
      const bool all = vis == 0xffffu;
      // DKV: per-query statistics of this thread's 16 columns, staged beside the block by the producer
      const float4* lse_col = reinterpret_cast<const float4*>(smem + L::OFF_STAT + ystage * 512) + 4 * wg;
      const float4* delta_col = lse_col + 16;
      if (!mbar_wait(&s_full[u], (sph >> u) & 1u, abort_flag, st, SITE_B_CW_S, budget)) {
        ok = false;
        break;
      }
      sph ^= 1u << u;
      if (DKV) {
        // S was computed from this stage, so its bytes have landed; the wait makes the statistics
        // written by the bulk copy visible to this thread
        if (!mbar_wait(&y_full[ystage], yphase, abort_flag, st, SITE_B_CW_S, budget)) {
          ok = false;
          break;
        }
      }
      // (the accumulate MMAs of block it - 2 read P^T / dS from this buffer; they were issued before
      // the S / dP MMAs of this block and the tensor core completes MMAs in issue order)
      tc_fence_after();
      uint32_t rs[16], rd[16];
      tmem_ld16(tmem_s(u) + lane_off + 16 * wg, rs);
      tmem_ld16(tmem_dp(u) + lane_off + 16 * wg, rd);
      tmem_ld_wait();
      // Eight columns at a time: probabilities and dS are packed and stored as soon as they exist.
      // MASKED = false is the path of a warp whose rows all see all 16 columns: no selects.
      auto compute16 = [&](auto masked_tag) {
        constexpr bool MASKED = decltype(masked_tag)::value;
#pragma unroll
        for (int gg = 0; gg < 2; ++gg) {
          uint32_t pw[4], dw[4];
#pragma unroll
          for (int h4 = 0; h4 < 2; ++h4) {
            const int e4 = gg * 2 + h4;                  // group of four of the 16 columns
            uint64_t l2[2], dl[2];                       // negated statistics, two columns per word
            if (DKV) {
              const float4 lv = lse_col[e4];
              const float4 dv = delta_col[e4];
              l2[0] = pack_f32x2(lv.x, lv.y);
              l2[1] = pack_f32x2(lv.z, lv.w);
              dl[0] = pack_f32x2(dv.x, dv.y);
              dl[1] = pack_f32x2(dv.z, dv.w);
            } else {
              l2[0] = l2[1] = pack_f32x2(neg_lse2, neg_lse2);
              dl[0] = dl[1] = pack_f32x2(neg_delta, neg_delta);
            }
            // p = exp2(s * scale - lse), dS = p * (dP - delta): two columns per packed instruction
#pragma unroll
            for (int pr = 0; pr < 2; ++pr) {
              const int e = e4 * 4 + pr * 2;
              const uint64_t x2 = fma_f32x2(pack_f32x2(__uint_as_float(rs[e]), __uint_as_float(rs[e + 1])), scale2, l2[pr]);
              float xa, xb;
              unpack_f32x2(x2, xa, xb);
              float pa = fast_exp2(xa), pb = fast_exp2(xb);
              if (MASKED) {
                if (!((vis >> e) & 1u)) pa = 0.f;
                if (!((vis >> (e + 1)) & 1u)) pb = 0.f;
              }
              const uint64_t d2 = add_f32x2(pack_f32x2(__uint_as_float(rd[e]), __uint_as_float(rd[e + 1])), dl[pr]);
              const uint64_t ds2 = mul_f32x2(pack_f32x2(pa, pb), d2);
              float da, db;
              unpack_f32x2(ds2, da, db);
              pw[h4 * 2 + pr] = pack_bf16(pa, pb);
              dw[h4 * 2 + pr] = pack_bf16(da, db);
            }
          }
          if (DKV) tmem_st4(tmem_s(u) + lane_off + 16 * wg + 4 * gg, pw);
          tmem_st4(tmem_dp(u) + lane_off + 16 * wg + 4 * gg, dw);
        }
      };
      if (__all_sync(0xffffffffu, all)) compute16(std::false_type{});
      else compute16(std::true_type{});
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&t_full[u]);
      if (++ystage == Y_STAGES) {
        ystage = 0;
        yphase ^= 1u;
      }
    }
    // the epilogue pairs the warpgroups: pair u converts accumulator u, each warpgroup half of it
    const int u = wg & 1;
    const int half = wg >> 1;
    // ---- epilogue: accumulators -> bf16 -> staging -> TMA store ----
    if (ok && n_iter > 0) {
      ok = mbar_wait(acc_full, 0, abort_flag, st, SITE_B_CW_ACC, budget);
      tc_fence_after();
    }
    const bool any_bad = named_bar_or(2 + u, 256, !ok);
    const bool writes = DKV || (u == 0);
    if (!any_bad && writes) {
      // DKV: warpgroup 0 stores dV, warpgroup 1 stores dK (scaled); DQ: warpgroup 0 stores dQ (scaled).
      const uint32_t acc = (DKV && u == 1) ? tmem_acc2 : tmem_acc1;
      const float mul = (DKV && u == 0) ? 1.f : args.scale;
      uint8_t* stage_buf = smem + L::OFF_X + u * L::XT;      // the resident tile u is dead now: [HALVES][128 rows][128 B]
      // the two warpgroups of the pair convert half of the head dimension each
#pragma unroll 1
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
        uint32_t rr[32];
        if (n_iter > 0) {
          tmem_ld32(acc + lane_off + c * 32, rr);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) rr[e] = 0u;
        }
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(rr[jj * 8 + 0]) * mul, __uint_as_float(rr[jj * 8 + 1]) * mul);
          v.y = pack_bf16(__uint_as_float(rr[jj * 8 + 2]) * mul, __uint_as_float(rr[jj * 8 + 3]) * mul);
          v.z = pack_bf16(__uint_as_float(rr[jj * 8 + 4]) * mul, __uint_as_float(rr[jj * 8 + 5]) * mul);
          v.w = pack_bf16(__uint_as_float(rr[jj * 8 + 6]) * mul, __uint_as_float(rr[jj * 8 + 7]) * mul);
          *reinterpret_cast<uint4*>(stage_buf + (c / 2) * 16384 + sw128_offset(r, (c % 2) * 4 + jj)) = v;
        }
      }
      fence_proxy_async_smem();
      named_bar_sync(4 + u, 256);
      if (r == 0 && half == 0) {
        const CUtensorMap* mo = (DKV && u == 1) ? &map_out2 : &map_out1;
        const int oh = DKV ? hkv : head;
        const int ob = DKV ? kbatch : b;
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) tma_store_4d(mo, stage_buf + hf * 16384, hf * 64, oh, x0, ob);
        tma_commit_group();
        tma_wait_group<0>();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D, int MODE>
int launch_bwd(const BwdCall& c) {
  using L = BwdSmem<D>;
  const bool grouped = c.grp.desc != nullptr;
  const int Sq = grouped ? c.gathered_rows : (c.Sq > 0 ? c.Sq : c.S);
  auto make = [&](const void* base, int heads, long row_stride, int rows, int seq, int batches) -> const CUtensorMap* {
    const uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(heads), static_cast<uint64_t>(seq),
                              static_cast<uint64_t>(batches)};
    const uint64_t strides[3] = {static_cast<uint64_t>(D), static_cast<uint64_t>(row_stride),
                                 static_cast<uint64_t>(row_stride) * seq};
    const uint32_t box[4] = {64, 1, static_cast<uint32_t>(rows), 1};
    return get_tensor_map_4d(base, Elt::BF16, dims, strides, box, true);
  };
  constexpr bool DKV = (MODE == MODE_DKV);
  // Resident operands use 128-row boxes, streamed operands 64-row boxes.
  // grouped: Q / dO / dQ are the gathered rows (one batch, one head)
  const int qh = grouped ? 1 : c.Hq, qb = grouped ? 1 : c.B;
  const CUtensorMap* mq = make(c.q, qh, c.q_row_stride, DKV ? 64 : 128, Sq, qb);
  const CUtensorMap* mk = make(c.k, c.Hkv, c.k_row_stride, DKV ? 128 : 64, c.S, c.B);
  const CUtensorMap* mv = make(c.v, c.Hkv, c.v_row_stride, DKV ? 128 : 64, c.S, c.B);
  const CUtensorMap* mdo = make(c.dout, qh, c.do_row_stride, DKV ? 64 : 128, Sq, qb);
  const CUtensorMap* mo1 = DKV ? make(c.dv, c.Hkv, c.dv_row_stride, 128, c.S, c.B)
                               : make(c.dq, qh, c.dq_row_stride, 128, Sq, qb);
  const CUtensorMap* mo2 = DKV ? make(c.dk, c.Hkv, c.dk_row_stride, 128, c.S, c.B) : mo1;
  if (!mq || !mk || !mv || !mdo || !mo1 || !mo2) return 1;
  BwdArgs a{};
  a.B = c.B; a.S = c.S; a.Hq = c.Hq; a.Hkv = c.Hkv;
  a.Sq = Sq; a.q_off = c.q_off;
  a.scale = c.scale;
  a.scale_log2 = c.scale * 1.4426950408889634f;
  a.seg = c.seg; a.lim = c.lim; a.kv_lo = c.kv_lo; a.kv_hi = c.kv_hi; a.q_lo = c.q_lo; a.q_hi = c.q_hi;
  a.run_start = c.run_start; a.run_end = c.run_end; a.first_q = c.first_q;
  a.neg_lse2 = c.neg_lse2; a.neg_delta = c.neg_delta;
  a.sp = c.sp;
  a.grp = c.grp;
  a.status = device_status();
  a.spin_budget = c.spin_budget > 0 ? c.spin_budget : CTB_SPIN_BUDGET;
  auto kern = attn_bwd_kernel<D, MODE>;
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    CTB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES));
    configured_dev = dev;
  }
  const int grid = grouped ? c.ctas : (DKV ? c.B * c.Hkv * (c.S / 128) : c.B * c.Hq * (Sq / 128));
  if (grid <= 0) return 0;
  kern<<<grid, BWD_THREADS, L::BYTES, static_cast<cudaStream_t>(c.stream)>>>(*mq, *mk, *mv, *mdo, *mo1, *mo2, a);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace attn
}  // namespace ctb

// mode 0: dK/dV kernel, mode 1: dQ kernel.  All tensors are [B,S,H,D] views with a row
// stride; neg_lse2 = -lse * log2(e) and neg_delta = -sum_d O dO are [B,Hq,S] fp32 (ctb_attn_bwd_stats).
CTB_API int ctb_attn_bwd(int mode, const void* q, const void* k, const void* v, const void* dout, void* dq, void* dk,
                         void* dv, const float* neg_lse2, const float* neg_delta, const int* seg, const int* lim,
                         const int* kv_lo, const int* kv_hi, const int* q_lo, const int* q_hi, const int* run_start, const int* run_end, const int* first_q, int B, int S, int Hq,
                         int Hkv, int D, long q_rs, long k_rs, long v_rs, long do_rs, long dq_rs, long dk_rs,
                         long dv_rs, float scale, long long spin_budget, void* stream) {
  if (S % 128) return ctb::fail("attention: sequence length must be a multiple of 128");
  if (Hq % Hkv) return ctb::fail("attention: Hq must be a multiple of Hkv");
  ctb::attn::BwdCall c{};
  c.q = q; c.k = k; c.v = v; c.dout = dout; c.dq = dq; c.dk = dk; c.dv = dv; c.neg_lse2 = neg_lse2; c.neg_delta = neg_delta;
  c.seg = seg; c.lim = lim; c.kv_lo = kv_lo; c.kv_hi = kv_hi; c.q_lo = q_lo; c.q_hi = q_hi;
  c.run_start = run_start; c.run_end = run_end; c.first_q = first_q;
  c.B = B; c.S = S; c.Hq = Hq; c.Hkv = Hkv;
  c.q_row_stride = q_rs; c.k_row_stride = k_rs; c.v_row_stride = v_rs; c.do_row_stride = do_rs;
  c.dq_row_stride = dq_rs; c.dk_row_stride = dk_rs; c.dv_row_stride = dv_rs;
  c.scale = scale; c.spin_budget = spin_budget; c.stream = stream;
  using namespace ctb::attn;
  if (D == 128) return mode == 0 ? launch_bwd<128, MODE_DKV>(c) : launch_bwd<128, MODE_DQ>(c);
  if (D == 64) return mode == 0 ? launch_bwd<64, MODE_DKV>(c) : launch_bwd<64, MODE_DQ>(c);
  return ctb::fail("attention: head_dim must be 64 or 128");
}

// Sequence-parallel backward: q / dout / dq, neg_lse2 and neg_delta hold the Sq queries [q_off, q_off + Sq)
// of every row; k / v / dk / dv cover all S keys (dk / dv are this rank's partial sums).
CTB_API int ctb_attn_bwd_range(int mode, const void* q, const void* k, const void* v, const void* dout, void* dq,
                               void* dk, void* dv, const float* neg_lse2, const float* neg_delta, const int* seg,
                               const int* lim, const int* kv_lo, const int* kv_hi, const int* q_lo, const int* q_hi,
                               const int* run_start, const int* run_end, const int* first_q, int B, int S, int Sq, int q_off, int Hq, int Hkv, int D,
                               long q_rs, long k_rs, long v_rs, long do_rs, long dq_rs, long dk_rs, long dv_rs,
                               float scale, long long spin_budget, void* stream) {
  if (S % 128 || Sq % 128 || q_off % 128 || q_off < 0 || q_off + Sq > S)
    return ctb::fail("attention: S, Sq and q_off must be multiples of 128 with q_off + Sq <= S");
  if (Hq % Hkv) return ctb::fail("attention: Hq must be a multiple of Hkv");
  ctb::attn::BwdCall c{};
  c.q = q; c.k = k; c.v = v; c.dout = dout; c.dq = dq; c.dk = dk; c.dv = dv; c.neg_lse2 = neg_lse2; c.neg_delta = neg_delta;
  c.seg = seg; c.lim = lim; c.kv_lo = kv_lo; c.kv_hi = kv_hi; c.q_lo = q_lo; c.q_hi = q_hi;
  c.run_start = run_start; c.run_end = run_end; c.first_q = first_q;
  c.B = B; c.S = S; c.Sq = Sq; c.q_off = q_off; c.Hq = Hq; c.Hkv = Hkv;
  c.q_row_stride = q_rs; c.k_row_stride = k_rs; c.v_row_stride = v_rs; c.do_row_stride = do_rs;
  c.dq_row_stride = dq_rs; c.dk_row_stride = dk_rs; c.dv_row_stride = dv_rs;
  c.scale = scale; c.spin_budget = spin_budget; c.stream = stream;
  using namespace ctb::attn;
  if (D == 128) return mode == 0 ? launch_bwd<128, MODE_DKV>(c) : launch_bwd<128, MODE_DQ>(c);
  if (D == 64) return mode == 0 ? launch_bwd<64, MODE_DKV>(c) : launch_bwd<64, MODE_DQ>(c);
  return ctb::fail("attention: head_dim must be 64 or 128");
}

// Block-sparse (MoBA) backward: `it_off` has one entry per CTA plus one, in grid order
// (mode 0: (key tile ascending, batch, kv head); mode 1: (query tile descending, batch, head));
// `it_list` holds 64-row block indices, with the head's index inside its GQA group in bits 24+
// for mode 0.
CTB_API int ctb_attn_bwd_sparse(int mode, const void* q, const void* k, const void* v, const void* dout, void* dq,
                                void* dk, void* dv, const float* neg_lse2, const float* neg_delta, const int* seg,
                                const int* lim, const int* kv_lo, const int* kv_hi, const int* q_lo, const int* q_hi,
                                const int* run_start, const int* run_end, const int* first_q, const int* it_off, const int* it_cnt, int it_stride,
                                const int* it_list, const unsigned* sel, const unsigned* allsel, const int* doc_start,
                                int block, int words, int B, int S, int Hq, int Hkv, int D,
                                long q_rs, long k_rs, long v_rs, long do_rs, long dq_rs, long dk_rs, long dv_rs,
                                float scale, long long spin_budget, void* stream) {
  if (S % 128) return ctb::fail("attention: sequence length must be a multiple of 128");
  if (Hq % Hkv) return ctb::fail("attention: Hq must be a multiple of Hkv");
  if (block < 128) return ctb::fail("sparse attention: the routing block must hold at least 128 tokens");
  ctb::attn::BwdCall c{};
  c.q = q; c.k = k; c.v = v; c.dout = dout; c.dq = dq; c.dk = dk; c.dv = dv; c.neg_lse2 = neg_lse2; c.neg_delta = neg_delta;
  c.seg = seg; c.lim = lim; c.kv_lo = kv_lo; c.kv_hi = kv_hi; c.q_lo = q_lo; c.q_hi = q_hi;
  c.run_start = run_start; c.run_end = run_end; c.first_q = first_q;
  c.B = B; c.S = S; c.Hq = Hq; c.Hkv = Hkv;
  c.q_row_stride = q_rs; c.k_row_stride = k_rs; c.v_row_stride = v_rs; c.do_row_stride = do_rs;
  c.dq_row_stride = dq_rs; c.dk_row_stride = dk_rs; c.dv_row_stride = dv_rs;
  c.scale = scale; c.spin_budget = spin_budget; c.stream = stream;
  c.sp.it_off = it_off; c.sp.it_cnt = it_cnt; c.sp.it_stride = it_stride; c.sp.it_list = it_list; c.sp.sel = sel;
  c.sp.doc_start = doc_start;
  c.sp.allsel = allsel; c.sp.block = block; c.sp.words = words;
  using namespace ctb::attn;
  if (D == 128) return mode == 0 ? launch_bwd<128, MODE_DKV>(c) : launch_bwd<128, MODE_DQ>(c);
  if (D == 64) return mode == 0 ? launch_bwd<64, MODE_DKV>(c) : launch_bwd<64, MODE_DQ>(c);
  return ctb::fail("attention: head_dim must be 64 or 128");
}

// Grouped MoBA backward (see GroupArgs).  mode 0 (dK/dV): one CTA per (group, 128-key tile), `ctas`
// descriptors; dk / dv are [B,S,Hkv,D] views that receive the history part (tiles of groups without
// rows are not written: clear the buffers first).  mode 1 (dQ): one CTA per 128 gathered rows,
// gathered_rows / 128 descriptors; dqg is [gathered_rows, D].  qg / dog / the statistics are the
// gathered rows ([gathered_rows, D] contiguous, [gathered_rows] fp32, padding rows zero).
CTB_API int ctb_attn_bwd_grouped(int mode, const void* qg, const void* k, const void* v, const void* dog, void* dqg,
                                 void* dk, void* dv, const float* neg_lse2_g, const float* neg_delta_g,
                                 const void* desc, int ctas, int gathered_rows, int block, int B, int S, int Hkv, int D,
                                 long k_rs, long v_rs, long dk_rs, long dv_rs, float scale, long long spin_budget,
                                 void* stream) {
  if (S % 128 || block % 128 || block < 128) return ctb::fail("grouped attention: S and the block must be multiples of 128");
  if (gathered_rows <= 0 || gathered_rows % 256) return ctb::fail("grouped attention: gathered rows must be a positive multiple of 256");
  ctb::attn::BwdCall c{};
  c.q = qg; c.k = k; c.v = v; c.dout = dog; c.dq = dqg; c.dk = dk; c.dv = dv;
  c.neg_lse2 = neg_lse2_g; c.neg_delta = neg_delta_g;
  c.B = B; c.S = S; c.Hq = Hkv; c.Hkv = Hkv;
  c.q_row_stride = D; c.do_row_stride = D; c.dq_row_stride = D;
  c.k_row_stride = k_rs; c.v_row_stride = v_rs; c.dk_row_stride = dk_rs; c.dv_row_stride = dv_rs;
  c.scale = scale; c.spin_budget = spin_budget; c.stream = stream;
  c.grp.desc = static_cast<const int4*>(desc); c.grp.block = block; c.gathered_rows = gathered_rows;
  c.ctas = mode == 0 ? ctas : gathered_rows / 128;
  using namespace ctb::attn;
  if (D == 128) return mode == 0 ? launch_bwd<128, MODE_DKV>(c) : launch_bwd<128, MODE_DQ>(c);
  if (D == 64) return mode == 0 ? launch_bwd<64, MODE_DKV>(c) : launch_bwd<64, MODE_DQ>(c);
  return ctb::fail("attention: head_dim must be 64 or 128");
}
