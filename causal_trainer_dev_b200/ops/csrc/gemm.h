// Shared declarations of the tcgen05 GEMM family (see gemm.cu for the design notes).
#pragma once
#include "host_common.h"

namespace ctb {

enum GemmEpilogue : int {
  EPI_STORE = 0,       // C = alpha * acc (+ bias), bf16 or fp32, store or reduce-add
  EPI_CE_STATS = 1,    // per-row max / sum-exp / target logit of each 256-column slab
  EPI_CE_DLOGITS = 2,  // C = (exp(acc - lse[row]) - onehot(target[row])) * coef[row], bf16
  EPI_PUSH = 3,        // bf16 partial tiles stored into the row owners' receive buffers (GemmPush)
};

// Reduce-scatter by push (tensor-parallel row-parallel projections): instead of storing a
// partial-sum tile into local memory, the epilogue writes it into the receive buffer of the
// rank that owns those rows, `dest[p] + ((src_rank * rows_per_rank + local_row) * ld + col)`,
// and the CTA that completes the last tile bound for rank p publishes `epoch` in `flag[p]`.
struct GemmPush {
  __nv_bfloat16* const* dest;            // device table: every rank's receive buffer [world][rows_per_rank][ld]
  unsigned* const* flag;                 // device table: &pads_of_rank_p[base + src_rank]
  unsigned* counters;                    // local, one per destination rank, self-resetting
  int rows_per_rank;
  int row_offset;                        // global row of row 0 of this GEMM (chunked callers)
  int src_rank;
  int tiles_per_dest;                    // tiles bound for one rank, summed over all launches of the op
  long ld;
  unsigned epoch;
  int enabled;
};

// Device-side argument block (passed by value).
struct GemmArgs {
  int M, N, K;
  int out_f32;
  int accumulate;
  int split_k;            // > 1: work units are (tile, K slice), every slice reduce-adds into C
  int tail_first;         // with tail_splits > 1: tiles [tail_first, tiles) are cut into K slices,
  int tail_splits;        //   tail_splits each; the tiles before them stay whole
  float alpha;
  const __nv_bfloat16* bias;
  DeviceStatus* status;
  long long spin_budget;
  const unsigned* b_flags;
  long b_flag_chunk;
  long b_flag_base;
  unsigned b_flag_epoch;
  int b_wait_all;
  int n_rotate;
  int m_rotate;
  long ldb;
  long lda;
  const unsigned* a_flags;
  long a_flag_chunk;
  long a_flag_base;
  unsigned a_flag_epoch;
  const int* ce_targets;
  float* ce_max;
  float* ce_sum;
  float* ce_target_logit;
  const float* ce_lse;
  const float* ce_coef;
  GemmPush push;
  int* tile_counter;     // [2]: next tile to claim, CTAs that stopped claiming (dynamic_tiles only)
  int dynamic_tiles;
};

// Host-side call description.
struct GemmCall {
  const void* A = nullptr;
  const void* B = nullptr;
  void* C = nullptr;
  int M = 0, N = 0, K = 0;
  long lda = 0, ldb = 0, ldc = 0;
  int a_mn = 0, b_mn = 0;
  int out_f32 = 0, accumulate = 0;
  float alpha = 1.f;
  const void* bias = nullptr;
  int epi = EPI_STORE;
  int max_ctas = 0;
  void* stream = nullptr;
  const unsigned* b_flags = nullptr;
  long b_flag_chunk = 0;
  long b_flag_base = 0;
  unsigned b_flag_epoch = 0;
  int b_wait_all = 0;
  int n_rotate = 0;
  int m_rotate = 0;
  const unsigned* a_flags = nullptr;
  long a_flag_chunk = 0;
  long a_flag_base = 0;
  unsigned a_flag_epoch = 0;
  long long spin_budget = 0;
  const int* ce_targets = nullptr;
  float* ce_max = nullptr;
  float* ce_sum = nullptr;
  float* ce_target_logit = nullptr;
  const float* ce_lse = nullptr;
  const float* ce_coef = nullptr;
  GemmPush push{};
};

int run_gemm(const GemmCall& call);

// Two-CTA variant (gemm_pair.cu): plain products on clusters of two CTAs with
// tcgen05.mma.cta_group::2, selected by run_gemm when the mode is on (CTB_GEMM_PAIR=1 or
// ctb_gemm_set_pair) and the call has no gathered operand, fused epilogue or bias.
bool gemm_pair_eligible(const GemmCall& c);
int launch_gemm_pair(const GemmCall& c);

}  // namespace ctb
