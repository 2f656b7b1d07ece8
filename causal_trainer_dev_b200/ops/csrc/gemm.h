// Shared declarations of the tcgen05 GEMM family (see gemm.cu for the design notes).
#pragma once
#include "host_common.h"

namespace ctb {

enum GemmEpilogue : int {
  EPI_STORE = 0,       // C = alpha * acc (+ bias), bf16 or fp32, store or reduce-add
  EPI_CE_STATS = 1,    // per-row max / sum-exp / target logit of each 256-column slab
  EPI_CE_DLOGITS = 2,  // C = (exp(acc - lse[row]) - onehot(target[row])) * coef[row], bf16
};

// Device-side argument block (passed by value).
struct GemmArgs {
  int M, N, K;
  int out_f32;
  int accumulate;
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
  long ldb;
  const int* ce_targets;
  float* ce_max;
  float* ce_sum;
  float* ce_target_logit;
  const float* ce_lse;
  const float* ce_coef;
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
  long long spin_budget = 0;
  const int* ce_targets = nullptr;
  float* ce_max = nullptr;
  float* ce_sum = nullptr;
  float* ce_target_logit = nullptr;
  const float* ce_lse = nullptr;
  const float* ce_coef = nullptr;
};

int run_gemm(const GemmCall& call);

}  // namespace ctb
