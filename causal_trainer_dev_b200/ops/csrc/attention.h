// Shared declarations of the flash-attention kernels (forward, dQ, dK/dV).
#pragma once
#include "host_common.h"

namespace ctb {
namespace attn {

// Visibility metadata, built once per step and shared by all layers:
//   seg    [B,S]      canonical run ids, 0 = padding
//   lim    [B,S]      inclusive last visible key index = max(i, attention_end[i]); null => i
//   kv_lo  [B,S/128]  first key index any row of the 128-row query block can see
//   kv_hi  [B,S/128]  one past the last such key index (kv_hi <= kv_lo: nothing visible)
//   kmin/kmax [B,S/128] min / max segment id inside each 128-key block
//   q_lo/q_hi [B,S/128] per 128-key block: range of query indices that can see it
struct FwdArgs {
  int B, S, Hq, Hkv;
  float scale_log2;
  const int* seg;
  const int* lim;
  const int* kv_lo;
  const int* kv_hi;
  const int* kmin;
  const int* kmax;
  float* lse;
  DeviceStatus* status;
  long long spin_budget;
};

struct FwdCall {
  const void* q; const void* k; const void* v; void* o; float* lse;
  const int* seg; const int* lim; const int* kv_lo; const int* kv_hi; const int* kmin; const int* kmax;
  int B, S, Hq, Hkv;
  long q_row_stride, k_row_stride, v_row_stride, o_row_stride;
  float scale;
  long long spin_budget;
  void* stream;
};

enum : int { MODE_DKV = 0, MODE_DQ = 1 };

// Extra metadata of the backward kernels, at 64-row granularity:
//   seg_min64 / seg_max64 [B,S/64]  min / max segment id of each 64-token block
//   lim_min64 / lim_max64 [B,S/64]  min / max of lim over each 64-token block
struct BwdArgs {
  int B, S, Hq, Hkv;
  float scale, scale_log2;
  const int* seg;
  const int* lim;
  const int* kv_lo;
  const int* kv_hi;
  const int* q_lo;
  const int* q_hi;
  const int* seg_min64;
  const int* seg_max64;
  const int* lim_min64;
  const int* lim_max64;
  const float* lse;
  const float* delta;
  DeviceStatus* status;
  long long spin_budget;
};

struct BwdCall {
  const void* q; const void* k; const void* v; const void* dout;
  void* dq; void* dk; void* dv;
  const float* lse; const float* delta;
  const int* seg; const int* lim; const int* kv_lo; const int* kv_hi; const int* q_lo; const int* q_hi;
  const int* seg_min64; const int* seg_max64; const int* lim_min64; const int* lim_max64;
  int B, S, Hq, Hkv;
  long q_row_stride, k_row_stride, v_row_stride, do_row_stride, dq_row_stride, dk_row_stride, dv_row_stride;
  float scale;
  long long spin_budget;
  void* stream;
};

}  // namespace attn
}  // namespace ctb
