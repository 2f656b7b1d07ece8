// Memory-bound kernels of the decoder layer and the optimizer (sm_100a, HBM3e bound):
// RMSNorm forward/backward (optional fused residual add), RoPE (in place on the packed QKV
// projection, both pairings, partial rotary, arbitrary positions), SwiGLU forward/backward
// on the packed gate|up projection, embedding gather, the attention delta = rowsum(O*dO),
// cut-CE partial-statistics combine, sum of squares for the global gradient norm and the
// fused AdamW update with moments in the parameter dtype.
//
// All of them move 16 bytes per thread per access and keep reductions in fp32.
// Reference semantics: rms_norm (src/causal_trainer/modeling/architecture.py:155-162),
// apply_rotary_cos_sin (src/causal_trainer/modeling/rotary.py:132-204), _mlp_projection
// (architecture.py:205-229), optimizer update (src/causal_trainer/training/steps.py:172-186,
// src/causal_trainer/training/optimizer.py:42-75).
#include <cuda_bf16.h>

#include "host_common.h"

namespace ctb {
namespace ew {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV = 8;  // 8-element vectors per thread: hidden size up to 16384

struct bf16x8 {
  uint4 raw;
};
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Sum over the block; every thread gets the result.  `scratch` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// ------------------------------------------------------------------------------------------
// RMSNorm forward.  y = bf16(x * rstd) * w   (normalised value rounded to bf16 before the
// scale, as the reference does).  With `residual` set: h = x + residual is written to
// `h_out` first and normalised.
// ------------------------------------------------------------------------------------------
template <int NV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int rows, int d, float eps) {
  __shared__ float scratch[33];
  const int nvec = d / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * d);
    const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + static_cast<size_t>(row) * d) : nullptr;
    uint4 hv[NV];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float f[8];
        unpack8(xr[v], f);
        if (rr) {
          float g[8];
          unpack8(rr[v], g);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __bfloat162float(__float2bfloat16(f[e] + g[e]));
          hv[i] = pack8(f);
          reinterpret_cast<uint4*>(h_out + static_cast<size_t>(row) * d)[v] = hv[i];
        } else {
          hv[i] = xr[v];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
      }
    }
    const float total = block_sum(ss, scratch);
    const float rstd = rsqrtf(total / d + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float f[8], g[8];
        unpack8(hv[i], f);
        unpack8(reinterpret_cast<const uint4*>(w)[v], g);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = __bfloat162float(__float2bfloat16(f[e] * rstd)) * g[e];
        reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * d)[v] = pack8(f);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// RMSNorm backward.  dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres), and per-CTA
// partial sums of dw = sum_rows dy * xhat into `dw_partial[gridDim.x][d]` (fp32 scratch),
// reduced by rmsnorm_dw_reduce_kernel.  No atomics: the result is deterministic.
// ------------------------------------------------------------------------------------------
template <int NV>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int rows, int d) {
  __shared__ float scratch[33];
  const int nvec = d / 8;
  float dw_acc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) dw_acc[i][e] = 0.f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rs = rstd[row];
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * d);
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * d);
    float gx[NV][8], xh[NV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float a[8], b[8], c[8];
        unpack8(dyr[v], a);
        unpack8(xr[v], b);
        unpack8(reinterpret_cast<const uint4*>(w)[v], c);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[i][e] = b[e] * rs;
          gx[i][e] = a[e] * c[e];
          dot += gx[i][e] * xh[i][e];
          dw_acc[i][e] += a[e] * xh[i][e];
        }
      }
    }
    const float mean = block_sum(dot, scratch) / d;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rs * (gx[i][e] - xh[i][e] * mean);
        if (dres) {
          float r[8];
          unpack8(reinterpret_cast<const uint4*>(dres + static_cast<size_t>(row) * d)[v], r);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += r[e];
        }
        reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * d)[v] = pack8(o);
      }
    }
  }
  float* out = dw_partial + static_cast<size_t>(blockIdx.x) * d;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
      float4* o4 = reinterpret_cast<float4*>(out + v * 8);
      o4[0] = make_float4(dw_acc[i][0], dw_acc[i][1], dw_acc[i][2], dw_acc[i][3]);
      o4[1] = make_float4(dw_acc[i][4], dw_acc[i][5], dw_acc[i][6], dw_acc[i][7]);
    }
  }
}

// dw[c] (+)= sum_p partial[p][c]; out dtype bf16 or fp32.
__global__ void rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, int parts, int d, void* __restrict__ dw,
                                         int out_f32, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[static_cast<size_t>(p) * d + c];
  if (out_f32) {
    float* o = static_cast<float*>(dw);
    o[c] = accumulate ? o[c] + s : s;
  } else {
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(dw);
    o[c] = __float2bfloat16(accumulate ? __bfloat162float(o[c]) + s : s);
  }
}

// ------------------------------------------------------------------------------------------
// RoPE, in place on `heads` consecutive heads of a packed projection row.
//   x: [T][row_stride] with head h at columns h*D..h*D+D-1; cos/sin: [T][rot/2] fp32.
//   style 0 = gpt-j (adjacent pairs), 1 = gpt-neox (half split).  sign=-1 applies the
//   inverse rotation (the backward pass).
// ------------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cosv,
                            const float* __restrict__ sinv, long row_stride, int T, int heads, int D, int rot,
                            int style, float sign) {
  const int half = rot / 2;
  const long total = static_cast<long>(T) * heads * half;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int p = static_cast<int>(i % half);
    const long th = i / half;
    const int h = static_cast<int>(th % heads);
    const long t = th / heads;
    const float c = cosv[t * half + p];
    const float s = sinv[t * half + p] * sign;
    __nv_bfloat16* base = x + t * row_stride + static_cast<long>(h) * D;
    const int i0 = style == 0 ? 2 * p : p;
    const int i1 = style == 0 ? 2 * p + 1 : p + half;
    const float a = __bfloat162float(base[i0]);
    const float b = __bfloat162float(base[i1]);
    base[i0] = __float2bfloat16(a * c - b * s);
    base[i1] = __float2bfloat16(b * c + a * s);
  }
}

// cos/sin tables from arbitrary integer positions: angle = pos * inv_freq[p] in fp32.
__global__ void rope_table_kernel(const int* __restrict__ pos, const float* __restrict__ inv_freq,
                                  float* __restrict__ cosv, float* __restrict__ sinv, int T, int half) {
  const long total = static_cast<long>(T) * half;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int p = static_cast<int>(i % half);
    const long t = i / half;
    const float ang = static_cast<float>(pos[t]) * inv_freq[p];
    float s, c;
    sincosf(ang, &s, &c);
    // the reference casts the table to the compute dtype once per step
    cosv[i] = __bfloat162float(__float2bfloat16(c));
    sinv[i] = __bfloat162float(__float2bfloat16(s));
  }
}

// ------------------------------------------------------------------------------------------
// SwiGLU on the packed projection gu[T][2f] = [gate | up]:  h = silu(gate) * up.
// Backward writes d(gate|up) in the same packed layout.
// ------------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h, long T, int f) {
  const int nvec = f / 8;
  const long total = T * nvec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = i / nvec;
    const int v = static_cast<int>(i % nvec);
    const uint4* row = reinterpret_cast<const uint4*>(gu + t * 2 * f);
    float g[8], u[8], o[8];
    unpack8(row[v], g);
    unpack8(row[nvec + v], u);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float act = __bfloat162float(__float2bfloat16(g[e] / (1.f + __expf(-g[e]))));
      o[e] = act * u[e];
    }
    reinterpret_cast<uint4*>(h + t * f)[v] = pack8(o);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dh,
                                  __nv_bfloat16* __restrict__ dgu, long T, int f) {
  const int nvec = f / 8;
  const long total = T * nvec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = i / nvec;
    const int v = static_cast<int>(i % nvec);
    const uint4* row = reinterpret_cast<const uint4*>(gu + t * 2 * f);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(row[v], g);
    unpack8(row[nvec + v], u);
    unpack8(reinterpret_cast<const uint4*>(dh + t * f)[v], d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sg = 1.f / (1.f + __expf(-g[e]));
      const float act = g[e] * sg;
      du[e] = d[e] * act;
      dg[e] = d[e] * u[e] * sg * (1.f + g[e] * (1.f - sg));
    }
    uint4* orow = reinterpret_cast<uint4*>(dgu + t * 2 * f);
    orow[v] = pack8(dg);
    orow[nvec + v] = pack8(du);
  }
}

// ------------------------------------------------------------------------------------------
// Embedding gather: out[t] = table[ids[t]] (the stored pad row is returned as is).
// ------------------------------------------------------------------------------------------
__global__ void embedding_gather_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                        __nv_bfloat16* __restrict__ out, long T, int d, int vocab) {
  const int nvec = d / 8;
  const long total = T * nvec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = i / nvec;
    const int v = static_cast<int>(i % nvec);
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    reinterpret_cast<uint4*>(out + t * d)[v] = reinterpret_cast<const uint4*>(table + static_cast<long>(id) * d)[v];
  }
}

// ------------------------------------------------------------------------------------------
// delta[b][h][s] = sum_d O[b][s][h][d] * dO[b][s][h][d]   (one warp per (token, head))
// ------------------------------------------------------------------------------------------
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, int B, int S, int H, int D, long o_rs, long do_rs) {
  const long warp_id = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long total = static_cast<long>(B) * S * H;
  if (warp_id >= total) return;
  const int h = static_cast<int>(warp_id % H);
  const long t = warp_id / H;
  const __nv_bfloat16* op = o + t * o_rs + static_cast<long>(h) * D;
  const __nv_bfloat16* dp = dout + t * do_rs + static_cast<long>(h) * D;
  float acc = 0.f;
  for (int c = lane * 2; c < D; c += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(op + c));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dp + c));
    acc += a.x * b.x + a.y * b.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    const long b_idx = t / S, s_idx = t % S;
    delta[(b_idx * H + h) * S + s_idx] = acc;
  }
}

// ------------------------------------------------------------------------------------------
// Per-query statistics of the attention backward, in the form its kernels consume:
//   neg_delta[b][h][s] = -sum_d O dO        neg_lse2[b][h][s] = -lse[b][h][s] * log2(e)
// (one warp per (token, head)), so the inner loops use packed fma / add without a negation.
// ------------------------------------------------------------------------------------------
__global__ void attn_bwd_stats_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                      const float* __restrict__ lse, float* __restrict__ neg_lse2,
                                      float* __restrict__ neg_delta, int B, int S, int H, int D, long o_rs, long do_rs) {
  const long warp_id = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long total = static_cast<long>(B) * S * H;
  if (warp_id >= total) return;
  const int h = static_cast<int>(warp_id % H);
  const long t = warp_id / H;
  const __nv_bfloat16* op = o + t * o_rs + static_cast<long>(h) * D;
  const __nv_bfloat16* dp = dout + t * do_rs + static_cast<long>(h) * D;
  float acc = 0.f;
  for (int c = lane * 2; c < D; c += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(op + c));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dp + c));
    acc += a.x * b.x + a.y * b.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    const long b_idx = t / S, s_idx = t % S;
    const long i = (b_idx * H + h) * S + s_idx;
    neg_delta[i] = -acc;
    neg_lse2[i] = -lse[i] * 1.4426950408889634f;
  }
}

// ------------------------------------------------------------------------------------------
// Cut-CE combine: merges per-slab (max, sumexp) into lse[row], emits the weighted NLL per
// row, the backward coefficient coef[row] = weight * grad_scale, and block partial sums of
// (nll, weight) which the host-side wrapper adds up (fp32, fixed order: deterministic).
// ------------------------------------------------------------------------------------------
__global__ void ce_combine_kernel(const float* __restrict__ pmax, const float* __restrict__ psum, int slabs,
                                  const float* __restrict__ target_logit, const float* __restrict__ weights,
                                  float grad_scale, float* __restrict__ lse, float* __restrict__ coef,
                                  float* __restrict__ block_nll, float* __restrict__ block_w, int rows) {
  __shared__ float scratch[33];
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  float nll = 0.f, w = 0.f;
  if (row < rows) {
    float m = -INFINITY;
    for (int s = 0; s < slabs; ++s) m = fmaxf(m, pmax[static_cast<size_t>(s) * rows + row]);
    float acc = 0.f;
    for (int s = 0; s < slabs; ++s) {
      const size_t i = static_cast<size_t>(s) * rows + row;
      acc += psum[i] * __expf(pmax[i] - m);
    }
    const float l = m + logf(acc);
    lse[row] = l;
    w = weights[row];
    coef[row] = w * grad_scale;
    nll = (w != 0.f) ? (l - target_logit[row]) * w : 0.f;
  }
  const float bn = block_sum(nll, scratch);
  const float bw = block_sum(w, scratch);
  if (threadIdx.x == 0) {
    block_nll[blockIdx.x] = bn;
    block_w[blockIdx.x] = bw;
  }
}

// ------------------------------------------------------------------------------------------
// Cross-entropy over a materialised logits slab [rows, vocab] (bf16): one CTA per row.
//   stats:    lse[row] = logsumexp(logits[row, :]), target_logit[row] (0 when the target is < 0)
//   backward: logits[row, v] <- (exp(logits[row, v] - lse[row]) - [v == target]) * coef[row], in place
// The projection-fused cut cross-entropy never writes logits; these two kernels are the variant
// that does (the reference's `pallas` loss backend, src/causal_trainer/kernels/cross_entropy.py:
// 99-189, 254-322), for when the slab is wanted anyway.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
logits_ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, long ld, int vocab, const int* __restrict__ targets,
                       float* __restrict__ lse, float* __restrict__ target_logit) {
  __shared__ float scratch[33];
  __shared__ float s_max;
  const long row = blockIdx.x;
  const __nv_bfloat16* x = logits + row * ld;
  const int nvec = vocab / 8;
  float m = -INFINITY;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 raw = reinterpret_cast<const uint4*>(x)[v];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      m = fmaxf(m, fmaxf(f.x, f.y));
    }
  }
  for (int c = nvec * 8 + threadIdx.x; c < vocab; c += blockDim.x) m = fmaxf(m, __bfloat162float(x[c]));
  // block max through the sum helper's scratch: reduce per warp, then across warps
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = -INFINITY;
    for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) t = fmaxf(t, scratch[w]);
    s_max = t;
  }
  __syncthreads();
  const float mx = s_max;
  float acc = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 raw = reinterpret_cast<const uint4*>(x)[v];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      acc += __expf(f.x - mx) + __expf(f.y - mx);
    }
  }
  for (int c = nvec * 8 + threadIdx.x; c < vocab; c += blockDim.x) acc += __expf(__bfloat162float(x[c]) - mx);
  const float total = block_sum(acc, scratch);
  if (threadIdx.x == 0) {
    lse[row] = mx + logf(total);
    const int t = targets[row];
    target_logit[row] = (t >= 0 && t < vocab) ? __bfloat162float(x[t]) : 0.f;
  }
}

__global__ void __launch_bounds__(256)
logits_ce_backward_kernel(__nv_bfloat16* __restrict__ logits, long ld, int vocab, const int* __restrict__ targets,
                          const float* __restrict__ lse, const float* __restrict__ coef) {
  const long row = blockIdx.x;
  __nv_bfloat16* x = logits + row * ld;
  const float l = lse[row], c = coef[row];
  const int t = targets[row];
  const int nvec = vocab / 8;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 raw = reinterpret_cast<uint4*>(x)[v];
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      const int col = v * 8 + e * 2;
      const float a = (__expf(f.x - l) - (col == t ? 1.f : 0.f)) * c;
      const float b = (__expf(f.y - l) - (col + 1 == t ? 1.f : 0.f)) * c;
      h[e] = __floats2bfloat162_rn(a, b);
    }
    reinterpret_cast<uint4*>(x)[v] = raw;
  }
  for (int col = nvec * 8 + threadIdx.x; col < vocab; col += blockDim.x)
    x[col] = __float2bfloat16((__expf(__bfloat162float(x[col]) - l) - (col == t ? 1.f : 0.f)) * c);
}

// ------------------------------------------------------------------------------------------
// Sum of squares (fp32) of a bf16 / fp32 vector into per-block partials.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ x, long n, float* __restrict__ partial, int round_bf16) {
  __shared__ float scratch[33];
  float acc = 0.f;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float v = static_cast<float>(x[i]);
    if (round_bf16) v = __bfloat162float(__float2bfloat16(v));
    acc += v * v;
  }
  const float t = block_sum(acc, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = t;
}

// ------------------------------------------------------------------------------------------
// Fused AdamW on a flat shard.  Moments are stored in the parameter dtype; the arithmetic is
// fp32.  `clip` points at a device scalar (global-norm clip coefficient, <= 1) so the
// optimizer never waits for the host; `decay` is 0 for vectors (norm scales, biases).
//   g' = g*clip; m = b1 m + (1-b1) g'; v = b2 v + (1-b2) g'^2
//   p += bf16( -lr * ( m/(1-b1^t) / (sqrt(v/(1-b2^t)) + eps) + decay * p ) )
// ------------------------------------------------------------------------------------------
template <typename GT>
__global__ void adamw_kernel(__nv_bfloat16* __restrict__ p, const GT* __restrict__ g, __nv_bfloat16* __restrict__ m,
                             __nv_bfloat16* __restrict__ v, long n, float lr, float b1, float b2, float eps,
                             float decay, float bc1, float bc2, const float* __restrict__ clip, float gscale,
                             int round_bf16) {
  const float cs = (clip ? *clip : 1.f) * gscale;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float graw = static_cast<float>(g[i]);
    if (round_bf16) graw = __bfloat162float(__float2bfloat16(graw));
    const float gi = graw * cs;
    const float mi = b1 * __bfloat162float(m[i]) + (1.f - b1) * gi;
    const float vi = b2 * __bfloat162float(v[i]) + (1.f - b2) * gi * gi;
    const float pi = __bfloat162float(p[i]);
    const float upd = -lr * ((mi / bc1) / (sqrtf(vi / bc2) + eps) + decay * pi);
    m[i] = __float2bfloat16(mi);
    v[i] = __float2bfloat16(vi);
    p[i] = __float2bfloat16(pi + __bfloat162float(__float2bfloat16(upd)));
  }
}

// ------------------------------------------------------------------------------------------
// AdamW over a whole flat arena in one launch.  The arena is a sequence of regions
// [bounds[r], bounds[r+1]) with a mode each: 1 = weight decay, 0 = no decay, -1 = frozen (the
// region is skipped: no update, moments untouched).  16-byte accesses: eight elements of the
// parameter, both moments and the gradient per thread per round, two rounds in flight.
// ------------------------------------------------------------------------------------------
constexpr int ADAM_MAX_REGIONS = 512;

__device__ __forceinline__ float fast_sqrt(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename GT>
__global__ void __launch_bounds__(256)
adamw_regions_kernel(__nv_bfloat16* __restrict__ p, const GT* __restrict__ g, __nv_bfloat16* __restrict__ m,
                     __nv_bfloat16* __restrict__ v, long n, const long* __restrict__ bounds,
                     const int* __restrict__ modes, int nreg, float lr, float b1, float b2, float eps, float decay,
                     float bc1, float bc2, const float* __restrict__ clip, float gscale, int round_bf16) {
  __shared__ long sb[ADAM_MAX_REGIONS + 1];
  __shared__ int sm[ADAM_MAX_REGIONS];
  for (int i = threadIdx.x; i <= nreg; i += blockDim.x) sb[i] = bounds[i];
  for (int i = threadIdx.x; i < nreg; i += blockDim.x) sm[i] = modes[i];
  __syncthreads();
  const float cs = (clip ? *clip : 1.f) * gscale;
  const float inv_bc1 = 1.f / bc1, inv_bc2 = 1.f / bc2;
  auto region_of = [&](long e) {
    int lo = 0, hi = nreg - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (sb[mid] <= e) lo = mid; else hi = mid - 1;
    }
    return lo;
  };
  const long nvec = n / 8;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  int cached = 0;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < nvec; i += stride) {
    const long e0 = i * 8;
    if (!(sb[cached] <= e0 && e0 < sb[cached + 1])) cached = region_of(e0);
    const bool uniform = sb[cached + 1] >= e0 + 8;
    if (uniform && sm[cached] < 0) continue;
    uint4 pr = reinterpret_cast<const uint4*>(p)[i];
    uint4 mr = reinterpret_cast<const uint4*>(m)[i];
    uint4 vr = reinterpret_cast<const uint4*>(v)[i];
    float gf[8];
    if constexpr (sizeof(GT) == 4) {
      const float4 g0 = reinterpret_cast<const float4*>(g)[2 * i];
      const float4 g1 = reinterpret_cast<const float4*>(g)[2 * i + 1];
      gf[0] = g0.x; gf[1] = g0.y; gf[2] = g0.z; gf[3] = g0.w;
      gf[4] = g1.x; gf[5] = g1.y; gf[6] = g1.z; gf[7] = g1.w;
      if (round_bf16) {
#pragma unroll
        for (int e = 0; e < 8; ++e) gf[e] = __bfloat162float(__float2bfloat16(gf[e]));
      }
    } else {
      const uint4 gr = reinterpret_cast<const uint4*>(g)[i];
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gr);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(gh[e]);
        gf[2 * e] = f.x;
        gf[2 * e + 1] = f.y;
      }
    }
    __nv_bfloat16* pe = reinterpret_cast<__nv_bfloat16*>(&pr);
    __nv_bfloat16* me = reinterpret_cast<__nv_bfloat16*>(&mr);
    __nv_bfloat16* ve = reinterpret_cast<__nv_bfloat16*>(&vr);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int mode = uniform ? sm[cached] : sm[region_of(e0 + e)];
      if (mode < 0) continue;
      const float gi = gf[e] * cs;
      const float mi = b1 * __bfloat162float(me[e]) + (1.f - b1) * gi;
      const float vi = b2 * __bfloat162float(ve[e]) + (1.f - b2) * gi * gi;
      const float pi = __bfloat162float(pe[e]);
      // one sqrt.approx and one rcp.approx per element (2 ulp each, far below the bf16 rounding of the
      // update): with IEEE division and square root the sweep is bound by instruction issue, not by HBM
      const float upd = -lr * ((mi * inv_bc1) * fast_rcp(fast_sqrt(vi * inv_bc2) + eps) + (mode ? decay : 0.f) * pi);
      me[e] = __float2bfloat16(mi);
      ve[e] = __float2bfloat16(vi);
      pe[e] = __float2bfloat16(pi + __bfloat162float(__float2bfloat16(upd)));
    }
    reinterpret_cast<uint4*>(p)[i] = pr;
    reinterpret_cast<uint4*>(m)[i] = mr;
    reinterpret_cast<uint4*>(v)[i] = vr;
  }
}

// ------------------------------------------------------------------------------------------
// Active-row compaction (rows whose loss weight is non-zero go through the LM head; the others do
// not).  Stable: the compacted order is the row order, so results do not depend on it.
//   active_count   rows with weight != 0 per block of 1024 rows
//   active_fill    idx[k] = k-th active row; total[0] = number of active rows
//   gather_rows    dst[j] = src[idx[j]]
//   scatter_rows   dst[idx[j]] = src[j] for j < total (dst cleared by the caller)
// ------------------------------------------------------------------------------------------
constexpr int ACTIVE_BLOCK = 1024;

__global__ void __launch_bounds__(ACTIVE_BLOCK)
active_count_kernel(const float* __restrict__ w, int rows, int* __restrict__ block_counts) {
  const int r = blockIdx.x * ACTIVE_BLOCK + threadIdx.x;
  const int flag = (r < rows && w[r] != 0.f) ? 1 : 0;
  const int n = __syncthreads_count(flag);
  if (threadIdx.x == 0) block_counts[blockIdx.x] = n;
}

__global__ void __launch_bounds__(ACTIVE_BLOCK)
active_fill_kernel(const float* __restrict__ w, int rows, const int* __restrict__ block_counts, int* __restrict__ idx,
                   int* __restrict__ total) {
  __shared__ int warp_sums[ACTIVE_BLOCK / 32];
  __shared__ int base_s;
  const int r = blockIdx.x * ACTIVE_BLOCK + threadIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool flag = r < rows && w[r] != 0.f;
  const unsigned votes = __ballot_sync(0xffffffffu, flag);
  if (lane == 0) warp_sums[warp] = __popc(votes);
  if (threadIdx.x == 0) {
    int base = 0;
    for (int b = 0; b < static_cast<int>(blockIdx.x); ++b) base += block_counts[b];
    base_s = base;
  }
  __syncthreads();
  int before = base_s;
  for (int x = 0; x < warp; ++x) before += warp_sums[x];
  if (flag) idx[before + __popc(votes & ((1u << lane) - 1u))] = r;
  if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) {
    int sum = base_s;
    for (int x = 0; x < ACTIVE_BLOCK / 32; ++x) sum += warp_sums[x];
    total[0] = sum;
  }
}

// Row indices come from device memory: an index outside [0, rows) is recorded in the status word
// (site, position, value) and the row is skipped; nothing is read or written out of bounds.
enum : unsigned { SITE_GATHER_INDEX = 0x0601, SITE_SCATTER_INDEX = 0x0602 };

__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ src, long src_stride, const int* __restrict__ idx,
                                   __nv_bfloat16* __restrict__ dst, long n, int d, int rows, DeviceStatus* st) {
  const int nvec = d / 8;
  const long work = n * nvec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < work;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long j = i / nvec;
    const int v = static_cast<int>(i % nvec);
    const int r = idx[j];
    if (r < 0 || r >= rows) {
      if (v == 0) report_failure(st, SITE_GATHER_INDEX, static_cast<unsigned>(j), static_cast<unsigned>(r));
      reinterpret_cast<uint4*>(dst + j * d)[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    reinterpret_cast<uint4*>(dst + j * d)[v] = reinterpret_cast<const uint4*>(src + r * src_stride)[v];
  }
}

__global__ void scatter_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ idx,
                                    const int* __restrict__ total, __nv_bfloat16* __restrict__ dst, long dst_stride,
                                    long n, int d, int rows, DeviceStatus* st) {
  const int nvec = d / 8;
  const long live = min(n, static_cast<long>(total[0]));
  const long work = live * nvec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < work;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long j = i / nvec;
    const int v = static_cast<int>(i % nvec);
    const int r = idx[j];
    if (r < 0 || r >= rows) {
      if (v == 0) report_failure(st, SITE_SCATTER_INDEX, static_cast<unsigned>(j), static_cast<unsigned>(r));
      continue;
    }
    reinterpret_cast<uint4*>(dst + r * dst_stride)[v] = reinterpret_cast<const uint4*>(src + j * d)[v];
  }
}

}  // namespace ew
}  // namespace ctb

using namespace ctb;
using namespace ctb::ew;

static inline int grid_for(long work, int threads, int cap_per_sm = 8) {
  long blocks = (work + threads - 1) / threads;
  const long cap = static_cast<long>(sm_count()) * cap_per_sm;
  if (blocks > cap) blocks = cap;
  return static_cast<int>(blocks < 1 ? 1 : blocks);
}

CTB_API int ctb_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out, float* rstd,
                            int rows, int d, float eps, void* stream) {
  if (d % 8 || d > NORM_MAXV * NORM_THREADS * 8) return fail("rmsnorm: hidden size must be a multiple of 8, <= 16384");
  if (residual && !h_out) return fail("rmsnorm: residual given without h_out");
  const int grid = rows < sm_count() * 8 ? rows : sm_count() * 8;
  const int nv = (d / 8 + NORM_THREADS - 1) / NORM_THREADS;
#define CTB_NORM_FWD(NV)                                                                                         \
  rmsnorm_fwd_kernel<NV><<<grid, NORM_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(                          \
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual),                         \
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(h_out),  \
      rstd, rows, d, eps)
  if (nv <= 1) CTB_NORM_FWD(1);
  else if (nv <= 2) CTB_NORM_FWD(2);
  else if (nv <= 4) CTB_NORM_FWD(4);
  else CTB_NORM_FWD(8);
#undef CTB_NORM_FWD
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Number of per-CTA partial rows the backward kernel writes; `dw_partial` must hold
// ctb_rmsnorm_bwd_parts(rows) * d floats.
CTB_API int ctb_rmsnorm_bwd_parts(int rows) {
  const int cap = sm_count() * 2;
  return rows < cap ? rows : cap;
}

CTB_API int ctb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                            void* dx, float* dw_partial, void* dw, int dw_f32, int dw_accumulate, int rows, int d,
                            void* stream) {
  if (d % 8 || d > NORM_MAXV * NORM_THREADS * 8) return fail("rmsnorm: hidden size must be a multiple of 8, <= 16384");
  const int parts = ctb_rmsnorm_bwd_parts(rows);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int nv = (d / 8 + NORM_THREADS - 1) / NORM_THREADS;
#define CTB_NORM_BWD(NV)                                                                       \
  rmsnorm_bwd_kernel<NV><<<parts, NORM_THREADS, 0, s>>>(                                       \
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),             \
      static_cast<const __nv_bfloat16*>(w), rstd, static_cast<const __nv_bfloat16*>(dres),     \
      static_cast<__nv_bfloat16*>(dx), dw_partial, rows, d)
  if (nv <= 1) CTB_NORM_BWD(1);
  else if (nv <= 2) CTB_NORM_BWD(2);
  else if (nv <= 4) CTB_NORM_BWD(4);
  else CTB_NORM_BWD(8);
#undef CTB_NORM_BWD
  CTB_CUDA_OK(cudaGetLastError());
  if (dw != nullptr) {
    rmsnorm_dw_reduce_kernel<<<(d + 255) / 256, 256, 0, s>>>(dw_partial, parts, d, dw, dw_f32, dw_accumulate);
    CTB_CUDA_OK(cudaGetLastError());
  }
  return 0;
}

CTB_API int ctb_rope_table(const int* pos, const float* inv_freq, float* cosv, float* sinv, int T, int half,
                           void* stream) {
  rope_table_kernel<<<grid_for(static_cast<long>(T) * half, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      pos, inv_freq, cosv, sinv, T, half);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_rope(void* x, const float* cosv, const float* sinv, long row_stride, int T, int heads, int D, int rot,
                     int style, int inverse, void* stream) {
  if (rot % 2 || rot > D) return fail("rope: rotary_dim must be even and <= head_dim");
  rope_kernel<<<grid_for(static_cast<long>(T) * heads * (rot / 2), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(x), cosv, sinv, row_stride, T, heads, D, rot, style, inverse ? -1.f : 1.f);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_swiglu_fwd(const void* gu, void* h, long T, int f, void* stream) {
  if (f % 8) return fail("swiglu: intermediate size must be a multiple of 8");
  swiglu_fwd_kernel<<<grid_for(T * (f / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(h), T, f);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_swiglu_bwd(const void* gu, const void* dh, void* dgu, long T, int f, void* stream) {
  if (f % 8) return fail("swiglu: intermediate size must be a multiple of 8");
  swiglu_bwd_kernel<<<grid_for(T * (f / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dh), static_cast<__nv_bfloat16*>(dgu),
      T, f);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_embedding_gather(const int* ids, const void* table, void* out, long T, int d, int vocab,
                                 void* stream) {
  if (d % 8) return fail("embedding: hidden size must be a multiple of 8");
  embedding_gather_kernel<<<grid_for(T * (d / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), T, d, vocab);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_attn_delta(const void* o, const void* dout, float* delta, int B, int S, int H, int D, long o_rs,
                           long do_rs, void* stream) {
  const long warps = static_cast<long>(B) * S * H;
  const int threads = 256;
  const long blocks = (warps * 32 + threads - 1) / threads;
  attn_delta_kernel<<<static_cast<unsigned>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dout), delta, B, S, H, D, o_rs, do_rs);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// o, dout: [B,S,H,D] bf16 views (row strides in elements); lse, neg_lse2, neg_delta: [B,H,S] fp32.
CTB_API int ctb_attn_bwd_stats(const void* o, const void* dout, const float* lse, float* neg_lse2, float* neg_delta,
                               int B, int S, int H, int D, long o_rs, long do_rs, void* stream) {
  const long warps = static_cast<long>(B) * S * H;
  const int threads = 256;
  const long blocks = (warps * 32 + threads - 1) / threads;
  attn_bwd_stats_kernel<<<static_cast<unsigned>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dout), lse, neg_lse2, neg_delta, B, S, H,
      D, o_rs, do_rs);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// block_nll / block_w must hold ceil(rows / 256) floats each.
CTB_API int ctb_ce_combine(const float* pmax, const float* psum, int slabs, const float* target_logit,
                           const float* weights, float grad_scale, float* lse, float* coef, float* block_nll,
                           float* block_w, int rows, void* stream) {
  ce_combine_kernel<<<(rows + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      pmax, psum, slabs, target_logit, weights, grad_scale, lse, coef, block_nll, block_w, rows);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// logits: [rows, vocab] bf16 with row stride ld (elements, multiple of 8); lse/target_logit: [rows].
CTB_API int ctb_logits_ce_stats(const void* logits, long ld, int rows, int vocab, const int* targets, float* lse,
                                float* target_logit, void* stream) {
  if (ld % 8) return fail("logits_ce: row stride must be a multiple of 8 elements");
  if (rows <= 0) return 0;
  logits_ce_stats_kernel<<<rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), ld, vocab, targets, lse, target_logit);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_logits_ce_backward(void* logits, long ld, int rows, int vocab, const int* targets, const float* lse,
                                   const float* coef, void* stream) {
  if (ld % 8) return fail("logits_ce: row stride must be a multiple of 8 elements");
  if (rows <= 0) return 0;
  logits_ce_backward_kernel<<<rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(logits), ld, vocab, targets, lse, coef);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// partial must hold ctb_sumsq_parts() floats.
CTB_API int ctb_sumsq_parts() { return sm_count() * 4; }
// round_bf16: square the bf16 rounding of each fp32 element (the norm of gradients "cast to
// the parameter dtype" without materialising the cast).
CTB_API int ctb_sumsq(const void* x, long n, int is_f32, int round_bf16, float* partial, void* stream) {
  const int grid = ctb_sumsq_parts();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (is_f32) sumsq_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), n, partial, round_bf16);
  else sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), n, partial, 0);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

CTB_API int ctb_adamw(void* p, const void* g, int g_f32, void* m, void* v, long n, float lr, float b1, float b2,
                      float eps, float decay, float bc1, float bc2, const float* clip, float gscale, int round_bf16,
                      void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n, 256, 16);
  if (g_f32)
    adamw_kernel<float><<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(p), static_cast<const float*>(g),
                                              static_cast<__nv_bfloat16*>(m), static_cast<__nv_bfloat16*>(v), n, lr,
                                              b1, b2, eps, decay, bc1, bc2, clip, gscale, round_bf16);
  else
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(p),
                                                      static_cast<const __nv_bfloat16*>(g),
                                                      static_cast<__nv_bfloat16*>(m), static_cast<__nv_bfloat16*>(v), n,
                                                      lr, b1, b2, eps, decay, bc1, bc2, clip, gscale, 0);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// AdamW over a flat arena of n elements (n % 8 == 0, 16-byte aligned bases) split into nreg
// regions: bounds[nreg + 1] (device, ascending, bounds[0] = 0, bounds[nreg] = n) and
// modes[nreg] (device: 1 decay, 0 no decay, -1 frozen).  One launch.
CTB_API int ctb_adamw_regions(void* p, const void* g, int g_f32, void* m, void* v, long n, const long* bounds,
                              const int* modes, int nreg, float lr, float b1, float b2, float eps, float decay,
                              float bc1, float bc2, const float* clip, float gscale, int round_bf16, void* stream) {
  if (n % 8) return fail("adamw_regions: the arena must be a whole number of 16-byte vectors");
  if (nreg < 1 || nreg > ADAM_MAX_REGIONS) return fail("adamw_regions: between 1 and 512 regions");
  auto misaligned = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) != 0; };
  if (misaligned(p) || misaligned(g) || misaligned(m) || misaligned(v))
    return fail("adamw_regions: parameter, gradient and moment arenas must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n / 8, 256, 8);
  if (g_f32)
    adamw_regions_kernel<float><<<grid, 256, 0, s>>>(
        static_cast<__nv_bfloat16*>(p), static_cast<const float*>(g), static_cast<__nv_bfloat16*>(m),
        static_cast<__nv_bfloat16*>(v), n, bounds, modes, nreg, lr, b1, b2, eps, decay, bc1, bc2, clip, gscale,
        round_bf16);
  else
    adamw_regions_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(
        static_cast<__nv_bfloat16*>(p), static_cast<const __nv_bfloat16*>(g), static_cast<__nv_bfloat16*>(m),
        static_cast<__nv_bfloat16*>(v), n, bounds, modes, nreg, lr, b1, b2, eps, decay, bc1, bc2, clip, gscale, 0);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// idx[k] = k-th row with w != 0 (k < total[0]); block_counts is scratch of ceil(rows / 1024) ints.
CTB_API int ctb_active_rows(const float* w, int rows, int* block_counts, int* idx, int* total, void* stream) {
  if (rows <= 0) return fail("active_rows: no rows");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int blocks = (rows + ACTIVE_BLOCK - 1) / ACTIVE_BLOCK;
  active_count_kernel<<<blocks, ACTIVE_BLOCK, 0, s>>>(w, rows, block_counts);
  CTB_CUDA_OK(cudaGetLastError());
  active_fill_kernel<<<blocks, ACTIVE_BLOCK, 0, s>>>(w, rows, block_counts, idx, total);
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// dst[j, :] = src[idx[j], :] for j < n (bf16 rows of d elements, d % 8 == 0; src has `rows` rows).
CTB_API int ctb_gather_rows(const void* src, long src_stride, int rows, const int* idx, void* dst, long n, int d,
                            void* stream) {
  if (d % 8 || src_stride % 8) return fail("gather_rows: rows must be whole 16-byte vectors");
  if (n <= 0) return 0;
  gather_rows_kernel<<<grid_for(n * (d / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), src_stride, idx, static_cast<__nv_bfloat16*>(dst), n, d, rows,
      device_status());
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}

// dst[idx[j], :] = src[j, :] for j < min(n, total[0]); dst has `rows` rows, those no j names are left alone.
CTB_API int ctb_scatter_rows(const void* src, const int* idx, const int* total, void* dst, long dst_stride, int rows,
                             long n, int d, void* stream) {
  if (d % 8 || dst_stride % 8) return fail("scatter_rows: rows must be whole 16-byte vectors");
  if (n <= 0) return 0;
  scatter_rows_kernel<<<grid_for(n * (d / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), idx, total, static_cast<__nv_bfloat16*>(dst), dst_stride, n, d, rows,
      device_status());
  CTB_CUDA_OK(cudaGetLastError());
  return 0;
}
