// See rmsnorm_noalloc.h for who this is for and the full contract.
//
// The weight gradient of RMSNorm is a column sum over all rows.  Each CTA walks a strided
// set of rows, keeps its column sums in registers and writes them as one row of a
// [parts][d] fp32 table; a second kernel adds the table's rows in a fixed order (no
// atomics, so the result does not depend on scheduling).  In the regular entry point that
// table is caller-provided scratch; here it is the static array below.
#include "rmsnorm_noalloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

namespace {

constexpr int THREADS = 256;
constexpr int MAX_DEVICES = 64;

// Partial column sums, one row per CTA.  Lives in the library image on every device that
// loads it.  In host code this name is only a handle for cudaGetSymbolAddress: it is NOT a
// device pointer and must never be passed to a kernel as one.
static __device__ __align__(256) float g_dw_partials[CTB_NOALLOC_MAX_PARTS * CTB_NOALLOC_MAX_D];

thread_local char t_error[256] = "";

int refuse(const char* what) {
  snprintf(t_error, sizeof(t_error), "%s", what);
  return 1;
}
int refuse_cuda(const char* what, cudaError_t e) {
  snprintf(t_error, sizeof(t_error), "%s: %s", what, cudaGetErrorString(e));
  return 1;
}

std::mutex g_mutex;
float* g_table[MAX_DEVICES] = {nullptr};   // device address of g_dw_partials, per device
int g_sms[MAX_DEVICES] = {0};

// Resolves (once per device, with that device current) the device address of the table.
int table_for_current_device(float** table, int* sms) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return refuse_cuda("cudaGetDevice", e);
  if (dev < 0 || dev >= MAX_DEVICES) return refuse("device index out of range for the per-device table");
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_table[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_dw_partials);
    if (e != cudaSuccess) return refuse_cuda("cudaGetSymbolAddress(g_dw_partials)", e);
    int n = 0;
    e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return refuse_cuda("cudaDeviceGetAttribute", e);
    g_sms[dev] = n > 0 ? n : 1;
    g_table[dev] = p;
  }
  *table = g_table[dev];
  *sms = g_sms[dev];
  return 0;
}

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
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < THREADS / 32) ? scratch[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres); row `blockIdx.x` of `table` receives
// this CTA's sums of dy * xhat.  NV = 8-element vectors per thread (d <= NV * 2048).
template <int NV>
__global__ void __launch_bounds__(THREADS)
rmsnorm_bwd_static_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                          const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                          const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                          float* __restrict__ table, int rows, int d) {
  __shared__ float scratch[33];
  const int nvec = d / 8;
  float acc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rs = rstd[row];
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(row) * d);
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * d);
    float gx[NV][8], xh[NV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * THREADS;
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
          acc[i][e] += a[e] * xh[i][e];
        }
      }
    }
    const float mean = block_sum(dot, scratch) / d;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * THREADS;
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
  // Every CTA writes its whole row of the table, including CTAs that saw no row (zeros),
  // so the reduce below never reads a stale element of an earlier call.
  float* out = table + static_cast<size_t>(blockIdx.x) * d;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * THREADS;
    if (v < nvec) {
      float4* o4 = reinterpret_cast<float4*>(out + v * 8);
      o4[0] = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
      o4[1] = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    }
  }
}

__global__ void dw_from_table_kernel(const float* __restrict__ table, int parts, int d, void* __restrict__ dw,
                                     int out_f32, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += table[static_cast<size_t>(p) * d + c];
  if (out_f32) {
    float* o = static_cast<float*>(dw);
    o[c] = accumulate ? o[c] + s : s;
  } else {
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(dw);
    o[c] = __float2bfloat16(accumulate ? __bfloat162float(o[c]) + s : s);
  }
}

}  // namespace

extern "C" __attribute__((visibility("default"))) const char* ctb_noalloc_last_error(void) { return t_error; }

extern "C" __attribute__((visibility("default"))) int ctb_rmsnorm_bwd_noalloc(
    const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx, void* dw, int dw_f32,
    int dw_accumulate, int rows, int d, void* stream) {
  if (rows <= 0 || d <= 0) return refuse("rmsnorm_bwd_noalloc: rows and d must be positive");
  if (d % 8) return refuse("rmsnorm_bwd_noalloc: d must be a multiple of 8");
  if (d > CTB_NOALLOC_MAX_D)
    return refuse("rmsnorm_bwd_noalloc: d exceeds CTB_NOALLOC_MAX_D (8192), the size the static scratch was built for");
  if (!dy || !x || !w || !rstd || !dx) return refuse("rmsnorm_bwd_noalloc: dy, x, w, rstd and dx are required");
  // The kernel moves rows in 16-byte vectors.  A pointer into the middle of a vector (a sliced
  // view, an odd offset into a pool) would fault on the device, so it is refused here instead.
  auto misaligned = [](const void* p, uintptr_t a) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) % a) != 0; };
  if (misaligned(dy, 16) || misaligned(x, 16) || misaligned(w, 16) || misaligned(dres, 16) || misaligned(dx, 16))
    return refuse("rmsnorm_bwd_noalloc: dy, x, w, dres and dx must be 16-byte aligned");
  if (misaligned(rstd, 4) || misaligned(dw, dw_f32 ? 4 : 2))
    return refuse("rmsnorm_bwd_noalloc: rstd and dw must be aligned to their element size");
  float* table = nullptr;
  int sms = 0;
  if (table_for_current_device(&table, &sms)) return 1;   // first call on this device resolves the address
  int parts = sms * 2;
  if (parts > CTB_NOALLOC_MAX_PARTS) parts = CTB_NOALLOC_MAX_PARTS;
  if (parts > rows) parts = rows;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int nv = (d / 8 + THREADS - 1) / THREADS;
#define CTB_LAUNCH(NV)                                                                               \
  rmsnorm_bwd_static_kernel<NV><<<parts, THREADS, 0, s>>>(                                           \
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),                   \
      static_cast<const __nv_bfloat16*>(w), rstd, static_cast<const __nv_bfloat16*>(dres),           \
      static_cast<__nv_bfloat16*>(dx), table, rows, d)
  if (nv <= 1) CTB_LAUNCH(1);
  else if (nv <= 2) CTB_LAUNCH(2);
  else CTB_LAUNCH(4);
#undef CTB_LAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return refuse_cuda("rmsnorm_bwd_noalloc launch", e);
  if (dw != nullptr) {
    dw_from_table_kernel<<<(d + 255) / 256, 256, 0, s>>>(table, parts, d, dw, dw_f32, dw_accumulate);
    e = cudaGetLastError();
    if (e != cudaSuccess) return refuse_cuda("rmsnorm_bwd_noalloc reduce launch", e);
  }
  return 0;
}
