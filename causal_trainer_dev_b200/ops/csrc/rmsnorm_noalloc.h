// RMSNorm backward for callers that may not allocate device memory.
//
// This entry point has no counterpart in the reference trainer; it exists for embedders
// of this library.
//
// Who needs it: a host application that reserves the GPU's memory for its own pool (a
// serving runtime, a trainer with a pre-sized arena) and therefore forbids cudaMalloc in
// the libraries it loads, and any caller on a path where the implicit device-wide
// synchronisation of cudaMalloc / cudaFree cannot be tolerated.  The regular entry point
// (ctb_rmsnorm_bwd) asks its caller for a scratch buffer of ctb_rmsnorm_bwd_parts(rows) * d
// floats; the Python wrapper gets that buffer from torch's allocator.  This variant needs
// no buffer: the per-CTA partial sums of the weight gradient live in a fixed array inside
// the library image.
//
// Contract
//   * same arguments and results as ctb_rmsnorm_bwd minus the scratch pointer: the caller
//     still passes inputs (dy, x, w, rstd, optional dres) and outputs (dx, dw);
//   * limit: d <= CTB_NOALLOC_MAX_D (8192) and d a multiple of 8; larger sizes are refused
//     with a message (ctb_noalloc_last_error), nothing is launched;
//   * dy, x, w, dres and dx are read and written in 16-byte vectors and must be 16-byte
//     aligned (rstd and dw: aligned to their element); a misaligned pointer is refused the
//     same way, before any launch;
//   * cost: CTB_NOALLOC_MAX_PARTS * CTB_NOALLOC_MAX_D floats (9.5 MiB) of device memory on
//     every GPU that loads the library, held until the process exits;
//   * the first call on a device resolves the device address of the array (one
//     cudaGetSymbolAddress with that device current).  Make that first call during set-up,
//     before any stream capture begins on that device;
//   * the array is shared by all calls and keeps the previous call's contents.  Nothing in
//     it has to start at zero: each call overwrites every element it later reads.  Two
//     calls whose kernels overlap on the GPU (different streams, no ordering) race on the
//     array; order them on one stream or with events;
//   * no cudaMalloc, cudaFree or allocating library routine is called, on any path.
#pragma once

#define CTB_NOALLOC_MAX_D 8192
#define CTB_NOALLOC_MAX_PARTS 304

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0 on success.  dw may be null (only dx is wanted); dw_f32 selects fp32 / bf16
// for dw; dw_accumulate adds to the existing contents of dw.
int ctb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                            void* dx, void* dw, int dw_f32, int dw_accumulate, int rows, int d, void* stream);

// Message of the last failure of ctb_rmsnorm_bwd_noalloc on the calling thread.
const char* ctb_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
