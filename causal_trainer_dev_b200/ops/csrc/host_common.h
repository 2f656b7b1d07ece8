// Host-side helpers shared by the launchers: error strings, tensor-map construction
// through the driver entry point (no link-time dependency on libcuda), a small cache
// of encoded maps, and the per-device status word.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <unordered_map>

#include "tc05.cuh"

#define CTB_API extern "C" __attribute__((visibility("default")))

namespace ctb {

// Last error message of the calling thread (returned by ctb_last_error()).
void set_error(const std::string& msg);
int fail(const std::string& msg);  // sets the message, returns a non-zero code

#define CTB_CUDA_OK(expr)                                                                        \
  do {                                                                                           \
    cudaError_t _e = (expr);                                                                     \
    if (_e != cudaSuccess) return ::ctb::fail(std::string(#expr) + ": " + cudaGetErrorString(_e)); \
  } while (0)

enum class Elt : int { BF16 = 0, F32 = 1 };

// Encodes (or fetches from cache) a tiled tensor map over a row-major 2-D view.
//   inner/outer: extents in elements; row_stride: elements between rows;
//   box_inner/box_outer: tile; swizzle128: 128-byte swizzle or none.
// Returns nullptr and sets the error message on failure.
const CUtensorMap* get_tensor_map_2d(const void* base, Elt elt, uint64_t inner, uint64_t outer, uint64_t row_stride,
                                     uint32_t box_inner, uint32_t box_outer, bool swizzle128);
// 3-D variant: dims {d0 (contiguous), d1, d2} with element strides s1, s2.
const CUtensorMap* get_tensor_map_3d(const void* base, Elt elt, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1,
                                     uint64_t s2, uint32_t b0, uint32_t b1, uint32_t b2, bool swizzle128);

// 4-D variant used by attention: dims {d0 (contiguous), d1, d2, d3}, element strides s1..s3.
const CUtensorMap* get_tensor_map_4d(const void* base, Elt elt, const uint64_t dims[4], const uint64_t strides[3],
                                     const uint32_t box[4], bool swizzle128);

// Per-device status word in device memory (allocated on first use).
DeviceStatus* device_status();

int sm_count();

}  // namespace ctb
