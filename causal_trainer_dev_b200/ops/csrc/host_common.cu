#include "host_common.h"

#include <cudaTypedefs.h>

#include <cstring>
#include <vector>

namespace ctb {

static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }
int fail(const std::string& msg) {
  g_last_error = msg;
  return 1;
}

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeFn>(p);
    }
  });
  return fn;
}

struct MapKey {
  uint64_t v[16];
  bool operator==(const MapKey& o) const { return std::memcmp(v, o.v, sizeof(v)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (uint64_t x : k.v) {
      h ^= x;
      h *= 1099511628211ull;
    }
    return static_cast<size_t>(h);
  }
};

std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap*, MapKeyHash> g_maps;

const CUtensorMap* lookup_or_encode(const MapKey& key, const void* base, Elt elt, uint32_t rank, const uint64_t* dims,
                                    const uint64_t* strides_elems, const uint32_t* box, bool swizzle128) {
  std::lock_guard<std::mutex> lock(g_map_mutex);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) return it->second;
  EncodeFn fn = encode_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return nullptr;
  }
  const uint64_t esize = (elt == Elt::BF16) ? 2 : 4;
  cuuint64_t gdims[4];
  cuuint64_t gstrides[3];
  cuuint32_t gbox[4];
  cuuint32_t estr[4] = {1, 1, 1, 1};
  for (uint32_t i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
  }
  for (uint32_t i = 0; i + 1 < rank; ++i) gstrides[i] = strides_elems[i] * esize;
  auto* map = new CUtensorMap;
  CUresult r = fn(map, elt == Elt::BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, rank,
                  const_cast<void*>(base), gdims, gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    delete map;
    set_error("cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)) +
              " (base must be 16-byte aligned, strides multiples of 16 bytes)");
    return nullptr;
  }
  if (g_maps.size() > 65536) {  // bound the cache; maps are tiny but pointers churn under allocator reuse
    for (auto& kv : g_maps) delete kv.second;
    g_maps.clear();
  }
  g_maps.emplace(key, map);
  return map;
}

}  // namespace

const CUtensorMap* get_tensor_map_2d(const void* base, Elt elt, uint64_t inner, uint64_t outer, uint64_t row_stride,
                                     uint32_t box_inner, uint32_t box_outer, bool swizzle128) {
  MapKey key{};
  key.v[0] = reinterpret_cast<uint64_t>(base);
  key.v[1] = static_cast<uint64_t>(elt) | (2ull << 8) | (swizzle128 ? 1ull << 16 : 0);
  key.v[2] = inner;
  key.v[3] = outer;
  key.v[4] = row_stride;
  key.v[5] = box_inner;
  key.v[6] = box_outer;
  int dev = 0;
  cudaGetDevice(&dev);
  key.v[7] = static_cast<uint64_t>(dev);
  uint64_t dims[2] = {inner, outer};
  uint64_t strides[1] = {row_stride};
  uint32_t box[2] = {box_inner, box_outer};
  return lookup_or_encode(key, base, elt, 2, dims, strides, box, swizzle128);
}

const CUtensorMap* get_tensor_map_3d(const void* base, Elt elt, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1,
                                     uint64_t s2, uint32_t b0, uint32_t b1, uint32_t b2, bool swizzle128) {
  MapKey key{};
  key.v[0] = reinterpret_cast<uint64_t>(base);
  key.v[1] = static_cast<uint64_t>(elt) | (3ull << 8) | (swizzle128 ? 1ull << 16 : 0);
  key.v[2] = d0;
  key.v[3] = d1;
  key.v[4] = d2;
  key.v[5] = s1;
  key.v[6] = s2;
  key.v[7] = b0;
  key.v[8] = b1;
  key.v[9] = b2;
  int dev = 0;
  cudaGetDevice(&dev);
  key.v[10] = static_cast<uint64_t>(dev);
  uint64_t dims[3] = {d0, d1, d2};
  uint64_t strides[2] = {s1, s2};
  uint32_t box[3] = {b0, b1, b2};
  return lookup_or_encode(key, base, elt, 3, dims, strides, box, swizzle128);
}

const CUtensorMap* get_tensor_map_4d(const void* base, Elt elt, const uint64_t dims[4], const uint64_t strides[3],
                                     const uint32_t box[4], bool swizzle128) {
  MapKey key{};
  key.v[0] = reinterpret_cast<uint64_t>(base);
  key.v[1] = static_cast<uint64_t>(elt) | (4ull << 8) | (swizzle128 ? 1ull << 16 : 0);
  for (int i = 0; i < 4; ++i) key.v[2 + i] = dims[i];
  for (int i = 0; i < 3; ++i) key.v[6 + i] = strides[i];
  for (int i = 0; i < 4; ++i) key.v[9 + i] = box[i];
  int dev = 0;
  cudaGetDevice(&dev);
  key.v[13] = static_cast<uint64_t>(dev);
  return lookup_or_encode(key, base, elt, 4, dims, strides, box, swizzle128);
}

namespace {
std::mutex g_status_mutex;
DeviceStatus* g_status[64] = {nullptr};
int g_sm_count[64] = {0};
}  // namespace

DeviceStatus* device_status() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (g_status[dev] == nullptr) {
    DeviceStatus* p = nullptr;
    if (cudaMalloc(&p, sizeof(DeviceStatus)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(DeviceStatus));
    g_status[dev] = p;
  }
  return g_status[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sm_count[dev] = n > 0 ? n : 148;
  }
  return g_sm_count[dev];
}

}  // namespace ctb

CTB_API const char* ctb_last_error() { return ctb::g_last_error.c_str(); }

// Copies the device status word to `out[4]` (code, block, detail0, detail1) and clears it.
// Synchronises the given stream first.
CTB_API int ctb_status(unsigned int* out, void* stream) {
  ctb::DeviceStatus* st = ctb::device_status();
  if (st == nullptr) return ctb::fail("no status word on this device");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CTB_CUDA_OK(cudaStreamSynchronize(s));
  CTB_CUDA_OK(cudaMemcpy(out, st, sizeof(ctb::DeviceStatus), cudaMemcpyDeviceToHost));
  if (out[0] != 0) CTB_CUDA_OK(cudaMemset(st, 0, sizeof(ctb::DeviceStatus)));
  return 0;
}
