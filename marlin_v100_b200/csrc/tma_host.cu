// Host-side tensor-map encoding.  The driver entry point is resolved through the runtime, so the
// library carries no link-time dependency on libcuda.
#include <array>
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tma.cuh"

namespace mb200 {

namespace {
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
std::once_flag g_once;
}  // namespace

int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides, const uint32_t* box,
                      CUtensorMapSwizzle swizzle) {
  std::call_once(g_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeFn>(fn);
  });
  if (g_encode == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return MARLIN_B200_ECUDA;
  }
  cuuint64_t gdims[5], gstrides[4];
  cuuint32_t gbox[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstrides[i - 1] = strides[i - 1];
  }
  const CUresult r = g_encode(map, dtype, (cuuint32_t)rank, const_cast<void*>(base), gdims, gstrides, gbox, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (rank %d, dims %llu x %llu, box %u x %u)", (int)r, rank,
              (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 0), box[0],
              rank > 1 ? box[1] : 0);
    return MARLIN_B200_ECUDA;
  }
  return 0;
}

namespace {
struct MapKey {
  const void* ptr;
  std::array<uint64_t, 16> v;  // dtype, rank, swizzle, dims[5], strides[4], box[4] (rank <= 4 in this library)
  bool operator==(const MapKey& o) const { return ptr == o.ptr && v == o.v; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    for (uint64_t x : k.v) h = h * 1000003u ^ std::hash<uint64_t>()(x);
    return h;
  }
};
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;
}  // namespace

int cached_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides, const uint32_t* box,
                      CUtensorMapSwizzle swizzle) {
  if (rank > 4) return encode_tensor_map(map, dtype, rank, base, dims, strides, box, swizzle);
  MapKey key{};
  key.ptr = base;
  key.v[0] = (uint64_t)dtype; key.v[1] = (uint64_t)rank; key.v[2] = (uint64_t)swizzle;
  for (int i = 0; i < rank; ++i) { key.v[3 + i] = dims[i]; key.v[12 + i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) key.v[8 + i] = strides[i];
  std::lock_guard<std::mutex> lock(g_map_mutex);
  auto it = g_map_cache.find(key);
  if (it != g_map_cache.end()) {
    *map = it->second;
    return 0;
  }
  if (int rc = encode_tensor_map(map, dtype, rank, base, dims, strides, box, swizzle)) return rc;
  if (g_map_cache.size() > 4096) g_map_cache.clear();
  g_map_cache.emplace(key, *map);
  return 0;
}

}  // namespace mb200
