#include "tensormap.h"

#include "agb.h"

#include <cstdio>
#include <cstring>
#include <mutex>
#include <unordered_map>

namespace agb {
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) ==
            cudaSuccess &&
        result == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeFn>(ptr);
    }
  });
  return fn;
}

}  // namespace

namespace {
thread_local const char* g_detail = "";

// A tensor map is a pure function of (base, rank, dims, strides, box) for the fixed type,
// swizzle and fill used here, and the allocator hands the same addresses back step after
// step, so encoded maps are kept per host thread and looked up instead of re-encoded
// (two or more encodes per launch otherwise, a few thousand launches per training step).
struct MapKey {
  uint64_t words[16];
  bool operator==(const MapKey& other) const { return memcmp(words, other.words, sizeof(words)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& key) const {
    uint64_t h = 0x9e3779b97f4a7c15ull;
    for (uint64_t w : key.words) h = (h ^ w) * 0x100000001b3ull + (h >> 29);
    return size_t(h);
  }
};
constexpr size_t kMaxCachedMaps = 1 << 14;
}
void set_error_detail(const char* text) { g_detail = text; }
const char* error_detail() { return g_detail; }

bool make_tensor_map_bf16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  // The driver call needs a current context; a thread that has only used the runtime API
  // lazily (e.g. an autograd worker) may not have bound the primary context yet.
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
  if (rank < 1 || rank > 5) return false;
  MapKey key{};
  key.words[0] = reinterpret_cast<uint64_t>(base);
  key.words[1] = uint64_t(rank);
  for (int i = 0; i < rank; ++i) {
    key.words[2 + i] = dims[i];
    key.words[11 + i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) key.words[7 + i] = strides_bytes[i];
  static thread_local std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  auto found = cache.find(key);
  if (found != cache.end()) {
    *map = found->second;
    return true;
  }
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estrides[5] = {1, 1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) gstrides[i] = strides_bytes[i];
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank),
                  const_cast<void*>(base), gdims, gstrides, gbox, estrides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    static thread_local char text[256];
    snprintf(text, sizeof(text),
             "cuTensorMapEncodeTiled -> %d (base %p rank %d dims %llu %llu %llu stride0 %llu box %u %u)",
             int(r), base, rank, (unsigned long long)dims[0],
             (unsigned long long)(rank > 1 ? dims[1] : 0), (unsigned long long)(rank > 2 ? dims[2] : 0),
             (unsigned long long)(rank > 1 ? strides_bytes[0] : 0), box[0], rank > 1 ? box[1] : 0);
    set_error_detail(text);
    return false;
  }
  if (cache.size() >= kMaxCachedMaps) cache.clear();
  cache.emplace(key, *map);
  return true;
}

}  // namespace agb
