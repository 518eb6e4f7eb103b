// Host-side cache of encoded TMA tensor maps.
//
// Every GEMM launch needs three CUtensorMap objects (A, B, C).  cuTensorMapEncodeTiled costs about a microsecond
// each on the host, which shows in host-bound steps (decode, small chunks).  Parameters and, thanks to the
// framework's caching allocator, most activations come back at the same address with the same shape, so the encoded
// maps are kept in a small table keyed by (address, rows, cols, leading dimension, box) and reused.  A map depends
// on nothing else: it does not go stale when the memory behind the address is rewritten or re-allocated.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace rwkv_tmap {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

struct Key {
  uintptr_t ptr;
  long long rows, cols, ld;
  int box_cols, box_rows;
  bool operator==(const Key& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_cols == o.box_cols && box_rows == o.box_rows;
  }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    uint64_t h = (uint64_t)k.ptr * 0x9E3779B97F4A7C15ull;
    h ^= ((uint64_t)k.rows + 0x7F4A7C15ull) * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    h ^= ((uint64_t)k.cols * 0x165667B19E3779F9ull) + (h << 6) + (h >> 2);
    h ^= ((uint64_t)k.ld * 0x27D4EB2F165667C5ull) + (h << 6) + (h >> 2);
    h ^= (uint64_t)(k.box_cols * 131 + k.box_rows) + (h << 6) + (h >> 2);
    return (size_t)h;
  }
};

constexpr size_t MAX_ENTRIES = 8192;

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with leading dimension `ld` (elements),
// box = {box_cols, box_rows}, 128-byte swizzle.
inline int make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld, int box_cols,
                    int box_rows) {
  if (((uintptr_t)ptr & 15) || (ld * 2) % 16) return RWKV_ERR_BAD_ALIGNMENT;
  static std::mutex mu;
  static std::unordered_map<Key, CUtensorMap, KeyHash> table;
  const Key key{(uintptr_t)ptr, rows, cols, ld, box_cols, box_rows};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = table.find(key);
    if (it != table.end()) {
      *map = it->second;
      return RWKV_OK;
    }
  }
  EncodeTiledFn enc = get_encode();
  if (!enc) return RWKV_ERR_NOT_INITIALISED;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // The encoder is a driver entry point and wants a current context.  A thread whose first CUDA work is this call
    // (an autograd worker starting a backward pass with a GEMM) has none yet: a runtime call binds the device's
    // primary context.  (Never reached while a stream is being captured: the capturing thread has a context.)
    cudaFree(nullptr);
    r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) return RWKV_ERR_CUDA_BASE + 900 + (int)r;
  std::lock_guard<std::mutex> lock(mu);
  if (table.size() >= MAX_ENTRIES) table.clear();
  table.emplace(key, *map);
  return RWKV_OK;
}

}  // namespace rwkv_tmap
