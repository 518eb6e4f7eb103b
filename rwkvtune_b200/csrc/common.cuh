// Shared device helpers for the sm_100a kernels of rwkvtune_b200.
// Everything here is header-only; kernels are exported with C linkage and take raw
// device pointers plus a cudaStream_t so the library has no dependency on libtorch.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define RWKV_EXPORT extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;

// Error codes returned by the C entry points (0 = ok).  Launch failures return the
// cudaError_t value offset by 1000 so the Python side can print cudaGetErrorString.
enum RwkvStatus : int {
  RWKV_OK = 0,
  RWKV_ERR_BAD_SHAPE = 1,
  RWKV_ERR_BAD_ALIGNMENT = 2,
  RWKV_ERR_TOO_LARGE = 3,
  RWKV_ERR_NOT_INITIALISED = 4,
  RWKV_ERR_WAIT_TIMEOUT = 5,
  RWKV_ERR_CUDA_BASE = 1000,
};

static inline int rwkv_launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? RWKV_OK : RWKV_ERR_CUDA_BASE + (int)e;
}

// ------------------------------------------------------------------------------------------------------------------
// Chained launches (programmatic dependent launch).  A decode step is ~250 kernels of a few microseconds each, so the
// gap between two kernels of the stream costs as much as the kernels.  When chaining is on (`rwkv_set_launch_chaining`,
// switched on by the inference engine around its decode loop), the kernels of the decode path are launched with the
// programmatic-stream-serialisation attribute: a kernel may be scheduled while its predecessor is still running, does
// whatever does not depend on it, and `rwkv_chain_wait()` then blocks until the predecessor has completed and its
// writes are visible.  Every chained kernel calls `rwkv_chain_begin()` (or `rwkv_chain_trigger()` then, later,
// `rwkv_chain_wait()`) before its first access to anything another kernel of the chain writes, so the order of the
// stream is kept transitively; model parameters - constant while chaining is on - may be requested before the wait.
// Launched the ordinary way the two instructions do nothing.
__device__ __forceinline__ void rwkv_chain_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void rwkv_chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void rwkv_chain_begin() {
  rwkv_chain_trigger();
  rwkv_chain_wait();
}
inline int& rwkv_chain_flag() {
  static int flag = 0;
  return flag;
}
template <typename... KArgs, typename... Args>
static inline void rwkv_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                               Args... args) {
  if (!rwkv_chain_flag()) {
    kernel<<<grid, block, smem, st>>>(args...);
    return;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

// 8 bf16 values (one 16-byte vector) -> 8 floats
__device__ __forceinline__ void unpack8(const uint4& p, float* f) {
  f[0] = bf16_lo(p.x); f[1] = bf16_hi(p.x);
  f[2] = bf16_lo(p.y); f[3] = bf16_hi(p.y);
  f[4] = bf16_lo(p.z); f[5] = bf16_hi(p.z);
  f[6] = bf16_lo(p.w); f[7] = bf16_hi(p.w);
}

__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 p;
  p.x = pack_bf16(f[0], f[1]);
  p.y = pack_bf16(f[2], f[3]);
  p.z = pack_bf16(f[4], f[5]);
  p.w = pack_bf16(f[6], f[7]);
  return p;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }


// ------------------------------------------------------------------------------------------------------------------
// Debug build (`python -m rwkvtune_b200.csrc.build --debug`, -DRWKV_DEBUG_BOUNDS): data-dependent indices (token ids,
// labels, gather indices, row permutations) are range-checked where they are used.  An index out of range is
// *recorded* - event count, kernel tag, the index and its limit - and the access is skipped; nothing traps, asserts or
// faults, so the context stays usable and the host reads the record afterwards (`rwkv_debug_read_<file>`).  In the
// release build the same call is the plain range test the kernels rely on anyway.
// Each translation unit that uses the check instantiates its own record with RWKV_DEFINE_DEBUG_EVENTS(tag).
#ifdef RWKV_DEBUG_BOUNDS
#define RWKV_DEFINE_DEBUG_EVENTS(tag)                                                                     \
  static __device__ long long rwkv_debug_events_[4];   /* count, kernel tag of the first event, index, limit */ \
  RWKV_EXPORT int rwkv_debug_read_##tag(long long* out4, int reset) {                                     \
    cudaError_t e = cudaMemcpyFromSymbol(out4, rwkv_debug_events_, 4 * sizeof(long long));                \
    if (e == cudaSuccess && reset) {                                                                      \
      const long long zero[4] = {0, 0, 0, 0};                                                             \
      e = cudaMemcpyToSymbol(rwkv_debug_events_, zero, sizeof(zero));                                     \
    }                                                                                                     \
    return e == cudaSuccess ? RWKV_OK : RWKV_ERR_CUDA_BASE + (int)e;                                      \
  }
#define RWKV_IN_RANGE(i, n, kernel_tag) rwkv_in_range_dbg_((long long)(i), (long long)(n), (kernel_tag), rwkv_debug_events_)
__device__ __forceinline__ bool rwkv_in_range_dbg_(long long i, long long n, int kernel_tag, long long* ev) {
  if (i >= 0 && i < n) return true;
  if (atomicAdd(reinterpret_cast<unsigned long long*>(&ev[0]), 1ull) == 0ull) {
    ev[1] = kernel_tag; ev[2] = i; ev[3] = n;
  }
  return false;
}
#else
#define RWKV_DEFINE_DEBUG_EVENTS(tag)
#define RWKV_IN_RANGE(i, n, kernel_tag) ((long long)(i) >= 0 && (long long)(i) < (long long)(n))
#endif
