// Skeleton shared by the fused element-wise kernels: a CTA walks a strip of consecutive
// time steps of one batch row; thread i owns channels [8i, 8i+8) for the whole strip, so
// per-channel parameters live in registers and per-channel parameter gradients accumulate
// in registers without any cross-thread traffic.  Row statistics (LayerNorm) go through a
// double-buffered shared-memory block reduction; per-head statistics (64 channels = 8
// threads) go through three shuffle stages.
#pragma once
#include "common.cuh"

constexpr int EW_MAX_WARPS = 32;

struct RowCtx {
  int b, t0, t1, T, C;
  int col;        // first channel of this thread
  bool active;    // col < C
};

__device__ __forceinline__ RowCtx make_row_ctx(int T, int C, int strip) {
  RowCtx c;
  c.b = blockIdx.y;
  c.t0 = blockIdx.x * strip;
  c.t1 = min(T, c.t0 + strip);
  c.T = T;
  c.C = C;
  c.col = threadIdx.x * 8;
  c.active = c.col < C;
  return c;
}

__device__ __forceinline__ void load8f(const float* p, float* f) {
  const float4 a = reinterpret_cast<const float4*>(p)[0];
  const float4 b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void store8f(float* p, const float* f) {
  reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
}
__device__ __forceinline__ uint4 ldg16(const bf16* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void stg16(bf16* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }

// round-trip through bf16 so that recomputed values match what was stored
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// Block-wide sum of NV values per thread.  `buf` is [2][EW_MAX_WARPS][NV]; `phase` alternates
// between calls so one barrier per call is enough.
template <int NV>
__device__ __forceinline__ void block_sum(float (&v)[NV], float* buf, int& phase) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int i = 0; i < NV; ++i) v[i] = warp_sum(v[i]);
  float* slot = buf + phase * EW_MAX_WARPS * NV;
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < NV; ++i) slot[warp * NV + i] = v[i];
  }
  __syncthreads();
  // every warp folds the per-warp partials itself: lane w reads warp w's value, then one shuffle tree
#pragma unroll
  for (int i = 0; i < NV; ++i) v[i] = warp_sum(lane < nw ? slot[lane * NV + i] : 0.f);
  phase ^= 1;
}

// sum over the 8 threads that share a 64-channel head
__device__ __forceinline__ float head_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}
