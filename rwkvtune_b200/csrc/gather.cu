// Row gathers and the embedding gradient.
//
//   rwkv_gather_rows        dst[i, :] = src[index[i], :] on rows of `row_bytes` bytes (multiple of 16).
//                           One kernel serves the embedding lookup ([V, C] table), the fan-out of a
//                           prefilled recurrent state to G sampling paths, and the compaction of the
//                           live rows of a state pool (rwkvtune/inference/grpo_batch_generator.py:245-300
//                           does these with index_select / repeat_interleave per tensor).
//   rwkv_embedding_backward dW[idx, :] = sum of dy rows with that index, accumulated in fp32 in a fixed
//                           order (positions sorted by index), so the result is deterministic.
#include "common.cuh"

RWKV_DEFINE_DEBUG_EVENTS(gather)

namespace {

__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ src, const long long* __restrict__ index, uint4* __restrict__ dst,
                   long long n_out, long long n_src, int vec_per_row) {
  const long long total = n_out * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = (int)(i - r * vec_per_row);
    const long long s = index[r];
    dst[i] = RWKV_IN_RANGE(s, n_src, 1) ? src[s * vec_per_row + c] : make_uint4(0u, 0u, 0u, 0u);
  }
}

// grid = M sorted positions; a block works only if it is the first of its run of equal indices.
__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const bf16* __restrict__ dy, const long long* __restrict__ sorted_idx,
                     const long long* __restrict__ order, bf16* __restrict__ dW, long long M, long long V, int C) {
  const long long i = blockIdx.x;
  const long long tok = sorted_idx[i];
  if (!RWKV_IN_RANGE(tok, V, 2)) return;
  if (i > 0 && sorted_idx[i - 1] == tok) return;
  for (int c = threadIdx.x * 8; c < C; c += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (long long j = i; j < M && sorted_idx[j] == tok; ++j) {
      float f[8];
      if (!RWKV_IN_RANGE(order[j], M, 3)) continue;
      unpack8(*reinterpret_cast<const uint4*>(dy + order[j] * C + c), f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
    *reinterpret_cast<uint4*>(dW + tok * C + c) = pack8(acc);
  }
}

}  // namespace

RWKV_EXPORT int rwkv_gather_rows(const void* src, const void* index, void* dst, long long n_out, long long n_src,
                                 long long row_bytes, void* stream) {
  if (n_out <= 0) return RWKV_OK;
  if (row_bytes <= 0 || (row_bytes & 15) || row_bytes / 16 > 0x7fffffffLL) return RWKV_ERR_BAD_SHAPE;
  if (((uintptr_t)src | (uintptr_t)dst) & 15) return RWKV_ERR_BAD_ALIGNMENT;
  const int vec = (int)(row_bytes / 16);
  const long long total = n_out * vec;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  gather_rows_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, (const long long*)index,
                                                                        (uint4*)dst, n_out, n_src, vec);
  return rwkv_launch_status();
}

// dW must be zero-filled by the caller (rows whose token does not occur stay zero).
RWKV_EXPORT int rwkv_embedding_backward(const void* dy, const void* sorted_idx, const void* order, void* dW,
                                        long long M, long long V, int C, void* stream) {
  if (M <= 0) return RWKV_OK;
  if (C <= 0 || (C & 7) || M > 0x7fffffffLL) return RWKV_ERR_BAD_SHAPE;
  embedding_bwd_kernel<<<(unsigned)M, 256, 0, (cudaStream_t)stream>>>((const bf16*)dy, (const long long*)sorted_idx,
                                                                      (const long long*)order, (bf16*)dW, M, V, C);
  return rwkv_launch_status();
}
