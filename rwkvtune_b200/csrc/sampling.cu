// Token sampling over a full vocabulary row without sorting it: repetition penalty (from a bitmap of tokens already
// seen), banned ids, temperature, additive logit bias, top-k, top-p, the draw (or the arg-max when greedy), the
// token's log-probability and the update of the seen-bitmap, in one kernel.
//
// One 1024-thread CTA per row; each thread keeps up to 64 probabilities, 24 in registers and 40 in shared memory
// (V <= 65536).  The nucleus is "the sorted prefix whose cumulative mass is <= top_p, plus
// always the most likely token" -- i.e. token i is kept iff the mass of all tokens at least as
// likely as i is <= top_p.  That set is {p >= theta*} for a threshold found by bisection on
// theta (each probe is one pass over registers and shared memory + one block reduction), so no sort, no cumsum and no
// scatter is needed.  The draw is an inverse-CDF walk over the kept tokens in index order with a
// Philox4x32-10 uniform keyed by (seed, row).  Replaces the full 65536-way sort + cumsum +
// unsort + softmax + multinomial sequence of the reference
// (rwkvtune/inference/core.py:165-238) and its per-sequence Python repetition penalty
// (rwkvtune/inference/grpo_batch_generator.py:25-42).  Top-k keeps every value >= the k-th largest (ties kept, as
// `logits < kth` masking does); the k-th largest is found exactly by a 32-step radix descent over the
// order-preserving integer image of the floats (one count reduction per bit).
#include "common.cuh"

namespace {

constexpr int ST = 1024;       // threads per row
constexpr int SPT = 64;        // values per thread
constexpr int SPT_REG = 24;    // of which in registers; the rest in shared memory (160 KB)
constexpr int SAMPLE_SMEM = (SPT - SPT_REG) * ST * 4;

__device__ __forceinline__ uint2 mulhilo(uint32_t a, uint32_t b) {
  const unsigned long long p = (unsigned long long)a * b;
  return make_uint2((uint32_t)p, (uint32_t)(p >> 32));
}

// Philox4x32-10; returns a uniform in (0, 1)
__device__ float philox_uniform(unsigned long long seed, unsigned long long ctr) {
  uint32_t c0 = (uint32_t)ctr, c1 = (uint32_t)(ctr >> 32), c2 = 0x243F6A88u, c3 = 0x85A308D3u;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint2 m0 = mulhilo(0xD2511F53u, c0), m1 = mulhilo(0xCD9E8D57u, c2);
    const uint32_t n0 = m1.y ^ c1 ^ k0, n1 = m1.x, n2 = m0.y ^ c3 ^ k1, n3 = m0.x;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return ((c0 >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = (threadIdx.x < 32) ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) s = warp_sum(s);
  if (threadIdx.x == 0) red[32] = s;
  __syncthreads();
  return red[32];
}

__device__ __forceinline__ float block_reduce_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = (threadIdx.x < 32) ? red[threadIdx.x] : -INFINITY;
  if (threadIdx.x < 32) s = warp_max(s);
  if (threadIdx.x == 0) red[32] = s;
  __syncthreads();
  return red[32];
}

struct SampleArgs {
  const float* bias;            // [V] additive bias applied after temperature scaling, or null
  unsigned char* seen;          // [*, V] bitmap of tokens already in each sequence's history, or null
  const long long* seen_rows;   // [n] row of `seen` that belongs to batch row i (null: row i)
  float penalty;                // repetition penalty (> 0, != 1 to have an effect)
  int top_k;                    // 0 = off
  int greedy;                   // 1: arg-max of the penalised, biased logits (no temperature)
  int update_seen;              // 1: mark the sampled token in `seen`
};

__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

#define PGET(j) ((j) < SPT_REG ? p_reg[(j) < SPT_REG ? (j) : 0] : p_sh[((j) - SPT_REG) * ST + tid])
#define PSET(j, v)                                         \
  do {                                                     \
    const float pset_v_ = (v);                             \
    if ((j) < SPT_REG) p_reg[(j) < SPT_REG ? (j) : 0] = pset_v_; \
    else p_sh[((j) - SPT_REG) * ST + tid] = pset_v_;       \
  } while (0)

template <typename T>
__global__ void __launch_bounds__(ST)
sample_top_p_kernel(const T* __restrict__ logits, int V, int n_valid, float inv_temp, float top_p,
                    unsigned long long seed, long long* __restrict__ tokens, float* __restrict__ logps,
                    const SampleArgs sa) {
  __shared__ float red[33];
  __shared__ float scan[ST / 32];
  __shared__ int winner;
  __shared__ int amax;
  rwkv_chain_begin();
  const int row = blockIdx.x, tid = threadIdx.x;
  const T* x = logits + (size_t)row * V;
  unsigned char* seen_row = nullptr;
  if (sa.seen) seen_row = sa.seen + (size_t)(sa.seen_rows ? sa.seen_rows[row] : row) * V;
  const bool penalise = seen_row && sa.penalty > 0.f && sa.penalty != 1.f;
  const float inv_pen = penalise ? 1.f / sa.penalty : 1.f;
  const float scale = sa.greedy ? 1.f : inv_temp;

  // half of the row's values live in registers, half in shared memory (column j of thread tid at [j][tid]: conflict-
  // free): 64 registers per thread are all a 1024-thread CTA can have, and values spilled to local memory made
  // every pass of the searches below a trip through L1/L2
  extern __shared__ float p_sh[];
  float p_reg[SPT_REG];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < SPT; ++j) {
    const int i = tid + j * ST;
    float v = -INFINITY;
    if (i < n_valid) {
      if constexpr (sizeof(T) == 2) v = __bfloat162float(x[i]);
      else v = x[i];
      if (penalise && seen_row[i]) v = v > 0.f ? v * inv_pen : v * sa.penalty;
      v *= scale;
      if (sa.bias) v += sa.bias[i];
      if (!(v == v)) v = -INFINITY;   // NaN logits are never sampled
    }
    PSET(j, v);
    mx = fmaxf(mx, v);
  }
  mx = block_reduce_max(mx, red);
  if (sa.greedy) {   // first index of the maximum; log-probability under the plain softmax of the same logits
    if (tid == 0) amax = 0x7fffffff;
    __syncthreads();
    float zg = 0.f;
#pragma unroll
    for (int j = 0; j < SPT; ++j) {
      if (PGET(j) == mx) atomicMin(&amax, tid + j * ST);
      zg += (PGET(j) == -INFINITY) ? 0.f : __expf(PGET(j) - mx);
    }
    zg = block_reduce_sum(zg, red);
    if (tid == 0) {
      tokens[row] = amax;
      logps[row] = -__logf(zg);
      if (sa.update_seen && seen_row) seen_row[amax] = 1;
    }
    return;
  }
  if (sa.top_k > 0 && sa.top_k < n_valid) {   // radix descent for the key of the k-th largest value
    uint32_t prefix = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = prefix | (1u << bit);
      float cnt = 0.f;
#pragma unroll
      for (int j = 0; j < SPT; ++j) cnt += (order_key(PGET(j)) >= cand) ? 1.f : 0.f;
      cnt = block_reduce_sum(cnt, red);
      if (cnt >= (float)sa.top_k) prefix = cand;
    }
#pragma unroll
    for (int j = 0; j < SPT; ++j)
      if (order_key(PGET(j)) < prefix) PSET(j, -INFINITY);
  }
  float z = 0.f;
#pragma unroll
  for (int j = 0; j < SPT; ++j) {
    PSET(j, (PGET(j) == -INFINITY) ? 0.f : __expf(PGET(j) - mx));
    z += PGET(j);
  }
  z = block_reduce_sum(z, red);
  const float inv_z = 1.f / z;
  float pmax = 0.f;
#pragma unroll
  for (int j = 0; j < SPT; ++j) {
    PSET(j, PGET(j) * (inv_z));
    pmax = fmaxf(pmax, PGET(j));
  }
  if (tid == 0) amax = 0x7fffffff;
  pmax = block_reduce_max(pmax, red);
#pragma unroll
  for (int j = 0; j < SPT; ++j)
    if (PGET(j) == pmax) atomicMin(&amax, tid + j * ST);

  // bisection for the smallest theta with mass({p >= theta}) <= top_p
  float theta = 0.f;
  if (top_p < 1.f) {
    float lo = 0.f, hi = pmax;          // mass(lo) > top_p (or lo == 0), mass(hi) may or may not qualify
    float m_hi = 0.f;
#pragma unroll
    for (int j = 0; j < SPT; ++j) m_hi += (PGET(j) >= hi) ? PGET(j) : 0.f;
    m_hi = block_reduce_sum(m_hi, red);
    if (m_hi > top_p) {
      theta = pmax;                      // even the top token alone exceeds top_p: keep just it
    } else {
      for (int it = 0; it < 30; ++it) {
        const float mid = 0.5f * (lo + hi);
        float m = 0.f;
#pragma unroll
        for (int j = 0; j < SPT; ++j) m += (PGET(j) >= mid) ? PGET(j) : 0.f;
        m = block_reduce_sum(m, red);
        if (m <= top_p) hi = mid; else lo = mid;
      }
      theta = hi;
    }
  }

  float kept = 0.f;
#pragma unroll
  for (int j = 0; j < SPT; ++j) kept += (PGET(j) >= theta && PGET(j) > 0.f) ? PGET(j) : 0.f;
  // block-wide exclusive scan of the per-thread kept mass
  const int lane = tid & 31, warp = tid >> 5;
  float incl = kept;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) scan[warp] = incl;
  if (tid == 0) winner = -1;
  __syncthreads();
  if (warp == 0) {
    float w = scan[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    scan[lane] = w;   // inclusive over warps
  }
  __syncthreads();
  const float total = scan[ST / 32 - 1];
  const float excl = (warp ? scan[warp - 1] : 0.f) + incl - kept;
  const float u = philox_uniform(seed, (unsigned long long)row) * total;
  if (kept > 0.f && u >= excl && u < excl + kept) {
    float acc = excl;
    int pick = -1;
#pragma unroll
    for (int j = 0; j < SPT; ++j) {
      if (PGET(j) >= theta && PGET(j) > 0.f) {
        if (pick < 0) pick = j;          // first kept value as a floor
        if (u >= acc) pick = j;
        acc += PGET(j);
      }
    }
    atomicMax(&winner, tid + pick * ST);
    // the token's log-probability under the renormalised nucleus
    float pv = 0.f;
#pragma unroll
    for (int j = 0; j < SPT; ++j) if (j == pick) pv = PGET(j);
    logps[row] = __logf(pv / total);
  }
  __syncthreads();
  if (tid == 0) {
    if (winner < 0) {   // rounding left u at the very end of the CDF: take the most likely token
      winner = amax;
      logps[row] = __logf(pmax / total);
    }
    tokens[row] = winner;
    if (sa.update_seen && seen_row) seen_row[winner] = 1;
  }
}

#undef PGET
#undef PSET

}  // namespace

// logits: [n, V] fp32 (is_bf16 = 0) or bf16 (1); ids >= n_valid are banned; tokens int64 [n], logps fp32 [n].
// bias: fp32 [V] or null.  seen: uint8 [rows, V] or null, seen_rows: int64 [n] or null (row i of the batch uses
// seen[seen_rows[i]]); penalty <= 0 or == 1 disables the repetition penalty; top_k = 0 disables top-k; greedy = 1
// takes the arg-max (temperature ignored); update_seen = 1 marks the sampled token in the bitmap.
RWKV_EXPORT int rwkv_sample_tokens(const void* logits, int is_bf16, int n, int V, int n_valid, float inv_temp,
                                   float top_p, int top_k, int greedy, const void* bias, void* seen,
                                   const void* seen_rows, float penalty, int update_seen, long long seed,
                                   void* tokens, void* logps, void* stream) {
  if (n <= 0 || V <= 0 || V > ST * SPT || n_valid <= 0 || n_valid > V || top_k < 0) return RWKV_ERR_BAD_SHAPE;
  SampleArgs sa;
  sa.bias = (const float*)bias;
  sa.seen = (unsigned char*)seen;
  sa.seen_rows = (const long long*)seen_rows;
  sa.penalty = penalty;
  sa.top_k = top_k;
  sa.greedy = greedy;
  sa.update_seen = update_seen;
  cudaStream_t st = (cudaStream_t)stream;
  static bool configured = false;
  if (!configured) {
    cudaError_t e1 = cudaFuncSetAttribute(sample_top_p_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SAMPLE_SMEM);
    cudaError_t e2 = cudaFuncSetAttribute(sample_top_p_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, SAMPLE_SMEM);
    if (e1 != cudaSuccess || e2 != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)(e1 != cudaSuccess ? e1 : e2);
    configured = true;
  }
  if (is_bf16)
    rwkv_launch(sample_top_p_kernel<bf16>, dim3(n), dim3(ST), SAMPLE_SMEM, st, (const bf16*)logits, V, n_valid, inv_temp, top_p,
                (unsigned long long)seed, (long long*)tokens, (float*)logps, sa);
  else
    rwkv_launch(sample_top_p_kernel<float>, dim3(n), dim3(ST), SAMPLE_SMEM, st, (const float*)logits, V, n_valid, inv_temp,
                top_p, (unsigned long long)seed, (long long*)tokens, (float*)logps, sa);
  return rwkv_launch_status();
}

// Temperature + top-p only (the call above with every other feature off).
RWKV_EXPORT int rwkv_sample_top_p(const void* logits, int is_bf16, int n, int V, int n_valid, float inv_temp,
                                  float top_p, long long seed, void* tokens, void* logps, void* stream) {
  return rwkv_sample_tokens(logits, is_bf16, n, V, n_valid, inv_temp, top_p, 0, 0, nullptr, nullptr, nullptr, 1.f, 0,
                            seed, tokens, logps, stream);
}

namespace {

// Per-step bookkeeping of a lock-step rollout, for the live paths i = 0 .. n_live-1 (path i is row rows[i] of the
// rollout): store the sampled token (0 once the row has finished), count it, mark the row finished on an end-of-sequence
// id or at the last step, and hand the token to the next decode step's input buffer.
__global__ void __launch_bounds__(256)
rollout_advance_kernel(const long long* __restrict__ tok, const long long* __restrict__ rows,
                       unsigned char* __restrict__ finished, long long* __restrict__ out_ids,
                       long long* __restrict__ lengths, const long long* __restrict__ eos, int n_eos, int step,
                       int max_new, int n_live, long long* __restrict__ next_tok) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_live) return;
  const long long r = rows[i];
  const long long t = tok[i];
  const bool live = finished[r] == 0;
  out_ids[r * max_new + step] = live ? t : 0;
  if (live) {
    lengths[r] += 1;
    bool done = step + 1 >= max_new;
    for (int e = 0; e < n_eos; ++e) done = done || (t == eos[e]);
    if (done) finished[r] = 1;
  }
  if (next_tok) next_tok[i] = t;
}

}  // namespace

// tok, rows: int64 [n_live] (rows distinct); finished: bool [n]; out_ids: int64 [n, max_new]; lengths: int64 [n];
// eos: int64 [n_eos] or null; next_tok: int64 [n_live] or null.
RWKV_EXPORT int rwkv_rollout_advance(const void* tok, const void* rows, void* finished, void* out_ids, void* lengths,
                                     const void* eos, int n_eos, int step, int max_new, int n_live, void* next_tok,
                                     void* stream) {
  if (n_live <= 0) return RWKV_OK;
  if (step < 0 || step >= max_new || n_eos < 0 || (n_eos > 0 && !eos)) return RWKV_ERR_BAD_SHAPE;
  rollout_advance_kernel<<<(n_live + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      (const long long*)tok, (const long long*)rows, (unsigned char*)finished, (long long*)out_ids, (long long*)lengths,
      (const long long*)eos, n_eos, step, max_new, n_live, (long long*)next_tok);
  return rwkv_launch_status();
}
