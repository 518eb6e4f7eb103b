// ZeRO-2 step over NVLink peer memory: gradient reduce-scatter fused with the bf16->fp32 cast,
// the 1/(N*accum) scale and the grad-norm partial sum (phase A); global-norm clip, AdamW on the
// owned shard and write-back of the new bf16 parameters into every rank's parameter buffer
// (phase B).  Data moves by plain peer loads/stores issued from inside the kernels on buffers
// that every rank has mapped (symmetric memory); no NCCL call is on this path.
//
// Cross-rank ordering uses flag words in a small symmetric control block (int32 words):
//   ctrl[r][0 .. 16)             barrier flags: slot p of rank r's block is written by rank p
//   ctrl[r][64 .. 80)  (float)   slot p holds rank p's squared-norm partial
//   ctrl[r][128 + 16 b + p]      "bucket b of rank p's gradients is complete" (epoch value), b < MAX_BUCKETS
// Gradient buckets make the reduce-scatter overlap with backward: as soon as the last gradient of a bucket has been
// written, the rank raises the bucket's flag in every peer's block (rwkv_p2p_signal, on the compute stream) and the
// owner of that range reduces it on a side stream after a bounded wait for all ranks' flags (rwkv_p2p_wait +
// rwkv_zero2_reduce_bucket), while backward continues with the next layers.
// Every data kernel reads the status word first and returns without writing when a wait has expired earlier in
// the step, so a timed-out step changes neither gradients-in-flight nor parameters ("poisoned step").
// A barrier stores a monotonically increasing epoch into slot `rank` of every peer's block with
// release semantics at system scope and then waits, with a globaltimer deadline, until all slots
// of its own block have reached the epoch.  A wait that expires records a code in `status` and
// the kernel returns; nothing spins forever.
//
// Replaces DeepSpeed's stage-2 reduce-scatter / FusedAdam / all-gather sequence that the
// reference selects with strategy="deepspeed_stage_2" (rwkvtune/training/sft_trainer.py:392-412).
#include "common.cuh"

namespace {

constexpr int MAX_RANKS = 16;
constexpr int NORM_OFFSET_WORDS = 64;   // float slots start 256 bytes into the control block

struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// One block; thread t talks to rank t.
__global__ void p2p_barrier_kernel(PeerPtrs ctrl, int rank, int world, int epoch, int* status,
                                   unsigned long long timeout_ns) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  st_release_sys(reinterpret_cast<int*>(ctrl.p[t]) + rank, epoch);
  const int* mine = reinterpret_cast<const int*>(ctrl.p[rank]) + t;
  const unsigned long long deadline = globaltimer_ns() + timeout_ns;
  while (ld_acquire_sys(mine) < epoch) {
    if (globaltimer_ns() > deadline) {
      atomicCAS(status, 0, RWKV_ERR_WAIT_TIMEOUT * 100 + t);
      return;
    }
    __nanosleep(64);
  }
}

// One block; thread t raises flag word `word + rank` in rank t's control block.
__global__ void p2p_signal_kernel(PeerPtrs ctrl, int rank, int world, int word, int value) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  st_release_sys(reinterpret_cast<int*>(ctrl.p[t]) + word + rank, value);
}

// One block; thread t waits (bounded) until flag word `word + t` of this rank's block has reached `value`.
__global__ void p2p_wait_kernel(PeerPtrs ctrl, int rank, int world, int word, int value, int* status,
                                unsigned long long timeout_ns) {
  const int t = threadIdx.x;
  if (t >= world) return;
  const int* mine = reinterpret_cast<const int*>(ctrl.p[rank]) + word + t;
  const unsigned long long deadline = globaltimer_ns() + timeout_ns;
  while (ld_acquire_sys(mine) < value) {
    if (globaltimer_ns() > deadline) {
      atomicCAS(status, 0, RWKV_ERR_WAIT_TIMEOUT * 100 + t);
      return;
    }
    __nanosleep(64);
  }
}

// Phase A.  out[i] (+)= scale * sum_p grad_p[lo + i]  (fp32, fixed rank order); partial[b] = sum of out^2.
// With `accumulate` the reduced micro-batch gradient is added to what `out` holds (fp32 accumulation of
// micro-batches on the owner) and the norm partial is taken of the accumulated value.
// WMAX: compile-time bound on the rank count (2, 4, 8, 16).  A peer load takes microseconds, so throughput is bytes
// in flight over latency: every thread issues the loads of all ranks for ITER consecutive vectors before it adds.
template <int WMAX>
__global__ void __launch_bounds__(256)
zero2_reduce_kernel(PeerPtrs grads, int world, size_t lo, size_t n, float scale, float* __restrict__ out,
                    float* __restrict__ partial, int accumulate, const int* __restrict__ status) {
  constexpr int ITER = WMAX >= 8 ? 1 : (WMAX == 4 ? 2 : 4);
  __shared__ float red[8];
  if (status && *reinterpret_cast<const volatile int*>(status)) return;   // poisoned step: touch nothing
  float acc = 0.f;
  const size_t n8 = n / 8;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i0 = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i0 < n8; i0 += stride * ITER) {
    uint4 raw[ITER][WMAX];
#pragma unroll
    for (int u = 0; u < ITER; ++u) {
      const size_t i = i0 + u * stride;
#pragma unroll
      for (int p = 0; p < WMAX; ++p)
        if (p < world && i < n8)
          raw[u][p] = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(grads.p[p]) + lo) + i);
    }
#pragma unroll
    for (int u = 0; u < ITER; ++u) {
      const size_t i = i0 + u * stride;
      if (i >= n8) break;
      float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int p = 0; p < WMAX; ++p) {
        if (p < world) {
          float f[8];
          unpack8(raw[u][p], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) s[e] += f[e];
        }
      }
      float4* o4 = reinterpret_cast<float4*>(out + i * 8);
      if (accumulate) {
        const float4 a0 = o4[0], a1 = o4[1];
        s[0] = s[0] * scale + a0.x; s[1] = s[1] * scale + a0.y; s[2] = s[2] * scale + a0.z; s[3] = s[3] * scale + a0.w;
        s[4] = s[4] * scale + a1.x; s[5] = s[5] * scale + a1.y; s[6] = s[6] * scale + a1.z; s[7] = s[7] * scale + a1.w;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) s[e] *= scale;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) acc += s[e] * s[e];
      o4[0] = make_float4(s[0], s[1], s[2], s[3]);
      o4[1] = make_float4(s[4], s[5], s[6], s[7]);
    }
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    partial[blockIdx.x] = t;
  }
}

// Sums the block partials and publishes this rank's squared-norm partial into slot `rank` of every
// rank's control block.
__global__ void __launch_bounds__(256)
zero2_publish_norm_kernel(const float* __restrict__ partial, int nblocks, PeerPtrs ctrl, int rank, int world,
                          const float* __restrict__ extra) {
  __shared__ float red[8];
  float acc = (extra && threadIdx.x == 0) ? extra[0] : 0.f;   // squared norm of gradients reduced elsewhere
  for (int i = threadIdx.x; i < nblocks; i += 256) acc += partial[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    for (int p = 0; p < world; ++p)
      reinterpret_cast<volatile float*>(reinterpret_cast<int*>(ctrl.p[p]) + NORM_OFFSET_WORDS)[rank] = t;
    __threadfence_system();
  }
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, clip;
};

// Phase B on one (group, shard) segment: `seg` elements starting at flat offset `flat0`; master/m/v/gred
// are the shard-local arrays already offset to the segment.  New bf16 parameters go to every rank.
__global__ void __launch_bounds__(256)
zero2_adam_bcast_kernel(PeerPtrs params, int world, const float* __restrict__ my_norms, size_t flat0, size_t seg,
                        float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                        const float* __restrict__ gred, AdamArgs a, const int* __restrict__ status) {
  if (status && *reinterpret_cast<const volatile int*>(status)) return;   // poisoned step: parameters stay as they are
  float coef = 1.f;
  if (a.clip > 0.f) {
    float nsq = 0.f;
    for (int p = 0; p < world; ++p) nsq += my_norms[p];
    coef = fminf(1.f, a.clip / (sqrtf(nsq) + 1e-6f));
  }
  const float step_size = a.lr / a.bc1;
  const float inv_bc2_sqrt = rsqrtf(a.bc2);
  const float decay = 1.f - a.lr * a.weight_decay;
  const size_t n8 = seg / 8;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float g[8], pm[8], mm[8], vv[8], o[8];
    const float4* g4 = reinterpret_cast<const float4*>(gred + i * 8);
    float4* p4 = reinterpret_cast<float4*>(master + i * 8);
    float4* m4 = reinterpret_cast<float4*>(m + i * 8);
    float4* v4 = reinterpret_cast<float4*>(v + i * 8);
    *reinterpret_cast<float4*>(g) = g4[0]; *reinterpret_cast<float4*>(g + 4) = g4[1];
    *reinterpret_cast<float4*>(pm) = p4[0]; *reinterpret_cast<float4*>(pm + 4) = p4[1];
    *reinterpret_cast<float4*>(mm) = m4[0]; *reinterpret_cast<float4*>(mm + 4) = m4[1];
    *reinterpret_cast<float4*>(vv) = v4[0]; *reinterpret_cast<float4*>(vv + 4) = v4[1];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float ge = g[e] * coef;
      mm[e] = a.beta1 * mm[e] + (1.f - a.beta1) * ge;
      vv[e] = a.beta2 * vv[e] + (1.f - a.beta2) * ge * ge;
      const float denom = sqrtf(vv[e]) * inv_bc2_sqrt + a.eps;
      pm[e] = pm[e] * decay - step_size * mm[e] / denom;
      o[e] = pm[e];
    }
    p4[0] = *reinterpret_cast<float4*>(pm); p4[1] = *reinterpret_cast<float4*>(pm + 4);
    m4[0] = *reinterpret_cast<float4*>(mm); m4[1] = *reinterpret_cast<float4*>(mm + 4);
    v4[0] = *reinterpret_cast<float4*>(vv); v4[1] = *reinterpret_cast<float4*>(vv + 4);
    const uint4 packed = pack8(o);
    for (int p = 0; p < world; ++p)
      reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(params.p[p]) + flat0)[i] = packed;
  }
}

int fill_ptrs(PeerPtrs* out, const unsigned long long* ptrs, int world) {
  if (world <= 0 || world > MAX_RANKS) return RWKV_ERR_BAD_SHAPE;
  for (int i = 0; i < MAX_RANKS; ++i) out->p[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return RWKV_OK;
}

}  // namespace

// ctrl_ptrs: host array of `world` device addresses (each rank's control block as mapped in this process)
RWKV_EXPORT int rwkv_p2p_barrier(const unsigned long long* ctrl_ptrs, int rank, int world, int epoch, void* status,
                                 long long timeout_ns, void* stream) {
  PeerPtrs c;
  int r = fill_ptrs(&c, ctrl_ptrs, world);
  if (r) return r;
  if (rank < 0 || rank >= world || timeout_ns <= 0) return RWKV_ERR_BAD_SHAPE;
  p2p_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(c, rank, world, epoch, (int*)status,
                                                         (unsigned long long)timeout_ns);
  return rwkv_launch_status();
}

// Raise flag word `word + rank` (0 <= word, word + world <= control block size) in every rank's control block.
RWKV_EXPORT int rwkv_p2p_signal(const unsigned long long* ctrl_ptrs, int rank, int world, int word, int value,
                                void* stream) {
  PeerPtrs c;
  int r = fill_ptrs(&c, ctrl_ptrs, world);
  if (r) return r;
  if (rank < 0 || rank >= world || word < 0) return RWKV_ERR_BAD_SHAPE;
  p2p_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(c, rank, world, word, value);
  return rwkv_launch_status();
}

// Wait until flag words `word .. word + world` of this rank's block have all reached `value`; on expiry
// `status` receives 500 + the rank that was missing.
RWKV_EXPORT int rwkv_p2p_wait(const unsigned long long* ctrl_ptrs, int rank, int world, int word, int value,
                              void* status, long long timeout_ns, void* stream) {
  PeerPtrs c;
  int r = fill_ptrs(&c, ctrl_ptrs, world);
  if (r) return r;
  if (rank < 0 || rank >= world || word < 0 || timeout_ns <= 0 || !status) return RWKV_ERR_BAD_SHAPE;
  p2p_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(c, rank, world, word, value, (int*)status,
                                                      (unsigned long long)timeout_ns);
  return rwkv_launch_status();
}

// Phase A on one range: out[0 .. n) (+)= scale * sum over ranks of grads[lo .. lo + n); `partial` receives `blocks`
// floats (block sums of out^2).  n and lo multiples of 8; 1 <= blocks <= 1024.  `status` (may be null): the step's
// status word; when it is non-zero the kernel writes nothing.
RWKV_EXPORT int rwkv_zero2_reduce_bucket(const unsigned long long* grad_ptrs, int world, long long lo, long long n,
                                         float scale, void* out, void* partial, int blocks, int accumulate,
                                         const void* status, void* stream) {
  PeerPtrs g;
  int r = fill_ptrs(&g, grad_ptrs, world);
  if (r) return r;
  if (n <= 0 || (n & 7) || (lo & 7)) return RWKV_ERR_BAD_ALIGNMENT;
  if (blocks <= 0 || blocks > 1024) return RWKV_ERR_BAD_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
#define RWKV_REDUCE(WM)                                                                                              \
  zero2_reduce_kernel<WM><<<blocks, 256, 0, st>>>(g, world, (size_t)lo, (size_t)n, scale, (float*)out, (float*)partial, \
                                                  accumulate, (const int*)status)
  if (world <= 2) RWKV_REDUCE(2);
  else if (world <= 4) RWKV_REDUCE(4);
  else if (world <= 8) RWKV_REDUCE(8);
  else RWKV_REDUCE(16);
#undef RWKV_REDUCE
  return rwkv_launch_status();
}

// Sum `n_partials` block partials (+ `extra[0]` when given) and publish the result as this rank's squared-norm
// share in every rank's control block.
RWKV_EXPORT int rwkv_zero2_publish_norm(const void* partial, int n_partials, const void* extra,
                                        const unsigned long long* ctrl_ptrs, int rank, int world, void* stream) {
  PeerPtrs c;
  int r = fill_ptrs(&c, ctrl_ptrs, world);
  if (r) return r;
  if (n_partials < 0 || rank < 0 || rank >= world) return RWKV_ERR_BAD_SHAPE;
  zero2_publish_norm_kernel<<<1, 256, 0, (cudaStream_t)stream>>>((const float*)partial, n_partials, c, rank, world,
                                                                 (const float*)extra);
  return rwkv_launch_status();
}

// Phase A in one call (whole shard, no buckets): reduced fp32 gradients of [lo, lo + n) into `out`, this rank's
// squared norm published to all ranks.  `scratch` needs 1024 floats.  n and lo must be multiples of 8.
RWKV_EXPORT int rwkv_zero2_reduce_scatter(const unsigned long long* grad_ptrs, const unsigned long long* ctrl_ptrs,
                                          int rank, int world, long long lo, long long n, float scale, void* out,
                                          void* scratch, const void* status, void* stream) {
  int r = rwkv_zero2_reduce_bucket(grad_ptrs, world, lo, n, scale, out, scratch, 1024, 0, status, stream);
  if (r) return r;
  return rwkv_zero2_publish_norm(scratch, 1024, nullptr, ctrl_ptrs, rank, world, stream);
}

// Phase B on one segment.  flat0: offset of the segment in the flat parameter space (multiple of 8).
RWKV_EXPORT int rwkv_zero2_adam_broadcast(const unsigned long long* param_ptrs, const unsigned long long* ctrl_ptrs,
                                          int rank, int world, long long flat0, long long seg, void* master, void* m,
                                          void* v, const void* gred, float lr, float beta1, float beta2, float eps,
                                          float weight_decay, int step, float clip, const void* status, void* stream) {
  PeerPtrs p;
  int r = fill_ptrs(&p, param_ptrs, world);
  if (r) return r;
  if (seg <= 0 || (seg & 7) || (flat0 & 7) || step <= 0 || world > MAX_RANKS) return RWKV_ERR_BAD_ALIGNMENT;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  a.clip = clip;
  const float* norms = reinterpret_cast<const float*>(reinterpret_cast<const int*>(ctrl_ptrs[rank]) + NORM_OFFSET_WORDS);
  const long long n8 = seg / 8;
  const int blocks = (int)((n8 + 255) / 256 < 148 * 8 ? (n8 + 255) / 256 : 148 * 8);
  zero2_adam_bcast_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(p, world, norms, (size_t)flat0, (size_t)seg,
                                                                    (float*)master, (float*)m, (float*)v,
                                                                    (const float*)gred, a, (const int*)status);
  return rwkv_launch_status();
}

// ---------------------------------------------------------------------------------------------------------------
// ZeRO-3 helpers for weights stored as K-panels (rank p owns columns [p*Kp, (p+1)*Kp) of a [N, K] matrix as a
// contiguous [N, Kp] array).
namespace {

// Gather: staged[n][p*Kp + c] = panel_p[n][c] for every rank p, starting with the local panel.  Plain peer loads,
// eight 16-byte loads in flight per thread (a peer load takes microseconds: throughput = bytes in flight / latency).
__global__ void __launch_bounds__(256)
ag_gather_kernel(PeerPtrs panels, int rank, int world, int N, int K, int Kp, bf16* __restrict__ staged) {
  constexpr int UNROLL = 8;
  const int vec_per_row = Kp / 8;
  const long long total = (long long)N * vec_per_row;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int s = 0; s < world; ++s) {
    const int p = (rank + s) % world;
    const uint4* src = reinterpret_cast<const uint4*>(panels.p[p]);
    bf16* dst = staged + (long long)p * Kp;
    for (long long v0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; v0 < total; v0 += stride * UNROLL) {
      uint4 val[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long v = v0 + u * stride;
        if (v < total) val[u] = __ldcg(src + v);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long v = v0 + u * stride;
        if (v < total) {
          const long long row = v / vec_per_row;
          const int c = (int)(v - row * vec_per_row);
          *reinterpret_cast<uint4*>(dst + row * K + c * 8) = val[u];
        }
      }
    }
  }
}

// Reduce-scatter of a full [N, K] weight gradient held by every rank: this rank sums columns [col0, col0 + Kp) of all
// ranks' matrices (fixed rank order, fp32) into its panel gradient out[N][Kp] (+= when `accumulate`).
__global__ void __launch_bounds__(256)
zero3_reduce_panel_kernel(PeerPtrs dw, int world, int N, int K, int Kp, int col0, float scale, float* __restrict__ out,
                          float* __restrict__ partial, int accumulate, const int* __restrict__ status) {
  __shared__ float red[8];
  if (status && *reinterpret_cast<const volatile int*>(status)) return;
  float acc = 0.f;
  const int vec_per_row = Kp / 8;
  const long long total = (long long)N * vec_per_row;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (long long)gridDim.x * blockDim.x) {
    const long long row = v / vec_per_row;
    const int c = (int)(v - row * vec_per_row);
    const long long src_off = row * K + col0 + c * 8;
    uint4 raw[MAX_RANKS];
#pragma unroll
    for (int p = 0; p < MAX_RANKS; ++p)
      if (p < world) raw[p] = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(dw.p[p]) + src_off));
    float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int p = 0; p < MAX_RANKS; ++p) {
      if (p < world) {
        float f[8];
        unpack8(raw[p], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) s[e] += f[e];
      }
    }
    float4* o4 = reinterpret_cast<float4*>(out + v * 8);
    if (accumulate) {
      const float4 a0 = o4[0], a1 = o4[1];
      s[0] = s[0] * scale + a0.x; s[1] = s[1] * scale + a0.y; s[2] = s[2] * scale + a0.z; s[3] = s[3] * scale + a0.w;
      s[4] = s[4] * scale + a1.x; s[5] = s[5] * scale + a1.y; s[6] = s[6] * scale + a1.z; s[7] = s[7] * scale + a1.w;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) s[e] *= scale;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += s[e] * s[e];
    o4[0] = make_float4(s[0], s[1], s[2], s[3]);
    o4[1] = make_float4(s[4], s[5], s[6], s[7]);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0 && partial) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    partial[blockIdx.x] = t;
  }
}

}  // namespace

// staged ([N, K] bf16, local) <- the `world` K-panels ([N, K/world] each) at panel_ptrs (peer-mapped addresses).
RWKV_EXPORT int rwkv_ag_gather(const unsigned long long* panel_ptrs, int rank, int world, int N, int K, void* staged,
                               int blocks, void* stream) {
  PeerPtrs p;
  int r = fill_ptrs(&p, panel_ptrs, world);
  if (r) return r;
  if (N <= 0 || K <= 0 || K % world || (K / world) % 8 || rank < 0 || rank >= world || blocks <= 0) return RWKV_ERR_BAD_SHAPE;
  if ((uintptr_t)staged & 15) return RWKV_ERR_BAD_ALIGNMENT;
  ag_gather_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(p, rank, world, N, K, K / world, (bf16*)staged);
  return rwkv_launch_status();
}

// out[N][Kp] (+)= scale * sum over ranks of dw_r[:, rank*Kp : (rank+1)*Kp]; dw_ptrs: every rank's [N, K] bf16 gradient.
// `partial` (may be null) receives `blocks` block sums of out^2.
RWKV_EXPORT int rwkv_zero3_reduce_panel(const unsigned long long* dw_ptrs, int rank, int world, int N, int K,
                                        float scale, void* out, void* partial, int blocks, int accumulate,
                                        const void* status, void* stream) {
  PeerPtrs p;
  int r = fill_ptrs(&p, dw_ptrs, world);
  if (r) return r;
  if (N <= 0 || K <= 0 || K % world || (K / world) % 8 || rank < 0 || rank >= world || blocks <= 0 || blocks > 1024)
    return RWKV_ERR_BAD_SHAPE;
  const int Kp = K / world;
  zero3_reduce_panel_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(p, world, N, K, Kp, rank * Kp, scale, (float*)out,
                                                                      (float*)partial, accumulate, (const int*)status);
  return rwkv_launch_status();
}
