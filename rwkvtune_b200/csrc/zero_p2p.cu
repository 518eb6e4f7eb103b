// ZeRO-2 step over NVLink peer memory: gradient reduce-scatter fused with the bf16->fp32 cast,
// the 1/(N*accum) scale and the grad-norm partial sum (phase A); global-norm clip, AdamW on the
// owned shard and write-back of the new bf16 parameters into every rank's parameter buffer
// (phase B).  Data moves by plain peer loads/stores issued from inside the kernels on buffers
// that every rank has mapped (symmetric memory); no NCCL call is on this path.
//
// Cross-rank ordering uses flag words in a small symmetric control block:
//   ctrl[r] (int32 [MAX_RANKS])  flags:  slot p of rank r's block is written by rank p
//   ctrl[r] + 64 (float [MAX_RANKS])     slot p holds rank p's squared-norm partial
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

// Phase A.  out[i] = scale * sum_p grad_p[lo + i]  (fp32, fixed rank order); partial[b] = sum of out^2.
__global__ void __launch_bounds__(256)
zero2_reduce_kernel(PeerPtrs grads, int world, size_t lo, size_t n, float scale, float* __restrict__ out,
                    float* __restrict__ partial) {
  __shared__ float red[8];
  float acc = 0.f;
  const size_t n8 = n / 8;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int p = 0; p < world; ++p) {
      const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(grads.p[p]) + lo) + i);
      float f[8];
      unpack8(raw, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) s[e] += f[e];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) { s[e] *= scale; acc += s[e] * s[e]; }
    reinterpret_cast<float4*>(out + i * 8)[0] = make_float4(s[0], s[1], s[2], s[3]);
    reinterpret_cast<float4*>(out + i * 8)[1] = make_float4(s[4], s[5], s[6], s[7]);
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
zero2_publish_norm_kernel(const float* __restrict__ partial, int nblocks, PeerPtrs ctrl, int rank, int world) {
  __shared__ float red[8];
  float acc = 0.f;
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
                        const float* __restrict__ gred, AdamArgs a) {
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

// Phase A: reduced fp32 gradients of [lo, lo + n) into `out`, this rank's squared norm published to all ranks.
// `scratch` needs 1024 floats.  n must be a multiple of 8 and lo a multiple of 8.
RWKV_EXPORT int rwkv_zero2_reduce_scatter(const unsigned long long* grad_ptrs, const unsigned long long* ctrl_ptrs,
                                          int rank, int world, long long lo, long long n, float scale, void* out,
                                          void* scratch, void* stream) {
  PeerPtrs g, c;
  int r = fill_ptrs(&g, grad_ptrs, world);
  if (r) return r;
  r = fill_ptrs(&c, ctrl_ptrs, world);
  if (r) return r;
  if (n <= 0 || (n & 7) || (lo & 7)) return RWKV_ERR_BAD_ALIGNMENT;
  const int blocks = 1024;
  cudaStream_t st = (cudaStream_t)stream;
  zero2_reduce_kernel<<<blocks, 256, 0, st>>>(g, world, (size_t)lo, (size_t)n, scale, (float*)out, (float*)scratch);
  zero2_publish_norm_kernel<<<1, 256, 0, st>>>((const float*)scratch, blocks, c, rank, world);
  return rwkv_launch_status();
}

// Phase B on one segment.  flat0: offset of the segment in the flat parameter space (multiple of 8).
RWKV_EXPORT int rwkv_zero2_adam_broadcast(const unsigned long long* param_ptrs, const unsigned long long* ctrl_ptrs,
                                          int rank, int world, long long flat0, long long seg, void* master, void* m,
                                          void* v, const void* gred, float lr, float beta1, float beta2, float eps,
                                          float weight_decay, int step, float clip, void* stream) {
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
                                                                    (const float*)gred, a);
  return rwkv_launch_status();
}
