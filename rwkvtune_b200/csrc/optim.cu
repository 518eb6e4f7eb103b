// Optimiser-side kernels on flat buffers: gradient sum of squares (two-stage, fixed
// summation order) and AdamW with decoupled weight decay on an fp32 master copy that also
// writes the bf16 compute copy.  The clip coefficient is derived on the device from the
// squared norm, so a training step needs no host synchronisation between backward and
// the parameter update.  Stands in for DeepSpeed's FusedAdam plus Lightning's
// gradient_clip_val (reference: rwkvtune/training/lightning_module.py:278-288,
// rwkvtune/training/sft_trainer.py:448).
#include "common.cuh"

namespace {

constexpr int SUMSQ_BLOCKS = 1024;

__global__ void __launch_bounds__(256)
sumsq_stage1(const bf16* __restrict__ g, size_t n, float scale, float* __restrict__ partial) {
  __shared__ float red[8];
  float acc = 0.f;
  const size_t n8 = n / 8;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(g + i * 8), f);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += f[e] * f[e];
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {   // ragged tail
    const float x = __bfloat162float(g[n8 * 8 + threadIdx.x]);
    acc += x * x;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) s += red[i];
    partial[blockIdx.x] = s * scale * scale;
  }
}

// out[0] (+)= sum(partial)
__global__ void __launch_bounds__(256)
sumsq_stage2(const float* __restrict__ partial, int n, float* __restrict__ out, int accumulate) {
  __shared__ float red[8];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) acc += partial[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) s += red[i];
    out[0] = accumulate ? out[0] + s : s;
  }
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale, clip;
};

template <typename GradT>
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
             const GradT* __restrict__ grad, bf16* __restrict__ param_out, size_t n,
             const float* __restrict__ norm_sq, AdamArgs a) {
  float coef = a.grad_scale;
  if (norm_sq && a.clip > 0.f) {
    const float nrm = sqrtf(norm_sq[0]);
    coef *= fminf(1.f, a.clip / (nrm + 1e-6f));
  }
  const float step_size = a.lr / a.bc1;
  const float inv_bc2_sqrt = rsqrtf(a.bc2);
  const float decay = 1.f - a.lr * a.weight_decay;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float g;
    if constexpr (sizeof(GradT) == 2) g = __bfloat162float(grad[i]) * coef;
    else g = grad[i] * coef;
    const float mi = a.beta1 * m[i] + (1.f - a.beta1) * g;
    const float vi = a.beta2 * v[i] + (1.f - a.beta2) * g * g;
    const float denom = sqrtf(vi) * inv_bc2_sqrt + a.eps;
    const float p = master[i] * decay - step_size * mi / denom;
    m[i] = mi;
    v[i] = vi;
    master[i] = p;
    if (param_out) param_out[i] = __float2bfloat16_rn(p);
  }
}

}  // namespace

// out[0] = (accumulate ? out[0] : 0) + sum((g * scale)^2).  `scratch` holds >= 1024 floats.
RWKV_EXPORT int rwkv_grad_sumsq_bf16(const void* g, long long n, float scale, void* scratch, void* out,
                                     int accumulate, void* stream) {
  if (n < 0) return RWKV_ERR_BAD_SHAPE;
  if (((uintptr_t)g) & 15) return RWKV_ERR_BAD_ALIGNMENT;
  cudaStream_t st = (cudaStream_t)stream;
  sumsq_stage1<<<SUMSQ_BLOCKS, 256, 0, st>>>((const bf16*)g, (size_t)n, scale, (float*)scratch);
  sumsq_stage2<<<1, 256, 0, st>>>((const float*)scratch, SUMSQ_BLOCKS, (float*)out, accumulate);
  return rwkv_launch_status();
}

// grad_is_fp32: 0 = bf16 gradients, 1 = fp32 gradients.  norm_sq may be null (no clipping).
RWKV_EXPORT int rwkv_adamw_step(void* master, void* m, void* v, const void* grad, int grad_is_fp32, void* param_out,
                                long long n, const void* norm_sq, float lr, float beta1, float beta2, float eps,
                                float weight_decay, int step, float grad_scale, float clip, void* stream) {
  if (n <= 0 || step <= 0) return RWKV_ERR_BAD_SHAPE;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  a.grad_scale = grad_scale; a.clip = clip;
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  cudaStream_t st = (cudaStream_t)stream;
  if (grad_is_fp32)
    adamw_kernel<float><<<blocks, 256, 0, st>>>((float*)master, (float*)m, (float*)v, (const float*)grad,
                                                (bf16*)param_out, (size_t)n, (const float*)norm_sq, a);
  else
    adamw_kernel<bf16><<<blocks, 256, 0, st>>>((float*)master, (float*)m, (float*)v, (const bf16*)grad,
                                               (bf16*)param_out, (size_t)n, (const float*)norm_sq, a);
  return rwkv_launch_status();
}

namespace {

// out[w] = sum_r partials[r][w]: the per-CTA partial sums of a parameter gradient ([rows, W] fp32, rows = CTAs of the
// backward kernel, W = a few thousand) into the gradient.  A block owns 32 columns: 8 row groups of 32 lanes read
// 128 contiguous bytes each and stride over the rows, then the 8 groups meet in shared memory (fixed order).
template <typename OutT>
__global__ void __launch_bounds__(256)
colsum_kernel(const float* __restrict__ partials, int rows, long long W, OutT* __restrict__ out) {
  __shared__ float part[8][32];
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const long long col = (long long)blockIdx.x * 32 + lane;
  float acc = 0.f;
  if (col < W)
    for (int r = grp; r < rows; r += 8) acc += partials[(long long)r * W + col];
  part[grp][lane] = acc;
  __syncthreads();
  if (grp == 0 && col < W) {
    float s = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) s += part[g][lane];
    if constexpr (sizeof(OutT) == 2) out[col] = __float2bfloat16_rn(s);
    else out[col] = s;
  }
}

}  // namespace

// partials: fp32 [rows, W] contiguous; out: [W], fp32 (out_bf16 = 0) or bf16 (1: the sum is rounded once, at the end).
RWKV_EXPORT int rwkv_colsum_f32(const void* partials, int rows, long long W, void* out, int out_bf16, void* stream) {
  if (rows <= 0 || W <= 0) return RWKV_ERR_BAD_SHAPE;
  const unsigned blocks = (unsigned)((W + 31) / 32);
  if (out_bf16)
    colsum_kernel<bf16><<<blocks, 256, 0, (cudaStream_t)stream>>>((const float*)partials, rows, W, (bf16*)out);
  else
    colsum_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((const float*)partials, rows, W, (float*)out);
  return rwkv_launch_status();
}
