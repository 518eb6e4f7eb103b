// Row-wise softmax statistics and gradients over vocabulary logits, in place on the bf16 GEMM output.
//
// The head GEMM (tcgen05) writes a slab of logits [R, V] in bf16; these kernels make ONE statistics sweep and,
// for training, ONE rewrite sweep per row (the second sweep hits L2: a 65 536-entry row is 128 KB), replacing
// the chain  float() -> max -> exp -> sum -> gather -> divide -> scatter -> to(bf16)  that re-reads the slab
// ten times.  The rewritten slab is the gradient w.r.t. the logits and feeds the two backward GEMMs directly.
//
//   rwkv_ce_rows                 cross-entropy (ignore_index, mean over valid targets) + L2Wrap
//                                (rwkvtune/training/lightning_module.py:23-39, :147-156)
//   rwkv_logprob_entropy_rows_*  selective log-softmax and entropy of logits / temperature
//                                (rwkvtune/training/grpo/utils.py:13-152)
#include "common.cuh"

RWKV_DEFINE_DEBUG_EVENTS(loss_rows)

namespace {

constexpr int LNT = 256;

struct RowStats {
  float m;     // max
  float s;     // sum exp(x - m)
  float sx;    // sum exp(x - m) * x
  int am;      // arg max
};

__device__ __forceinline__ void merge(RowStats& a, const RowStats& b) {
  if (b.s == 0.f) return;          // empty partial (a thread that saw no element)
  if (a.s == 0.f) { a = b; return; }
  if (b.m > a.m || (b.m == a.m && b.am < a.am)) {
    const float r = __expf(a.m - b.m);
    a.s = a.s * r + b.s;
    a.sx = a.sx * r + b.sx;
    a.m = b.m;
    a.am = b.am;
  } else {
    const float r = __expf(b.m - a.m);
    a.s += b.s * r;
    a.sx += b.sx * r;
  }
}

// One sweep over a row of V (multiple of 8) bf16 logits scaled by `mul`; result valid in every thread.
template <bool WITH_SX>
__device__ __forceinline__ RowStats row_stats(const bf16* __restrict__ p, int V, float mul, RowStats* red) {
  RowStats st{-INFINITY, 0.f, 0.f, 0};
  for (int i = threadIdx.x; i < V / 8; i += LNT) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(p + (size_t)i * 8), f);
    float lm = -INFINITY;
    int la = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      f[k] *= mul;
      if (f[k] > lm) { lm = f[k]; la = k; }
    }
    if (lm > st.m) {
      const float r = __expf(st.m - lm);
      st.s *= r;
      st.sx *= r;
      st.m = lm;
      st.am = i * 8 + la;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float e = __expf(f[k] - st.m);
      st.s += e;
      if (WITH_SX) st.sx += e * f[k];
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    RowStats other;
    other.m = __shfl_xor_sync(0xffffffffu, st.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, st.s, o);
    other.sx = __shfl_xor_sync(0xffffffffu, st.sx, o);
    other.am = __shfl_xor_sync(0xffffffffu, st.am, o);
    merge(st, other);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = st;
  __syncthreads();
  RowStats tot = red[0];
#pragma unroll
  for (int w = 1; w < LNT / 32; ++w) merge(tot, red[w]);
  return tot;
}

__global__ void __launch_bounds__(LNT)
ce_rows_kernel(bf16* __restrict__ logits, const long long* __restrict__ labels, const float* __restrict__ inv_nvalid,
               float l2_factor, long long ignore_index, float* __restrict__ loss_rows, int write_grad, int V) {
  __shared__ RowStats red[LNT / 32];
  __shared__ float tgt_s;
  const int row = blockIdx.x;
  bf16* p = logits + (size_t)row * V;
  const long long label = labels[row];
  const bool valid = label != ignore_index && RWKV_IN_RANGE(label, V, 11);
  if (threadIdx.x == 0) tgt_s = valid ? __bfloat162float(p[label]) : 0.f;   // before the row is overwritten
  const RowStats st = row_stats<false>(p, V, 1.f, red);
  const float lse = st.m + __logf(st.s);
  if (threadIdx.x == 0) loss_rows[row] = valid ? lse - tgt_s : 0.f;
  if (!write_grad) return;
  const float scale = valid ? *inv_nvalid : 0.f;
  const float l2 = st.m * l2_factor;
  const int lab = valid ? (int)label : -1;
  for (int i = threadIdx.x; i < V / 8; i += LNT) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(p + (size_t)i * 8), f);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int j = i * 8 + k;
      float g = __expf(f[k] - lse) * scale;
      if (j == lab) g -= scale;
      if (j == st.am) g += l2;
      f[k] = g;
    }
    *reinterpret_cast<uint4*>(p + (size_t)i * 8) = pack8(f);
  }
}

__global__ void __launch_bounds__(LNT)
logprob_entropy_fwd_kernel(const bf16* __restrict__ logits, const long long* __restrict__ targets, float inv_t,
                           float* __restrict__ logp, float* __restrict__ ent, int V) {
  __shared__ RowStats red[LNT / 32];
  const int row = blockIdx.x;
  const bf16* p = logits + (size_t)row * V;
  const RowStats st = row_stats<true>(p, V, inv_t, red);
  if (threadIdx.x == 0) {
    const float lse = st.m + __logf(st.s);
    const long long t = targets[row];
    const float zt = RWKV_IN_RANGE(t, V, 12) ? __bfloat162float(p[t]) * inv_t : 0.f;
    logp[row] = zt - lse;
    if (ent) ent[row] = lse - st.sx / st.s;
  }
}

// In place: logits -> d loss / d logits, given per-row d loss / d logp and d loss / d entropy (either may be null).
__global__ void __launch_bounds__(LNT)
logprob_entropy_bwd_kernel(bf16* __restrict__ logits, const long long* __restrict__ targets, float inv_t,
                           const float* __restrict__ g_logp, const float* __restrict__ g_ent, int V) {
  __shared__ RowStats red[LNT / 32];
  const int row = blockIdx.x;
  bf16* p = logits + (size_t)row * V;
  const RowStats st = row_stats<true>(p, V, inv_t, red);
  const float lse = st.m + __logf(st.s);
  const float h = lse - st.sx / st.s;
  const float gl = g_logp ? g_logp[row] : 0.f;
  const float ge = g_ent ? g_ent[row] : 0.f;
  const long long t = targets[row];
  const int lab = (t >= 0 && t < V) ? (int)t : -1;
  for (int i = threadIdx.x; i < V / 8; i += LNT) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(p + (size_t)i * 8), f);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float z = f[k] * inv_t;
      const float pr = __expf(z - lse);
      float g = -pr * (gl + ge * (z - lse + h));
      if (i * 8 + k == lab) g += gl;
      f[k] = g * inv_t;
    }
    *reinterpret_cast<uint4*>(p + (size_t)i * 8) = pack8(f);
  }
}

bool bad_rows(long long R, int V, const void* p) {
  return R <= 0 || R > 0x7fffffffLL || V <= 0 || (V & 7) || ((uintptr_t)p & 15);
}

}  // namespace

// logits: bf16 [R, V] (V % 8 == 0, 16-byte aligned), overwritten with the gradient when write_grad != 0.
// labels: int64 [R]; inv_nvalid: device scalar 1 / (number of non-ignored targets);
// l2_factor: L2Wrap factor (0 disables); loss_rows: fp32 [R] = logsumexp - target logit (0 on ignored rows).
RWKV_EXPORT int rwkv_ce_rows(void* logits, const void* labels, const void* inv_nvalid, float l2_factor,
                             long long ignore_index, void* loss_rows, int write_grad, long long R, int V,
                             void* stream) {
  if (bad_rows(R, V, logits)) return RWKV_ERR_BAD_SHAPE;
  ce_rows_kernel<<<(unsigned)R, LNT, 0, (cudaStream_t)stream>>>((bf16*)logits, (const long long*)labels,
                                                                (const float*)inv_nvalid, l2_factor, ignore_index,
                                                                (float*)loss_rows, write_grad, V);
  return rwkv_launch_status();
}

RWKV_EXPORT int rwkv_logprob_entropy_rows_fwd(const void* logits, const void* targets, float inv_t, void* logp,
                                              void* ent, long long R, int V, void* stream) {
  if (bad_rows(R, V, logits)) return RWKV_ERR_BAD_SHAPE;
  logprob_entropy_fwd_kernel<<<(unsigned)R, LNT, 0, (cudaStream_t)stream>>>((const bf16*)logits, (const long long*)targets,
                                                                            inv_t, (float*)logp, (float*)ent, V);
  return rwkv_launch_status();
}

RWKV_EXPORT int rwkv_logprob_entropy_rows_bwd(void* logits, const void* targets, float inv_t, const void* g_logp,
                                              const void* g_ent, long long R, int V, void* stream) {
  if (bad_rows(R, V, logits)) return RWKV_ERR_BAD_SHAPE;
  logprob_entropy_bwd_kernel<<<(unsigned)R, LNT, 0, (cudaStream_t)stream>>>((bf16*)logits, (const long long*)targets,
                                                                            inv_t, (const float*)g_logp,
                                                                            (const float*)g_ent, V);
  return rwkv_launch_status();
}
