// One decoding step of the recurrent core of a time-mix block, in one kernel per layer:
//
//   key / decay / value preparation   (w = -softplus(-(w0 + w_lin)) - 0.5, a = sigmoid(a0 + a_lin), kk = normalize(k * k_k),
//                                      k' = k (1 + (a - 1) k_a), v' = v + (v_first - v) sigmoid(v0 + v_lin), -kk, kk a)
//   WKV7 state update and read-out    (S = S diag(d) + (S a~) b~^T + v' k'^T with d = exp(-exp(w)),  y = S r)
//   GroupNorm + bonus + gate          (z = (GN(y) + (sum_head r k' r_k) v') g)
//
// for one token per sequence.  During training these are three kernels over long sequences (timemix_fused.cu,
// wkv7.cu / wkv7_tc.cu); at one token per sequence each of them is a launch plus a memory round trip, and the
// general WKV7 kernel carries 58 KB of chunk staging per CTA that limits it to three CTAs per SM.  Here a CTA
// owns one (sequence, head): 64 threads prepare one channel of the head each while all 128 threads are already
// loading their 8 x 4 slice of the 64 x 64 fp32 state; 2.5 KB of shared memory and 72 registers (seven CTAs per SM), so that the
// 32 KB of state traffic per CTA is spread over many resident CTAs.  The new state goes to a second tensor or back
// into the first (in place), which may be a [B, H, 64, 64] tensor or a slot-indexed pool (continuous batching).
//
// Every intermediate that the three-kernel path stores as bf16 (w, k', v', -kk, kk a, y) is rounded to bf16
// here as well and the reductions are taken in the same order, so the fused step reproduces that path to the last
// bit, except for the occasional element where the compiler contracts a multiply-add differently in the two places.
//
// Reference statement: rwkvtune/models/rwkv7/model.py:146-200 at T = 1.
#include "common.cuh"
#include "elementwise.cuh"

namespace {

constexpr int DC_N = 64;         // head size
constexpr int DC_THREADS = 128;

enum { DQ = 0, DD, DK_, DV, DA, DB, DC_NIN };

struct DecodeCoreArgs {
  const bf16 *r, *k, *v, *wlin, *alin, *vlin, *vfirst, *g;                 // [B, C]; vlin / vfirst null in the first block
  const float *w0, *a0, *v0, *k_k, *k_a, *r_k, *gn_w, *gn_b;             // [C]
  const float* state;          // [B or n_slots, H, 64, 64] fp32
  float* state_out;            // same shape; may be `state` itself (update in place)
  const long long* slots;      // [B] state row of each sequence, or null (row = sequence index)
  bf16* z;                     // [B, C]
  int H;
  float eps;
};

__device__ __forceinline__ float dc_softplus(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

__device__ __forceinline__ void dc_ld4_as2(const float* p, float2& lo, float2& hi) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  lo = make_float2(x.x, x.y);
  hi = make_float2(x.z, x.w);
}

// v[0..7] and v[8..15] are two sets of per-row partial sums over this lane's 4 columns; the 16 lanes that share the
// rows are summed with 15 shuffles.  On return v[0] holds, for lanes with (lane & 8) == 0, the total of the first set
// for row (lane & 7); for the other lanes the total of the second set for that row.  (Same order of additions as the
// general forward kernel.)
__device__ __forceinline__ void dc_butterfly(float (&v)[16], int lane) {
  {
    const bool hi = lane & 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float send = hi ? v[i] : v[i + 8];
      const float keep = hi ? v[i + 8] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
  }
  {
    const bool hi = lane & 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float send = hi ? v[i] : v[i + 4];
      const float keep = hi ? v[i + 4] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
  }
  {
    const bool hi = lane & 2;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float send = hi ? v[i] : v[i + 2];
      const float keep = hi ? v[i + 2] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
    }
  }
  {
    const bool hi = lane & 1;
    const float send = hi ? v[0] : v[1];
    const float keep = hi ? v[1] : v[0];
    v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
  }
}

// Sum over the head's 64 channels of the values in `vals`, in the order the row kernels use: eight consecutive
// channels are added sequentially (a thread's eight channels there), the eight partial sums with an xor butterfly.
// Called by the 64 preparation threads (warps 0 and 1); `slot` receives the total.
__device__ __forceinline__ float dc_head_total(float mine, float* vals, float* slot, int tid) {
  vals[tid] = mine;
  asm volatile("bar.sync 1, 64;" ::: "memory");
  if (tid < 32) {   // the whole first warp takes part in the shuffles; lanes 0..7 carry the eight partial sums
    float g = 0.f;
    if (tid < 8) {
#pragma unroll
      for (int e = 0; e < 8; ++e) g += vals[tid * 8 + e];
    }
    g = head_sum(g);
    if (tid == 0) *slot = g;
  }
  asm volatile("bar.sync 1, 64;" ::: "memory");
  return *slot;
}

__global__ void __launch_bounds__(DC_THREADS, 7)
wkv7_decode_core_kernel(const DecodeCoreArgs A) {
  __shared__ __align__(16) float in[DC_NIN][DC_N];   // r, decay, k', v', -kk, kk a of this head
  __shared__ __align__(16) float sabuf[DC_N];
  __shared__ __align__(16) float ybuf[DC_N];
  __shared__ float scratch[2][DC_N];
  __shared__ float totals[4];
  rwkv_chain_trigger();
  const int h = blockIdx.x, bb = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int C = A.H * DC_N;
  const bool prep = tid < DC_N;                       // threads 0..63: one channel of the head each
  const int ch = h * DC_N + (prep ? tid : 0);

  // parameters do not depend on the predecessor kernel
  float w0 = 0.f, a0 = 0.f, v0 = 0.f, kk_p = 0.f, ka_p = 0.f, gw = 0.f, gb = 0.f, rk = 0.f;
  if (prep) {
    w0 = A.w0[ch];
    a0 = A.a0[ch];
    if (A.vfirst) v0 = A.v0[ch];
    kk_p = A.k_k[ch];
    ka_p = A.k_a[ch];
    gw = A.gn_w[ch];     // needed last, requested first: no memory round trip left in the GroupNorm phase
    gb = A.gn_b[ch];
    rk = A.r_k[ch];
  }
  rwkv_chain_wait();

  // every thread: its 8 rows x 4 columns of the state (requested first, so that it is in flight during the preparation)
  const size_t srow = A.slots ? (size_t)A.slots[bb] : (size_t)bb;
  const float* sp = A.state + (srow * A.H + h) * DC_N * DC_N;
  float* sp_out = A.state_out + (srow * A.H + h) * DC_N * DC_N;
  const int rg = lane >> 4, cg = lane & 15;
  const int r0 = warp * 16 + rg * 8, c0 = cg * 4;
  float2 S2[8][2];
#pragma unroll
  for (int i = 0; i < 8; ++i) dc_ld4_as2(sp + (r0 + i) * DC_N + c0, S2[i][0], S2[i][1]);

  float gate = 0.f;
  if (prep) {
    const size_t off = (size_t)bb * C + ch;
    const float rf = __bfloat162float(A.r[off]), kf = __bfloat162float(A.k[off]);
    float vf = __bfloat162float(A.v[off]);
    const float wl = __bfloat162float(A.wlin[off]), al = __bfloat162float(A.alin[off]);
    gate = __bfloat162float(A.g[off]);
    float v1 = 0.f, vl = 0.f;
    if (A.vfirst) { v1 = __bfloat162float(A.vfirst[off]); vl = __bfloat162float(A.vlin[off]); }
    const float nrm2 = dc_head_total((kf * kk_p) * (kf * kk_p), scratch[0], &totals[0], tid);
    const float inv = 1.f / fmaxf(sqrtf(nrm2), 1e-12f);
    if (A.vfirst) vf = round_bf16(vf + (v1 - vf) * sigmoidf_(v0 + vl));
    const float w = round_bf16(-dc_softplus(-(w0 + wl)) - 0.5f);
    const float a = sigmoidf_(a0 + al);
    const float kkn = kf * kk_p * inv;
    in[DQ][tid] = rf;
    in[DD][tid] = __expf(-__expf(w));
    in[DK_][tid] = round_bf16(kf * (1.f + (a - 1.f) * ka_p));
    in[DV][tid] = vf;
    in[DA][tid] = round_bf16(-kkn);
    in[DB][tid] = round_bf16(kkn * a);
  }
  __syncthreads();

  float red[16];
  {   // sa = S a~ with the state before the update
    float2 a0v, a1v;
    dc_ld4_as2(&in[DA][c0], a0v, a1v);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 acc = __ffma2_rn(S2[i][1], a1v, __fmul2_rn(S2[i][0], a0v));
      red[i] = 0.f;
      red[8 + i] = acc.x + acc.y;
    }
    dc_butterfly(red, lane);
    if (cg & 8) sabuf[r0 + (cg & 7)] = red[0];
    __syncwarp();
  }
  {   // update and read-out
    float2 d0, d1, b0, b1, k0, k1, q0, q1;
    dc_ld4_as2(&in[DD][c0], d0, d1);
    dc_ld4_as2(&in[DB][c0], b0, b1);
    dc_ld4_as2(&in[DK_][c0], k0, k1);
    dc_ld4_as2(&in[DQ][c0], q0, q1);
    const float4 saA = *reinterpret_cast<const float4*>(&sabuf[r0]);
    const float4 saB = *reinterpret_cast<const float4*>(&sabuf[r0 + 4]);
    const float4 vA = *reinterpret_cast<const float4*>(&in[DV][r0]);
    const float4 vB = *reinterpret_cast<const float4*>(&in[DV][r0 + 4]);
    const float sa[8] = {saA.x, saA.y, saA.z, saA.w, saB.x, saB.y, saB.z, saB.w};
    const float vv[8] = {vA.x, vA.y, vA.z, vA.w, vB.x, vB.y, vB.z, vB.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 sai = make_float2(sa[i], sa[i]), vi = make_float2(vv[i], vv[i]);
      S2[i][0] = __ffma2_rn(S2[i][0], d0, __ffma2_rn(sai, b0, __fmul2_rn(vi, k0)));
      S2[i][1] = __ffma2_rn(S2[i][1], d1, __ffma2_rn(sai, b1, __fmul2_rn(vi, k1)));
      const float2 yy = __ffma2_rn(S2[i][1], q1, __fmul2_rn(S2[i][0], q0));
      red[i] = yy.x + yy.y;
      red[8 + i] = 0.f;
    }
    dc_butterfly(red, lane);
    if (!(cg & 8)) ybuf[r0 + cg] = red[0];
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
    *reinterpret_cast<float4*>(sp_out + (r0 + i) * DC_N + c0) = make_float4(S2[i][0].x, S2[i][0].y, S2[i][1].x, S2[i][1].y);
  __syncthreads();

  if (prep) {   // GroupNorm over the head, bonus, gate
    const float yf = round_bf16(ybuf[tid]);
    const float s = dc_head_total(yf, scratch[0], &totals[1], tid);
    const float bonus = dc_head_total(in[DQ][tid] * in[DK_][tid] * rk, scratch[1], &totals[2], tid);
    const float mean = s * (1.f / 64.f);
    const float q = dc_head_total((yf - mean) * (yf - mean), scratch[0], &totals[3], tid);
    const float rstd = rsqrtf(q * (1.f / 64.f) + A.eps);
    const float o = ((yf - mean) * rstd * gw + gb + bonus * in[DV][tid]) * gate;
    A.z[(size_t)bb * C + ch] = __float2bfloat16_rn(o);
  }
}

}  // namespace

// r, k, v, wlin, alin, g (and vlin, vfirst, or both null): bf16 [B, H * 64]; parameters fp32 [H * 64] (v0 may be null when
// vfirst is); state / state_out fp32 [rows, H, 64, 64] (the same pointer: update in place), row = slots[i] (int64 [B],
// distinct) or i when slots is null; z: bf16 [B, H * 64].
RWKV_EXPORT int rwkv_wkv7_decode_core(const void* r, const void* k, const void* v, const void* wlin, const void* alin,
                                      const void* vlin, const void* vfirst, const void* g, const void* w0,
                                      const void* a0, const void* v0, const void* k_k, const void* k_a,
                                      const void* r_k, const void* gn_w, const void* gn_b, const void* state,
                                      void* state_out, const void* slots, void* z, int B, int H, float eps, void* stream) {
  if (B <= 0 || H <= 0 || B > 65535) return RWKV_ERR_BAD_SHAPE;
  if ((vfirst == nullptr) != (vlin == nullptr) || (vfirst && !v0) || !state || !state_out) return RWKV_ERR_BAD_SHAPE;
  DecodeCoreArgs a;
  a.r = (const bf16*)r; a.k = (const bf16*)k; a.v = (const bf16*)v; a.wlin = (const bf16*)wlin;
  a.alin = (const bf16*)alin; a.vlin = (const bf16*)vlin; a.vfirst = (const bf16*)vfirst; a.g = (const bf16*)g;
  a.w0 = (const float*)w0; a.a0 = (const float*)a0; a.v0 = (const float*)v0; a.k_k = (const float*)k_k;
  a.k_a = (const float*)k_a; a.r_k = (const float*)r_k; a.gn_w = (const float*)gn_w; a.gn_b = (const float*)gn_b;
  a.state = (const float*)state; a.state_out = (float*)state_out; a.slots = (const long long*)slots; a.z = (bf16*)z; a.H = H; a.eps = eps;
  rwkv_launch(wkv7_decode_core_kernel, dim3(H, B), dim3(DC_THREADS), 0, (cudaStream_t)stream, a);
  return rwkv_launch_status();
}
