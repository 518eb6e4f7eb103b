// WKV7 state recurrence for head size 64: forward with state in/out and the
// reverse-time backward with state-gradient in/out.
//
//   sa = S a ;  S <- S diag(d) + sa b^T + v k^T ;  y = S q ,   d = exp(-exp(w))
//
// S is [value row][key column] in fp32.  Every row of S evolves independently of
// the others (only the emitted gradients sum over rows), so one CTA owns a
// (batch, head) pair and its four warps each own 16 rows.  Inputs are staged for
// 16 time steps at a time, which leaves two block barriers per 16 steps instead of
// two per step; the next 16 steps are prefetched into registers while the current
// ones are computed.
//
// Replaces the reference's three kernels (training: wkv7_cuda.cu:10-134, stateful
// inference: wkv7s.cu:5-54, infinite-context: wkv7_infctx_cuda.cu:28-342) with one
// forward and one backward that take optional state / state-gradient pointers.
#include "common.cuh"

namespace {

constexpr int N = 64;        // head size
constexpr int CH = 16;       // staged time steps
constexpr int NTHREADS = 128;

enum { IQ = 0, ID = 1, IK = 2, IV = 3, IA = 4, IB = 5 };

// ------------------------------------------------------------------------------------------
// Forward.  Four warps per head, a warp owns 16 rows: 2 row groups x 16 column groups, a
// thread holds an 8 x 4 block of S as packed float2.  The recurrence is latency bound (one
// dependent chain per step), so each step does one combined reduction: the row sums of
// y_t = S_t q_t and of sa_{t+1} = S_t a_{t+1} go through the same halving butterfly
// (16 values over 16 lanes, 15 shuffles, 4 stages).
// ------------------------------------------------------------------------------------------
struct FwdSmem {
  float in[6][CH][N];
  float ybuf[CH][N];
  float sabuf[CH + 1][N];
  uint4 raw[2][6][CH][N / 8];
};

// v[0..7] = y partials, v[8..15] = sa partials.  On return v[0] holds, for lanes with
// (lane & 8) == 0, the y total of row (lane & 7); for the other lanes the sa total of that row.
__device__ __forceinline__ void fwd_butterfly(float (&v)[16], int lane) {
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

__device__ __forceinline__ void cp_async16_f(void* smem_dst, const void* gsrc, bool pred) {
  uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc), "r"(sz) : "memory");
}

__device__ __forceinline__ void ld4_as2(const float* p, float2& lo, float2& hi) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  lo = make_float2(x.x, x.y);
  hi = make_float2(x.z, x.w);
}

__global__ void __launch_bounds__(NTHREADS)
wkv7_fwd_kernel(const bf16* __restrict__ q_, const bf16* __restrict__ w_, const bf16* __restrict__ k_,
                const bf16* __restrict__ v_, const bf16* __restrict__ a_, const bf16* __restrict__ b_,
                const float* __restrict__ s0, bf16* __restrict__ y_, float* __restrict__ sa_out,
                float* __restrict__ ckpt, float* __restrict__ s_final, const long long* __restrict__ slots,
                int T, int H) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>(smem_raw);
  rwkv_chain_begin();

  const int h = blockIdx.x, bb = blockIdx.y;
  // state row of this sequence: its batch index, or its slot in a state pool (continuous batching keeps the
  // states of all admitted sequences in one pool and decodes any subset of them in place)
  const size_t srow = slots ? (size_t)slots[bb] : (size_t)bb;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = lane >> 4, cg = lane & 15;
  const int r0 = warp * 16 + rg * 8;     // first of this thread's 8 rows
  const int c0 = cg * 4;                 // first of its 4 columns
  const int NC = (T + CH - 1) / CH;
  const size_t tok_stride = (size_t)H * N;
  const size_t base = ((size_t)bb * T * H + h) * N;
  const bf16* src[6] = {q_, w_, k_, v_, a_, b_};

  float2 S2[8][2];
  if (s0) {
    const float* p = s0 + (srow * H + h) * N * N;
#pragma unroll
    for (int i = 0; i < 8; ++i) ld4_as2(p + (r0 + i) * N + c0, S2[i][0], S2[i][1]);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) S2[i][0] = S2[i][1] = make_float2(0.f, 0.f);
  }

  // staging: 6 tensors x 16 steps x 8 parts = 768 vectors, 6 per thread (tensor u, step tid/8, part tid%8)
  const int st_step = tid >> 3, st_part = tid & 7;
  auto stage = [&](int c, int buf) {
    const int t = c * CH + st_step;
    const bool live = t < T;
    const size_t off = base + (size_t)(live ? t : 0) * tok_stride + st_part * 8;
#pragma unroll
    for (int u = 0; u < 6; ++u) cp_async16_f(&sm.raw[buf][u][st_step][st_part], src[u] + off, live);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  stage(0, 0);

  for (int c = 0; c < NC; ++c) {
    const int buf = c & 1;
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();   // raw[buf] landed; previous chunk's ybuf/sabuf fully written out
    if (c + 1 < NC) stage(c + 1, buf ^ 1);
    {
      const bool live = (c * CH + st_step) < T;
#pragma unroll
      for (int u = 0; u < 6; ++u) {
        float f[8];
        unpack8(sm.raw[buf][u][st_step][st_part], f);
        if (u == ID) {
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = live ? __expf(-__expf(f[e])) : 1.f;
        } else if (!live) {
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = 0.f;
        }
        float4* dst = reinterpret_cast<float4*>(&sm.in[u][st_step][st_part * 8]);
        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
      }
    }
    __syncthreads();

    float red[16];
    // sa of the chunk's first step
    {
      float2 a0, a1;
      ld4_as2(&sm.in[IA][0][c0], a0, a1);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 acc = __ffma2_rn(S2[i][1], a1, __fmul2_rn(S2[i][0], a0));
        red[i] = 0.f;
        red[8 + i] = acc.x + acc.y;
      }
      fwd_butterfly(red, lane);
      if (cg & 8) sm.sabuf[0][r0 + (cg & 7)] = red[0];
      __syncwarp();
    }

    const int nsteps = min(CH, T - c * CH);   // the last chunk may be short (decode runs one step)
#pragma unroll 1
    for (int t = 0; t < nsteps; ++t) {
      float2 d0, d1, b0, b1, k0, k1, q0, q1, a0, a1;
      ld4_as2(&sm.in[ID][t][c0], d0, d1);
      ld4_as2(&sm.in[IB][t][c0], b0, b1);
      ld4_as2(&sm.in[IK][t][c0], k0, k1);
      ld4_as2(&sm.in[IQ][t][c0], q0, q1);
      const int tn = (t + 1 < CH) ? t + 1 : t;
      ld4_as2(&sm.in[IA][tn][c0], a0, a1);
      const float4 saA = *reinterpret_cast<const float4*>(&sm.sabuf[t][r0]);
      const float4 saB = *reinterpret_cast<const float4*>(&sm.sabuf[t][r0 + 4]);
      const float4 vA = *reinterpret_cast<const float4*>(&sm.in[IV][t][r0]);
      const float4 vB = *reinterpret_cast<const float4*>(&sm.in[IV][t][r0 + 4]);
      const float sa[8] = {saA.x, saA.y, saA.z, saA.w, saB.x, saB.y, saB.z, saB.w};
      const float vv[8] = {vA.x, vA.y, vA.z, vA.w, vB.x, vB.y, vB.z, vB.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 sai = make_float2(sa[i], sa[i]), vi = make_float2(vv[i], vv[i]);
        S2[i][0] = __ffma2_rn(S2[i][0], d0, __ffma2_rn(sai, b0, __fmul2_rn(vi, k0)));
        S2[i][1] = __ffma2_rn(S2[i][1], d1, __ffma2_rn(sai, b1, __fmul2_rn(vi, k1)));
        const float2 yy = __ffma2_rn(S2[i][1], q1, __fmul2_rn(S2[i][0], q0));
        const float2 ss = __ffma2_rn(S2[i][1], a1, __fmul2_rn(S2[i][0], a0));
        red[i] = yy.x + yy.y;
        red[8 + i] = ss.x + ss.y;
      }
      fwd_butterfly(red, lane);
      if (cg & 8) sm.sabuf[t + 1][r0 + (cg & 7)] = red[0];
      else sm.ybuf[t][r0 + cg] = red[0];
      __syncwarp();
    }
    __syncthreads();

    // coalesced write-out: y as bf16, sa as fp32 (one 8-element vector per thread each)
    {
      const int t = c * CH + st_step;
      if (t < T) {
        const size_t off = base + (size_t)t * tok_stride + st_part * 8;
        *reinterpret_cast<uint4*>(y_ + off) = pack8(&sm.ybuf[st_step][st_part * 8]);
        if (sa_out) {
          float4* d4 = reinterpret_cast<float4*>(sa_out + off);
          const float4* s4 = reinterpret_cast<const float4*>(&sm.sabuf[st_step][st_part * 8]);
          d4[0] = s4[0];
          d4[1] = s4[1];
        }
      }
    }
    if (ckpt) {
      float* p = ckpt + (((size_t)bb * H + h) * NC + c) * N * N;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        *reinterpret_cast<float4*>(p + (r0 + i) * N + c0) = make_float4(S2[i][0].x, S2[i][0].y, S2[i][1].x, S2[i][1].y);
    }
  }
  if (s_final) {
    float* p = s_final + (srow * H + h) * N * N;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      *reinterpret_cast<float4*>(p + (r0 + i) * N + c0) = make_float4(S2[i][0].x, S2[i][0].y, S2[i][1].x, S2[i][1].y);
  }
}

// ------------------------------------------------------------------------------------------
// Backward.  A warp owns 16 rows, a lane owns 2 columns of S and dS for all 16 rows, so the
// column sums (dq, dw, dk, db, da) are thread-local per warp and only cross the four warps
// through shared-memory adds; the row sums (dv, dsa) go through a halving butterfly.
// S_{t-1} is rebuilt from S_t by inverting the update (d >= 0.545 because w <= -0.5) and is
// re-synchronised from the forward's checkpoint at every 16-step boundary.
// ------------------------------------------------------------------------------------------
enum { BQ = 0, BK, BV, BA, BB, BDY, BSA, BD, BINVD, BDWF, B_NIN };
enum { OQ = 0, OW, OK_, OB, OA, OV, B_NOUT };

struct BwdSmem {
  float in[B_NIN][CH][N];
  float part[4][CH / 2][5][N];   // per-warp column sums for half a chunk: dq dw dk db da
  float ov[CH / 2][N];           // dv for half a chunk
  uint4 raw[7][CH][N / 8];       // bf16 staging: q w k v a b dy
  float raw_sa[CH][N];
  float dsa[4][16];
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool pred) {
  uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// 8 per-lane partials -> v[0] = total over the 16 column-group lanes of row ((lane >> 1) & 7)
__device__ __forceinline__ void row8x16_butterfly(float (&v)[8], int lane) {
  {
    const bool hi = lane & 8;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float send = hi ? v[i] : v[i + 4];
      const float keep = hi ? v[i + 4] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
  }
  {
    const bool hi = lane & 4;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float send = hi ? v[i] : v[i + 2];
      const float keep = hi ? v[i + 2] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
  }
  {
    const bool hi = lane & 2;
    const float send = hi ? v[0] : v[1];
    const float keep = hi ? v[1] : v[0];
    v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
  v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
}

__device__ __forceinline__ float2 bc2(float x) { return make_float2(x, x); }
__device__ __forceinline__ float2 neg2(float2 x) { return make_float2(-x.x, -x.y); }

// Thread layout: warp = 16 rows (2 row groups of 8) x 64 columns (16 column groups of 4).
// A thread holds an 8 x 4 block of S and of dS as packed float2.
__global__ void __launch_bounds__(NTHREADS, 2)
wkv7_bwd_kernel(const bf16* __restrict__ q_, const bf16* __restrict__ w_, const bf16* __restrict__ k_,
                const bf16* __restrict__ v_, const bf16* __restrict__ a_, const bf16* __restrict__ b_,
                const bf16* __restrict__ dy_, const float* __restrict__ sa_, const float* __restrict__ ckpt,
                const float* __restrict__ ds_T, bf16* __restrict__ dq_, bf16* __restrict__ dw_,
                bf16* __restrict__ dk_, bf16* __restrict__ dv_, bf16* __restrict__ da_, bf16* __restrict__ db_,
                float* __restrict__ ds0, int T, int H) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  BwdSmem& sm = *reinterpret_cast<BwdSmem*>(smem_raw);

  const int h = blockIdx.x, bb = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = lane >> 4, cg = lane & 15;
  const int R = warp * 16 + rg * 8;   // first of this thread's 8 rows
  const int cl = cg * 4;              // first of its 4 columns
  const int NC = (T + CH - 1) / CH;
  const size_t tok_stride = (size_t)H * N;
  const size_t base = ((size_t)bb * T * H + h) * N;
  const bf16* src[7] = {q_, w_, k_, v_, a_, b_, dy_};
  const float* ck_base = ckpt + ((size_t)bb * H + h) * NC * N * N;
  const int st_step = tid >> 3, st_part = tid & 7;

  auto stage = [&](int c) {
    const int t = c * CH + st_step;
    const bool live = t < T;
    const size_t off = base + (size_t)(live ? t : 0) * tok_stride + st_part * 8;
#pragma unroll
    for (int i = 0; i < 7; ++i) cp_async16(&sm.raw[i][st_step][st_part], src[i] + off, live);
    cp_async16(&sm.raw_sa[st_step][st_part * 8], sa_ + off, live);
    cp_async16(&sm.raw_sa[st_step][st_part * 8 + 4], sa_ + off + 4, live);
    cp_async_commit();
  };

  float2 S2[8][2], dS2[8][2];
  if (ds_T) {
    const float* p = ds_T + ((size_t)bb * H + h) * N * N;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 t = *reinterpret_cast<const float4*>(p + (R + i) * N + cl);
      dS2[i][0] = make_float2(t.x, t.y); dS2[i][1] = make_float2(t.z, t.w);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) dS2[i][0] = dS2[i][1] = make_float2(0.f, 0.f);
  }

  float4 ckn[8];   // checkpoint of the chunk about to be processed, prefetched one chunk ahead
  {
    const float* cp = ck_base + (size_t)(NC - 1) * N * N;
#pragma unroll
    for (int i = 0; i < 8; ++i) ckn[i] = __ldg(reinterpret_cast<const float4*>(cp + (R + i) * N + cl));
  }
  stage(NC - 1);
  for (int c = NC - 1; c >= 0; --c) {
    cp_async_wait_all();
    __syncthreads();   // staged data visible; previous chunk's outputs fully written out
    {
      const bool live = (c * CH + st_step) < T;
      float f[8];
      const int dstmap[7] = {BQ, -1, BK, BV, BA, BB, BDY};
#pragma unroll
      for (int i = 0; i < 7; ++i) {
        unpack8(sm.raw[i][st_step][st_part], f);
        if (i == 1) {
          float d[8], id[8], wf[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float ew = __expf(f[e]);
            d[e] = live ? __expf(-ew) : 1.f;
            id[e] = 1.f / d[e];
            wf[e] = live ? -ew * d[e] : 0.f;
          }
          float4* p0 = reinterpret_cast<float4*>(&sm.in[BD][st_step][st_part * 8]);
          float4* p1 = reinterpret_cast<float4*>(&sm.in[BINVD][st_step][st_part * 8]);
          float4* p2 = reinterpret_cast<float4*>(&sm.in[BDWF][st_step][st_part * 8]);
          p0[0] = make_float4(d[0], d[1], d[2], d[3]);     p0[1] = make_float4(d[4], d[5], d[6], d[7]);
          p1[0] = make_float4(id[0], id[1], id[2], id[3]); p1[1] = make_float4(id[4], id[5], id[6], id[7]);
          p2[0] = make_float4(wf[0], wf[1], wf[2], wf[3]); p2[1] = make_float4(wf[4], wf[5], wf[6], wf[7]);
        } else {
          float4* p = reinterpret_cast<float4*>(&sm.in[dstmap[i]][st_step][st_part * 8]);
          p[0] = live ? make_float4(f[0], f[1], f[2], f[3]) : make_float4(0, 0, 0, 0);
          p[1] = live ? make_float4(f[4], f[5], f[6], f[7]) : make_float4(0, 0, 0, 0);
        }
      }
      float4* ps = reinterpret_cast<float4*>(&sm.in[BSA][st_step][st_part * 8]);
      const float4* rs = reinterpret_cast<const float4*>(&sm.raw_sa[st_step][st_part * 8]);
      ps[0] = live ? rs[0] : make_float4(0, 0, 0, 0);
      ps[1] = live ? rs[1] : make_float4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) { S2[i][0] = make_float2(ckn[i].x, ckn[i].y); S2[i][1] = make_float2(ckn[i].z, ckn[i].w); }
    __syncthreads();
    if (c > 0) {
      stage(c - 1);
      const float* cp = ck_base + (size_t)(c - 1) * N * N;
#pragma unroll
      for (int i = 0; i < 8; ++i) ckn[i] = __ldg(reinterpret_cast<const float4*>(cp + (R + i) * N + cl));
    }

#pragma unroll 1
    for (int hb = 1; hb >= 0; --hb) {
#pragma unroll 1
    for (int t = hb * 8 + 7; t >= hb * 8; --t) {
      const int t8 = t & 7;
      float2 q2[2], k2[2], b2[2], id2[2];
      {
        const float4 x = *reinterpret_cast<const float4*>(&sm.in[BQ][t][cl]);
        q2[0] = make_float2(x.x, x.y); q2[1] = make_float2(x.z, x.w);
        const float4 y = *reinterpret_cast<const float4*>(&sm.in[BK][t][cl]);
        k2[0] = make_float2(y.x, y.y); k2[1] = make_float2(y.z, y.w);
        const float4 z = *reinterpret_cast<const float4*>(&sm.in[BB][t][cl]);
        b2[0] = make_float2(z.x, z.y); b2[1] = make_float2(z.z, z.w);
        const float4 u = *reinterpret_cast<const float4*>(&sm.in[BINVD][t][cl]);
        id2[0] = make_float2(u.x, u.y); id2[1] = make_float2(u.z, u.w);
      }
      float vv[8], ss[8], yy[8];
      {
        const float4 a0 = *reinterpret_cast<const float4*>(&sm.in[BV][t][R]);
        const float4 a1 = *reinterpret_cast<const float4*>(&sm.in[BV][t][R + 4]);
        vv[0] = a0.x; vv[1] = a0.y; vv[2] = a0.z; vv[3] = a0.w; vv[4] = a1.x; vv[5] = a1.y; vv[6] = a1.z; vv[7] = a1.w;
        const float4 b0 = *reinterpret_cast<const float4*>(&sm.in[BSA][t][R]);
        const float4 b1 = *reinterpret_cast<const float4*>(&sm.in[BSA][t][R + 4]);
        ss[0] = b0.x; ss[1] = b0.y; ss[2] = b0.z; ss[3] = b0.w; ss[4] = b1.x; ss[5] = b1.y; ss[6] = b1.z; ss[7] = b1.w;
        const float4 c0 = *reinterpret_cast<const float4*>(&sm.in[BDY][t][R]);
        const float4 c1 = *reinterpret_cast<const float4*>(&sm.in[BDY][t][R + 4]);
        yy[0] = c0.x; yy[1] = c0.y; yy[2] = c0.z; yy[3] = c0.w; yy[4] = c1.x; yy[5] = c1.y; yy[6] = c1.z; yy[7] = c1.w;
      }
      // column accumulators: [0..1]=dq, [2..3]=dw, [4..5]=dk, [6..7]=db, [8..9]=da (packed pairs)
      float2 col[10];
#pragma unroll
      for (int j = 0; j < 10; ++j) col[j] = make_float2(0.f, 0.f);
      float dvp[8], dsap[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 dyi = bc2(yy[i]), vi = bc2(vv[i]), si = bc2(ss[i]);
        const float2 nvi = neg2(vi), nsi = neg2(si);
        float2 tv = make_float2(0.f, 0.f), ts = make_float2(0.f, 0.f);
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          col[0 + p] = __ffma2_rn(S2[i][p], dyi, col[0 + p]);
          dS2[i][p] = __ffma2_rn(dyi, q2[p], dS2[i][p]);
          float2 sp = __ffma2_rn(nvi, k2[p], S2[i][p]);
          sp = __ffma2_rn(nsi, b2[p], sp);
          sp = __fmul2_rn(sp, id2[p]);
          col[2 + p] = __ffma2_rn(dS2[i][p], sp, col[2 + p]);
          col[4 + p] = __ffma2_rn(dS2[i][p], vi, col[4 + p]);
          col[6 + p] = __ffma2_rn(dS2[i][p], si, col[6 + p]);
          tv = __ffma2_rn(dS2[i][p], k2[p], tv);
          ts = __ffma2_rn(dS2[i][p], b2[p], ts);
          S2[i][p] = sp;
        }
        dvp[i] = tv.x + tv.y;
        dsap[i] = ts.x + ts.y;
      }
      row8x16_butterfly(dvp, lane);
      row8x16_butterfly(dsap, lane);
      if ((cg & 1) == 0) {
        sm.ov[t8][R + (cg >> 1)] = dvp[0];
        sm.dsa[warp][rg * 8 + (cg >> 1)] = dsap[0];
      }
      __syncwarp();
      {
        const float4 e0 = *reinterpret_cast<const float4*>(&sm.dsa[warp][rg * 8]);
        const float4 e1 = *reinterpret_cast<const float4*>(&sm.dsa[warp][rg * 8 + 4]);
        const float ds_[8] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w};
        float2 a2[2], d2[2];
        const float4 x = *reinterpret_cast<const float4*>(&sm.in[BA][t][cl]);
        a2[0] = make_float2(x.x, x.y); a2[1] = make_float2(x.z, x.w);
        const float4 y = *reinterpret_cast<const float4*>(&sm.in[BD][t][cl]);
        d2[0] = make_float2(y.x, y.y); d2[1] = make_float2(y.z, y.w);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 di = bc2(ds_[i]);
#pragma unroll
          for (int p = 0; p < 2; ++p) {
            col[8 + p] = __ffma2_rn(S2[i][p], di, col[8 + p]);
            dS2[i][p] = __ffma2_rn(dS2[i][p], d2[p], __fmul2_rn(di, a2[p]));
          }
        }
      }
      __syncwarp();
      // sum the two row groups (lanes l and l^16); each keeps half of the 20 column values
      {
        float cv[20];
#pragma unroll
        for (int j = 0; j < 10; ++j) { cv[2 * j] = col[j].x; cv[2 * j + 1] = col[j].y; }
        const bool hi = lane & 16;
#pragma unroll
        for (int j = 0; j < 10; ++j) {
          const float send = hi ? cv[j] : cv[j + 10];
          const float keep = hi ? cv[j + 10] : cv[j];
          cv[j] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
        }
        // value index j (0..19) -> array j/4, column cl + j%4; low lanes hold 0..9, high lanes 10..19
        float* pw = &sm.part[warp][t8][0][0];
        if (!hi) {
          *reinterpret_cast<float4*>(pw + 0 * N + cl) = make_float4(cv[0], cv[1], cv[2], cv[3]);
          *reinterpret_cast<float4*>(pw + 1 * N + cl) = make_float4(cv[4], cv[5], cv[6], cv[7]);
          *reinterpret_cast<float2*>(pw + 2 * N + cl) = make_float2(cv[8], cv[9]);
        } else {
          *reinterpret_cast<float2*>(pw + 2 * N + cl + 2) = make_float2(cv[0], cv[1]);
          *reinterpret_cast<float4*>(pw + 3 * N + cl) = make_float4(cv[2], cv[3], cv[4], cv[5]);
          *reinterpret_cast<float4*>(pw + 4 * N + cl) = make_float4(cv[6], cv[7], cv[8], cv[9]);
        }
      }
    }
    __syncthreads();
    // half-chunk write-out: threads 0..63 emit dq dw dk, threads 64..127 emit db da dv
    {
      const int grp = tid >> 6, s8 = (tid >> 3) & 7, part = tid & 7;
      const int tl = hb * 8 + s8, t = c * CH + tl;
      if (t < T) {
        const size_t off = base + (size_t)t * tok_stride + part * 8;
        bf16* dst[6] = {dq_, dw_, dk_, db_, da_, dv_};
#pragma unroll
        for (int u = 0; u < 3; ++u) {
          const int o = grp * 3 + u;   // 0..5 ; 5 = dv
          float f[8];
          if (o < 5) {
#pragma unroll
            for (int e = 0; e < 8; ++e)
              f[e] = sm.part[0][s8][o][part * 8 + e] + sm.part[1][s8][o][part * 8 + e] +
                     sm.part[2][s8][o][part * 8 + e] + sm.part[3][s8][o][part * 8 + e];
            if (o == OW) {
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] *= sm.in[BDWF][tl][part * 8 + e];
            }
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = sm.ov[s8][part * 8 + e];
          }
          *reinterpret_cast<uint4*>(dst[o] + off) = pack8(f);
        }
      }
    }
    __syncthreads();
    }   // hb
  }
  if (ds0) {
    float* p = ds0 + ((size_t)bb * H + h) * N * N;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      *reinterpret_cast<float4*>(p + (R + i) * N + cl) = make_float4(dS2[i][0].x, dS2[i][0].y, dS2[i][1].x, dS2[i][1].y);
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------
// C entry points.  All tensors are contiguous; q,w,k,v,a,b,y,dy and the gradients are
// bf16 [B,T,H,64]; sa is fp32 [B,T,H,64]; ckpt is fp32 [B,H,ceil(T/16),64,64]; states are
// fp32 [B,H,64,64].  Nullable: s0, sa, ckpt, s_final (forward); ds_T, ds0 (backward).
// ------------------------------------------------------------------------------------------
RWKV_EXPORT int rwkv_wkv7_forward(const void* q, const void* w, const void* k, const void* v, const void* a,
                                  const void* b, const void* s0, void* y, void* sa, void* ckpt, void* s_final,
                                  int B, int T, int H, void* stream) {
  if (B <= 0 || T <= 0 || H <= 0 || B > 65535) return RWKV_ERR_BAD_SHAPE;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(wkv7_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(FwdSmem));
    if (e != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)e;
    configured = true;
  }
  dim3 grid(H, B);
  rwkv_launch(wkv7_fwd_kernel, grid, dim3(NTHREADS), sizeof(FwdSmem), (cudaStream_t)stream,
      (const bf16*)q, (const bf16*)w, (const bf16*)k, (const bf16*)v, (const bf16*)a, (const bf16*)b,
      (const float*)s0, (bf16*)y, (float*)sa, (float*)ckpt, (float*)s_final, nullptr, T, H);
  return rwkv_launch_status();
}

// Forward on a state pool: sequence i reads and writes pool[slots[i]] ([n_slots, H, 64, 64] fp32) in place; no
// gather before and no scatter after the step.  q .. b, y: bf16 [B, T, H, 64]; slots: int64 [B], distinct.
RWKV_EXPORT int rwkv_wkv7_forward_slots(const void* q, const void* w, const void* k, const void* v, const void* a,
                                        const void* b, void* pool, const void* slots, void* y, int B, int T, int H,
                                        void* stream) {
  if (B <= 0 || T <= 0 || H <= 0 || B > 65535 || !pool || !slots) return RWKV_ERR_BAD_SHAPE;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(wkv7_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(FwdSmem));
    if (e != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)e;
    configured = true;
  }
  dim3 grid(H, B);
  rwkv_launch(wkv7_fwd_kernel, grid, dim3(NTHREADS), sizeof(FwdSmem), (cudaStream_t)stream,
      (const bf16*)q, (const bf16*)w, (const bf16*)k, (const bf16*)v, (const bf16*)a, (const bf16*)b,
      (const float*)pool, (bf16*)y, nullptr, nullptr, (float*)pool, (const long long*)slots, T, H);
  return rwkv_launch_status();
}

RWKV_EXPORT int rwkv_wkv7_backward(const void* q, const void* w, const void* k, const void* v, const void* a,
                                   const void* b, const void* dy, const void* sa, const void* ckpt,
                                   const void* ds_T, void* dq, void* dw, void* dk, void* dv, void* da, void* db,
                                   void* ds0, int B, int T, int H, void* stream) {
  if (B <= 0 || T <= 0 || H <= 0 || B > 65535) return RWKV_ERR_BAD_SHAPE;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(wkv7_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(BwdSmem));
    if (e != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)e;
    configured = true;
  }
  dim3 grid(H, B);
  wkv7_bwd_kernel<<<grid, NTHREADS, sizeof(BwdSmem), (cudaStream_t)stream>>>(
      (const bf16*)q, (const bf16*)w, (const bf16*)k, (const bf16*)v, (const bf16*)a, (const bf16*)b,
      (const bf16*)dy, (const float*)sa, (const float*)ckpt, (const float*)ds_T, (bf16*)dq, (bf16*)dw,
      (bf16*)dk, (bf16*)dv, (bf16*)da, (bf16*)db, (float*)ds0, T, H);
  return rwkv_launch_status();
}
