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
// Forward.  Thread layout inside a warp: 8 row pairs x 4 column quarters; a thread holds
// S[2][16].  Row sums need two shuffle stages.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NTHREADS)
wkv7_fwd_kernel(const bf16* __restrict__ q_, const bf16* __restrict__ w_, const bf16* __restrict__ k_,
                const bf16* __restrict__ v_, const bf16* __restrict__ a_, const bf16* __restrict__ b_,
                const float* __restrict__ s0, bf16* __restrict__ y_, float* __restrict__ sa_out,
                float* __restrict__ ckpt, float* __restrict__ s_final, int T, int H) {
  __shared__ __align__(16) float in[6][CH][N];
  __shared__ __align__(16) float ybuf[CH][N];
  __shared__ __align__(16) float sabuf[CH][N];

  const int h = blockIdx.x, bb = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r0 = warp * 16 + (lane >> 2) * 2;   // first of this thread's two rows
  const int c0 = (lane & 3) * 16;               // first of its sixteen columns
  const int NC = (T + CH - 1) / CH;
  const size_t tok_stride = (size_t)H * N;
  const size_t base = ((size_t)bb * T * H + h) * N;
  const bf16* src[6] = {q_, w_, k_, v_, a_, b_};

  float S[2][16];
  if (s0) {
    const float* p = s0 + ((size_t)bb * H + h) * N * N;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        float4 t = *reinterpret_cast<const float4*>(p + (r0 + i) * N + c0 + j);
        S[i][j] = t.x; S[i][j + 1] = t.y; S[i][j + 2] = t.z; S[i][j + 3] = t.w;
      }
  } else {
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 16; ++j) S[i][j] = 0.f;
  }

  // staging assignment: tensor i, step tid/8, 8-element part tid%8
  const int st_step = tid >> 3, st_part = tid & 7;
  uint4 pre[6];
  auto prefetch = [&](int c) {
    const int t = c * CH + st_step;
#pragma unroll
    for (int i = 0; i < 6; ++i) {
      if (t < T) pre[i] = *reinterpret_cast<const uint4*>(src[i] + base + (size_t)t * tok_stride + st_part * 8);
      else pre[i] = make_uint4(0, 0, 0, 0);
    }
  };
  prefetch(0);

  for (int c = 0; c < NC; ++c) {
    // registers -> shared (fp32); decay computed once here
    {
      const bool live = (c * CH + st_step) < T;
#pragma unroll
      for (int i = 0; i < 6; ++i) {
        float f[8];
        unpack8(pre[i], f);
        if (i == ID) {
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = live ? __expf(-__expf(f[e])) : 1.f;
        }
        float4* dst = reinterpret_cast<float4*>(&in[i][st_step][st_part * 8]);
        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
      }
    }
    __syncthreads();
    if (c + 1 < NC) prefetch(c + 1);

#pragma unroll 2
    for (int t = 0; t < CH; ++t) {
      float sa0 = 0.f, sa1 = 0.f;
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        float4 av = *reinterpret_cast<const float4*>(&in[IA][t][c0 + j]);
        sa0 += S[0][j] * av.x + S[0][j + 1] * av.y + S[0][j + 2] * av.z + S[0][j + 3] * av.w;
        sa1 += S[1][j] * av.x + S[1][j + 1] * av.y + S[1][j + 2] * av.z + S[1][j + 3] * av.w;
      }
      sa0 += __shfl_xor_sync(0xffffffffu, sa0, 1);
      sa1 += __shfl_xor_sync(0xffffffffu, sa1, 1);
      sa0 += __shfl_xor_sync(0xffffffffu, sa0, 2);
      sa1 += __shfl_xor_sync(0xffffffffu, sa1, 2);
      const float2 vv = *reinterpret_cast<const float2*>(&in[IV][t][r0]);
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        const float4 dv = *reinterpret_cast<const float4*>(&in[ID][t][c0 + j]);
        const float4 bv = *reinterpret_cast<const float4*>(&in[IB][t][c0 + j]);
        const float4 kv = *reinterpret_cast<const float4*>(&in[IK][t][c0 + j]);
        const float4 qv = *reinterpret_cast<const float4*>(&in[IQ][t][c0 + j]);
        const float dd[4] = {dv.x, dv.y, dv.z, dv.w}, bbv[4] = {bv.x, bv.y, bv.z, bv.w};
        const float kk[4] = {kv.x, kv.y, kv.z, kv.w}, qq[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          S[0][j + e] = S[0][j + e] * dd[e] + (sa0 * bbv[e] + vv.x * kk[e]);
          S[1][j + e] = S[1][j + e] * dd[e] + (sa1 * bbv[e] + vv.y * kk[e]);
          y0 += S[0][j + e] * qq[e];
          y1 += S[1][j + e] * qq[e];
        }
      }
      y0 += __shfl_xor_sync(0xffffffffu, y0, 1);
      y1 += __shfl_xor_sync(0xffffffffu, y1, 1);
      y0 += __shfl_xor_sync(0xffffffffu, y0, 2);
      y1 += __shfl_xor_sync(0xffffffffu, y1, 2);
      if ((lane & 3) == 0) {
        *reinterpret_cast<float2*>(&ybuf[t][r0]) = make_float2(y0, y1);
        *reinterpret_cast<float2*>(&sabuf[t][r0]) = make_float2(sa0, sa1);
      }
    }
    __syncthreads();

    // coalesced write-out of this chunk: y as bf16 (8 per thread), sa as fp32
    {
      const int t = c * CH + st_step;
      if (t < T) {
        const float* ysrc = &ybuf[st_step][st_part * 8];
        *reinterpret_cast<uint4*>(y_ + base + (size_t)t * tok_stride + st_part * 8) = pack8(ysrc);
        if (sa_out) {
          float4* d4 = reinterpret_cast<float4*>(sa_out + base + (size_t)t * tok_stride + st_part * 8);
          const float4* s4 = reinterpret_cast<const float4*>(&sabuf[st_step][st_part * 8]);
          d4[0] = s4[0];
          d4[1] = s4[1];
        }
      }
    }
    if (ckpt) {
      float* p = ckpt + (((size_t)bb * H + h) * NC + c) * N * N;
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          *reinterpret_cast<float4*>(p + (r0 + i) * N + c0 + j) =
              make_float4(S[i][j], S[i][j + 1], S[i][j + 2], S[i][j + 3]);
    }
  }
  if (s_final) {
    float* p = s_final + ((size_t)bb * H + h) * N * N;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 16; j += 4)
        *reinterpret_cast<float4*>(p + (r0 + i) * N + c0 + j) =
            make_float4(S[i][j], S[i][j + 1], S[i][j + 2], S[i][j + 3]);
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
  float out[B_NOUT][CH][N];
  float ck[N][N];
  uint4 raw[7][CH][N / 8];   // bf16 staging: q w k v a b dy
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

// 16 per-lane partial values -> lane holds the warp total of row ((lane >> 1) & 15) in v[0]
__device__ __forceinline__ void row_butterfly(float (&v)[16], int lane) {
  {
    const bool hi = lane & 16;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float send = hi ? v[i] : v[i + 8];
      float keep = hi ? v[i + 8] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
  }
  {
    const bool hi = lane & 8;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float send = hi ? v[i] : v[i + 4];
      float keep = hi ? v[i + 4] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
  }
  {
    const bool hi = lane & 4;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float send = hi ? v[i] : v[i + 2];
      float keep = hi ? v[i + 2] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
  }
  {
    const bool hi = lane & 2;
    float send = hi ? v[0] : v[1];
    float keep = hi ? v[1] : v[0];
    v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
  v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
}

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
  const int R = warp * 16;
  const int cl = lane * 2;
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
    const float* cp = ck_base + (size_t)c * N * N;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = (tid + i * NTHREADS) * 4;
      cp_async16(&sm.ck[0][0] + e, cp + e, true);
    }
    cp_async_commit();
  };

  float S[16][2], dS[16][2];
  if (ds_T) {
    const float* p = ds_T + ((size_t)bb * H + h) * N * N;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float2 t = *reinterpret_cast<const float2*>(p + (R + i) * N + cl);
      dS[i][0] = t.x; dS[i][1] = t.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) dS[i][0] = dS[i][1] = 0.f;
  }

  stage(NC - 1);
  for (int c = NC - 1; c >= 0; --c) {
    cp_async_wait_all();
    __syncthreads();   // staged data visible; previous chunk's outputs fully written out
    // convert staged bf16 -> fp32 working arrays
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
      float4 z = make_float4(0, 0, 0, 0);
#pragma unroll
      for (int o = 0; o < B_NOUT - 1; ++o) {   // the five atomically accumulated arrays
        float4* p = reinterpret_cast<float4*>(&sm.out[o][st_step][st_part * 8]);
        p[0] = z; p[1] = z;
      }
    }
    // state at the end of this chunk, from the forward's checkpoint
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float2 t = *reinterpret_cast<const float2*>(&sm.ck[R + i][cl]);
      S[i][0] = t.x; S[i][1] = t.y;
    }
    __syncthreads();
    if (c > 0) stage(c - 1);

    for (int t = CH - 1; t >= 0; --t) {
      const float2 q2 = *reinterpret_cast<const float2*>(&sm.in[BQ][t][cl]);
      const float2 k2 = *reinterpret_cast<const float2*>(&sm.in[BK][t][cl]);
      const float2 b2 = *reinterpret_cast<const float2*>(&sm.in[BB][t][cl]);
      const float2 a2 = *reinterpret_cast<const float2*>(&sm.in[BA][t][cl]);
      const float2 d2 = *reinterpret_cast<const float2*>(&sm.in[BD][t][cl]);
      const float2 i2 = *reinterpret_cast<const float2*>(&sm.in[BINVD][t][cl]);
      float dq0 = 0, dq1 = 0, dw0 = 0, dw1 = 0, dk0 = 0, dk1 = 0, db0 = 0, db1 = 0;
      float dvp[16], dsap[16];
#pragma unroll
      for (int g = 0; g < 16; g += 4) {
        const float4 v4 = *reinterpret_cast<const float4*>(&sm.in[BV][t][R + g]);
        const float4 s4 = *reinterpret_cast<const float4*>(&sm.in[BSA][t][R + g]);
        const float4 y4 = *reinterpret_cast<const float4*>(&sm.in[BDY][t][R + g]);
        const float vv[4] = {v4.x, v4.y, v4.z, v4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
        const float yy[4] = {y4.x, y4.y, y4.z, y4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = g + e;
          dq0 += S[i][0] * yy[e];
          dq1 += S[i][1] * yy[e];
          dS[i][0] += yy[e] * q2.x;
          dS[i][1] += yy[e] * q2.y;
          const float sp0 = (S[i][0] - vv[e] * k2.x - ss[e] * b2.x) * i2.x;
          const float sp1 = (S[i][1] - vv[e] * k2.y - ss[e] * b2.y) * i2.y;
          dw0 += dS[i][0] * sp0;
          dw1 += dS[i][1] * sp1;
          dk0 += dS[i][0] * vv[e];
          dk1 += dS[i][1] * vv[e];
          db0 += dS[i][0] * ss[e];
          db1 += dS[i][1] * ss[e];
          dvp[i] = dS[i][0] * k2.x + dS[i][1] * k2.y;
          dsap[i] = dS[i][0] * b2.x + dS[i][1] * b2.y;
          S[i][0] = sp0;
          S[i][1] = sp1;
        }
      }
      row_butterfly(dvp, lane);
      row_butterfly(dsap, lane);
      if ((lane & 1) == 0) {
        const int row = (lane >> 1) & 15;
        sm.out[OV][t][R + row] = dvp[0];
        sm.dsa[warp][row] = dsap[0];
      }
      __syncwarp();
      float da0 = 0, da1 = 0;
#pragma unroll
      for (int g = 0; g < 16; g += 4) {
        const float4 s4 = *reinterpret_cast<const float4*>(&sm.dsa[warp][g]);
        const float ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = g + e;
          da0 += S[i][0] * ss[e];
          da1 += S[i][1] * ss[e];
          dS[i][0] = dS[i][0] * d2.x + ss[e] * a2.x;
          dS[i][1] = dS[i][1] * d2.y + ss[e] * a2.y;
        }
      }
      __syncwarp();
      atomicAdd(&sm.out[OQ][t][cl], dq0);  atomicAdd(&sm.out[OQ][t][cl + 1], dq1);
      atomicAdd(&sm.out[OW][t][cl], dw0);  atomicAdd(&sm.out[OW][t][cl + 1], dw1);
      atomicAdd(&sm.out[OK_][t][cl], dk0); atomicAdd(&sm.out[OK_][t][cl + 1], dk1);
      atomicAdd(&sm.out[OB][t][cl], db0);  atomicAdd(&sm.out[OB][t][cl + 1], db1);
      atomicAdd(&sm.out[OA][t][cl], da0);  atomicAdd(&sm.out[OA][t][cl + 1], da1);
    }
    __syncthreads();
    // write the six gradients of this chunk (bf16, 8 per thread per tensor)
    {
      const int t = c * CH + st_step;
      if (t < T) {
        const size_t off = base + (size_t)t * tok_stride + st_part * 8;
        float f[8];
        bf16* dst[6] = {dq_, dw_, dk_, db_, da_, dv_};
#pragma unroll
        for (int o = 0; o < B_NOUT; ++o) {
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = sm.out[o][st_step][st_part * 8 + e];
          if (o == OW) {
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] *= sm.in[BDWF][st_step][st_part * 8 + e];
          }
          *reinterpret_cast<uint4*>(dst[o] + off) = pack8(f);
        }
      }
    }
  }
  if (ds0) {
    float* p = ds0 + ((size_t)bb * H + h) * N * N;
#pragma unroll
    for (int i = 0; i < 16; ++i) *reinterpret_cast<float2*>(p + (R + i) * N + cl) = make_float2(dS[i][0], dS[i][1]);
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
  dim3 grid(H, B);
  wkv7_fwd_kernel<<<grid, NTHREADS, 0, (cudaStream_t)stream>>>(
      (const bf16*)q, (const bf16*)w, (const bf16*)k, (const bf16*)v, (const bf16*)a, (const bf16*)b,
      (const float*)s0, (bf16*)y, (float*)sa, (float*)ckpt, (float*)s_final, T, H);
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
