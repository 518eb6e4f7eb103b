// WKV7 in chunked, tensor-core form (head size 64, chunks of 16 steps).
//
// Within a chunk the recurrence  S_t = S_{t-1} diag(d_t) + (S_{t-1} a_t) b_t^T + v_t k_t^T,  y_t = S_t q_t
// is rewritten with cumulative decays  gamma_t = prod_{i<=t} d_i  and the scaled operands
//   At = a * gamma_{t-1},  Bt = b / gamma_t,  Kt = k / gamma_t,  Qt = q * gamma_t,
//   Bb = b * gamma_L / gamma_t,  Kb = k * gamma_L / gamma_t
// as a handful of small matrix products (all indices s, t inside the chunk, j over key channels):
//   Mab = striu(Bt At^T)  Mka = striu(Kt At^T)  Pb = triu(Bt Qt^T)  Pk = triu(Kt Qt^T)      [16 x 16]
//   R = S0 At^T + V Mka ;   U = R (I - Mab)^-1 ;   Y = S0 Qt^T + U Pb + V Pk               [64 x 16]
//   S_L = S0 diag(gamma_L) + U Bb + V Kb                                                    [64 x 64]
// The diagonal decay of the carried state stays in fp32; only the rank-16 corrections go through bf16
// tensor-core operands (mma.sync m16n8k16, fp32 accumulation), so rounding does not compound through
// the decay.  One CTA per (batch, head); warp w owns state rows [16w, 16w+16) as accumulator
// fragments.  The 16x16 unit-triangular inverse is a forward substitution in fp32.
//
// The backward pass is the transpose of these products, chunk by chunk in reverse, recomputing the
// intra-chunk matrices from the inputs and the saved chunk-start state (bf16); it never inverts the
// recurrence.  Gradients w.r.t. the decay follow from d(log gamma_t), reverse-cumulated over t.
//
// These small dependent products are issued with mma.sync from registers: tcgen05 needs operands in
// shared memory and results read back from tensor memory between every dependent product, which costs
// more than the 16x16x64 products themselves.
#include "common.cuh"

namespace {

constexpr int N = 64;
constexpr int L = 16;
constexpr int LDS_ = 72;     // padded row length (bf16) of the [16][64] operand arrays
constexpr int LDM = 24;      // padded row length (bf16) of the [16][16] matrices
constexpr int NT = 128;

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// A fragment (16 x 16) of a row-major array X[row][col] (leading dimension ld elements): rows r0.., cols c0..
__device__ __forceinline__ void load_a(uint32_t (&a)[4], const bf16* X, int ld, int r0, int c0, int lane) {
  ldsm4(a, s32(X + (r0 + (lane & 15)) * ld + c0 + (lane >> 4) * 8));
}
// A fragment of the transpose: A[m][k] = X[k][m]; X row-major [k][m]: rows k0.., cols m0..
__device__ __forceinline__ void load_a_t(uint32_t (&a)[4], const bf16* X, int ld, int k0, int m0, int lane) {
  const int mi = lane >> 3, r = lane & 7;
  ldsm4t(a, s32(X + (k0 + (mi >> 1) * 8 + r) * ld + m0 + (mi & 1) * 8));
}
// B fragments for two adjacent n-tiles (n0..n0+15) and one k-step (k0..k0+15) from storage Z[n][k]:
// out[0],out[1] = tile n0 ; out[2],out[3] = tile n0+8
__device__ __forceinline__ void load_b(uint32_t (&b)[4], const bf16* Z, int ld, int n0, int k0, int lane) {
  const int mi = lane >> 3, r = lane & 7;
  ldsm4(b, s32(Z + (n0 + (mi >> 1) * 8 + r) * ld + k0 + (mi & 1) * 8));
}
// Same, from storage W[k][n] (n contiguous): B[k][n] = W[k][n]
__device__ __forceinline__ void load_b_t(uint32_t (&b)[4], const bf16* W, int ld, int k0, int n0, int lane) {
  const int mi = lane >> 3, r = lane & 7;
  ldsm4t(b, s32(W + (k0 + (mi & 1) * 8 + r) * ld + n0 + (mi >> 1) * 8));
}
// accumulator (16 x 16 as two n-tiles) -> A fragment
__device__ __forceinline__ void acc_to_a(uint32_t (&a)[4], const float (&c0)[4], const float (&c1)[4]) {
  a[0] = pack_bf16(c0[0], c0[1]);
  a[1] = pack_bf16(c0[2], c0[3]);
  a[2] = pack_bf16(c1[0], c1[1]);
  a[3] = pack_bf16(c1[2], c1[3]);
}

struct FwdSm {
  uint4 raw[2][6][L][N / 8];      // q w k v a b (bf16), double buffered
  float cs[L][N];                 // cumulative log decay
  bf16 At[L][LDS_], Bt[L][LDS_], Kt[L][LDS_], Qt[L][LDS_], Bb[L][LDS_], Kb[L][LDS_], Vs[L][LDS_];
  float Mab[L][L + 1];
  bf16 MkaT[L][LDM], PbT[L][LDM], PkT[L][LDM], TinvT[L][LDM];
  float gL[N];
  float ybuf[L][N];
};

enum { RQ = 0, RW, RK, RV, RA, RB };

__device__ __forceinline__ void cp16(void* dst, const void* src, bool pred) {
  const int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s32(dst)), "l"(src), "r"(sz) : "memory");
}

// Builds cs, gL and the seven operand arrays of one chunk from sm.raw[buf].  All threads.
template <class SM>
__device__ __forceinline__ void build_operands(SM& sm, int buf, int chunk, int T) {
  const int tid = threadIdx.x;
  if (tid < N) {
    const bf16* wrow = reinterpret_cast<const bf16*>(&sm.raw[buf][RW][0][0]);
    float acc = 0.f;
#pragma unroll
    for (int t = 0; t < L; ++t) {
      const bool live = chunk * L + t < T;
      acc += live ? -__expf(__bfloat162float(wrow[t * N + tid])) : 0.f;
      sm.cs[t][tid] = acc;
    }
    sm.gL[tid] = __expf(acc);
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < (L * N) / NT; ++i) {
    const int e = tid + i * NT, t = e >> 6, j = e & 63;
    const float c = sm.cs[t][j], cp = t ? sm.cs[t - 1][j] : 0.f, cl = sm.cs[L - 1][j];
    const float ec = __expf(c), enc = __expf(-c), ecp = __expf(cp), el = __expf(cl - c);
    const float qv = __bfloat162float(reinterpret_cast<const bf16*>(&sm.raw[buf][RQ][0][0])[e]);
    const float kv = __bfloat162float(reinterpret_cast<const bf16*>(&sm.raw[buf][RK][0][0])[e]);
    const float av = __bfloat162float(reinterpret_cast<const bf16*>(&sm.raw[buf][RA][0][0])[e]);
    const float bv = __bfloat162float(reinterpret_cast<const bf16*>(&sm.raw[buf][RB][0][0])[e]);
    sm.At[t][j] = __float2bfloat16_rn(av * ecp);
    sm.Bt[t][j] = __float2bfloat16_rn(bv * enc);
    sm.Kt[t][j] = __float2bfloat16_rn(kv * enc);
    sm.Qt[t][j] = __float2bfloat16_rn(qv * ec);
    sm.Bb[t][j] = __float2bfloat16_rn(bv * el);
    sm.Kb[t][j] = __float2bfloat16_rn(kv * el);
    sm.Vs[t][j] = reinterpret_cast<const bf16*>(&sm.raw[buf][RV][0][0])[e];
  }
  __syncthreads();
}

// 16x16 product  C[s][t] = sum_j X[s][j] Z[t][j]  by one warp; c0 = columns 0..7, c1 = columns 8..15
__device__ __forceinline__ void small_xzt(float (&c0)[4], float (&c1)[4], const bf16* X, const bf16* Z, int lane) {
#pragma unroll
  for (int e = 0; e < 4; ++e) c0[e] = c1[e] = 0.f;
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    uint32_t a[4], b[4];
    load_a(a, X, LDS_, 0, kk * 16, lane);
    load_b(b, Z, LDS_, 0, kk * 16, lane);
    mma16816(c0, a, b[0], b[1]);
    mma16816(c1, a, b[2], b[3]);
  }
}

// Intra-chunk matrices (independent of the state): Mab (fp32), MkaT, PbT, PkT (bf16, transposed), then TinvT.
template <class SM>
__device__ __forceinline__ void build_small_matrices(SM& sm) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  float c0[4], c1[4];
  const bf16* X = (warp == 0 || warp == 2) ? &sm.Bt[0][0] : &sm.Kt[0][0];
  const bf16* Z = (warp < 2) ? &sm.At[0][0] : &sm.Qt[0][0];
  small_xzt(c0, c1, X, Z, lane);
  const bool strict = warp < 2;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int s = g + (e >> 1) * 8, t = half * 8 + tq * 2 + (e & 1);
      float val = half ? c1[e] : c0[e];
      if (strict ? (s >= t) : (s > t)) val = 0.f;
      if (warp == 0) sm.Mab[s][t] = val;
      else if (warp == 1) sm.MkaT[t][s] = __float2bfloat16_rn(val);
      else if (warp == 2) sm.PbT[t][s] = __float2bfloat16_rn(val);
      else sm.PkT[t][s] = __float2bfloat16_rn(val);
    }
  }
  __syncthreads();
  if (warp == 0 && lane < L) {   // row `lane` of (I - Mab)^-1 by forward substitution
    float x[L];
#pragma unroll
    for (int t = 0; t < L; ++t) {
      float acc = (lane == t) ? 1.f : 0.f;
#pragma unroll
      for (int s = 0; s < t; ++s) acc += x[s] * sm.Mab[s][t];
      x[t] = acc;
      sm.TinvT[t][lane] = __float2bfloat16_rn(acc);
    }
  }
}

__global__ void __launch_bounds__(NT)
wkv7_tc_fwd_kernel(const bf16* __restrict__ q_, const bf16* __restrict__ w_, const bf16* __restrict__ k_,
                   const bf16* __restrict__ v_, const bf16* __restrict__ a_, const bf16* __restrict__ b_,
                   const float* __restrict__ s0, bf16* __restrict__ y_, bf16* __restrict__ chunk_states,
                   float* __restrict__ s_final, int T, int H) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  FwdSm& sm = *reinterpret_cast<FwdSm*>(smem_raw);
  const int h = blockIdx.x, bb = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int m0 = warp * 16;
  const int NC = (T + L - 1) / L;
  const size_t tok_stride = (size_t)H * N;
  const size_t base = ((size_t)bb * T * H + h) * N;
  const bf16* src[6] = {q_, w_, k_, v_, a_, b_};
  const int st_step = tid >> 3, st_part = tid & 7;

  auto stage = [&](int c, int buf) {
    const int t = c * L + st_step;
    const bool live = t < T;
    const size_t off = base + (size_t)(live ? t : 0) * tok_stride + st_part * 8;
#pragma unroll
    for (int u = 0; u < 6; ++u) cp16(&sm.raw[buf][u][st_step][st_part], src[u] + off, live);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // state rows [m0, m0+16) as 8 accumulator tiles: S[n][e]: row m0+g+(e>>1)*8, col 8n+2tq+(e&1)
  float S[8][4];
  if (s0) {
    const float* p = s0 + ((size_t)bb * H + h) * N * N;
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const float2 t2 = *reinterpret_cast<const float2*>(p + (m0 + g + hh * 8) * N + n * 8 + tq * 2);
        S[n][hh * 2] = t2.x; S[n][hh * 2 + 1] = t2.y;
      }
  } else {
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) S[n][e] = 0.f;
  }

  stage(0, 0);
  for (int c = 0; c < NC; ++c) {
    const int buf = c & 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (c + 1 < NC) stage(c + 1, buf ^ 1);
    if (chunk_states) {   // state at the start of this chunk, bf16 (what the backward multiplies with)
      bf16* p = chunk_states + (((size_t)bb * H + h) * NC + c) * N * N;
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
          *reinterpret_cast<uint32_t*>(p + (m0 + g + hh * 8) * N + n * 8 + tq * 2) = pack_bf16(S[n][hh * 2], S[n][hh * 2 + 1]);
    }
    build_operands(sm, buf, c, T);
    build_small_matrices(sm);

    // S0 as A fragments (4 k-steps over the key channels)
    uint32_t sa[4][4];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) acc_to_a(sa[kk], S[2 * kk], S[2 * kk + 1]);
    uint32_t va[4];                                   // V rows of this warp, transposed: A[m=v][k=s]
    load_a_t(va, &sm.Vs[0][0], LDS_, 0, m0, lane);

    float r0[4] = {0, 0, 0, 0}, r1[4] = {0, 0, 0, 0};   // R = S0 At^T + V Mka
    float y0[4] = {0, 0, 0, 0}, y1[4] = {0, 0, 0, 0};   // Y = S0 Qt^T + ...
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t b[4];
      load_b(b, &sm.At[0][0], LDS_, 0, kk * 16, lane);
      mma16816(r0, sa[kk], b[0], b[1]);
      mma16816(r1, sa[kk], b[2], b[3]);
      load_b(b, &sm.Qt[0][0], LDS_, 0, kk * 16, lane);
      mma16816(y0, sa[kk], b[0], b[1]);
      mma16816(y1, sa[kk], b[2], b[3]);
    }
    {
      uint32_t b[4];
      load_b(b, &sm.MkaT[0][0], LDM, 0, 0, lane);
      mma16816(r0, va, b[0], b[1]);
      mma16816(r1, va, b[2], b[3]);
      load_b(b, &sm.PkT[0][0], LDM, 0, 0, lane);
      mma16816(y0, va, b[0], b[1]);
      mma16816(y1, va, b[2], b[3]);
    }
    __syncthreads();   // TinvT ready
    float u0[4] = {0, 0, 0, 0}, u1[4] = {0, 0, 0, 0};
    uint32_t ua[4];
    {
      uint32_t ra[4], b[4];
      acc_to_a(ra, r0, r1);
      load_b(b, &sm.TinvT[0][0], LDM, 0, 0, lane);
      mma16816(u0, ra, b[0], b[1]);
      mma16816(u1, ra, b[2], b[3]);
      acc_to_a(ua, u0, u1);
      load_b(b, &sm.PbT[0][0], LDM, 0, 0, lane);
      mma16816(y0, ua, b[0], b[1]);
      mma16816(y1, ua, b[2], b[3]);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int row = m0 + g + (e >> 1) * 8;
      sm.ybuf[tq * 2 + (e & 1)][row] = y0[e];
      sm.ybuf[8 + tq * 2 + (e & 1)][row] = y1[e];
    }
    // S <- S diag(gamma_L) + U Bb + V Kb
#pragma unroll
    for (int n = 0; n < 8; n += 2) {
      uint32_t b[4];
      const float2 g0 = *reinterpret_cast<const float2*>(&sm.gL[n * 8 + tq * 2]);
      const float2 g1 = *reinterpret_cast<const float2*>(&sm.gL[(n + 1) * 8 + tq * 2]);
      S[n][0] *= g0.x; S[n][1] *= g0.y; S[n][2] *= g0.x; S[n][3] *= g0.y;
      S[n + 1][0] *= g1.x; S[n + 1][1] *= g1.y; S[n + 1][2] *= g1.x; S[n + 1][3] *= g1.y;
      load_b_t(b, &sm.Bb[0][0], LDS_, 0, n * 8, lane);
      mma16816(S[n], ua, b[0], b[1]);
      mma16816(S[n + 1], ua, b[2], b[3]);
      load_b_t(b, &sm.Kb[0][0], LDS_, 0, n * 8, lane);
      mma16816(S[n], va, b[0], b[1]);
      mma16816(S[n + 1], va, b[2], b[3]);
    }
    __syncthreads();
    {
      const int t = c * L + st_step;
      if (t < T) *reinterpret_cast<uint4*>(y_ + base + (size_t)t * tok_stride + st_part * 8) = pack8(&sm.ybuf[st_step][st_part * 8]);
    }
  }
  if (s_final) {
    float* p = s_final + ((size_t)bb * H + h) * N * N;
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
        *reinterpret_cast<float2*>(p + (m0 + g + hh * 8) * N + n * 8 + tq * 2) = make_float2(S[n][hh * 2], S[n][hh * 2 + 1]);
  }
}

}  // namespace

// q,w,k,v,a,b,y: bf16 [B,T,H,64];  s0 / s_final: fp32 [B,H,64,64] (nullable);
// chunk_states: bf16 [B,H,ceil(T/16),64,64] (nullable) = state at the start of every chunk, for the backward.
RWKV_EXPORT int rwkv_wkv7_tc_forward(const void* q, const void* w, const void* k, const void* v, const void* a,
                                     const void* b, const void* s0, void* y, void* chunk_states, void* s_final, int B,
                                     int T, int H, void* stream) {
  if (B <= 0 || T <= 0 || H <= 0 || B > 65535) return RWKV_ERR_BAD_SHAPE;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(wkv7_tc_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(FwdSm));
    if (e != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)e;
    configured = true;
  }
  wkv7_tc_fwd_kernel<<<dim3(H, B), NT, sizeof(FwdSm), (cudaStream_t)stream>>>(
      (const bf16*)q, (const bf16*)w, (const bf16*)k, (const bf16*)v, (const bf16*)a, (const bf16*)b, (const float*)s0,
      (bf16*)y, (bf16*)chunk_states, (float*)s_final, T, H);
  return rwkv_launch_status();
}
