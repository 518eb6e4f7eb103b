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
// the decay.  The 16x16 unit-triangular inverse is a forward substitution in fp32.
//
// Kernels:
//   prep        one CTA per chunk (full occupancy): everything that does not depend on the carried
//               state - cumulative decays, scaled operands, the 16x16 matrices, the inverse - written
//               to a workspace (10.5 KB per chunk) that the forward scan AND, if the caller keeps it,
//               both backward kernels read.
//   fwd scan    one CTA per (batch, head), warp w owns state rows [16w, 16w+16) as accumulator
//               fragments; walks the chunks issuing only tensor-core products on operands prefetched
//               with cp.async; stores the bf16 state at the start of every chunk for the backward.
//   bwd scan    the same walk in reverse for dS:  dU = dY Pb^T + dS Bb^T,  dR = dU Tinv^T,
//               dS0 = dY Qt + dS diag(gamma_L) + dR At;  stores dS at the end of every chunk (bf16).
//   bwd chunk   one CTA per chunk (three per SM): loads the workspace operands, recomputes R, U from the
//               saved chunk-start state and forms all six input gradients from the transposed products
//               (optionally adding them to gradients already in the output buffers).  It never inverts
//               the recurrence.  The decay gradient is the reverse cumulative sum over t of d(log gamma_t).
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
constexpr int NP = 72;       // padded row length (fp32) of [16][64] arrays read by accumulator-layout threads
constexpr int RAWLD = 9;     // uint4 per row of the raw input tiles (8 used): 144-byte rows avoid bank conflicts

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

enum { RQ = 0, RW, RK, RV, RA, RB };

__device__ __forceinline__ void cp16(void* dst, const void* src, bool pred) {
  const int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s32(dst)), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int K>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(K) : "memory"); }

__device__ __forceinline__ void ld8f(float (&f)[8], const float* p) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// Prefix products of the decay over the 16 steps of a chunk: E[t][j] = exp(sum_{i<=t} -exp(w_i[j])) (fp32) and,
// with WRITE_GL, gL[j] = E[15][j].  Thread (channel j, half h) scans steps 8h .. 8h+7, the second half then adds
// the first half's total (`scratch`: 64 floats).  All NT threads; ends with a block barrier.
template <bool WRITE_GL>
__device__ __forceinline__ void decay_scan(const bf16* wrow, int ld, float (*E)[NP], float* gL, float* scratch,
                                           int chunk, int T) {
  const int tid = threadIdx.x;
  const int j = tid & (N - 1), hf = tid >> 6;
  float c[8];
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int t = hf * 8 + i;
    const bool live = chunk * L + t < T;
    acc += live ? -__expf(__bfloat162float(wrow[t * ld + j])) : 0.f;
    c[i] = acc;
  }
  if (hf == 0) scratch[j] = acc;
  __syncthreads();
  const float base = hf ? scratch[j] : 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) E[hf * 8 + i][j] = __expf(c[i] + base);
  if (WRITE_GL && hf) gL[j] = __expf(c[7] + base);
  __syncthreads();
}

// From sm.raw (q w k v a b of one chunk, bf16, rows past the sequence end zero-filled) builds
//   E[t][j] = gamma_t (fp32), gL = gamma_L, and the bf16 operand arrays At Bt Kt Qt Bb Kb Vs.
// All NT threads; thread (row, part) handles 8 consecutive channels of one step.
template <class SM>
__device__ __forceinline__ void build_operands(SM& sm, int chunk, int T) {
  const int tid = threadIdx.x;
  decay_scan<true>(reinterpret_cast<const bf16*>(&sm.raw[RW][0][0]), RAWLD * 8, sm.E, sm.gL, &sm.Mab[0][0], chunk, T);
  const int row = tid >> 3, part = tid & 7, j0 = part * 8;
  float e[8], ep[8], gl[8], qv[8], kv[8], av[8], bv[8];
  ld8f(e, &sm.E[row][j0]);
  if (row) ld8f(ep, &sm.E[row - 1][j0]);
  else {
#pragma unroll
    for (int i = 0; i < 8; ++i) ep[i] = 1.f;
  }
  ld8f(gl, &sm.gL[j0]);
  unpack8(sm.raw[RQ][row][part], qv);
  unpack8(sm.raw[RK][row][part], kv);
  unpack8(sm.raw[RA][row][part], av);
  unpack8(sm.raw[RB][row][part], bv);
  float at[8], bt[8], kt[8], qt[8], bb[8], kb[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float inv = __fdividef(1.f, e[i]), el = gl[i] * inv;
    at[i] = av[i] * ep[i];
    bt[i] = bv[i] * inv;
    kt[i] = kv[i] * inv;
    qt[i] = qv[i] * e[i];
    bb[i] = bv[i] * el;
    kb[i] = kv[i] * el;
  }
  *reinterpret_cast<uint4*>(&sm.At[row][j0]) = pack8(at);
  *reinterpret_cast<uint4*>(&sm.Bt[row][j0]) = pack8(bt);
  *reinterpret_cast<uint4*>(&sm.Kt[row][j0]) = pack8(kt);
  *reinterpret_cast<uint4*>(&sm.Qt[row][j0]) = pack8(qt);
  *reinterpret_cast<uint4*>(&sm.Bb[row][j0]) = pack8(bb);
  *reinterpret_cast<uint4*>(&sm.Kb[row][j0]) = pack8(kb);
  *reinterpret_cast<uint4*>(&sm.Vs[row][j0]) = sm.raw[RV][row][part];
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

// Intra-chunk matrices (independent of the state): Mab (fp32), Mka, Pb, Pk and Tinv = (I - Mab)^-1 in bf16,
// stored transposed (xT[t][s] = x[s][t]).  Ends with a block barrier: all outputs are visible on return.
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
      const bf16 hv = __float2bfloat16_rn(val);
      if (warp == 0) sm.Mab[s][t] = val;
      else if (warp == 1) sm.MkaT[t][s] = hv;
      else if (warp == 2) sm.PbT[t][s] = hv;
      else sm.PkT[t][s] = hv;
    }
  }
  __syncthreads();
  if (warp == 0 && lane < L) {
    // Row `lane` of X = (I - Mab)^-1:  x[t] = [t == lane] + sum_{s<t} x[s] Mab[s][t].  Column-oriented: as soon as
    // x[s] is known it is pushed into every later accumulator, so the dependent chain is one FMA per step and the
    // other 15 - s FMAs of the step are independent.
    float acc[L];
#pragma unroll
    for (int t = 0; t < L; ++t) acc[t] = (lane == t) ? 1.f : 0.f;
#pragma unroll
    for (int s_ = 0; s_ < L; ++s_) {
      const float xs = acc[s_];
#pragma unroll
      for (int t = s_ + 1; t < L; ++t) acc[t] += xs * sm.Mab[s_][t];
      sm.TinvT[s_][lane] = __float2bfloat16_rn(xs);
    }
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------------ prep
struct WsFwd {          // per chunk, 10496 bytes
  bf16 At[L][N], Qt[L][N], Bb[L][N], Kb[L][N];
  bf16 MkaT[L][L], PbT[L][L], PkT[L][L], TinvT[L][L];
  float gL[N];
};
struct PrepSm {
  uint4 raw[6][L][RAWLD];
  float E[L][NP];
  float gL[N];
  bf16 At[L][LDS_], Bt[L][LDS_], Kt[L][LDS_], Qt[L][LDS_], Bb[L][LDS_], Kb[L][LDS_], Vs[L][LDS_];
  float Mab[L][L + 1];
  bf16 MkaT[L][LDM], PbT[L][LDM], PkT[L][LDM], TinvT[L][LDM];
};

// Loads the six raw input tiles of chunk c (rows past T zero-filled) with cp.async; caller waits.
template <class SM>
__device__ __forceinline__ void load_raw_chunk(SM& sm, const bf16* const (&src)[6], size_t base, size_t tok_stride,
                                               int c, int T) {
  const int row = threadIdx.x >> 3, part = threadIdx.x & 7;
  const int t = c * L + row;
  const bool live = t < T;
  const size_t off = base + (size_t)(live ? t : 0) * tok_stride + part * 8;
#pragma unroll
  for (int u = 0; u < 6; ++u) cp16(&sm.raw[u][row][part], src[u] + off, live);
}

// grid (NC, H, B): one chunk per CTA, writes that chunk's WsFwd.
__global__ void __launch_bounds__(NT)
wkv7_tc_prep_kernel(const bf16* __restrict__ q_, const bf16* __restrict__ w_, const bf16* __restrict__ k_,
                    const bf16* __restrict__ v_, const bf16* __restrict__ a_, const bf16* __restrict__ b_,
                    unsigned char* __restrict__ ws, int T, int H) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  PrepSm& sm = *reinterpret_cast<PrepSm*>(smem_raw);
  const int c = blockIdx.x, h = blockIdx.y, bb = blockIdx.z;
  const int NC = gridDim.x;
  const int tid = threadIdx.x;
  const bf16* const src[6] = {q_, w_, k_, v_, a_, b_};
  load_raw_chunk(sm, src, ((size_t)bb * T * H + h) * N, (size_t)H * N, c, T);
  cp_commit();
  cp_wait<0>();
  __syncthreads();
  build_operands(sm, c, T);
  build_small_matrices(sm);
  const size_t chunk_id = ((size_t)bb * H + h) * NC + c;
  const int row = tid >> 3, part = tid & 7, j0 = part * 8;
  auto cpy = [](bf16* dst, const bf16* src_) { *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src_); };
  WsFwd* o = reinterpret_cast<WsFwd*>(ws + chunk_id * sizeof(WsFwd));
  cpy(&o->At[row][j0], &sm.At[row][j0]);
  cpy(&o->Qt[row][j0], &sm.Qt[row][j0]);
  cpy(&o->Bb[row][j0], &sm.Bb[row][j0]);
  cpy(&o->Kb[row][j0], &sm.Kb[row][j0]);
  if (part < 2) {
    cpy(&o->MkaT[row][j0], &sm.MkaT[row][j0]);
    cpy(&o->PbT[row][j0], &sm.PbT[row][j0]);
    cpy(&o->PkT[row][j0], &sm.PkT[row][j0]);
    cpy(&o->TinvT[row][j0], &sm.TinvT[row][j0]);
  }
  if (tid < N) o->gL[tid] = sm.gL[tid];
}

// ------------------------------------------------------------------------------------------ scans
constexpr int STAGES = 3;

// accumulator rows [m0, m0+16) x 64 columns <-> global fp32 / bf16 [64][64]
__device__ __forceinline__ void load_state_f32(float (&S)[8][4], const float* p, int m0, int g, int tq) {
#pragma unroll
  for (int n = 0; n < 8; ++n)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const float2 t2 = *reinterpret_cast<const float2*>(p + (m0 + g + hh * 8) * N + n * 8 + tq * 2);
      S[n][hh * 2] = t2.x; S[n][hh * 2 + 1] = t2.y;
    }
}
__device__ __forceinline__ void store_state_f32(const float (&S)[8][4], float* p, int m0, int g, int tq) {
#pragma unroll
  for (int n = 0; n < 8; ++n)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
      *reinterpret_cast<float2*>(p + (m0 + g + hh * 8) * N + n * 8 + tq * 2) = make_float2(S[n][hh * 2], S[n][hh * 2 + 1]);
}

// bf16 copy of a warp's 16 x 64 state rows to global memory through a per-warp staging tile, so that the global stores
// are 16 bytes wide and every 128-byte row leaves as two full requests.  (Stored straight from the accumulator layout
// the same data takes sixteen 4-byte store instructions per thread with eight partial sectors each; on the forward
// scan that cost a third of the kernel's time.)
struct StateStage { bf16 t[4][16][LDS_]; };
__device__ __forceinline__ void store_state_bf16_wide(const float (&S)[8][4], bf16* p, StateStage& stg, int warp, int m0,
                                                      int lane) {
  const int g = lane >> 2, tq = lane & 3;
  __syncwarp();      // the previous chunk's reads of the staging tile are done
#pragma unroll
  for (int n = 0; n < 8; ++n)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
      *reinterpret_cast<uint32_t*>(&stg.t[warp][g + hh * 8][n * 8 + tq * 2]) = pack_bf16(S[n][hh * 2], S[n][hh * 2 + 1]);
  __syncwarp();
  const int r = lane >> 1, hf = lane & 1;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<uint4*>(p + (m0 + r) * N + hf * 32 + i * 8) =
        *reinterpret_cast<const uint4*>(&stg.t[warp][r][hf * 32 + i * 8]);
}

struct ScanStage {
  bf16 At[L][LDS_], Qt[L][LDS_], Bb[L][LDS_], Kb[L][LDS_], Vs[L][LDS_];
  bf16 MkaT[L][LDM], PbT[L][LDM], PkT[L][LDM], TinvT[L][LDM];
  float gL[N];
};
struct ScanSm {
  ScanStage st[STAGES];
  StateStage stg;
};

__global__ void __launch_bounds__(NT)
wkv7_tc_scan_kernel(const bf16* __restrict__ v_, const unsigned char* __restrict__ ws, const float* __restrict__ s0,
                    bf16* __restrict__ y_, bf16* __restrict__ chunk_states, float* __restrict__ s_final, int T, int H) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  ScanSm& sm = *reinterpret_cast<ScanSm*>(smem_raw);
  const int h = blockIdx.x, bb = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int m0 = warp * 16;
  const int NC = (T + L - 1) / L;
  const size_t tok_stride = (size_t)H * N;
  const size_t base = ((size_t)bb * T * H + h) * N;
  const int row = tid >> 3, part = tid & 7;

  auto stage = [&](int c) {
    if (c < NC) {
      ScanStage& s = sm.st[c % STAGES];
      const WsFwd* w = reinterpret_cast<const WsFwd*>(ws + (((size_t)bb * H + h) * NC + c) * sizeof(WsFwd));
      cp16(&s.At[row][part * 8], &w->At[row][part * 8], true);
      cp16(&s.Qt[row][part * 8], &w->Qt[row][part * 8], true);
      cp16(&s.Bb[row][part * 8], &w->Bb[row][part * 8], true);
      cp16(&s.Kb[row][part * 8], &w->Kb[row][part * 8], true);
      const int t = c * L + row;
      const bool live = t < T;
      cp16(&s.Vs[row][part * 8], v_ + base + (size_t)(live ? t : 0) * tok_stride + part * 8, live);
      if (part < 2) {
        cp16(&s.MkaT[row][part * 8], &w->MkaT[row][part * 8], true);
        cp16(&s.PbT[row][part * 8], &w->PbT[row][part * 8], true);
        cp16(&s.PkT[row][part * 8], &w->PkT[row][part * 8], true);
        cp16(&s.TinvT[row][part * 8], &w->TinvT[row][part * 8], true);
      }
      if (tid < 16) cp16(&s.gL[tid * 4], &w->gL[tid * 4], true);
    }
    cp_commit();   // committed even when empty so the wait count below stays uniform
  };

  float S[8][4];
  if (s0) load_state_f32(S, s0 + ((size_t)bb * H + h) * N * N, m0, g, tq);
  else {
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) S[n][e] = 0.f;
  }

#pragma unroll
  for (int c = 0; c < STAGES - 1; ++c) stage(c);
  for (int c = 0; c < NC; ++c) {
    cp_wait<STAGES - 2>();
    __syncthreads();   // chunk c landed for all threads; the buffer of chunk c-1 is free
    stage(c + STAGES - 1);
    const ScanStage& s = sm.st[c % STAGES];
    if (chunk_states)
      store_state_bf16_wide(S, chunk_states + (((size_t)bb * H + h) * NC + c) * N * N, sm.stg, warp, m0, lane);

    // all operand fragments first, so the loads overlap the dependent products
    uint32_t bAt[4][4], bQt[4][4], bBb[4][4], bKb[4][4], bMka[4], bPk[4], bTinv[4], bPb[4], va[4];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      load_b(bAt[kk], &s.At[0][0], LDS_, 0, kk * 16, lane);
      load_b(bQt[kk], &s.Qt[0][0], LDS_, 0, kk * 16, lane);
    }
    load_a_t(va, &s.Vs[0][0], LDS_, 0, m0, lane);
    load_b(bMka, &s.MkaT[0][0], LDM, 0, 0, lane);
    load_b(bPk, &s.PkT[0][0], LDM, 0, 0, lane);
    load_b(bTinv, &s.TinvT[0][0], LDM, 0, 0, lane);
    load_b(bPb, &s.PbT[0][0], LDM, 0, 0, lane);
#pragma unroll
    for (int n2 = 0; n2 < 4; ++n2) {
      load_b_t(bBb[n2], &s.Bb[0][0], LDS_, 0, n2 * 16, lane);
      load_b_t(bKb[n2], &s.Kb[0][0], LDS_, 0, n2 * 16, lane);
    }
    float2 gl[8];          // decay of this thread's state columns, read with the other operands (no load on the path)
#pragma unroll
    for (int n = 0; n < 8; ++n) gl[n] = *reinterpret_cast<const float2*>(&s.gL[n * 8 + tq * 2]);
    uint32_t sa[4][4];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) acc_to_a(sa[kk], S[2 * kk], S[2 * kk + 1]);

    // The chunk-to-chunk dependency runs  S -> R -> U -> S.  A dependent mma.sync costs its full latency, so every
    // product on that path gets its own accumulator (summed with plain adds afterwards) and everything that does not
    // depend on U (V Kb, V Mka, the Y terms) is issued off the path: three dependent products per chunk instead of eight.
    float rp[5][2][4];                                   // R = S0 At^T (four k-steps) + V Mka, as independent partials
    float y0[4] = {0, 0, 0, 0}, y1[4] = {0, 0, 0, 0};   // Y = S0 Qt^T + U Pb + V Pk
#pragma unroll
    for (int i = 0; i < 5; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) rp[i][0][e] = rp[i][1][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      mma16816(rp[kk][0], sa[kk], bAt[kk][0], bAt[kk][1]);
      mma16816(rp[kk][1], sa[kk], bAt[kk][2], bAt[kk][3]);
    }
    mma16816(rp[4][0], va, bMka[0], bMka[1]);
    mma16816(rp[4][1], va, bMka[2], bMka[3]);
    float tk[8][4];                                      // V Kb: the part of the state update that does not need U
#pragma unroll
    for (int n2 = 0; n2 < 4; ++n2) {
#pragma unroll
      for (int e = 0; e < 4; ++e) tk[2 * n2][e] = tk[2 * n2 + 1][e] = 0.f;
      mma16816(tk[2 * n2], va, bKb[n2][0], bKb[n2][1]);
      mma16816(tk[2 * n2 + 1], va, bKb[n2][2], bKb[n2][3]);
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      mma16816(y0, sa[kk], bQt[kk][0], bQt[kk][1]);
      mma16816(y1, sa[kk], bQt[kk][2], bQt[kk][3]);
    }
    mma16816(y0, va, bPk[0], bPk[1]);
    mma16816(y1, va, bPk[2], bPk[3]);
    float r0[4], r1[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      r0[e] = (rp[0][0][e] + rp[1][0][e]) + (rp[2][0][e] + rp[3][0][e]) + rp[4][0][e];
      r1[e] = (rp[0][1][e] + rp[1][1][e]) + (rp[2][1][e] + rp[3][1][e]) + rp[4][1][e];
    }
    uint32_t ra[4], ua[4];
    float u0[4] = {0, 0, 0, 0}, u1[4] = {0, 0, 0, 0};
    acc_to_a(ra, r0, r1);
    mma16816(u0, ra, bTinv[0], bTinv[1]);
    mma16816(u1, ra, bTinv[2], bTinv[3]);
    acc_to_a(ua, u0, u1);
    mma16816(y0, ua, bPb[0], bPb[1]);
    mma16816(y1, ua, bPb[2], bPb[3]);
    // S <- S diag(gamma_L) + U Bb + V Kb
#pragma unroll
    for (int n2 = 0; n2 < 4; ++n2) {
      const int n = 2 * n2;
      const float2 g0 = gl[n], g1 = gl[n + 1];
      S[n][0] = S[n][0] * g0.x + tk[n][0]; S[n][1] = S[n][1] * g0.y + tk[n][1];
      S[n][2] = S[n][2] * g0.x + tk[n][2]; S[n][3] = S[n][3] * g0.y + tk[n][3];
      S[n + 1][0] = S[n + 1][0] * g1.x + tk[n + 1][0]; S[n + 1][1] = S[n + 1][1] * g1.y + tk[n + 1][1];
      S[n + 1][2] = S[n + 1][2] * g1.x + tk[n + 1][2]; S[n + 1][3] = S[n + 1][3] * g1.y + tk[n + 1][3];
      mma16816(S[n], ua, bBb[n2][0], bBb[n2][1]);
      mma16816(S[n + 1], ua, bBb[n2][2], bBb[n2][3]);
    }
    // y of this warp's 16 value rows: element (v, t) of the accumulator goes to y[t][v].  Sixteen lanes with the same t
    // write one 32-byte sector between them, so the scattered 2-byte stores stay sector-efficient and nothing on the
    // in-order instruction stream waits for a shared-memory round trip.
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int vrow = m0 + g + (e >> 1) * 8;
      const int ta = c * L + tq * 2 + (e & 1), tb = ta + 8;
      if (ta < T) y_[base + (size_t)ta * tok_stride + vrow] = __float2bfloat16_rn(y0[e]);
      if (tb < T) y_[base + (size_t)tb * tok_stride + vrow] = __float2bfloat16_rn(y1[e]);
    }
  }
  if (s_final) store_state_f32(S, s_final + ((size_t)bb * H + h) * N * N, m0, g, tq);
}

struct BScanStage {
  bf16 At[L][LDS_], Qt[L][LDS_], Bb[L][LDS_], dYs[L][LDS_];
  bf16 PbT[L][LDM], TinvT[L][LDM];
  float gL[N];
};
struct BScanSm {
  BScanStage st[STAGES];
  StateStage stg;
};

// Reverse walk.  dstates[c] = dS at the END of chunk c (bf16); ds0 = dS at the start of the sequence.
// `ws` is a forward workspace (WsFwd): Pb and Tinv are stored transposed.
__global__ void __launch_bounds__(NT)
wkv7_tc_bwd_scan_kernel(const bf16* __restrict__ dy_, const unsigned char* __restrict__ ws,
                        const float* __restrict__ ds_final, bf16* __restrict__ dstates, float* __restrict__ ds0,
                        int T, int H) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  BScanSm& sm = *reinterpret_cast<BScanSm*>(smem_raw);
  const int h = blockIdx.x, bb = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int m0 = warp * 16;
  const int NC = (T + L - 1) / L;
  const size_t tok_stride = (size_t)H * N;
  const size_t base = ((size_t)bb * T * H + h) * N;
  const int row = tid >> 3, part = tid & 7;

  // i counts walked chunks: chunk index c = NC-1-i
  auto stage = [&](int i) {
    if (i < NC) {
      const int c = NC - 1 - i;
      BScanStage& s = sm.st[i % STAGES];
      const WsFwd* w = reinterpret_cast<const WsFwd*>(ws + (((size_t)bb * H + h) * NC + c) * sizeof(WsFwd));
      cp16(&s.At[row][part * 8], &w->At[row][part * 8], true);
      cp16(&s.Qt[row][part * 8], &w->Qt[row][part * 8], true);
      cp16(&s.Bb[row][part * 8], &w->Bb[row][part * 8], true);
      const int t = c * L + row;
      const bool live = t < T;
      cp16(&s.dYs[row][part * 8], dy_ + base + (size_t)(live ? t : 0) * tok_stride + part * 8, live);
      if (part < 2) {
        cp16(&s.PbT[row][part * 8], &w->PbT[row][part * 8], true);
        cp16(&s.TinvT[row][part * 8], &w->TinvT[row][part * 8], true);
      }
      if (tid < 16) cp16(&s.gL[tid * 4], &w->gL[tid * 4], true);
    }
    cp_commit();
  };

  float S[8][4];   // dS rows [m0, m0+16)
  if (ds_final) load_state_f32(S, ds_final + ((size_t)bb * H + h) * N * N, m0, g, tq);
  else {
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) S[n][e] = 0.f;
  }
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) stage(i);
  for (int i = 0; i < NC; ++i) {
    const int c = NC - 1 - i;
    cp_wait<STAGES - 2>();
    __syncthreads();
    stage(i + STAGES - 1);
    const BScanStage& s = sm.st[i % STAGES];
    store_state_bf16_wide(S, dstates + (((size_t)bb * H + h) * NC + c) * N * N, sm.stg, warp, m0, lane);

    uint32_t bBb[4][4], bQt[4][4], bAt[4][4], bPb[4], bTinv[4], dya[4];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) load_b(bBb[kk], &s.Bb[0][0], LDS_, 0, kk * 16, lane);
    load_a_t(dya, &s.dYs[0][0], LDS_, 0, m0, lane);
    load_b_t(bPb, &s.PbT[0][0], LDM, 0, 0, lane);      // stored [t][s]: B[k=t][n=s] is a transposed load
    load_b_t(bTinv, &s.TinvT[0][0], LDM, 0, 0, lane);
#pragma unroll
    for (int n2 = 0; n2 < 4; ++n2) {
      load_b_t(bQt[n2], &s.Qt[0][0], LDS_, 0, n2 * 16, lane);
      load_b_t(bAt[n2], &s.At[0][0], LDS_, 0, n2 * 16, lane);
    }
    float2 gl[8];
#pragma unroll
    for (int n = 0; n < 8; ++n) gl[n] = *reinterpret_cast<const float2*>(&s.gL[n * 8 + tq * 2]);
    uint32_t dsa[4][4];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) acc_to_a(dsa[kk], S[2 * kk], S[2 * kk + 1]);
    // same latency argument as in the forward scan: independent accumulators on the dS -> dU -> dR -> dS path
    float up[5][2][4];                                   // dU = dS Bb^T (four k-steps) + dY Pb^T
#pragma unroll
    for (int i = 0; i < 5; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) up[i][0][e] = up[i][1][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      mma16816(up[kk][0], dsa[kk], bBb[kk][0], bBb[kk][1]);
      mma16816(up[kk][1], dsa[kk], bBb[kk][2], bBb[kk][3]);
    }
    mma16816(up[4][0], dya, bPb[0], bPb[1]);
    mma16816(up[4][1], dya, bPb[2], bPb[3]);
    float tq_[8][4];                                     // dY Qt: independent of dR
#pragma unroll
    for (int n2 = 0; n2 < 4; ++n2) {
#pragma unroll
      for (int e = 0; e < 4; ++e) tq_[2 * n2][e] = tq_[2 * n2 + 1][e] = 0.f;
      mma16816(tq_[2 * n2], dya, bQt[n2][0], bQt[n2][1]);
      mma16816(tq_[2 * n2 + 1], dya, bQt[n2][2], bQt[n2][3]);
    }
    float u0[4], u1[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      u0[e] = (up[0][0][e] + up[1][0][e]) + (up[2][0][e] + up[3][0][e]) + up[4][0][e];
      u1[e] = (up[0][1][e] + up[1][1][e]) + (up[2][1][e] + up[3][1][e]) + up[4][1][e];
    }
    uint32_t dua[4], dra[4];
    acc_to_a(dua, u0, u1);
    float r0[4] = {0, 0, 0, 0}, r1[4] = {0, 0, 0, 0};   // dR = dU Tinv^T
    mma16816(r0, dua, bTinv[0], bTinv[1]);
    mma16816(r1, dua, bTinv[2], bTinv[3]);
    acc_to_a(dra, r0, r1);
    // dS0 = dS diag(gamma_L) + dY Qt + dR At
#pragma unroll
    for (int n2 = 0; n2 < 4; ++n2) {
      const int n = 2 * n2;
      const float2 g0 = gl[n], g1 = gl[n + 1];
      S[n][0] = S[n][0] * g0.x + tq_[n][0]; S[n][1] = S[n][1] * g0.y + tq_[n][1];
      S[n][2] = S[n][2] * g0.x + tq_[n][2]; S[n][3] = S[n][3] * g0.y + tq_[n][3];
      S[n + 1][0] = S[n + 1][0] * g1.x + tq_[n + 1][0]; S[n + 1][1] = S[n + 1][1] * g1.y + tq_[n + 1][1];
      S[n + 1][2] = S[n + 1][2] * g1.x + tq_[n + 1][2]; S[n + 1][3] = S[n + 1][3] * g1.y + tq_[n + 1][3];
      mma16816(S[n], dra, bAt[n2][0], bAt[n2][1]);
      mma16816(S[n + 1], dra, bAt[n2][2], bAt[n2][3]);
    }
  }
  if (ds0) store_state_f32(S, ds0 + ((size_t)bb * H + h) * N * N, m0, g, tq);
}

// ------------------------------------------------------------------------------------------ bwd chunk
struct BwdSm {
  bf16 wraw[L][N];                                 // log-decay inputs of the chunk
  float E[L][NP];
  float gL[N];
  bf16 At[L][LDS_], Bt[L][LDS_], Kt[L][LDS_], Qt[L][LDS_], Bb[L][LDS_], Kb[L][LDS_], Vs[L][LDS_];
  bf16 dYs[L][LDS_];
  bf16 S0s[N][LDS_], dSs[N][LDS_];
  bf16 MkaT[L][LDM], PbT[L][LDM], PkT[L][LDM], TinvT[L][LDM];       // from the forward workspace
  bf16 dPbN[L][LDM], dPkN[L][LDM], dMkaN[L][LDM], dMabN[L][LDM];
  bf16 Us[4][L][LDM], dRs[4][L][LDM];              // per warp: [v_local][s]
  bf16 dVs[L][LDS_];
  float sds[4][N], extra[N], scratch[N];
  union {
    float part2[2][4][L][L + 1];                   // partial dPb dPk dMka dMab: warps 0,1 store, warps 2,3 add
    struct { float Gs[L][NP], ada[L][NP], xs[L][NP]; } fin;
  } u;
};
static_assert(sizeof(BwdSm) <= 74 * 1024, "three CTAs of the chunk backward must fit one SM");
enum { A_DPB = 0, A_DPK, A_DMKA, A_DMAB };

__device__ __forceinline__ void store_tile(float (*dst)[L + 1], const float (&c0)[4], const float (&c1)[4], int g, int tq) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int s = g + (e >> 1) * 8, t = tq * 2 + (e & 1);
    dst[s][t] = c0[e];
    dst[s][t + 8] = c1[e];
  }
}

// grid (NC, H, B)
__global__ void __launch_bounds__(NT)
wkv7_tc_bwd_chunk_kernel(const bf16* __restrict__ q_, const bf16* __restrict__ w_, const bf16* __restrict__ k_,
                         const bf16* __restrict__ v_, const bf16* __restrict__ a_, const bf16* __restrict__ b_,
                         const bf16* __restrict__ dy_, const bf16* __restrict__ chunk_states,
                         const bf16* __restrict__ dstates, const unsigned char* __restrict__ ws, bf16* __restrict__ dq_, bf16* __restrict__ dw_,
                         bf16* __restrict__ dk_, bf16* __restrict__ dv_, bf16* __restrict__ da_, bf16* __restrict__ db_,
                         int acc_qkv, int T, int H) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  BwdSm& sm = *reinterpret_cast<BwdSm*>(smem_raw);
  const int c = blockIdx.x, h = blockIdx.y, bb = blockIdx.z;
  const int NC = gridDim.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int m0 = warp * 16;
  const size_t tok_stride = (size_t)H * N;
  const size_t base = ((size_t)bb * T * H + h) * N;
  const int row = tid >> 3, part = tid & 7, j0 = part * 8;
  const size_t chunk_id = ((size_t)bb * H + h) * NC + c;

  {
    // scaled operands and the four 16x16 matrices come from the forward pass's workspace; raw v, dy, w and the
    // two 64x64 states from their own tensors
    const WsFwd* w = reinterpret_cast<const WsFwd*>(ws + chunk_id * sizeof(WsFwd));
    cp16(&sm.At[row][j0], &w->At[row][j0], true);
    cp16(&sm.Qt[row][j0], &w->Qt[row][j0], true);
    cp16(&sm.Bb[row][j0], &w->Bb[row][j0], true);
    cp16(&sm.Kb[row][j0], &w->Kb[row][j0], true);
    if (part < 2) {
      cp16(&sm.MkaT[row][j0], &w->MkaT[row][j0], true);
      cp16(&sm.PbT[row][j0], &w->PbT[row][j0], true);
      cp16(&sm.PkT[row][j0], &w->PkT[row][j0], true);
      cp16(&sm.TinvT[row][j0], &w->TinvT[row][j0], true);
    }
    if (tid < 16) cp16(&sm.gL[tid * 4], &w->gL[tid * 4], true);
    const int t = c * L + row;
    const bool live = t < T;
    const size_t off = base + (size_t)(live ? t : 0) * tok_stride + j0;
    cp16(&sm.wraw[row][j0], w_ + off, live);
    cp_commit();      // group 1: what the decay scan and the Bt / Kt rescaling need
    cp16(&sm.Vs[row][j0], v_ + off, live);
    cp16(&sm.dYs[row][j0], dy_ + off, live);
    const bf16* s0p = chunk_states + chunk_id * N * N;
    const bf16* dsp = dstates + chunk_id * N * N;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = row + 16 * i;
      cp16(&sm.S0s[r][j0], s0p + r * N + j0, true);
      cp16(&sm.dSs[r][j0], dsp + r * N + j0, true);
    }
    cp_commit();      // group 2: values, output gradient and the two 64x64 states, still in flight during the scan
  }
  // acc_qkv: this thread's tiles of the gradients already in dq / dk / dv, requested now and added in the output pass
  uint4 acc_in[3] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
  if (acc_qkv && c * L + row < T) {
    const size_t off = base + (size_t)(c * L + row) * tok_stride + j0;
    acc_in[0] = *reinterpret_cast<const uint4*>(dq_ + off);
    acc_in[1] = *reinterpret_cast<const uint4*>(dk_ + off);
    acc_in[2] = *reinterpret_cast<const uint4*>(dv_ + off);
  }
  cp_wait<1>();
  __syncthreads();
  decay_scan<false>(&sm.wraw[0][0], N, sm.E, nullptr, sm.scratch, c, T);
  {  // Bt = b / gamma_t = Bb / gamma_L, Kt likewise (thread (row, part): 8 channels of one step)
    float bbv[8], kbv[8], gl[8];
    unpack8(*reinterpret_cast<const uint4*>(&sm.Bb[row][j0]), bbv);
    unpack8(*reinterpret_cast<const uint4*>(&sm.Kb[row][j0]), kbv);
    ld8f(gl, &sm.gL[j0]);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float inv = __fdividef(1.f, gl[i]);
      bbv[i] *= inv;
      kbv[i] *= inv;
    }
    *reinterpret_cast<uint4*>(&sm.Bt[row][j0]) = pack8(bbv);
    *reinterpret_cast<uint4*>(&sm.Kt[row][j0]) = pack8(kbv);
  }
  cp_wait<0>();
  __syncthreads();

  {  // sds[q][j] = gamma_L[j] * sum over 16 value rows of S0[v][j] dS[v][j]   (d log gamma_L through the carried state)
    const int jp = tid & 31, qd = tid >> 5;
    float ax = 0.f, ay = 0.f;
#pragma unroll
    for (int vv = 0; vv < 16; ++vv) {
      const float2 s2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&sm.S0s[qd * 16 + vv][jp * 2]));
      const float2 d2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&sm.dSs[qd * 16 + vv][jp * 2]));
      ax += s2.x * d2.x; ay += s2.y * d2.y;
    }
    sm.sds[qd][jp * 2] = ax * sm.gL[jp * 2];
    sm.sds[qd][jp * 2 + 1] = ay * sm.gL[jp * 2 + 1];
  }

  // ---- value-row phase: warp owns rows [m0, m0+16)
  {
    uint32_t sa[4][4], dsa[4][4], va[4], dya[4], b[4];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      load_a(sa[kk], &sm.S0s[0][0], LDS_, m0, kk * 16, lane);
      load_a(dsa[kk], &sm.dSs[0][0], LDS_, m0, kk * 16, lane);
    }
    load_a_t(va, &sm.Vs[0][0], LDS_, 0, m0, lane);
    load_a_t(dya, &sm.dYs[0][0], LDS_, 0, m0, lane);
    float r0[4] = {0, 0, 0, 0}, r1[4] = {0, 0, 0, 0};       // R = S0 At^T + V Mka
    float du0[4] = {0, 0, 0, 0}, du1[4] = {0, 0, 0, 0};     // dU = dY Pb^T + dS Bb^T
    float dv0[4] = {0, 0, 0, 0}, dv1[4] = {0, 0, 0, 0};     // dV = dY Pk^T + dS Kb^T + dR Mka^T
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      load_b(b, &sm.At[0][0], LDS_, 0, kk * 16, lane);
      mma16816(r0, sa[kk], b[0], b[1]);
      mma16816(r1, sa[kk], b[2], b[3]);
      load_b(b, &sm.Bb[0][0], LDS_, 0, kk * 16, lane);
      mma16816(du0, dsa[kk], b[0], b[1]);
      mma16816(du1, dsa[kk], b[2], b[3]);
      load_b(b, &sm.Kb[0][0], LDS_, 0, kk * 16, lane);
      mma16816(dv0, dsa[kk], b[0], b[1]);
      mma16816(dv1, dsa[kk], b[2], b[3]);
    }
    load_b(b, &sm.MkaT[0][0], LDM, 0, 0, lane);
    mma16816(r0, va, b[0], b[1]);
    mma16816(r1, va, b[2], b[3]);
    load_b_t(b, &sm.PbT[0][0], LDM, 0, 0, lane);
    mma16816(du0, dya, b[0], b[1]);
    mma16816(du1, dya, b[2], b[3]);
    load_b_t(b, &sm.PkT[0][0], LDM, 0, 0, lane);
    mma16816(dv0, dya, b[0], b[1]);
    mma16816(dv1, dya, b[2], b[3]);
    uint32_t ra[4], dua[4], dra[4];
    float u0[4] = {0, 0, 0, 0}, u1[4] = {0, 0, 0, 0}, dr0[4] = {0, 0, 0, 0}, dr1[4] = {0, 0, 0, 0};
    acc_to_a(ra, r0, r1);
    load_b(b, &sm.TinvT[0][0], LDM, 0, 0, lane);
    mma16816(u0, ra, b[0], b[1]);
    mma16816(u1, ra, b[2], b[3]);
    acc_to_a(dua, du0, du1);
    load_b_t(b, &sm.TinvT[0][0], LDM, 0, 0, lane);
    mma16816(dr0, dua, b[0], b[1]);
    mma16816(dr1, dua, b[2], b[3]);
    acc_to_a(dra, dr0, dr1);
    load_b_t(b, &sm.MkaT[0][0], LDM, 0, 0, lane);
    mma16816(dv0, dra, b[0], b[1]);
    mma16816(dv1, dra, b[2], b[3]);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int vl = g + (e >> 1) * 8, s = tq * 2 + (e & 1);
      sm.Us[warp][vl][s] = __float2bfloat16_rn(u0[e]);
      sm.Us[warp][vl][s + 8] = __float2bfloat16_rn(u1[e]);
      sm.dRs[warp][vl][s] = __float2bfloat16_rn(dr0[e]);
      sm.dRs[warp][vl][s + 8] = __float2bfloat16_rn(dr1[e]);
      sm.dVs[s][m0 + vl] = __float2bfloat16_rn(dv0[e]);
      sm.dVs[s + 8][m0 + vl] = __float2bfloat16_rn(dv1[e]);
    }
    __syncwarp();
    // partial 16x16 sums over this warp's value rows
    uint32_t aUt[4], aV[4], bdY[4], bdR[4];
    load_a_t(aUt, &sm.Us[warp][0][0], LDM, 0, 0, lane);     // A[s][v] = U[v][s]
    load_a(aV, &sm.Vs[0][0], LDS_, 0, m0, lane);            // A[s][v] = V[s][v]
    load_b(bdY, &sm.dYs[0][0], LDS_, 0, m0, lane);          // B[v][t] = dY[t][v]
    load_b_t(bdR, &sm.dRs[warp][0][0], LDM, 0, 0, lane);    // B[v][t] = dR[v][t]
    float pc[4][2][4];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
#pragma unroll
      for (int e = 0; e < 4; ++e) pc[m][0][e] = pc[m][1][e] = 0.f;
      const uint32_t (&A_)[4] = (m == A_DPB || m == A_DMAB) ? aUt : aV;
      const uint32_t (&B_)[4] = (m == A_DPB || m == A_DPK) ? bdY : bdR;
      mma16816(pc[m][0], A_, B_[0], B_[1]);
      mma16816(pc[m][1], A_, B_[2], B_[3]);
    }
    // cross-warp sum in two rounds: warps 0,1 store their fragments, warps 2,3 add theirs at the same positions
    if (warp < 2) {
#pragma unroll
      for (int m = 0; m < 4; ++m) store_tile(sm.u.part2[warp][m], pc[m][0], pc[m][1], g, tq);
    }
    __syncthreads();
    if (warp >= 2) {
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        float (*dst)[L + 1] = sm.u.part2[warp - 2][m];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int s_ = g + (e >> 1) * 8, t_ = tq * 2 + (e & 1);
          dst[s_][t_] += pc[m][0][e];
          dst[s_][t_ + 8] += pc[m][1][e];
        }
      }
    }
  }
  __syncthreads();
  // masks (Pb, Pk: s <= t; Mka, Mab: s < t), bf16
  for (int e = tid; e < 4 * L * L; e += NT) {
    const int m = e >> 8, s_ = (e >> 4) & 15, t_ = e & 15;
    const float val = sm.u.part2[0][m][s_][t_] + sm.u.part2[1][m][s_][t_];
    const bool keep = (m == A_DPB || m == A_DPK) ? (s_ <= t_) : (s_ < t_);
    const bf16 hv = __float2bfloat16_rn(keep ? val : 0.f);
    bf16 (*dst)[LDM] = m == A_DPB ? sm.dPbN : m == A_DPK ? sm.dPkN : m == A_DMKA ? sm.dMkaN : sm.dMabN;
    dst[s_][t_] = hv;
  }
  __syncthreads();

  // q, k, a, b at this thread's output positions, requested now so that they arrive during the products below
  // (the chunk's inputs were read by the prep kernel moments ago: L2 hits)
  float2 rq[2][2], rk[2][2], ra2[2][2], rb[2][2];
  {
    auto raw2 = [&](const bf16* src, int t, int j) {
      const int tt = c * L + t;
      if (tt >= T) return make_float2(0.f, 0.f);
      return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + base + (size_t)tt * tok_stride + j));
    };
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int t = g + hh * 8, j = m0 + i * 8 + tq * 2;
        rq[i][hh] = raw2(q_, t, j);
        rk[i][hh] = raw2(k_, t, j);
        ra2[i][hh] = raw2(a_, t, j);
        rb[i][hh] = raw2(b_, t, j);
      }
  }

  // ---- key-channel phase: warp owns channels [m0, m0+16) of the six [16 x 64] gradients
  float dQt[2][4], dAt[2][4], dKt[2][4], dBt[2][4], dBb[2][4], dKb[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) dQt[i][e] = dAt[i][e] = dKt[i][e] = dBt[i][e] = dBb[i][e] = dKb[i][e] = 0.f;
  {
    uint32_t a[4], b[4];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {     // contractions over the 64 value rows
      uint32_t bS0[4], bdS[4];
      load_b_t(bS0, &sm.S0s[0][0], LDS_, kk * 16, m0, lane);
      load_b_t(bdS, &sm.dSs[0][0], LDS_, kk * 16, m0, lane);
      load_a(a, &sm.dYs[0][0], LDS_, 0, kk * 16, lane);          // A[t][v] = dY[t][v]
      mma16816(dQt[0], a, bS0[0], bS0[1]);
      mma16816(dQt[1], a, bS0[2], bS0[3]);
      load_a_t(a, &sm.dRs[kk][0][0], LDM, 0, 0, lane);           // A[t][v] = dR[v][t]
      mma16816(dAt[0], a, bS0[0], bS0[1]);
      mma16816(dAt[1], a, bS0[2], bS0[3]);
      load_a_t(a, &sm.Us[kk][0][0], LDM, 0, 0, lane);            // A[s][v] = U[v][s]
      mma16816(dBb[0], a, bdS[0], bdS[1]);
      mma16816(dBb[1], a, bdS[2], bdS[3]);
      load_a(a, &sm.Vs[0][0], LDS_, 0, kk * 16, lane);           // A[s][v] = V[s][v]
      mma16816(dKb[0], a, bdS[0], bdS[1]);
      mma16816(dKb[1], a, bdS[2], bdS[3]);
    }
    // contractions over the 16 steps
    load_b_t(b, &sm.Bt[0][0], LDS_, 0, m0, lane);
    load_a_t(a, &sm.dPbN[0][0], LDM, 0, 0, lane);
    mma16816(dQt[0], a, b[0], b[1]); mma16816(dQt[1], a, b[2], b[3]);
    load_a_t(a, &sm.dMabN[0][0], LDM, 0, 0, lane);
    mma16816(dAt[0], a, b[0], b[1]); mma16816(dAt[1], a, b[2], b[3]);
    load_b_t(b, &sm.Kt[0][0], LDS_, 0, m0, lane);
    load_a_t(a, &sm.dPkN[0][0], LDM, 0, 0, lane);
    mma16816(dQt[0], a, b[0], b[1]); mma16816(dQt[1], a, b[2], b[3]);
    load_a_t(a, &sm.dMkaN[0][0], LDM, 0, 0, lane);
    mma16816(dAt[0], a, b[0], b[1]); mma16816(dAt[1], a, b[2], b[3]);
    load_b_t(b, &sm.At[0][0], LDS_, 0, m0, lane);
    load_a(a, &sm.dMkaN[0][0], LDM, 0, 0, lane);
    mma16816(dKt[0], a, b[0], b[1]); mma16816(dKt[1], a, b[2], b[3]);
    load_a(a, &sm.dMabN[0][0], LDM, 0, 0, lane);
    mma16816(dBt[0], a, b[0], b[1]); mma16816(dBt[1], a, b[2], b[3]);
    load_b_t(b, &sm.Qt[0][0], LDS_, 0, m0, lane);
    load_a(a, &sm.dPkN[0][0], LDM, 0, 0, lane);
    mma16816(dKt[0], a, b[0], b[1]); mma16816(dKt[1], a, b[2], b[3]);
    load_a(a, &sm.dPbN[0][0], LDM, 0, 0, lane);
    mma16816(dBt[0], a, b[0], b[1]); mma16816(dBt[1], a, b[2], b[3]);
  }
  __syncthreads();   // every warp is done reading the operand arrays: reuse them as output staging

  // ---- undo the decay scaling; G = d loss / d log gamma_t
  bf16 (*odq)[LDS_] = sm.At, (*oda)[LDS_] = sm.Bt, (*odb)[LDS_] = sm.Kt, (*odk)[LDS_] = sm.Qt;
  auto st2 = [](bf16* p, float x, float y) { *reinterpret_cast<uint32_t*>(p) = pack_bf16(x, y); };
#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int t = g + hh * 8, j = m0 + i * 8 + tq * 2, e0 = hh * 2, e1 = hh * 2 + 1;
      const float2 E = *reinterpret_cast<const float2*>(&sm.E[t][j]);
      const float2 Ep = t ? *reinterpret_cast<const float2*>(&sm.E[t - 1][j]) : make_float2(1.f, 1.f);
      const float2 gl = *reinterpret_cast<const float2*>(&sm.gL[j]);
      const float2 qv = rq[i][hh], kv = rk[i][hh], av = ra2[i][hh], bv = rb[i][hh];
      const float ix = __fdividef(1.f, E.x), iy = __fdividef(1.f, E.y);
      const float lx = gl.x * ix, ly = gl.y * iy;
      const float dqx = dQt[i][e0] * E.x, dqy = dQt[i][e1] * E.y;
      const float dax = dAt[i][e0] * Ep.x, day = dAt[i][e1] * Ep.y;
      const float dbbx = dBb[i][e0] * lx, dbby = dBb[i][e1] * ly;
      const float dkbx = dKb[i][e0] * lx, dkby = dKb[i][e1] * ly;
      const float dbx = dBt[i][e0] * ix + dbbx, dby = dBt[i][e1] * iy + dbby;
      const float dkx = dKt[i][e0] * ix + dkbx, dky = dKt[i][e1] * iy + dkby;
      st2(&odq[t][j], dqx, dqy);
      st2(&oda[t][j], dax, day);
      st2(&odb[t][j], dbx, dby);
      st2(&odk[t][j], dkx, dky);
      *reinterpret_cast<float2*>(&sm.u.fin.Gs[t][j]) =
          make_float2(qv.x * dqx - bv.x * dbx - kv.x * dkx, qv.y * dqy - bv.y * dby - kv.y * dky);
      *reinterpret_cast<float2*>(&sm.u.fin.ada[t][j]) = make_float2(av.x * dax, av.y * day);
      // gamma_L enters Bb, Kb of every step
      *reinterpret_cast<float2*>(&sm.u.fin.xs[t][j]) = make_float2(bv.x * dbbx + kv.x * dkbx, bv.y * dbby + kv.y * dkby);
    }
  }
  __syncthreads();
  bf16 (*odw)[LDS_] = sm.Bb;      // free since the value-row phase
  {
    // d loss / d log-decay: suffix sums over the steps of  G_total[t] = Gs[t] + (a da)[t+1]  (gamma_t scales a_{t+1});
    // the last step also receives everything that flows through gamma_L.  Thread (channel j, half h) owns steps
    // 8h .. 8h+7 of one column: scalar, conflict-free shared-memory reads.
    const int j = tid & (N - 1), hf = tid >> 6;
    float ex = sm.sds[0][j] + sm.sds[1][j] + sm.sds[2][j] + sm.sds[3][j];
#pragma unroll
    for (int t = 0; t < L; ++t) ex += sm.u.fin.xs[t][j];
    float run = 0.f, r[8];
#pragma unroll
    for (int i = 7; i >= 0; --i) {
      const int t = hf * 8 + i;
      run += sm.u.fin.Gs[t][j] + (t + 1 < L ? sm.u.fin.ada[t + 1][j] : ex);
      r[i] = run;
    }
    if (hf) sm.scratch[j] = run;
    __syncthreads();
    const float later = hf ? 0.f : sm.scratch[j];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = hf * 8 + i;
      odw[t][j] = __float2bfloat16_rn(-__expf(__bfloat162float(sm.wraw[t][j])) * (r[i] + later));
    }
  }
  __syncthreads();
  {
    const int t = c * L + row;
    if (t < T) {
      const size_t off = base + (size_t)t * tok_stride + j0;
      *reinterpret_cast<uint4*>(dw_ + off) = *reinterpret_cast<const uint4*>(&odw[row][j0]);
      // acc_qkv: dq / dk / dv already hold another consumer's gradient of the same tensors (the bonus term of the
      // output normalisation reads r, k, v too); it is summed here instead of by a separate pass
      auto put = [&](bf16* dst, const bf16* stage, const uint4& prior) {
        uint4 val = *reinterpret_cast<const uint4*>(stage);
        if (acc_qkv) {
          float fa[8], fb[8];
          unpack8(val, fa);
          unpack8(prior, fb);
#pragma unroll
          for (int i = 0; i < 8; ++i) fa[i] += fb[i];
          val = pack8(fa);
        }
        *reinterpret_cast<uint4*>(dst) = val;
      };
      put(dq_ + off, &odq[row][j0], acc_in[0]);
      put(dk_ + off, &odk[row][j0], acc_in[1]);
      put(dv_ + off, &sm.dVs[row][j0], acc_in[2]);
      *reinterpret_cast<uint4*>(da_ + off) = *reinterpret_cast<const uint4*>(&oda[row][j0]);
      *reinterpret_cast<uint4*>(db_ + off) = *reinterpret_cast<const uint4*>(&odb[row][j0]);
    }
  }
}

}  // namespace

namespace {
template <class K>
cudaError_t set_smem(K kernel, size_t bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}
int configure_once() {
  static int status = -1;
  if (status >= 0) return status;
  cudaError_t e = set_smem(wkv7_tc_prep_kernel, sizeof(PrepSm));
  if (e == cudaSuccess) e = set_smem(wkv7_tc_scan_kernel, sizeof(ScanSm));
  if (e == cudaSuccess) e = set_smem(wkv7_tc_bwd_scan_kernel, sizeof(BScanSm));
  if (e == cudaSuccess) e = set_smem(wkv7_tc_bwd_chunk_kernel, sizeof(BwdSm));
  if (e != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)e;
  status = 0;
  return 0;
}
}  // namespace

// Bytes of the chunk-product workspace the forward fills and the backward reads.
RWKV_EXPORT long long rwkv_wkv7_tc_ws_bytes(int B, int T, int H) {
  const long long NC = (T + L - 1) / L;
  return (long long)B * H * NC * (long long)sizeof(WsFwd);
}

// q,w,k,v,a,b,y: bf16 [B,T,H,64]; s0/s_final: fp32 [B,H,64,64] or null (row = value channel, column = key
// channel); chunk_states: bf16 [B,H,ceil(T/16),64,64] or null - the state at the START of each chunk;
// ws: rwkv_wkv7_tc_ws_bytes() bytes, 16-byte aligned; it may be kept for the backward call.
RWKV_EXPORT int rwkv_wkv7_tc_forward(const void* q, const void* w, const void* k, const void* v, const void* a,
                                     const void* b, const void* s0, void* y, void* chunk_states, void* s_final,
                                     void* ws, int B, int T, int H, void* stream) {
  if (B <= 0 || T <= 0 || H <= 0 || B > 65535 || H > 65535) return RWKV_ERR_BAD_SHAPE;
  if (int rc = configure_once()) return rc;
  const int NC = (T + L - 1) / L;
  cudaStream_t st = (cudaStream_t)stream;
  wkv7_tc_prep_kernel<<<dim3(NC, H, B), NT, sizeof(PrepSm), st>>>((const bf16*)q, (const bf16*)w, (const bf16*)k,
                                                                  (const bf16*)v, (const bf16*)a, (const bf16*)b,
                                                                  (unsigned char*)ws, T, H);
  wkv7_tc_scan_kernel<<<dim3(H, B), NT, sizeof(ScanSm), st>>>((const bf16*)v, (const unsigned char*)ws, (const float*)s0,
                                                              (bf16*)y, (bf16*)chunk_states, (float*)s_final, T, H);
  return rwkv_launch_status();
}

// dy and the six gradients: bf16 [B,T,H,64]; chunk_states from the forward; ds_final (in) / ds0 (out): fp32
// [B,H,64,64] or null; dstates: scratch bf16 [B,H,ceil(T/16),64,64].
// acc_qkv = 1: dq, dk, dv are added to what the three buffers already contain.
// ws: rwkv_wkv7_tc_ws_bytes() bytes.  ws_is_forward = 1: it still holds what the forward call on the SAME inputs
// wrote (kept by the caller); ws_is_forward = 0: scratch, refilled here by the prep kernel.
RWKV_EXPORT int rwkv_wkv7_tc_backward(const void* q, const void* w, const void* k, const void* v, const void* a,
                                      const void* b, const void* dy, const void* chunk_states, const void* ds_final,
                                      void* dstates, void* ws, int ws_is_forward, void* dq, void* dw, void* dk,
                                      void* dv, void* da, void* db, void* ds0, int acc_qkv, int B, int T, int H,
                                      void* stream) {
  if (B <= 0 || T <= 0 || H <= 0 || B > 65535 || H > 65535) return RWKV_ERR_BAD_SHAPE;
  if (int rc = configure_once()) return rc;
  const int NC = (T + L - 1) / L;
  cudaStream_t st = (cudaStream_t)stream;
  if (!ws_is_forward)
    wkv7_tc_prep_kernel<<<dim3(NC, H, B), NT, sizeof(PrepSm), st>>>((const bf16*)q, (const bf16*)w, (const bf16*)k,
                                                                    (const bf16*)v, (const bf16*)a, (const bf16*)b,
                                                                    (unsigned char*)ws, T, H);
  wkv7_tc_bwd_scan_kernel<<<dim3(H, B), NT, sizeof(BScanSm), st>>>((const bf16*)dy, (const unsigned char*)ws,
                                                                   (const float*)ds_final, (bf16*)dstates, (float*)ds0,
                                                                   T, H);
  wkv7_tc_bwd_chunk_kernel<<<dim3(NC, H, B), NT, sizeof(BwdSm), st>>>(
      (const bf16*)q, (const bf16*)w, (const bf16*)k, (const bf16*)v, (const bf16*)a, (const bf16*)b, (const bf16*)dy,
      (const bf16*)chunk_states, (const bf16*)dstates, (const unsigned char*)ws, (bf16*)dq, (bf16*)dw, (bf16*)dk, (bf16*)dv, (bf16*)da,
      (bf16*)db, acc_qkv, T, H);
  return rwkv_launch_status();
}
