// Fused element-wise stages of the RWKV-7 time-mix block.
//
// prep  (between the projections and the recurrence; model.py:147-161 of the reference):
//   w    = -softplus(-(w0 + w_lin)) - 0.5
//   a    = sigmoid(a0 + a_lin)
//   v'   = v + (v_first - v) * sigmoid(v0 + v_lin)           (layers > 0)
//   kk   = normalize_per_head(k * k_k);  k' = k * (1 + (a - 1) * k_a)
//   outputs: w, k', v', -kk, kk * a
//
// post  (after the recurrence; model.py:166-170):
//   z = (GroupNorm_head(y) + (sum_n r k' r_k) v') * g
//
// Thread i owns channels [8i, 8i+8) of a strip of time steps; the 8 threads of a head
// reduce with three shuffles.  Backward kernels recompute the cheap intermediates instead
// of reading saved copies and leave per-CTA partial sums of the parameter gradients.
#include "elementwise.cuh"

namespace {

__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

struct PrepParams {
  float w0[8], a0[8], v0[8], kk[8], ka[8];
};

__global__ void __launch_bounds__(512)
timemix_prep_fwd_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v, const bf16* __restrict__ vfirst,
                        const bf16* __restrict__ wlin, const bf16* __restrict__ alin, const bf16* __restrict__ vlin,
                        const float* __restrict__ w0, const float* __restrict__ a0, const float* __restrict__ v0,
                        const float* __restrict__ k_k, const float* __restrict__ k_a, bf16* __restrict__ w_out,
                        bf16* __restrict__ k_out, bf16* __restrict__ v_out, bf16* __restrict__ an_out,
                        bf16* __restrict__ b_out, int T, int C, int strip) {
  rwkv_chain_trigger();
  const RowCtx rc = make_row_ctx(T, C, strip);
  PrepParams p;
#pragma unroll
  for (int e = 0; e < 8; ++e) p.w0[e] = p.a0[e] = p.v0[e] = p.kk[e] = p.ka[e] = 0.f;
  if (rc.active) {
    load8f(w0 + rc.col, p.w0);
    load8f(a0 + rc.col, p.a0);
    if (vfirst) load8f(v0 + rc.col, p.v0);
    load8f(k_k + rc.col, p.kk);
    load8f(k_a + rc.col, p.ka);
  }
  rwkv_chain_wait();   // parameters before, activations after (see common.cuh)
  for (int t = rc.t0; t < rc.t1; ++t) {
    const size_t off = ((size_t)rc.b * T + t) * C + rc.col;
    float kf[8] = {0, 0, 0, 0, 0, 0, 0, 0}, vf[8], wl[8], al[8];
    if (rc.active) {
      unpack8(ldg16(k + off), kf);
      unpack8(ldg16(v + off), vf);
      unpack8(ldg16(wlin + off), wl);
      unpack8(ldg16(alin + off), al);
    }
    float nrm2 = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) nrm2 += (kf[e] * p.kk[e]) * (kf[e] * p.kk[e]);
    nrm2 = head_sum(nrm2);
    if (!rc.active) continue;
    const float inv = 1.f / fmaxf(sqrtf(nrm2), 1e-12f);
    float wo[8], ko[8], ano[8], bo[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      wo[e] = -softplusf_(-(p.w0[e] + wl[e])) - 0.5f;
      const float a = sigmoidf_(p.a0[e] + al[e]);
      const float kkn = kf[e] * p.kk[e] * inv;
      ko[e] = kf[e] * (1.f + (a - 1.f) * p.ka[e]);
      ano[e] = -kkn;
      bo[e] = kkn * a;
    }
    if (vfirst) {
      float v1[8], vl[8];
      unpack8(ldg16(vfirst + off), v1);
      unpack8(ldg16(vlin + off), vl);
#pragma unroll
      for (int e = 0; e < 8; ++e) vf[e] = vf[e] + (v1[e] - vf[e]) * sigmoidf_(p.v0[e] + vl[e]);
      stg16(v_out + off, pack8(vf));
    }
    stg16(w_out + off, pack8(wo));
    stg16(k_out + off, pack8(ko));
    stg16(an_out + off, pack8(ano));
    stg16(b_out + off, pack8(bo));
  }
}

// partials [nCTA][5][C]: dw0, da0, dv0, dk_k, dk_a
__global__ void __launch_bounds__(512)
timemix_prep_bwd_kernel(const bf16* __restrict__ gw, const bf16* __restrict__ gk, const bf16* __restrict__ gv,
                        const bf16* __restrict__ gan, const bf16* __restrict__ gb, const bf16* __restrict__ k,
                        const bf16* __restrict__ v, const bf16* __restrict__ vfirst, const bf16* __restrict__ wlin,
                        const bf16* __restrict__ alin, const bf16* __restrict__ vlin, const float* __restrict__ w0,
                        const float* __restrict__ a0, const float* __restrict__ v0, const float* __restrict__ k_k,
                        const float* __restrict__ k_a, bf16* __restrict__ dk, bf16* __restrict__ dv,
                        bf16* __restrict__ dvfirst, bf16* __restrict__ dwlin, bf16* __restrict__ dalin,
                        bf16* __restrict__ dvlin, float* __restrict__ partials, int T, int C, int strip) {
  const RowCtx rc = make_row_ctx(T, C, strip);
  PrepParams p;
  float acc[5][8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    p.w0[e] = p.a0[e] = p.v0[e] = p.kk[e] = p.ka[e] = 0.f;
#pragma unroll
    for (int i = 0; i < 5; ++i) acc[i][e] = 0.f;
  }
  if (rc.active) {
    load8f(w0 + rc.col, p.w0);
    load8f(a0 + rc.col, p.a0);
    if (vfirst) load8f(v0 + rc.col, p.v0);
    load8f(k_k + rc.col, p.kk);
    load8f(k_a + rc.col, p.ka);
  }
  for (int t = rc.t0; t < rc.t1; ++t) {
    const size_t off = ((size_t)rc.b * T + t) * C + rc.col;
    // every tile of this row is requested up front: one memory round trip per row instead of three
    const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
    const bool on = rc.active;
    const uint4 q_k = on ? ldg16(k + off) : z4, q_al = on ? ldg16(alin + off) : z4;
    const uint4 q_gan = on ? ldg16(gan + off) : z4, q_gb = on ? ldg16(gb + off) : z4;
    const uint4 q_gk = on ? ldg16(gk + off) : z4, q_gw = on ? ldg16(gw + off) : z4, q_wl = on ? ldg16(wlin + off) : z4;
    const uint4 q_gv = on ? ldg16(gv + off) : z4;
    const bool mixv = on && vfirst != nullptr;
    const uint4 q_v = mixv ? ldg16(v + off) : z4, q_vf = mixv ? ldg16(vfirst + off) : z4;
    const uint4 q_vl = mixv ? ldg16(vlin + off) : z4;
    float kf[8], al[8], g_an[8], g_b[8];
    unpack8(q_k, kf);
    unpack8(q_al, al);
    unpack8(q_gan, g_an);
    unpack8(q_gb, g_b);
    float a[8], kr[8], dkk[8];
    float nrm2 = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      a[e] = sigmoidf_(p.a0[e] + al[e]);
      kr[e] = kf[e] * p.kk[e];
      nrm2 += kr[e] * kr[e];
      dkk[e] = -g_an[e] + g_b[e] * a[e];
    }
    nrm2 = head_sum(nrm2);
    const float inv = 1.f / fmaxf(sqrtf(nrm2), 1e-12f);
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) dot += kr[e] * inv * dkk[e];
    dot = head_sum(dot);
    if (!rc.active) continue;
    float g_k[8], g_w[8], wl[8];
    unpack8(q_gk, g_k);
    unpack8(q_gw, g_w);
    unpack8(q_wl, wl);
    float o_dk[8], o_dw[8], o_da[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float kkn = kr[e] * inv;
      const float dkr = (dkk[e] - kkn * dot) * inv;
      const float modf = 1.f + (a[e] - 1.f) * p.ka[e];
      o_dk[e] = dkr * p.kk[e] + g_k[e] * modf;
      acc[3][e] += dkr * kf[e];
      acc[4][e] += g_k[e] * kf[e] * (a[e] - 1.f);
      const float da = g_b[e] * kkn + g_k[e] * kf[e] * p.ka[e];
      o_da[e] = da * a[e] * (1.f - a[e]);
      acc[1][e] += o_da[e];
      o_dw[e] = g_w[e] * sigmoidf_(-(p.w0[e] + wl[e]));
      acc[0][e] += o_dw[e];
    }
    stg16(dk + off, pack8(o_dk));
    stg16(dwlin + off, pack8(o_dw));
    stg16(dalin + off, pack8(o_da));
    float g_v[8];
    unpack8(q_gv, g_v);
    if (vfirst) {
      float vf[8], v1[8], vl[8], o_dv[8], o_dvf[8], o_dvl[8];
      unpack8(q_v, vf);
      unpack8(q_vf, v1);
      unpack8(q_vl, vl);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float s = sigmoidf_(p.v0[e] + vl[e]);
        o_dv[e] = g_v[e] * (1.f - s);
        o_dvf[e] = g_v[e] * s;
        o_dvl[e] = g_v[e] * (v1[e] - vf[e]) * s * (1.f - s);
        acc[2][e] += o_dvl[e];
      }
      stg16(dv + off, pack8(o_dv));
      stg16(dvfirst + off, pack8(o_dvf));
      stg16(dvlin + off, pack8(o_dvl));
    } else {
      stg16(dv + off, pack8(g_v));
    }
  }
  if (rc.active) {
    float* pp = partials + ((size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 5) * C + rc.col;
#pragma unroll
    for (int i = 0; i < 5; ++i) store8f(pp + (size_t)i * C, acc[i]);
  }
}

__global__ void __launch_bounds__(512)
gn_bonus_gate_fwd_kernel(const bf16* __restrict__ y, const bf16* __restrict__ r, const bf16* __restrict__ k,
                         const bf16* __restrict__ v, const bf16* __restrict__ g, const float* __restrict__ gn_w,
                         const float* __restrict__ gn_b, const float* __restrict__ r_k, bf16* __restrict__ z, int T,
                         int C, int strip, float eps) {
  rwkv_chain_trigger();
  const RowCtx rc = make_row_ctx(T, C, strip);
  float gw[8] = {0, 0, 0, 0, 0, 0, 0, 0}, gb[8] = {0, 0, 0, 0, 0, 0, 0, 0}, rk[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (rc.active) { load8f(gn_w + rc.col, gw); load8f(gn_b + rc.col, gb); load8f(r_k + rc.col, rk); }
  rwkv_chain_wait();   // parameters before, activations after (see common.cuh)
  for (int t = rc.t0; t < rc.t1; ++t) {
    const size_t off = ((size_t)rc.b * T + t) * C + rc.col;
    float yf[8] = {0, 0, 0, 0, 0, 0, 0, 0}, rf[8] = {0, 0, 0, 0, 0, 0, 0, 0}, kf[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (rc.active) {
      unpack8(ldg16(y + off), yf);
      unpack8(ldg16(r + off), rf);
      unpack8(ldg16(k + off), kf);
    }
    float s = 0.f, bonus = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) { s += yf[e]; bonus += rf[e] * kf[e] * rk[e]; }
    s = head_sum(s);
    bonus = head_sum(bonus);
    const float mean = s * (1.f / 64.f);
    float q = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) q += (yf[e] - mean) * (yf[e] - mean);
    q = head_sum(q);
    if (!rc.active) continue;
    const float rstd = rsqrtf(q * (1.f / 64.f) + eps);
    float vf[8], gf[8], o[8];
    unpack8(ldg16(v + off), vf);
    unpack8(ldg16(g + off), gf);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = ((yf[e] - mean) * rstd * gw[e] + gb[e] + bonus * vf[e]) * gf[e];
    stg16(z + off, pack8(o));
  }
}

// partials [nCTA][3][C]: dgn_w, dgn_b, dr_k
__global__ void __launch_bounds__(512)
gn_bonus_gate_bwd_kernel(const bf16* __restrict__ dz, const bf16* __restrict__ y, const bf16* __restrict__ r,
                         const bf16* __restrict__ k, const bf16* __restrict__ v, const bf16* __restrict__ g,
                         const float* __restrict__ gn_w, const float* __restrict__ gn_b,
                         const float* __restrict__ r_k, bf16* __restrict__ dy, bf16* __restrict__ dr,
                         bf16* __restrict__ dk, bf16* __restrict__ dv, bf16* __restrict__ dg,
                         float* __restrict__ partials, int T, int C, int strip, float eps) {
  const RowCtx rc = make_row_ctx(T, C, strip);
  float gw[8] = {0, 0, 0, 0, 0, 0, 0, 0}, gb[8] = {0, 0, 0, 0, 0, 0, 0, 0}, rk[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float acc[3][8];
#pragma unroll
  for (int i = 0; i < 3; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
  if (rc.active) { load8f(gn_w + rc.col, gw); load8f(gn_b + rc.col, gb); load8f(r_k + rc.col, rk); }
  for (int t = rc.t0; t < rc.t1; ++t) {
    const size_t off = ((size_t)rc.b * T + t) * C + rc.col;
    float yf[8] = {0, 0, 0, 0, 0, 0, 0, 0}, rf[8] = {0, 0, 0, 0, 0, 0, 0, 0}, kf[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float vf[8] = {0, 0, 0, 0, 0, 0, 0, 0}, gf[8] = {0, 0, 0, 0, 0, 0, 0, 0}, dzf[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (rc.active) {
      unpack8(ldg16(y + off), yf);
      unpack8(ldg16(r + off), rf);
      unpack8(ldg16(k + off), kf);
      unpack8(ldg16(v + off), vf);
      unpack8(ldg16(g + off), gf);
      unpack8(ldg16(dz + off), dzf);
    }
    float s = 0.f, bonus = 0.f, drk = 0.f;
    float du[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      du[e] = dzf[e] * gf[e];
      s += yf[e];
      bonus += rf[e] * kf[e] * rk[e];
      drk += du[e] * vf[e];
    }
    s = head_sum(s);
    bonus = head_sum(bonus);
    drk = head_sum(drk);
    const float mean = s * (1.f / 64.f);
    float q = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) q += (yf[e] - mean) * (yf[e] - mean);
    q = head_sum(q);
    const float rstd = rsqrtf(q * (1.f / 64.f) + eps);
    float xh[8], c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      xh[e] = (yf[e] - mean) * rstd;
      const float gg = du[e] * gw[e];
      c1 += gg;
      c2 += gg * xh[e];
    }
    c1 = head_sum(c1) * (1.f / 64.f);
    c2 = head_sum(c2) * (1.f / 64.f);
    if (!rc.active) continue;
    float o_dy[8], o_dr[8], o_dk[8], o_dv[8], o_dg[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      o_dy[e] = rstd * (du[e] * gw[e] - c1 - xh[e] * c2);
      o_dr[e] = drk * kf[e] * rk[e];
      o_dk[e] = drk * rf[e] * rk[e];
      o_dv[e] = du[e] * bonus;
      o_dg[e] = dzf[e] * (xh[e] * gw[e] + gb[e] + bonus * vf[e]);
      acc[0][e] += du[e] * xh[e];
      acc[1][e] += du[e];
      acc[2][e] += drk * rf[e] * kf[e];
    }
    stg16(dy + off, pack8(o_dy));
    stg16(dr + off, pack8(o_dr));
    stg16(dk + off, pack8(o_dk));
    stg16(dv + off, pack8(o_dv));
    stg16(dg + off, pack8(o_dg));
  }
  if (rc.active) {
    float* pp = partials + ((size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 3) * C + rc.col;
#pragma unroll
    for (int i = 0; i < 3; ++i) store8f(pp + (size_t)i * C, acc[i]);
  }
}

// relu(x)^2 and its backward (2 * relu(x) * dy), 8 elements per thread
__global__ void relu_sq_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, size_t n8) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(ldg16(x + i * 8), f);
#pragma unroll
    for (int e = 0; e < 8; ++e) { const float r = fmaxf(f[e], 0.f); f[e] = r * r; }
    stg16(y + i * 8, pack8(f));
  }
}
// from_output = 1: the first argument is y = relu(x)^2 (what the fused GEMM epilogue stored) and relu(x) = sqrt(y)
__global__ void relu_sq_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy, bf16* __restrict__ dx,
                                   size_t n8, int from_output) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float f[8], g[8];
    unpack8(ldg16(x + i * 8), f);
    unpack8(ldg16(dy + i * 8), g);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = 2.f * (from_output ? sqrtf(fmaxf(f[e], 0.f)) : fmaxf(f[e], 0.f)) * g[e];
    stg16(dx + i * 8, pack8(f));
  }
}

inline int threads_for(int C) { return ((C / 8 + 31) / 32) * 32; }
inline bool shape_ok(int B, int T, int C, int strip) {
  return C % 64 == 0 && C / 8 <= 512 && strip > 0 && B > 0 && B <= 65535 && T > 0;
}

}  // namespace

RWKV_EXPORT int rwkv_timemix_prep_forward(const void* k, const void* v, const void* vfirst, const void* wlin,
                                          const void* alin, const void* vlin, const void* w0, const void* a0,
                                          const void* v0, const void* k_k, const void* k_a, void* w_out,
                                          void* k_out, void* v_out, void* an_out, void* b_out, int B, int T, int C,
                                          int strip, void* stream) {
  if (!shape_ok(B, T, C, strip)) return RWKV_ERR_BAD_SHAPE;
  dim3 grid((T + strip - 1) / strip, B);
  rwkv_launch(timemix_prep_fwd_kernel, grid, dim3(threads_for(C)), 0, (cudaStream_t)stream,
      (const bf16*)k, (const bf16*)v, (const bf16*)vfirst, (const bf16*)wlin, (const bf16*)alin, (const bf16*)vlin,
      (const float*)w0, (const float*)a0, (const float*)v0, (const float*)k_k, (const float*)k_a, (bf16*)w_out,
      (bf16*)k_out, (bf16*)v_out, (bf16*)an_out, (bf16*)b_out, T, C, strip);
  return rwkv_launch_status();
}

RWKV_EXPORT int rwkv_timemix_prep_backward(const void* gw, const void* gk, const void* gv, const void* gan,
                                           const void* gb, const void* k, const void* v, const void* vfirst,
                                           const void* wlin, const void* alin, const void* vlin, const void* w0,
                                           const void* a0, const void* v0, const void* k_k, const void* k_a,
                                           void* dk, void* dv, void* dvfirst, void* dwlin, void* dalin, void* dvlin,
                                           void* partials, int B, int T, int C, int strip, void* stream) {
  if (!shape_ok(B, T, C, strip)) return RWKV_ERR_BAD_SHAPE;
  dim3 grid((T + strip - 1) / strip, B);
  timemix_prep_bwd_kernel<<<grid, threads_for(C), 0, (cudaStream_t)stream>>>(
      (const bf16*)gw, (const bf16*)gk, (const bf16*)gv, (const bf16*)gan, (const bf16*)gb, (const bf16*)k,
      (const bf16*)v, (const bf16*)vfirst, (const bf16*)wlin, (const bf16*)alin, (const bf16*)vlin,
      (const float*)w0, (const float*)a0, (const float*)v0, (const float*)k_k, (const float*)k_a, (bf16*)dk,
      (bf16*)dv, (bf16*)dvfirst, (bf16*)dwlin, (bf16*)dalin, (bf16*)dvlin, (float*)partials, T, C, strip);
  return rwkv_launch_status();
}

RWKV_EXPORT int rwkv_gn_bonus_gate_forward(const void* y, const void* r, const void* k, const void* v,
                                           const void* g, const void* gn_w, const void* gn_b, const void* r_k,
                                           void* z, int B, int T, int C, int strip, float eps, void* stream) {
  if (!shape_ok(B, T, C, strip)) return RWKV_ERR_BAD_SHAPE;
  dim3 grid((T + strip - 1) / strip, B);
  rwkv_launch(gn_bonus_gate_fwd_kernel, grid, dim3(threads_for(C)), 0, (cudaStream_t)stream,
      (const bf16*)y, (const bf16*)r, (const bf16*)k, (const bf16*)v, (const bf16*)g, (const float*)gn_w,
      (const float*)gn_b, (const float*)r_k, (bf16*)z, T, C, strip, eps);
  return rwkv_launch_status();
}

RWKV_EXPORT int rwkv_gn_bonus_gate_backward(const void* dz, const void* y, const void* r, const void* k,
                                            const void* v, const void* g, const void* gn_w, const void* gn_b,
                                            const void* r_k, void* dy, void* dr, void* dk, void* dv, void* dg,
                                            void* partials, int B, int T, int C, int strip, float eps,
                                            void* stream) {
  if (!shape_ok(B, T, C, strip)) return RWKV_ERR_BAD_SHAPE;
  dim3 grid((T + strip - 1) / strip, B);
  gn_bonus_gate_bwd_kernel<<<grid, threads_for(C), 0, (cudaStream_t)stream>>>(
      (const bf16*)dz, (const bf16*)y, (const bf16*)r, (const bf16*)k, (const bf16*)v, (const bf16*)g,
      (const float*)gn_w, (const float*)gn_b, (const float*)r_k, (bf16*)dy, (bf16*)dr, (bf16*)dk, (bf16*)dv,
      (bf16*)dg, (float*)partials, T, C, strip, eps);
  return rwkv_launch_status();
}

RWKV_EXPORT int rwkv_relu_sq_forward(const void* x, void* y, long long n, void* stream) {
  if (n % 8) return RWKV_ERR_BAD_SHAPE;
  const size_t n8 = (size_t)n / 8;
  const int blocks = (int)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
  relu_sq_fwd_kernel<<<blocks > 0 ? blocks : 1, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, n8);
  return rwkv_launch_status();
}

RWKV_EXPORT int rwkv_relu_sq_backward(const void* x, const void* dy, void* dx, long long n, int from_output,
                                      void* stream) {
  if (n % 8) return RWKV_ERR_BAD_SHAPE;
  const size_t n8 = (size_t)n / 8;
  const int blocks = (int)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
  relu_sq_bwd_kernel<<<blocks > 0 ? blocks : 1, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (const bf16*)dy,
                                                                               (bf16*)dx, n8, from_output);
  return rwkv_launch_status();
}
