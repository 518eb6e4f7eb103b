// LayerNorm + token shift + K-way lerp in one pass over the residual stream (forward and
// backward), and a plain LayerNorm built from the same pieces.
//
//   h = LN(x);  out_k[t] = h[t] + (h[t-1] - h[t]) * mix_k     (h[-1] = carried row or 0)
//
// The reference runs this as LayerNorm, ZeroPad2d, a subtraction and six multiply-adds,
// each a separate pass over [B,T,C] (model.py:138-144, :305-306, :373).  Here x is read once
// and the K outputs are written once.  h is rounded to bf16 before it is mixed, so a
// sequence processed in chunks with the carried row gives bit-identical results.
#include <stdlib.h>

#include "elementwise.cuh"

namespace {

template <int K>
__global__ void __launch_bounds__(512)
ln_shift_mix_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ ln_w, const float* __restrict__ ln_b,
                        const float* __restrict__ mix, const bf16* __restrict__ prev, bf16* __restrict__ outs,
                        bf16* __restrict__ last, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                        int B, int T, int C, int strip, float eps) {
  __shared__ float red[2 * EW_MAX_WARPS * 4];
  rwkv_chain_trigger();
  int phase = 0;
  const RowCtx rc = make_row_ctx(T, C, strip);
  const size_t row0 = (size_t)rc.b * T;
  const size_t plane = (size_t)B * T * C;
  const float invC = 1.f / C;

  float w[8], bb[8], mu[K][8], hprev[8];
  if (rc.active) {
    load8f(ln_w + rc.col, w);
    load8f(ln_b + rc.col, bb);
#pragma unroll
    for (int k = 0; k < K; ++k) load8f(mix + (size_t)k * C + rc.col, mu[k]);
  }
  // parameters (constant while launches are chained) are requested before the predecessor kernel has finished,
  // activations after
  rwkv_chain_wait();
#pragma unroll
  for (int e = 0; e < 8; ++e) hprev[e] = 0.f;

  // halo: h of the row before the strip
  if (rc.t0 == 0) {
    if (prev && rc.active) unpack8(ldg16(prev + (size_t)rc.b * C + rc.col), hprev);
  } else {
    float xf[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (rc.active) unpack8(ldg16(x + (row0 + rc.t0 - 1) * C + rc.col), xf);
    float s[1] = {0.f};
#pragma unroll
    for (int e = 0; e < 8; ++e) s[0] += xf[e];
    block_sum<1>(s, red, phase);
    const float mean = s[0] * invC;
    float q[1] = {0.f};
    if (rc.active) {
#pragma unroll
      for (int e = 0; e < 8; ++e) q[0] += (xf[e] - mean) * (xf[e] - mean);
    }
    block_sum<1>(q, red, phase);
    const float rstd = rsqrtf(q[0] * invC + eps);
#pragma unroll
    for (int e = 0; e < 8; ++e) hprev[e] = round_bf16((xf[e] - mean) * rstd * w[e] + bb[e]);
  }

  // raw tiles of the next four rows are fetched before the reductions of the current four
  uint4 xq[4];
  auto fetch4 = [&](int tg) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = tg + i;
      xq[i] = (t < rc.t1 && rc.active) ? ldg16(x + (row0 + t) * C + rc.col) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  fetch4(rc.t0);
  for (int tg = rc.t0; tg < rc.t1; tg += 4) {
    float xf[4][8];
    float s[4], q[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s[i] = 0.f;
      unpack8(xq[i], xf[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) s[i] += xf[i][e];
    }
    if (tg + 4 < rc.t1) fetch4(tg + 4);
    block_sum<4>(s, red, phase);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s[i] *= invC;
      q[i] = 0.f;
      if (rc.active) {
#pragma unroll
        for (int e = 0; e < 8; ++e) q[i] += (xf[i][e] - s[i]) * (xf[i][e] - s[i]);
      }
    }
    block_sum<4>(q, red, phase);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = tg + i;
      if (t >= rc.t1) break;
      const float rstd = rsqrtf(q[i] * invC + eps);
      if (threadIdx.x == 0 && mean_out) {
        mean_out[row0 + t] = s[i];
        rstd_out[row0 + t] = rstd;
      }
      if (rc.active) {
        float hcur[8], o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) hcur[e] = round_bf16((xf[i][e] - s[i]) * rstd * w[e] + bb[e]);
#pragma unroll
        for (int k = 0; k < K; ++k) {
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = hcur[e] + (hprev[e] - hcur[e]) * mu[k][e];
          stg16(outs + (size_t)k * plane + (row0 + t) * C + rc.col, pack8(o));
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) hprev[e] = hcur[e];
      }
    }
  }
  if (last && rc.t1 == T && rc.active) stg16(last + (size_t)rc.b * C + rc.col, pack8(hprev));
}

// Backward.  Walks the strip in reverse; `carry` holds sum_k dO_k[t+1]*mix_k.  Emits dx, the
// gradient of the carried row (dprev) and per-CTA partial sums of the parameter gradients in
// `partials` [gridDim.y*gridDim.x][K+2][C]: rows 0..K-1 = dmix, K = dln_w, K+1 = dln_b.
struct DOutPtrs { const bf16* p[6]; };   // the K output gradients may live in separate allocations

template <int K>
__global__ void __launch_bounds__(512)
ln_shift_mix_bwd_kernel(const DOutPtrs dO, const bf16* __restrict__ dlast, const bf16* __restrict__ dres,
                        const bf16* __restrict__ x,
                        const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                        const float* __restrict__ ln_w, const float* __restrict__ ln_b,
                        const float* __restrict__ mix, const bf16* __restrict__ prev, bf16* __restrict__ dx,
                        float* __restrict__ dprev, float* __restrict__ partials, int B, int T, int C, int strip) {
  __shared__ float red[2 * EW_MAX_WARPS * 2];
  int phase = 0;
  const RowCtx rc = make_row_ctx(T, C, strip);
  const size_t row0 = (size_t)rc.b * T;
  const float invC = 1.f / C;

  float w[8], bb[8], mu[K][8];
  float acc_mu[K][8], acc_w[8], acc_b[8], carry[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    w[e] = bb[e] = 0.f;
    acc_w[e] = acc_b[e] = carry[e] = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) { acc_mu[k][e] = 0.f; mu[k][e] = 0.f; }
  }
  if (rc.active) {
    load8f(ln_w + rc.col, w);
    load8f(ln_b + rc.col, bb);
#pragma unroll
    for (int k = 0; k < K; ++k) load8f(mix + (size_t)k * C + rc.col, mu[k]);
    if (rc.t1 < T) {   // halo: contribution of the row after the strip
#pragma unroll
      for (int k = 0; k < K; ++k) {
        float g[8];
        unpack8(ldg16(dO.p[k] + (row0 + rc.t1) * C + rc.col), g);
#pragma unroll
        for (int e = 0; e < 8; ++e) carry[e] += g[e] * mu[k][e];
      }
    } else if (dlast) {
      float g[8];
      unpack8(ldg16(dlast + (size_t)rc.b * C + rc.col), g);
#pragma unroll
      for (int e = 0; e < 8; ++e) carry[e] += g[e];
    }
  }

  // h of row t (recomputed exactly as the forward rounded it)
  auto h_of_row = [&](int t, float* xh, float* h) {
    if (t < 0) {
#pragma unroll
      for (int e = 0; e < 8; ++e) { xh[e] = 0.f; h[e] = 0.f; }
      if (prev && rc.active) unpack8(ldg16(prev + (size_t)rc.b * C + rc.col), h);
      return;
    }
    float xf[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (rc.active) unpack8(ldg16(x + (row0 + t) * C + rc.col), xf);
    const float m = mean_in[row0 + t], r = rstd_in[row0 + t];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      xh[e] = (xf[e] - m) * r;
      h[e] = round_bf16(xh[e] * w[e] + bb[e]);
    }
  };

  float xh_cur[8], h_cur[8], xh_prev[8], h_prev[8];
  h_of_row(rc.t1 - 1, xh_cur, h_cur);
  for (int t = rc.t1 - 1; t >= rc.t0; --t) {
    h_of_row(t - 1, xh_prev, h_prev);
    float dh[8], ncarry[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { dh[e] = carry[e]; ncarry[e] = 0.f; }
    if (rc.active) {
#pragma unroll
      for (int k = 0; k < K; ++k) {
        float g[8];
        unpack8(ldg16(dO.p[k] + (row0 + t) * C + rc.col), g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          dh[e] += g[e] * (1.f - mu[k][e]);
          ncarry[e] += g[e] * mu[k][e];
          acc_mu[k][e] += g[e] * (h_prev[e] - h_cur[e]);
        }
      }
    }
    float c[2] = {0.f, 0.f};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float g = dh[e] * w[e];
      c[0] += g;
      c[1] += g * xh_cur[e];
      acc_w[e] += dh[e] * xh_cur[e];
      acc_b[e] += dh[e];
    }
    block_sum<2>(c, red, phase);
    if (rc.active) {
      const float r = rstd_in[row0 + t];
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = r * (dh[e] * w[e] - c[0] * invC - xh_cur[e] * c[1] * invC);
      if (dres) {   // gradient arriving through the residual connection around this LayerNorm
        float rr[8];
        unpack8(ldg16(dres + (row0 + t) * C + rc.col), rr);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += rr[e];
      }
      stg16(dx + (row0 + t) * C + rc.col, pack8(o));
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      carry[e] = ncarry[e];
      xh_cur[e] = xh_prev[e];
      h_cur[e] = h_prev[e];
    }
  }
  if (rc.active) {
    if (dprev && rc.t0 == 0) store8f(dprev + (size_t)rc.b * C + rc.col, carry);
    float* p = partials + ((size_t)(blockIdx.y * gridDim.x + blockIdx.x) * (K + 2)) * C + rc.col;
#pragma unroll
    for (int k = 0; k < K; ++k) store8f(p + (size_t)k * C, acc_mu[k]);
    store8f(p + (size_t)K * C, acc_w);
    store8f(p + (size_t)(K + 1) * C, acc_b);
  }
}

// Plain LayerNorm over the last dimension of a [rows, C] tensor, `strip` rows per CTA.
__global__ void __launch_bounds__(512)
layer_norm_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ ln_w, const float* __restrict__ ln_b,
                      bf16* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows,
                      int C, int strip, float eps) {
  __shared__ float red[2 * EW_MAX_WARPS * 4];
  rwkv_chain_begin();
  int phase = 0;
  const int col = threadIdx.x * 8;
  const bool active = col < C;
  const int r0 = blockIdx.x * strip, r1 = min(rows, r0 + strip);
  const float invC = 1.f / C;
  float w[8] = {0, 0, 0, 0, 0, 0, 0, 0}, bb[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (active) { load8f(ln_w + col, w); load8f(ln_b + col, bb); }
  for (int rg = r0; rg < r1; rg += 4) {
    float xf[4][8], s[4], q[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s[i] = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) xf[i][e] = 0.f;
      if (rg + i < r1 && active) {
        unpack8(ldg16(x + (size_t)(rg + i) * C + col), xf[i]);
#pragma unroll
        for (int e = 0; e < 8; ++e) s[i] += xf[i][e];
      }
    }
    block_sum<4>(s, red, phase);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s[i] *= invC;
      q[i] = 0.f;
      if (active) {
#pragma unroll
        for (int e = 0; e < 8; ++e) q[i] += (xf[i][e] - s[i]) * (xf[i][e] - s[i]);
      }
    }
    block_sum<4>(q, red, phase);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = rg + i;
      if (r >= r1) break;
      const float rstd = rsqrtf(q[i] * invC + eps);
      if (threadIdx.x == 0 && mean_out) { mean_out[r] = s[i]; rstd_out[r] = rstd; }
      if (active) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (xf[i][e] - s[i]) * rstd * w[e] + bb[e];
        stg16(y + (size_t)r * C + col, pack8(o));
      }
    }
  }
}

// partials: [gridDim.x][2][C] (dln_w, dln_b)
__global__ void __launch_bounds__(512)
layer_norm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const float* __restrict__ mean_in,
                      const float* __restrict__ rstd_in, const float* __restrict__ ln_w, bf16* __restrict__ dx,
                      float* __restrict__ partials, int rows, int C, int strip) {
  __shared__ float red[2 * EW_MAX_WARPS * 2];
  int phase = 0;
  const int col = threadIdx.x * 8;
  const bool active = col < C;
  const int r0 = blockIdx.x * strip, r1 = min(rows, r0 + strip);
  const float invC = 1.f / C;
  float w[8] = {0, 0, 0, 0, 0, 0, 0, 0}, acc_w[8] = {0, 0, 0, 0, 0, 0, 0, 0}, acc_b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (active) load8f(ln_w + col, w);
  for (int r = r0; r < r1; ++r) {
    float g[8] = {0, 0, 0, 0, 0, 0, 0, 0}, xh[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const float m = mean_in[r], rs = rstd_in[r];
    if (active) {
      float xf[8];
      unpack8(ldg16(dy + (size_t)r * C + col), g);
      unpack8(ldg16(x + (size_t)r * C + col), xf);
#pragma unroll
      for (int e = 0; e < 8; ++e) xh[e] = (xf[e] - m) * rs;
    }
    float c[2] = {0.f, 0.f};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      c[0] += g[e] * w[e];
      c[1] += g[e] * w[e] * xh[e];
      acc_w[e] += g[e] * xh[e];
      acc_b[e] += g[e];
    }
    block_sum<2>(c, red, phase);
    if (active) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = rs * (g[e] * w[e] - c[0] * invC - xh[e] * c[1] * invC);
      stg16(dx + (size_t)r * C + col, pack8(o));
    }
  }
  if (active) {
    float* p = partials + (size_t)blockIdx.x * 2 * C + col;
    store8f(p, acc_w);
    store8f(p + C, acc_b);
  }
}

__device__ __forceinline__ void unpack4(const uint2& p, float* f) {
  f[0] = bf16_lo(p.x); f[1] = bf16_hi(p.x); f[2] = bf16_lo(p.y); f[3] = bf16_hi(p.y);
}
__device__ __forceinline__ uint2 pack4(const float* f) { return make_uint2(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3])); }
__device__ __forceinline__ void load4f(const float* p, float* f) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
}
__device__ __forceinline__ void store4f(float* p, const float* f) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}

// Same backward with four channels per thread (C/4 threads): the K mix coefficients and the K+2 parameter-gradient
// accumulators then take half the registers, which leaves room to fetch the next row's K gradient tiles before
// the block reduction of the current row.  Same `partials` layout as the kernel above.
template <int K>
__global__ void __launch_bounds__(512)
ln_shift_mix_bwd_v4_kernel(const DOutPtrs dO, const bf16* __restrict__ dlast, const bf16* __restrict__ dres,
                           const bf16* __restrict__ x,
                           const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                           const float* __restrict__ ln_w, const float* __restrict__ ln_b,
                           const float* __restrict__ mix, const bf16* __restrict__ prev, bf16* __restrict__ dx,
                           float* __restrict__ dprev, float* __restrict__ partials, int B, int T, int C, int strip) {
  __shared__ float red[2 * EW_MAX_WARPS * 2];
  int phase = 0;
  const int b = blockIdx.y, t0 = blockIdx.x * strip, t1 = min(T, t0 + strip);
  const int col = threadIdx.x * 4;
  const bool active = col < C;
  const size_t row0 = (size_t)b * T;
  const float invC = 1.f / C;
  auto ld4 = [](const bf16* p) { return *reinterpret_cast<const uint2*>(p); };

  float w[4], bb[4], mu[K][4];
  float acc_mu[K][4], acc_w[4], acc_b[4], carry[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    w[e] = bb[e] = 0.f;
    acc_w[e] = acc_b[e] = carry[e] = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) { acc_mu[k][e] = 0.f; mu[k][e] = 0.f; }
  }
  if (active) {
    load4f(ln_w + col, w);
    load4f(ln_b + col, bb);
#pragma unroll
    for (int k = 0; k < K; ++k) load4f(mix + (size_t)k * C + col, mu[k]);
    if (t1 < T) {   // halo: contribution of the row after the strip
#pragma unroll
      for (int k = 0; k < K; ++k) {
        float g[4];
        unpack4(ld4(dO.p[k] + (row0 + t1) * C + col), g);
#pragma unroll
        for (int e = 0; e < 4; ++e) carry[e] += g[e] * mu[k][e];
      }
    } else if (dlast) {
      float g[4];
      unpack4(ld4(dlast + (size_t)b * C + col), g);
#pragma unroll
      for (int e = 0; e < 4; ++e) carry[e] += g[e];
    }
  }
  // raw row t (x tile, mean, rstd), fetched one iteration before it is turned into h / xhat
  uint2 xq = make_uint2(0u, 0u);
  float mq = 0.f, rq = 0.f;
  auto fetch_x = [&](int t) {
    if (t >= 0) {
      xq = active ? ld4(x + (row0 + t) * C + col) : make_uint2(0u, 0u);
      mq = mean_in[row0 + t];
      rq = rstd_in[row0 + t];
    } else {
      xq = (prev && active) ? ld4(prev + (size_t)b * C + col) : make_uint2(0u, 0u);
    }
  };
  auto h_from_fetched = [&](int t, float* xh, float* h) {
    float xf[4];
    unpack4(xq, xf);
    if (t < 0) {   // carried row: already h
#pragma unroll
      for (int e = 0; e < 4; ++e) { xh[e] = 0.f; h[e] = xf[e]; }
      return;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      xh[e] = (xf[e] - mq) * rq;
      h[e] = round_bf16(xh[e] * w[e] + bb[e]);
    }
  };
  uint2 gq[K];
  auto fetch = [&](int t) {
#pragma unroll
    for (int k = 0; k < K; ++k)
      gq[k] = (active && t >= t0) ? ld4(dO.p[k] + (row0 + t) * C + col) : make_uint2(0u, 0u);
  };

  float xh_cur[4], h_cur[4], xh_prev[4], h_prev[4];
  fetch_x(t1 - 1);
  h_from_fetched(t1 - 1, xh_cur, h_cur);
  float r_cur = rq, r_prev = 0.f;     // rstd of the row being finished, kept in a register (no load after the barrier)
  fetch(t1 - 1);
  fetch_x(t1 - 2);
  for (int t = t1 - 1; t >= t0; --t) {
    uint2 gc[K];
#pragma unroll
    for (int k = 0; k < K; ++k) gc[k] = gq[k];
    h_from_fetched(t - 1, xh_prev, h_prev);
    r_prev = rq;
    if (t - 1 >= t0) {   // next row's tiles are in flight during this row's reduction
      fetch(t - 1);
      fetch_x(t - 2);
    }
    float dh[4], ncarry[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) { dh[e] = carry[e]; ncarry[e] = 0.f; }
    float dlt[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) dlt[e] = h_prev[e] - h_cur[e];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      float g[4];
      unpack4(gc[k], g);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        dh[e] += g[e];                       // sum_k g_k (1 - mu_k) = sum_k g_k - ncarry, finished below
        ncarry[e] += g[e] * mu[k][e];
        acc_mu[k][e] += g[e] * dlt[e];
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) dh[e] -= ncarry[e];
    float c[2] = {0.f, 0.f};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float g = dh[e] * w[e];
      c[0] += g;
      c[1] += g * xh_cur[e];
      acc_w[e] += dh[e] * xh_cur[e];
      acc_b[e] += dh[e];
    }
    block_sum<2>(c, red, phase);
    if (active) {
      const float r = r_cur;
      float o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = r * (dh[e] * w[e] - c[0] * invC - xh_cur[e] * c[1] * invC);
      if (dres) {
        float rr[4];
        unpack4(ld4(dres + (row0 + t) * C + col), rr);
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] += rr[e];
      }
      *reinterpret_cast<uint2*>(dx + (row0 + t) * C + col) = pack4(o);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      carry[e] = ncarry[e];
      xh_cur[e] = xh_prev[e];
      h_cur[e] = h_prev[e];
    }
    r_cur = r_prev;
  }
  if (active) {
    if (dprev && t0 == 0) store4f(dprev + (size_t)b * C + col, carry);
    float* p = partials + ((size_t)(blockIdx.y * gridDim.x + blockIdx.x) * (K + 2)) * C + col;
#pragma unroll
    for (int k = 0; k < K; ++k) store4f(p + (size_t)k * C, acc_mu[k]);
    store4f(p + (size_t)K * C, acc_w);
    store4f(p + (size_t)(K + 1) * C, acc_b);
  }
}

// K = 1 (channel mix): two rows per block reduction.  The single-output backward is bound by the round trip of one
// row's tiles plus one barrier; handling rows t and t-1 together halves the barriers and doubles the bytes in flight.
__global__ void __launch_bounds__(512, 2)
ln_shift_mix_bwd1_pair_kernel(const bf16* __restrict__ dO, const bf16* __restrict__ dlast, const bf16* __restrict__ dres,
                              const bf16* __restrict__ x, const float* __restrict__ mean_in,
                              const float* __restrict__ rstd_in, const float* __restrict__ ln_w,
                              const float* __restrict__ ln_b, const float* __restrict__ mix,
                              const bf16* __restrict__ prev, bf16* __restrict__ dx, float* __restrict__ dprev,
                              float* __restrict__ partials, int B, int T, int C, int strip) {
  __shared__ float red[2 * EW_MAX_WARPS * 4];
  int phase = 0;
  const int b = blockIdx.y, t0 = blockIdx.x * strip, t1 = min(T, t0 + strip);
  const int col = threadIdx.x * 4;
  const bool active = col < C;
  const size_t row0 = (size_t)b * T;
  const float invC = 1.f / C;
  auto ld4 = [](const bf16* p) { return *reinterpret_cast<const uint2*>(p); };
  const uint2 z2 = make_uint2(0u, 0u);

  float w[4] = {0, 0, 0, 0}, bb[4] = {0, 0, 0, 0}, mu[4] = {0, 0, 0, 0};
  float acc_mu[4] = {0, 0, 0, 0}, acc_w[4] = {0, 0, 0, 0}, acc_b[4] = {0, 0, 0, 0}, carry[4] = {0, 0, 0, 0};
  if (active) {
    load4f(ln_w + col, w);
    load4f(ln_b + col, bb);
    load4f(mix + col, mu);
    if (t1 < T) {
      float g[4];
      unpack4(ld4(dO + (row0 + t1) * C + col), g);
#pragma unroll
      for (int e = 0; e < 4; ++e) carry[e] = g[e] * mu[e];
    } else if (dlast) {
      unpack4(ld4(dlast + (size_t)b * C + col), carry);
    }
  }
  struct Raw { uint2 x; float m, r; };
  auto fetch_row = [&](int t) {          // rows below t0 - 1 are never used
    Raw q{z2, 0.f, 0.f};
    if (t < t0 - 1) return q;
    if (t >= 0) {
      q.x = active ? ld4(x + (row0 + t) * C + col) : z2;
      q.m = mean_in[row0 + t];
      q.r = rstd_in[row0 + t];
    } else if (prev && active) {
      q.x = ld4(prev + (size_t)b * C + col);
    }
    return q;
  };
  auto h_of = [&](int t, const Raw& q, float* xh, float* h) {
    float xf[4];
    unpack4(q.x, xf);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      xh[e] = t < 0 ? 0.f : (xf[e] - q.m) * q.r;
      h[e] = t < 0 ? xf[e] : round_bf16(xh[e] * w[e] + bb[e]);
    }
  };
  auto fetch_g = [&](int t) { return (active && t >= t0) ? ld4(dO + (row0 + t) * C + col) : z2; };

  uint2 gA = fetch_g(t1 - 1), gB = fetch_g(t1 - 2);
  float xh_a[4], h_a[4];
  h_of(t1 - 1, fetch_row(t1 - 1), xh_a, h_a);
  Raw raw1 = fetch_row(t1 - 2), raw2 = fetch_row(t1 - 3);
  for (int t = t1 - 1; t >= t0; t -= 2) {
    const bool two = t - 1 >= t0;
    float xh_b[4], h_b[4], xh_c[4], h_c[4];
    h_of(t - 1, raw1, xh_b, h_b);
    h_of(t - 2, raw2, xh_c, h_c);
    const uint2 gA_c = gA, gB_c = gB;
    if (t - 2 >= t0) {      // next pair's tiles are in flight during this pair's reduction
      gA = fetch_g(t - 2);
      gB = fetch_g(t - 3);
      raw1 = fetch_row(t - 3);
      raw2 = fetch_row(t - 4);
    }
    float ga[4], gb[4], dh_a[4], dh_b[4], nc[4];
    unpack4(gA_c, ga);
    unpack4(gB_c, gb);
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float ca = ga[e] * mu[e];
      dh_a[e] = carry[e] + ga[e] - ca;
      acc_mu[e] += ga[e] * (h_b[e] - h_a[e]);
      const float cb = gb[e] * mu[e];
      dh_b[e] = ca + gb[e] - cb;
      nc[e] = two ? cb : ca;
      if (two) acc_mu[e] += gb[e] * (h_c[e] - h_b[e]);
      const float wa = dh_a[e] * w[e];
      c[0] += wa;
      c[1] += wa * xh_a[e];
      acc_w[e] += dh_a[e] * xh_a[e];
      acc_b[e] += dh_a[e];
      if (two) {
        const float wb = dh_b[e] * w[e];
        c[2] += wb;
        c[3] += wb * xh_b[e];
        acc_w[e] += dh_b[e] * xh_b[e];
        acc_b[e] += dh_b[e];
      }
    }
    block_sum<4>(c, red, phase);
    if (active) {
      auto emit = [&](int tt, const float* dh, const float* xh, float s0, float s1) {
        const float r = rstd_in[row0 + tt];
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = r * (dh[e] * w[e] - s0 * invC - xh[e] * s1 * invC);
        if (dres) {
          float rr[4];
          unpack4(ld4(dres + (row0 + tt) * C + col), rr);
#pragma unroll
          for (int e = 0; e < 4; ++e) o[e] += rr[e];
        }
        *reinterpret_cast<uint2*>(dx + (row0 + tt) * C + col) = pack4(o);
      };
      emit(t, dh_a, xh_a, c[0], c[1]);
      if (two) emit(t - 1, dh_b, xh_b, c[2], c[3]);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      carry[e] = nc[e];
      xh_a[e] = xh_c[e];
      h_a[e] = h_c[e];
    }
  }
  if (active) {
    if (dprev && t0 == 0) store4f(dprev + (size_t)b * C + col, carry);
    float* p = partials + ((size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 3) * C + col;
    store4f(p, acc_mu);
    store4f(p + (size_t)C, acc_w);
    store4f(p + (size_t)2 * C, acc_b);
  }
}

// ------------------------------------------------------------------------------------------------------------
// Backward, pipelined version (K = 1 or 6, up to 2048 channels): four channels per thread held as two float2 pairs
// (packed fp32x2 arithmetic), two rows per block reduction, and the tiles of the next two rows (K gradients, x of the
// row before, the residual gradient) fetched with 8-byte cp.async into a per-thread slot of a double-buffered
// shared-memory ring while the current two rows are processed.  The per-channel state (K mix coefficients, K + 2
// parameter-gradient accumulators, the LayerNorm weight and bias, the carry) fills the register file of one CTA per
// SM, so loads in flight cannot come from other CTAs or from more registers: the ring supplies them.
// Same `partials` layout and the same arithmetic order per channel as the kernels above.
constexpr int V5_MAX_THREADS = 512;
// HBM latency under load is several thousand cycles; one row pair is 8 KB per tensor per CTA, so keeping the memory
// system busy from a single resident CTA takes two (K = 6: 3 x 64 KB of ring) or three (K = 1) row pairs in flight.
__host__ __device__ constexpr int V5_NBUF(int K) { return K >= 4 ? 3 : 4; }

__device__ __forceinline__ float2 bf2_to_f2(uint32_t u) { return make_float2(bf16_lo(u), bf16_hi(u)); }
__device__ __forceinline__ float2 f2_fma(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 f2_add(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 f2_mul(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 f2_sub(float2 a, float2 b) { return __fadd2_rn(a, make_float2(-b.x, -b.y)); }
__device__ __forceinline__ float2 f2_set(float v) { return make_float2(v, v); }
__device__ __forceinline__ void cp8(void* dst, const void* src, bool pred) {
  const int sz = pred ? 8 : 0;     // size 0: the 8 bytes are zero-filled, nothing is read
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src),
               "r"(sz)
               : "memory");
}

template <int K>
__global__ void __launch_bounds__(V5_MAX_THREADS, 1)
ln_shift_mix_bwd_v5_kernel(const DOutPtrs dO, const bf16* __restrict__ dlast, const bf16* __restrict__ dres,
                           const bf16* __restrict__ x, const float* __restrict__ mean_in,
                           const float* __restrict__ rstd_in, const float* __restrict__ ln_w,
                           const float* __restrict__ ln_b, const float* __restrict__ mix,
                           const bf16* __restrict__ prev, bf16* __restrict__ dx, float* __restrict__ dprev,
                           float* __restrict__ partials, int B, int T, int C, int strip) {
  constexpr int NTEN = K + 2;                       // per row slot: K gradient tiles, x of the row before, dres
  constexpr int NBUF = V5_NBUF(K);                  // ring depth: NBUF - 1 row pairs in flight ahead of the one in work
  extern __shared__ __align__(16) unsigned char v5_smem[];
  uint2* ring = reinterpret_cast<uint2*>(v5_smem);  // [NBUF buffers][2 rows][NTEN][blockDim.x]
  __shared__ float red[2 * EW_MAX_WARPS * 4];
  int phase = 0;
  const int nt = blockDim.x;
  const int b = blockIdx.y, t0 = blockIdx.x * strip, t1 = min(T, t0 + strip);
  const int tid = threadIdx.x, col = tid * 4;
  const bool active = col < C;
  const size_t row0 = (size_t)b * T;
  const float invC = 1.f / C;
  auto slot = [&](int bf_, int r, int ten) { return ring + ((size_t)((bf_ * 2 + r) * NTEN + ten)) * nt + tid; };

  float2 w2[2], b2[2], mu2[K][2], accmu2[K][2], accw2[2], accb2[2], carry2[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    w2[i] = b2[i] = accw2[i] = accb2[i] = carry2[i] = f2_set(0.f);
#pragma unroll
    for (int k = 0; k < K; ++k) mu2[k][i] = accmu2[k][i] = f2_set(0.f);
  }
  if (active) {
    const float4 w4 = *reinterpret_cast<const float4*>(ln_w + col), b4 = *reinterpret_cast<const float4*>(ln_b + col);
    w2[0] = make_float2(w4.x, w4.y); w2[1] = make_float2(w4.z, w4.w);
    b2[0] = make_float2(b4.x, b4.y); b2[1] = make_float2(b4.z, b4.w);
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const float4 m4 = *reinterpret_cast<const float4*>(mix + (size_t)k * C + col);
      mu2[k][0] = make_float2(m4.x, m4.y); mu2[k][1] = make_float2(m4.z, m4.w);
    }
    if (t1 < T) {   // halo: contribution of the row after the strip
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const uint2 g = *reinterpret_cast<const uint2*>(dO.p[k] + (row0 + t1) * C + col);
        carry2[0] = f2_fma(bf2_to_f2(g.x), mu2[k][0], carry2[0]);
        carry2[1] = f2_fma(bf2_to_f2(g.y), mu2[k][1], carry2[1]);
      }
    } else if (dlast) {
      const uint2 g = *reinterpret_cast<const uint2*>(dlast + (size_t)b * C + col);
      carry2[0] = bf2_to_f2(g.x); carry2[1] = bf2_to_f2(g.y);
    }
  }

  // Row slot r of a buffer describes output row tt: gradients of row tt, x of row tt - 1 (to rebuild h of the row
  // before), dres of row tt.  Rows below t0 are never processed; x of row t0 - 1 is a halo read (the carried row
  // `prev` stands in for row -1).
  auto issue = [&](int buf, int t_hi) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int tt = t_hi - r;
      const bool live = active && tt >= t0;
      const size_t off = (row0 + (live ? tt : t0)) * C + (active ? col : 0);   // always an address inside the tensors
#pragma unroll
      for (int k = 0; k < K; ++k) cp8(slot(buf, r, k), dO.p[k] + off, live);
      const bool has_x = live && tt - 1 >= 0;
      const bool has_prev = live && tt - 1 < 0 && prev != nullptr;
      const bf16* xsrc = has_x ? x + (row0 + tt - 1) * C + col : (has_prev ? prev + (size_t)b * C + col : x + off);
      cp8(slot(buf, r, K), xsrc, has_x || has_prev);
      cp8(slot(buf, r, K + 1), dres ? dres + off : x + off, live && dres != nullptr);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // h and xhat of a row from its raw x tile; row -1 is the carried row (already h), rows without data are zero
  auto rebuild = [&](const uint2& raw, int t, float2* xh, float2* h) {
    const float2 x0 = bf2_to_f2(raw.x), x1 = bf2_to_f2(raw.y);
    if (t < 0) {
      xh[0] = xh[1] = f2_set(0.f);
      h[0] = x0; h[1] = x1;
      return;
    }
    const float m = mean_in[row0 + t], r = rstd_in[row0 + t];
    const float2 r2 = f2_set(r), nmr = f2_set(-m * r);
    xh[0] = f2_fma(x0, r2, nmr);
    xh[1] = f2_fma(x1, r2, nmr);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 hv = f2_fma(xh[i], w2[i], b2[i]);
      h[i] = bf2_to_f2(pack_bf16(hv.x, hv.y));      // rounded exactly as the forward stored it
    }
  };

  float2 xh_a[2], h_a[2];
  {
    uint2 raw = make_uint2(0u, 0u);
    if (active) raw = *reinterpret_cast<const uint2*>(x + (row0 + t1 - 1) * C + col);
    rebuild(raw, t1 - 1, xh_a, h_a);
  }
  // prologue: NBUF - 1 row pairs in flight (empty groups keep the group count uniform past the end of the strip)
#pragma unroll
  for (int i = 0; i < NBUF - 1; ++i) {
    if (t1 - 1 - 2 * i >= t0) issue(i, t1 - 1 - 2 * i);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  int buf = 0;
  for (int t = t1 - 1; t >= t0; t -= 2) {
    const bool two = t - 1 >= t0;
    {
      const int ahead = t - 2 * (NBUF - 1);
      int nb = buf + NBUF - 1;
      if (nb >= NBUF) nb -= NBUF;
      if (ahead >= t0) issue(nb, ahead);
      else asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group %0;" ::"n"(NBUF - 1) : "memory");
    }
    float2 xh_b[2], h_b[2], xh_c[2], h_c[2];
    rebuild(*slot(buf, 0, K), t - 1, xh_b, h_b);
    rebuild(*slot(buf, 1, K), t - 2, xh_c, h_c);
    float2 dh_a[2], dh_b[2], nc_a[2], nc_b[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) { dh_a[i] = carry2[i]; nc_a[i] = nc_b[i] = dh_b[i] = f2_set(0.f); }
    const float2 dlt_a[2] = {f2_sub(h_b[0], h_a[0]), f2_sub(h_b[1], h_a[1])};
    const float2 dlt_b[2] = {f2_sub(h_c[0], h_b[0]), f2_sub(h_c[1], h_b[1])};
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const uint2 ga = *slot(buf, 0, k), gb = *slot(buf, 1, k);     // zero for rows that are not processed
      const float2 ga2[2] = {bf2_to_f2(ga.x), bf2_to_f2(ga.y)}, gb2[2] = {bf2_to_f2(gb.x), bf2_to_f2(gb.y)};
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        dh_a[i] = f2_add(dh_a[i], ga2[i]);
        nc_a[i] = f2_fma(ga2[i], mu2[k][i], nc_a[i]);
        accmu2[k][i] = f2_fma(ga2[i], dlt_a[i], accmu2[k][i]);
        dh_b[i] = f2_add(dh_b[i], gb2[i]);
        nc_b[i] = f2_fma(gb2[i], mu2[k][i], nc_b[i]);
        accmu2[k][i] = f2_fma(gb2[i], dlt_b[i], accmu2[k][i]);
      }
    }
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    float2 gw_a[2], gw_b[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      dh_a[i] = f2_sub(dh_a[i], nc_a[i]);                   // sum_k g_k (1 - mu_k) + carry
      dh_b[i] = f2_add(f2_sub(dh_b[i], nc_b[i]), nc_a[i]);  // row t-1 receives row t's shifted share
      gw_a[i] = f2_mul(dh_a[i], w2[i]);
      gw_b[i] = f2_mul(dh_b[i], w2[i]);
      const float2 pa = f2_mul(gw_a[i], xh_a[i]), pb = f2_mul(gw_b[i], xh_b[i]);
      c[0] += gw_a[i].x + gw_a[i].y;
      c[1] += pa.x + pa.y;
      accw2[i] = f2_fma(dh_a[i], xh_a[i], accw2[i]);
      accb2[i] = f2_add(accb2[i], dh_a[i]);
      if (two) {
        c[2] += gw_b[i].x + gw_b[i].y;
        c[3] += pb.x + pb.y;
        accw2[i] = f2_fma(dh_b[i], xh_b[i], accw2[i]);
        accb2[i] = f2_add(accb2[i], dh_b[i]);
      }
    }
    block_sum<4>(c, red, phase);
    if (active) {
      auto emit = [&](int tt, const float2* gw, const float2* xh, float s0, float s1, const uint2& rres) {
        const float2 r2 = f2_set(rstd_in[row0 + tt]);
        const float2 n0 = f2_set(-s0 * invC), n1 = f2_set(-s1 * invC);
        float2 o[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) o[i] = f2_mul(r2, f2_fma(xh[i], n1, f2_add(gw[i], n0)));
        if (dres) {
          o[0] = f2_add(o[0], bf2_to_f2(rres.x));
          o[1] = f2_add(o[1], bf2_to_f2(rres.y));
        }
        *reinterpret_cast<uint2*>(dx + (row0 + tt) * C + col) = make_uint2(pack_bf16(o[0].x, o[0].y), pack_bf16(o[1].x, o[1].y));
      };
      emit(t, gw_a, xh_a, c[0], c[1], *slot(buf, 0, K + 1));
      if (two) emit(t - 1, gw_b, xh_b, c[2], c[3], *slot(buf, 1, K + 1));
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      carry2[i] = two ? nc_b[i] : nc_a[i];
      xh_a[i] = two ? xh_c[i] : xh_b[i];
      h_a[i] = two ? h_c[i] : h_b[i];
    }
    if (++buf == NBUF) buf = 0;
  }
  if (active) {
    if (dprev && t0 == 0) *reinterpret_cast<float4*>(dprev + (size_t)b * C + col) = make_float4(carry2[0].x, carry2[0].y, carry2[1].x, carry2[1].y);
    float* p = partials + ((size_t)(blockIdx.y * gridDim.x + blockIdx.x) * (K + 2)) * C + col;
#pragma unroll
    for (int k = 0; k < K; ++k)
      *reinterpret_cast<float4*>(p + (size_t)k * C) = make_float4(accmu2[k][0].x, accmu2[k][0].y, accmu2[k][1].x, accmu2[k][1].y);
    *reinterpret_cast<float4*>(p + (size_t)K * C) = make_float4(accw2[0].x, accw2[0].y, accw2[1].x, accw2[1].y);
    *reinterpret_cast<float4*>(p + (size_t)(K + 1) * C) = make_float4(accb2[0].x, accb2[0].y, accb2[1].x, accb2[1].y);
  }
}

template <int K>
int launch_bwd_v5(const DOutPtrs& dptrs, const void* dlast, const void* dres, const void* x, const void* mean,
                  const void* rstd, const void* ln_w, const void* ln_b, const void* mix, const void* prev, void* dx,
                  void* dprev, void* partials, int B, int T, int C, int strip, cudaStream_t st) {
  const int nt = ((C / 4 + 31) / 32) * 32;
  const int smem = V5_NBUF(K) * 2 * (K + 2) * nt * (int)sizeof(uint2);
  auto kern = ln_shift_mix_bwd_v5_kernel<K>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, V5_NBUF(K) * 2 * (K + 2) * V5_MAX_THREADS * (int)sizeof(uint2));
    if (e != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)e;
    configured = true;
  }
  dim3 grid((T + strip - 1) / strip, B);
  kern<<<grid, nt, smem, st>>>(dptrs, (const bf16*)dlast, (const bf16*)dres, (const bf16*)x, (const float*)mean,
                               (const float*)rstd, (const float*)ln_w, (const float*)ln_b, (const float*)mix,
                               (const bf16*)prev, (bf16*)dx, (float*)dprev, (float*)partials, B, T, C, strip);
  return rwkv_launch_status();
}

inline int threads_for(int C) { return ((C / 8 + 31) / 32) * 32; }

}  // namespace

RWKV_EXPORT int rwkv_ln_shift_mix_forward(const void* x, const void* ln_w, const void* ln_b, const void* mix,
                                          const void* prev, void* outs, void* last, void* mean, void* rstd, int K,
                                          int B, int T, int C, int strip, float eps, void* stream) {
  if (C % 8 || C > 8 * 512 * 2 || C / 8 > 512 || strip <= 0 || B > 65535) return RWKV_ERR_BAD_SHAPE;
  dim3 grid((T + strip - 1) / strip, B);
  const int nt = threads_for(C);
  cudaStream_t st = (cudaStream_t)stream;
#define LAUNCH(KK)                                                                                              \
  rwkv_launch(ln_shift_mix_fwd_kernel<KK>, grid, dim3(nt), 0, st, (const bf16*)x, (const float*)ln_w,          \
              (const float*)ln_b, (const float*)mix, (const bf16*)prev, (bf16*)outs, (bf16*)last, (float*)mean,  \
              (float*)rstd, B, T, C, strip, eps)
  if (K == 6) LAUNCH(6);
  else if (K == 1) LAUNCH(1);
  else return RWKV_ERR_BAD_SHAPE;
#undef LAUNCH
  return rwkv_launch_status();
}

// dO: host array of K device pointers, each a bf16 [B, T, C] gradient of one mixed output.
// dres: optional bf16 [B, T, C] added to dx (the gradient of a residual connection that bypasses this operator).
RWKV_EXPORT int rwkv_ln_shift_mix_backward(const void* const* dO, const void* dlast, const void* dres, const void* x,
                                           const void* mean,
                                           const void* rstd, const void* ln_w, const void* ln_b, const void* mix,
                                           const void* prev, void* dx, void* dprev, void* partials, int K, int B,
                                           int T, int C, int strip, void* stream) {
  if (C % 8 || C / 8 > 512 || strip <= 0 || B > 65535) return RWKV_ERR_BAD_SHAPE;
  dim3 grid((T + strip - 1) / strip, B);
  const int nt = threads_for(C);
  cudaStream_t st = (cudaStream_t)stream;
  if (K != 1 && K != 6) return RWKV_ERR_BAD_SHAPE;
  DOutPtrs dptrs = {};
  for (int k = 0; k < K; ++k) {
    if (!dO[k] || ((uintptr_t)dO[k] & 15)) return RWKV_ERR_BAD_ALIGNMENT;
    dptrs.p[k] = (const bf16*)dO[k];
  }
#define LAUNCH(KK)                                                                                             \
  ln_shift_mix_bwd_kernel<KK><<<grid, nt, 0, st>>>(dptrs, (const bf16*)dlast, (const bf16*)dres, (const bf16*)x, \
                                                   (const float*)mean, (const float*)rstd, (const float*)ln_w, \
                                                   (const float*)ln_b, (const float*)mix, (const bf16*)prev,   \
                                                   (bf16*)dx, (float*)dprev, (float*)partials, B, T, C, strip)
#define LAUNCH_V4(KK)                                                                                          \
  ln_shift_mix_bwd_v4_kernel<KK><<<grid, ((C / 4 + 31) / 32) * 32, 0, st>>>(                                    \
      dptrs, (const bf16*)dlast, (const bf16*)dres, (const bf16*)x, (const float*)mean, (const float*)rstd,      \
      (const float*)ln_w, (const float*)ln_b, (const float*)mix, (const bf16*)prev, (bf16*)dx, (float*)dprev,    \
      (float*)partials, B, T, C, strip)
  static int use_v5 = -1;
  if (use_v5 < 0) {
    const char* e = getenv("RWKVTUNE_LN_BWD_V5");
    use_v5 = (e && e[0] == '0') ? 0 : 1;
  }
  if (use_v5 && C % 4 == 0 && C / 4 <= V5_MAX_THREADS) {   // pipelined kernel: packed arithmetic, two rows per reduction
    if (K == 6)
      return launch_bwd_v5<6>(dptrs, dlast, dres, x, mean, rstd, ln_w, ln_b, mix, prev, dx, dprev, partials, B, T, C, strip, st);
    return launch_bwd_v5<1>(dptrs, dlast, dres, x, mean, rstd, ln_w, ln_b, mix, prev, dx, dprev, partials, B, T, C, strip, st);
  }
  if (C / 4 <= 512) {   // four channels per thread with row prefetch
    if (K == 6) LAUNCH_V4(6);
    else
      ln_shift_mix_bwd1_pair_kernel<<<grid, ((C / 4 + 31) / 32) * 32, 0, st>>>(
          dptrs.p[0], (const bf16*)dlast, (const bf16*)dres, (const bf16*)x, (const float*)mean, (const float*)rstd,
          (const float*)ln_w, (const float*)ln_b, (const float*)mix, (const bf16*)prev, (bf16*)dx, (float*)dprev,
          (float*)partials, B, T, C, strip);
  } else if (K == 6) LAUNCH(6);
  else if (K == 1) LAUNCH(1);
  else return RWKV_ERR_BAD_SHAPE;
#undef LAUNCH
#undef LAUNCH_V4
  return rwkv_launch_status();
}

RWKV_EXPORT int rwkv_layer_norm_forward(const void* x, const void* ln_w, const void* ln_b, void* y, void* mean,
                                        void* rstd, int rows, int C, int strip, float eps, void* stream) {
  if (C % 8 || C / 8 > 512 || strip <= 0) return RWKV_ERR_BAD_SHAPE;
  rwkv_launch(layer_norm_fwd_kernel, dim3((rows + strip - 1) / strip), dim3(threads_for(C)), 0, (cudaStream_t)stream,
              (const bf16*)x, (const float*)ln_w, (const float*)ln_b, (bf16*)y, (float*)mean, (float*)rstd, rows, C,
              strip, eps);
  return rwkv_launch_status();
}

RWKV_EXPORT int rwkv_layer_norm_backward(const void* dy, const void* x, const void* mean, const void* rstd,
                                         const void* ln_w, void* dx, void* partials, int rows, int C, int strip,
                                         void* stream) {
  if (C % 8 || C / 8 > 512 || strip <= 0) return RWKV_ERR_BAD_SHAPE;
  layer_norm_bwd_kernel<<<(rows + strip - 1) / strip, threads_for(C), 0, (cudaStream_t)stream>>>(
      (const bf16*)dy, (const bf16*)x, (const float*)mean, (const float*)rstd, (const float*)ln_w, (bf16*)dx,
      (float*)partials, rows, C, strip);
  return rwkv_launch_status();
}


// ------------------------------------------------------------------------------------------
// Allocation-free variant of the LayerNorm backward (see no_alloc.h for who needs it and the
// rules).  Same kernel as above; the per-block partial sums land in a library-owned device
// array and a second small kernel folds them into dw / db.
// ------------------------------------------------------------------------------------------
#include "no_alloc.h"

static __device__ __align__(256) float g_ln_bwd_scratch[RWKV_NOALLOC_LN_SCRATCH_FLOATS];

namespace {

__global__ void __launch_bounds__(256)
ln_partials_reduce_kernel(const float* __restrict__ partials, int nblocks, int C, float* __restrict__ dw,
                          float* __restrict__ db) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float sw = 0.f, sb = 0.f;
  for (int b = 0; b < nblocks; ++b) {
    sw += partials[(size_t)b * 2 * C + c];
    sb += partials[(size_t)b * 2 * C + C + c];
  }
  dw[c] = sw;
  db[c] = sb;
}

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device, resolved once per device.
int noalloc_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)e;
  if (dev < 0 || dev >= kMaxDevices) return RWKV_ERR_BAD_SHAPE;
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_ln_bwd_scratch);
    if (e != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)e;
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return RWKV_OK;
}

}  // namespace

RWKV_EXPORT int rwkv_layer_norm_backward_noalloc(const void* dy, const void* x, const void* mean, const void* rstd,
                                                 const void* ln_w, void* dx, void* dw, void* db, int rows, int C,
                                                 int strip, void* stream) {
  if (rows <= 0 || C <= 0 || C % 8 || C / 8 > 512 || strip <= 0) return RWKV_ERR_BAD_SHAPE;
  const long long nblocks = ((long long)rows + strip - 1) / strip;
  if (nblocks * 2 * C > (long long)RWKV_NOALLOC_LN_SCRATCH_FLOATS) return RWKV_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int st = noalloc_scratch(&scratch);
  if (st != RWKV_OK) return st;
  cudaStream_t s = (cudaStream_t)stream;
  layer_norm_bwd_kernel<<<(int)nblocks, threads_for(C), 0, s>>>(
      (const bf16*)dy, (const bf16*)x, (const float*)mean, (const float*)rstd, (const float*)ln_w, (bf16*)dx, scratch,
      rows, C, strip);
  ln_partials_reduce_kernel<<<(C + 255) / 256, 256, 0, s>>>(scratch, (int)nblocks, C, (float*)dw, (float*)db);
  return rwkv_launch_status();
}
