// LayerNorm + token shift + K-way lerp in one pass over the residual stream (forward and
// backward), and a plain LayerNorm built from the same pieces.
//
//   h = LN(x);  out_k[t] = h[t] + (h[t-1] - h[t]) * mix_k     (h[-1] = carried row or 0)
//
// The reference runs this as LayerNorm, ZeroPad2d, a subtraction and six multiply-adds,
// each a separate pass over [B,T,C] (model.py:138-144, :305-306, :373).  Here x is read once
// and the K outputs are written once.  h is rounded to bf16 before it is mixed, so a
// sequence processed in chunks with the carried row gives bit-identical results.
#include "elementwise.cuh"

namespace {

template <int K>
__global__ void __launch_bounds__(512)
ln_shift_mix_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ ln_w, const float* __restrict__ ln_b,
                        const float* __restrict__ mix, const bf16* __restrict__ prev, bf16* __restrict__ outs,
                        bf16* __restrict__ last, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                        int B, int T, int C, int strip, float eps) {
  __shared__ float red[2 * EW_MAX_WARPS * 4];
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
  ln_shift_mix_fwd_kernel<KK><<<grid, nt, 0, st>>>((const bf16*)x, (const float*)ln_w, (const float*)ln_b,      \
                                                   (const float*)mix, (const bf16*)prev, (bf16*)outs,           \
                                                   (bf16*)last, (float*)mean, (float*)rstd, B, T, C, strip, eps)
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
  layer_norm_fwd_kernel<<<(rows + strip - 1) / strip, threads_for(C), 0, (cudaStream_t)stream>>>(
      (const bf16*)x, (const float*)ln_w, (const float*)ln_b, (bf16*)y, (float*)mean, (float*)rstd, rows, C, strip,
      eps);
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
