// WKV7 recurrence on the host CPU: forward (keeping one state per 16 steps for the backward, or none) and the
// closed-form backward, one (batch, head) problem per work item spread over std::threads.  The counterpart of the
// reference's CPU operator (rwkvtune/models/rwkv7/operators/wkv_cpu.py:9-80, a Python loop over time traced by
// autograd); bound in ops/cpu_ops.py, which keeps a pure-PyTorch version of the same algebra as fallback and oracle.
//
// Per head, with S indexed [value row i][key column j] and d = exp(-exp(w)):
//   u_i = sum_j S[i][j] a[j];   S'[i][j] = S[i][j] d[j] + u_i b[j] + v[i] k[j];   y_i = sum_j S'[i][j] r[j]
// Row i of S' depends on row i of S only, so the update runs row by row (in place when no state history is kept).
// Layouts: inputs and outputs [B, T, H, N] fp32 contiguous; state [B, H, N, N]; history [B*H, ceil(T/16), N, N]: the
// state at the start of every 16-step chunk (the backward rebuilds the others chunk by chunk in a thread-local buffer).
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#define RWKV_API extern "C" __attribute__((visibility("default")))
#if defined(__x86_64__) && defined(__GNUC__)
#define RWKV_CLONES __attribute__((target_clones("avx2,fma", "default")))
#else
#define RWKV_CLONES
#endif

namespace {

constexpr int MAX_N = 256;
constexpr int CHUNK = 16;      // the backward keeps one state per CHUNK steps and rebuilds the others

template <typename F>
void parallel_for(int n, int threads, F&& body) {
  if (threads < 1) threads = 1;
  if (threads > n) threads = n > 0 ? n : 1;
  if (threads == 1) {
    for (int i = 0; i < n; ++i) body(i);
    return;
  }
  std::atomic<int> next{0};
  auto work = [&]() {
    while (true) {
      const int i = next.fetch_add(1);
      if (i >= n) break;
      body(i);
    }
  };
  std::vector<std::thread> pool;
  pool.reserve(threads);
  for (int k = 0; k < threads; ++k) pool.emplace_back(work);
  for (auto& th : pool) th.join();
}

// One step for one head: cur (may alias prev) = prev diag(d) + (prev a) b^T + v k^T; y = cur r (skipped when y is null).
RWKV_CLONES inline void step_forward(const float* prev, float* cur, const float* rt, const float* kt, const float* vt,
                                     const float* at, const float* bt, const float* d, float* yt, int N) {
  for (int i = 0; i < N; ++i) {
    const float* p = prev + (int64_t)i * N;
    float* c = cur + (int64_t)i * N;
    float u = 0.f;
    for (int j = 0; j < N; ++j) u += p[j] * at[j];
    const float vi = vt[i];
    float acc = 0.f;
    for (int j = 0; j < N; ++j) {
      const float s = p[j] * d[j] + u * bt[j] + vi * kt[j];
      c[j] = s;
      acc += s * rt[j];
    }
    if (yt != nullptr) yt[i] = acc;
  }
}

// history (optional) receives the state at the start of every CHUNK-step chunk: S_0, S_CHUNK, S_2CHUNK, ...
RWKV_CLONES void forward_head(const float* r, const float* w, const float* k, const float* v, const float* a, const float* b,
                              const float* state0, float* history, float* final_state, float* y, float* decay, int T,
                              int N, int64_t step_stride) {
  const int64_t NN = (int64_t)N * N;
  std::vector<float> S(NN);
  if (state0 != nullptr) std::memcpy(S.data(), state0, NN * sizeof(float));
  else std::memset(S.data(), 0, NN * sizeof(float));
  float d[MAX_N];
  for (int t = 0; t < T; ++t) {
    if (history != nullptr && t % CHUNK == 0) std::memcpy(history + (int64_t)(t / CHUNK) * NN, S.data(), NN * sizeof(float));
    const int64_t off = (int64_t)t * step_stride;
    const float* wt = w + off;
    for (int j = 0; j < N; ++j) d[j] = std::exp(-std::exp(wt[j]));
    if (decay != nullptr) std::memcpy(decay + off, d, N * sizeof(float));
    step_forward(S.data(), S.data(), r + off, k + off, v + off, a + off, b + off, d, y + off, N);
  }
  std::memcpy(final_state, S.data(), NN * sizeof(float));
}

RWKV_CLONES void backward_head(const float* r, const float* w, const float* k, const float* v, const float* a, const float* b,
                               const float* decay, const float* history, const float* dy, const float* dstate, float* dr,
                               float* dw, float* dk, float* dv, float* da, float* db, float* dstate0, int T, int N,
                               int64_t step_stride) {
  const int64_t NN = (int64_t)N * N;
  std::vector<float> G(NN);
  if (dstate != nullptr) std::memcpy(G.data(), dstate, NN * sizeof(float));
  else std::memset(G.data(), 0, NN * sizeof(float));
  std::vector<float> local((int64_t)(CHUNK + 1) * NN);      // the states of one chunk, rebuilt from its first one
  float dd[MAX_N];
  const int n_chunks = (T + CHUNK - 1) / CHUNK;
  for (int c = n_chunks - 1; c >= 0; --c) {
    const int t0 = c * CHUNK, t1 = (t0 + CHUNK < T) ? t0 + CHUNK : T;
    std::memcpy(local.data(), history + (int64_t)c * NN, NN * sizeof(float));
    for (int t = t0; t < t1; ++t) {
      const int64_t off = (int64_t)t * step_stride;
      float* prev = local.data() + (int64_t)(t - t0) * NN;
      step_forward(prev, prev + NN, r + off, k + off, v + off, a + off, b + off, decay + off, nullptr, N);
    }
    for (int t = t1 - 1; t >= t0; --t) {
      const int64_t off = (int64_t)t * step_stride;
      const float *rt = r + off, *wt = w + off, *kt = k + off, *vt = v + off, *at = a + off, *bt = b + off;
      const float *dt = decay + off, *dyt = dy + off;
      float *drt = dr + off, *dwt = dw + off, *dkt = dk + off, *dvt = dv + off, *dat = da + off, *dbt = db + off;
      const float* prev = local.data() + (int64_t)(t - t0) * NN;
      const float* cur = prev + NN;
      for (int j = 0; j < N; ++j) drt[j] = dkt[j] = dbt[j] = dat[j] = dd[j] = 0.f;
      for (int i = 0; i < N; ++i) {
        float* g = G.data() + (int64_t)i * N;
        const float* p = prev + (int64_t)i * N;
        const float* cr = cur + (int64_t)i * N;
        const float dyi = dyt[i], vi = vt[i];
        float dvi = 0.f, e = 0.f, u = 0.f;
        for (int j = 0; j < N; ++j) {
          const float gij = g[j] + dyi * rt[j];            // dL/dS_t
          g[j] = gij;
          drt[j] += cr[j] * dyi;
          dvi += gij * kt[j];
          e += gij * bt[j];
          u += p[j] * at[j];
        }
        dvt[i] = dvi;
        for (int j = 0; j < N; ++j) {
          const float gij = g[j];
          dkt[j] += gij * vi;
          dbt[j] += gij * u;
          dd[j] += gij * p[j];
          dat[j] += p[j] * e;
          g[j] = gij * dt[j] + e * at[j];                   // dL/dS_{t-1}
        }
      }
      for (int j = 0; j < N; ++j) dwt[j] = -dd[j] * dt[j] * std::exp(wt[j]);
    }
  }
  if (dstate0 != nullptr) std::memcpy(dstate0, G.data(), NN * sizeof(float));
}

}  // namespace

// history (optional): [B*H, rwkv_wkv7_cpu_history_states(T), N, N]; decay (optional): [B, T, H, N] receives exp(-exp(w)).
RWKV_API int rwkv_wkv7_cpu_history_states(int T) { return (T + CHUNK - 1) / CHUNK > 0 ? (T + CHUNK - 1) / CHUNK : 1; }

RWKV_API int rwkv_wkv7_cpu_forward(const float* r, const float* w, const float* k, const float* v, const float* a,
                                   const float* b, const float* state0, float* history, float* final_state, float* y,
                                   float* decay, int B, int T, int H, int N, int threads) {
  if (B < 1 || T < 0 || H < 1 || N < 1 || N > MAX_N) return 1;
  const int64_t NN = (int64_t)N * N;
  const int64_t step = (int64_t)H * N;
  parallel_for(B * H, threads, [&](int bh) {
    const int bi = bh / H, h = bh % H;
    const int64_t base = ((int64_t)bi * T * H + h) * N;
    forward_head(r + base, w + base, k + base, v + base, a + base, b + base, state0 ? state0 + bh * NN : nullptr,
                 history ? history + (int64_t)bh * rwkv_wkv7_cpu_history_states(T) * NN : nullptr, final_state + bh * NN, y + base,
                 decay ? decay + base : nullptr, T, N, step);
  });
  return 0;
}

RWKV_API int rwkv_wkv7_cpu_backward(const float* r, const float* w, const float* k, const float* v, const float* a,
                                    const float* b, const float* decay, const float* history, const float* dy,
                                    const float* dstate, float* dr, float* dw, float* dk, float* dv, float* da, float* db,
                                    float* dstate0, int B, int T, int H, int N, int threads) {
  if (B < 1 || T < 0 || H < 1 || N < 1 || N > MAX_N || history == nullptr || decay == nullptr) return 1;
  const int64_t NN = (int64_t)N * N;
  const int64_t step = (int64_t)H * N;
  parallel_for(B * H, threads, [&](int bh) {
    const int bi = bh / H, h = bh % H;
    const int64_t base = ((int64_t)bi * T * H + h) * N;
    backward_head(r + base, w + base, k + base, v + base, a + base, b + base, decay + base,
                  history + (int64_t)bh * rwkv_wkv7_cpu_history_states(T) * NN, dy + base, dstate ? dstate + bh * NN : nullptr, dr + base,
                  dw + base, dk + base, dv + base, da + base, db + base, dstate0 ? dstate0 + bh * NN : nullptr, T, N, step);
  });
  return 0;
}
