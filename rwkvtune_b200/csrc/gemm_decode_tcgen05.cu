// Decode-sized grouped GEMM on the 5th-generation tensor cores:
//   y_i[M, N_i] = act_i(alpha_i * x_i[M, K_i] @ W_i) + residual_i   (or act_i(alpha_i * x_i W_i + residual_i))
// for up to 12 problems in ONE launch, M <= 128.
//
// With M = number of sequences being decoded, every projection is bound by streaming its weight matrix once,
// and a 24-layer step issues some 330 of them, so both the launch count and the bytes in flight per SM matter.
// The product is computed transposed: the WEIGHT tile (128 output columns x 64 k) is the A operand of a
// 128-row tcgen05.mma and the activations (M rows, padded to a multiple of 16) are the B operand, so the
// 128-lane tensor-memory accumulator is full whatever M is.  Weights may be stored [N, K] (nn.Linear) or
// [K, N] (the low-rank maps); both are expressed through the shared-memory and instruction descriptors.
//
// Grid = (column tiles of all problems) x (K slices).  The S CTAs that share a column tile form one thread-
// block cluster: each streams its K slice through a TMA ring into tensor memory, parks its fp32 partial tile
// in its own shared memory, and after one cluster barrier CTA z sums rows [z * M/S, (z+1) * M/S) of all S
// partial tiles through distributed shared memory in a fixed order (bit-reproducible, no atomics, no
// workspace), applies the activation, adds the residual and stores bf16.  A C x C projection thus runs on
// 128 SMs instead of 16, and r/k/v plus the four low-rank first stages of a block go out as one launch.
//
// Every mbarrier wait is bounded by a deadline; on expiry the waiter records a code in `status`, every role
// still reaches both cluster barriers, tensor memory is released and the kernel returns.
//
// Replaces the cuBLAS calls behind nn.Linear and the low-rank matmuls on the rollout path
// (rwkvtune/models/rwkv7/model.py:134-172, :307-308 at T = 1).
#include <cuda.h>

#include "common.cuh"
#include "tensormap_cache.cuh"

namespace {

constexpr int DN = 128;                      // weight rows (output columns) per CTA = rows of the MMA
constexpr int DK = 64;                       // contraction elements per ring stage (one 128-byte swizzled row)
constexpr int D_THREADS = 192;
constexpr int D_MAX_PROBLEMS = 12;
constexpr int D_MAX_STAGES = 8;
constexpr int D_MAX_M = 128;
constexpr int D_MAX_SPLIT = 8;               // portable cluster size
constexpr int D_MAX_NEXT = 4;                // weight matrices of later launches to prefetch into L2
constexpr int W_BYTES = DN * DK * 2;         // 16 KiB
constexpr unsigned long long D_WAIT_NS = 2000000000ull;

struct alignas(64) DecodeProblem {
  CUtensorMap map_w;
  CUtensorMap map_x;
  bf16* y;
  const bf16* residual;
  int N, K;
  int epi;          // 0 none, 1 relu(x)^2, 3 tanh, 4 sigmoid
  int w_kn;         // weight stored [K, N] (N contiguous) instead of [N, K]
  int tile_start;   // first blockIdx.x of this problem
  float alpha;      // scale of the product (a LoRA adapter's alpha / r; 1 otherwise)
  int res_first;    // 1: y = act(alpha * acc + residual)   0: y = act(alpha * acc) + residual
  int pad_[1];
};
struct alignas(64) DecodeParams {
  DecodeProblem p[D_MAX_PROBLEMS];
  int count, M, Mpad, stages, tmem_cols;
  int prefetch;     // weights are not written by any kernel of the chain: stream them before the chain wait
  int* status;
  unsigned long long* trace;   // optional [CTAs][16] globaltimer stamps of the phases of every CTA (null: off)
  // Weights of the products that follow this launch in the step (null / 0: none).  Once a CTA has requested all of its own
  // tiles it asks for its share of these to be brought into L2, so that HBM keeps streaming during this launch's
  // epilogue and the next launch's prologue instead of idling through both.
  const void* next_w[D_MAX_NEXT];
  unsigned next_bytes[D_MAX_NEXT];
};

struct DBarriers {
  uint64_t full[D_MAX_STAGES];
  uint64_t empty[D_MAX_STAGES];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t d_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void d_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(d_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void d_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(d_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool d_mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(d_smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long d_globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false once the deadline has passed (code recorded in `status`) or another role of this CTA gave up.
__device__ __forceinline__ bool d_mbar_wait(uint64_t* bar, uint32_t parity, DBarriers* bars, int* status, int code) {
  if (d_mbar_try_wait(bar, parity)) return true;
  const unsigned long long deadline = d_globaltimer_ns() + D_WAIT_NS;
  for (uint32_t i = 1;; ++i) {
    if (d_mbar_try_wait(bar, parity)) return true;
    if ((i & 0x3ff) == 0) {
      if (*reinterpret_cast<volatile int*>(&bars->abort_flag)) return false;
      if (d_globaltimer_ns() > deadline) break;
    }
  }
  *reinterpret_cast<volatile int*>(&bars->abort_flag) = 1;
  if (status) atomicCAS(status, 0, code);
  return false;
}
__device__ __forceinline__ void d_tma_load_2d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(d_smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// 128-byte swizzle, 8-row groups 1024 B apart; lbo_16 = 1 for a K-major operand (unused), for an MN-major one the
// distance between two 64-element chunks of the M/N dimension, >> 4.
__device__ __forceinline__ uint64_t d_smem_desc(uint32_t addr, uint32_t lbo_16) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fff);
  d |= (uint64_t)(lbo_16 & 0x3fff) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ void d_umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void d_umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(d_smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void d_tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void d_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void d_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// every thread of every CTA of the cluster passes through here (the roles have diverged: unaligned form)
__device__ __forceinline__ void d_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release;\nbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ float4 d_ld_cluster_f4(uint32_t local_addr, uint32_t cta) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(cta));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(remote)
               : "memory");
  return v;
}
__device__ __forceinline__ float d_act(float x, int epi) {
  if (epi == 1) { x = fmaxf(x, 0.f); return x * x; }
  if (epi == 3) return 1.f - __fdividef(2.f, __expf(2.f * x) + 1.f);
  if (epi == 4) return __fdividef(1.f, 1.f + __expf(-x));
  return x;
}

// phase stamps for `benchmarks/decode_gemm_timeline.py`: 0 CTA started, 1 barriers armed and tensor memory allocated,
// 2 predecessor kernel complete (chain wait returned), 3 first ring stage landed, 4 last ring stage landed,
// 5 accumulator complete, 6 partial tile in shared memory, 7 cluster barrier passed, 8 rows summed and stored,
// 9 tensor memory released
#define D_STAMP(i)                                                                                              \
  do {                                                                                                          \
    if (prm.trace) prm.trace[((size_t)blockIdx.z * gridDim.x + blockIdx.x) * 16 + (i)] = d_globaltimer_ns();    \
  } while (0)

__global__ void __launch_bounds__(D_THREADS)
gemm_decode_kernel(const __grid_constant__ DecodeParams prm) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ DBarriers bars;
  const uint32_t raw = d_smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - raw);

  rwkv_chain_trigger();
  if (threadIdx.x == 0) D_STAMP(0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = (int)gridDim.z, z = (int)blockIdx.z;       // cluster = the S CTAs with the same blockIdx.x
  int pi = 0;
#pragma unroll
  for (int i = 1; i < D_MAX_PROBLEMS; ++i)
    if (i < prm.count && (int)blockIdx.x >= prm.p[i].tile_start) pi = i;
  const DecodeProblem& P = prm.p[pi];
  const int n0 = ((int)blockIdx.x - P.tile_start) * DN;
  const int N = P.N, M = prm.M, Mpad = prm.Mpad;
  const int num_kb = (P.K + DK - 1) / DK;
  const int kb_lo = (int)((long long)num_kb * z / S), kb_hi = (int)((long long)num_kb * (z + 1) / S);
  const int stages = prm.stages;
  const uint32_t stage_bytes = (uint32_t)(W_BYTES + Mpad * 128);
  int* status = prm.status;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { d_mbar_init(&bars.full[s], 1); d_mbar_init(&bars.empty[s], 1); }
    d_mbar_init(&bars.acc_full, 1);
    bars.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(d_smem_u32(&bars.tmem_base)),
                 "r"(prm.tmem_cols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  d_fence_before();
  __syncthreads();
  d_fence_after();
  const uint32_t tmem_base = bars.tmem_base;
  if (threadIdx.x == 0) D_STAMP(1);
  // everything that reads activations or writes results comes after the predecessor kernel has completed; the
  // producer thread decides for itself (it may start the weight stream first)
  if (threadIdx.x != 0) rwkv_chain_wait();

  if (warp == 0) {
    if (lane == 0) {   // -------------------------------------------------------------- TMA producer
      // The first ring fill is split: the weight tiles do not depend on the predecessor kernel, so (when the caller
      // vouches that no kernel of the chain writes weights) they are requested before the chain wait and only the
      // activation tiles after it.
      const int pre = prm.prefetch ? min(stages, kb_hi - kb_lo) : 0;
      for (int i = 0; i < pre; ++i) {
        d_mbar_expect_tx(&bars.full[i], stage_bytes);
        const uint32_t sw = base + i * stage_bytes;
        const int kb = kb_lo + i;
        if (P.w_kn) {
          d_tma_load_2d(sw, &P.map_w, &bars.full[i], n0, kb * DK);
          d_tma_load_2d(sw + DK * 128, &P.map_w, &bars.full[i], n0 + 64, kb * DK);
        } else {
          d_tma_load_2d(sw, &P.map_w, &bars.full[i], kb * DK, n0);
        }
      }
      rwkv_chain_wait();
      D_STAMP(2);
      for (int i = 0; i < pre; ++i)
        d_tma_load_2d(base + i * stage_bytes + W_BYTES, &P.map_x, &bars.full[i], (kb_lo + i) * DK, 0);
      int stage = pre == stages ? 0 : pre;
      uint32_t phase = pre == stages ? 1u : 0u;
      for (int kb = kb_lo + pre; kb < kb_hi; ++kb) {
        if (!d_mbar_wait(&bars.empty[stage], phase ^ 1, &bars, status, 201)) break;
        d_mbar_expect_tx(&bars.full[stage], stage_bytes);
        const uint32_t sw = base + stage * stage_bytes, sx = sw + W_BYTES;
        if (P.w_kn) {   // [K, N]: two 64-column chunks, each 64 k-rows of 128 bytes
          d_tma_load_2d(sw, &P.map_w, &bars.full[stage], n0, kb * DK);
          d_tma_load_2d(sw + DK * 128, &P.map_w, &bars.full[stage], n0 + 64, kb * DK);
        } else {
          d_tma_load_2d(sw, &P.map_w, &bars.full[stage], kb * DK, n0);
        }
        d_tma_load_2d(sx, &P.map_x, &bars.full[stage], kb * DK, 0);
        if (++stage == stages) { stage = 0; phase ^= 1; }
      }
      // this CTA's share of the following launches' weights: L2 prefetch, 16-byte granules, at most 32 KB per request
      const unsigned cta = blockIdx.z * gridDim.x + blockIdx.x, n_cta = gridDim.x * gridDim.z;
#pragma unroll
      for (int j = 0; j < D_MAX_NEXT; ++j) {
        const unsigned total = prm.next_bytes[j];
        if (!prm.next_w[j] || !total) continue;
        const unsigned share = ((total / n_cta) + 15u) & ~15u;
        const unsigned lo = cta * share;
        const unsigned hi = min(total, lo + share);
        const char* basep = reinterpret_cast<const char*>(prm.next_w[j]);
        for (unsigned off = lo; off < hi; off += 32768u) {
          const unsigned sz = min(32768u, hi - off) & ~15u;
          if (sz) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(basep + off), "r"(sz) : "memory");
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && kb_hi > kb_lo) {   // --------------------------------------------- MMA issuer
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((P.w_kn ? 1u : 0u) << 15) |
                             ((uint32_t)(Mpad >> 3) << 17) | ((uint32_t)(DN >> 4) << 24);
      const uint32_t a_lbo = P.w_kn ? (DK * 128) >> 4 : 1;
      const uint32_t a_adv = P.w_kn ? (2 * 1024) >> 4 : 32 >> 4;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb_lo; kb < kb_hi; ++kb) {
        if (!d_mbar_wait(&bars.full[stage], phase, &bars, status, 203)) { ok = false; break; }
        if (kb == kb_lo) D_STAMP(3);
        if (kb == kb_hi - 1) D_STAMP(4);
        d_fence_after();
        const uint32_t sw = base + stage * stage_bytes, sx = sw + W_BYTES;
        const uint64_t adesc = d_smem_desc(sw, a_lbo);
        const uint64_t bdesc = d_smem_desc(sx, 1);
#pragma unroll
        for (int k = 0; k < DK / 16; ++k)
          d_umma(tmem_base, adesc + (uint64_t)(k * a_adv), bdesc + (uint64_t)(k * 2), idesc, ((kb - kb_lo) | k) ? 1u : 0u);
        d_umma_commit(&bars.empty[stage]);
        if (++stage == stages) { stage = 0; phase ^= 1; }
      }
      if (ok) d_umma_commit(&bars.acc_full);
    }
  } else {
    // ---------------------------------------------------------------------------------- accumulator -> shared memory
    // P[m][n] fp32, 128 columns per row, over the (by then idle) ring: the commit behind acc_full completes after
    // every MMA has read its operands, and every TMA write was consumed by one of those MMAs.
    const int quarter = warp & 3;
    const int n = quarter * 32 + lane;
    bool have = kb_hi > kb_lo;
    if (have) have = d_mbar_wait(&bars.acc_full, 0, &bars, status, 204);
    have = __all_sync(0xffffffffu, have);
    if (threadIdx.x == 64) D_STAMP(5);
    // the four warps start overwriting the ring only when all of them know the MMAs are done (or that none ran)
    asm volatile("bar.sync 1, 128;" ::: "memory");
    d_fence_after();
    float* Pm = reinterpret_cast<float*>(base_ptr);
    for (int c = 0; c < Mpad; c += 16) {
      uint32_t v[16];
      if (have) {
        d_tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0u;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) Pm[(c + i) * DN + n] = __uint_as_float(v[i]);
    }
    d_fence_before();
    if (threadIdx.x == 64) D_STAMP(6);
  }

  d_cluster_sync();   // every CTA's partial tile is in its shared memory
  if (threadIdx.x == 64) D_STAMP(7);

  if (warp >= 2) {
    // ---------------------------------------------------------------------------------- cluster reduction + store
    const int t = (int)threadIdx.x - 64;
    const int rp = (M + S - 1) / S;
    const int m_lo = z * rp, m_hi = min(M, m_lo + rp);
    const int n4 = (t & 31) * 4;
    const int epi = P.epi;
    const float alpha = P.alpha;
    const bool res_first = P.res_first != 0;
    if (n0 + n4 < N) {
      const float* Pm = reinterpret_cast<const float*>(base_ptr);
      for (int m = m_lo + (t >> 5); m < m_hi; m += 4) {
        const uint32_t local = d_smem_u32(Pm + m * DN + n4);
        float4 part[D_MAX_SPLIT];
#pragma unroll
        for (int zz = 0; zz < D_MAX_SPLIT; ++zz)
          if (zz < S) part[zz] = d_ld_cluster_f4(local, (uint32_t)zz);
        float4 acc = part[0];
#pragma unroll
        for (int zz = 1; zz < D_MAX_SPLIT; ++zz)
          if (zz < S) { acc.x += part[zz].x; acc.y += part[zz].y; acc.z += part[zz].z; acc.w += part[zz].w; }
        const size_t off = (size_t)m * N + n0 + n4;
        float4 res = make_float4(0.f, 0.f, 0.f, 0.f);
        if (P.residual) {   // plain load: the residual may be the output buffer itself (in-place accumulation)
          const uint2 r = *reinterpret_cast<const uint2*>(P.residual + off);
          res = make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u),
                            __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xffff0000u));
        }
        acc.x *= alpha; acc.y *= alpha; acc.z *= alpha; acc.w *= alpha;
        if (res_first) { acc.x += res.x; acc.y += res.y; acc.z += res.z; acc.w += res.w; }
        acc.x = d_act(acc.x, epi); acc.y = d_act(acc.y, epi); acc.z = d_act(acc.z, epi); acc.w = d_act(acc.w, epi);
        if (!res_first) { acc.x += res.x; acc.y += res.y; acc.z += res.z; acc.w += res.w; }
        *reinterpret_cast<uint2*>(P.y + off) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
      }
    }
  }

  if (threadIdx.x == 64) D_STAMP(8);
  d_cluster_sync();   // nobody leaves while a peer may still read its partial tile
  __syncthreads();
  if (warp == 1) {
    d_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(prm.tmem_cols));
    if (lane == 0) D_STAMP(9);
  }
}

}  // namespace

// count <= 12 problems sharing M <= 128.  xs: [M, K_i] bf16 row-major contiguous; ws: [N_i, K_i] (w_kn[i] = 0) or
// [K_i, N_i] (w_kn[i] = 1) bf16 row-major contiguous; ys: [M, N_i] bf16 contiguous; residuals[i] may be null, else
// [M, N_i] bf16 added after the activation, or before it where res_first[i] (may be ys[i] itself: accumulation in place);
// epis[i]: 0 none, 1 relu^2, 3 tanh, 4 sigmoid; alphas[i] scales the product (null: 1).
// Every N_i a multiple of 8, every K_i a multiple of 8, all pointers 16-byte aligned.  split: K slices per column
// tile (1, 2, 4 or 8), 0 = choose.  prefetch_weights: with chained launches, request weight tiles before the
// predecessor kernel has finished (only when no kernel in flight writes any of the weights).  status: device int, set non-zero if a device-side wait ran out.
// next_ws / next_bytes (next_count <= 4, may be null): device pointers (16-byte aligned) and sizes (below 4 GB) of weight
// matrices that later launches of the same stream will read; they are prefetched into L2.
// trace: optional device buffer of 16 x (number of CTAs) uint64, zeroed by the caller: globaltimer stamps of the phases of
// every CTA (see D_STAMP), for benchmarks/decode_gemm_timeline.py.
RWKV_EXPORT int rwkv_gemm_decode_tcgen05_traced(const void* const* xs, const void* const* ws, void* const* ys,
                                                const void* const* residuals, const int* Ns, const int* Ks,
                                                const int* epis, const int* w_kn, const float* alphas,
                                                const int* res_first, int count, int M, int split,
                                                int prefetch_weights, void* status, void* stream, void* trace,
                                                const void* const* next_ws, const long long* next_bytes,
                                                int next_count) {
  if (count <= 0 || count > D_MAX_PROBLEMS || M <= 0 || M > D_MAX_M) return RWKV_ERR_BAD_SHAPE;
  if (split != 0 && split != 1 && split != 2 && split != 4 && split != 8) return RWKV_ERR_BAD_SHAPE;
  DecodeParams prm;
  memset(&prm, 0, sizeof(prm));
  const int Mpad = (M + 15) / 16 * 16;
  prm.count = count;
  prm.M = M;
  prm.Mpad = Mpad;
  prm.status = (int*)status;
  prm.trace = (unsigned long long*)trace;
  for (int j = 0; j < D_MAX_NEXT; ++j) {
    const bool on = next_ws && next_bytes && j < next_count && next_ws[j] && !((uintptr_t)next_ws[j] & 15) &&
                    next_bytes[j] > 0 && next_bytes[j] < 0xffff0000ll;
    prm.next_w[j] = on ? next_ws[j] : nullptr;
    prm.next_bytes[j] = on ? (unsigned)next_bytes[j] : 0u;
  }
  prm.prefetch = prefetch_weights ? 1 : 0;
  int cols = 32;
  while (cols < Mpad) cols *= 2;
  prm.tmem_cols = cols;
  int tiles = 0, kb_min = 1 << 30, kb_max = 0;
  for (int i = 0; i < count; ++i) {
    const int N = Ns[i], K = Ks[i];
    if (N <= 0 || N % 8 || K <= 0 || K % 8) return RWKV_ERR_BAD_SHAPE;
    if (((uintptr_t)ys[i] & 7) || (residuals && residuals[i] && ((uintptr_t)residuals[i] & 7))) return RWKV_ERR_BAD_ALIGNMENT;
    DecodeProblem& p = prm.p[i];
    int rc;
    if (w_kn && w_kn[i]) rc = rwkv_tmap::make_map(&p.map_w, ws[i], K, N, N, 64, DK);
    else rc = rwkv_tmap::make_map(&p.map_w, ws[i], N, K, K, DK, DN);
    if (rc != RWKV_OK) return rc;
    rc = rwkv_tmap::make_map(&p.map_x, xs[i], M, K, K, DK, Mpad);
    if (rc != RWKV_OK) return rc;
    p.y = (bf16*)ys[i];
    p.residual = residuals ? (const bf16*)residuals[i] : nullptr;
    p.N = N;
    p.K = K;
    p.epi = epis ? epis[i] : 0;
    p.w_kn = (w_kn && w_kn[i]) ? 1 : 0;
    p.alpha = alphas ? alphas[i] : 1.f;
    p.res_first = (res_first && res_first[i]) ? 1 : 0;
    p.tile_start = tiles;
    tiles += (N + DN - 1) / DN;
    const int kb = (K + DK - 1) / DK;
    kb_min = kb < kb_min ? kb : kb_min;
    kb_max = kb > kb_max ? kb : kb_max;
  }
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  if (split == 0) {   // enough CTAs for every SM, never more slices than the shortest contraction has blocks
    split = 1;
    while (split < D_MAX_SPLIT && tiles * split < sms && split * 2 <= kb_min) split *= 2;
  }
  const int stage_bytes = W_BYTES + Mpad * 128;
  const int kb_per_cta = (kb_max + split - 1) / split;
  int stages = (110 * 1024 - 1024) / stage_bytes;            // two CTAs per SM when the ring is this small
  if (stages > kb_per_cta) stages = kb_per_cta;
  if (stages > D_MAX_STAGES) stages = D_MAX_STAGES;
  if (stages < 2) stages = 2;                                // the partial tile (Mpad x 128 fp32) reuses the ring
  prm.stages = stages;
  const int smem = stages * stage_bytes + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         D_MAX_STAGES * (W_BYTES + D_MAX_M * 128) / 2 + 1024);
    if (e != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles, 1, split);
  cfg.blockDim = dim3(D_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (split > 1) {   // a single K slice needs no cluster (the kernel's cluster barriers are then CTA-local)
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 1;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = split;
    ++n_attr;
  }
  if (rwkv_chain_flag()) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_decode_kernel, prm);
  return e == cudaSuccess ? rwkv_launch_status() : RWKV_ERR_CUDA_BASE + (int)e;
}

RWKV_EXPORT int rwkv_gemm_decode_tcgen05(const void* const* xs, const void* const* ws, void* const* ys,
                                         const void* const* residuals, const int* Ns, const int* Ks, const int* epis,
                                         const int* w_kn, const float* alphas, const int* res_first, int count, int M,
                                         int split, int prefetch_weights, void* status, void* stream) {
  return rwkv_gemm_decode_tcgen05_traced(xs, ws, ys, residuals, Ns, Ks, epis, w_kn, alphas, res_first, count, M, split,
                                         prefetch_weights, status, stream, nullptr, nullptr, nullptr, 0);
}

// Chained launches for the kernels of the decode path (see common.cuh): 1 = on, 0 = off.  Returns the previous value.
RWKV_EXPORT int rwkv_set_launch_chaining(int on) {
  const int prev = rwkv_chain_flag();
  rwkv_chain_flag() = on ? 1 : 0;
  return prev;
}
