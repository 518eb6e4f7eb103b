// bf16 GEMM on pairs of SMs: C[M,N] = op(A) * op(B), one 256x256 output tile per cluster of two CTAs, issued as
// tcgen05.mma.cta_group::2.  Operands may be K-major (contraction index contiguous) or MN-major, as in the
// single-CTA kernel, so x@W^T (NT), x@W (NN) and dy^T@x (TN) all run here without transposing anything.
//
// Each CTA of a pair stages ITS OWN halves of the operands with TMA - 128 rows of A and 128 rows of B per
// 64-wide K block (every load reads this GPU's memory into the issuing CTA's own shared memory; nothing is
// broadcast across the cluster) - and
// both CTAs' loads complete on the leader CTA's "full" mbarrier (cp.async.bulk.tensor ... .cta_group::2).  One
// elected thread of the leader issues the MMAs: the tensor cores of both SMs read A from their own shared
// memory and the two B halves from both, so each SM fills 32 KB of shared memory per 256x256x64 step instead
// of the 48 KB per 128x256x64 step of the single-CTA kernel (half the B traffic per FLOP, six ring stages
// instead of four).  The accumulator rows 0-127 live in the leader's tensor memory, rows 128-255 in the
// peer's; tcgen05.commit with a CTA mask releases ring stages and publishes finished accumulators in both
// CTAs, each CTA's four epilogue warps drain their own 128 rows (tcgen05.ld, optional relu^2 / add, bf16,
// swizzled staging, TMA store) and report back to the leader's "accumulator empty" mbarrier.  Two accumulators
// per CTA let the epilogue of tile i overlap the MMAs of tile i+1.
//
// A second operand pair (A2 [M, K2], B2 [N, K2], same layouts as the first) may be appended to the contraction:
// C = op(A) op(B) + op(A2) op(B2), its K blocks simply following the first pair's in the ring.  That is the LoRA
// linear in one launch - x W^T + (s x A^T) B^T with the rank-r factor as one extra 64-wide K block - instead of a
// base GEMM followed by a second GEMM that re-reads and re-writes the whole output to accumulate into it.
//
// Every mbarrier wait is bounded: on expiry the waiter records a code in `status`, all roles leave their
// loops, the two CTAs meet at the cluster barrier, tensor memory is released and the kernel returns.
//
// Replaces the cuBLAS calls behind the nn.Linear forward projections of the reference
// (rwkvtune/models/rwkv7/model.py:146-170, :307-308).
#include <cuda.h>

#include "common.cuh"
#include "tensormap_cache.cuh"

namespace {

constexpr int BM = 128;            // rows of A (and of C) per CTA; the pair covers 256
constexpr int BN = 256;            // columns of C per pair
constexpr int BNH = 128;           // rows of B staged by each CTA
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;           // 16 KiB
constexpr int B_BYTES = BNH * BK * 2;          // 16 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int C_CHUNK_BYTES = BM * 64 * 2;     // 128 rows x 64 bf16
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr unsigned long long WAIT_NS = 4000000000ull;      // every wait gives up after four seconds

struct Barriers {
  uint64_t full[STAGES];      // leader only: both CTAs' loads of a stage have landed
  uint64_t empty[STAGES];     // every CTA: the MMAs that read this stage have completed
  uint64_t acc_full[2];       // every CTA: accumulator complete
  uint64_t acc_empty[2];      // leader only: all eight epilogue warps of the pair have drained the accumulator
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * C_CHUNK_BYTES + 1024 + 256;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.aligned;\nbarrier.cluster.wait.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// arrive on an mbarrier given by its shared::cluster address (this CTA's or the peer's)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false when the deadline passes (after recording `code` and raising the abort flag of both
// CTAs of the pair) or when another role has already aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Barriers* bars, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long deadline = globaltimer_ns() + WAIT_NS;
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 0x3ff) == 0) {
      if (*reinterpret_cast<volatile int*>(&bars->abort_flag)) return false;
      if (globaltimer_ns() > deadline) break;
    }
  }
  *reinterpret_cast<volatile int*>(&bars->abort_flag) = 1;
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(map_to_cta(smem_u32(&bars->abort_flag), cluster_ctarank() ^ 1u)), "r"(1)
               : "memory");
  if (status) atomicCAS(status, 0, code);
  return false;
}

// TMA load into this CTA's shared memory, completing on an mbarrier of the pair given by its shared::cluster address
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y)
               : "memory");
}

// 128-byte swizzle, 8-row groups 1024 B apart.  lbo_16: leading-dimension byte offset >> 4 (1 for K-major, where it
// is unused; for MN-major the distance between two 64-element chunks of the M/N dimension).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_16) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fff);
  d |= (uint64_t)(lbo_16 & 0x3fff) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;        // stride between 8-row groups
  d |= (uint64_t)1 << 46;                  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;                  // 128-byte swizzle
  return d;
}

__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
// arrive on the mbarrier at this shared-memory offset in both CTAs of the pair once all prior MMAs have completed
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// EPI: 0 = plain store, 1 = relu(x)^2, 2 = add the bf16 [M,N] matrix c_in (row stride ldc; may be C itself),
//      5 = x * 2 sqrt(c_in): the derivative of relu(p)^2 expressed through its output, applied to a data gradient
template <bool A_MN, bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_c, int M, int N, int K, int* status,
                         const bf16* __restrict__ c_in, long long ldc, const __grid_constant__ CUtensorMap map_a2,
                         const __grid_constant__ CUtensorMap map_b2, int K2) {
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - raw);
  const uint32_t c_stage = base + STAGES * STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(base_ptr + STAGES * STAGE_BYTES + 2 * C_CHUNK_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();            // 0 = leader
  const int pair = (int)blockIdx.x >> 1, n_pairs = (int)gridDim.x >> 1;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb1 = (K + BK - 1) / BK;                    // K blocks of the first operand pair
  const int num_kb = num_kb1 + (K2 + BK - 1) / BK;          // ... followed by those of the second (K2 = 0: none)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&bars->acc_full[a], 1); mbar_init(&bars->acc_empty[a], 8); }
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();            // the peer's barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        const int m0 = (tile / tiles_n) * (2 * BM) + (int)rank * BM;
        const int n0 = (tile % tiles_n) * BN + (int)rank * BNH;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, bars, status, 201)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(&bars->full[stage], 2 * STAGE_BYTES);
          const uint32_t full_leader = map_to_cta(smem_u32(&bars->full[stage]), 0);
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          const bool second = kb >= num_kb1;
          const CUtensorMap* ma = second ? &map_a2 : &map_a;
          const CUtensorMap* mb = second ? &map_b2 : &map_b;
          const int k0 = (second ? kb - num_kb1 : kb) * BK;
          if (A_MN) {   // A stored [K, M]: two boxes of 64 m-columns x 64 k-rows
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d_pair(sa + c * (BK * 128), ma, full_leader, m0 + c * 64, k0);
          } else {
            tma_load_2d_pair(sa, ma, full_leader, k0, m0);
          }
          if (B_MN) {   // B stored [K, N]: this CTA's 128 n-columns as two boxes
#pragma unroll
            for (int c = 0; c < BNH / 64; ++c) tma_load_2d_pair(sb + c * (BK * 128), mb, full_leader, n0 + c * 64, k0);
          } else {
            tma_load_2d_pair(sb, mb, full_leader, k0, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      // kind::f16: D fp32 (bit 4), A bf16 (bit 7), B bf16 (bit 10), both K-major, N = 256, M = 256 across the pair
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) |
                                 ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                                 ((uint32_t)((2 * BM) >> 4) << 24);
      constexpr uint32_t a_lbo = A_MN ? (BK * 128) >> 4 : 1, b_lbo = B_MN ? (BK * 128) >> 4 : 1;
      constexpr uint32_t a_adv = A_MN ? (2 * 1024) >> 4 : 32 >> 4, b_adv = B_MN ? (2 * 1024) >> 4 : 32 >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1, bars, status, 202)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, bars, status, 203)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          const uint64_t adesc = make_smem_desc(sa, a_lbo), bdesc = make_smem_desc(sb, b_lbo);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_f16_pair(d_tmem, adesc + (uint64_t)(k * a_adv), bdesc + (uint64_t)(k * b_adv), idesc, (kb | k) ? 1u : 0u);
          umma_commit_pair(&bars->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(&bars->acc_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quarter = warp & 3;                 // tensor-memory lanes [32q, 32q+32)
    const int row = quarter * 32 + lane;          // row of this CTA's 128-row half owned by this thread
    int local = 0;
    int cbuf = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, ++local) {
      const int m0 = (tile / tiles_n) * (2 * BM) + (int)rank * BM, n0 = (tile % tiles_n) * BN;
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      mbar_wait(&bars->acc_full[acc], acc_phase, bars, status, 204);
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*reinterpret_cast<volatile int*>(&bars->abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int chunk = 0; chunk < BN / 64; ++chunk) {
        uint32_t v0[32], v1[32];
        tmem_ld32(t_row + chunk * 64, v0);
        tmem_ld32(t_row + chunk * 64 + 32, v1);
        uint4 cin[(EPI == 2 || EPI == 5) ? 8 : 1];
        if (EPI == 2 || EPI == 5) {
          const long long gm = m0 + row;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int gn = n0 + chunk * 64 + j * 8;
            cin[j] = (gm < M && gn < N) ? __ldcg(reinterpret_cast<const uint4*>(c_in + gm * ldc + gn))
                                        : make_uint4(0u, 0u, 0u, 0u);
          }
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (threadIdx.x == 64) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const uint32_t cs = c_stage + cbuf * C_CHUNK_BYTES + row * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float f[8], prev[8];
          if (EPI == 2 || EPI == 5) unpack8(cin[j], prev);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int col = j * 8 + e;
            float x = __uint_as_float(col < 32 ? v0[col] : v1[col - 32]);
            if (EPI == 1) { x = fmaxf(x, 0.f); x = x * x; }
            if (EPI == 2) x += prev[e];
            if (EPI == 5) x *= 2.f * sqrtf(prev[e]);
            f[e] = x;
          }
          const uint4 packed = pack8(f);
          const uint32_t dst = cs + ((j ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed.x), "r"(packed.y),
                       "r"(packed.z), "r"(packed.w)
                       : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          tma_store_2d(&map_c, c_stage + cbuf * C_CHUNK_BYTES, n0 + chunk * 64, m0);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        cbuf ^= 1;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bars->acc_empty[acc]), 0));
    }
    if (threadIdx.x == 64) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();            // neither CTA leaves (or frees tensor memory) while the other may still signal or read it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
}

using rwkv_tmap::make_map;   // encoded maps are cached per (address, shape, stride, box)

template <bool A_MN, bool B_MN, int EPI>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, int M, int N, int K, int* status,
           int sms, const bf16* c_in, long long ldc, cudaStream_t st, const CUtensorMap& ma2, const CUtensorMap& mb2,
           int K2) {
  auto kern = gemm_tcgen05_2cta_kernel<A_MN, B_MN, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)e;
    configured = true;
  }
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  int pairs = sms / 2;
  if (tiles < pairs) pairs = tiles;
  kern<<<2 * pairs, NUM_THREADS, SMEM_BYTES, st>>>(ma, mb, mc, M, N, K, status, c_in, ldc, ma2, mb2, K2);
  return rwkv_launch_status();
}

}  // namespace

// C[M,N] (row-major, ldc) = op(A) op(B), bf16 in/out, fp32 accumulation, on pairs of SMs.
//   a_mn = 0: A is [M,K] row-major (lda);  a_mn = 1: A is stored [K,M] row-major (lda)
//   b_mn = 0: B is [N,K] row-major (ldb);  b_mn = 1: B is stored [K,N] row-major (ldb)
//   epilogue: 0 none, 1 relu(x)^2, 5 multiply by 2 sqrt(residual), 2 add a bf16 [M,N] matrix: `residual` (row stride
//   ldr) or, when that is null, the values already in C (in place).
//   status: device int, set non-zero if a device-side wait expired.
//   a2 / b2 (optional, K2 > 0): a second operand pair in the same layouts, appended to the contraction:
//   C = op(A) op(B) + op(A2) op(B2)   (A2 is [M,K2] or stored [K2,M]; B2 is [N,K2] or stored [K2,N])
RWKV_EXPORT int rwkv_gemm_bf16_tcgen05_2cta_dual(const void* a, const void* b, void* c, int M, int N, int K,
                                                 long long lda, long long ldb, long long ldc, int a_mn, int b_mn,
                                                 int epilogue, void* status, const void* residual, long long ldr,
                                                 const void* a2, const void* b2, int K2, long long lda2, long long ldb2,
                                                 void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K2 < 0 || !(epilogue == 0 || epilogue == 1 || epilogue == 2 || epilogue == 5))
    return RWKV_ERR_BAD_SHAPE;
  if (K2 > 0 && (!a2 || !b2)) return RWKV_ERR_BAD_SHAPE;
  if ((epilogue == 2 || epilogue == 5) && residual && (((uintptr_t)residual & 15) || (ldr * 2) % 16))
    return RWKV_ERR_BAD_ALIGNMENT;
  if (epilogue == 5 && !residual) return RWKV_ERR_BAD_SHAPE;
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap ma, mb, mc;
  int r = a_mn ? make_map(&ma, a, K, M, lda, 64, BK) : make_map(&ma, a, M, K, lda, BK, BM);
  if (r) return r;
  r = b_mn ? make_map(&mb, b, K, N, ldb, 64, BK) : make_map(&mb, b, N, K, ldb, BK, BNH);
  if (r) return r;
  r = make_map(&mc, c, M, N, ldc, 64, BM);
  if (r) return r;
  CUtensorMap ma2 = ma, mb2 = mb;     // placeholders when there is no second pair (never dereferenced: K2 = 0)
  if (K2 > 0) {
    r = a_mn ? make_map(&ma2, a2, K2, M, lda2, 64, BK) : make_map(&ma2, a2, M, K2, lda2, BK, BM);
    if (r) return r;
    r = b_mn ? make_map(&mb2, b2, K2, N, ldb2, 64, BK) : make_map(&mb2, b2, N, K2, ldb2, BK, BNH);
    if (r) return r;
  }
  cudaStream_t st = (cudaStream_t)stream;
  int* sp = (int*)status;
  const bf16* cp = residual ? (const bf16*)residual : (const bf16*)c;
  if (residual) ldc = ldr;
#define DISPATCH(AM, BMN)                                                                 \
  (epilogue == 1   ? launch<AM, BMN, 1>(ma, mb, mc, M, N, K, sp, sms, cp, ldc, st, ma2, mb2, K2)         \
   : epilogue == 2 ? launch<AM, BMN, 2>(ma, mb, mc, M, N, K, sp, sms, cp, ldc, st, ma2, mb2, K2)         \
   : epilogue == 5 ? launch<AM, BMN, 5>(ma, mb, mc, M, N, K, sp, sms, cp, ldc, st, ma2, mb2, K2)         \
                   : launch<AM, BMN, 0>(ma, mb, mc, M, N, K, sp, sms, cp, ldc, st, ma2, mb2, K2))
  if (!a_mn && !b_mn) return DISPATCH(false, false);
  if (!a_mn && b_mn) return DISPATCH(false, true);
  if (a_mn && b_mn) return DISPATCH(true, true);
  return DISPATCH(true, false);
#undef DISPATCH
}

RWKV_EXPORT int rwkv_gemm_bf16_tcgen05_2cta(const void* a, const void* b, void* c, int M, int N, int K, long long lda,
                                            long long ldb, long long ldc, int a_mn, int b_mn, int epilogue,
                                            void* status, const void* residual, long long ldr, void* stream) {
  return rwkv_gemm_bf16_tcgen05_2cta_dual(a, b, c, M, N, K, lda, ldb, ldc, a_mn, b_mn, epilogue, status, residual, ldr,
                                          nullptr, nullptr, 0, 0, 0, stream);
}
