// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = op(A) * op(B), fp32 accumulation in
// tensor memory, operands streamed by TMA.
//
// One persistent CTA per SM, six warps with fixed roles:
//   warp 0    TMA producer: fills a 4-stage ring of {A 128x64, B 256x64} bf16 tiles (128-byte
//             swizzle), one mbarrier transaction per stage
//   warp 1    allocates the 512 tensor-memory columns and issues tcgen05.mma (128x256x16 per
//             instruction, one elected thread); tcgen05.commit releases ring stages and signals
//             a finished accumulator
//   warps 2-5 epilogue: tcgen05.ld the 128x256 fp32 accumulator quarter by quarter, optional
//             fused relu(x)^2, convert to bf16, stage in swizzled shared memory, TMA store
// Two accumulators (2 x 256 columns) let the epilogue of tile i overlap the MMAs of tile i+1.
//
// Operand layouts: an operand is "K-major" when the contraction index is contiguous in memory
// and "MN-major" when the M (or N) index is.  Both are expressed through the shared-memory and
// instruction descriptors, so x@W^T (NT), x@W (NN) and dy^T@x (TN) run in the same kernel without
// transposing anything in memory.
//
// Every mbarrier wait is bounded: on expiry the waiter records a code in `status`, all roles
// leave their loops, tensor memory is released and the kernel returns.
//
// Replaces the cuBLAS calls behind every nn.Linear / matmul of the reference
// (rwkvtune/models/rwkv7/model.py:146-170, :307-308).
#include <cuda.h>

#include "common.cuh"
#include "tensormap_cache.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;          // 16 KiB
constexpr int B_BYTES = BN * BK * 2;          // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int C_CHUNK_BYTES = BM * 64 * 2;    // 128 rows x 64 bf16
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr uint32_t WAIT_LIMIT = 1u << 28;
constexpr int MAX_RANKS = 16;

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * C_CHUNK_BYTES + 1024 + 256;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (after recording `code`) when the limit is hit or another role aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Barriers* bars, int* status, int code) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 0xffff) == 0xffff && *reinterpret_cast<volatile int*>(&bars->abort_flag)) return false;
  }
  *reinterpret_cast<volatile int*>(&bars->abort_flag) = 1;
  if (status) atomicCAS(status, 0, code);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_16, uint32_t sbo_16) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fff);
  d |= (uint64_t)(lbo_16 & 0x3fff) << 16;
  d |= (uint64_t)(sbo_16 & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version for sm_100
  d |= (uint64_t)2 << 61;   // 128-byte swizzle
  return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
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

// All-gather fused into the GEMM (ZeRO-3): the weight is stored as K-panels, rank p owning columns
// [p*Kp, (p+1)*Kp) as a contiguous [N, Kp] matrix.  Every CTA of the GEMM carries four extra "copy" warps.
// Copy warp q of every CTA works on the row blocks j = q, q + 4, ... of the weight (a row block = 256 weight
// rows = one output-column tile, all panels): the 148 warps with the same q pull that row block from the owners'
// memory - plain peer loads over NVLink, eight 16-byte loads in flight per thread, all peers at once - into a
// local [N, K] staging matrix and each adds one arrival to the row block's counter.  Four row blocks are in
// flight at any time and they complete in order.  The tiles are walked in groups of column tiles, and the TMA
// producer of a tile waits only for the row block it is about to load: the MMAs of the first column tiles run
// while the rest of the weight is still crossing NVLink, no SM is set aside for copying, and each remote byte
// crosses the link once.
struct AgParams {
  const bf16* shard[MAX_RANKS];
  bf16* staged;
  int* blk_count;      // [n_rb] arrival counters, monotonically increasing over calls
  int rank, world, Kp, n_rb;
  int target;          // a row block has landed when its counter has reached this value
  int group;           // column tiles per tile group (see the tile order below)
  // optional second operand pair (local memory, K-major), appended to the contraction: y = x W^T + x2 W2^T.  The LoRA
  // term of a sharded frozen weight rides here as one extra K block instead of a second, accumulating GEMM.
  int K2;
  CUtensorMap map_a2, map_b2;
};
constexpr int AG_COPY_WARPS = 4;

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Runs in warps NUM_THREADS/32 .. NUM_THREADS/32 + AG_COPY_WARPS - 1 of every CTA.
__device__ void ag_copy_role(const AgParams& ag, int N, int K, int cta, int n_cta) {
  constexpr int UNROLL = 8;
  const int wq = ((int)threadIdx.x - NUM_THREADS) >> 5;
  const int lane = threadIdx.x & 31;
  const long long g = (long long)cta * 32 + lane;          // this thread among the threads that share a row block
  const long long G = (long long)n_cta * 32;
  const int vec_per_prow = ag.Kp / 8;                      // 16-byte vectors per panel row
  const int vec_per_row = K / 8;
  for (int j = wq; j < ag.n_rb; j += AG_COPY_WARPS) {
    const int r0 = j * BN;
    const int rows = min(BN, N - r0);
    const long long total = (long long)rows * vec_per_row;
    for (long long v0 = g; v0 < total; v0 += G * UNROLL) {
      uint4 val[UNROLL];
      long long dst_off[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long v = v0 + u * G;
        if (v < total) {
          const int row = (int)(v / vec_per_row);
          const int cv = (int)(v - (long long)row * vec_per_row);
          const int p = cv / vec_per_prow;
          const int c = cv - p * vec_per_prow;
          val[u] = __ldcg(reinterpret_cast<const uint4*>(ag.shard[p]) + (long long)(r0 + row) * vec_per_prow + c);
          dst_off[u] = (long long)(r0 + row) * K + (long long)cv * 8;
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long v = v0 + u * G;
        if (v < total) *reinterpret_cast<uint4*>(ag.staged + dst_off[u]) = val[u];
      }
    }
    __threadfence();
    asm volatile("fence.proxy.async;" ::: "memory");
    __syncwarp();
    if (lane == 0) atomicAdd(&ag.blk_count[j], 1);
  }
}

// EPI: 0 = plain store, 1 = relu(x)^2, 2 = add to the bf16 values already in C (in place: C += A B),
//      3 = tanh(x), 4 = sigmoid(x)  (the bottleneck activations of the low-rank decay and gate chains),
//      5 = x * 2 sqrt(Y) with Y a bf16 [M,N] matrix: the derivative of relu(p)^2 expressed through its output Y,
//          applied to the dgrad of the channel-mix value projection (no separate activation-backward pass)
template <bool A_MN, bool B_MN, int EPI, bool AG>
__global__ void __launch_bounds__(AG ? NUM_THREADS + AG_COPY_WARPS * 32 : NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_c, int M, int N, int K, int* status,
                    const bf16* __restrict__ c_in, long long ldc, int splits, float* __restrict__ partial,
                    const __grid_constant__ AgParams ag) {
  const int cta = (int)blockIdx.x;
  const int n_cta = (int)gridDim.x;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - raw);
  const uint32_t c_stage = base + STAGES * STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(base_ptr + STAGES * STAGE_BYTES + 2 * C_CHUNK_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  // split-K (splits > 1): a work item is (tile, K slice); the slice's fp32 tile goes to `partial[slice]` and a small
  // kernel sums the slices.  For products with few output tiles and a long contraction (weight gradients of the
  // low-rank maps: 16 tiles, K = tokens) this is what fills the SMs.  splits == 1 is the plain path.
  const int num_items = num_tiles * splits;
  // plain GEMM: row-tile-major (consecutive CTAs share the A tile's row panel and sweep B, which stays in L2).
  // All-gather variant: the column tiles are taken in groups of `ag.group`, group after group in the order in which
  // their weight rows arrive, and row-tile-major inside a group: early tiles need only the first row blocks of the
  // weight, while A is re-read once per group instead of once per column tile.
  auto tile_m0 = [&](int tile) {
    if (!AG) return (tile / tiles_n) * BM;
    const int per_group = tiles_m * ag.group;
    const int g = tile / per_group;
    const int gn = min(ag.group, tiles_n - g * ag.group);
    return ((tile - g * per_group) / gn) * BM;
  };
  auto tile_n0 = [&](int tile) {
    if (!AG) return (tile % tiles_n) * BN;
    const int per_group = tiles_m * ag.group;
    const int g = tile / per_group;
    const int gn = min(ag.group, tiles_n - g * ag.group);
    return (g * ag.group + (tile - g * per_group) % gn) * BN;
  };
  const int num_kb2 = AG ? (ag.K2 + BK - 1) / BK : 0;      // K blocks of the appended operand pair (all-gather variant)
  auto kb_range = [&](int sp, int& lo, int& hi) {
    lo = (int)((long long)num_kb * sp / splits);
    hi = (int)((long long)num_kb * (sp + 1) / splits) + (sp == splits - 1 ? num_kb2 : 0);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&bars->acc_full[a], 1); mbar_init(&bars->acc_empty[a], 4); }
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = cta; item < num_items && ok; item += n_cta) {
        const int tile = item / splits;
        const int m0 = tile_m0(tile), n0 = tile_n0(tile);
        int kb_lo, kb_hi;
        kb_range(item - tile * splits, kb_lo, kb_hi);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          const int k0 = kb * BK;
          if (AG && kb == kb_lo) {   // the row block of the weight that this column tile reads must have landed
            const int* cnt = &ag.blk_count[n0 / BN];
            bool landed = false;
            for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
              if (ld_acquire_gpu(cnt) >= ag.target) { landed = true; break; }
              if ((it & 0xfff) == 0xfff && *reinterpret_cast<volatile int*>(&bars->abort_flag)) break;
              __nanosleep(32);
            }
            if (!landed) {
              *reinterpret_cast<volatile int*>(&bars->abort_flag) = 1;
              if (status) atomicCAS(status, 0, 105);
              ok = false;
              break;
            }
            asm volatile("fence.proxy.async;" ::: "memory");
          }
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, bars, status, 101)) { ok = false; break; }
          mbar_expect_tx(&bars->full[stage], STAGE_BYTES);
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          if (AG && kb >= num_kb) {   // appended pair: both operands K-major, from this GPU's memory
            tma_load_2d(sa, &ag.map_a2, &bars->full[stage], (kb - num_kb) * BK, m0);
            tma_load_2d(sb, &ag.map_b2, &bars->full[stage], (kb - num_kb) * BK, n0);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
            continue;
          }
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * (BK * 128), &map_a, &bars->full[stage], m0 + c * 64, k0);
          } else {
            tma_load_2d(sa, &map_a, &bars->full[stage], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * (BK * 128), &map_b, &bars->full[stage], n0 + c * 64, k0);
          } else {
            tma_load_2d(sb, &map_b, &bars->full[stage], k0, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) |
                                 ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      constexpr uint32_t a_lbo = A_MN ? (BK * 128) >> 4 : 1, b_lbo = B_MN ? (BK * 128) >> 4 : 1;
      constexpr uint32_t a_adv = A_MN ? (2 * 1024) >> 4 : 32 >> 4, b_adv = B_MN ? (2 * 1024) >> 4 : 32 >> 4;
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int item = cta; item < num_items && ok; item += n_cta, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1, bars, status, 102)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        int kb_lo, kb_hi;
        kb_range(item % splits, kb_lo, kb_hi);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, bars, status, 103)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_BYTES;
          const uint64_t adesc = make_smem_desc(sa, a_lbo, 1024 >> 4);
          const uint64_t bdesc = make_smem_desc(sb, b_lbo, 1024 >> 4);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_f16(d_tmem, adesc + (uint64_t)(k * a_adv), bdesc + (uint64_t)(k * b_adv), idesc,
                     ((kb - kb_lo) | k) ? 1u : 0u);
          umma_commit(&bars->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&bars->acc_full[acc]);
      }
    }
  } else if (AG && warp >= NUM_THREADS / 32) {
    // ------------------------------------------------------------------ panel copy (all-gather variant only)
    ag_copy_role(ag, N, K, cta, n_cta);
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;                 // tensor-memory lanes [32q, 32q+32)
    const int row = quarter * 32 + lane;          // row of the tile owned by this thread
    int local = 0;
    int cbuf = 0;
    bool ok = true;
    for (int item = cta; item < num_items && ok; item += n_cta, ++local) {
      const int tile = item / splits, sp = item - tile * splits;
      const int m0 = tile_m0(tile), n0 = tile_n0(tile);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      mbar_wait(&bars->acc_full[acc], acc_phase, bars, status, 104);
      // the four epilogue warps must take the same branch: a timeout is published in abort_flag before
      // this barrier and read by everyone after it
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
        if (EPI == 2 || EPI == 5) {   // this thread's 64 output columns of the existing C, fetched while the TMEM load is in flight
          const long long gm = m0 + row;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int gn = n0 + chunk * 64 + j * 8;
            cin[j] = (gm < M && gn < N) ? __ldcg(reinterpret_cast<const uint4*>(c_in + gm * ldc + gn))
                                        : make_uint4(0u, 0u, 0u, 0u);
          }
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (splits > 1) {   // fp32 slice tile straight from the registers: 256 contiguous bytes per thread and chunk
          const long long gm = m0 + row;
          if (gm < M) {
            float* dst = partial + ((size_t)sp * M + gm) * N + n0 + chunk * 64;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int col = j * 4;
              if (n0 + chunk * 64 + col < N) {
                const uint32_t* v = col < 32 ? &v0[col] : &v1[col - 32];
                *reinterpret_cast<float4*>(dst + col) = make_float4(__uint_as_float(v[0]), __uint_as_float(v[1]),
                                                                    __uint_as_float(v[2]), __uint_as_float(v[3]));
              }
            }
          }
          continue;
        }
        // the staging buffer we are about to overwrite must have been read by its TMA store
        if (threadIdx.x == 64) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const uint32_t cs = c_stage + cbuf * C_CHUNK_BYTES + row * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {   // eight 16-byte pieces of this row, XOR-swizzled by (row % 8)
          float f[8], prev[8];
          if (EPI == 2 || EPI == 5) unpack8(cin[j], prev);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int col = j * 8 + e;
            float x = __uint_as_float(col < 32 ? v0[col] : v1[col - 32]);
            if (EPI == 1) { x = fmaxf(x, 0.f); x = x * x; }
            if (EPI == 2) x += prev[e];
            if (EPI == 3) x = 1.f - __fdividef(2.f, __expf(2.f * x) + 1.f);     // tanh, saturates cleanly at +-1
            if (EPI == 4) x = __fdividef(1.f, 1.f + __expf(-x));
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
      if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
    }
    if (threadIdx.x == 64) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
}

// ------------------------------------------------------------------------------------------ host side
using rwkv_tmap::make_map;   // encoded maps are cached per (address, shape, stride, box)

template <bool A_MN, bool B_MN, int EPI>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, int M, int N, int K, int* status,
           int sms, const bf16* c_in, long long ldc, cudaStream_t st) {
  auto kern = gemm_tcgen05_kernel<A_MN, B_MN, EPI, false>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)e;
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sms ? tiles : sms;
  AgParams none = {};
  kern<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ma, mb, mc, M, N, K, status, c_in, ldc, 1, nullptr, none);
  return rwkv_launch_status();
}

// Sums the `splits` fp32 slice tiles of a split-K product and writes bf16 C.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ partial, bf16* __restrict__ c, int M, int N, long long ldc, int splits) {
  const long long n4 = N / 4;
  const long long total = (long long)M * n4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / n4;
    const int n = (int)(i - m * n4) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sp = 0; sp < splits; ++sp) {
      const float4 v = *reinterpret_cast<const float4*>(partial + ((size_t)sp * M + m) * N + n);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<uint2*>(c + m * ldc + n) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
  }
}

template <bool A_MN, bool B_MN>
int launch_splitk(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, int M, int N, int K, int* status,
                  int sms, int splits, float* partial, bf16* c, long long ldc, cudaStream_t st) {
  auto kern = gemm_tcgen05_kernel<A_MN, B_MN, 0, false>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)e;
    configured = true;
  }
  const int items = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * splits;
  const int grid = items < sms ? items : sms;
  AgParams none = {};
  kern<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(ma, mb, mc, M, N, K, status, nullptr, 0, splits, partial, none);
  const long long total = (long long)M * (N / 4);
  long long blocks = (total + 255) / 256;
  if (blocks > sms * 8) blocks = sms * 8;
  splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, st>>>(partial, c, M, N, ldc, splits);
  return rwkv_launch_status();
}

template <int EPI>
int launch_ag(CUtensorMap ma, CUtensorMap mb, CUtensorMap mc, int M, int N, int K, int* status, int sms,
              AgParams ag, int* arrivals_io, const bf16* c_in, long long ldc, cudaStream_t st) {
  auto kern = gemm_tcgen05_kernel<false, false, EPI, true>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)e;
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sms ? tiles : sms;
  // every row block receives one arrival per CTA of the grid
  *arrivals_io += grid;
  ag.target = *arrivals_io;
  // tile producers wait for copy warps of other CTAs of the same grid: a cooperative launch guarantees that all
  // CTAs are resident together
  int splits = 1;
  float* partial = nullptr;
  void* args[] = {&ma, &mb, &mc, &M, &N, &K, &status, &c_in, &ldc, &splits, &partial, &ag};
  cudaError_t e = cudaLaunchCooperativeKernel((void*)kern, dim3(grid), dim3(NUM_THREADS + AG_COPY_WARPS * 32), args,
                                              SMEM_BYTES, st);
  return e == cudaSuccess ? rwkv_launch_status() : RWKV_ERR_CUDA_BASE + (int)e;
}

}  // namespace

// C[M,N] (row-major, ldc) = op(A) op(B) in bf16 with fp32 accumulation.
//   a_mn = 0: A is [M,K] row-major (lda);  a_mn = 1: A is stored [K,M] row-major (lda)
//   b_mn = 0: B is [N,K] row-major (ldb);  b_mn = 1: B is stored [K,N] row-major (ldb)
//   epilogue: 0 none, 1 relu(x)^2, 3 tanh, 4 sigmoid, 5 multiply by 2 sqrt(residual), 2 add a bf16 [M,N] matrix: `residual` (row stride ldr) or, when that is null,
//   the values already in C (in place).   status: device int, set non-zero if a device-side wait timed out.
RWKV_EXPORT int rwkv_gemm_bf16_tcgen05(const void* a, const void* b, void* c, int M, int N, int K, long long lda,
                                       long long ldb, long long ldc, int a_mn, int b_mn, int epilogue, void* status,
                                       const void* residual, long long ldr, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return RWKV_ERR_BAD_SHAPE;
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
  int r;
  r = a_mn ? make_map(&ma, a, K, M, lda, 64, BK) : make_map(&ma, a, M, K, lda, BK, BM);
  if (r) return r;
  r = b_mn ? make_map(&mb, b, K, N, ldb, 64, BK) : make_map(&mb, b, N, K, ldb, BK, BN);
  if (r) return r;
  r = make_map(&mc, c, M, N, ldc, 64, BM);
  if (r) return r;
  cudaStream_t st = (cudaStream_t)stream;
  int* sp = (int*)status;
  const bf16* cp = residual ? (const bf16*)residual : (const bf16*)c;
  if (residual) ldc = ldr;      // from here on ldc is only the row stride of the matrix added in the epilogue
#define DISPATCH(AM, BMN)                                                                        \
  (epilogue == 1   ? launch<AM, BMN, 1>(ma, mb, mc, M, N, K, sp, sms, cp, ldc, st)                \
   : epilogue == 2 ? launch<AM, BMN, 2>(ma, mb, mc, M, N, K, sp, sms, cp, ldc, st)                \
   : epilogue == 3 ? launch<AM, BMN, 3>(ma, mb, mc, M, N, K, sp, sms, cp, ldc, st)                \
   : epilogue == 4 ? launch<AM, BMN, 4>(ma, mb, mc, M, N, K, sp, sms, cp, ldc, st)                \
   : epilogue == 5 ? launch<AM, BMN, 5>(ma, mb, mc, M, N, K, sp, sms, cp, ldc, st)                \
                   : launch<AM, BMN, 0>(ma, mb, mc, M, N, K, sp, sms, cp, ldc, st))
  if (!a_mn && !b_mn) return DISPATCH(false, false);
  if (!a_mn && b_mn) return DISPATCH(false, true);
  if (a_mn && b_mn) return DISPATCH(true, true);
  return DISPATCH(true, false);
#undef DISPATCH
}

// Split-K variant of rwkv_gemm_bf16_tcgen05 (no epilogue): the contraction is cut into `splits` slices
// (1 < splits <= ceil(K / 64)), each (tile, slice) is one work item; `workspace` holds splits * M * N floats.
// N must be a multiple of 8.  For products with few output tiles and a long contraction.
RWKV_EXPORT int rwkv_gemm_bf16_tcgen05_splitk(const void* a, const void* b, void* c, int M, int N, int K, long long lda,
                                              long long ldb, long long ldc, int a_mn, int b_mn, int splits,
                                              void* workspace, void* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (N & 7) || splits < 2 || splits > (K + BK - 1) / BK || !workspace)
    return RWKV_ERR_BAD_SHAPE;
  if ((uintptr_t)workspace & 15) return RWKV_ERR_BAD_ALIGNMENT;
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap ma, mb, mc;
  int r;
  r = a_mn ? make_map(&ma, a, K, M, lda, 64, BK) : make_map(&ma, a, M, K, lda, BK, BM);
  if (r) return r;
  r = b_mn ? make_map(&mb, b, K, N, ldb, 64, BK) : make_map(&mb, b, N, K, ldb, BK, BN);
  if (r) return r;
  r = make_map(&mc, c, M, N, ldc, 64, BM);
  if (r) return r;
  cudaStream_t st = (cudaStream_t)stream;
  int* sp = (int*)status;
  float* ws = (float*)workspace;
  bf16* cp = (bf16*)c;
  if (!a_mn && !b_mn) return launch_splitk<false, false>(ma, mb, mc, M, N, K, sp, sms, splits, ws, cp, ldc, st);
  if (!a_mn && b_mn) return launch_splitk<false, true>(ma, mb, mc, M, N, K, sp, sms, splits, ws, cp, ldc, st);
  if (a_mn && b_mn) return launch_splitk<true, true>(ma, mb, mc, M, N, K, sp, sms, splits, ws, cp, ldc, st);
  return launch_splitk<true, false>(ma, mb, mc, M, N, K, sp, sms, splits, ws, cp, ldc, st);
}

// y[M,N] = x[M,K] @ W[N,K]^T where W is stored as `world` K-panels, panel p ([N, K/world], row-major) living at
// shard_ptrs[p] (peer-mapped addresses; shard_ptrs[rank] is local).  `staged` ([N,K] bf16, local) receives the
// gathered weight and can be reused afterwards (e.g. by the backward pass).  blk_count: ceil(N / 256)
// device ints, zero-initialised once; *arrivals_io: host-side running total of arrivals per counter (0 before the
// first call on these buffers), advanced by this call.
// x2 / w2 (optional): a second, local operand pair ([M, K2] and [N, K2], row-major contiguous) appended to the
// contraction: y = x W^T + x2 w2^T.  epilogue: 0 none, 1 relu(.)^2, 2 add `residual` ([M, N] bf16, row stride ldr).
RWKV_EXPORT int rwkv_ag_gemm_bf16_tcgen05_fused(const void* x, const unsigned long long* shard_ptrs, void* staged,
                                                void* y, int M, int N, int K, int rank, int world, void* blk_count,
                                                int* arrivals_io, void* status, const void* x2, const void* w2, int K2,
                                                int epilogue, const void* residual, long long ldr, void* stream) {
  if (K2 < 0 || (K2 > 0 && (!x2 || !w2))) return RWKV_ERR_BAD_SHAPE;
  if (epilogue < 0 || epilogue > 2 || (epilogue == 2 && (!residual || ((uintptr_t)residual & 15) || (ldr * 2) % 16)))
    return RWKV_ERR_BAD_SHAPE;
  if (M <= 0 || N <= 0 || K <= 0 || world <= 0 || world > MAX_RANKS || rank < 0 || rank >= world) return RWKV_ERR_BAD_SHAPE;
  if (K % world || (K / world) % BK || !arrivals_io || !blk_count) return RWKV_ERR_BAD_SHAPE;
  if (*arrivals_io > 0x70000000) return RWKV_ERR_TOO_LARGE;
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap ma, mb, mc;
  int r = make_map(&ma, x, M, K, K, BK, BM);
  if (r) return r;
  r = make_map(&mb, staged, N, K, K, BK, BN);
  if (r) return r;
  r = make_map(&mc, y, M, N, N, 64, BM);
  if (r) return r;
  AgParams ag = {};
  for (int i = 0; i < world; ++i) ag.shard[i] = reinterpret_cast<const bf16*>(shard_ptrs[i]);
  ag.staged = (bf16*)staged;
  ag.blk_count = (int*)blk_count;
  ag.rank = rank; ag.world = world; ag.Kp = K / world; ag.n_rb = (N + BN - 1) / BN;
  ag.group = ag.n_rb >= 16 ? 8 : 4;
  ag.K2 = K2;
  if (K2 > 0) {
    r = make_map(&ag.map_a2, x2, M, K2, K2, BK, BM);
    if (r) return r;
    r = make_map(&ag.map_b2, w2, N, K2, K2, BK, BN);
    if (r) return r;
  }
  const bf16* c_in = (const bf16*)residual;
  cudaStream_t st = (cudaStream_t)stream;
  if (epilogue == 1) return launch_ag<1>(ma, mb, mc, M, N, K, (int*)status, sms, ag, arrivals_io, nullptr, 0, st);
  if (epilogue == 2) return launch_ag<2>(ma, mb, mc, M, N, K, (int*)status, sms, ag, arrivals_io, c_in, ldr, st);
  return launch_ag<0>(ma, mb, mc, M, N, K, (int*)status, sms, ag, arrivals_io, nullptr, 0, st);
}

RWKV_EXPORT int rwkv_ag_gemm_bf16_tcgen05_dual(const void* x, const unsigned long long* shard_ptrs, void* staged, void* y,
                                               int M, int N, int K, int rank, int world, void* blk_count,
                                               int* arrivals_io, void* status, const void* x2, const void* w2, int K2,
                                               void* stream) {
  return rwkv_ag_gemm_bf16_tcgen05_fused(x, shard_ptrs, staged, y, M, N, K, rank, world, blk_count, arrivals_io, status,
                                         x2, w2, K2, 0, nullptr, 0, stream);
}

RWKV_EXPORT int rwkv_ag_gemm_bf16_tcgen05(const void* x, const unsigned long long* shard_ptrs, void* staged, void* y,
                                          int M, int N, int K, int rank, int world, void* blk_count,
                                          int* arrivals_io, void* status, void* stream) {
  return rwkv_ag_gemm_bf16_tcgen05_dual(x, shard_ptrs, staged, y, M, N, K, rank, world, blk_count, arrivals_io, status,
                                        nullptr, nullptr, 0, stream);
}
