// Small-M ("decode") GEMM:  y_i[M, N_i] = x_i[M, K_i] @ W_i[N_i, K_i]^T  for up to 8 problems in ONE launch.
//
// With M = number of sequences being decoded (tens to a few hundred) every projection is bound by streaming
// its weight matrix once, and a 24-layer step issues ~300 of them, so launch count matters as much as the
// kernel: the r/k/v projections (three inputs, three weights) or the four low-rank first stages go out as one
// grouped launch.  Each CTA owns 64 output columns of one problem (16 per warp), a block of 64 rows and one
// slice of K: every weight element is read exactly once from HBM, x comes from L2 once per 64 columns.  When
// there are fewer column tiles than SMs the contraction is split over blockIdx.z; partial sums meet in an fp32
// workspace through atomics and the LAST CTA to arrive at a tile (a counter, no waiting) converts it to bf16
// and leaves workspace and counter zeroed for the next call.  cp.async 3-stage ring, ldmatrix + mma.sync
// m16n8k16 (the tile is far too small for a 128-row tcgen05 instruction; the tensor pipe is idle either way).
// Replaces the cuBLAS calls behind nn.Linear on the rollout path (rwkvtune/models/rwkv7/model.py:134-172 at T=1).
#include "common.cuh"

namespace {

constexpr int SM_BM = 64, SM_BN = 64, SM_BK = 128, SM_STAGES = 3, SM_NT = 128;
constexpr int SM_LD = SM_BK + 8;   // padded row (bf16): 272-byte rows keep ldmatrix conflict-free

struct SmallMProblem {
  const bf16* x;
  const bf16* w;
  bf16* y;
  int N, K;
  long long ws_off;    // float offset of this problem's [M, N] partial-sum area
};
struct SmallMParams {
  SmallMProblem p[8];
  int tile_start[9];   // prefix sums of ceil(N_i / 64)
  int count, M, split_k;
  float* ws;
  unsigned* counters;  // one per (tile, m-block)
};

struct SmallMStage {
  bf16 xs[SM_BM][SM_LD];
  bf16 ws[SM_BN][SM_LD];
};

__device__ __forceinline__ uint32_t sm_s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void sm_cp16(void* dst, const void* src, bool pred) {
  const int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sm_s32(dst)), "l"(src), "r"(sz) : "memory");
}

__global__ void __launch_bounds__(SM_NT)
gemm_small_m_kernel(const __grid_constant__ SmallMParams prm) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ unsigned arrival;
  SmallMStage* st = reinterpret_cast<SmallMStage*>(smem_raw);
  int pi = 0;
#pragma unroll
  for (int i = 1; i < 8; ++i)
    if (i < prm.count && (int)blockIdx.x >= prm.tile_start[i]) pi = i;
  const SmallMProblem P = prm.p[pi];
  const int n0 = ((int)blockIdx.x - prm.tile_start[pi]) * SM_BN;
  const int m0 = blockIdx.y * SM_BM;
  const int M = prm.M, K = P.K, N = P.N;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // K slice of this CTA, in blocks of SM_BK
  const int nkb_all = (K + SM_BK - 1) / SM_BK;
  const int per = (nkb_all + prm.split_k - 1) / prm.split_k;
  const int kb0 = blockIdx.z * per;
  const int nkb = max(0, min(per, nkb_all - kb0));

  auto stage = [&](int i) {
    if (i < nkb) {
      SmallMStage& s = st[i % SM_STAGES];
      const int k0 = (kb0 + i) * SM_BK;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int e = tid + u * SM_NT, r = e >> 4, c = (e & 15) * 8;
        const bool okx = (m0 + r < M) && (k0 + c < K);
        sm_cp16(&s.xs[r][c], P.x + (size_t)(okx ? m0 + r : 0) * K + (okx ? k0 + c : 0), okx);
        const bool okw = (n0 + r < N) && (k0 + c < K);
        sm_cp16(&s.ws[r][c], P.w + (size_t)(okw ? n0 + r : 0) * K + (okw ? k0 + c : 0), okw);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float acc[4][2][4];
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mt][nt][e] = 0.f;
#pragma unroll
  for (int i = 0; i < SM_STAGES - 1; ++i) stage(i);
  for (int i = 0; i < nkb; ++i) {
    asm volatile("cp.async.wait_group %0;" ::"n"(SM_STAGES - 2) : "memory");
    __syncthreads();
    stage(i + SM_STAGES - 1);
    const SmallMStage& s = st[i % SM_STAGES];
#pragma unroll
    for (int kk = 0; kk < SM_BK / 16; ++kk) {
      uint32_t b[4];
      const int mi = lane >> 3, r = lane & 7;
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                   : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3])
                   : "r"(sm_s32(&s.ws[warp * 16 + (mi >> 1) * 8 + r][kk * 16 + (mi & 1) * 8])));
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        uint32_t a[4];
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
                     : "r"(sm_s32(&s.xs[mt * 16 + (lane & 15)][kk * 16 + (lane >> 4) * 8])));
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
          asm volatile(
              "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
              : "+f"(acc[mt][nt][0]), "+f"(acc[mt][nt][1]), "+f"(acc[mt][nt][2]), "+f"(acc[mt][nt][3])
              : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[nt * 2]), "r"(b[nt * 2 + 1]));
      }
    }
  }
  const int g = lane >> 2, tq = lane & 3;
  const int ncol = n0 + warp * 16 + tq * 2;     // this thread's first column (tile nt adds 8)
  if (prm.split_k == 1) {
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int m = m0 + mt * 16 + g + hh * 8;
        if (m < M) {
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
            if (ncol + nt * 8 < N)
              *reinterpret_cast<uint32_t*>(P.y + (size_t)m * N + ncol + nt * 8) =
                  pack_bf16(acc[mt][nt][hh * 2], acc[mt][nt][hh * 2 + 1]);
        }
      }
    return;
  }
  // split-K: add into the fp32 area, then the last CTA of this (tile, m-block) finishes the tile
  float* area = prm.ws + P.ws_off;
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int m = m0 + mt * 16 + g + hh * 8;
      if (m < M) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
          if (ncol + nt * 8 < N) {
            atomicAdd(area + (size_t)m * N + ncol + nt * 8, acc[mt][nt][hh * 2]);
            atomicAdd(area + (size_t)m * N + ncol + nt * 8 + 1, acc[mt][nt][hh * 2 + 1]);
          }
      }
    }
  __threadfence();
  __syncthreads();
  unsigned* ctr = prm.counters + blockIdx.y * gridDim.x + blockIdx.x;
  if (tid == 0) arrival = atomicAdd(ctr, 1u);
  __syncthreads();
  if (arrival != (unsigned)prm.split_k - 1) return;
  __threadfence();
  for (int e = tid; e < SM_BM * (SM_BN / 2); e += SM_NT) {
    const int r = e / (SM_BN / 2), c = (e % (SM_BN / 2)) * 2;
    const int m = m0 + r, n = n0 + c;
    if (m < M && n < N) {
      float2* src = reinterpret_cast<float2*>(area + (size_t)m * N + n);
      const float2 v = __ldcg(src);
      *reinterpret_cast<uint32_t*>(P.y + (size_t)m * N + n) = pack_bf16(v.x, v.y);
      __stcg(src, make_float2(0.f, 0.f));
    }
  }
  if (tid == 0) *ctr = 0u;
}

}  // namespace

// count <= 8 problems sharing M.  xs / ws / ys: host arrays of device pointers (bf16, row-major, 16-byte aligned);
// Ns / Ks: host arrays; every N even, every K a multiple of 8.  split_k > 1 needs `workspace` (fp32, at least
// sum_i M * N_i floats, zero before the first call; left zero on return) and `counters` (uint32, at least
// (sum_i ceil(N_i / 64)) * ceil(M / 64) entries, same rule).
RWKV_EXPORT int rwkv_gemm_small_m(const void* const* xs, const void* const* ws, void* const* ys, const int* Ns,
                                  const int* Ks, int count, int M, int split_k, void* workspace, void* counters,
                                  void* stream) {
  if (count <= 0 || count > 8 || M <= 0 || split_k < 1 || split_k > 64) return RWKV_ERR_BAD_SHAPE;
  if (split_k > 1 && (!workspace || !counters)) return RWKV_ERR_NOT_INITIALISED;
  SmallMParams prm;
  prm.count = count;
  prm.M = M;
  prm.split_k = split_k;
  prm.ws = (float*)workspace;
  prm.counters = (unsigned*)counters;
  int tiles = 0;
  long long off = 0;
  for (int i = 0; i < count; ++i) {
    if (Ns[i] <= 0 || Ns[i] % 2 || Ks[i] <= 0 || Ks[i] % 8) return RWKV_ERR_BAD_SHAPE;
    if (((uintptr_t)xs[i] | (uintptr_t)ws[i]) & 15) return RWKV_ERR_BAD_ALIGNMENT;
    if ((uintptr_t)ys[i] & 3) return RWKV_ERR_BAD_ALIGNMENT;
    prm.p[i] = SmallMProblem{(const bf16*)xs[i], (const bf16*)ws[i], (bf16*)ys[i], Ns[i], Ks[i], off};
    prm.tile_start[i] = tiles;
    tiles += (Ns[i] + SM_BN - 1) / SM_BN;
    off += (long long)M * Ns[i];
  }
  for (int i = count; i < 9; ++i) prm.tile_start[i] = tiles;
  static bool configured = false;
  const int smem = (int)(sizeof(SmallMStage) * SM_STAGES);
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_small_m_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return RWKV_ERR_CUDA_BASE + (int)e;
    configured = true;
  }
  dim3 grid(tiles, (M + SM_BM - 1) / SM_BM, split_k);
  gemm_small_m_kernel<<<grid, SM_NT, smem, (cudaStream_t)stream>>>(prm);
  return rwkv_launch_status();
}
