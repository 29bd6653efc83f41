// The tile of tile_gemm.cuh on the tensor cores, for bfloat16: C = A . B^T with A's rows
// given as pointers (gathered rows, null = zeros) and one or two B matrices [N, K] that
// share the A tile (a gate and an up projection, say).  128 threads, a tile of BM x 64
// outputs per B matrix, k in steps of 32 through a cp.async ring of four stages (dynamic
// shared memory: the caller passes sizeof(MmaTileSmem<BM, NB>) at the launch),
// mma.sync m16n8k16 with float32 accumulators.  An output's k terms are added in the
// same order whatever else is in the tile, and BM = 16 and BM = 64 give the same bits.
// Needs K % 8 == 0 and 16-byte aligned rows of A and B.
#pragma once
#include "common.cuh"

#define TGM_THREADS 128
#define TGM_BN 64
#define TGM_BK 32
#define TGM_LD (TGM_BK + 8)      // bf16 elements per shared row: 80 bytes, conflict-free fragment loads

#define TGM_STAGES 4

template <int BM, int NB>
struct MmaTileSmem {
  bf16 A[TGM_STAGES][BM][TGM_LD];
  bf16 B[TGM_STAGES][NB * TGM_BN][TGM_LD];
  const void* rows[BM];
};

// the kernel's dynamic shared memory as the tile's buffers
template <int BM, int NB>
__device__ __forceinline__ MmaTileSmem<BM, NB>& tgm_smem() {
  extern __shared__ __align__(16) unsigned char tgm_raw[];
  return *reinterpret_cast<MmaTileSmem<BM, NB>*>(tgm_raw);
}
template <typename K, int BM, int NB>
static inline void tgm_allow_smem(K kernel) {
  if (sizeof(MmaTileSmem<BM, NB>) > 48 * 1024)
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(MmaTileSmem<BM, NB>));
}

__device__ __forceinline__ void tgm_cp16(void* smem_dst, const void* src, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void tgm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tgm_wait_ring() { asm volatile("cp.async.wait_group %0;" ::"n"(TGM_STAGES - 2) : "memory"); }

__device__ __forceinline__ void tgm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void tgm_ldmatrix4(uint32_t (&r)[4], const void* smem_row) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// NT: n-tiles of 8 columns a warp owns (BM 64: 8, all 64 columns of its 16 rows; BM 16: 2)
template <int BM> struct TgmShape { static constexpr int NT = (BM == 64) ? 8 : 2; };

// What a thread copies in every stage, worked out once: its 16-byte chunk sits at the same k offset
// (kc) of every row it serves, rows (tid + 128 i) / 4 of A and of each B matrix; a null pointer is zeros.
template <int BM, int NB>
struct TgmPlan {
  static constexpr int AS = (BM * 4 + TGM_THREADS - 1) / TGM_THREADS;
  const bf16* a[AS];
  const bf16* b[NB][2];
  int kc;
};

template <int BM, int NB>
__device__ __forceinline__ void tgm_plan(TgmPlan<BM, NB>& p, const MmaTileSmem<BM, NB>& sm, const bf16* const (&B)[NB],
                                         long long ldb, int n0, int N) {
  const int tid = threadIdx.x;
  p.kc = (tid & 3) * 8;
#pragma unroll
  for (int i = 0; i < TgmPlan<BM, NB>::AS; ++i) {
    const int r = (tid + TGM_THREADS * i) >> 2;
    const bf16* row = (r < BM) ? (const bf16*)sm.rows[r] : nullptr;
    p.a[i] = row ? row + p.kc : nullptr;
  }
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int n = (tid + TGM_THREADS * i) >> 2;
      p.b[b][i] = (n0 + n < N) ? B[b] + (long long)(n0 + n) * ldb + p.kc : nullptr;
    }
}

template <int BM, int NB>
__device__ __forceinline__ void tgm_load_stage(MmaTileSmem<BM, NB>& sm, int st, const TgmPlan<BM, NB>& p,
                                               const void* dummy, int K, int k0) {
  const int tid = threadIdx.x;
  const bool in_k = k0 + p.kc < K;
#pragma unroll
  for (int i = 0; i < TgmPlan<BM, NB>::AS; ++i) {
    const int r = (tid + TGM_THREADS * i) >> 2;
    if (r < BM) {
      const bool ok = in_k && p.a[i] != nullptr;
      tgm_cp16(&sm.A[st][r][p.kc], ok ? (const void*)(p.a[i] + k0) : dummy, ok);
    }
  }
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int n = (tid + TGM_THREADS * i) >> 2;
      const bool ok = in_k && p.b[b][i] != nullptr;
      tgm_cp16(&sm.B[st][b * TGM_BN + n][p.kc], ok ? (const void*)(p.b[b][i] + k0) : dummy, ok);
    }
}

// How the tile is shared out.  BM 64: the four warps form a 2 x 2 grid of 32 x 32 outputs (two row tiles of
// 16 by four n-tiles of 8 a warp), so a warp reads half of A's and half of B's rows of a stage.  BM 16: a warp
// owns 16 columns (two n-tiles) of the 16 rows.  acc[b][nt][4] holds B matrix b's fragments, nt = row tile * NTL
// + n-tile; tgm_coord gives the output (row, col) within the CTA's tile of element i of fragment nt.
template <int BM>
__device__ __forceinline__ void tgm_coord(int nt, int i, int& row, int& col) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  if (BM == 64) {
    row = (warp >> 1) * 32 + (nt >> 2) * 16 + g + 8 * (i >> 1);
    col = (warp & 1) * 32 + (nt & 3) * 8 + 2 * t + (i & 1);
  } else {
    row = g + 8 * (i >> 1);
    col = warp * 16 + nt * 8 + 2 * t + (i & 1);
  }
}

template <int BM, int NB>
__device__ __forceinline__ void tile_gemm_mma(MmaTileSmem<BM, NB>& sm, const bf16* const (&B)[NB], long long ldb,
                                              int n0, int N, int K, float (&acc)[NB][TgmShape<BM>::NT][4]) {
  constexpr int NT = TgmShape<BM>::NT;
  constexpr int MTW = (BM == 64) ? 2 : 1, NTL = NT / MTW;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row0 = (BM == 64) ? (warp >> 1) * 32 : 0;
  const int col0 = (BM == 64) ? (warp & 1) * 32 : warp * 16;
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[b][nt][i] = 0.f;
  const int steps = (K + TGM_BK - 1) / TGM_BK;
  // a group is committed for every step of the ring, also an empty one, so that "all but the last
  // TGM_STAGES - 2 groups have landed" always means: the stage about to be read has
  TgmPlan<BM, NB> plan;
  tgm_plan<BM, NB>(plan, sm, B, ldb, n0, N);
  for (int s = 0; s < TGM_STAGES - 1; ++s) {
    if (s < steps) tgm_load_stage<BM, NB>(sm, s, plan, B[0], K, s * TGM_BK);
    tgm_commit();
  }
  for (int s = 0; s < steps; ++s) {
    const int st = s % TGM_STAGES;
    tgm_wait_ring();
    __syncthreads();               // stage st has landed for everyone, and everyone has left step s - 1
    if (s + TGM_STAGES - 1 < steps)
      tgm_load_stage<BM, NB>(sm, (s + TGM_STAGES - 1) % TGM_STAGES, plan, B[0], K, (s + TGM_STAGES - 1) * TGM_BK);
    tgm_commit();
#pragma unroll
    for (int kk = 0; kk < TGM_BK; kk += 16) {
      // fragments by ldmatrix: A's 16 x 16 in one, B's 8 x 16 of two n-tiles in one
      uint32_t a[MTW][4];
#pragma unroll
      for (int mt = 0; mt < MTW; ++mt)
        tgm_ldmatrix4(a[mt], &sm.A[st][row0 + mt * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int nt = 0; nt < NTL; nt += 2) {
          uint32_t bb[4];
          tgm_ldmatrix4(bb, &sm.B[st][b * TGM_BN + col0 + nt * 8 + (lane & 7) + ((lane >> 4) & 1) * 8][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
          for (int mt = 0; mt < MTW; ++mt) {
            tgm_mma(acc[b][mt * NTL + nt], a[mt], bb[0], bb[1]);
            tgm_mma(acc[b][mt * NTL + nt + 1], a[mt], bb[2], bb[3]);
          }
        }
    }
  }
  __syncthreads();
}

// whether RLLM_TILE_GEMM=simt keeps these products on the CUDA cores (for tests and comparisons)
static inline bool tgm_disabled() {
  static int off = -1;
  if (off < 0) { const char* e = getenv("RLLM_TILE_GEMM"); off = (e && e[0] == 's') ? 1 : 0; }
  return off == 1;
}
