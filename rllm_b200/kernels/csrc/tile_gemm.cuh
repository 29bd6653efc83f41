// A tile of C = A . B on CUDA cores with float32 accumulation, shared by the
// kernels whose matrix products are not one plain [M, K] x [N, K]^T: products
// per head over strided slices, and products per expert over gathered rows.
//
// 256 threads compute BM x 64 outputs; a thread owns BM / 16 rows x 4 columns
// and adds its k terms in the order k = 0 .. K-1, so an output depends on its
// own row of A and column of B only: not on the other rows of the tile, not on
// the tile it fell into.  A's rows are given as pointers (shared memory), so a
// caller may gather them; a null pointer is a row of zeros.  B is either
// [N, K] (an element (n, k) at B[n * ldb + k]) or [K, N] (at B[k * ldb + n]).
#pragma once
#include "common.cuh"

#define TG_BN 64
#define TG_BK 16
#define TG_THREADS 256

template <int BM>
struct TileGemmSmem {
  float As[TG_BK][BM + 4];
  float Bs[TG_BK][TG_BN + 4];
  const void* rows[BM];
};

template <typename T, int BM, bool B_KN>
__device__ __forceinline__ void tile_gemm_accumulate(TileGemmSmem<BM>& sm, const T* __restrict__ B,
                                                     long long ldb, int n0, int N, int K,
                                                     float (&acc)[BM / 16][4]) {
  constexpr int TM = BM / 16;
  const int tid = threadIdx.x;
  const int tm = (tid / 16) * TM, tn = (tid % 16) * 4;
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += TG_BK) {
#pragma unroll
    for (int u = 0; u < TM; ++u) {
      const int e = tid + TG_THREADS * u, r = e >> 4, kk = e & 15;
      const T* p = (const T*)sm.rows[r];
      sm.As[kk][r] = (p != nullptr && k0 + kk < K) ? to_f32(p[k0 + kk]) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = tid + TG_THREADS * u;
      if (B_KN) {
        const int kk = e >> 6, n = e & 63;
        sm.Bs[kk][n] = (k0 + kk < K && n0 + n < N) ? to_f32(B[(long long)(k0 + kk) * ldb + n0 + n]) : 0.f;
      } else {
        const int n = e >> 4, kk = e & 15;
        sm.Bs[kk][n] = (k0 + kk < K && n0 + n < N) ? to_f32(B[(long long)(n0 + n) * ldb + k0 + kk]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TG_BK; ++k) {
      float a[TM], b[4];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = sm.As[k][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = sm.Bs[k][tn + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
}
