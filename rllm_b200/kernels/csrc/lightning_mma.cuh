// The lightning recurrence's chunk passes on the tensor cores (bfloat16 activations, mma.sync m16n8k16,
// float32 accumulators), for heads whose sizes are instantiated below.  For a chunk of C = 64 tokens with
// start state S_0 (float32 [d, dv]) and decay lambda:
//   pass 1 (end state from zero):   Z = (K * w)^T V,                 w_j = lambda^(n - 1 - j)
//   pass 2 (outputs):               O = ((Q K^T) * D) V + diag(lambda^(t + 1)) (Q S_0),
//                                   D[t, j] = lambda^(t - j) for j <= t, else 0
// with Q, K, V the chunk's activated rows (silu in float32, then rounded to bfloat16: a projection's
// activation).  What is float32 by this design's rules never passes through one bfloat16 number: the
// weights (Q K^T) * D, the start state S_0 and the weighted keys K * w each go into their product as the
// sum of two bfloat16 numbers (value and remainder), which keeps 16 bits of mantissa, and all sums are
// float32.  Every operand lies in shared memory as it lies in global memory (tokens by channels, the state
// [d][dv]); where a product sums over the rows of such an array (V, S_0, K * w), its fragments come from
// ldmatrix with .trans.
#pragma once
#include "tile_gemm_mma.cuh"

#define LTC_CHUNK 64
#define LTC_THREADS 256
template <int D, int DV> struct LtcSmem1 {
  bf16 kh[LTC_CHUNK][D + 8], kl[LTC_CHUNK][D + 8], v[LTC_CHUNK][DV + 8];
};
// pass 2 works on DVB value columns a block (all of them, or half where two blocks then fit an SM)
template <int D, int DVB> struct LtcSmem2 {
  bf16 q[LTC_CHUNK][D + 8], k[LTC_CHUNK][D + 8], v[LTC_CHUNK][DVB + 8], sh[D][DVB + 8], sl[D][DVB + 8];
};
template <int D, int DV> struct LtcSplit { static constexpr int N = (D > 64 && DV > 64) ? 2 : 1; };

__device__ __forceinline__ float ltc_silu(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ uint32_t ltc_pack(bf16 a, bf16 b) {
  __nv_bfloat162 p;
  p.x = a;
  p.y = b;
  return *(uint32_t*)&p;
}
// lambda^e for an integer e >= 0 (lambda^0 = 1 also where lambda is 0)
__device__ __forceinline__ float ltc_pow(float log2_lam, int e) { return e == 0 ? 1.0f : exp2f((float)e * log2_lam); }

__device__ __forceinline__ void ltc_ldmatrix4_trans(uint32_t (&r)[4], const void* smem_row) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// Fragments from row-major shared arrays with LD elements a row.
// ltc_a / ltc_b: the array's rows are the product's rows (A: [m][k]; B: [n][k], two n-tiles of 8).
// ltc_a_t / ltc_b_t: the array's rows are the summed index ([k][m], [k][n]): the 8 x 8 blocks are transposed
// by the load.
template <int LD>
__device__ __forceinline__ void ltc_a(uint32_t (&a)[4], const bf16* base, int r0, int k0) {
  const int lane = threadIdx.x & 31;
  tgm_ldmatrix4(a, base + (size_t)(r0 + (lane & 15)) * LD + k0 + (lane >> 4) * 8);
}
template <int LD>
__device__ __forceinline__ void ltc_b(uint32_t (&b)[4], const bf16* base, int n0, int k0) {
  const int lane = threadIdx.x & 31;
  tgm_ldmatrix4(b, base + (size_t)(n0 + (lane & 7) + ((lane >> 4) & 1) * 8) * LD + k0 + ((lane >> 3) & 1) * 8);
}
template <int LD>
__device__ __forceinline__ void ltc_a_t(uint32_t (&a)[4], const bf16* base, int m0, int k0) {
  const int lane = threadIdx.x & 31;
  ltc_ldmatrix4_trans(a, base + (size_t)(k0 + (lane & 7) + ((lane >> 4) & 1) * 8) * LD + m0 + ((lane >> 3) & 1) * 8);
}
template <int LD>
__device__ __forceinline__ void ltc_b_t(uint32_t (&b)[4], const bf16* base, int n0, int k0) {
  const int lane = threadIdx.x & 31;
  ltc_ldmatrix4_trans(b, base + (size_t)(k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + n0 + ((lane >> 4) & 1) * 8);
}

// Four consecutive projections of a token's row, activated (zeros behind the chunk's n tokens).  `wide`: the
// rows are 8-byte aligned and one load fetches the four.
__device__ __forceinline__ void ltc_fetch4(const bf16* src, bool on, bool wide, float (&o)[4]) {
  if (!on) {
    o[0] = o[1] = o[2] = o[3] = 0.f;
  } else if (wide) {
    const uint2 raw = *(const uint2*)src;
    const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
    o[0] = ltc_silu(a.x); o[1] = ltc_silu(a.y); o[2] = ltc_silu(b.x); o[3] = ltc_silu(b.y);
  } else {
#pragma unroll
    for (int x = 0; x < 4; ++x) o[x] = ltc_silu(__bfloat162float(src[x]));
  }
}
__device__ __forceinline__ void ltc_store4(bf16* dst, const float (&o)[4]) {
  uint2 t;
  *(__nv_bfloat162*)&t.x = __floats2bfloat162_rn(o[0], o[1]);
  *(__nv_bfloat162*)&t.y = __floats2bfloat162_rn(o[2], o[3]);
  *(uint2*)dst = t;
}

// a chunk's rows of one projection into shared memory [token][W + 8], activated and rounded
// (W columns from column `col0` of the head's HW)
template <int W, int HW>
__device__ __forceinline__ void ltc_stage_rows(bf16 (*dst)[W + 8], const bf16* src, int stride, int t0, int n, int h,
                                               int col0, bool wide) {
#pragma unroll
  for (int e0 = 0; e0 < LTC_CHUNK * W; e0 += LTC_THREADS * 4) {
    const int e = e0 + threadIdx.x * 4;
    const int j = e / W, c = e - j * W;
    float o[4];
    ltc_fetch4(src + (size_t)(t0 + j) * stride + (size_t)h * HW + col0 + c, j < n, wide, o);
    ltc_store4(&dst[j][c], o);
  }
}

template <int D, int DV>
__global__ void __launch_bounds__(LTC_THREADS)
lightning_mma_pass1_kernel(const bf16* k, const bf16* v, int stride, int wide, const float* decay, float* work,
                           const int* q_start, int max_chunks, int heads) {
  extern __shared__ __align__(16) unsigned char ltc_raw[];
  LtcSmem1<D, DV>& sm = *reinterpret_cast<LtcSmem1<D, DV>*>(ltc_raw);
  pdl_wait();
  pdl_launch();
  const int h = blockIdx.x, s = blockIdx.y / max_chunks, chunk = blockIdx.y % max_chunks;
  const int t0 = q_start[s] + chunk * LTC_CHUNK;
  const int n = min(LTC_CHUNK, q_start[s + 1] - t0);
  if (n <= 0) return;
  const float l2 = log2f(decay[h]);
#pragma unroll
  for (int e0 = 0; e0 < LTC_CHUNK * D; e0 += LTC_THREADS * 4) {
    const int e = e0 + threadIdx.x * 4;
    const int j = e / D, i = e - j * D;
    float o[4], hi[4], lo[4];
    ltc_fetch4(k + (size_t)(t0 + j) * stride + (size_t)h * D + i, j < n, wide != 0, o);
    const float w = (j < n) ? ltc_pow(l2, n - 1 - j) : 0.f;
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const float kw = __bfloat162float(__float2bfloat16_rn(o[x])) * w;      // the rounded key, weighted
      hi[x] = __bfloat162float(__float2bfloat16_rn(kw));
      lo[x] = kw - hi[x];
    }
    ltc_store4(&sm.kh[j][i], hi);
    ltc_store4(&sm.kl[j][i], lo);
  }
  ltc_stage_rows<DV, DV>(sm.v, v, stride, t0, n, h, 0, wide != 0);
  __syncthreads();
  // a warp owns DV / 4 value columns and half of the d rows
  constexpr int MT = D / 32, NT = DV / 32;
  static_assert(NT >= 2 && NT % 2 == 0 && MT >= 1, "a warp takes pairs of n-tiles and whole m-tiles");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, c0 = (warp & 3) * (DV / 4), m0 = (warp >> 2) * (D / 2);
  float acc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int x = 0; x < 4; ++x) acc[mt][nt][x] = 0.f;
#pragma unroll
  for (int kk = 0; kk < LTC_CHUNK; kk += 16) {
    uint32_t b[NT / 2][4];
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) ltc_b_t<DV + 8>(b[np], &sm.v[0][0], c0 + np * 16, kk);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      uint32_t ah[4], al[4];
      ltc_a_t<D + 8>(ah, &sm.kh[0][0], m0 + mt * 16, kk);
      ltc_a_t<D + 8>(al, &sm.kl[0][0], m0 + mt * 16, kk);
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        tgm_mma(acc[mt][2 * np], ah, b[np][0], b[np][1]);
        tgm_mma(acc[mt][2 * np + 1], ah, b[np][2], b[np][3]);
        tgm_mma(acc[mt][2 * np], al, b[np][0], b[np][1]);
        tgm_mma(acc[mt][2 * np + 1], al, b[np][2], b[np][3]);
      }
    }
  }
  float* z = work + ((size_t)blockIdx.y * heads + h) * D * DV;
  const int g = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int c = c0 + nt * 8 + 2 * tq;
      *(float2*)(z + (size_t)(m0 + mt * 16 + g) * DV + c) = make_float2(acc[mt][nt][0], acc[mt][nt][1]);
      *(float2*)(z + (size_t)(m0 + mt * 16 + g + 8) * DV + c) = make_float2(acc[mt][nt][2], acc[mt][nt][3]);
    }
}

template <int D, int DV>
__global__ void __launch_bounds__(LTC_THREADS)
lightning_mma_pass2_kernel(const bf16* q, const bf16* k, const bf16* v, int stride, int wide, const float* decay,
                           const float* work, const int* q_start, int max_chunks, float* out, int heads) {
  constexpr int DVB = DV / LtcSplit<D, DV>::N;
  extern __shared__ __align__(16) unsigned char ltc_raw[];
  LtcSmem2<D, DVB>& sm = *reinterpret_cast<LtcSmem2<D, DVB>*>(ltc_raw);
  pdl_wait();
  pdl_launch();
  const int h = blockIdx.x, s = blockIdx.y / max_chunks, chunk = blockIdx.y % max_chunks;
  const int cb = blockIdx.z * DVB;                // this block's value columns
  const int t0 = q_start[s] + chunk * LTC_CHUNK;
  const int n = min(LTC_CHUNK, q_start[s + 1] - t0);
  if (n <= 0) return;
  const float l2 = log2f(decay[h]);
  ltc_stage_rows<D, D>(sm.q, q, stride, t0, n, h, 0, wide != 0);
  ltc_stage_rows<D, D>(sm.k, k, stride, t0, n, h, 0, wide != 0);
  ltc_stage_rows<DVB, DV>(sm.v, v, stride, t0, n, h, cb, wide != 0);
  const float* s0 = work + ((size_t)blockIdx.y * heads + h) * D * DV;      // the chunk's start state [i][c]
#pragma unroll 8
  for (int e0 = 0; e0 < D * DVB; e0 += LTC_THREADS * 4) {
    const int e = e0 + threadIdx.x * 4;
    const int i = e / DVB, c = e - i * DVB;
    const float4 x = *(const float4*)(s0 + (size_t)i * DV + cb + c);
    float hi[4] = {x.x, x.y, x.z, x.w}, lo[4];
#pragma unroll
    for (int y = 0; y < 4; ++y) {
      const float r = __bfloat162float(__float2bfloat16_rn(hi[y]));
      lo[y] = hi[y] - r;
      hi[y] = r;
    }
    ltc_store4(&sm.sh[i][c], hi);
    ltc_store4(&sm.sl[i][c], lo);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int r0 = (warp & 3) * 16;                 // this warp's 16 tokens,
  const int cbase = (warp >> 2) * (DVB / 2);      // and its half of the block's value columns (the weights are computed
  if (r0 >= n) return;                            // by every warp that needs them)
  constexpr int NT = DVB / 16;
  static_assert(NT >= 2 && NT % 2 == 0, "a warp takes pairs of n-tiles");
  float o[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int x = 0; x < 4; ++x) o[nt][x] = 0.f;
  // what the start state gives: (Q S_0), the state as value + remainder; then row t times lambda^(t + 1)
#pragma unroll
  for (int kk = 0; kk < D; kk += 16) {
    uint32_t a[4];
    ltc_a<D + 8>(a, &sm.q[0][0], r0, kk);
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t bh[4], bl[4];
      ltc_b_t<DVB + 8>(bh, &sm.sh[0][0], cbase + np * 16, kk);
      ltc_b_t<DVB + 8>(bl, &sm.sl[0][0], cbase + np * 16, kk);
      tgm_mma(o[2 * np], a, bh[0], bh[1]);
      tgm_mma(o[2 * np + 1], a, bh[2], bh[3]);
      tgm_mma(o[2 * np], a, bl[0], bl[1]);
      tgm_mma(o[2 * np + 1], a, bl[2], bl[3]);
    }
  }
  const float up = ltc_pow(l2, r0 + g + 1), dn = ltc_pow(l2, r0 + g + 9);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    o[nt][0] *= up; o[nt][1] *= up;
    o[nt][2] *= dn; o[nt][3] *= dn;
  }
  // the chunk's own tokens: scores against the keys up to this warp's last row, times the decays
  float p[LTC_CHUNK / 8][4];
#pragma unroll
  for (int nt = 0; nt < LTC_CHUNK / 8; ++nt)
#pragma unroll
    for (int x = 0; x < 4; ++x) p[nt][x] = 0.f;
#pragma unroll
  for (int kk = 0; kk < D; kk += 16) {
    uint32_t a[4];
    ltc_a<D + 8>(a, &sm.q[0][0], r0, kk);
#pragma unroll
    for (int np = 0; np < LTC_CHUNK / 16; ++np) {
      if (np * 16 <= r0) {                         // later keys are hidden from all 16 rows (one branch a warp)
        uint32_t b[4];
        ltc_b<D + 8>(b, &sm.k[0][0], np * 16, kk);
        tgm_mma(p[2 * np], a, b[0], b[1]);
        tgm_mma(p[2 * np + 1], a, b[2], b[3]);
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < LTC_CHUNK / 8; ++nt)
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int t = r0 + g + 8 * (x >> 1), j = nt * 8 + 2 * tq + (x & 1);
      p[nt][x] = (j <= t) ? p[nt][x] * ltc_pow(l2, t - j) : 0.f;
    }
  // weights times values, the weights as value + remainder
#pragma unroll
  for (int ks = 0; ks < LTC_CHUNK / 16; ++ks) {
    if (ks * 16 <= r0) {
      uint32_t ah[4], al[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        // fragment element x: n-tile 2 ks + (x >> 1), accumulator pair (x & 1): rows g and g + 8
        const float f0 = p[2 * ks + (x >> 1)][2 * (x & 1)], f1 = p[2 * ks + (x >> 1)][2 * (x & 1) + 1];
        const bf16 h0 = __float2bfloat16_rn(f0), h1 = __float2bfloat16_rn(f1);
        ah[x] = ltc_pack(h0, h1);
        al[x] = ltc_pack(__float2bfloat16_rn(f0 - __bfloat162float(h0)), __float2bfloat16_rn(f1 - __bfloat162float(h1)));
      }
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        uint32_t b[4];
        ltc_b_t<DVB + 8>(b, &sm.v[0][0], cbase + np * 16, ks * 16);
        tgm_mma(o[2 * np], ah, b[0], b[1]);
        tgm_mma(o[2 * np + 1], ah, b[2], b[3]);
        tgm_mma(o[2 * np], al, b[0], b[1]);
        tgm_mma(o[2 * np + 1], al, b[2], b[3]);
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int c = cb + cbase + nt * 8 + 2 * tq;
    const int ta = r0 + g, tb = r0 + g + 8;
    if (ta < n) *(float2*)(out + ((size_t)(t0 + ta) * heads + h) * DV + c) = make_float2(o[nt][0], o[nt][1]);
    if (tb < n) *(float2*)(out + ((size_t)(t0 + tb) * heads + h) * DV + c) = make_float2(o[nt][2], o[nt][3]);
  }
}

// Launches the two passes around `chain` (the caller's kernel that turns end-from-zero states into start
// states).  Returns false if this head shape is not instantiated.
template <int D, int DV, typename Chain>
static bool ltc_launch(const bf16* q, const bf16* k, const bf16* v, int stride, const float* decay, float* work,
                       const int* q_start, int num_seqs, int max_chunks, float* out, int heads, cudaStream_t stream,
                       Chain chain) {
  const dim3 grid(heads, num_seqs * max_chunks);
  const size_t s1 = sizeof(LtcSmem1<D, DV>), s2 = sizeof(LtcSmem2<D, DV / LtcSplit<D, DV>::N>);
  static bool allowed = false;
  if (!allowed) {
    cudaFuncSetAttribute(lightning_mma_pass1_kernel<D, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s1);
    cudaFuncSetAttribute(lightning_mma_pass2_kernel<D, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s2);
    allowed = true;
  }
  // rows that start on 8-byte boundaries are fetched four values a load
  const int wide = stride % 4 == 0 && (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 7) == 0;
  rllm_launch_pdl(lightning_mma_pass1_kernel<D, DV>, grid, dim3(LTC_THREADS), s1, stream, k, v, stride, wide, decay, work,
                  q_start, max_chunks, heads);
  chain();
  rllm_launch_pdl(lightning_mma_pass2_kernel<D, DV>, dim3(grid.x, grid.y, LtcSplit<D, DV>::N), dim3(LTC_THREADS), s2, stream, q, k, v, stride, wide, decay,
                  (const float*)work, q_start, max_chunks, out, heads);
  return true;
}
