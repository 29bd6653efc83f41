// Hyper-connections: the residual is S parallel streams x_1 .. x_S (float32,
// [S, T, H]) instead of one.  A sublayer reads a weighted sum of the streams,
//   u = sum_s a[s] x_s,
// and its result y is written back into all streams at once, from the old ones,
//   x_t <- sum_s M[s, t] x_s + b[t] * (g * y)          (g: a per-channel scale, may be absent),
// with a [S], M [S, S] ("from" row, "to" column) and b [S] learned per sublayer.
// Everything is element-wise over (token, channel), so the kernels here fuse what
// follows: the write-back of one sublayer, the read of the next and the norm on
// that read are one pass over the streams.
//
// The norm that can be fused is the dynamic tanh, which needs no statistics:
//   n(u) = tanh(alpha * u) * w + c        (alpha a scalar; w, c [H]).
// All arithmetic is float32; only the norm's output is rounded to the activation
// dtype.  A row's result depends on that row alone.
#include "common.cuh"
#include <math.h>

#define HS_MAX_STREAMS 8
#define HS_THREADS 256

// four (or one) consecutive values in registers
template <int V> struct HsVec { float v[V]; };
template <int V> __device__ __forceinline__ HsVec<V> hs_ld(const float* p) {
  HsVec<V> r;
  if (V == 4) { const float4 t = *(const float4*)p; r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; }
  else r.v[0] = p[0];
  return r;
}
template <int V> __device__ __forceinline__ HsVec<V> hs_ld(const bf16* p) {
  HsVec<V> r;
  if (V == 4) {
    const uint2 t = *(const uint2*)p;
    const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&t.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&t.y);
    r.v[0] = a.x; r.v[1] = a.y; r.v[2] = b.x; r.v[3] = b.y;
  } else r.v[0] = __bfloat162float(p[0]);
  return r;
}
template <int V> __device__ __forceinline__ void hs_st(float* p, const HsVec<V>& r) {
  if (V == 4) *(float4*)p = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
  else p[0] = r.v[0];
}
template <int V> __device__ __forceinline__ void hs_st(bf16* p, const HsVec<V>& r) {
  if (V == 4) {
    uint2 t;
    *(__nv_bfloat162*)&t.x = __floats2bfloat162_rn(r.v[0], r.v[1]);
    *(__nv_bfloat162*)&t.y = __floats2bfloat162_rn(r.v[2], r.v[3]);
    *(uint2*)p = t;
  } else p[0] = __float2bfloat16_rn(r.v[0]);
}

// The coefficient tensors are tiny weights (no kernel writes them, so they may be read before the dependency
// wait); a block brings them into shared memory once.
struct HsCoeff {
  float a[HS_MAX_STREAMS];                       // read weights (of the read this kernel performs)
  float m[HS_MAX_STREAMS * HS_MAX_STREAMS];      // mix [from][to]
  float b[HS_MAX_STREAMS];                       // write weights
};

// out[r, :] = norm(sum_s a[s] xs[s, row(r), :]);  a == nullptr: all ones (the plain sum of the streams).
// norm_w == nullptr: no norm (out is then float32, the sum itself).  A thread takes V consecutive channels.
template <typename TO, typename TW, int V>
__global__ void __launch_bounds__(HS_THREADS)
hs_read_kernel(const float* xs, const float* a, const int* rows, const float* alpha, const TW* norm_w,
               const TW* norm_c, TO* out, int S, long long T, int H, long long total) {
  __shared__ HsCoeff co;
  if (threadIdx.x < S) co.a[threadIdx.x] = a ? a[threadIdx.x] : 1.0f;
  const float al = alpha ? alpha[0] : 0.f;
  __syncthreads();
  pdl_wait();
  pdl_launch();
  const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (idx >= total) return;
  const long long r = idx / H;
  const int i = (int)(idx - r * H);
  const long long src = rows ? (long long)rows[r] : r;
  HsVec<V> u;
#pragma unroll
  for (int e = 0; e < V; ++e) u.v[e] = 0.f;
  for (int s = 0; s < S; ++s) {
    const HsVec<V> x = hs_ld<V>(xs + ((size_t)s * T + src) * H + i);
#pragma unroll
    for (int e = 0; e < V; ++e) u.v[e] = fmaf(co.a[s], x.v[e], u.v[e]);
  }
  if (norm_w) {
    const HsVec<V> w = hs_ld<V>(norm_w + i), c = hs_ld<V>(norm_c + i);
#pragma unroll
    for (int e = 0; e < V; ++e) u.v[e] = fmaf(tanhf(al * u.v[e]), w.v[e], c.v[e]);
  }
  hs_st<V>(out + idx, u);
}

// xs (in place): x_t <- sum_s M[s, t] x_s + b[t] * g * y;  then, if a_next is given, the next read and its
// norm: out = norm(sum_t a_next[t] x_t).  sum_out (float32 [T, H], optional): the plain sum of the new streams.
template <typename TY, typename TO, typename TW, int V>
__global__ void __launch_bounds__(HS_THREADS)
hs_write_kernel(float* xs, const TY* y, const TW* g, const float* m, const float* b, const float* a_next,
                const float* alpha, const TW* norm_w, const TW* norm_c, TO* out, float* sum_out, int S,
                long long T, int H, long long total) {
  __shared__ HsCoeff co;
  for (int e = threadIdx.x; e < S * S; e += blockDim.x) co.m[e] = m[e];
  if (threadIdx.x < S) {
    co.b[threadIdx.x] = b[threadIdx.x];
    co.a[threadIdx.x] = a_next ? a_next[threadIdx.x] : 0.f;
  }
  const float al = alpha ? alpha[0] : 0.f;
  __syncthreads();
  pdl_wait();
  pdl_launch();
  const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (idx >= total) return;
  const int i = (int)(idx % H);
  HsVec<V> x[HS_MAX_STREAMS];
#pragma unroll
  for (int s = 0; s < HS_MAX_STREAMS; ++s)
    if (s < S) x[s] = hs_ld<V>(xs + (size_t)s * T * H + idx);
  HsVec<V> yy = hs_ld<V>(y + idx);
  if (g) {
    const HsVec<V> gg = hs_ld<V>(g + i);
#pragma unroll
    for (int e = 0; e < V; ++e) yy.v[e] *= gg.v[e];
  }
  HsVec<V> u, all;
#pragma unroll
  for (int e = 0; e < V; ++e) u.v[e] = all.v[e] = 0.f;
  for (int t = 0; t < S; ++t) {
    HsVec<V> v;
#pragma unroll
    for (int e = 0; e < V; ++e) v.v[e] = 0.f;
#pragma unroll
    for (int s = 0; s < HS_MAX_STREAMS; ++s) {
      if (s < S) {
#pragma unroll
        for (int e = 0; e < V; ++e) v.v[e] = fmaf(co.m[s * S + t], x[s].v[e], v.v[e]);
      }
    }
#pragma unroll
    for (int e = 0; e < V; ++e) {
      v.v[e] = fmaf(co.b[t], yy.v[e], v.v[e]);
      u.v[e] = fmaf(co.a[t], v.v[e], u.v[e]);
      all.v[e] += v.v[e];
    }
    hs_st<V>(xs + (size_t)t * T * H + idx, v);
  }
  if (sum_out) hs_st<V>(sum_out + idx, all);
  if (a_next && out) {
    if (norm_w) {
      const HsVec<V> w = hs_ld<V>(norm_w + i), c = hs_ld<V>(norm_c + i);
#pragma unroll
      for (int e = 0; e < V; ++e) u.v[e] = fmaf(tanhf(al * u.v[e]), w.v[e], c.v[e]);
    }
    hs_st<V>(out + idx, u);
  }
}

// the dynamic tanh alone, on a float32 row set:  out[r] = tanh(alpha (x[row(r)] + delta[row(r)])) * w + c
template <typename TO, typename TW>
__global__ void __launch_bounds__(HS_THREADS)
dyt_kernel(float* x, const TO* delta, const int* rows, const float* alpha, const TW* w, const TW* c, TO* out,
           int H, long long total, int writeback) {
  const float al = alpha[0];
  pdl_wait();
  pdl_launch();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long r = idx / H;
  const int i = (int)(idx - r * H);
  const size_t at = (size_t)(rows ? (long long)rows[r] : r) * H + i;
  float v = x[at];
  if (delta) {
    v += to_f32(delta[at]);
    if (writeback) x[at] = v;
  }
  out[idx] = from_f32<TO>(fmaf(tanhf(al * v), to_f32(w[i]), to_f32(c[i])));
}

static inline unsigned hs_blocks(long long total) { return (unsigned)((total + HS_THREADS - 1) / HS_THREADS); }
static inline bool hs_aligned(const void* p) { return ((uintptr_t)p & 15) == 0; }

// w_dtype: the dtype of the norm's w and c and of g;  out_dtype: the activation dtype (float32: also "no norm")
RLLM_EXPORT int rllm_hs_read(const float* xs, const float* a, const int* rows, const float* alpha,
                             const void* norm_w, const void* norm_c, int w_dtype, void* out, int out_dtype, int S,
                             long long T, int R, int H, cudaStream_t stream) {
  const long long total = (long long)R * H;
  if (total <= 0) return 0;
  if (S <= 0 || S > HS_MAX_STREAMS || T <= 0) return RLLM_E_BADARG;
  if ((norm_w == nullptr) != (norm_c == nullptr) || (norm_w && !alpha)) return RLLM_E_BADARG;
  if (!norm_w && out_dtype != RLLM_DT_F32) return RLLM_E_BADARG;
  const bool v4 = H % 4 == 0 && hs_aligned(xs) && hs_aligned(norm_w) && hs_aligned(norm_c) && hs_aligned(out);
  RLLM_DISPATCH_DTYPE(out_dtype, TO, RLLM_DISPATCH_DTYPE(w_dtype, TW, {
    if (v4)
      rllm_launch_pdl(hs_read_kernel<TO, TW, 4>, dim3(hs_blocks(total / 4)), dim3(HS_THREADS), (size_t)0, stream, xs, a,
                      rows, alpha, (const TW*)norm_w, (const TW*)norm_c, (TO*)out, S, T, H, total);
    else
      rllm_launch_pdl(hs_read_kernel<TO, TW, 1>, dim3(hs_blocks(total)), dim3(HS_THREADS), (size_t)0, stream, xs, a,
                      rows, alpha, (const TW*)norm_w, (const TW*)norm_c, (TO*)out, S, T, H, total);
  }));
  RLLM_LAUNCH_CHECK();
  return 0;
}

RLLM_EXPORT int rllm_hs_write(float* xs, const void* y, int y_dtype, const void* g, const float* m, const float* b,
                              const float* a_next, const float* alpha, const void* norm_w, const void* norm_c,
                              int w_dtype, void* out, float* sum_out, int S, long long T, int H,
                              cudaStream_t stream) {
  const long long total = T * H;
  if (total <= 0) return 0;
  if (S <= 0 || S > HS_MAX_STREAMS) return RLLM_E_BADARG;
  if ((norm_w == nullptr) != (norm_c == nullptr) || (norm_w && !alpha)) return RLLM_E_BADARG;
  const bool v4 = H % 4 == 0 && hs_aligned(xs) && hs_aligned(y) && hs_aligned(g) && hs_aligned(norm_w) &&
                  hs_aligned(norm_c) && hs_aligned(out) && hs_aligned(sum_out);
#define HS_WRITE(TY_, TO_)                                                                                            \
  RLLM_DISPATCH_DTYPE(w_dtype, TW, {                                                                                  \
    if (v4)                                                                                                           \
      rllm_launch_pdl(hs_write_kernel<TY_, TO_, TW, 4>, dim3(hs_blocks(total / 4)), dim3(HS_THREADS), (size_t)0, stream, \
                      xs, (const TY_*)y, (const TW*)g, m, b, a_next, alpha, (const TW*)norm_w, (const TW*)norm_c,     \
                      (TO_*)out, sum_out, S, T, H, total);                                                            \
    else                                                                                                              \
      rllm_launch_pdl(hs_write_kernel<TY_, TO_, TW, 1>, dim3(hs_blocks(total)), dim3(HS_THREADS), (size_t)0, stream,  \
                      xs, (const TY_*)y, (const TW*)g, m, b, a_next, alpha, (const TW*)norm_w, (const TW*)norm_c,     \
                      (TO_*)out, sum_out, S, T, H, total);                                                            \
  })
  // out has the dtype of y (the activation dtype) when a norm follows, float32 when the bare read is asked for
  if (y_dtype == RLLM_DT_BF16 && (norm_w || !out)) HS_WRITE(bf16, bf16);
  else if (y_dtype == RLLM_DT_BF16) HS_WRITE(bf16, float);
  else if (y_dtype == RLLM_DT_F32) HS_WRITE(float, float);
  else return RLLM_E_BADARG;
#undef HS_WRITE
  RLLM_LAUNCH_CHECK();
  return 0;
}

RLLM_EXPORT int rllm_dyt(float* x, const void* delta, const int* rows, const float* alpha, const void* w,
                         const void* c, int w_dtype, void* out, int out_dtype, int R, int H, int writeback,
                         cudaStream_t stream) {
  const long long total = (long long)R * H;
  if (total <= 0) return 0;
  if (!alpha || !w || !c) return RLLM_E_BADARG;
  RLLM_DISPATCH_DTYPE(out_dtype, TO, RLLM_DISPATCH_DTYPE(w_dtype, TW,
    (rllm_launch_pdl(dyt_kernel<TO, TW>, dim3(hs_blocks(total)), dim3(HS_THREADS), (size_t)0, stream, x,
                     (const TO*)delta, rows, alpha, (const TW*)w, (const TW*)c, (TO*)out, H, total, writeback))));
  RLLM_LAUNCH_CHECK();
  return 0;
}
