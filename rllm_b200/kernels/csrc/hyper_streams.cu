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

struct HsCoeff {
  float a[HS_MAX_STREAMS];                       // read weights (of the read this kernel performs)
  float m[HS_MAX_STREAMS * HS_MAX_STREAMS];      // mix [from][to]
  float b[HS_MAX_STREAMS];                       // write weights
};

// The coefficient tensors are tiny; every thread takes them from global memory (they are weights: no kernel
// writes them, so they may be read before the dependency wait).
__device__ __forceinline__ void hs_load(const float* p, float* dst, int n) {
  for (int i = 0; i < n; ++i) dst[i] = p[i];
}

// out[r, :] = norm(sum_s a[s] xs[s, row(r), :]);  a == nullptr: all ones (the plain sum of the streams).
// norm_w == nullptr: no norm (out is then float32, the sum itself).
template <typename TO, typename TW>
__global__ void __launch_bounds__(HS_THREADS)
hs_read_kernel(const float* xs, const float* a, const int* rows, const float* alpha, const TW* norm_w,
               const TW* norm_c, TO* out, int S, long long T, int H, long long total) {
  float ca[HS_MAX_STREAMS];
  for (int s = 0; s < S; ++s) ca[s] = a ? a[s] : 1.0f;
  const float al = alpha ? alpha[0] : 0.f;
  pdl_wait();
  pdl_launch();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long r = idx / H;
  const int i = (int)(idx - r * H);
  const long long src = rows ? (long long)rows[r] : r;
  float u = 0.f;
  for (int s = 0; s < S; ++s) u = fmaf(ca[s], xs[((size_t)s * T + src) * H + i], u);
  if (norm_w) u = fmaf(tanhf(al * u), to_f32(norm_w[i]), to_f32(norm_c[i]));
  out[idx] = from_f32<TO>(u);
}

// xs (in place): x_t <- sum_s M[s, t] x_s + b[t] * g * y;  then, if a_next is given, the next read and its
// norm: out = norm(sum_t a_next[t] x_t).  sum_out (float32 [T, H], optional): the plain sum of the new streams.
template <typename TY, typename TO, typename TW>
__global__ void __launch_bounds__(HS_THREADS)
hs_write_kernel(float* xs, const TY* y, const TW* g, const float* m, const float* b, const float* a_next,
                const float* alpha, const TW* norm_w, const TW* norm_c, TO* out, float* sum_out, int S,
                long long T, int H, long long total) {
  float cm[HS_MAX_STREAMS * HS_MAX_STREAMS], cb[HS_MAX_STREAMS], ca[HS_MAX_STREAMS];
  hs_load(m, cm, S * S);
  hs_load(b, cb, S);
  if (a_next) hs_load(a_next, ca, S);
  const float al = alpha ? alpha[0] : 0.f;
  pdl_wait();
  pdl_launch();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int i = (int)(idx % H);
  float x[HS_MAX_STREAMS];
  for (int s = 0; s < S; ++s) x[s] = xs[(size_t)s * T * H + idx];
  float yy = to_f32(y[idx]);
  if (g) yy *= to_f32(g[i]);
  float u = 0.f, total_sum = 0.f;
  for (int t = 0; t < S; ++t) {
    float v = 0.f;
    for (int s = 0; s < S; ++s) v = fmaf(cm[s * S + t], x[s], v);
    v = fmaf(cb[t], yy, v);
    xs[(size_t)t * T * H + idx] = v;
    if (a_next) u = fmaf(ca[t], v, u);
    total_sum += v;
  }
  if (sum_out) sum_out[idx] = total_sum;
  if (a_next && out) {
    if (norm_w) u = fmaf(tanhf(al * u), to_f32(norm_w[i]), to_f32(norm_c[i]));
    out[idx] = from_f32<TO>(u);
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

// w_dtype: the dtype of the norm's w and c and of g;  out_dtype: the activation dtype (float32: also "no norm")
RLLM_EXPORT int rllm_hs_read(const float* xs, const float* a, const int* rows, const float* alpha,
                             const void* norm_w, const void* norm_c, int w_dtype, void* out, int out_dtype, int S,
                             long long T, int R, int H, cudaStream_t stream) {
  const long long total = (long long)R * H;
  if (total <= 0) return 0;
  if (S <= 0 || S > HS_MAX_STREAMS || T <= 0) return RLLM_E_BADARG;
  if ((norm_w == nullptr) != (norm_c == nullptr) || (norm_w && !alpha)) return RLLM_E_BADARG;
  if (!norm_w && out_dtype != RLLM_DT_F32) return RLLM_E_BADARG;
  RLLM_DISPATCH_DTYPE(out_dtype, TO, RLLM_DISPATCH_DTYPE(w_dtype, TW,
    (rllm_launch_pdl(hs_read_kernel<TO, TW>, dim3(hs_blocks(total)), dim3(HS_THREADS), (size_t)0, stream, xs, a, rows,
                     alpha, (const TW*)norm_w, (const TW*)norm_c, (TO*)out, S, T, H, total))));
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
  // out has the dtype of y (the activation dtype) when a norm follows, float32 when the bare read is asked for
  if (y_dtype == RLLM_DT_BF16 && (norm_w || !out)) {
    RLLM_DISPATCH_DTYPE(w_dtype, TW,
      (rllm_launch_pdl(hs_write_kernel<bf16, bf16, TW>, dim3(hs_blocks(total)), dim3(HS_THREADS), (size_t)0, stream, xs,
                       (const bf16*)y, (const TW*)g, m, b, a_next, alpha, (const TW*)norm_w, (const TW*)norm_c,
                       (bf16*)out, sum_out, S, T, H, total)));
  } else if (y_dtype == RLLM_DT_BF16) {
    RLLM_DISPATCH_DTYPE(w_dtype, TW,
      (rllm_launch_pdl(hs_write_kernel<bf16, float, TW>, dim3(hs_blocks(total)), dim3(HS_THREADS), (size_t)0, stream, xs,
                       (const bf16*)y, (const TW*)g, m, b, a_next, alpha, (const TW*)norm_w, (const TW*)norm_c,
                       (float*)out, sum_out, S, T, H, total)));
  } else if (y_dtype == RLLM_DT_F32) {
    RLLM_DISPATCH_DTYPE(w_dtype, TW,
      (rllm_launch_pdl(hs_write_kernel<float, float, TW>, dim3(hs_blocks(total)), dim3(HS_THREADS), (size_t)0, stream, xs,
                       (const float*)y, (const TW*)g, m, b, a_next, alpha, (const TW*)norm_w, (const TW*)norm_c,
                       (float*)out, sum_out, S, T, H, total)));
  } else {
    return RLLM_E_BADARG;
  }
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
