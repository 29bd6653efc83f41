// Linear attention with a fixed decay per head ("lightning attention"):
//   q_t = silu(a_q), k_t = silu(a_k) [heads, d],  v_t = silu(a_v) [heads, dv]   (a_*: the token's projections)
//   S_t = lambda_h S_{t-1} + k_t v_t^T        (S: [d, dv] per head, float32, per request)
//   o_t = S_t^T q_t                            (no other scale)
// The state lives in the request's state slot [heads, d, dv] and is carried from step to step.
// Activations, state, products and sums are float32; the output is float32 (a norm reads it).
//
// One thread owns a value column j of a head and keeps S[:, j] in registers; a block walks
// the tokens in order, eight at a time (their q and k rows are staged in shared memory).  So
// a token's result does not depend on how the sequence was cut or on the batch.
//
// Long portions: the tokens of a sequence in this step are cut into chunks of LT_CHUNK that run
// side by side.  The recurrence is linear in S: first every chunk computes its end state from a
// zero start, then a small kernel chains them (start of chunk c+1 = lambda^len(c) * start of
// chunk c + end-from-zero of chunk c, in order, and the sequence's new state), then every chunk
// walks its tokens from its start.  Results differ from the plain walk by rounding only.
#include "common.cuh"
#include <math.h>

#define LT_THREADS 64
#define LT_TOKENS 8
#define LT_CHUNK 64

__device__ __forceinline__ float lt_silu(float v) { return v / (1.0f + expf(-v)); }

// mode 0: whole portion from the slot's state, state written back
// mode 1: one chunk from a zero start, end state to work[chunk], no output
// mode 2: one chunk from work[chunk], output, nothing written back
template <typename T, int D, int MODE>
__global__ void __launch_bounds__(LT_THREADS)
lightning_kernel(const T* q, const T* k, const T* v, int stride, const float* decay, float* state, float* work,
                 const int* q_start, const int* slots, int num_slots, int max_chunks, float* out, int heads, int d,
                 int dv, int* err) {
  __shared__ float qs[LT_TOKENS][D], ks[LT_TOKENS][D];
  pdl_wait();
  pdl_launch();
  const int h = blockIdx.x;
  const int s = (MODE == 0) ? blockIdx.y : blockIdx.y / max_chunks;
  const int chunk = (MODE == 0) ? 0 : blockIdx.y % max_chunks;
  const int j = blockIdx.z * LT_THREADS + threadIdx.x;
  const bool mine = j < dv;
  int t0 = q_start[s], t1 = q_start[s + 1];
  if (MODE != 0) {
    t0 += chunk * LT_CHUNK;
    t1 = min(t1, t0 + LT_CHUNK);
    if (t0 >= t1) return;
  }
  const int slot = slots[s];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, 8);
    return;
  }
  const float lam = decay[h];
  float S[D];
  float* sp = (MODE == 0) ? state + ((size_t)slot * heads + h) * d * dv
                          : work + ((size_t)blockIdx.y * heads + h) * d * dv;
#pragma unroll
  for (int i = 0; i < D; ++i) S[i] = (MODE != 1 && mine && i < d) ? sp[(size_t)i * dv + j] : 0.f;
  for (int tb = t0; tb < t1; tb += LT_TOKENS) {
    const int n = min(LT_TOKENS, t1 - tb);
    __syncthreads();
    for (int e = threadIdx.x; e < LT_TOKENS * D; e += LT_THREADS) {
      const int tt = e / D, i = e - tt * D;
      float qv = 0.f, kv = 0.f;
      if (tt < n && i < d) {
        const size_t at = (size_t)(tb + tt) * stride + (size_t)h * d + i;
        if (MODE != 1) qv = lt_silu(to_f32(q[at]));
        kv = lt_silu(to_f32(k[at]));
      }
      qs[tt][i] = qv;
      ks[tt][i] = kv;
    }
    float vv[LT_TOKENS];
#pragma unroll
    for (int tt = 0; tt < LT_TOKENS; ++tt)
      vv[tt] = (mine && tt < n) ? lt_silu(to_f32(v[(size_t)(tb + tt) * stride + (size_t)h * dv + j])) : 0.f;
    __syncthreads();
#pragma unroll
    for (int tt = 0; tt < LT_TOKENS; ++tt) {
      if (tt < n) {
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < D; ++i) {
          S[i] = fmaf(lam, S[i], ks[tt][i] * vv[tt]);
          if (MODE != 1) o = fmaf(S[i], qs[tt][i], o);
        }
        if (MODE != 1 && mine) out[((size_t)(tb + tt) * heads + h) * dv + j] = o;
      }
    }
  }
  if (MODE != 2 && mine) {
#pragma unroll
    for (int i = 0; i < D; ++i)
      if (i < d) sp[(size_t)i * dv + j] = S[i];
  }
}

// work[s * max_chunks + c] holds chunk c's end state from a zero start; afterwards it holds chunk c's start
// state, and the slot holds the sequence's state after its last token.
__global__ void __launch_bounds__(256)
lightning_chain_kernel(const float* decay, float* state, float* work, const int* q_start, const int* slots,
                       int num_slots, int max_chunks, int heads, int d, int dv) {
  pdl_wait();
  pdl_launch();
  const int h = blockIdx.x, s = blockIdx.y;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;
  if (e >= d * dv) return;
  const int slot = slots[s];
  if (slot < 0 || slot >= num_slots) return;
  const int len = q_start[s + 1] - q_start[s];
  if (len <= 0) return;
  const float lam = decay[h];
  const float full = powf(lam, (float)LT_CHUNK);
  float* sp = state + ((size_t)slot * heads + h) * d * dv + e;
  float cur = *sp;
  const int chunks = (len + LT_CHUNK - 1) / LT_CHUNK;
  for (int c = 0; c < chunks; ++c) {
    float* wp = work + (((size_t)s * max_chunks + c) * heads + h) * d * dv + e;
    const float z = *wp;
    *wp = cur;
    const int n = min(LT_CHUNK, len - c * LT_CHUNK);
    cur = fmaf(n == LT_CHUNK ? full : powf(lam, (float)n), cur, z);
  }
  *sp = cur;
}

template <typename T, int D>
static int lightning_launch(const T* q, const T* k, const T* v, int stride, const float* decay, float* state,
                            float* work, const int* q_start, const int* slots, int num_slots, int num_seqs,
                            int max_chunks, float* out, int heads, int d, int dv, int* err, cudaStream_t stream) {
  const unsigned vt = (unsigned)((dv + LT_THREADS - 1) / LT_THREADS);
  if (max_chunks <= 0) {
    rllm_launch_pdl(lightning_kernel<T, D, 0>, dim3(heads, num_seqs, vt), dim3(LT_THREADS), (size_t)0, stream, q, k, v,
                    stride, decay, state, work, q_start, slots, num_slots, 1, out, heads, d, dv, err);
  } else {
    const dim3 grid(heads, num_seqs * max_chunks, vt);
    rllm_launch_pdl(lightning_kernel<T, D, 1>, grid, dim3(LT_THREADS), (size_t)0, stream, q, k, v, stride, decay,
                    state, work, q_start, slots, num_slots, max_chunks, out, heads, d, dv, err);
    rllm_launch_pdl(lightning_chain_kernel, dim3(heads, num_seqs, (d * dv + 255) / 256), dim3(256), (size_t)0, stream,
                    decay, state, work, q_start, slots, num_slots, max_chunks, heads, d, dv);
    rllm_launch_pdl(lightning_kernel<T, D, 2>, grid, dim3(LT_THREADS), (size_t)0, stream, q, k, v, stride, decay,
                    state, work, q_start, slots, num_slots, max_chunks, out, heads, d, dv, err);
  }
  return 0;
}

// max_chunks 0: the plain walk.  > 0: ceil(longest portion / LT_CHUNK); work then holds
// num_seqs * max_chunks * heads * d * dv floats.
RLLM_EXPORT int rllm_lightning_chunk() { return LT_CHUNK; }

RLLM_EXPORT int rllm_lightning_scan(const void* q, const void* k, const void* v, int stride, int dtype,
                                    const float* decay, float* state, float* work, const int* q_start,
                                    const int* slots, int num_slots, int num_seqs, int max_chunks, float* out,
                                    int heads, int d, int dv, int* err, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (heads <= 0 || d <= 0 || dv <= 0 || num_slots <= 0 || max_chunks < 0) return RLLM_E_BADARG;
  if (max_chunks > 0 && !work) return RLLM_E_BADARG;
  if (d > 128) return RLLM_E_UNSUPPORTED;               // a thread keeps a column of the state in registers
  if ((long long)num_seqs * (max_chunks > 0 ? max_chunks : 1) > 65535) return RLLM_E_UNSUPPORTED;
#define LT_GO(T_, D_)                                                                                          \
  lightning_launch<T_, D_>((const T_*)q, (const T_*)k, (const T_*)v, stride, decay, state, work, q_start, slots, \
                           num_slots, num_seqs, max_chunks, out, heads, d, dv, err, stream)
  RLLM_DISPATCH_DTYPE(dtype, TT, {
    if (d <= 16) LT_GO(TT, 16);
    else if (d <= 32) LT_GO(TT, 32);
    else if (d <= 64) LT_GO(TT, 64);
    else LT_GO(TT, 128);
  });
#undef LT_GO
  RLLM_LAUNCH_CHECK();
  return 0;
}
