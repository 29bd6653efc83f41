// The selective state-space recurrence (Mamba) and the short causal convolution ahead of it.
//
//   convolution: c_t = silu(bias + sum_j w[ch, j] x_{t - (taps - 1) + j})   per channel, zeros before the
//                sequence's start; the last taps - 1 inputs are per-request state (float32 [taps - 1, E])
//   recurrence:  dt = softplus(r_t + dt_bias)     (r_t: the token's step projection, one per channel)
//                S[ch, n] <- exp(dt A[ch, n]) S[ch, n] + dt c_t B_t[n],   A = -exp(A_log)
//                y = sum_n S[ch, n] C_t[n] + D c_t,   out = y * silu(z_t)
//                S is per-request state (float32, kept as [N, E]).
// Step sizes, decays, exponentials, state and sums are float32.  One thread owns a channel of a
// sequence and walks the sequence's tokens of the step in order, so a token's result does not depend
// on how the sequence was cut or on the batch.
//
// Long portions run as chunks of SS_CHUNK side by side: the recurrence is linear in S, and the product
// of a chunk's decays is exp(A * sum of its dt).  First every chunk computes (sum of dt, end state from
// zero), then a small kernel chains the chunks in order (and leaves the sequence's new state), then
// every chunk walks its tokens from its start.  Results differ from the plain walk by rounding only.
#include "common.cuh"
#include <math.h>

#define SS_THREADS 128
#define SS_TOKENS 8
#define SS_CHUNK 64

__device__ __forceinline__ float ss_silu(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float ss_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// x: T rows with stride `stride` (the first E columns are read).  One thread a (token, channel).
template <typename T, typename TW>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const T* x, int stride, const TW* w, const TW* bias, float* tail, const int* q_start,
                   const int* token_seq, const int* slots, int num_slots, T* out, int E, int taps, long long total,
                   int* err) {
  pdl_wait();
  pdl_launch();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int t = (int)(idx / E), c = (int)(idx - (long long)t * E);
  const int s = token_seq[t];
  const int first = q_start[s], qlen = q_start[s + 1] - first;
  const int slot = slots[s];
  if (slot < 0 || slot >= num_slots) {
    atomicOr(err, 8);
    return;
  }
  float* tl = tail + (size_t)slot * (taps - 1) * E + c;
  const int li = t - first;
  float acc = to_f32(bias[c]);
  for (int j = 0; j < taps; ++j) {
    const int src = li - (taps - 1) + j;
    const float v = (src >= 0) ? to_f32(x[(size_t)(first + src) * stride + c]) : tl[(size_t)(taps - 1 + src) * E];
    acc = fmaf(to_f32(w[(size_t)c * taps + j]), v, acc);
  }
  out[(size_t)t * E + c] = from_f32<T>(ss_silu(acc));
  if (qlen == 1) {                       // the only reader of this sequence's tail: move it on by one input
    for (int k = 0; k + 1 < taps - 1; ++k) tl[(size_t)k * E] = tl[(size_t)(k + 1) * E];
    if (taps > 1) tl[(size_t)(taps - 2) * E] = to_f32(x[(size_t)t * stride + c]);
  }
}

// Up to CV_TAPS taps: one thread takes a channel and CV_RUN consecutive tokens of the step and keeps the
// last taps - 1 inputs in registers, so that a token costs one load (the window is fetched anew where the
// run crosses into another sequence).  Weights and window are held right-aligned: entry CV_TAPS - 1 is the
// current token's.
#define CV_TAPS 8
#define CV_RUN 8
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
causal_conv_run_kernel(const T* x, int stride, const TW* w, const TW* bias, float* tail, const int* q_start,
                       const int* token_seq, const int* slots, int num_slots, T* out, int E, int taps, int T_tokens,
                       int* err) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const bool mine = c < E;
  float wv[CV_TAPS];
#pragma unroll
  for (int k = 0; k < CV_TAPS; ++k) wv[CV_TAPS - 1 - k] = (mine && k < taps) ? to_f32(w[(size_t)c * taps + taps - 1 - k]) : 0.f;
  const float b = mine ? to_f32(bias[c]) : 0.f;
  pdl_wait();
  pdl_launch();
  if (!mine) return;
  float win[CV_TAPS - 1];
  int cur = -1, first = 0, qlen = 0;
  float* tl = nullptr;
  const int t_end = min(T_tokens, (int)(blockIdx.y + 1) * CV_RUN);
  for (int t = blockIdx.y * CV_RUN; t < t_end; ++t) {
    const int s = token_seq[t];
    if (s != cur) {
      cur = s;
      first = q_start[s];
      qlen = q_start[s + 1] - first;
      const int slot = slots[s];
      if (slot < 0 || slot >= num_slots) {
        atomicOr(err, 8);
        return;
      }
      tl = tail + (size_t)slot * (taps - 1) * E + c;
      const int li = t - first;
#pragma unroll
      for (int k = 1; k < CV_TAPS; ++k) {              // the input k places back
        float v = 0.f;
        if (k <= taps - 1) {
          const int src = li - k;
          v = (src >= 0) ? to_f32(x[(size_t)(first + src) * stride + c]) : tl[(size_t)(taps - 1 + src) * E];
        }
        win[CV_TAPS - 1 - k] = v;
      }
    }
    const float xv = to_f32(x[(size_t)t * stride + c]);
    float acc = b;
#pragma unroll
    for (int j = 0; j < CV_TAPS - 1; ++j) acc = fmaf(wv[j], win[j], acc);
    acc = fmaf(wv[CV_TAPS - 1], xv, acc);
    out[(size_t)t * E + c] = from_f32<T>(ss_silu(acc));
#pragma unroll
    for (int j = 0; j < CV_TAPS - 2; ++j) win[j] = win[j + 1];
    win[CV_TAPS - 2] = xv;
    if (qlen == 1) {                     // the only reader of this sequence's tail: move it on by one input
      for (int k = 0; k + 1 < taps - 1; ++k) tl[(size_t)k * E] = tl[(size_t)(k + 1) * E];
      if (taps > 1) tl[(size_t)(taps - 2) * E] = xv;
    }
  }
}

// sequences that brought more than one token: the tail becomes their last taps - 1 inputs
template <typename T>
__global__ void __launch_bounds__(256)
conv_tail_kernel(const T* x, int stride, float* tail, const int* q_start, const int* slots, int num_slots, int E,
                 int taps) {
  pdl_wait();
  pdl_launch();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
  if (c >= E) return;
  const int first = q_start[s], qlen = q_start[s + 1] - first;
  const int slot = slots[s];
  if (qlen <= 1 || slot < 0 || slot >= num_slots) return;
  float* tl = tail + (size_t)slot * (taps - 1) * E + c;
  // new[k] = input number qlen - (taps - 1) + k of this step, or old[qlen + k] if that lies before the step;
  // old[qlen + k] is behind new[k], so walking k upwards reads every old value before it is overwritten
  for (int k = 0; k < taps - 1; ++k) {
    const int src = qlen - (taps - 1) + k;
    tl[(size_t)k * E] = (src >= 0) ? to_f32(x[(size_t)(first + src) * stride + c]) : tl[(size_t)(qlen + k) * E];
  }
}

// mode 0: whole portion from the slot's state, state written back
// mode 1: one chunk from zero: end state and the sum of dt to work, no output
// mode 2: one chunk from work[chunk] (its start state), output, nothing written back
template <typename T, typename TW, int NMAX, int MODE>
__global__ void __launch_bounds__(SS_THREADS)
selective_scan_kernel(const T* xc, const float* dt_raw, const TW* dt_bias, const T* bc, int bc_stride, int b_off,
                      int c_off, const TW* a_log, const TW* dskip, const T* z, int z_stride, float* state,
                      float* work, float* work_dt, const int* q_start, const int* slots, int num_slots, int max_chunks,
                      T* out, int E, int N, int* err) {
  __shared__ float Bs[SS_TOKENS][NMAX], Cs[SS_TOKENS][NMAX];
  const int c = blockIdx.x * SS_THREADS + threadIdx.x;
  const bool mine = c < E;
  float A[NMAX];
#pragma unroll
  // A times log2(e): the decay exp(dt A) is then one exp2 (a single special-function instruction)
  for (int n = 0; n < NMAX; ++n) A[n] = (mine && n < N) ? -expf(to_f32(a_log[(size_t)c * N + n])) * 1.4426950408889634f : 0.f;
  const float bias = mine ? to_f32(dt_bias[c]) : 0.f, dsk = mine ? to_f32(dskip[c]) : 0.f;
  pdl_wait();
  pdl_launch();
  const int s = (MODE == 0) ? blockIdx.y : blockIdx.y / max_chunks;
  const int chunk = (MODE == 0) ? 0 : blockIdx.y % max_chunks;
  int t0 = q_start[s], t1 = q_start[s + 1];
  if (MODE != 0) {
    t0 += chunk * SS_CHUNK;
    t1 = min(t1, t0 + SS_CHUNK);
    if (t0 >= t1) return;
  }
  const int slot = slots[s];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, 8);
    return;
  }
  float* sp = (MODE == 0) ? state + (size_t)slot * N * E : work + (size_t)blockIdx.y * N * E;
  float S[NMAX];
#pragma unroll
  for (int n = 0; n < NMAX; ++n) S[n] = (MODE != 1 && mine && n < N) ? sp[(size_t)n * E + c] : 0.f;
  float dt_sum = 0.f;
  // The next eight tokens' values are fetched into registers before this eight's arithmetic starts, so that
  // the loads' latency lies behind it.
  constexpr int PB = (SS_TOKENS * NMAX + SS_THREADS - 1) / SS_THREADS;
  T px[SS_TOKENS], pz[SS_TOKENS], pb[PB], pc[PB];
  float pd[SS_TOKENS];
  auto fetch = [&](int tb) {
    const int cnt = min(SS_TOKENS, t1 - tb);
#pragma unroll
    for (int u = 0; u < PB; ++u) {
      const int e = threadIdx.x + u * SS_THREADS;
      const int tt = e / NMAX, n = e - tt * NMAX;
      const bool on = e < SS_TOKENS * NMAX && tt < cnt && n < N;
      const T* row = bc + (size_t)(tb + tt) * bc_stride;
      pb[u] = on ? row[b_off + n] : from_f32<T>(0.f);
      pc[u] = on ? row[c_off + n] : from_f32<T>(0.f);
    }
#pragma unroll
    for (int tt = 0; tt < SS_TOKENS; ++tt) {
      const bool on = mine && tt < cnt;
      const size_t t = (size_t)(tb + tt);
      px[tt] = on ? xc[t * E + c] : from_f32<T>(0.f);
      pd[tt] = on ? dt_raw[t * E + c] : 0.f;
      pz[tt] = (on && MODE != 1) ? z[t * z_stride + c] : from_f32<T>(0.f);
    }
  };
  fetch(t0);
  for (int tb = t0; tb < t1; tb += SS_TOKENS) {
    const int cnt = min(SS_TOKENS, t1 - tb);
    __syncthreads();
#pragma unroll
    for (int u = 0; u < PB; ++u) {
      const int e = threadIdx.x + u * SS_THREADS;
      if (e < SS_TOKENS * NMAX) {
        (&Bs[0][0])[e] = to_f32(pb[u]);
        (&Cs[0][0])[e] = to_f32(pc[u]);
      }
    }
    float xv[SS_TOKENS], dv[SS_TOKENS], zv[SS_TOKENS];
#pragma unroll
    for (int tt = 0; tt < SS_TOKENS; ++tt) {
      const bool on = mine && tt < cnt;
      xv[tt] = to_f32(px[tt]);
      dv[tt] = on ? ss_softplus(pd[tt] + bias) : 0.f;
      zv[tt] = to_f32(pz[tt]);
    }
    __syncthreads();
    if (tb + SS_TOKENS < t1) fetch(tb + SS_TOKENS);
#pragma unroll
    for (int tt = 0; tt < SS_TOKENS; ++tt) {
      if (tt < cnt) {
        const float dt = dv[tt], dx = dt * xv[tt];
        float y = 0.f;
#pragma unroll
        for (int n = 0; n < NMAX; ++n) {
          S[n] = fmaf(exp2f(dt * A[n]), S[n], dx * Bs[tt][n]);
          if (MODE != 1) y = fmaf(S[n], Cs[tt][n], y);
        }
        dt_sum += dt;
        if (MODE != 1 && mine) {
          y = fmaf(dsk, xv[tt], y);
          out[(size_t)(tb + tt) * E + c] = from_f32<T>(y * ss_silu(zv[tt]));
        }
      }
    }
  }
  if (MODE != 2 && mine) {
#pragma unroll
    for (int n = 0; n < NMAX; ++n)
      if (n < N) sp[(size_t)n * E + c] = S[n];
    if (MODE == 1) work_dt[(size_t)blockIdx.y * E + c] = dt_sum;
  }
}

// work[s * max_chunks + k]: chunk k's end state from zero, replaced by chunk k's start state; the slot gets
// the state after the sequence's last token.
template <typename TW>
__global__ void __launch_bounds__(256)
selective_chain_kernel(const TW* a_log, float* state, float* work, const float* work_dt, const int* q_start,
                       const int* slots, int num_slots, int max_chunks, int E, int N) {
  pdl_wait();
  pdl_launch();
  const int s = blockIdx.y;
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (long long)N * E) return;
  const int n = (int)(e / E), c = (int)(e - (long long)n * E);
  const int slot = slots[s];
  if (slot < 0 || slot >= num_slots) return;
  const int len = q_start[s + 1] - q_start[s];
  if (len <= 0) return;
  const float a = -expf(to_f32(a_log[(size_t)c * N + n]));
  float* sp = state + (size_t)slot * N * E + e;
  float cur = *sp;
  const int chunks = (len + SS_CHUNK - 1) / SS_CHUNK;
  // eight chunks' summaries are fetched before the chain runs over them (the loads do not depend on it)
  for (int k0 = 0; k0 < chunks; k0 += 8) {
    float zend[8], dts[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const size_t w = (size_t)s * max_chunks + k0 + u;
      zend[u] = (k0 + u < chunks) ? work[w * N * E + e] : 0.f;
      dts[u] = (k0 + u < chunks) ? work_dt[w * E + c] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (k0 + u < chunks) {
        work[((size_t)s * max_chunks + k0 + u) * N * E + e] = cur;
        cur = fmaf(expf(a * dts[u]), cur, zend[u]);
      }
    }
  }
  *sp = cur;
}

RLLM_EXPORT int rllm_scan_chunk() { return SS_CHUNK; }

RLLM_EXPORT int rllm_causal_conv(const void* x, int stride, int dtype, const void* w, const void* bias, int w_dtype,
                                 float* tail, const int* q_start, const int* token_seq, const int* slots,
                                 int num_slots, int num_seqs, int any_long, void* out, int T, int E, int taps,
                                 int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E <= 0 || taps <= 0 || taps > 64 || num_slots <= 0) return RLLM_E_BADARG;
  const long long total = (long long)T * E;
  if (taps <= CV_TAPS && (T + CV_RUN - 1) / CV_RUN <= 65535) {
    RLLM_DISPATCH_DTYPE(dtype, TT, RLLM_DISPATCH_DTYPE(w_dtype, TW,
      (rllm_launch_pdl(causal_conv_run_kernel<TT, TW>, dim3((unsigned)((E + 127) / 128), (unsigned)((T + CV_RUN - 1) / CV_RUN)),
                       dim3(128), (size_t)0, stream, (const TT*)x, stride, (const TW*)w, (const TW*)bias, tail, q_start,
                       token_seq, slots, num_slots, (TT*)out, E, taps, T, err))));
  } else {
    RLLM_DISPATCH_DTYPE(dtype, TT, RLLM_DISPATCH_DTYPE(w_dtype, TW,
      (rllm_launch_pdl(causal_conv_kernel<TT, TW>, dim3((unsigned)((total + 255) / 256)), dim3(256), (size_t)0, stream,
                       (const TT*)x, stride, (const TW*)w, (const TW*)bias, tail, q_start, token_seq, slots, num_slots,
                       (TT*)out, E, taps, total, err))));
  }
  if (any_long && taps > 1) {
    if (num_seqs > 65535) return RLLM_E_UNSUPPORTED;
    RLLM_DISPATCH_DTYPE(dtype, TT,
      (rllm_launch_pdl(conv_tail_kernel<TT>, dim3((E + 255) / 256, num_seqs), dim3(256), (size_t)0, stream,
                       (const TT*)x, stride, tail, q_start, slots, num_slots, E, taps)));
  }
  RLLM_LAUNCH_CHECK();
  return 0;
}

template <typename T, typename TW, int NMAX>
static void scan_launch(const T* xc, const float* dt_raw, const TW* dt_bias, const T* bc, int bc_stride, int b_off,
                        int c_off, const TW* a_log, const TW* dskip, const T* z, int z_stride, float* state,
                        float* work, float* work_dt, const int* q_start, const int* slots, int num_slots,
                        int num_seqs, int max_chunks, T* out, int E, int N, int* err, cudaStream_t stream) {
  const unsigned bx = (unsigned)((E + SS_THREADS - 1) / SS_THREADS);
  if (max_chunks <= 0) {
    rllm_launch_pdl(selective_scan_kernel<T, TW, NMAX, 0>, dim3(bx, num_seqs), dim3(SS_THREADS), (size_t)0, stream, xc,
                    dt_raw, dt_bias, bc, bc_stride, b_off, c_off, a_log, dskip, z, z_stride, state, work, work_dt,
                    q_start, slots, num_slots, 1, out, E, N, err);
    return;
  }
  const dim3 grid(bx, num_seqs * max_chunks);
  rllm_launch_pdl(selective_scan_kernel<T, TW, NMAX, 1>, grid, dim3(SS_THREADS), (size_t)0, stream, xc, dt_raw, dt_bias,
                  bc, bc_stride, b_off, c_off, a_log, dskip, z, z_stride, state, work, work_dt, q_start, slots,
                  num_slots, max_chunks, out, E, N, err);
  rllm_launch_pdl(selective_chain_kernel<TW>, dim3((unsigned)(((long long)N * E + 255) / 256), num_seqs), dim3(256),
                  (size_t)0, stream, a_log, state, work, (const float*)work_dt, q_start, slots, num_slots, max_chunks,
                  E, N);
  rllm_launch_pdl(selective_scan_kernel<T, TW, NMAX, 2>, grid, dim3(SS_THREADS), (size_t)0, stream, xc, dt_raw, dt_bias,
                  bc, bc_stride, b_off, c_off, a_log, dskip, z, z_stride, state, work, work_dt, q_start, slots,
                  num_slots, max_chunks, out, E, N, err);
}

// max_chunks 0: the plain walk.  > 0: ceil(longest portion / SS_CHUNK); work holds num_seqs * max_chunks * N * E
// floats and work_dt num_seqs * max_chunks * E.
RLLM_EXPORT int rllm_selective_scan(const void* xc, const float* dt_raw, const void* dt_bias, const void* bc,
                                    int bc_stride, int b_off, int c_off, const void* a_log, const void* dskip,
                                    const void* z, int z_stride, int dtype, int w_dtype, float* state, float* work,
                                    float* work_dt, const int* q_start, const int* slots, int num_slots, int num_seqs,
                                    int max_chunks, void* out, int E, int N, int* err, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (E <= 0 || N <= 0 || num_slots <= 0 || max_chunks < 0) return RLLM_E_BADARG;
  if (max_chunks > 0 && (!work || !work_dt)) return RLLM_E_BADARG;
  if (N > 128) return RLLM_E_UNSUPPORTED;              // a thread keeps a channel's states in registers
  if ((long long)num_seqs * (max_chunks > 0 ? max_chunks : 1) > 65535) return RLLM_E_UNSUPPORTED;
#define SS_GO(T_, TW_, N_)                                                                                         \
  scan_launch<T_, TW_, N_>((const T_*)xc, dt_raw, (const TW_*)dt_bias, (const T_*)bc, bc_stride, b_off, c_off,     \
                           (const TW_*)a_log, (const TW_*)dskip, (const T_*)z, z_stride, state, work, work_dt,     \
                           q_start, slots, num_slots, num_seqs, max_chunks, (T_*)out, E, N, err, stream)
  RLLM_DISPATCH_DTYPE(dtype, TT, RLLM_DISPATCH_DTYPE(w_dtype, TW, {
    if (N <= 16) SS_GO(TT, TW, 16);
    else if (N <= 32) SS_GO(TT, TW, 32);
    else if (N <= 64) SS_GO(TT, TW, 64);
    else SS_GO(TT, TW, 128);
  }));
#undef SS_GO
  RLLM_LAUNCH_CHECK();
  return 0;
}
