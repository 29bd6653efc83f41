// Linear attention with a fixed decay per head ("lightning attention"):
//   q_t = silu(a_q), k_t = silu(a_k) [heads, d],  v_t = silu(a_v) [heads, dv]   (a_*: the token's projections)
//   S_t = lambda_h S_{t-1} + k_t v_t^T        (S: [d, dv] per head, float32, per request)
//   o_t = S_t^T q_t                            (no other scale)
// The state lives in the request's state slot [heads, d, dv] and is carried from step to step.
// Activations, state, products and sums are float32; the output is float32 (a norm reads it).
//
// A block owns a head of a sequence (and a range of value columns); a thread keeps an 8 x 8 tile of S in
// registers, eight rows of the head's d (its "slice") by eight value columns.  The block walks the tokens
// in order, eight at a time (their activated q, k and v rows are staged in shared memory); a token's
// output column is the sum over the slices, taken with shuffles inside the warp.  So a token's result
// does not depend on how the sequence was cut or on the batch.
//
// Long portions: the tokens of a sequence in this step are cut into chunks of LT_CHUNK that run
// side by side.  The recurrence is linear in S: first every chunk computes its end state from a
// zero start, then a small kernel chains them (start of chunk c+1 = lambda^len(c) * start of
// chunk c + end-from-zero of chunk c, in order, and the sequence's new state), then every chunk
// walks its tokens from its start.  Results differ from the plain walk by rounding only.
#include "common.cuh"
#include "lightning_mma.cuh"
#include <math.h>

#define LT_TOKENS 8
#define LT_CHUNK 64
#define LT_TILE 8            // a thread's tile of S is LT_TILE x LT_TILE
#define LT_MAX_COLS 256      // value columns a block covers at most

__device__ __forceinline__ float lt_silu(float v) { return v / (1.0f + expf(-v)); }

// mode 0: whole portion from the slot's state, state written back
// mode 1: one chunk from a zero start, end state to work[chunk], no output
// mode 2: one chunk from work[chunk], output, nothing written back
// NS: slices of d (a power of two up to 32; d <= 8 NS); thread = slice + NS * (tile of columns)
template <typename T, int NS, int MODE>
__global__ void __launch_bounds__(256)
lightning_kernel(const T* q, const T* k, const T* v, int stride, const float* decay, float* state, float* work,
                 const int* q_start, const int* slots, int num_slots, int max_chunks, float* out, int heads, int d,
                 int dv, int* err) {
  constexpr int D = NS * LT_TILE;
  __shared__ __align__(16) float qs[LT_TOKENS][D], ks[LT_TOKENS][D], vs[LT_TOKENS][LT_MAX_COLS];
  pdl_wait();
  pdl_launch();
  const int h = blockIdx.x;
  const int s = (MODE == 0) ? blockIdx.y : blockIdx.y / max_chunks;
  const int chunk = (MODE == 0) ? 0 : blockIdx.y % max_chunks;
  const int cols = (int)blockDim.x / NS * LT_TILE;              // value columns of this block
  const int col0 = blockIdx.z * cols;
  const int ds = threadIdx.x % NS, vt = threadIdx.x / NS;
  const int i0 = ds * LT_TILE, jl = vt * LT_TILE, j0 = col0 + jl;
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
  // which finished output columns this lane holds after the sum over the slices (see below)
  int colbase = 0, last = LT_TILE;
  bool writer = true;
#pragma unroll
  for (int off = NS / 2; off > 0; off >>= 1) {
    const bool upper = (ds & off) != 0;
    if (last > 1) {
      last >>= 1;
      colbase += upper ? last : 0;
    } else {
      writer = writer && !upper;
    }
  }
  float S[LT_TILE][LT_TILE];
  float* sp = (MODE == 0) ? state + ((size_t)slot * heads + h) * d * dv
                          : work + ((size_t)blockIdx.y * heads + h) * d * dv;
  // a tile's rows are eight consecutive floats: two 16-byte accesses where the head's sizes allow it
  const bool wide = (dv & 3) == 0 && j0 + LT_TILE <= dv && (((uintptr_t)sp) & 15) == 0;
#pragma unroll
  for (int a = 0; a < LT_TILE; ++a) {
    if (MODE != 1 && wide && i0 + a < d) {
      *(float4*)&S[a][0] = *(const float4*)(sp + (size_t)(i0 + a) * dv + j0);
      *(float4*)&S[a][4] = *(const float4*)(sp + (size_t)(i0 + a) * dv + j0 + 4);
    } else {
#pragma unroll
      for (int b = 0; b < LT_TILE; ++b)
        S[a][b] = (MODE != 1 && i0 + a < d && j0 + b < dv) ? sp[(size_t)(i0 + a) * dv + j0 + b] : 0.f;
    }
  }
  // The next eight tokens' rows are fetched into registers before this eight's arithmetic starts, so that the
  // loads' latency lies behind it (with four slices or more: a thread then stages at most 8 + 8 + 16 values).
  constexpr bool PF = NS >= 4;
  constexpr int PQ = 8, PV = PF ? 64 / NS : 1;
  T rq[PQ], rk[PQ], rv[PV];
  auto fetch = [&](int tb) {
    const int n = min(LT_TOKENS, t1 - tb);
#pragma unroll
    for (int u = 0; u < PQ; ++u) {
      const int e = threadIdx.x + u * blockDim.x;
      const int tt = e / D, i = e - tt * D;
      const bool on = e < LT_TOKENS * D && tt < n && i < d;
      const size_t at = (size_t)(tb + tt) * stride + (size_t)h * d + i;
      rq[u] = (on && MODE != 1) ? q[at] : from_f32<T>(0.f);
      rk[u] = on ? k[at] : from_f32<T>(0.f);
    }
#pragma unroll
    for (int u = 0; u < PV; ++u) {
      const int e = threadIdx.x + u * blockDim.x;
      const int tt = e / cols, j = e - tt * cols;
      const bool on = e < LT_TOKENS * cols && tt < n && col0 + j < dv;
      rv[u] = on ? v[(size_t)(tb + tt) * stride + (size_t)h * dv + col0 + j] : from_f32<T>(0.f);
    }
  };
  if (PF) fetch(t0);
  for (int tb = t0; tb < t1; tb += LT_TOKENS) {
    const int n = min(LT_TOKENS, t1 - tb);
    __syncthreads();
    if (PF) {
#pragma unroll
      for (int u = 0; u < PQ; ++u) {
        const int e = threadIdx.x + u * blockDim.x;
        if (e < LT_TOKENS * D) {
          (&qs[0][0])[e] = lt_silu(to_f32(rq[u]));                 // silu(0) = 0 where nothing was fetched
          (&ks[0][0])[e] = lt_silu(to_f32(rk[u]));
        }
      }
#pragma unroll
      for (int u = 0; u < PV; ++u) {
        const int e = threadIdx.x + u * blockDim.x;
        if (e < LT_TOKENS * cols) vs[e / cols][e % cols] = lt_silu(to_f32(rv[u]));
      }
    } else {
      for (int e = threadIdx.x; e < LT_TOKENS * D; e += blockDim.x) {
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
      for (int e = threadIdx.x; e < LT_TOKENS * cols; e += blockDim.x) {
        const int tt = e / cols, j = e - tt * cols;
        vs[tt][j] = (tt < n && col0 + j < dv) ? lt_silu(to_f32(v[(size_t)(tb + tt) * stride + (size_t)h * dv + col0 + j])) : 0.f;
      }
    }
    __syncthreads();
    if (PF && tb + LT_TOKENS < t1) fetch(tb + LT_TOKENS);
    for (int tt = 0; tt < n; ++tt) {
      float kk[LT_TILE], qq[LT_TILE], vv[LT_TILE], o[LT_TILE];
      *(float4*)&kk[0] = *(const float4*)&ks[tt][i0];
      *(float4*)&kk[4] = *(const float4*)&ks[tt][i0 + 4];
      *(float4*)&vv[0] = *(const float4*)&vs[tt][jl];
      *(float4*)&vv[4] = *(const float4*)&vs[tt][jl + 4];
      if (MODE != 1) {
        *(float4*)&qq[0] = *(const float4*)&qs[tt][i0];
        *(float4*)&qq[4] = *(const float4*)&qs[tt][i0 + 4];
      }
#pragma unroll
      for (int b = 0; b < LT_TILE; ++b) o[b] = 0.f;
#pragma unroll
      for (int a = 0; a < LT_TILE; ++a)
#pragma unroll
        for (int b = 0; b < LT_TILE; ++b) {
          S[a][b] = fmaf(lam, S[a][b], kk[a] * vv[b]);
          if (MODE != 1) o[b] = fmaf(S[a][b], qq[a], o[b]);
        }
      if (MODE != 1) {
        // The sum over the slices by halving: in every round a lane hands half of its partial sums to its
        // partner and adds the partner's for the half it keeps (8 shuffles for 16 slices instead of 32);
        // at the end a lane holds the finished sums of `last` columns from `colbase` on.
        int cnt = LT_TILE;
#pragma unroll
        for (int off = NS / 2; off > 0; off >>= 1) {
          const bool upper = (ds & off) != 0;
          if (cnt > 1) {
            cnt >>= 1;
#pragma unroll
            for (int b = 0; b < LT_TILE / 2; ++b) {
              if (b < cnt) {
                const float send = upper ? o[b] : o[b + cnt];
                const float recv = __shfl_xor_sync(0xffffffffu, send, off);
                o[b] = (upper ? o[b + cnt] : o[b]) + recv;
              }
            }
          } else {
            o[0] += __shfl_xor_sync(0xffffffffu, o[0], off);
          }
        }
        if (writer) {
          float* op = out + ((size_t)(tb + tt) * heads + h) * dv + j0 + colbase;
#pragma unroll
          for (int b = 0; b < LT_TILE; ++b)
            if (b < last && j0 + colbase + b < dv) op[b] = o[b];
        }
      }
    }
  }
  if (MODE != 2) {
#pragma unroll
    for (int a = 0; a < LT_TILE; ++a) {
      if (wide && i0 + a < d) {
        *(float4*)(sp + (size_t)(i0 + a) * dv + j0) = *(const float4*)&S[a][0];
        *(float4*)(sp + (size_t)(i0 + a) * dv + j0 + 4) = *(const float4*)&S[a][4];
      } else {
#pragma unroll
        for (int b = 0; b < LT_TILE; ++b)
          if (i0 + a < d && j0 + b < dv) sp[(size_t)(i0 + a) * dv + j0 + b] = S[a][b];
      }
    }
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
  float* w0 = work + ((size_t)s * max_chunks * heads + h) * d * dv + e;
  const size_t step = (size_t)heads * d * dv;
  // eight chunks' end states are fetched before the chain runs over them (the loads do not depend on it)
  for (int c0 = 0; c0 < chunks; c0 += 8) {
    float z[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) z[u] = (c0 + u < chunks) ? w0[(size_t)(c0 + u) * step] : 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (c0 + u < chunks) {
        w0[(size_t)(c0 + u) * step] = cur;
        const int n = min(LT_CHUNK, len - (c0 + u) * LT_CHUNK);
        cur = fmaf(n == LT_CHUNK ? full : powf(lam, (float)n), cur, z[u]);
      }
    }
  }
  *sp = cur;
}

template <typename T, int NS>
static int lightning_launch(const T* q, const T* k, const T* v, int stride, const float* decay, float* state,
                            float* work, const int* q_start, const int* slots, int num_slots, int num_seqs,
                            int max_chunks, float* out, int heads, int d, int dv, int* err, cudaStream_t stream) {
  // tiles of eight value columns a block: as many as the head has, up to 256 threads and LT_MAX_COLS columns,
  // and whole warps (a slice's partners in the sum are lanes of one warp)
  int vt = (dv + LT_TILE - 1) / LT_TILE;
  vt = vt > 8 ? vt : 8;                          // at least as many threads as a row of q has values (8 NS)
  vt = vt < 256 / NS ? vt : 256 / NS;
  vt = vt < LT_MAX_COLS / LT_TILE ? vt : LT_MAX_COLS / LT_TILE;
  while ((vt * NS) % 32) ++vt;
  const unsigned threads = (unsigned)(vt * NS), gz = (unsigned)((dv + vt * LT_TILE - 1) / (vt * LT_TILE));
  if (max_chunks <= 0) {
    rllm_launch_pdl(lightning_kernel<T, NS, 0>, dim3(heads, num_seqs, gz), dim3(threads), (size_t)0, stream, q, k, v,
                    stride, decay, state, work, q_start, slots, num_slots, 1, out, heads, d, dv, err);
  } else {
    const dim3 grid(heads, num_seqs * max_chunks, gz);
    rllm_launch_pdl(lightning_kernel<T, NS, 1>, grid, dim3(threads), (size_t)0, stream, q, k, v, stride, decay,
                    state, work, q_start, slots, num_slots, max_chunks, out, heads, d, dv, err);
    rllm_launch_pdl(lightning_chain_kernel, dim3(heads, num_seqs, (d * dv + 255) / 256), dim3(256), (size_t)0, stream,
                    decay, state, work, q_start, slots, num_slots, max_chunks, heads, d, dv);
    rllm_launch_pdl(lightning_kernel<T, NS, 2>, grid, dim3(threads), (size_t)0, stream, q, k, v, stride, decay,
                    state, work, q_start, slots, num_slots, max_chunks, out, heads, d, dv, err);
  }
  return 0;
}

// max_chunks 0: the plain walk.  > 0: ceil(longest portion / LT_CHUNK); work then holds
// num_seqs * max_chunks * heads * d * dv floats.
RLLM_EXPORT int rllm_lightning_chunk() { return LT_CHUNK; }

// RLLM_LIGHTNING=simt keeps the chunk passes on the CUDA cores (for tests and comparisons)
static inline bool lightning_mma_disabled() {
  static int off = -1;
  if (off < 0) { const char* e = getenv("RLLM_LIGHTNING"); off = (e && e[0] == 's') ? 1 : 0; }
  return off == 1;
}

RLLM_EXPORT int rllm_lightning_scan(const void* q, const void* k, const void* v, int stride, int dtype,
                                    const float* decay, float* state, float* work, const int* q_start,
                                    const int* slots, int num_slots, int num_seqs, int max_chunks, float* out,
                                    int heads, int d, int dv, int* err, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (heads <= 0 || d <= 0 || dv <= 0 || num_slots <= 0 || max_chunks < 0) return RLLM_E_BADARG;
  if (max_chunks > 0 && !work) return RLLM_E_BADARG;
  if (d > 256) return RLLM_E_UNSUPPORTED;               // 32 slices of eight rows: the partners of a sum are one warp
  if ((long long)num_seqs * (max_chunks > 0 ? max_chunks : 1) > 65535) return RLLM_E_UNSUPPORTED;
  static_assert(LT_CHUNK == LTC_CHUNK, "the chain kernel serves both forms of the chunk passes");
  if (dtype == RLLM_DT_BF16 && max_chunks > 0 && !lightning_mma_disabled() && stride % 2 == 0) {
    // long portions of bfloat16 activations: the chunk passes on the tensor cores, where the head's sizes are built
    auto chain = [&]() {
      rllm_launch_pdl(lightning_chain_kernel, dim3(heads, num_seqs, (d * dv + 255) / 256), dim3(256), (size_t)0, stream,
                      decay, state, work, q_start, slots, num_slots, max_chunks, heads, d, dv);
    };
    bool done = false;
#define LTC_GO(D_, DV_)                                                                                          \
  if (!done && d == D_ && dv == DV_)                                                                             \
    done = ltc_launch<D_, DV_>((const bf16*)q, (const bf16*)k, (const bf16*)v, stride, decay, work, q_start,     \
                               num_seqs, max_chunks, out, heads, stream, chain)
    LTC_GO(32, 64); LTC_GO(32, 128); LTC_GO(64, 64); LTC_GO(64, 128); LTC_GO(128, 64); LTC_GO(128, 128);
#undef LTC_GO
    if (done) {
      RLLM_LAUNCH_CHECK();
      return 0;
    }
  }
#define LT_GO(T_, NS_)                                                                                          \
  lightning_launch<T_, NS_>((const T_*)q, (const T_*)k, (const T_*)v, stride, decay, state, work, q_start, slots, \
                           num_slots, num_seqs, max_chunks, out, heads, d, dv, err, stream)
  RLLM_DISPATCH_DTYPE(dtype, TT, {
    if (d <= 8) LT_GO(TT, 1);
    else if (d <= 16) LT_GO(TT, 2);
    else if (d <= 32) LT_GO(TT, 4);
    else if (d <= 64) LT_GO(TT, 8);
    else if (d <= 128) LT_GO(TT, 16);
    else LT_GO(TT, 32);
  });
#undef LT_GO
  RLLM_LAUNCH_CHECK();
  return 0;
}
