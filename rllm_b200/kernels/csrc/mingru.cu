// minGRU: a gated recurrence whose gates read the current token only,
//   z = sigmoid(a_z + b_z),  u = a_x + b_x,  c = u + 1/2 (u >= 0) | sigmoid(u) (u < 0),
//   S_t = (1 - z) S_{t-1} + z c,   y_t = S_t * silu(a_g),
// with a_z, a_x, a_g the token's three projections side by side in one row.  The
// state is float32, one row per request slot, carried from step to step; gates,
// candidate, state and the output gate are float32 arithmetic.  One thread owns
// a channel of a sequence and walks the sequence's tokens of this step in
// order, so a token's state does not depend on how the sequence was cut.
#include "common.cuh"

#define MG_THREADS 128
#define MG_AHEAD 4

__device__ __forceinline__ float sigmoid_f32(float v) { return 1.0f / (1.0f + expf(-v)); }

template <typename TA, typename TW>
__global__ void __launch_bounds__(MG_THREADS)
mingru_scan_kernel(const TA* zxg, int stride, const TW* bz, const TW* bx,
                   float* state, const int* q_start, const int* slots,
                   int num_slots, TA* out, int W, int* err) {
  // (Every kernel of this file starts with the wait for the kernel ahead of it in the stream and lets the
  // next one in right after: launches overlap the tails of their predecessors.  The pointer parameters
  // carry no __restrict__, so that no load is proved independent of that wait and moved above it.)
  pdl_wait();
  pdl_launch();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
  if (c >= W) return;
  const int slot = slots[s];
  if (slot < 0 || slot >= num_slots) {
    atomicOr(err, 8);
    return;
  }
  const float biasz = to_f32(bz[c]), biasx = to_f32(bx[c]);
  float S = state[(size_t)slot * W + c];
  const int t1 = q_start[s + 1];
  for (int t0 = q_start[s]; t0 < t1; t0 += MG_AHEAD) {
    float az[MG_AHEAD], ax[MG_AHEAD], ag[MG_AHEAD];
#pragma unroll
    for (int i = 0; i < MG_AHEAD; ++i) {
      const int t = min(t0 + i, t1 - 1);
      const TA* r = zxg + (size_t)t * stride + c;
      az[i] = to_f32(r[0]); ax[i] = to_f32(r[W]); ag[i] = to_f32(r[2 * W]);
    }
#pragma unroll
    for (int i = 0; i < MG_AHEAD; ++i) {
      if (t0 + i < t1) {
        const float z = sigmoid_f32(az[i] + biasz), u = ax[i] + biasx;
        const float cand = (u >= 0.f) ? u + 0.5f : sigmoid_f32(u);
        S = fmaf(1.0f - z, S, z * cand);
        out[(size_t)(t0 + i) * W + c] = from_f32<TA>(S * (ag[i] * sigmoid_f32(ag[i])));
      }
    }
  }
  state[(size_t)slot * W + c] = S;
}

// Long portions: the sequence's tokens of this step are cut into chunks of MG_CHUNK.  The recurrence is
// linear in the state, S_t = a_t S_{t-1} + b_t with a_t = 1 - z_t and b_t = z_t c_t, so a chunk is
// summarised by (A, B) = (product of its a_t, its end state from a zero start): first every chunk
// computes its (A, B) at once, then every chunk rebuilds its start state from the sequence's state and
// the chunks before it (in order) and walks its tokens as the plain kernel does.  Results differ from the
// plain kernel's by rounding only, and do not depend on what else is in the batch.
#define MG_CHUNK 64
#define MG_BATCH 8

template <typename TA, typename TW>
__global__ void __launch_bounds__(MG_THREADS)
mingru_chunk_summary_kernel(const TA* zxg, int stride, const TW* bz,
                            const TW* bx, const float* state,
                            const int* q_start, const int* slots, int num_slots,
                            int max_chunks, float* carry, float* init, int W) {
  pdl_wait();
  pdl_launch();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y / max_chunks, k = blockIdx.y % max_chunks;
  if (c >= W) return;
  const int t0 = q_start[s] + k * MG_CHUNK, t1 = min(q_start[s + 1], t0 + MG_CHUNK);
  if (t0 >= t1) return;
  const int slot = slots[s];
  if (slot < 0 || slot >= num_slots) return;
  if (k == 0) init[(size_t)s * W + c] = state[(size_t)slot * W + c];
  const float biasz = to_f32(bz[c]), biasx = to_f32(bx[c]);
  float A = 1.f, B = 0.f;
  for (int tb = t0; tb < t1; tb += MG_BATCH) {        // a batch of tokens' values are fetched before the chain runs
    float az[MG_BATCH], ax[MG_BATCH];
#pragma unroll
    for (int i = 0; i < MG_BATCH; ++i) {
      const TA* r = zxg + (size_t)min(tb + i, t1 - 1) * stride + c;
      az[i] = to_f32(r[0]); ax[i] = to_f32(r[W]);
    }
#pragma unroll
    for (int i = 0; i < MG_BATCH; ++i) {
      if (tb + i < t1) {
        const float z = sigmoid_f32(az[i] + biasz), u = ax[i] + biasx;
        const float cand = (u >= 0.f) ? u + 0.5f : sigmoid_f32(u);
        A *= 1.0f - z;
        B = fmaf(1.0f - z, B, z * cand);
      }
    }
  }
  float* o = carry + ((size_t)blockIdx.y * 2) * W + c;
  o[0] = A;
  o[W] = B;
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(MG_THREADS)
mingru_chunk_scan_kernel(const TA* zxg, int stride, const TW* bz,
                         const TW* bx, float* state, const int* q_start,
                         const int* slots, int num_slots, int max_chunks,
                         const float* carry, const float* init, TA* out,
                         int W, int* err) {
  pdl_wait();
  pdl_launch();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y / max_chunks, k = blockIdx.y % max_chunks;
  if (c >= W) return;
  const int t0 = q_start[s] + k * MG_CHUNK, t1 = min(q_start[s + 1], t0 + MG_CHUNK);
  if (t0 >= t1) return;
  const int slot = slots[s];
  if (slot < 0 || slot >= num_slots) {
    atomicOr(err, 8);
    return;
  }
  float S = init[(size_t)s * W + c];
  for (int j = 0; j < k; ++j) {
    const float* p = carry + ((size_t)(s * max_chunks + j) * 2) * W + c;
    S = fmaf(p[0], S, p[W]);
  }
  const float biasz = to_f32(bz[c]), biasx = to_f32(bx[c]);
  for (int tb = t0; tb < t1; tb += MG_BATCH) {
    float az[MG_BATCH], ax[MG_BATCH], ag[MG_BATCH];
#pragma unroll
    for (int i = 0; i < MG_BATCH; ++i) {
      const TA* r = zxg + (size_t)min(tb + i, t1 - 1) * stride + c;
      az[i] = to_f32(r[0]); ax[i] = to_f32(r[W]); ag[i] = to_f32(r[2 * W]);
    }
#pragma unroll
    for (int i = 0; i < MG_BATCH; ++i) {
      if (tb + i < t1) {
        const float z = sigmoid_f32(az[i] + biasz), u = ax[i] + biasx;
        const float cand = (u >= 0.f) ? u + 0.5f : sigmoid_f32(u);
        S = fmaf(1.0f - z, S, z * cand);
        out[(size_t)(tb + i) * W + c] = from_f32<TA>(S * (ag[i] * sigmoid_f32(ag[i])));
      }
    }
  }
  if (t1 == q_start[s + 1]) state[(size_t)slot * W + c] = S;
}

// work: float32 [S * max_chunks * 2 * W + S * W], max_chunks = ceil(max_q / 64)
RLLM_EXPORT int rllm_mingru_scan_chunked(const void* zxg, int stride, const void* bz, const void* bx, float* state,
                                         const int* q_start, const int* slots, int num_slots, void* out, int S,
                                         int W, int max_q, float* work, int act_dtype, int w_dtype, int* err,
                                         cudaStream_t stream) {
  if (S <= 0 || max_q <= 0) return 0;
  const int max_chunks = (max_q + MG_CHUNK - 1) / MG_CHUNK;
  if (W <= 0 || stride < 3 * W || num_slots <= 0 || (long long)S * max_chunks > 65535) return RLLM_E_BADARG;
  dim3 grid((W + MG_THREADS - 1) / MG_THREADS, S * max_chunks);
  float* carry = work;
  float* init = work + (size_t)S * max_chunks * 2 * W;
#define MG_LAUNCH(TA, TW)                                                                                   \
  do {                                                                                                      \
    rllm_launch_pdl(mingru_chunk_summary_kernel<TA, TW>, dim3(grid), dim3(MG_THREADS), (size_t)(0), stream, (const TA*)zxg, stride, (const TW*)bz, \
        (const TW*)bx, state, q_start, slots, num_slots, max_chunks, carry, init, W);                       \
    rllm_launch_pdl(mingru_chunk_scan_kernel<TA, TW>, dim3(grid), dim3(MG_THREADS), (size_t)(0), stream, (const TA*)zxg, stride, (const TW*)bz, \
        (const TW*)bx, state, q_start, slots, num_slots, max_chunks, carry, init, (TA*)out, W, err);        \
  } while (0)
  RLLM_DISPATCH_DTYPE(act_dtype, TA_, RLLM_DISPATCH_DTYPE(w_dtype, TW_, MG_LAUNCH(TA_, TW_)));
#undef MG_LAUNCH
  RLLM_LAUNCH_CHECK();
  return 0;
}

RLLM_EXPORT int rllm_mingru_scan(const void* zxg, int stride, const void* bz, const void* bx, float* state,
                                 const int* q_start, const int* slots, int num_slots, void* out, int S, int W,
                                 int act_dtype, int w_dtype, int* err, cudaStream_t stream) {
  if (S <= 0) return 0;
  if (W <= 0 || stride < 3 * W || num_slots <= 0 || S > 65535) return RLLM_E_BADARG;
  dim3 grid((W + MG_THREADS - 1) / MG_THREADS, S);
#define MG_LAUNCH(TA, TW)                                                                              \
  rllm_launch_pdl(mingru_scan_kernel<TA, TW>, dim3(grid), dim3(MG_THREADS), (size_t)(0), stream, (const TA*)zxg, stride, (const TW*)bz,   \
      (const TW*)bx, state, q_start, slots, num_slots, (TA*)out, W, err)
  RLLM_DISPATCH_DTYPE(act_dtype, TA_, RLLM_DISPATCH_DTYPE(w_dtype, TW_, MG_LAUNCH(TA_, TW_)));
#undef MG_LAUNCH
  RLLM_LAUNCH_CHECK();
  return 0;
}
