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
mingru_scan_kernel(const TA* __restrict__ zxg, int stride, const TW* __restrict__ bz, const TW* __restrict__ bx,
                   float* __restrict__ state, const int* __restrict__ q_start, const int* __restrict__ slots,
                   int num_slots, TA* __restrict__ out, int W, int* __restrict__ err) {
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

RLLM_EXPORT int rllm_mingru_scan(const void* zxg, int stride, const void* bz, const void* bx, float* state,
                                 const int* q_start, const int* slots, int num_slots, void* out, int S, int W,
                                 int act_dtype, int w_dtype, int* err, cudaStream_t stream) {
  if (S <= 0) return 0;
  if (W <= 0 || stride < 3 * W || num_slots <= 0 || S > 65535) return RLLM_E_BADARG;
  dim3 grid((W + MG_THREADS - 1) / MG_THREADS, S);
#define MG_LAUNCH(TA, TW)                                                                              \
  mingru_scan_kernel<TA, TW><<<grid, MG_THREADS, 0, stream>>>((const TA*)zxg, stride, (const TW*)bz,   \
      (const TW*)bx, state, q_start, slots, num_slots, (TA*)out, W, err)
  RLLM_DISPATCH_DTYPE(act_dtype, TA_, RLLM_DISPATCH_DTYPE(w_dtype, TW_, MG_LAUNCH(TA_, TW_)));
#undef MG_LAUNCH
  RLLM_LAUNCH_CHECK();
  return 0;
}
