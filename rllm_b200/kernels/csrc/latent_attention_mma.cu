// Attention over cached latent rows on the tensor cores (bfloat16 rows, float32
// scores, softmax and sums): the kernel of prompt portions and of decoding alike.
//
// All heads of a token read the same rows, so a CTA takes ROWS = 16 * MT consecutive
// (token, head) pairs of ONE sequence as the rows of its tiles, and walks the keys in
// tiles of 32 aligned to absolute positions (the arithmetic of a row does not depend
// on the cut of the sequence, the batch or the pages).  Per key tile: the 32 cached
// rows come in by cp.async through the block table (double buffered); warp w
// computes the scores of keys 8w .. 8w+7 for all rows (Q . K^T, mma.sync m16n8k16);
// the running max and sum of a row are combined across the warps in shared memory;
// the weights are written to shared memory as bfloat16 and each warp adds P . V for
// its own quarter of the value columns, V being the first dv columns of the very rows
// that served as keys (ldmatrix.trans).  A sink starts a row's running max at
// sink[h] and its sum at 1.  Exponentials are base 2 with log2(e) folded into the scale.
//
// Few rows and many keys (decoding): the key tiles are also cut into splits of
// `split_keys` keys at absolute positions, one CTA each (grid z); a split leaves
// its unnormalised sums, running max and sum in a work buffer and a second kernel
// adds the splits of a row in order (and the sink).  Where the cuts fall depends on
// the row's own sequence only.
#include "common.cuh"
#include <math.h>

// NW warps a CTA (4, or 8 where the values are wider than 64: their columns are shared out among more
// warps); a key tile has 8 keys a warp.

__device__ __forceinline__ void lam_cp16(void* smem_dst, const void* src, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void lam_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MT, int NVT, int NW>
__global__ void __launch_bounds__(32 * NW)
latent_attention_mma_kernel(const bf16* q, bf16* out, const bf16* cache,
                            const int* block_table, int max_blocks, const int* q_start,
                            const int* seq_lens, int heads, int dk, int dv, int ld, int page_size,
                            int num_pages, int window, float scale_log2, const float* sink,
                            int split_keys, float* work, int* err) {
  // (Every kernel of this file starts with the wait for the kernel ahead of it in the stream and lets the
  // next one in right after: launches overlap the tails of their predecessors.  The pointer parameters
  // carry no __restrict__, so that no load is proved independent of that wait and moved above it.)
  pdl_wait();
  pdl_launch();
  constexpr int ROWS = 16 * MT, LAM_THREADS = 32 * NW, LAM_KEYS = 8 * NW;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = (bf16*)smem_raw;                               // [ROWS][ld]
  bf16* Ks = Qs + (size_t)ROWS * ld;                        // [2][LAM_KEYS][ld]
  bf16* Ps = Ks + (size_t)2 * LAM_KEYS * ld;                // [ROWS][LAM_KEYS + 8]
  float* wmax = (float*)(Ps + ROWS * (LAM_KEYS + 8));       // [2][NW][ROWS]
  float* wsum = wmax + 2 * NW * ROWS;                       // [2][NW][ROWS]
  float* m_cur = wsum + 2 * NW * ROWS;                      // [ROWS]
  float* l_cur = m_cur + ROWS;                              // [ROWS]

  const int s = blockIdx.y;
  const int t0 = q_start[s], nq = q_start[s + 1] - t0;
  // among the sequence's nq * heads rows; the last rows see the most keys, so they are handed out first
  const int row_tiles = (nq * heads + ROWS - 1) / ROWS;
  if ((int)blockIdx.x >= row_tiles) return;
  const int row_base = (row_tiles - 1 - (int)blockIdx.x) * ROWS;
  const int seq_len = seq_lens[s];
  const int pos0 = seq_len - nq;                            // position of the sequence's first token of this step
  const int rows_here = min(ROWS, nq * heads - row_base);
  const int tok_lo = row_base / heads, tok_hi = (row_base + rows_here - 1) / heads;
  const int p_lo = pos0 + tok_lo, p_hi = pos0 + tok_hi;
  const int k_lo = (window > 0 && p_lo - window + 1 > 0) ? p_lo - window + 1 : 0;
  int tile_lo = k_lo / LAM_KEYS, tile_hi = p_hi / LAM_KEYS;           // inclusive
  const int dvp = 8 * NVT * NW;
  float* wrow = nullptr;              // split mode: where this CTA's rows leave their partial results
  const int split_tiles = split_keys / LAM_KEYS;
  if (split_tiles > 0) {
    tile_lo = max(tile_lo, (int)blockIdx.z * split_tiles);
    tile_hi = min(tile_hi, (int)(blockIdx.z + 1) * split_tiles - 1);
    wrow = work + (((size_t)s * gridDim.x * ROWS + row_base) * gridDim.z + blockIdx.z) * (dvp + 2);
    if (tile_lo > tile_hi) {          // nothing of this split is visible: an empty partial result
      if (threadIdx.x < rows_here) {
        float* w = wrow + (size_t)threadIdx.x * gridDim.z * (dvp + 2);
        w[dvp] = -INFINITY;
        w[dvp + 1] = 0.f;
      }
      return;
    }
  }
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int chunks = ld / 8 - 1;                            // 16-byte chunks of a row that are loaded (the pad is not)
  const int* bt = block_table + (size_t)s * max_blocks;

  // queries: rows row_base .. of the sequence's (token, head) pairs lie one behind the other in q
  const bf16* qsrc = q + ((size_t)t0 * heads + row_base) * dk;
  for (int c = tid; c < ROWS * chunks; c += LAM_THREADS) {
    const int r = c / chunks, kc = (c - r * chunks) * 8;
    const bool ok = r < rows_here && kc < dk;
    lam_cp16(Qs + (size_t)r * ld + kc, ok ? (const void*)(qsrc + (size_t)r * dk + kc) : (const void*)q, ok);
  }
  if (tid < ROWS) {
    const int h = (row_base + tid) % heads;
    const bool with_sink = sink != nullptr && split_keys <= 0;      // split mode: the merge adds the sink
    m_cur[tid] = with_sink ? sink[h] * 1.4426950408889634f : -INFINITY;
    l_cur[tid] = with_sink ? 1.f : 0.f;
  }

  // four threads a key row: the row's page is looked up once a tile, its 16-byte chunks are shared out by fours
  auto load_keys = [&](int tile, int st) {
    const int r = tid >> 2, j = tile * LAM_KEYS + r;
    bf16* dst = Ks + ((size_t)st * LAM_KEYS + r) * ld;
    bool ok = j >= k_lo && j <= p_hi;
    const bf16* src = cache;
    if (ok) {
      const int page = bt[j / page_size];
      if (page < 0 || page >= num_pages) {
        if ((tid & 3) == 0) atomicOr(err, 4);
        ok = false;
      } else {
        src = cache + ((size_t)page * page_size + (j % page_size)) * dk;
      }
    }
    for (int kc = (tid & 3) * 8; kc < chunks * 8; kc += 32) {
      const bool here = ok && kc < dk;
      lam_cp16(dst + kc, here ? (const void*)(src + kc) : (const void*)cache, here);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float o[MT][NVT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NVT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[mt][nt][i] = 0.f;
  // position of each row this thread holds scores of: rows mt * 16 + g and + 8
  int rpos[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int r = mt * 16 + g + 8 * hf;
      rpos[mt][hf] = (r < rows_here) ? pos0 + (row_base + r) / heads : -1;
    }

  load_keys(tile_lo, 0);
  const int ksteps = (dk + 31) / 32 * 2;                    // in pairs; the rows are zero beyond dk
  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    const int st = (tile - tile_lo) & 1, par = st;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (tile < tile_hi) load_keys(tile + 1, st ^ 1);
    const bf16* K = Ks + (size_t)st * LAM_KEYS * ld;
    // ---- scores of keys 8 warp .. 8 warp + 7 for all rows
    float sc[MT][4], sc2[MT][4];       // even and odd k steps add up apart: twice as many MMAs in flight
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[mt][i] = sc2[mt][i] = 0.f;
    // two k steps of 16 a round: one ldmatrix.x4 brings the keys' fragments of both (8 keys x 32 values),
    // one ldmatrix.x4 per row tile and k step the queries'
    const unsigned kaddr = (unsigned)__cvta_generic_to_shared(K + (size_t)(warp * 8 + (lane & 7)) * ld + (lane >> 3) * 8);
    const unsigned qaddr = (unsigned)__cvta_generic_to_shared(Qs + (size_t)(lane & 15) * ld + (lane >> 4) * 8);
    for (int ks = 0; ks < ksteps; ks += 2) {
      uint32_t b[4];
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                   : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(kaddr + ks * 32));
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t a[4];
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
                       : "r"(qaddr + (unsigned)((mt * 16 * ld + (ks + half) * 16) * 2)));
          if (half == 0) lam_mma(sc[mt], a, b[0], b[1]);
          else lam_mma(sc2[mt], a, b[2], b[3]);
        }
      }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[mt][i] += sc2[mt][i];
    const int jbase = tile * LAM_KEYS + warp * 8 + 2 * t;
    float* wm = wmax + (size_t)par * NW * ROWS;
    float* ws = wsum + (size_t)par * NW * ROWS;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int p = rpos[mt][hf];
        float mx = -INFINITY;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = jbase + e;
          const bool vis = p >= 0 && j <= p && (window <= 0 || p - j < window);
          const float v = vis ? sc[mt][2 * hf + e] * scale_log2 : -INFINITY;
          sc[mt][2 * hf + e] = v;
          mx = fmaxf(mx, v);
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        if (t == 0) wm[warp * ROWS + mt * 16 + g + 8 * hf] = mx;
      }
    __syncthreads();
    // ---- weights, their sums, and the factor that the rows' old sums shrink by
    float corr[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int r = mt * 16 + g + 8 * hf;
        const float mo = m_cur[r];
        float mn = mo;
#pragma unroll
        for (int w = 0; w < NW; ++w) mn = fmaxf(mn, wm[w * ROWS + r]);
        corr[mt][hf] = (mn == -INFINITY) ? 1.f : exp2f(mo - mn);
        float p0 = 0.f, p1 = 0.f;
        if (mn != -INFINITY) {
          p0 = exp2f(sc[mt][2 * hf] - mn);
          p1 = exp2f(sc[mt][2 * hf + 1] - mn);
        }
        float sum = p0 + p1;
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (t == 0) ws[warp * ROWS + r] = sum;
        *(__nv_bfloat162*)(Ps + (size_t)r * (LAM_KEYS + 8) + warp * 8 + 2 * t) = __floats2bfloat162_rn(p0, p1);
      }
    __syncthreads();
    if (tid < ROWS) {
      const int r = tid;
      const float mo = m_cur[r];
      float mn = mo, sum = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        mn = fmaxf(mn, wm[w * ROWS + r]);
        sum += ws[w * ROWS + r];
      }
      if (mn != -INFINITY) {
        l_cur[r] = l_cur[r] * exp2f(mo - mn) + sum;
        m_cur[r] = mn;
      }
    }
    // ---- O = O * corr + P . V for value columns [warp * NVT * 8, (warp + 1) * NVT * 8)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NVT; ++nt) {
        o[mt][nt][0] *= corr[mt][0]; o[mt][nt][1] *= corr[mt][0];
        o[mt][nt][2] *= corr[mt][1]; o[mt][nt][3] *= corr[mt][1];
      }
#pragma unroll
    for (int kk = 0; kk < LAM_KEYS; kk += 16) {
      uint32_t a[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const unsigned paddr = (unsigned)__cvta_generic_to_shared(
            Ps + (size_t)(mt * 16 + (lane & 15)) * (LAM_KEYS + 8) + kk + (lane >> 4) * 8);
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(a[mt][0]), "=r"(a[mt][1]), "=r"(a[mt][2]), "=r"(a[mt][3]) : "r"(paddr));
      }
      if constexpr (NVT % 2 == 0) {
#pragma unroll
        for (int nt = 0; nt < NVT; nt += 2) {
          // V^T fragments of two n-tiles: keys kk .. kk+15 (rows of K), columns col .. col+15
          const int col = (warp * NVT + nt) * 8;
          const unsigned addr = (unsigned)__cvta_generic_to_shared(
              K + (size_t)(kk + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + col + ((lane >> 4) & 1) * 8);
          uint32_t b[4];
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(addr));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            lam_mma(o[mt][nt], a[mt], b[0], b[1]);
            lam_mma(o[mt][nt + 1], a[mt], b[2], b[3]);
          }
        }
      } else {
#pragma unroll
        for (int nt = 0; nt < NVT; ++nt) {
          // V^T fragment: keys kk .. kk+15 (rows of K), columns col .. col+7; lanes 0-15 give the row addresses
          const int col = (warp * NVT + nt) * 8;
          const unsigned addr = (unsigned)__cvta_generic_to_shared(K + (size_t)(kk + (lane & 15)) * ld + col);
          uint32_t b0, b1;
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) lam_mma(o[mt][nt], a[mt], b0, b1);
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int r = mt * 16 + g + 8 * hf;
      if (r >= rows_here) continue;
      if (wrow != nullptr) {
        float* w = wrow + (size_t)r * gridDim.z * (dvp + 2);
#pragma unroll
        for (int nt = 0; nt < NVT; ++nt) {
          const int col = (warp * NVT + nt) * 8 + 2 * t;
          w[col] = o[mt][nt][2 * hf];
          w[col + 1] = o[mt][nt][2 * hf + 1];
        }
        if (warp == 0 && t == 0) { w[dvp] = m_cur[r]; w[dvp + 1] = l_cur[r]; }
        continue;
      }
      const float l = l_cur[r];
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      bf16* orow = out + ((size_t)t0 * heads + row_base + r) * dv;
#pragma unroll
      for (int nt = 0; nt < NVT; ++nt) {
        const int col = (warp * NVT + nt) * 8 + 2 * t;
        if (col + 1 < dv) {
          *(__nv_bfloat162*)(orow + col) = __floats2bfloat162_rn(o[mt][nt][2 * hf] * inv, o[mt][nt][2 * hf + 1] * inv);
        } else if (col < dv) {
          orow[col] = __float2bfloat16_rn(o[mt][nt][2 * hf] * inv);
        }
      }
    }
}

// one CTA per (sequence, row): the splits' factors first (running max over the splits and the sink), then a
// thread a value column adds the splits' partial sums in order
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const float* work, bf16* out, const int* q_start, int heads, int dv, int dvp,
                              int max_rows, int nsplit, const float* sink) {
  pdl_wait();
  pdl_launch();
  extern __shared__ float fac[];      // [nsplit]: 2^(m_z - M), 0 for a split that saw nothing
  __shared__ float red[32];
  const int row = blockIdx.x, s = blockIdx.y;
  const int t0 = q_start[s], nq = q_start[s + 1] - t0;
  if (row >= nq * heads) return;
  const float* w = work + (((size_t)s * max_rows + row) * nsplit) * (dvp + 2);
  const float sk = sink ? sink[row % heads] * 1.4426950408889634f : -INFINITY;
  float mx = sk;
  for (int z = threadIdx.x; z < nsplit; z += blockDim.x) mx = fmaxf(mx, w[(size_t)z * (dvp + 2) + dvp]);
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  const float M = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  __syncthreads();
  float part = 0.f;
  for (int z = threadIdx.x; z < nsplit; z += blockDim.x) {
    const float m = w[(size_t)z * (dvp + 2) + dvp], l = w[(size_t)z * (dvp + 2) + dvp + 1];
    const float fz = (l > 0.f && m != -INFINITY) ? exp2f(m - M) : 0.f;
    fac[z] = fz;
    part += l * fz;
  }
  part = block_sum(part, red);          // (its order depends on nsplit and the block size only)
  const float L = part + (sink ? exp2f(sk - M) : 0.f);
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  bf16* orow = out + ((size_t)t0 * heads + row) * dv;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float acc = 0.f;
    for (int z = 0; z < nsplit; ++z) {
      const float fz = fac[z];
      const float v = w[(size_t)z * (dvp + 2) + c];
      acc = fmaf(fz != 0.f ? v : 0.f, fz, acc);
    }
    orow[c] = __float2bfloat16_rn(acc * inv);
  }
}

template <int MT, int NVT, int NW>
static int lam_launch(const bf16* q, bf16* out, const bf16* cache, const int* block_table, int max_blocks,
                      const int* q_start, const int* seq_lens, int S, int max_q, int heads, int dk, int dv,
                      int page_size, int num_pages, int window, float scale, const float* sink, int split_keys,
                      int nsplit, float* work, int* err, cudaStream_t stream) {
  constexpr int ROWS = 16 * MT, LAM_THREADS = 32 * NW, LAM_KEYS = 8 * NW;
  const int dkp = (dk + 31) / 32 * 32;
  const int ld = max(dkp, 8 * NVT * NW) + 8;
  const size_t smem = ((size_t)ROWS * ld + 2 * LAM_KEYS * ld + ROWS * (LAM_KEYS + 8)) * sizeof(bf16) +
                      (size_t)(2 * NW * ROWS * 2 + 2 * ROWS) * sizeof(float);
  if (smem > 220 * 1024) return RLLM_E_UNSUPPORTED;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(latent_attention_mma_kernel<MT, NVT, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const long long blocks_x = ((long long)max_q * heads + ROWS - 1) / ROWS;
  if (blocks_x > 2147483647LL || S > 65535) return RLLM_E_UNSUPPORTED;
  dim3 grid((unsigned)blocks_x, S, split_keys > 0 ? nsplit : 1);
  rllm_launch_pdl(latent_attention_mma_kernel<MT, NVT, NW>, dim3(grid), dim3(LAM_THREADS), (size_t)(smem), stream, 
      q, out, cache, block_table, max_blocks, q_start, seq_lens, heads, dk, dv, ld, page_size, num_pages, window,
      scale * 1.4426950408889634f, sink, split_keys, work, err);
  RLLM_LAUNCH_CHECK();
  if (split_keys > 0) {
    const int max_rows = (int)blocks_x * ROWS;
    dim3 mg(max_rows, S);
    rllm_launch_pdl(latent_attention_merge_kernel, dim3(mg), dim3(128), (size_t)nsplit * sizeof(float), stream, work, out, q_start, heads, dv, 8 * NVT * NW, max_rows, nsplit, sink);
    RLLM_LAUNCH_CHECK();
  }
  return 0;
}

// work size in floats for a split launch: rows are padded to the row tile the launch will choose
RLLM_EXPORT long long rllm_latent_attention_mma_work(int S, int max_q, int heads, int dv, int nsplit) {
  const long long rows = (long long)max_q * heads;
  const int mt = rows <= 16 ? 1 : (rows <= 32 ? 2 : (dv > 256 ? 2 : 4));
  const int nvt = dv <= 32 ? 1 : (dv <= 64 ? 2 : (dv <= 128 ? 4 : (dv <= 256 ? 8 : 16)));
  const long long padded = (rows + 16 * mt - 1) / (16 * mt) * (16 * mt);
  return (long long)S * padded * nsplit * (32 * nvt + 2);
}

// q [T, heads * dk], out [T, heads * dv], cache [pages, 1, page_size, dk]; sequence s owns tokens
// q_start[s] .. q_start[s+1] and holds seq_lens[s] tokens after this step; max_q: the most tokens a
// sequence brings.  Needs dk % 8 == 0, dv <= min(dk, 512) and 16-byte aligned buffers.
RLLM_EXPORT int rllm_latent_attention_mma(const void* q, void* out, const void* cache, const int* block_table,
                                          int max_blocks, const int* q_start, const int* seq_lens, int S, int max_q,
                                          int heads, int dk, int dv, int page_size, int num_pages, int window,
                                          float scale, const float* sink, int split_keys, int nsplit, float* work,
                                          int* err, cudaStream_t stream) {
  if (S <= 0 || max_q <= 0) return 0;
  if (split_keys > 0 && (split_keys % 64 != 0 || nsplit <= 0 || nsplit > 8192 || work == nullptr)) return RLLM_E_BADARG;
  if (heads <= 0 || dk <= 0 || dv <= 0 || dv > dk || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 ||
      window < 0)
    return RLLM_E_BADARG;
  if (dk % 8 != 0 || dv > 512 || (((uintptr_t)q | (uintptr_t)out | (uintptr_t)cache) & 15) != 0)
    return RLLM_E_UNSUPPORTED;
#define LAM_GO(MT_, NVT_, NW_)                                                                              \
  return lam_launch<MT_, NVT_, NW_>((const bf16*)q, (bf16*)out, (const bf16*)cache, block_table, max_blocks, q_start, \
                               seq_lens, S, max_q, heads, dk, dv, page_size, num_pages, window, scale, sink,   \
                               split_keys, nsplit, work, err, stream)
  // as many row tiles of 16 as the sequences' rows fill, up to what the accumulators leave room for
  const long long rows = (long long)max_q * heads;
  const int mt = rows <= 16 ? 1 : (rows <= 32 ? 2 : 4);
#define LAM_PICK(NVT_, MAXMT_, NW_)                      \
  do {                                                   \
    if (mt == 1) LAM_GO(1, NVT_, NW_);                   \
    if (mt == 2 || MAXMT_ == 2) LAM_GO(2, NVT_, NW_);    \
    LAM_GO(MAXMT_, NVT_, NW_);                           \
  } while (0)
  if (dv <= 32) LAM_PICK(1, 4, 4);
  if (dv <= 64) LAM_PICK(2, 4, 4);
  if (dv <= 128) LAM_PICK(2, 4, 8);
  if (dv <= 256) LAM_PICK(4, 4, 8);
  LAM_PICK(8, 2, 8);
#undef LAM_PICK
#undef LAM_GO
}
