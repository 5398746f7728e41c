// Routed feed-forward (mixture of experts): router, grouping of tokens by expert, the experts' products
// over the grouped rows, and the weighted sum back into token order.
//
// qv_moe_route    logits = Wr h in float32 (fixed summation order), the `top` largest per token (ties: the lower
//                 index), weights = softmax over the chosen logits only; optionally one more row of the router
//                 matrix' companion (a scalar gate per token: sigmoid(ws . h)).
// qv_moe_route_table  no router: row `token id` of an integer table [vocab, top] lists the token's experts, each weighted 1/top.
// qv_moe_group    counting sort of the (token, choice) pairs by expert, all on the device (a step never waits
//                 for the host): row_token[r] = token of sorted row r, slot_row[token * top + j] = its sorted row,
//                 and a table of row tiles (expert, first row, rows) for the products' grids.
// qv_moe_experts  CUDA-core products over the grouped rows, float32 multiply-adds with k ascending:
//                   UP (1):   act[r] = silu(Wg_e h[row_token[r]]) * (Wu_e h[row_token[r]])
//                   UP (2):   act[r] = relu(Wu_e h[row_token[r]])^2            (ungated experts)
//                   DOWN (0): y[r]   = Wd_e act[r]   (float32)
// qv_moe_combine  delta[t] = (mixer output) * s_mix + (sum_j weight[t, j] * y[slot_row[t, j]] + gate[t] * shared[t]) * s_ff
//                 in float32, choices summed in the order the router ranked them; s_mix, s_ff: per-feature factors or none.
#include "common.cuh"

#define ROUTE_WARPS 8
// One warp's dot product of a weight row with the token's inputs (float32 in shared memory), summed over the warp.
template <typename TW>
__device__ __forceinline__ float route_dot(const TW* __restrict__ w, const float* __restrict__ xs, int d, int lane) {
  // 16-byte loads, eight in flight per lane, where the rows allow; the order of the sum depends on d only
    float acc = 0.f;
    constexpr int VEC = 16 / (int)sizeof(TW);
    int i = 0;
    if ((d % VEC) == 0 && (((uintptr_t)w) & 15) == 0) {
      for (i = lane * VEC; i + 7 * 32 * VEC < d; i += 8 * 32 * VEC) {
        uint4 wv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) wv[u] = *(const uint4*)(w + i + u * 32 * VEC);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const TW* p = (const TW*)&wv[u];
#pragma unroll
          for (int k = 0; k < VEC; ++k) acc = fmaf(to_f(p[k]), xs[i + u * 32 * VEC + k], acc);
        }
      }
      for (; i < d; i += 32 * VEC) {
        const uint4 wv = *(const uint4*)(w + i);
        const TW* p = (const TW*)&wv;
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc = fmaf(to_f(p[k]), xs[i + k], acc);
      }
    } else {
      for (i = lane; i + 7 * 32 < d; i += 8 * 32) {
        float wv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) wv[u] = to_f(w[i + u * 32]);
#pragma unroll
        for (int u = 0; u < 8; ++u) acc = fmaf(wv[u], xs[i + u * 32], acc);
      }
      for (; i < d; i += 32) acc = fmaf(to_f(w[i]), xs[i], acc);
    }
    return warp_sum(acc);
}

// logits[t][e] = wr[e] . h[t] for e < E, and logits[t][E] = wg . h[t] when wg is given: eight rows a CTA, so that a
// step of few tokens still spreads the router's matrix over many SMs.
template <typename T, typename TW>
__global__ void __launch_bounds__(ROUTE_WARPS * 32) moe_logits_kernel(float* __restrict__ logits, const T* __restrict__ h, int ld_h,
                                                                      const TW* __restrict__ wr, const TW* __restrict__ wg, int d, int E) {
  extern __shared__ float xs_only[];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* x = h + (size_t)t * ld_h;
  for (int i = threadIdx.x; i < d; i += blockDim.x) xs_only[i] = to_f(x[i]);
  __syncthreads();
  const int e = blockIdx.y * ROUTE_WARPS + warp;
  if (e >= E + (wg ? 1 : 0)) return;
  const float acc = route_dot(e < E ? wr + (size_t)e * d : wg, xs_only, d, lane);
  if (lane == 0) logits[(size_t)t * (E + 1) + e] = acc;
}

// The same dot products for ROUTE_TOKENS tokens at once: a weight row is read once for all of them, and every token's sum has
// the order route_dot gives it (a lane's elements ascending, then the warp's tree), so the logits do not depend on which kernel
// formed them.  xs: [ROUTE_TOKENS][d] float32 in shared memory.
#define ROUTE_TOKENS 8
template <typename TW>
__device__ __forceinline__ void route_dot_tokens(const TW* __restrict__ w, const float* __restrict__ xs, int d, int lane, float (&acc)[ROUTE_TOKENS]) {
  constexpr int VEC = 16 / (int)sizeof(TW);
#pragma unroll
  for (int t = 0; t < ROUTE_TOKENS; ++t) acc[t] = 0.f;
  int i = 0;
  if ((d % VEC) == 0 && (((uintptr_t)w) & 15) == 0) {
    for (i = lane * VEC; i + 7 * 32 * VEC < d; i += 8 * 32 * VEC) {
      uint4 wv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) wv[u] = *(const uint4*)(w + i + u * 32 * VEC);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const TW* p = (const TW*)&wv[u];
        float wf[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) wf[k] = to_f(p[k]);
#pragma unroll
        for (int t = 0; t < ROUTE_TOKENS; ++t) {
          const float4* x4 = (const float4*)(xs + (size_t)t * d + i + u * 32 * VEC);
#pragma unroll
          for (int k4 = 0; k4 < VEC / 4; ++k4) {
            const float4 xv = x4[k4];
            acc[t] = fmaf(wf[4 * k4], xv.x, acc[t]); acc[t] = fmaf(wf[4 * k4 + 1], xv.y, acc[t]);
            acc[t] = fmaf(wf[4 * k4 + 2], xv.z, acc[t]); acc[t] = fmaf(wf[4 * k4 + 3], xv.w, acc[t]);
          }
        }
      }
    }
    for (; i < d; i += 32 * VEC) {
      const uint4 wv = *(const uint4*)(w + i);
      const TW* p = (const TW*)&wv;
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        const float wf = to_f(p[k]);
#pragma unroll
        for (int t = 0; t < ROUTE_TOKENS; ++t) acc[t] = fmaf(wf, xs[(size_t)t * d + i + k], acc[t]);
      }
    }
  } else {
    for (i = lane; i + 7 * 32 < d; i += 8 * 32) {
      float wv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) wv[u] = to_f(w[i + u * 32]);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
#pragma unroll
        for (int t = 0; t < ROUTE_TOKENS; ++t) acc[t] = fmaf(wv[u], xs[(size_t)t * d + i + u * 32], acc[t]);
      }
    }
    for (; i < d; i += 32) {
      const float wf = to_f(w[i]);
#pragma unroll
      for (int t = 0; t < ROUTE_TOKENS; ++t) acc[t] = fmaf(wf, xs[(size_t)t * d + i], acc[t]);
    }
  }
#pragma unroll
  for (int t = 0; t < ROUTE_TOKENS; ++t) acc[t] = warp_sum(acc[t]);
}

// Many tokens: a CTA takes ROUTE_TOKENS tokens and eight rows, so the router's matrix is read once per group of tokens
// instead of once per token.  d a multiple of 4 (16-byte reads of the tokens' rows in shared memory).
template <typename T, typename TW>
__global__ void __launch_bounds__(ROUTE_WARPS * 32) moe_logits_tokens_kernel(float* __restrict__ logits, const T* __restrict__ h, int ld_h,
                                                                             const TW* __restrict__ wr, const TW* __restrict__ wg, int d,
                                                                             int E, int T_all) {
  extern __shared__ __align__(16) float xs_tokens[];
  pdl_wait();
  pdl_launch_dependents();
  const int t0 = blockIdx.x * ROUTE_TOKENS, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < ROUTE_TOKENS * d; i += blockDim.x) {
    const int t = i / d, c = i - t * d;
    xs_tokens[i] = t0 + t < T_all ? to_f(h[(size_t)(t0 + t) * ld_h + c]) : 0.f;
  }
  __syncthreads();
  const int e = blockIdx.y * ROUTE_WARPS + warp;
  if (e >= E + (wg ? 1 : 0)) return;
  float acc[ROUTE_TOKENS];
  route_dot_tokens(e < E ? wr + (size_t)e * d : wg, xs_tokens, d, lane, acc);
  if (lane == 0) {
#pragma unroll
    for (int t = 0; t < ROUTE_TOKENS; ++t)
      if (t0 + t < T_all) logits[(size_t)(t0 + t) * (E + 1) + e] = acc[t];
  }
}

// pre: logits worked out by moe_logits_kernel ([T][E + 1]), or null: then this kernel forms them itself.
template <typename T, typename TW>
__global__ void __launch_bounds__(ROUTE_WARPS * 32) moe_route_kernel(int* __restrict__ top_idx, float* __restrict__ top_w, float* __restrict__ gate_out,
                                                        const T* __restrict__ h, int ld_h, const TW* __restrict__ wr,
                                                        const TW* __restrict__ wg, int d, int E, int top, const float* __restrict__ pre) {
  extern __shared__ float logit[];           // E floats, then the token's d inputs
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* xs = logit + E;
  if (pre) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) logit[e] = pre[(size_t)t * (E + 1) + e];
    if (wg && threadIdx.x == 0) gate_out[t] = 1.0f / (1.0f + expf(-pre[(size_t)t * (E + 1) + E]));
  } else {
    const T* x = h + (size_t)t * ld_h;
    for (int i = threadIdx.x; i < d; i += blockDim.x) xs[i] = to_f(x[i]);
    __syncthreads();
  }
  for (int e = warp; e < E + (wg ? 1 : 0) && !pre; e += ROUTE_WARPS) {
    float acc = route_dot(e < E ? wr + (size_t)e * d : wg, xs, d, lane);
    if (lane == 0) {
      if (e < E) logit[e] = acc;
      else gate_out[t] = 1.0f / (1.0f + expf(-acc));
    }
  }
  __syncthreads();
  if (warp != 0) return;
  float first = 0.f, denom = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = logit[e];
      if (v > best) { best = v; bi = e; }      // ascending e: the lowest index wins a tie within a lane
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (j == 0) first = best;
    const float p = expf(best - first);         // the first choice is the largest: exponents are <= 0
    denom += p;
    if (lane == 0) {
      top_idx[(size_t)t * top + j] = bi < E ? bi : 0;          // (not-a-number logits: still an expert that exists)
      top_w[(size_t)t * top + j] = p;
      if (bi < E) logit[bi] = -INFINITY;
    }
    __syncwarp();
  }
  for (int j = lane; j < top; j += 32) top_w[(size_t)t * top + j] /= denom;
}

// logits_ws: room for T * (E + 1) floats, or null.  With it, the logits are formed in a launch of their own: for steps of up to
// 256 tokens over (tokens x groups of eight rows) CTAs, for longer ones over (groups of eight tokens x groups of eight rows); the
// result is the same whichever kernel forms them (same sums, same order).
extern "C" int qv_moe_route(int* top_idx, float* top_w, float* gate_out, const void* h, int ld_h, const void* wr, const void* wg,
                            float* logits_ws, int T, int d, int E, int top, int dt, int w_dt, void* stream) {
  if (T <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || E > 8192) return QV_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)(E + d) * sizeof(float);
  if (smem > 48 * 1024) return QV_ERR_TOO_LARGE;
  const bool split = logits_ws && T <= 256;
  // more tokens: the logits by groups of tokens, where the group's rows fit shared memory
  const size_t tsmem = (size_t)ROUTE_TOKENS * d * sizeof(float);
  const bool tokens = logits_ws && !split && d % 4 == 0 && tsmem <= 160 * 1024;
  const dim3 lgrid(T, (E + (wg ? 1 : 0) + ROUTE_WARPS - 1) / ROUTE_WARPS);
  const dim3 tgrid((T + ROUTE_TOKENS - 1) / ROUTE_TOKENS, (E + (wg ? 1 : 0) + ROUTE_WARPS - 1) / ROUTE_WARPS);
#define ROUTE(TT, TW)                                                                                                        \
  do {                                                                                                                       \
    if (split) {                                                                                                             \
      const int rc = qv_launch(moe_logits_kernel<TT, TW>, lgrid, dim3(ROUTE_WARPS * 32), (size_t)d * sizeof(float), st, logits_ws, \
                               (const TT*)h, ld_h, (const TW*)wr, (const TW*)wg, d, E);                                      \
      if (rc) return rc;                                                                                                     \
    } else if (tokens) {                                                                                                     \
      if (tsmem > 48 * 1024)                                                                                                 \
        cudaFuncSetAttribute(moe_logits_tokens_kernel<TT, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tsmem);     \
      const int rc = qv_launch(moe_logits_tokens_kernel<TT, TW>, tgrid, dim3(ROUTE_WARPS * 32), tsmem, st, logits_ws,        \
                               (const TT*)h, ld_h, (const TW*)wr, (const TW*)wg, d, E, T);                                   \
      if (rc) return rc;                                                                                                     \
    }                                                                                                                        \
    return qv_launch(moe_route_kernel<TT, TW>, dim3(T), dim3(ROUTE_WARPS * 32), smem, st, top_idx, top_w, gate_out, (const TT*)h, \
                     ld_h, (const TW*)wr, (const TW*)wg, d, E, top,                                                          \
                     (split || tokens) ? (const float*)logits_ws : (const float*)nullptr);                                   \
  } while (0)
  if (dt == QV_DT_F32 && w_dt == QV_DT_F32) ROUTE(float, float);
  if (dt == QV_DT_BF16 && w_dt == QV_DT_BF16) ROUTE(bf16, bf16);
  if (dt == QV_DT_BF16 && w_dt == QV_DT_F32) ROUTE(bf16, float);
  if (dt == QV_DT_F32 && w_dt == QV_DT_BF16) ROUTE(float, bf16);
#undef ROUTE
  return QV_ERR_UNSUPPORTED;
}

// top_idx[t][j] = table[ids[t]][j] (an entry outside 0..E-1, which a sound table has not, reads as expert 0), top_w = 1/top.
__global__ void moe_route_table_kernel(int* __restrict__ top_idx, float* __restrict__ top_w, const int* __restrict__ table,
                                       const int* __restrict__ ids, int n, int top, int vocab, int E) {
  pdl_wait();
  pdl_launch_dependents();
  const float w = 1.0f / (float)top;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int t = i / top, j = i - t * top;
    int id = ids[t];
    if (id < 0 || id >= vocab) id = 0;
    const int e = table[(size_t)id * top + j];
    top_idx[i] = (e >= 0 && e < E) ? e : 0;
    top_w[i] = w;
  }
}

extern "C" int qv_moe_route_table(int* top_idx, float* top_w, const int* table, const int* ids, int T, int top, int vocab, int E,
                                  void* stream) {
  if (T <= 0) return 0;
  if (top <= 0 || E <= 0 || top > E) return QV_ERR_UNSUPPORTED;
  const int n = T * top;
  const int blocks = (n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8;
  return qv_launch(moe_route_table_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, top_idx, top_w, table, ids, n, top, vocab, E);
}

// One block.  tiles: [max_tiles][3] = (expert or -1, first sorted row, rows).
__global__ void __launch_bounds__(1024) moe_group_kernel(int* __restrict__ row_token, int* __restrict__ slot_row, int* __restrict__ tiles,
                                                         int max_tiles, const int* __restrict__ top_idx, int* __restrict__ rank_tmp,
                                                         int R, int top, int E, int bm) {
  extern __shared__ int cnt[];               // E counts, then E offsets
  pdl_wait();
  pdl_launch_dependents();
  int* off = cnt + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int r = threadIdx.x; r < R; r += blockDim.x) rank_tmp[r] = atomicAdd(&cnt[top_idx[r]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, n = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = o;
      for (int r0 = 0; r0 < cnt[e] && n < max_tiles; r0 += bm, ++n) {
        tiles[3 * n] = e;
        tiles[3 * n + 1] = o + r0;
        tiles[3 * n + 2] = cnt[e] - r0 < bm ? cnt[e] - r0 : bm;
      }
      o += cnt[e];
    }
    for (; n < max_tiles; ++n) { tiles[3 * n] = -1; tiles[3 * n + 1] = 0; tiles[3 * n + 2] = 0; }
  }
  __syncthreads();
  for (int r = threadIdx.x; r < R; r += blockDim.x) {
    const int pos = off[top_idx[r]] + rank_tmp[r];
    slot_row[r] = pos;
    row_token[pos] = r / top;
  }
}

#define MOE_BM 32
#define MOE_BN 64
#define MOE_BK 16

#define MOE_TC_BM 64       // rows of a tile of the tensor-core kernel

extern "C" int qv_moe_tile_rows(int tensor_cores) { return tensor_cores ? MOE_TC_BM : MOE_BM; }

extern "C" int qv_moe_max_tiles(int R, int E, int bm) {
  const int a = (R + bm - 1) / bm + E;
  return a < R ? a : R;
}

extern "C" int qv_moe_group(int* row_token, int* slot_row, int* tiles, const int* top_idx, int* rank_tmp, int T, int top, int E,
                            int bm, void* stream) {
  if (T <= 0) return 0;
  if (E > 8192 || bm <= 0) return QV_ERR_UNSUPPORTED;
  const int R = T * top;
  return qv_launch(moe_group_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), (cudaStream_t)stream, row_token, slot_row, tiles,
                   qv_moe_max_tiles(R, E, bm), top_idx, rank_tmp, R, top, E, bm);
}

// Tile of 32 rows x 64 columns, 256 threads, each 2 rows x 4 columns; k in steps of 16, ascending.
// MODE 1 (gated up): a = h (rows gathered by row_token), w1/w2 = gate/up matrices [E][N][K]; out act [R, N] in the compute type.
// MODE 2 (ungated up): as 1 with w1 the up matrices alone and the square of relu as activation.
// MODE 0 (down): a = act [R, K]; w1 = down matrices [E][N][K]; out y [R, N] float32.
template <typename T, typename TW, int MODE>
__global__ void __launch_bounds__(256) moe_experts_kernel(void* __restrict__ out_, int ld_out, const T* __restrict__ a, int ld_a,
                                                          const TW* __restrict__ w1, const TW* __restrict__ w2,
                                                          const int* __restrict__ row_token, const int* __restrict__ tiles, int N, int K) {
  constexpr bool GATHER = MODE != 0;         // rows of a are gathered, the output is in the compute type
  constexpr bool UP = MODE == 1;             // a second matrix (the gate's partner)
  __shared__ float As[MOE_BK][MOE_BM + 1];
  __shared__ float B1[MOE_BK][MOE_BN + 1];
  __shared__ float B2[UP ? MOE_BK : 1][MOE_BN + 1];
  pdl_wait();
  pdl_launch_dependents();
  const int e = tiles[3 * blockIdx.y];
  if (e < 0) return;
  const int row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
  const int n0 = blockIdx.x * MOE_BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const TW* W1 = w1 + (size_t)e * N * K;
  const TW* W2 = UP ? w2 + (size_t)e * N * K : nullptr;
  float acc1[2][4] = {}, acc2[2][4] = {};
  // loaders: A tile 32 x 16 (2 elements a thread), B tiles 64 x 16 (4 elements a thread)
  const int ar = threadIdx.x >> 3, ak = (threadIdx.x & 7) * 2;
  size_t a_row = 0;
  const bool a_ok = ar < rows;
  if (a_ok) a_row = GATHER ? (size_t)row_token[row0 + ar] : (size_t)(row0 + ar);
  const int bn = threadIdx.x >> 2, bk = (threadIdx.x & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += MOE_BK) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int k = k0 + ak + i;
      As[ak + i][ar] = (a_ok && k < K) ? to_f(a[a_row * ld_a + k]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + bk + i, n = n0 + bn;
      const bool ok = n < N && k < K;
      B1[bk + i][bn] = ok ? to_f(W1[(size_t)n * K + k]) : 0.f;
      if (UP) B2[bk + i][bn] = ok ? to_f(W2[(size_t)n * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < MOE_BK; ++k) {
      const float a0 = As[k][ty * 2], a1 = As[k][ty * 2 + 1];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float b = B1[k][tx * 4 + c];
        acc1[0][c] = fmaf(a0, b, acc1[0][c]);
        acc1[1][c] = fmaf(a1, b, acc1[1][c]);
        if (UP) {
          const float b2 = B2[k][tx * 4 + c];
          acc2[0][c] = fmaf(a0, b2, acc2[0][c]);
          acc2[1][c] = fmaf(a1, b2, acc2[1][c]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = ty * 2 + r;
    if (row >= rows) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int n = n0 + tx * 4 + c;
      if (n >= N) continue;
      if (UP) {
        const float g = acc1[r][c];
        ((T*)out_)[(size_t)(row0 + row) * ld_out + n] = from_f<T>(g / (1.0f + expf(-g)) * acc2[r][c]);
      } else if (MODE == 2) {
        const float g = fmaxf(acc1[r][c], 0.f);
        ((T*)out_)[(size_t)(row0 + row) * ld_out + n] = from_f<T>(g * g);
      } else {
        ((float*)out_)[(size_t)(row0 + row) * ld_out + n] = acc1[r][c];
      }
    }
  }
}

extern "C" int qv_moe_experts(int up, void* out, int ld_out, const void* a, int ld_a, const void* w1, const void* w2,
                              const int* row_token, const int* tiles, int R, int E, int N, int K, int dt, int w_dt, void* stream) {
  if (R <= 0) return 0;
  const int max_tiles = qv_moe_max_tiles(R, E, MOE_BM);
  if (max_tiles > 65535) return QV_ERR_TOO_LARGE;
  dim3 grid((N + MOE_BN - 1) / MOE_BN, max_tiles);
  cudaStream_t st = (cudaStream_t)stream;
#define EXPERTS(TT, TW)                                                                                                        \
  do {                                                                                                                         \
    if (up == 1) return qv_launch(moe_experts_kernel<TT, TW, 1>, grid, dim3(256), 0, st, out, ld_out, (const TT*)a, ld_a, (const TW*)w1, \
                                  (const TW*)w2, row_token, tiles, N, K);                                                      \
    if (up == 2) return qv_launch(moe_experts_kernel<TT, TW, 2>, grid, dim3(256), 0, st, out, ld_out, (const TT*)a, ld_a, (const TW*)w1, \
                                  (const TW*)w2, row_token, tiles, N, K);                                                      \
    return qv_launch(moe_experts_kernel<TT, TW, 0>, grid, dim3(256), 0, st, out, ld_out, (const TT*)a, ld_a, (const TW*)w1,      \
                     (const TW*)w2, row_token, tiles, N, K);                                                                   \
  } while (0)
  if (dt == QV_DT_F32 && w_dt == QV_DT_F32) EXPERTS(float, float);
  if (dt == QV_DT_BF16 && w_dt == QV_DT_BF16) EXPERTS(bf16, bf16);
  if (dt == QV_DT_BF16 && w_dt == QV_DT_F32) EXPERTS(bf16, float);
  if (dt == QV_DT_F32 && w_dt == QV_DT_BF16) EXPERTS(float, bf16);
#undef EXPERTS
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- the experts' products on the tensor cores (bfloat16)
// Tile of 64 grouped rows x 64 columns, k in steps of BK through a cp.async ring of STAGES buffers; four warps, each
// 32 x 32 as mma.sync m16n8k16 with float32 accumulators; rows of A are gathered by row_token (UP) while they
// are copied, rows past the tile's end and k past K are zero-filled.  K must be a multiple of 8.
#define TC_BN 64

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int bytes) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MODE, int BK, int STAGES>
__global__ void __launch_bounds__(128) moe_experts_tc_kernel(void* __restrict__ out_, int ld_out, const bf16* __restrict__ a, int ld_a,
                                                             const bf16* __restrict__ w1, const bf16* __restrict__ w2,
                                                             const int* __restrict__ row_token, const int* __restrict__ tiles, int N, int K) {
  constexpr bool GATHER = MODE != 0;         // modes as in moe_experts_kernel
  constexpr bool UP = MODE == 1;
  constexpr int LD = BK + 8;                 // padded row of a staged tile: ldmatrix without bank conflicts
  constexpr int PIECES = BK / 8;             // 16-byte pieces of a row
  constexpr int TILE = 64 * LD;              // elements of one staged 64-row tile
  extern __shared__ __align__(16) unsigned char moe_smem[];
  bf16* As = (bf16*)moe_smem;                // [STAGES][64][LD]
  bf16* B1 = As + STAGES * TILE;             // [STAGES][64][LD]
  bf16* B2 = B1 + STAGES * TILE;             // [STAGES][64][LD] (UP)
  pdl_wait();
  pdl_launch_dependents();
  const int e = tiles[3 * blockIdx.y];
  if (e < 0) return;
  const int row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
  const int n0 = blockIdx.x * TC_BN;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 1, wn = warp & 1;
  // weights are packed: [expert][N/64][K/64] tiles of 64 rows x 64 k, each 8 KB contiguous (zero-padded at the edges)
  static_assert(BK == 64, "a stage is one packed tile");
  const int NT = (N + 63) / 64, KT = (K + 63) / 64;
  const bf16* W1 = w1 + ((size_t)e * NT + blockIdx.x) * KT * 4096;
  const bf16* W2 = UP ? w2 + ((size_t)e * NT + blockIdx.x) * KT * 4096 : nullptr;
  auto stage = [&](int buf, int k0) {
    if (k0 < K) {
      const size_t tile_off = (size_t)(k0 / 64) * 4096;
      for (int c = tid; c < 64 * PIECES; c += 128) {
        const int r = c / PIECES, pc = c - r * PIECES, k = k0 + pc * 8;
        const bool kin = k < K, aok = r < rows && kin;
        const size_t src_row = aok ? (GATHER ? (size_t)row_token[row0 + r] : (size_t)(row0 + r)) : 0;
        cp_async16(As + buf * TILE + r * LD + pc * 8, a + src_row * ld_a + (kin ? k : 0), aok ? 16 : 0);
        cp_async16(B1 + buf * TILE + r * LD + pc * 8, W1 + tile_off + c * 8, 16);
        if (UP) cp_async16(B2 + buf * TILE + r * LD + pc * 8, W2 + tile_off + c * 8, 16);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");      // one group a stage, empty past the end, so the counts below hold
  };
  float acc1[2][4][4] = {}, acc2[UP ? 2 : 1][4][4] = {};
  const int nk = (K + BK - 1) / BK;
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) stage(st, st * BK);
  for (int kt = 0; kt < nk; ++kt) {
    const int buf = kt % STAGES;
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();                         // stage kt has landed for everyone; the buffer refilled next was read a round ago
    stage((kt + STAGES - 1) % STAGES, (kt + STAGES - 1) * BK);
    const bf16* Ab = As + buf * TILE;
    const bf16* B1b = B1 + buf * TILE;
    const bf16* B2b = B2 + buf * TILE;
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
      uint32_t af[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
        ldsm4(af[mt][0], af[mt][1], af[mt][2], af[mt][3], Ab + (wm * 32 + mt * 16 + (lane & 15)) * LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int pr = 0; pr < 2; ++pr) {
        const int n = wn * 32 + pr * 16 + (lane >> 4) * 8 + (lane & 7), k = ks * 16 + ((lane >> 3) & 1) * 8;
        uint32_t b[4];
        ldsm4(b[0], b[1], b[2], b[3], B1b + n * LD + k);
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          mma16816(acc1[mt][pr * 2], af[mt], b[0], b[1]);
          mma16816(acc1[mt][pr * 2 + 1], af[mt], b[2], b[3]);
        }
        if (UP) {
          ldsm4(b[0], b[1], b[2], b[3], B2b + n * LD + k);
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            mma16816(acc2[mt][pr * 2], af[mt], b[0], b[1]);
            mma16816(acc2[mt][pr * 2 + 1], af[mt], b[2], b[3]);
          }
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  // accumulator (mt, nt): rows wm*32 + mt*16 + lane/4 (+8), columns wn*32 + nt*8 + 2*(lane%4) (+1)
#pragma unroll
  for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * 32 + mt * 16 + (lane >> 2) + half * 8;
      if (r >= rows) continue;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int n = n0 + wn * 32 + nt * 8 + 2 * (lane & 3) + j;
          if (n >= N) continue;
          const float v = acc1[mt][nt][half * 2 + j];
          if (UP) ((bf16*)out_)[(size_t)(row0 + r) * ld_out + n] = __float2bfloat16_rn(v / (1.0f + expf(-v)) * acc2[mt][nt][half * 2 + j]);
          else if (MODE == 2) ((bf16*)out_)[(size_t)(row0 + r) * ld_out + n] = __float2bfloat16_rn(fmaxf(v, 0.f) * fmaxf(v, 0.f));
          else ((float*)out_)[(size_t)(row0 + r) * ld_out + n] = v;
        }
      }
    }
  }
}

// As qv_moe_experts for bfloat16 operands, on the tensor cores, with the experts' matrices packed in tiles of 64 x 64
// ([E][ceil(N/64)][ceil(K/64)][64][64], zero-padded: what a stage copies is 8 KB in one piece, which memory delivers
// several times faster than 64 rows that lie a whole matrix row apart).  The tile table must have been made for tiles
// of qv_moe_tile_rows(1) rows.  Refuses rows of `a` that do not start on 16 bytes.
extern "C" int qv_moe_experts_tc(int up, void* out, int ld_out, const void* a, int ld_a, const void* w1, const void* w2,
                                 const int* row_token, const int* tiles, int R, int E, int N, int K, void* stream) {
  if (R <= 0) return 0;
  if ((ld_a & 7) || (((uintptr_t)a | (uintptr_t)w1 | (uintptr_t)w2) & 15)) return QV_ERR_UNSUPPORTED;
  const int max_tiles = qv_moe_max_tiles(R, E, MOE_TC_BM);
  if (max_tiles > 65535) return QV_ERR_TOO_LARGE;
  dim3 grid((N + TC_BN - 1) / TC_BN, max_tiles);
  cudaStream_t st = (cudaStream_t)stream;
  // k in steps of 64 through three stages: a row of a weight tile is then a whole 128-byte line and two stages of
  // copies are in flight while one is multiplied
  constexpr int BK = 64, STAGES = 3;
  const size_t smem = (size_t)STAGES * 64 * (BK + 8) * 2 * (up == 1 ? 3 : 2);
  if (up == 1) {
    cudaFuncSetAttribute(moe_experts_tc_kernel<1, BK, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return qv_launch(moe_experts_tc_kernel<1, BK, STAGES>, grid, dim3(128), smem, st, out, ld_out, (const bf16*)a, ld_a, (const bf16*)w1,
                     (const bf16*)w2, row_token, tiles, N, K);
  }
  if (up == 2) {
    cudaFuncSetAttribute(moe_experts_tc_kernel<2, BK, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return qv_launch(moe_experts_tc_kernel<2, BK, STAGES>, grid, dim3(128), smem, st, out, ld_out, (const bf16*)a, ld_a, (const bf16*)w1,
                     (const bf16*)w2, row_token, tiles, N, K);
  }
  cudaFuncSetAttribute(moe_experts_tc_kernel<0, BK, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return qv_launch(moe_experts_tc_kernel<0, BK, STAGES>, grid, dim3(128), smem, st, out, ld_out, (const bf16*)a, ld_a, (const bf16*)w1,
                   (const bf16*)w2, row_token, tiles, N, K);
}

// delta [T, d] float32.  mix, shared: [T, d] in the compute type or null; gate [T] float32 or null.
template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(float* __restrict__ delta, const T* __restrict__ mix, const float* __restrict__ y,
                                                          const int* __restrict__ slot_row, const float* __restrict__ top_w,
                                                          const T* __restrict__ shared, const float* __restrict__ gate, int d, int top,
                                                          const float* __restrict__ s_mix, const float* __restrict__ s_ff) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float g = gate ? gate[t] : 1.f;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < d; i += gridDim.y * blockDim.x) {
    float routed = 0.f;
    for (int j = 0; j < top; ++j) routed = fmaf(top_w[(size_t)t * top + j], y[(size_t)slot_row[(size_t)t * top + j] * d + i], routed);
    float v = routed;
    if (shared) v = fmaf(g, to_f(shared[(size_t)t * d + i]), v);
    if (s_ff) v *= s_ff[i];
    if (mix) v = fmaf(to_f(mix[(size_t)t * d + i]), s_mix ? s_mix[i] : 1.f, v);
    delta[(size_t)t * d + i] = v;
  }
}

extern "C" int qv_moe_combine(float* delta, const void* mix, const float* y, const int* slot_row, const float* top_w,
                              const void* shared, const float* gate, int T, int d, int top, int dt, const float* s_mix,
                              const float* s_ff, void* stream) {
  if (T <= 0) return 0;
  QV_DISPATCH_DT(dt, TT,
                 return qv_launch(moe_combine_kernel<TT>, dim3(T, T < 256 ? (d + 255) / 256 : 1), dim3(256), 0, (cudaStream_t)stream, delta, (const TT*)mix, y, slot_row,
                                  top_w, (const TT*)shared, gate, d, top, s_mix, s_ff));
  return QV_ERR_UNSUPPORTED;
}
