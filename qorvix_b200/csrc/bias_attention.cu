// Causal grouped-query softmax attention without rotation, whose positions enter through a learned bias on the
// scores and a temperature on the queries:
//
//   score(i, j, h) = (temp(i) q_i,h . k_j,g) * scale + bias[bucket[min(i - j, far)], h],     temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1)
//
// `bucket` (int32, far + 1 entries) maps a distance to a row of the bias table [rows, H] (float32); distances from `far` on
// share the last entry.  The table of buckets is built by the host, so the rule that spaces the rows is not part of the kernels.
// A token's cache row holds the keys of all key/value heads, then their values: [G * n | G * dv].
//
// qv_bias_attn_prepare      adds the projections' biases, scales q by the temperature of its position (float32, then rounded to
//                           the compute type) and writes k and v into the token's cache row.
// qv_bias_attention_generic one warp per (token, head), keys in blocks of 32 aligned to absolute positions, float32 throughout:
//                           the order of every sum depends on the token's position alone.
#include "common.cuh"

#define BA_MAX_DV 256

// proj [T, >= (H + G) * n + G * dv] float32: [q | k | v] starting at column offsets q_off, k_off, v_off.
template <typename T>
__global__ void __launch_bounds__(256) bias_attn_prepare_kernel(T* __restrict__ q_out, int ld_qo, const float* __restrict__ proj, int ld_p,
                                                               int q_off, int k_off, int v_off, const float* __restrict__ bq,
                                                               const float* __restrict__ bk, const float* __restrict__ bv,
                                                               T* __restrict__ cache, const int* __restrict__ tok_pos,
                                                               const int* __restrict__ tok_seg, const int* __restrict__ block_table,
                                                               int max_blocks, int H, int G, int n, int dv, int page, float coef, int every) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const float* row = proj + (size_t)t * ld_p;
  const float temp = 1.0f + coef * logf((float)((pos + 1) / every + 1));
  const int nq = H * n, nk = G * n, nv = G * dv;
  const size_t width = (size_t)nk + nv;
  const int pg = block_table[(size_t)tok_seg[t] * max_blocks + pos / page];
  T* crow = cache + ((size_t)pg * page + (size_t)(pos % page)) * width;
  for (int i = threadIdx.x; i < nq + nk + nv; i += blockDim.x) {
    if (i < nq) {
      q_out[(size_t)t * ld_qo + i] = from_f<T>((row[q_off + i] + (bq ? bq[i] : 0.f)) * temp);
    } else if (i < nq + nk) {
      const int c = i - nq;
      crow[c] = from_f<T>(row[k_off + c] + (bk ? bk[c] : 0.f));
    } else {
      const int c = i - nq - nk;
      crow[nk + c] = from_f<T>(row[v_off + c] + (bv ? bv[c] : 0.f));
    }
  }
}

extern "C" int qv_bias_attn_prepare(void* q_out, int ld_qo, const float* proj, int ld_p, int q_off, int k_off, int v_off, const float* bq,
                                    const float* bk, const float* bv, void* cache, const int* tok_pos, const int* tok_seg,
                                    const int* block_table, int max_blocks, int T, int H, int G, int n, int dv, int page, float coef,
                                    int every, int dt, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || n <= 0 || dv <= 0 || every <= 0) return QV_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t esz = dt == QV_DT_F32 ? 4 : 2;
  for (int done = 0; done < T; done += 65535) {
    const int rows = T - done < 65535 ? T - done : 65535;
    int rc = QV_ERR_UNSUPPORTED;
    QV_DISPATCH_DT(dt, TT,
                   rc = qv_launch(bias_attn_prepare_kernel<TT>, dim3(rows), dim3(256), 0, st,
                                  (TT*)((char*)q_out + (size_t)done * ld_qo * esz), ld_qo, proj + (size_t)done * ld_p, ld_p, q_off, k_off,
                                  v_off, bq, bk, bv, (TT*)cache, tok_pos + done, tok_seg + done, block_table, max_blocks, H, G, n, dv,
                                  page, coef, every));
    if (rc) return rc;
  }
  return 0;
}

template <typename T>
__global__ void __launch_bounds__(128) bias_attention_generic_kernel(
    T* __restrict__ out, int ld_out, const T* __restrict__ q, int ld_q, const T* __restrict__ cache, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_seg, const int* __restrict__ block_table, int max_blocks, int H, int G, int n, int dv, int page,
    float scale, const int* __restrict__ bucket, int far, const float* __restrict__ bias, const float* __restrict__ gate, int ld_g,
    float factor) {
  extern __shared__ float qs_all[];              // 4 warps x n floats
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x * 4 + warp;
  const int t = blockIdx.y;
  if (h >= H) return;                            // whole warp leaves together
  float* qs = qs_all + (size_t)warp * n;
  const T* qrow = q + (size_t)t * ld_q + (size_t)h * n;
  for (int i = lane; i < n; i += 32) qs[i] = to_f(qrow[i]);
  __syncwarp();
  const int pos = tok_pos[t];
  const int* bt = block_table + (size_t)tok_seg[t] * max_blocks;
  const int g = h / (H / G);
  const size_t width = (size_t)G * (n + dv);
  const size_t k_off = (size_t)g * n, v_off = (size_t)G * n + (size_t)g * dv;

  constexpr int NREG = BA_MAX_DV / 32;
  float o[NREG];
#pragma unroll
  for (int j = 0; j < NREG; ++j) o[j] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int kb = 0; kb <= pos; kb += 32) {
    const int tk = kb + lane;
    const bool valid = tk <= pos;
    size_t base = 0;
    float s = -INFINITY;
    if (valid) {
      base = ((size_t)bt[tk / page] * page + (size_t)(tk % page)) * width;
      const T* kp = cache + base + k_off;
      float d = 0.f;
      for (int i = 0; i < n; ++i) d = fmaf(qs[i], to_f(kp[i]), d);
      const int dist = pos - tk < far ? pos - tk : far;
      s = fmaf(d, scale, bias ? bias[(size_t)bucket[dist] * H + h] : 0.f);
    }
    const float mn = fmaxf(m, warp_max(s));      // finite: the block holds a valid key
    const float p = valid ? expf(s - mn) : 0.f;
    const float c = expf(m - mn);
    l = l * c + warp_sum(p);
#pragma unroll
    for (int j = 0; j < NREG; ++j) o[j] *= c;
    const int nkeys = pos - kb + 1 < 32 ? pos - kb + 1 : 32;
    for (int j = 0; j < nkeys; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const size_t bj = __shfl_sync(0xffffffffu, (unsigned long long)base, j);
      if (pj == 0.f) continue;
      const T* vp = cache + bj + v_off;
#pragma unroll
      for (int r = 0; r < NREG; ++r) {
        const int i = lane + 32 * r;
        if (i < dv) o[r] = fmaf(pj, to_f(vp[i]), o[r]);
      }
    }
    m = mn;
  }
  const float inv = 1.0f / l;
  T* orow = out + (size_t)t * ld_out + (size_t)h * dv;
  const float* grow = gate ? gate + (size_t)t * ld_g + (size_t)h * dv : nullptr;
#pragma unroll
  for (int r = 0; r < NREG; ++r) {
    const int i = lane + 32 * r;
    if (i < dv) {
      float v = o[r] * inv;
      if (grow) v *= 1.0f / (1.0f + expf(-grow[i]));
      orow[i] = from_f<T>(v * factor);
    }
  }
}

// gate (float32 [T, H * dv], row stride ld_g, or null): the heads' outputs are multiplied by sigmoid(gate) and by `factor`.
extern "C" int qv_bias_attention_generic(void* out, int ld_out, const void* q, int ld_q, const void* cache, const int* tok_pos,
                                         const int* tok_seg, const int* block_table, int max_blocks, int T, int H, int G, int n, int dv,
                                         int page, float scale, const int* bucket, int far, const float* bias, const float* gate,
                                         int ld_g, float factor, int dt, void* stream) {
  if (T <= 0) return 0;
  if (dv > BA_MAX_DV || dv <= 0 || n <= 0 || G <= 0 || H % G || far < 0) return QV_ERR_UNSUPPORTED;
  const size_t smem = (size_t)4 * n * sizeof(float);
  if (smem > 48 * 1024) return QV_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t esz = dt == QV_DT_F32 ? 4 : 2;
  for (int done = 0; done < T; done += 65535) {            // rows are independent: several launches for very many tokens
    const int rows = T - done < 65535 ? T - done : 65535;
    dim3 grid((H + 3) / 4, rows);
    int rc = QV_ERR_UNSUPPORTED;
    QV_DISPATCH_DT(dt, TT,
                   rc = qv_launch(bias_attention_generic_kernel<TT>, grid, dim3(128), smem, st,
                                  (TT*)((char*)out + (size_t)done * ld_out * esz), ld_out, (const TT*)((const char*)q + (size_t)done * ld_q * esz),
                                  ld_q, (const TT*)cache, tok_pos + done, tok_seg + done, block_table, max_blocks, H, G, n, dv, page, scale,
                                  bucket, far, bias, gate ? gate + (size_t)done * ld_g : nullptr, ld_g, factor));
    if (rc) return rc;
  }
  return 0;
}
