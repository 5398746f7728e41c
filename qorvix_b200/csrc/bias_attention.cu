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
// qv_rot_norm_prepare       for attention without a bias table over the same cache rows: rotation of part of every head, unit
//                           norm of q and k, a temperature per head on q, values blended with another layer's.
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

// Queries and keys that are rotated and then unit-normed, values that may be blended with another layer's:
//   q, k heads: the first `rot` entries rotated in split halves (entry i with entry i + rot/2, angles of row tok_pos of cos_sin),
//   then, if `unit`, divided by the root mean square over the head (eps under the root); q also times head_temp[h] (or 1);
//   v = (1 - lam) v + lam v_first[t] where v_first is given (float32 [T, G * dv], row stride ld_vf).
// proj [T, ...] float32 with [q | k | v] at q_off, k_off, v_off; q -> q_out (compute type), k and v -> the token's cache row
// [G * n | G * dv].  All arithmetic float32.  One block per token, a warp per head in turn (staged in shared memory).
template <typename T>
__global__ void __launch_bounds__(256) rot_norm_prepare_kernel(T* __restrict__ q_out, int ld_qo, const float* __restrict__ proj, int ld_p,
                                                              int q_off, int k_off, int v_off, T* __restrict__ cache,
                                                              const float2* __restrict__ cos_sin, int table_rows, int rot, int unit,
                                                              float eps, const float* __restrict__ head_temp,
                                                              const float* __restrict__ v_first, int ld_vf, float lam,
                                                              const int* __restrict__ tok_pos, const int* __restrict__ tok_seg,
                                                              const int* __restrict__ block_table, int max_blocks, int H, int G, int n,
                                                              int dv, int page) {
  extern __shared__ float rn_smem[];               // 8 warps x n floats
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = tok_pos[t];
  const float* row = proj + (size_t)t * ld_p;
  const int half = rot >> 1;
  const float2* cs = rot ? cos_sin + (size_t)(pos < table_rows ? pos : table_rows - 1) * half : nullptr;
  const int nk = G * n, nv = G * dv;
  const int pg = block_table[(size_t)tok_seg[t] * max_blocks + pos / page];
  T* crow = cache + ((size_t)pg * page + (size_t)(pos % page)) * ((size_t)nk + nv);
  float* x = rn_smem + (size_t)warp * n;
  for (int hs = warp; hs < H + G; hs += 8) {
    const bool isq = hs < H;
    const float* src = isq ? row + q_off + (size_t)hs * n : row + k_off + (size_t)(hs - H) * n;
    for (int i = lane; i < n; i += 32) x[i] = src[i];
    __syncwarp();
    for (int i = lane; i < half; i += 32) {
      const float a = x[i], b = x[i + half];
      const float2 c = cs[i];
      x[i] = a * c.x - b * c.y;
      x[i + half] = b * c.x + a * c.y;
    }
    __syncwarp();
    float sc = 1.0f;
    if (unit) {
      float ss = 0.f;
      for (int i = lane; i < n; i += 32) ss = fmaf(x[i], x[i], ss);
      ss = warp_sum(ss);
      sc = 1.0f / sqrtf(ss / (float)n + eps);
    }
    if (isq) {
      const float temp = head_temp ? head_temp[hs] : 1.0f;
      T* dst = q_out + (size_t)t * ld_qo + (size_t)hs * n;
      for (int i = lane; i < n; i += 32) dst[i] = from_f<T>(x[i] * sc * temp);
    } else {
      T* dst = crow + (size_t)(hs - H) * n;
      for (int i = lane; i < n; i += 32) dst[i] = from_f<T>(x[i] * sc);
    }
    __syncwarp();
  }
  const float* vf = v_first ? v_first + (size_t)t * ld_vf : nullptr;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float v = row[v_off + i];
    if (vf) v = (1.0f - lam) * v + lam * vf[i];
    crow[nk + i] = from_f<T>(v);
  }
}

extern "C" int qv_rot_norm_prepare(void* q_out, int ld_qo, const float* proj, int ld_p, int q_off, int k_off, int v_off, void* cache,
                                   const float* cos_sin, int table_rows, int rot, int unit, float eps, const float* head_temp,
                                   const float* v_first, int ld_vf, float lam, const int* tok_pos, const int* tok_seg,
                                   const int* block_table, int max_blocks, int T, int H, int G, int n, int dv, int page, int dt,
                                   void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || n <= 0 || dv <= 0 || rot < 0 || rot > n || (rot & 1) || (rot && cos_sin == nullptr)) return QV_ERR_UNSUPPORTED;
  const size_t smem = (size_t)8 * n * sizeof(float);
  if (smem > 48 * 1024) return QV_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t esz = dt == QV_DT_F32 ? 4 : 2;
  for (int done = 0; done < T; done += 65535) {
    const int rows = T - done < 65535 ? T - done : 65535;
    int rc = QV_ERR_UNSUPPORTED;
    QV_DISPATCH_DT(dt, TT,
                   rc = qv_launch(rot_norm_prepare_kernel<TT>, dim3(rows), dim3(256), smem, st,
                                  (TT*)((char*)q_out + (size_t)done * ld_qo * esz), ld_qo, proj + (size_t)done * ld_p, ld_p, q_off, k_off,
                                  v_off, (TT*)cache, (const float2*)cos_sin, table_rows, rot, unit, eps, head_temp,
                                  v_first ? v_first + (size_t)done * ld_vf : nullptr, ld_vf, lam, tok_pos + done, tok_seg + done,
                                  block_table, max_blocks, H, G, n, dv, page));
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

// ---------------------------------------------------------------- tensor cores (bfloat16)
// qv_bias_attention_mma   mma.sync m16n8k16 (bfloat16 in, float32 sums), keys and values in blocks of 32 through two
//                         stages of cp.async, fragments by ldmatrix, online softmax in float32 (base 2: the scale and
//                         the table of biases carry log2 e).  The bias comes from a table per head over the distance
//                         (dist_bias [H, far + 1], the bucket rule already applied by the host).  The softmax weights
//                         enter the product with the values as three bfloat16 terms that together hold their 24 bits,
//                         so the weights stay 32-bit.
//   portions       a CTA of four warps owns 64 consecutive tokens of one head (16 rows a warp); a block of keys needs
//                  a strip of 95 consecutive distances of the head's table, which rides in the stage.
//   single tokens  a CTA of one warp owns the (up to 16) query heads that share a key/value head, and one slice of
//                  `slice_keys` keys (slices are aligned to absolute positions; how many there are follows from the longest
//                  context the step may hold, and those past a token's position leave at once); with more than one slice a
//                  step, bias_attention_merge_kernel joins a token's slices in ascending order.
// Key and value sizes: multiples of 8, padded with zeros to NP and DP (64 or 128).
#define BT_KEYS 32

struct BiasMmaArgs {
  bf16* out; int ld_out;
  const bf16* q; int ld_q;
  const bf16* cache;
  const int* seg_q_start; const int* seg_pos0; const int* block_table; int max_blocks;
  int H, G, n, dv, page;
  float scale_log2;
  const float* dist_bias; int far;                 // [H, far + 1], times log2 e
  const float* gate; int ld_g; float factor;
  float* partial; int slices; int slice_keys;      // single tokens: [S, H, slices, 2 + dv] (m, l, o); unused with one slice
};

__device__ __forceinline__ void bt_ldmatrix4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void bt_ldmatrix4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void bt_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16 bytes, or 16 zero bytes where `valid` is false (src must still be an address that may be formed)
__device__ __forceinline__ void bt_cp16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bt_cp4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t bt_pack(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&h;
}
// the three bfloat16 terms of two float32 weights (a pair is rounded by one instruction; its halves are floats again by a shift and a mask)
__device__ __forceinline__ void bt_split3(float x, float y, uint32_t& t0, uint32_t& t1, uint32_t& t2) {
  t0 = bt_pack(x, y);
  const float xr = x - __uint_as_float(t0 << 16), yr = y - __uint_as_float(t0 & 0xffff0000u);
  t1 = bt_pack(xr, yr);
  t2 = bt_pack(xr - __uint_as_float(t1 << 16), yr - __uint_as_float(t1 & 0xffff0000u));
}

static inline size_t bt_smem_bytes(int NP, int DP, int warps) {
  return (size_t)(16 * warps * (NP + 8) + 2 * BT_KEYS * ((NP + 8) + (DP + 8))) * sizeof(bf16) + 2 * 96 * sizeof(float);
}

template <int NP, int DP, int WARPS, bool SINGLE>
__global__ void __launch_bounds__(32 * WARPS) bias_attention_mma_kernel(BiasMmaArgs a) {
  extern __shared__ __align__(16) unsigned char bt_smem[];
  constexpr int ROWS = 16 * WARPS, NT = 32 * WARPS;
  constexpr int KS = NP + 8, VS = DP + 8;                 // row strides (elements): an odd number of 16-byte units
  constexpr int KC = NP / 8, VC = DP / 8;                 // 16-byte chunks a row
  bf16* sQ = (bf16*)bt_smem;                              // [ROWS][KS]
  bf16* sK = sQ + ROWS * KS;                              // [2][32][KS]
  bf16* sV = sK + 2 * BT_KEYS * KS;                       // [2][32][VS]
  float* sB = (float*)(sV + 2 * BT_KEYS * VS);            // [2][96]: the strip of the head's table (portions)
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g8 = lane >> 2, tg = lane & 3;
  const int H = a.H, G = a.G, n = a.n, dv = a.dv, page = a.page, gs = H / G, far = a.far;
  const int s = blockIdx.z;
  const int q0 = a.seg_q_start[s];
  const int pos0 = a.seg_pos0[s];
  const int* bt = a.block_table + (size_t)s * a.max_blocks;
  int h, kvh, i0, rows_valid, k_lo, k_hi;                 // keys k_lo .. k_hi - 1; rows of the tile that exist
  if (SINGLE) {
    kvh = blockIdx.y; h = kvh * gs; i0 = pos0; rows_valid = gs;
    k_lo = blockIdx.x * a.slice_keys;
    k_hi = a.slices > 1 ? min(k_lo + a.slice_keys, pos0 + 1) : pos0 + 1;
  } else {
    h = blockIdx.y; kvh = h / gs;
    const int rb = gridDim.x - 1 - blockIdx.x;            // the longest tiles first
    const int len = a.seg_q_start[s + 1] - q0;
    if (rb * ROWS >= len) return;
    i0 = pos0 + rb * ROWS;
    rows_valid = min(ROWS, len - rb * ROWS);
    k_lo = 0; k_hi = i0 + rows_valid;
  }
  const int r_lo = warp * 16 + g8, r_hi = r_lo + 8;       // this thread's two rows of the tile
  const bool ok_lo = r_lo < rows_valid, ok_hi = r_hi < rows_valid;
  if (SINGLE && k_lo >= k_hi) return;                     // a slice past the token: the merge does not read it
  const size_t width = (size_t)G * (n + dv);
  const size_t k_col = (size_t)kvh * n, v_col = (size_t)G * n + (size_t)kvh * dv;

  // queries: the tile's rows, zeros beyond the rows that exist and beyond the key size
  for (int idx = tid; idx < ROWS * KC; idx += NT) {
    const int r = idx / KC, c = idx % KC;
    const bool valid = r < rows_valid && c * 8 < n;
    const bf16* src = a.q;
    if (valid) src = SINGLE ? a.q + (size_t)q0 * a.ld_q + (size_t)(h + r) * n + c * 8
                            : a.q + (size_t)(q0 + (i0 - pos0) + r) * a.ld_q + (size_t)h * n + c * 8;
    bt_cp16(sQ + r * KS + c * 8, src, valid);
  }
  auto load = [&](int stage, int j0) {
    bf16* dK = sK + stage * BT_KEYS * KS;
    bf16* dV = sV + stage * BT_KEYS * VS;
    // lane r of every warp works out where key j0 + r lies (one division a block and lane); the pieces of 16 bytes ask for it
    const int jr = j0 + lane;
    unsigned long long row_at = 0;
    if (jr < k_hi) row_at = ((unsigned long long)bt[jr / page] * page + (unsigned long long)(jr % page)) * width;
    for (int idx = tid; idx < BT_KEYS * (KC + VC); idx += NT) {       // the same number of rounds for every lane: (KC + VC) % 4 == 0
      const int r = idx / (KC + VC), c = idx % (KC + VC);
      const unsigned long long at = __shfl_sync(0xffffffffu, row_at, r);
      const bool isk = c < KC;
      const int cc = isk ? c : c - KC;
      const bool valid = j0 + r < k_hi && cc * 8 < (isk ? n : dv);
      const bf16* src = valid ? a.cache + at + (isk ? k_col : v_col) + cc * 8 : a.cache;
      bt_cp16(isk ? dK + r * KS + cc * 8 : dV + r * VS + cc * 8, src, valid);
    }
    if (!SINGLE) {
      const int d0 = i0 - j0 - (BT_KEYS - 1);             // strip[x] = table[clamp(d0 + x)], x = row - key + 31
      for (int x = tid; x < 96; x += NT) {
        const int d = min(max(d0 + x, 0), far);
        bt_cp4(sB + stage * 96 + x, a.dist_bias + (size_t)h * (far + 1) + d);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  const int pos_lo = SINGLE ? pos0 : min(i0 + r_lo, k_hi - 1);        // rows that do not exist look like the last one
  const int pos_hi = SINGLE ? pos0 : min(i0 + r_hi, k_hi - 1);
  const int warp_last = SINGLE ? pos0 : min(i0 + warp * 16 + 15, k_hi - 1);
  const int head_lo = h + (SINGLE ? min(r_lo, gs - 1) : 0), head_hi = h + (SINGLE ? min(r_hi, gs - 1) : 0);
  const float* tab_lo = a.dist_bias + (size_t)head_lo * (far + 1);
  const float* tab_hi = a.dist_bias + (size_t)head_hi * (far + 1);
  const int mat = lane >> 3, r8 = lane & 7;

  uint32_t qf[NP / 16][4];
  float o[DP / 8][4];
#pragma unroll
  for (int i = 0; i < DP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  const int nkb = (k_hi - k_lo + BT_KEYS - 1) / BT_KEYS;
  load(0, k_lo);
  for (int kb = 0; kb < nkb; ++kb) {
    const int stage = kb & 1, j0 = k_lo + kb * BT_KEYS;
    if (kb + 1 < nkb) {
      load(stage ^ 1, j0 + BT_KEYS);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    if (kb == 0) {
#pragma unroll
      for (int kk = 0; kk < NP / 16; ++kk)
        bt_ldmatrix4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], sQ + (warp * 16 + (mat & 1) * 8 + r8) * KS + kk * 16 + (mat >> 1) * 8);
    }
    if (j0 <= warp_last) {
      const bf16* tK = sK + stage * BT_KEYS * KS;
      const bf16* tV = sV + stage * BT_KEYS * VS;
      float sc[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < NP / 16; ++kk) {
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          uint32_t b0, b1, b2, b3;
          bt_ldmatrix4(b0, b1, b2, b3, tK + (nb * 16 + (mat >> 1) * 8 + r8) * KS + kk * 16 + (mat & 1) * 8);
          bt_mma(sc[2 * nb], qf[kk], b0, b1);
          bt_mma(sc[2 * nb + 1], qf[kk], b2, b3);
        }
      }
      // scores in base 2 with the bias of the distance; keys behind a row's position drop out
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = nt * 8 + 2 * tg + (e & 1), j = j0 + col;
          const bool hi = e >= 2;
          const int pos = hi ? pos_hi : pos_lo;
          float v = -INFINITY;
          if (j <= pos) {
            float b;
            if (SINGLE) b = __ldg((hi ? tab_hi : tab_lo) + min(pos - j, far));
            else b = sB[stage * 96 + (hi ? r_hi : r_lo) - col + (BT_KEYS - 1)];
            v = fmaf(sc[nt][e], a.scale_log2, b);
          }
          sc[nt][e] = v;
          if (hi) mx_hi = fmaxf(mx_hi, v); else mx_lo = fmaxf(mx_lo, v);
        }
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);     // finite: a row's first block holds a key it sees
      const float c_lo = exp2f(m_lo - mn_lo), c_hi = exp2f(m_hi - mn_hi);
      m_lo = mn_lo; m_hi = mn_hi;
      float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        sc[nt][0] = exp2f(sc[nt][0] - mn_lo); sc[nt][1] = exp2f(sc[nt][1] - mn_lo);
        sc[nt][2] = exp2f(sc[nt][2] - mn_hi); sc[nt][3] = exp2f(sc[nt][3] - mn_hi);
        sum_lo += sc[nt][0] + sc[nt][1];
        sum_hi += sc[nt][2] + sc[nt][3];
      }
      l_lo = l_lo * c_lo + sum_lo;                         // a thread's share of the row's sum; joined at the end
      l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
      for (int i = 0; i < DP / 8; ++i) { o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi; }
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        uint32_t t[3][4];
        bt_split3(sc[2 * kk][0], sc[2 * kk][1], t[0][0], t[1][0], t[2][0]);
        bt_split3(sc[2 * kk][2], sc[2 * kk][3], t[0][1], t[1][1], t[2][1]);
        bt_split3(sc[2 * kk + 1][0], sc[2 * kk + 1][1], t[0][2], t[1][2], t[2][2]);
        bt_split3(sc[2 * kk + 1][2], sc[2 * kk + 1][3], t[0][3], t[1][3], t[2][3]);
#pragma unroll
        for (int np = 0; np < DP / 16; np += 2) {          // four accumulators in turn: no product waits for the one before it
          uint32_t b[8];
          bt_ldmatrix4_trans(b[0], b[1], b[2], b[3], tV + (kk * 16 + (mat & 1) * 8 + r8) * VS + (np * 2 + (mat >> 1)) * 8);
          bt_ldmatrix4_trans(b[4], b[5], b[6], b[7], tV + (kk * 16 + (mat & 1) * 8 + r8) * VS + (np * 2 + 2 + (mat >> 1)) * 8);
#pragma unroll
          for (int term = 2; term >= 0; --term) {          // the small terms first
            bt_mma(o[2 * np], t[term], b[0], b[1]);
            bt_mma(o[2 * np + 1], t[term], b[2], b[3]);
            bt_mma(o[2 * np + 2], t[term], b[4], b[5]);
            bt_mma(o[2 * np + 3], t[term], b[6], b[7]);
          }
        }
      }
    }
    __syncthreads();
  }
  pdl_launch_dependents();                                // not earlier: the next kernel's waiting CTAs would share the SMs with the tiles
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

  if (SINGLE && a.slices > 1) {                            // the slice's maximum, sum and unnormalised values
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (!(half ? ok_hi : ok_lo)) continue;
      float* p = a.partial + (((size_t)s * H + h + (half ? r_hi : r_lo)) * a.slices + blockIdx.x) * (2 + dv);
      if (tg == 0) { p[0] = half ? m_hi : m_lo; p[1] = half ? l_hi : l_lo; }
#pragma unroll
      for (int i = 0; i < DP / 8; ++i) {
        const int col = i * 8 + 2 * tg;
        if (col < dv) { p[2 + col] = o[i][2 * half]; p[2 + col + 1] = o[i][2 * half + 1]; }
      }
    }
    return;
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    if (!(half ? ok_hi : ok_lo)) continue;
    const int r = half ? r_hi : r_lo;
    const size_t t = SINGLE ? (size_t)q0 : (size_t)(q0 + (i0 - pos0) + r);
    const int head = SINGLE ? h + r : h;
    const float inv = 1.0f / (half ? l_hi : l_lo);
    bf16* orow = a.out + t * a.ld_out + (size_t)head * dv;
    const float* grow = a.gate ? a.gate + t * a.ld_g + (size_t)head * dv : nullptr;
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) {
      const int col = i * 8 + 2 * tg;
      if (col < dv) {
        float v0 = o[i][2 * half] * inv, v1 = o[i][2 * half + 1] * inv;
        if (grow) { v0 *= 1.0f / (1.0f + expf(-grow[col])); v1 *= 1.0f / (1.0f + expf(-grow[col + 1])); }
        *(uint32_t*)(orow + col) = bt_pack(v0 * a.factor, v1 * a.factor);
      }
    }
  }
}

// joins a token's slices (ascending), then gate and factor.  One warp per (token, head): the lanes share out the slices for the
// maximum, the sum and the slices' weights, and the columns for the values, whose loads for several slices are in flight together
// (read one slice after the other, a (token, head) waited for some fifty loads in a row).  dv <= 128.
__global__ void __launch_bounds__(128) bias_attention_merge_kernel(bf16* __restrict__ out, int ld_out, const float* __restrict__ partial,
                                                                  const int* __restrict__ seg_q_start, const int* __restrict__ seg_pos0,
                                                                  int H, int dv, int all_slices, int slice_keys,
                                                                  const float* __restrict__ gate, int ld_g, float factor) {
  pdl_wait();
  pdl_launch_dependents();
  const int s = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= H) return;
  const int stride = 2 + dv;
  const float* p = partial + ((size_t)s * H + h) * all_slices * stride;
  const int slices = min(all_slices, seg_pos0[s] / slice_keys + 1);       // the slices that hold keys of this token
  float M = -INFINITY, L = 0.f;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (slices <= 32) {                            // a lane a slice: maximum and sum are read once, the values' loads do not wait for them
    const float mi = lane < slices ? p[(size_t)lane * stride] : -INFINITY;
    const float li = lane < slices ? p[(size_t)lane * stride + 1] : 0.f;
    M = warp_max(mi);
    const float wi = exp2f(mi - M);
    L = warp_sum(li * wi);
#pragma unroll 8
    for (int j = 0; j < slices; ++j) {
      const float wj = __shfl_sync(0xffffffffu, wi, j);
      const float* ps = p + (size_t)j * stride + 2;
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int c = lane + 32 * r;
        if (c < dv) acc[r] = fmaf(ps[c], wj, acc[r]);
      }
    }
  } else {
    for (int i = lane; i < slices; i += 32) M = fmaxf(M, p[(size_t)i * stride]);
    M = warp_max(M);
    for (int i = lane; i < slices; i += 32) L += p[(size_t)i * stride + 1] * exp2f(p[(size_t)i * stride] - M);
    L = warp_sum(L);
    for (int base = 0; base < slices; base += 32) {
      const float wi = base + lane < slices ? exp2f(p[(size_t)(base + lane) * stride] - M) : 0.f;
      const int cnt = min(32, slices - base);
#pragma unroll 4
      for (int j = 0; j < cnt; ++j) {
        const float wj = __shfl_sync(0xffffffffu, wi, j);
        const float* ps = p + (size_t)(base + j) * stride + 2;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int c = lane + 32 * r;
          if (c < dv) acc[r] = fmaf(ps[c], wj, acc[r]);
        }
      }
    }
  }
  const size_t t = (size_t)seg_q_start[s];
  const float inv = 1.0f / L;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int c = lane + 32 * r;
    if (c < dv) {
      float v = acc[r] * inv;
      if (gate) v *= 1.0f / (1.0f + expf(-gate[t * ld_g + (size_t)h * dv + c]));
      out[t * ld_out + (size_t)h * dv + c] = __float2bfloat16_rn(v * factor);
    }
  }
}

// S segments starting at rows seg_q_start[s] and positions seg_pos0[s].  max_q_len == 1: single tokens (H / G <= 16), their keys
// in `slices` slices of slice_keys (a multiple of 32) with `partial` [S, H, slices, 2 + dv] when slices > 1.
// dist_bias [H, far + 1] float32 holds bias * log2 e per distance.  QV_ERR_UNSUPPORTED for sizes it does not take.
extern "C" int qv_bias_attention_mma(void* out, int ld_out, const void* q, int ld_q, const void* cache, const int* seg_q_start,
                                     const int* seg_pos0, const int* block_table, int max_blocks, int S, int max_q_len, int H, int G, int n,
                                     int dv, int page, float scale, const float* dist_bias, int far, const float* gate, int ld_g,
                                     float factor, float* partial, int slices, int slice_keys, void* stream) {
  if (S <= 0) return 0;
  if (n <= 0 || dv <= 0 || n % 8 || dv % 8 || n > 128 || dv > 128 || G <= 0 || H % G || far < 0 || ld_q % 8 || ld_out % 2) return QV_ERR_UNSUPPORTED;
  const bool single = max_q_len == 1;
  if (single && H / G > 16) return QV_ERR_UNSUPPORTED;
  if (single && slices > 1 && (partial == nullptr || slice_keys <= 0 || slice_keys % BT_KEYS)) return QV_ERR_UNSUPPORTED;
  if (!single) slices = 1;
  if (S > 65535 || H > 65535) return QV_ERR_TOO_LARGE;
  BiasMmaArgs a;
  a.out = (bf16*)out; a.ld_out = ld_out; a.q = (const bf16*)q; a.ld_q = ld_q; a.cache = (const bf16*)cache; a.seg_q_start = seg_q_start;
  a.seg_pos0 = seg_pos0; a.block_table = block_table; a.max_blocks = max_blocks; a.H = H; a.G = G; a.n = n; a.dv = dv; a.page = page;
  a.scale_log2 = scale * 1.4426950408889634f; a.dist_bias = dist_bias; a.far = far; a.gate = gate; a.ld_g = ld_g; a.factor = factor;
  a.partial = partial; a.slices = slices < 1 ? 1 : slices; a.slice_keys = slice_keys;
  cudaStream_t st = (cudaStream_t)stream;
  const int NP = n <= 64 ? 64 : 128, DP = dv <= 64 ? 64 : 128;
  int rc = QV_ERR_UNSUPPORTED;
#define BT_LAUNCH(NP_, DP_)                                                                                                      \
  do {                                                                                                                           \
    if (single) {                                                                                                                \
      const size_t smem = bt_smem_bytes(NP_, DP_, 1);                                                                            \
      cudaFuncSetAttribute(bias_attention_mma_kernel<NP_, DP_, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      rc = qv_launch(bias_attention_mma_kernel<NP_, DP_, 1, true>, dim3(a.slices, G, S), dim3(32), smem, st, a);                 \
    } else {                                                                                                                     \
      const size_t smem = bt_smem_bytes(NP_, DP_, 4);                                                                            \
      cudaFuncSetAttribute(bias_attention_mma_kernel<NP_, DP_, 4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      rc = qv_launch(bias_attention_mma_kernel<NP_, DP_, 4, false>, dim3((max_q_len + 63) / 64, H, S), dim3(128), smem, st, a);   \
    }                                                                                                                            \
  } while (0)
  if (NP == 64 && DP == 64) BT_LAUNCH(64, 64);
  else if (NP == 64) BT_LAUNCH(64, 128);
  else if (DP == 64) BT_LAUNCH(128, 64);
  else BT_LAUNCH(128, 128);
#undef BT_LAUNCH
  if (rc) return rc;
  if (single && a.slices > 1)
    rc = qv_launch(bias_attention_merge_kernel, dim3(S, (H + 3) / 4), dim3(128), 0, st, (bf16*)out, ld_out, (const float*)partial, seg_q_start,
                   seg_pos0, H, dv, a.slices, slice_keys, gate, ld_g, factor);
  return rc;
}
