// Attention over a paged cache of low-rank latents (one row per token: the normed latent c of `rank`
// entries followed by one rotated key part of `dr` entries that all heads share).
//
// Per head h the unrotated key of token j is Wuk_h c_j and its value Wuv_h c_j.  Neither is ever formed:
//   score(t, j) = (q_plain . Wuk_h c_j + q_rot . kr_j) * scale = ((Wuk_h^T q_plain) . c_j + q_rot . kr_j) * scale
//   out(t)      = Wuv_h (sum_j p_j c_j)
// so a query is first carried into the latent space (rank entries), attention then runs as if all heads
// shared one key/value head whose key row is [c | kr] and whose value row is c, and the head's value
// matrix is applied to the weighted latent afterwards.  A sigmoid gate multiplies the output.
//
// qv_latent_prepare: per token, RMS norm of the latent part of the down projection, rotation of the shared
//   key part (neighbouring pairs or split halves), write of both into the token's cache row; rotation of
//   every head's query part in place.
// qv_latent_attention_generic: one warp per (token, head), float32 arithmetic whatever the storage type,
//   keys in blocks of 32 aligned to absolute positions with a running maximum and sum, so a position's
//   result depends on the position and the cache only.  Serves the true 32-bit path and every size.
#include "common.cuh"

// proj[t] = [... down: rank + dr at kv_off ...], row stride ld; q[t] = H * (dn + dr) entries, row stride ld_q (the queries may
// be columns of proj or a tensor of their own).  Rotation of the first `rot` entries of a rotated part by the angles of row
// tok_pos of cos_sin: split_half 0 pairs entries (2i, 2i+1), 1 pairs entries (i, i + rot/2).
template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(
    T* __restrict__ proj, int ld, T* __restrict__ q, int ld_q, int kv_off, T* __restrict__ cache, const float* __restrict__ norm_w,
    float eps, const float2* __restrict__ cos_sin, int table_rows, const int* __restrict__ tok_pos, const int* __restrict__ tok_seg,
    const int* __restrict__ block_table, int max_blocks, int H, int dn, int dr, int rank, int rot, int page, int split_half) {
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  T* row = proj + (size_t)t * ld;
  const float2* cs = cos_sin + (size_t)(pos < table_rows ? pos : table_rows - 1) * (rot >> 1);
  const int pg = block_table[(size_t)tok_seg[t] * max_blocks + pos / page];
  T* dst = cache + ((size_t)pg * page + (size_t)(pos % page)) * (rank + dr);
  // the latent: x * rsqrt(mean(x^2) + eps) * w
  const T* lat = row + kv_off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = to_f(lat[i]); ss += v * v; }
  const float total = block_sum(ss, red);
  const float sc = 1.0f / sqrtf(total / (float)rank + eps);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f<T>(to_f(lat[i]) * sc * norm_w[i]);
  // the shared rotated key part
  const int pairs = rot >> 1;
  const T* kr = lat + rank;
  for (int i = threadIdx.x; i < dr; i += blockDim.x) {
    float v = to_f(kr[i]);
    if (i < rot) {
      if (split_half) {
        const bool first = i < pairs;
        const float2 c = cs[first ? i : i - pairs];
        const float other = to_f(kr[first ? i + pairs : i - pairs]);
        v = first ? v * c.x - other * c.y : v * c.x + other * c.y;
      } else {
        const float2 c = cs[i >> 1];
        const float other = to_f(kr[i ^ 1]);
        v = (i & 1) ? v * c.x + other * c.y : v * c.x - other * c.y;
      }
    }
    dst[rank + i] = from_f<T>(v);
  }
  // every head's rotated query part, in place (a pair is handled by one thread)
  const int step = split_half ? pairs : 1;
  for (int k = threadIdx.x; k < H * pairs; k += blockDim.x) {
    const int h = k / pairs, i = k - h * pairs;
    T* qr = q + (size_t)t * ld_q + (size_t)h * (dn + dr) + dn + (split_half ? i : 2 * i);
    const float a = to_f(qr[0]), b = to_f(qr[step]);
    const float2 c = cs[i];
    qr[0] = from_f<T>(a * c.x - b * c.y);
    qr[step] = from_f<T>(b * c.x + a * c.y);
  }
}

extern "C" int qv_latent_prepare(void* proj, int ld, void* q, int ld_q, int kv_off, void* cache, const float* norm_w, float eps,
                                 const float* cos_sin, int table_rows, const int* tok_pos, const int* tok_seg,
                                 const int* block_table, int max_blocks, int T, int H, int dn, int dr, int rank, int rot,
                                 int page, int split_half, int dt, void* stream) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > dr || (rot & 1) || rank <= 0) return QV_ERR_UNSUPPORTED;
  QV_DISPATCH_DT(dt, TT,
                 return qv_launch(latent_prepare_kernel<TT>, dim3(T), dim3(256), 0, (cudaStream_t)stream, (TT*)proj, ld, (TT*)q, ld_q,
                                  kv_off, (TT*)cache, norm_w, eps, (const float2*)cos_sin, table_rows, tok_pos, tok_seg, block_table,
                                  max_blocks, H, dn, dr, rank, rot, page, split_half));
  return QV_ERR_UNSUPPORTED;
}

#define LAT_MAX_RANK 1024

// q: rows of [dn unrotated | dr rotated] per head at q (row stride ld_q); wuk [H * dn, rank]; wuv [H * dv, rank];
// gate (may be null) and out: [T, H * dv] with their row strides.
template <typename T, typename TW>
__global__ void __launch_bounds__(128) latent_attention_generic_kernel(
    T* __restrict__ out, int ld_out, const T* __restrict__ q, int ld_q, const T* __restrict__ gate, int ld_gate,
    const T* __restrict__ cache, const TW* __restrict__ wuk, const TW* __restrict__ wuv, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_seg, const int* __restrict__ block_table, int max_blocks, int H, int dn, int dr, int dv,
    int rank, int page, int window, float scale) {
  extern __shared__ float sm_all[];              // 4 warps x (rank + dr + dn) floats
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x * 4 + warp;
  const int t = blockIdx.y;
  if (h >= H) return;
  const int kw = rank + dr;
  float* qs = sm_all + (size_t)warp * (kw + dn);   // [rank latent query | dr rotated query]
  float* qp = qs + kw;                             // dn unrotated query entries
  const T* qrow = q + (size_t)t * ld_q + (size_t)h * (dn + dr);
  for (int i = lane; i < dn; i += 32) qp[i] = to_f(qrow[i]);
  for (int i = lane; i < dr; i += 32) qs[rank + i] = to_f(qrow[dn + i]);
  __syncwarp();
  // the query in the latent space: qs[r] = sum_i q_plain[i] * wuk[h * dn + i][r]
  for (int r = lane; r < rank; r += 32) {
    float acc = 0.f;
    for (int i = 0; i < dn; ++i) acc = fmaf(qp[i], to_f(wuk[((size_t)h * dn + i) * rank + r]), acc);
    qs[r] = acc;
  }
  __syncwarp();

  const int pos = tok_pos[t];
  const int* bt = block_table + (size_t)tok_seg[t] * max_blocks;
  const int lo = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;
  constexpr int NREG = LAT_MAX_RANK / 32;
  float o[NREG];
#pragma unroll
  for (int j = 0; j < NREG; ++j) o[j] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int kb = (lo >> 5) << 5; kb <= pos; kb += 32) {
    const int tk = kb + lane;
    const bool valid = tk >= lo && tk <= pos;
    size_t base = 0;
    float s = -INFINITY;
    if (valid) {
      base = ((size_t)bt[tk / page] * page + (size_t)(tk % page)) * kw;
      const T* kp = cache + base;
      float dot = 0.f;
      for (int i = 0; i < kw; ++i) dot = fmaf(qs[i], to_f(kp[i]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int j = 0; j < NREG; ++j) o[j] *= corr;
    const int nk = pos - kb + 1 < 32 ? pos - kb + 1 : 32;
    for (int j = 0; j < nk; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const size_t bj = __shfl_sync(0xffffffffu, (unsigned long long)base, j);
      if (pj == 0.f) continue;
      const T* vp = cache + bj;
#pragma unroll
      for (int r = 0; r < NREG; ++r) {
        const int i = lane + 32 * r;
        if (i < rank) o[r] = fmaf(pj, to_f(vp[i]), o[r]);
      }
    }
    m = m_new;
  }
  // the weighted latent, then the head's value matrix and the gate
  __syncwarp();
  const float inv = 1.0f / l;
#pragma unroll
  for (int r = 0; r < NREG; ++r) {
    const int i = lane + 32 * r;
    if (i < rank) qs[i] = o[r] * inv;
  }
  __syncwarp();
  T* orow = out + (size_t)t * ld_out + (size_t)h * dv;
  const T* grow = gate ? gate + (size_t)t * ld_gate + (size_t)h * dv : nullptr;
  for (int j = 0; j < dv; ++j) {
    const TW* wr = wuv + ((size_t)h * dv + j) * rank;
    float acc = 0.f;
    for (int r = lane; r < rank; r += 32) acc = fmaf(to_f(wr[r]), qs[r], acc);
    acc = warp_sum(acc);
    if (lane == 0) {
      if (grow) acc *= 1.0f / (1.0f + expf(-to_f(grow[j])));
      orow[j] = from_f<T>(acc);
    }
  }
}

extern "C" int qv_latent_attention_generic(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate,
                                           const void* cache, const void* wuk, const void* wuv, const int* tok_pos,
                                           const int* tok_seg, const int* block_table, int max_blocks, int T, int H, int dn,
                                           int dr, int dv, int rank, int page, int window, float scale, int dt, int w_dt,
                                           void* stream) {
  if (T <= 0) return 0;
  if (rank > LAT_MAX_RANK || rank <= 0 || dn < 0 || dr < 0 || dv <= 0) return QV_ERR_UNSUPPORTED;
  const size_t smem = (size_t)4 * (rank + dr + dn) * sizeof(float);
  if (smem > 200 * 1024) return QV_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  int done = 0;
  while (done < T) {                               // rows are independent; the grid's second dimension is limited
    const int n = T - done < 65535 ? T - done : 65535;
    const size_t esz = dt == QV_DT_F32 ? 4 : 2;
    void* o = (char*)out + (size_t)done * ld_out * esz;
    const void* qq = (const char*)q + (size_t)done * ld_q * esz;
    const void* gg = gate ? (const char*)gate + (size_t)done * ld_gate * esz : nullptr;
    dim3 grid((H + 3) / 4, n);
    int rc;
#define LAT_GENERIC(TT, TW)                                                                                              \
  do {                                                                                                                   \
    if (smem > 48 * 1024)                                                                                                \
      cudaFuncSetAttribute(latent_attention_generic_kernel<TT, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    rc = qv_launch(latent_attention_generic_kernel<TT, TW>, grid, dim3(128), smem, st, (TT*)o, ld_out, (const TT*)qq, ld_q, \
                   (const TT*)gg, ld_gate, (const TT*)cache, (const TW*)wuk, (const TW*)wuv, tok_pos + done, tok_seg + done, \
                   block_table, max_blocks, H, dn, dr, dv, rank, page, window, scale);                                   \
  } while (0)
    if (dt == QV_DT_F32 && w_dt == QV_DT_F32) LAT_GENERIC(float, float);
    else if (dt == QV_DT_BF16 && w_dt == QV_DT_BF16) LAT_GENERIC(bf16, bf16);
    else if (dt == QV_DT_BF16 && w_dt == QV_DT_F32) LAT_GENERIC(bf16, float);
    else if (dt == QV_DT_F32 && w_dt == QV_DT_BF16) LAT_GENERIC(float, bf16);
    else return QV_ERR_UNSUPPORTED;
#undef LAT_GENERIC
    if (rc) return rc;
    done += n;
  }
  return 0;
}

// ---------------------------------------------------------------- tensor-core path (bfloat16)
// Three launches: (1) qv_latent_absorb carries every (token, head) query into the latent space, giving rows
// [Wuk_h^T q_plain | q_rot] of rank + dr entries; (2) latent_attention_tc_kernel runs attention with all heads
// sharing the cache rows as keys ([c | kr]) and as values (c): a CTA of eight warps takes 32 consecutive
// (token, head) rows of one segment and walks its keys in blocks of 64 staged by cp.async in two buffers;
// Q.K^T and P.V are mma.sync m16n8k16 with float32 accumulators, the softmax is float32 with a running
// maximum; the keys of a tile may be split over several CTAs, each leaving an unnormalised partial result;
// (3) qv_latent_expand merges the partial results, applies the head's value matrix and the gate.
#define LT_BM 32
#define LT_BK 64
#define LT_WARPS 8

__device__ __forceinline__ void lt_cp16(void* smem, const void* gmem, int bytes) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void lt_ldsm4(uint32_t* r, const void* p) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void lt_ldsm2(uint32_t* r, const void* p) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(s));
}
__device__ __forceinline__ void lt_ldsm2t(uint32_t* r, const void* p) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(s));
}
__device__ __forceinline__ void lt_mma(float* c, const uint32_t* a, const uint32_t* b) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Per-head products on the tensor cores: for head e, out[t, e*out_off + n] = f(sum_k a[t, e*a_off + k] * w[e][n][k]),
// t < R, n < N; tiles of 64 tokens x 64 columns, k in steps of 32 through a two-stage cp.async ring, four warps of
// 32 x 32 (mma.sync m16n8k16, float32 accumulators).  GATED: f multiplies by sigmoid(gate[t, e*gate_off + n]).
// tail > 0: the `tail` entries that follow a head's K inputs are copied behind its N outputs (the rotated query part
// rides along with the query's move into the latent space).  K a multiple of 8, rows of a on 16 bytes.
#define HG_LD 40
template <bool GATED>
__global__ void __launch_bounds__(128) heads_gemm_kernel(bf16* __restrict__ out, int ld_out, int out_off, const bf16* __restrict__ a, int ld_a,
                                                         int a_off, const bf16* __restrict__ w, const bf16* __restrict__ gate, int ld_gate,
                                                         int gate_off, int R, int N, int K, int tail) {
  __shared__ __align__(16) bf16 As[2][64][HG_LD];
  __shared__ __align__(16) bf16 Bs[2][64][HG_LD];
  pdl_wait();
  pdl_launch_dependents();
  const int e = blockIdx.z, row0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int rows = min(64, R - row0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, wm = warp >> 1, wn = warp & 1;
  const bf16* A = a + (size_t)e * a_off;
  const bf16* W = w + (size_t)e * N * K;
  if (tail > 0 && blockIdx.x == 0)
    for (int c = tid; c < rows * tail; c += 128) {
      const int r = c / tail, i = c - r * tail;
      out[(size_t)(row0 + r) * ld_out + (size_t)e * out_off + N + i] = A[(size_t)(row0 + r) * ld_a + K + i];
    }
  auto stage = [&](int buf, int k0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = tid + i * 128, r = c >> 2, k = k0 + (c & 3) * 8;
      const bool kin = k < K, aok = r < rows && kin, bok = n0 + r < N && kin;
      lt_cp16(&As[buf][r][(c & 3) * 8], A + (aok ? (size_t)(row0 + r) * ld_a + k : 0), aok ? 16 : 0);
      lt_cp16(&Bs[buf][r][(c & 3) * 8], W + (bok ? (size_t)(n0 + r) * K + k : 0), bok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float acc[2][4][4] = {};
  const int nk = (K + 31) / 32;
  stage(0, 0);
  for (int kt = 0; kt < nk; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < nk) {
      stage(buf ^ 1, (kt + 1) * 32);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      uint32_t af[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) lt_ldsm4(af[mt], &As[buf][wm * 32 + mt * 16 + (lane & 15)][ks * 16 + (lane >> 4) * 8]);
#pragma unroll
      for (int pr = 0; pr < 2; ++pr) {
        uint32_t b[4];
        lt_ldsm4(b, &Bs[buf][wn * 32 + pr * 16 + (lane >> 4) * 8 + (lane & 7)][ks * 16 + ((lane >> 3) & 1) * 8]);
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          lt_mma(acc[mt][pr * 2], af[mt], b);
          lt_mma(acc[mt][pr * 2 + 1], af[mt], b + 2);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * 32 + mt * 16 + (lane >> 2) + half * 8;
      if (r >= rows) continue;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int n = n0 + wn * 32 + nt * 8 + 2 * (lane & 3) + j;
          if (n >= N) continue;
          float v = acc[mt][nt][half * 2 + j];
          if (GATED) v *= 1.0f / (1.0f + expf(-to_f(gate[(size_t)(row0 + r) * ld_gate + (size_t)e * gate_off + n])));
          out[(size_t)(row0 + r) * ld_out + (size_t)e * out_off + n] = __float2bfloat16_rn(v);
        }
    }
}

template <int NTW>
__global__ void __launch_bounds__(LT_WARPS * 32) latent_attention_tc_kernel(
    float* __restrict__ part_o, float* __restrict__ part_ml, const bf16* __restrict__ qlat, const bf16* __restrict__ cache,
    const int* __restrict__ seg_q_start, const int* __restrict__ seg_pos0, const int* __restrict__ block_table, int max_blocks,
    int H, int dr, int page, int window, float scale, int splits, int total_rows) {
  constexpr int RANK = NTW * 64;
  extern __shared__ __align__(16) unsigned char lt_smem[];
  const int kw = RANK + dr, ldk = kw + 8;
  bf16* Qs = (bf16*)lt_smem;                               // [32][ldk]
  bf16* Ks = Qs + (size_t)LT_BM * ldk;                     // [2][64][ldk]
  bf16* Ps = Ks + (size_t)2 * LT_BK * ldk;                 // [32][72]
  float* st_max = (float*)(Ps + LT_BM * (LT_BK + 8));      // [8][32]
  float* st_sum = st_max + LT_WARPS * LT_BM;               // [8][32]
  pdl_wait();
  pdl_launch_dependents();
  const int s = blockIdx.y, split = blockIdx.z;
  const int q0 = seg_q_start[s], q1 = seg_q_start[s + 1];
  const int row_first = q0 * H + blockIdx.x * LT_BM;       // global (token, head) row of this tile's first row
  const int rows = min(LT_BM, q1 * H - row_first);
  if (rows <= 0) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pos0 = seg_pos0[s];
  const int pos_first = pos0 + row_first / H - q0, pos_last = pos0 + (row_first + rows - 1) / H - q0;
  const int lo_tile = window > 0 ? max(0, pos_first - window + 1) : 0;
  const int b_first = lo_tile / LT_BK, nb_all = pos_last / LT_BK - b_first + 1;
  const int b_lo = b_first + (int)((long long)nb_all * split / splits), b_hi = b_first + (int)((long long)nb_all * (split + 1) / splits);
  const int* bt = block_table + (size_t)s * max_blocks;
  const int pieces = kw / 8;                               // 16-byte pieces of a row

  // a warp copies whole rows (one page lookup a row, the row's 16-byte pieces dealt to the lanes)
  auto load_keys = [&](int buf, int blk) {
    bf16* dst = Ks + (size_t)buf * LT_BK * ldk;
    for (int r = warp; r < LT_BK; r += LT_WARPS) {
      const int key = blk * LT_BK + r;
      const bool ok = key <= pos_last;
      const bf16* src = cache + (ok ? ((size_t)bt[key / page] * page + (size_t)(key % page)) * kw : 0);
      for (int p = lane; p < pieces; p += 32) lt_cp16(dst + (size_t)r * ldk + p * 8, src + (ok ? p * 8 : 0), ok ? 16 : 0);
    }
  };
  for (int r = warp; r < LT_BM; r += LT_WARPS) {
    const bool ok = r < rows;
    const bf16* src = qlat + (ok ? (size_t)(row_first + r) * kw : 0);
    for (int p = lane; p < pieces; p += 32) lt_cp16(Qs + (size_t)r * ldk + p * 8, src + (ok ? p * 8 : 0), ok ? 16 : 0);
  }
  if (b_lo < b_hi) load_keys(0, b_lo);
  asm volatile("cp.async.commit_group;" ::: "memory");

  // this thread's four rows (m-tile mt, half hf): tile row mt*16 + hf*8 + lane/4, with position and window start
  int rpos[2][2], rlo[2][2];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int r = mt * 16 + hf * 8 + (lane >> 2);
      rpos[mt][hf] = r < rows ? pos0 + (row_first + r) / H - q0 : -1;
      rlo[mt][hf] = window > 0 ? max(0, rpos[mt][hf] - window + 1) : 0;
    }
  float m_run[2][2], l_run[2][2], o[2][NTW][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) { m_run[mt][hf] = -INFINITY; l_run[mt][hf] = 0.f; }
#pragma unroll
    for (int nt = 0; nt < NTW; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[mt][nt][e] = 0.f;
  }

  for (int blk = b_lo; blk < b_hi; ++blk) {
    const int buf = (blk - b_lo) & 1;
    if (blk + 1 < b_hi) {
      load_keys(buf ^ 1, blk + 1);
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const bf16* Kb = Ks + (size_t)buf * LT_BK * ldk;
    // scores of this warp's eight keys for all 32 rows
    float sc[2][4] = {}, sd[2][4] = {};                      // two chains of dependent products instead of one
    const int nks = kw / 16;
    for (int ks = 0; ks < nks; ks += 2) {
      uint32_t a[2][4], b[2];
      lt_ldsm4(a[0], Qs + (size_t)(lane & 15) * ldk + ks * 16 + (lane >> 4) * 8);
      lt_ldsm4(a[1], Qs + (size_t)(16 + (lane & 15)) * ldk + ks * 16 + (lane >> 4) * 8);
      lt_ldsm2(b, Kb + (size_t)(warp * 8 + (lane & 7)) * ldk + ks * 16 + ((lane >> 3) & 1) * 8);
      lt_mma(sc[0], a[0], b);
      lt_mma(sc[1], a[1], b);
      if (ks + 1 < nks) {
        uint32_t c[2][4], e[2];
        lt_ldsm4(c[0], Qs + (size_t)(lane & 15) * ldk + (ks + 1) * 16 + (lane >> 4) * 8);
        lt_ldsm4(c[1], Qs + (size_t)(16 + (lane & 15)) * ldk + (ks + 1) * 16 + (lane >> 4) * 8);
        lt_ldsm2(e, Kb + (size_t)(warp * 8 + (lane & 7)) * ldk + (ks + 1) * 16 + ((lane >> 3) & 1) * 8);
        lt_mma(sd[0], c[0], e);
        lt_mma(sd[1], c[1], e);
      }
    }
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int x = 0; x < 4; ++x) sc[mt][x] += sd[mt][x];
    const int key0 = blk * LT_BK + warp * 8 + 2 * (lane & 3);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int key = key0 + j;
          float v = sc[mt][hf * 2 + j] * scale;
          if (key > rpos[mt][hf] || key < rlo[mt][hf]) v = -INFINITY;
          sc[mt][hf * 2 + j] = v;
          mx = fmaxf(mx, v);
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        if ((lane & 3) == 0) st_max[warp * LT_BM + mt * 16 + hf * 8 + (lane >> 2)] = mx;
      }
    __syncthreads();
    float corr[2][2];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int r = mt * 16 + hf * 8 + (lane >> 2);
        float bm = st_max[r];
#pragma unroll
        for (int w = 1; w < LT_WARPS; ++w) bm = fmaxf(bm, st_max[w * LT_BM + r]);
        const float m_new = fmaxf(m_run[mt][hf], bm);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        corr[mt][hf] = expf(m_run[mt][hf] - m_use);
        m_run[mt][hf] = m_new;
        const float p0 = expf(sc[mt][hf * 2] - m_use), p1 = expf(sc[mt][hf * 2 + 1] - m_use);
        *(__nv_bfloat162*)(Ps + (size_t)r * (LT_BK + 8) + warp * 8 + 2 * (lane & 3)) = __floats2bfloat162_rn(p0, p1);
        float sum = p0 + p1;
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((lane & 3) == 0) st_sum[warp * LT_BM + r] = sum;
      }
    __syncthreads();
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int r = mt * 16 + hf * 8 + (lane >> 2);
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < LT_WARPS; ++w) sum += st_sum[w * LT_BM + r];
        l_run[mt][hf] = l_run[mt][hf] * corr[mt][hf] + sum;
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) { o[mt][nt][hf * 2] *= corr[mt][hf]; o[mt][nt][hf * 2 + 1] *= corr[mt][hf]; }
      }
    // weighted latents: this warp's NTW * 8 columns
#pragma unroll
    for (int kk = 0; kk < LT_BK / 16; ++kk) {
      uint32_t a[2][4];
      lt_ldsm4(a[0], Ps + (size_t)(lane & 15) * (LT_BK + 8) + kk * 16 + (lane >> 4) * 8);
      lt_ldsm4(a[1], Ps + (size_t)(16 + (lane & 15)) * (LT_BK + 8) + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int nt = 0; nt < NTW; ++nt) {
        uint32_t b[2];
        lt_ldsm2t(b, Kb + (size_t)(kk * 16 + (lane & 15)) * ldk + (warp * NTW + nt) * 8);
        lt_mma(o[0][nt], a[0], b);
        lt_mma(o[1][nt], a[1], b);
      }
    }
    __syncthreads();
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int r = mt * 16 + hf * 8 + (lane >> 2);
      if (r >= rows) continue;
      const size_t prow = (size_t)split * total_rows + row_first + r;
      if (warp == 0 && (lane & 3) == 0) { part_ml[2 * prow] = m_run[mt][hf]; part_ml[2 * prow + 1] = l_run[mt][hf]; }
#pragma unroll
      for (int nt = 0; nt < NTW; ++nt)
        *(float2*)(part_o + prow * RANK + (warp * NTW + nt) * 8 + 2 * (lane & 3)) = make_float2(o[mt][nt][hf * 2], o[mt][nt][hf * 2 + 1]);
    }
}

// lat[row][:] (bfloat16) = the partial results of a (token, head) row merged: sum_s e^(m_s - M) o_s / sum_s e^(m_s - M) l_s
__global__ void __launch_bounds__(128) latent_merge_kernel(bf16* __restrict__ lat, const float* __restrict__ part_o,
                                                           const float* __restrict__ part_ml, int rank, int splits, int total_rows) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t row = blockIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[2 * ((size_t)s * total_rows + row)]);
  float L = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float m = part_ml[2 * ((size_t)s * total_rows + row)];
    if (m != -INFINITY) L += expf(m - M) * part_ml[2 * ((size_t)s * total_rows + row) + 1];
  }
  const float inv = 1.0f / L;
  for (int r = threadIdx.x * 2; r < rank; r += blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float m = part_ml[2 * ((size_t)s * total_rows + row)];
      if (m == -INFINITY) continue;
      const float w = expf(m - M);
      const float2 v = *(const float2*)(part_o + ((size_t)s * total_rows + row) * rank + r);
      a0 = fmaf(w, v.x, a0);
      a1 = fmaf(w, v.y, a1);
    }
    *(__nv_bfloat162*)(lat + row * rank + r) = __floats2bfloat162_rn(a0 * inv, a1 * inv);
  }
}

extern "C" long long qv_latent_tc_workspace_bytes(int T, int H, int dr, int rank, int splits) {
  const long long rows = (long long)T * H;
  return rows * (rank + dr) * 2 + (long long)splits * rows * rank * 4 + (long long)splits * rows * 2 * 4 + rows * rank * 2 + 64;
}

// bfloat16 operands; rank a multiple of 64 up to 512 (not 320 or 448), dr a multiple of 16, dn a multiple of 8.
// wuk_t: the heads' key matrices transposed, [H][rank][dn].  workspace: what qv_latent_tc_workspace_bytes says,
// 16-byte aligned.  Refuses other sizes (the caller then takes the generic kernel).
extern "C" int qv_latent_attention_tc(void* out, int ld_out, const void* q, int ld_q, const void* gate, int ld_gate, const void* cache,
                                      const void* wuk_t, const void* wuv, const int* seg_q_start, const int* seg_pos0,
                                      const int* block_table, int max_blocks, int T, int S, int max_q_len, int H, int dn, int dr,
                                      int dv, int rank, int page, int window, float scale, int splits, void* workspace, void* stream) {
  if (T <= 0) return 0;
  if (rank % 64 || rank > 512 || dr % 16 || dr < 0 || dn % 8 || dn <= 0 || ld_q % 8 || splits < 1 || S > 65535 || splits > 65535 || H > 65535)
    return QV_ERR_UNSUPPORTED;
  if ((T + 63) / 64 > 65535) return QV_ERR_TOO_LARGE;
  const int ntw = rank / 64;
  if (ntw == 5 || ntw == 7) return QV_ERR_UNSUPPORTED;
  const int kw = rank + dr, ldk = kw + 8;
  const size_t smem = ((size_t)LT_BM * ldk + (size_t)2 * LT_BK * ldk + (size_t)LT_BM * (LT_BK + 8)) * 2 + (size_t)2 * LT_WARPS * LT_BM * 4;
  if (smem > 220 * 1024) return QV_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  const long long rows = (long long)T * H;
  bf16* qlat = (bf16*)workspace;
  float* part_o = (float*)((char*)workspace + ((rows * kw * 2 + 15) / 16) * 16);
  float* part_ml = part_o + (size_t)splits * rows * rank;
  bf16* lat = (bf16*)(part_ml + (((size_t)splits * rows * 2 + 3) / 4) * 4);
  // the queries' move into the latent space: per head q_plain [T, dn] x Wuk_h [dn, rank], the rotated part copied behind
  int rc = qv_launch(heads_gemm_kernel<false>, dim3((rank + 63) / 64, (T + 63) / 64, H), dim3(128), 0, st, qlat, H * kw, kw,
                     (const bf16*)q, ld_q, dn + dr, (const bf16*)wuk_t, (const bf16*)nullptr, 0, 0, T, rank, dn, dr);
  if (rc) return rc;
  dim3 grid(((size_t)max_q_len * H + LT_BM - 1) / LT_BM, S, splits);
#define LT_LAUNCH(N)                                                                                                        \
  case N:                                                                                                                   \
    cudaFuncSetAttribute(latent_attention_tc_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
    rc = qv_launch(latent_attention_tc_kernel<N>, grid, dim3(LT_WARPS * 32), smem, st, part_o, part_ml, (const bf16*)qlat,  \
                   (const bf16*)cache, seg_q_start, seg_pos0, block_table, max_blocks, H, dr, page, window, scale, splits,  \
                   (int)rows);                                                                                              \
    break;
  switch (ntw) {
    LT_LAUNCH(1) LT_LAUNCH(2) LT_LAUNCH(3) LT_LAUNCH(4) LT_LAUNCH(6) LT_LAUNCH(8)
    default: return QV_ERR_UNSUPPORTED;
  }
#undef LT_LAUNCH
  if (rc) return rc;
  rc = qv_launch(latent_merge_kernel, dim3((unsigned)rows), dim3(128), 0, st, lat, (const float*)part_o, (const float*)part_ml, rank,
                 splits, (int)rows);
  if (rc) return rc;
  // the heads' value matrices and the gate: per head latent [T, rank] x Wuv_h^T [rank, dv]
  if (gate)
    return qv_launch(heads_gemm_kernel<true>, dim3((dv + 63) / 64, (T + 63) / 64, H), dim3(128), 0, st, (bf16*)out, ld_out, dv,
                     (const bf16*)lat, H * rank, rank, (const bf16*)wuv, (const bf16*)gate, ld_gate, dv, T, dv, rank, 0);
  return qv_launch(heads_gemm_kernel<false>, dim3((dv + 63) / 64, (T + 63) / 64, H), dim3(128), 0, st, (bf16*)out, ld_out, dv,
                   (const bf16*)lat, H * rank, rank, (const bf16*)wuv, (const bf16*)nullptr, 0, 0, T, dv, rank, 0);
}
