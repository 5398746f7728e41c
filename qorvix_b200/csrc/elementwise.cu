// Memory-bound kernels of the step: embedding gather, (residual add +) RMSNorm (+ row
// gather), rotary encoding fused with the paged key/value write, SwiGLU, casts.
// Formulas follow the reference's CPU ops (runtime/src/ops.cpp:8-13 rmsnorm, :96-100 swiglu,
// :127-148 split-half rope) and its CUDA twins (cuda/src/cuda_backend.cu:231-340), rebuilt
// for batches of tokens, a float32 residual stream and a paged cache.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] as float32 (the residual stream is float32).
template <typename TW>
__global__ void embed_kernel(float* __restrict__ out, const TW* __restrict__ table,
                             const int* __restrict__ ids, int d, int vocab) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;   // ids are validated on the host; never read out of bounds
  const TW* row = table + (size_t)id * d;
  float* o = out + (size_t)t * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f(row[i]);
}

extern "C" int qv_embed(float* out, const void* table, const int* ids, int T, int d, int vocab,
                        int table_dt, void* stream) {
  if (T <= 0) return 0;
  QV_DISPATCH_DT(table_dt, TW,
                 return qv_launch(embed_kernel<TW>, dim3(T), dim3(256), 0, (cudaStream_t)stream, out, (const TW*)table, ids, d, vocab));
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- add + rmsnorm (+ gather)
// row r reads source row s = row_idx ? row_idx[r] : r.
//   x = residual[s] + (delta ? delta[s] : 0)        (float32 sum)
//   if write_residual: residual[s] = x              (only without row_idx)
//   out[r] = (x * rsqrt(mean(x^2) + eps)) * w
// One block per row; the row is staged in shared memory so it is read once.
template <typename TD> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *(const float4*)p; }
};
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ float4 load(const bf16* p) {
    const uint2 v = *(const uint2*)p;
    const __nv_bfloat162 a = *(const __nv_bfloat162*)&v.x, b = *(const __nv_bfloat162*)&v.y;
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
};
__device__ __forceinline__ void store4(float* p, float4 v) { *(float4*)p = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u; u.x = *(uint32_t*)&a; u.y = *(uint32_t*)&b;
  *(uint2*)p = u;
}

// VEC: rows are read four elements at a time, all loads of a thread issued before any is used
// (d a multiple of 4, at most 4 * 4 * blockDim elements); else one element at a time.
template <typename TD, typename TO, bool VEC>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(TO* __restrict__ out, float* __restrict__ residual,
                                   const TD* __restrict__ delta, const float* __restrict__ w,
                                   const int* __restrict__ row_idx, int d, float eps,
                                   int write_residual) {
  extern __shared__ float smem[];
  pdl_wait();
  pdl_launch_dependents();
  float* xs = smem;            // d floats
  float* red = VEC ? smem : smem + d;       // 33 floats
  const int r = blockIdx.x;
  const int s = row_idx ? row_idx[r] : r;
  float* res = residual + (size_t)s * d;
  const TD* dl = delta ? delta + (size_t)s * d : nullptr;
  TO* o = out + (size_t)r * d;
  float ss = 0.f;
  if constexpr (VEC) {
    constexpr int MAXV = 4;
    float4 x[MAXV];
    const int nvec = d >> 2;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = threadIdx.x + k * 256;
      x[k] = i < nvec ? *(const float4*)(res + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (dl) {
#pragma unroll
      for (int k = 0; k < MAXV; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < nvec) {
          const float4 dv = Vec4<TD>::load(dl + 4 * i);
          x[k].x += dv.x; x[k].y += dv.y; x[k].z += dv.z; x[k].w += dv.w;
        }
      }
    }
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < nvec) {
        if (write_residual) *(float4*)(res + 4 * i) = x[k];
        ss += x[k].x * x[k].x + x[k].y * x[k].y + x[k].z * x[k].z + x[k].w * x[k].w;
      }
    }
    const float total = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(total / (float)d + eps);
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < nvec) {
        const float4 wv = *(const float4*)(w + 4 * i);
        store4(o + 4 * i, make_float4(x[k].x * scale * wv.x, x[k].y * scale * wv.y, x[k].z * scale * wv.z, x[k].w * scale * wv.w));
      }
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      float x = res[i];
      if (dl) x += to_f(dl[i]);
      xs[i] = x;
      if (write_residual) res[i] = x;
      ss += x * x;
    }
    const float total = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(total / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_f<TO>(xs[i] * scale * w[i]);
  }
}

extern "C" int qv_add_rmsnorm(void* out, float* residual, const void* delta, const float* w,
                              const int* row_idx, int rows, int d, float eps, int write_residual,
                              int delta_dt, int out_dt, void* stream) {
  if (rows <= 0) return 0;
  const size_t smem = (size_t)(d + 33) * sizeof(float);
  if (smem > 200 * 1024) return QV_ERR_TOO_LARGE;
  if (row_idx && write_residual) return QV_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  int rc = 0;
  // the vector path keeps the row in registers: d a multiple of 4, at most 4096 elements, rows 16-byte aligned
  const bool vec = (d % 4 == 0) && d <= 4 * 4 * 256 && (((uintptr_t)out | (uintptr_t)residual | (uintptr_t)delta | (uintptr_t)w) & 15) == 0;
#define LAUNCH_NORM(TD, TO)                                                                          \
  do {                                                                                               \
    if (vec) {                                                                                       \
      rc = qv_launch(add_rmsnorm_kernel<TD, TO, true>, dim3(rows), dim3(256), 48 * sizeof(float), st, \
          (TO*)out, residual, (const TD*)delta, w, row_idx, d, eps, write_residual);                 \
    } else {                                                                                         \
      if (smem > 48 * 1024)                                                                          \
        cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO, false>,                                      \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                \
      rc = qv_launch(add_rmsnorm_kernel<TD, TO, false>, dim3(rows), dim3(256), smem, st, (TO*)out, residual, \
                                                 (const TD*)delta, w, row_idx, d, eps, write_residual); \
    }                                                                                                \
  } while (0)
  if (delta_dt == QV_DT_F32 && out_dt == QV_DT_F32) LAUNCH_NORM(float, float);
  else if (delta_dt == QV_DT_BF16 && out_dt == QV_DT_BF16) LAUNCH_NORM(bf16, bf16);
  else if (delta_dt == QV_DT_F32 && out_dt == QV_DT_BF16) LAUNCH_NORM(float, bf16);
  else if (delta_dt == QV_DT_BF16 && out_dt == QV_DT_F32) LAUNCH_NORM(bf16, float);
  else return QV_ERR_UNSUPPORTED;
#undef LAUNCH_NORM
  return rc;
}

// ---------------------------------------------------------------- rotary + paged KV write
// qkv[t] = [q: H*hd | k: Hkv*hd | v: Hkv*hd] in the compute dtype (row stride `ld`).
// For token t at position p (table row p holds cos/sin of p*inv_freq[i], i < rot/2):
//   q heads and k heads: pairs (i, i + rot/2) of the first `rot` dims are rotated
//   (split-half), the other dims pass through.  q is rewritten in place; the rotated k and
//   the plain v go to the cache slot of (request, position):
//   page = block_table[seg, p / page], cache[page][0|1][kv head][p % page][:]
// If `cache` is null only q and k are rotated in place (k is then written back to qkv).
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int ld, T* __restrict__ cache,
                                     const float2* __restrict__ cos_sin, int table_rows,
                                     const int* __restrict__ tok_pos, const int* __restrict__ tok_seg,
                                     const int* __restrict__ block_table, int max_blocks, int H,
                                     int Hkv, int hd, int rot, int page) {
  // grid (token, groups of 8 head slots), one warp per slot: slots 0..H-1 are q heads,
  // H..H+Hkv-1 k heads, H+Hkv..H+2Hkv-1 v heads
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int head = blockIdx.y * 8 + (threadIdx.x >> 5);
  if (head >= H + 2 * Hkv) return;
  const int lane = threadIdx.x & 31;
  const int pos = tok_pos[t];
  T* row = qkv + (size_t)t * ld;
  const int half = rot >> 1;
  const float2* cs = cos_sin + (size_t)(pos < table_rows ? pos : table_rows - 1) * half;
  T* kdst = nullptr;
  T* vdst = nullptr;
  if (cache) {
    const int pg = block_table[(size_t)tok_seg[t] * max_blocks + pos / page];
    const size_t page_elems = (size_t)2 * Hkv * page * hd;
    kdst = cache + (size_t)pg * page_elems + (size_t)(pos % page) * hd;
    vdst = kdst + (size_t)Hkv * page * hd;
  }
  if (head < H + Hkv) {
    T* v = row + (size_t)head * hd;
    const bool to_cache = head >= H && cache;
    T* dst = to_cache ? kdst + (size_t)(head - H) * page * hd : v;
    if (sizeof(T) == 2 && (half & 1) == 0 && (((uintptr_t)v | (uintptr_t)dst) & 3) == 0) {
      // bfloat16: two neighbouring pairs per lane, 4-byte loads and stores
      for (int i = 2 * lane; i < half; i += 64) {
        const __nv_bfloat162 a2 = *(const __nv_bfloat162*)((const bf16*)v + i);
        const __nv_bfloat162 b2 = *(const __nv_bfloat162*)((const bf16*)v + i + half);
        const float2 c0 = cs[i], c1 = cs[i + 1];
        const float a0 = __low2float(a2), a1 = __high2float(a2), b0 = __low2float(b2), b1 = __high2float(b2);
        *(__nv_bfloat162*)((bf16*)dst + i) = __floats2bfloat162_rn(a0 * c0.x - b0 * c0.y, a1 * c1.x - b1 * c1.y);
        *(__nv_bfloat162*)((bf16*)dst + i + half) = __floats2bfloat162_rn(a0 * c0.y + b0 * c0.x, a1 * c1.y + b1 * c1.x);
      }
    } else {
      for (int i = lane; i < half; i += 32) {
        const float a = to_f(v[i]), b = to_f(v[i + half]);
        const float2 c = cs[i];
        dst[i] = from_f<T>(a * c.x - b * c.y);
        dst[i + half] = from_f<T>(a * c.y + b * c.x);
      }
    }
    if (to_cache)      // dims beyond the rotated ones pass through
      for (int i = rot + lane; i < hd; i += 32) dst[i] = v[i];
  } else if (cache) {
    const int vh = head - H - Hkv;
    const T* v = row + (size_t)head * hd;
    T* dst = vdst + (size_t)vh * page * hd;
    if (sizeof(T) == 2 && (hd & 7) == 0 && (((uintptr_t)v | (uintptr_t)dst) & 15) == 0) {
      for (int i = 8 * lane; i < hd; i += 256) *(uint4*)((bf16*)dst + i) = *(const uint4*)((const bf16*)v + i);
    } else {
      for (int i = lane; i < hd; i += 32) dst[i] = v[i];
    }
  }
}

extern "C" int qv_rope_kv_write(void* qkv, int ld, void* cache, const float* cos_sin, int table_rows,
                                const int* tok_pos, const int* tok_seg, const int* block_table,
                                int max_blocks, int T, int H, int Hkv, int hd, int rot, int page,
                                int dt, void* stream) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > hd || (rot & 1)) return QV_ERR_UNSUPPORTED;
  if ((H + 2 * Hkv + 7) / 8 > 65535) return QV_ERR_TOO_LARGE;
  QV_DISPATCH_DT(dt, TT,
                 return qv_launch(rope_kv_write_kernel<TT>, dim3(T, (H + 2 * Hkv + 7) / 8), dim3(256), 0, (cudaStream_t)stream,
                     (TT*)qkv, ld, (TT*)cache, (const float2*)cos_sin, table_rows, tok_pos, tok_seg,
                     block_table, max_blocks, H, Hkv, hd, rot, page));
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- swiglu
// out[t, i] = gate/(1+exp(-gate)) * up, with gu[t] (row stride 2f) either [gate: f | up: f] or, when
// `interleaved`, groups of 32 columns holding 16 gate values and then the 16 up values of the same
// features (the layout the fused tensor-core epilogue uses; f a multiple of 16).
template <typename T>
__global__ void swiglu_kernel(T* __restrict__ out, const T* __restrict__ gu, size_t n, int f, int interleaved) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / f;
    const int i = (int)(idx - t * f);
    const int gi = interleaved ? ((i >> 4) << 5) + (i & 15) : i;
    const int ui = interleaved ? gi + 16 : f + i;
    const float g = to_f(gu[t * 2 * f + gi]);
    const float u = to_f(gu[t * 2 * f + ui]);
    out[idx] = from_f<T>(g / (1.0f + expf(-g)) * u);
  }
}

extern "C" int qv_swiglu(void* out, const void* gu, int T, int f, int interleaved, int dt, void* stream) {
  const size_t n = (size_t)T * f;
  if (n == 0) return 0;
  if (interleaved && (f & 15)) return QV_ERR_UNSUPPORTED;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  QV_DISPATCH_DT(dt, TT, return qv_launch(swiglu_kernel<TT>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (TT*)out, (const TT*)gu, n, f, interleaved));
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- casts
template <typename TI, typename TO>
__global__ void cast_kernel(TO* __restrict__ out, const TI* __restrict__ in, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f<TO>(to_f(in[i]));
}

extern "C" int qv_cast(void* out, const void* in, long long n, int in_dt, int out_dt, void* stream) {
  if (n <= 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  cudaStream_t st = (cudaStream_t)stream;
  if (in_dt == QV_DT_F32 && out_dt == QV_DT_BF16) cast_kernel<float, bf16><<<blocks, 256, 0, st>>>((bf16*)out, (const float*)in, (size_t)n);
  else if (in_dt == QV_DT_BF16 && out_dt == QV_DT_F32) cast_kernel<bf16, float><<<blocks, 256, 0, st>>>((float*)out, (const bf16*)in, (size_t)n);
  else return QV_ERR_UNSUPPORTED;
  return qv_launch_status();
}

// out[r, c] = in[r, c] for matrices whose rows are contiguous but may lie any stride apart, with a
// change of type on the way if asked: what makes an aligned, dense copy of a column slice of a wider
// buffer, or of float32 rows for a kernel that takes bfloat16.
template <typename FROM, typename TO>
__global__ void cast_rows_kernel(TO* __restrict__ out, long long ld_out, const FROM* __restrict__ in, long long ld_in, int rows, int cols) {
  const size_t n = (size_t)rows * cols;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / cols, c = i - r * cols;
    out[r * ld_out + c] = from_f<TO>(to_f(in[r * ld_in + c]));
  }
}

extern "C" int qv_cast_rows(void* out, long long ld_out, const void* in, long long ld_in, int rows, int cols, int in_dt, int out_dt, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  const size_t n = (size_t)rows * cols;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  cudaStream_t st = (cudaStream_t)stream;
#define QV_CAST_ROWS(FROM, TO) cast_rows_kernel<FROM, TO><<<blocks, 256, 0, st>>>((TO*)out, ld_out, (const FROM*)in, ld_in, rows, cols)
  if (in_dt == QV_DT_F32 && out_dt == QV_DT_BF16) QV_CAST_ROWS(float, bf16);
  else if (in_dt == QV_DT_BF16 && out_dt == QV_DT_F32) QV_CAST_ROWS(bf16, float);
  else if (in_dt == QV_DT_F32 && out_dt == QV_DT_F32) QV_CAST_ROWS(float, float);
  else if (in_dt == QV_DT_BF16 && out_dt == QV_DT_BF16) QV_CAST_ROWS(bf16, bf16);
  else return QV_ERR_UNSUPPORTED;
#undef QV_CAST_ROWS
  return qv_launch_status();
}

// ---------------------------------------------------------------- embedding + hashed pair table
// out[t, :] = table[ids[t], :] + pair[row, :] as float32, where row hashes the token with the one before
// it in its request: (prev * mul_prev + id * mul_cur) mod buckets, and is `buckets` (the table's last row)
// for a request's first token.  The token before a segment's first one is kept per request in
// last_token[slot] (int32), which the block of a segment's first token reads and then sets to the
// segment's last token, so that portions cut anywhere see the same pairs.
template <typename TW>
__global__ void embed_pair_kernel(float* __restrict__ out, const TW* __restrict__ table, const TW* __restrict__ pair,
                                  const int* __restrict__ ids, const int* __restrict__ tok_pos, const int* __restrict__ tok_seg,
                                  const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot,
                                  int* __restrict__ last_token, int d, int vocab, int buckets, int mul_prev, int mul_cur) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const int s = tok_seg[t];
  const int first = seg_q_start[s];
  long long row = buckets;
  if (tok_pos[t] > 0) {
    int prev = t > first ? ids[t - 1] : last_token[seg_slot[s]];
    if (prev < 0 || prev >= vocab) prev = 0;
    row = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
    if (row < 0) row += buckets;            // the mathematical remainder, also for negative multipliers
  }
  __syncthreads();                          // every thread has read the kept token before it is replaced
  if (t == first && threadIdx.x == 0) last_token[seg_slot[s]] = ids[seg_q_start[s + 1] - 1];
  const TW* a = table + (size_t)id * d;
  const TW* b = pair + (size_t)row * d;
  float* o = out + (size_t)t * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f(a[i]) + to_f(b[i]);
}

extern "C" int qv_embed_pair(float* out, const void* table, const void* pair, const int* ids, const int* tok_pos,
                             const int* tok_seg, const int* seg_q_start, const int* seg_slot, int* last_token, int T, int d,
                             int vocab, int buckets, int mul_prev, int mul_cur, int table_dt, void* stream) {
  if (T <= 0) return 0;
  if (buckets <= 0) return QV_ERR_UNSUPPORTED;
  QV_DISPATCH_DT(table_dt, TW,
                 return qv_launch(embed_pair_kernel<TW>, dim3(T), dim3(256), 0, (cudaStream_t)stream, out, (const TW*)table,
                                  (const TW*)pair, ids, tok_pos, tok_seg, seg_q_start, seg_slot, last_token, d, vocab, buckets,
                                  mul_prev, mul_cur));
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- add + two rmsnorms of the same stream
// x = residual[r] (+ delta[r]), written back; out1[r] = x * rsqrt(mean(x^2) + eps) * w1, out2[r] likewise
// with w2: the two norms of a block whose mixer and feed-forward both read the stream as it enters.
template <typename TD, typename TO>
__global__ void __launch_bounds__(256) add_rmsnorm2_kernel(TO* __restrict__ out1, TO* __restrict__ out2, float* __restrict__ residual,
                                                           const TD* __restrict__ delta, const float* __restrict__ w1,
                                                           const float* __restrict__ w2, int d, float eps) {
  extern __shared__ float smem[];
  pdl_wait();
  pdl_launch_dependents();
  float* xs = smem;
  float* red = smem + d;
  const int r = blockIdx.x;
  float* res = residual + (size_t)r * d;
  const TD* dl = delta ? delta + (size_t)r * d : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float x = res[i];
    if (dl) { x += to_f(dl[i]); res[i] = x; }
    xs[i] = x;
    ss += x * x;
  }
  const float total = block_sum(ss, red);
  const float scale = 1.0f / sqrtf(total / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = xs[i] * scale;
    out1[(size_t)r * d + i] = from_f<TO>(v * w1[i]);
    if (out2) out2[(size_t)r * d + i] = from_f<TO>(v * w2[i]);
  }
}

extern "C" int qv_add_rmsnorm2(void* out1, void* out2, float* residual, const void* delta, const float* w1, const float* w2,
                               int rows, int d, float eps, int delta_dt, int out_dt, void* stream) {
  if (rows <= 0) return 0;
  const size_t smem = (size_t)(d + 33) * sizeof(float);
  if (smem > 200 * 1024) return QV_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
#define LAUNCH_NORM2(TD, TO)                                                                                     \
  do {                                                                                                           \
    if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm2_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    return qv_launch(add_rmsnorm2_kernel<TD, TO>, dim3(rows), dim3(256), smem, st, (TO*)out1, (TO*)out2, residual, \
                     (const TD*)delta, w1, w2, d, eps);                                                          \
  } while (0)
  if (delta_dt == QV_DT_F32 && out_dt == QV_DT_F32) LAUNCH_NORM2(float, float);
  else if (delta_dt == QV_DT_BF16 && out_dt == QV_DT_BF16) LAUNCH_NORM2(bf16, bf16);
  else if (delta_dt == QV_DT_F32 && out_dt == QV_DT_BF16) LAUNCH_NORM2(float, bf16);
  else if (delta_dt == QV_DT_BF16 && out_dt == QV_DT_F32) LAUNCH_NORM2(bf16, float);
#undef LAUNCH_NORM2
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- sum of two deltas, tanh cap
// out (float32) = a + b, each float32 or the compute type: what a block that runs two parts side by side
// hands on as one delta.
template <typename TA, typename TB>
__global__ void sum2_kernel(float* __restrict__ out, const TA* __restrict__ a, const TB* __restrict__ b, size_t n) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = to_f(a[i]) + to_f(b[i]);
}

extern "C" int qv_sum2(float* out, const void* a, const void* b, long long n, int a_dt, int b_dt, void* stream) {
  if (n <= 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  cudaStream_t st = (cudaStream_t)stream;
#define QV_SUM2(TA, TB) return qv_launch(sum2_kernel<TA, TB>, dim3(blocks), dim3(256), 0, st, out, (const TA*)a, (const TB*)b, (size_t)n)
  if (a_dt == QV_DT_F32 && b_dt == QV_DT_F32) QV_SUM2(float, float);
  if (a_dt == QV_DT_BF16 && b_dt == QV_DT_BF16) QV_SUM2(bf16, bf16);
  if (a_dt == QV_DT_F32 && b_dt == QV_DT_BF16) QV_SUM2(float, bf16);
  if (a_dt == QV_DT_BF16 && b_dt == QV_DT_F32) QV_SUM2(bf16, float);
#undef QV_SUM2
  return QV_ERR_UNSUPPORTED;
}

// x = cap * tanh(x / cap) in place, float32 (a soft limit on logits).
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] / cap);
}

extern "C" int qv_softcap(float* x, long long n, float cap, void* stream) {
  if (n <= 0) return 0;
  if (!(cap > 0.f)) return QV_ERR_UNSUPPORTED;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  return qv_launch(softcap_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, (size_t)n, cap);
}

// ---------------------------------------------------------------- scaled sum of two parts' outputs
// out[t, i] (float32) = a[t, i] * sa[i] + b[t, i] * sb[i]; sa, sb (float32 [d]) and b may be null (factor one, no
// second term): what a block that runs two parts side by side hands on when their outputs have per-feature factors.
template <typename TA, typename TB>
__global__ void scale_sum2_kernel(float* __restrict__ out, const TA* __restrict__ a, const float* __restrict__ sa,
                                  const TB* __restrict__ b, const float* __restrict__ sb, size_t n, int d) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % d);
    float v = to_f(a[i]) * (sa ? sa[c] : 1.f);
    if (b) v = fmaf(to_f(b[i]), sb ? sb[c] : 1.f, v);
    out[i] = v;
  }
}

extern "C" int qv_scale_sum2(float* out, const void* a, const float* sa, const void* b, const float* sb, int T, int d, int a_dt,
                             int b_dt, void* stream) {
  const size_t n = (size_t)T * d;
  if (n == 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  cudaStream_t st = (cudaStream_t)stream;
#define QV_SS2(TA, TB) return qv_launch(scale_sum2_kernel<TA, TB>, dim3(blocks), dim3(256), 0, st, out, (const TA*)a, sa, (const TB*)b, sb, n, d)
  if (a_dt == QV_DT_F32 && b_dt == QV_DT_F32) QV_SS2(float, float);
  if (a_dt == QV_DT_BF16 && b_dt == QV_DT_BF16) QV_SS2(bf16, bf16);
  if (a_dt == QV_DT_F32 && b_dt == QV_DT_BF16) QV_SS2(float, bf16);
  if (a_dt == QV_DT_BF16 && b_dt == QV_DT_F32) QV_SS2(bf16, float);
#undef QV_SS2
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- re-entry of the stream: [x + delta ; x0]
// out[t] = [residual[t] + delta[t] (float32 sum) | x0[t]] in the compute type, 2d wide: the input of the product
// that carries the stream and the embedding's output back into a stretch of layers that runs again.
template <typename TD, typename TO>
__global__ void stream_concat_kernel(TO* __restrict__ out, const float* __restrict__ residual, const TD* __restrict__ delta,
                                     const float* __restrict__ x0, size_t n, int d) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / d;
    const int c = (int)(i - t * d);
    out[t * 2 * d + c] = from_f<TO>(residual[i] + (delta ? to_f(delta[i]) : 0.f));
    out[t * 2 * d + d + c] = from_f<TO>(x0[i]);
  }
}

extern "C" int qv_stream_concat(void* out, const float* residual, const void* delta, const float* x0, int T, int d, int delta_dt,
                                int out_dt, void* stream) {
  const size_t n = (size_t)T * d;
  if (n == 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  cudaStream_t st = (cudaStream_t)stream;
#define QV_SC(TD, TO) return qv_launch(stream_concat_kernel<TD, TO>, dim3(blocks), dim3(256), 0, st, (TO*)out, residual, (const TD*)delta, x0, n, d)
  if (delta_dt == QV_DT_F32 && out_dt == QV_DT_F32) QV_SC(float, float);
  if (delta_dt == QV_DT_BF16 && out_dt == QV_DT_BF16) QV_SC(bf16, bf16);
  if (delta_dt == QV_DT_F32 && out_dt == QV_DT_BF16) QV_SC(float, bf16);
  if (delta_dt == QV_DT_BF16 && out_dt == QV_DT_F32) QV_SC(bf16, float);
#undef QV_SC
  return QV_ERR_UNSUPPORTED;
}

// x[t, :] += v[:] (float32), one vector for all rows.
__global__ void add_vector_kernel(float* __restrict__ x, const float* __restrict__ v, size_t n, int d) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] += v[i % d];
}

extern "C" int qv_add_vector(float* x, const float* v, int T, int d, void* stream) {
  const size_t n = (size_t)T * d;
  if (n == 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  return qv_launch(add_vector_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, v, n, d);
}

// ---------------------------------------------------------------- ungated activations
// out = act(x) elementwise in place or not; kind 0: the square of relu, 1: the tanh form of GELU.
template <typename T>
__global__ void activation_kernel(T* __restrict__ out, const T* __restrict__ x, size_t n, int kind) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float z = to_f(x[i]);
    float r;
    if (kind == 1) {
      r = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    } else {
      const float v = fmaxf(z, 0.f);
      r = v * v;
    }
    out[i] = from_f<T>(r);
  }
}

extern "C" int qv_activation(void* out, const void* x, long long n, int kind, int dt, void* stream) {
  if (n <= 0) return 0;
  if (kind != 0 && kind != 1) return QV_ERR_UNSUPPORTED;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  QV_DISPATCH_DT(dt, TT, return qv_launch(activation_kernel<TT>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (TT*)out, (const TT*)x, (size_t)n, kind));
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- norm without statistics (Dynamic Tanh)
// row r reads source row s = row_idx ? row_idx[r] : r.
//   x = residual[s] + (delta ? delta[s] : 0)        (float32 sum; written back unless row_idx is given)
//   out[r] = tanh(alpha * x) * w + b                (float32 arithmetic; no mean, no variance)
template <typename TD, typename TO>
__global__ void __launch_bounds__(256) add_tanhnorm_kernel(TO* __restrict__ out, float* __restrict__ residual, const TD* __restrict__ delta,
                                                          const float* __restrict__ w, const float* __restrict__ b, float alpha,
                                                          const int* __restrict__ row_idx, int d, int write_residual) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int s = row_idx ? row_idx[r] : r;
  float* res = residual + (size_t)s * d;
  const TD* dl = delta ? delta + (size_t)s * d : nullptr;
  TO* o = out + (size_t)r * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float x = res[i];
    if (dl) x += to_f(dl[i]);
    if (write_residual && dl) res[i] = x;
    o[i] = from_f<TO>(fmaf(tanhf(alpha * x), w[i], b ? b[i] : 0.f));
  }
}

extern "C" int qv_add_tanhnorm(void* out, float* residual, const void* delta, const float* w, const float* b, float alpha,
                               const int* row_idx, int rows, int d, int write_residual, int delta_dt, int out_dt, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
#define LAUNCH_TN(TD, TO)                                                                                                   \
  return qv_launch(add_tanhnorm_kernel<TD, TO>, dim3(rows), dim3(256), 0, st, (TO*)out, residual, (const TD*)delta, w, b, alpha, \
                   row_idx, d, write_residual)
  if (delta_dt == QV_DT_F32 && out_dt == QV_DT_F32) LAUNCH_TN(float, float);
  if (delta_dt == QV_DT_BF16 && out_dt == QV_DT_BF16) LAUNCH_TN(bf16, bf16);
  if (delta_dt == QV_DT_F32 && out_dt == QV_DT_BF16) LAUNCH_TN(float, bf16);
  if (delta_dt == QV_DT_BF16 && out_dt == QV_DT_F32) LAUNCH_TN(bf16, float);
#undef LAUNCH_TN
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- token row + learned position row (+ tanh norm)
// out[t] (float32) = table[ids[t]] + pos_scale * pos_table[tok_pos[t]], the sum in float32; with w also
// out = tanh(alpha * out) * w + b.  Ids and positions outside their tables are clamped.
template <typename TW>
__global__ void __launch_bounds__(256) embed_pos_kernel(float* __restrict__ out, const TW* __restrict__ table, const TW* __restrict__ pos_table,
                                                       const int* __restrict__ ids, const int* __restrict__ tok_pos, int d, int vocab,
                                                       int positions, float pos_scale, const float* __restrict__ w,
                                                       const float* __restrict__ b, float alpha) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t], p = tok_pos[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  p = p < 0 ? 0 : (p >= positions ? positions - 1 : p);
  const TW* e = table + (size_t)id * d;
  const TW* q = pos_table + (size_t)p * d;
  float* o = out + (size_t)t * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float x = fmaf(pos_scale, to_f(q[i]), to_f(e[i]));
    if (w) x = fmaf(tanhf(alpha * x), w[i], b ? b[i] : 0.f);
    o[i] = x;
  }
}

extern "C" int qv_embed_pos(float* out, const void* table, const void* pos_table, const int* ids, const int* tok_pos, int T, int d,
                            int vocab, int positions, float pos_scale, const float* w, const float* b, float alpha, int table_dt,
                            void* stream) {
  if (T <= 0) return 0;
  QV_DISPATCH_DT(table_dt, TW,
                 return qv_launch(embed_pos_kernel<TW>, dim3(T), dim3(256), 0, (cudaStream_t)stream, out, (const TW*)table,
                                  (const TW*)pos_table, ids, tok_pos, d, vocab, positions, pos_scale, w, b, alpha));
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- gated feed-forward activations
// out[t, i] = act(gate_i) * up_i; act 0: SiLU, 1: the tanh form of GELU.  gu is [gate | up], or with `interleaved` groups of
// 32 columns: 16 gate values, then the 16 up values of the same features.  Float32 arithmetic.
template <typename T>
__global__ void glu_act_kernel(T* __restrict__ out, const T* __restrict__ gu, size_t n, int f, int act, int interleaved) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / f;
    const int i = (int)(idx - t * f);
    const int gi = interleaved ? ((i >> 4) << 5) + (i & 15) : i;
    const int ui = interleaved ? gi + 16 : f + i;
    const float g = to_f(gu[t * 2 * f + gi]);
    const float u = to_f(gu[t * 2 * f + ui]);
    float a;
    if (act == 1) a = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    else a = g / (1.0f + expf(-g));
    out[idx] = from_f<T>(a * u);
  }
}

extern "C" int qv_glu_act(void* out, const void* gu, int T, int f, int act, int interleaved, int dt, void* stream) {
  const size_t n = (size_t)T * f;
  if (n == 0) return 0;
  if ((act != 0 && act != 1) || (interleaved && (f & 15))) return QV_ERR_UNSUPPORTED;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  QV_DISPATCH_DT(dt, TT, return qv_launch(glu_act_kernel<TT>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (TT*)out, (const TT*)gu, n, f, act, interleaved));
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- gate of a sublayer's result
// out[t, i] (float32) = y[t, i] * sigmoid(g[t, i] + bias[i]): y in float32 or the compute type (row stride ld_y), g
// float32 pre-activations (row stride ld_g, so a column slice of a wider product serves).
template <typename TY>
__global__ void sigmoid_gate_kernel(float* __restrict__ out, const TY* __restrict__ y, int ld_y, const float* __restrict__ g, int ld_g,
                                    const float* __restrict__ bias, size_t n, int d) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / d;
    const int i = (int)(idx - t * d);
    const float z = g[t * ld_g + i] + (bias ? bias[i] : 0.f);
    out[idx] = to_f(y[t * ld_y + i]) * (1.0f / (1.0f + expf(-z)));
  }
}

extern "C" int qv_sigmoid_gate(float* out, const void* y, int ld_y, const float* g, int ld_g, const float* bias, int T, int d, int y_dt,
                               void* stream) {
  const size_t n = (size_t)T * d;
  if (n == 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  QV_DISPATCH_DT(y_dt, TY, return qv_launch(sigmoid_gate_kernel<TY>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, out, (const TY*)y,
                                            ld_y, g, ld_g, bias, n, d));
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- weighted sum over the streams kept so far
// stack [slots][n] float32 keeps the embedding's output and every run's result.  The run's result, x + delta (delta may be null,
// float32), goes into slot `count - 1`; x then becomes sum over j < count of w[j] * stack[j][.], added up in the order of j.
__global__ void depth_mix_kernel(float* __restrict__ x, const float* __restrict__ delta, float* __restrict__ stack, size_t n,
                                 const float* __restrict__ w, int count) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float cur = x[i];
    if (delta) cur += delta[i];
    stack[(size_t)(count - 1) * n + i] = cur;
    float acc = 0.f;
    for (int j = 0; j + 1 < count; ++j) acc = fmaf(w[j], stack[(size_t)j * n + i], acc);
    x[i] = fmaf(w[count - 1], cur, acc);
  }
}

extern "C" int qv_depth_mix(float* x, const float* delta, float* stack, long long n, const float* w, int count, void* stream) {
  if (n <= 0) return 0;
  if (count < 1) return QV_ERR_UNSUPPORTED;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  return qv_launch(depth_mix_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, delta, stack, (size_t)n, w, count);
}

// x *= s in place, float32 (a fixed factor on logits).
__global__ void scale_kernel(float* __restrict__ x, size_t n, float s) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] *= s;
}

extern "C" int qv_scale(float* x, long long n, float s, void* stream) {
  if (n <= 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  return qv_launch(scale_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, (size_t)n, s);
}

extern "C" const char* qv_error_string(int code) {
  if (code == QV_ERR_UNSUPPORTED) return "size or dtype not supported by this kernel";
  if (code == QV_ERR_TOO_LARGE) return "size exceeds what this kernel can hold on chip";
  return cudaGetErrorString((cudaError_t)code);
}

// ---------------------------------------------------------------- norm on a sublayer's output (post-norm blocks)
// residual[t] += y[t] * rsqrt(mean(y[t]^2) + eps) * w     (float32; y in the compute type or float32, row stride ld_y)
// cast[t] = residual[t] in the compute type, if cast is given: what the next sublayer's products read.
// One block per row; the sum's order depends on d alone.  VEC: the row of y stays in registers and is read once, four elements
// at a time (d a multiple of 4, at most 4 * 4 * blockDim elements, rows that start on 16 bytes).
template <typename TY, typename TO, bool VEC>
__global__ void __launch_bounds__(256) post_rmsnorm_add_kernel(float* __restrict__ residual, const TY* __restrict__ y, int ld_y,
                                                              const float* __restrict__ w, float eps, TO* __restrict__ cast, int d) {
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const TY* yr = y + (size_t)t * ld_y;
  float* res = residual + (size_t)t * d;
  float ss = 0.f;
  if constexpr (VEC) {
    constexpr int MAXV = 4;
    float4 v[MAXV], r[MAXV];
    const int nvec = d >> 2;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = threadIdx.x + k * 256;
      v[k] = i < nvec ? Vec4<TY>::load(yr + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
      r[k] = i < nvec ? *(const float4*)(res + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < MAXV; ++k) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    const float total = block_sum(ss, red);
    const float sc = 1.0f / sqrtf(total / (float)d + eps);
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < nvec) {
        const float4 wv = *(const float4*)(w + 4 * i);
        const float4 x = make_float4(r[k].x + v[k].x * sc * wv.x, r[k].y + v[k].y * sc * wv.y, r[k].z + v[k].z * sc * wv.z,
                                     r[k].w + v[k].w * sc * wv.w);
        *(float4*)(res + 4 * i) = x;
        if (cast) store4(cast + (size_t)t * d + 4 * i, x);
      }
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) { const float v = to_f(yr[i]); ss = fmaf(v, v, ss); }
    const float total = block_sum(ss, red);
    const float sc = 1.0f / sqrtf(total / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      const float x = res[i] + to_f(yr[i]) * sc * w[i];
      res[i] = x;
      if (cast) cast[(size_t)t * d + i] = from_f<TO>(x);
    }
  }
}

extern "C" int qv_post_rmsnorm_add(float* residual, const void* y, int ld_y, const float* w, float eps, void* cast, int T, int d,
                                   int y_dt, int cast_dt, void* stream) {
  if (T <= 0 || d <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = d % 4 == 0 && d <= 4 * 4 * 256 && ld_y % 4 == 0 &&
                   (((uintptr_t)residual | (uintptr_t)y | (uintptr_t)w | (uintptr_t)cast) & 15) == 0;
#define LAUNCH_POST(TY, TO)                                                                                                        \
  do {                                                                                                                             \
    if (vec) return qv_launch(post_rmsnorm_add_kernel<TY, TO, true>, dim3(T), dim3(256), 0, st, residual, (const TY*)y, ld_y, w,   \
                              eps, (TO*)cast, d);                                                                                  \
    return qv_launch(post_rmsnorm_add_kernel<TY, TO, false>, dim3(T), dim3(256), 0, st, residual, (const TY*)y, ld_y, w, eps,      \
                     (TO*)cast, d);                                                                                                \
  } while (0)
  if (y_dt == QV_DT_F32 && cast_dt == QV_DT_F32) LAUNCH_POST(float, float);
  if (y_dt == QV_DT_BF16 && cast_dt == QV_DT_BF16) LAUNCH_POST(bf16, bf16);
  if (y_dt == QV_DT_F32 && cast_dt == QV_DT_BF16) LAUNCH_POST(float, bf16);
  if (y_dt == QV_DT_BF16 && cast_dt == QV_DT_F32) LAUNCH_POST(bf16, float);
#undef LAUNCH_POST
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- RMS norm of rows that are slices
// out[t, :n] = in[t, :n] * rsqrt(mean(in[t, :n]^2) + eps) * w (w may be null), rows with strides; float32 arithmetic.
// One warp per row, four rows a block.
template <typename TI, typename TO>
__global__ void __launch_bounds__(128) rmsnorm_rows_kernel(TO* __restrict__ out, int ld_out, const TI* __restrict__ in, int ld_in,
                                                          const float* __restrict__ w, float eps, int T, int n) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const TI* x = in + (size_t)t * ld_in;
  float ss = 0.f;
  for (int i = lane; i < n; i += 32) { const float v = to_f(x[i]); ss = fmaf(v, v, ss); }
  ss = warp_sum(ss);
  const float sc = 1.0f / sqrtf(ss / (float)n + eps);
  TO* o = out + (size_t)t * ld_out;
  for (int i = lane; i < n; i += 32) o[i] = from_f<TO>(to_f(x[i]) * sc * (w ? w[i] : 1.0f));
}

extern "C" int qv_rmsnorm_rows(void* out, int ld_out, const void* in, int ld_in, const float* w, float eps, int T, int n, int in_dt,
                               int out_dt, void* stream) {
  if (T <= 0 || n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid((T + 3) / 4);
#define LAUNCH_ROWS(TI, TO) \
  return qv_launch(rmsnorm_rows_kernel<TI, TO>, grid, dim3(128), 0, st, (TO*)out, ld_out, (const TI*)in, ld_in, w, eps, T, n)
  if (in_dt == QV_DT_F32 && out_dt == QV_DT_F32) LAUNCH_ROWS(float, float);
  if (in_dt == QV_DT_BF16 && out_dt == QV_DT_BF16) LAUNCH_ROWS(bf16, bf16);
  if (in_dt == QV_DT_F32 && out_dt == QV_DT_BF16) LAUNCH_ROWS(float, bf16);
  if (in_dt == QV_DT_BF16 && out_dt == QV_DT_F32) LAUNCH_ROWS(bf16, float);
#undef LAUNCH_ROWS
  return QV_ERR_UNSUPPORTED;
}
