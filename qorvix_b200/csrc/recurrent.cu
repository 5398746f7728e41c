// Recurrent mixers' kernels: a per-request state of fixed size carried from token to token.
//
// qv_conv_state     short causal convolution per channel with optional bias, optional SiLU and optionally the input
//                   added to the result, the last taps-1 inputs of a request kept as state so that a portion continues
//                   where the last one ended.
// qv_linear_scan    S_t = a_t S_(t-1) + b_t k_t v_t^T;  y_t = S_t^T q_t  per head, S in float32, in two kinds:
//                     GATED_MAX  exponential gates stabilised by a running maximum (matrix-memory LSTM):
//                                log i = cap tanh((gi + bi)/cap), log f = logsigmoid(cap tanh((gf + bf)/cap)),
//                                m_t = max(log f + m_(t-1), log i), a = exp(log f + m_(t-1) - m_t), b = exp(log i - m_t),
//                                n_t = a n_(t-1) + b k_t,  y_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//                     DECAY      selective state space with a scalar decay per head:
//                                dt = softplus(g + bias), a = exp(-exp(A_log) dt), b = dt, y_t = S_t^T q_t + D v_t
// qv_gated_group_norm  the unit norm (RMS over equal parts of a row) with weight and gate that follows a scan.
//
// All state arithmetic, gates, decays and norms are float32; q, k and v are read in the compute type.
#include "common.cuh"

#define CONV_MAX_TAPS 16
#define CONV_CHUNK 16

// in/out: [T, channels] with row strides and types of their own; w [channels, taps] (last column: the current token),
// bias [channels] or null; tail [slots][(taps-1) * channels] float32, oldest input first.  act 1: SiLU of the sum, 0: the sum
// as it is; add_input 1: the current input is added to the result (out = in + conv(in), after the activation).
// grid (segments, channel tiles, time chunks).  MT: the most taps this instance takes (its arrays stay in registers).
template <typename TI, typename TO, int MT>
__global__ void __launch_bounds__(128) conv_state_kernel(TO* __restrict__ out, int ld_out, const TI* __restrict__ in, int ld_in,
                                                         const float* __restrict__ w, const float* __restrict__ bias,
                                                         float* __restrict__ tail, long long slot_stride,
                                                         const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot,
                                                         int channels, int taps, int act, int add_input) {
  pdl_wait();
  pdl_launch_dependents();
  const int s = blockIdx.x;
  const int c = blockIdx.y * 128 + threadIdx.x;
  const int q0 = seg_q_start[s], len = seg_q_start[s + 1] - q0;
  const int j0 = blockIdx.z * CONV_CHUNK;
  if (c >= channels || j0 >= len) return;
  const int j1 = j0 + CONV_CHUNK < len ? j0 + CONV_CHUNK : len;
  float* tl = tail + (size_t)seg_slot[s] * slot_stride;
  float curs[CONV_CHUNK];                        // the chunk's inputs, all loads in flight before the first is used
#pragma unroll
  for (int jj = 0; jj < CONV_CHUNK; ++jj) curs[jj] = j0 + jj < j1 ? to_f(in[(size_t)(q0 + j0 + jj) * ld_in + c]) : 0.f;
  float wt[MT], win[MT];
  // win[i]: the input taps - 1 - i places ahead of the token in turn; a chunk is at least as long as the longest filter reaches
  // back, so only the first chunk reads the state
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    wt[i] = i < taps ? w[(size_t)c * taps + i] : 0.f;
    win[i] = 0.f;
    if (i < taps - 1) {
      const int idx = j0 - (taps - 1) + i;
      win[i] = idx >= 0 ? to_f(in[(size_t)(q0 + idx) * ld_in + c]) : tl[(size_t)(taps - 1 + idx) * channels + c];
    }
  }
  if (blockIdx.z == 0) {
    // the state after this segment: its last taps - 1 inputs, or, of a segment shorter than that, what is left of the old state
    // ahead of its own inputs.  Written now from values in registers (only this thread reads or writes these entries).
#pragma unroll
    for (int i = 0; i < MT - 1; ++i) {
      if (i < taps - 1) {
        const int idx = len - (taps - 1) + i;             // place in the segment; below zero: entry len + i of the old state
        float v = 0.f;
        if (idx < 0) {
#pragma unroll
          for (int k = 0; k < MT - 1; ++k)
            if (k == len + i) v = win[k];
        } else if (idx < CONV_CHUNK) {
#pragma unroll
          for (int k = 0; k < CONV_CHUNK; ++k)
            if (k == idx) v = curs[k];
        } else {
          v = to_f(in[(size_t)(q0 + idx) * ld_in + c]);
        }
        tl[(size_t)i * channels + c] = v;
      }
    }
  }
  const float b = bias ? bias[c] : 0.f;
#pragma unroll
  for (int jj = 0; jj < CONV_CHUNK; ++jj) {
    if (j0 + jj >= j1) break;
    const float cur = curs[jj];
    float acc = b;
#pragma unroll
    for (int i = 0; i < MT - 1; ++i) {
      if (i < taps - 1) acc = fmaf(wt[i], win[i], acc);
    }
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (i == taps - 1) acc = fmaf(wt[i], cur, acc);
    }
#pragma unroll
    for (int i = 0; i < MT - 1; ++i) {
      if (i < taps - 2) win[i] = win[i + 1];
      else if (i == taps - 2) win[i] = cur;
    }
    if (act) acc = acc / (1.0f + expf(-acc));
    if (add_input) acc += cur;
    out[(size_t)(q0 + j0 + jj) * ld_out + c] = from_f<TO>(acc);
  }
}

extern "C" int qv_conv_state(void* out, int ld_out, const void* in, int ld_in, const float* w, const float* bias, float* tail,
                             long long slot_stride, const int* seg_q_start, const int* seg_slot, int S, int max_q_len,
                             int channels, int taps, int in_dt, int out_dt, int act, int add_input, void* stream) {
  if (S <= 0 || channels <= 0) return 0;
  if (taps < 1 || taps > CONV_MAX_TAPS) return QV_ERR_UNSUPPORTED;
  const int chunks = max_q_len > 0 ? (max_q_len + CONV_CHUNK - 1) / CONV_CHUNK : 1;
  if (chunks > 65535 || (channels + 127) / 128 > 65535) return QV_ERR_TOO_LARGE;
  dim3 grid(S, (channels + 127) / 128, chunks);
#define LAUNCH_CONV(TI, TO)                                                                                                    \
  do {                                                                                                                         \
    if (taps <= 4)                                                                                                             \
      return qv_launch(conv_state_kernel<TI, TO, 4>, grid, dim3(128), 0, (cudaStream_t)stream, (TO*)out, ld_out, (const TI*)in, \
                       ld_in, w, bias, tail, slot_stride, seg_q_start, seg_slot, channels, taps, act, add_input);              \
    return qv_launch(conv_state_kernel<TI, TO, CONV_MAX_TAPS>, grid, dim3(128), 0, (cudaStream_t)stream, (TO*)out, ld_out,     \
                     (const TI*)in, ld_in, w, bias, tail, slot_stride, seg_q_start, seg_slot, channels, taps, act, add_input); \
  } while (0)
  if (in_dt == QV_DT_F32 && out_dt == QV_DT_F32) LAUNCH_CONV(float, float);
  if (in_dt == QV_DT_BF16 && out_dt == QV_DT_BF16) LAUNCH_CONV(bf16, bf16);
  if (in_dt == QV_DT_F32 && out_dt == QV_DT_BF16) LAUNCH_CONV(float, bf16);
  if (in_dt == QV_DT_BF16 && out_dt == QV_DT_F32) LAUNCH_CONV(bf16, float);
#undef LAUNCH_CONV
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- the scan
#define SCAN_VT 32          // value columns per block (one per lane)
#define SCAN_WARPS 8        // the key rows are dealt to the warps
#define SCAN_GATED_MAX 0
#define SCAN_DECAY 1

struct ScanArgs {
  float* out; int ld_out;                 // [T, H * dv] float32
  const void* q; int ld_q; int q_group;   // head h reads columns (h / q_group) * dk ... of q and of k
  const void* k; int ld_k;
  const void* v; int ld_v;                // head h reads columns h * dv ...
  const float* g1; int ld_g1;             // [T, >= H]: input-gate pre-activation | step pre-activation
  const float* g2; int ld_g2;             // [T, >= H]: forget-gate pre-activation (GATED_MAX)
  const float* p1; const float* p2; const float* p3;   // per head: bi | dt bias;  bf | A_log;  - | D
  float cap; float q_scale;
  float* state; long long slot_stride;    // per slot: [H][tiles][dk * 32 (+ dk + 1 for GATED_MAX)]
  const int* seg_q_start; const int* seg_slot;
  int H, dk, dv;
};

__host__ __device__ inline int scan_tile_floats(int kind, int dk, int vt = SCAN_VT) { return dk * vt + (kind == SCAN_GATED_MAX ? dk + 1 : 0); }
// Value columns a CTA owns: 32, or 16 for key sizes of 129..256, where a thread would else keep 32 rows (more than
// its registers hold) and wide heads give few CTAs.  A function of the key size alone: the state's layout follows it.
static inline int scan_vt(int dk) { return (dk > 128 && dk <= 256) ? 16 : 32; }

template <typename T, int KIND>
__global__ void __launch_bounds__(SCAN_VT * SCAN_WARPS) linear_scan_kernel(ScanArgs a) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int s = blockIdx.x, h = blockIdx.y, tile = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int dk = a.dk, dv = a.dv;
  const int tiles = (dv + SCAN_VT - 1) / SCAN_VT;
  float* S = sm;                           // [dk][32]
  float* qs = S + (size_t)dk * SCAN_VT;    // [dk]
  float* ks = qs + dk;                     // [dk]
  float* ns = ks + dk;                     // [dk] (GATED_MAX)
  float* red = ns + dk;                    // [SCAN_WARPS][32]
  float* sc = red + SCAN_WARPS * SCAN_VT;  // [2]: n . q, spare
  const int q0 = a.seg_q_start[s], len = a.seg_q_start[s + 1] - q0;
  float* st = a.state + (size_t)a.seg_slot[s] * a.slot_stride + ((size_t)h * tiles + tile) * scan_tile_floats(KIND, dk);
  for (int i = threadIdx.x; i < dk * SCAN_VT; i += blockDim.x) S[i] = st[i];
  float m = 0.f;
  if (KIND == SCAN_GATED_MAX) {
    for (int i = threadIdx.x; i < dk; i += blockDim.x) ns[i] = st[dk * SCAN_VT + i];
    m = st[dk * SCAN_VT + dk];
  }
  const int col = tile * SCAN_VT + lane;
  const bool live = col < dv;
  const T* qb = (const T*)a.q + (size_t)(h / a.q_group) * dk;
  const T* kb = (const T*)a.k + (size_t)(h / a.q_group) * dk;
  const T* vb = (const T*)a.v + (size_t)h * dv;
  const float b1 = a.p1 ? a.p1[h] : 0.f, b2 = a.p2 ? a.p2[h] : 0.f, b3 = a.p3 ? a.p3[h] : 0.f;
  __syncthreads();
  for (int j = 0; j < len; ++j) {
    const size_t t = (size_t)(q0 + j);
    for (int i = threadIdx.x; i < dk; i += blockDim.x) {
      qs[i] = to_f(qb[t * a.ld_q + i]) * a.q_scale;
      ks[i] = to_f(kb[t * a.ld_k + i]);
    }
    const float vv = live ? to_f(vb[t * a.ld_v + col]) : 0.f;
    float keep, take;
    if (KIND == SCAN_GATED_MAX) {
      const float li = a.cap * tanhf((a.g1[t * a.ld_g1 + h] + b1) / a.cap);
      const float zf = a.cap * tanhf((a.g2[t * a.ld_g2 + h] + b2) / a.cap);
      const float lf = fminf(zf, 0.f) - log1pf(expf(-fabsf(zf)));          // log sigmoid
      const float m_new = fmaxf(lf + m, li);
      keep = expf(lf + m - m_new);
      take = expf(li - m_new);
      m = m_new;
    } else {
      const float z = a.g1[t * a.ld_g1 + h] + b1;
      const float dt = z > 20.f ? z : log1pf(expf(z));                      // softplus
      keep = expf(-expf(b2) * dt);
      take = dt;
    }
    __syncthreads();                       // qs, ks are in place; red of the last token has been read
    if (KIND == SCAN_GATED_MAX && warp == 0) {
      float dot = 0.f;
      for (int i = lane; i < dk; i += 32) {
        const float n = keep * ns[i] + take * ks[i];
        ns[i] = n;
        dot = fmaf(n, qs[i], dot);
      }
      dot = warp_sum(dot);
      if (lane == 0) sc[0] = dot;
    }
    float acc = 0.f;
    const float tv = take * vv;
    for (int i = warp; i < dk; i += SCAN_WARPS) {
      const float sv = fmaf(keep, S[i * SCAN_VT + lane], tv * ks[i]);
      S[i * SCAN_VT + lane] = sv;
      acc = fmaf(sv, qs[i], acc);
    }
    red[warp * SCAN_VT + lane] = acc;
    __syncthreads();
    if (warp == 0 && live) {
      float y = 0.f;
#pragma unroll
      for (int w = 0; w < SCAN_WARPS; ++w) y += red[w * SCAN_VT + lane];
      if (KIND == SCAN_GATED_MAX) y = y / (fmaxf(fabsf(sc[0]), expf(-m)) + 1e-6f);
      else y = fmaf(b3, vv, y);
      a.out[t * a.ld_out + (size_t)h * dv + col] = y;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < dk * SCAN_VT; i += blockDim.x) st[i] = S[i];
  if (KIND == SCAN_GATED_MAX) {
    for (int i = threadIdx.x; i < dk; i += blockDim.x) st[dk * SCAN_VT + i] = ns[i];
    if (threadIdx.x == 0) st[dk * SCAN_VT + dk] = m;
  }
}

// The same recurrence with the state in registers (key sizes up to 8 * RPT rows: a thread keeps RPT rows of its value
// column) and tokens taken four at a time: their inputs are fetched together, the block meets twice per four tokens
// instead of twice per token, and each of the first four warps sums one token's partial outputs.  Arithmetic and
// summation order are those of linear_scan_kernel; the state's layout in memory is the same.
#define SCAN_TB 4
#define SCAN_CH 256      // tokens whose gates are worked out together (one a thread)
// ASYNC: the rows of q and k start on 16 bytes, and the next four tokens' rows are copied into the other of two
// buffers by cp.async while the present four are worked on (else plain loads ahead of the work).
template <typename T, int KIND, int RPT, bool ASYNC, int VT>
__global__ void __launch_bounds__(SCAN_VT * SCAN_WARPS) linear_scan_reg_kernel(ScanArgs a) {
  extern __shared__ __align__(16) float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int s = blockIdx.x, h = blockIdx.y, tile = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int dk = a.dk, dv = a.dv;
  constexpr int RS = 32 / VT;                       // row groups a warp: with 16 columns a tile, the lanes' halves take alternate rows
  const int cl = lane % VT, rsub = lane / VT;
  const int tiles = (dv + VT - 1) / VT;
  const int rowpad = (dk + 7) & ~7;                // a token's row in the buffers (elements): whole 16-byte pieces
  T* raw = (T*)sm;                                 // [2 buffers][q, k][TB][rowpad] as stored (the scale of q is applied to the sums)
  float* ns = sm + (4 * SCAN_TB * rowpad * sizeof(T) + 3) / 4;   // [dk]
  float* red = ns + dk;                            // [TB][SCAN_WARPS][32]
  float* sc = red + SCAN_TB * SCAN_WARPS * SCAN_VT;  // [TB]
  float* gk = sc + SCAN_TB;                        // [SCAN_CH] keep factors of the tokens in work
  float* gt = gk + SCAN_CH;                        // [SCAN_CH] take factors
  float* ge = gt + SCAN_CH;                        // [SCAN_CH] exp(-m) (GATED_MAX)
  float* gm = ge + SCAN_CH;                        // [SCAN_CH] scratch of the running maximum
  const int q0 = a.seg_q_start[s], len = a.seg_q_start[s + 1] - q0;
  float* st = a.state + (size_t)a.seg_slot[s] * a.slot_stride + ((size_t)h * tiles + tile) * scan_tile_floats(KIND, dk, VT);
  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int k = warp * RS + rsub + SCAN_WARPS * RS * i;
    S[i] = k < dk ? st[k * VT + cl] : 0.f;
  }
  float m = 0.f;
  if (KIND == SCAN_GATED_MAX) {
    for (int i = threadIdx.x; i < dk; i += blockDim.x) ns[i] = st[dk * VT + i];
    m = st[dk * VT + dk];
  }
  const int col = tile * VT + cl;
  const bool live = col < dv;
  const T* qb = (const T*)a.q + (size_t)(h / a.q_group) * dk;
  const T* kb = (const T*)a.k + (size_t)(h / a.q_group) * dk;
  const T* vb = (const T*)a.v + (size_t)h * dv;
  const float b1 = a.p1 ? a.p1[h] : 0.f, b2 = a.p2 ? a.p2[h] : 0.f, b3 = a.p3 ? a.p3[h] : 0.f;
  const float rate = KIND == SCAN_DECAY ? expf(b2) : 0.f;
  auto issue = [&](int buf, int j0) {
    const int nb = len - j0 < SCAN_TB ? len - j0 : SCAN_TB;
    const int pieces = dk * (int)sizeof(T) / 16, per = 16 / (int)sizeof(T);
    T* dst = raw + (size_t)buf * 2 * SCAN_TB * rowpad;
    for (int c = threadIdx.x; c < 2 * nb * pieces; c += blockDim.x) {
      const int which = c / (nb * pieces), rem = c - which * nb * pieces, tt = rem / pieces, pc = rem - tt * pieces;
      const T* src = (which ? kb + (size_t)(q0 + j0 + tt) * a.ld_k : qb + (size_t)(q0 + j0 + tt) * a.ld_q) + pc * per;
      const unsigned sa = (unsigned)__cvta_generic_to_shared(dst + (which * SCAN_TB + tt) * rowpad + pc * per);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(src) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (ASYNC) issue(0, 0);
  // Gates are worked out for 256 tokens at a time, one token a thread, and kept in shared memory: the transcendental
  // functions then lie off the path from one token to the next.  Only the running maximum is a chain (thread 0).
  for (int c0 = 0; c0 < len; c0 += SCAN_CH) {
    const int nch = len - c0 < SCAN_CH ? len - c0 : SCAN_CH;
    __syncthreads();                         // the gates of the last 256 tokens have been used
    if ((int)threadIdx.x < nch) {
      const size_t t = (size_t)(q0 + c0 + threadIdx.x);
      if (KIND == SCAN_GATED_MAX) {
        const float zf = a.cap * tanhf((a.g2[t * a.ld_g2 + h] + b2) / a.cap);
        gk[threadIdx.x] = fminf(zf, 0.f) - log1pf(expf(-fabsf(zf)));          // log forget gate
        gt[threadIdx.x] = a.cap * tanhf((a.g1[t * a.ld_g1 + h] + b1) / a.cap);  // log input gate
      } else {
        const float z = a.g1[t * a.ld_g1 + h] + b1;
        const float dt = z > 20.f ? z : log1pf(expf(z));
        gk[threadIdx.x] = expf(-rate * dt);
        gt[threadIdx.x] = dt;
      }
    }
    if (KIND == SCAN_GATED_MAX) {
      __syncthreads();
      if (threadIdx.x == 0) {
        float mm = m;
        for (int j = 0; j < nch; ++j) {
          const float m_new = fmaxf(gk[j] + mm, gt[j]);
          gm[j] = mm;                          // the maximum before this token
          ge[j] = m_new;                       // and after it
          mm = m_new;
        }
      }
      __syncthreads();
      m = ge[nch - 1];
      __syncthreads();                       // everyone has the maximum before its place is used for exp(-m)
      if ((int)threadIdx.x < nch) {
        const float lf = gk[threadIdx.x], li = gt[threadIdx.x], mp = gm[threadIdx.x], mc = ge[threadIdx.x];
        gk[threadIdx.x] = expf(lf + mp - mc);
        gt[threadIdx.x] = expf(li - mc);
        ge[threadIdx.x] = expf(-mc);
      }
    }
    __syncthreads();
  for (int j0 = c0; j0 < c0 + nch; j0 += SCAN_TB) {
    const int nb = c0 + nch - j0 < SCAN_TB ? c0 + nch - j0 : SCAN_TB;
    const size_t t0 = (size_t)(q0 + j0);
    const int buf = (j0 / SCAN_TB) & 1;
    const T* qs = raw + (size_t)buf * 2 * SCAN_TB * rowpad;
    const T* ks = qs + SCAN_TB * rowpad;
    if (ASYNC) {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
      T* wq = raw + (size_t)buf * 2 * SCAN_TB * rowpad;
      for (int c = threadIdx.x; c < nb * dk; c += blockDim.x) {
        const int tt = c / dk, i = c - tt * dk;
        wq[tt * rowpad + i] = qb[(t0 + tt) * a.ld_q + i];
        wq[(SCAN_TB + tt) * rowpad + i] = kb[(t0 + tt) * a.ld_k + i];
      }
    }
    float vv[SCAN_TB], keep[SCAN_TB], take[SCAN_TB], mt[SCAN_TB];
#pragma unroll
    for (int tt = 0; tt < SCAN_TB; ++tt) {
      vv[tt] = 0.f; keep[tt] = 1.f; take[tt] = 0.f; mt[tt] = 1.f;
      if (tt < nb) {
        vv[tt] = live ? to_f(vb[(t0 + tt) * a.ld_v + col]) : 0.f;
        keep[tt] = gk[j0 - c0 + tt];
        take[tt] = gt[j0 - c0 + tt];
        if (KIND == SCAN_GATED_MAX) mt[tt] = ge[j0 - c0 + tt];          // exp(-m) after the token
      }
    }
    __syncthreads();                       // the four tokens' q and k are in place; red and sc of the last four have been read
    if (ASYNC && j0 + SCAN_TB < len) issue(buf ^ 1, j0 + SCAN_TB);
    if (KIND == SCAN_GATED_MAX && warp == 0) {
      for (int tt = 0; tt < nb; ++tt) {
        float dot = 0.f;
        for (int i = lane; i < dk; i += 32) {
          const float n = keep[tt] * ns[i] + take[tt] * to_f(ks[tt * rowpad + i]);
          ns[i] = n;
          dot = fmaf(n, to_f(qs[tt * rowpad + i]), dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) sc[tt] = dot * a.q_scale;
      }
    }
#pragma unroll
    for (int tt = 0; tt < SCAN_TB; ++tt) {
      if (tt < nb) {
        float acc = 0.f;
        const float tv = take[tt] * vv[tt];
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
          const int k = warp * RS + rsub + SCAN_WARPS * RS * i;
          if (k < dk) {
            S[i] = fmaf(keep[tt], S[i], tv * to_f(ks[tt * rowpad + k]));
            acc = fmaf(S[i], to_f(qs[tt * rowpad + k]), acc);
          }
        }
        red[(tt * SCAN_WARPS + warp) * SCAN_VT + lane] = acc;
      }
    }
    __syncthreads();
    if (warp < nb && live && rsub == 0) {
      const int tt = warp;
      float y = 0.f;
#pragma unroll
      for (int w = 0; w < SCAN_WARPS; ++w)
#pragma unroll
        for (int g = 0; g < RS; ++g) y += red[(tt * SCAN_WARPS + w) * SCAN_VT + g * VT + cl];
      y *= a.q_scale;
      // vv and mt of token tt, which this thread holds at a compile-time index only: pick without indexing registers
      float v_tt = vv[0], m_tt = mt[0];
#pragma unroll
      for (int x = 1; x < SCAN_TB; ++x) if (x == tt) { v_tt = vv[x]; m_tt = mt[x]; }
      if (KIND == SCAN_GATED_MAX) y = y / (fmaxf(fabsf(sc[tt]), m_tt) + 1e-6f);
      else y = fmaf(b3, v_tt, y);
      a.out[(t0 + tt) * a.ld_out + (size_t)h * dv + col] = y;
    }
  }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int k = warp * RS + rsub + SCAN_WARPS * RS * i;
    if (k < dk) st[k * VT + cl] = S[i];
  }
  if (KIND == SCAN_GATED_MAX) {
    for (int i = threadIdx.x; i < dk; i += blockDim.x) st[dk * VT + i] = ns[i];
    if (threadIdx.x == 0) st[dk * VT + dk] = m;
  }
}

extern "C" long long qv_linear_scan_state_floats(int kind, int H, int dk, int dv) {
  const int vt = scan_vt(dk);
  return (long long)H * ((dv + vt - 1) / vt) * scan_tile_floats(kind, dk, vt);
}

extern "C" int qv_linear_scan(int kind, float* out, int ld_out, const void* q, int ld_q, int q_group, const void* k, int ld_k,
                              const void* v, int ld_v, const float* g1, int ld_g1, const float* g2, int ld_g2, const float* p1,
                              const float* p2, const float* p3, float cap, float q_scale, float* state, long long slot_stride,
                              const int* seg_q_start, const int* seg_slot, int S, int H, int dk, int dv, int dt, void* stream) {
  if (S <= 0) return 0;
  if (kind != SCAN_GATED_MAX && kind != SCAN_DECAY) return QV_ERR_UNSUPPORTED;
  if (H <= 0 || dk <= 0 || dv <= 0 || q_group <= 0 || H > 65535) return QV_ERR_UNSUPPORTED;
  const int vt = scan_vt(dk);
  const int tiles = (dv + vt - 1) / vt;
  const size_t smem = ((size_t)dk * SCAN_VT + 3 * (size_t)dk + SCAN_WARPS * SCAN_VT + 2) * sizeof(float);
  if (smem > 200 * 1024 || tiles > 65535) return QV_ERR_TOO_LARGE;
  ScanArgs a;
  a.out = out; a.ld_out = ld_out; a.q = q; a.ld_q = ld_q; a.q_group = q_group; a.k = k; a.ld_k = ld_k; a.v = v; a.ld_v = ld_v;
  a.g1 = g1; a.ld_g1 = ld_g1; a.g2 = g2; a.ld_g2 = ld_g2; a.p1 = p1; a.p2 = p2; a.p3 = p3; a.cap = cap; a.q_scale = q_scale;
  a.state = state; a.slot_stride = slot_stride; a.seg_q_start = seg_q_start; a.seg_slot = seg_slot; a.H = H; a.dk = dk; a.dv = dv;
  dim3 grid(S, H, tiles);
  cudaStream_t st = (cudaStream_t)stream;
  if (dk <= 8 * 32) {                      // the state fits the registers
    const size_t esz = dt == QV_DT_F32 ? 4 : 2;
    const size_t rowpad = (size_t)((dk + 7) & ~7);
    const size_t smem_r = ((4 * SCAN_TB * rowpad * esz + 3) / 4 + dk + SCAN_TB * SCAN_WARPS * SCAN_VT + SCAN_TB + 4 * SCAN_CH) * sizeof(float);
    const bool async = (dk * esz) % 16 == 0 && ((size_t)ld_q * esz) % 16 == 0 && ((size_t)ld_k * esz) % 16 == 0 &&
                       (((uintptr_t)q | (uintptr_t)k) & 15) == 0;
    const int rpt = dk <= 32 ? 4 : dk <= 64 ? 8 : 16;          // 129..256 rows: 16 columns a tile, two row groups a warp
#define LAUNCH_REG(TT, KIND, RPT)                                                                                             \
  do {                                                                                                                        \
    if (vt == 16) {                                                                                                           \
      if (async) return qv_launch(linear_scan_reg_kernel<TT, KIND, 16, true, 16>, grid, dim3(SCAN_VT * SCAN_WARPS), smem_r, st, a); \
      return qv_launch(linear_scan_reg_kernel<TT, KIND, 16, false, 16>, grid, dim3(SCAN_VT * SCAN_WARPS), smem_r, st, a);     \
    }                                                                                                                         \
    if (async) return qv_launch(linear_scan_reg_kernel<TT, KIND, RPT, true, 32>, grid, dim3(SCAN_VT * SCAN_WARPS), smem_r, st, a); \
    return qv_launch(linear_scan_reg_kernel<TT, KIND, RPT, false, 32>, grid, dim3(SCAN_VT * SCAN_WARPS), smem_r, st, a);      \
  } while (0)
#define LAUNCH_REG_RPT(TT, KIND)                  \
  do {                                            \
    if (rpt == 4) LAUNCH_REG(TT, KIND, 4);        \
    if (rpt == 8) LAUNCH_REG(TT, KIND, 8);        \
    LAUNCH_REG(TT, KIND, 16);                     \
  } while (0)
    if (dt == QV_DT_F32 && kind == SCAN_GATED_MAX) LAUNCH_REG_RPT(float, SCAN_GATED_MAX);
    if (dt == QV_DT_F32 && kind == SCAN_DECAY) LAUNCH_REG_RPT(float, SCAN_DECAY);
    if (dt == QV_DT_BF16 && kind == SCAN_GATED_MAX) LAUNCH_REG_RPT(bf16, SCAN_GATED_MAX);
    if (dt == QV_DT_BF16 && kind == SCAN_DECAY) LAUNCH_REG_RPT(bf16, SCAN_DECAY);
#undef LAUNCH_REG_RPT
#undef LAUNCH_REG
    return QV_ERR_UNSUPPORTED;
  }
#define LAUNCH_SCAN(TT, KIND)                                                                                               \
  do {                                                                                                                      \
    if (smem > 48 * 1024) cudaFuncSetAttribute(linear_scan_kernel<TT, KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    return qv_launch(linear_scan_kernel<TT, KIND>, grid, dim3(SCAN_VT * SCAN_WARPS), smem, st, a);                          \
  } while (0)
  if (dt == QV_DT_F32 && kind == SCAN_GATED_MAX) LAUNCH_SCAN(float, SCAN_GATED_MAX);
  if (dt == QV_DT_F32 && kind == SCAN_DECAY) LAUNCH_SCAN(float, SCAN_DECAY);
  if (dt == QV_DT_BF16 && kind == SCAN_GATED_MAX) LAUNCH_SCAN(bf16, SCAN_GATED_MAX);
  if (dt == QV_DT_BF16 && kind == SCAN_DECAY) LAUNCH_SCAN(bf16, SCAN_DECAY);
#undef LAUNCH_SCAN
  return QV_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------- unit norm in equal parts, weight, gate
// y [T, width] float32 in `groups` equal parts; gate [T, width] in the compute type (row stride ld_gate).
//   gate_first = 0:  out = y / rms_part(y) * w * sigmoid(gate)
//   gate_first = 1:  u = y * silu(gate);  out = u / rms_part(u) * w
// One block per (token, part).
template <typename T>
__global__ void __launch_bounds__(1024) gated_group_norm_kernel(T* __restrict__ out, int ld_out, const float* __restrict__ y, int ld_y,
                                                               const T* __restrict__ gate, int ld_gate, const float* __restrict__ w,
                                                               int part, float eps, int gate_first) {
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, g = blockIdx.y;
  const float* yr = y + (size_t)t * ld_y + (size_t)g * part;
  const T* gr = gate + (size_t)t * ld_gate + (size_t)g * part;
  T* o = out + (size_t)t * ld_out + (size_t)g * part;
  const float* wr = w + (size_t)g * part;
  float ss = 0.f;
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    float v = yr[i];
    if (gate_first) { const float z = to_f(gr[i]); v *= z / (1.0f + expf(-z)); }
    ss += v * v;
  }
  const float total = block_sum(ss, red);
  const float sc = 1.0f / sqrtf(total / (float)part + eps);
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    const float z = to_f(gr[i]);
    float v = yr[i];
    if (gate_first) v = v * (z / (1.0f + expf(-z))) * sc * wr[i];
    else v = v * sc * wr[i] * (1.0f / (1.0f + expf(-z)));
    o[i] = from_f<T>(v);
  }
}

extern "C" int qv_gated_group_norm(void* out, int ld_out, const float* y, int ld_y, const void* gate, int ld_gate, const float* w,
                                   int T, int width, int groups, float eps, int gate_first, int dt, void* stream) {
  if (T <= 0) return 0;
  if (groups <= 0 || width % groups || groups > 65535) return QV_ERR_UNSUPPORTED;
  // one element a thread up to 1024; the block's size, and so the order of the sums, follows from the part's width alone
  const int part_w = width / groups;
  const int threads = part_w >= 1024 ? 1024 : (part_w <= 128 ? 128 : ((part_w + 31) / 32) * 32);
  QV_DISPATCH_DT(dt, TT,
                 return qv_launch(gated_group_norm_kernel<TT>, dim3(T, groups), dim3(threads), 0, (cudaStream_t)stream, (TT*)out, ld_out, y,
                                  ld_y, (const TT*)gate, ld_gate, w, width / groups, eps, gate_first));
  return QV_ERR_UNSUPPORTED;
}
