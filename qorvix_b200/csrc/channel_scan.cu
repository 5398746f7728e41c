// Recurrences whose decay is a vector over the key channels, with or without the delta rule's removal term:
//
//   S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,      y_t = S_t^T q_t * q_scale
//
// per request and head, S [dk x dv] float32 in the request's state slot, both first terms reading the old state.
// Without removal (au, u null) this is gated linear attention's S_t = diag(w_t) S_(t-1) + k_t v_t^T.
//
// qv_channel_gates    per-channel factors from a low-rank pre-activation: z = W2 f(x1) + b, then
//                       POW_SIGMOID      sigmoid(z)^p                  (a decay with temperature 1/p)
//                       EXP_NEG_SIGMOID  exp(-p * sigmoid(z))          (a decay bounded below by exp(-p))
//                       EXP_NEG_SOFTPLUS exp(-rate_c * softplus(z))    (a step size times a rate per channel)
//                       LINEAR           z                             (a pre-activation for a later kernel)
//                     f the identity or tanh.
// qv_unit_keys        u = k / sqrt(sum(k^2) + eps) per head and au = sigmoid(a + bias) * u.
// qv_channel_scan     the recurrence.  The columns of S are independent of one another: a few lanes own a column, each a run of
//                     its rows in registers, so u^T S and S^T q are short sums in a fixed order; the warps of a CTA share the
//                     tokens' vectors, which arrive in shared memory by cp.async a chunk ahead.  Only u^T S lies on the chain
//                     from token to token.
// qv_head_norm_gate   the unit norm per head (RMS over a head's values) with weight, gate (sigmoid or SiLU, behind the norm)
//                     and a fixed factor that follows a scan.
//
// Everything is float32: the inputs are column slices of float32 products (row strides given), the state, the
// factors and all sums.  The order of every sum depends on the sizes alone, so a token's result does not depend
// on how its request was cut into steps or on what else is in the batch.
#include "common.cuh"

#define GATE_POW_SIGMOID 0
#define GATE_EXP_NEG_SIGMOID 1
#define GATE_EXP_NEG_SOFTPLUS 2
#define GATE_LINEAR 3

// x1 [T, R] (row stride ld_x), W2 transposed [R, N] float32, bias [N] or null -> out [T, N] (row stride ld_out).
// A CTA takes CG_TOKENS tokens and CG_CHANNELS channels, so that an entry of W2 is read once for all of its tokens; the sum over r
// is cut into four quarters (r ascending in each, by four groups of threads) that are added in order, so that a step of
// few tokens still has many loads in flight and the order of a sum depends on R alone.
#define CG_TOKENS 8
#define CG_CHANNELS 64
__global__ void __launch_bounds__(4 * CG_CHANNELS) channel_gates_kernel(float* __restrict__ out, int ld_out, const float* __restrict__ x1,
                                                                       int ld_x, const float* __restrict__ w2t,
                                                                       const float* __restrict__ bias, int T, int N, int R,
                                                                       int pre_tanh, int kind, float p, const float* __restrict__ rate) {
  extern __shared__ float cg_smem[];               // [CG_TOKENS][R] the tokens' low-rank rows, then [4][CG_TOKENS][CG_CHANNELS] partial sums
  float* xs = cg_smem;
  float* part = cg_smem + CG_TOKENS * R;
  pdl_wait();
  pdl_launch_dependents();
  const int t0 = blockIdx.x * CG_TOKENS;
  const int nt = min(CG_TOKENS, T - t0);
  for (int i = threadIdx.x; i < CG_TOKENS * R; i += blockDim.x) {
    const int j = i / R, r = i % R;
    float v = 0.f;
    if (j < nt) {
      v = x1[(size_t)(t0 + j) * ld_x + r];
      if (pre_tanh) v = tanhf(v);
    }
    xs[i] = v;
  }
  __syncthreads();
  const int cq = threadIdx.x / CG_CHANNELS, cl = threadIdx.x % CG_CHANNELS;
  const int c = blockIdx.y * CG_CHANNELS + cl;
  const int rq = (R + 3) / 4;
  const int r_lo = cq * rq, r_hi = min(R, r_lo + rq);
  float z[CG_TOKENS];
#pragma unroll
  for (int j = 0; j < CG_TOKENS; ++j) z[j] = 0.f;
  if (c < N) {
#pragma unroll 8
    for (int r = r_lo; r < r_hi; ++r) {
      const float wv = w2t[(size_t)r * N + c];
#pragma unroll
      for (int j = 0; j < CG_TOKENS; ++j) z[j] = fmaf(xs[j * R + r], wv, z[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < CG_TOKENS; ++j) part[(cq * CG_TOKENS + j) * CG_CHANNELS + cl] = z[j];
  __syncthreads();
  if (c >= N) return;
  const float bc = bias ? bias[c] : 0.f;
  for (int j = cq; j < nt; j += 4) {               // the four groups share the tokens' last step
    float zz = part[j * CG_CHANNELS + cl];
#pragma unroll
    for (int q = 1; q < 4; ++q) zz += part[(q * CG_TOKENS + j) * CG_CHANNELS + cl];
    zz += bc;
    float g;
    if (kind == GATE_POW_SIGMOID) {
      const float ls = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));          // log sigmoid(z)
      g = expf(p * ls);
    } else if (kind == GATE_EXP_NEG_SIGMOID) {
      g = expf(-p * (1.0f / (1.0f + expf(-zz))));
    } else if (kind == GATE_EXP_NEG_SOFTPLUS) {
      const float sp = fmaxf(zz, 0.f) + log1pf(expf(-fabsf(zz)));          // softplus(z)
      g = expf(-rate[c] * sp);
    } else {
      g = zz;
    }
    out[(size_t)(t0 + j) * ld_out + c] = g;
  }
}

// rate [N] float32: the factor per channel of GATE_EXP_NEG_SOFTPLUS (null for the other kinds).
extern "C" int qv_channel_gates(float* out, int ld_out, const float* x1, int ld_x, const float* w2t, const float* bias, int T, int N,
                                int R, int pre_tanh, int kind, float p, const float* rate, void* stream) {
  if (T <= 0 || N <= 0) return 0;
  const size_t smem = ((size_t)CG_TOKENS * R + 4 * CG_TOKENS * CG_CHANNELS) * sizeof(float);
  if (R <= 0 || smem > 48 * 1024) return QV_ERR_UNSUPPORTED;
  if (kind < GATE_POW_SIGMOID || kind > GATE_LINEAR || (kind == GATE_EXP_NEG_SOFTPLUS && rate == nullptr)) return QV_ERR_UNSUPPORTED;
  const int by = (N + CG_CHANNELS - 1) / CG_CHANNELS;
  if (by > 65535) return QV_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const int per = 65535 * CG_TOKENS;
  for (int done = 0; done < T; done += per) {
    const int rows = T - done < per ? T - done : per;
    const int rc = qv_launch(channel_gates_kernel, dim3((rows + CG_TOKENS - 1) / CG_TOKENS, by), dim3(4 * CG_CHANNELS), smem, st,
                             out + (size_t)done * ld_out, ld_out, x1 + (size_t)done * ld_x, ld_x, w2t, bias, rows, N, R, pre_tanh, kind, p, rate);
    if (rc) return rc;
  }
  return 0;
}

// k, a [T, H * n] float32 (row strides) -> u, au [T, H * n] dense.  One warp per (token, head).
__global__ void __launch_bounds__(128) unit_keys_kernel(float* __restrict__ u, float* __restrict__ au, const float* __restrict__ k, int ld_k,
                                                       const float* __restrict__ a, int ld_a, const float* __restrict__ a_bias, int H, int n,
                                                       float eps) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= H) return;
  const float* kr = k + (size_t)t * ld_k + (size_t)h * n;
  const float* ar = a + (size_t)t * ld_a + (size_t)h * n;
  float ss = 0.f;
  for (int i = lane; i < n; i += 32) ss = fmaf(kr[i], kr[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss + eps);
  const size_t o = ((size_t)t * H + h) * n;
  for (int i = lane; i < n; i += 32) {
    const float uu = kr[i] * inv;
    const float z = ar[i] + (a_bias ? a_bias[(size_t)h * n + i] : 0.f);
    u[o + i] = uu;
    au[o + i] = uu * (1.0f / (1.0f + expf(-z)));
  }
}

extern "C" int qv_unit_keys(float* u, float* au, const float* k, int ld_k, const float* a, int ld_a, const float* a_bias, int T, int H,
                            int n, float eps, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || n <= 0) return QV_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  for (int done = 0; done < T; done += 65535) {
    const int rows = T - done < 65535 ? T - done : 65535;
    const int rc = qv_launch(unit_keys_kernel, dim3(rows, (H + 3) / 4), dim3(128), 0, st, u + (size_t)done * H * n,
                             au + (size_t)done * H * n, k + (size_t)done * ld_k, ld_k, a + (size_t)done * ld_a, ld_a, a_bias, H, n, eps);
    if (rc) return rc;
  }
  return 0;
}

// The operands of the delta rule whose removal reads the decayed state,
//   S' = diag(g) S,  S = S' + k (beta (v - S'^T k))^T = diag(g) S - (beta k) ((g * k)^T S) + (beta k) v^T,
// in the scan's terms: w = g, u = g * k, au = beta k and the written key beta k, with k and q unit vectors per head
// (x / sqrt(sum x^2 + eps)) and q times q_scale.  q, k [T, G * n] float32 (row strides; head h reads group h / (H / G)),
// b [T, H] the pre-activation of beta = sigmoid(b), g [T, H * n] -> qh, kb, ug dense [T, H * n].  One warp per (token, head).
__global__ void __launch_bounds__(128) delta_operands_kernel(float* __restrict__ qh, float* __restrict__ kb, float* __restrict__ ug,
                                                            const float* __restrict__ q, int ld_q, const float* __restrict__ k, int ld_k,
                                                            const float* __restrict__ b, int ld_b, const float* __restrict__ g, int ld_g,
                                                            int H, int G, int n, float eps, float q_scale) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= H) return;
  const int grp = h / (H / G);
  const float* qr = q + (size_t)t * ld_q + (size_t)grp * n;
  const float* kr = k + (size_t)t * ld_k + (size_t)grp * n;
  const float* gr = g + (size_t)t * ld_g + (size_t)h * n;
  float sq = 0.f, sk = 0.f;
  for (int i = lane; i < n; i += 32) { sq = fmaf(qr[i], qr[i], sq); sk = fmaf(kr[i], kr[i], sk); }
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  const float iq = q_scale / sqrtf(sq + eps), ik = 1.0f / sqrtf(sk + eps);
  const float beta = 1.0f / (1.0f + expf(-b[(size_t)t * ld_b + h]));
  const size_t o = ((size_t)t * H + h) * n;
  for (int i = lane; i < n; i += 32) {
    const float kk = kr[i] * ik;
    qh[o + i] = qr[i] * iq;
    kb[o + i] = beta * kk;
    ug[o + i] = gr[i] * kk;
  }
}

extern "C" int qv_delta_operands(float* qh, float* kb, float* ug, const float* q, int ld_q, const float* k, int ld_k, const float* b,
                                 int ld_b, const float* g, int ld_g, int T, int H, int G, int n, float eps, float q_scale, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || n <= 0) return QV_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  for (int done = 0; done < T; done += 65535) {
    const int rows = T - done < 65535 ? T - done : 65535;
    const size_t o = (size_t)done * H * n;
    const int rc = qv_launch(delta_operands_kernel, dim3(rows, (H + 3) / 4), dim3(128), 0, st, qh + o, kb + o, ug + o,
                             q + (size_t)done * ld_q, ld_q, k + (size_t)done * ld_k, ld_k, b + (size_t)done * ld_b, ld_b,
                             g + (size_t)done * ld_g, ld_g, H, G, n, eps, q_scale);
    if (rc) return rc;
  }
  return 0;
}

// ---------------------------------------------------------------- the scan
// A column of S belongs to LPC lanes that hold CS_ROWS rows each (rows lic * CS_ROWS ..), so LPC = 1, 2, 4, 8, 16 serves key
// sizes up to 16, 32, 64, 128, 256; a warp holds 32 / LPC columns, a CTA four times that.  (Eight rows a lane and the next
// token's vectors fetched into registers ahead were measured and were slower: more shuffles and more registers.)  The sums over a column's rows
// are CS_ROWS multiply-adds a lane (four partial sums, a fixed order) and log2(LPC) shuffles.  The tokens' vectors arrive in
// shared memory by cp.async, a chunk of tokens ahead of the warps that work through them, and are read 16 bytes at a time.
// The state of a request is kept in the order of the registers ([head][warp tile][row of the lane][lane]), so that it is read and
// written in whole lines; rows and columns beyond the sizes hold zeros.
#define CS_WARPS 4
#define CS_ROWS 16
#define CS_PAD 20           // floats a lane's rows take in a stage: 16 and 4 of padding, so that 16-byte reads of the LPC lanes miss one another's banks

struct ChannelScanArgs {
  float* out; int ld_out;                 // [T, H * dv]
  const float* q; int ld_q;               // [T, H * dk] ...
  const float* k; int ld_k;
  const float* v; int ld_v;               // [T, H * dv]
  const float* w; int ld_w;               // decay per key channel
  const float* au; int ld_au;             // removal: a * u and u, or null
  const float* u; int ld_u;
  float q_scale;
  float* state; long long slot_stride;    // per slot: [H][tiles][CS_ROWS][32]
  const int* seg_q_start; const int* seg_slot;
  int H, dk, dv;
};

// 4 or 16 bytes, or as many zero bytes where `valid` is false
__device__ __forceinline__ void cs_cp4(float* dst, const float* src, bool valid) {
  const int bytes = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cs_cp16(float* dst, const float* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ float cs_sum4(const float* p) { return (p[0] + p[1]) + (p[2] + p[3]); }

// `chunk` tokens a stage, two stages.  vec4: every vector starts on 16 bytes and dk is a multiple of 4 (16-byte copies).
template <int LPC, bool REMOVAL>
__global__ void __launch_bounds__(32 * CS_WARPS) channel_scan_kernel(ChannelScanArgs a, int chunk, int vec4) {
  extern __shared__ __align__(16) float cs_ring[];
  constexpr int NV = REMOVAL ? 5 : 3;
  constexpr int CPW = 32 / LPC, CTA_COLS = CS_WARPS * CPW, NTH = 32 * CS_WARPS;
  constexpr int VEC = CS_PAD * LPC;                // floats a vector takes in a stage
  constexpr int ROW = NV * VEC + CTA_COLS;         // floats a token takes
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int lic = lane % LPC, cw = lane / LPC;
  const int dk = a.dk, dv = a.dv;
  const int cta_col0 = blockIdx.z * CTA_COLS;
  const int col = cta_col0 + warp * CPW + cw;
  const int tiles = (dv + CPW - 1) / CPW;
  const int q0 = a.seg_q_start[s], len = a.seg_q_start[s + 1] - q0;
  const int tile = blockIdx.z * CS_WARPS + warp;
  const bool active = tile < tiles;
  float* st = a.state + (size_t)a.seg_slot[s] * a.slot_stride + ((size_t)h * tiles + tile) * (CS_ROWS * 32) + lane;
  float S[CS_ROWS];
#pragma unroll
  for (int i = 0; i < CS_ROWS; ++i) S[i] = active ? st[i * 32] : 0.f;
  const size_t hk = (size_t)h * dk, hv = (size_t)h * dv;
  const float* srcs[5] = {a.w + hk, a.k + hk, a.q + hk, REMOVAL ? a.au + hk : nullptr, REMOVAL ? a.u + hk : nullptr};
  const int lds[5] = {a.ld_w, a.ld_k, a.ld_q, a.ld_au, a.ld_u};
  auto issue = [&](int c) {
    float* base = cs_ring + (size_t)(c & 1) * chunk * ROW;
    const int j0 = c * chunk, nt = min(chunk, len - j0);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      if (vec4) {
        constexpr int PER = CS_ROWS * LPC / 4;       // 16-byte pieces a vector (padding rows included)
        for (int i = tid; i < nt * PER; i += NTH) {
          const int j = i / PER, r = (i % PER) * 4;
          cs_cp16(base + j * ROW + v * VEC + r + (r / CS_ROWS) * (CS_PAD - CS_ROWS), srcs[v] + (size_t)(q0 + j0 + j) * lds[v] + r, r < dk);
        }
      } else {
        constexpr int PER = CS_ROWS * LPC;
        for (int i = tid; i < nt * PER; i += NTH) {
          const int j = i / PER, r = i % PER;
          cs_cp4(base + j * ROW + v * VEC + r + (r / CS_ROWS) * (CS_PAD - CS_ROWS), srcs[v] + (size_t)(q0 + j0 + j) * lds[v] + r, r < dk);
        }
      }
    }
    for (int i = tid; i < nt * CTA_COLS; i += NTH) {
      const int j = i / CTA_COLS, cc = i % CTA_COLS;
      cs_cp4(base + j * ROW + NV * VEC + cc, a.v + (size_t)(q0 + j0 + j) * a.ld_v + hv + cta_col0 + cc, cta_col0 + cc < dv);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int nchunks = (len + chunk - 1) / chunk;
  if (nchunks > 0) issue(0);
  for (int c = 0; c < nchunks; ++c) {
    if (c + 1 < nchunks) {
      issue(c + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int j0 = c * chunk, nt = min(chunk, len - j0);
    if (active) {
#pragma unroll(REMOVAL ? 2 : 4)
      for (int j = 0; j < nt; ++j) {
        const float* d = cs_ring + ((size_t)(c & 1) * chunk + j) * ROW;
        const float4* pw = (const float4*)(d + lic * CS_PAD);
        const float4* pk = (const float4*)(d + VEC + lic * CS_PAD);
        const float4* pq = (const float4*)(d + 2 * VEC + lic * CS_PAD);
        const float vv = d[NV * VEC + warp * CPW + cw];
        float dd = 0.f;
        if (REMOVAL) {
          const float4* pu = (const float4*)(d + 4 * VEC + lic * CS_PAD);
          float p[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int i = 0; i < CS_ROWS / 4; ++i) {
            const float4 u4 = pu[i];
            p[0] = fmaf(u4.x, S[4 * i], p[0]); p[1] = fmaf(u4.y, S[4 * i + 1], p[1]);
            p[2] = fmaf(u4.z, S[4 * i + 2], p[2]); p[3] = fmaf(u4.w, S[4 * i + 3], p[3]);
          }
          dd = cs_sum4(p);
#pragma unroll
          for (int o = LPC / 2; o > 0; o >>= 1) dd += __shfl_xor_sync(0xffffffffu, dd, o);
        }
        float y[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < CS_ROWS / 4; ++i) {
          const float4 w4 = pw[i], k4 = pk[i], q4 = pq[i];
          float n0 = fmaf(k4.x, vv, w4.x * S[4 * i]), n1 = fmaf(k4.y, vv, w4.y * S[4 * i + 1]);
          float n2 = fmaf(k4.z, vv, w4.z * S[4 * i + 2]), n3 = fmaf(k4.w, vv, w4.w * S[4 * i + 3]);
          if (REMOVAL) {
            const float4 a4 = ((const float4*)(d + 3 * VEC + lic * CS_PAD))[i];
            n0 = fmaf(-a4.x, dd, n0); n1 = fmaf(-a4.y, dd, n1); n2 = fmaf(-a4.z, dd, n2); n3 = fmaf(-a4.w, dd, n3);
          }
          S[4 * i] = n0; S[4 * i + 1] = n1; S[4 * i + 2] = n2; S[4 * i + 3] = n3;
          y[0] = fmaf(q4.x, n0, y[0]); y[1] = fmaf(q4.y, n1, y[1]); y[2] = fmaf(q4.z, n2, y[2]); y[3] = fmaf(q4.w, n3, y[3]);
        }
        float yy = cs_sum4(y);
#pragma unroll
        for (int o = LPC / 2; o > 0; o >>= 1) yy += __shfl_xor_sync(0xffffffffu, yy, o);
        if (lic == 0 && col < dv) a.out[(size_t)(q0 + j0 + j) * a.ld_out + hv + col] = yy * a.q_scale;
      }
    }
    __syncthreads();
  }
  pdl_launch_dependents();
  if (!active) return;
#pragma unroll
  for (int i = 0; i < CS_ROWS; ++i) st[i * 32] = S[i];
}

// A launch that starts only when the kernel before it has ended.  For portions the scan is a long kernel of few CTAs that wants an
// SM each: launched ahead (programmatic dependent launch) its CTAs are placed while the kernel before it still fills the SMs, several
// on one SM, and the scan of a 2,048-token prompt was measured to take 1.6 to 2 times as long.
template <typename... KArgs, typename... Args>
static inline int cs_launch_after(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  return (int)cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

static inline int cs_lanes_per_column(int dk) { return dk <= 16 ? 1 : dk <= 32 ? 2 : dk <= 64 ? 4 : dk <= 128 ? 8 : 16; }

extern "C" long long qv_channel_scan_state_floats(int H, int dk, int dv) {
  const int cpw = 32 / cs_lanes_per_column(dk);
  return (long long)H * ((dv + cpw - 1) / cpw) * CS_ROWS * 32;
}

// max_q_len: the longest segment of the step (how many tokens a stage of the ring holds follows from it).
extern "C" int qv_channel_scan(float* out, int ld_out, const float* q, int ld_q, const float* k, int ld_k, const float* v, int ld_v,
                               const float* w, int ld_w, const float* au, int ld_au, const float* u, int ld_u, float q_scale,
                               float* state, long long slot_stride, const int* seg_q_start, const int* seg_slot, int S, int max_q_len,
                               int H, int dk, int dv, void* stream) {
  if (S <= 0) return 0;
  if (H <= 0 || dk <= 0 || dv <= 0 || H > 65535 || (au == nullptr) != (u == nullptr)) return QV_ERR_UNSUPPORTED;
  if (dk > 256) return QV_ERR_TOO_LARGE;
  ChannelScanArgs a;
  a.out = out; a.ld_out = ld_out; a.q = q; a.ld_q = ld_q; a.k = k; a.ld_k = ld_k; a.v = v; a.ld_v = ld_v; a.w = w; a.ld_w = ld_w;
  a.au = au; a.ld_au = ld_au; a.u = u; a.ld_u = ld_u; a.q_scale = q_scale; a.state = state; a.slot_stride = slot_stride;
  a.seg_q_start = seg_q_start; a.seg_slot = seg_slot; a.H = H; a.dk = dk; a.dv = dv;
  const int lpc = cs_lanes_per_column(dk);
  const int cta_cols = CS_WARPS * 32 / lpc;
  const int ctas = (dv + cta_cols - 1) / cta_cols;
  if (ctas > 65535) return QV_ERR_TOO_LARGE;
  dim3 grid(S, H, ctas), block(32 * CS_WARPS);
  cudaStream_t st = (cudaStream_t)stream;
  const bool rem = au != nullptr;
  const int row = (rem ? 5 : 3) * CS_PAD * lpc + cta_cols;
  int chunk = max_q_len < 1 ? 1 : (max_q_len > 16 ? 16 : max_q_len);
  while (chunk > 1 && (size_t)2 * chunk * row * sizeof(float) > 64 * 1024) chunk >>= 1;
  const size_t smem = (size_t)2 * chunk * row * sizeof(float);
  auto aligned = [](const float* p, int ld) { return p == nullptr || (((uintptr_t)p & 15) == 0 && ld % 4 == 0); };
  const bool long_rows = max_q_len >= 16;
  const int vec4 = dk % 4 == 0 && aligned(q, ld_q) && aligned(k, ld_k) && aligned(w, ld_w) && aligned(au, ld_au) && aligned(u, ld_u);
#define CS_LAUNCH(LPC_)                                                                                                  \
  do {                                                                                                                   \
    if (rem) {                                                                                                           \
      cudaFuncSetAttribute(channel_scan_kernel<LPC_, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);     \
      if (long_rows) return cs_launch_after(channel_scan_kernel<LPC_, true>, grid, block, smem, st, a, chunk, vec4);     \
      return qv_launch(channel_scan_kernel<LPC_, true>, grid, block, smem, st, a, chunk, vec4);                          \
    }                                                                                                                    \
    cudaFuncSetAttribute(channel_scan_kernel<LPC_, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);      \
    if (long_rows) return cs_launch_after(channel_scan_kernel<LPC_, false>, grid, block, smem, st, a, chunk, vec4);      \
    return qv_launch(channel_scan_kernel<LPC_, false>, grid, block, smem, st, a, chunk, vec4);                           \
  } while (0)
  if (lpc == 1) CS_LAUNCH(1);
  if (lpc == 2) CS_LAUNCH(2);
  if (lpc == 4) CS_LAUNCH(4);
  if (lpc == 8) CS_LAUNCH(8);
  CS_LAUNCH(16);
#undef CS_LAUNCH
}

// ---------------------------------------------------------------- unit norm per head, weight, gate, factor
// y [T, H * dv] float32 -> out[t, h, i] = y / sqrt(mean_i(y^2) + eps) * w[h * dv + i] * gate(g[t, h * dv + i]) * factor,
// gate 0: sigmoid, 1: SiLU; g float32 (row stride ld_g).  One warp per (token, head); the sum's order follows dv alone.
template <typename T>
__global__ void __launch_bounds__(128) head_norm_gate_kernel(T* __restrict__ out, int ld_out, const float* __restrict__ y, int ld_y,
                                                            const float* __restrict__ g, int ld_g, const float* __restrict__ w, int H,
                                                            int dv, float eps, int gate, float factor) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= H) return;
  const float* yr = y + (size_t)t * ld_y + (size_t)h * dv;
  const float* gr = g + (size_t)t * ld_g + (size_t)h * dv;
  const float* wr = w + (size_t)h * dv;
  T* o = out + (size_t)t * ld_out + (size_t)h * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss = fmaf(yr[i], yr[i], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  for (int i = lane; i < dv; i += 32) {
    const float z = gr[i];
    const float sg = 1.0f / (1.0f + expf(-z));
    const float gv = gate == 1 ? z * sg : sg;
    o[i] = from_f<T>(yr[i] * inv * wr[i] * gv * factor);
  }
}

extern "C" int qv_head_norm_gate(void* out, int ld_out, const float* y, int ld_y, const float* g, int ld_g, const float* w, int T, int H,
                                 int dv, float eps, int gate, float factor, int out_dt, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || dv <= 0 || (gate != 0 && gate != 1)) return QV_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t esz = out_dt == QV_DT_F32 ? 4 : 2;
  for (int done = 0; done < T; done += 65535) {
    const int rows = T - done < 65535 ? T - done : 65535;
    int rc = QV_ERR_UNSUPPORTED;
    QV_DISPATCH_DT(out_dt, TT,
                   rc = qv_launch(head_norm_gate_kernel<TT>, dim3(rows, (H + 3) / 4), dim3(128), 0, st,
                                  (TT*)((char*)out + (size_t)done * ld_out * esz), ld_out, y + (size_t)done * ld_y, ld_y,
                                  g + (size_t)done * ld_g, ld_g, w, H, dv, eps, gate, factor));
    if (rc) return rc;
  }
  return 0;
}
