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
//                     f the identity or tanh.
// qv_unit_keys        u = k / sqrt(sum(k^2) + eps) per head and au = sigmoid(a + bias) * u.
// qv_channel_scan     the recurrence.  The columns of S are independent of one another, so a warp owns C of them, its lanes
//                     owning the rows (row = lane + 32 i): u^T S and S^T q are sums over a warp (shuffles, a fixed order), and
//                     warps never wait for one another.  Only u^T S lies on the chain from token to token; the next token's
//                     vectors are fetched while the present one is worked on.
// qv_head_norm_gate   the unit norm per head (RMS over a head's values) with weight, gate (sigmoid or SiLU, behind the norm)
//                     and a fixed factor that follows a scan.
//
// Everything is float32: the inputs are column slices of float32 products (row strides given), the state, the
// factors and all sums.  The order of every sum depends on the sizes alone, so a token's result does not depend
// on how its request was cut into steps or on what else is in the batch.
#include "common.cuh"

#define GATE_POW_SIGMOID 0
#define GATE_EXP_NEG_SIGMOID 1

// x1 [T, R] (row stride ld_x), W2 [N, R] float32, bias [N] or null -> out [T, N] (row stride ld_out)
__global__ void __launch_bounds__(256) channel_gates_kernel(float* __restrict__ out, int ld_out, const float* __restrict__ x1, int ld_x,
                                                           const float* __restrict__ w2, const float* __restrict__ bias, int N, int R,
                                                           int pre_tanh, int kind, float p) {
  extern __shared__ float xs[];                    // R floats: the token's low-rank row
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int r = threadIdx.x; r < R; r += blockDim.x) {
    const float v = x1[(size_t)t * ld_x + r];
    xs[r] = pre_tanh ? tanhf(v) : v;
  }
  __syncthreads();
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < N; c += gridDim.y * blockDim.x) {
    const float* wr = w2 + (size_t)c * R;
    float z = 0.f;
    for (int r = 0; r < R; ++r) z = fmaf(xs[r], wr[r], z);
    if (bias) z += bias[c];
    float g;
    if (kind == GATE_POW_SIGMOID) {
      const float ls = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));          // log sigmoid(z)
      g = expf(p * ls);
    } else {
      g = expf(-p * (1.0f / (1.0f + expf(-z))));
    }
    out[(size_t)t * ld_out + c] = g;
  }
}

extern "C" int qv_channel_gates(float* out, int ld_out, const float* x1, int ld_x, const float* w2, const float* bias, int T, int N,
                                int R, int pre_tanh, int kind, float p, void* stream) {
  if (T <= 0 || N <= 0) return 0;
  if (R <= 0 || (size_t)R * sizeof(float) > 48 * 1024) return QV_ERR_UNSUPPORTED;
  if (kind != GATE_POW_SIGMOID && kind != GATE_EXP_NEG_SIGMOID) return QV_ERR_UNSUPPORTED;
  const int by = (N + 255) / 256 < 64 ? (N + 255) / 256 : 64;
  cudaStream_t st = (cudaStream_t)stream;
  for (int done = 0; done < T; done += 65535) {
    const int rows = T - done < 65535 ? T - done : 65535;
    const int rc = qv_launch(channel_gates_kernel, dim3(rows, by), dim3(256), (size_t)R * sizeof(float), st,
                             out + (size_t)done * ld_out, ld_out, x1 + (size_t)done * ld_x, ld_x, w2, bias, N, R, pre_tanh, kind, p);
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

// ---------------------------------------------------------------- the scan
#define CS_WARPS 4
#define CS_COLS 4           // value columns a warp owns

struct ChannelScanArgs {
  float* out; int ld_out;                 // [T, H * dv]
  const float* q; int ld_q;               // [T, H * dk] ...
  const float* k; int ld_k;
  const float* v; int ld_v;               // [T, H * dv]
  const float* w; int ld_w;               // decay per key channel
  const float* au; int ld_au;             // removal: a * u and u, or null
  const float* u; int ld_u;
  float q_scale;
  float* state; long long slot_stride;    // per slot: [H][dv][dk]
  const int* seg_q_start; const int* seg_slot;
  int H, dk, dv;
};

template <int RPL, bool REMOVAL>
__global__ void __launch_bounds__(32 * CS_WARPS) channel_scan_kernel(ChannelScanArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  const int s = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int dk = a.dk, dv = a.dv;
  const int col0 = (blockIdx.z * CS_WARPS + warp) * CS_COLS;
  if (col0 >= dv) return;                          // warps are on their own: nothing waits for this one
  const int q0 = a.seg_q_start[s], len = a.seg_q_start[s + 1] - q0;
  float* st = a.state + (size_t)a.seg_slot[s] * a.slot_stride + ((size_t)h * dv + col0) * dk;
  float S[CS_COLS][RPL];
#pragma unroll
  for (int c = 0; c < CS_COLS; ++c)
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      const int r = lane + 32 * i;
      S[c][i] = (r < dk && col0 + c < dv) ? st[(size_t)c * dk + r] : 0.f;
    }
  const size_t hk = (size_t)h * dk, hv = (size_t)h * dv + col0;
  float wn[RPL], kn[RPL], qn[RPL], aun[RPL], un[RPL], vn[CS_COLS];
  auto fetch = [&](int j) {
    const size_t t = (size_t)(q0 + j);
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      const int r = lane + 32 * i;
      const bool ok = r < dk;
      wn[i] = ok ? a.w[t * a.ld_w + hk + r] : 0.f;
      kn[i] = ok ? a.k[t * a.ld_k + hk + r] : 0.f;
      qn[i] = ok ? a.q[t * a.ld_q + hk + r] : 0.f;
      if (REMOVAL) {
        aun[i] = ok ? a.au[t * a.ld_au + hk + r] : 0.f;
        un[i] = ok ? a.u[t * a.ld_u + hk + r] : 0.f;
      }
    }
#pragma unroll
    for (int c = 0; c < CS_COLS; ++c) vn[c] = col0 + c < dv ? a.v[t * a.ld_v + hv + c] : 0.f;
  };
  if (len > 0) fetch(0);
  for (int j = 0; j < len; ++j) {
    float wc[RPL], kc[RPL], qc[RPL], auc[RPL], uc[RPL], vc[CS_COLS];
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      wc[i] = wn[i]; kc[i] = kn[i]; qc[i] = qn[i];
      if (REMOVAL) { auc[i] = aun[i]; uc[i] = un[i]; }
    }
#pragma unroll
    for (int c = 0; c < CS_COLS; ++c) vc[c] = vn[c];
    if (j + 1 < len) fetch(j + 1);
    float d[CS_COLS];
    if (REMOVAL) {
#pragma unroll
      for (int c = 0; c < CS_COLS; ++c) {
        float p = 0.f;
#pragma unroll
        for (int i = 0; i < RPL; ++i) p = fmaf(uc[i], S[c][i], p);
        d[c] = p;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int c = 0; c < CS_COLS; ++c) d[c] += __shfl_xor_sync(0xffffffffu, d[c], o);
    }
    float y[CS_COLS];
#pragma unroll
    for (int c = 0; c < CS_COLS; ++c) {
      float p = 0.f;
#pragma unroll
      for (int i = 0; i < RPL; ++i) {
        float nv = fmaf(kc[i], vc[c], wc[i] * S[c][i]);
        if (REMOVAL) nv = fmaf(-auc[i], d[c], nv);
        S[c][i] = nv;
        p = fmaf(qc[i], nv, p);
      }
      y[c] = p;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int c = 0; c < CS_COLS; ++c) y[c] += __shfl_xor_sync(0xffffffffu, y[c], o);
    float mine = y[0];
#pragma unroll
    for (int c = 1; c < CS_COLS; ++c) if (lane == c) mine = y[c];
    if (lane < CS_COLS && col0 + lane < dv) a.out[(size_t)(q0 + j) * a.ld_out + hv + lane] = mine * a.q_scale;
  }
#pragma unroll
  for (int c = 0; c < CS_COLS; ++c)
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      const int r = lane + 32 * i;
      if (r < dk && col0 + c < dv) st[(size_t)c * dk + r] = S[c][i];
    }
}

extern "C" long long qv_channel_scan_state_floats(int H, int dk, int dv) { return (long long)H * dk * dv; }

extern "C" int qv_channel_scan(float* out, int ld_out, const float* q, int ld_q, const float* k, int ld_k, const float* v, int ld_v,
                               const float* w, int ld_w, const float* au, int ld_au, const float* u, int ld_u, float q_scale,
                               float* state, long long slot_stride, const int* seg_q_start, const int* seg_slot, int S, int H, int dk,
                               int dv, void* stream) {
  if (S <= 0) return 0;
  if (H <= 0 || dk <= 0 || dv <= 0 || H > 65535 || (au == nullptr) != (u == nullptr)) return QV_ERR_UNSUPPORTED;
  if (dk > 256) return QV_ERR_TOO_LARGE;
  ChannelScanArgs a;
  a.out = out; a.ld_out = ld_out; a.q = q; a.ld_q = ld_q; a.k = k; a.ld_k = ld_k; a.v = v; a.ld_v = ld_v; a.w = w; a.ld_w = ld_w;
  a.au = au; a.ld_au = ld_au; a.u = u; a.ld_u = ld_u; a.q_scale = q_scale; a.state = state; a.slot_stride = slot_stride;
  a.seg_q_start = seg_q_start; a.seg_slot = seg_slot; a.H = H; a.dk = dk; a.dv = dv;
  const int per_cta = CS_WARPS * CS_COLS;
  const int tiles = (dv + per_cta - 1) / per_cta;
  if (tiles > 65535) return QV_ERR_TOO_LARGE;
  dim3 grid(S, H, tiles), block(32 * CS_WARPS);
  cudaStream_t st = (cudaStream_t)stream;
  const bool rem = au != nullptr;
#define CS_LAUNCH(RPL)                                                                   \
  do {                                                                                   \
    if (rem) return qv_launch(channel_scan_kernel<RPL, true>, grid, block, 0, st, a);    \
    return qv_launch(channel_scan_kernel<RPL, false>, grid, block, 0, st, a);            \
  } while (0)
  if (dk <= 32) CS_LAUNCH(1);
  if (dk <= 64) CS_LAUNCH(2);
  if (dk <= 128) CS_LAUNCH(4);
  CS_LAUNCH(8);
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
