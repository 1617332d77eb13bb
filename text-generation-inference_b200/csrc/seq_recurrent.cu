// Recurrent mixers with a matrix state per head, carried from token to token in fp32 state slots:
//
//   ssm_scan_kernel   (selective state space, "Mamba-2" form)  S_t = a_t S_(t-1) + dt_t B_t x_t^T ,  y_t = S_t^T C_t + D x_t
//                     a_t = exp(-exp(A_log) dt_t), dt_t = softplus(raw + bias); B / C shared by the heads of a group.
//   mlstm_scan_kernel (matrix memory with exponential gating)  m_t = max(f_t + m_(t-1), i_t),
//                     S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) + e^(i_t - m_t) k_t v_t^T, n_t likewise with k_t alone,
//                     y_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6); i_t = cap tanh(raw/cap), f_t = logsigmoid(cap tanh(raw/cap)).
//   delta_scan_kernel (gated delta rule)  S <- g_t S, u_t = beta_t (v_t - S^T k_t), S <- S + k_t u_t^T, y_t = S^T q_t (the read-out sees the
//                     token's own write); q_t, k_t unit vectors (x / sqrt(sum x^2 + 1e-6)), q_t times q_scale; beta_t = sigmoid(raw),
//                     g_t = exp(-exp(A_log) softplus(raw + dt_bias)); q / k shared by the heads of a group.
//   gdelta_scan_kernel (generalised delta rule)  S <- diag(w_t) S - (a_t * u_t)(u_t^T S) + k_t v_t^T, y_t = S^T r_t with u_t the unit-length
//                     key, a decay w_t = exp(-c sigmoid(.)) and a removal rate a_t = sigmoid(.) per key channel.
//   mingru_scan_kernel / mingru_scan_runs_kernel (minimal gated recurrent unit, a state per channel)  S <- (1 - z_t) S + z_t c_t.
//   causal_conv_silu_kernel / conv_state_update_kernel: short depth-wise causal convolution whose last taps-1 inputs are state.
//
// One block owns (sequence, head, 32 value columns) and walks the sequence's tokens of this step in order, whether they are a
// whole prompt, a portion of one or a single decoded token: the arithmetic per token is the same in every case, so the state
// and the outputs do not depend on how a sequence was cut into steps.  A thread holds a column's state entries for every 8th
// state row in registers; 8 neighbouring lanes reduce the read-out.  A sequence whose first token of the step is at position 0
// starts from a zero state and never reads its (possibly reused) slot.
#include "seq_common.cuh"

namespace b200 {
namespace seq {

constexpr int kScanThreads = 256, kCols = 32, kSplit = 8, kChunk = 16;

__device__ __forceinline__ float group8_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

template <typename TP, int KMAX>
__global__ void __launch_bounds__(kScanThreads) ssm_scan_kernel(
    const float* __restrict__ xbc, int64_t ld_xbc, int col_x, int col_B, int col_C, const float* __restrict__ dt_raw, int64_t ld_dt, int col_dt,
    const TP* __restrict__ dt_bias, const TP* __restrict__ A_log, const TP* __restrict__ Dskip, float* __restrict__ state,
    const int32_t* __restrict__ state_slots, const int32_t* __restrict__ cu_q, const int64_t* __restrict__ position_ids, float* __restrict__ y,
    int64_t ld_y, int H, int P, int N, int heads_per_group) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* Bs = sm;                      // [kChunk][N]
  float* Cs = Bs + kChunk * N;         // [kChunk][N]
  float* xs = Cs + kChunk * N;         // [kChunk][kCols]
  float* ys = xs + kChunk * kCols;     // [kChunk][kCols]
  float* dts = ys + kChunk * kCols;    // [kChunk]
  float* dec = dts + kChunk;           // [kChunk]
  const int b = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * kCols;
  const int g = h / heads_per_group;
  const int col = threadIdx.x / kSplit, ks = threadIdx.x % kSplit;
  const int t_begin = cu_q[b], t_end = cu_q[b + 1];
  if (t_begin >= t_end) return;
  const bool fresh = position_ids[t_begin] == 0;
  float* sp = state + ((int64_t)state_slots[b] * H + h) * N * P;
  float S[KMAX];
  float* stage = dec + kChunk;  // [N][kCols + 1]: the state tile passes through shared memory so that global rows are read whole
  if (!fresh) {
    for (int idx = threadIdx.x; idx < N * kCols; idx += kScanThreads) {
      const int n = idx / kCols, c = idx % kCols;
      stage[n * (kCols + 1) + c] = (v0 + c < P) ? sp[(int64_t)n * P + v0 + c] : 0.f;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < KMAX; ++i) {
    const int n = ks + kSplit * i;
    S[i] = (!fresh && n < N) ? stage[n * (kCols + 1) + col] : 0.f;
  }
  const float bias = ldf(dt_bias + h), A = expf(ldf(A_log + h)), Dh = ldf(Dskip + h);
  for (int t0 = t_begin; t0 < t_end; t0 += kChunk) {
    const int nt = min(kChunk, t_end - t0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * N; idx += kScanThreads) {
      const int tt = idx / N, n = idx % N;
      const float* row = xbc + (int64_t)(t0 + tt) * ld_xbc;
      Bs[tt * N + n] = row[col_B + g * N + n];
      Cs[tt * N + n] = row[col_C + g * N + n];
    }
    for (int idx = threadIdx.x; idx < nt * kCols; idx += kScanThreads) {
      const int tt = idx / kCols, c = idx % kCols;
      xs[idx] = (v0 + c < P) ? xbc[(int64_t)(t0 + tt) * ld_xbc + col_x + h * P + v0 + c] : 0.f;
    }
    if (threadIdx.x < nt) {
      const float d = softplus_f(dt_raw[(int64_t)(t0 + threadIdx.x) * ld_dt + col_dt + h] + bias);
      dts[threadIdx.x] = d;
      dec[threadIdx.x] = expf(-A * d);
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float a = dec[tt], xv = xs[tt * kCols + col];
      const float coef = dts[tt] * xv;
      float part = 0.f;
#pragma unroll
      for (int i = 0; i < KMAX; ++i) {
        const int n = ks + kSplit * i;
        if (n < N) {
          S[i] = fmaf(a, S[i], coef * Bs[tt * N + n]);
          part = fmaf(S[i], Cs[tt * N + n], part);
        }
      }
      part = group8_sum(part);
      if (ks == 0) ys[tt * kCols + col] = part + Dh * xv;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * kCols; idx += kScanThreads) {
      const int tt = idx / kCols, c = idx % kCols;
      if (v0 + c < P) y[(int64_t)(t0 + tt) * ld_y + h * P + v0 + c] = ys[idx];
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < KMAX; ++i) {
    const int n = ks + kSplit * i;
    if (n < N) stage[n * (kCols + 1) + col] = S[i];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < N * kCols; idx += kScanThreads) {
    const int n = idx / kCols, c = idx % kCols;
    if (v0 + c < P) sp[(int64_t)n * P + v0 + c] = stage[n * (kCols + 1) + c];
  }
}

template <typename TP, int KMAX>
__global__ void __launch_bounds__(kScanThreads) mlstm_scan_kernel(
    const float* __restrict__ proj, int64_t ld, int col_q, int col_k, int col_v, int col_i, int col_f, const TP* __restrict__ i_bias,
    const TP* __restrict__ f_bias, float cap, float q_scale, float* __restrict__ S_state, float* __restrict__ n_state, float* __restrict__ m_state,
    const int32_t* __restrict__ state_slots, const int32_t* __restrict__ cu_q, const int64_t* __restrict__ position_ids, float* __restrict__ y,
    int64_t ld_y, int H, int dk, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* qs = sm;                       // [kChunk][dk]
  float* kk = qs + kChunk * dk;         // [kChunk][dk]
  float* vs = kk + kChunk * dk;         // [kChunk][kCols]
  float* ys = vs + kChunk * kCols;      // [kChunk][kCols]
  float* ig = ys + kChunk * kCols;      // [kChunk]
  float* fg = ig + kChunk;              // [kChunk]
  const int b = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * kCols;
  const int col = threadIdx.x / kSplit, ks = threadIdx.x % kSplit;
  const int t_begin = cu_q[b], t_end = cu_q[b + 1];
  if (t_begin >= t_end) return;
  const bool fresh = position_ids[t_begin] == 0;
  const int64_t slot = state_slots[b];
  float* Sp = S_state + (slot * H + h) * dk * dv;
  float* np = n_state + (slot * H + h) * dk;
  float S[KMAX], nn[KMAX];
  float* stage = fg + kChunk;  // [dk][kCols + 1]: the state tile passes through shared memory so that global rows are read whole
  if (!fresh) {
    for (int idx = threadIdx.x; idx < dk * kCols; idx += kScanThreads) {
      const int n = idx / kCols, c = idx % kCols;
      stage[n * (kCols + 1) + c] = (v0 + c < dv) ? Sp[(int64_t)n * dv + v0 + c] : 0.f;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < KMAX; ++i) {
    const int n = ks + kSplit * i;
    S[i] = (!fresh && n < dk) ? stage[n * (kCols + 1) + col] : 0.f;
    nn[i] = (!fresh && n < dk) ? np[n] : 0.f;
  }
  float m = fresh ? 0.f : m_state[slot * H + h];
  const float ib = ldf(i_bias + h), fb = ldf(f_bias + h);
  for (int t0 = t_begin; t0 < t_end; t0 += kChunk) {
    const int nt = min(kChunk, t_end - t0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * dk; idx += kScanThreads) {
      const int tt = idx / dk, n = idx % dk;
      const float* row = proj + (int64_t)(t0 + tt) * ld;
      qs[idx] = row[col_q + h * dk + n] * q_scale;
      kk[idx] = row[col_k + h * dk + n];
    }
    for (int idx = threadIdx.x; idx < nt * kCols; idx += kScanThreads) {
      const int tt = idx / kCols, c = idx % kCols;
      vs[idx] = (v0 + c < dv) ? proj[(int64_t)(t0 + tt) * ld + col_v + h * dv + v0 + c] : 0.f;
    }
    if (threadIdx.x < nt) {
      const float* row = proj + (int64_t)(t0 + threadIdx.x) * ld;
      ig[threadIdx.x] = cap * tanhf((row[col_i + h] + ib) / cap);
      fg[threadIdx.x] = logsigmoid_f(cap * tanhf((row[col_f + h] + fb) / cap));
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float fm = fg[tt] + m;
      const float m_new = fmaxf(fm, ig[tt]);
      const float keep = expf(fm - m_new), take = expf(ig[tt] - m_new);
      m = m_new;
      const float tv = take * vs[tt * kCols + col];
      float num = 0.f, nq = 0.f;
#pragma unroll
      for (int i = 0; i < KMAX; ++i) {
        const int n = ks + kSplit * i;
        if (n < dk) {
          const float kv = kk[tt * dk + n], qv = qs[tt * dk + n];
          S[i] = fmaf(keep, S[i], kv * tv);
          nn[i] = fmaf(keep, nn[i], take * kv);
          num = fmaf(S[i], qv, num);
          nq = fmaf(nn[i], qv, nq);
        }
      }
      num = group8_sum(num);
      nq = group8_sum(nq);
      if (ks == 0) ys[tt * kCols + col] = num / (fmaxf(fabsf(nq), expf(-m)) + 1e-6f);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * kCols; idx += kScanThreads) {
      const int tt = idx / kCols, c = idx % kCols;
      if (v0 + c < dv) y[(int64_t)(t0 + tt) * ld_y + h * dv + v0 + c] = ys[idx];
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < KMAX; ++i) {
    const int n = ks + kSplit * i;
    if (n < dk) {
      stage[n * (kCols + 1) + col] = S[i];
      if (blockIdx.z == 0 && col == 0) np[n] = nn[i];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < dk * kCols; idx += kScanThreads) {
    const int n = idx / kCols, c = idx % kCols;
    if (v0 + c < dv) Sp[(int64_t)n * dv + v0 + c] = stage[n * (kCols + 1) + c];
  }
  if (blockIdx.z == 0 && threadIdx.x == 0) m_state[slot * H + h] = m;
}

// Gated delta rule.  c: the convolved, activated [q | k | v] rows; raw: the rows holding the write-strength and decay projections.
template <typename TP, int KMAX>
__global__ void __launch_bounds__(kScanThreads) delta_scan_kernel(
    const float* __restrict__ c, int64_t ldc, int col_q, int col_k, int col_v, const float* __restrict__ raw, int64_t ldr, int col_b, int col_a,
    const TP* __restrict__ A_log, const TP* __restrict__ dt_bias, float q_scale, float* __restrict__ S_state, const int32_t* __restrict__ state_slots,
    const int32_t* __restrict__ cu_q, const int64_t* __restrict__ position_ids, float* __restrict__ y, int64_t ld_y, int H, int dk, int dv,
    int heads_per_group) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* qs = sm;                       // [kChunk][dk]
  float* kk = qs + kChunk * dk;         // [kChunk][dk]
  float* vs = kk + kChunk * dk;         // [kChunk][kCols]
  float* ys = vs + kChunk * kCols;      // [kChunk][kCols]
  float* bt = ys + kChunk * kCols;      // [kChunk] write strength
  float* dc = bt + kChunk;              // [kChunk] decay
  const int b = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * kCols;
  const int g = h / heads_per_group;
  const int col = threadIdx.x / kSplit, ks = threadIdx.x % kSplit;
  const int t_begin = cu_q[b], t_end = cu_q[b + 1];
  if (t_begin >= t_end) return;
  const bool fresh = position_ids[t_begin] == 0;
  float* Sp = S_state + ((int64_t)state_slots[b] * H + h) * dk * dv;
  float S[KMAX];
  float* stage = dc + kChunk;  // [dk][kCols + 1]
  if (!fresh) {
    for (int idx = threadIdx.x; idx < dk * kCols; idx += kScanThreads) {
      const int n = idx / kCols, cc = idx % kCols;
      stage[n * (kCols + 1) + cc] = (v0 + cc < dv) ? Sp[(int64_t)n * dv + v0 + cc] : 0.f;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < KMAX; ++i) {
    const int n = ks + kSplit * i;
    S[i] = (!fresh && n < dk) ? stage[n * (kCols + 1) + col] : 0.f;
  }
  const float A = expf(ldf(A_log + h)), bias = ldf(dt_bias + h);
  for (int t0 = t_begin; t0 < t_end; t0 += kChunk) {
    const int nt = min(kChunk, t_end - t0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * dk; idx += kScanThreads) {
      const int tt = idx / dk, n = idx % dk;
      const float* row = c + (int64_t)(t0 + tt) * ldc;
      qs[idx] = row[col_q + g * dk + n];
      kk[idx] = row[col_k + g * dk + n];
    }
    for (int idx = threadIdx.x; idx < nt * kCols; idx += kScanThreads) {
      const int tt = idx / kCols, cc = idx % kCols;
      vs[idx] = (v0 + cc < dv) ? c[(int64_t)(t0 + tt) * ldc + col_v + h * dv + v0 + cc] : 0.f;
    }
    if (threadIdx.x < nt) {
      const float* row = raw + (int64_t)(t0 + threadIdx.x) * ldr;
      bt[threadIdx.x] = sigmoid_f(row[col_b + h]);
      dc[threadIdx.x] = expf(-A * softplus_f(row[col_a + h] + bias));
    }
    __syncthreads();
    for (int tt = warp_id(); tt < nt; tt += kScanThreads / 32) {  // unit length, one warp per token
      float sq = 0.f, sk = 0.f;
      for (int n = lane_id(); n < dk; n += 32) {
        sq = fmaf(qs[tt * dk + n], qs[tt * dk + n], sq);
        sk = fmaf(kk[tt * dk + n], kk[tt * dk + n], sk);
      }
      const float rq = q_scale / sqrtf(warp_sum(sq) + 1e-6f), rk = 1.f / sqrtf(warp_sum(sk) + 1e-6f);
      for (int n = lane_id(); n < dk; n += 32) {
        qs[tt * dk + n] *= rq;
        kk[tt * dk + n] *= rk;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float a = dc[tt];
      float pred = 0.f;
#pragma unroll
      for (int i = 0; i < KMAX; ++i) {
        const int n = ks + kSplit * i;
        if (n < dk) {
          S[i] *= a;
          pred = fmaf(S[i], kk[tt * dk + n], pred);
        }
      }
      pred = group8_sum(pred);
      const float u = bt[tt] * (vs[tt * kCols + col] - pred);
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < KMAX; ++i) {
        const int n = ks + kSplit * i;
        if (n < dk) {
          S[i] = fmaf(kk[tt * dk + n], u, S[i]);
          o = fmaf(S[i], qs[tt * dk + n], o);
        }
      }
      o = group8_sum(o);
      if (ks == 0) ys[tt * kCols + col] = o;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * kCols; idx += kScanThreads) {
      const int tt = idx / kCols, cc = idx % kCols;
      if (v0 + cc < dv) y[(int64_t)(t0 + tt) * ld_y + h * dv + v0 + cc] = ys[idx];
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < KMAX; ++i) {
    const int n = ks + kSplit * i;
    if (n < dk) stage[n * (kCols + 1) + col] = S[i];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < dk * kCols; idx += kScanThreads) {
    const int n = idx / kCols, cc = idx % kCols;
    if (v0 + cc < dv) Sp[(int64_t)n * dv + v0 + cc] = stage[n * (kCols + 1) + cc];
  }
}

// Generalised delta rule.  Per head a [dk, dv] memory; every token, with the unit key u = k / sqrt(sum k^2 + 1e-6):
//   S <- diag(w) S - (a * u) (u^T S) + k v^T   (both subtrahend and decay read the old memory),   y = S^T r
// w = exp(-decay_scale * sigmoid(dlogit + w0)) and a = sigmoid(alogit + a_bias) per head and key channel.
// raw: rows holding r, k (H x dk each), v (H x dv) and the removal logits (H x dk); dec: rows holding the decay logits (H x dk).
template <typename TP, int KMAX>
__global__ void __launch_bounds__(kScanThreads, KMAX <= 16 ? 3 : 1) gdelta_scan_kernel(
    const float* __restrict__ raw, int64_t ldr, int col_r, int col_k, int col_v, int col_a, const float* __restrict__ dec, int64_t ldd, int col_d,
    const TP* __restrict__ a_bias, const TP* __restrict__ w0, float decay_scale, float* __restrict__ S_state, const int32_t* __restrict__ state_slots,
    const int32_t* __restrict__ cu_q, const int64_t* __restrict__ position_ids, float* __restrict__ y, int64_t ld_y, int H, int dk, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* rs = sm;                       // [kChunk][dk] read vector
  float* kk = rs + kChunk * dk;         // [kChunk][dk] key
  float* uu = kk + kChunk * dk;         // [kChunk][dk] unit key
  float* au = uu + kChunk * dk;         // [kChunk][dk] removal rate times unit key
  float* ws = au + kChunk * dk;         // [kChunk][dk] decay
  float* vs = ws + kChunk * dk;         // [kChunk][kCols]
  float* ys = vs + kChunk * kCols;      // [kChunk][kCols]
  float* stage = ys + kChunk * kCols;   // [dk][kCols + 1]
  const int b = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * kCols;
  const int col = threadIdx.x / kSplit, ks = threadIdx.x % kSplit;
  const int t_begin = cu_q[b], t_end = cu_q[b + 1];
  if (t_begin >= t_end) return;
  const bool fresh = position_ids[t_begin] == 0;
  float* Sp = S_state + ((int64_t)state_slots[b] * H + h) * dk * dv;
  float S[KMAX];
  if (!fresh) {
    for (int idx = threadIdx.x; idx < dk * kCols; idx += kScanThreads) {
      const int n = idx / kCols, cc = idx % kCols;
      stage[n * (kCols + 1) + cc] = (v0 + cc < dv) ? Sp[(int64_t)n * dv + v0 + cc] : 0.f;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < KMAX; ++i) {
    const int n = ks + kSplit * i;
    S[i] = (!fresh && n < dk) ? stage[n * (kCols + 1) + col] : 0.f;
  }
  for (int t0 = t_begin; t0 < t_end; t0 += kChunk) {
    const int nt = min(kChunk, t_end - t0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * dk; idx += kScanThreads) {
      const int tt = idx / dk, n = idx % dk;
      const float* row = raw + (int64_t)(t0 + tt) * ldr;
      rs[idx] = row[col_r + h * dk + n];
      kk[idx] = row[col_k + h * dk + n];
      au[idx] = sigmoid_f(row[col_a + h * dk + n] + ldf(a_bias + h * dk + n));
      ws[idx] = expf(-decay_scale * sigmoid_f(dec[(int64_t)(t0 + tt) * ldd + col_d + h * dk + n] + ldf(w0 + h * dk + n)));
    }
    for (int idx = threadIdx.x; idx < nt * kCols; idx += kScanThreads) {
      const int tt = idx / kCols, cc = idx % kCols;
      vs[idx] = (v0 + cc < dv) ? raw[(int64_t)(t0 + tt) * ldr + col_v + h * dv + v0 + cc] : 0.f;
    }
    __syncthreads();
    for (int tt = warp_id(); tt < nt; tt += kScanThreads / 32) {  // unit key, one warp per token
      float sk = 0.f;
      for (int n = lane_id(); n < dk; n += 32) sk = fmaf(kk[tt * dk + n], kk[tt * dk + n], sk);
      const float rk = 1.f / sqrtf(warp_sum(sk) + 1e-6f);
      for (int n = lane_id(); n < dk; n += 32) {
        const float u = kk[tt * dk + n] * rk;
        uu[tt * dk + n] = u;
        au[tt * dk + n] *= u;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      float along = 0.f;   // u^T S of this column, from the old memory
#pragma unroll
      for (int i = 0; i < KMAX; ++i) {
        const int n = ks + kSplit * i;
        if (n < dk) along = fmaf(S[i], uu[tt * dk + n], along);
      }
      along = group8_sum(along);
      const float vv = vs[tt * kCols + col];
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < KMAX; ++i) {
        const int n = ks + kSplit * i;
        if (n < dk) {
          S[i] = fmaf(kk[tt * dk + n], vv, fmaf(-au[tt * dk + n], along, ws[tt * dk + n] * S[i]));
          o = fmaf(S[i], rs[tt * dk + n], o);
        }
      }
      o = group8_sum(o);
      if (ks == 0) ys[tt * kCols + col] = o;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * kCols; idx += kScanThreads) {
      const int tt = idx / kCols, cc = idx % kCols;
      if (v0 + cc < dv) y[(int64_t)(t0 + tt) * ld_y + h * dv + v0 + cc] = ys[idx];
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < KMAX; ++i) {
    const int n = ks + kSplit * i;
    if (n < dk) stage[n * (kCols + 1) + col] = S[i];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < dk * kCols; idx += kScanThreads) {
    const int n = idx / kCols, cc = idx % kCols;
    if (v0 + cc < dv) Sp[(int64_t)n * dv + v0 + cc] = stage[n * (kCols + 1) + cc];
  }
}

// Minimal gated recurrent unit: per channel S <- (1 - z) S + z c with z = sigmoid(zlogit + z_bias) and the candidate
// c = x + 1/2 for x >= 0, sigmoid(x) below (x = xlogit + x_bias); out = S * SiLU(gate) * out_scale in the projections' element type.
// One thread per (sequence, channel) walks the sequence's rows of the step in order.
constexpr int kGruThreads = 128;

template <typename TP, typename TO>
__global__ void __launch_bounds__(kGruThreads) mingru_scan_kernel(const float* __restrict__ proj, int64_t ld, int col_z, int col_x, int col_g,
                                                                  const TP* __restrict__ z_bias, const TP* __restrict__ x_bias,
                                                                  float* __restrict__ state, const int32_t* __restrict__ state_slots,
                                                                  const int32_t* __restrict__ cu_q, const int64_t* __restrict__ position_ids,
                                                                  TO* __restrict__ out, int64_t ld_out, float out_scale, int C) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, c = blockIdx.y * kGruThreads + threadIdx.x;
  const int t_begin = cu_q[b], t_end = cu_q[b + 1];
  if (c >= C || t_begin >= t_end) return;
  float* sp = state + (int64_t)state_slots[b] * C + c;
  float S = position_ids[t_begin] == 0 ? 0.f : *sp;
  const float zb = z_bias ? ldf(z_bias + c) : 0.f, xb = x_bias ? ldf(x_bias + c) : 0.f;
#pragma unroll 4
  for (int t = t_begin; t < t_end; ++t) {
    const float* row = proj + (int64_t)t * ld;
    const float z = sigmoid_f(row[col_z + c] + zb), x = row[col_x + c] + xb;
    const float cand = x >= 0.f ? x + 0.5f : sigmoid_f(x);
    S = fmaf(z, cand - S, S);
    stf(out + (int64_t)t * ld_out + c, (col_g >= 0 ? S * silu_f(row[col_g + c]) : S) * out_scale);
  }
  *sp = S;
}

// The same recurrence for steps that bring many rows per sequence.  S_t = a_t S_(t-1) + b_t is linear in S, so a sequence's rows are
// dealt out in NSEG consecutive runs: a block owns (sequence, 32 channels), warp j walks run j from a zero state and leaves the run's
// product of a_t and its end state; after one barrier every warp folds the runs before its own into its true start state and walks
// its run again, writing the results.  Chains are NSEG times shorter than in the one-thread-per-channel form; the results differ
// from it by fp32 rounding only.
template <typename TP, typename TO, int NSEG>
__global__ void __launch_bounds__(32 * NSEG) mingru_scan_runs_kernel(const float* __restrict__ proj, int64_t ld, int col_z, int col_x, int col_g,
                                                                     const TP* __restrict__ z_bias, const TP* __restrict__ x_bias,
                                                                     float* __restrict__ state, const int32_t* __restrict__ state_slots,
                                                                     const int32_t* __restrict__ cu_q, const int64_t* __restrict__ position_ids,
                                                                     TO* __restrict__ out, int64_t ld_out, float out_scale, int C) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[NSEG][32], Bs[NSEG][32];
  const int b = blockIdx.x, lane = threadIdx.x & 31, seg = threadIdx.x >> 5, c = blockIdx.y * 32 + lane;
  const int t_begin = cu_q[b], t_end = cu_q[b + 1];
  if (t_begin >= t_end) return;   // block-uniform
  const bool live = c < C;
  const int per = (t_end - t_begin + NSEG - 1) / NSEG;
  const int t0 = min(t_begin + seg * per, t_end), t1 = min(t0 + per, t_end);
  const float zb = (live && z_bias) ? ldf(z_bias + c) : 0.f, xb = (live && x_bias) ? ldf(x_bias + c) : 0.f;
  float A = 1.f, S = 0.f;
  if (live) {
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
      const float* row = proj + (int64_t)t * ld;
      const float z = sigmoid_f(row[col_z + c] + zb), x = row[col_x + c] + xb;
      const float cand = x >= 0.f ? x + 0.5f : sigmoid_f(x);
      A *= 1.f - z;
      S = fmaf(z, cand - S, S);
    }
  }
  As[seg][lane] = A;
  Bs[seg][lane] = S;
  __syncthreads();
  if (!live) return;
  float* sp = state + (int64_t)state_slots[b] * C + c;
  S = position_ids[t_begin] == 0 ? 0.f : *sp;
  for (int j = 0; j < seg; ++j) S = fmaf(As[j][lane], S, Bs[j][lane]);
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
    const float* row = proj + (int64_t)t * ld;
    const float z = sigmoid_f(row[col_z + c] + zb), x = row[col_x + c] + xb;
    const float cand = x >= 0.f ? x + 0.5f : sigmoid_f(x);
    S = fmaf(z, cand - S, S);
    stf(out + (int64_t)t * ld_out + c, (col_g >= 0 ? S * silu_f(row[col_g + c]) : S) * out_scale);
  }
  if (seg == NSEG - 1) *sp = S;   // the last run ends the sequence's rows (an empty run passes its start state on)
}

constexpr int kMaxTaps = 8;

// out[t, c] = silu(bias[c] + sum_j w[c, j] * in(p - (taps-1) + j)), p the token's position; inputs before this step's first token
// come from the sequence's conv state (positions >= 0) or are zero (before the sequence starts)
template <typename TP, int ACT>  // ACT 0: no activation, 1: SiLU
__global__ void causal_conv_silu_kernel(const float* __restrict__ u, int64_t ld_u, int col0, int C, int taps, const TP* __restrict__ w,
                                        const TP* __restrict__ bias, const float* __restrict__ conv_state, const int32_t* __restrict__ state_slots,
                                        const int32_t* __restrict__ seq_of_token, const int32_t* __restrict__ cu_q,
                                        const int64_t* __restrict__ position_ids, float* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = seq_of_token[t];
  const int row0 = cu_q[b];
  const int64_t s = position_ids[row0], p = position_ids[t];
  const float* st = conv_state + (int64_t)state_slots[b] * (taps - 1) * C;
  float acc = bias ? ldf(bias + c) : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int64_t pp = p - (taps - 1) + j;
    float val = 0.f;
    if (pp >= s) val = u[(row0 + (pp - s)) * ld_u + col0 + c];
    else if (pp >= 0) val = st[(pp - s + taps - 1) * C + c];
    acc = fmaf(ldf(w + (int64_t)c * taps + j), val, acc);
  }
  out[t * C + c] = ACT == 1 ? silu_f(acc) : acc;
}

// after the convolution: the state becomes the last taps-1 inputs of the sequence (older state entries shift when the step
// brought fewer tokens than that)
__global__ void conv_state_update_kernel(const float* __restrict__ u, int64_t ld_u, int col0, int C, int taps, float* __restrict__ conv_state,
                                         const int32_t* __restrict__ state_slots, const int32_t* __restrict__ cu_q,
                                         const int64_t* __restrict__ position_ids) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int row0 = cu_q[b], nq = cu_q[b + 1] - row0;
  if (nq <= 0) return;
  const int64_t s = position_ids[row0], e = s + nq;
  float* st = conv_state + (int64_t)state_slots[b] * (taps - 1) * C;
  float old[kMaxTaps];
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) old[k] = (k < taps - 1 && s > 0) ? st[(int64_t)k * C + c] : 0.f;
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) {
    if (k >= taps - 1) break;
    const int64_t pp = e - (taps - 1) + k;
    float val = 0.f;
    if (pp >= s) val = u[(row0 + (pp - s)) * ld_u + col0 + c];
    else if (pp >= 0) {
      const int idx = (int)(pp - s + taps - 1);
#pragma unroll
      for (int q = 0; q < kMaxTaps; ++q)
        if (q == idx) val = old[q];
    }
    st[(int64_t)k * C + c] = val;
  }
}

}  // namespace seq
}  // namespace b200

using namespace b200::seq;

// act 0: out = convolution (+ bias when given); act 1: SiLU of that
extern "C" int b200_seq_causal_conv(const float* u, int64_t ld_u, int col0, int C, int taps, const void* w, const void* bias, int dt, int act,
                                    float* conv_state, const int32_t* state_slots, const int32_t* seq_of_token, const int32_t* cu_q,
                                    const int64_t* position_ids, float* out, int64_t T, int B, void* stream) {
  if (T == 0) return B200_OK;
  if (taps < 1 || taps > kMaxTaps) { b200_set_last_error("seq_causal_conv: 1 <= taps <= 8"); return B200_ERR_ARG; }
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned cb = (unsigned)((C + 255) / 256);
  if (act == 1)
    B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((causal_conv_silu_kernel<E, 1>), dim3((unsigned)T, cb), dim3(256), 0, st, u, ld_u, col0, C, taps, (const E*)w,
                                         (const E*)bias, (const float*)conv_state, state_slots, seq_of_token, cu_q, position_ids, out));
  else
    B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((causal_conv_silu_kernel<E, 0>), dim3((unsigned)T, cb), dim3(256), 0, st, u, ld_u, col0, C, taps, (const E*)w,
                                         (const E*)bias, (const float*)conv_state, state_slots, seq_of_token, cu_q, position_ids, out));
  if (taps > 1)
    B200_LAUNCH(conv_state_update_kernel, dim3((unsigned)B, cb), dim3(256), 0, st, u, ld_u, col0, C, taps, conv_state, state_slots, cu_q, position_ids);
  b200_count_launches(2);
  return B200_OK;
}

extern "C" int b200_seq_causal_conv_silu(const float* u, int64_t ld_u, int col0, int C, int taps, const void* w, const void* bias, int dt,
                                         float* conv_state, const int32_t* state_slots, const int32_t* seq_of_token, const int32_t* cu_q,
                                         const int64_t* position_ids, float* out, int64_t T, int B, void* stream) {
  return b200_seq_causal_conv(u, ld_u, col0, C, taps, w, bias, dt, 1, conv_state, state_slots, seq_of_token, cu_q, position_ids, out, T, B, stream);
}

template <typename TP, int KMAX>
static int launch_ssm(const float* xbc, int64_t ld_xbc, int col_x, int col_B, int col_C, const float* dt_raw, int64_t ld_dt, int col_dt,
                      const void* dt_bias, const void* A_log, const void* Dskip, float* state, const int32_t* state_slots, const int32_t* cu_q,
                      const int64_t* position_ids, float* y, int64_t ld_y, int B, int H, int P, int N, int hpg, cudaStream_t st) {
  const size_t smem = ((size_t)2 * kChunk * N + 2 * kChunk * kCols + 2 * kChunk + (size_t)N * (kCols + 1)) * 4;
  static bool cfg = false;
  if (!cfg) { cudaFuncSetAttribute(ssm_scan_kernel<TP, KMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); cfg = true; }
  dim3 grid((unsigned)B, (unsigned)H, (unsigned)((P + kCols - 1) / kCols));
  B200_LAUNCH((ssm_scan_kernel<TP, KMAX>), grid, dim3(kScanThreads), smem, st, xbc, ld_xbc, col_x, col_B, col_C, dt_raw, ld_dt, col_dt,
              (const TP*)dt_bias, (const TP*)A_log, (const TP*)Dskip, state, state_slots, cu_q, position_ids, y, ld_y, H, P, N, hpg);
  b200_count_launches(1);
  return B200_OK;
}

extern "C" int b200_seq_ssm_scan(const float* xbc, int64_t ld_xbc, int col_x, int col_B, int col_C, const float* dt_raw, int64_t ld_dt, int col_dt,
                                 const void* dt_bias, const void* A_log, const void* Dskip, int dt, float* state, const int32_t* state_slots,
                                 const int32_t* cu_q, const int64_t* position_ids, float* y, int64_t ld_y, int B, int H, int P, int N, int groups,
                                 void* stream) {
  if (B == 0) return B200_OK;
  if (groups <= 0 || H % groups != 0 || N > 256) { b200_set_last_error("seq_ssm_scan: need heads % groups == 0 and state <= 256"); return B200_ERR_ARG; }
  const int hpg = H / groups;
  cudaStream_t st = (cudaStream_t)stream;
#define SSM(K)                                                                                                                                  \
  B200_SEQ_DISPATCH(dt, E, return (launch_ssm<E, K>(xbc, ld_xbc, col_x, col_B, col_C, dt_raw, ld_dt, col_dt, dt_bias, A_log, Dskip, state, state_slots, \
                                                   cu_q, position_ids, y, ld_y, B, H, P, N, hpg, st)))
  if (N <= 64) SSM(8);
  else if (N <= 128) SSM(16);
  else SSM(32);
#undef SSM
}

template <typename TP, int KMAX>
static int launch_mlstm(const float* proj, int64_t ld, int col_q, int col_k, int col_v, int col_i, int col_f, const void* i_bias, const void* f_bias,
                        float cap, float q_scale, float* S_state, float* n_state, float* m_state, const int32_t* state_slots, const int32_t* cu_q,
                        const int64_t* position_ids, float* y, int64_t ld_y, int B, int H, int dk, int dv, cudaStream_t st) {
  const size_t smem = ((size_t)2 * kChunk * dk + 2 * kChunk * kCols + 2 * kChunk + (size_t)dk * (kCols + 1)) * 4;
  static bool cfg = false;
  if (!cfg) { cudaFuncSetAttribute(mlstm_scan_kernel<TP, KMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); cfg = true; }
  dim3 grid((unsigned)B, (unsigned)H, (unsigned)((dv + kCols - 1) / kCols));
  B200_LAUNCH((mlstm_scan_kernel<TP, KMAX>), grid, dim3(kScanThreads), smem, st, proj, ld, col_q, col_k, col_v, col_i, col_f, (const TP*)i_bias,
              (const TP*)f_bias, cap, q_scale, S_state, n_state, m_state, state_slots, cu_q, position_ids, y, ld_y, H, dk, dv);
  b200_count_launches(1);
  return B200_OK;
}

extern "C" int b200_seq_mlstm_scan(const float* proj, int64_t ld, int col_q, int col_k, int col_v, int col_i, int col_f, const void* i_bias,
                                   const void* f_bias, int dt, float cap, float q_scale, float* S_state, float* n_state, float* m_state,
                                   const int32_t* state_slots, const int32_t* cu_q, const int64_t* position_ids, float* y, int64_t ld_y, int B, int H,
                                   int dk, int dv, void* stream) {
  if (B == 0) return B200_OK;
  if (dk > 256) { b200_set_last_error("seq_mlstm_scan: key size <= 256"); return B200_ERR_ARG; }
  cudaStream_t st = (cudaStream_t)stream;
#define ML(K)                                                                                                                               \
  B200_SEQ_DISPATCH(dt, E, return (launch_mlstm<E, K>(proj, ld, col_q, col_k, col_v, col_i, col_f, i_bias, f_bias, cap, q_scale, S_state, n_state, \
                                                     m_state, state_slots, cu_q, position_ids, y, ld_y, B, H, dk, dv, st)))
  if (dk <= 64) ML(8);
  else if (dk <= 128) ML(16);
  else ML(32);
#undef ML
}

template <typename TP, int KMAX>
static int launch_delta(const float* c, int64_t ldc, int col_q, int col_k, int col_v, const float* raw, int64_t ldr, int col_b, int col_a,
                        const void* A_log, const void* dt_bias, float q_scale, float* S_state, const int32_t* state_slots, const int32_t* cu_q,
                        const int64_t* position_ids, float* y, int64_t ld_y, int B, int H, int dk, int dv, int hpg, cudaStream_t st) {
  const size_t smem = ((size_t)2 * kChunk * dk + 2 * kChunk * kCols + 2 * kChunk + (size_t)dk * (kCols + 1)) * 4;
  static bool cfg = false;
  if (!cfg) { cudaFuncSetAttribute(delta_scan_kernel<TP, KMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); cfg = true; }
  dim3 grid((unsigned)B, (unsigned)H, (unsigned)((dv + kCols - 1) / kCols));
  B200_LAUNCH((delta_scan_kernel<TP, KMAX>), grid, dim3(kScanThreads), smem, st, c, ldc, col_q, col_k, col_v, raw, ldr, col_b, col_a,
              (const TP*)A_log, (const TP*)dt_bias, q_scale, S_state, state_slots, cu_q, position_ids, y, ld_y, H, dk, dv, hpg);
  b200_count_launches(1);
  return B200_OK;
}

// c fp32 [T, ldc]: activated q / k (kv_heads x dk each) and v (H x dv) columns; raw fp32 [T, ldr]: write-strength and decay logits, one per
// head; A_log, dt_bias [H] of element type dt; S_state fp32 [slots, H, dk, dv] advanced in place -> y fp32 [T, H * dv]
extern "C" int b200_seq_delta_scan(const float* c, int64_t ldc, int col_q, int col_k, int col_v, const float* raw, int64_t ldr, int col_b, int col_a,
                                   const void* A_log, const void* dt_bias, int dt, float q_scale, float* S_state, const int32_t* state_slots,
                                   const int32_t* cu_q, const int64_t* position_ids, float* y, int64_t ld_y, int B, int H, int kv_heads, int dk,
                                   int dv, void* stream) {
  if (B == 0) return B200_OK;
  if (kv_heads <= 0 || H % kv_heads != 0 || dk > 256) { b200_set_last_error("seq_delta_scan: need heads % kv_heads == 0 and key size <= 256"); return B200_ERR_ARG; }
  const int hpg = H / kv_heads;
  cudaStream_t st = (cudaStream_t)stream;
#define DL(K)                                                                                                                                  \
  B200_SEQ_DISPATCH(dt, E, return (launch_delta<E, K>(c, ldc, col_q, col_k, col_v, raw, ldr, col_b, col_a, A_log, dt_bias, q_scale, S_state,    \
                                                     state_slots, cu_q, position_ids, y, ld_y, B, H, dk, dv, hpg, st)))
  if (dk <= 64) DL(8);
  else if (dk <= 128) DL(16);
  else DL(32);
#undef DL
}

template <typename TP, int KMAX>
static int launch_gdelta(const float* raw, int64_t ldr, int col_r, int col_k, int col_v, int col_a, const float* dec, int64_t ldd, int col_d,
                         const void* a_bias, const void* w0, float decay_scale, float* S_state, const int32_t* state_slots, const int32_t* cu_q,
                         const int64_t* position_ids, float* y, int64_t ld_y, int B, int H, int dk, int dv, cudaStream_t st) {
  const size_t smem = ((size_t)5 * kChunk * dk + 2 * kChunk * kCols + (size_t)dk * (kCols + 1)) * 4;
  static bool cfg = false;
  if (!cfg) { cudaFuncSetAttribute(gdelta_scan_kernel<TP, KMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); cfg = true; }
  dim3 grid((unsigned)B, (unsigned)H, (unsigned)((dv + kCols - 1) / kCols));
  B200_LAUNCH((gdelta_scan_kernel<TP, KMAX>), grid, dim3(kScanThreads), smem, st, raw, ldr, col_r, col_k, col_v, col_a, dec, ldd, col_d,
              (const TP*)a_bias, (const TP*)w0, decay_scale, S_state, state_slots, cu_q, position_ids, y, ld_y, H, dk, dv);
  b200_count_launches(1);
  return B200_OK;
}

// raw fp32 [T, ldr]: read vectors, keys (H x dk each), values (H x dv) and removal logits (H x dk) at col_r / col_k / col_v / col_a;
// dec fp32 [T, ldd]: decay logits (H x dk) at col_d; a_bias, w0 [H * dk] of element type dt; S_state fp32 [slots, H, dk, dv] advanced
// in place -> y fp32 [T, H * dv]
extern "C" int b200_seq_gdelta_scan(const float* raw, int64_t ldr, int col_r, int col_k, int col_v, int col_a, const float* dec, int64_t ldd,
                                    int col_d, const void* a_bias, const void* w0, int dt, float decay_scale, float* S_state,
                                    const int32_t* state_slots, const int32_t* cu_q, const int64_t* position_ids, float* y, int64_t ld_y, int B,
                                    int H, int dk, int dv, void* stream) {
  if (B == 0) return B200_OK;
  if (dk <= 0 || dk > 256 || dv <= 0) { b200_set_last_error("seq_gdelta_scan: need 0 < key size <= 256"); return B200_ERR_ARG; }
  cudaStream_t st = (cudaStream_t)stream;
#define GD(K)                                                                                                                                \
  B200_SEQ_DISPATCH(dt, E, return (launch_gdelta<E, K>(raw, ldr, col_r, col_k, col_v, col_a, dec, ldd, col_d, a_bias, w0, decay_scale, S_state, \
                                                      state_slots, cu_q, position_ids, y, ld_y, B, H, dk, dv, st)))
  if (dk <= 64) GD(8);
  else if (dk <= 128) GD(16);
  else GD(32);
#undef GD
}

// proj fp32 [T, ld]: update-gate logits, candidate inputs and output-gate logits (C columns each) at col_z / col_x / col_g (col_g < 0:
// no output gate); z_bias, x_bias [C] of element type dt (may be NULL); state fp32 [slots, C] advanced in place -> out [T, ld_out] of
// type out_dt, times out_scale.  T: token rows of the step (steps with many rows per sequence take the kernel that walks runs of rows)
extern "C" int b200_seq_mingru_scan(const float* proj, int64_t ld, int col_z, int col_x, int col_g, const void* z_bias, const void* x_bias, int dt,
                                    float* state, const int32_t* state_slots, const int32_t* cu_q, const int64_t* position_ids, void* out,
                                    int out_dt, int64_t ld_out, float out_scale, int64_t T, int B, int C, void* stream) {
  if (B == 0 || C == 0) return B200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (T >= 8 * (int64_t)B) {   // prompts and portions: a sequence's rows in 16 runs per block of 32 channels
    constexpr int kRuns = 16;
    dim3 grid_r((unsigned)B, (unsigned)((C + 31) / 32));
#define MGR(TO)                                                                                                                              \
  B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((mingru_scan_runs_kernel<E, TO, kRuns>), grid_r, dim3(32 * kRuns), 0, st, proj, ld, col_z, col_x, col_g, \
                                       (const E*)z_bias, (const E*)x_bias, state, state_slots, cu_q, position_ids, (TO*)out, ld_out, out_scale, C))
    if (out_dt == B200_DT_F32) MGR(float);
    else if (out_dt == B200_DT_BF16) MGR(__nv_bfloat16);
    else { b200_set_last_error("unknown element type"); return B200_ERR_ARG; }
#undef MGR
    b200_count_launches(1);
    return B200_OK;
  }
  dim3 grid((unsigned)B, (unsigned)((C + kGruThreads - 1) / kGruThreads));
#define MG(TO)                                                                                                                          \
  B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((mingru_scan_kernel<E, TO>), grid, dim3(kGruThreads), 0, st, proj, ld, col_z, col_x, col_g,      \
                                       (const E*)z_bias, (const E*)x_bias, state, state_slots, cu_q, position_ids, (TO*)out, ld_out, out_scale, C))
  if (out_dt == B200_DT_F32) MG(float);
  else if (out_dt == B200_DT_BF16) MG(__nv_bfloat16);
  else { b200_set_last_error("unknown element type"); return B200_ERR_ARG; }
#undef MG
  b200_count_launches(1);
  return B200_OK;
}
