// Row kernels around an fp32 residual stream: embedding lookup (scaled, or plus a learned position row), layer norm in and out of
// the stream, RMS norm of the stream with an offset weight, RMS norm of a
// column slice, grouped RMS norm with a gate, the clamped gated feed-forward activation, the per-layer token side input, the step
// between two sublayers of a decoder with several residual streams (write all streams, read and norm the next input), plain
// activations, and the turn-back + gate of attention heads whose values carry their position.
// One block per token row; all statistics and the residual sum in fp32.
#include "seq_common.cuh"

namespace b200 {
namespace seq {

constexpr int kRowThreads = 256;

// x[t, :] = table[id[t], :] * scale  (fp32 residual stream)
template <typename T>
__global__ void __launch_bounds__(kRowThreads) embed_scale_kernel(const T* __restrict__ table, const int64_t* __restrict__ ids, float scale,
                                                                  float* __restrict__ out, int W, int64_t V) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t t = blockIdx.x;
  int64_t id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  for (int i = threadIdx.x; i < W; i += kRowThreads) out[t * W + i] = ldf(table + id * W + i) * scale;
}

// x[t, :] = table[id[t], :] + pos_table[position[t], :]  (learned absolute positions; fp32 residual stream)
template <typename T>
__global__ void __launch_bounds__(kRowThreads) embed_add_pos_kernel(const T* __restrict__ table, const T* __restrict__ pos_table,
                                                                    const int64_t* __restrict__ ids, const int64_t* __restrict__ position_ids,
                                                                    float* __restrict__ out, int W, int64_t V, int64_t P) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t t = blockIdx.x;
  int64_t id = ids[t], p = position_ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  p = p < 0 ? 0 : (p >= P ? P - 1 : p);
  for (int i = threadIdx.x; i < W; i += kRowThreads) out[t * W + i] = ldf(table + id * W + i) + ldf(pos_table + p * W + i);
}

// out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * (w + w_offset): RMS norm of the fp32 stream whose weight is stored around -w_offset
// (w_offset 1: "one plus weight"; 0: plain weight)
template <typename TP>
__global__ void __launch_bounds__(kRowThreads) rmsnorm_rows_kernel(const float* __restrict__ x, const TP* __restrict__ w, float w_offset,
                                                                   TP* __restrict__ out, int W, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += kRowThreads) {
    const float v = x[t * W + i];
    q += v * v;
  }
  const float rstd = 1.f / sqrtf(block_sum(q, red) / W + eps);
  for (int i = threadIdx.x; i < W; i += kRowThreads) stf(out + t * W + i, x[t * W + i] * rstd * (ldf(w + i) + w_offset));
}

// mode 0: out[t] = LN(x[t]) * w + b  (x fp32 or T, out T)      mode 1: resid[t] += LN(x[t]) * w + b  (resid fp32)
// In mode 1 `out`, when given, also receives the updated residual row in the activation type (the next projection's input).
template <typename TX, typename TP, typename TO>
__global__ void __launch_bounds__(kRowThreads) layernorm_kernel(const TX* __restrict__ x, const TP* __restrict__ w, const TP* __restrict__ b,
                                                                TO* __restrict__ out, float* __restrict__ resid, int W, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row[];
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += kRowThreads) {
    const float v = ldf(x + t * W + i);
    row[i] = v;
    s += v;
  }
  const float mean = block_sum(s, red) / W;
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += kRowThreads) {
    const float d = row[i] - mean;
    q += d * d;
  }
  const float rstd = 1.f / sqrtf(block_sum(q, red) / W + eps);
  for (int i = threadIdx.x; i < W; i += kRowThreads) {
    const float y = (row[i] - mean) * rstd * ldf(w + i) + ldf(b + i);
    if (resid) {
      const float r = resid[t * W + i] + y;
      resid[t * W + i] = r;
      if (out) stf(out + t * W + i, r);
    } else {
      stf(out + t * W + i, y);
    }
  }
}

// out[t, g*n + i] = gate_after * w[g*n+i] * v / sqrt(mean_i(v^2) + eps), v = x[t, g*n + i] * gate_before, per group g of n
// columns.  gate kinds: 0 none, 1 SiLU(gate) multiplied in before the statistics, 2 sigmoid(gate) multiplied in after the
// weight, 3 SiLU(gate) multiplied in after the weight.  groups == 0: no normalisation (gate only).  x and gate are column slices (leading dimensions given) of fp32 buffers.
template <typename TP, typename TO>
__global__ void __launch_bounds__(kRowThreads) group_rmsnorm_gate_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ gate,
                                                                         int64_t ldg, int gate_kind, const TP* __restrict__ w, int groups, int n,
                                                                         int C, float eps, TO* __restrict__ out, int64_t ldo) {
  // grid (rows, parts): a part is one group of n columns (groups > 0) or a run of n columns of an un-normalised row (groups == 0)
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const int c0 = blockIdx.y * n, c1 = min(C, c0 + n);
  float rstd = 1.f;
  if (groups > 0) {
    float q = 0.f;
    for (int c = c0 + threadIdx.x; c < c1; c += kRowThreads) {
      float v = x[t * ldx + c];
      if (gate_kind == 1) v *= silu_f(gate[t * ldg + c]);
      q += v * v;
    }
    rstd = 1.f / sqrtf(block_sum(q, red) / n + eps);
  }
  for (int c = c0 + threadIdx.x; c < c1; c += kRowThreads) {
    float v = x[t * ldx + c];
    if (gate_kind == 1) v *= silu_f(gate[t * ldg + c]);
    v *= rstd;
    if (w) v *= ldf(w + c);
    if (gate_kind == 2) v *= sigmoid_f(gate[t * ldg + c]);
    else if (gate_kind == 3) v *= silu_f(gate[t * ldg + c]);
    stf(out + t * ldo + c, v);
  }
}

// y = g' * sigmoid(alpha g') * (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit); gu = [g | u] per row
template <typename T>
__global__ void ff_clamped_gate_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t rows, int F, float limit, float alpha) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = rows * F;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / F, c = i % F;
    const float g = fminf(ldf(gu + r * 2 * F + c), limit);
    const float u = fminf(fmaxf(ldf(gu + r * 2 * F + F + c), -limit), limit);
    stf(out + i, g * sigmoid_f(alpha * g) * (u + 1.f));
  }
}

// Per-layer token input, the two row kernels around its projections:  g = gelu_tanh(a) * table[id, col0 : col0 + dim]  (a = Wg x),
// and  resid += y / sqrt(mean(y^2) + eps) * w  (y = Wp g).
template <typename T>
__global__ void side_gate_kernel(const float* __restrict__ a, const int64_t* __restrict__ ids, const T* __restrict__ table, int64_t ld_table,
                                 int64_t col0, int dim, int64_t V, T* __restrict__ out, int64_t rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = rows * dim;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / dim, j = i % dim;
    int64_t id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    stf(out + i, gelu_tanh_f(a[i]) * ldf(table + id * ld_table + col0 + j));
  }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads) rms_add_kernel(const float* __restrict__ y, const T* __restrict__ w, float* __restrict__ resid, int W,
                                                              float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += kRowThreads) {
    const float v = y[t * W + i];
    q += v * v;
  }
  const float rstd = 1.f / sqrtf(block_sum(q, red) / W + eps);
  for (int i = threadIdx.x; i < W; i += kRowThreads) resid[t * W + i] += y[t * W + i] * rstd * ldf(w + i);
}

// resid[t] += v / sqrt(mean(v^2) + eps) * w with v = y[t] * sigmoid(gate[t]) (gate NULL: v = y[t]): a sublayer's result, gated per
// channel, normalised and added to the fp32 stream.  `typed`, when given, also receives the updated row in the projections' type.
template <typename T>
__global__ void __launch_bounds__(kRowThreads) gated_rms_add_kernel(const float* __restrict__ y, const float* __restrict__ gate,
                                                                    const T* __restrict__ w, float* __restrict__ resid, T* __restrict__ typed, int W,
                                                                    float eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row[];
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += kRowThreads) {
    float v = y[t * W + i];
    if (gate) v *= sigmoid_f(gate[t * W + i]);
    row[i] = v;
    q += v * v;
  }
  const float rstd = 1.f / sqrtf(block_sum(q, red) / W + eps);
  for (int i = threadIdx.x; i < W; i += kRowThreads) {
    const float r = resid[t * W + i] + row[i] * rstd * ldf(w + i);
    resid[t * W + i] = r;
    if (typed) stf(typed + t * W + i, r);
  }
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ out, int64_t n) {
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) stf(out + i, x[i]);
}

// out = act(g) * u over rows [g | u]; act 0: SiLU, 1: GELU (tanh form)
template <typename T, int ACT>
__global__ void ff_gate_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t rows, int F) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = rows * F;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / F, c = i % F;
    const float g = ldf(gu + r * 2 * F + c), u = ldf(gu + r * 2 * F + F + c);
    stf(out + i, (ACT == 1 ? gelu_tanh_f(g) : silu_f(g)) * u);
  }
}

// Several residual streams per token ("hyper-connections"): X [T, S, W] fp32.  One launch does what lies between two sublayers:
//   write   (y given)        every stream at once from the old ones, X_t <- sum_s mix[s, t] X_s + out_coef[t] * y
//   read    (in_coef given)  u = sum_s in_coef[s] X_s of the (new) streams; typed <- u / sqrt(mean(u^2) + eps) * w (w NULL: typed <- u)
// `init`, when given, is the row every stream starts from (the embedding output) and X is not read.  One block per token; the
// row of u waits in shared memory between the two passes; S <= kMaxStreams.
constexpr int kMaxStreams = 8;

// VEC consecutive fp32 values in one access (VEC 4: 16 bytes, the pointer 16-byte aligned)
template <int VEC>
__device__ __forceinline__ void ld_vec(const float* p, float (&v)[VEC]) {
  if constexpr (VEC == 4) {
    const float4 f = *reinterpret_cast<const float4*>(p);
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
  } else {
#pragma unroll
    for (int k = 0; k < VEC; ++k) v[k] = p[k];
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void st_vec(T* p, const float (&v)[VEC]) {
  if constexpr (VEC == 4 && sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else if constexpr (VEC == 4 && sizeof(T) == 2) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
  } else {
#pragma unroll
    for (int k = 0; k < VEC; ++k) stf(p + k, v[k]);
  }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(kRowThreads) streams_step_kernel(float* __restrict__ X, int S, const float* __restrict__ init,
                                                                   const float* __restrict__ y, const float* __restrict__ mix,
                                                                   const float* __restrict__ out_coef, const float* __restrict__ in_coef,
                                                                   const T* __restrict__ w, T* __restrict__ typed, int W, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float row[];
  __shared__ float red[32];
  __shared__ float cm[kMaxStreams * kMaxStreams], co[kMaxStreams], ci[kMaxStreams];
  if (threadIdx.x < S * S) cm[threadIdx.x] = mix ? mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    co[threadIdx.x] = out_coef ? out_coef[threadIdx.x] : 0.f;
    ci[threadIdx.x] = in_coef ? in_coef[threadIdx.x] : 0.f;
  }
  __syncthreads();
  const int64_t t = blockIdx.x;
  float* xr = X + t * S * W;
  float q = 0.f;
  for (int i = threadIdx.x * VEC; i < W; i += kRowThreads * VEC) {
    float x[kMaxStreams][VEC];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s)
      if (s < S) ld_vec<VEC>(init ? init + t * W + i : xr + (int64_t)s * W + i, x[s]);
    float u[VEC];   // the read of the new streams, gathered while they are written
#pragma unroll
    for (int k = 0; k < VEC; ++k) u[k] = 0.f;
    if (y) {
      float yv[VEC];
      ld_vec<VEC>(y + t * W + i, yv);
#pragma unroll
      for (int o = 0; o < kMaxStreams; ++o) {
        if (o >= S) break;
        float nx[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) nx[k] = co[o] * yv[k];
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s)
          if (s < S) {
            const float c = cm[s * S + o];
#pragma unroll
            for (int k = 0; k < VEC; ++k) nx[k] = fmaf(c, x[s][k], nx[k]);
          }
        st_vec<float, VEC>(xr + (int64_t)o * W + i, nx);   // every old stream of this column is in registers already
#pragma unroll
        for (int k = 0; k < VEC; ++k) u[k] = fmaf(ci[o], nx[k], u[k]);
      }
    } else {
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s)
        if (s < S) {
          if (init) st_vec<float, VEC>(xr + (int64_t)s * W + i, x[s]);
#pragma unroll
          for (int k = 0; k < VEC; ++k) u[k] = fmaf(ci[s], x[s][k], u[k]);
        }
    }
    if (in_coef) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) q += u[k] * u[k];
      st_vec<float, VEC>(row + i, u);
    }
  }
  if (!in_coef) return;
  const float rstd = w ? 1.f / sqrtf(block_sum(q, red) / W + eps) : 1.f;
  for (int i = threadIdx.x * VEC; i < W; i += kRowThreads * VEC) {   // every thread reads back what it wrote itself
    float u[VEC];
    ld_vec<VEC>(row + i, u);
    if (w) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) u[k] = u[k] * rstd * ldf(w + i + k);
    }
    st_vec<T, VEC>(typed + t * W + i, u);
  }
}

// out = act(in) element by element over rows of F columns (in may be a column slice: leading dimension ld_in);
// act 0: SiLU, 1: GELU (tanh form), 2: tanh.  Evaluated in fp32.
template <typename TI, typename TO, int ACT>
__global__ void ff_act_kernel(const TI* __restrict__ in, int64_t ld_in, TO* __restrict__ out, int64_t rows, int F) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = rows * F;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / F, c = i % F;
    const float z = ldf(in + r * ld_in + c);
    stf(out + i, ACT == 1 ? gelu_tanh_f(z) : (ACT == 2 ? tanhf(z) : silu_f(z)));
  }
}

// Attention heads on their way to the output projection: a [T, H, dv] fp32; every head's first `rot` columns are turned by
// -position (pairs: column i with column i + rot / 2 when `interleaved` is 0, columns 2i and 2i + 1 otherwise; cos / sin
// [positions, rot / 2]), then the head is multiplied by sigmoid(gate[t, h]) (gate NULL: by 1) and by out_scale -> out rows of
// H * dv columns of type T (leading dimension ld_out: the rows may be a column slice of a wider buffer).
template <typename T>
__global__ void __launch_bounds__(kRowThreads) heads_turn_gate_kernel(const float* __restrict__ a, const float* __restrict__ gate, int64_t ld_gate,
                                                                      const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                                                                      int interleaved, const int64_t* __restrict__ position_ids,
                                                                      T* __restrict__ out, int64_t ld_out, float out_scale, int H, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t t = blockIdx.x;
  const int half = rot / 2;
  const float* cs = rot ? cos_t + position_ids[t] * half : nullptr;
  const float* sn = rot ? sin_t + position_ids[t] * half : nullptr;
  const float* row = a + t * H * dv;
  for (int e = threadIdx.x; e < H * dv; e += kRowThreads) {
    const int h = e / dv, i = e % dv;
    float x = row[e];
    if (i < rot) {
      int f, partner;
      bool first;
      if (interleaved) { f = i >> 1; first = (i & 1) == 0; partner = first ? e + 1 : e - 1; }
      else { first = i < half; f = first ? i : i - half; partner = first ? e + half : e - half; }
      const float yv = row[partner];
      // the inverse turn: (u, v) -> (u cos + v sin, v cos - u sin)
      x = first ? x * cs[f] + yv * sn[f] : x * cs[f] - yv * sn[f];
    }
    if (gate) x *= sigmoid_f(gate[t * ld_gate + h]);
    stf(out + t * ld_out + e, x * out_scale);
  }
}

}  // namespace seq
}  // namespace b200

using namespace b200::seq;

extern "C" int b200_seq_embed_scale(const void* table, int dt, const int64_t* ids, float scale, float* out, int64_t T, int64_t W, int64_t V,
                                    void* stream) {
  if (T == 0) return B200_OK;
  B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((embed_scale_kernel<E>), dim3((unsigned)T), dim3(kRowThreads), 0, (cudaStream_t)stream, (const E*)table, ids,
                                       scale, out, (int)W, V));
  b200_count_launches(1);
  return B200_OK;
}

extern "C" int b200_seq_embed_add_pos(const void* table, const void* pos_table, int dt, const int64_t* ids, const int64_t* position_ids,
                                      float* out, int64_t T, int64_t W, int64_t V, int64_t P, void* stream) {
  if (T == 0) return B200_OK;
  B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((embed_add_pos_kernel<E>), dim3((unsigned)T), dim3(kRowThreads), 0, (cudaStream_t)stream, (const E*)table,
                                       (const E*)pos_table, ids, position_ids, out, (int)W, V, P));
  b200_count_launches(1);
  return B200_OK;
}

extern "C" int b200_seq_rmsnorm_rows(const float* x, const void* w, int dt, float w_offset, void* out, int64_t T, int64_t W, float eps,
                                     void* stream) {
  if (T == 0) return B200_OK;
  B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((rmsnorm_rows_kernel<E>), dim3((unsigned)T), dim3(kRowThreads), 0, (cudaStream_t)stream, x, (const E*)w,
                                       w_offset, (E*)out, (int)W, eps));
  b200_count_launches(1);
  return B200_OK;
}

// x_dt: element type of x (fp32 stream or an activation of type dt).  resid == nullptr: out (type dt) = LN(x); else resid += LN(x).
extern "C" int b200_seq_layernorm(const void* x, int x_dt, const void* w, const void* b, int dt, void* out, float* resid, int64_t T, int64_t W,
                                  float eps, void* stream) {
  if (T == 0) return B200_OK;
  if (W * 4 > 160 * 1024) { b200_set_last_error("seq_layernorm: row too wide"); return B200_ERR_ARG; }
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)W * 4;
#define LN_LAUNCH(TX, TP)                                                                                                              \
  do {                                                                                                                                 \
    static bool cfg = false;                                                                                                           \
    if (!cfg) { cudaFuncSetAttribute(layernorm_kernel<TX, TP, TP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); cfg = true; } \
    B200_LAUNCH((layernorm_kernel<TX, TP, TP>), dim3((unsigned)T), dim3(kRowThreads), smem, st, (const TX*)x, (const TP*)w, (const TP*)b,   \
                (TP*)out, resid, (int)W, eps);                                                                                         \
  } while (0)
  if (dt == B200_DT_F32 && x_dt == B200_DT_F32) LN_LAUNCH(float, float);
  else if (dt == B200_DT_BF16 && x_dt == B200_DT_F32) LN_LAUNCH(float, __nv_bfloat16);
  else if (dt == B200_DT_BF16 && x_dt == B200_DT_BF16) LN_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else { b200_set_last_error("seq_layernorm: unsupported element types"); return B200_ERR_UNSUPPORTED; }
#undef LN_LAUNCH
  b200_count_launches(1);
  return B200_OK;
}

extern "C" int b200_seq_group_rmsnorm_gate(const float* x, int64_t ldx, const float* gate, int64_t ldg, int gate_kind, const void* w, int w_dt,
                                           int groups, int n, float eps, void* out, int out_dt, int64_t ldo, int64_t T, void* stream) {
  if (T == 0) return B200_OK;
  if (gate_kind != 0 && gate == nullptr) { b200_set_last_error("seq_group_rmsnorm_gate: gate missing"); return B200_ERR_ARG; }
  cudaStream_t st = (cudaStream_t)stream;
  const int C = groups > 0 ? groups * n : n;
  const int part = groups > 0 ? n : 2048;
  const dim3 grid((unsigned)T, (unsigned)((C + part - 1) / part));
#define GN_LAUNCH(TP, TO)                                                                                                                   \
  B200_LAUNCH((group_rmsnorm_gate_kernel<TP, TO>), grid, dim3(kRowThreads), 0, st, x, ldx, gate, ldg, gate_kind, (const TP*)w, groups, part, \
              C, eps, (TO*)out, ldo)
  if (w_dt == B200_DT_F32 && out_dt == B200_DT_F32) GN_LAUNCH(float, float);
  else if (w_dt == B200_DT_BF16 && out_dt == B200_DT_BF16) GN_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (w_dt == B200_DT_BF16 && out_dt == B200_DT_F32) GN_LAUNCH(__nv_bfloat16, float);
  else { b200_set_last_error("seq_group_rmsnorm_gate: unsupported element types"); return B200_ERR_UNSUPPORTED; }
#undef GN_LAUNCH
  b200_count_launches(1);
  return B200_OK;
}

extern "C" int b200_seq_ff_clamped_gate(const void* gu, void* out, int dt, int64_t rows, int64_t F, float limit, float alpha, void* stream) {
  if (rows == 0 || F == 0) return B200_OK;
  int64_t blocks = (rows * F + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((ff_clamped_gate_kernel<E>), dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const E*)gu, (E*)out,
                                       rows, (int)F, limit, alpha));
  b200_count_launches(1);
  return B200_OK;
}

extern "C" int b200_seq_side_gate(const float* a, const int64_t* ids, const void* table, int64_t ld_table, int64_t col0, int dim, int64_t V,
                                  void* out, int dt, int64_t rows, void* stream) {
  if (rows == 0 || dim == 0) return B200_OK;
  int64_t blocks = (rows * dim + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((side_gate_kernel<E>), dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, a, ids, (const E*)table,
                                       ld_table, col0, dim, V, (E*)out, rows));
  b200_count_launches(1);
  return B200_OK;
}

extern "C" int b200_seq_rms_add(const float* y, const void* w, int dt, float* resid, int64_t T, int64_t W, float eps, void* stream) {
  if (T == 0) return B200_OK;
  B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((rms_add_kernel<E>), dim3((unsigned)T), dim3(kRowThreads), 0, (cudaStream_t)stream, y, (const E*)w, resid,
                                       (int)W, eps));
  b200_count_launches(1);
  return B200_OK;
}

extern "C" int b200_seq_gated_rms_add(const float* y, const float* gate, const void* w, int dt, float* resid, void* typed, int64_t T, int64_t W,
                                      float eps, void* stream) {
  if (T == 0) return B200_OK;
  if (W * 4 > 160 * 1024) { b200_set_last_error("seq_gated_rms_add: row too wide"); return B200_ERR_ARG; }
#define GRA(E)                                                                                                                          \
  do {                                                                                                                                  \
    static bool cfg = false;                                                                                                            \
    if (!cfg) { cudaFuncSetAttribute(gated_rms_add_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); cfg = true; }   \
    B200_LAUNCH((gated_rms_add_kernel<E>), dim3((unsigned)T), dim3(kRowThreads), (size_t)W * 4, (cudaStream_t)stream, y, gate, (const E*)w, \
                resid, (E*)typed, (int)W, eps);                                                                                         \
  } while (0)
  if (dt == B200_DT_F32) GRA(float);
  else if (dt == B200_DT_BF16) GRA(__nv_bfloat16);
  else { b200_set_last_error("unknown element type"); return B200_ERR_ARG; }
#undef GRA
  b200_count_launches(1);
  return B200_OK;
}

extern "C" int b200_seq_cast_rows(const float* x, void* out, int dt, int64_t n, void* stream) {
  if (n == 0) return B200_OK;
  int64_t blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((cast_rows_kernel<E>), dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, x, (E*)out, n));
  b200_count_launches(1);
  return B200_OK;
}

// act 0: SiLU(g) * u, 1: GELU_tanh(g) * u
extern "C" int b200_seq_ff_gate(const void* gu, void* out, int dt, int64_t rows, int64_t F, int act, void* stream) {
  if (rows == 0 || F == 0) return B200_OK;
  int64_t blocks = (rows * F + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (act == 1)
    B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((ff_gate_kernel<E, 1>), dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const E*)gu, (E*)out,
                                         rows, (int)F));
  else
    B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((ff_gate_kernel<E, 0>), dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const E*)gu, (E*)out,
                                         rows, (int)F));
  b200_count_launches(1);
  return B200_OK;
}

// X fp32 [T, S, W] in place (S <= 8).  init fp32 [T, W] or NULL; y fp32 [T, W] or NULL (with mix fp32 [S, S] indexed [from, to] and
// out_coef fp32 [S]); in_coef fp32 [S] or NULL (with typed [T, W] of type dt and, optionally, the norm weight w of type dt).
extern "C" int b200_seq_streams_step(float* X, int S, const float* init, const float* y, const float* mix, const float* out_coef,
                                     const float* in_coef, const void* w, int dt, void* typed, int64_t T, int64_t W, float eps, void* stream) {
  if (T == 0) return B200_OK;
  if (S < 1 || S > kMaxStreams || (y && (!mix || !out_coef)) || (in_coef && !typed) || W > 40000) {
    b200_set_last_error("seq_streams_step: 1 <= streams <= 8; a write needs mix and out_coef, a read needs an output");
    return B200_ERR_ARG;
  }
#define SST(E, V)                                                                                                                        \
  do {                                                                                                                                   \
    static bool cfg = false;                                                                                                             \
    if (!cfg) { cudaFuncSetAttribute(streams_step_kernel<E, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); cfg = true; }  \
    B200_LAUNCH((streams_step_kernel<E, V>), dim3((unsigned)T), dim3(kRowThreads), (size_t)W * 4, (cudaStream_t)stream, X, S, init, y, mix, \
                out_coef, in_coef, (const E*)w, (E*)typed, (int)W, eps);                                                                 \
  } while (0)
  // 16-byte accesses when every row starts on a 16-byte boundary
  const bool vec = W % 4 == 0 && ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(init) | reinterpret_cast<uintptr_t>(y) |
                                   reinterpret_cast<uintptr_t>(typed)) & 15) == 0;
  if (dt == B200_DT_F32) { if (vec) SST(float, 4); else SST(float, 1); }
  else if (dt == B200_DT_BF16) { if (vec) SST(__nv_bfloat16, 4); else SST(__nv_bfloat16, 1); }
  else { b200_set_last_error("unknown element type"); return B200_ERR_ARG; }
#undef SST
  b200_count_launches(1);
  return B200_OK;
}

// in: rows of type in_dt (leading dimension ld_in), out: dense rows of type out_dt; act 0 SiLU, 1 GELU (tanh form), 2 tanh
extern "C" int b200_seq_ff_act(const void* in, int in_dt, int64_t ld_in, void* out, int out_dt, int64_t rows, int64_t F, int act, void* stream) {
  if (rows == 0 || F == 0) return B200_OK;
  int64_t blocks = (rows * F + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (act < 0 || act > 2) { b200_set_last_error("seq_ff_act: unknown activation"); return B200_ERR_ARG; }
#define FA(TI, TO, A) B200_LAUNCH((ff_act_kernel<TI, TO, A>), dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const TI*)in, ld_in, (TO*)out, rows, (int)F)
#define FA_ACT(TI, TO)            \
  do {                            \
    if (act == 0) FA(TI, TO, 0);  \
    else if (act == 1) FA(TI, TO, 1); \
    else FA(TI, TO, 2);           \
  } while (0)
  if (in_dt == B200_DT_F32 && out_dt == B200_DT_F32) FA_ACT(float, float);
  else if (in_dt == B200_DT_F32 && out_dt == B200_DT_BF16) FA_ACT(float, __nv_bfloat16);
  else if (in_dt == B200_DT_BF16 && out_dt == B200_DT_BF16) FA_ACT(__nv_bfloat16, __nv_bfloat16);
  else { b200_set_last_error("seq_ff_act: element types must be fp32 -> any or bf16 -> bf16"); return B200_ERR_ARG; }
#undef FA_ACT
#undef FA
  b200_count_launches(1);
  return B200_OK;
}

// a fp32 [T, H, dv]; gate fp32 rows (leading dimension ld_gate, one logit per head) or NULL; cos / sin fp32 [positions, rot / 2]
// (rot 0: no turn) -> out [T, ld_out] of type dt, H * dv columns written, times out_scale
extern "C" int b200_seq_heads_turn_gate(const float* a, const float* gate, int64_t ld_gate, const float* cos_t, const float* sin_t, int rot,
                                        int interleaved, const int64_t* position_ids, void* out, int dt, int64_t ld_out, float out_scale,
                                        int64_t T, int H, int dv, void* stream) {
  if (T == 0) return B200_OK;
  if (rot < 0 || rot > dv || rot % 2 != 0 || (rot > 0 && (!cos_t || !sin_t || !position_ids))) {
    b200_set_last_error("seq_heads_turn_gate: turned columns must be even, at most the head size, with tables and positions");
    return B200_ERR_ARG;
  }
  B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((heads_turn_gate_kernel<E>), dim3((unsigned)T), dim3(kRowThreads), 0, (cudaStream_t)stream, a, gate, ld_gate,
                                       cos_t, sin_t, rot, interleaved, position_ids, (E*)out, ld_out, out_scale, H, dv));
  b200_count_launches(1);
  return B200_OK;
}
