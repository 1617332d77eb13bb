// Routed feed-forward (mixture of experts): every token picks `top` experts and weighs them, by one of two rules:
//   mode 0  the largest router logits; weights = soft-max over the picked logits only;
//   mode 1  scores s = sigmoid(logit); the largest s + correction[expert] are picked, the weights are the picked plain scores
//           divided by their sum (+ 1e-20), times a constant.
//
//   moe_route_kernel   : one warp per token: top-k of the fp32 logits (ties: the lower expert), weights, and the token's place in
//                        each picked expert's list (an atomic counter per expert; the order inside a list changes no result).
//   moe_plan_kernel    : lists -> one compact row order (expert by expert) cut into tiles of 64 rows that never span two
//                        experts; row <-> (token, pick) maps in both directions.
//   moe_linear_kernel  : C[row] = W[expert of row's tile] A[row] over that plan; A rows are either the compact rows or gathered
//                        through the row -> token map.  fp32 accumulation in ascending k: a row's result does not depend on what
//                        else the step holds.
//   moe_linear_mma_kernel : the same product on tensor cores for bfloat16 operands (see the note above the kernel).
//   moe_combine_add_kernel : resid[t] += mix[t] + sum over the token's picks, in pick order, of weight * y[row(t, pick)].
//
// Plan workspace (int32): [counts E][offsets E + 1][n_tiles 1][tile_expert max_tiles][tile_row0 max_tiles][place R][row_of R]
// [token_of_row R] with R = T * top and max_tiles = ceil(R / 64) + E.
#include "seq_common.cuh"

#include <cstdlib>

namespace b200 {
namespace seq {

constexpr int kMoeTile = 64, kMoeStep = 16, kMaxTop = 16, kMaxExpertsPerLane = 8;

struct MoePlan {
  int32_t *counts, *offsets, *n_tiles, *tile_expert, *tile_row0, *place, *row_of, *token_of_row;
  int64_t max_tiles;
};

__host__ __device__ inline int64_t moe_max_tiles(int64_t T, int E, int top) { return (T * top + kMoeTile - 1) / kMoeTile + E; }

__host__ __device__ inline MoePlan moe_plan_view(int32_t* base, int64_t T, int E, int top) {
  MoePlan p;
  const int64_t R = T * top;
  p.max_tiles = moe_max_tiles(T, E, top);
  p.counts = base;
  p.offsets = p.counts + E;
  p.n_tiles = p.offsets + E + 1;
  p.tile_expert = p.n_tiles + 1;
  p.tile_row0 = p.tile_expert + p.max_tiles;
  p.place = p.tile_row0 + p.max_tiles;
  p.row_of = p.place + R;
  p.token_of_row = p.row_of + R;
  return p;
}

template <int MODE>
__global__ void __launch_bounds__(256) moe_route_kernel(const float* __restrict__ logits, int64_t T, int E, int top, int32_t* __restrict__ ids,
                                                        float* __restrict__ weights, int32_t* __restrict__ counts, int32_t* __restrict__ place,
                                                        const void* __restrict__ correction, int corr_dt, float weight_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t t = (int64_t)blockIdx.x * 8 + warp_id();
  if (t >= T) return;
  const int lane = lane_id();
  float z[kMaxExpertsPerLane], sc[kMaxExpertsPerLane];
#pragma unroll
  for (int i = 0; i < kMaxExpertsPerLane; ++i) {
    const int e = lane + 32 * i;
    z[i] = e < E ? logits[t * E + e] : -INFINITY;
    sc[i] = 0.f;
    if (MODE == 1 && e < E) {
      sc[i] = sigmoid_f(z[i]);
      z[i] = sc[i] + (correction ? ld_any(correction, e, corr_dt) : 0.f);
    }
  }
  float val[kMaxTop];
  int idx[kMaxTop];
#pragma unroll
  for (int k = 0; k < kMaxTop; ++k) {
    if (k >= top) break;
    float best = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      if (e < E && (z[i] > best || (z[i] == best && e < be))) { best = z[i]; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > best || (ov == best && oe < be)) { best = ov; be = oe; }
    }
    if (MODE == 1) {  // the weight uses the plain score of the pick, which its owning lane holds
      float mine = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxExpertsPerLane; ++i)
        if (lane + 32 * i == be) mine = sc[i];
      best = __shfl_sync(0xffffffffu, mine, be & 31);
    }
    val[k] = best;
    idx[k] = be;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i)
      if (lane + 32 * i == be) z[i] = -INFINITY;
  }
  if (lane == 0) {
    float den = 0.f, w[kMaxTop];
#pragma unroll
    for (int k = 0; k < kMaxTop; ++k) {
      if (k >= top) break;
      w[k] = MODE == 1 ? val[k] : expf(val[k] - val[0]);  // mode 0: val[0] is the largest
      den += w[k];
    }
    const float norm = MODE == 1 ? weight_scale / (den + 1e-20f) : 1.f / den;
#pragma unroll
    for (int k = 0; k < kMaxTop; ++k) {
      if (k >= top) break;
      ids[t * top + k] = idx[k];
      weights[t * top + k] = w[k] * norm;
      place[t * top + k] = atomicAdd(counts + idx[k], 1);
    }
  }
}

__global__ void __launch_bounds__(256) moe_plan_kernel(const int32_t* __restrict__ ids, int64_t R, int top, int E, MoePlan p) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      p.offsets[e] = off;
      const int c = p.counts[e];
      for (int r = 0; r < c; r += kMoeTile) {
        p.tile_expert[nt] = e;
        p.tile_row0[nt] = off + r;
        ++nt;
      }
      off += c;
    }
    p.offsets[E] = off;
    *p.n_tiles = nt;
  }
  __syncthreads();
  for (int64_t i = threadIdx.x; i < R; i += blockDim.x) {
    const int row = p.offsets[ids[i]] + p.place[i];
    p.row_of[i] = row;
    p.token_of_row[row] = (int32_t)(i / top);
  }
}

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) moe_linear_kernel(const TA* __restrict__ A, int64_t lda, int gather, const TW* __restrict__ W,
                                                         TC* __restrict__ C, int64_t ldc, MoePlan p, int N, int K) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[kMoeStep][kMoeTile + 4];
  __shared__ float Ws[kMoeStep][kMoeTile + 4];
  __shared__ int64_t a_row[kMoeTile];
  const int tile = blockIdx.y;
  if (tile >= *p.n_tiles) return;
  const int e = p.tile_expert[tile], m0 = p.tile_row0[tile], m_end = p.offsets[e + 1];
  W += (int64_t)e * N * K;
  const int n0 = blockIdx.x * kMoeTile;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  if (tid < kMoeTile) {
    const int m = m0 + tid;
    a_row[tid] = m < m_end ? (gather ? (int64_t)p.token_of_row[m] : (int64_t)m) : -1;
  }
  __syncthreads();
  float acc[4][4] = {};
  const int64_t ar = a_row[lr];
  for (int k0 = 0; k0 < K; k0 += kMoeStep) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      const int n = n0 + lr;
      As[lk + i][lr] = (ar >= 0 && k < K) ? ldf(A + ar * lda + k) : 0.f;
      Ws[lk + i][lr] = (n < N && k < K) ? ldf(W + (int64_t)n * K + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kMoeStep; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = As[k][ty * 4 + i];
        w[i] = Ws[k][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= m_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) stf(C + (int64_t)m * ldc + n, acc[i][j]);
    }
  }
}

// Tensor-core form of moe_linear_kernel for bfloat16 operands: 64 x 64 output tile per block of four warps (each 32 x 32), k in
// steps of 64 through a three-stage cp.async pipeline, m16n8k16 products with fp32 accumulation in ascending k.  With the few
// rows per expert of a decoding step the work is streaming each picked expert's weights once; the tiles of the plan keep that
// to the experts that were picked.  Needs K % 8 == 0 and 16-byte aligned rows.
constexpr int kMmaBK = 64, kMmaStages = 3, kMmaLd = kMmaBK + 8;

template <typename TC>
__global__ void __launch_bounds__(128) moe_linear_mma_kernel(const __nv_bfloat16* __restrict__ A, int64_t lda, int gather,
                                                             const __nv_bfloat16* __restrict__ W, TC* __restrict__ C, int64_t ldc, MoePlan p, int N,
                                                             int K) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char moe_smem[];
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(moe_smem);      // [stages][64][kMmaLd]
  __nv_bfloat16* Ws = As + kMmaStages * kMoeTile * kMmaLd;             // [stages][64][kMmaLd]
  const int tile = blockIdx.y;
  if (tile >= *p.n_tiles) return;
  const int e = p.tile_expert[tile], m0 = p.tile_row0[tile], m_end = p.offsets[e + 1];
  W += (int64_t)e * N * K;
  const int n0 = blockIdx.x * kMoeTile;
  const int tid = threadIdx.x, w = warp_id(), lane = lane_id();
  // loader: chunk c = tid + 128 i covers row c / 8, k offset (c % 8) * 8 of the 64 x 64 tile
  const int kc = (tid & 7) * 8;
  const __nv_bfloat16* a_src[4];
  const __nv_bfloat16* w_src[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = (tid >> 3) + i * 16;
    const int m = m0 + row, n = n0 + row;
    a_src[i] = m < m_end ? A + (gather ? (int64_t)p.token_of_row[m] : (int64_t)m) * lda : nullptr;
    w_src[i] = n < N ? W + (int64_t)n * K : nullptr;
  }
  auto load = [&](int stage, int kt) {
    const int k = kt * kMmaBK + kc;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = (tid >> 3) + i * 16;
      const bool pa = a_src[i] != nullptr && k < K, pw = w_src[i] != nullptr && k < K;
      cp_async_16(As + (stage * kMoeTile + row) * kMmaLd + kc, pa ? a_src[i] + k : A, pa);
      cp_async_16(Ws + (stage * kMoeTile + row) * kMmaLd + kc, pw ? w_src[i] + k : W, pw);
    }
    cp_async_commit();
  };
  const int nk = (K + kMmaBK - 1) / kMmaBK;
  load(0, 0);
  if (nk > 1) load(1, 1);
  float acc[2][4][4] = {};
  const int wm = w >> 1, wn = w & 1, lm = lane >> 3, lr = lane & 7;
  const uint32_t as_addr = smem_u32(As), ws_addr = smem_u32(Ws);
  for (int kt = 0; kt < nk; ++kt) {
    const int stage = kt % kMmaStages;
    if (kt + 1 < nk) cp_async_wait<1>();
    else cp_async_wait<0>();
    __syncthreads();  // stage kt has landed; everyone is done with the stage that the next load overwrites
    if (kt + 2 < nk) load((kt + 2) % kMmaStages, kt + 2);
    const uint32_t a_lane = as_addr + (uint32_t)(((stage * kMoeTile + wm * 32 + (lm & 1) * 8 + lr) * kMmaLd + (lm >> 1) * 8) * 2);
    const uint32_t b_lane = ws_addr + (uint32_t)(((stage * kMoeTile + wn * 32 + (lm >> 1) * 8 + lr) * kMmaLd + (lm & 1) * 8) * 2);
#pragma unroll
    for (int kk = 0; kk < kMmaBK; kk += 16) {
      uint32_t a[2][4], b[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) ldmatrix_x4(a[mt][0], a[mt][1], a[mt][2], a[mt][3], a_lane + (uint32_t)((mt * 16 * kMmaLd + kk) * 2));
#pragma unroll
      for (int np = 0; np < 2; ++np) ldmatrix_x4(b[np][0], b[np][1], b[np][2], b[np][3], b_lane + (uint32_t)((np * 16 * kMmaLd + kk) * 2));
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          mma_m16n8k16_bf16f32(acc[mt][2 * np], a[mt], b[np][0], b[np][1]);
          mma_m16n8k16_bf16f32(acc[mt][2 * np + 1], a[mt], b[np][2], b[np][3]);
        }
    }
  }
  const int cq = (lane & 3) * 2;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int el = 0; el < 4; ++el) {
        const int m = m0 + wm * 32 + mt * 16 + (lane >> 2) + (el >> 1) * 8;
        const int n = n0 + wn * 32 + nt * 8 + cq + (el & 1);
        if (m < m_end && n < N) stf(C + (int64_t)m * ldc + n, acc[mt][nt][el]);
      }
}

// out[row] = A[token(row)] for the compact rows of the plan (what a dense product per expert reads)
template <typename T>
__global__ void __launch_bounds__(256) moe_gather_rows_kernel(const T* __restrict__ A, int64_t lda, T* __restrict__ out, const int32_t* __restrict__ token_of_row,
                                                              int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const T* src = A + (int64_t)token_of_row[row] * lda;
  for (int i = threadIdx.x; i < K; i += 256) out[row * K + i] = src[i];
}

// top == 0 (or y == nullptr): resid += mix only
__global__ void __launch_bounds__(256) moe_combine_add_kernel(float* __restrict__ resid, const float* __restrict__ mix, const float* __restrict__ y,
                                                              int64_t ldy, const float* __restrict__ weights, const int32_t* __restrict__ row_of,
                                                              int top, int W) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t t = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += 256) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) acc = fmaf(weights[t * top + k], y[(int64_t)row_of[t * top + k] * ldy + i], acc);
    resid[t * W + i] += (mix ? mix[t * W + i] : 0.f) + acc;
  }
}

}  // namespace seq
}  // namespace b200

using namespace b200::seq;

extern "C" int64_t b200_seq_moe_plan_ints(int64_t T, int E, int top) {
  return (int64_t)E + E + 1 + 1 + 2 * moe_max_tiles(T, E, top) + 3 * T * top;
}

// logits fp32 [T, E] -> ids int32 [T, top], weights fp32 [T, top] and the plan (b200_seq_moe_plan_ints int32 values)
// mode 0: soft-max over the picked logits (correction, weight_scale unused); mode 1: sigmoid scores, picks by score + correction
// (element type corr_dt, may be NULL), weights = score / sum of the picked scores * weight_scale
extern "C" int b200_seq_moe_route_scored(const float* logits, int64_t T, int E, int top, int mode, const void* correction, int corr_dt,
                                         float weight_scale, int32_t* ids, float* weights, int32_t* plan, void* stream) {
  if (T == 0) return B200_OK;
  if (E < 1 || E > 32 * kMaxExpertsPerLane || top < 1 || top > kMaxTop || top > E) {
    b200_set_last_error("seq_moe_route: need 1 <= top <= min(16, experts), experts <= 256");
    return B200_ERR_ARG;
  }
  cudaStream_t st = (cudaStream_t)stream;
  MoePlan p = moe_plan_view(plan, T, E, top);
  if (cudaMemsetAsync(p.counts, 0, sizeof(int32_t) * E, st) != cudaSuccess) { b200_set_last_error("seq_moe_route: memset failed"); return B200_ERR_CUDA; }
  if (mode == 1)
    B200_LAUNCH(moe_route_kernel<1>, dim3((unsigned)((T + 7) / 8)), dim3(256), 0, st, logits, T, E, top, ids, weights, p.counts, p.place, correction,
                corr_dt, weight_scale);
  else
    B200_LAUNCH(moe_route_kernel<0>, dim3((unsigned)((T + 7) / 8)), dim3(256), 0, st, logits, T, E, top, ids, weights, p.counts, p.place, correction,
                corr_dt, weight_scale);
  B200_LAUNCH(moe_plan_kernel, dim3(1), dim3(256), 0, st, (const int32_t*)ids, T * top, top, E, p);
  b200_count_launches(2);
  return B200_OK;
}

extern "C" int b200_seq_moe_route(const float* logits, int64_t T, int E, int top, int32_t* ids, float* weights, int32_t* plan, void* stream) {
  return b200_seq_moe_route_scored(logits, T, E, top, 0, nullptr, B200_DT_F32, 1.f, ids, weights, plan, stream);
}

template <typename TA, typename TW, typename TC>
static int launch_moe_linear(const void* A, int64_t lda, int gather, const void* W, void* C, int64_t ldc, MoePlan p, int64_t N, int64_t K,
                             cudaStream_t st) {
  dim3 grid((unsigned)((N + kMoeTile - 1) / kMoeTile), (unsigned)p.max_tiles);
  B200_LAUNCH((moe_linear_kernel<TA, TW, TC>), grid, dim3(256), 0, st, (const TA*)A, lda, gather, (const TW*)W, (TC*)C, ldc, p, (int)N, (int)K);
  b200_count_launches(1);
  return B200_OK;
}

// C[row, :N] = W[expert(row)] [N, K] . A[gather ? token(row) : row, :K] for the T * top compact rows of the plan; W [E, N, K] dense
extern "C" int b200_seq_moe_linear(const void* A, int a_dt, int64_t lda, int gather, const void* W, int w_dt, void* C, int c_dt, int64_t ldc,
                                   int32_t* plan, int64_t T, int E, int top, int64_t N, int64_t K, void* stream) {
  if (T == 0 || N == 0) return B200_OK;
  MoePlan p = moe_plan_view(plan, T, E, top);
  if (p.max_tiles > 65535 || K <= 0) { b200_set_last_error("seq_moe_linear: bad sizes"); return B200_ERR_ARG; }
  cudaStream_t st = (cudaStream_t)stream;
  static const bool use_mma = []() { const char* e = getenv("B200_SEQ_MOE_MMA"); return !(e && e[0] == '0'); }();
  if (use_mma && a_dt == B200_DT_BF16 && w_dt == B200_DT_BF16 && K % 8 == 0 && lda % 8 == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(W) & 15) == 0) {
    const size_t smem = (size_t)2 * kMmaStages * kMoeTile * kMmaLd * 2;
    dim3 grid((unsigned)((N + kMoeTile - 1) / kMoeTile), (unsigned)p.max_tiles);
#define MMA_LAUNCH(TC)                                                                                                                  \
  do {                                                                                                                                  \
    static bool cfg = false;                                                                                                            \
    if (!cfg) { cudaFuncSetAttribute(moe_linear_mma_kernel<TC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); cfg = true; }   \
    B200_LAUNCH((moe_linear_mma_kernel<TC>), grid, dim3(128), smem, st, (const __nv_bfloat16*)A, lda, gather, (const __nv_bfloat16*)W,   \
                (TC*)C, ldc, p, (int)N, (int)K);                                                                                        \
    b200_count_launches(1);                                                                                                             \
    return B200_OK;                                                                                                                     \
  } while (0)
    if (c_dt == B200_DT_F32) MMA_LAUNCH(float);
    else MMA_LAUNCH(__nv_bfloat16);
#undef MMA_LAUNCH
  }
  const int key = a_dt * 4 + w_dt * 2 + c_dt;
#define CASE(a, w, c, TA, TW, TC) \
  case a * 4 + w * 2 + c: return launch_moe_linear<TA, TW, TC>(A, lda, gather, W, C, ldc, p, N, K, st)
  switch (key) {
    CASE(0, 0, 0, __nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    CASE(0, 0, 1, __nv_bfloat16, __nv_bfloat16, float);
    CASE(1, 0, 1, float, __nv_bfloat16, float);
    CASE(1, 1, 1, float, float, float);
    default: break;
  }
#undef CASE
  b200_set_last_error("seq_moe_linear: unsupported combination of element types");
  return B200_ERR_UNSUPPORTED;
}

// resid fp32 [T, W] += mix (fp32 [T, W] or NULL) + sum_k weights[t, k] y[row_of(t, k)];  y NULL / top 0: the sum is empty
extern "C" int b200_seq_moe_combine_add(float* resid, const float* mix, const float* y, int64_t ldy, const float* weights, int32_t* plan,
                                        int64_t T, int E, int top, int64_t W, void* stream) {
  if (T == 0) return B200_OK;
  const int32_t* row_of = nullptr;
  if (y != nullptr && top > 0) row_of = moe_plan_view(plan, T, E, top).row_of;
  else top = 0;
  B200_LAUNCH(moe_combine_add_kernel, dim3((unsigned)T), dim3(256), 0, (cudaStream_t)stream, resid, mix, y, ldy, weights, row_of, top, (int)W);
  b200_count_launches(1);
  return B200_OK;
}

// out [T * top, K] (type dt) = A[token(row)]: the compact rows, for callers that run one dense product per expert
extern "C" int b200_seq_moe_gather_rows(const void* A, int dt, int64_t lda, void* out, int32_t* plan, int64_t T, int E, int top, int64_t K,
                                        void* stream) {
  if (T == 0) return B200_OK;
  MoePlan p = moe_plan_view(plan, T, E, top);
  B200_SEQ_DISPATCH(dt, El, B200_LAUNCH((moe_gather_rows_kernel<El>), dim3((unsigned)(T * top)), dim3(256), 0, (cudaStream_t)stream, (const El*)A, lda,
                                        (El*)out, (const int32_t*)p.token_of_row, (int)K));
  b200_count_launches(1);
  return B200_OK;
}
