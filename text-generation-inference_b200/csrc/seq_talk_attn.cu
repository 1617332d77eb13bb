// Grouped-query attention whose scaled scores are mixed across the query heads before the soft-max ("talking heads":
// s'_h = sum_g M[h, g] s_g with a learned [heads, heads] matrix), over a paged cache of rotated keys and values, with a chunked
// causal mask (a query sees the earlier keys of its own chunk of `chunk` positions, chunks counted from position 0 of the
// sequence) and / or a sliding window.  Because every head's weights depend on every head's scores, one block owns ALL heads of
// its query rows, unlike the per-key-head kernels of seq_paged_attn.cu.
//
// Cache row of a token (token-major: `page` rows of `row_width` elements per block):
//   [ ... keys of the G key heads (from k_off, G * dim) ... | ... values of the G value heads (from v_off, G * vdim) ... ]
//
//   qk_rot_prepare_kernel : from a token's projected row [q | k | v] (fp32): RMS norm over the WHOLE q projection and over the
//                           whole k projection (one statistic for all heads, a weight per column), rotation of the first
//                           `rot` columns of every head in the rotate-half layout (column i pairs with column i + rot/2; the
//                           cos / sin tables carry frequency scaling and amplitude), keys and values into the token's cache
//                           slot, queries into a dense fp32 buffer.
//   talk_attn_kernel      : plain form, any element type and shape.  One block per (query token, slab of 8 heads): raw scores of
//                           all heads against a tile of 32 keys, the mix, fp32 online soft-max and P V for the slab's heads (a
//                           warp each).  Prompts, portions and decoded tokens are one case: keys come back from the cache.
//   talk_attn_mma_kernel  : bfloat16 caches, m16n8k16 tensor-core products; see the note above the kernel.
#include "seq_common.cuh"

#include <cstdlib>

namespace b200 {
namespace seq {

constexpr int kTalkPrepThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kTalkPrepThreads) qk_rot_prepare_kernel(
    const float* __restrict__ src, int64_t ld, int col_q, int col_k, int col_v, int H, int G, int d, int dv, const T* __restrict__ qnorm_w,
    const T* __restrict__ knorm_w, int whole_norm, float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
    const int64_t* __restrict__ position_ids, const int64_t* __restrict__ slot_mapping, T* __restrict__ cache, int64_t RW, int k_off, int v_off,
    float* __restrict__ q_out) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const int64_t pos = position_ids[t], slot = slot_mapping[t];
  const float* row = src + t * ld;
  const int nq = H * d, nk = G * d, half = rot / 2;
  float rq = 1.f, rk = 1.f;
  if (whole_norm) {
    float s = 0.f;
    for (int i = threadIdx.x; i < nq; i += kTalkPrepThreads) s += row[col_q + i] * row[col_q + i];
    rq = 1.f / sqrtf(block_sum(s, red) / nq + eps);
    s = 0.f;
    for (int i = threadIdx.x; i < nk; i += kTalkPrepThreads) s += row[col_k + i] * row[col_k + i];
    rk = 1.f / sqrtf(block_sum(s, red) / nk + eps);
  }
  const float* cs = cos_t + pos * half;
  const float* sn = sin_t + pos * half;
  T* crow = slot >= 0 ? cache + slot * RW : nullptr;
  for (int e = threadIdx.x; e < nq + nk; e += kTalkPrepThreads) {
    const bool is_q = e < nq;
    const int c = is_q ? e : e - nq;          // column inside the projection
    const int i = c % d;
    const float* v = row + (is_q ? col_q : col_k);
    const T* w = is_q ? qnorm_w : knorm_w;
    const float r = is_q ? rq : rk;
    float x = v[c] * r * (w ? ldf(w + c) : 1.f);
    if (i < rot) {
      const int partner = i < half ? c + half : c - half;
      const float y = v[partner] * r * (w ? ldf(w + partner) : 1.f);
      const int f = i < half ? i : i - half;
      x = i < half ? x * cs[f] - y * sn[f] : x * cs[f] + y * sn[f];
    }
    if (is_q) q_out[t * nq + c] = x;
    else if (crow) stf(crow + k_off + c, x);
  }
  if (crow)
    for (int c = threadIdx.x; c < G * dv; c += kTalkPrepThreads) stf(crow + v_off + c, row[col_v + c]);
}

constexpr int kTalkWarps = 8, kTalkKeys = 32;

__device__ __forceinline__ int first_visible(int p, int chunk, int window) {
  int lo = chunk > 0 ? (p / chunk) * chunk : 0;
  if (window > 0) lo = max(lo, p - window + 1);
  return lo;
}

template <typename T, int NV>  // NV = ceil(vdim / 32) value columns per lane
__global__ void __launch_bounds__(kTalkWarps * 32) talk_attn_kernel(
    const float* __restrict__ q, const T* __restrict__ cache, int64_t RW, int k_off, int v_off, const int32_t* __restrict__ block_table,
    int64_t bt_stride, const int32_t* __restrict__ seq_of_token, const int64_t* __restrict__ position_ids, const float* __restrict__ talk,
    float* __restrict__ out, int H, int G, int d, int dv, int chunk, int window, float scale, int page) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int KD = G * d, KP = KD + 1, VD = G * dv, rep = H / G;
  float* qs = sm;                          // [H][d], scaled
  float* ss = qs + H * d;                  // [H][32] raw scores of the tile
  float* kv = ss + H * kTalkKeys;          // keys [32][KP], then values [32][VD]
  const int64_t t = blockIdx.x;
  const int w = warp_id(), lane = lane_id(), nthreads = kTalkWarps * 32;
  const int h = blockIdx.y * kTalkWarps + w;  // the head whose soft-max and output this warp owns
  const bool own = h < H;
  const int b = seq_of_token[t];
  const int p = (int)position_ids[t];
  const int j_lo = first_visible(p, chunk, window);
  for (int idx = threadIdx.x; idx < H * d; idx += nthreads) qs[idx] = q[t * H * d + idx] * scale;
  float m = -INFINITY, l = 0.f, acc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) acc[i] = 0.f;
  const int32_t* table = block_table + (int64_t)b * bt_stride;
  for (int j0 = j_lo; j0 <= p; j0 += kTalkKeys) {
    const int nk = min(kTalkKeys, p - j0 + 1);
    __syncthreads();  // the previous tile's values are no longer read
    for (int idx = threadIdx.x; idx < nk * KD; idx += nthreads) {
      const int jj = idx / KD, c = idx % KD, j = j0 + jj;
      kv[jj * KP + c] = ldf(cache + ((int64_t)table[j / page] * page + j % page) * RW + k_off + c);
    }
    __syncthreads();
    for (int g = w; g < H; g += kTalkWarps) {
      float dot = 0.f;
      if (lane < nk) {
        const float* kq = kv + lane * KP + (g / rep) * d;
        const float* qq = qs + g * d;
        for (int i = 0; i < d; ++i) dot = fmaf(qq[i], kq[i], dot);
      }
      ss[g * kTalkKeys + lane] = dot;
    }
    __syncthreads();  // scores complete, keys no longer read
    for (int idx = threadIdx.x; idx < nk * VD; idx += nthreads) {
      const int jj = idx / VD, c = idx % VD, j = j0 + jj;
      kv[idx] = ldf(cache + ((int64_t)table[j / page] * page + j % page) * RW + v_off + c);
    }
    float s = -INFINITY;
    if (own && lane < nk) {
      if (talk) {
        s = 0.f;
        for (int g = 0; g < H; ++g) s = fmaf(talk[h * H + g], ss[g * kTalkKeys + lane], s);
      } else {
        s = ss[h * kTalkKeys + lane];
      }
    }
    __syncthreads();  // values loaded
    if (own) {
      const float m_new = fmaxf(m, warp_max(s));
      const float pr = lane < nk ? expf(s - m_new) : 0.f;
      const float corr = expf(m - m_new);
      l = l * corr + warp_sum(pr);
      m = m_new;
#pragma unroll
      for (int i = 0; i < NV; ++i) acc[i] *= corr;
      const float* vbase = kv + (h / rep) * dv;
      for (int jj = 0; jj < nk; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, pr, jj);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int c = lane + 32 * i;
          if (c < dv) acc[i] = fmaf(pj, vbase[jj * VD + c], acc[i]);
        }
      }
    }
  }
  if (own) {
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < dv) out[(t * H + h) * dv + c] = acc[i] * inv;
    }
  }
}

}  // namespace seq
}  // namespace b200

using namespace b200::seq;

// src fp32 [T, ld] holds the projections at columns col_q (H * d), col_k (G * d), col_v (G * dv).  whole_norm: RMS norm over each of
// the q and k projections as a whole (weights per column, may be NULL).  cos / sin fp32 [positions, rot / 2]; rot 0: no rotation.
extern "C" int b200_seq_qk_rot_prepare(const float* src, int64_t ld, int col_q, int col_k, int col_v, int H, int G, int d, int dv,
                                       const void* qnorm_w, const void* knorm_w, int whole_norm, float eps, const float* cos_t, const float* sin_t,
                                       int rot, const int64_t* position_ids, const int64_t* slot_mapping, void* cache, int dt, int64_t row_width,
                                       int k_off, int v_off, float* q_out, int64_t T, void* stream) {
  if (T == 0) return B200_OK;
  if (rot < 0 || rot > d || rot % 2 != 0 || (rot > 0 && (cos_t == nullptr || sin_t == nullptr))) {
    b200_set_last_error("seq_qk_rot_prepare: rotated columns must be even, at most the head size, with tables");
    return B200_ERR_ARG;
  }
  B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((qk_rot_prepare_kernel<E>), dim3((unsigned)T), dim3(kTalkPrepThreads), 0, (cudaStream_t)stream, src, ld, col_q,
                                       col_k, col_v, H, G, d, dv, (const E*)qnorm_w, (const E*)knorm_w, whole_norm, eps, cos_t, sin_t, rot,
                                       position_ids, slot_mapping, (E*)cache, row_width, k_off, v_off, q_out));
  b200_count_launches(1);
  return B200_OK;
}

template <typename E, int NV>
static int launch_talk_plain(const float* q, const void* cache, int64_t RW, int k_off, int v_off, const int32_t* block_table, int64_t bt_stride,
                             const int32_t* seq_of_token, const int64_t* position_ids, const float* talk, float* out, int64_t T, int H, int G, int d,
                             int dv, int chunk, int window, float scale, int page, cudaStream_t st) {
  const size_t kvbuf = (size_t)kTalkKeys * (size_t)max(G * d + 1, G * dv);
  const size_t smem = ((size_t)H * d + (size_t)H * kTalkKeys + kvbuf) * 4;
  if (smem > 200 * 1024) { b200_set_last_error("seq_talk_attn: heads x size too large for the plain kernel"); return B200_ERR_UNSUPPORTED; }
  static bool cfg = false;
  if (!cfg) { cudaFuncSetAttribute(talk_attn_kernel<E, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); cfg = true; }
  dim3 grid((unsigned)T, (unsigned)((H + kTalkWarps - 1) / kTalkWarps));
  B200_LAUNCH((talk_attn_kernel<E, NV>), grid, dim3(kTalkWarps * 32), smem, st, q, (const E*)cache, RW, k_off, v_off, block_table, bt_stride,
              seq_of_token, position_ids, talk, out, H, G, d, dv, chunk, window, scale, page);
  b200_count_launches(1);
  return B200_OK;
}

// q fp32 [T, H, d]; cache rows as above; talk fp32 [H, H] or NULL (no mix); chunk / window <= 0: none -> out fp32 [T, H, dv]
extern "C" int b200_seq_talk_attn(const float* q, const void* cache, int dt, int64_t row_width, int k_off, int v_off, const int32_t* block_table,
                                  int64_t bt_stride, const int32_t* seq_of_token, const int32_t* cu_q, int B, const int64_t* position_ids,
                                  const float* talk, float* out, int64_t T, int H, int G, int d, int dv, int chunk, int window, float scale,
                                  int page, void* stream) {
  if (T == 0) return B200_OK;
  if (G <= 0 || H % G != 0 || d <= 0 || dv <= 0 || dv > 256) {
    b200_set_last_error("seq_talk_attn: need heads % kv_heads == 0 and 0 < vdim <= 256");
    return B200_ERR_ARG;
  }
  cudaStream_t st = (cudaStream_t)stream;
  (void)cu_q;
  (void)B;
#define TALK(N)                                                                                                                              \
  B200_SEQ_DISPATCH(dt, E, return (launch_talk_plain<E, N>(q, cache, row_width, k_off, v_off, block_table, bt_stride, seq_of_token, position_ids, \
                                                          talk, out, T, H, G, d, dv, chunk, window, scale, page, st)))
  const int nv = (dv + 31) / 32;
  if (nv <= 1) TALK(1);
  else if (nv <= 2) TALK(2);
  else if (nv <= 4) TALK(4);
  else TALK(8);
#undef TALK
}
