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
//                           slot, queries into a dense fp32 buffer.  Optionally the values turn as well, by their own position
//                           over the first `v_rot` columns of every value head (halves or neighbouring columns as pairs).
//   talk_attn_kernel      : plain form, any element type and shape.  One block per (query token, slab of 8 heads): raw scores of
//                           all heads against a tile of 32 keys, the mix, fp32 online soft-max and P V for the slab's heads (a
//                           warp each).  Prompts, portions and decoded tokens are one case: keys come back from the cache.
//   group_attn_kernel     : plain form without a mix: one block per (query token, key / value head group, 8 heads of the group).
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
    float* __restrict__ q_out, const float* __restrict__ vcos_t, const float* __restrict__ vsin_t, int v_rot, int v_interleaved) {
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
  if (crow) {
    // values: the first v_rot columns of every value head turn with the token's own position (tables of their own)
    const int vhalf = v_rot / 2;
    const float* vc = v_rot ? vcos_t + pos * vhalf : nullptr;
    const float* vs = v_rot ? vsin_t + pos * vhalf : nullptr;
    for (int c = threadIdx.x; c < G * dv; c += kTalkPrepThreads) {
      const int i = c % dv;
      float x = row[col_v + c];
      if (i < v_rot) {
        int f, partner;
        bool first;
        if (v_interleaved) { f = i >> 1; first = (i & 1) == 0; partner = first ? c + 1 : c - 1; }
        else { first = i < vhalf; f = first ? i : i - vhalf; partner = first ? c + vhalf : c - vhalf; }
        const float y = row[col_v + partner];
        x = first ? x * vc[f] - y * vs[f] : x * vc[f] + y * vs[f];
      }
      stf(crow + v_off + c, x);
    }
  }
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
    float* __restrict__ out, int H, int G, int d, int dv, int chunk, int window, float scale, int page, const float* __restrict__ sink) {
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
  // a sink logit sits in the soft-max denominator like one more key (unscaled, never mixed) whose value is zero
  float m = (sink && own) ? sink[h] : -INFINITY, l = (sink && own) ? 1.f : 0.f, acc[NV];
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

// Plain form without a head mix: no head needs another head's scores, so a block owns (query token, key / value head group, up
// to 8 query heads of that group) and stages only that group's keys and values - shared memory does not grow with the number of
// groups.  Same tiles of 32 keys, a warp per head, fp32 online soft-max, window, chunk and sink as above.
template <typename T, int NV>  // NV = ceil(vdim / 32) value columns per lane
__global__ void __launch_bounds__(kTalkWarps * 32) group_attn_kernel(
    const float* __restrict__ q, const T* __restrict__ cache, int64_t RW, int k_off, int v_off, const int32_t* __restrict__ block_table,
    int64_t bt_stride, const int32_t* __restrict__ seq_of_token, const int64_t* __restrict__ position_ids, float* __restrict__ out, int H, int G,
    int d, int dv, int chunk, int window, float scale, int page, const float* __restrict__ sink) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int KP = d + 1, rep = H / G, slabs = (rep + kTalkWarps - 1) / kTalkWarps;
  float* qs = sm;                          // [8][d], scaled
  float* kv = qs + kTalkWarps * d;         // keys [32][KP], then values [32][dv]
  const int64_t t = blockIdx.x;
  const int g = blockIdx.y / slabs, sub = blockIdx.y % slabs;
  const int w = warp_id(), lane = lane_id(), nthreads = kTalkWarps * 32;
  const int hh = sub * kTalkWarps + w;     // head of the group that this warp owns
  const bool own = hh < rep;
  const int h = g * rep + (own ? hh : 0);
  const int b = seq_of_token[t];
  const int p = (int)position_ids[t];
  const int j_lo = first_visible(p, chunk, window);
  for (int idx = threadIdx.x; idx < kTalkWarps * d; idx += nthreads) {
    const int ww = idx / d, head = sub * kTalkWarps + ww;
    qs[idx] = head < rep ? q[(t * H + g * rep + head) * d + idx % d] * scale : 0.f;
  }
  float m = (sink && own) ? sink[h] : -INFINITY, l = (sink && own) ? 1.f : 0.f, acc[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) acc[i] = 0.f;
  const int32_t* table = block_table + (int64_t)b * bt_stride;
  const int kcol = k_off + g * d, vcol = v_off + g * dv;
  for (int j0 = j_lo; j0 <= p; j0 += kTalkKeys) {
    const int nk = min(kTalkKeys, p - j0 + 1);
    __syncthreads();  // the previous tile's values are no longer read (first time round: qs is complete after the next barrier)
    for (int idx = threadIdx.x; idx < nk * d; idx += nthreads) {
      const int jj = idx / d, c = idx % d, j = j0 + jj;
      kv[jj * KP + c] = ldf(cache + ((int64_t)table[j / page] * page + j % page) * RW + kcol + c);
    }
    __syncthreads();
    float s = -INFINITY;
    if (own && lane < nk) {
      const float* kq = kv + lane * KP;
      const float* qq = qs + w * d;
      s = 0.f;
      for (int i = 0; i < d; ++i) s = fmaf(qq[i], kq[i], s);
    }
    __syncthreads();  // keys no longer read
    for (int idx = threadIdx.x; idx < nk * dv; idx += nthreads) {
      const int jj = idx / dv, c = idx % dv, j = j0 + jj;
      kv[idx] = ldf(cache + ((int64_t)table[j / page] * page + j % page) * RW + vcol + c);
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
      for (int jj = 0; jj < nk; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, pr, jj);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int c = lane + 32 * i;
          if (c < dv) acc[i] = fmaf(pj, kv[jj * dv + c], acc[i]);
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

// ------------------------------------------------------------------------------------------------------------------------
// Tensor-core form for bfloat16 caches.  One block per (sequence, tile of QT query tokens): its R = QT * heads rows are ordered
// (key head group, token, query head of the group), so that the 16 rows of a warp share one group and read that group's key and
// value columns; R / 16 warps.  Per tile of KT keys (16-byte cp.async; a tile holds the keys and values of ALL groups): every
// warp computes the raw scores of its rows with m16n8k16 products and leaves them, scaled, in shared memory in fp32; after a
// barrier each thread gathers, for the (row, key) elements of its own accumulator fragment, the scores of all heads of the same
// token and mixes them with FFMAs in fp32 (the mix is the one step that crosses warps); mask, fp32 online soft-max and
// O += P V follow per warp with P in registers.  There is ONE key buffer and ONE value buffer, so that two blocks share an SM at
// the sizes of a real model: the next tile's keys are fetched as soon as the scores are done (while the mix, the soft-max and
// P V run), its values when P V is done (while the next scores run).  gridDim.z > 1 deals the tile's keys out in runs whose partial
// (output, max, sum) talk_attn_merge_kernel joins.  Needs dim % 16 == 0, vdim % 16 == 0, vdim <= 128 and QT * (heads / kv_heads)
// a multiple of 16; everything else takes the plain kernel.
// ------------------------------------------------------------------------------------------------------------------------
constexpr int kTalkPad = 8;

// acc += t * v on both halves at once (packed fp32 FMA of sm_100)
__device__ __forceinline__ void ffma2(float2& acc, float t, float vx, float vy) {
  asm("{ .reg .b64 a, b, c; mov.b64 a, {%2, %2}; mov.b64 b, {%3, %4}; mov.b64 c, {%0, %1}; fma.rn.f32x2 c, a, b, c; mov.b64 {%0, %1}, c; }"
      : "+f"(acc.x), "+f"(acc.y)
      : "f"(t), "f"(vx), "f"(vy));
}

// which (sequence, tile of QT of its rows) block `tile` has; b == B: none
__device__ __forceinline__ void talk_find_tile(const int32_t* cu_q, int B, int QT, int tile, int& b, int& row0, int& ntok) {
  for (b = 0; b < B; ++b) {
    const int n = cu_q[b + 1] - cu_q[b];
    const int nt = (n + QT - 1) / QT;
    if (tile < nt) {
      row0 = cu_q[b] + tile * QT;
      ntok = min(QT, cu_q[b + 1] - row0);
      return;
    }
    tile -= nt;
  }
}

template <int NDV, int KT>  // NDV = vdim / 8 output n-tiles per warp, KT keys per tile
__global__ void __launch_bounds__(512) talk_attn_mma_kernel(
    const float* __restrict__ q, const __nv_bfloat16* __restrict__ cache, int64_t RW, int k_off, int v_off, const int32_t* __restrict__ block_table,
    int64_t bt_stride, const int32_t* __restrict__ cu_q, int B, const int64_t* __restrict__ position_ids, const float* __restrict__ talk,
    float* __restrict__ out, int H, int G, int d, int QT, int chunk, int window, float scale, int page, float* __restrict__ partial,
    const float* __restrict__ sink) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int dv = NDV * 8, SP = KT == 16 ? 16 : KT + 4;   // row stride of the score tile: conflict-free 16-byte accesses
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int rep = H / G, R = QT * H, rows_g = QT * rep;
  const int KD = G * d, KP = KD + kTalkPad, VD = G * dv, VP = VD + kTalkPad, DP = d + kTalkPad;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [R][DP]
  __nv_bfloat16* Ks = Qs + R * DP;                                   // [KT][KP]
  __nv_bfloat16* Vs = Ks + KT * KP;                                  // [KT][VP]
  float* Ss = reinterpret_cast<float*>(Vs + KT * VP);                // [R][SP] scaled raw scores of the tile
  float* Ts = Ss + R * SP;                                           // [H][H] the mixing matrix
  int b, row0 = 0, ntok = 0;
  talk_find_tile(cu_q, B, QT, blockIdx.x, b, row0, ntok);
  if (b >= B) return;  // block-uniform: no barrier has been met yet
  const int nthreads = blockDim.x;
  const int p0 = (int)position_ids[row0], p_last = p0 + ntok - 1;
  const int j_first = first_visible(p0, chunk, window);
  const int n_ktiles = (p_last - j_first + KT) / KT;
  const int per_split = (n_ktiles + gridDim.z - 1) / gridDim.z;
  const int j_start = j_first + (int)blockIdx.z * per_split * KT;
  const int j_end = min(p_last, j_start + per_split * KT - 1);   // last key of this block's run
  const int w = warp_id(), lane = lane_id();
  const int32_t* table = block_table + (int64_t)b * bt_stride;
  for (int r = w; r < R; r += nthreads / 32) {
    const int c = r / rows_g, rr = r % rows_g, tok = rr / rep, hh = rr % rep;
    const float* src = q + ((int64_t)(row0 + tok) * H + c * rep + hh) * d;
    const bool live = tok < ntok;
    for (int i = lane; i < d; i += 32) Qs[r * DP + i] = __float2bfloat16_rn(live ? src[i] : 0.f);
  }
  if (talk)
    for (int i = threadIdx.x; i < H * H; i += nthreads) Ts[i] = talk[i];
  const int kchunks = KD / 8, vchunks = VD / 8;
  const int page_shift = (page & (page - 1)) == 0 ? 31 - __clz(page) : -1;
  // one block-table lookup per thread and row, then the row's 16-byte pieces go round eight threads
  auto load_rows = [&](__nv_bfloat16* dst, int ld, int off, int chunks, int j0) {
    for (int row = threadIdx.x >> 3; row < KT; row += nthreads >> 3) {
      const int j = j0 + row;
      __nv_bfloat16* drow = dst + row * ld;
      if (j <= j_end) {
        const int64_t blk = table[page_shift >= 0 ? j >> page_shift : j / page];
        const int tk = page_shift >= 0 ? j & (page - 1) : j % page;
        const __nv_bfloat16* src = cache + (blk * page + tk) * RW + off;
        for (int ch = threadIdx.x & 7; ch < chunks; ch += 8) cp_async_16(drow + ch * 8, src + ch * 8, true);
      } else {
        for (int ch = threadIdx.x & 7; ch < chunks; ch += 8) *reinterpret_cast<uint4*>(drow + ch * 8) = make_uint4(0u, 0u, 0u, 0u);  // finite: p = 0
      }
    }
    cp_async_commit();
  };
  // this thread's two accumulator rows
  const int cq = (lane & 3) * 2;
  const int c_w = (w * 16) / rows_g;   // the warp's key / value head group
  int p_row[2], lo_row[2], h_row[2], tok_row[2];
  bool valid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = w * 16 + (lane >> 2) + i * 8, rr = r % rows_g;
    tok_row[i] = rr / rep;
    valid[i] = tok_row[i] < ntok;
    p_row[i] = valid[i] ? p0 + tok_row[i] : p0;
    lo_row[i] = first_visible(p_row[i], chunk, window);
    h_row[i] = c_w * rep + rr % rep;
  }
  const bool warp_active = ((w * 16) % rows_g) / rep < ntok;  // rows of a warp ascend in token: its first row decides
  const int lo_last = first_visible(p_last, chunk, window);
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  if (sink && blockIdx.z == 0) {   // the sink counts once: in the first run of the keys
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      m_run[i] = sink[h_row[i]];
      l_run[i] = 1.f;
    }
  }
  float o[NDV][4];
#pragma unroll
  for (int i = 0; i < NDV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const uint32_t qs_addr = smem_u32(Qs), ks_addr = smem_u32(Ks), vs_addr = smem_u32(Vs);
  const int lm = lane >> 3, lr = lane & 7;
  const uint32_t a_lane = qs_addr + (uint32_t)(((w * 16 + (lm & 1) * 8 + lr) * DP + (lm >> 1) * 8) * 2);
  if (j_start <= j_end) load_rows(Ks, KP, k_off, kchunks, j_start);
  for (int j0 = j_start; j0 <= j_end; j0 += KT) {
    load_rows(Vs, VP, v_off, vchunks, j0);   // the value buffer is free: the previous tile ended with a barrier
    cp_async_wait<1>();                      // this tile's keys have landed (its values may still be in flight)
    __syncthreads();                         // ... for every thread; first time round Qs is complete as well
    float s[KT / 8][4];
#pragma unroll
    for (int i = 0; i < KT / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    if (warp_active) {
      const uint32_t b_lane = ks_addr + (uint32_t)((((lm >> 1) * 8 + lr) * KP + c_w * d + (lm & 1) * 8) * 2);
      for (int kk = 0; kk < d; kk += 16) {
        uint32_t a[4];
        ldmatrix_x4(a[0], a[1], a[2], a[3], a_lane + kk * 2);
#pragma unroll
        for (int kg = 0; kg < KT / 16; ++kg) {
          uint32_t bb[4];
          ldmatrix_x4(bb[0], bb[1], bb[2], bb[3], b_lane + (uint32_t)((kg * 16 * KP + kk) * 2));
          mma_m16n8k16_bf16f32(s[2 * kg], a, bb[0], bb[1]);
          mma_m16n8k16_bf16f32(s[2 * kg + 1], a, bb[2], bb[3]);
        }
      }
#pragma unroll
      for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] *= scale;
    }
    if (talk) {
      // all heads' scores of the tile meet in shared memory; every thread then mixes the elements of its own fragment.  A row of
      // the tile is stored with each quad lane's KT / 4 columns side by side (the mix is column-wise, so any order serves as long
      // as writer and reader agree), which makes the stores and the mix's loads 16 bytes wide
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        float* dst = Ss + (w * 16 + (lane >> 2) + i * 8) * SP + (lane & 3) * (KT / 4);
#pragma unroll
        for (int nt = 0; nt < KT / 8; nt += 2)
          *reinterpret_cast<float4*>(dst + nt * 2) = make_float4(s[nt][i * 2], s[nt][i * 2 + 1], s[nt + 1][i * 2], s[nt + 1][i * 2 + 1]);
      }
    }
    cp_async_wait<0>();   // this tile's values have landed
    __syncthreads();      // scores and values are visible to all; nobody reads the key buffer any more
    if (j0 + KT <= j_end) load_rows(Ks, KP, k_off, kchunks, j0 + KT);
    else cp_async_commit();
    if (talk) {
      if (warp_active) {
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        // rows of tokens that the tile does not have (a decoding step fills one token of QT) are left at zero
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if (!valid[i]) continue;
          float2 acc[KT / 8];
#pragma unroll
          for (int nt = 0; nt < KT / 8; ++nt) acc[nt] = make_float2(0.f, 0.f);
          const float* trow = Ts + h_row[i] * H;
          const float* srow = Ss + tok_row[i] * rep * SP + (lane & 3) * (KT / 4);
          for (int c = 0; c < G; ++c) {   // head g = c * rep + hh of the same token: row c * rows_g + tok * rep + hh
            const float* rc = srow + c * rows_g * SP;
            const float* tc = trow + c * rep;
            if ((rep & 3) == 0) {
              for (int hh = 0; hh < rep; hh += 4) {
                const float4 t4 = *reinterpret_cast<const float4*>(tc + hh);
                const float tg[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  const float* ra = rc + (hh + u) * SP;
#pragma unroll
                  for (int nt = 0; nt < KT / 8; nt += 2) {
                    const float4 v = *reinterpret_cast<const float4*>(ra + nt * 2);
                    ffma2(acc[nt], tg[u], v.x, v.y);
                    ffma2(acc[nt + 1], tg[u], v.z, v.w);
                  }
                }
              }
            } else {
              for (int hh = 0; hh < rep; ++hh) {
                const float tg = tc[hh];
                const float* ra = rc + hh * SP;
#pragma unroll
                for (int nt = 0; nt < KT / 8; nt += 2) {
                  const float4 v = *reinterpret_cast<const float4*>(ra + nt * 2);
                  ffma2(acc[nt], tg, v.x, v.y);
                  ffma2(acc[nt + 1], tg, v.z, v.w);
                }
              }
            }
          }
#pragma unroll
          for (int nt = 0; nt < KT / 8; ++nt) {
            s[nt][i * 2] = acc[nt].x;
            s[nt][i * 2 + 1] = acc[nt].y;
          }
        }
      }
    }
    if (warp_active) {
      float mx[2] = {-INFINITY, -INFINITY};
      if (j0 + KT - 1 <= min(j_end, p0) && j0 >= lo_last) {
        // an interior tile: every key is visible to every row
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
      } else {
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = e >> 1, j = j0 + nt * 8 + cq + (e & 1);
            if (j > p_row[i] || j < lo_row[i] || j > j_end) s[nt][e] = -INFINITY;
            mx[i] = fmaxf(mx[i], s[nt][e]);
          }
      }
      float m_use[2], corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        const float m_new = fmaxf(m_run[i], mx[i]);
        m_use[i] = m_new == -INFINITY ? 0.f : m_new;  // a row that has met no visible key yet
        corr[i] = expf(m_run[i] - m_use[i]);
        m_run[i] = m_new;
      }
      uint32_t pa[KT / 16][4];
#pragma unroll
      for (int nt = 0; nt < KT / 8; ++nt) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(expf(s[nt][0] - m_use[0]), expf(s[nt][1] - m_use[0]));
        const __nv_bfloat162 hi = __floats2bfloat162_rn(expf(s[nt][2] - m_use[1]), expf(s[nt][3] - m_use[1]));
        // the sums use the rounded probabilities: numerator and denominator see the same weights
        sum[0] += __low2float(lo) + __high2float(lo);
        sum[1] += __low2float(hi) + __high2float(hi);
        pa[nt >> 1][(nt & 1) * 2] = *reinterpret_cast<const uint32_t*>(&lo);
        pa[nt >> 1][(nt & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&hi);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
        sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
        l_run[i] = l_run[i] * corr[i] + sum[i];
      }
#pragma unroll
      for (int i = 0; i < NDV; ++i) {
        o[i][0] *= corr[0];
        o[i][1] *= corr[0];
        o[i][2] *= corr[1];
        o[i][3] *= corr[1];
      }
      const uint32_t v_lane = vs_addr + (uint32_t)((((lm & 1) * 8 + lr) * VP + c_w * dv + (lm >> 1) * 8) * 2);
#pragma unroll
      for (int kg = 0; kg < KT / 16; ++kg) {
#pragma unroll
        for (int nt = 0; nt < NDV; nt += 2) {
          uint32_t bb[4];
          ldmatrix_x4_trans(bb[0], bb[1], bb[2], bb[3], v_lane + (uint32_t)((kg * 16 * VP + nt * 8) * 2));
          mma_m16n8k16_bf16f32(o[nt], pa[kg], bb[0], bb[1]);
          mma_m16n8k16_bf16f32(o[nt + 1], pa[kg], bb[2], bb[3]);
        }
      }
    }
    __syncthreads();  // everyone is done with the values and the scores before the next iteration overwrites them
  }
  if (gridDim.z > 1) {
    // partial [tile][split][R rows][dv + 2]: unnormalised output, then the running max and sum
    float* base = partial + (((int64_t)blockIdx.x * gridDim.z + blockIdx.z) * R) * (dv + 2);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (!valid[i]) continue;
      float* dst = base + (int64_t)(w * 16 + (lane >> 2) + i * 8) * (dv + 2);
#pragma unroll
      for (int nt = 0; nt < NDV; ++nt) {
        dst[nt * 8 + cq] = o[nt][i * 2];
        dst[nt * 8 + cq + 1] = o[nt][i * 2 + 1];
      }
      if ((lane & 3) == 0) {
        dst[dv] = m_run[i];
        dst[dv + 1] = l_run[i];
      }
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!valid[i]) continue;
    float* dst = out + ((int64_t)(row0 + tok_row[i]) * H + h_row[i]) * dv;
    const float inv = 1.f / l_run[i];
#pragma unroll
    for (int nt = 0; nt < NDV; ++nt) {
      dst[nt * 8 + cq] = o[nt][i * 2] * inv;
      dst[nt * 8 + cq + 1] = o[nt][i * 2 + 1] * inv;
    }
  }
}

// out[row] = sum_z e^(m_z - M) O_z / sum_z e^(m_z - M) l_z over the key runs of talk_attn_mma_kernel; one warp per row, blocks (query tile, 8 rows)
__global__ void __launch_bounds__(256) talk_attn_merge_kernel(const float* __restrict__ partial, float* __restrict__ out, const int32_t* __restrict__ cu_q,
                                                             int B, int H, int G, int QT, int dv, int nsplit) {
  pdl_launch_dependents();
  pdl_wait();
  int b, row0 = 0, ntok = 0;
  talk_find_tile(cu_q, B, QT, blockIdx.x, b, row0, ntok);
  if (b >= B) return;
  const int rep = H / G, R = QT * H, rows_g = QT * rep, lane = lane_id();
  constexpr int kMaxSplit = 8;
  for (int r = blockIdx.y * 8 + warp_id(); r < R; r += 8 * gridDim.y) {
    const int c = r / rows_g, rr = r % rows_g, tok = rr / rep;
    if (tok >= ntok) continue;
    const float* base = partial + (((int64_t)blockIdx.x * nsplit) * R + r) * (dv + 2);
    const int64_t zs = (int64_t)R * (dv + 2);
    float M = -INFINITY, wz[kMaxSplit];
#pragma unroll
    for (int z = 0; z < kMaxSplit; ++z) {
      wz[z] = z < nsplit ? base[z * zs + dv] : -INFINITY;
      M = fmaxf(M, wz[z]);
    }
    float den = 0.f;
#pragma unroll
    for (int z = 0; z < kMaxSplit; ++z) {
      wz[z] = wz[z] > -INFINITY ? expf(wz[z] - M) : 0.f;  // an empty run carries no weight
      if (z < nsplit) den += wz[z] * base[z * zs + dv + 1];
    }
    const float inv = 1.f / den;
    float* dst = out + ((int64_t)(row0 + tok) * H + c * rep + rr % rep) * dv;
    for (int col = lane; col < dv; col += 32) {
      float acc = 0.f;
#pragma unroll
      for (int z = 0; z < kMaxSplit; ++z)
        if (z < nsplit) acc = fmaf(wz[z], base[z * zs + col], acc);
      dst[col] = acc * inv;
    }
  }
}

}  // namespace seq
}  // namespace b200

using namespace b200::seq;

// src fp32 [T, ld] holds the projections at columns col_q (H * d), col_k (G * d), col_v (G * dv).  whole_norm: RMS norm over each of
// the q and k projections as a whole (weights per column, may be NULL).  cos / sin fp32 [positions, rot / 2]; rot 0: no rotation.
// vcos / vsin fp32 [positions, v_rot / 2]: the values' own turn (v_rot 0: stored as projected; v_interleaved: pairs are neighbours).
extern "C" int b200_seq_qk_rot_prepare(const float* src, int64_t ld, int col_q, int col_k, int col_v, int H, int G, int d, int dv,
                                       const void* qnorm_w, const void* knorm_w, int whole_norm, float eps, const float* cos_t, const float* sin_t,
                                       int rot, const int64_t* position_ids, const int64_t* slot_mapping, void* cache, int dt, int64_t row_width,
                                       int k_off, int v_off, float* q_out, int64_t T, const float* vcos_t, const float* vsin_t, int v_rot,
                                       int v_interleaved, void* stream) {
  if (T == 0) return B200_OK;
  if (v_rot < 0 || v_rot > dv || v_rot % 2 != 0 || (v_rot > 0 && (vcos_t == nullptr || vsin_t == nullptr))) {
    b200_set_last_error("seq_qk_rot_prepare: turned value columns must be even, at most the value size, with tables");
    return B200_ERR_ARG;
  }
  if (rot < 0 || rot > d || rot % 2 != 0 || (rot > 0 && (cos_t == nullptr || sin_t == nullptr))) {
    b200_set_last_error("seq_qk_rot_prepare: rotated columns must be even, at most the head size, with tables");
    return B200_ERR_ARG;
  }
  B200_SEQ_DISPATCH(dt, E, B200_LAUNCH((qk_rot_prepare_kernel<E>), dim3((unsigned)T), dim3(kTalkPrepThreads), 0, (cudaStream_t)stream, src, ld, col_q,
                                       col_k, col_v, H, G, d, dv, (const E*)qnorm_w, (const E*)knorm_w, whole_norm, eps, cos_t, sin_t, rot,
                                       position_ids, slot_mapping, (E*)cache, row_width, k_off, v_off, q_out, vcos_t, vsin_t, v_rot, v_interleaved));
  b200_count_launches(1);
  return B200_OK;
}

template <typename E, int NV>
static int launch_talk_plain(const float* q, const void* cache, int64_t RW, int k_off, int v_off, const int32_t* block_table, int64_t bt_stride,
                             const int32_t* seq_of_token, const int64_t* position_ids, const float* talk, float* out, int64_t T, int H, int G, int d,
                             int dv, int chunk, int window, float scale, int page, const float* sink, cudaStream_t st) {
  const size_t kvbuf = (size_t)kTalkKeys * (size_t)max(G * d + 1, G * dv);
  const size_t smem = ((size_t)H * d + (size_t)H * kTalkKeys + kvbuf) * 4;
  if (smem > 200 * 1024) { b200_set_last_error("seq_talk_attn: heads x size too large for the plain kernel"); return B200_ERR_UNSUPPORTED; }
  static bool cfg = false;
  if (!cfg) { cudaFuncSetAttribute(talk_attn_kernel<E, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); cfg = true; }
  dim3 grid((unsigned)T, (unsigned)((H + kTalkWarps - 1) / kTalkWarps));
  B200_LAUNCH((talk_attn_kernel<E, NV>), grid, dim3(kTalkWarps * 32), smem, st, q, (const E*)cache, RW, k_off, v_off, block_table, bt_stride,
              seq_of_token, position_ids, talk, out, H, G, d, dv, chunk, window, scale, page, sink);
  b200_count_launches(1);
  return B200_OK;
}

template <typename E, int NV>
static int launch_group_plain(const float* q, const void* cache, int64_t RW, int k_off, int v_off, const int32_t* block_table, int64_t bt_stride,
                              const int32_t* seq_of_token, const int64_t* position_ids, float* out, int64_t T, int H, int G, int d, int dv, int chunk,
                              int window, float scale, int page, const float* sink, cudaStream_t st) {
  const size_t smem = ((size_t)kTalkWarps * d + (size_t)kTalkKeys * (size_t)max(d + 1, dv)) * 4;
  if (smem > 200 * 1024) { b200_set_last_error("seq_talk_attn: head size too large for the plain kernel"); return B200_ERR_UNSUPPORTED; }
  static bool cfg = false;
  if (!cfg) { cudaFuncSetAttribute(group_attn_kernel<E, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); cfg = true; }
  const int rep = H / G;
  dim3 grid((unsigned)T, (unsigned)(G * ((rep + kTalkWarps - 1) / kTalkWarps)));
  B200_LAUNCH((group_attn_kernel<E, NV>), grid, dim3(kTalkWarps * 32), smem, st, q, (const E*)cache, RW, k_off, v_off, block_table, bt_stride,
              seq_of_token, position_ids, out, H, G, d, dv, chunk, window, scale, page, sink);
  b200_count_launches(1);
  return B200_OK;
}

// How the tensor-core kernel would run a step: tokens per query tile (0: the shape takes the plain kernel), keys per tile, shared memory
struct TalkPlan { int QT, KT; size_t smem; };

static TalkPlan talk_mma_plan(int dt, int64_t T, int B, int H, int G, int d, int dv, bool has_talk) {
  static const bool use_mma = []() { const char* e = getenv("B200_SEQ_ATTN_MMA"); return !(e && e[0] == '0'); }();
  TalkPlan p{0, 0, 0};
  if (!use_mma || dt != B200_DT_BF16 || G <= 0 || H % G != 0 || d % 16 != 0 || dv % 16 != 0 || dv > 128 || (dv / 8 != 2 && dv / 8 != 4 && dv / 8 != 8 && dv / 8 != 16))
    return p;
  const int rep = H / G;
  int g16 = 16, x = rep;
  while (x % 2 == 0 && g16 > 1) { x /= 2; g16 /= 2; }   // g16 = 16 / gcd(16, rep)
  int QT = g16;
  if ((int64_t)QT * H > 256) return p;
  if (T > 2 * (int64_t)B)                                // prompts and portions: larger tiles share each key tile among more rows
    while ((int64_t)QT * 2 * H <= 128) QT *= 2;
  const int R = QT * H;
  auto bytes = [&](int KT) {
    return ((size_t)R * (d + kTalkPad) + (size_t)KT * (G * d + kTalkPad) + (size_t)KT * (G * dv + kTalkPad)) * 2 +
           ((size_t)R * (KT == 16 ? 16 : KT + 4) + (has_talk ? (size_t)H * H : 0)) * 4;
  };
  // the largest key tile with which two blocks share an SM (228 KB, 1 KB reserved per block); failing that, the largest that fits at all
  for (size_t limit : {(size_t)(233472 / 2 - 1024), (size_t)200 * 1024})
    for (int KT : {64, 32, 16})
      if (bytes(KT) <= limit) { p.QT = QT; p.KT = KT; p.smem = bytes(KT); return p; }
  return p;
}

// Over how many blocks the tensor-core kernel should split each query tile's keys in this step (1: no split; 0: the plain kernel runs)
// and the fp32 workspace (`partial`) that takes
extern "C" int b200_seq_talk_attn_splits(int dt, int64_t T, int B, int H, int G, int d, int dv, int64_t* workspace_floats) {
  if (workspace_floats) *workspace_floats = 0;
  const TalkPlan p = talk_mma_plan(dt, T, B, H, G, d, dv, true);
  if (p.QT == 0) return 0;
  const int64_t tiles = (T + p.QT - 1) / p.QT + B;
  const int64_t busy = (T + p.QT - 1) / p.QT > B ? (T + p.QT - 1) / p.QT : B;
  // as many runs as keep all blocks resident at once (shared memory decides how many share an SM)
  int64_t per_sm = (int64_t)233472 / (int64_t)(p.smem + 1024);   // 228 KB per SM, 1 KB reserved per block
  per_sm = per_sm < 1 ? 1 : per_sm;
  int64_t n = (148 * per_sm) / (busy > 0 ? busy : 1);
  n = n < 1 ? 1 : (n > 8 ? 8 : n);
  if (n > 1 && workspace_floats) *workspace_floats = tiles * n * p.QT * H * (dv + 2);
  return (int)n;
}

// q fp32 [T, H, d]; cache rows as above; talk fp32 [H, H] or NULL (no mix); chunk / window <= 0: none -> out fp32 [T, H, dv].
// sink fp32 [H] or NULL: a logit per head that joins the soft-max denominator (after the mix, unscaled) and carries no value.
// `partial` / nsplit: from b200_seq_talk_attn_splits (NULL / <= 1: no split).
extern "C" int b200_seq_talk_attn(const float* q, const void* cache, int dt, int64_t row_width, int k_off, int v_off, const int32_t* block_table,
                                  int64_t bt_stride, const int32_t* seq_of_token, const int32_t* cu_q, int B, const int64_t* position_ids,
                                  const float* talk, float* out, int64_t T, int H, int G, int d, int dv, int chunk, int window, float scale,
                                  int page, float* partial, int nsplit, const float* sink, void* stream) {
  if (T == 0) return B200_OK;
  if (G <= 0 || H % G != 0 || d <= 0 || dv <= 0 || dv > 256) {
    b200_set_last_error("seq_talk_attn: need heads % kv_heads == 0 and 0 < vdim <= 256");
    return B200_ERR_ARG;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const TalkPlan plan = talk_mma_plan(dt, T, B, H, G, d, dv, talk != nullptr);
  if (plan.QT > 0 && cu_q != nullptr && row_width % 8 == 0 && k_off % 8 == 0 && v_off % 8 == 0 && (reinterpret_cast<uintptr_t>(cache) & 15) == 0) {
    const int64_t tiles = (T + plan.QT - 1) / plan.QT + B;  // upper bound of sum_b ceil(n_b / QT); surplus blocks return at once
    if (!partial || nsplit < 1) nsplit = 1;
    if (nsplit > 8) nsplit = 8;
    if (tiles <= 0x7fffffff) {
      dim3 grid((unsigned)tiles, 1, (unsigned)nsplit);
      const unsigned threads = (unsigned)(plan.QT * H / 16 * 32);
#define TAM(N, KT)                                                                                                                       \
  do {                                                                                                                                   \
    static bool cfg = false;                                                                                                             \
    if (!cfg) { cudaFuncSetAttribute(talk_attn_mma_kernel<N, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); cfg = true; } \
    B200_LAUNCH((talk_attn_mma_kernel<N, KT>), grid, dim3(threads), plan.smem, st, q, (const __nv_bfloat16*)cache, row_width, k_off, v_off, \
                block_table, bt_stride, cu_q, B, position_ids, talk, out, H, G, d, plan.QT, chunk, window, scale, page, partial, sink);  \
  } while (0)
#define TAM_KT(N)                 \
  do {                            \
    if (plan.KT == 64) TAM(N, 64); \
    else if (plan.KT == 32) TAM(N, 32); \
    else TAM(N, 16);              \
  } while (0)
      switch (dv / 8) {
        case 2: TAM_KT(2); break;
        case 4: TAM_KT(4); break;
        case 8: TAM_KT(8); break;
        default: TAM_KT(16); break;
      }
#undef TAM_KT
#undef TAM
      if (nsplit > 1)
        B200_LAUNCH(talk_attn_merge_kernel, dim3((unsigned)tiles, (unsigned)((plan.QT * H + 7) / 8)), dim3(256), 0, st, (const float*)partial, out, cu_q, B, H, G, plan.QT, dv, nsplit);
      b200_count_launches(nsplit > 1 ? 2 : 1);
      return B200_OK;
    }
  }
#define TALK(N)                                                                                                                              \
  B200_SEQ_DISPATCH(dt, E, return (launch_talk_plain<E, N>(q, cache, row_width, k_off, v_off, block_table, bt_stride, seq_of_token, position_ids, \
                                                          talk, out, T, H, G, d, dv, chunk, window, scale, page, sink, st)))
  const int nv = (dv + 31) / 32;
  if (talk == nullptr) {   // no mix: blocks per key / value head group
#define GRP(N)                                                                                                                                \
  B200_SEQ_DISPATCH(dt, E, return (launch_group_plain<E, N>(q, cache, row_width, k_off, v_off, block_table, bt_stride, seq_of_token, position_ids, \
                                                           out, T, H, G, d, dv, chunk, window, scale, page, sink, st)))
    if (nv <= 1) GRP(1);
    else if (nv <= 2) GRP(2);
    else if (nv <= 4) GRP(4);
    else GRP(8);
#undef GRP
  }
  if (nv <= 1) TALK(1);
  else if (nv <= 2) TALK(2);
  else if (nv <= 4) TALK(4);
  else TALK(8);
#undef TALK
}
