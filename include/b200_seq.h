/* C ABI of libb200_seq.so: kernels of the decoder families with an fp32 residual stream (latent attention over a paged latent cache,
 * multi-head attention with differential maps or a distance bias over paged heads, state-space and matrix-memory mixers over fp32
 * state slots, routed feed-forward, row kernels around the stream).
 *
 * Conventions as in b200_tgis.h: plain device pointers + sizes + a cudaStream_t (void*), status-code return (0 = ok, the
 * message through b200_last_error()), no allocation, enqueue-only.  Element types are passed as codes: 0 = bfloat16,
 * 1 = float32.  Everything called "state", "residual", soft-max and norm statistics is fp32 whatever the element type.
 * The library also exports b200_last_error, b200_cuda_peek_error, b200_launch_count, b200_kv_alloc_* and b200_decode_advance
 * with the signatures b200_tgis.h gives them.
 *
 * A ragged step: T token rows of B sequences; sequence b owns rows cu_q[b] .. cu_q[b+1], at consecutive positions
 * position_ids[row]; seq_of_token[row] = b; slot_mapping[row] = cache row (block * page + offset); state_slots[b] = the
 * sequence's recurrent-state slot.  A sequence whose first row of the step is at position 0 starts from a zero state.
 */
#ifndef B200_SEQ_H
#define B200_SEQ_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define B200_DT_BF16 0
#define B200_DT_F32 1

/* C[z][m][n] = sum_k A[z][m][k] W[z][n][k] (+ bias[n]); fp32 accumulation in ascending k; strides in elements */
int b200_seq_linear(const void* A, int a_dt, int64_t lda, int64_t strideA, const void* W, int w_dt, int64_t ldw, int64_t strideW,
                    const void* bias, void* C, int c_dt, int64_t ldc, int64_t strideC, int64_t M, int64_t N, int64_t K, int64_t Z,
                    void* stream);
/* out[t] = table[ids[t]] * scale, fp32 */
int b200_seq_embed_scale(const void* table, int dt, const int64_t* ids, float scale, float* out, int64_t T, int64_t W, int64_t V,
                         void* stream);
/* LayerNorm with weight and bias of rows of type x_dt; resid == NULL: out (type dt) = LN(x), else resid (fp32) += LN(x) and out,
 * when given, receives the updated residual rows in type dt */
int b200_seq_layernorm(const void* x, int x_dt, const void* w, const void* b, int dt, void* out, float* resid, int64_t T, int64_t W,
                       float eps, void* stream);
/* per group of n columns: v / sqrt(mean v^2 + eps) * w; gate_kind 0 none, 1 SiLU(gate) before the statistics, 2 sigmoid(gate)
 * after the weight; groups == 0: gate only */
int b200_seq_group_rmsnorm_gate(const float* x, int64_t ldx, const float* gate, int64_t ldg, int gate_kind, const void* w, int w_dt,
                                int groups, int n, float eps, void* out, int out_dt, int64_t ldo, int64_t T, void* stream);
/* [g | u] rows -> min(g, limit) sigmoid(alpha min(g, limit)) (clamp(u, +-limit) + 1) */
int b200_seq_ff_clamped_gate(const void* gu, void* out, int dt, int64_t rows, int64_t F, float limit, float alpha, void* stream);
/* per-layer token input, around its two projections: out = gelu_tanh(a) * table[id, col0 : col0 + dim]; resid += unit_rms(y) * w */
int b200_seq_side_gate(const float* a, const int64_t* ids, const void* table, int64_t ld_table, int64_t col0, int dim, int64_t V, void* out,
                       int dt, int64_t rows, void* stream);
int b200_seq_rms_add(const float* y, const void* w, int dt, float* resid, int64_t T, int64_t W, float eps, void* stream);
/* cache row of every token = [unit_rms(latent) * w | rotated key part]; q_abs[:, :, R:] = rotated query parts */
int b200_seq_latent_prepare(const float* down, int64_t ld_down, int col_c, int col_kr, const float* q, int64_t ld_q, int q_head_stride,
                            int q_rot_off, const void* cnorm_w, const float* cos_t, const float* sin_t, const int64_t* position_ids,
                            const int64_t* slot_mapping, void* cache, int dt, float* q_abs, int64_t T, int H, int R, int r, int rot_dims,
                            float eps, void* stream);
/* out[t, h, :R] = sum_j softmax_j((q_abs[t, h] . cache_row(j)) * scale) cache_row(j)[:R], j over (p - window, p] of t's sequence.
 * b200_seq_latent_attn_splits: over how many blocks the tensor-core kernel should split each token's keys for this shape (0: the
 * shape takes the plain kernel) and the fp32 workspace (`partial`) that takes; partial NULL / nsplit <= 1: no split */
int b200_seq_latent_attn_splits(int dt, int64_t Tq, int H, int R, int r, int64_t* workspace_floats);
int b200_seq_latent_attn(const float* q_abs, const void* cache, int dt, const int32_t* block_table, int64_t bt_stride,
                         const int32_t* seq_of_token, const int64_t* position_ids, float* out, int64_t Tq, int H, int R, int r, int window,
                         float scale, int page, float* partial, int nsplit, void* stream);
/* SiLU(depth-wise causal convolution) of columns [col0, col0 + C) of u; conv_state [slots, taps - 1, C] read and advanced */
int b200_seq_causal_conv_silu(const float* u, int64_t ld_u, int col0, int C, int taps, const void* w, const void* bias, int dt,
                              float* conv_state, const int32_t* state_slots, const int32_t* seq_of_token, const int32_t* cu_q,
                              const int64_t* position_ids, float* out, int64_t T, int B, void* stream);
/* S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x, dt = softplus(raw + bias); state [slots, H, N, P] */
int b200_seq_ssm_scan(const float* xbc, int64_t ld_xbc, int col_x, int col_B, int col_C, const float* dt_raw, int64_t ld_dt, int col_dt,
                      const void* dt_bias, const void* A_log, const void* Dskip, int dt, float* state, const int32_t* state_slots,
                      const int32_t* cu_q, const int64_t* position_ids, float* y, int64_t ld_y, int B, int H, int P, int N, int groups,
                      void* stream);
/* matrix memory with exponential gating and a running maximum from 0; S [slots, H, dk, dv], n [slots, H, dk], m [slots, H] */
int b200_seq_mlstm_scan(const float* proj, int64_t ld, int col_q, int col_k, int col_v, int col_i, int col_f, const void* i_bias,
                        const void* f_bias, int dt, float cap, float q_scale, float* S_state, float* n_state, float* m_state,
                        const int32_t* state_slots, const int32_t* cu_q, const int64_t* position_ids, float* y, int64_t ld_y, int B, int H,
                        int dk, int dv, void* stream);

/* same convolution with the activation as a parameter: act 0 none, 1 SiLU; bias may be NULL */
int b200_seq_causal_conv(const float* u, int64_t ld_u, int col0, int C, int taps, const void* w, const void* bias, int dt, int act,
                         float* conv_state, const int32_t* state_slots, const int32_t* seq_of_token, const int32_t* cu_q,
                         const int64_t* position_ids, float* out, int64_t T, int B, void* stream);
/* out[t] = table[ids[t]] + pos_table[position_ids[t]], fp32 */
int b200_seq_embed_add_pos(const void* table, const void* pos_table, int dt, const int64_t* ids, const int64_t* position_ids, float* out,
                           int64_t T, int64_t W, int64_t V, int64_t P, void* stream);
/* out (type dt) = x / sqrt(mean x^2 + eps) * (w + w_offset) of fp32 rows */
int b200_seq_rmsnorm_rows(const float* x, const void* w, int dt, float w_offset, void* out, int64_t T, int64_t W, float eps, void* stream);
/* per token: unit-RMS (normalise != 0) of Hq query heads and Hk key heads of d elements, optional weights, queries times
 * 1 + temp_coef ln(floor((p + 1) / temp_every) + 1); keys to cache[slot, k_off ..], Cv values to cache[slot, v_off ..], queries to
 * q_out fp32 [T, Hq, d].  col_k / col_v < 0: the layer writes no keys / values.  Inside a block of `page` tokens the pool is
 * head-group-major: a group's k_group key heads (v_width value columns) of the block's tokens lie together */
int b200_seq_heads_prepare(const float* src, int64_t ld, int col_q, int Hq, int d, const void* qnorm_w, float temp_coef, int temp_every,
                           int col_k, int Hk, const void* knorm_w, int col_v, int Cv, int normalise, const int64_t* position_ids,
                           const int64_t* slot_mapping, void* cache, int dt, int64_t row_width, int k_off, int v_off, int page, int k_group,
                           int v_width, float* q_out, int64_t T, float eps, void* stream);
/* soft-max attention of H * maps query rows per token over G * maps paged key heads (d) and G value heads (dv) of its own sequence,
 * causal, optional window, optional bias rel[bucket(distance), head] (fp32 [rel_rows, H]) after the scale; out fp32 [Tq, H * maps, dv] */
int b200_seq_paged_attn(const float* q, const void* cache, int dt, int64_t row_width, int k_off, int v_off, const int32_t* block_table,
                        int64_t bt_stride, const int32_t* seq_of_token, const int32_t* cu_q, int B, const int64_t* position_ids, float* out,
                        int64_t Tq, int H, int G, int maps, int d, int dv, int window, float scale, int page, const float* rel,
                        const int32_t* bucket_tab, int n_bucket_tab, int rel_rows, float* partial, int nsplit, void* stream);
/* blocks to split each query tile's keys over for this step (0: plain kernel, 1: no split) and the fp32 workspace for `partial` */
int b200_seq_paged_attn_splits(int dt, int64_t Tq, int B, int H, int G, int maps, int d, int dv, int64_t* workspace_floats);
/* in fp32 [T, H, 2, dv] -> out [T, H * dv]: (a1 - lambda a2) / sqrt(mean(.^2) + eps) * out_scale */
int b200_seq_diff_combine(const float* in, void* out, int out_dt, int64_t T, int H, int dv, float lambda, float out_scale, float eps,
                          void* stream);
/* routed feed-forward: top-k of fp32 router logits with soft-max weights over the picked logits, and the plan (compact rows expert by
 * expert, tiles of 64 rows) that the grouped products and the combine read; plan = b200_seq_moe_plan_ints int32 values */
int64_t b200_seq_moe_plan_ints(int64_t T, int E, int top);
int b200_seq_moe_route(const float* logits, int64_t T, int E, int top, int32_t* ids, float* weights, int32_t* plan, void* stream);
/* C[row] = W[expert(row)] A[gather ? token(row) : row] for the T * top rows of the plan; W [E, N, K] */
int b200_seq_moe_linear(const void* A, int a_dt, int64_t lda, int gather, const void* W, int w_dt, void* C, int c_dt, int64_t ldc,
                        int32_t* plan, int64_t T, int E, int top, int64_t N, int64_t K, void* stream);
/* out [T * top, K] = A[token(row)]: compact rows for callers that run one dense product per expert (plan offsets at int E of plan) */
int b200_seq_moe_gather_rows(const void* A, int dt, int64_t lda, void* out, int32_t* plan, int64_t T, int E, int top, int64_t K, void* stream);
/* resid += mix + sum_k weights[t, k] y[row(t, k)]; mix and y may be NULL */
int b200_seq_moe_combine_add(float* resid, const float* mix, const float* y, int64_t ldy, const float* weights, int32_t* plan, int64_t T,
                             int E, int top, int64_t W, void* stream);
/* mode 0: as b200_seq_moe_route; mode 1: scores = sigmoid(logit), the picks are the largest score + correction[expert] (element type
 * corr_dt, may be NULL), weights = picked score / (sum of the picked scores + 1e-20) * weight_scale */
int b200_seq_moe_route_scored(const float* logits, int64_t T, int E, int top, int mode, const void* correction, int corr_dt, float weight_scale,
                              int32_t* ids, float* weights, int32_t* plan, void* stream);
/* resid (fp32) += v / sqrt(mean v^2 + eps) * w, v = y * sigmoid(gate) (gate NULL: y); typed (type dt, may be NULL) = the updated rows */
int b200_seq_gated_rms_add(const float* y, const float* gate, const void* w, int dt, float* resid, void* typed, int64_t T, int64_t W, float eps,
                           void* stream);
/* out (type dt) = x, n fp32 values */
int b200_seq_cast_rows(const float* x, void* out, int dt, int64_t n, void* stream);
/* rows [g | u] (type dt, 2F wide) -> act(g) * u; act 0: SiLU, 1: GELU in its tanh form */
int b200_seq_ff_gate(const void* gu, void* out, int dt, int64_t rows, int64_t F, int act, void* stream);
/* gated delta rule over fp32 state slots S [slots, H, dk, dv]: per token S <- g S, u = beta (v - S^T k), S <- S + k u^T, y = S^T q; q and k
 * (kv_heads x dk, shared by H / kv_heads heads) are made unit vectors, q times q_scale; beta = sigmoid(raw[col_b + h]),
 * g = exp(-exp(A_log[h]) softplus(raw[col_a + h] + dt_bias[h])); c holds the activated q / k / v columns; y fp32 [T, H * dv] */
int b200_seq_delta_scan(const float* c, int64_t ldc, int col_q, int col_k, int col_v, const float* raw, int64_t ldr, int col_b, int col_a,
                        const void* A_log, const void* dt_bias, int dt, float q_scale, float* S_state, const int32_t* state_slots,
                        const int32_t* cu_q, const int64_t* position_ids, float* y, int64_t ld_y, int B, int H, int kv_heads, int dk, int dv,
                        void* stream);
/* per token: RMS norm over the whole q projection (H * d columns) and the whole k projection (G * d) when whole_norm != 0 (weights per
 * column, may be NULL), rotation of the first `rot` columns of every head, column i paired with i + rot / 2 (cos / sin fp32
 * [positions, rot / 2]); keys and values to the token-major cache row [k_off: G * d | v_off: G * dv], queries to q_out fp32 [T, H * d].
 * v_rot > 0: the first v_rot columns of every value head turn by the token's position too (vcos / vsin fp32 [positions, v_rot / 2];
 * pairs are column i with i + v_rot / 2, or columns 2i and 2i + 1 when v_interleaved != 0) */
int b200_seq_qk_rot_prepare(const float* src, int64_t ld, int col_q, int col_k, int col_v, int H, int G, int d, int dv, const void* qnorm_w,
                            const void* knorm_w, int whole_norm, float eps, const float* cos_t, const float* sin_t, int rot,
                            const int64_t* position_ids, const int64_t* slot_mapping, void* cache, int dt, int64_t row_width, int k_off,
                            int v_off, float* q_out, int64_t T, const float* vcos_t, const float* vsin_t, int v_rot, int v_interleaved,
                            void* stream);
/* attention with the scaled scores mixed over the heads before the soft-max (talk fp32 [H, H], NULL: none); a query at p sees keys
 * j <= p with floor(j / chunk) == floor(p / chunk) (chunk > 0) and p - j < window (window > 0); sink fp32 [H] (NULL: none): exp(sink[h])
 * joins head h's soft-max denominator (after the mix, unscaled) and carries no value; out fp32 [T, H, dv] */
int b200_seq_talk_attn(const float* q, const void* cache, int dt, int64_t row_width, int k_off, int v_off, const int32_t* block_table,
                       int64_t bt_stride, const int32_t* seq_of_token, const int32_t* cu_q, int B, const int64_t* position_ids,
                       const float* talk, float* out, int64_t T, int H, int G, int d, int dv, int chunk, int window, float scale, int page,
                       float* partial, int nsplit, const float* sink, void* stream);
/* blocks to split each query tile's keys over for this step (0: plain kernel, 1: no split) and the fp32 workspace for `partial` */
int b200_seq_talk_attn_splits(int dt, int64_t T, int B, int H, int G, int d, int dv, int64_t* workspace_floats);
/* several residual streams per token, X fp32 [T, S, W] in place (S <= 8).  init (fp32 [T, W], may be NULL): every stream starts as this
 * row and X is not read.  y (fp32 [T, W], may be NULL): all streams at once from the old ones, X_t <- sum_s mix[s * S + t] X_s +
 * out_coef[t] y.  in_coef (fp32 [S], may be NULL): u = sum_s in_coef[s] X_s of the new streams and typed (type dt) <-
 * u / sqrt(mean u^2 + eps) * w (w of type dt; NULL: typed <- u) */
int b200_seq_streams_step(float* X, int S, const float* init, const float* y, const float* mix, const float* out_coef, const float* in_coef,
                          const void* w, int dt, void* typed, int64_t T, int64_t W, float eps, void* stream);
/* out (dense rows of type out_dt) = act(in) over rows of F columns with leading dimension ld_in; act 0: SiLU, 1: GELU in its tanh form,
 * 2: tanh; element types fp32 -> any or bf16 -> bf16 */
int b200_seq_ff_act(const void* in, int in_dt, int64_t ld_in, void* out, int out_dt, int64_t rows, int64_t F, int act, void* stream);
/* a fp32 [T, H, dv]: the first `rot` columns of every head turn by minus the token's position (cos / sin fp32 [positions, rot / 2]; pairs
 * as in b200_seq_qk_rot_prepare's values), the head is multiplied by sigmoid(gate[t * ld_gate + h]) (gate NULL: by 1) and by out_scale
 * -> out rows of type dt with leading dimension ld_out, H * dv columns written */
int b200_seq_heads_turn_gate(const float* a, const float* gate, int64_t ld_gate, const float* cos_t, const float* sin_t, int rot,
                             int interleaved, const int64_t* position_ids, void* out, int dt, int64_t ld_out, float out_scale, int64_t T, int H,
                             int dv, void* stream);
/* generalised delta rule over fp32 state slots S [slots, H, dk, dv]: per token, with u = k / sqrt(sum k^2 + 1e-6),
 * S <- diag(w) S - (a * u)(u^T S) + k v^T (the old S on the right), y = S^T r; w = exp(-decay_scale sigmoid(dec[col_d + h dk + n] +
 * w0[h dk + n])), a = sigmoid(raw[col_a + h dk + n] + a_bias[h dk + n]); r, k, a: H x dk columns of raw, v: H x dv; y fp32 [T, H * dv] */
int b200_seq_gdelta_scan(const float* raw, int64_t ldr, int col_r, int col_k, int col_v, int col_a, const float* dec, int64_t ldd, int col_d,
                         const void* a_bias, const void* w0, int dt, float decay_scale, float* S_state, const int32_t* state_slots,
                         const int32_t* cu_q, const int64_t* position_ids, float* y, int64_t ld_y, int B, int H, int dk, int dv, void* stream);
/* minimal gated recurrent unit over fp32 state slots [slots, C]: z = sigmoid(proj[col_z + c] + z_bias[c]), x = proj[col_x + c] + x_bias[c],
 * candidate = x + 1/2 (x >= 0) or sigmoid(x), S <- (1 - z) S + z candidate; out (type out_dt) = S * SiLU(proj[col_g + c]) (col_g < 0: S), times out_scale */
int b200_seq_mingru_scan(const float* proj, int64_t ld, int col_z, int col_x, int col_g, const void* z_bias, const void* x_bias, int dt,
                         float* state, const int32_t* state_slots, const int32_t* cu_q, const int64_t* position_ids, void* out, int out_dt,
                         int64_t ld_out, float out_scale, int64_t T, int B, int C, void* stream);

#ifdef __cplusplus
}
#endif
#endif
