"""Sequence mixers beyond plain multi-head attention, each with its constants as constructor arguments so that any decoder
family can compose them: latent attention over a paged latent cache (sliding window, rotary part with optional YaRN frequency
scaling), the selective state-space mixer (Mamba-2 form), the matrix-memory mixer (mLSTM), differential attention (two soft-max
maps per head, short convolutions after the projections, optionally over another layer's keys and values), attention with a
learned bias per log-spaced distance bucket, the gated delta rule, attention with head-mixed scores under a chunked mask,
windowed attention with sink logits, position-carrying values and a gate per head, the minimal gated recurrent unit, two mixers
side by side on shared products, the generalised delta rule, and the feed-forward layers (clamped gated MLP, gated MLP with
biases, plain MLP, routed experts with an optional shared expert).

A mixer declares what it keeps per sequence (`cache_spec`): a row of the paged cache per token, or fp32 state tensors in a
state slot.  `forward(h, step, store)` takes the normed hidden states of a ragged step (ops_seq.RaggedStep: any mix of whole
prompts, portions of prompts and single decoded tokens) and the layer's store from the cache manager (utils/paged.py
`HybridCacheManager`).  Kernels: csrc/seq_*.cu through ops_seq.py.  Projections accumulate in fp32; soft-max, norms, gates of
the recurrences and the states are fp32 whatever the element type.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
from torch import nn

from .. import ops_seq as ops
from .paged import LayerCacheSpec


def _need_single_rank(weights, what: str):
    if weights.process_group.size() != 1:
        raise NotImplementedError(f"{what} is not sharded: run it on one rank")


class ScaledRotaryTables:
    """cos / sin of position * frequency of every rotated pair, fp32 [positions, dims / 2], grown on demand (which columns form
    pair i - neighbours or halves - is the kernel's business).
    frequency_i = base^(-2i/dims).  With `scaling` = {factor, original, fast, slow} (YaRN): pairs that turn more than `fast`
    times over `original` positions keep their frequency, pairs that turn fewer than `slow` times are slowed by `factor`, a
    linear ramp over the pair index in between; cos and sin are multiplied by 0.1 ln(factor) + 1."""

    def __init__(self, dims: int, base: float, scaling: Optional[dict] = None):
        if dims % 2:
            raise ValueError("rotary dims must be even")
        self.dims, self.base, self.scaling = int(dims), float(base), scaling
        self._cos = self._sin = None

    def frequencies(self) -> torch.Tensor:
        i = torch.arange(self.dims // 2, dtype=torch.float64)
        freq = self.base ** (-2.0 * i / self.dims)
        sc = self.scaling
        if sc:
            def pair_turning(turns: float) -> float:  # (fractional) pair index that makes `turns` turns over the original length
                return self.dims * math.log(float(sc["original"]) / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
            lo = max(math.floor(pair_turning(float(sc["fast"]))), 0)
            hi = min(math.ceil(pair_turning(float(sc["slow"]))), self.dims - 1)
            ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            freq = freq / float(sc["factor"]) * ramp + freq * (1.0 - ramp)
        return freq

    def amplitude(self) -> float:
        return 0.1 * math.log(float(self.scaling["factor"])) + 1.0 if self.scaling else 1.0

    def tables(self, n_pos: int, device):
        if self._cos is None or self._cos.shape[0] < n_pos or self._cos.device != torch.device(device):
            n = max(256, 1 << (max(int(n_pos), 1) - 1).bit_length())
            ang = torch.arange(n, dtype=torch.float64)[:, None] * self.frequencies()[None, :]
            amp = self.amplitude()
            self._cos = (torch.cos(ang) * amp).to(torch.float32).to(device).contiguous()
            self._sin = (torch.sin(ang) * amp).to(torch.float32).to(device).contiguous()
        return self._cos, self._sin


class LatentAttention(nn.Module):
    """Multi-head attention whose keys and values are up-projections of one latent per token (rank `kv_rank`) plus one rotated
    key part (`rot_dim`) shared by all heads; queries go through a latent of rank `q_rank`.  Only the normalised latent and the
    rotated key part are cached: `kv_rank + rot_dim` elements per token and layer.  The kernels work in the absorbed form (the
    key up-projection is applied to the query, the value up-projection to the attention output), for prompts and decoding alike.
    Tensors under `prefix`: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g (sigmoid gate on the concatenated heads), o."""

    def __init__(self, prefix: str, weights, *, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, q_rank: int, scale: float,
                 window: Optional[int], rotary: ScaledRotaryTables, eps: float):
        super().__init__()
        _need_single_rank(weights, "LatentAttention")
        self.H, self.d, self.r, self.dv, self.R, self.Q = heads, dim, rot_dim, vdim, kv_rank, q_rank
        self.scale, self.window, self.rotary, self.eps = float(scale), int(window or 0), rotary, float(eps)
        if rotary.dims > rot_dim:
            raise ValueError("rotary dims exceed the rotated part")
        get = lambda n: weights.get_tensor(f"{prefix}.{n}")  # noqa: E731
        self.w_in = torch.cat([get("dq"), get("dkv"), get("g")], 0).contiguous()          # -> [q latent | kv latent | key part | gate]
        self.dq_norm, self.dkv_norm = get("dq.norm"), get("dkv.norm")
        self.w_uq = get("uq").contiguous()                                               # rows head by head: [dim plain | rot_dim rotated]
        self.w_uk_t = get("uk").view(heads, dim, kv_rank).transpose(1, 2).contiguous()   # [H, R, d]: q~ = Wuk_h^T q_plain
        self.w_uv = get("uv").view(heads, vdim, kv_rank).contiguous()
        self.w_o = get("o").contiguous()
        self.dtype = self.w_o.dtype

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="paged", row_width=self.R + self.r)

    def forward(self, h: torch.Tensor, step: ops.RaggedStep, store, max_s: int) -> torch.Tensor:
        H, d, r, dv, R, Q = self.H, self.d, self.r, self.dv, self.R, self.Q
        T = step.T
        down = ops.linear(h, self.w_in, out_dtype=torch.float32)
        cq = ops.group_rmsnorm_gate(down[:, :Q], self.dq_norm, 1, self.eps, self.dtype)
        q = ops.linear(cq, self.w_uq, out_dtype=torch.float32)
        q_abs = torch.empty(T, H, R + r, dtype=torch.float32, device=h.device)
        cos, sin = self.rotary.tables(max_s, h.device)
        ops.latent_prepare(down, Q, Q + R, q, d + r, d, self.dkv_norm, cos, sin, step, store, q_abs, H, R, r, self.rotary.dims, self.eps)
        ops.linear_per_head(q.view(T, H, d + r)[:, :, :d], self.w_uk_t, q_abs[:, :, :R])
        o_lat = ops.latent_attn(q_abs, store, step, R, r, self.window, self.scale)
        o = torch.empty(T, H, dv, dtype=torch.float32, device=h.device)
        ops.linear_per_head(o_lat, self.w_uv, o)
        gated = ops.group_rmsnorm_gate(o.view(T, H * dv), None, 0, self.eps, self.dtype, gate=down[:, Q + R + r:],
                                       gate_kind=ops.GATE_SIGMOID_AFTER)
        return ops.linear(gated, self.w_o)


class Mamba2Mixer(nn.Module):
    """Selective state-space mixer: in-projection [z | x | B | C | dt], depth-wise causal convolution + SiLU over [x | B | C],
    per head S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x, then y * SiLU(z), RMS norm in `norm_groups` parts, out-projection.
    State per sequence: S [heads, state, vdim] and the last conv - 1 convolution inputs, both fp32.
    Tensors under `prefix`: in, conv, conv.b, dt_bias, A_log, D, norm, o."""

    def __init__(self, prefix: str, weights, *, heads: int, vdim: int, state: int, groups: int, conv: int, norm_groups: int, eps: float):
        super().__init__()
        _need_single_rank(weights, "Mamba2Mixer")
        self.H, self.P, self.N, self.G, self.taps, self.norm_groups, self.eps = heads, vdim, state, groups, conv, norm_groups, float(eps)
        get = lambda n: weights.get_tensor(f"{prefix}.{n}").contiguous()  # noqa: E731
        self.w_in, self.conv_w, self.conv_b = get("in"), get("conv"), get("conv.b")
        self.dt_bias, self.A_log, self.D, self.norm_w, self.w_o = get("dt_bias"), get("A_log"), get("D"), get("norm"), get("o")
        self.inner = heads * vdim
        self.channels = self.inner + 2 * groups * state
        self.dtype = self.w_o.dtype

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="state", state={"S": (self.H, self.N, self.P), "conv": (max(self.taps - 1, 1), self.channels)})

    def forward(self, h: torch.Tensor, step: ops.RaggedStep, store: Dict[str, torch.Tensor], max_s: int) -> torch.Tensor:
        inner, GN = self.inner, self.G * self.N
        u = ops.linear(h, self.w_in, out_dtype=torch.float32)
        xbc = ops.causal_conv_silu(u, inner, self.channels, self.conv_w, self.conv_b, store["conv"], step)
        y = ops.ssm_scan(xbc, 0, inner, inner + GN, u, 2 * inner + 2 * GN, self.dt_bias, self.A_log, self.D, store["S"], step, self.H, self.P,
                         self.N, self.G)
        gated = ops.group_rmsnorm_gate(y, self.norm_w, self.norm_groups, self.eps, self.dtype, gate=u[:, :inner], gate_kind=ops.GATE_SILU_BEFORE)
        return ops.linear(gated, self.w_o)


class MLSTMMixer(nn.Module):
    """Matrix-memory mixer: per head a [dim, vdim] memory S, a normaliser n and a running maximum m (from 0) of the log gates;
    log input gate cap tanh(./cap), log forget gate logsigmoid(cap tanh(./cap)); read-out S^T q / (max(|n.q|, e^-m) + 1e-6) with
    q scaled by dim^-1/2, per-head unit-RMS, weight, sigmoid output gate, out-projection.  State fp32.
    Tensors under `prefix`: q, k, v, g, i, i.b, f, f.b, norm, o."""

    def __init__(self, prefix: str, weights, *, heads: int, dim: int, vdim: int, gate_cap: float, eps: float,
                 out_dtype: Optional[torch.dtype] = None):
        """`out_dtype`: element type of the result (None: the projections' type; torch.float32 for a stream that adds it in fp32)"""
        super().__init__()
        _need_single_rank(weights, "MLSTMMixer")
        self.out_dtype = out_dtype
        self.H, self.d, self.dv, self.cap, self.eps = heads, dim, vdim, float(gate_cap), float(eps)
        get = lambda n: weights.get_tensor(f"{prefix}.{n}").contiguous()  # noqa: E731
        self.w_in = torch.cat([get("q"), get("k"), get("v"), get("g"), get("i"), get("f")], 0).contiguous()
        self.i_b, self.f_b, self.norm_w, self.w_o = get("i.b"), get("f.b"), get("norm"), get("o")
        self.dtype = self.w_o.dtype

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="state", state={"S": (self.H, self.d, self.dv), "n": (self.H, self.d), "m": (self.H,)})

    def forward(self, h: torch.Tensor, step: ops.RaggedStep, store: Dict[str, torch.Tensor], max_s: int) -> torch.Tensor:
        H, d, dv = self.H, self.d, self.dv
        qk, vg = 2 * H * d, 2 * H * dv
        proj = ops.linear(h, self.w_in, out_dtype=torch.float32)  # [q | k | v | g | i | f]
        y = ops.mlstm_scan(proj, 0, H * d, qk, qk + vg, qk + vg + H, self.i_b, self.f_b, self.cap, d ** -0.5, store["S"], store["n"],
                           store["m"], step, H, d, dv)
        gated = ops.group_rmsnorm_gate(y, self.norm_w, H, self.eps, self.dtype, gate=proj[:, qk + H * dv:qk + vg],
                                       gate_kind=ops.GATE_SIGMOID_AFTER)
        return ops.linear(gated, self.w_o, out_dtype=self.out_dtype)


class ClampedGatedMLP(nn.Module):
    """down(g' * sigmoid(alpha g') * (u' + 1)) with g' = min(gate(x), limit), u' = clamp(up(x), -limit, limit).
    Tensors under `prefix`: gate, up, down."""

    def __init__(self, prefix: str, weights, *, limit: float, alpha: float = 1.702):
        super().__init__()
        _need_single_rank(weights, "ClampedGatedMLP")
        self.limit, self.alpha = float(limit), float(alpha)
        self.w_gate_up = torch.cat([weights.get_tensor(f"{prefix}.gate"), weights.get_tensor(f"{prefix}.up")], 0).contiguous()
        self.w_down = weights.get_tensor(f"{prefix}.down").contiguous()

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return ops.linear(ops.ff_clamped_gate(ops.linear(h, self.w_gate_up), self.limit, self.alpha), self.w_down)


def log_distance_buckets(rows: int, far: float) -> List[int]:
    """bucket of every distance up to the first one that reaches the last row: distances below rows // 2 have a row each, from there
    rows are spaced evenly in ln(distance) up to `far`; every larger distance takes the last row"""
    half = rows // 2
    if half < 1 or far <= half:
        raise ValueError("distance buckets need at least two rows and a far distance beyond rows / 2")
    out, n = [], 0
    while True:
        b = n if n < half else min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))
        out.append(b)
        if b >= rows - 1:
            return out
        n += 1


class DifferentialAttention(nn.Module):
    """Grouped-query attention with two soft-max maps per head over the same values: o = a1 - lambda a2, unit-RMS per head, times
    (1 - diff); lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff.  Queries and keys hold [map 1 | map 2] per head.  A depth-wise
    causal convolution (`conv` taps, no bias) follows each of the q / k / v projections; queries and keys are then RMS-normed per
    head and map with a weight shared by all heads, and queries are multiplied by 1 + temp_coef ln(floor((p + 1) / temp_every) + 1).
    No rotation.  Per sequence and token: the keys after convolution and norm and the values after convolution in the block pool
    (head-group-major inside a block, ops_seq.heads_prepare), and the last
    conv - 1 projected rows (fp32 state slot).  `own_kv` False: the layer has no key / value tensors and reads the rows of another
    layer with the same head counts (its `forward` is given that layer's pool).
    Tensors under `prefix`: q, q.conv, q.norm, [k, k.conv, k.norm, v, v.conv,] lq1, lk1, lq2, lk2, o."""

    def __init__(self, prefix: str, weights, *, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, scale: float, diff: float,
                 temp_coef: float, temp_every: int, eps: float, own_kv: bool = True, window: Optional[int] = None):
        super().__init__()
        _need_single_rank(weights, "DifferentialAttention")
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.H, self.G, self.d, self.dv, self.taps = heads, kv_heads, dim, vdim, int(conv)
        self.scale, self.diff, self.eps, self.own_kv, self.window = float(scale), float(diff), float(eps), bool(own_kv), int(window or 0)
        self.temp_coef, self.temp_every = float(temp_coef), int(temp_every)
        get = lambda n: weights.get_tensor(f"{prefix}.{n}")  # noqa: E731
        names = ["q", "k", "v"] if own_kv else ["q"]
        self.w_in = torch.cat([get(n) for n in names], 0).contiguous()                   # -> [q | k | v]
        self.conv_w = torch.cat([get(f"{n}.conv") for n in names], 0).contiguous()
        self.q_norm = get("q.norm").contiguous()
        self.k_norm = get("k.norm").contiguous() if own_kv else None
        lam = [(get(a).float() * get(b).float()).sum() for a, b in (("lq1", "lk1"), ("lq2", "lk2"))]
        self.lam = float(torch.exp(lam[0]) - torch.exp(lam[1])) + self.diff
        self.w_o = get("o").contiguous()
        self.dtype = self.w_o.dtype
        self.cq, self.ck, self.cv = heads * 2 * dim, kv_heads * 2 * dim, kv_heads * vdim
        self.channels = self.cq + (self.ck + self.cv if own_kv else 0)
        if self.w_in.shape[0] != self.channels or self.conv_w.shape != (self.channels, self.taps):
            raise ValueError(f"{prefix}: projection / convolution shapes do not match the head sizes")

    def cache_spec(self) -> LayerCacheSpec:
        state = {"conv": (max(self.taps - 1, 1), self.channels)}
        return LayerCacheSpec(kind="paged", row_width=self.ck + self.cv, state=state) if self.own_kv else LayerCacheSpec(kind="state", state=state)

    def forward(self, h: torch.Tensor, step: ops.RaggedStep, pages: torch.Tensor, state: Dict[str, torch.Tensor], max_s: int) -> torch.Tensor:
        """`pages`: this layer's pool, or the pool of the layer whose keys and values it reads -> fp32 [T, width]"""
        u = ops.linear(h, self.w_in, out_dtype=torch.float32)
        c = ops.causal_conv(u, 0, self.channels, self.conv_w, None, state["conv"], step)
        own = self.own_kv
        q = ops.heads_prepare(c, col_q=0, q_heads=self.H * 2, dim=self.d, q_norm_w=self.q_norm, temp_coef=self.temp_coef,
                              temp_every=self.temp_every, col_k=self.cq if own else -1, k_heads=self.G * 2, k_norm_w=self.k_norm,
                              col_v=self.cq + self.ck if own else -1, v_width=self.cv, normalise=True, step=step, cache=pages, k_off=0,
                              v_off=self.ck, k_group=2, v_group_width=self.dv, eps=self.eps)
        a = ops.paged_attn(q, pages, step, heads=self.H, kv_heads=self.G, maps=2, vdim=self.dv, k_off=0, v_off=self.ck, scale=self.scale,
                           window=self.window)
        o = ops.diff_combine(a, self.H, self.dv, self.lam, 1.0 - self.diff, self.eps, self.dtype)
        return ops.linear(o, self.w_o, out_dtype=torch.float32)


class BucketBiasAttention(nn.Module):
    """Grouped-query attention whose values are the keys as projected (there is no value projection), with biases on the q / k
    projections, queries and keys divided by their RMS per head (no weight), a learned bias rel[bucket(i - j), head] added to the
    scaled score (`log_distance_buckets` over the table's rows and `bias_max`), and sigmoid(W_g h) multiplied into the concatenated
    heads before the output projection.  No rotation.  Cached per token: the unit-RMS keys and the keys as projected (the values).
    Tensors under `prefix`: q, q.b, k, k.b, rel, g, o."""

    def __init__(self, prefix: str, weights, *, heads: int, kv_heads: int, dim: int, scale: float, bias_max: float, eps: float,
                 window: Optional[int] = None):
        super().__init__()
        _need_single_rank(weights, "BucketBiasAttention")
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.H, self.G, self.d, self.scale, self.eps, self.window = heads, kv_heads, dim, float(scale), float(eps), int(window or 0)
        get = lambda n: weights.get_tensor(f"{prefix}.{n}")  # noqa: E731
        self.w_in = torch.cat([get("q"), get("k"), get("g")], 0).contiguous()            # -> [q | k | gate]
        self.b_in = torch.cat([get("q.b"), get("k.b"), torch.zeros_like(get("q.b"))], 0).contiguous()
        rel = get("rel")
        if rel.shape[1] != heads:
            raise ValueError(f"{prefix}.rel: one column per head expected")
        self.rel = rel.float().contiguous()
        self.bucket_tab = torch.tensor(log_distance_buckets(rel.shape[0], float(bias_max)), dtype=torch.int32).to(rel.device)
        self.w_o = get("o").contiguous()
        self.dtype = self.w_o.dtype

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="paged", row_width=2 * self.G * self.d)

    def forward(self, h: torch.Tensor, step: ops.RaggedStep, pages: torch.Tensor, state, max_s: int) -> torch.Tensor:
        H, G, d = self.H, self.G, self.d
        u = ops.linear(h, self.w_in, self.b_in, out_dtype=torch.float32)
        q = ops.heads_prepare(u, col_q=0, q_heads=H, dim=d, q_norm_w=None, temp_coef=0.0, temp_every=0, col_k=H * d, k_heads=G, k_norm_w=None,
                              col_v=H * d, v_width=G * d, normalise=True, step=step, cache=pages, k_off=0, v_off=G * d, k_group=1,
                              v_group_width=d, eps=self.eps)
        a = ops.paged_attn(q, pages, step, heads=H, kv_heads=G, maps=1, vdim=d, k_off=0, v_off=G * d, scale=self.scale, window=self.window,
                           rel=self.rel, bucket_tab=self.bucket_tab)
        gated = ops.group_rmsnorm_gate(a.view(step.T, H * d), None, 0, self.eps, self.dtype, gate=u[:, (H + G) * d:],
                                       gate_kind=ops.GATE_SIGMOID_AFTER)
        return ops.linear(gated, self.w_o, out_dtype=torch.float32)


class RoutedExperts(nn.Module):
    """Mixture of gated experts without biases: router logits in fp32, `top` experts per token.  Routing rule: the largest logits
    with weights = soft-max over the picked logits, or (`sigmoid_scores`) the largest sigmoid(logit) + correction with weights =
    picked sigmoid(logit) / their sum * `weight_scale`.  Expert: down(act(gate x) . up x), act = the clamped form of
    `ClampedGatedMLP` (`limit` given: g' sigmoid(alpha g') (u' + 1)) or plain SiLU(g) u (`limit` None).  `forward` returns the
    experts' outputs as compact rows (expert by expert) with the routing; `ops.moe_combine_add` sums them into the stream.
    Tensors under `prefix`: router, [correction,] e<j>.gate, e<j>.up, e<j>.down."""

    dense_rows_per_expert = 64   # average rows per expert from which a step runs one dense product per expert

    def __init__(self, prefix: str, weights, *, experts: int, top: int, limit: Optional[float], alpha: float = 1.702,
                 sigmoid_scores: bool = False, correction: bool = False, weight_scale: float = 1.0):
        super().__init__()
        _need_single_rank(weights, "RoutedExperts")
        self.E, self.top, self.limit, self.alpha = int(experts), int(top), None if limit is None else float(limit), float(alpha)
        self.sigmoid_scores, self.weight_scale = bool(sigmoid_scores), float(weight_scale)
        get = lambda n: weights.get_tensor(f"{prefix}.{n}")  # noqa: E731
        self.correction = get("correction").contiguous() if correction else None
        self.w_router = get("router").contiguous()
        self.w_gate_up = torch.stack([torch.cat([get(f"e{e}.gate"), get(f"e{e}.up")], 0) for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([get(f"e{e}.down") for e in range(self.E)]).contiguous()
        if self.w_router.shape[0] != self.E:
            raise ValueError(f"{prefix}.router: one row per expert expected")

    def _act(self, gu: torch.Tensor) -> torch.Tensor:
        return ops.ff_gate(gu, ops.ACT_SILU) if self.limit is None else ops.ff_clamped_gate(gu, self.limit, self.alpha)

    def forward(self, h: torch.Tensor):
        routing = ops.moe_route(ops.linear(h, self.w_router, out_dtype=torch.float32), self.top, sigmoid_scores=self.sigmoid_scores,
                                correction=self.correction, weight_scale=self.weight_scale)
        rows = h.shape[0] * self.top
        if h.dtype == torch.bfloat16 and rows >= self.dense_rows_per_expert * self.E and not torch.cuda.is_current_stream_capturing():
            # prompts: enough rows per expert for the tcgen05 product (ops.linear) to pay - one product per expert over its run of
            # compact rows; the runs' bounds are read back once per layer, so this form stays out of captured decode graphs
            offs = ops.moe_expert_offsets(routing)
            a = ops.moe_gather_rows(h, routing)
            gu = torch.empty(rows, self.w_gate_up.shape[1], dtype=h.dtype, device=h.device)
            for e in range(self.E):
                if offs[e + 1] > offs[e]:
                    ops.linear(a[offs[e]:offs[e + 1]], self.w_gate_up[e], out=gu[offs[e]:offs[e + 1]])
            act = self._act(gu)
            y = torch.empty(rows, self.w_down.shape[1], dtype=torch.float32, device=h.device)
            for e in range(self.E):
                if offs[e + 1] > offs[e]:
                    ops.linear(act[offs[e]:offs[e + 1]], self.w_down[e], out=y[offs[e]:offs[e + 1]])
            return y, routing
        gu = ops.moe_linear(h, self.w_gate_up, routing, gather=True, out_dtype=h.dtype)
        return ops.moe_linear(self._act(gu), self.w_down, routing, gather=False, out_dtype=torch.float32), routing


class GatedMLP(nn.Module):
    """down(act(gate x + b_g) * (up x + b_u)) + b_d with act SiLU or the tanh form of GELU; biases optional.  The result is fp32.
    Tensors under `prefix`: gate, up, down [, gate.b, up.b, down.b]."""

    def __init__(self, prefix: str, weights, *, activation: str, bias: bool):
        super().__init__()
        _need_single_rank(weights, "GatedMLP")
        if activation not in ("silu", "gelu_tanh"):
            raise NotImplementedError(f"activation {activation!r}")
        self.act = ops.ACT_SILU if activation == "silu" else ops.ACT_GELU_TANH
        get = lambda n: weights.get_tensor(f"{prefix}.{n}")  # noqa: E731
        self.w_gate_up = torch.cat([get("gate"), get("up")], 0).contiguous()
        self.w_down = get("down").contiguous()
        self.b_gate_up = torch.cat([get("gate.b"), get("up.b")], 0).contiguous() if bias else None
        self.b_down = get("down.b").contiguous() if bias else None

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return ops.linear(ops.ff_gate(ops.linear(h, self.w_gate_up, self.b_gate_up), self.act), self.w_down, self.b_down, out_dtype=torch.float32)


class GatedDeltaMixer(nn.Module):
    """Gated delta rule: per head a [dim, vdim] memory S in fp32; every token S <- g S, u = beta (v - S^T k), S <- S + k u^T,
    o = S^T q (the read-out sees the token's own write).  q / k (kv_heads x dim, shared by heads / kv_heads heads) and v
    (heads x vdim) pass a depth-wise causal convolution (`conv` taps, no bias) and SiLU; q and k become unit vectors
    (x / sqrt(sum x^2 + 1e-6)), q times dim^-1/2; beta = sigmoid(W_b h), g = exp(-exp(A_log) softplus(W_a h + dt_bias)).  Each
    head's o is divided by its RMS, times a weight shared by the heads, times SiLU(W_g h); then the output projection.
    State per sequence: S and the last conv - 1 convolution inputs, both fp32.
    Tensors under `prefix`: q, q.conv, k, k.conv, v, v.conv, b, a, A_log, dt_bias, g, norm, o."""

    def __init__(self, prefix: str, weights, *, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, eps: float):
        super().__init__()
        _need_single_rank(weights, "GatedDeltaMixer")
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.H, self.G, self.d, self.dv, self.taps, self.eps = int(heads), int(kv_heads), int(dim), int(vdim), int(conv), float(eps)
        get = lambda n: weights.get_tensor(f"{prefix}.{n}")  # noqa: E731
        self.cqk, self.cv = self.G * self.d, self.H * self.dv
        self.channels = 2 * self.cqk + self.cv                                            # convolved columns [q | k | v]
        self.w_in = torch.cat([get(n) for n in ("q", "k", "v", "g", "b", "a")], 0).contiguous()   # -> [q | k | v | gate | beta | decay]
        self.conv_w = torch.cat([get(f"{n}.conv") for n in ("q", "k", "v")], 0).contiguous()
        self.A_log, self.dt_bias = get("A_log").contiguous(), get("dt_bias").contiguous()
        self.norm_w = get("norm").repeat(self.H).contiguous()                            # one entry per column of the heads
        self.w_o = get("o").contiguous()
        self.dtype = self.w_o.dtype
        if self.w_in.shape[0] != self.channels + self.cv + 2 * self.H or self.conv_w.shape != (self.channels, self.taps):
            raise ValueError(f"{prefix}: projection / convolution shapes do not match the head sizes")

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="state", state={"S": (self.H, self.d, self.dv), "conv": (max(self.taps - 1, 1), self.channels)})

    def forward(self, h: torch.Tensor, step: ops.RaggedStep, pages, state: Dict[str, torch.Tensor], max_s: int) -> torch.Tensor:
        """-> fp32 [T, width]"""
        C, cv, H = self.channels, self.cv, self.H
        u = ops.linear(h, self.w_in, out_dtype=torch.float32)
        c = ops.causal_conv(u, 0, C, self.conv_w, None, state["conv"], step, act_silu=True)
        y = ops.delta_scan(c, 0, self.cqk, 2 * self.cqk, u, C + cv, C + cv + H, self.A_log, self.dt_bias, self.d ** -0.5, state["S"], step,
                           H, self.G, self.d, self.dv)
        gated = ops.group_rmsnorm_gate(y, self.norm_w, H, self.eps, self.dtype, gate=u[:, C:C + cv], gate_kind=ops.GATE_SILU_AFTER)
        return ops.linear(gated, self.w_o, out_dtype=torch.float32)


class TalkingHeadsAttention(nn.Module):
    """Grouped-query attention whose scaled scores are mixed over the query heads before the soft-max, s'_h = sum_g talk[h, g] s_g.
    Queries and keys are RMS-normed over their whole projection (all heads at once, a weight per column) and then rotated on the
    first `rotary.dims` columns of every head in the rotate-half layout (column i with column i + dims / 2; `rotary` None: no
    rotation).  Mask: causal, within chunks of `chunk` positions counted from the start of the sequence (None: plain causal),
    optionally a sliding window.  Cached per token: the rotated keys and the values of all key heads (token-major row).
    Tensors under `prefix`: q, k, v, q.norm, k.norm, talk, o."""

    def __init__(self, prefix: str, weights, *, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, rotary: Optional[ScaledRotaryTables],
                 chunk: Optional[int], eps: float, window: Optional[int] = None, talk: bool = True):
        super().__init__()
        _need_single_rank(weights, "TalkingHeadsAttention")
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.H, self.G, self.d, self.dv = int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.rotary, self.chunk, self.window, self.eps = float(scale), rotary, int(chunk or 0), int(window or 0), float(eps)
        if rotary is not None and rotary.dims > dim:
            raise ValueError("rotary dims exceed the head size")
        get = lambda n: weights.get_tensor(f"{prefix}.{n}")  # noqa: E731
        self.w_in = torch.cat([get("q"), get("k"), get("v")], 0).contiguous()
        self.q_norm, self.k_norm = get("q.norm").contiguous(), get("k.norm").contiguous()
        self.talk = get("talk").float().contiguous() if talk else None
        self.w_o = get("o").contiguous()
        self.dtype = self.w_o.dtype
        self.cq, self.ck, self.cv = self.H * self.d, self.G * self.d, self.G * self.dv
        if self.w_in.shape[0] != self.cq + self.ck + self.cv or (self.talk is not None and self.talk.shape != (self.H, self.H)):
            raise ValueError(f"{prefix}: projection shapes do not match the head sizes")

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="paged", row_width=self.ck + self.cv)

    def forward(self, h: torch.Tensor, step: ops.RaggedStep, pages: torch.Tensor, state, max_s: int) -> torch.Tensor:
        """-> fp32 [T, width]"""
        u = ops.linear(h, self.w_in, out_dtype=torch.float32)
        cos, sin = self.rotary.tables(max_s, h.device) if self.rotary is not None else (None, None)
        q = ops.qk_rot_prepare(u, col_q=0, col_k=self.cq, col_v=self.cq + self.ck, heads=self.H, kv_heads=self.G, dim=self.d, vdim=self.dv,
                               q_norm_w=self.q_norm, k_norm_w=self.k_norm, whole_norm=True, eps=self.eps, cos=cos, sin=sin,
                               rot=self.rotary.dims if self.rotary is not None else 0, step=step, cache=pages, k_off=0, v_off=self.ck)
        a = ops.talk_attn(q, pages, step, kv_heads=self.G, vdim=self.dv, k_off=0, v_off=self.ck, scale=self.scale, talk=self.talk,
                          chunk=self.chunk, window=self.window)
        o = ops.cast_rows(a.view(step.T, self.H * self.dv), self.dtype)
        return ops.linear(o, self.w_o, out_dtype=torch.float32)


class SinkRotaryAttention(nn.Module):
    """Grouped-query attention over a sliding window with a learned sink logit per head in the soft-max denominator (the sink has
    no key and no value: it only takes weight), a sigmoid gate per head on the result, and values that carry their position:
    a value is turned over `value_rotary.dims` of its columns by its own position before it is cached, and every head's result
    is turned back by the query's position, so the result only sees position differences.  Before that: an optional depth-wise
    causal convolution (`conv` taps, no bias, no activation) after each of the q / k / v projections, an RMS norm over the whole q
    and the whole k projection (a weight per column), rotation of the first `rotary.dims` columns of every q / k head (column i
    with column i + dims / 2).  Cached per token: rotated keys and turned values of all key heads (token-major row); per
    sequence: the last conv - 1 projected rows (fp32).
    A mixer that can share its input and output products with a neighbour: `in_rows()` are the rows it adds to the input
    projection, `from_projection` continues from the fp32 projection and leaves the gated heads, times `out_scale`, in `out`;
    `w_o` finishes.
    Tensors under `prefix`: q, k, v, [q.conv, k.conv, v.conv,] q.norm, k.norm, [sink,] [g,] o."""

    def __init__(self, prefix: str, weights, *, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, rotary: Optional[ScaledRotaryTables],
                 value_rotary: Optional[ScaledRotaryTables], value_pairs: str = "halves", conv: int = 0, window: Optional[int] = None,
                 sink: bool = True, head_gate: bool = True, eps: float = 1e-6):
        super().__init__()
        _need_single_rank(weights, "SinkRotaryAttention")
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if value_pairs not in ("halves", "interleaved"):
            raise ValueError("value_pairs is 'halves' or 'interleaved'")
        self.H, self.G, self.d, self.dv, self.taps = int(heads), int(kv_heads), int(dim), int(vdim), int(conv or 0)
        self.scale, self.rotary, self.value_rotary, self.window, self.eps = float(scale), rotary, value_rotary, int(window or 0), float(eps)
        self.value_interleaved = value_pairs == "interleaved"
        if rotary is not None and rotary.dims > dim:
            raise ValueError("rotary dims exceed the head size")
        if value_rotary is not None and value_rotary.dims > vdim:
            raise ValueError("turned value columns exceed the value size")
        get = lambda n: weights.get_tensor(f"{prefix}.{n}")  # noqa: E731
        self.cq, self.ck, self.cv = self.H * self.d, self.G * self.d, self.G * self.dv
        self.channels = self.cq + self.ck + self.cv
        self.w_in = torch.cat([get(n) for n in (("q", "k", "v", "g") if head_gate else ("q", "k", "v"))], 0).contiguous()
        self.n_in = self.channels + (self.H if head_gate else 0)
        self.head_gate = bool(head_gate)
        self.conv_w = torch.cat([get(f"{n}.conv") for n in ("q", "k", "v")], 0).contiguous() if self.taps >= 1 else None
        self.q_norm, self.k_norm = get("q.norm").contiguous(), get("k.norm").contiguous()
        self.sink = get("sink").float().contiguous() if sink else None
        self.w_o = get("o").contiguous()
        self.dtype = self.w_o.dtype
        self.n_out = self.H * self.dv
        if self.w_in.shape[0] != self.n_in or (self.conv_w is not None and self.conv_w.shape != (self.channels, self.taps)) or \
                self.w_o.shape[1] != self.n_out or (self.sink is not None and self.sink.shape != (self.H,)):
            raise ValueError(f"{prefix}: tensor shapes do not match the head sizes")

    def in_rows(self) -> torch.Tensor:
        return self.w_in

    def cache_spec(self) -> LayerCacheSpec:
        state = {"conv": (max(self.taps - 1, 1), self.channels)} if self.taps >= 1 else {}   # a single tap is a weight per channel
        return LayerCacheSpec(kind="paged", row_width=self.ck + self.cv, state=state)

    def prepare_positions(self, n_pos: int, device) -> None:
        for r in (self.rotary, self.value_rotary):
            if r is not None:
                r.tables(n_pos, device)

    def from_projection(self, u: torch.Tensor, col0: int, step: ops.RaggedStep, pages: torch.Tensor, state, max_s: int, out: torch.Tensor,
                        out_scale: float = 1.0) -> None:
        """u fp32 [T, >= col0 + n_in]: this mixer's input projection from column col0 -> out [T, heads * vdim] (a column slice is fine)"""
        c, cq = u, col0
        if self.conv_w is not None:
            c, cq = ops.causal_conv(u, col0, self.channels, self.conv_w, None, state["conv"], step), 0
        cos, sin = self.rotary.tables(max_s, u.device) if self.rotary is not None else (None, None)
        vr = self.value_rotary
        vcos, vsin = vr.tables(max_s, u.device) if vr is not None else (None, None)
        q = ops.qk_rot_prepare(c, col_q=cq, col_k=cq + self.cq, col_v=cq + self.cq + self.ck, heads=self.H, kv_heads=self.G, dim=self.d,
                               vdim=self.dv, q_norm_w=self.q_norm, k_norm_w=self.k_norm, whole_norm=True, eps=self.eps, cos=cos, sin=sin,
                               rot=self.rotary.dims if self.rotary is not None else 0, step=step, cache=pages, k_off=0, v_off=self.ck,
                               v_cos=vcos, v_sin=vsin, v_rot=vr.dims if vr is not None else 0, v_interleaved=self.value_interleaved)
        a = ops.talk_attn(q, pages, step, kv_heads=self.G, vdim=self.dv, k_off=0, v_off=self.ck, scale=self.scale, window=self.window,
                          sink=self.sink)
        gate = u[:, col0 + self.channels:col0 + self.channels + self.H] if self.head_gate else None
        ops.heads_turn_gate(a, gate, vcos, vsin, vr.dims if vr is not None else 0, self.value_interleaved, step, self.dtype, out=out,
                            out_scale=out_scale)

    def forward(self, h: torch.Tensor, step: ops.RaggedStep, pages: torch.Tensor, state, max_s: int) -> torch.Tensor:
        """-> fp32 [T, width]"""
        u = ops.linear(h, self.w_in, out_dtype=torch.float32)
        o = torch.empty(step.T, self.n_out, dtype=self.dtype, device=h.device)
        self.from_projection(u, 0, step, pages, state, max_s, o)
        return ops.linear(o, self.w_o, out_dtype=torch.float32)


class MinGRUMixer(nn.Module):
    """Minimal gated recurrent unit: per channel S <- (1 - z) S + z c, the gates reading only the current token:
    z = sigmoid(W_z h + b_z), c = g(W_x h + b_x) with g(u) = u + 1/2 for u >= 0 and sigmoid(u) below; the result is
    W_o (S * SiLU(W_g h)).  State per sequence: S [width] in fp32.  Shares products with a neighbour like `SinkRotaryAttention`.
    Tensors under `prefix`: z, z.b, x, x.b, g, o."""

    def __init__(self, prefix: str, weights, *, width: int):
        super().__init__()
        _need_single_rank(weights, "MinGRUMixer")
        self.C = int(width)
        get = lambda n: weights.get_tensor(f"{prefix}.{n}")  # noqa: E731
        self.w_in = torch.cat([get("z"), get("x"), get("g")], 0).contiguous()
        self.z_b, self.x_b = get("z.b").contiguous(), get("x.b").contiguous()
        self.w_o = get("o").contiguous()
        self.dtype = self.w_o.dtype
        self.n_in, self.n_out = 3 * self.C, self.C
        if self.w_in.shape[0] != self.n_in or self.w_o.shape[1] != self.C:
            raise ValueError(f"{prefix}: projection shapes do not match the width")

    def in_rows(self) -> torch.Tensor:
        return self.w_in

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="state", state={"S": (self.C,)})

    def from_projection(self, u: torch.Tensor, col0: int, step: ops.RaggedStep, pages, state, max_s: int, out: torch.Tensor,
                        out_scale: float = 1.0) -> None:
        C = self.C
        ops.mingru_scan(u, col0, col0 + C, col0 + 2 * C, self.z_b, self.x_b, state["S"], step, C, self.dtype, out=out, out_scale=out_scale)

    def forward(self, h: torch.Tensor, step: ops.RaggedStep, pages, state, max_s: int) -> torch.Tensor:
        """-> fp32 [T, width]"""
        u = ops.linear(h, self.w_in, out_dtype=torch.float32)
        o = torch.empty(step.T, self.C, dtype=self.dtype, device=h.device)
        self.from_projection(u, 0, step, pages, state, max_s, o)
        return ops.linear(o, self.w_o, out_dtype=torch.float32)


class ParallelMixers(nn.Module):
    """Two mixers side by side that read the same input: left_scale * left(h) + right_scale * right(h).  Both must offer
    `in_rows` / `from_projection` / `w_o` / `n_in` / `n_out`: their input projections run as ONE product, each leaves what its
    output projection reads - times its scale, before the rounding to the projections' element type - in its columns of one
    buffer, and ONE product over [left | right] columns adds the two results.  At most one of them keeps paged rows; the state
    tensors of both live in the layer's slot under `left.` / `right.` names."""

    def __init__(self, left: nn.Module, right: nn.Module, left_scale: float, right_scale: float):
        super().__init__()
        self.left, self.right, self.ls, self.rs = left, right, float(left_scale), float(right_scale)
        self.w_in = torch.cat([left.in_rows(), right.in_rows()], 0).contiguous()
        self.w_o = torch.cat([left.w_o, right.w_o], 1).contiguous()
        self.dtype = self.w_o.dtype
        sl, sr = left.cache_spec(), right.cache_spec()
        if sl.kind == "paged" and sr.kind == "paged":
            raise NotImplementedError("two paged mixers in one layer")
        self._spec = LayerCacheSpec(kind="paged" if "paged" in (sl.kind, sr.kind) else "state", row_width=max(sl.row_width, sr.row_width),
                                    state={**{f"left.{k}": v for k, v in (sl.state or {}).items()},
                                           **{f"right.{k}": v for k, v in (sr.state or {}).items()}})

    def cache_spec(self) -> LayerCacheSpec:
        return self._spec

    def prepare_positions(self, n_pos: int, device) -> None:
        for m in (self.left, self.right):
            if hasattr(m, "prepare_positions"):
                m.prepare_positions(n_pos, device)

    def forward(self, h: torch.Tensor, step: ops.RaggedStep, pages, state: Dict[str, torch.Tensor], max_s: int) -> torch.Tensor:
        """-> fp32 [T, width]"""
        L, R = self.left, self.right
        u = ops.linear(h, self.w_in, out_dtype=torch.float32)
        o = torch.empty(step.T, L.n_out + R.n_out, dtype=self.dtype, device=h.device)
        side = lambda p: {k[len(p):]: v for k, v in (state or {}).items() if k.startswith(p)}  # noqa: E731
        L.from_projection(u, 0, step, pages, side("left."), max_s, o[:, :L.n_out], self.ls)
        R.from_projection(u, L.n_in, step, pages, side("right."), max_s, o[:, L.n_out:], self.rs)
        return ops.linear(o, self.w_o, out_dtype=torch.float32)


class GeneralDeltaMixer(nn.Module):
    """Generalised delta rule: per head a [dim, dim] memory S in fp32; every token, with the unit-length key u,
    S <- diag(w) S - (a * u)(u^T S) + k v^T (decay and removal both read the old memory), o = S^T r.  The decay per head and key
    channel comes from a low-rank projection, w = exp(-decay_scale * sigmoid(W_w2 tanh(W_w1 h) + w0)), the removal rate is
    a = sigmoid(W_a h + b_a).  Each head's o is divided by its RMS, times a weight per column, times sigmoid(W_g h); then the
    output projection.  State per sequence: S in fp32.
    Tensors under `prefix`: r, k, v, g, a, a.b, w1, w2, w0, norm, o."""

    def __init__(self, prefix: str, weights, *, heads: int, dim: int, eps: float, decay_scale: float = math.exp(-0.5)):
        super().__init__()
        _need_single_rank(weights, "GeneralDeltaMixer")
        self.H, self.d, self.eps, self.decay_scale = int(heads), int(dim), float(eps), float(decay_scale)
        get = lambda n: weights.get_tensor(f"{prefix}.{n}")  # noqa: E731
        self.n = self.H * self.d
        self.w_in = torch.cat([get(n) for n in ("r", "k", "v", "g", "a", "w1")], 0).contiguous()    # -> [r | k | v | gate | removal | low rank]
        self.rank = get("w1").shape[0]
        self.w2 = get("w2").contiguous()
        self.a_b, self.w0, self.norm_w = get("a.b").contiguous(), get("w0").contiguous(), get("norm").contiguous()
        self.w_o = get("o").contiguous()
        self.dtype = self.w_o.dtype
        if self.w_in.shape[0] != 5 * self.n + self.rank or self.w2.shape != (self.n, self.rank) or self.norm_w.shape != (self.n,):
            raise ValueError(f"{prefix}: projection shapes do not match the head sizes")

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="state", state={"S": (self.H, self.d, self.d)})

    def forward(self, h: torch.Tensor, step: ops.RaggedStep, pages, state: Dict[str, torch.Tensor], max_s: int) -> torch.Tensor:
        """-> fp32 [T, width]"""
        n = self.n
        u = ops.linear(h, self.w_in, out_dtype=torch.float32)
        low = ops.ff_act(u[:, 5 * n:5 * n + self.rank], ops.ACT_TANH, out_dtype=self.dtype)
        dec = ops.linear(low, self.w2, out_dtype=torch.float32)
        y = ops.gdelta_scan(u, 0, n, 2 * n, 4 * n, dec, 0, self.a_b, self.w0, self.decay_scale, state["S"], step, self.H, self.d, self.d)
        gated = ops.group_rmsnorm_gate(y, self.norm_w, self.H, self.eps, self.dtype, gate=u[:, 3 * n:4 * n], gate_kind=ops.GATE_SIGMOID_AFTER)
        return ops.linear(gated, self.w_o, out_dtype=torch.float32)


class PlainMLP(nn.Module):
    """down(act(up x)) with act SiLU or the tanh form of GELU, no gate, no biases.  The result is fp32.
    Tensors under `prefix`: up, down."""

    def __init__(self, prefix: str, weights, *, activation: str):
        super().__init__()
        _need_single_rank(weights, "PlainMLP")
        if activation not in ("silu", "gelu_tanh"):
            raise NotImplementedError(f"activation {activation!r}")
        self.act = ops.ACT_SILU if activation == "silu" else ops.ACT_GELU_TANH
        self.w_up = weights.get_tensor(f"{prefix}.up").contiguous()
        self.w_down = weights.get_tensor(f"{prefix}.down").contiguous()

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return ops.linear(ops.ff_act(ops.linear(h, self.w_up), self.act), self.w_down, out_dtype=torch.float32)
