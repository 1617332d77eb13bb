"""Slow reference of the Nasozen decoder: plain PyTorch on the CPU, one function per mechanism, whole sequences at once.

Test infrastructure only.  It shares no code with the product path (no paged cache, no state slots, no kernels): every mixer
recomputes a sequence from its first token (dense score matrices, token-by-token recurrences), so a test can compare any cut
of a prompt, any batch and any reuse of pages and slots in the product against it.  `dtype` is torch.float64 by default.

The model.  x = embed[token] is copied into `streams` residual streams X_1 .. X_n (hyper-connections).  A sublayer q of a layer
(1: the mixer, 2: the feed-forward) reads u = sum_s in_q[s] X_s, computes y = sublayer(unit_rms(u) * norm_q) and rewrites all
streams at once, X_t <- sum_s mix_q[s, t] X_s + residual_mult * out_q[t] * y.  A configuration without `streams` keeps one
stream with plain sums, x <- x + residual_mult * y.  Layers `loop.start .. loop.stop - 1` run `loop.times` times in a row with
the same tensors (every pass has a memory of its own).  At the end x = sum_s X_s, logits = embed (unit_rms(x) * final.norm).

Mixers:
  parallel       left_scale * attention(h) + right_scale * minGRU(h), both reading the same h.  The attention: grouped
                 queries, a short causal convolution after each of the q / k / v projections, an RMS norm over the whole q and
                 the whole k projection, rotation of the first rot.dims columns of every q / k head (column i with column
                 i + dims / 2), values rotated over all their columns by their own position and the head's result rotated back
                 by the query's position, a sliding window, a learned sink logit per head in the soft-max denominator, a
                 sigmoid gate per head.  The minGRU: z = sigmoid(W_z h + b), candidate c = g(W_x h + b) with g(u) = u + 1/2
                 for u >= 0 and sigmoid(u) below, S <- (1 - z) S + z c, out = W_o (S * silu(W_g h)).
  mlstm          matrix memory with capped log gates and a running maximum that starts at 0.
  general_delta  S <- diag(w) S - (a * u)(u^T S) + k v^T with u the unit-length key, a decay w per key channel from a low-rank
                 projection and a removal rate a per key channel; o = S^T r.
Feed-forward: down(gelu_tanh(up h)), or `top` of `experts` SiLU-gated experts weighted by their soft-max scores over the
picked scores' sum.

Checkpoint naming: `embed`, `l<i>.norm1|norm2`, `l<i>.hc1|hc2.in|out|mix`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------ small pieces
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def logsigmoid(z):
    return -torch.nn.functional.softplus(-z)


def short_conv(u, w):
    """u [L, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the first row."""
    L, taps = u.shape[0], w.shape[1]
    pad = torch.cat([u.new_zeros(taps - 1, u.shape[1]), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + w[:, j] * pad[j:j + L]
    return y


def sub(sd: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}


# ------------------------------------------------------------------------------------------------ rotation
def turn_halves(x, positions, dims: int, base: float, sign: float = 1.0):
    """x [L, heads, n]: the first `dims` columns of every head, column i paired with column i + dims / 2, pair i turned by
    sign * position * base^(-2i / dims); the other columns pass"""
    i = torch.arange(dims // 2, dtype=x.dtype)
    ang = sign * positions.to(x.dtype)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], -1)


# ------------------------------------------------------------------------------------------------ mixers
def sink_window_attention(h, p, m: dict, eps: float):
    """h [L, W] -> [L, W]: the attention half of the parallel mixer"""
    L, H, G, d, dv = h.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    pos = torch.arange(L)
    q, k, v = h @ p["q"].T, h @ p["k"].T, h @ p["v"].T
    if m.get("conv"):
        q, k, v = short_conv(q, p["q.conv"]), short_conv(k, p["k.conv"]), short_conv(v, p["v.conv"])
    q = (unit_rms(q, eps) * p["q.norm"]).view(L, H, d)
    k = (unit_rms(k, eps) * p["k.norm"]).view(L, G, d)
    v = v.view(L, G, dv)
    base = 10000.0
    if m.get("rot"):
        base = float(m["rot"]["base"])
        q, k = turn_halves(q, pos, int(m["rot"]["dims"]), base), turn_halves(k, pos, int(m["rot"]["dims"]), base)
    v = turn_halves(v, pos, dv, base)                                  # every value column turns with the value's position
    rep = H // G
    s = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(rep, dim=1)) * float(m["scale"])
    see = pos[None, :] <= pos[:, None]
    if m.get("mask"):
        see = see & (pos[:, None] - pos[None, :] < int(m["mask"]["size"]))
    s = s.masked_fill(~see, float("-inf"))
    sink = p["sink"][:, None, None].expand(H, L, 1) if "sink" in p else s.new_full((H, L, 1), float("-inf"))
    a = torch.softmax(torch.cat([s, sink], -1), -1)[..., :L]           # the sink takes weight and gives nothing
    o = torch.einsum("hij,jhv->ihv", a, v.repeat_interleave(rep, dim=1))
    o = turn_halves(o, pos, dv, base, sign=-1.0)                       # back by the query's position
    o = o * torch.sigmoid(h @ p["g"].T)[:, :, None]
    return o.reshape(L, H * dv) @ p["o"].T


def min_gru(h, p):
    """h [L, W] -> [L, W]: S <- (1 - z) S + z c per channel, gates from the current token only"""
    z = torch.sigmoid(h @ p["z"].T + p["z.b"])
    u = h @ p["x"].T + p["x.b"]
    c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = torch.zeros(z.shape[1], dtype=h.dtype)
    out = torch.zeros_like(z)
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        out[t] = S
    return (out * silu(h @ p["g"].T)) @ p["o"].T


def parallel_mixer(h, p, m: dict, eps: float):
    return float(m["left_scale"]) * sink_window_attention(h, sub(p, "left."), m["left"], eps) + float(m["right_scale"]) * min_gru(h, sub(p, "right."))


def mlstm(h, p, m: dict, eps: float):
    """h [L, W] -> [L, W]: per head S [dim, vdim], normaliser n [dim], running maximum (from 0) of the log gates"""
    L, H, d, dv, cap = h.shape[0], int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = (h @ p["q"].T).view(L, H, d) * d ** -0.5
    k = (h @ p["k"].T).view(L, H, d)
    v = (h @ p["v"].T).view(L, H, dv)
    ig = cap * torch.tanh((h @ p["i"].T + p["i.b"]) / cap)
    fg = logsigmoid(cap * torch.tanh((h @ p["f"].T + p["f.b"]) / cap))
    o = torch.zeros(L, H, dv, dtype=h.dtype)
    for hd in range(H):
        S, n, mx = torch.zeros(d, dv, dtype=h.dtype), torch.zeros(d, dtype=h.dtype), torch.zeros((), dtype=h.dtype)
        for t in range(L):
            m_new = torch.maximum(fg[t, hd] + mx, ig[t, hd])
            keep, write = torch.exp(fg[t, hd] + mx - m_new), torch.exp(ig[t, hd] - m_new)
            S = keep * S + write * torch.outer(k[t, hd], v[t, hd])
            n = keep * n + write * k[t, hd]
            mx = m_new
            o[t, hd] = (S.T @ q[t, hd]) / (torch.maximum(torch.abs(n @ q[t, hd]), torch.exp(-mx)) + 1e-6)
    o = (unit_rms(o, eps).reshape(L, H * dv) * p["norm"]) * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T


def general_delta(h, p, m: dict, eps: float):
    """h [L, W] -> [L, W]: per head S [dim, dim]; every token decays the key rows, removes along the unit key, then writes"""
    L, H, d = h.shape[0], int(m["heads"]), int(m["dim"])
    r, k, v = (h @ p["r"].T).view(L, H, d), (h @ p["k"].T).view(L, H, d), (h @ p["v"].T).view(L, H, d)
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ p["w1"].T) @ p["w2"].T + p["w0"])).view(L, H, d)
    a = torch.sigmoid(h @ p["a"].T + p["a.b"]).view(L, H, d)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    o = torch.zeros(L, H, d, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(d, d, dtype=h.dtype)
        for t in range(L):
            ut = u[t, hd]
            S = w[t, hd][:, None] * S - torch.outer(a[t, hd] * ut, ut @ S) + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ r[t, hd]
    o = (unit_rms(o, eps).reshape(L, H * d) * p["norm"]) * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T


MIXERS = {"parallel": parallel_mixer, "mlstm": mlstm, "general_delta": general_delta}


# ------------------------------------------------------------------------------------------------ feed-forward
def dense_mlp(h, p):
    return gelu_tanh(h @ p["up"].T) @ p["down"].T


def silu_expert(h, p, prefix: str):
    return (silu(h @ p[prefix + "gate"].T) * (h @ p[prefix + "up"].T)) @ p[prefix + "down"].T


def routed_experts(h, p, f: dict, margins: Optional[list] = None):
    """soft-max scores over all experts; the `top` largest are picked and weighted by score / (sum of the picked scores + 1e-20).
    `margins`, when a list, receives per row the gap in score between the last pick and the best expert left out"""
    E, top = int(f["router"]["experts"]), int(f["router"]["top"])
    s = torch.softmax(h @ p["router"].T, -1)
    val, idx = torch.topk(s, top, dim=-1)
    if margins is not None:
        margins.append(val[:, -1] - torch.topk(s, top + 1, dim=-1).values[:, -1] if top < E else torch.full_like(val[:, 0], float("inf")))
    wgt = val / (val.sum(-1, keepdim=True) + 1e-20)
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for e in range(E):
        out = out + silu_expert(h, p, f"e{e}.") * (wgt * (idx == e)).sum(-1, keepdim=True)
    return out


# ------------------------------------------------------------------------------------------------ the model
def layer_runs(config: dict) -> List[int]:
    """the layer index of every layer run, in order (looped layers appear `times` times)"""
    n, loop = len(config["layers"]), config.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(config: dict, sd: Dict[str, torch.Tensor], tokens: List[int], dtype=F64, residuals: Optional[list] = None,
            margins: Optional[list] = None):
    """logits [L, vocab] of one sequence; `residuals`, when a list, receives the sum of the streams after every layer run,
    `margins` the routing margin of every position in every routed layer run"""
    sd = {k: v.to(dtype) for k, v in sd.items() if v.is_floating_point()}
    eps, mult = float(config["norm"]["eps"]), float(config.get("residual_mult", 1.0))
    n_streams = int(config["streams"]) if config.get("streams") else 0
    x = sd["embed"][torch.tensor(tokens, dtype=torch.int64)]
    X = x[None].repeat(max(n_streams, 1), 1, 1)                         # [streams, L, W]

    def sublayer(X, pre, q, fn):
        if not n_streams:
            return X + mult * fn(unit_rms(X[0], eps) * sd[f"{pre}.norm{q}"])[None]
        y = fn(unit_rms(torch.einsum("s,slw->lw", sd[f"{pre}.hc{q}.in"], X), eps) * sd[f"{pre}.norm{q}"])
        return torch.einsum("st,slw->tlw", sd[f"{pre}.hc{q}.mix"], X) + mult * sd[f"{pre}.hc{q}.out"][:, None, None] * y[None]

    for i in layer_runs(config):
        layer, pre = config["layers"][i], f"l{i}"
        p = sub(sd, pre + ".mix.")
        X = sublayer(X, pre, 1, lambda h: MIXERS[layer["type"]](h, p, layer["mixer"], eps))
        f = layer.get("mlp")
        if f:
            pf = sub(sd, pre + ".mlp.")
            X = sublayer(X, pre, 2, (lambda h: dense_mlp(h, pf)) if f["kind"] == "dense" else (lambda h: routed_experts(h, pf, f, margins)))
        if residuals is not None:
            residuals.append(X.sum(0))
    return (unit_rms(X.sum(0), eps) * sd["final.norm"]) @ sd["embed"].T
