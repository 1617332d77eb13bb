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


def turn_neighbours(x, positions, dims: int, base: float, sign: float = 1.0):
    """as turn_halves with columns 2i and 2i + 1 as pair i (the model does not use it; the kernels offer both layouts)"""
    i = torch.arange(dims // 2, dtype=x.dtype)
    ang = sign * positions.to(x.dtype)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2], out[..., 1:dims:2] = a * c - b * s, b * c + a * s
    return out


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
    rot = m.get("rot")
    if rot:
        q, k = turn_halves(q, pos, int(rot["dims"]), float(rot["base"])), turn_halves(k, pos, int(rot["dims"]), float(rot["base"]))
        v = turn_halves(v, pos, dv, float(rot["base"]))                # every value column turns with the value's position
    rep = H // G
    s = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(rep, dim=1)) * float(m["scale"])
    see = pos[None, :] <= pos[:, None]
    if m.get("mask"):
        see = see & (pos[:, None] - pos[None, :] < int(m["mask"]["size"]))
    s = s.masked_fill(~see, float("-inf"))
    sink = p["sink"][:, None, None].expand(H, L, 1) if "sink" in p else s.new_full((H, L, 1), float("-inf"))
    a = torch.softmax(torch.cat([s, sink], -1), -1)[..., :L]           # the sink takes weight and gives nothing
    o = torch.einsum("hij,jhv->ihv", a, v.repeat_interleave(rep, dim=1))
    if rot:
        o = turn_halves(o, pos, dv, float(rot["base"]), sign=-1.0)     # back by the query's position
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
    `margins`, when a list, receives per row the gap in router logit between the last pick and the best expert left out"""
    E, top = int(f["router"]["experts"]), int(f["router"]["top"])
    z = h @ p["router"].T
    s = torch.softmax(z, -1)
    val, idx = torch.topk(s, top, dim=-1)
    if margins is not None:
        zs = torch.topk(z, min(top + 1, E), dim=-1).values
        margins.append(zs[:, top - 1] - zs[:, top] if top < E else torch.full_like(val[:, 0], float("inf")))
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


# ------------------------------------------------------------------------------------------------ random models
def random_config(*, width: int = 40, vocab: int = 72, order=("parallel", "mlstm", "general_delta", "parallel"), loop=(1, 3, 2), streams=3,
                  residual_mult: float = 0.7, heads: int = 6, kv_heads: int = 2, dim: int = 10, vdim: int = 12, rot_dims=6, base: float = 100.0,
                  window=20, conv=3, sharp: float = 1.0, gru_width: int = 28, left_scale: float = 0.8, right_scale: float = 0.6,
                  m_heads: int = 3, m_dim: int = 6, m_vdim: int = 10, gate_cap: float = 9.0, d_heads: int = 2, d_dim: int = 12,
                  mlp=("dense", "moe", "moe", None), experts: int = 5, top: int = 2, ff: int = 24, eps: float = 1e-5) -> dict:
    """a small configuration; `loop` = (start, stop, times) or None, `streams` None for a single plain stream, `rot_dims` / `window` /
    `conv` None to leave the entry out, `sharp` multiplies the attention's score scale"""
    layers = []
    for i, kind in enumerate(order):
        if kind == "parallel":
            left = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "scale": dim ** -0.5 * sharp}
            if conv:
                left["conv"] = conv
            if rot_dims:
                left["rot"] = {"base": base, "dims": rot_dims}
            if window:
                left["mask"] = {"size": window}
            mixer = {"left": left, "left_scale": left_scale, "right": {"width": gru_width}, "right_scale": right_scale}
        elif kind == "mlstm":
            mixer = {"dim": m_dim, "gate_cap": gate_cap, "heads": m_heads, "vdim": m_vdim}
        else:
            mixer = {"dim": d_dim, "heads": d_heads}
        f = mlp[i]
        if f == "dense":
            f = {"kind": "dense", "ff": ff + 4}
        elif f == "moe":
            f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
        layers.append({"type": kind, "mixer": mixer, "mlp": f})
    out = {"architecture": "Nasozen", "layers": layers, "norm": {"eps": eps}, "residual_mult": residual_mult, "vocab": vocab, "width": width}
    if streams:
        out["streams"] = streams
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


def tensor_shapes(config: dict, decay_rank: int = 5) -> Dict[str, tuple]:
    W, V = int(config["width"]), int(config["vocab"])
    S = int(config["streams"]) if config.get("streams") else 0
    out = {"embed": (V, W), "final.norm": (W,)}
    for i, layer in enumerate(config["layers"]):
        m, pre = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "parallel":
            a, C = m["left"], m["right"]["width"]
            H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            mix = {"left.q": (H * d, W), "left.k": (G * d, W), "left.v": (G * dv, W), "left.q.norm": (H * d,), "left.k.norm": (G * d,),
                   "left.sink": (H,), "left.g": (H, W), "left.o": (W, H * dv)}
            if a.get("conv"):
                mix.update({"left.q.conv": (H * d, a["conv"]), "left.k.conv": (G * d, a["conv"]), "left.v.conv": (G * dv, a["conv"])})
            mix.update({"right.z": (C, W), "right.z.b": (C,), "right.x": (C, W), "right.x.b": (C,), "right.g": (C, W), "right.o": (W, C)})
        elif layer["type"] == "mlstm":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            mix = {"q": (H * d, W), "k": (H * d, W), "v": (H * dv, W), "g": (H * dv, W), "i": (H, W), "i.b": (H,), "f": (H, W), "f.b": (H,),
                   "norm": (H * dv,), "o": (W, H * dv)}
        else:
            n = m["heads"] * m["dim"]
            mix = {"r": (n, W), "k": (n, W), "v": (n, W), "g": (n, W), "a": (n, W), "a.b": (n,), "w1": (decay_rank, W), "w2": (n, decay_rank),
                   "w0": (n,), "norm": (n,), "o": (W, n)}
        out.update({pre + k: v for k, v in mix.items()})
        subs = [1] + ([2] if layer.get("mlp") else [])
        for q in subs:
            out[f"l{i}.norm{q}"] = (W,)
            if S:
                out.update({f"l{i}.hc{q}.in": (S,), f"l{i}.hc{q}.out": (S,), f"l{i}.hc{q}.mix": (S, S)})
        f = layer.get("mlp")
        if f and f["kind"] == "dense":
            out.update({f"l{i}.mlp.up": (int(f["ff"]), W), f"l{i}.mlp.down": (W, int(f["ff"]))})
        elif f:
            E, n = int(f["router"]["experts"]), int(f["expert"]["ff"])
            out[f"l{i}.mlp.router"] = (E, W)
            for e in range(E):
                out.update({f"l{i}.mlp.e{e}.gate": (n, W), f"l{i}.mlp.e{e}.up": (n, W), f"l{i}.mlp.e{e}.down": (W, n)})
    return out


def random_state_dict(config: dict, seed: int = 0, decay_rank: int = 5) -> Dict[str, torch.Tensor]:
    """weights that are exactly representable in bfloat16, so that every element type starts from the same numbers"""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in tensor_shapes(config, decay_rank).items():
        parts = name.split(".")
        leaf = parts[-1]
        if ".hc" in name:
            S = shape[0]
            t = {"in": torch.full(shape, 1.0 / S), "out": torch.ones(shape), "mix": torch.eye(S)}[leaf] + torch.randn(shape, generator=g) * 0.25
        elif leaf == "conv":
            t = torch.randn(shape, generator=g) * 0.6
        elif leaf == "sink":
            t = torch.randn(shape, generator=g) * 1.5
        elif leaf == "w0":
            t = torch.randn(shape, generator=g) * 1.5
        elif leaf == "b":
            t = torch.randn(shape, generator=g) * (2.0 if parts[-2] in ("i", "f") else 0.7)
        elif leaf == "w2":
            t = torch.randn(shape, generator=g) * 1.2
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g) * ((0.7 if name == "embed" else 1.5 / math.sqrt(shape[1])))
        else:  # norm weights
            t = 1.0 + torch.randn(shape, generator=g) * 0.3
        sd[name] = t.to(torch.bfloat16).to(torch.float32)
    return sd
