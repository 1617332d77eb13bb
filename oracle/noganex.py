"""Slow reference of the Noganex decoder: plain PyTorch on the CPU, one function per mechanism, whole sequences at once.

Test infrastructure only.  It shares no code with the product path (no paged cache, no state slots, no kernels): every mixer
recomputes a sequence from its first token (dense score matrices, a token-by-token recurrence), so a test can compare any cut
of a prompt, any batch and any reuse of pages and slots in the product against it.  `dtype` is torch.float64 by default.

The model: x = embed[token]; every layer is x += N1(s1 * mixer(x)) then x += N2(s2 * ff(x)) with N = unit-RMS times a weight
and s = sigmoid(R x + r) (a gate per channel, computed from the sublayer's input); both sublayers read the stream itself, the
norm sits on their result.  The mixer is the gated delta rule (short convolutions + SiLU on q / k / v, unit-length q and k, a
write strength and a decay per head) or grouped-query attention with an RMS norm over the whole q and k projections, a partly
rotated head (rotate-half pairs, optional YaRN scaling), scores mixed across heads before the soft-max, and a chunked causal
mask.  The feed-forward is a gated MLP (tanh-GELU, biases) or sigmoid-routed experts (SiLU) with a shared expert.  A layer may
use another layer's tensors with a state of its own.  logits = head (N_final x) * logit_scale.

Checkpoint naming: `embed`, `l<i>.norm1|norm2`, `l<i>.rg1|rg2` (+ `.b`), `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------ small pieces
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def unit_length(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


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
def rotary_frequencies(rot: dict, dtype=F64):
    """frequency of every rotated pair and the amplitude of cos / sin"""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def pair_of(turns):
        return dims * math.log(float(sc["original"]) / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / float(sc["factor"]) * ramp + f * (1.0 - ramp), 0.1 * math.log(float(sc["factor"])) + 1.0


def rotate_half(x, rot: dict):
    """x [L, heads, dim]: the first rot.dims columns of every head, column i paired with column i + dims / 2"""
    dims = int(rot["dims"])
    f, amp = rotary_frequencies(rot, x.dtype)
    ang = torch.arange(x.shape[0], dtype=x.dtype)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * amp)[:, None, :], (torch.sin(ang) * amp)[:, None, :]
    a, b = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], -1)


# ------------------------------------------------------------------------------------------------ mixers
def talking_attention(h, p, m: dict, eps: float):
    """h [L, W] -> [L, W]: grouped-query attention, whole-projection q / k norm, partial rotation, scores mixed over the heads,
    chunked causal mask"""
    L, H, G, d, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms(h @ p["q"].T, eps) * p["q.norm"]
    k = unit_rms(h @ p["k"].T, eps) * p["k.norm"]
    v = (h @ p["v"].T).view(L, G, dv)
    q, k = q.view(L, H, d), k.view(L, G, d)
    if m.get("rot"):
        q, k = rotate_half(q, m["rot"]), rotate_half(k, m["rot"])
    rep = H // G
    s = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(rep, dim=1)) * float(m["scale"])
    if "talk" in p:
        s = torch.einsum("hg,gij->hij", p["talk"], s)
    pos = torch.arange(L)
    see = pos[None, :] <= pos[:, None]
    if m.get("mask"):
        size = int(m["mask"]["size"])
        see = see & ((pos[None, :] // size) == (pos[:, None] // size))
    a = torch.softmax(s.masked_fill(~see, float("-inf")), -1)
    o = torch.einsum("hij,jhv->ihv", a, v.repeat_interleave(rep, dim=1)).reshape(L, H * dv)
    return o @ p["o"].T


def gated_delta(h, p, m: dict, eps: float):
    """h [L, W] -> [L, W]: per head a [dim, vdim] memory S; every token S <- g S, then writes beta (v - S^T k) at k and reads at q"""
    L, H, G, d, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ p["q"].T, p["q.conv"])).view(L, G, d)
    k = silu(short_conv(h @ p["k"].T, p["k.conv"])).view(L, G, d)
    v = silu(short_conv(h @ p["v"].T, p["v.conv"])).view(L, H, dv)
    q, k = unit_length(q) * d ** -0.5, unit_length(k)
    beta = torch.sigmoid(h @ p["b"].T)                                                  # [L, H]
    g = torch.exp(-torch.exp(p["A_log"]) * softplus(h @ p["a"].T + p["dt_bias"]))      # [L, H]
    rep = H // G
    o = torch.zeros(L, H, dv, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(L):
            kt, qt = k[t, hd // rep], q[t, hd // rep]
            S = g[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ kt)
            S = S + torch.outer(kt, u)
            o[t, hd] = S.T @ qt
    o = unit_rms(o, eps) * p["norm"] * silu(h @ p["g"].T).view(L, H, dv)
    return o.reshape(L, H * dv) @ p["o"].T


# ------------------------------------------------------------------------------------------------ feed-forward
def dense_mlp(h, p):
    return (gelu_tanh(h @ p["gate"].T + p["gate.b"]) * (h @ p["up"].T + p["up.b"])) @ p["down"].T + p["down.b"]


def silu_expert(h, p, prefix: str):
    return (silu(h @ p[prefix + "gate"].T) * (h @ p[prefix + "up"].T)) @ p[prefix + "down"].T


def routed_experts(h, p, f: dict, margins: Optional[list] = None):
    """sigmoid scores; the picks are the `top` largest of score + correction, their weights the plain scores over their sum, times
    router.scale; a shared expert is added for every token.  `margins`, when a list, receives per row the gap in choice score
    between the last pick and the best expert left out"""
    E, top, scale = int(f["router"]["experts"]), int(f["router"]["top"]), float(f["router"].get("scale", 1.0))
    s = torch.sigmoid(h @ p["router"].T)
    choice = s + p["correction"] if "correction" in p else s
    val, idx = torch.topk(choice, top, dim=-1)
    if margins is not None:
        margins.append(val[:, -1] - torch.topk(choice, top + 1, dim=-1).values[:, -1] if top < E else torch.full_like(val[:, 0], float("inf")))
    picked = torch.gather(s, 1, idx)
    wgt = picked / (picked.sum(-1, keepdim=True) + 1e-20) * scale
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for e in range(E):
        out = out + silu_expert(h, p, f"e{e}.") * (wgt * (idx == e)).sum(-1, keepdim=True)
    if f.get("shared"):
        out = out + silu_expert(h, p, "shared.")
    return out


# ------------------------------------------------------------------------------------------------ the model
def weight_layer(config: dict, i: int) -> int:
    """the layer whose tensors layer i uses"""
    seen = set()
    while config["layers"][i].get("weights_of") is not None and i not in seen:
        seen.add(i)
        i = int(config["layers"][i]["weights_of"])
    return i


def forward(config: dict, sd: Dict[str, torch.Tensor], tokens: List[int], dtype=F64, residuals: Optional[list] = None,
            margins: Optional[list] = None):
    """logits [L, vocab] of one sequence; `residuals`, when a list, receives the stream after every layer, `margins` the routing
    margin of every position in every routed layer (a reduced-precision run may pick other experts where it is small)"""
    sd = {k: v.to(dtype) for k, v in sd.items() if v.is_floating_point()}
    eps = float(config["norm"]["eps"])
    x = sd["embed"][torch.tensor(tokens, dtype=torch.int64)]
    for i, layer in enumerate(config["layers"]):
        pre = f"l{weight_layer(config, i)}"
        m, p = layer["mixer"], sub(sd, pre + ".mix.")
        y = talking_attention(x, p, m, eps) if layer["type"] == "attention" else gated_delta(x, p, m, eps)
        y = y * torch.sigmoid(x @ sd[pre + ".rg1"].T + sd[pre + ".rg1.b"])
        x = x + unit_rms(y, eps) * sd[pre + ".norm1"]
        f = layer.get("mlp")
        if f:
            pf = sub(sd, pre + ".mlp.")
            y = dense_mlp(x, pf) if f["kind"] == "dense" else routed_experts(x, pf, f, margins)
            y = y * torch.sigmoid(x @ sd[pre + ".rg2"].T + sd[pre + ".rg2.b"])
            x = x + unit_rms(y, eps) * sd[pre + ".norm2"]
        if residuals is not None:
            residuals.append(x.clone())
    return (unit_rms(x, eps) * sd["final.norm"]) @ sd["head"].T * float(config.get("logit_scale", 1.0))
