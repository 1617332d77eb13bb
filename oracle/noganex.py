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


# ------------------------------------------------------------------------------------------------ random models
def random_config(*, width: int = 40, vocab: int = 72, order=("delta", "attention", "delta", "attention"), weights_of=(None, None, 0, None),
                  heads=(6, 4), kv_heads=(3, 2), dim=(10, 12), vdim=(14, 20), rot_dims: int = 8, base: float = 100.0, scaling="yarn",
                  chunk: int = 24, conv: int = 3, mlp=("moe", "dense", "moe", None), experts: int = 5, top: int = 2, ff: int = 24, shared_ff=16,
                  router_scale: float = 1.5, logit_scale: float = 0.5, eps: float = 1e-5) -> dict:
    """a small configuration; `heads`, `kv_heads`, `dim`, `vdim` are (attention, delta)"""
    layers = []
    for i, kind in enumerate(order):
        if kind == "attention":
            rot = {"base": base, "dims": rot_dims}
            if scaling == "yarn":
                rot["scaling"] = {"factor": 4.0, "fast": 8.0, "original": 32, "slow": 1.0}
            mixer = {"dim": dim[0], "heads": heads[0], "kv_heads": kv_heads[0], "vdim": vdim[0], "scale": dim[0] ** -0.5 * 1.6, "rot": rot}
            if chunk:
                mixer["mask"] = {"size": chunk}
        else:
            mixer = {"conv": conv, "dim": dim[1], "heads": heads[1], "kv_heads": kv_heads[1], "vdim": vdim[1]}
        f = mlp[i]
        if f == "dense":
            f = {"kind": "dense", "ff": ff + 4}
        elif f == "moe":
            f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": router_scale},
                 "shared": {"ff": shared_ff} if shared_ff else None}
        layer = {"type": kind, "mixer": mixer, "mlp": f}
        if weights_of[i] is not None:
            src = layers[int(weights_of[i])]
            layer = {"type": src["type"], "mixer": src["mixer"], "mlp": src["mlp"], "weights_of": int(weights_of[i])}
        layers.append(layer)
    return {"architecture": "Noganex", "layers": layers, "logit_scale": logit_scale, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def tensor_shapes(config: dict) -> Dict[str, tuple]:
    W, V = int(config["width"]), int(config["vocab"])
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(config["layers"]):
        if layer.get("weights_of") is not None:
            continue
        m, pre = layer["mixer"], f"l{i}"
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({f"{pre}.norm1": (W,), f"{pre}.rg1": (W, W), f"{pre}.rg1.b": (W,)})
        if layer["type"] == "attention":
            mix = {"q": (H * d, W), "k": (G * d, W), "v": (G * dv, W), "q.norm": (H * d,), "k.norm": (G * d,), "talk": (H, H), "o": (W, H * dv)}
        else:
            t = int(m["conv"])
            mix = {"q": (G * d, W), "q.conv": (G * d, t), "k": (G * d, W), "k.conv": (G * d, t), "v": (H * dv, W), "v.conv": (H * dv, t),
                   "b": (H, W), "a": (H, W), "A_log": (H,), "dt_bias": (H,), "g": (H * dv, W), "norm": (dv,), "o": (W, H * dv)}
        out.update({f"{pre}.mix.{k}": v for k, v in mix.items()})
        f = layer.get("mlp")
        if not f:
            continue
        out.update({f"{pre}.norm2": (W,), f"{pre}.rg2": (W, W), f"{pre}.rg2.b": (W,)})
        if f["kind"] == "dense":
            n = int(f["ff"])
            out.update({f"{pre}.mlp.gate": (n, W), f"{pre}.mlp.gate.b": (n,), f"{pre}.mlp.up": (n, W), f"{pre}.mlp.up.b": (n,),
                        f"{pre}.mlp.down": (W, n), f"{pre}.mlp.down.b": (W,)})
        else:
            E, n = int(f["router"]["experts"]), int(f["expert"]["ff"])
            out.update({f"{pre}.mlp.router": (E, W), f"{pre}.mlp.correction": (E,)})
            for e in range(E):
                out.update({f"{pre}.mlp.e{e}.gate": (n, W), f"{pre}.mlp.e{e}.up": (n, W), f"{pre}.mlp.e{e}.down": (W, n)})
            if f.get("shared"):
                n = int(f["shared"]["ff"])
                out.update({f"{pre}.mlp.shared.gate": (n, W), f"{pre}.mlp.shared.up": (n, W), f"{pre}.mlp.shared.down": (W, n)})
    return out


def random_state_dict(config: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """weights that are exactly representable in bfloat16, so that every element type starts from the same numbers"""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if name.endswith(".talk"):
            t = torch.eye(shape[0]) + torch.randn(shape, generator=g) * 0.35
        elif leaf == "conv":
            t = torch.randn(shape, generator=g) * 0.6
        elif leaf == "correction":
            t = torch.randn(shape, generator=g) * 0.3
        elif leaf == "A_log":
            t = torch.randn(shape, generator=g) * 0.5 - 1.0
        elif leaf == "dt_bias":
            t = torch.randn(shape, generator=g) * 0.5
        elif leaf == "b" and len(shape) == 1:
            t = torch.randn(shape, generator=g) * 0.5
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g) * ((0.7 if name == "embed" else 1.5 / math.sqrt(shape[1])))
        else:  # norm weights
            t = 1.0 + torch.randn(shape, generator=g) * 0.3
        sd[name] = t.to(torch.bfloat16).to(torch.float32)
    return sd
