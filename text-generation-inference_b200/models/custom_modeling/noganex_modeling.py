"""Noganex: a decoder whose sublayers read the fp32 residual stream itself and are normalised on the way back,
x += N1(s1 . mixer(x)) then x += N2(s2 . ff(x)), with N = x / sqrt(mean x^2 + eps) * w and a gate per channel
s = sigmoid(R x + r) computed from the sublayer's input.  The mixer of a layer is the gated delta rule (recurrent, fp32 state) or
grouped-query attention with head-mixed scores, a whole-projection q / k norm, partial rotate-half rotation (optionally YaRN
scaled) and a chunked causal mask; the feed-forward is a gated MLP with biases (tanh-GELU) or sigmoid-routed SiLU experts plus a
shared expert.  A layer may use another layer's tensors (`weights_of`) with a cache or state of its own.
logits = head (N_final x) * logit_scale.

config.json: {"architecture": "Noganex", "vocab", "width", "norm": {"eps"}, "logit_scale", "layers": [{"type": "attention" |
"delta", "mixer": {...}, "mlp": null | {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top",
"scale"}, "shared": null | {"ff"}} [, "weights_of": j]}, ...]}.
  attention: heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling: null | {factor, original, fast, slow}}, mask {size}
  delta:     heads, kv_heads, dim, vdim, conv (taps)
Checkpoint tensors: `embed`, `l<i>.norm1|norm2`, `l<i>.rg1|rg2` (+ `.b`), `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.

The mixers and feed-forwards (utils/mixers.py) and their kernels know nothing of this family; this file reads the configuration,
loads the tensors under the family's names and composes the layers.  Steps are ragged (ragged_decoder.py).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional

import torch
from torch import nn

from ... import ops_seq as ops
from ...utils.mixers import GatedDeltaMixer, GatedMLP, RoutedExperts, ScaledRotaryTables, TalkingHeadsAttention
from ...utils.paged import HybridCacheManager
from .ragged_decoder import RaggedDecoderForCausalLM

ARCHITECTURE = "Noganex"
MIXER_TYPES = ("attention", "delta")


class NoganexConfig:
    """config.json of the family, with the attribute names the runtime reads on any model config."""
    model_type = "noganex"

    def __init__(self, raw: Dict[str, Any]):
        if raw.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} configuration")
        self.raw = raw
        self.architecture = ARCHITECTURE
        self.vocab_size = int(raw["vocab"])
        self.hidden_size = int(raw["width"])
        self.layers: List[Dict[str, Any]] = list(raw["layers"])
        self.num_hidden_layers = len(self.layers)
        self.norm_eps = float(raw["norm"]["eps"])
        self.logit_scale = float(raw.get("logit_scale", 1.0))
        self.eos_token_id = raw.get("eos_token_id")
        self.pad_token_id = raw.get("pad_token_id")
        self.quantize = None
        for i, layer in enumerate(self.layers):
            if layer["type"] not in MIXER_TYPES:
                raise NotImplementedError(f"mixer type {layer['type']!r}")
            f = layer.get("mlp")
            if f and f.get("kind") not in ("dense", "moe"):
                raise NotImplementedError(f"mlp kind {f.get('kind')!r}")
            j = self.weight_layer(i)
            if j != i:
                own = self.layers[j]
                if own["type"] != layer["type"] or own["mixer"] != layer["mixer"] or own.get("mlp") != layer.get("mlp"):
                    raise ValueError(f"layer {i}: weights_of {j} names a layer of another shape")

    def weight_layer(self, i: int) -> int:
        """the layer whose tensors layer i uses (itself unless `weights_of` says otherwise)"""
        seen = set()
        while self.layers[i].get("weights_of") is not None:
            if i in seen or not 0 <= int(self.layers[i]["weights_of"]) < len(self.layers):
                raise ValueError(f"layer {i}: weights_of does not lead to a layer with tensors")
            seen.add(i)
            i = int(self.layers[i]["weights_of"])
        return i

    @classmethod
    def from_pretrained(cls, model_path: str) -> "NoganexConfig":
        with open(os.path.join(model_path, "config.json")) as f:
            return cls(json.load(f))


def tensor_shapes(raw: Dict[str, Any]) -> Dict[str, tuple]:
    """name -> shape of every checkpoint tensor of a configuration (synthetic checkpoints, load-time validation)"""
    W, V = int(raw["width"]), int(raw["vocab"])
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(raw["layers"]):
        if layer.get("weights_of") is not None:
            continue
        m, pre = layer["mixer"], f"l{i}"
        H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        if layer["type"] == "attention":
            mix = {"q": (H * d, W), "k": (G * d, W), "v": (G * dv, W), "q.norm": (H * d,), "k.norm": (G * d,), "talk": (H, H), "o": (W, H * dv)}
        else:
            taps = int(m["conv"])
            mix = {"q": (G * d, W), "q.conv": (G * d, taps), "k": (G * d, W), "k.conv": (G * d, taps), "v": (H * dv, W), "v.conv": (H * dv, taps),
                   "b": (H, W), "A_log": (H,), "norm": (dv,), "a": (H, W), "dt_bias": (H,), "g": (H * dv, W), "o": (W, H * dv)}
        out.update({f"{pre}.norm1": (W,), f"{pre}.rg1": (W, W), f"{pre}.rg1.b": (W,)})
        out.update({f"{pre}.mix.{k}": v for k, v in mix.items()})
        f = layer.get("mlp")
        if not f:
            continue
        out.update({f"{pre}.norm2": (W,), f"{pre}.rg2": (W, W), f"{pre}.rg2.b": (W,)})
        if f["kind"] == "dense":
            ff = int(f["ff"])
            out.update({f"{pre}.mlp.gate": (ff, W), f"{pre}.mlp.gate.b": (ff,), f"{pre}.mlp.up": (ff, W), f"{pre}.mlp.up.b": (ff,),
                        f"{pre}.mlp.down": (W, ff), f"{pre}.mlp.down.b": (W,)})
        else:
            E, ff = int(f["router"]["experts"]), int(f["expert"]["ff"])
            out.update({f"{pre}.mlp.router": (E, W), f"{pre}.mlp.correction": (E,)})
            for e in range(E):
                out.update({f"{pre}.mlp.e{e}.gate": (ff, W), f"{pre}.mlp.e{e}.up": (ff, W), f"{pre}.mlp.e{e}.down": (W, ff)})
            if f.get("shared"):
                sf = int(f["shared"]["ff"])
                out.update({f"{pre}.mlp.shared.gate": (sf, W), f"{pre}.mlp.shared.up": (sf, W), f"{pre}.mlp.shared.down": (W, sf)})
    return out


def build_mixer(kind: str, prefix: str, m: Dict[str, Any], weights, eps: float) -> nn.Module:
    common = dict(heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), eps=eps)
    if kind == "attention":
        rot, mask = m.get("rot"), m.get("mask")
        rotary = ScaledRotaryTables(int(rot["dims"]), float(rot["base"]), rot.get("scaling")) if rot and int(rot.get("dims", 0)) > 0 else None
        return TalkingHeadsAttention(prefix, weights, scale=float(m["scale"]), rotary=rotary, chunk=int(mask["size"]) if mask else None, **common)
    if kind == "delta":
        return GatedDeltaMixer(prefix, weights, conv=int(m["conv"]), **common)
    raise NotImplementedError(f"mixer type {kind!r}")


class RoutedWithShared(nn.Module):
    """sigmoid-routed SiLU experts plus an expert that every token uses -> fp32 [T, width]"""

    def __init__(self, prefix: str, f: Dict[str, Any], weights):
        super().__init__()
        r = f["router"]
        self.routed = RoutedExperts(prefix, weights, experts=int(r["experts"]), top=int(r["top"]), limit=None, sigmoid_scores=True,
                                    correction=True, weight_scale=float(r.get("scale", 1.0)))
        self.shared = GatedMLP(f"{prefix}.shared", weights, activation="silu", bias=False) if f.get("shared") else None

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        y, routing = self.routed(h)
        out = self.shared(h) if self.shared is not None else torch.zeros(h.shape[0], y.shape[1], dtype=torch.float32, device=h.device)
        ops.moe_combine_add(out, None, y, routing)
        return out


class _GatedSublayer(nn.Module):
    """what surrounds a sublayer: the channel gate from the sublayer's input and the norm on its result"""

    def __init__(self, pre: str, n: int, weights, eps: float):
        super().__init__()
        self.w_gate = weights.get_tensor(f"{pre}.rg{n}").contiguous()
        self.b_gate = weights.get_tensor(f"{pre}.rg{n}.b").contiguous()
        self.norm_w = weights.get_tensor(f"{pre}.norm{n}").contiguous()
        self.eps = eps

    def add(self, x: torch.Tensor, xt: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        """x (fp32 stream, in place) += N(sigmoid(R xt + r) . y) -> the updated stream in the projections' element type"""
        gate = ops.linear(xt, self.w_gate, self.b_gate, out_dtype=torch.float32)
        return ops.gated_rms_add(x, y, gate, self.norm_w, self.eps, typed_copy=True)


class NoganexLayer(nn.Module):
    def __init__(self, index: int, config: NoganexConfig, weights, share: Optional["NoganexLayer"] = None):
        super().__init__()
        self.index = index
        if share is not None:  # another layer's modules; the cache or state is this layer's own (looked up by index)
            self.mixer, self.mlp, self.around1, self.around2 = share.mixer, share.mlp, share.around1, share.around2
            return
        spec, pre, eps = config.layers[index], f"l{index}", config.norm_eps
        self.mixer = build_mixer(spec["type"], f"{pre}.mix", spec["mixer"], weights, eps)
        self.around1 = _GatedSublayer(pre, 1, weights, eps)
        f = spec.get("mlp")
        self.mlp, self.around2 = None, None
        if f:
            self.mlp = (GatedMLP(f"{pre}.mlp", weights, activation="gelu_tanh", bias=True) if f["kind"] == "dense"
                        else RoutedWithShared(f"{pre}.mlp", f, weights))
            self.around2 = _GatedSublayer(pre, 2, weights, eps)

    def forward(self, x: torch.Tensor, xt: torch.Tensor, step: ops.RaggedStep, manager: HybridCacheManager, max_s: int) -> torch.Tensor:
        """advances the fp32 stream x in place; xt is x in the projections' element type, the new one is returned"""
        y = self.mixer(xt, step, manager.layer_pages(self.index), manager.layer_state(self.index), max_s)
        xt = self.around1.add(x, xt, y)
        if self.mlp is not None:
            xt = self.around2.add(x, xt, self.mlp(xt))
        return xt


class _PlainNorm(nn.Module):
    def __init__(self, name: str, weights, eps: float):
        super().__init__()
        self.w, self.eps = weights.get_tensor(name).contiguous(), eps

    def forward(self, x):
        return ops.rmsnorm_rows(x, self.w, self.eps)


class NoganexModel(nn.Module):
    def __init__(self, config: NoganexConfig, weights):
        super().__init__()
        self.config = config
        self.embed = weights.get_tensor("embed").contiguous()
        self.dtype = self.embed.dtype
        layers: List[Optional[NoganexLayer]] = [None] * config.num_hidden_layers
        for i in range(config.num_hidden_layers):      # layers with tensors first: a sharing layer may come before its source
            if config.weight_layer(i) == i:
                layers[i] = NoganexLayer(i, config, weights)
        for i in range(config.num_hidden_layers):
            if layers[i] is None:
                layers[i] = NoganexLayer(i, config, weights, share=layers[config.weight_layer(i)])
        self.layers = nn.ModuleList(layers)
        self.final_norm = _PlainNorm("final.norm", weights, config.norm_eps)
        self.kv_cache_manager: Optional[HybridCacheManager] = None
        self.residual_probe: Optional[list] = None  # when a list: receives a copy of the stream after every layer (tests)

    def forward(self, input_ids, step: ops.RaggedStep, max_s: int) -> torch.Tensor:
        x = ops.embed_scale(self.embed, input_ids, 1.0)
        xt = ops.cast_rows(x, self.dtype)
        for layer in self.layers:
            xt = layer(x, xt, step, self.kv_cache_manager, max_s)
            if self.residual_probe is not None:
                self.residual_probe.append(x.clone())
        return x


class NoganexForCausalLM(RaggedDecoderForCausalLM):
    def __init__(self, config: NoganexConfig, weights):
        super().__init__(config, weights, NoganexModel(config, weights))
        self.logit_scale = config.logit_scale
