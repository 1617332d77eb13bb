"""Nasozen: a pre-norm decoder on several fp32 residual streams ("hyper-connections") whose layers pick one of three mixers, with
a run of layers that repeats with the same tensors.

x = embed[token] starts `streams` copies X_1 .. X_n.  Sublayer q of a layer (1: mixer, 2: feed-forward) reads
u = sum_s in_q[s] X_s, computes y = sublayer(N_q(u)) with N = u / sqrt(mean u^2 + eps) * w, and rewrites all streams at once,
X_t <- sum_s mix_q[s, t] X_s + residual_mult * out_q[t] * y.  Without `streams` in the configuration there is one stream and
x <- x + residual_mult * y.  Layers loop.start .. loop.stop - 1 run loop.times times in a row with the same tensors; every pass
is a layer run with a cache and state of its own.  After the last run x = sum_s X_s and logits = embed (N_final x): the
embedding table is the vocabulary head.

Mixers: "parallel" = left_scale * (windowed grouped-query attention with short convolutions, a whole-projection q / k norm,
partly rotated heads, position-carrying values, a sink logit and a gate per head) + right_scale * (a minimal gated recurrent
unit), both reading the same input; "mlstm" = the matrix memory with capped log gates; "general_delta" = the generalised
delta rule with a decay and a removal rate per key channel.  Feed-forward: up / tanh-GELU / down, or soft-max routed SiLU
experts weighted by their scores over the picked scores' sum.

config.json: {"architecture": "Nasozen", "vocab", "width", "norm": {"eps"}, "residual_mult", ["streams",] ["loop": {"start",
"stop", "times"},] "layers": [{"type": "parallel" | "mlstm" | "general_delta", "mixer": {...}, "mlp": null | {"kind": "dense",
"ff"} | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}}}, ...]}.
  parallel:      left {heads, kv_heads, dim, vdim, scale, [conv,] [rot {base, dims},] [mask {size}]}, left_scale, right {width}, right_scale
  mlstm:         heads, dim, vdim, gate_cap
  general_delta: heads, dim
Checkpoint tensors: `embed`, `l<i>.norm1|norm2`, `l<i>.hc1|hc2.in|out|mix`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`.

The mixers and feed-forwards (utils/mixers.py) and their kernels know nothing of this family; this file reads the configuration,
loads the tensors under the family's names and composes the layer runs.  Steps are ragged (ragged_decoder.py).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional

import torch
from torch import nn

from ... import ops_seq as ops
from ...utils.mixers import (GeneralDeltaMixer, MinGRUMixer, MLSTMMixer, ParallelMixers, PlainMLP, RoutedExperts, ScaledRotaryTables,
                             SinkRotaryAttention)
from ...utils.paged import HybridCacheManager
from .ragged_decoder import RaggedDecoderForCausalLM

ARCHITECTURE = "Nasozen"
MIXER_TYPES = ("parallel", "mlstm", "general_delta")
MAX_STREAMS = 8


class NasozenConfig:
    """config.json of the family, with the attribute names the runtime reads on any model config."""
    model_type = "nasozen"

    def __init__(self, raw: Dict[str, Any]):
        if raw.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} configuration")
        self.raw = raw
        self.architecture = ARCHITECTURE
        self.vocab_size = int(raw["vocab"])
        self.hidden_size = int(raw["width"])
        self.layers: List[Dict[str, Any]] = list(raw["layers"])
        self.norm_eps = float(raw["norm"]["eps"])
        self.residual_mult = float(raw.get("residual_mult", 1.0))
        self.streams = int(raw["streams"]) if raw.get("streams") else 0      # 0: one stream with plain sums, no hc tensors
        if self.streams > MAX_STREAMS:
            raise NotImplementedError(f"at most {MAX_STREAMS} residual streams")
        self.eos_token_id = raw.get("eos_token_id")
        self.pad_token_id = raw.get("pad_token_id")
        self.quantize = None
        n, loop = len(self.layers), raw.get("loop")
        if loop:
            a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
            if not (0 <= a <= b <= n) or times < 1:
                raise ValueError("loop: need 0 <= start <= stop <= number of layers and times >= 1")
            self.layer_runs = list(range(a)) + list(range(a, b)) * times + list(range(b, n))
        else:
            self.layer_runs = list(range(n))
        self.num_hidden_layers = len(self.layer_runs)     # what the cache manager books: one entry per layer run
        for layer in self.layers:
            if layer["type"] not in MIXER_TYPES:
                raise NotImplementedError(f"mixer type {layer['type']!r}")
            f = layer.get("mlp")
            if f and f.get("kind") not in ("dense", "moe"):
                raise NotImplementedError(f"mlp kind {f.get('kind')!r}")

    @classmethod
    def from_pretrained(cls, model_path: str) -> "NasozenConfig":
        with open(os.path.join(model_path, "config.json")) as f:
            return cls(json.load(f))


def tensor_shapes(raw: Dict[str, Any], decay_rank: int = 16) -> Dict[str, tuple]:
    """name -> shape of every checkpoint tensor of a configuration (synthetic checkpoints).  The rank of the delta rule's decay
    projection is not part of the configuration: a checkpoint's `w1` decides it, a synthetic one takes `decay_rank`."""
    W, V = int(raw["width"]), int(raw["vocab"])
    S = int(raw["streams"]) if raw.get("streams") else 0
    out = {"embed": (V, W), "final.norm": (W,)}
    for i, layer in enumerate(raw["layers"]):
        m, pre = layer["mixer"], f"l{i}"
        if layer["type"] == "parallel":
            a, C = m["left"], int(m["right"]["width"])
            H, G, d, dv = int(a["heads"]), int(a["kv_heads"]), int(a["dim"]), int(a["vdim"])
            mix = {"left.q": (H * d, W), "left.k": (G * d, W), "left.v": (G * dv, W), "left.q.norm": (H * d,), "left.k.norm": (G * d,),
                   "left.sink": (H,), "left.g": (H, W), "left.o": (W, H * dv), "right.z": (C, W), "right.z.b": (C,), "right.x": (C, W),
                   "right.x.b": (C,), "right.g": (C, W), "right.o": (W, C)}
            taps = int(a.get("conv") or 0)
            if taps >= 1:
                mix.update({"left.q.conv": (H * d, taps), "left.k.conv": (G * d, taps), "left.v.conv": (G * dv, taps)})
        elif layer["type"] == "mlstm":
            H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
            mix = {"q": (H * d, W), "k": (H * d, W), "v": (H * dv, W), "g": (H * dv, W), "o": (W, H * dv), "norm": (H * dv,), "i": (H, W),
                   "i.b": (H,), "f": (H, W), "f.b": (H,)}
        else:
            H, d = int(m["heads"]), int(m["dim"])
            rank = int(decay_rank)
            mix = {n: (H * d, W) for n in ("r", "k", "v", "g", "a")}
            mix.update({"a.b": (H * d,), "w1": (rank, W), "w2": (H * d, rank), "w0": (H * d,), "norm": (H * d,), "o": (W, H * d)})
        out[f"{pre}.norm1"] = (W,)
        out.update({f"{pre}.mix.{k}": v for k, v in mix.items()})
        f = layer.get("mlp")
        subs = (1, 2) if f else (1,)
        if S:
            for q in subs:
                out.update({f"{pre}.hc{q}.in": (S,), f"{pre}.hc{q}.out": (S,), f"{pre}.hc{q}.mix": (S, S)})
        if not f:
            continue
        out[f"{pre}.norm2"] = (W,)
        if f["kind"] == "dense":
            ff = int(f["ff"])
            out.update({f"{pre}.mlp.up": (ff, W), f"{pre}.mlp.down": (W, ff)})
        else:
            E, ff = int(f["router"]["experts"]), int(f["expert"]["ff"])
            out[f"{pre}.mlp.router"] = (E, W)
            for e in range(E):
                out.update({f"{pre}.mlp.e{e}.gate": (ff, W), f"{pre}.mlp.e{e}.up": (ff, W), f"{pre}.mlp.e{e}.down": (W, ff)})
    return out


def build_mixer(kind: str, prefix: str, m: Dict[str, Any], weights, eps: float) -> nn.Module:
    if kind == "parallel":
        a = m["left"]
        rot, mask, vdim = a.get("rot"), a.get("mask"), int(a["vdim"])
        rotary = ScaledRotaryTables(int(rot["dims"]), float(rot["base"])) if rot and int(rot.get("dims", 0)) > 0 else None
        # the values turn over all their columns with the rotation's base, pair m by position * base^(-2m / vdim), whatever part
        # of a key head turns
        value_rotary = ScaledRotaryTables(vdim, float(rot["base"])) if rot else None
        left = SinkRotaryAttention(f"{prefix}.left", weights, heads=int(a["heads"]), kv_heads=int(a["kv_heads"]), dim=int(a["dim"]), vdim=vdim,
                                   scale=float(a["scale"]), rotary=rotary, value_rotary=value_rotary, value_pairs="halves",
                                   conv=int(a.get("conv") or 0), window=int(mask["size"]) if mask else None, sink=True, head_gate=True, eps=eps)
        right = MinGRUMixer(f"{prefix}.right", weights, width=int(m["right"]["width"]))
        return ParallelMixers(left, right, float(m["left_scale"]), float(m["right_scale"]))
    if kind == "mlstm":
        return MLSTMMixer(prefix, weights, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), gate_cap=float(m["gate_cap"]), eps=eps,
                          out_dtype=torch.float32)
    if kind == "general_delta":
        return GeneralDeltaMixer(prefix, weights, heads=int(m["heads"]), dim=int(m["dim"]), eps=eps)
    raise NotImplementedError(f"mixer type {kind!r}")


class SoftmaxRouted(nn.Module):
    """`top` of `experts` SiLU-gated experts, weights = soft-max scores of the picked experts over their sum (which is the soft-max
    over the picked logits alone) -> fp32 [T, width]"""

    def __init__(self, prefix: str, f: Dict[str, Any], weights):
        super().__init__()
        r = f["router"]
        self.routed = RoutedExperts(prefix, weights, experts=int(r["experts"]), top=int(r["top"]), limit=None)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        y, routing = self.routed(h)
        out = torch.zeros(h.shape[0], y.shape[1], dtype=torch.float32, device=h.device)
        ops.moe_combine_add(out, None, y, routing)
        return out


class _Sublayer(nn.Module):
    """the way in and out of one sublayer: read coefficients, norm weight, mixing matrix and write coefficients (fp32, the write
    coefficients already times residual_mult)"""

    def __init__(self, pre: str, q: int, weights, config: NasozenConfig):
        super().__init__()
        dev = weights.device
        self.norm_w = weights.get_tensor(f"{pre}.norm{q}").contiguous()
        if config.streams:
            f32 = lambda n: weights.get_tensor(f"{pre}.hc{q}.{n}").to(torch.float32).contiguous()  # noqa: E731
            self.c_in, self.c_mix, self.c_out = f32("in"), f32("mix"), (f32("out") * config.residual_mult).contiguous()
            S = config.streams
            if self.c_in.shape != (S,) or self.c_mix.shape != (S, S) or self.c_out.shape != (S,):
                raise ValueError(f"{pre}.hc{q}: coefficient shapes do not match {S} streams")
        else:
            self.c_in = torch.ones(1, dtype=torch.float32, device=dev)
            self.c_mix = torch.ones(1, 1, dtype=torch.float32, device=dev)
            self.c_out = torch.full((1,), config.residual_mult, dtype=torch.float32, device=dev)


class NasozenLayer(nn.Module):
    """one layer run: `index` is the run (its cache and state), the modules may be another run's (a looped layer)"""

    def __init__(self, index: int, layer: int, config: NasozenConfig, weights, share: Optional["NasozenLayer"] = None):
        super().__init__()
        self.index, self.layer = index, layer
        if share is not None:
            self.mixer, self.mlp, self.sub1, self.sub2 = share.mixer, share.mlp, share.sub1, share.sub2
            return
        spec, pre, eps = config.layers[layer], f"l{layer}", config.norm_eps
        self.mixer = build_mixer(spec["type"], f"{pre}.mix", spec["mixer"], weights, eps)
        self.sub1 = _Sublayer(pre, 1, weights, config)
        f = spec.get("mlp")
        self.mlp, self.sub2 = None, None
        if f:
            self.mlp = PlainMLP(f"{pre}.mlp", weights, activation="gelu_tanh") if f["kind"] == "dense" else SoftmaxRouted(f"{pre}.mlp", f, weights)
            self.sub2 = _Sublayer(pre, 2, weights, config)

    def subs(self):
        return [self.sub1] + ([self.sub2] if self.sub2 is not None else [])

    def mix(self, h, step, manager: HybridCacheManager, max_s: int) -> torch.Tensor:
        if isinstance(self.mixer, MLSTMMixer):
            return self.mixer(h, step, manager.layer_state(self.index), max_s)
        return self.mixer(h, step, manager.layer_pages(self.index), manager.layer_state(self.index), max_s)


class _SumNorm(nn.Module):
    """the model's norm over the sum of the streams (what `final_norm` means for this family: it takes the streams [T, S, W])"""

    def __init__(self, name: str, weights, eps: float, streams: int):
        super().__init__()
        self.w, self.eps = weights.get_tensor(name).contiguous(), eps
        self.ones = torch.ones(max(streams, 1), dtype=torch.float32, device=weights.device)

    def forward(self, X):
        return ops.streams_step(X, in_coef=self.ones, norm_w=self.w, eps=self.eps)


class NasozenModel(nn.Module):
    def __init__(self, config: NasozenConfig, weights):
        super().__init__()
        self.config = config
        self.embed = weights.get_tensor("embed").contiguous()
        self.dtype = self.embed.dtype
        first: Dict[int, NasozenLayer] = {}
        runs = []
        for i, layer in enumerate(config.layer_runs):
            run = NasozenLayer(i, layer, config, weights, share=first.get(layer))
            first.setdefault(layer, run)
            runs.append(run)
        self.layers = nn.ModuleList(runs)
        self.final_norm = _SumNorm("final.norm", weights, config.norm_eps, config.streams)
        self.kv_cache_manager: Optional[HybridCacheManager] = None
        self.residual_probe: Optional[list] = None  # when a list: receives the sum of the streams after every layer run (tests)

    def forward(self, input_ids, step: ops.RaggedStep, max_s: int) -> torch.Tensor:
        """-> the streams, fp32 [T, S, W].  Between two sublayers ONE launch writes the streams with the last result and reads the
        next sublayer's normed input; the first launch also spreads the embedding output over the streams."""
        x0 = ops.embed_scale(self.embed, input_ids, 1.0)
        T, W, eps = x0.shape[0], x0.shape[1], self.config.norm_eps
        X = torch.empty(T, max(self.config.streams, 1), W, dtype=torch.float32, device=x0.device)
        subs = [(run, q, s) for run in self.layers for q, s in enumerate(run.subs())]
        h = ops.streams_step(X, init=x0, in_coef=subs[0][2].c_in, norm_w=subs[0][2].norm_w, eps=eps)
        for n, (run, q, s) in enumerate(subs):
            y = run.mix(h, step, self.kv_cache_manager, max_s) if q == 0 else run.mlp(h)
            last_of_run = n + 1 == len(subs) or subs[n + 1][0] is not run
            nxt = subs[n + 1][2] if n + 1 < len(subs) else None
            h = ops.streams_step(X, y=y, mix=s.c_mix, out_coef=s.c_out, in_coef=nxt.c_in if nxt else None, norm_w=nxt.norm_w if nxt else None,
                                 eps=eps)
            if last_of_run and self.residual_probe is not None:
                self.residual_probe.append(X.sum(1))
        return X


class NasozenForCausalLM(RaggedDecoderForCausalLM):
    def __init__(self, config: NasozenConfig, weights):
        super().__init__(config, weights, NasozenModel(config, weights), head_tensor="embed")
