"""Nasozen without a GPU: the configuration reader (layer runs of a loop, optional entries) and its refusals, the checkpoint table
against the reference's, the cache manager's bookkeeping for a stack whose looped layers keep a store per pass, and properties
of the slow reference itself (so that a GPU test that agrees with it agrees with the mechanism)."""
import copy
import math

import pytest
import torch

from oracle import nasozen as orc


def test_config_reader_layer_runs_and_refusals():
    import tgis_b200  # noqa: F401
    from tgis_b200.models.custom_modeling.nasozen_modeling import NasozenConfig, tensor_shapes
    raw = orc.random_config()
    cfg = NasozenConfig(raw)
    assert cfg.model_type == "nasozen" and cfg.hidden_size == 40 and cfg.streams == 3 and cfg.residual_mult == 0.7
    assert cfg.layer_runs == orc.layer_runs(raw) == [0, 1, 2, 1, 2, 3] and cfg.num_hidden_layers == 6
    assert tensor_shapes(raw, 5) == orc.tensor_shapes(raw, 5)
    assert "head" not in tensor_shapes(raw)                                   # the embedding table is the head
    plain = orc.random_config(streams=None, loop=None, conv=None, rot_dims=None, window=None)
    cfg = NasozenConfig(plain)
    assert cfg.streams == 0 and cfg.layer_runs == [0, 1, 2, 3]
    names = tensor_shapes(plain)
    assert not any(".hc" in k or k.endswith(".conv") for k in names) and tensor_shapes(plain, 5) == orc.tensor_shapes(plain, 5)
    assert NasozenConfig(orc.random_config(loop=(0, 4, 3))).layer_runs == [0, 1, 2, 3] * 3
    assert NasozenConfig(orc.random_config(loop=(2, 2, 5))).layer_runs == [0, 1, 2, 3]      # an empty run of layers repeats nothing
    with pytest.raises(ValueError):
        NasozenConfig(dict(raw, architecture="Other"))
    with pytest.raises(ValueError):
        NasozenConfig(dict(raw, loop={"start": 3, "stop": 2, "times": 2}))
    with pytest.raises(NotImplementedError):
        NasozenConfig(dict(raw, streams=9))
    bad = copy.deepcopy(raw)
    bad["layers"][1]["type"] = "conv_only"
    with pytest.raises(NotImplementedError):
        NasozenConfig(bad)
    bad = copy.deepcopy(raw)
    bad["layers"][0]["mlp"]["kind"] = "sparse"
    with pytest.raises(NotImplementedError):
        NasozenConfig(bad)


def test_engine_recognises_the_architecture(tmp_path):
    import json
    import tgis_b200  # noqa: F401
    from tgis_b200.inference_engine import FLASH_TYPES, load_config
    with open(tmp_path / "config.json", "w") as f:
        json.dump(orc.random_config(), f)
    cfg = load_config(str(tmp_path))
    assert cfg.model_type == "nasozen" and cfg.model_type in FLASH_TYPES


def test_cache_specs_book_a_store_per_layer_run():
    import tgis_b200  # noqa: F401
    from tgis_b200.utils.paged import HybridCacheManager, LayerCacheSpec
    # parallel / delta / delta again (the same layer's second pass) : what the runs of such a stack declare
    par = LayerCacheSpec("paged", row_width=2 * (10 + 12), state={"left.conv": (2, 104), "right.S": (28,)})
    delta = LayerCacheSpec("state", state={"S": (2, 12, 12)})
    mgr = HybridCacheManager([par, delta, delta], torch.float32, "cpu", total_num_gpu_blocks=5, num_state_slots=2)
    assert mgr.layer_pages(0).shape == (5, 16, 44) and mgr.layer_pages(1) is None
    assert mgr.layer_state(0)["right.S"].shape == (2, 28)
    assert mgr.layer_state(1)["S"].data_ptr() != mgr.layer_state(2)["S"].data_ptr()
    (a,) = mgr.allocate_tokens([33])
    assert mgr.free_blocks == 2 and mgr.free_state_slots == 1
    mgr.free_sequences([a])
    assert mgr.free_blocks == 5 and mgr.free_state_slots == 2


def _attention(seed=1, **kw):
    cfg = orc.random_config(order=("parallel",), loop=None, mlp=(None,), **kw)
    sd = orc.random_state_dict(cfg, seed=seed)
    return cfg["layers"][0]["mixer"]["left"], {k: v.double() for k, v in orc.sub(sd, "l0.mix.left.").items()}, cfg


def test_reference_attention_properties():
    m, p, cfg = _attention(window=8, conv=None)
    g = torch.Generator().manual_seed(0)
    h = torch.randn(30, cfg["width"], dtype=torch.float64, generator=g)
    full = orc.sink_window_attention(h, p, m, 1e-5)
    # a row sees itself and the window - 1 rows before it, nothing older: rows 20.. do not move when rows 0..12 change, row 19 does
    h2 = h.clone()
    h2[:13] = torch.randn(13, cfg["width"], dtype=torch.float64, generator=g)
    other = orc.sink_window_attention(h2, p, m, 1e-5)
    assert torch.allclose(other[20:], full[20:], atol=1e-12) and not torch.allclose(other[19], full[19], atol=1e-4)
    # the values' turn and the turn back cancel for the query's own position and depend on differences only: without a window, a
    # sequence whose keys and values are all equal gives that value back, scaled by what the sink leaves
    m2, p2, cfg2 = _attention(window=None, conv=None, seed=3)
    x = torch.randn(4, 2, m2["vdim"], dtype=torch.float64, generator=g)
    pos = torch.tensor([3, 9, 0, 100])
    there = orc.turn_halves(x, pos, m2["vdim"], 50.0)
    assert torch.allclose(orc.turn_halves(there, pos, m2["vdim"], 50.0, sign=-1.0), x, atol=1e-12)
    assert torch.allclose(there.norm(dim=-1), x.norm(dim=-1))
    assert torch.equal(orc.turn_halves(x, torch.zeros(4, dtype=torch.long), 6, 50.0), x)
    shifted = orc.turn_halves(orc.turn_halves(x, pos + 17, m2["vdim"], 50.0), torch.full((4,), 17), m2["vdim"], 50.0, sign=-1.0)
    assert torch.allclose(shifted, there, atol=1e-12)
    assert torch.allclose(orc.turn_neighbours(orc.turn_neighbours(x, pos, 8, 50.0), pos, 8, 50.0, sign=-1.0), x, atol=1e-12)
    # the sink: minus infinity is a plain soft-max, a huge one silences the head; a sink weighs once whatever the row's length
    no_sink = orc.sink_window_attention(h, {k: v for k, v in p.items() if k != "sink"}, m, 1e-5)
    low = orc.sink_window_attention(h, dict(p, sink=torch.full_like(p["sink"], -1e4)), m, 1e-5)
    high = orc.sink_window_attention(h, dict(p, sink=torch.full_like(p["sink"], 1e4)), m, 1e-5)
    assert torch.allclose(low, no_sink, atol=1e-12) and float(high.abs().max()) < 1e-12 and not torch.allclose(full, no_sink, atol=1e-3)
    # a single tap is a weight per channel, not the identity
    m3, p3, cfg3 = _attention(conv=1, seed=4)
    h3 = torch.randn(6, cfg3["width"], dtype=torch.float64, generator=g)
    assert torch.allclose(orc.short_conv(h3 @ p3["v"].T, p3["v.conv"]), (h3 @ p3["v"].T) * p3["v.conv"][:, 0])


def test_reference_recurrences():
    g = torch.Generator().manual_seed(5)
    # the gated unit: z = 1 copies the candidate, z = 0 keeps the (zero) state; the candidate's branches are u + 1/2 and sigmoid(u)
    W, C = 8, 6
    rnd = lambda *shape: torch.randn(*shape, dtype=torch.float64, generator=g)  # noqa: E731
    p = {"z": torch.zeros(C, W, dtype=torch.float64), "x": rnd(C, W), "g": rnd(C, W), "z.b": torch.full((C,), 40.0, dtype=torch.float64),
         "x.b": rnd(C), "o": torch.eye(C, dtype=torch.float64)}
    h = rnd(5, W)
    u = h @ p["x"].T + p["x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    assert torch.allclose(orc.min_gru(h, p), cand * orc.silu(h @ p["g"].T), atol=1e-12)
    assert float(orc.min_gru(h, dict(p, **{"z.b": torch.full((C,), -800.0, dtype=torch.float64)})).abs().max()) == 0.0
    # the delta rule: with no decay (w = 1) and full removal (a = 1), writing at a unit key and reading there returns the value,
    # and a second write at the same key replaces the first
    d = 5
    k = torch.zeros(d, dtype=torch.float64)
    k[1] = 1.0
    S = torch.zeros(d, d, dtype=torch.float64)
    for v in (torch.arange(5.0, dtype=torch.float64), torch.full((d,), 7.0, dtype=torch.float64)):
        S = S - torch.outer(k, k @ S) + torch.outer(k, v)
    assert torch.allclose(S.T @ k, torch.full((d,), 7.0, dtype=torch.float64))
    # the decay lies in (exp(-exp(-1/2)), 1)
    cfg = orc.random_config(order=("general_delta", "mlstm"), loop=None, mlp=(None, None), streams=2)
    sd = orc.random_state_dict(cfg, seed=2)
    assert 0.54 < math.exp(-math.exp(-0.5)) < 0.55
    toks = list(range(4, 30))
    a, b = orc.forward(cfg, sd, toks), orc.forward(cfg, sd, toks[:20])
    assert torch.allclose(a[:20], b, atol=1e-12)                                             # causal


def test_reference_streams_and_loop():
    """one stream with unit coefficients is the plain pre-norm sum; a loop of one pass is no loop; a loop shares tensors, not memory"""
    base = orc.random_config(streams=None, loop=None)
    sd = orc.random_state_dict(base, seed=6)
    toks = list(range(5, 25))
    ref = orc.forward(base, sd, toks)
    one = dict(base, streams=1)
    sd1 = dict(sd)
    for i, layer in enumerate(base["layers"]):
        for q in (1, 2) if layer.get("mlp") else (1,):
            sd1.update({f"l{i}.hc{q}.in": torch.ones(1), f"l{i}.hc{q}.out": torch.ones(1), f"l{i}.hc{q}.mix": torch.ones(1, 1)})
    assert torch.allclose(orc.forward(one, sd1, toks), ref, atol=1e-12)
    assert torch.allclose(orc.forward(dict(base, loop={"start": 1, "stop": 3, "times": 1}), sd, toks), ref, atol=1e-12)
    twice = orc.forward(dict(base, loop={"start": 1, "stop": 3, "times": 2}), sd, toks)
    unrolled = copy.deepcopy(base)
    unrolled["layers"] = [base["layers"][i] for i in (0, 1, 2, 1, 2, 3)]
    sdu = {}
    for new, old in enumerate((0, 1, 2, 1, 2, 3)):
        sdu.update({f"l{new}." + k[len(f"l{old}."):]: v for k, v in sd.items() if k.startswith(f"l{old}.")})
    sdu.update({k: v for k, v in sd.items() if not k.startswith("l")})
    assert torch.allclose(orc.forward(unrolled, sdu, toks), twice, atol=1e-12)
    res = []
    orc.forward(dict(base, loop={"start": 1, "stop": 3, "times": 2}), sd, toks, residuals=res)
    assert len(res) == 6
