"""Noganex without a GPU: the configuration reader and its refusals, the checkpoint table against the reference's, the cache
manager's bookkeeping for a stack that mixes paged and state layers with shared tensors, and properties of the slow reference
itself (so that a GPU test that agrees with it agrees with the mechanism)."""
import copy

import pytest
import torch

from oracle import noganex as orc


def test_config_reader_and_refusals():
    import tgis_b200  # noqa: F401
    from tgis_b200.models.custom_modeling.noganex_modeling import NoganexConfig, tensor_shapes
    raw = orc.random_config()
    cfg = NoganexConfig(raw)
    assert cfg.model_type == "noganex" and cfg.num_hidden_layers == 4 and cfg.hidden_size == 40 and cfg.logit_scale == 0.5
    assert [cfg.weight_layer(i) for i in range(4)] == [0, 1, 0, 3]
    assert tensor_shapes(raw) == orc.tensor_shapes(raw)
    assert not any(k.startswith("l2.") for k in tensor_shapes(raw))          # a sharing layer has no tensors
    with pytest.raises(ValueError):
        NoganexConfig(dict(raw, architecture="Other"))
    bad = copy.deepcopy(raw)
    bad["layers"][1]["type"] = "conv_only"
    with pytest.raises(NotImplementedError):
        NoganexConfig(bad)
    bad = copy.deepcopy(raw)
    bad["layers"][2]["weights_of"] = 1                                       # an attention layer's tensors for a delta layer
    with pytest.raises(ValueError):
        NoganexConfig(bad)
    bad = copy.deepcopy(raw)
    bad["layers"][0]["weights_of"] = 2                                       # a ring
    with pytest.raises(ValueError):
        NoganexConfig(bad)
    chain = copy.deepcopy(raw)
    chain["layers"].append(dict(chain["layers"][2], weights_of=2))           # 4 -> 2 -> 0
    assert NoganexConfig(chain).weight_layer(4) == 0


def test_engine_recognises_the_architecture(tmp_path):
    import json
    import tgis_b200  # noqa: F401
    from tgis_b200.inference_engine import FLASH_TYPES, load_config
    with open(tmp_path / "config.json", "w") as f:
        json.dump(orc.random_config(), f)
    cfg = load_config(str(tmp_path))
    assert cfg.model_type == "noganex" and cfg.model_type in FLASH_TYPES


def test_cache_specs_book_pages_and_slots_per_layer():
    import tgis_b200  # noqa: F401
    from tgis_b200.utils.paged import HybridCacheManager, LayerCacheSpec
    # delta / attention / delta (shared tensors, own state): what the layers of such a stack declare
    delta = LayerCacheSpec("state", state={"S": (4, 12, 20), "conv": (2, 2 * 24 + 80)})
    attn = LayerCacheSpec("paged", row_width=3 * (10 + 14))
    mgr = HybridCacheManager([delta, attn, delta], torch.float32, "cpu", total_num_gpu_blocks=5, num_state_slots=2)
    assert mgr.layer_pages(0) is None and mgr.layer_pages(1).shape == (5, 16, 72)
    assert mgr.layer_state(0)["S"].data_ptr() != mgr.layer_state(2)["S"].data_ptr()
    (a,) = mgr.allocate_tokens([33])
    assert mgr.free_blocks == 2 and mgr.free_state_slots == 1
    mgr.free_sequences([a])
    assert mgr.free_blocks == 5 and mgr.free_state_slots == 2


def test_reference_properties():
    cfg = orc.random_config(order=("attention",), weights_of=(None,), mlp=(None,), chunk=8)
    sd = orc.random_state_dict(cfg, seed=1)
    p = {k: v.double() for k, v in orc.sub(sd, "l0.mix.").items()}
    m = cfg["layers"][0]["mixer"]
    h = torch.randn(30, cfg["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    full = orc.talking_attention(h, p, m, 1e-5)
    # a chunk sees nothing before it: rows 16..23 computed from the chunk alone, at their true positions, are the same
    alone = copy.deepcopy(m)
    h2 = h.clone()
    h2[:16] = torch.randn(16, cfg["width"], dtype=torch.float64)
    assert torch.allclose(orc.talking_attention(h2, p, alone, 1e-5)[16:24], full[16:24], atol=1e-12)
    assert not torch.allclose(orc.talking_attention(h2, p, alone, 1e-5)[8:16], full[8:16], atol=1e-3)
    # an identity mixing matrix is plain attention; any other moves the result
    p_id = dict(p, talk=torch.eye(m["heads"], dtype=torch.float64))
    p_no = {k: v for k, v in p.items() if k != "talk"}
    assert torch.allclose(orc.talking_attention(h, p_id, m, 1e-5), orc.talking_attention(h, p_no, m, 1e-5), atol=1e-12)
    assert not torch.allclose(orc.talking_attention(h, p_id, m, 1e-5), full, atol=1e-3)
    # rotation keeps lengths up to the amplitude and leaves the columns past rot.dims alone
    x = torch.randn(5, 2, m["dim"], dtype=torch.float64)
    y = orc.rotate_half(x, m["rot"])
    _, amp = orc.rotary_frequencies(m["rot"])
    d = m["rot"]["dims"]
    assert torch.allclose(y[..., :d].norm(dim=-1), x[..., :d].norm(dim=-1) * amp) and torch.equal(y[..., d:], x[..., d:])
    assert torch.allclose(y[0], torch.cat([x[0, :, :d] * amp, x[0, :, d:]], -1))        # position 0: no turn


def test_reference_delta_rule_is_a_memory():
    """with full write strength and no decay, writing v at a unit key and reading at the same key gives v back"""
    d, dv = 6, 4
    k = torch.zeros(d, dtype=torch.float64)
    k[2] = 1.0
    S = torch.zeros(d, dv, dtype=torch.float64)
    v1, v2 = torch.arange(4.0, dtype=torch.float64), torch.ones(4, dtype=torch.float64) * 7
    for v in (v1, v2):      # the second write replaces the first: u = v - S^T k
        S = S + torch.outer(k, 1.0 * (v - S.T @ k))
    assert torch.allclose(S.T @ k, v2)
    cfg = orc.random_config(order=("delta",), weights_of=(None,), mlp=(None,))
    sd = orc.random_state_dict(cfg, seed=2)
    toks = list(range(4, 30))
    a = orc.forward(cfg, sd, toks)
    b = orc.forward(cfg, sd, toks[:20])
    assert torch.allclose(a[:20], b, atol=1e-12)                                          # causal
