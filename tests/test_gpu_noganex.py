"""Noganex on the GPU against the slow CPU reference (oracle/noganex.py, float64): each mechanism alone, then the model through
the engine's step function and cache manager - whole prompts, token-by-token decoding, portions down to two tokens, ragged
batches, pages and state slots that are freed and used again - and greedy generation through FlashCausalLM.generate_token.

The configurations are small and uneven (key size != value size, head counts that differ between the two mixers, one and several
query heads per key head, one to four convolution taps, partial and full rotation, one expert per token and all experts per
token).  Where random weights would hide a fault the test makes it show: a key that must win the soft-max from far away, at a page
border, at the first positions, just inside and just outside a chunk; a head whose weights come from another head's scores
through the mixing matrix; a correction that changes the picked experts but not their weights."""
import copy
import json
import math
import os

import pytest
import torch

from oracle import noganex as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL32, TOL16 = 2e-4, 0.3


# ------------------------------------------------------------------------------------------------ helpers
def _model(tmp_path, config, sd, dtype=torch.float32, blocks=64, slots=4):
    from safetensors.torch import save_file
    import tgis_b200  # noqa: F401
    from tgis_b200.inference_engine import InferenceEngine
    from tgis_b200.models.flash_causal_lm import FlashCausalLM
    from tgis_b200.utils.dist import FakeGroup
    from tgis_b200.utils.synthetic import make_tokenizer
    from tgis_b200.utils.weights import Weights

    d = str(tmp_path)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(config, f)
    path = os.path.join(d, "model.safetensors")
    save_file({k: v.contiguous() for k, v in sd.items()}, path)
    weights = Weights([path], device=DEV, dtype=dtype, process_group=FakeGroup(0, 1))
    engine = InferenceEngine(d, None, dtype, None, None, None, weights=weights, tokenizer=make_tokenizer(config["vocab"]))
    return FlashCausalLM(d, None, "tgis_native", dtype, None, None, engine=engine, num_kv_blocks=blocks, num_state_slots=slots)


def _tokens(seed, n, vocab):
    return torch.randint(4, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _rel(got, ref):
    """largest row error relative to the spread of the reference logits"""
    got, ref = got.double().cpu(), ref.double()
    return float(((got - ref).pow(2).mean(-1).sqrt() / ref.std()).max())


def _decided(config, sd, tokens, least=0.05):
    """positions whose routing is no close call in any layer: where bfloat16 must pick the reference's experts"""
    margins = []
    orc.forward(config, sd, tokens, margins=margins)
    if not margins:
        return torch.ones(len(tokens), dtype=torch.bool)
    return torch.stack(margins).min(0).values > least


def _run_cut(model, tokens, cuts):
    """one sequence in portions of the given sizes (the rest token by token) -> logits of every position"""
    sid, at, rows = None, 0, []
    sizes = list(cuts) + [1] * (len(tokens) - sum(cuts))
    for n in sizes:
        sids, lg = model.step_ragged([sid], [tokens[at:at + n]])
        sid, at = sids[0], at + n
        rows.append(lg)
    model.kv_cache_manager.free_sequences([sid])
    return torch.cat(rows)


class _DictWeights:
    def __init__(self, sd, dtype):
        from tgis_b200.utils.dist import FakeGroup
        self.sd, self.dtype, self.device, self.process_group = sd, dtype, DEV, FakeGroup(0, 1)

    def get_tensor(self, name):
        return self.sd[name].to(self.dtype).to(DEV)


def _step(starts_and_counts, tables):
    """RaggedStep for sequences (start, count) whose pages are given by `tables` (one list of block ids per sequence)"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq
    pos, seq, slots, cu = [], [], [], [0]
    for b, (start, n) in enumerate(starts_and_counts):
        for p in range(start, start + n):
            pos.append(p)
            seq.append(b)
            slots.append(tables[b][p // 16] * 16 + p % 16)
        cu.append(cu[-1] + n)
    width = max(len(t) for t in tables)
    bt = torch.zeros(len(tables), width, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t)
    return ops_seq.RaggedStep(T=len(pos), B=len(tables), position_ids=torch.tensor(pos, dtype=torch.int64, device=DEV),
                              cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV), seq_of_token=torch.tensor(seq, dtype=torch.int32, device=DEV),
                              slot_mapping=torch.tensor(slots, dtype=torch.int64, device=DEV), block_table=bt.to(DEV),
                              state_slots=torch.arange(len(tables), dtype=torch.int32, device=DEV))


# ------------------------------------------------------------------------------------------------ mechanisms alone
def test_row_kernels_match_reference():
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    g = torch.Generator().manual_seed(0)
    T, W, eps = 7, 52, 1e-5
    y, gate, x0 = torch.randn(T, W, generator=g) * 3, torch.randn(T, W, generator=g) * 2, torch.randn(T, W, generator=g)
    for dtype in (torch.float32, torch.bfloat16):
        w = (1 + 0.3 * torch.randn(W, generator=g)).to(dtype)
        for gt in (gate, None):
            v = y.double() * (torch.sigmoid(gt.double()) if gt is not None else 1.0)
            ref = x0.double() + orc.unit_rms(v, eps) * w.double()
            x = x0.clone().to(DEV)
            typed = ops.gated_rms_add(x, y.to(DEV), None if gt is None else gt.to(DEV), w.to(DEV), eps, typed_copy=True)
            assert float((x.cpu().double() - ref).abs().max()) < 2e-5
            assert typed.dtype == dtype and float((typed.cpu().double() - ref).abs().max()) < (2e-5 if dtype == torch.float32 else 0.04)
        assert torch.equal(ops.cast_rows(x0.to(DEV), dtype).cpu(), x0.to(dtype))
        gu = (torch.randn(T, 2 * 18, generator=g) * 2).to(dtype)
        for act, fn in ((ops.ACT_SILU, orc.silu), (ops.ACT_GELU_TANH, orc.gelu_tanh)):
            ref = fn(gu[:, :18].double()) * gu[:, 18:].double()
            got = ops.ff_gate(gu.to(DEV), act).cpu().double()
            assert float((got - ref).abs().max()) < (1e-5 if dtype == torch.float32 else 0.05)
    # unit-RMS per group, a weight per column, SiLU gate after the weight
    H, dv = 3, 14
    o, gl, wn = torch.randn(T, H * dv, generator=g), torch.randn(T, H * dv, generator=g), 1 + 0.3 * torch.randn(dv, generator=g)
    ref = (orc.unit_rms(o.double().view(T, H, dv), eps) * wn.double()).view(T, H * dv) * orc.silu(gl.double())
    got = ops.group_rmsnorm_gate(o.to(DEV), wn.repeat(H).to(DEV), H, eps, torch.float32, gate=gl.to(DEV), gate_kind=ops.GATE_SILU_AFTER)
    assert float((got.cpu().double() - ref).abs().max()) < 1e-5


@pytest.mark.parametrize("scaling", [None, {"factor": 4.0, "fast": 8.0, "original": 32, "slow": 1.0}, {"factor": 6.0, "fast": 16.0, "original": 64, "slow": 2.0}])
def test_rotary_tables_match_reference(scaling):
    import tgis_b200  # noqa: F401
    from tgis_b200.utils.mixers import ScaledRotaryTables
    rot = {"base": 100.0, "dims": 12, "scaling": scaling}
    f, amp = orc.rotary_frequencies(rot)
    cos, sin = ScaledRotaryTables(12, 100.0, scaling).tables(300, DEV)
    ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    assert float((cos[:300].cpu().double() - torch.cos(ang) * amp).abs().max()) < 1e-6
    assert float((sin[:300].cpu().double() - torch.sin(ang) * amp).abs().max()) < 1e-6
    if scaling:
        plain, _ = orc.rotary_frequencies({"base": 100.0, "dims": 12})
        assert float(f[0]) == float(plain[0]) and float(f[-1]) < float(plain[-1]) and amp > 1.0   # fast pairs kept, slow ones slowed


@pytest.mark.parametrize("E,top", [(5, 2), (3, 3), (7, 1), (40, 4)])
def test_scored_routing_picks_and_weights(E, top):
    """picks by sigmoid + correction, weights by the plain sigmoid: a correction large enough to change the picks leaves the weights
    of the picks as the scores say"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    g = torch.Generator().manual_seed(E)
    T = 33
    z = torch.randn(T, E, generator=g) * 2
    corr = torch.randn(E, generator=g) * 0.8
    s = torch.sigmoid(z.double())
    val, idx = torch.topk(s + corr.double(), top, dim=-1)
    picked = torch.gather(s, 1, idx)
    want = picked / picked.sum(-1, keepdim=True) * 1.7
    r = ops.moe_route(z.to(DEV), top, sigmoid_scores=True, correction=corr.to(DEV), weight_scale=1.7)
    ids, wg = r.ids.cpu().long(), r.weights.cpu().double()
    order = ids.argsort(-1)
    assert torch.equal(torch.gather(ids, 1, order), idx.sort(-1).values)
    assert float((torch.gather(wg, 1, order) - torch.gather(want, 1, idx.argsort(-1))).abs().max()) < 1e-6
    if top < E:
        assert not torch.equal(idx.sort(-1).values, torch.topk(s, top, dim=-1).indices.sort(-1).values)   # the correction matters
    plain = ops.moe_route(z.to(DEV), top)   # the other rule still holds: soft-max over the largest logits
    v0, i0 = torch.topk(z.double(), top, dim=-1)
    assert torch.equal(plain.ids.cpu().long().sort(-1).values, i0.sort(-1).values)
    assert float((plain.weights.cpu().double().sort(-1).values - torch.softmax(v0, -1).sort(-1).values).abs().max()) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,ff,shared", [(5, 2, 24, 16), (3, 3, 10, None), (6, 1, 72, 8), (16, 4, 64, 64)])
def test_routed_experts_with_shared_match_reference(E, top, ff, shared, dtype):
    import tgis_b200  # noqa: F401
    from tgis_b200.models.custom_modeling.noganex_modeling import RoutedWithShared
    W = 64
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": E, "top": top, "scale": 2.5}, "shared": {"ff": shared} if shared else None}
    cfg = {"architecture": "Noganex", "layers": [{"type": "delta", "mixer": {"conv": 2, "dim": 4, "heads": 1, "kv_heads": 1, "vdim": 4}, "mlp": f}],
           "norm": {"eps": 1e-5}, "vocab": 8, "width": W}
    sd = orc.random_state_dict(cfg, seed=3)
    mod = RoutedWithShared("l0.mlp", f, _DictWeights(sd, dtype))
    p64 = {k: v.double() for k, v in orc.sub(sd, "l0.mlp.").items()}
    g = torch.Generator().manual_seed(2)
    for T in (1, 9, 200):
        h = torch.randn(T, W, generator=g).to(dtype)
        margins = []
        ref = orc.routed_experts(h.double(), p64, f, margins)
        got = mod(h.to(DEV)).cpu().double()
        sure = margins[0] > (0.0 if dtype == torch.float32 else 0.03)
        if not bool(sure.any()):
            continue
        err = float((got[sure] - ref[sure]).abs().max() / ref.abs().max())
        assert err < (2e-5 if dtype == torch.float32 else 0.05), (T, err)
        if T > 1:   # a row's result does not depend on the rest of the step
            alone = mod(h[3:4].to(DEV)).cpu().double()
            assert float((alone - got[3:4]).abs().max()) < (1e-5 if dtype == torch.float32 else 0.05) * float(ref.abs().max())


MIXER_CASES = [
    ("delta", {"conv": 3, "dim": 12, "heads": 4, "kv_heads": 2, "vdim": 20}),
    ("delta", {"conv": 1, "dim": 70, "heads": 2, "kv_heads": 2, "vdim": 40}),     # key size past 64, two blocks of value columns
    ("delta", {"conv": 4, "dim": 8, "heads": 6, "kv_heads": 1, "vdim": 5}),
    ("delta", {"conv": 2, "dim": 32, "heads": 3, "kv_heads": 3, "vdim": 64}),
    ("attention", {"dim": 10, "heads": 6, "kv_heads": 3, "vdim": 14, "scale": 0.6, "mask": {"size": 24},
                   "rot": {"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "fast": 8.0, "original": 32, "slow": 1.0}}}),
    ("attention", {"dim": 12, "heads": 5, "kv_heads": 1, "vdim": 36, "scale": 0.5, "mask": {"size": 7}, "rot": {"base": 50.0, "dims": 12}}),
    ("attention", {"dim": 6, "heads": 12, "kv_heads": 4, "vdim": 6, "scale": 0.9, "rot": {"base": 10.0, "dims": 2}}),       # no chunks, two slabs of heads
    ("attention", {"dim": 8, "heads": 3, "kv_heads": 3, "vdim": 8, "scale": 0.7, "mask": {"size": 16}}),                      # no rotation
    # shapes that take the tensor-core attention kernel when the cache is bfloat16 (sizes in 16s)
    ("attention", {"dim": 16, "heads": 8, "kv_heads": 2, "vdim": 32, "scale": 0.5, "mask": {"size": 20},
                   "rot": {"base": 100.0, "dims": 16, "scaling": {"factor": 4.0, "fast": 8.0, "original": 32, "slow": 1.0}}}),
    ("attention", {"dim": 32, "heads": 4, "kv_heads": 4, "vdim": 16, "scale": 0.3, "mask": {"size": 33}, "rot": {"base": 100.0, "dims": 8}}),
    ("attention", {"dim": 64, "heads": 16, "kv_heads": 2, "vdim": 64, "scale": 0.2, "rot": {"base": 1000.0, "dims": 32}}),
    # three heads per key head (a query tile of 16 tokens), the widest value size of the tensor-core kernel, and as many key heads as
    # heads with too many rows for one block (plain kernel although the sizes are in 16s)
    ("attention", {"dim": 32, "heads": 6, "kv_heads": 2, "vdim": 64, "scale": 0.3, "mask": {"size": 18}, "rot": {"base": 100.0, "dims": 32}}),
    ("attention", {"dim": 32, "heads": 4, "kv_heads": 2, "vdim": 128, "scale": 0.3, "mask": {"size": 40}, "rot": {"base": 100.0, "dims": 16}}),
    ("attention", {"dim": 16, "heads": 24, "kv_heads": 24, "vdim": 16, "scale": 0.4, "mask": {"size": 29}, "rot": {"base": 100.0, "dims": 16}}),
]


@pytest.mark.parametrize("kind,m", MIXER_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mixer_alone_any_cut(kind, m, dtype):
    """one mixer, two sequences of unequal length, fed whole / in ragged portions / token by token, pages out of order, stores
    filled with NaN first"""
    import tgis_b200  # noqa: F401
    from tgis_b200.models.custom_modeling.noganex_modeling import build_mixer
    W, eps = 64, 1e-5
    cfg = {"architecture": "Noganex", "layers": [{"type": kind, "mixer": m, "mlp": None}], "norm": {"eps": eps}, "vocab": 8, "width": W}
    sd = orc.random_state_dict(cfg, seed=5)
    p64 = {k: v.double() for k, v in orc.sub(sd, "l0.mix.").items()}
    mixer = build_mixer(kind, "l0.mix", m, _DictWeights(sd, dtype), eps)
    spec = mixer.cache_spec()
    g = torch.Generator().manual_seed(1)
    lens = [45, 19]
    hs = [torch.randn(L, W, generator=g).to(dtype) for L in lens]
    fn = orc.talking_attention if kind == "attention" else orc.gated_delta
    refs = [fn(h.double(), p64, m, eps) for h in hs]
    tables = [[5, 0, 3], [7, 1]]
    for cuts in ([(45,), (19,)], [(16, 2, 27), (1, 18)], [(1,) * 45, (1,) * 19], [(7, 30, 8), (5, 5, 9)]):
        pages = torch.full((8, 16, max(spec.row_width, 1)), float("nan"), dtype=dtype, device=DEV)
        state = {n: torch.full((2, *s), float("nan"), dtype=torch.float32, device=DEV) for n, s in (spec.state or {}).items()}
        outs, done, k = [[], []], [0, 0], 0
        while any(d < L for d, L in zip(done, lens)):
            active = [(b, cuts[b][k]) for b in range(2) if k < len(cuts[b])]
            k += 1
            st = _step([(done[b], n) for b, n in active], [tables[b] for b, _ in active])
            st.state_slots = torch.tensor([b for b, _ in active], dtype=torch.int32, device=DEV)
            h = torch.cat([hs[b][done[b]:done[b] + n] for b, n in active]).to(DEV)
            y = mixer(h, st, pages, state, max(lens))
            at = 0
            for b, n in active:
                outs[b].append(y[at:at + n])
                at += n
                done[b] += n
        for b in range(2):
            got = torch.cat(outs[b]).double().cpu()
            err = float((got - refs[b]).abs().max() / refs[b].abs().max())
            assert err < (2e-5 if dtype == torch.float32 else 0.08), (kind, cuts, b, err)


def test_delta_state_long_run():
    """300 tokens one by one: the memory is carried from step to step in its fp32 slot without drift"""
    import tgis_b200  # noqa: F401
    from tgis_b200.models.custom_modeling.noganex_modeling import build_mixer
    m = {"conv": 2, "dim": 16, "heads": 2, "kv_heads": 1, "vdim": 24}
    cfg = {"architecture": "Noganex", "layers": [{"type": "delta", "mixer": m, "mlp": None}], "norm": {"eps": 1e-5}, "vocab": 8, "width": 64}
    sd = orc.random_state_dict(cfg, seed=9)
    mixer = build_mixer("delta", "l0.mix", m, _DictWeights(sd, torch.float32), 1e-5)
    spec = mixer.cache_spec()
    h = torch.randn(300, 64, generator=torch.Generator().manual_seed(3))
    ref = orc.gated_delta(h.double(), {k: v.double() for k, v in orc.sub(sd, "l0.mix.").items()}, m, 1e-5)
    state = {n: torch.full((1, *s), float("nan"), dtype=torch.float32, device=DEV) for n, s in spec.state.items()}
    out = []
    for t in range(300):
        out.append(mixer(h[t:t + 1].to(DEV), _step([(t, 1)], [list(range(19))]), None, state, 300))
    got = torch.cat(out).cpu().double()
    assert float((got - ref).abs().max() / ref.abs().max()) < 2e-5


def _talk_reference(q, K, V, q_pos, talk, G, scale, chunk):
    """q [n, H, d] at positions q_pos over keys K [L, G, d], V [L, G, dv] -> [n, H, dv] (float64, dense)"""
    H = q.shape[1]
    rep = H // G
    s = torch.einsum("ihd,jhd->hij", q.double(), K.double().repeat_interleave(rep, dim=1)) * scale
    if talk is not None:
        s = torch.einsum("hg,gij->hij", talk.double(), s)
    j = torch.arange(K.shape[0])
    p = torch.tensor(q_pos)
    see = j[None, :] <= p[:, None]
    if chunk:
        see = see & ((j[None, :] // chunk) == (p[:, None] // chunk))
    a = torch.softmax(s.masked_fill(~see, float("-inf")), -1)
    return torch.einsum("hij,jhv->ihv", a, V.double().repeat_interleave(rep, dim=1))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,chunk", [(6, 3, 10, 14, 100), (4, 1, 16, 32, 64), (8, 2, 32, 16, 0), (16, 4, 16, 64, 150), (3, 3, 8, 8, 37)])
def test_attention_loud_keys_at_edges(dtype, H, G, d, dv, chunk):
    """One key is made to dominate ONE head's raw score; the mixing matrix hands that score to another head, whose output must
    then be that key's value - or must not move at all when the key lies outside the query's chunk.  The loud key sits far back,
    on both sides of page borders, at the first positions, at the first and last position of a chunk and just before it; queries
    are single decoded tokens and rows inside a prompt portion."""
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    g = torch.Generator().manual_seed(7)
    L, page = 420, 16
    table = torch.randperm(32, generator=g)[:(L + page - 1) // page].tolist()
    K, V = torch.randn(L, G, d, generator=g) * 0.3, torch.randn(L, G, dv, generator=g)
    qdir = torch.randn(d, generator=g)
    qdir = qdir / qdir.norm()
    talk = torch.eye(H) * 0.5 + torch.randn(H, H, generator=g) * 0.1
    src, dst = 0, H - 1                 # head `src` hears the loud key; head `dst` gets most of its weight from src's score
    talk[dst, src] = 1.5
    scale = 0.8
    size = chunk or 10 ** 9
    q_pos = [400, 419, 17, 2] + ([(400 // size) * size, (400 // size) * size + 1] if chunk else [])
    loud = [0, 1, 15, 16, 17, 31, 32, 200, 399] + ([(400 // size) * size - 1, (400 // size) * size] if chunk else [])
    pool = torch.full((32, page, G * (d + dv)), float("nan"), dtype=dtype, device=DEV)
    for j_loud in loud:
        K2 = K.clone()
        K2[j_loud, src // (H // G)] = qdir * 40.0
        rows = torch.cat([K2.reshape(L, G * d), V.reshape(L, G * dv)], 1).to(dtype)
        for j in range(L):
            pool[table[j // page], j % page] = rows[j].to(DEV)
        Kr, Vr = rows[:, :G * d].float().view(L, G, d), rows[:, G * d:].float().view(L, G, dv)
        q = torch.randn(len(q_pos), H, d, generator=g) * 0.2
        q[:, src] = qdir * 1.0
        ref = _talk_reference(q, Kr, Vr, q_pos, talk, G, scale, chunk)
        # (a) every query as a decoded token of its own sequence (same pages), (b) the queries at 400.. as rows of one portion
        for qs in ([[p] for p in q_pos], [[399 + i for i in range(21)]]):
            if len(qs) == 1:
                qq = torch.randn(21, H, d, generator=g) * 0.2
                qq[:, src] = qdir
                rr = _talk_reference(qq, Kr, Vr, qs[0], talk, G, scale, chunk)
                st = _step([(399, 21)], [table])
            else:
                qq, rr = q, ref
                st = _step([(p, 1) for p in q_pos], [table] * len(q_pos))
            got = ops.talk_attn(qq.to(DEV), pool, st, kv_heads=G, vdim=dv, k_off=0, v_off=G * d, scale=scale, talk=talk.to(DEV), chunk=chunk)
            err = float((got.cpu().double() - rr).abs().max())
            assert err < (1e-4 if dtype == torch.float32 else 0.06), (j_loud, len(qs), err)
        # the test is live: with the key one position off the reference moves far
        seen = [p for p in q_pos if j_loud <= p and (not chunk or j_loud // size == p // size)]
        if seen and j_loud + 1 < L:
            K3 = K.clone()
            K3[j_loud + 1, src // (H // G)] = qdir * 40.0
            off = _talk_reference(q, K3.to(dtype).float(), Vr, q_pos, talk, G, scale, chunk)
            assert float((off - ref).abs().max()) > 0.3


# ------------------------------------------------------------------------------------------------ the model through the engine
def _sharp(config, factor=4.0):
    """soft-max sharp enough that single keys matter to the logits"""
    c = copy.deepcopy(config)
    done = set()
    for layer in c["layers"]:
        if layer["type"] == "attention" and id(layer["mixer"]) not in done:
            layer["mixer"]["scale"] *= factor
            done.add(id(layer["mixer"]))
    return c


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompt_portions_and_decoding_agree_with_reference(tmp_path, dtype):
    # bfloat16: a pick that flips on a near tie would stay in the recurrent memory for many tokens, so no row after it could be
    # compared; there every expert is picked (the weights still come from the scores) and the picks themselves are tested per row
    # in test_routed_experts_with_shared_match_reference
    cfg = _sharp(orc.random_config(order=("delta", "attention", "delta", "attention", "attention"), weights_of=(None, None, 0, None, 1),
                                   mlp=("moe", "dense", "moe", None, "dense"), **({} if dtype == torch.float32 else {"experts": 3, "top": 3})),
                 4.0 if dtype == torch.float32 else 2.0)
    sd = orc.random_state_dict(cfg, seed=11)
    model = _model(tmp_path, cfg, sd, dtype)
    toks = _tokens(2, 75, cfg["vocab"])
    ref = orc.forward(cfg, sd, toks)
    tol = TOL32 if dtype == torch.float32 else TOL16
    sure = _decided(cfg, sd, toks) if dtype == torch.bfloat16 else torch.ones(75, dtype=torch.bool)
    assert bool(sure.all())
    whole = _run_cut(model, toks, [75])
    assert _rel(whole[sure], ref[sure]) < tol
    # the mechanisms are live in this configuration: a reference with a chunk one token longer, without the shared tensors'
    # separate state, with another router scale or logit scale, or with the correction ignored is far outside the tolerance
    if dtype == torch.float32:
        def changed(edit, state=None):
            c2, s2 = copy.deepcopy(cfg), dict(state or sd)
            edit(c2, s2)
            return _rel(orc.forward(c2, s2, toks), ref)
        assert changed(lambda c, s: c["layers"][1]["mixer"]["mask"].update(size=25)) > 20 * TOL32
        assert changed(lambda c, s: c["layers"][1]["mixer"]["rot"].update(dims=6)) > 20 * TOL32
        assert changed(lambda c, s: c["layers"][1]["mixer"]["rot"].pop("scaling")) > 20 * TOL32
        assert changed(lambda c, s: c["layers"][0]["mlp"]["router"].update(scale=1.4)) > 20 * TOL32
        assert changed(lambda c, s: c.update(logit_scale=0.55)) > 20 * TOL32
        assert changed(lambda c, s: s.update({"l0.mlp.correction": torch.zeros_like(s["l0.mlp.correction"])})) > 20 * TOL32
        assert changed(lambda c, s: s.update({"l1.mix.talk": torch.eye(s["l1.mix.talk"].shape[0])})) > 20 * TOL32
        assert changed(lambda c, s: s.update({"l0.rg1.b": s["l0.rg1.b"] + 1.0})) > 20 * TOL32
    for cuts in ([], [40], [2, 2, 2, 19, 3, 16, 17, 2], [16, 16, 16, 16], [24, 24, 24], [23, 2, 23, 2], [1, 20, 22, 31]):
        got = _run_cut(model, toks, cuts)
        assert _rel(got[sure], ref[sure]) < tol, cuts
        if dtype == torch.float32:
            assert _rel(got, whole.cpu()) < 1e-5, cuts  # the cut itself changes nothing beyond rounding
    assert model.kv_cache_manager.free_blocks == model.kv_cache_manager.total_num_gpu_blocks
    assert model.kv_cache_manager.free_state_slots == 4


def test_tensor_core_shapes_through_the_engine(tmp_path):
    """bfloat16 with head sizes in 16s: prompts, portions and decoded tokens take the tensor-core attention kernel; a step mixes
    a long portion (several query tiles) with single tokens"""
    cfg = _sharp(orc.random_config(width=64, order=("attention", "delta", "attention"), weights_of=(None, None, 0), heads=(8, 4), kv_heads=(2, 2),
                                   dim=(32, 16), vdim=(16, 32), rot_dims=16, chunk=60, mlp=("dense", "moe", "dense"), experts=4, top=4), 2.0)
    sd = orc.random_state_dict(cfg, seed=12)
    model = _model(tmp_path, cfg, sd, torch.bfloat16)
    toks = _tokens(3, 150, cfg["vocab"])
    ref, sure = orc.forward(cfg, sd, toks), _decided(cfg, sd, toks)
    assert bool(sure.all())   # every expert is picked: see test_prompt_portions_and_decoding_agree_with_reference
    for cuts in ([150], [100, 2, 40], [1, 70, 33], [5]):
        assert _rel(_run_cut(model, toks, cuts)[sure], ref[sure]) < TOL16, cuts
    other = _tokens(4, 90, cfg["vocab"])
    ref_o, sure_o = orc.forward(cfg, sd, other), _decided(cfg, sd, other)
    (a,), la = model.step_ragged([None], [toks[:20]])
    (a, b), l2 = model.step_ragged([a, None], [toks[20:21], other[:80]])
    (b, a), l3 = model.step_ragged([b, a], [other[80:], toks[21:150]])
    model.kv_cache_manager.free_sequences([a, b])
    assert _rel(torch.cat([la, l2[:1], l3[10:]])[sure], ref[sure]) < TOL16
    assert _rel(torch.cat([l2[1:], l3[:10]])[sure_o], ref_o[sure_o]) < TOL16


def test_residual_stream_after_every_layer(tmp_path):
    cfg = orc.random_config()
    sd = orc.random_state_dict(cfg, seed=4)
    model = _model(tmp_path, cfg, sd, torch.float32)
    toks = _tokens(5, 30, cfg["vocab"])
    want = []
    orc.forward(cfg, sd, toks, residuals=want)
    probe = []
    model.model.model.residual_probe = probe
    sids, _ = model.step_ragged([None], [toks])
    model.model.model.residual_probe = None
    model.kv_cache_manager.free_sequences(sids)
    assert len(probe) == len(want) == 4
    for i, (a, b) in enumerate(zip(probe, want)):
        assert float((a.cpu().double() - b).abs().max()) < 1e-4 * float(b.abs().max()), i


@pytest.mark.parametrize("variant", ["one_key_head", "equal_heads_top1", "all_experts_no_shared", "attention_only_shared_later"])
def test_other_sizes(tmp_path, variant):
    """sizes that a usual configuration makes equal or 1: one key head, as many key heads as query heads, one expert per token,
    every expert per token, one / two / four taps, full and no rotation, a chunk of two tokens, a layer that borrows the tensors of a
    LATER layer, no feed-forward at all, a logit scale of 1"""
    kw = {"one_key_head": dict(heads=(5, 3), kv_heads=(1, 1), dim=(6, 16), vdim=(8, 8), conv=1, experts=4, top=3, rot_dims=6, chunk=2),
          "equal_heads_top1": dict(heads=(3, 2), kv_heads=(3, 2), dim=(14, 6), vdim=(36, 36), conv=4, experts=6, top=1, rot_dims=2, scaling=None,
                                   chunk=0, logit_scale=1.0),
          "all_experts_no_shared": dict(heads=(8, 6), kv_heads=(4, 2), dim=(8, 10), vdim=(10, 40), conv=2, experts=3, top=3, shared_ff=None, width=56,
                                        rot_dims=8, chunk=31, router_scale=1.0),
          "attention_only_shared_later": dict(order=("attention", "attention", "attention"), weights_of=(None, None, None),
                                              mlp=(None, "dense", None), heads=(10, 2), kv_heads=(5, 1), chunk=16)}[variant]
    cfg = _sharp(orc.random_config(**kw), 3.0)
    if variant == "attention_only_shared_later":   # layer 0 uses layer 2's tensors
        cfg["layers"][0] = dict(cfg["layers"][2], weights_of=2)
    sd = orc.random_state_dict(cfg, seed=31)
    model = _model(tmp_path, cfg, sd, torch.float32)
    toks = _tokens(6, 60, cfg["vocab"])
    ref = orc.forward(cfg, sd, toks)
    for cuts in ([60], [3, 30, 2], [17]):
        assert _rel(_run_cut(model, toks, cuts), ref) < TOL32, (variant, cuts)


def test_ragged_batches_reused_pages_and_slots(tmp_path):
    """four requests of unequal length run as mixed steps (portions beside decoded tokens, requests joining and leaving) in a pool
    that is too small for all of them at once and is filled with garbage first: every request equals its run alone"""
    cfg = _sharp(orc.random_config())
    sd = orc.random_state_dict(cfg, seed=21)
    model = _model(tmp_path, cfg, sd, torch.float32, blocks=12, slots=2)
    mgr = model.kv_cache_manager
    for p in mgr.pages:
        if p is not None:
            p.fill_(float("nan"))
    for st in mgr.states:
        for t in (st or {}).values():
            t.fill_(float("nan"))
    lens = {"a": 70, "b": 33, "c": 1, "d": 50}
    toks = {k: _tokens(30 + i, n, cfg["vocab"]) for i, (k, n) in enumerate(lens.items())}
    refs = {k: orc.forward(cfg, sd, v) for k, v in toks.items()}
    plan = [[("a", 20), ("b", 2)], [("a", 1), ("b", 31)], [("a", 30)], [("a", 1)], [("a", 18), ("c", 1)],   # b ends at step 1, a at 4
            [("d", 17)], [("d", 2)], [("d", 1)], [("d", 30)]]
    got = {k: [] for k in lens}
    at = {k: 0 for k in lens}
    live = {}
    for step in plan:
        ids = [live.get(k) for k, _ in step]
        sids, lg = model.step_ragged(ids, [toks[k][at[k]:at[k] + n] for k, n in step])
        o = 0
        for (k, n), sid in zip(step, sids):
            live[k] = sid
            got[k].append(lg[o:o + n])
            o += n
            at[k] += n
            if at[k] == lens[k]:
                mgr.free_sequences([live.pop(k)])
        assert len(live) <= 2
    for k in lens:
        assert at[k] == lens[k]
        assert _rel(torch.cat(got[k]), refs[k]) < TOL32, k
    assert mgr.free_blocks == mgr.total_num_gpu_blocks and mgr.free_state_slots == 2


def test_long_decoding_and_first_tokens(tmp_path):
    """three prompt tokens, then 197 single steps: chunk edges (every 64) pass inside the decoded tokens; the first tokens have
    fewer inputs than taps"""
    cfg = _sharp(orc.random_config(chunk=64, conv=4))
    sd = orc.random_state_dict(cfg, seed=8)
    model = _model(tmp_path, cfg, sd, torch.float32)
    toks = _tokens(9, 200, cfg["vocab"])
    ref = orc.forward(cfg, sd, toks)
    c2 = copy.deepcopy(cfg)
    c2["layers"][1]["mixer"]["mask"]["size"] = 65
    assert _rel(orc.forward(c2, sd, toks)[60:70], ref[60:70]) > 20 * TOL32   # the chunk's edge is live
    got = _run_cut(model, toks, [3])
    assert _rel(got[:8], ref[:8]) < TOL32
    assert _rel(got, ref) < TOL32
    one = _run_cut(model, toks[:1], [1])  # a request of a single token
    assert _rel(one, ref[:1]) < TOL32


def test_greedy_generation_through_generate_token(tmp_path):
    """from_pb -> generate_token (prefill, decode steps, a second batch joined by concatenate, prune of a finished request):
    the engine's own scheduler path picks the reference's greedy tokens wherever the reference's top-2 gap is decisive"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import pb
    cfg = orc.random_config()
    sd = orc.random_state_dict(cfg, seed=13)
    model = _model(tmp_path, cfg, sd, torch.float32, blocks=64, slots=6)
    tok = model.tokenizer
    V = cfg["vocab"]

    def text(ids):
        return " ".join("test" if i == 3 else f"<tok{i}>" for i in ids)

    def batch_of(bid, prompts, n_new, first_id):
        reqs = [pb.Request(id=first_id + i, inputs=text(p), input_length=len(p), truncate=False, max_output_length=n_new,
                           parameters=pb.NextTokenChooserParameters(temperature=0.0, top_p=1.0, min_new_tokens=n_new))
                for i, p in enumerate(prompts)]
        return pb.Batch(id=bid, requests=reqs)

    def oracle_greedy(prompt, n_new):
        seq, out, sure = list(prompt), [], n_new
        for s in range(n_new):
            lg = orc.forward(cfg, sd, seq)[-1]
            lg[2] = float("-inf")  # min_new_tokens bans EOS
            top = lg.topk(2).values
            if float(top[0] - top[1]) < 1e-3 * float(lg[torch.isfinite(lg)].std()):
                sure = min(sure, s)
            out.append(int(lg.argmax()))
            seq.append(out[-1])
        return out, sure

    n_new = 7
    p1 = [_tokens(40, 9, V), _tokens(41, 23, V)]
    p2 = [_tokens(42, 5, V)]
    got = {0: [], 1: [], 2: []}
    with torch.inference_mode():
        b1, errs = model.batch_type.from_pb(batch_of(0, p1, n_new, 0), tok, model.dtype, model.device, None, None, True)
        assert not errs
        for t in model.generate_token(b1, first=True)[0]:
            got[t.request_id].append(t.token_id)
        for _ in range(2):
            for t in model.generate_token(b1)[0]:
                got[t.request_id].append(t.token_id)
        b2, errs = model.batch_type.from_pb(batch_of(1, p2, n_new, 2), tok, model.dtype, model.device, None, None, True)
        for t in model.generate_token(b2, first=True, for_concat=True)[0]:
            got[t.request_id].append(t.token_id)
        both = model.batch_type.concatenate([b1, b2])
        for _ in range(n_new - 3):
            for t in model.generate_token(both)[0]:
                got[t.request_id].append(t.token_id)
        assert len(got[0]) == n_new and len(got[1]) == n_new
        rest = model.batch_type.prune(both, [0, 1])
        assert len(rest) == 1
        while len(got[2]) < n_new:
            for t in model.generate_token(rest)[0]:
                got[t.request_id].append(t.token_id)
        model.kv_cache_manager.free_sequences(rest.sequence_ids)
    sure_total = 0
    for rid, prompt in enumerate(p1 + p2):
        ref, sure = oracle_greedy(prompt, n_new)
        assert got[rid][:sure] == ref[:sure], (rid, got[rid], ref)
        sure_total += sure
    assert sure_total >= 12
    mgr = model.kv_cache_manager
    assert mgr.free_blocks == mgr.total_num_gpu_blocks and mgr.free_state_slots == 6
