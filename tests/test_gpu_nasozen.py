"""Nasozen on the GPU against the slow CPU reference (oracle/nasozen.py, float64): each mechanism alone, then the model through
the engine's step function and cache manager - whole prompts, token-by-token decoding, portions down to two tokens, ragged
batches, pages and state slots that are freed and used again - and greedy generation through FlashCausalLM.generate_token.

The configurations are small and uneven (key size != value size, several key heads and one, two to five residual streams and
none, loops of one and three passes and none, one to four convolution taps and none, partial and full rotation and none).  Where
random weights would hide a fault the test makes it show: a key that must win the soft-max from the window's far edge, from
just outside it, at a page border or at the first positions; a sink that swallows the soft-max; a recurrent state filled with
garbage before its slot is used again."""
import copy
import json
import math
import os

import pytest
import torch

from oracle import nasozen as orc

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
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in sd.items()}, path)
    weights = Weights([path], device=DEV, dtype=dtype, process_group=FakeGroup(0, 1))
    engine = InferenceEngine(d, None, dtype, None, None, None, weights=weights, tokenizer=make_tokenizer(config["vocab"]))
    return FlashCausalLM(d, None, "tgis_native", dtype, None, None, engine=engine, num_kv_blocks=blocks, num_state_slots=slots)


def _tokens(seed, n, vocab):
    return torch.randint(4, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _rel(got, ref):
    """largest row error relative to the spread of the reference logits"""
    got, ref = got.double().cpu(), ref.double()
    return float(((got - ref).pow(2).mean(-1).sqrt() / ref.std()).max())


def _decided(config, sd, tokens, least=0.15):
    """positions whose routing is no close call in any layer run: where bfloat16 must pick the reference's experts"""
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


def _step(starts_and_counts, tables, slots=None):
    """RaggedStep for sequences (start, count) whose pages are given by `tables` (one list of block ids per sequence)"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq
    pos, seq, rows, cu = [], [], [], [0]
    for b, (start, n) in enumerate(starts_and_counts):
        for p in range(start, start + n):
            pos.append(p)
            seq.append(b)
            rows.append(tables[b][p // 16] * 16 + p % 16)
        cu.append(cu[-1] + n)
    width = max(len(t) for t in tables)
    bt = torch.zeros(len(tables), width, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t)
    slots = list(range(len(tables))) if slots is None else slots
    return ops_seq.RaggedStep(T=len(pos), B=len(tables), position_ids=torch.tensor(pos, dtype=torch.int64, device=DEV),
                              cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV), seq_of_token=torch.tensor(seq, dtype=torch.int32, device=DEV),
                              slot_mapping=torch.tensor(rows, dtype=torch.int64, device=DEV), block_table=bt.to(DEV),
                              state_slots=torch.tensor(slots, dtype=torch.int32, device=DEV))


def _feed(mixer, spec, h, cuts, dtype, blocks=40):
    """one sequence through a mixer alone in portions of the given sizes, over NaN-filled pages (out of order) and state -> [L, W]"""
    L = h.shape[0]
    pages = torch.full((blocks, 16, spec.row_width), float("nan"), dtype=dtype, device=DEV) if spec.kind == "paged" else None
    state = {k: torch.full((3, *shape), float("nan"), dtype=torch.float32, device=DEV) for k, shape in (spec.state or {}).items()}
    table = [(7 * i + 3) % blocks for i in range((L + 15) // 16)]
    assert len(set(table)) == len(table)
    out, at = [], 0
    for n in list(cuts) + [1] * (L - sum(cuts)):
        st = _step([(at, n)], [table], slots=[2])
        out.append(mixer(h[at:at + n].to(dtype).to(DEV).contiguous(), st, pages, state, L + 1))
        at += n
    return torch.cat(out).double().cpu()


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("S", [1, 2, 3, 5])
def test_streams_step_write_and_read(S):
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    g = torch.Generator().manual_seed(S)
    T, W, eps = 6, 44, 1e-5
    X0, y, x0 = torch.randn(T, S, W, generator=g) * 2, torch.randn(T, W, generator=g), torch.randn(T, W, generator=g)
    mix, co, ci = torch.eye(S) + 0.3 * torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
    new = torch.einsum("su,tsw->tuw", mix.double(), X0.double()) + co.double()[None, :, None] * y.double()[:, None, :]
    for dtype in (torch.float32, torch.bfloat16):
        w = (1 + 0.3 * torch.randn(W, generator=g)).to(dtype)
        tol = 2e-5 if dtype == torch.float32 else 0.05
        # write and read in one launch
        X = X0.clone().to(DEV)
        h = ops.streams_step(X, y=y.to(DEV), mix=mix.to(DEV), out_coef=co.to(DEV), in_coef=ci.to(DEV), norm_w=w.to(DEV), eps=eps)
        assert float((X.cpu().double() - new).abs().max()) < 2e-5
        ref_h = orc.unit_rms(torch.einsum("s,tsw->tw", ci.double(), new), eps) * w.double()
        assert h.dtype == dtype and float((h.cpu().double() - ref_h).abs().max()) < tol
        # the same as two launches
        X = X0.clone().to(DEV)
        assert ops.streams_step(X, y=y.to(DEV), mix=mix.to(DEV), out_coef=co.to(DEV)) is None
        assert float((X.cpu().double() - new).abs().max()) < 2e-5
        h2 = ops.streams_step(X, in_coef=ci.to(DEV), norm_w=w.to(DEV), eps=eps)
        assert torch.equal(h2, h) and float((X.cpu().double() - new).abs().max()) < 2e-5   # a read leaves the streams alone
        # every stream starts as the given row (what X held before is never read)
        X = torch.full((T, S, W), float("nan"), device=DEV)
        h = ops.streams_step(X, init=x0.to(DEV), in_coef=ci.to(DEV), norm_w=w.to(DEV), eps=eps)
        assert torch.equal(X.cpu(), x0[:, None, :].expand(T, S, W))
        ref_h = orc.unit_rms(x0.double() * ci.double().sum(), eps) * w.double()
        assert float((h.cpu().double() - ref_h).abs().max()) < tol
    # the plain sum without a norm
    X = X0.clone().to(DEV)
    u = ops.streams_step(X, in_coef=torch.ones(S, device=DEV), out_dtype=torch.float32)
    assert float((u.cpu().double() - X0.double().sum(1)).abs().max()) < 1e-5


def test_activation_and_head_epilogue_kernels():
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    from tgis_b200.utils.mixers import ScaledRotaryTables
    g = torch.Generator().manual_seed(1)
    T = 9
    wide = torch.randn(T, 50, generator=g) * 2
    for act, fn in ((ops.ACT_SILU, orc.silu), (ops.ACT_GELU_TANH, orc.gelu_tanh), (ops.ACT_TANH, torch.tanh)):
        ref = fn(wide[:, 7:30].double())
        assert float((ops.ff_act(wide.to(DEV)[:, 7:30], act).cpu().double() - ref).abs().max()) < 1e-5          # a column slice
        assert float((ops.ff_act(wide.to(DEV)[:, 7:30], act, out_dtype=torch.bfloat16).cpu().double() - ref).abs().max()) < 0.05
        b16 = wide.to(torch.bfloat16)
        assert float((ops.ff_act(b16.to(DEV), act).cpu().double() - fn(b16.double())).abs().max()) < 0.05
    H, dv, base = 3, 10, 50.0
    a, gate = torch.randn(T, H, dv, generator=g), torch.randn(T, H + 4, generator=g)
    pos = torch.tensor([0, 1, 2, 3, 40, 41, 7, 300, 5])
    st = _step([(0, 4), (40, 2), (7, 1), (300, 1), (5, 1)], [list(range(20))] * 5)
    for rot, pairs in ((10, "halves"), (6, "halves"), (10, "interleaved"), (4, "interleaved"), (0, "halves")):
        tab = ScaledRotaryTables(rot, base) if rot else None
        cos, sin = tab.tables(301, DEV) if rot else (None, None)
        turn = orc.turn_halves if pairs == "halves" else orc.turn_neighbours
        ref = (turn(a.double(), pos, rot, base, sign=-1.0) if rot else a.double()) * torch.sigmoid(gate[:, 2:2 + H].double())[:, :, None] * 0.7
        buf = torch.zeros(T, H * dv + 5, device=DEV)
        ops.heads_turn_gate(a.to(DEV), gate.to(DEV)[:, 2:2 + H], cos, sin, rot, pairs == "interleaved", st, torch.float32, out=buf[:, 5:], out_scale=0.7)
        assert float((buf[:, 5:].cpu().double() - ref.reshape(T, H * dv)).abs().max()) < 1e-5, (rot, pairs)
        assert float(buf[:, :5].abs().max()) == 0.0
    plain = ops.heads_turn_gate(a.to(DEV), None, None, None, 0, False, st, torch.bfloat16)
    assert plain.dtype == torch.bfloat16 and float((plain.float().cpu() - a.reshape(T, H * dv)).abs().max()) < 0.02


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C", [5, 130, 300])
def test_min_gru_any_cut_and_reused_slot(C, dtype):
    import tgis_b200  # noqa: F401
    from tgis_b200.utils.mixers import MinGRUMixer
    g = torch.Generator().manual_seed(C)
    W, L = 24, 45
    sd = {"m.z": torch.randn(C, W, generator=g) * 0.4, "m.x": torch.randn(C, W, generator=g) * 0.5, "m.g": torch.randn(C, W, generator=g) * 0.4,
          "m.z.b": torch.randn(C, generator=g), "m.x.b": torch.randn(C, generator=g), "m.o": torch.randn(W, C, generator=g) / math.sqrt(C)}
    sd = {k: v.to(torch.bfloat16).float() for k, v in sd.items()}
    h = (torch.randn(L, W, generator=g)).to(torch.bfloat16).float()
    ref = orc.min_gru(h.double(), {k[2:]: v.double() for k, v in sd.items()})
    mixer = MinGRUMixer("m", _DictWeights(sd, dtype), width=C)
    tol = 1e-4 if dtype == torch.float32 else 0.06
    for cuts in ([L], [], [2, 2, 30, 3], [1, 43]):
        got = _feed(mixer, mixer.cache_spec(), h, cuts, dtype)
        assert float((got - ref).abs().max()) < tol * float(ref.abs().max()), cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,rank", [(3, 10, 4), (2, 72, 16), (1, 132, 3)])
def test_general_delta_any_cut(H, d, rank, dtype):
    import tgis_b200  # noqa: F401
    from tgis_b200.utils.mixers import GeneralDeltaMixer
    g = torch.Generator().manual_seed(H * d)
    W, L, eps = 32, 40, 1e-5
    cfg = {"width": W, "vocab": 8, "layers": [{"type": "general_delta", "mixer": {"heads": H, "dim": d}, "mlp": None}]}
    sd = {k[7:]: v for k, v in orc.random_state_dict(cfg, seed=H, decay_rank=rank).items() if k.startswith("l0.mix.")}
    h = torch.randn(L, W, generator=g).to(torch.bfloat16).float()
    ref = orc.general_delta(h.double(), {k: v.double() for k, v in sd.items()}, cfg["layers"][0]["mixer"], eps)
    mixer = GeneralDeltaMixer("m", _DictWeights({"m." + k: v for k, v in sd.items()}, dtype), heads=H, dim=d, eps=eps)
    tol = 2e-4 if dtype == torch.float32 else 0.08
    for cuts in ([L], [], [2, 17, 2, 16], [1, 38]):
        got = _feed(mixer, mixer.cache_spec(), h, cuts, dtype)
        assert float((got - ref).abs().max()) < tol * float(ref.abs().max()), cuts


def test_recurrent_states_long_run():
    """300 single steps of the delta memory and the gated unit: the state neither drifts from the reference nor depends on the cut"""
    import tgis_b200  # noqa: F401
    from tgis_b200.utils.mixers import GeneralDeltaMixer, MinGRUMixer
    g = torch.Generator().manual_seed(77)
    W, L, H, d, C, eps = 20, 300, 2, 12, 30, 1e-5
    cfg = {"width": W, "vocab": 8, "layers": [{"type": "general_delta", "mixer": {"heads": H, "dim": d}, "mlp": None}]}
    sd = {k[7:]: v for k, v in orc.random_state_dict(cfg, seed=5).items() if k.startswith("l0.mix.")}
    h = torch.randn(L, W, generator=g).to(torch.bfloat16).float()
    ref = orc.general_delta(h.double(), {k: v.double() for k, v in sd.items()}, cfg["layers"][0]["mixer"], eps)
    mixer = GeneralDeltaMixer("m", _DictWeights({"m." + k: v for k, v in sd.items()}, torch.float32), heads=H, dim=d, eps=eps)
    for cuts in ([], [150, 150]):
        assert float((_feed(mixer, mixer.cache_spec(), h, cuts, torch.float32) - ref).abs().max()) < 3e-4 * float(ref.abs().max())
    gs = {"m.z": torch.randn(C, W, generator=g) * 0.4, "m.x": torch.randn(C, W, generator=g) * 0.5, "m.g": torch.randn(C, W, generator=g) * 0.4,
          "m.z.b": torch.randn(C, generator=g) - 2.0, "m.x.b": torch.randn(C, generator=g), "m.o": torch.randn(W, C, generator=g) / math.sqrt(C)}
    ref = orc.min_gru(h.double(), {k[2:]: v.double() for k, v in gs.items()})
    gru = MinGRUMixer("m", _DictWeights(gs, torch.float32), width=C)
    assert float((_feed(gru, gru.cache_spec(), h, [], torch.float32) - ref).abs().max()) < 1e-4 * float(ref.abs().max())


def _attention_case(H, G, d, dv, rot, window, conv, sharp, seed, W=32):
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": d ** -0.5 * sharp}
    if rot:
        m["rot"] = {"base": 100.0, "dims": rot}
    if window:
        m["mask"] = {"size": window}
    if conv:
        m["conv"] = conv
    cfg = {"width": W, "vocab": 8, "layers": [{"type": "parallel", "mlp": None,
                                                "mixer": {"left": m, "right": {"width": 4}, "left_scale": 1.0, "right_scale": 1.0}}]}
    sd = {k[12:]: v for k, v in orc.random_state_dict(cfg, seed=seed).items() if k.startswith("l0.mix.left.")}
    return m, sd


def _attention(m, sd, dtype, eps=1e-5):
    from tgis_b200.utils.mixers import ScaledRotaryTables, SinkRotaryAttention
    rot = m.get("rot")
    return SinkRotaryAttention("a", _DictWeights({"a." + k: v for k, v in sd.items()}, dtype), heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"],
                               vdim=m["vdim"], scale=m["scale"], rotary=ScaledRotaryTables(rot["dims"], rot["base"]) if rot else None,
                               value_rotary=ScaledRotaryTables(m["vdim"], rot["base"]) if rot else None, conv=m.get("conv", 0),
                               window=m["mask"]["size"] if m.get("mask") else None, eps=eps)


ATTENTION_CASES = [  # heads, kv heads, dim, vdim, rotated columns, window, taps
    (6, 2, 10, 12, 6, 20, 3),      # the plain kernel: sizes that are no multiples of 16
    (4, 4, 16, 32, 16, 37, 4),     # as many key heads as heads, full rotation
    (8, 1, 32, 16, 8, 16, 2),      # one key head, a window of exactly one page
    (16, 4, 16, 64, 0, 50, 0),     # no rotation (the values stay as projected), no convolution
    (3, 1, 8, 8, 4, 0, 1),         # no window at all, a single tap
    (8, 2, 64, 128, 32, 5, 4),     # a window shorter than a page
    (16, 16, 64, 256, 32, 50, 2),  # many key heads of wide values: more than one block's shared memory if all groups were staged
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ATTENTION_CASES)
def test_attention_alone_any_cut(case, dtype):
    import tgis_b200  # noqa: F401
    m, sd = _attention_case(*case, sharp=1.5, seed=sum(case))
    g = torch.Generator().manual_seed(3)
    L, eps = 70, 1e-5
    h = torch.randn(L, 32, generator=g).to(torch.bfloat16).float()
    ref = orc.sink_window_attention(h.double(), {k: v.double() for k, v in sd.items()}, m, eps)
    mixer = _attention(m, sd, dtype)
    tol = 1e-4 if dtype == torch.float32 else 0.08
    for cuts in ([L], [], [2, 33, 2, 31], [16, 16, 16, 16], [1, 20, 47]):
        got = _feed(mixer, mixer.cache_spec(), h, cuts, dtype)
        assert float((got - ref).abs().max()) < tol * float(ref.abs().max()), cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,window", [(6, 3, 10, 14, 100), (4, 1, 16, 32, 64), (8, 2, 32, 16, 33), (16, 4, 16, 64, 150), (2, 2, 64, 128, 17)])
def test_attention_loud_keys_at_window_edges_and_sinks(dtype, H, G, d, dv, window):
    """One key is made to win the soft-max of every head (a query and a key scaled along the same direction): the output must be
    that key's value when the key is the window's oldest, at a page border, at position 0 or the query itself, and must not move
    at all when the key is one step outside the window - for a decoded token and for a row inside a portion.  Then the sinks:
    a huge sink swallows every head's weight, a very negative one leaves the plain soft-max."""
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    g = torch.Generator().manual_seed(window)
    L, scale = 420, 1.0
    cases = [(L - 1, L - window, True), (L - 1, L - window - 1, False), (L - 1, L - 1, True), (window - 1, 0, True), (window, 0, False),
             (200, 192, True), (207, 191, True), (L - 1, 2, False), (16 + window - 1, 16, True), (16 + window, 16, False), (15 + window, 15, False)]
    cases = [c for c in cases if 0 <= c[1] <= c[0] < L]
    blocks = (L + 15) // 16
    table = [(7 * i + 1) % (blocks + 3) for i in range(blocks)]
    assert len(set(table)) == blocks
    RW = G * d + G * dv
    for qpos, kpos, inside in cases:
        q = torch.randn(L, H, d, generator=g) * 0.3
        k = torch.randn(L, G, d, generator=g) * 0.3
        v = torch.randn(L, G, dv, generator=g)
        direction = torch.nn.functional.normalize(torch.randn(d, generator=g), dim=0)
        q[qpos] = direction * 9.0
        k[kpos] = direction * 9.0                      # every head's score against kpos: 81, against the rest: small
        pool = torch.full((blocks + 3, 16, RW), float("nan"), dtype=dtype, device=DEV)
        rows = torch.tensor([table[p // 16] * 16 + p % 16 for p in range(L)], device=DEV)
        pool.view(-1, RW)[rows] = torch.cat([k.reshape(L, -1), v.reshape(L, -1)], 1).to(dtype).to(DEV)
        sink = torch.randn(H, generator=g)
        for start, n in ((qpos, 1), (max(qpos - 40, 0), min(41, qpos + 1) + (3 if qpos + 3 < L else 0))):   # decoded alone / inside a portion
            st = _step([(start, n)], [table])
            row = qpos - start

            def run(qq, sk=sink):
                return ops.talk_attn(qq[start:start + n].contiguous().to(DEV), pool, st, kv_heads=G, vdim=dv, k_off=0, v_off=G * d, scale=scale,
                                     window=window, sink=None if sk is None else sk.to(DEV))[row].cpu()
            got = run(q)
            vv = v.to(dtype).float()
            if inside:
                want = vv[kpos].repeat_interleave(H // G, dim=0)
                assert float((got - want).abs().max()) < 1e-3, (qpos, kpos, n)
            else:
                lo = max(qpos - window + 1, 0)
                s = torch.einsum("hd,jhd->hj", q[qpos].double(), k[lo:qpos + 1].to(dtype).double().repeat_interleave(H // G, dim=1))
                w = torch.softmax(torch.cat([s, sink.double()[:, None]], 1), 1)[:, :-1]
                want = torch.einsum("hj,jhv->hv", w, vv[lo:qpos + 1].double().repeat_interleave(H // G, dim=1))
                tol = 1e-4 if dtype == torch.float32 else 0.03
                assert float((got.double() - want).abs().max()) < tol, (qpos, kpos, n)     # the loud key outside adds nothing
                assert float((got - vv[kpos].repeat_interleave(H // G, dim=0)).abs().max()) > 0.3
            if n == 1 and inside:
                assert float(run(q, torch.full((H,), 200.0)).abs().max()) < 1e-6          # the sink takes everything
                assert float((run(q, torch.full((H,), -200.0)) - run(q, None)).abs().max()) < 1e-6


@pytest.mark.parametrize("pairs", ["halves", "interleaved"])
def test_values_turn_with_their_position(pairs):
    """the value columns of the cache row are the projected values turned by the token's position, in both pair layouts"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    from tgis_b200.utils.mixers import ScaledRotaryTables
    g = torch.Generator().manual_seed(9)
    H, G, d, dv, base, T = 4, 2, 8, 12, 30.0, 6
    u = torch.randn(T, H * d + G * d + G * dv + 3, generator=g)
    st = _step([(37, T)], [[4, 2, 0]])
    pool = torch.zeros(5, 16, G * d + G * dv, device=DEV)
    for v_rot in (12, 8):
        tab = ScaledRotaryTables(v_rot, base)
        cos, sin = tab.tables(64, DEV)
        ops.qk_rot_prepare(u.to(DEV), col_q=0, col_k=H * d, col_v=H * d + G * d, heads=H, kv_heads=G, dim=d, vdim=dv, q_norm_w=None, k_norm_w=None,
                           whole_norm=False, eps=1e-5, cos=None, sin=None, rot=0, step=st, cache=pool, k_off=0, v_off=G * d, v_cos=cos, v_sin=sin,
                           v_rot=v_rot, v_interleaved=pairs == "interleaved")
        vals = u[:, H * d + G * d:H * d + G * d + G * dv].double().view(T, G, dv)
        turn = orc.turn_halves if pairs == "halves" else orc.turn_neighbours
        want = turn(vals, torch.arange(37, 37 + T), v_rot, base)
        rows = st.slot_mapping
        got = pool.view(-1, G * d + G * dv)[rows][:, G * d:].cpu().double().view(T, G, dv)
        assert float((got - want).abs().max()) < 1e-5
        keys = pool.view(-1, G * d + G * dv)[rows][:, :G * d].cpu()
        assert float((keys - u[:, H * d:H * d + G * d]).abs().max()) < 1e-6


@pytest.mark.parametrize("E,top", [(5, 2), (3, 3), (7, 1), (24, 6)])
def test_softmax_routing_weights_are_scores_over_their_sum(E, top):
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    g = torch.Generator().manual_seed(E)
    z = torch.randn(50, E, generator=g) * 2
    s = torch.softmax(z.double(), -1)
    val, idx = torch.topk(s, top, dim=-1)
    want = val / (val.sum(-1, keepdim=True) + 1e-20)
    r = ops.moe_route(z.to(DEV), top)
    order = r.ids.cpu().long().argsort(1)
    assert torch.equal(r.ids.cpu().long().gather(1, order), idx.sort(1).values)
    got = r.weights.cpu().double().gather(1, order)
    assert float((got - want.gather(1, idx.argsort(1))).abs().max()) < 1e-6


# ------------------------------------------------------------------------------------------------ the model
def _vary(cfg, sd, fn):
    c2, s2 = copy.deepcopy(cfg), {k: v.clone() for k, v in sd.items()}
    fn(c2, s2)
    return c2, s2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompt_portions_and_decoding_agree_with_reference(tmp_path, dtype):
    cfg = orc.random_config(sharp=3.0, window=24)
    sd = orc.random_state_dict(cfg, seed=2)
    for k in sd:
        if k.endswith(".router"):   # decisive routers: fewer close calls for the bfloat16 run to flip
            sd[k] = (sd[k] * 4.0).to(torch.bfloat16).float()
    model = _model(tmp_path, cfg, sd, dtype)
    toks = _tokens(1, 90, cfg["vocab"])
    ref = orc.forward(cfg, sd, toks)
    sure = _decided(cfg, sd, toks) if dtype == torch.bfloat16 else torch.ones(len(toks), dtype=torch.bool)
    assert int(sure.sum()) > 40
    tol = TOL32 if dtype == torch.float32 else TOL16
    whole = _run_cut(model, toks, [len(toks)])
    assert _rel(whole[sure], ref[sure]) < tol
    if dtype == torch.float32:
        # what the configuration and the tensors say is live in this test: each of these, when wrong, is far outside the tolerance
        def changed(fn):
            c2, s2 = _vary(cfg, sd, fn)
            return _rel(orc.forward(c2, s2, toks), ref)
        left = lambda c, i=0: c["layers"][i]["mixer"]["left"]  # noqa: E731
        assert changed(lambda c, s: left(c)["mask"].update(size=25)) > 20 * TOL32
        assert changed(lambda c, s: left(c)["mask"].update(size=23)) > 20 * TOL32
        assert changed(lambda c, s: left(c)["rot"].update(dims=4)) > 20 * TOL32
        assert changed(lambda c, s: left(c)["rot"].update(base=90.0)) > 20 * TOL32
        assert changed(lambda c, s: left(c).update(scale=left(c)["scale"] * 1.05)) > 20 * TOL32
        assert changed(lambda c, s: s.update({"l0.mix.left.sink": s["l0.mix.left.sink"] - 1.0})) > 20 * TOL32
        assert changed(lambda c, s: s.update({"l0.mix.left.g": s["l0.mix.left.g"] * 0.5})) > 20 * TOL32
        assert changed(lambda c, s: c["layers"][0]["mixer"].update(left_scale=0.7)) > 20 * TOL32
        assert changed(lambda c, s: c["layers"][3]["mixer"].update(right_scale=0.7)) > 20 * TOL32
        assert changed(lambda c, s: c.update(residual_mult=0.75)) > 20 * TOL32
        assert changed(lambda c, s: c["loop"].update(times=3)) > 20 * TOL32
        assert changed(lambda c, s: c["loop"].update(stop=2)) > 20 * TOL32
        assert changed(lambda c, s: s.update({"l1.hc2.mix": s["l1.hc2.mix"].T.contiguous()})) > 20 * TOL32
        assert changed(lambda c, s: s.update({"l2.hc1.in": s["l2.hc1.in"].flip(0)})) > 20 * TOL32
        assert changed(lambda c, s: c["layers"][1]["mixer"].update(gate_cap=4.0)) > 20 * TOL32
        assert changed(lambda c, s: s.update({"l2.mix.w0": s["l2.mix.w0"] + 1.0})) > 20 * TOL32
        assert changed(lambda c, s: s.update({"l2.mix.a.b": s["l2.mix.a.b"] + 1.0})) > 20 * TOL32
        assert changed(lambda c, s: c["layers"][1]["mlp"]["router"].update(top=3)) > 20 * TOL32
    for cuts in ([], [40], [2, 2, 2, 19, 3, 16, 17, 2], [16, 16, 16, 16], [24, 24, 24], [23, 2, 23, 2], [1, 25, 22, 31]):
        got = _run_cut(model, toks, cuts)
        assert _rel(got[sure], ref[sure]) < tol, cuts
        if dtype == torch.float32:
            assert _rel(got, whole.cpu()) < 1e-5, cuts  # the cut itself changes nothing beyond rounding
    assert model.kv_cache_manager.free_blocks == model.kv_cache_manager.total_num_gpu_blocks
    assert model.kv_cache_manager.free_state_slots == 4


def test_tensor_core_shapes_through_the_engine(tmp_path):
    """bfloat16 with head sizes in 16s: prompts, portions and decoded tokens take the tensor-core attention kernel and the
    tensor-core products; a step mixes a long portion (several query tiles) with single tokens"""
    cfg = orc.random_config(width=64, order=("parallel", "general_delta", "parallel", "mlstm"), loop=(0, 2, 2), streams=2, heads=8, kv_heads=2, dim=32,
                            vdim=16, rot_dims=16, window=60, sharp=2.0, gru_width=64, d_heads=2, d_dim=16, m_heads=2, m_dim=16, m_vdim=32,
                            mlp=("moe", "dense", None, "moe"), experts=4, top=4)
    sd = orc.random_state_dict(cfg, seed=12, decay_rank=8)
    model = _model(tmp_path, cfg, sd, torch.bfloat16)
    toks = _tokens(3, 150, cfg["vocab"])
    ref = orc.forward(cfg, sd, toks)
    for cuts in ([150], [100, 2, 40], [1, 70, 33], [5]):
        assert _rel(_run_cut(model, toks, cuts), ref) < TOL16, cuts
    other = _tokens(4, 90, cfg["vocab"])
    ref_o = orc.forward(cfg, sd, other)
    (a,), la = model.step_ragged([None], [toks[:20]])
    (a, b), l2 = model.step_ragged([a, None], [toks[20:21], other[:80]])
    (b, a), l3 = model.step_ragged([b, a], [other[80:], toks[21:150]])
    model.kv_cache_manager.free_sequences([a, b])
    assert _rel(torch.cat([la, l2[:1], l3[10:]]), ref) < TOL16
    assert _rel(torch.cat([l2[1:], l3[:10]]), ref_o) < TOL16


def test_residual_stream_after_every_layer_run(tmp_path):
    cfg = orc.random_config(loop=(1, 3, 3))
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
    assert len(probe) == len(want) == 8
    for i, (a, b) in enumerate(zip(probe, want)):
        assert float((a.cpu().double() - b).abs().max()) < 1e-4 * float(b.abs().max()), i


OTHER_SIZES = {
    "plain_stream_no_loop": dict(streams=None, loop=None, residual_mult=1.0, kv_heads=1, heads=5, conv=None, top=1, experts=6),
    "one_stream_one_pass": dict(streams=1, loop=(0, 4, 1), kv_heads=6, heads=6, dim=14, vdim=8, rot_dims=14, conv=2, top=3, experts=3, window=2),
    "five_streams_whole_loop": dict(streams=5, loop=(0, 3, 2), order=("general_delta", "parallel", "mlstm"), mlp=("moe", None, "dense"), width=56,
                                    heads=8, kv_heads=4, dim=8, vdim=10, rot_dims=2, conv=4, window=31, d_heads=1, d_dim=70, m_heads=1, m_dim=20,
                                    m_vdim=36, left_scale=1.0, right_scale=1.0),
    "no_rotation_no_window": dict(rot_dims=None, window=None, order=("parallel", "parallel"), loop=(1, 2, 3), mlp=(None, "dense"), streams=2,
                                  gru_width=70, conv=1),
    "recurrent_only": dict(order=("mlstm", "general_delta", "mlstm"), loop=(2, 3, 2), mlp=("dense", "dense", "moe"), streams=4, gate_cap=3.0),
}


@pytest.mark.parametrize("variant", sorted(OTHER_SIZES))
def test_other_sizes(tmp_path, variant):
    """sizes that a usual configuration makes equal or 1, and entries it may leave out: no `streams` and no `loop` at all, one
    stream, a loop of one pass, a loop over every layer, one key head and as many key heads as heads, one expert per token and
    every expert per token, a window of two tokens and none, full rotation and none (then the values do not turn either), one to
    four taps and none, layers without a feed-forward, attention-free stacks"""
    cfg = orc.random_config(sharp=3.0, **OTHER_SIZES[variant])
    sd = orc.random_state_dict(cfg, seed=31, decay_rank=7)
    model = _model(tmp_path, cfg, sd, torch.float32)
    toks = _tokens(6, 60, cfg["vocab"])
    ref = orc.forward(cfg, sd, toks)
    for cuts in ([60], [3, 30, 2], [17]):
        assert _rel(_run_cut(model, toks, cuts), ref) < TOL32, (variant, cuts)


def test_ragged_batches_reused_pages_and_slots(tmp_path):
    """four requests of unequal length run as mixed steps (portions beside decoded tokens, requests joining and leaving) in a pool
    that is too small for all of them at once and is filled with garbage first: every request equals its run alone"""
    cfg = orc.random_config(sharp=3.0)
    sd = orc.random_state_dict(cfg, seed=21)
    model = _model(tmp_path, cfg, sd, torch.float32, blocks=12, slots=2)
    mgr = model.kv_cache_manager
    assert len(mgr.pages) == 6   # one store per layer run
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
    """three prompt tokens, then 197 single steps: the window (40) passes over decoded tokens only; the first tokens have fewer
    inputs than taps"""
    cfg = orc.random_config(sharp=3.0, window=40, conv=4)
    sd = orc.random_state_dict(cfg, seed=8)
    model = _model(tmp_path, cfg, sd, torch.float32)
    toks = _tokens(9, 200, cfg["vocab"])
    ref = orc.forward(cfg, sd, toks)
    c2, _ = _vary(cfg, sd, lambda c, s: [layer["mixer"]["left"]["mask"].update(size=41) for layer in c["layers"] if layer["type"] == "parallel"])
    assert _rel(orc.forward(c2, sd, toks)[45:], ref[45:]) > 20 * TOL32   # the window's edge is live
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


def test_sampling_and_logprobs_through_generate_token(tmp_path):
    """requests that sample (temperature, top-k, a seed) and ask for log-probabilities take the chooser chain on the fp32 logits:
    the same seed draws the same tokens, ids stay inside the top-k set of the reference's logits, log-probabilities are finite"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import pb
    cfg = orc.random_config(order=("parallel", "general_delta"), loop=(1, 2, 2), mlp=("dense", None), streams=2, window=10)
    sd = orc.random_state_dict(cfg, seed=17)
    model = _model(tmp_path, cfg, sd, torch.float32, blocks=32, slots=4)
    tok, V = model.tokenizer, cfg["vocab"]
    prompt = _tokens(50, 11, V)
    text = " ".join(f"<tok{i}>" for i in prompt)
    n_new, top_k = 5, 4

    def run(batch_id):
        reqs = [pb.Request(id=i, inputs=text, input_length=len(prompt), truncate=False, max_output_length=n_new,
                           parameters=pb.NextTokenChooserParameters(temperature=0.9, top_k=top_k, top_p=1.0, seed=1234, min_new_tokens=n_new),
                           details=pb.RequestedDetails(logprobs=True)) for i in range(2)]
        out = [[], []]
        with torch.inference_mode():
            batch, errs = model.batch_type.from_pb(pb.Batch(id=batch_id, requests=reqs), tok, model.dtype, model.device, None, None, True)
            assert not errs
            infos = model.generate_token(batch, first=True)[0]
            for _ in range(n_new):
                for t in infos:
                    out[t.request_id].append((t.token_id, t.logprob))
                if len(out[0]) == n_new:
                    break
                infos = model.generate_token(batch)[0]
            model.kv_cache_manager.free_sequences(batch.sequence_ids)
        return out

    first, again = run(0), run(1)
    assert [t for t, _ in first[0]] == [t for t, _ in again[0]] and [t for t, _ in first[1]] == [t for t, _ in again[1]]
    assert [t for t, _ in first[0]] == [t for t, _ in first[1]]  # two requests with the same seed and prompt in one batch
    seq = list(prompt)
    for t, lp in first[0]:
        ref = orc.forward(cfg, sd, seq)[-1]
        ref[2] = float("-inf")
        assert t in ref.topk(top_k + 1).indices.tolist()
        assert lp is not None and lp <= 0.0 and lp > -30.0
        seq.append(t)
    mgr = model.kv_cache_manager
    assert mgr.free_blocks == mgr.total_num_gpu_blocks and mgr.free_state_slots == 4
