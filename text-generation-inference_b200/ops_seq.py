"""Tensor-level wrappers over libb200_seq.so: the kernels of the decoder families with an fp32 stream (latent attention over a paged latent
cache, differential and distance-biased attention over paged heads, head-mixed and sink attention over token-major rows, state-space,
matrix-memory, delta-rule and gated-unit mixers over fp32 state slots, routed feed-forward, the row kernels around one or several
residual streams).

Element type `dtype` is torch.bfloat16 or torch.float32 (weights, activations between projections, cache pages); statistics,
soft-max, recurrences, states and the residual stream are fp32 in both.  CUDA tensors only; there is no eager fallback.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

_DT = {torch.bfloat16: 0, torch.float32: 1}


def _dt(t) -> int:
    d = t if isinstance(t, torch.dtype) else t.dtype
    if d not in _DT:
        raise _lib.B200Error(f"element type {d}: the hybrid-family kernels take bfloat16 or float32")
    return _DT[d]


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _lib.B200Error("expected CUDA tensors (the B200 path has no CPU fallback)")


@dataclass
class RaggedStep:
    """Index tensors of one step over a ragged batch: sequence b brings the token rows cu_q[b] .. cu_q[b+1] at consecutive
    positions position_ids[row]; whether that is a prompt, a portion of one or one decoded token makes no difference."""
    T: int
    B: int
    position_ids: torch.Tensor   # [T] int64
    cu_q: torch.Tensor           # [B + 1] int32
    seq_of_token: torch.Tensor   # [T] int32
    slot_mapping: torch.Tensor   # [T] int64: cache row of each token (block * page + offset)
    block_table: torch.Tensor    # [B, max_blocks] int32
    state_slots: Optional[torch.Tensor]  # [B] int32


_TC_GEMM = os.getenv("B200_SEQ_TC_GEMM", "1") != "0"
_ATTN_SPLIT = os.getenv("B200_SEQ_ATTN_SPLIT", "1") != "0"
_gemm_ws = {}


def _gemm_workspace(device, N: int, K: int) -> torch.Tensor:
    """per-device split-K workspace of the tensor-core product (tile counters zeroed once; the kernel re-arms them)"""
    need = _lib.load_seq().b200_gemm_workspace_bytes_max(N, K)
    ws = _gemm_ws.get(device)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _gemm_ws[device] = ws
    return ws


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M, K] @ w [N, K]^T -> [M, N], fp32 accumulation.  bfloat16 operands go to the tcgen05 product (csrc/gemm_f16.cu,
    output bfloat16 or fp32) when they are dense and K is a multiple of 8 of at least 64; everything else - float32 operands
    (a true 32-bit product), row-strided slices, small or odd K - to the plain product with ascending-k accumulation."""
    _cuda(x, w, bias)
    assert x.dim() == 2 and w.dim() == 2 and x.stride(1) == 1 and w.stride(1) == 1 and x.shape[1] == w.shape[1]
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or x.dtype, device=x.device)
    assert out.stride(1) == 1
    if (_TC_GEMM and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
            and K % 8 == 0 and K >= 64 and x.is_contiguous() and w.is_contiguous() and out.is_contiguous()
            and (bias is None or bias.dtype == torch.bfloat16) and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and M > 0):
        ws = _gemm_workspace(x.device, N, K)
        _lib.check_seq(_lib.load_seq().b200_gemm_bf16(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), int(out.dtype == torch.float32), M, N, K,
                                                      _ptr(ws), _stream()), "gemm_bf16")
        return out
    _lib.check_seq(_lib.load_seq().b200_seq_linear(_ptr(x), _dt(x), x.stride(0), 0, _ptr(w), _dt(w), w.stride(0), 0, _ptr(bias), _ptr(out),
                                                   _dt(out), out.stride(0), 0, M, N, K, 1, _stream()), "seq_linear")
    return out


def linear_per_head(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """x [M, Z, K], w [Z, N, K], out [M, Z, N] (all may be slices with a wider last-but-one stride): out[:, z] = x[:, z] @ w[z]^T."""
    _cuda(x, w, out)
    M, Z, K = x.shape
    N = w.shape[1]
    assert w.shape == (Z, N, K) and out.shape == (M, Z, N) and x.stride(2) == 1 and w.stride(2) == 1 and out.stride(2) == 1
    _lib.check_seq(_lib.load_seq().b200_seq_linear(_ptr(x), _dt(x), x.stride(0), x.stride(1), _ptr(w), _dt(w), w.stride(1), w.stride(0), None,
                                                   _ptr(out), _dt(out), out.stride(0), out.stride(1), M, N, K, Z, _stream()), "seq_linear")
    return out


def embed_scale(table: torch.Tensor, ids: torch.Tensor, scale: float) -> torch.Tensor:
    """-> fp32 [T, W] = table[ids] * scale (the residual stream starts here)."""
    _cuda(table, ids)
    assert ids.dtype == torch.int64 and table.is_contiguous()
    out = torch.empty(ids.shape[0], table.shape[1], dtype=torch.float32, device=table.device)
    _lib.check_seq(_lib.load_seq().b200_seq_embed_scale(_ptr(table), _dt(table), _ptr(ids), float(scale), _ptr(out), ids.shape[0],
                                                        table.shape[1], table.shape[0], _stream()), "seq_embed_scale")
    return out


def layernorm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    """LayerNorm with weight and bias of a contiguous [T, W] tensor (fp32 stream or an activation); result has w's type."""
    _cuda(x, w, b)
    assert x.is_contiguous()
    out = torch.empty(x.shape, dtype=w.dtype, device=x.device)
    _lib.check_seq(_lib.load_seq().b200_seq_layernorm(_ptr(x), _dt(x), _ptr(w), _ptr(b), _dt(w), _ptr(out), None, x.shape[0], x.shape[1],
                                                      float(eps), _stream()), "seq_layernorm")
    return out


def layernorm_into_residual(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float, residual: torch.Tensor,
                            typed_copy: bool = False) -> Optional[torch.Tensor]:
    """residual (fp32, in place) += LayerNorm(x) * w + b.  typed_copy: also returns the updated residual in w's element type
    (the input of the next projection); for float32 that is the residual itself."""
    _cuda(x, w, b, residual)
    assert x.is_contiguous() and residual.is_contiguous() and residual.dtype == torch.float32 and x.shape == residual.shape
    copy = torch.empty(x.shape, dtype=w.dtype, device=x.device) if typed_copy and w.dtype != torch.float32 else None
    _lib.check_seq(_lib.load_seq().b200_seq_layernorm(_ptr(x), _dt(x), _ptr(w), _ptr(b), _dt(w), _ptr(copy), _ptr(residual), x.shape[0],
                                                      x.shape[1], float(eps), _stream()), "seq_layernorm")
    return (copy if copy is not None else residual) if typed_copy else None


GATE_NONE, GATE_SILU_BEFORE, GATE_SIGMOID_AFTER, GATE_SILU_AFTER = 0, 1, 2, 3


def group_rmsnorm_gate(x: torch.Tensor, weight: Optional[torch.Tensor], groups: int, eps: float, out_dtype: torch.dtype,
                       gate: Optional[torch.Tensor] = None, gate_kind: int = GATE_NONE) -> torch.Tensor:
    """x, gate: fp32 [T, C] column slices.  Per group of C / groups columns: v / sqrt(mean(v^2) + eps) * weight, with the gate
    multiplied in before the statistics (SiLU) or after the weight (sigmoid, or SiLU with GATE_SILU_AFTER).  groups == 0: no
    normalisation.  `weight` has one entry per column."""
    _cuda(x, weight, gate)
    assert x.dtype == torch.float32 and x.stride(1) == 1 and (gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1))
    T, C = x.shape
    n = C // groups if groups > 0 else C
    assert groups == 0 or n * groups == C
    out = torch.empty(T, C, dtype=out_dtype, device=x.device)
    w_dt = _dt(weight) if weight is not None else _dt(out_dtype)
    _lib.check_seq(_lib.load_seq().b200_seq_group_rmsnorm_gate(
        _ptr(x), x.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, gate_kind, _ptr(weight), w_dt, groups, n, float(eps),
        _ptr(out), _dt(out), out.stride(0), T, _stream()), "seq_group_rmsnorm_gate")
    return out


def ff_clamped_gate(gate_up: torch.Tensor, limit: float, alpha: float = 1.702) -> torch.Tensor:
    """[T, 2F] = [g | u] -> [T, F]: min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u, -limit, limit) + 1)."""
    _cuda(gate_up)
    assert gate_up.is_contiguous()
    T, F2 = gate_up.shape
    out = torch.empty(T, F2 // 2, dtype=gate_up.dtype, device=gate_up.device)
    _lib.check_seq(_lib.load_seq().b200_seq_ff_clamped_gate(_ptr(gate_up), _ptr(out), _dt(gate_up), T, F2 // 2, float(limit), float(alpha),
                                                            _stream()), "seq_ff_clamped_gate")
    return out


def token_side(residual: torch.Tensor, residual_typed: torch.Tensor, ids: torch.Tensor, table: torch.Tensor, col0: int, dim: int,
               w_gate: torch.Tensor, w_proj: torch.Tensor, norm_w: torch.Tensor, eps: float) -> None:
    """residual (fp32, in place) += unit_rms(w_proj (gelu_tanh(w_gate x) * table[id, col0:col0+dim])) * norm_w.  `residual_typed` is x
    in the projections' element type (layernorm_into_residual(..., typed_copy=True))."""
    _cuda(residual, residual_typed, ids, table, w_gate, w_proj, norm_w)
    assert residual.dtype == torch.float32 and residual.is_contiguous()
    T, W = residual.shape
    lib = _lib.load_seq()
    a = linear(residual_typed, w_gate, out_dtype=torch.float32)
    g = torch.empty(T, dim, dtype=table.dtype, device=table.device)
    _lib.check_seq(lib.b200_seq_side_gate(_ptr(a), _ptr(ids), _ptr(table), table.stride(0), col0, dim, table.shape[0], _ptr(g), _dt(table), T,
                                          _stream()), "seq_side_gate")
    y = linear(g, w_proj, out_dtype=torch.float32)
    _lib.check_seq(lib.b200_seq_rms_add(_ptr(y), _ptr(norm_w), _dt(norm_w), _ptr(residual), T, W, float(eps), _stream()), "seq_rms_add")


def latent_prepare(down: torch.Tensor, col_c: int, col_kr: int, q: torch.Tensor, q_head_stride: int, q_rot_off: int,
                   cnorm_w: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, step: RaggedStep, cache: torch.Tensor, q_abs: torch.Tensor,
                   H: int, R: int, r: int, rot_dims: int, eps: float) -> None:
    """Writes each token's cache row [unit_rms(latent) * w | rotated key part] and the rotated query parts q_abs[:, :, R:]."""
    _cuda(down, q, cache, q_abs)
    assert down.dtype == torch.float32 and q.dtype == torch.float32 and q_abs.dtype == torch.float32 and cos.dtype == torch.float32
    assert q_abs.is_contiguous() and cache.is_contiguous() and cos.is_contiguous() and sin.is_contiguous()
    _lib.check_seq(_lib.load_seq().b200_seq_latent_prepare(
        _ptr(down), down.stride(0), col_c, col_kr, _ptr(q), q.stride(0), q_head_stride, q_rot_off, _ptr(cnorm_w), _ptr(cos), _ptr(sin),
        _ptr(step.position_ids), _ptr(step.slot_mapping), _ptr(cache), _dt(cache), _ptr(q_abs), step.T, H, R, r, rot_dims, float(eps),
        _stream()), "seq_latent_prepare")


def latent_attn(q_abs: torch.Tensor, cache: torch.Tensor, step: RaggedStep, R: int, r: int, window: int, scale: float) -> torch.Tensor:
    """q_abs fp32 [T, H, R + r], cache [blocks, page, R + r] -> fp32 [T, H, R]: soft-max attention of every token over the cache
    rows of its own sequence at positions (p - window, p], in latent space."""
    _cuda(q_abs, cache)
    T, H, D = q_abs.shape
    assert D == R + r and cache.shape[-1] == D and q_abs.is_contiguous() and cache.is_contiguous()
    out = torch.empty(T, H, R, dtype=torch.float32, device=q_abs.device)
    lib = _lib.load_seq()
    need = ctypes.c_int64(0)
    nsplit = lib.b200_seq_latent_attn_splits(_dt(cache), T, H, R, r, ctypes.byref(need)) if _ATTN_SPLIT else 1
    partial = torch.empty(need.value, dtype=torch.float32, device=q_abs.device) if nsplit > 1 else None
    _lib.check_seq(lib.b200_seq_latent_attn(
        _ptr(q_abs), _ptr(cache), _dt(cache), _ptr(step.block_table), step.block_table.stride(0), _ptr(step.seq_of_token),
        _ptr(step.position_ids), _ptr(out), T, H, R, r, int(window), float(scale), cache.shape[1], _ptr(partial), nsplit, _stream()),
        "seq_latent_attn")
    return out


def causal_conv_silu(u: torch.Tensor, col0: int, channels: int, w: torch.Tensor, bias: torch.Tensor, conv_state: torch.Tensor,
                     step: RaggedStep) -> torch.Tensor:
    """SiLU(depth-wise causal convolution) of the columns [col0, col0 + channels) of u (fp32); conv_state [slots, taps - 1, channels]
    supplies the inputs before this step's first token and is advanced to the sequence's last taps - 1 inputs."""
    _cuda(u, w, bias, conv_state)
    assert u.dtype == torch.float32 and conv_state.dtype == torch.float32 and w.is_contiguous() and conv_state.is_contiguous()
    taps = w.shape[1]
    out = torch.empty(step.T, channels, dtype=torch.float32, device=u.device)
    _lib.check_seq(_lib.load_seq().b200_seq_causal_conv_silu(
        _ptr(u), u.stride(0), col0, channels, taps, _ptr(w), _ptr(bias), _dt(w), _ptr(conv_state), _ptr(step.state_slots),
        _ptr(step.seq_of_token), _ptr(step.cu_q), _ptr(step.position_ids), _ptr(out), step.T, step.B, _stream()), "seq_causal_conv_silu")
    return out


def ssm_scan(xbc: torch.Tensor, col_x: int, col_B: int, col_C: int, dt_raw: torch.Tensor, col_dt: int, dt_bias: torch.Tensor,
             A_log: torch.Tensor, D: torch.Tensor, state: torch.Tensor, step: RaggedStep, H: int, P: int, N: int, groups: int) -> torch.Tensor:
    """-> y fp32 [T, H * P]; state fp32 [slots, H, N, P] advanced in place."""
    _cuda(xbc, dt_raw, state)
    assert xbc.dtype == torch.float32 and dt_raw.dtype == torch.float32 and state.dtype == torch.float32 and state.is_contiguous()
    y = torch.empty(step.T, H * P, dtype=torch.float32, device=xbc.device)
    _lib.check_seq(_lib.load_seq().b200_seq_ssm_scan(
        _ptr(xbc), xbc.stride(0), col_x, col_B, col_C, _ptr(dt_raw), dt_raw.stride(0), col_dt, _ptr(dt_bias), _ptr(A_log), _ptr(D),
        _dt(dt_bias), _ptr(state), _ptr(step.state_slots), _ptr(step.cu_q), _ptr(step.position_ids), _ptr(y), y.stride(0), step.B, H, P, N,
        groups, _stream()), "seq_ssm_scan")
    return y


def mlstm_scan(proj: torch.Tensor, col_q: int, col_k: int, col_v: int, col_i: int, col_f: int, i_bias: torch.Tensor, f_bias: torch.Tensor,
               cap: float, q_scale: float, S: torch.Tensor, n: torch.Tensor, m: torch.Tensor, step: RaggedStep, H: int, dk: int, dv: int
               ) -> torch.Tensor:
    """-> y fp32 [T, H * dv]; S [slots, H, dk, dv], n [slots, H, dk], m [slots, H] (fp32) advanced in place."""
    _cuda(proj, S, n, m)
    assert proj.dtype == torch.float32 and S.is_contiguous() and n.is_contiguous() and m.is_contiguous()
    y = torch.empty(step.T, H * dv, dtype=torch.float32, device=proj.device)
    _lib.check_seq(_lib.load_seq().b200_seq_mlstm_scan(
        _ptr(proj), proj.stride(0), col_q, col_k, col_v, col_i, col_f, _ptr(i_bias), _ptr(f_bias), _dt(i_bias), float(cap), float(q_scale),
        _ptr(S), _ptr(n), _ptr(m), _ptr(step.state_slots), _ptr(step.cu_q), _ptr(step.position_ids), _ptr(y), y.stride(0), step.B, H, dk, dv,
        _stream()), "seq_mlstm_scan")
    return y


def causal_conv(u: torch.Tensor, col0: int, channels: int, w: torch.Tensor, bias: Optional[torch.Tensor], conv_state: torch.Tensor,
                step: RaggedStep, act_silu: bool = False) -> torch.Tensor:
    """Depth-wise causal convolution (optionally + bias, optionally SiLU) of the columns [col0, col0 + channels) of u (fp32); state as
    in causal_conv_silu."""
    _cuda(u, w, bias, conv_state)
    assert u.dtype == torch.float32 and conv_state.dtype == torch.float32 and w.is_contiguous() and conv_state.is_contiguous()
    out = torch.empty(step.T, channels, dtype=torch.float32, device=u.device)
    _lib.check_seq(_lib.load_seq().b200_seq_causal_conv(
        _ptr(u), u.stride(0), col0, channels, w.shape[1], _ptr(w), _ptr(bias), _dt(w), int(act_silu), _ptr(conv_state), _ptr(step.state_slots),
        _ptr(step.seq_of_token), _ptr(step.cu_q), _ptr(step.position_ids), _ptr(out), step.T, step.B, _stream()), "seq_causal_conv")
    return out


def embed_add_pos(table: torch.Tensor, pos_table: torch.Tensor, ids: torch.Tensor, position_ids: torch.Tensor) -> torch.Tensor:
    """-> fp32 [T, W] = table[ids] + pos_table[position_ids] (learned absolute positions)."""
    _cuda(table, pos_table, ids, position_ids)
    assert ids.dtype == torch.int64 and position_ids.dtype == torch.int64 and table.is_contiguous() and pos_table.is_contiguous()
    assert table.dtype == pos_table.dtype and table.shape[1] == pos_table.shape[1]
    out = torch.empty(ids.shape[0], table.shape[1], dtype=torch.float32, device=table.device)
    _lib.check_seq(_lib.load_seq().b200_seq_embed_add_pos(_ptr(table), _ptr(pos_table), _dt(table), _ptr(ids), _ptr(position_ids), _ptr(out),
                                                          ids.shape[0], table.shape[1], table.shape[0], pos_table.shape[0], _stream()),
                   "seq_embed_add_pos")
    return out


def rmsnorm_rows(x: torch.Tensor, w: torch.Tensor, eps: float, w_offset: float = 0.0) -> torch.Tensor:
    """x fp32 [T, W] -> x / sqrt(mean(x^2) + eps) * (w + w_offset) in w's element type."""
    _cuda(x, w)
    assert x.dtype == torch.float32 and x.is_contiguous()
    out = torch.empty(x.shape, dtype=w.dtype, device=x.device)
    _lib.check_seq(_lib.load_seq().b200_seq_rmsnorm_rows(_ptr(x), _ptr(w), _dt(w), float(w_offset), _ptr(out), x.shape[0], x.shape[1], float(eps),
                                                         _stream()), "seq_rmsnorm_rows")
    return out


def heads_prepare(src: torch.Tensor, *, col_q: int, q_heads: int, dim: int, q_norm_w: Optional[torch.Tensor], temp_coef: float, temp_every: int,
                  col_k: int, k_heads: int, k_norm_w: Optional[torch.Tensor], col_v: int, v_width: int, normalise: bool, step: RaggedStep,
                  cache: torch.Tensor, k_off: int, v_off: int, k_group: int, v_group_width: int, eps: float) -> torch.Tensor:
    """src fp32 [T, C]: unit-RMS per head (optional weight) of the query heads at col_q and the key heads at col_k, the queries times
    the position's temperature; keys -> cache[slot, k_off:], v_width values from col_v -> cache[slot, v_off:]; -> queries fp32
    [T, q_heads, dim].  col_k / col_v < 0: the layer writes no keys / values (it reads another layer's rows).  Inside a block the
    pool is head-group-major (what `paged_attn` reads): `k_group` key heads and `v_group_width` value columns per key/value head
    group; of a block's tokens, one group's keys lie together, then the next group's, and after all keys the values likewise."""
    _cuda(src, cache, q_norm_w, k_norm_w)
    assert src.dtype == torch.float32 and src.stride(1) == 1 and cache.is_contiguous()
    q = torch.empty(step.T, q_heads, dim, dtype=torch.float32, device=src.device)
    _lib.check_seq(_lib.load_seq().b200_seq_heads_prepare(
        _ptr(src), src.stride(0), col_q, q_heads, dim, _ptr(q_norm_w), float(temp_coef), int(temp_every), col_k, k_heads, _ptr(k_norm_w), col_v,
        v_width, int(normalise), _ptr(step.position_ids), _ptr(step.slot_mapping), _ptr(cache), _dt(cache), cache.shape[-1], k_off, v_off,
        cache.shape[1], int(k_group), int(v_group_width), _ptr(q), step.T, float(eps), _stream()), "seq_heads_prepare")
    return q


def paged_attn(q: torch.Tensor, cache: torch.Tensor, step: RaggedStep, *, heads: int, kv_heads: int, maps: int, vdim: int, k_off: int,
               v_off: int, scale: float, window: int = 0, rel: Optional[torch.Tensor] = None, bucket_tab: Optional[torch.Tensor] = None
               ) -> torch.Tensor:
    """q fp32 [T, heads * maps, dim]; cache [blocks, page, row] (head-group-major inside a block, as `heads_prepare` writes it) with
    kv_heads * maps key heads from column k_off and kv_heads value heads (vdim) from column v_off -> fp32 [T, heads * maps, vdim]: causal soft-max attention of every token over its own sequence's cache rows.
    rel fp32 [rows, heads] + bucket_tab int32 [n]: rel[bucket(i - j), head] is added to the scaled score, bucket(n) = bucket_tab[n]
    below len(bucket_tab), rows - 1 from there on."""
    _cuda(q, cache, rel, bucket_tab)
    T, Hq, d = q.shape
    assert Hq == heads * maps and q.is_contiguous() and cache.is_contiguous() and q.dtype == torch.float32
    assert rel is None or (rel.dtype == torch.float32 and rel.is_contiguous() and rel.shape[1] == heads and bucket_tab.dtype == torch.int32)
    out = torch.empty(T, Hq, vdim, dtype=torch.float32, device=q.device)
    lib = _lib.load_seq()
    need = ctypes.c_int64(0)
    nsplit = lib.b200_seq_paged_attn_splits(_dt(cache), T, step.B, heads, kv_heads, maps, d, vdim, ctypes.byref(need)) if _ATTN_SPLIT else 1
    partial = torch.empty(need.value, dtype=torch.float32, device=q.device) if nsplit > 1 else None
    _lib.check_seq(lib.b200_seq_paged_attn(
        _ptr(q), _ptr(cache), _dt(cache), cache.shape[-1], k_off, v_off, _ptr(step.block_table), step.block_table.stride(0),
        _ptr(step.seq_of_token), _ptr(step.cu_q), step.B, _ptr(step.position_ids), _ptr(out), T, heads, kv_heads, maps, d, vdim, int(window),
        float(scale),
        cache.shape[1], _ptr(rel), _ptr(bucket_tab), 0 if bucket_tab is None else bucket_tab.shape[0], 0 if rel is None else rel.shape[0],
        _ptr(partial), nsplit, _stream()), "seq_paged_attn")
    return out


def diff_combine(maps_out: torch.Tensor, heads: int, vdim: int, lam: float, out_scale: float, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """maps_out fp32 [T, heads * 2, vdim] -> [T, heads * vdim]: (a1 - lam a2) / sqrt(mean(.^2) + eps) * out_scale per head."""
    _cuda(maps_out)
    assert maps_out.dtype == torch.float32 and maps_out.is_contiguous() and maps_out.shape[1:] == (heads * 2, vdim)
    T = maps_out.shape[0]
    out = torch.empty(T, heads * vdim, dtype=out_dtype, device=maps_out.device)
    _lib.check_seq(_lib.load_seq().b200_seq_diff_combine(_ptr(maps_out), _ptr(out), _dt(out), T, heads, vdim, float(lam), float(out_scale),
                                                         float(eps), _stream()), "seq_diff_combine")
    return out


@dataclass
class MoeRouting:
    """picks of a step's tokens and the compact row plan the grouped products read"""
    T: int
    experts: int
    top: int
    ids: torch.Tensor       # [T, top] int32
    weights: torch.Tensor   # [T, top] fp32
    plan: torch.Tensor      # int32 workspace (b200_seq_moe_plan_ints)


def moe_route(logits: torch.Tensor, top: int, *, sigmoid_scores: bool = False, correction: Optional[torch.Tensor] = None,
              weight_scale: float = 1.0) -> MoeRouting:
    """logits fp32 [T, E] -> the `top` largest per token (ties: the lower expert), weights = soft-max over the picked logits.
    sigmoid_scores: the picks are the largest sigmoid(logit) + correction[expert]; the weights are the picked sigmoid(logit)
    divided by their sum and multiplied by weight_scale."""
    _cuda(logits, correction)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    T, E = logits.shape
    lib = _lib.load_seq()
    ids = torch.empty(T, top, dtype=torch.int32, device=logits.device)
    weights = torch.empty(T, top, dtype=torch.float32, device=logits.device)
    plan = torch.empty(int(lib.b200_seq_moe_plan_ints(T, E, top)), dtype=torch.int32, device=logits.device)
    if sigmoid_scores:
        assert correction is None or (correction.is_contiguous() and correction.shape == (E,))
        _lib.check_seq(lib.b200_seq_moe_route_scored(_ptr(logits), T, E, top, 1, _ptr(correction), 1 if correction is None else _dt(correction),
                                                     float(weight_scale), _ptr(ids), _ptr(weights), _ptr(plan), _stream()), "seq_moe_route")
    else:
        _lib.check_seq(lib.b200_seq_moe_route(_ptr(logits), T, E, top, _ptr(ids), _ptr(weights), _ptr(plan), _stream()), "seq_moe_route")
    return MoeRouting(T, E, top, ids, weights, plan)


def moe_linear(a: torch.Tensor, w: torch.Tensor, r: MoeRouting, gather: bool, out_dtype: torch.dtype) -> torch.Tensor:
    """w [E, N, K]; a [T, K] (gather: the row of each pick's token) or [T * top, K] (compact rows) -> [T * top, N] compact rows."""
    _cuda(a, w)
    E, N, K = w.shape
    assert w.is_contiguous() and a.stride(1) == 1 and a.shape[1] == K and E == r.experts and a.shape[0] == (r.T if gather else r.T * r.top)
    out = torch.empty(r.T * r.top, N, dtype=out_dtype, device=a.device)
    _lib.check_seq(_lib.load_seq().b200_seq_moe_linear(_ptr(a), _dt(a), a.stride(0), int(gather), _ptr(w), _dt(w), _ptr(out), _dt(out),
                                                       out.stride(0), _ptr(r.plan), r.T, E, r.top, N, K, _stream()), "seq_moe_linear")
    return out


def moe_gather_rows(a: torch.Tensor, r: MoeRouting) -> torch.Tensor:
    """a [T, K] -> [T * top, K]: the compact rows (row i holds the token of pick i in expert order), for one dense product per expert."""
    _cuda(a)
    assert a.stride(1) == 1 and a.shape[0] == r.T
    out = torch.empty(r.T * r.top, a.shape[1], dtype=a.dtype, device=a.device)
    _lib.check_seq(_lib.load_seq().b200_seq_moe_gather_rows(_ptr(a), _dt(a), a.stride(0), _ptr(out), _ptr(r.plan), r.T, r.experts, r.top, a.shape[1],
                                                            _stream()), "seq_moe_gather_rows")
    return out


def moe_expert_offsets(r: MoeRouting) -> list:
    """first compact row of every expert, and the row count at the end (a device-to-host read: not inside a captured graph)"""
    return r.plan[r.experts:2 * r.experts + 1].tolist()


def moe_combine_add(resid: torch.Tensor, mix: Optional[torch.Tensor], y: Optional[torch.Tensor], r: Optional[MoeRouting]) -> None:
    """resid (fp32, in place) += mix + sum_k weights[t, k] y[row(t, k)]; either addend may be None."""
    _cuda(resid, mix, y)
    assert resid.dtype == torch.float32 and resid.is_contiguous() and (mix is None or (mix.dtype == torch.float32 and mix.is_contiguous()))
    assert y is None or (y.dtype == torch.float32 and y.stride(1) == 1 and r is not None)
    T, W = resid.shape
    _lib.check_seq(_lib.load_seq().b200_seq_moe_combine_add(
        _ptr(resid), _ptr(mix), _ptr(y), 0 if y is None else y.stride(0), None if y is None else _ptr(r.weights), None if y is None else _ptr(r.plan),
        T, 0 if y is None else r.experts, 0 if y is None else r.top, W, _stream()), "seq_moe_combine_add")


def gated_rms_add(resid: torch.Tensor, y: torch.Tensor, gate: Optional[torch.Tensor], w: torch.Tensor, eps: float,
                  typed_copy: bool = False) -> Optional[torch.Tensor]:
    """resid (fp32, in place) += v / sqrt(mean(v^2) + eps) * w with v = y * sigmoid(gate) (gate None: v = y); y and gate fp32 [T, W].
    typed_copy: also returns the updated stream in w's element type (the input of the next projection); for float32 that is the
    stream itself."""
    _cuda(resid, y, gate, w)
    assert resid.dtype == torch.float32 and resid.is_contiguous() and y.dtype == torch.float32 and y.is_contiguous() and y.shape == resid.shape
    assert gate is None or (gate.dtype == torch.float32 and gate.is_contiguous() and gate.shape == resid.shape)
    copy = torch.empty(resid.shape, dtype=w.dtype, device=resid.device) if typed_copy and w.dtype != torch.float32 else None
    _lib.check_seq(_lib.load_seq().b200_seq_gated_rms_add(_ptr(y), _ptr(gate), _ptr(w), _dt(w), _ptr(resid), _ptr(copy), resid.shape[0],
                                                          resid.shape[1], float(eps), _stream()), "seq_gated_rms_add")
    return (copy if copy is not None else resid) if typed_copy else None


def cast_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """the fp32 stream in the projections' element type (float32: the stream itself)"""
    _cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    if dtype == torch.float32:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _lib.check_seq(_lib.load_seq().b200_seq_cast_rows(_ptr(x), _ptr(out), _dt(dtype), x.numel(), _stream()), "seq_cast_rows")
    return out


ACT_SILU, ACT_GELU_TANH = 0, 1


def ff_gate(gate_up: torch.Tensor, act: int) -> torch.Tensor:
    """[T, 2F] = [g | u] -> [T, F]: act(g) * u with act SiLU or the tanh form of GELU, evaluated in fp32."""
    _cuda(gate_up)
    assert gate_up.is_contiguous()
    T, F2 = gate_up.shape
    out = torch.empty(T, F2 // 2, dtype=gate_up.dtype, device=gate_up.device)
    _lib.check_seq(_lib.load_seq().b200_seq_ff_gate(_ptr(gate_up), _ptr(out), _dt(gate_up), T, F2 // 2, int(act), _stream()), "seq_ff_gate")
    return out


def delta_scan(c: torch.Tensor, col_q: int, col_k: int, col_v: int, raw: torch.Tensor, col_b: int, col_a: int, A_log: torch.Tensor,
               dt_bias: torch.Tensor, q_scale: float, S: torch.Tensor, step: RaggedStep, H: int, kv_heads: int, dk: int, dv: int) -> torch.Tensor:
    """Gated delta rule -> y fp32 [T, H * dv]; S fp32 [slots, H, dk, dv] advanced in place.  c fp32: activated q / k (kv_heads x dk
    each) and v (H x dv) columns; raw fp32: write-strength logits at col_b and decay logits at col_a, one per head."""
    _cuda(c, raw, S, A_log, dt_bias)
    assert c.dtype == torch.float32 and raw.dtype == torch.float32 and S.dtype == torch.float32 and S.is_contiguous()
    assert c.stride(1) == 1 and raw.stride(1) == 1 and A_log.dtype == dt_bias.dtype
    y = torch.empty(step.T, H * dv, dtype=torch.float32, device=c.device)
    _lib.check_seq(_lib.load_seq().b200_seq_delta_scan(
        _ptr(c), c.stride(0), col_q, col_k, col_v, _ptr(raw), raw.stride(0), col_b, col_a, _ptr(A_log), _ptr(dt_bias), _dt(A_log), float(q_scale),
        _ptr(S), _ptr(step.state_slots), _ptr(step.cu_q), _ptr(step.position_ids), _ptr(y), y.stride(0), step.B, H, kv_heads, dk, dv, _stream()),
        "seq_delta_scan")
    return y


def qk_rot_prepare(src: torch.Tensor, *, col_q: int, col_k: int, col_v: int, heads: int, kv_heads: int, dim: int, vdim: int,
                   q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], whole_norm: bool, eps: float, cos: Optional[torch.Tensor],
                   sin: Optional[torch.Tensor], rot: int, step: RaggedStep, cache: torch.Tensor, k_off: int, v_off: int,
                   v_cos: Optional[torch.Tensor] = None, v_sin: Optional[torch.Tensor] = None, v_rot: int = 0, v_interleaved: bool = False
                   ) -> torch.Tensor:
    """src fp32 [T, C] = [q | k | v] projections: RMS norm over the whole q and the whole k projection (whole_norm), rotation of the
    first `rot` columns of every head in the rotate-half layout with the cos / sin tables, keys and values into the token's row of
    `cache` [blocks, page, row] (token-major: keys of all key heads from k_off, values from v_off) -> queries fp32 [T, heads, dim].
    v_rot > 0: the first v_rot columns of every value head turn by the token's position as well, with tables of their own
    (v_cos / v_sin [positions, v_rot / 2]); pairs are column i with i + v_rot / 2, or neighbours (v_interleaved)."""
    _cuda(src, cache, q_norm_w, k_norm_w, cos, sin, v_cos, v_sin)
    assert src.dtype == torch.float32 and src.stride(1) == 1 and cache.is_contiguous()
    assert rot == 0 or (cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous() and cos.shape[1] == rot // 2)
    assert v_rot == 0 or (v_cos.dtype == torch.float32 and v_cos.is_contiguous() and v_sin.is_contiguous() and v_cos.shape[1] == v_rot // 2)
    q = torch.empty(step.T, heads, dim, dtype=torch.float32, device=src.device)
    _lib.check_seq(_lib.load_seq().b200_seq_qk_rot_prepare(
        _ptr(src), src.stride(0), col_q, col_k, col_v, heads, kv_heads, dim, vdim, _ptr(q_norm_w), _ptr(k_norm_w), int(whole_norm), float(eps),
        _ptr(cos), _ptr(sin), int(rot), _ptr(step.position_ids), _ptr(step.slot_mapping), _ptr(cache), _dt(cache), cache.shape[-1], k_off, v_off,
        _ptr(q), step.T, _ptr(v_cos), _ptr(v_sin), int(v_rot), int(v_interleaved), _stream()), "seq_qk_rot_prepare")
    return q


def talk_attn(q: torch.Tensor, cache: torch.Tensor, step: RaggedStep, *, kv_heads: int, vdim: int, k_off: int, v_off: int, scale: float,
              talk: Optional[torch.Tensor] = None, chunk: int = 0, window: int = 0, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q fp32 [T, heads, dim]; cache [blocks, page, row] token-major as `qk_rot_prepare` writes it -> fp32 [T, heads, vdim]: attention
    of every token over its own sequence's cache rows; the scaled scores of all heads are mixed by talk fp32 [heads, heads]
    (s'_h = sum_g talk[h, g] s_g) before the soft-max.  chunk > 0: a query sees only keys of its own chunk of `chunk` positions
    (counted from position 0); window > 0: only the last `window` keys.  sink fp32 [heads]: exp(sink[h]) joins head h's soft-max
    denominator (after the mix, not scaled) and carries no value."""
    _cuda(q, cache, talk, sink)
    T, H, d = q.shape
    assert q.is_contiguous() and cache.is_contiguous() and q.dtype == torch.float32
    assert talk is None or (talk.dtype == torch.float32 and talk.is_contiguous() and talk.shape == (H, H))
    assert sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.shape == (H,))
    out = torch.empty(T, H, vdim, dtype=torch.float32, device=q.device)
    lib = _lib.load_seq()
    need = ctypes.c_int64(0)
    nsplit = lib.b200_seq_talk_attn_splits(_dt(cache), T, step.B, H, kv_heads, d, vdim, ctypes.byref(need)) if _ATTN_SPLIT else 1
    partial = torch.empty(need.value, dtype=torch.float32, device=q.device) if nsplit > 1 else None
    _lib.check_seq(lib.b200_seq_talk_attn(
        _ptr(q), _ptr(cache), _dt(cache), cache.shape[-1], k_off, v_off, _ptr(step.block_table), step.block_table.stride(0),
        _ptr(step.seq_of_token), _ptr(step.cu_q), step.B, _ptr(step.position_ids), _ptr(talk), _ptr(out), T, H, kv_heads, d, vdim, int(chunk),
        int(window), float(scale), cache.shape[1], _ptr(partial), nsplit, _ptr(sink), _stream()), "seq_talk_attn")
    return out


def streams_step(X: torch.Tensor, *, init: Optional[torch.Tensor] = None, y: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
                 out_coef: Optional[torch.Tensor] = None, in_coef: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
                 eps: float = 0.0, out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """Several residual streams per token, X fp32 [T, S, W] in place; one launch does what lies between two sublayers.
    init [T, W]: every stream starts as this row.  y [T, W] (+ mix [S, S] indexed [from, to], out_coef [S]): all streams at once
    from the old ones, X_t <- sum_s mix[s, t] X_s + out_coef[t] y.  in_coef [S]: returns unit_rms(sum_s in_coef[s] X_s) * norm_w of
    the new streams in norm_w's element type (norm_w None: the plain sum in `out_dtype`).  All coefficients fp32."""
    _cuda(X, init, y, mix, out_coef, in_coef, norm_w)
    assert X.dtype == torch.float32 and X.is_contiguous() and X.dim() == 3
    T, S, W = X.shape
    for t, shape in ((init, (T, W)), (y, (T, W)), (mix, (S, S)), (out_coef, (S,)), (in_coef, (S,))):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous() and tuple(t.shape) == shape)
    dt = norm_w.dtype if norm_w is not None else (out_dtype or torch.float32)
    typed = torch.empty(T, W, dtype=dt, device=X.device) if in_coef is not None else None
    _lib.check_seq(_lib.load_seq().b200_seq_streams_step(_ptr(X), S, _ptr(init), _ptr(y), _ptr(mix), _ptr(out_coef), _ptr(in_coef), _ptr(norm_w),
                                                         _dt(dt), _ptr(typed), T, W, float(eps), _stream()), "seq_streams_step")
    return typed


ACT_TANH = 2


def ff_act(x: torch.Tensor, act: int, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """act(x) element by element (ACT_SILU, ACT_GELU_TANH, ACT_TANH), evaluated in fp32; x [T, F] may be a column slice; fp32 rows may
    come out in another element type."""
    _cuda(x)
    assert x.dim() == 2 and x.stride(1) == 1
    out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    _lib.check_seq(_lib.load_seq().b200_seq_ff_act(_ptr(x), _dt(x), x.stride(0), _ptr(out), _dt(out), x.shape[0], x.shape[1], int(act), _stream()),
                   "seq_ff_act")
    return out


def heads_turn_gate(a: torch.Tensor, gate: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rot: int,
                    interleaved: bool, step: RaggedStep, out_dtype: torch.dtype, out: Optional[torch.Tensor] = None, out_scale: float = 1.0
                    ) -> torch.Tensor:
    """a fp32 [T, H, dv] -> [T, H * dv] in out_dtype: the first `rot` columns of every head turned back by the token's position (the
    inverse of the values' turn in `qk_rot_prepare`), then the head times sigmoid(gate[t, h]) (gate fp32 [T, H], may be a column slice)
    and times out_scale.  `out` may be a column slice of a wider buffer (the input of a product that several mixers share)."""
    _cuda(a, gate, cos, sin)
    T, H, dv = a.shape
    assert a.dtype == torch.float32 and a.is_contiguous() and (gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape == (T, H)))
    assert rot == 0 or (cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous() and cos.shape[1] == rot // 2)
    if out is None:
        out = torch.empty(T, H * dv, dtype=out_dtype, device=a.device)
    assert out.dtype == out_dtype and out.shape == (T, H * dv) and out.stride(1) == 1
    _lib.check_seq(_lib.load_seq().b200_seq_heads_turn_gate(_ptr(a), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(cos), _ptr(sin),
                                                            int(rot), int(interleaved), _ptr(step.position_ids), _ptr(out), _dt(out),
                                                            out.stride(0), float(out_scale), T, H, dv, _stream()), "seq_heads_turn_gate")
    return out


def gdelta_scan(raw: torch.Tensor, col_r: int, col_k: int, col_v: int, col_a: int, dec: torch.Tensor, col_d: int, a_bias: torch.Tensor,
                w0: torch.Tensor, decay_scale: float, S: torch.Tensor, step: RaggedStep, H: int, dk: int, dv: int) -> torch.Tensor:
    """Generalised delta rule -> y fp32 [T, H * dv]; S fp32 [slots, H, dk, dv] advanced in place.  raw fp32: read vectors, keys and
    removal logits (H x dk each) and values (H x dv) at the given columns; dec fp32: decay logits (H x dk) at col_d; per token
    S <- diag(w) S - (a * u)(u^T S) + k v^T with u the unit-length key, w = exp(-decay_scale sigmoid(dec + w0)), a = sigmoid(. + a_bias)."""
    _cuda(raw, dec, S, a_bias, w0)
    assert raw.dtype == torch.float32 and dec.dtype == torch.float32 and S.dtype == torch.float32 and S.is_contiguous()
    assert raw.stride(1) == 1 and dec.stride(1) == 1 and a_bias.dtype == w0.dtype and a_bias.is_contiguous() and w0.is_contiguous()
    y = torch.empty(step.T, H * dv, dtype=torch.float32, device=raw.device)
    _lib.check_seq(_lib.load_seq().b200_seq_gdelta_scan(
        _ptr(raw), raw.stride(0), col_r, col_k, col_v, col_a, _ptr(dec), dec.stride(0), col_d, _ptr(a_bias), _ptr(w0), _dt(w0), float(decay_scale),
        _ptr(S), _ptr(step.state_slots), _ptr(step.cu_q), _ptr(step.position_ids), _ptr(y), y.stride(0), step.B, H, dk, dv, _stream()),
        "seq_gdelta_scan")
    return y


def mingru_scan(proj: torch.Tensor, col_z: int, col_x: int, col_g: int, z_bias: Optional[torch.Tensor], x_bias: Optional[torch.Tensor],
                state: torch.Tensor, step: RaggedStep, width: int, out_dtype: torch.dtype, out: Optional[torch.Tensor] = None,
                out_scale: float = 1.0) -> torch.Tensor:
    """Minimal gated recurrent unit -> S_t * SiLU(gate) * out_scale [T, width] in out_dtype (col_g < 0: S_t), optionally into `out`, a
    column slice of a wider buffer; state fp32 [slots, width] advanced in place.  proj fp32: update-gate logits, candidate inputs and output-gate logits at the given columns; z = sigmoid(. + z_bias),
    candidate = x + 1/2 for x >= 0 and sigmoid(x) below, S <- (1 - z) S + z candidate."""
    _cuda(proj, state, z_bias, x_bias)
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and state.dtype == torch.float32 and state.is_contiguous()
    assert z_bias is None or x_bias is None or z_bias.dtype == x_bias.dtype
    b = z_bias if z_bias is not None else x_bias
    if out is None:
        out = torch.empty(step.T, width, dtype=out_dtype, device=proj.device)
    assert out.dtype == out_dtype and out.shape == (step.T, width) and out.stride(1) == 1
    _lib.check_seq(_lib.load_seq().b200_seq_mingru_scan(
        _ptr(proj), proj.stride(0), col_z, col_x, col_g, _ptr(z_bias), _ptr(x_bias), 1 if b is None else _dt(b), _ptr(state),
        _ptr(step.state_slots), _ptr(step.cu_q), _ptr(step.position_ids), _ptr(out), _dt(out), out.stride(0), float(out_scale), step.T, step.B, width, _stream()),
        "seq_mingru_scan")
    return out
