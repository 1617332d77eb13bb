"""The row kernel of the residual streams and the two elementwise / matrix scans alone at a served shape, for an `ncu` capture or a
CUDA-event timing.

    python tools/profile_stream_scans.py [--seqs 4 --len 1024 --width 2048 --heads 16 --dim 128 --streams 3]

One ragged step of N sequences of L tokens: `gdelta_scan` (generalised delta rule), `streams_step` (write + read + norm of the
residual streams in one launch) and `mingru_scan` (minimal gated recurrent unit) on random inputs that are larger than L2 together;
L2 is flushed before every timed call.  Prints the CUDA-event time of each call and tokens/s or bytes/s.
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqs", type=int, default=4)
    ap.add_argument("--len", type=int, default=1024)
    ap.add_argument("--width", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--streams", type=int, default=3)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    import torch
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    dev = "cuda:0"
    B, L, W, H, d, S = a.seqs, a.len, a.width, a.heads, a.dim, a.streams
    T, n = B * L, H * d
    g = torch.Generator(device=dev).manual_seed(0)
    step = ops.RaggedStep(T=T, B=B, position_ids=torch.arange(L, device=dev).repeat(B),
                          cu_q=torch.arange(0, T + 1, L, dtype=torch.int32, device=dev),
                          seq_of_token=torch.arange(B, dtype=torch.int32, device=dev).repeat_interleave(L),
                          slot_mapping=torch.zeros(T, dtype=torch.int64, device=dev), block_table=torch.zeros(B, 1, dtype=torch.int32, device=dev),
                          state_slots=torch.arange(B, dtype=torch.int32, device=dev))
    raw = torch.randn(T, 5 * n + 16, device=dev, generator=g)
    dec = torch.randn(T, n, device=dev, generator=g)
    a_b, w0 = torch.zeros(n, device=dev, dtype=torch.bfloat16), torch.ones(n, device=dev, dtype=torch.bfloat16)
    mem = torch.zeros(B, H, d, d, device=dev)
    X = torch.randn(T, S, W, device=dev, generator=g)
    y = torch.randn(T, W, device=dev, generator=g)
    mix, co, ci = torch.eye(S, device=dev), torch.ones(S, device=dev), torch.full((S,), 1.0 / S, device=dev)
    nw = torch.ones(W, device=dev, dtype=torch.bfloat16)
    proj = torch.randn(T, 3 * W, device=dev, generator=g)
    gru = torch.zeros(B, W, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        total = 0.0
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / a.iters

    calls = {
        "gdelta_scan": lambda: ops.gdelta_scan(raw, 0, n, 2 * n, 4 * n, dec, 0, a_b, w0, 0.6065, mem, step, H, d, d),
        "streams_step": lambda: ops.streams_step(X, y=y, mix=mix, out_coef=co, in_coef=ci, norm_w=nw, eps=1e-5),
        "mingru_scan": lambda: ops.mingru_scan(proj, 0, W, 2 * W, None, None, gru, step, W, torch.bfloat16),
    }
    for fn in calls.values():
        fn()
    torch.cuda.synchronize()
    ms = {k: timed(fn) for k, fn in calls.items()}
    print(f"gdelta_scan  {ms['gdelta_scan']:.4f} ms  {T / ms['gdelta_scan'] * 1e3:.0f} tokens/s  ({B} x {L} tokens, {H} heads of {d} x {d})")
    print(f"streams_step {ms['streams_step']:.4f} ms  {T * W * (S * 8 + 4 + 2) / ms['streams_step'] / 1e6:.0f} GB/s  ({S} streams of width {W})")
    print(f"mingru_scan  {ms['mingru_scan']:.4f} ms  {T * W * 14 / ms['mingru_scan'] / 1e6:.0f} GB/s  (width {W})")


if __name__ == "__main__":
    main()
