"""The head-mixed attention kernel alone at a served shape, for an `ncu` capture or a CUDA-event timing.

    python tools/profile_talk_attn.py [--mode prefill|decode] [--heads 32 --kv-heads 8 --dim 128 --vdim 128] [--seqs N --len L]

prefill: N sequences of L tokens as one ragged step; decode: N sequences with L cached tokens, one new token each.  The cache holds
random rows (> L2 for the default decode shape).  Prints the CUDA-event time of the call and the achieved FLOP/s or bytes/s.
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="decode", choices=["prefill", "decode"])
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--vdim", type=int, default=128)
    ap.add_argument("--seqs", type=int, default=32)
    ap.add_argument("--len", type=int, default=1040)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    import torch
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    dev = "cuda:0"
    H, G, d, dv, B, L, page = a.heads, a.kv_heads, a.dim, a.vdim, a.seqs, a.len, 16
    per_seq = (L + page) // page + 1
    cache = torch.randn(B * per_seq, page, G * (d + dv), device=dev).to(torch.bfloat16)
    table = torch.randperm(B * per_seq, device=dev).to(torch.int32).view(B, per_seq)
    n = L if a.mode == "prefill" else 1
    start = 0 if a.mode == "prefill" else L
    pos = (torch.arange(n, device=dev)[None, :] + start).expand(B, n).reshape(-1).contiguous()
    seq = torch.arange(B, device=dev, dtype=torch.int32)[:, None].expand(B, n).reshape(-1).contiguous()
    slots = (table.long()[seq.long(), pos // page] * page + pos % page).contiguous()
    step = ops.RaggedStep(T=B * n, B=B, position_ids=pos, cu_q=(torch.arange(B + 1, device=dev, dtype=torch.int32) * n).contiguous(),
                          seq_of_token=seq, slot_mapping=slots, block_table=table, state_slots=None)
    q = torch.randn(B * n, H, d, device=dev)
    talk = (torch.eye(H, device=dev) + 0.02 * torch.randn(H, H, device=dev)).contiguous()

    def run():
        return ops.talk_attn(q, cache, step, kv_heads=G, vdim=dv, k_off=0, v_off=G * d, scale=d ** -0.5, talk=talk, chunk=a.chunk)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(3):
        run()
    ms = []
    for _ in range(a.iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    t = sorted(ms)[len(ms) // 2] * 1e-3
    if a.mode == "prefill":
        flops = B * (L * (L + 1) // 2) * H * (d + dv + H) * 2
        print(f"prefill {B} x {L}: {t * 1e3:.3f} ms, {flops / t / 1e12:.1f} TFLOP/s (products + mix)")
    else:
        byts = B * (L + 1) * G * (d + dv) * 2
        print(f"decode {B} x {L}: {t * 1e6:.1f} us, {byts / t / 1e9:.0f} GB/s over {byts / 1e6:.0f} MB of cache rows")


if __name__ == "__main__":
    main()
