#!/usr/bin/env python
"""bench.py — decode throughput of the TGIS continuous-batching hot path on B200 (contract in the task prompt / DESIGN.md).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference] [--no-extra]

Workloads (BASELINE.json):
  llama3-8b-gptq   the north-star target "batched int4 Llama-8B decode at bs=64": Llama-3-8B (GQA-8) GPTQ int4 g128, bs=64,
                   seq 1024->2048, tensor parallel over N GPUs.  DEFAULT AT EVERY N: it is the one int4 model that shards at
                   tp = 1/2/4/8, so the driver's 1/2/4/8 curve compares like with like.
  llama2-7b-gptq   config[2]: Llama-2-7B GPTQ int4, 1 GPU, bs=64, 1024->2048 (row-sharding stops at tp=2: 11008/tp % 128).
                   Measured in the same run at N=1 and reported under "extra".
  llama2-7b-fp16   config[3]: Llama-2-7B fp16, tensor parallel, bs=64.  Measured in the same run at N>1, under "extra".
  tinyllama-fp16   config[1]: TinyLlama-1.1B fp16, bs=32, 512->1024 (on request).
  llama3-70b-gptq-mixed   config[4]: Llama-3-70B int4, NUM_SHARD=8, continuous batching (Poisson arrivals, prompts U[256,1024], outputs
                   U[128,512], up to 128 running) through Prefill / NextToken with prune + concatenate; llama3-8b-gptq-mixed is the
                   same session on one GPU (on request).

A "step" is one decode step of the whole batch (one token per sequence).  The run really generates the whole trajectory
L0 -> L1 from the prompt, so KV contents, block tables and lengths are what the serving path produces:
  value : B*K / device time of K consecutive graph-replayed steps centred on the mean context (L0+L1)/2, inputs resident in
          HBM, no host round trip (CUDA events, max over ranks)
  e2e   : the same metric over ALL the other decode steps of the trajectory through the public API
          `FlashCausalLM.generate_token(batch)` driven from host buffers: every step copies the step's input token ids from
          pinned host memory and reads the chosen ids back to the host
  roofline : attn_decode_paged kernel, algorithmic KV bytes per launch / CUDA-event time per launch vs the measured HBM peak;
          "gemm" beside it: the int4 / fp16 linears' weight bytes per step / their CUDA-event time per step
  self_check : greedy ids of a 2-layer model of the same widths through the same code path vs the CPU oracle (tests' rule:
          exact outside the 2-ulp tie band)
  cpu_baseline : the reference's CPU CausalLM path (HF eager fp32, padded batch, greedy) on a bounded sample
`--impl reference` times that CPU path alone (rank 0 only) and prints the same JSON line with "impl": "reference".
Data is synthetic: seeded random weights of the named architecture, prompts "test " * L0 (the reference's own
load recipe, utils/memory_characterizer.py:219-240).
"""
from __future__ import annotations

import argparse
import ctypes
import gc
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (arch, quantize, batch, prompt_len, end_len)
    "llama3-8b-gptq": ("llama-3-8b", "gptq", 64, 1024, 2048),
    "llama2-7b-gptq": ("llama-2-7b", "gptq", 64, 1024, 2048),
    "llama2-7b-fp16": ("llama-2-7b", None, 64, 1024, 2048),
    "llama3-70b-gptq": ("llama-3-70b", "gptq", 128, 512, 1024),  # steady-state sibling of config[4]; needs --gpus 2 or more
    "pythia-12b-fp16": ("pythia-12b", None, 64, 1024, 2048),  # GPT-NeoX, the second flash family (parallel residual, partial rotary)
    "tiny-neox": ("tiny-neox", None, 4, 32, 256),
    "neox-w2048": ("neox-w2048", None, 32, 1024, 1088),  # equal-size partners of --hybrid-compare (3 layers of a real model's widths)
    "neox-w4096": ("neox-w4096", None, 32, 1024, 1088),
    "tinyllama-fp16": ("tinyllama-1.1b", None, 32, 512, 1024),
    "tiny-test": ("tiny-test", None, 4, 32, 256),
}
# continuous-batching sessions (BASELINE config[4] and a single-GPU sibling): (arch, quantize, max batch, prompt range, output range,
# requests, Poisson arrivals per second)
MIXED_WORKLOADS = {
    "llama3-70b-gptq-mixed": ("llama-3-70b", "gptq", 128, (256, 1024), (128, 512), 384, 60.0),
    "llama3-8b-gptq-mixed": ("llama-3-8b", "gptq", 128, (256, 1024), (128, 512), 384, 120.0),
    "tiny-test-mixed": ("tiny-test", None, 8, (8, 60), (4, 24), 40, 2000.0),
}
DEFAULT_WORKLOAD = "llama3-8b-gptq"
METRIC = "decode_tokens_per_s"
UNIT = "tokens/s"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled during the timed region (B200_PROFILING.md recipe).  Started well before
    the timed region (nvidia-smi needs a second to enumerate an 8-GPU box); only samples between mark() and stop() count."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.lines = []
        self.proc = None
        self.index = index
        self.first = 0

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self, wait_s: float = 5.0):
        """call right before the timed region: waits until nvidia-smi delivers, then forgets the earlier samples"""
        if self.proc is None:
            return
        t_end = time.time() + wait_s
        while not self.lines and time.time() < t_end:
            time.sleep(0.02)
        self.first = max(0, len(self.lines) - 1)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.12)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for ln in self.lines[self.first:]:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ======================================================================================================
# CPU baseline: the reference's CausalLM path (models/causal_lm.py:548-739 on the hf_transformers engine) restated
# ======================================================================================================
def cpu_reference_decode(arch: str, B: int, ctx: int, steps: int, warmup: int, sample_layers: int):
    """Times greedy decode steps of the reference's CPU path on a bounded sample: `sample_layers` of the model's layers
    (same widths, fp32, HF eager attention, padded rectangular KV at context `ctx`), scaled to the full depth.
    -> dict(value tokens/s of the full model, cores, sample, ms_per_step full depth, steps timed per sample)."""
    from oracle import causal_lm as ocl  # oracle/ is the checker + CPU baseline only (never on the product path)
    return ocl.time_decode(arch, B, ctx, steps, warmup, sample_layers)


def run_reference(args, workload):
    arch, quantize, B, L0, L1 = WORKLOADS[workload]
    rank = int(os.getenv("RANK", "0"))
    if rank != 0:
        return 0
    ctx = (L0 + L1) // 2
    r = cpu_reference_decode(arch, B, ctx, args.steps, args.warmup, args.cpu_layers)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "arch": arch, "batch": B, "prompt_len": L0, "end_len": L1, "context": ctx,
                   "steps_timed_per_sample": r["steps_timed"], "extrapolated_in_depth": r["extrapolated"]},
        "cpu_baseline": {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port", "sample": r["sample"]},
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if not args.no_extra and workload != "tiny-test":
        try:  # BASELINE config[0]: gpt2 CausalLM fp32 CPU, bs=4, 128 -> 256 (whole model, really run; random-init: no weights here)
            from oracle import causal_lm as ocl
            line["extra"] = {"config0_gpt2_cpu": ocl.time_decode_gpt2(4, 192, steps=8, warmup=2)}
        except Exception as e:  # noqa: BLE001
            line["extra"] = {"config0_gpt2_cpu": {"failed": f"{type(e).__name__}: {e}"}}
    print(json.dumps(line), flush=True)
    return 0


# ======================================================================================================
# GPU arm
# ======================================================================================================
def build_model(workload, world, rank, num_layers=None, cfg_override=None, weights=None, blocks=None):
    import torch
    import tgis_b200  # noqa: F401
    from tgis_b200.inference_engine import InferenceEngine
    from tgis_b200.models.flash_causal_lm import FlashCausalLM
    from tgis_b200.utils.dist import initialize_torch_distributed
    from tgis_b200.utils.synthetic import SyntheticWeights, make_tokenizer, model_config

    arch, quantize, B, L0, L1 = WORKLOADS[workload]
    cfg = cfg_override or model_config(arch, quantize=quantize, max_position_embeddings=max(4096, L1 + 64), num_layers=num_layers)
    local = int(os.getenv("LOCAL_RANK", rank))
    torch.cuda.set_device(local % torch.cuda.device_count())
    device = torch.device("cuda", torch.cuda.current_device())
    pg = initialize_torch_distributed(world, rank)
    if weights is None:
        weights = SyntheticWeights(cfg, device, torch.float16, pg, quantize=quantize)
    tok = make_tokenizer(cfg.vocab_size)
    engine = InferenceEngine("<synthetic>", None, torch.float16, quantize, cfg, L1, weights=weights, tokenizer=tok)
    if blocks is None:
        blocks = B * ((L1 + 16) // 16 + 1) + 8
    model = FlashCausalLM("<synthetic>", None, "tgis_native", torch.float16, quantize, cfg, engine=engine, num_kv_blocks=blocks)
    return model, cfg


def make_batch_pb(B, L0, n_new, batch_id=0):
    from tgis_b200 import pb
    reqs = []
    for i in range(B):
        reqs.append(pb.Request(
            id=i, inputs="test " * 10000, input_length=L0, truncate=True, max_output_length=n_new,
            parameters=pb.NextTokenChooserParameters(temperature=0.0, top_k=0, top_p=1.0, typical_p=0.0, min_new_tokens=n_new)))
    return pb.Batch(id=batch_id, requests=reqs, total_tokens=B * (L0 + n_new))


def algorithmic_bytes_per_step(cfg, quantize, B, ctx, tp):
    """SURVEY.md §8d formula, per GPU -> (whole step, attention KV read of one layer, linear weights incl. head)."""
    H, I, V, nl = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers
    d = H // cfg.num_attention_heads
    h, kv = cfg.num_attention_heads, cfg.num_key_value_heads
    mlp_mats = 2 if getattr(cfg, "model_type", "llama") == "gpt_neox" else 3  # h_to_4h, 4h_to_h | gate, up, down
    lin_params = nl * ((h + 2 * kv) * d * H + h * d * H + mlp_mats * I * H)
    if quantize == "gptq":
        w_lin = lin_params * (0.5 + (2 + 0.5) / 128)
    else:
        w_lin = lin_params * 2
    w_head = V * H * 2
    kv_read = B * ctx * nl * 2 * kv * d * 2
    kv_write = B * nl * 2 * kv * d * 2
    logits = B * V * 2
    return (w_lin + w_head + kv_read + kv_write + logits) / tp, kv_read / tp / nl, (w_lin + w_head) / tp


def measure_workload(args, workload, world, rank, full: bool):
    """One workload, the whole L0 -> L1 trajectory.  `full`: also the per-kernel rooflines (eager passes) and prefill detail."""
    import torch
    import torch.distributed as dist

    arch, quantize, B, L0, L1 = WORKLOADS[workload]
    K, W = args.steps, args.warmup
    model, cfg = build_model(workload, world, rank, args.layers)
    from tgis_b200 import _lib
    lib = _lib.load()
    dev = model.device
    n_new = L1 - L0
    mid = (L0 + L1) // 2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    # ---------------------------------------------------------------- prefill (timed once, reported beside the metric)
    batch, errs = model.batch_type.from_pb(make_batch_pb(B, L0, n_new), model.tokenizer, model.dtype, dev, None, None, True)
    assert not errs
    e2e_ms, e2e_steps, e2e_ctx_sum = 0.0, 0, 0.0
    host_ids = torch.empty(B, dtype=torch.int64).pin_memory()
    with torch.inference_mode():
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        toks = model.generate_token(batch, first=True)[0]
        e1.record()
        barrier()
        prefill_ms = max_over_ranks(e0.elapsed_time(e1))
        cur = L0  # tokens cached before the next decode step (that step attends over cur + 1)

        def e2e_segment(n_steps, toks, cur):
            """n_steps decode steps through generate_token with host buffers in the timed region; -> (ms, toks, cur)"""
            if n_steps <= 0:
                return 0.0, toks, cur
            barrier()
            t0 = time.perf_counter()
            e0.record()
            for _ in range(n_steps):
                host_ids.copy_(torch.tensor([t.token_id for t in toks], dtype=torch.int64))
                batch.input_ids.copy_(host_ids, non_blocking=True)      # H2D: this step's input token ids
                toks = model.generate_token(batch)[0]                    # D2H: the chosen ids (one read per step)
            e1.record()
            barrier()
            wall = (time.perf_counter() - t0) * 1e3
            return max_over_ranks(max(e0.elapsed_time(e1), wall)), toks, cur + n_steps

        # ---- e2e, first half of the trajectory (3 untimed steps first: the fused state and its CUDA graph come to exist)
        for _ in range(3):
            toks = model.generate_token(batch)[0]
            cur += 1
        n_eager = K if full else 0
        start_a = mid - (K + n_eager) // 2 - W
        seg_steps = max(0, start_a - cur)
        ctx0 = cur
        ms, toks, cur = e2e_segment(seg_steps, toks, cur)
        e2e_ms += ms
        e2e_steps += seg_steps
        e2e_ctx_sum += seg_steps * (ctx0 + (seg_steps + 1) / 2.0)

        # ---- device-resident window around the mean context: no host round trip inside the timed region
        st = batch._fused
        batch.input_ids.copy_(torch.tensor([t.token_id for t in toks], dtype=torch.int64))

        def device_step(use_graph=True):
            model._run_fused_step(batch, st, use_graph)  # chains the chosen ids into input_ids on the device

        for _ in range(W):
            device_step()
            cur += 1
        attn_ms = gemm_ms = None
        n_attn = n_gemm = 0
        ctx_roof = None
        if full:
            # eager steps carry the per-kernel events (events are not captured into graphs); two kernel families, K/2 steps each
            which_gemm = 2 if quantize == "gptq" else 3  # B200_TIME_GEMM_W4A16 / B200_TIME_GEMM_F16
            halves = [(1, K - K // 2), (which_gemm, K // 2)]
            for which, n_steps in halves:
                timing = lib.b200_timing_create(n_steps * (4 * cfg.num_hidden_layers + 2) + 8)
                lib.b200_timing_attach(timing, which)
                barrier()
                for _ in range(n_steps):
                    device_step(use_graph=False)
                barrier()
                lib.b200_timing_attach(None, 0)
                tot = ctypes.c_float(0)
                n_timed = lib.b200_timing_collect(timing, ctypes.byref(tot))
                if n_timed < 0:
                    raise RuntimeError(lib.b200_last_error().decode())
                lib.b200_timing_destroy(timing)
                if which == 1:
                    attn_ms, n_attn = tot.value / max(n_timed, 1), n_timed
                    ctx_roof = cur + (n_steps + 1) / 2.0
                else:
                    gemm_ms, n_gemm = tot.value / max(n_steps, 1), n_timed  # per step
                cur += n_steps
        # headline pass
        launches0 = lib.b200_launch_count()
        sampler.mark()
        barrier()
        e0.record()
        for _ in range(K):
            device_step()
        e1.record()
        barrier()
        dev_ms = max_over_ranks(e0.elapsed_time(e1))
        clocks = sampler.stop()
        ctx_value = cur + (K + 1) / 2.0
        cur += K
        # the host mirrors of the lengths advance too (generate_token was bypassed for these steps)
        skipped = W + n_eager + K
        for i in range(B):
            batch.input_lengths[i] += skipped
            batch.next_token_chooser.current_tokens[i] += skipped
        batch.max_seqlen += skipped
        # graph replays launch the same kernels as an eager step; count them from one eager step's counter delta
        l0 = lib.b200_launch_count()
        device_step(use_graph=False)
        torch.cuda.synchronize()
        launches_per_step = lib.b200_launch_count() - l0
        cur += 1
        for i in range(B):
            batch.input_lengths[i] += 1
            batch.next_token_chooser.current_tokens[i] += 1
        batch.max_seqlen += 1

        # ---- e2e, second half of the trajectory: up to the last token the requests asked for
        toks = model.generate_token(batch)[0]
        cur += 1
        seg_steps = max(0, (L1 - 1) - cur)
        ctx0 = cur
        ms, toks, cur = e2e_segment(seg_steps, toks, cur)
        e2e_ms += ms
        e2e_steps += seg_steps
        e2e_ctx_sum += seg_steps * (ctx0 + (seg_steps + 1) / 2.0)

    hbm_peak, peak_kind = peaks()
    step_bytes, _, w_bytes = algorithmic_bytes_per_step(cfg, quantize, B, ctx_value, world)
    value = B * K / (dev_ms / 1e3)
    res = {
        "workload": workload, "value": value, "ms_per_step": dev_ms / K, "mean_context_timed": ctx_value,
        "step_roofline": {"algorithmic_bytes_per_step_per_gpu": step_bytes, "hbm_gbs_achieved": step_bytes / (dev_ms / K / 1e3) / 1e9,
                          "frac_of_hbm_peak": step_bytes / (dev_ms / K / 1e3) / 1e9 / hbm_peak, "peak_kind": peak_kind},
        "prefill": {"tokens": B * L0, "ms": prefill_ms, "tokens_per_s": B * L0 / (prefill_ms / 1e3)},
        "e2e": {"value": B * e2e_steps / (e2e_ms / 1e3) if e2e_ms > 0 else None, "unit": UNIT, "h2d_bytes_per_step": B * 8,
                "d2h_bytes_per_step": B * 8, "ms_per_step": e2e_ms / max(e2e_steps, 1), "steps": e2e_steps,
                "mean_context": e2e_ctx_sum / max(e2e_steps, 1), "api": "FlashCausalLM.generate_token",
                "trajectory": f"every decode step {L0}->{L1} outside the {skipped + 5}-step device-timed window"},
        "gpu_launches": int(launches_per_step * K), "launches_per_step": int(launches_per_step), "clocks": clocks,
        "arch": arch, "quantize": quantize, "batch": B, "prompt_len": L0, "end_len": L1, "layers": cfg.num_hidden_layers,
    }
    if full and attn_ms:
        _, attn_bytes_roof, _ = algorithmic_bytes_per_step(cfg, quantize, B, ctx_roof, world)
        achieved = attn_bytes_roof / (attn_ms / 1e3) / 1e9
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "roofline_traffic.json")
        if os.path.exists(tpath):
            try:
                with open(tpath) as f:
                    traffic = json.load(f).get(workload, {}).get("attn_decode_traffic_bytes_per_launch")
            except Exception:
                traffic = None
        res["roofline"] = {"kernel": "attn_decode_paged_kernel", "bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                           "frac": achieved / hbm_peak, "traffic": traffic, "peak_kind": peak_kind,
                           "algorithmic_bytes_per_launch": attn_bytes_roof, "avg_launch_ms": attn_ms, "launches_timed": n_attn,
                           "share_of_step": attn_ms * cfg.num_hidden_layers / (dev_ms / K),
                           "timing": "CUDA events around each eager launch (adds the event gaps: graph-replayed launches are shorter, "
                                     "see profiles/ step traces)"}
        if gemm_ms:
            res["roofline"]["gemm"] = {"kernel": "gemm_w4a16_kernel" if quantize == "gptq" else "gemm_f16_kernel", "bound": "hbm",
                                       "algorithmic_weight_bytes_per_step": w_bytes, "ms_per_step": gemm_ms,
                                       "achieved": w_bytes / (gemm_ms / 1e3) / 1e9, "unit": "GB/s",
                                       "frac": w_bytes / (gemm_ms / 1e3) / 1e9 / hbm_peak, "share_of_step": gemm_ms / (dev_ms / K),
                                       "launches_timed": n_gemm}
    # free everything before the next workload
    del batch, st, model
    gc.collect()
    torch.cuda.empty_cache()
    return res


def run_mixed(args, workload):
    """BASELINE config[4]: continuous batching with add-on prefills, driven through the shard's own Prefill / NextToken messages
    by tools/router_sim.py (the Rust router's loop restated).  Decode-step and prefill throughput are reported separately."""
    import torch
    import torch.distributed as dist

    from tools import router_sim

    world = int(os.getenv("WORLD_SIZE", "1"))
    rank = int(os.getenv("RANK", "0"))
    arch, quantize, max_bs, prompt_range, new_range, n_req, rate = MIXED_WORKLOADS[workload]
    n_req = args.requests or n_req
    max_len = prompt_range[1] + new_range[1]
    WORKLOADS[workload] = (arch, quantize, max_bs, prompt_range[1], max_len)
    blocks = max_bs * ((max_len + 16) // 16 + 1) + 8
    model, cfg = build_model(workload, world, rank, args.layers, blocks=blocks)
    from tgis_b200 import _lib, pb
    from tgis_b200.server import Cache, TextGenerationService
    lib = _lib.load()
    service = TextGenerationService(model, Cache(), ["unix:///dev/null"])
    requests = router_sim.make_requests(n_req, rate, prompt_range, new_range, cfg.vocab_size, seed=0, filler=3)  # "test " * L
    budget = max_bs * max_len
    bytes_acc = {"decode": 0.0}
    H, I, V, nl = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers
    d = H // cfg.num_attention_heads

    def on_step(bs, ctx_sum):
        step_bytes, _, _ = algorithmic_bytes_per_step(cfg, quantize, 1, 0, world)        # weights + head (+ 1 row of logits)
        kv = (ctx_sum + bs) * nl * 2 * cfg.num_key_value_heads * d * 2 / world              # KV read of every context (+ the new token)
        bytes_acc["decode"] += step_bytes + kv + (bs - 1) * V * 2 / world

    def sync():
        torch.cuda.synchronize()

    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    l0 = lib.b200_launch_count()
    if world > 1:
        dist.barrier()
    sampler.mark()
    def agree(dt):
        """every rank advances the session clock by the slowest rank's time: identical admission decisions on all shards"""
        if world == 1:
            return dt
        t = torch.tensor([dt], dtype=torch.float64, device=model.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    with torch.inference_mode():
        out = router_sim.run_session(service, pb, requests, max_bs, lambda p: "test " * len(p), max_batch_tokens=budget, sync=sync,
                                     on_decode_step=on_step, agree=agree)
    clocks = sampler.stop()
    st = out["stats"]
    launches = lib.b200_launch_count() - l0
    hbm_peak, peak_kind = peaks()

    def maxr(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=model.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    decode_s, prefill_s = maxr(st["decode_s"]), maxr(st["prefill_s"])
    value = st["decode_tokens"] / decode_s
    assert all(len(out["tokens"][r.id]) == r.max_new for r in requests), "a request did not receive all its tokens"
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": st["decode_steps"], "warmup": 0,
        "ms_per_step": decode_s / max(st["decode_steps"], 1) * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16" if quantize is None else "int4 weights x f16 activations, f32 accumulate", "data": "synthetic",
        "config": {"workload": workload, "arch": arch, "quantize": quantize, "max_batch": max_bs, "prompt_len": list(prompt_range),
                   "new_tokens": list(new_range), "requests": n_req, "poisson_arrivals_per_s": rate, "seed": 0, "kv_block": 16,
                   "parallelism": f"tp{world}", "layers": cfg.num_hidden_layers,
                   "driver": "tools/router_sim.py: add-on Prefill (to_prune) + NextToken over every cached batch id, as router/src/batcher.rs",
                   "timing": "wall clock around each RPC, device synchronised on both sides (host bookkeeping of prune / concatenate included)"},
        "tokens_per_s_per_gpu": value / world,
        "decode": {"tokens": st["decode_tokens"], "seconds": decode_s, "steps": st["decode_steps"],
                   "mean_batch": st["batch_size_sum"] / max(st["decode_steps"], 1), "max_batch": st["max_batch"],
                   "steps_after_a_concatenate": st["concat_steps"]},
        "prefill": {"tokens": st["prefill_tokens"], "ms": prefill_s * 1e3, "calls": st["prefill_calls"],
                    "tokens_per_s": st["prefill_tokens"] / prefill_s if prefill_s > 0 else None},
        "step_roofline": {"algorithmic_bytes_per_gpu_all_decode_steps": bytes_acc["decode"],
                          "hbm_gbs_achieved": bytes_acc["decode"] / decode_s / 1e9,
                          "frac_of_hbm_peak": bytes_acc["decode"] / decode_s / 1e9 / hbm_peak, "peak_kind": peak_kind},
        "e2e": {"value": (st["decode_tokens"] + st["prefill_calls"]) / (decode_s + prefill_s), "unit": UNIT,
                "note": "generated tokens / (prefill + decode time): the session as the router sees it, host buffers in and out of every RPC",
                "h2d_bytes_per_step": None, "d2h_bytes_per_step": None},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.cuda.synchronize()
        sys.stdout.flush()
        try:
            store = dist.distributed_c10d._get_default_store()
            store.add("bench_done", 1)
            t_end = time.time() + 30
            while int(store.add("bench_done", 0)) < world and time.time() < t_end:
                time.sleep(0.05)
        except Exception:
            time.sleep(1.0)
        os._exit(0)
    return 0


def self_check(arch: str, quantize):
    """2 layers of the workload's widths (small vocabulary), ragged prompts, greedy decode through from_pb / generate_token
    (prefill, eager steps, the CUDA-graph-replayed fused step) vs the CPU oracle; exact outside the 2-ulp tie band."""
    import tempfile

    import torch
    from safetensors.torch import save_file

    from oracle import llama as oll  # checker only
    from tgis_b200 import pb
    from tgis_b200.inference_engine import InferenceEngine
    from tgis_b200.models.flash_causal_lm import FlashCausalLM
    from tgis_b200.utils.dist import FakeGroup
    from tgis_b200.utils.synthetic import ARCHS, llama_config, make_tokenizer
    from tgis_b200.utils.weights import Weights

    H, I, _, h, kv, _ = ARCHS[arch]
    cfg = llama_config(arch, quantize=quantize, max_position_embeddings=512, num_layers=2)
    cfg.vocab_size = 4096
    ocfg = oll.LlamaConfig(H, I, 2, h, kv, cfg.vocab_size, cfg.rms_norm_eps, cfg.rope_theta)
    sd = oll.make_state_dict(ocfg, seed=11, quantize=quantize, std=0.02)
    dev = "cuda:0"
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "model.safetensors")
        save_file({k: v.contiguous() for k, v in sd.items()}, path)
        weights = Weights([path], device=dev, dtype=torch.float16, process_group=FakeGroup(0, 1))
        tok = make_tokenizer(cfg.vocab_size)
        engine = InferenceEngine(tmp, None, torch.float16, quantize, cfg, 512, weights=weights, tokenizer=tok)
        model = FlashCausalLM(tmp, None, "tgis_native", torch.float16, quantize, cfg, engine=engine, num_kv_blocks=128)
    g = torch.Generator().manual_seed(0)
    lens = (40, 64, 17, 33, 48, 5, 64, 21)
    prompts = [torch.randint(4, cfg.vocab_size, (L,), generator=g).tolist() for L in lens]
    n_new = 8
    reqs = [pb.Request(id=i, inputs=" ".join(f"<tok{t}>" for t in p), input_length=len(p), max_output_length=n_new,
                       parameters=pb.NextTokenChooserParameters(temperature=0.0, top_p=1.0, min_new_tokens=n_new))
            for i, p in enumerate(prompts)]
    got = [[] for _ in prompts]
    with torch.inference_mode():
        batch, errs = model.batch_type.from_pb(pb.Batch(id=0, requests=reqs), tok, torch.float16, model.device, None, None, True)
        assert not errs
        out = model.generate_token(batch, first=True)
        for _ in range(n_new - 1):
            for t in out[0]:
                got[t.request_id].append(t.token_id)
            out = model.generate_token(batch)
        for t in out[0]:
            got[t.request_id].append(t.token_id)
    torch.cuda.synchronize()
    oracle = oll.LlamaOracle(oll.build_shards(ocfg, sd, 1))
    ref, ref_logits = oracle.generate_greedy(prompts, n_new, banned_token=cfg.eos_token_id)
    checked = mismatches = ties = 0
    for b in range(len(prompts)):
        for step in range(n_new):
            lg = ref_logits[step][b].float().clone()
            lg[cfg.eos_token_id] = float("-inf")
            top2 = lg.topk(2).values
            if float(top2[0] - top2[1]) <= 2 * max(abs(float(top2[0])), 1.0) * 2.0 ** -10:
                ties += 1
                break  # after a tie the continuations may legitimately differ
            checked += 1
            if got[b][step] != int(ref[b, step]):
                mismatches += 1
                break
    del model, batch
    gc.collect()
    torch.cuda.empty_cache()
    return {"model": f"{arch} widths, 2 layers, vocab 4096, {quantize or 'fp16'}", "sequences": len(prompts), "new_tokens": n_new,
            "tokens_checked": checked, "ties_skipped": ties, "mismatches_outside_tie_band": mismatches,
            "steps_through_cuda_graph": max(0, n_new - 1 - 2)}


def run_gpu(args, workload):
    import torch
    import torch.distributed as dist

    world = int(os.getenv("WORLD_SIZE", "1"))
    rank = int(os.getenv("RANK", "0"))
    main = measure_workload(args, workload, world, rank, full=True)
    arch, quantize, B, L0, L1 = WORKLOADS[workload]
    line = {
        "metric": METRIC, "value": main["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16" if quantize is None else "int4 weights x f16 activations, f32 accumulate", "data": "synthetic",
        "config": {"workload": workload, "arch": arch, "quantize": quantize, "batch": B, "prompt_len": L0, "end_len": L1,
                   "mean_context_timed": main["mean_context_timed"], "kv_block": 16, "parallelism": f"tp{world}",
                   "l2_policy": "inputs larger than L2 (KV + weights per step >> 126 MB)", "layers": main["layers"]},
        "tokens_per_s_per_gpu": main["value"] / world,
        "step_roofline": main["step_roofline"], "prefill": main["prefill"], "e2e": main["e2e"],
        "gpu_launches": main["gpu_launches"], "clocks": main["clocks"],
    }
    if "roofline" in main:
        line["roofline"] = main["roofline"]
    extra = {}
    if not args.no_extra and args.workload is None:
        other = "llama2-7b-gptq" if world == 1 else "llama2-7b-fp16"  # BASELINE config[2] / config[3]
        try:
            r = measure_workload(args, other, world, rank, full=False)
            extra[other] = {k: r[k] for k in ("value", "ms_per_step", "mean_context_timed", "step_roofline", "prefill", "e2e", "clocks",
                                              "launches_per_step", "arch", "quantize", "batch", "prompt_len", "end_len")}
            extra[other]["parallelism"] = f"tp{world}"
        except Exception as e:  # noqa: BLE001
            extra[other] = {"failed": f"{type(e).__name__}: {e}"}
    if rank == 0:
        from tgis_b200.utils.synthetic import ARCHS as LLAMA_ARCHS
        llama_family = arch in LLAMA_ARCHS  # the self-check and the CPU arm restate the Llama graph
        if world == 1 and not args.no_extra and llama_family:
            try:
                line["self_check"] = self_check(arch, quantize)
            except Exception as e:  # noqa: BLE001
                line["self_check"] = {"failed": f"{type(e).__name__}: {e}"}
        if not args.no_cpu_baseline and world == 1 and llama_family:
            try:
                r = cpu_reference_decode(arch, B, (L0 + L1) // 2, max(2, min(4, args.steps)), 1, args.cpu_layers)
                line["cpu_baseline"] = {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port", "sample": r["sample"]}
            except Exception as e:  # noqa: BLE001
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                                        "sample": f"failed: {type(e).__name__}: {e}"}
        if extra:
            line["extra"] = extra
        print(json.dumps(line), flush=True)
    if world > 1:
        # collectives live inside the captured CUDA graphs: tearing the communicator down while they exist can hang, so
        # rendezvous on the host-side store instead of an NCCL barrier, then leave without destroy_process_group()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        try:
            store = dist.distributed_c10d._get_default_store()
            store.add("bench_done", 1)
            t_end = time.time() + 30
            while int(store.add("bench_done", 0)) < world and time.time() < t_end:
                time.sleep(0.05)
        except Exception:
            time.sleep(1.0)
        os._exit(0)
    return 0


# ------------------------------------------------------------------------------------------------ --hybrid-compare
def _timed_ops(module, names, log):
    """wraps module-level op functions with a CUDA-event pair per call; log gets (name, start, end) triples"""
    import torch
    saved = {}
    for n in names:
        fn = getattr(module, n)
        saved[n] = fn

        def wrapped(*a, __fn=fn, __n=n, **k):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = __fn(*a, **k)
            e1.record()
            log.append((__n, e0, e1))
            return out
        setattr(module, n, wrapped)
    return saved


def _by_op(log):
    import torch
    torch.cuda.synchronize()
    out = {}
    for n, e0, e1 in log:
        out[n] = out.get(n, 0.0) + e0.elapsed_time(e1)
    return out


def _traced_decode_step(model, batch, lib):
    """device time of every kernel of one fused decode step: the step is captured in a graph of its own with a time stamp after
    every launch of the library (host latency is out of the picture, L2 as in the served step).  -> ({kernel: us}, total us)"""
    import re
    import torch
    cap = 4096
    buf = torch.zeros(cap, dtype=torch.int64, device=model.device)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        lib.b200_debug_step_trace(buf.data_ptr(), cap)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            lib.b200_debug_step_trace_begin(torch.cuda.current_stream().cuda_stream)
            model._run_fused_step(batch, batch._fused, False)
        names_buf = ctypes.create_string_buffer(1 << 20)
        n = lib.b200_debug_step_trace_names(names_buf, len(names_buf))
        lib.b200_debug_step_trace(None, 0)
        for _ in range(3):
            g.replay()
        side.synchronize()
    torch.cuda.current_stream().wait_stream(side)
    names = names_buf.value.decode().strip().split("\n")
    t = buf[:n].cpu().tolist()
    out = {}
    for i in range(1, n):
        k = re.sub(r"<.*", "", names[i].replace("b200::", "").replace("seq::", "").strip("()"))
        out[k] = out.get(k, 0.0) + (t[i] - t[i - 1]) / 1e3
    return out, (t[n - 1] - t[0]) / 1e3


def _neox_partner(width, PB, PL, DB, DL, K, Wm, timed, hbm, tens, ctx):
    """GPT-NeoX (fp16, parallel residual, paged attention) with three layers at `width`, measured like the fp32-stream families:
    the equal-size partner of --hybrid-compare and --dubesun-compare"""
    import torch
    from tgis_b200 import ops as ops_f16
    wl = f"neox-w{width}"
    nmodel, ncfg = build_model(wl, 1, 0, blocks=(DB + PB) * ((DL + 96) // 16 + 2))
    tok = nmodel.tokenizer
    names16 = ["gemm_f16", "layernorm_residual", "rope_kv_write_paged", "attn_prefill_varlen", "attn_decode_paged", "gelu", "embedding",
               "argmax"]

    def nprefill(B, L, n_new, keep=False):
        batch, _ = nmodel.batch_type.from_pb(make_batch_pb(B, L, n_new), tok, torch.float16, nmodel.device, None, None, True)
        nmodel.generate_token(batch, first=True)
        if keep:
            return batch
        nmodel.kv_cache_manager.free_sequences(batch.sequence_ids)
    with torch.inference_mode():
        for _ in range(Wm):
            nprefill(PB, PL, 2)
        npre_ms = timed(lambda: nprefill(PB, PL, 2), K)
        log = []
        saved = _timed_ops(ops_f16, names16, log)
        nprefill(PB, PL, 2)
        npre_ops = _by_op(log)
        for n, fn in saved.items():
            setattr(ops_f16, n, fn)
        os.environ["B200_PY_FUSED_STEP"] = "0"  # op by op, as the hybrid model runs: like is compared with like
        batch = nprefill(DB, DL, Wm + K + 8, keep=True)
        for _ in range(Wm):
            nmodel.generate_token(batch)
        ndec_ms = timed(lambda: nmodel.generate_token(batch), K)
        log = []
        saved = _timed_ops(ops_f16, names16, log)
        nmodel.generate_token(batch)
        ndec_ops = _by_op(log)
        for n, fn in saved.items():
            setattr(ops_f16, n, fn)
        os.environ.pop("B200_PY_FUSED_STEP", None)
        nmodel.kv_cache_manager.free_sequences(batch.sequence_ids)
        batch = nprefill(DB, DL, Wm + K + 8, keep=True)  # and as served: the graph-replayed step
        for _ in range(Wm):
            nmodel.generate_token(batch)
        ngraph_ms = timed(lambda: nmodel.generate_token(batch), K)
        from tgis_b200 import _lib as _libmod
        ndec_k, ndec_total = _traced_decode_step(nmodel, batch, _libmod.load())
        nmodel.kv_cache_manager.free_sequences(batch.sequence_ids)
    hd, nh = 128, width // 128
    nattn_flops = PB * 4 * (PL * PL // 2) * hd * nh
    nlin_w = 3 * (4 * width * width + 2 * width * 4 * width) + ncfg.vocab_size * width
    nkernels = {
        "attn_prefill_varlen": {"ms": npre_ops.get("attn_prefill_varlen", 0.0),
                                "of_measured_tensor": nattn_flops / (max(npre_ops.get("attn_prefill_varlen", 0.0), 1e-9) * 1e-3) / tens},
        "attn_decode_paged": {"us": ndec_k.get("attn_decode_paged_kernel", 0.0) + ndec_k.get("attn_decode_combine_kernel", 0.0), "of_measured_hbm":
                              3 * DB * ctx * 2 * nh * hd * 2
                              / ((ndec_k.get("attn_decode_paged_kernel", 1e-9) + ndec_k.get("attn_decode_combine_kernel", 0.0)) * 1e-6) / hbm},
        "gemm_f16 prefill (all projections)": {"ms": npre_ops["gemm_f16"], "of_measured_tensor":
                                               (2 * PB * PL * (nlin_w - ncfg.vocab_size * width) + 2 * PB * ncfg.vocab_size * width)
                                               / (npre_ops["gemm_f16"] * 1e-3) / tens},
        "gemm_f16 decode (all projections)": {"us": ndec_k["gemm_f16_kernel"], "of_measured_hbm": nlin_w * 2 / (ndec_k["gemm_f16_kernel"] * 1e-6) / hbm},
    }
    result = ({"model": wl, "dtype": "fp16", "layers": 3, "prefill_tokens_per_s": PB * PL / (npre_ms * 1e-3),
                    "decode_tokens_per_s": DB / (ndec_ms * 1e-3), "prefill_ms": npre_ms, "decode_ms_per_step": ndec_ms,
                    "decode_mode": "op by op (B200_PY_FUSED_STEP=0)",
                    "decode_graph_tokens_per_s": DB / (ngraph_ms * 1e-3), "decode_graph_ms_per_step": ngraph_ms,
                    "prefill_ms_by_op": {k: round(v, 4) for k, v in npre_ops.items()},
                    "decode_ms_by_op": {k: round(v, 4) for k, v in ndec_ops.items()},
                    "decode_graph_us_by_kernel": {k: round(v, 2) for k, v in sorted(ndec_k.items(), key=lambda kv: -kv[1])},
                    "decode_graph_traced_us": ndec_total, "kernels": nkernels})
    del nmodel
    gc.collect()
    torch.cuda.empty_cache()
    return result


def run_hybrid_compare(args):
    """Fetotar (bfloat16) beside GPT-NeoX (fp16) at equal width and depth, random weights: prefill of 4 x 1024 tokens and decode of
    32 sequences at context 1024.  Per model: tokens/s through the engine's own step (device time by CUDA events, L2 flushed
    between timed calls) and the device time of every kernel family inside one step; for the kernels that carry a step, achieved
    FLOP/s or bytes/s against the measured peaks."""
    import torch
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops as ops_f16, ops_seq
    from tgis_b200.inference_engine import InferenceEngine
    from tgis_b200.models.custom_modeling.fetotar_modeling import FetotarConfig
    from tgis_b200.models.flash_causal_lm import FlashCausalLM
    from tgis_b200.utils.dist import FakeGroup
    from tgis_b200.utils.synthetic import SyntheticHybridWeights, fetotar_config, make_tokenizer

    pk = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")):
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        pk = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    hbm, tens = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    PB, PL, DB, DL = 4, 1024, 32, 1024
    K, Wm = max(args.steps // 4, 4), args.warmup
    results = []

    def timed(fn, n):
        total = 0.0
        for _ in range(n):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / n

    for width in (2048, 4096):
        # ---------------------------------------------------------------- the hybrid model
        raw = fetotar_config(f"fetotar-w{width}")
        cfg = FetotarConfig(raw)
        weights = SyntheticHybridWeights(raw, dev, torch.bfloat16, FakeGroup(0, 1))
        engine = InferenceEngine("<synthetic>", None, torch.bfloat16, None, cfg, None, weights=weights, tokenizer=make_tokenizer(cfg.vocab_size))
        model = FlashCausalLM("<synthetic>", None, "tgis_native", torch.bfloat16, None, cfg, engine=engine,
                              num_kv_blocks=(DB + PB) * ((DL + 64) // 16 + 2), num_state_slots=DB + PB)
        g = torch.Generator().manual_seed(0)
        prompt = lambda n, L: [torch.randint(4, cfg.vocab_size, (L,), generator=g).tolist() for _ in range(n)]  # noqa: E731

        def prefill_once():
            sids, _ = model.step_ragged([None] * PB, prompts_p, [PL * (i + 1) - 1 for i in range(PB)])
            model.kv_cache_manager.free_sequences(sids)
        prompts_p = prompt(PB, PL)
        for _ in range(Wm):
            prefill_once()
        pre_ms = timed(prefill_once, K)
        names = [n for n in ("linear", "linear_per_head", "embed_scale", "layernorm", "layernorm_into_residual", "group_rmsnorm_gate",
                             "ff_clamped_gate", "token_side", "latent_prepare", "latent_attn", "causal_conv_silu", "ssm_scan", "mlstm_scan")]
        log = []
        saved = _timed_ops(ops_seq, names, log)
        prefill_once()
        pre_ops = _by_op(log)
        sids, _ = model.step_ragged([None] * DB, prompt(DB, DL), [])
        nxt = [[7]] * DB

        def decode_once():
            model.step_ragged(sids, nxt, None)
        log.clear()
        for n, fn in saved.items():
            setattr(ops_seq, n, fn)
        for _ in range(Wm):
            decode_once()
        dec_ms = timed(decode_once, K)
        saved = _timed_ops(ops_seq, names, log)
        decode_once()
        dec_ops = _by_op(log)
        for n, fn in saved.items():
            setattr(ops_seq, n, fn)
        model.kv_cache_manager.free_sequences(sids)
        # the serving path: from_pb -> generate_token, plain greedy, replayed as one CUDA graph from the third step of the batch
        with torch.inference_mode():
            gbatch, _ = model.batch_type.from_pb(make_batch_pb(DB, DL, Wm + K + 8), model.tokenizer, torch.bfloat16, model.device, None, None, True)
            model.generate_token(gbatch, first=True)
            for _ in range(Wm):
                model.generate_token(gbatch)
            graph_ms = timed(lambda: model.generate_token(gbatch), K)
            from tgis_b200 import _lib as _libmod
            dec_k, dec_total = _traced_decode_step(model, gbatch, _libmod.load_seq())
            model.kv_cache_manager.free_sequences(gbatch.sequence_ids)
        la, ss, ml = raw["layers"][1]["mixer"], raw["layers"][2]["mixer"], raw["layers"][0]["mixer"]
        D, R, H = la["kv_rank"] + la["rot_dim"], la["kv_rank"], la["heads"]
        attn_flops = PB * (PL * (PL + 1) // 2) * H * (D + R) * 2
        ctx = DL + Wm + K + 2
        kernels = {
            "latent_attn prefill": {"ms": pre_ops["latent_attn"], "tflops": attn_flops / pre_ops["latent_attn"] / 1e9,
                                    "of_measured_tensor": attn_flops / (pre_ops["latent_attn"] * 1e-3) / tens},
            "latent_attn decode": {"us": dec_k.get("latent_attn_mma_kernel", 0.0) + dec_k.get("latent_attn_merge_kernel", 0.0), "of_measured_hbm":
                                   DB * ctx * D * 2 / ((dec_k.get("latent_attn_mma_kernel", 0.0) + dec_k.get("latent_attn_merge_kernel", 0.0)) * 1e-6) / hbm},
            "ssm_scan decode": {"us": dec_k["ssm_scan_kernel"], "of_measured_hbm":
                                DB * ss["heads"] * ss["state"] * ss["vdim"] * 8 / (dec_k["ssm_scan_kernel"] * 1e-6) / hbm},
            "mlstm_scan decode": {"us": dec_k["mlstm_scan_kernel"], "of_measured_hbm":
                                  DB * ml["heads"] * ml["dim"] * ml["vdim"] * 8 / (dec_k["mlstm_scan_kernel"] * 1e-6) / hbm},
            "ssm_scan prefill": {"ms": pre_ops["ssm_scan"], "tokens_per_s": PB * PL / (pre_ops["ssm_scan"] * 1e-3)},
            "mlstm_scan prefill": {"ms": pre_ops["mlstm_scan"], "tokens_per_s": PB * PL / (pre_ops["mlstm_scan"] * 1e-3)},
        }
        from tgis_b200.models.custom_modeling.fetotar_modeling import tensor_shapes
        shapes = tensor_shapes(raw)
        lin_w = sum(a * b for n, (a, *rest) in shapes.items() for b in rest[:1]
                    if n.split(".")[-1] in ("in", "o", "q", "k", "v", "g", "i", "f", "dq", "uq", "dkv", "gate", "up", "down", "head")
                    and not n.startswith("side") and ".side." not in n)
        lin_flops = 2 * PB * PL * (lin_w - shapes["head"][0] * shapes["head"][1]) + 2 * PB * shapes["head"][0] * shapes["head"][1]
        kernels["linear prefill (all projections)"] = {"ms": pre_ops["linear"], "of_measured_tensor": lin_flops / (pre_ops["linear"] * 1e-3) / tens}
        kernels["linear decode (tcgen05 projections)"] = {"us": dec_k["gemm_f16_kernel"], "of_measured_hbm": lin_w * 2 / (dec_k["gemm_f16_kernel"] * 1e-6) / hbm}
        results.append({"model": f"fetotar-w{width}", "dtype": "bf16", "layers": 3, "prefill_tokens_per_s": PB * PL / (pre_ms * 1e-3),
                        "decode_tokens_per_s": DB / (dec_ms * 1e-3), "prefill_ms": pre_ms, "decode_ms_per_step": dec_ms,
                        "decode_graph_tokens_per_s": DB / (graph_ms * 1e-3), "decode_graph_ms_per_step": graph_ms,
                        "prefill_ms_by_op": {k: round(v, 4) for k, v in pre_ops.items()},
                        "decode_ms_by_op": {k: round(v, 4) for k, v in dec_ops.items()},
                        "decode_graph_us_by_kernel": {k: round(v, 2) for k, v in sorted(dec_k.items(), key=lambda kv: -kv[1])},
                        "decode_graph_traced_us": dec_total, "kernels": kernels})
        del model, engine, weights
        gc.collect()
        torch.cuda.empty_cache()

        results.append(_neox_partner(width, PB, PL, DB, DL, K, Wm, timed, hbm, tens, ctx))
    kernels["latent_attn decode"]["note"] = "3 attention layers in the partner vs 1 latent-attention layer here: compare fractions, not ms"
    print(json.dumps({"metric": "hybrid_compare", "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": Wm, "data": "synthetic",
                      "config": {"prefill": [PB, PL], "decode": [DB, DL], "l2": "flushed between timed calls"},
                      "peaks": {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": pk.get("source")}, "models": results}))
    return 0


def run_dubesun_compare(args):
    """Dubesun (bfloat16) beside GPT-NeoX (fp16) at equal width and depth, random weights: prefill of 4 x 1024 tokens and decode of
    32 sequences at context 1024, measured as --hybrid-compare measures its pair: tokens/s through the engine's own step (device
    time by CUDA events, L2 flushed between timed calls), device time per op family and per kernel of the graph-replayed decode
    step, and for the kernels that carry a step the achieved FLOP/s or bytes/s against the measured peaks."""
    import torch
    import tgis_b200  # noqa: F401
    from tgis_b200 import _lib as _libmod, ops_seq
    from tgis_b200.inference_engine import InferenceEngine
    from tgis_b200.models.custom_modeling.dubesun_modeling import DubesunConfig, tensor_shapes
    from tgis_b200.models.flash_causal_lm import FlashCausalLM
    from tgis_b200.utils.dist import FakeGroup
    from tgis_b200.utils.synthetic import SyntheticHybridWeights, dubesun_config, make_tokenizer

    pk = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")):
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        pk = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    hbm, tens = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    PB, PL, DB, DL = 4, 1024, 32, 1024
    K, Wm = max(args.steps // 4, 4), args.warmup
    ctx = DL + Wm + K + 2
    results = []

    def timed(fn, n):
        total = 0.0
        for _ in range(n):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / n

    widths = (2048, 4096) if not args.layers else (2048,)
    for width in widths:
        raw = dubesun_config(f"dubesun-w{width}")
        cfg = DubesunConfig(raw)
        weights = SyntheticHybridWeights(raw, dev, torch.bfloat16, FakeGroup(0, 1))
        engine = InferenceEngine("<synthetic>", None, torch.bfloat16, None, cfg, None, weights=weights, tokenizer=make_tokenizer(cfg.vocab_size))
        model = FlashCausalLM("<synthetic>", None, "tgis_native", torch.bfloat16, None, cfg, engine=engine,
                              num_kv_blocks=(DB + PB) * ((DL + 64) // 16 + 2), num_state_slots=DB + PB)
        g = torch.Generator().manual_seed(0)
        prompt = lambda n, L: [torch.randint(4, cfg.vocab_size, (L,), generator=g).tolist() for _ in range(n)]  # noqa: E731
        prompts_p = prompt(PB, PL)

        def prefill_once():
            sids, _ = model.step_ragged([None] * PB, prompts_p, [PL * (i + 1) - 1 for i in range(PB)])
            model.kv_cache_manager.free_sequences(sids)
        for _ in range(Wm):
            prefill_once()
        pre_ms = timed(prefill_once, K)
        names = ["linear", "embed_add_pos", "rmsnorm_rows", "causal_conv", "heads_prepare", "paged_attn", "diff_combine", "group_rmsnorm_gate",
                 "moe_route", "moe_gather_rows", "moe_linear", "ff_clamped_gate", "moe_combine_add"]
        log = []
        saved = _timed_ops(ops_seq, names, log)
        prefill_once()
        pre_ops = _by_op(log)
        for n, fn in saved.items():
            setattr(ops_seq, n, fn)
        sids, _ = model.step_ragged([None] * DB, prompt(DB, DL), [])
        nxt = [[t[0]] for t in prompt(DB, 1)]   # a different token per sequence: the routing of the first layer sees only the token

        def decode_once():
            model.step_ragged(sids, nxt, None)
        for _ in range(Wm):
            decode_once()
        dec_ms = timed(decode_once, K)
        log, routes = [], []
        route = ops_seq.moe_route
        ops_seq.moe_route = lambda *a, **k: (routes.append(route(*a, **k)), routes[-1])[1]
        saved = _timed_ops(ops_seq, names, log)
        decode_once()
        dec_ops = _by_op(log)
        for n, fn in saved.items():
            setattr(ops_seq, n, fn)
        ops_seq.moe_route = route
        picked = sum(len(set(r.ids.flatten().tolist())) for r in routes)   # experts whose weights a decode step reads, all layers
        model.kv_cache_manager.free_sequences(sids)
        # the serving path: from_pb -> generate_token, plain greedy, replayed as one CUDA graph from the third step of the batch
        with torch.inference_mode():
            gpb = make_batch_pb(DB, DL, Wm + K + 8)
            for r, toks in zip(gpb.requests, prompt(DB, DL)):   # a prompt of its own per request: the routing differs between them
                r.inputs = " ".join(f"<tok{t}>" for t in toks)
            gbatch, _ = model.batch_type.from_pb(gpb, model.tokenizer, torch.bfloat16, model.device, None, None, True)
            model.generate_token(gbatch, first=True)
            for _ in range(Wm):
                model.generate_token(gbatch)
            graph_ms = timed(lambda: model.generate_token(gbatch), K)
            dec_k, dec_total = _traced_decode_step(model, gbatch, _libmod.load_seq())
            model.kv_cache_manager.free_sequences(gbatch.sequence_ids)
        shapes = tensor_shapes(raw)
        attn_flops, attn_rows = 0, 0
        for layer in raw["layers"]:
            m = layer["mixer"]
            maps = 2 if layer["type"] == "attention" else 1
            attn_flops += PB * (PL * (PL + 1) // 2) * m["heads"] * maps * (m["dim"] + m["vdim"]) * 2
            attn_rows += m["kv_heads"] * (maps * m["dim"] + m["vdim"])   # elements a decoding token reads per cached token
        f = raw["layers"][0]["mlp"]
        E, top, ff = f["router"]["experts"], f["router"]["top"], f["expert"]["ff"]
        L = len(raw["layers"])
        proj_w = sum(a * b for n, (a, *rest) in shapes.items() for b in rest[:1]
                     if n.split(".")[-1] in ("q", "k", "v", "g", "o", "router") and ".mlp.e" not in n)
        head_w = shapes["head"][0] * shapes["head"][1]
        expert_w = 3 * width * ff
        lin_flops = 2 * PB * PL * (proj_w + L * top * expert_w) + 2 * PB * head_w
        attn_us = sum(v for k, v in dec_k.items() if k.startswith("paged_heads_attn"))   # the attention kernel of the step and its merge
        moe_us = dec_k.get("moe_linear_mma_kernel", 0.0)
        kernels = {
            "paged_attn prefill (3 layers)": {"ms": pre_ops["paged_attn"], "tflops": attn_flops / pre_ops["paged_attn"] / 1e9,
                                              "of_measured_tensor": attn_flops / (pre_ops["paged_attn"] * 1e-3) / tens},
            "paged_attn decode (3 layers)": {"us": attn_us, "of_measured_hbm": DB * ctx * attn_rows * 2 / (max(attn_us, 1e-9) * 1e-6) / hbm},
            "linear prefill (projections + one product per expert)": {"ms": pre_ops["linear"], "of_measured_tensor": lin_flops / (pre_ops["linear"] * 1e-3) / tens},
            "moe_linear decode (grouped, picked experts' weights once)": {"us": moe_us, "experts_picked_all_layers": picked, "of_measured_hbm":
                                                                          picked * expert_w * 2 / (max(moe_us, 1e-9) * 1e-6) / hbm},
            "linear decode (tcgen05 projections)": {"us": dec_k.get("gemm_f16_kernel", 0.0), "of_measured_hbm":
                                                    (proj_w + head_w) * 2 / (max(dec_k.get("gemm_f16_kernel", 0.0), 1e-9) * 1e-6) / hbm},
        }
        results.append({"model": f"dubesun-w{width}", "dtype": "bf16", "layers": L, "experts": E, "top": top,
                        "prefill_tokens_per_s": PB * PL / (pre_ms * 1e-3), "decode_tokens_per_s": DB / (dec_ms * 1e-3), "prefill_ms": pre_ms,
                        "decode_ms_per_step": dec_ms, "decode_graph_tokens_per_s": DB / (graph_ms * 1e-3), "decode_graph_ms_per_step": graph_ms,
                        "prefill_ms_by_op": {k: round(v, 4) for k, v in pre_ops.items()},
                        "decode_ms_by_op": {k: round(v, 4) for k, v in dec_ops.items()},
                        "decode_graph_us_by_kernel": {k: round(v, 2) for k, v in sorted(dec_k.items(), key=lambda kv: -kv[1])},
                        "decode_graph_traced_us": dec_total, "kernels": kernels})
        del model, engine, weights
        gc.collect()
        torch.cuda.empty_cache()
        results.append(_neox_partner(width, PB, PL, DB, DL, K, Wm, timed, hbm, tens, ctx))
    print(json.dumps({"metric": "dubesun_compare", "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": Wm, "data": "synthetic",
                      "config": {"prefill": [PB, PL], "decode": [DB, DL], "l2": "flushed between timed calls"},
                      "peaks": {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": pk.get("source")}, "models": results}))
    return 0


def _stream_family_measure(raw, cfg, op_names, PB, PL, DB, DL, K, Wm, timed, lib):
    """one fp32-stream family through the engine: prefill PB x PL and decode DB sequences at context DL, as --dubesun-compare measures
    them -> dict of timings (ms per call, per op family, per kernel of the graph-replayed decode step) and the decode step's routings"""
    import torch
    from tgis_b200 import ops_seq
    from tgis_b200.inference_engine import InferenceEngine
    from tgis_b200.models.flash_causal_lm import FlashCausalLM
    from tgis_b200.utils.dist import FakeGroup
    from tgis_b200.utils.synthetic import SyntheticHybridWeights, make_tokenizer
    dev = torch.device("cuda", 0)
    weights = SyntheticHybridWeights(raw, dev, torch.bfloat16, FakeGroup(0, 1))
    engine = InferenceEngine("<synthetic>", None, torch.bfloat16, None, cfg, None, weights=weights, tokenizer=make_tokenizer(cfg.vocab_size))
    model = FlashCausalLM("<synthetic>", None, "tgis_native", torch.bfloat16, None, cfg, engine=engine,
                          num_kv_blocks=(DB + PB) * ((DL + 64) // 16 + 2), num_state_slots=DB + PB)
    g = torch.Generator().manual_seed(0)
    prompt = lambda n, L: [torch.randint(4, cfg.vocab_size, (L,), generator=g).tolist() for _ in range(n)]  # noqa: E731
    prompts_p = prompt(PB, PL)

    def prefill_once():
        sids, _ = model.step_ragged([None] * PB, prompts_p, [PL * (i + 1) - 1 for i in range(PB)])
        model.kv_cache_manager.free_sequences(sids)
    for _ in range(Wm):
        prefill_once()
    pre_ms = timed(prefill_once, K)
    log = []
    saved = _timed_ops(ops_seq, op_names, log)
    prefill_once()
    pre_ops = _by_op(log)
    for n, fn in saved.items():
        setattr(ops_seq, n, fn)
    sids, _ = model.step_ragged([None] * DB, prompt(DB, DL), [])
    nxt = [[t[0]] for t in prompt(DB, 1)]

    def decode_once():
        model.step_ragged(sids, nxt, None)
    for _ in range(Wm):
        decode_once()
    dec_ms = timed(decode_once, K)
    log, routes = [], []
    route = ops_seq.moe_route
    ops_seq.moe_route = lambda *a, **k: (routes.append(route(*a, **k)), routes[-1])[1]
    saved = _timed_ops(ops_seq, op_names, log)
    decode_once()
    dec_ops = _by_op(log)
    for n, fn in saved.items():
        setattr(ops_seq, n, fn)
    ops_seq.moe_route = route
    picked = sum(len(set(r.ids.flatten().tolist())) for r in routes)
    model.kv_cache_manager.free_sequences(sids)
    with torch.inference_mode():   # the serving path: from_pb -> generate_token, plain greedy, replayed as one CUDA graph
        gpb = make_batch_pb(DB, DL, Wm + K + 8)
        for r, toks in zip(gpb.requests, prompt(DB, DL)):
            r.inputs = " ".join(f"<tok{t}>" for t in toks)
        gbatch, _ = model.batch_type.from_pb(gpb, model.tokenizer, torch.bfloat16, model.device, None, None, True)
        model.generate_token(gbatch, first=True)
        for _ in range(Wm):
            model.generate_token(gbatch)
        graph_ms = timed(lambda: model.generate_token(gbatch), K)
        dec_k, dec_total = _traced_decode_step(model, gbatch, lib)
        model.kv_cache_manager.free_sequences(gbatch.sequence_ids)
    del model, engine, weights
    gc.collect()
    torch.cuda.empty_cache()
    return {"pre_ms": pre_ms, "pre_ops": pre_ops, "dec_ms": dec_ms, "dec_ops": dec_ops, "graph_ms": graph_ms, "dec_k": dec_k, "dec_total": dec_total,
            "picked": picked}


def _noganex_side(width, env):
    """the Noganex half of --noganex-compare (also the partner of --nasozen-compare) -> its result entry"""
    from tgis_b200.models.custom_modeling import noganex_modeling
    from tgis_b200.utils.synthetic import noganex_config
    PB, PL, DB, DL, K, Wm, ctx = (env[k] for k in ("PB", "PL", "DB", "DL", "K", "Wm", "ctx"))
    timed, lib, hbm, tens, common, us = (env[k] for k in ("timed", "lib", "hbm", "tens", "common", "us"))
    raw = noganex_config(f"noganex-w{width}")
    names = ["linear", "embed_scale", "cast_rows", "rmsnorm_rows", "gated_rms_add", "causal_conv", "delta_scan", "qk_rot_prepare", "talk_attn",
             "group_rmsnorm_gate", "moe_route", "moe_gather_rows", "moe_linear", "ff_gate", "moe_combine_add"]
    r = _stream_family_measure(raw, noganex_modeling.NoganexConfig(raw), names, PB, PL, DB, DL, K, Wm, timed, lib)
    shapes = noganex_modeling.tensor_shapes(raw)
    attn = [l["mixer"] for l in raw["layers"] if l["type"] == "attention"]
    delta = [l["mixer"] for l in raw["layers"] if l["type"] == "delta"]
    attn_flops = sum(PB * (PL * (PL + 1) // 2) * m["heads"] * (m["dim"] + m["vdim"] + m["heads"]) * 2 for m in attn)
    attn_row = sum(m["kv_heads"] * (m["dim"] + m["vdim"]) for m in attn)       # elements a decoding token reads per cached token
    state_b = sum(m["heads"] * m["dim"] * m["vdim"] * 4 * 2 for m in delta)    # state read + written per sequence and step
    moes = [l["mlp"] for l in raw["layers"] if l["mlp"] and l["mlp"]["kind"] == "moe"]
    expert_w = 3 * width * moes[0]["expert"]["ff"]
    top = moes[0]["router"]["top"]
    dense_w = sum(a * b for n, (a, *rest) in shapes.items() for b in rest[:1] if ".mlp.e" not in n and n not in ("embed", "head"))
    head_w = shapes["head"][0] * shapes["head"][1]
    lin_flops = 2 * PB * PL * (dense_w + len(moes) * top * expert_w) + 2 * PB * head_w
    a_us, s_us, m_us = us(r["dec_k"], "talk_attn"), us(r["dec_k"], "delta_scan"), r["dec_k"].get("moe_linear_mma_kernel", 0.0)
    g_us = r["dec_k"].get("gemm_f16_kernel", 0.0)
    kernels = {
        "talk_attn prefill": {"ms": r["pre_ops"]["talk_attn"], "tflops": attn_flops / r["pre_ops"]["talk_attn"] / 1e9,
                              "of_measured_tensor": attn_flops / (r["pre_ops"]["talk_attn"] * 1e-3) / tens},
        "talk_attn decode": {"us": a_us, "of_measured_hbm": DB * ctx * attn_row * 2 / (max(a_us, 1e-9) * 1e-6) / hbm},
        "delta_scan prefill": {"ms": r["pre_ops"]["delta_scan"], "tokens_per_s_per_layer": PB * PL * len(delta) / (r["pre_ops"]["delta_scan"] * 1e-3)},
        "delta_scan decode": {"us": s_us, "of_measured_hbm": DB * state_b / (max(s_us, 1e-9) * 1e-6) / hbm},
        "linear prefill (projections, gates, one product per expert)": {"ms": r["pre_ops"]["linear"],
                                                                        "of_measured_tensor": lin_flops / (r["pre_ops"]["linear"] * 1e-3) / tens},
        "moe_linear decode (grouped, picked experts' weights once)": {"us": m_us, "experts_picked_all_layers": r["picked"], "of_measured_hbm":
                                                                      r["picked"] * expert_w * 2 / (max(m_us, 1e-9) * 1e-6) / hbm},
        "linear decode (tcgen05 projections)": {"us": g_us, "of_measured_hbm": (dense_w + head_w) * 2 / (max(g_us, 1e-9) * 1e-6) / hbm},
    }
    return common(f"noganex-w{width}", raw, r, kernels, {"experts": moes[0]["router"]["experts"], "top": top})


def run_noganex_compare(args):
    """Noganex (bfloat16) beside Dubesun (bfloat16), the closest family of the engine (fp32 stream, attention over a paged cache, short
    convolutions, routed experts), at equal width and depth on random weights: prefill of 4 x 1024 tokens and decode of 32 sequences at
    context 1024, measured as --dubesun-compare measures its pair, with the achieved FLOP/s or bytes/s of the kernels that carry a step
    against the measured peaks."""
    import torch
    import tgis_b200  # noqa: F401
    from tgis_b200 import _lib as _libmod
    from tgis_b200.models.custom_modeling import dubesun_modeling
    from tgis_b200.utils.synthetic import dubesun_config

    pk = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")):
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        pk = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    hbm, tens = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    PB, PL, DB, DL = 4, 1024, 32, 1024
    K, Wm = max(args.steps // 4, 4), args.warmup
    ctx = DL + Wm + K + 2
    lib = _libmod.load_seq()
    results = []

    def timed(fn, n):
        total = 0.0
        for _ in range(n):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / n

    def common(name, raw, r, kernels, extra):
        out = {"model": name, "dtype": "bf16", "layers": len(raw["layers"]), "prefill_tokens_per_s": PB * PL / (r["pre_ms"] * 1e-3),
               "decode_tokens_per_s": DB / (r["dec_ms"] * 1e-3), "prefill_ms": r["pre_ms"], "decode_ms_per_step": r["dec_ms"],
               "decode_graph_tokens_per_s": DB / (r["graph_ms"] * 1e-3), "decode_graph_ms_per_step": r["graph_ms"],
               "prefill_ms_by_op": {k: round(v, 4) for k, v in r["pre_ops"].items()},
               "decode_ms_by_op": {k: round(v, 4) for k, v in r["dec_ops"].items()},
               "decode_graph_us_by_kernel": {k: round(v, 2) for k, v in sorted(r["dec_k"].items(), key=lambda kv: -kv[1])},
               "decode_graph_traced_us": r["dec_total"], "kernels": kernels}
        out.update(extra)
        return out

    def us(dec_k, *prefixes):
        return sum(v for k, v in dec_k.items() if k.startswith(prefixes))

    widths = (2048, 4096) if not args.layers else (2048,)
    env = dict(PB=PB, PL=PL, DB=DB, DL=DL, K=K, Wm=Wm, ctx=ctx, timed=timed, lib=lib, hbm=hbm, tens=tens, common=common, us=us)
    for width in widths:
        results.append(_noganex_side(width, env))
        # ---------------------------------------------------------------- Dubesun, the partner
        raw = dubesun_config(f"dubesun-w{width}")
        names = ["linear", "embed_add_pos", "rmsnorm_rows", "causal_conv", "heads_prepare", "paged_attn", "diff_combine", "group_rmsnorm_gate",
                 "moe_route", "moe_gather_rows", "moe_linear", "ff_clamped_gate", "moe_combine_add"]
        r = _stream_family_measure(raw, dubesun_modeling.DubesunConfig(raw), names, PB, PL, DB, DL, K, Wm, timed, lib)
        shapes = dubesun_modeling.tensor_shapes(raw)
        attn_flops, attn_row = 0, 0
        for layer in raw["layers"]:
            m = layer["mixer"]
            maps = 2 if layer["type"] == "attention" else 1
            attn_flops += PB * (PL * (PL + 1) // 2) * m["heads"] * maps * (m["dim"] + m["vdim"]) * 2
            attn_row += m["kv_heads"] * (maps * m["dim"] + m["vdim"])
        f = raw["layers"][0]["mlp"]
        expert_w, top, L = 3 * width * f["expert"]["ff"], f["router"]["top"], len(raw["layers"])
        proj_w = sum(a * b for n, (a, *rest) in shapes.items() for b in rest[:1]
                     if n.split(".")[-1] in ("q", "k", "v", "g", "o", "router") and ".mlp.e" not in n)
        head_w = shapes["head"][0] * shapes["head"][1]
        lin_flops = 2 * PB * PL * (proj_w + L * top * expert_w) + 2 * PB * head_w
        a_us, m_us, g_us = us(r["dec_k"], "paged_heads_attn"), r["dec_k"].get("moe_linear_mma_kernel", 0.0), r["dec_k"].get("gemm_f16_kernel", 0.0)
        kernels = {
            "paged_attn prefill": {"ms": r["pre_ops"]["paged_attn"], "tflops": attn_flops / r["pre_ops"]["paged_attn"] / 1e9,
                                   "of_measured_tensor": attn_flops / (r["pre_ops"]["paged_attn"] * 1e-3) / tens},
            "paged_attn decode": {"us": a_us, "of_measured_hbm": DB * ctx * attn_row * 2 / (max(a_us, 1e-9) * 1e-6) / hbm},
            "linear prefill (projections + one product per expert)": {"ms": r["pre_ops"]["linear"],
                                                                      "of_measured_tensor": lin_flops / (r["pre_ops"]["linear"] * 1e-3) / tens},
            "moe_linear decode (grouped, picked experts' weights once)": {"us": m_us, "experts_picked_all_layers": r["picked"], "of_measured_hbm":
                                                                          r["picked"] * expert_w * 2 / (max(m_us, 1e-9) * 1e-6) / hbm},
            "linear decode (tcgen05 projections)": {"us": g_us, "of_measured_hbm": (proj_w + head_w) * 2 / (max(g_us, 1e-9) * 1e-6) / hbm},
        }
        results.append(common(f"dubesun-w{width}", raw, r, kernels, {"experts": f["router"]["experts"], "top": top}))
    print(json.dumps({"metric": "noganex_compare", "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": Wm, "data": "synthetic",
                      "config": {"prefill": [PB, PL], "decode": [DB, DL], "l2": "flushed between timed calls"},
                      "peaks": {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": pk.get("source")}, "models": results}))
    return 0


def run_nasozen_compare(args):
    """Nasozen (bfloat16) beside Noganex (bfloat16), the closest family of the engine (fp32 stream, whole-projection q / k norm and
    rotate-half rotation in front of the same attention kernel, a delta-rule memory, routed experts), at equal width and depth on random
    weights: prefill of 4 x 1024 tokens and decode of 32 sequences at context 1024, measured as --noganex-compare measures its pair, with
    the achieved FLOP/s or bytes/s of the kernels that carry a step against the measured peaks."""
    import torch
    import tgis_b200  # noqa: F401
    from tgis_b200 import _lib as _libmod
    from tgis_b200.models.custom_modeling import nasozen_modeling
    from tgis_b200.utils.synthetic import nasozen_config

    pk = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")):
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        pk = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    hbm, tens = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    PB, PL, DB, DL = 4, 1024, 32, 1024
    K, Wm = max(args.steps // 4, 4), args.warmup
    ctx = DL + Wm + K + 2
    lib = _libmod.load_seq()
    results = []

    def timed(fn, n):
        total = 0.0
        for _ in range(n):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / n

    def common(name, raw, r, kernels, extra):
        out = {"model": name, "dtype": "bf16", "layers": len(raw["layers"]), "prefill_tokens_per_s": PB * PL / (r["pre_ms"] * 1e-3),
               "decode_tokens_per_s": DB / (r["dec_ms"] * 1e-3), "prefill_ms": r["pre_ms"], "decode_ms_per_step": r["dec_ms"],
               "decode_graph_tokens_per_s": DB / (r["graph_ms"] * 1e-3), "decode_graph_ms_per_step": r["graph_ms"],
               "prefill_ms_by_op": {k: round(v, 4) for k, v in r["pre_ops"].items()},
               "decode_ms_by_op": {k: round(v, 4) for k, v in r["dec_ops"].items()},
               "decode_graph_us_by_kernel": {k: round(v, 2) for k, v in sorted(r["dec_k"].items(), key=lambda kv: -kv[1])},
               "decode_graph_traced_us": r["dec_total"], "kernels": kernels}
        out.update(extra)
        return out

    def us(dec_k, *prefixes):
        return sum(v for k, v in dec_k.items() if k.startswith(prefixes))

    env = dict(PB=PB, PL=PL, DB=DB, DL=DL, K=K, Wm=Wm, ctx=ctx, timed=timed, lib=lib, hbm=hbm, tens=tens, common=common, us=us)
    widths = (2048, 4096) if not args.layers else (2048,)
    for width in widths:
        raw = nasozen_config(f"nasozen-w{width}")
        names = ["linear", "embed_scale", "streams_step", "causal_conv", "qk_rot_prepare", "talk_attn", "heads_turn_gate", "mingru_scan", "mlstm_scan",
                 "gdelta_scan", "group_rmsnorm_gate", "ff_act", "moe_route", "moe_gather_rows", "moe_linear", "ff_gate", "moe_combine_add"]
        cfg = nasozen_modeling.NasozenConfig(raw)
        r = _stream_family_measure(raw, cfg, names, PB, PL, DB, DL, K, Wm, timed, lib)
        shapes = nasozen_modeling.tensor_shapes(raw)
        par = [l["mixer"] for l in raw["layers"] if l["type"] == "parallel"]
        attn = [m["left"] for m in par]
        delta = [l["mixer"] for l in raw["layers"] if l["type"] == "general_delta"]
        mem = [l["mixer"] for l in raw["layers"] if l["type"] == "mlstm"]
        S, T = cfg.streams or 1, PB * PL
        subs = sum(2 if l["mlp"] else 1 for l in raw["layers"])
        attn_flops = sum(PB * (PL * (PL + 1) // 2) * m["heads"] * (m["dim"] + m["vdim"]) * 2 for m in attn)
        attn_row = sum(m["kv_heads"] * (m["dim"] + m["vdim"]) for m in attn)       # elements a decoding token reads per cached token
        delta_b = sum(m["heads"] * m["dim"] * m["dim"] * 4 * 2 for m in delta)     # state read + written per sequence and step
        mem_b = sum(m["heads"] * m["dim"] * m["vdim"] * 4 * 2 for m in mem)
        gru_b = sum(m["right"]["width"] * (4 * 2 + 3 * 4 + 2) for m in par)         # state in and out, three fp32 inputs, one typed result
        # streams in and out once per sublayer, the sublayer's result in, the typed copy out (+ the first launch: embedding row in)
        stream_b = subs * width * (S * 4 * 2 + 4 + 2) + width * (4 + 2 + S * 4)
        moes = [l["mlp"] for l in raw["layers"] if l["mlp"] and l["mlp"]["kind"] == "moe"]
        expert_w = 3 * width * moes[0]["expert"]["ff"]
        top = moes[0]["router"]["top"]
        dense_w = sum(a * b for n, (a, *rest) in shapes.items() for b in rest[:1] if ".mlp.e" not in n and n != "embed")
        head_w = shapes["embed"][0] * shapes["embed"][1]
        lin_flops = 2 * T * (dense_w + len(moes) * top * expert_w) + 2 * PB * head_w
        dk = r["dec_k"]
        a_us, m_us, g_us = us(dk, "talk_attn"), dk.get("moe_linear_mma_kernel", 0.0), dk.get("gemm_f16_kernel", 0.0)
        kernels = {
            "talk_attn prefill": {"ms": r["pre_ops"]["talk_attn"], "tflops": attn_flops / r["pre_ops"]["talk_attn"] / 1e9,
                                  "of_measured_tensor": attn_flops / (r["pre_ops"]["talk_attn"] * 1e-3) / tens},
            "talk_attn decode": {"us": a_us, "of_measured_hbm": DB * ctx * attn_row * 2 / (max(a_us, 1e-9) * 1e-6) / hbm},
            "gdelta_scan prefill": {"ms": r["pre_ops"]["gdelta_scan"], "tokens_per_s_per_layer": T * len(delta) / (r["pre_ops"]["gdelta_scan"] * 1e-3)},
            "gdelta_scan decode": {"us": us(dk, "gdelta_scan"), "of_measured_hbm": DB * delta_b / (max(us(dk, "gdelta_scan"), 1e-9) * 1e-6) / hbm},
            "mlstm_scan prefill": {"ms": r["pre_ops"]["mlstm_scan"], "tokens_per_s_per_layer": T * len(mem) / (r["pre_ops"]["mlstm_scan"] * 1e-3)},
            "mlstm_scan decode": {"us": us(dk, "mlstm_scan"), "of_measured_hbm": DB * mem_b / (max(us(dk, "mlstm_scan"), 1e-9) * 1e-6) / hbm},
            "mingru_scan prefill": {"ms": r["pre_ops"]["mingru_scan"], "tokens_per_s_per_layer": T * len(par) / (r["pre_ops"]["mingru_scan"] * 1e-3),
                                    "of_measured_hbm": T * sum(m["right"]["width"] for m in par) * 14 / (r["pre_ops"]["mingru_scan"] * 1e-3) / hbm},
            "mingru_scan decode": {"us": us(dk, "mingru_scan"), "of_measured_hbm": DB * gru_b / (max(us(dk, "mingru_scan"), 1e-9) * 1e-6) / hbm},
            "streams_step prefill": {"ms": r["pre_ops"]["streams_step"], "of_measured_hbm": T * stream_b / (r["pre_ops"]["streams_step"] * 1e-3) / hbm},
            "streams_step decode": {"us": us(dk, "streams_step"), "launches": subs + 1,
                                    "of_measured_hbm": DB * stream_b / (max(us(dk, "streams_step"), 1e-9) * 1e-6) / hbm},
            "linear prefill (projections, one product per expert)": {"ms": r["pre_ops"]["linear"],
                                                                     "of_measured_tensor": lin_flops / (r["pre_ops"]["linear"] * 1e-3) / tens},
            "moe_linear decode (grouped, picked experts' weights once)": {"us": m_us, "experts_picked_all_layers": r["picked"], "of_measured_hbm":
                                                                          r["picked"] * expert_w * 2 / (max(m_us, 1e-9) * 1e-6) / hbm},
            "linear decode (tcgen05 projections)": {"us": g_us, "of_measured_hbm": (dense_w + head_w) * 2 / (max(g_us, 1e-9) * 1e-6) / hbm},
        }
        results.append(common(f"nasozen-w{width}", raw, r, kernels, {"experts": moes[0]["router"]["experts"], "top": top, "streams": S}))
        results.append(_noganex_side(width, env))
    print(json.dumps({"metric": "nasozen_compare", "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": Wm, "data": "synthetic",
                      "config": {"prefill": [PB, PL], "decode": [DB, DL], "l2": "flushed between timed calls"},
                      "peaks": {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": pk["bf16_tflops"], "source": pk.get("source")}, "models": results}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=None, choices=list(WORKLOADS) + list(MIXED_WORKLOADS))
    ap.add_argument("--requests", type=int, default=None, help="mixed workloads: number of requests in the session")
    ap.add_argument("--layers", type=int, default=None, help="debug: override the number of layers")
    ap.add_argument("--cpu-layers", type=int, default=2, help="layers in the CPU baseline's bounded sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the second workload, the self-check and the gpt2 CPU line")
    ap.add_argument("--hybrid-compare", action="store_true",
                    help="Fetotar beside GPT-NeoX at equal size: prefill and decode throughput and per-kernel rooflines (one GPU)")
    ap.add_argument("--dubesun-compare", action="store_true",
                    help="Dubesun beside GPT-NeoX at equal size: prefill and decode throughput and per-kernel rooflines (one GPU)")
    ap.add_argument("--noganex-compare", action="store_true",
                    help="Noganex beside Dubesun at equal size: prefill and decode throughput and per-kernel rooflines (one GPU)")
    ap.add_argument("--nasozen-compare", action="store_true",
                    help="Nasozen beside Noganex at equal size: prefill and decode throughput and per-kernel rooflines (one GPU)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.hybrid_compare:
        return run_hybrid_compare(args)
    if args.dubesun_compare:
        return run_dubesun_compare(args)
    if args.noganex_compare:
        return run_noganex_compare(args)
    if args.nasozen_compare:
        return run_nasozen_compare(args)
    workload = args.workload or DEFAULT_WORKLOAD
    if workload in MIXED_WORKLOADS:
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the continuous-batching session is a GPU-arm workload; the CPU arm times "
                                                                  "single decode steps (use a decode workload)"}))
            return 0
        return run_mixed(args, workload)
    if args.impl == "reference":
        return run_reference(args, workload)
    return run_gpu(args, workload)


if __name__ == "__main__":
    sys.exit(main())
