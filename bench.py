#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of Qwen3-0.6B (28 layers, hidden 1024, 16
query heads, 8 kv heads, head size 128, feed-forward 3072, vocabulary 151936,
tied head) with seeded random weights in bfloat16, a batch of 8 requests and a
context of 4096 tokens.  A "step" is one decode step of the whole batch.  It
prints one JSON line:

  value      decoded tokens a second, timed on the device with CUDA events
  e2e        the same through the Python entry point (scheduler, host tokens in
             and out)
  prefill    one prompt of 2,048 tokens through the step function
  roofline   bytes a decode step has to read (every weight once, the cache of
             the live requests) / its time, against the measured copy bandwidth
  points     decode at batch 1 and 64

Peaks come from MEASURED_PEAKS.json beside this file when it is there.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_0_6B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 28, "hidden_size": 1024, "num_attention_heads": 16,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 3072, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 40960,
}
# the other sizes BASELINE.json names (configs[3] and [4]); `--model` runs one of them instead
SIZES = {
    "qwen3-0.6b": {},
    "qwen3-4b": {"num_hidden_layers": 36, "hidden_size": 2560, "num_attention_heads": 32,
                 "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 9728},
    "qwen3-8b": {"num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32,
                 "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
                 "tie_word_embeddings": False},
}
CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "source": "measured"}
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in self.samples)]
        return {"sm_mhz": statistics.median(int(s[0]) for s in self.samples),
                "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons, "samples": len(self.samples)}


def step_bytes(cfg, layers, batch, context, elem=2):
    """Bytes a decode step has to read: every weight it uses once, and the cache."""
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nq + 2 * nkv) * d * h + h * nq * d + 3 * i * h + 2 * h + 2 * d
    weights = layers * per_layer + v * h + h
    if not cfg["tie_word_embeddings"]:
        weights += 0          # the embedding table is only gathered from: a few rows
    cache = layers * batch * context * 2 * nkv * d
    return (weights + cache) * elem


def prefill_flops(cfg, layers, tokens):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = 2 * tokens * layers * ((nq + 2 * nkv) * d * h + h * nq * d + 3 * i * h)
    attention = layers * 4 * nq * d * tokens * (tokens + 1) // 2
    return linear + attention + 2 * v * h


def time_decode(runner, sampler, batch, context, steps, warmup, launches):
    """Decode `steps` tokens for `batch` requests that end at `context` tokens."""
    import torch

    from lockstep_b200 import StepEntry
    from lockstep_b200 import kernels as K
    from lockstep_b200.sampling import SamplingParams

    start_len = context - steps - warmup
    uids = [f"d{i}" for i in range(batch)]
    for u in uids:
        runner.open(u)
        runner.fill_random(u, start_len)
    tokens = [[(7 * i + 13) % 1000 for i in range(batch)]]
    params = [SamplingParams(uid=u) for u in uids]

    def one_step():
        entries = [StepEntry(uid=u, tokens=[tokens[0][i]], start=runner.kv_len(u), want=[0])
                   for i, u in enumerate(uids)]
        logits = runner.step(entries, check=False)
        return sampler.sample_device(logits, params)

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    K.LAUNCHES[0] = 0
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        one_step()
    b.record()
    torch.cuda.synchronize()
    launches[0] = K.LAUNCHES[0]
    K.raise_on_fault(runner.err)
    ms = a.elapsed_time(b) / steps
    for u in uids:
        runner.close(u)
    return ms


def time_e2e(engine, batch, context, steps, warmup):
    """The same decode through the scheduler: host tokens in, sampled tokens out."""
    import torch

    from lockstep_b200 import Request

    sched = engine.scheduler
    start_len = context - steps - warmup - 1
    reqs = []
    for i in range(batch):
        r = Request(uid=f"e{i}", prompt=[(11 * i + j) % 1000 for j in range(start_len)],
                    max_new_tokens=steps + warmup + 1)
        reqs.append(r)
        sched.submit(r)
        sched.waiting.remove(r)
        engine.runner.open(r.uid)
        engine.runner.fill_random(r.uid, start_len - 1)
        r.kv_len = start_len - 1
        sched.running.append(r)
    for _ in range(warmup):
        sched.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        sched.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    produced = sum(len(r.generated) for r in reqs)
    assert produced == batch * (steps + warmup), produced
    sched.drain()              # a step the scheduler launched ahead of its last collect
    for r in list(sched.running):
        sched.running.remove(r)
        engine.runner.close(r.uid)
    # per step: one pinned buffer in (token ids, positions, slots, wanted rows, attention work
    # lists: the recorded step's whole input), sampled ids and the error word out
    graphs = engine.runner.graphs
    if graphs is not None and graphs.graphs:
        h2d = max(ctx.size for _, ctx, _, _ in graphs.graphs.values()) * 4
    else:
        h2d = batch * 4 * 4 + batch * (context // 256 + 1) * 8 * 4 + batch * 16
    return batch * steps / dt, h2d, batch * 4 + 8


def time_prefill(runner, tokens, repeats=3):
    import torch

    from lockstep_b200 import StepEntry

    ids = [(5 * i + 3) % 1000 for i in range(tokens)]
    times = []
    for r in range(repeats + 1):
        uid = f"p{r}"
        runner.open(uid)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        runner.step([StepEntry(uid=uid, tokens=ids, start=0, want=[tokens - 1])], check=False)
        b.record()
        torch.cuda.synchronize()
        runner.close(uid)
        if r:
            times.append(a.elapsed_time(b))
    return statistics.median(times)


def run_ours(args):
    import torch

    from lockstep_b200 import Engine
    from lockstep_b200 import kernels as K
    from lockstep_b200.weights import write_random_model

    cfg = dict(QWEN3_0_6B)
    cfg.update(SIZES[args.model])
    label = args.model.replace("qwen3", "Qwen3").upper().replace("QWEN3", "Qwen3")
    layers_full = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    layers = cfg["num_hidden_layers"]
    pk = peaks()
    batches = sorted({args.batch, 1, 64} if not args.quick else {args.batch})
    max_batch = max(batches)
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_random_model(Path(tmp) / "qwen3-0.6b-random", cfg, seed=0, dtype="bfloat16",
                                    device="cuda:0")
        engine = Engine(folder, dtype="bfloat16", device="cuda:0",
                        num_pages=max_batch * (CONTEXT // PAGE) + 8, page_size=PAGE,
                        max_running=max_batch, max_step_tokens=max(PREFILL_TOKENS, max_batch),
                        max_seq_len=CONTEXT)
    runner = engine.runner
    launches = [0]
    if args.only == "decode":
        ms = time_decode(runner, engine.sampler, args.batch, args.context, args.steps, args.warmup, launches)
        print(json.dumps({"only": "decode", "layers": layers, "batch": args.batch, "context": args.context,
                          "ms_per_step": round(ms, 4), "launches": launches[0]}))
        return 0
    if args.only == "prefill":
        pre_ms = time_prefill(runner, PREFILL_TOKENS, repeats=max(1, args.steps))
        print(json.dumps({"only": "prefill", "layers": layers, "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3)}))
        return 0
    clocks = ClockSampler()
    points = {}
    for b in batches:
        if b == args.batch:
            continue
        steps = max(4, args.steps // 4)
        ms = time_decode(runner, engine.sampler, b, CONTEXT, steps, args.warmup, [0])
        points[f"decode_b{b}"] = round(b / ms * 1e3, 1)
    clocks.start()
    ms = time_decode(runner, engine.sampler, args.batch, CONTEXT, args.steps, args.warmup, launches)
    clock_info = clocks.stop()
    value = args.batch / ms * 1e3
    e2e, h2d, d2h = time_e2e(engine, args.batch, CONTEXT, args.steps, args.warmup)
    pre_ms = time_prefill(runner, PREFILL_TOKENS)
    flops = prefill_flops(cfg, layers, PREFILL_TOKENS)
    bytes_step = step_bytes(cfg, layers, args.batch, CONTEXT)
    achieved = bytes_step / (ms * 1e-3) / 1e9
    line = {
        "metric": f"decode tokens/s, {label} sizes, batch {args.batch}, context {CONTEXT}",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {
            "model": f"{label} sizes, random weights N(0,0.02)", "layers": layers,
            "layers_of_model": layers_full, "hidden": cfg["hidden_size"],
            "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "tied_head": True, "global_batch": args.batch,
            "seq_len": CONTEXT, "page": PAGE, "prefill_tokens": PREFILL_TOKENS,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (weights + cache per step)",
            "peaks": pk["source"],
        },
        "clocks": clock_info,
        "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches[0],
        "prefill": {"value": round(PREFILL_TOKENS / pre_ms * 1e3, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(pre_ms, 3), "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0,
                    help="run fewer layers than the model has (named in config)")
    ap.add_argument("--model", default="qwen3-0.6b", choices=sorted(SIZES),
                    help="layer sizes (the default is the configuration the headline is quoted on)")
    ap.add_argument("--quick", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--only", default="", choices=["", "decode", "prefill"],
                    help="time only this part and print a short line (for profiling a small case)")
    ap.add_argument("--context", type=int, default=CONTEXT, help="context length of the decode steps")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported by this engine")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        print(json.dumps({
            "impl": "reference",
            "unavailable": "u7k4rs6/LockStep does not install offline: pip's metadata step fails "
                           "(the project sets [tool.uv] package = false and setuptools refuses its "
                           "flat layout of several top-level packages)"}))
        return 0
    return run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
