#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of Qwen3-0.6B (28 layers, hidden 1024, 16
query heads, 8 kv heads, head size 128, feed-forward 3072, vocabulary 151936,
tied head) with seeded random weights in bfloat16, a batch of 8 requests and a
context of 4096 tokens.  A "step" is one decode step of the whole batch.  Every
timed region is run five times (W warm-up steps, then exactly K timed steps,
from the same start) and the median is reported with the spread.  It prints one
JSON line:

  value      decoded tokens a second, timed on the device with CUDA events
  e2e        the same through the Python entry point (scheduler, host tokens in
             and out)
  prefill    one prompt of 2,048 tokens through the step function
  roofline   bytes a decode step has to read (every weight once, the cache of
             the live requests) / its time, against the measured copy bandwidth
  points     decode at batch 1 and 64 at the same context, decode at batch
             1/8/64 from a prompt of 512 over 256 generated tokens, and decode
             and prefill on the true 32-bit path; point_frac gives each one's
             fraction of its roofline

Peaks come from MEASURED_PEAKS.json beside this file when it is there.

``--impl reference`` runs u7k4rs6/LockStep itself, unmodified, from the plain
copy of its tree under baseline/_ref (its stock ``Qwen3`` and ``Scheduler``,
Triton kernels, float16) on the same workload and prints the same line.
``--workload mixed`` runs a continuous batch of 64 requests with prompts of 64
to 2,048 tokens and 128 decoded tokens each through the entry point.
"""

from __future__ import annotations

import argparse
import json
import random
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
# the other sizes the headline's source names; `--model` runs one of them instead
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
LONG_PREFILL_TOKENS = 8192      # an extra point: a prompt four times the headline's
PAGE = 16
REPEATS = 5
SETTLE = 24            # untimed decode steps before the warm-up steps of every timed decode region
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
FP32_TFLOPS_NOMINAL = 80.0        # FFMA peak of the CUDA cores: the 32-bit path's compute roof


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
    """Bytes a decode step has to read: every weight it uses once, and the cache
    (``context`` keys of every live request)."""
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nq + 2 * nkv) * d * h + h * nq * d + 3 * i * h + 2 * h + 2 * d
    weights = layers * per_layer + v * h + h      # the embedding table is only gathered from
    cache = layers * batch * context * 2 * nkv * d
    return (weights + cache) * elem


def prefill_flops(cfg, layers, tokens):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = 2 * tokens * layers * ((nq + 2 * nkv) * d * h + h * nq * d + 3 * i * h)
    attention = layers * 4 * nq * d * tokens * (tokens + 1) // 2
    return linear + attention + 2 * v * h


def spread(values):
    return {"median": round(statistics.median(values), 4), "min": round(min(values), 4),
            "max": round(max(values), 4), "n": len(values)}


def time_decode(runner, sampler, batch, end_context, steps, warmup, repeats=REPEATS, launches=None):
    """`repeats` regions, each: `batch` requests filled to the same start, `warmup` untimed
    decode steps, then exactly `steps` timed ones that end at `end_context` tokens.  Returns
    the milliseconds per step of every region."""
    import torch

    from lockstep_b200 import StepEntry
    from lockstep_b200 import kernels as K
    from lockstep_b200.sampling import SamplingParams

    # (the device runs its first dozen steps after other work some 10 % slower: `settle` more
    # untimed steps come before the warm-up steps)
    settle = SETTLE if end_context - steps - warmup - SETTLE >= 64 else 0
    warmup = warmup + settle
    start_len = end_context - steps - warmup
    if start_len < 1:
        raise ValueError("more steps than the context holds")
    uids = [f"d{i}" for i in range(batch)]
    tokens = [(7 * i + 13) % 1000 for i in range(batch)]
    params = [SamplingParams(uid=u) for u in uids]

    def one_step():
        entries = [StepEntry(uid=u, tokens=[tokens[i]], start=runner.kv_len(u), want=[0])
                   for i, u in enumerate(uids)]
        logits = runner.step(entries, check=False)
        return sampler.sample_device(logits, params)

    out = []
    for _ in range(repeats):
        for u in uids:
            runner.open(u)
            runner.fill_random(u, start_len)
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
        if launches is not None:
            launches[0] = K.LAUNCHES[0]
        K.raise_on_fault(runner.err)
        out.append(a.elapsed_time(b) / steps)
        for u in uids:
            runner.close(u)
    return out


def time_e2e(engine, batch, context, steps, warmup, repeats=REPEATS):
    """The same decode through the entry point: requests are submitted with prompts of host
    token ids, the engine prefills them itself (untimed), and `steps` decode steps of the whole
    batch are timed by the host's clock, sampled tokens read back on the host every step."""
    import torch

    from lockstep_b200 import Request

    rates = []
    sched = engine.scheduler
    for rep in range(repeats):
        # (after the prompts' step the device runs its first dozen decode steps some 10 % slower:
        # SETTLE untimed steps come before the warm-up steps)
        start_len = context - steps - warmup - SETTLE - 4
        reqs = [Request(uid=f"e{rep}-{i}", prompt=[(11 * i + j) % 1000 for j in range(start_len)],
                        max_new_tokens=steps + warmup + SETTLE + 4) for i in range(batch)]
        for r in reqs:
            engine.submit(r)
        # the prompts go in one step (a budget for all of them), so that every request decodes
        # at the same context in the timed steps
        budget, sched.max_step_tokens = sched.max_step_tokens, batch * context
        while not all(r.generated for r in reqs):
            sched.step()
        sched.max_step_tokens = budget
        for _ in range(SETTLE + warmup):
            sched.step()
        sched.drain()
        torch.cuda.synchronize()
        before = sum(len(r.generated) for r in reqs)
        t0 = time.perf_counter()
        for _ in range(steps):
            sched.step()
        sched.drain()              # a step the scheduler launched ahead of its last collect
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        produced = sum(len(r.generated) for r in reqs) - before
        assert batch * steps <= produced <= batch * (steps + 1), produced
        rates.append(produced / dt)
        for r in reqs:
            r.max_new_tokens = len(r.generated) + 1      # let them end
        while sched.step():
            pass
        sched.drain()
        assert engine.cache.free_pages() == engine.cache.total_pages()
    # per step: one pinned buffer in (token ids, positions, slots, wanted rows, attention work
    # lists: the recorded step's whole input), sampled ids and the error word out
    graphs = engine.runner.graphs
    if graphs is not None and graphs.graphs:
        h2d = graphs.input_bytes()
    else:
        h2d = batch * 4 * 4 + batch * (context // 256 + 1) * 8 * 4 + batch * 16
    return rates, h2d, batch * 4 + 8


def time_prefill(runner, tokens, repeats=REPEATS):
    import torch

    from lockstep_b200 import StepEntry

    ids = [(5 * i + 3) % 1000 for i in range(tokens)]
    times = []
    warm = 3          # untimed: a step of a shape that comes for the third time is recorded, later ones replay it
    for r in range(repeats + warm):
        uid = f"p{r}"
        runner.open(uid)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        runner.step([StepEntry(uid=uid, tokens=ids, start=0, want=[tokens - 1])], check=False)
        b.record()
        torch.cuda.synchronize()
        runner.close(uid)
        if r >= warm:
            times.append(a.elapsed_time(b))
    return times


def time_generate(engine, batch, options, prompt=512, new=256, repeats=3):
    """Tokens a second of `batch` requests with prompts of `prompt` tokens generating `new` tokens
    each through ``Engine.generate`` (host tokens in and out, the prefill included); the median of
    `repeats` runs after one untimed run."""
    import time

    import torch

    from lockstep_b200 import Request

    rates = []
    for r in range(repeats + 1):
        requests = [Request(uid=f"g{r}_{i}", prompt=[(11 * i + 7 * j + r) % 1000 for j in range(prompt)],
                            max_new_tokens=new, **options) for i in range(batch)]
        torch.cuda.synchronize()
        start = time.perf_counter()
        out = engine.generate(requests)
        torch.cuda.synchronize()
        if r:
            rates.append(sum(len(v) for v in out.values()) / (time.perf_counter() - start))
    return statistics.median(rates)


def steps_for(ms_guess: float, least: int = 8, most: int = 400, region_ms: float = 220.0) -> int:
    """Steps that make a region last about `region_ms`."""
    return max(least, min(most, int(region_ms / max(ms_guess, 1e-3))))


def build_engine(cfg, dtype, max_batch, context, seed=0):
    from lockstep_b200 import Engine
    from lockstep_b200.weights import write_random_model

    with tempfile.TemporaryDirectory() as tmp:
        folder = write_random_model(Path(tmp) / "random-model", cfg, seed=seed, dtype=dtype, device="cuda:0")
        return Engine(folder, dtype=dtype, device="cuda:0", num_pages=max_batch * (context // PAGE) + 8,
                      page_size=PAGE, max_running=max_batch, max_step_tokens=max(PREFILL_TOKENS, max_batch),
                      max_seq_len=context)


def model_config(args):
    cfg = dict(QWEN3_0_6B)
    cfg.update(SIZES[args.model])
    label = "Qwen3-" + args.model.split("-")[1].upper()
    layers_full = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    return cfg, label, layers_full


def config_record(cfg, label, layers_full, args, pk, extra=None):
    """`config` of the JSON line: flat, every size named."""
    from lockstep_b200 import constants

    record = {
        "model": f"{label} sizes, random weights N(0,0.02)", "layers": cfg["num_hidden_layers"],
        "layers_of_model": layers_full, "hidden": cfg["hidden_size"],
        "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
        "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
        "vocab": cfg["vocab_size"], "tied_head": bool(cfg["tie_word_embeddings"]), "global_batch": args.batch,
        "seq_len": CONTEXT, "page": PAGE, "prefill_tokens": PREFILL_TOKENS,
        "parallelism": "single GPU",
        "l2": "inputs larger than L2 (weights + cache per step)",
        "timing": f"median of {REPEATS} regions of --steps steps after --warmup steps; peaks {pk['source']}",
        "kernel_constants": constants.describe(),
        "kernel_constants_sha256": constants.digest(),
    }
    if extra:
        record.update(extra)
    assert len(record) <= 20
    return record


def run_ours(args):
    import torch

    from lockstep_b200 import kernels as K

    cfg, label, layers_full = model_config(args)
    layers = cfg["num_hidden_layers"]
    pk = peaks()
    batches = sorted({args.batch, 1, 64} if not args.quick else {args.batch})
    max_batch = 1 if args.only == "prefill" else max(batches)      # (the cache pool is sized for batch x context)
    engine = build_engine(cfg, args.dtype if args.only else "bfloat16", max_batch,
                          max(CONTEXT, args.prefill_tokens + 64) if args.only == "prefill" else CONTEXT)
    runner = engine.runner
    launches = [0]
    if args.only == "decode":
        ms = time_decode(runner, engine.sampler, args.batch, args.context, args.steps, args.warmup, 1, launches)[0]
        print(json.dumps({"only": "decode", "dtype": args.dtype, "layers": layers, "batch": args.batch,
                          "context": args.context, "ms_per_step": round(ms, 4), "launches": launches[0]}))
        return 0
    if args.only == "prefill":
        pre = time_prefill(runner, args.prefill_tokens, repeats=max(1, args.steps))
        print(json.dumps({"only": "prefill", "dtype": args.dtype, "layers": layers, "tokens": args.prefill_tokens,
                          "ms": round(statistics.median(pre), 3)}))
        return 0

    def frac_of_hbm(batch, mean_context, ms, elem=2):
        return step_bytes(cfg, layers, batch, mean_context, elem) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]

    points, point_frac, point_spread = {}, {}, {}
    # the same context at batch 1 and 64; then a prompt of 512 and 256 generated tokens
    guess = {1: 1.0, 8: 1.5, 64: 6.5}
    for b in batches:
        if b == args.batch:
            continue
        steps = steps_for(guess.get(b, 2.0) * layers / 28)
        ms = time_decode(runner, engine.sampler, b, CONTEXT, steps, args.warmup)
        med = statistics.median(ms)
        points[f"decode_b{b}"] = round(b / med * 1e3, 1)
        point_frac[f"decode_b{b}"] = round(frac_of_hbm(b, CONTEXT - steps / 2, med), 4)
        point_spread[f"decode_b{b}"] = spread(ms)
    if not args.quick:
        for b in batches:
            ms = time_decode(runner, engine.sampler, b, 768, 256 - args.warmup - SETTLE, args.warmup, repeats=3)
            med = statistics.median(ms)
            points[f"decode_b{b}_prompt512_gen256"] = round(b / med * 1e3, 1)
            point_frac[f"decode_b{b}_prompt512_gen256"] = round(frac_of_hbm(b, 768 - (256 - args.warmup - SETTLE) / 2, med), 4)

    clocks = ClockSampler()
    clocks.start()
    ms_all = time_decode(runner, engine.sampler, args.batch, CONTEXT, args.steps, args.warmup, REPEATS, launches)
    clock_info = clocks.stop()
    ms = statistics.median(ms_all)
    value = args.batch / ms * 1e3
    e2e_all, h2d, d2h = time_e2e(engine, args.batch, CONTEXT, args.steps, args.warmup)
    pre_all = time_prefill(runner, PREFILL_TOKENS)
    pre_ms = statistics.median(pre_all)
    if not args.quick:
        # whole generations through the entry point (their prefill included), greedy and sampled
        for name, options in (("greedy", {}), ("temperature", {"temperature": 0.8, "seed": 3}),
                              ("top_p", {"temperature": 0.8, "top_p": 0.9, "seed": 3})):
            points[f"generate_b{args.batch}_p512_n256_{name}"] = round(time_generate(engine, args.batch, options), 1)
    flops = prefill_flops(cfg, layers, PREFILL_TOKENS)
    bytes_step = step_bytes(cfg, layers, args.batch, CONTEXT - args.steps / 2)
    achieved = bytes_step / (ms * 1e-3) / 1e9

    if not args.quick:
        # a longer prompt in one step: attention is most of its work
        engine = runner = None
        torch.cuda.empty_cache()
        engine_long = build_engine(cfg, "bfloat16", 1, LONG_PREFILL_TOKENS + 64)
        pre_long = statistics.median(time_prefill(engine_long.runner, LONG_PREFILL_TOKENS, repeats=3))
        points[f"prefill_{LONG_PREFILL_TOKENS}"] = round(LONG_PREFILL_TOKENS / pre_long * 1e3, 1)
        point_frac[f"prefill_{LONG_PREFILL_TOKENS}"] = round(
            prefill_flops(cfg, layers, LONG_PREFILL_TOKENS) / (pre_long * 1e-3) / 1e12 / pk["bf16_tflops"], 4)
        del engine_long
        torch.cuda.empty_cache()

    fp32 = None
    if not args.quick and not args.no_fp32:
        # the true 32-bit path (FFMA products): decode at the headline's batch and context, and the prefill
        engine = runner = None
        torch.cuda.empty_cache()
        engine32 = build_engine(cfg, "float32", args.batch, CONTEXT)
        ms32 = time_decode(engine32.runner, engine32.sampler, args.batch, CONTEXT, max(4, min(args.steps, 12)),
                           3, repeats=3)
        med32 = statistics.median(ms32)
        pre32 = statistics.median(time_prefill(engine32.runner, PREFILL_TOKENS, repeats=3))
        points["decode_float32"] = round(args.batch / med32 * 1e3, 1)
        points["prefill_float32"] = round(PREFILL_TOKENS / pre32 * 1e3, 1)
        point_frac["decode_float32"] = round(
            step_bytes(cfg, layers, args.batch, CONTEXT, 4) / (med32 * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        point_frac["prefill_float32"] = round(flops / (pre32 * 1e-3) / (FP32_TFLOPS_NOMINAL * 1e12), 4)
        fp32 = {"decode_ms_per_step": round(med32, 3), "prefill_ms": round(pre32, 2),
                "prefill_roof": f"{FP32_TFLOPS_NOMINAL:.0f} TFLOP/s FFMA (nominal)"}
        del engine32

    line = {
        "metric": f"decode tokens/s, {label} sizes, batch {args.batch}, context {CONTEXT}",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": config_record(cfg, label, layers_full, args, pk),
        "clocks": clock_info,
        "spread_ms_per_step": spread(ms_all),
        "e2e": {"value": round(statistics.median(e2e_all), 1), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "min": round(min(e2e_all), 1), "max": round(max(e2e_all), 1)},
        "gpu_launches": launches[0],
        "prefill": {"value": round(PREFILL_TOKENS / pre_ms * 1e3, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(pre_ms, 3), "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "min_ms": round(min(pre_all), 3), "max_ms": round(max(pre_all), 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "point_frac": point_frac,
        "point_spread_ms": point_spread,
    }
    if fp32:
        line["float32"] = fp32
    print(json.dumps(line))
    return 0


def run_mixed(args):
    """A continuous batch through the entry point: 64 requests, prompts of 64 to 2,048 random
    tokens, 128 decoded tokens each; tokens a second over the whole run (prompt and decoded)."""
    import torch

    from lockstep_b200 import Request

    cfg, label, layers_full = model_config(args)
    pk = peaks()
    rng = random.Random(0)
    n_req, new = 64, 128
    lengths = [rng.randint(64, 2048) for _ in range(n_req)]
    context = 2048 + new + 16
    engine = build_engine(cfg, "bfloat16", n_req, -(-context // PAGE) * PAGE)

    def requests(tag):
        return [Request(uid=f"{tag}{i}", prompt=[rng.randrange(1000) for _ in range(n)], max_new_tokens=new)
                for i, n in enumerate(lengths)]

    engine.generate(requests("w"))              # an untimed pass of the whole workload: kernels, recorded steps
    times = []
    for rep in range(3):
        reqs = requests(f"m{rep}-")
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = engine.generate(reqs)
        torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
        assert all(len(v) == new for v in out.values())
    dt = statistics.median(times)
    stats = engine.scheduler.stats
    print(json.dumps({
        "metric": f"mixed continuous batch, {label} sizes: 64 requests, prompts U[64,2048], 128 decoded tokens each",
        "value": round(n_req * new / dt, 1), "unit": "decoded tok/s", "n_gpus": 1, "higher_is_better": True,
        "dtype": "bf16", "data": "synthetic", "impl": "ours", "seconds": spread(times),
        "all_tokens_per_s": round((sum(lengths) + n_req * new) / dt, 1),
        "prompt_tokens": sum(lengths), "decoded_tokens": n_req * new,
        "scheduler": {k: stats[k] for k in ("steps", "mixed_steps", "preemptions", "launched_ahead")},
        "config": config_record(cfg, label, layers_full, args, pk, {"global_batch": n_req, "seq_len": context}),
    }))
    return 0


# ---------------------------------------------------------------------------
# the reference arm: LockStep itself, unmodified, from baseline/_ref
# ---------------------------------------------------------------------------

def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:600]}))
    return 0


def write_reference_folder(folder: Path, cfg: dict, seed: int = 0) -> Path:
    """config.json and model.safetensors for LockStep's loader, written with torch and
    safetensors alone: seeded N(0, 0.02) matrices, gains 1 + N(0, 0.02), float16 (its engine
    dtype, so its cast at load is exact)."""
    import torch
    from safetensors.torch import save_file

    folder.mkdir(parents=True, exist_ok=True)
    keys = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "head_dim", "vocab_size", "rms_norm_eps", "rope_theta",
            "max_position_embeddings", "tie_word_embeddings")
    (folder / "config.json").write_text(json.dumps({"model_type": "qwen3", **{k: cfg[k] for k in keys}}))
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    gen = torch.Generator(device="cuda").manual_seed(seed)

    def matrix(*shape):
        return (0.02 * torch.randn(shape, generator=gen, device="cuda")).to(torch.float16).cpu()

    def gain(n):
        return (1.0 + 0.02 * torch.randn(n, generator=gen, device="cuda")).to(torch.float16).cpu()

    t = {"model.embed_tokens.weight": matrix(v, h), "model.norm.weight": gain(h)}
    if not cfg["tie_word_embeddings"]:
        t["lm_head.weight"] = matrix(v, h)
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}"
        t[f"{p}.input_layernorm.weight"] = gain(h)
        t[f"{p}.post_attention_layernorm.weight"] = gain(h)
        t[f"{p}.self_attn.q_proj.weight"] = matrix(nq * d, h)
        t[f"{p}.self_attn.k_proj.weight"] = matrix(nkv * d, h)
        t[f"{p}.self_attn.v_proj.weight"] = matrix(nkv * d, h)
        t[f"{p}.self_attn.o_proj.weight"] = matrix(h, nq * d)
        t[f"{p}.self_attn.q_norm.weight"] = gain(d)
        t[f"{p}.self_attn.k_norm.weight"] = gain(d)
        t[f"{p}.mlp.gate_proj.weight"] = matrix(i, h)
        t[f"{p}.mlp.up_proj.weight"] = matrix(i, h)
        t[f"{p}.mlp.down_proj.weight"] = matrix(h, i)
    save_file(t, str(folder / "model.safetensors"))
    return folder


def run_reference(args):
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "engine" / "model" / "qwen3.py").is_file():
        return unavailable("baseline/_ref holds no copy of u7k4rs6/LockStep (copy its tree there; it does not "
                           "pip-install: [tool.uv] package = false and a flat layout of several top-level packages)")
    if args.model != "qwen3-0.6b" or args.layers:
        return unavailable("LockStep's kernel registry pins hidden size 1024 and head size 128 and its loader "
                           "reads all layers: only the Qwen3-0.6B configuration runs")
    if args.batch > 32:
        return unavailable("LockStep's default policy runs at most 32 requests at a time")
    # nothing of this repository's package is on the reference's path
    sys.path[:] = [p for p in sys.path if Path(p or ".").resolve() != ROOT]
    sys.path.insert(0, str(ref_root))
    try:
        import torch

        from engine.model.qwen3 import Qwen3
        from engine.sched.policy import FixedChunkPolicy
        from engine.sched.scheduler import Request, Scheduler
    except Exception as e:  # noqa: BLE001
        return unavailable(f"importing LockStep's engine failed: {type(e).__name__}: {e}")
    assert "lockstep_b200" not in sys.modules
    cfg = dict(QWEN3_0_6B)
    batch, steps, warmup = args.batch, args.steps, args.warmup
    start_len = CONTEXT - REPEATS * steps - warmup - 1
    if start_len < 16:
        return unavailable("more steps than the context of 4096 holds")
    try:
        with tempfile.TemporaryDirectory() as tmp:
            folder = write_reference_folder(Path(tmp) / "qwen3-0.6b-random", cfg)
            model = Qwen3(folder, device="cuda", max_len=CONTEXT)
        blocks = batch * (CONTEXT // PAGE) + 8
        # Its own fixed-portion policy, 512 tokens a request a step: it computes logits for every
        # fed row and its product kernel indexes rows x vocabulary in 32 bits, so a step must stay
        # below 14,133 rows (whole prompts of 8 x 4,000 tokens in one step overflowed that index
        # and faulted).  A decode step is a portion of one token under either policy.
        sched = Scheduler(model, num_blocks=blocks, block_size=PAGE, audit=False, policy=FixedChunkPolicy(512))
        rng = random.Random(0)
        reqs = [Request(uid=f"r{i:02d}", prompt=[rng.randrange(1000) for _ in range(start_len)], seed=i,
                        max_new_tokens=REPEATS * steps + warmup + 1, temperature=0.0) for i in range(batch)]
        for r in reqs:
            sched.submit(r)
        while not all(r.generated for r in reqs):      # its own prefill of the prompts, untimed
            sched.step()
        torch.cuda.synchronize()
        assert all(len(r.generated) == 1 for r in reqs)
        for _ in range(warmup):
            sched.step()
        torch.cuda.synchronize()
        clocks = ClockSampler()
        clocks.start()
        ms_all, wall_all = [], []
        for _ in range(REPEATS):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            a.record()
            for _ in range(steps):
                sched.step()
            b.record()
            torch.cuda.synchronize()
            wall_all.append(time.perf_counter() - t0)
            ms_all.append(a.elapsed_time(b) / steps)
        clock_info = clocks.stop()
        assert all(len(r.generated) == REPEATS * steps + warmup + 1 for r in reqs)
    except Exception as e:  # noqa: BLE001
        return unavailable(f"LockStep's engine did not run this workload on this GPU: {type(e).__name__}: {e}")
    ms = statistics.median(ms_all)
    e2e = [batch * steps / w for w in wall_all]
    pk = peaks()
    nkv, d, v = cfg["num_key_value_heads"], cfg["head_dim"], cfg["vocab_size"]
    layers = cfg["num_hidden_layers"]
    mean_context = CONTEXT - REPEATS * steps / 2
    achieved = step_bytes(cfg, layers, batch, mean_context) / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": f"decode tokens/s, Qwen3-0.6B sizes, batch {batch}, context {CONTEXT}",
        "value": round(batch / ms * 1e3, 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16", "data": "synthetic", "impl": "reference",
        "config": {
            "model": "Qwen3-0.6B sizes, random weights N(0,0.02)", "layers": layers, "layers_of_model": layers,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"], "kv_heads": nkv, "head_dim": d,
            "intermediate": cfg["intermediate_size"], "vocab": v, "tied_head": True, "global_batch": batch,
            "seq_len": CONTEXT, "page": PAGE, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (weights + cache per step)",
            "timing": f"median of {REPEATS} consecutive regions of --steps steps; contexts "
                      f"{start_len + 1 + warmup} to {CONTEXT}",
            "path": "engine.model.qwen3.Qwen3 + engine.sched.scheduler.Scheduler.step, its FixedChunkPolicy(512) "
                    "for the prompts, audit off",
        },
        "clocks": clock_info, "spread_ms_per_step": spread(ms_all),
        # the reference's step is synchronous (it reads every request's logits row on the host),
        # so the device-timed and the end-to-end rate are the same loop
        "e2e": {"value": round(statistics.median(e2e), 1), "unit": "tok/s",
                "h2d_bytes_per_step": batch * 16 + batch * layers * (CONTEXT // PAGE) * 4,
                "d2h_bytes_per_step": batch * v * 2},
        "gpu_launches": None,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }))
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
    ap.add_argument("--quick", action="store_true", help="the headline only: no points at other batches or in float32")
    ap.add_argument("--no-fp32", action="store_true", help="skip the float32 points")
    ap.add_argument("--only", default="", choices=["", "decode", "prefill"],
                    help="time only this part and print a short line (for profiling a small case)")
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed"],
                    help="mixed: a continuous batch of 64 requests through the entry point")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="element type of the --only runs (the full line always reports both)")
    ap.add_argument("--context", type=int, default=CONTEXT, help="context length of the decode steps (--only decode)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="tokens of the prompt that --only prefill runs in one step")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported by this engine")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "mixed":
        return run_mixed(args)
    return run_ours(args)


if __name__ == "__main__":
    raise SystemExit(main())
