"""What ``bench.py`` promises without a device: one GPU only, the bytes and flops its roofline
fractions are made of, and a flat ``config`` record of at most 20 keys."""

from __future__ import annotations

import argparse
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import bench  # noqa: E402


def test_more_than_one_gpu_is_refused_with_one_line():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--gpus", "2"], capture_output=True, text=True)
    assert proc.returncode == 2
    assert len(proc.stdout.strip().splitlines()) == 1 and "one GPU" in proc.stdout


def test_bytes_of_a_decode_step_and_flops_of_a_prefill():
    cfg = dict(bench.QWEN3_0_6B)
    # Qwen3-0.6B in bfloat16: 31.46 MB of weights a layer x 28 + the head's 311.2 MB = 1.192 GB,
    # and 114,688 bytes of keys and values per token of context and request
    weights = bench.step_bytes(cfg, 28, 1, 0)
    assert abs(weights - 1.192e9) < 2e6
    per_token = bench.step_bytes(cfg, 28, 1, 1) - weights
    assert per_token == 114688
    assert bench.step_bytes(cfg, 28, 8, 4096) == weights + 8 * 4096 * per_token
    assert bench.step_bytes(cfg, 28, 8, 4096, elem=4) == 2 * bench.step_bytes(cfg, 28, 8, 4096)
    # a prefill of 2,048 tokens: 1.804 TFLOP of products + 0.481 of attention (counted causally) + the head's row
    flops = bench.prefill_flops(cfg, 28, 2048)
    assert abs(flops - 2.285e12) < 0.01e12
    big = dict(cfg)
    big.update(bench.SIZES["qwen3-8b"])
    assert abs(bench.step_bytes(big, 36, 1, 0) - 15.14e9) < 0.05e9      # untied head: the table is only gathered from


def test_the_config_record_is_flat_and_short():
    args = argparse.Namespace(batch=8, model="qwen3-8b", layers=4)
    cfg, label, layers_full = bench.model_config(args)
    record = bench.config_record(cfg, label, layers_full, args, bench.peaks())
    assert len(record) <= 20
    assert all(not isinstance(v, (dict, list, tuple)) for v in record.values())
    assert record["layers"] == 4 and record["layers_of_model"] == 36 and record["tied_head"] is False
    assert record["hidden"] == 4096 and record["global_batch"] == 8 and record["seq_len"] == bench.CONTEXT
    assert len(record["kernel_constants_sha256"]) == 64
