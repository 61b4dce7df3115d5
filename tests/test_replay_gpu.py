"""Replay of the same requests cut in different ways, against the plain implementation.

Modes: each request alone and whole; most of it in one step and the last 32
tokens one by one; in portions of changing size, down to two tokens; and mixed,
up to four live requests, portions of some beside decoded tokens of others,
with so few pages that they are used again.  In float32 and in bfloat16.
"""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent

LENGTHS = {"A": [70, 300, 37, 560, 129], "B": [45, 270, 90, 33, 520], "C": [100, 290, 64, 75, 200]}


@pytest.fixture(scope="module")
def zoo(tmp_path_factory):
    """(config name, dtype) -> (folder, requests, plain logits by uid)."""
    cache = {}

    def get(name: str, dtype: str):
        key = (name, dtype)
        if key not in cache:
            config, _ = H.CONFIGS[name]
            folder = H.make_model_folder(tmp_path_factory.mktemp(f"m{name}{dtype}"), config,
                                         seed=11 + ord(name), dtype=dtype)
            requests = {f"r{i}": H.random_tokens(n, config["vocab_size"], seed=100 * ord(name) + i)
                        for i, n in enumerate(LENGTHS[name])}
            plain = {uid: H.plain_logits(folder, toks) for uid, toks in requests.items()}
            cache[key] = (folder, requests, plain)
        return cache[key]

    return get


def make_runner(folder, name, dtype, steps, slack_pages=0):
    from lockstep_b200.engine import ModelRunner

    page = H.CONFIGS[name][1]
    tokens = H.max_live_tokens(steps, round_to=page)
    return ModelRunner(folder, dtype=dtype, num_pages=tokens // page + slack_pages, page_size=page,
                       max_live=4, max_seq_len=1024)


PLANS = {
    "whole": H.plan_whole,
    "bulk_then_single": H.plan_bulk_then_single,
    "portions": H.plan_portions,
    "mixed": H.plan_mixed,
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("mode", list(PLANS))
def test_replay_matches_plain(zoo, name, dtype, mode):
    folder, requests, plain = zoo(name, dtype)
    steps = PLANS[mode](requests)
    runner = make_runner(folder, name, dtype, steps)
    rows = H.run_plan(runner, steps)
    assert len(rows) == sum(len(t) for t in requests.values())
    H.assert_rows_close(rows, plain, dtype, f"{name}/{dtype}/{mode}")
    runner.cache.audit()
    assert runner.cache.free_pages() == runner.cache.total_pages()
    if mode == "mixed":
        assert runner.cache.reused_pages() > 0, "the pool was too large: no page was used again"
        assert any(len(s["entries"]) > 1 and any(len(t) > 1 for _, t, _ in s["entries"])
                   and any(len(t) == 1 for _, t, _ in s["entries"]) for s in steps), \
            "no step held a portion beside a decoded token"
    if mode == "portions":
        assert any(len(t) == 2 for s in steps for _, t, _ in s["entries"])
    if mode == "bulk_then_single":
        assert runner.graphs is not None and runner.graphs.replays > 50, "decode steps were not replayed from graphs"


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_float32_cuttings_agree_bitwise(zoo, name):
    """In float32 every reduction's order is fixed by the row alone, so the bits agree."""
    folder, requests, _ = zoo(name, "float32")
    ref = None
    for mode, plan in PLANS.items():
        steps = plan(requests)
        rows = H.run_plan(make_runner(folder, name, "float32", steps), steps)
        if ref is None:
            ref = rows
            continue
        for key, row in rows.items():
            assert torch.equal(row, ref[key]), f"{mode}: request {key[0]} position {key[1]} differs in bits"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(zoo, tmp_path, dtype):
    """The program itself, as a user runs it: stdin in, files and ``done`` lines out."""
    folder, requests, plain = zoo("B", dtype)
    steps = H.plan_mixed(requests, seed=3)
    out = tmp_path / "logits"
    env = dict(os.environ)
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(H.max_live_tokens(steps)), "--page-size", "8"],
        input=H.plan_to_jsonl(steps), capture_output=True, text=True, env=env, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(steps))]
    vocab = H.TINY_B["vocab_size"]
    held: dict[str, int] = {}
    for i, step in enumerate(steps):
        got = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, vocab)
        r = 0
        for uid, toks, want in step["entries"]:
            start = held.get(uid, 0)
            for w in want:
                ref = plain[uid][start + w].float().numpy()
                assert np.abs(got[r] - ref).max() <= H.tolerance(dtype, plain[uid]), (i, uid, start + w)
                r += 1
            held[uid] = start + len(toks)
        assert r == got.shape[0]


def test_long_decoding_and_first_tokens(zoo):
    """Token-by-token from the very first token, across page and split edges."""
    for dtype in ("float32", "bfloat16"):
        folder, requests, plain = zoo("A", dtype)
        toks = requests["r1"]           # 300 tokens: crosses the 256-token split
        steps = [{"entries": [("r1", toks[i:i + 1], [0])], "end": ["r1"] if i == len(toks) - 1 else []}
                 for i in range(len(toks))]
        rows = H.run_plan(make_runner(folder, "A", dtype, steps), steps)
        H.assert_rows_close(rows, plain, dtype, f"token by token/{dtype}")
