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

LENGTHS = {"A": [70, 300, 37, 560, 129], "B": [45, 270, 90, 33, 520], "C": [100, 290, 64, 75, 200],
           "D": [70, 650, 260, 37, 330], "E": [45, 270, 600, 33, 140]}
# D and E have the sizes the tensor-core kernels take: their portions also go beyond 128 tokens
HOT = ("D", "E")


@pytest.fixture(scope="module")
def zoo(tmp_path_factory):
    """(config name, dtype) -> (folder, requests, plain logits by uid)."""
    cache = {}

    def get(name: str, dtype: str):
        key = (name, dtype)
        if key not in cache:
            config, _ = H.CONFIGS[name]
            folder = H.make_model_folder(tmp_path_factory.mktemp(f"m{name}{dtype}"), config,
                                         seed=11 + ord(name), dtype=dtype, init_std=H.INIT_STD[name])
            requests = {f"r{i}": H.random_tokens(n, config["vocab_size"], seed=100 * ord(name) + i)
                        for i, n in enumerate(LENGTHS[name])}
            plain = {uid: H.plain_logits(folder, toks).float() for uid, toks in requests.items()}
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


def make_plan(mode, name, requests):
    if name in HOT and mode in ("portions", "mixed"):
        return PLANS[mode](requests, sizes=H.SIZES_WIDE)
    return PLANS[mode](requests)


# kernels that a mode must have launched on the hot configurations in bfloat16
FIRED = {
    "whole": ["gemm_tc_rows_pair", "attention_prefill_tc", "qk_norm_rope_store_whole"],
    "bulk_then_single": ["gemm_tc_few", "gemm_tc_few_norm", "gemm_tc_few_qkv", "attention_decode_mma",
                         "attention_combine"],
    "portions": ["gemm_tc_few", "gemm_tc_few_qkv", "gemm_tc_cluster", "gemm_tc_rows_pair",
                 "attention_prefill_tc"],
    "mixed": ["gemm_tc_cluster", "gemm_tc_rows_pair", "attention_prefill_tc", "attention_decode_mma"],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("mode", list(PLANS))
def test_replay_matches_plain(zoo, name, dtype, mode):
    from lockstep_b200 import kernels as K

    folder, requests, plain = zoo(name, dtype)
    steps = make_plan(mode, name, requests)
    runner = make_runner(folder, name, dtype, steps)
    before = K.kernel_counts()
    rows = H.run_plan(runner, steps)
    after = K.kernel_counts()
    assert len(rows) == sum(len(t) for t in requests.values())
    H.assert_rows_close(rows, plain, dtype, f"{name}/{dtype}/{mode}", config=name)
    runner.cache.audit()
    assert runner.cache.free_pages() == runner.cache.total_pages()
    if name in HOT and dtype == "bfloat16":
        idle = [k for k in FIRED[mode] if after.get(k, 0) == before.get(k, 0)]
        assert not idle, f"{name}/{mode}: these kernels never ran: {idle}"
        if name == "D":
            assert after["gemm_tc_walk"] > before["gemm_tc_walk"], "the head product did not take the persistent kernel"
        if mode == "portions":
            assert any(len(t) > 128 for s in steps for _, t, _ in s["entries"])
            assert any(32 < len(t) <= 128 for s in steps for _, t, _ in s["entries"])
    if dtype == "float32":
        used = [k for k in after if after[k] != before.get(k, 0) and ("_tc" in k or "_mma" in k)]
        assert not used, f"a tensor-core kernel ran on the 32-bit path: {used}"
    if mode == "mixed":
        assert runner.cache.reused_pages() > 0, "the pool was too large: no page was used again"
        assert any(len(s["entries"]) > 1 and any(len(t) > 1 for _, t, _ in s["entries"])
                   and any(len(t) == 1 for _, t, _ in s["entries"]) for s in steps), \
            "no step held a portion beside a decoded token"
    if mode == "portions":
        assert any(len(t) == 2 for s in steps for _, t, _ in s["entries"])
    if mode == "bulk_then_single":
        assert runner.graphs is not None and runner.graphs.replays > 50, "decode steps were not replayed from graphs"


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_float32_cuttings_agree_bitwise(zoo, name):
    """In float32 every reduction's order is fixed by the row alone, so the bits agree."""
    folder, requests, _ = zoo(name, "float32")
    ref = None
    for mode in PLANS:
        steps = make_plan(mode, name, requests)
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
                assert np.abs(got[r] - ref).max() <= H.tolerance(dtype, plain[uid], "B"), (i, uid, start + w)
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
        H.assert_rows_close(rows, plain, dtype, f"token by token/{dtype}", config="A")


@pytest.mark.parametrize("name", ["D", "E"])
def test_prompt_attention_with_two_heads_a_block_gives_the_same_bits(zoo, name):
    """The tensor-core attention of prompts has a kernel with one query head a block and one with
    the two heads of a key head a block (taken where a launch has items enough); which one runs
    depends on the batch, so both must give every row the same bits."""
    from lockstep_b200 import kernels as K

    folder, requests, plain = zoo(name, "bfloat16")
    rows = {}
    try:
        for mode in (0, 2):
            K.set_attention_prefill_pairs(mode)
            steps = make_plan("portions", name, requests)
            rows[mode] = H.run_plan(make_runner(folder, name, "bfloat16", steps), steps)
    finally:
        K.set_attention_prefill_pairs(1)
    H.assert_rows_close(rows[2], plain, "bfloat16", f"{name}/two heads a block", config=name)
    assert rows[0].keys() == rows[2].keys()
    for key in rows[0]:
        assert torch.equal(rows[0][key], rows[2][key]), key


@pytest.mark.parametrize("name", ["D", "E"])
def test_bfloat16_rows_do_not_depend_on_the_neighbours(zoo, name):
    """One request, cut the same way, alone and beside other requests of other lengths (so that
    its products run in other kernels and its rows lie elsewhere in the batch): the same bits.
    Every sum's order is a function of the row alone, in bfloat16 too."""
    folder, requests, _ = zoo(name, "bfloat16")
    uid, toks = "r2", requests["r2"]
    cuts = [140, 30, 9] + [1] * 24                       # a long portion, shorter ones, then decoding
    mine, at = [], 0
    for n in cuts:
        mine.append((uid, toks[at:at + n], list(range(n))))
        at += n
    alone = [{"entries": [m], "end": []} for m in mine]
    alone[-1]["end"] = [uid]
    others = {"r1": requests["r1"], "r4": requests["r4"], "r0": requests["r0"]}
    # neighbours: a portion of 150 beside the first step (many-token kernel), 40 beside the second
    # (64-token tiles), decoded tokens and small portions beside the rest
    beside = []
    pos = {u: 0 for u in others}
    plan = [[("r1", 150)], [("r4", 40)], [("r0", 3), ("r1", 1)]] + [[("r1", 1), ("r4", 1), ("r0", 1)]] * 24
    for m, extra in zip(mine, plan):
        entries = []
        for u, n in extra[:1]:                           # one neighbour before, the others after
            entries.append((u, others[u][pos[u]:pos[u] + n], []))
            pos[u] += n
        entries.append(m)
        for u, n in extra[1:]:
            entries.append((u, others[u][pos[u]:pos[u] + n], []))
            pos[u] += n
        beside.append({"entries": entries, "end": []})
    beside[-1]["end"] = [uid, *others]
    rows_alone = H.run_plan(make_runner(folder, name, "bfloat16", alone), alone)
    rows_beside = H.run_plan(make_runner(folder, name, "bfloat16", beside), beside)
    assert len(rows_alone) == sum(cuts)
    for key, row in rows_alone.items():
        assert torch.equal(row, rows_beside[key]), f"position {key[1]} of {uid} changes with its neighbours"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D", "E"])
def test_steps_of_mixed_portions_are_recorded_when_their_shape_repeats(zoo, name, dtype):
    """Steps of the same shape (a step that fills a token budget, say) come again and again: from
    the second on they are recorded, later ones replay the recording.  Whole prompts of equal
    length one after the other, then portions beside decoded tokens of three other requests: the
    rows agree with the plain implementation and, bit for bit, with a runner that records nothing."""
    from lockstep_b200.engine import ModelRunner

    folder, _, _ = zoo(name, dtype)
    config, page = H.CONFIGS[name]
    vocab = config["vocab_size"]
    n = 320
    prompts = {u: H.random_tokens(n + 8, vocab, seed=900 + i) for i, u in enumerate("abcdefgh")}
    plain = {u: H.plain_logits(folder, t).float() for u, t in prompts.items()}
    plain["x"] = plain["y"] = plain["a"]
    steps = []
    for u in "abc":                                     # whole prompts, one a step: the same shape thrice
        steps.append({"entries": [(u, prompts[u][:n], [n - 1])], "end": []})
    for u in "xy":                                      # and twice more, by requests that end at once
        steps.append({"entries": [(u, prompts["a"][:n], [0, n - 1])], "end": [u]})
    at = {u: n for u in "abc"}
    for k, u in enumerate("defgh"):                     # a portion of 317 beside three decoded tokens, five times
        entries = [(v, prompts[v][at[v]:at[v] + 1], [0]) for v in "abc"]
        for v in "abc":
            at[v] += 1
        entries.insert(1, (u, prompts[u][:n - 3], [n - 4]))
        steps.append({"entries": entries, "end": [u]})
    steps[-1]["end"] = ["h", "a", "b", "c"]
    rows = {}
    for graphs in (True, False):
        runner = ModelRunner(folder, dtype=dtype, num_pages=4 * (-(-(n + 8) // page)) + 2, page_size=page,
                             max_live=4, max_seq_len=1024, use_graphs=graphs)
        rows[graphs] = H.run_plan(runner, steps)
        if graphs:
            assert runner.graphs.mixed_replays == 2 + 2, runner.graphs.mixed_replays
            assert len(runner.graphs.mixed) == 2
        runner.cache.audit()
    H.assert_rows_close(rows[True], plain, dtype, f"{name}/{dtype}/recorded mixed steps", config=name)
    assert rows[True].keys() == rows[False].keys()
    for key in rows[True]:
        assert torch.equal(rows[True][key], rows[False][key]), key
