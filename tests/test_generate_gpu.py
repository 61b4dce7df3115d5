"""Generation through the Python entry point against the plain implementation."""

from __future__ import annotations

import pytest
import torch

import helpers as H
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


def check_tokens(folder, prompt, generated, dtype, sampling=None, config="A"):
    """Every generated token is the plain implementation's choice on the same
    context, or (for greedy) within the engine's error bound of its best logit: the
    chosen logit and the best one may each be off by the bound."""
    cfg, w = plain.read_model_folder(folder, torch.float64)
    ids = list(prompt)
    for i, tok in enumerate(generated):
        row = plain.logits(cfg, w, ids, torch.float64)[-1]
        if sampling is None:
            margin = 2 * H.tolerance(dtype, row, config)
            assert float(row[tok]) >= float(row.max()) - margin, (i, tok, int(row.argmax()))
        else:
            want = plain.sample_top_p(row, sampling["seed"], sampling["uid"], len(ids) - 1,
                                      p=sampling["top_p"], temperature=sampling["temperature"])
            assert tok == want, (i, tok, want)
        ids.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_tiny_a(tmp_path, dtype):
    """Tiny A: prompts of 1, 7, 33 and 64 tokens, 16 greedy tokens each, all at once."""
    from lockstep_b200 import Engine, Request

    folder = H.make_model_folder(tmp_path, H.TINY_A, seed=21, dtype=dtype)
    engine = Engine(folder, dtype=dtype, num_pages=24, page_size=H.PAGE_A, max_running=4, audit=True)
    prompts = {f"r{i}": H.random_tokens(n, 256, 40 + i) for i, n in enumerate([1, 7, 33, 64])}
    out = engine.generate([Request(uid=u, prompt=p, max_new_tokens=16) for u, p in prompts.items()])
    for uid, prompt in prompts.items():
        assert len(out[uid]) == 16
        check_tokens(folder, prompt, out[uid], dtype)
    assert engine.cache.free_pages() == engine.cache.total_pages()
    one = engine.generate_greedy(prompts["r2"], 16)
    if dtype == "float32":
        assert one == out["r2"]          # alone or in a batch: the same tokens


def test_temperature_sampling_tiny_b_chunked(tmp_path):
    """Tiny B: prompts of 5, 19 and 40 tokens, 12 tokens at temperature 0.7 with a
    fixed seed, prompts cut into portions of 8 beside the others' decoded tokens."""
    from lockstep_b200 import Engine, Request
    from lockstep_b200.engine import FixedChunkPolicy

    dtype = "float32"
    folder = H.make_model_folder(tmp_path, H.TINY_B, seed=22, dtype=dtype)
    engine = Engine(folder, dtype=dtype, num_pages=32, page_size=H.PAGE_B, max_running=4,
                    policy=FixedChunkPolicy(8), audit=True)
    prompts = {f"s{i}": H.random_tokens(n, 500, 50 + i) for i, n in enumerate([5, 19, 40])}
    reqs = [Request(uid=u, prompt=p, seed=77, max_new_tokens=12, temperature=0.7, top_p=0.95)
            for u, p in prompts.items()]
    out = engine.generate(reqs)
    assert engine.scheduler.stats["mixed_steps"] > 0
    for uid, prompt in prompts.items():
        check_tokens(folder, prompt, out[uid], dtype, config="B",
                     sampling={"seed": 77, "uid": uid, "top_p": 0.95, "temperature": 0.7})
    assert len({tuple(v) for v in out.values()}) == 3


def test_portions_of_prompts_beside_decoded_tokens_in_bfloat16(tmp_path):
    """The fixed-portion policy on the device in bfloat16: portions of 8 beside decoded tokens."""
    from lockstep_b200 import Engine, Request
    from lockstep_b200.engine import FixedChunkPolicy

    folder = H.make_model_folder(tmp_path, H.TINY_B, seed=26, dtype="bfloat16")
    engine = Engine(folder, dtype="bfloat16", num_pages=32, page_size=H.PAGE_B, max_running=4,
                    policy=FixedChunkPolicy(8), audit=True)
    prompts = {f"s{i}": H.random_tokens(n, 500, 80 + i) for i, n in enumerate([5, 19, 40])}
    out = engine.generate([Request(uid=u, prompt=p, max_new_tokens=12) for u, p in prompts.items()])
    assert engine.scheduler.stats["mixed_steps"] > 0
    for uid, prompt in prompts.items():
        check_tokens(folder, prompt, out[uid], "bfloat16", config="B")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_and_prefix_reuse_do_not_change_the_tokens(tmp_path, dtype):
    from lockstep_b200 import Engine, Request

    folder = H.make_model_folder(tmp_path, H.TINY_A, seed=23, dtype=dtype)
    shared = H.random_tokens(48, 256, 7)
    prompts = {f"p{i}": shared + H.random_tokens(5 + 9 * i, 256, 60 + i) for i in range(4)}

    def run(**kw):
        engine = Engine(folder, dtype=dtype, page_size=H.PAGE_A, max_running=4, audit=True, **kw)
        out = engine.generate([Request(uid=u, prompt=p, max_new_tokens=24) for u, p in prompts.items()])
        return out, engine

    roomy, _ = run(num_pages=64)
    tight, engine = run(num_pages=13, max_step_tokens=32)
    assert engine.scheduler.stats["preemptions"] > 0 and engine.cache.reused_pages() > 0
    cached, engine = run(num_pages=64, enable_prefix_cache=True)
    again = engine.generate([Request(uid="again", prompt=prompts["p3"], max_new_tokens=24)])
    assert any(e[1] == "cache_hit" for e in engine.scheduler.events)
    if dtype == "float32":
        # every row has the same bits however it was reached, so the tokens are the same
        assert tight == roomy
        assert cached == roomy and again["again"] == roomy["p3"]
    else:
        # a preempted request's decoded positions are computed again as a prompt, by the prompt
        # kernels: the same values beyond rounding, so each run is checked against the plain one
        for out in (roomy, tight, cached):
            for uid, prompt in prompts.items():
                check_tokens(folder, prompt, out[uid], dtype)
        check_tokens(folder, prompts["p3"], again["again"], dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_layers_through_the_entry_point_reuse_pages_behind_the_window(tmp_path, dtype):
    """Configuration C (two of three layers read a window of 40 keys) through the scheduler, with
    a pool so small that the pages a window has passed are taken again while requests still run."""
    from lockstep_b200 import Engine, Request

    folder = H.make_model_folder(tmp_path, H.TINY_C, seed=27, dtype=dtype)
    prompts = {f"w{i}": H.random_tokens(n, H.TINY_C["vocab_size"], 90 + i) for i, n in enumerate([150, 70, 101])}
    # all keys: 3 requests x up to 7 pages of 32; the pool holds 22 and the windowed group frees as it goes
    engine = Engine(folder, dtype=dtype, num_pages=22, page_size=H.PAGE_C, max_running=3, max_step_tokens=48,
                    max_seq_len=256, audit=True)
    assert len(engine.cache.paged) == 2
    out = engine.generate([Request(uid=u, prompt=p, max_new_tokens=60) for u, p in prompts.items()])
    windowed = [g for g in engine.cache.paged if g.window][0]
    assert windowed.allocator.stats["freed"] > 0 and windowed.allocator.stats["reused"] > 0
    for uid, prompt in prompts.items():
        assert len(out[uid]) == 60
        check_tokens(folder, prompt, out[uid], dtype, config="C")
    assert engine.cache.free_pages() == engine.cache.total_pages()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefix_reuse_with_windowed_layers_serves_the_next_turn(tmp_path, dtype):
    """Configuration C (a group that keeps all keys, a group with a window of 40) with prefix
    reuse: the next turn of a finished conversation adopts the whole prefix (in the windowed
    group only the window's pages are left, and only they are needed), pages that were freed
    are poisoned, and the tokens are those of a run without reuse."""
    from lockstep_b200 import Engine, Request

    folder = H.make_model_folder(tmp_path, H.TINY_C, seed=31, dtype=dtype)
    vocab = H.TINY_C["vocab_size"]
    first = H.random_tokens(150, vocab, 120)

    def run(**kw):
        engine = Engine(folder, dtype=dtype, num_pages=40, page_size=H.PAGE_C, max_running=2, max_step_tokens=64,
                        max_seq_len=320, audit=True, **kw)
        a = engine.generate([Request(uid="turn1", prompt=first, max_new_tokens=30)])["turn1"]
        follow = first + a + H.random_tokens(21, vocab, 121)
        b = engine.generate([Request(uid="turn2", prompt=follow, max_new_tokens=30)])["turn2"]
        return a, follow, b, engine

    a0, follow0, b0, _ = run()
    a1, follow1, b1, engine = run(enable_prefix_cache=True, poison_freed_pages=True)
    hits = [e for e in engine.scheduler.events if e[1] == "cache_hit"]
    assert len(hits) == 1 and hits[0][2] == "turn2"
    held = (len(first) + 30 - 1) // H.PAGE_C * H.PAGE_C          # whole pages of what turn 1 fed
    assert hits[0][3] == (held,)
    windowed = [g for g in engine.cache.paged if g.window][0]
    assert windowed.poisoned > 0
    if dtype == "float32":
        assert (a1, b1) == (a0, b0)                              # the same bits however a row was reached
    assert follow1[:len(first)] == first
    check_tokens(folder, first, a1, dtype, config="C")
    check_tokens(folder, follow1, b1, dtype, config="C")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_command_line_runs_a_workload(tmp_path, dtype):
    """``bin/lockstep run --workload``: a model folder and a file of requests in, token ids out."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    folder = H.make_model_folder(tmp_path, H.TINY_B, seed=28, dtype=dtype)
    prompts = {f"c{i}": H.random_tokens(n, 500, 95 + i) for i, n in enumerate([4, 23, 50])}
    workload = tmp_path / "workload.json"
    workload.write_text(json.dumps([{"uid": u, "prompt": p, "max_new_tokens": 10} for u, p in prompts.items()]))
    proc = subprocess.run(
        [sys.executable, str(root / "bin" / "lockstep"), "run", "--model", str(folder), "--dtype", dtype,
         "--workload", str(workload), "--policy", "fixed-chunk:16", "--num-blocks", "40", "--block-size", "8",
         "--max-running", "4"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]
    assert [l["uid"] for l in lines] == list(prompts)
    for line in lines:
        assert line["prompt_tokens"] == len(prompts[line["uid"]]) and len(line["generated"]) == 10
        check_tokens(folder, prompts[line["uid"]], line["generated"], dtype, config="B")
    assert "3 requests" in proc.stderr


def test_two_runs_have_the_same_trajectory_and_poisoned_pages_change_nothing(tmp_path):
    """The per-step record (work, tokens, logits bytes, cache digests) of two runs of the same
    requests agrees; with freed pages filled with the poison value, and so few pages that they
    are used again at once, the tokens and the logits bytes are still the same: no kernel gives
    weight to a key beyond a request's length."""
    from lockstep_b200 import Engine, Request

    for dtype in ("float32", "bfloat16"):
        folder = H.make_model_folder(tmp_path, H.TINY_A, seed=29, dtype=dtype)
        prompts = {f"t{i}": H.random_tokens(n, 256, 110 + i) for i, n in enumerate([30, 9, 47, 18, 5, 64])}

        def run(**kw):
            engine = Engine(folder, dtype=dtype, num_pages=14, page_size=H.PAGE_A, max_running=3,
                            max_step_tokens=40, trajectory=True, **kw)
            out = engine.generate([Request(uid=u, prompt=p, max_new_tokens=20) for u, p in prompts.items()])
            return out, engine

        out_a, a = run()
        out_b, b = run()
        out_p, p = run(poison_freed_pages=True)
        assert a.scheduler.trajectory.steps > 20
        assert a.scheduler.trajectory.first_divergence(b.scheduler.trajectory) is None
        assert a.scheduler.trajectory.hexdigest() == b.scheduler.trajectory.hexdigest()
        assert a.cache.reused_pages() > 0 and p.cache.paged[0].poisoned > 0
        assert out_p == out_a
        assert a.scheduler.trajectory.first_divergence(p.scheduler.trajectory) is None


def test_forward_batch_gives_logits_for_every_position(tmp_path):
    from lockstep_b200 import Engine

    folder = H.make_model_folder(tmp_path, H.TINY_B, seed=24, dtype="float32")
    engine = Engine(folder, dtype="float32", num_pages=16, page_size=H.PAGE_B)
    toks = H.random_tokens(21, 500, 3)
    a = engine.forward_batch([("x", toks[:13], 0)])["x"]
    b = engine.forward_batch([("x", toks[13:], 13)])["x"]
    engine.release("x")
    want = H.plain_logits(folder, toks)
    got = torch.cat([a, b]).cpu()
    assert (got - want.float()).abs().max() <= H.tolerance("float32", want)


def test_a_fault_in_a_kernel_is_reported(tmp_path):
    from lockstep_b200 import ModelRunner, StepEntry
    from lockstep_b200.kernels import KernelError

    folder = H.make_model_folder(tmp_path, H.TINY_A, seed=25, dtype="float32")
    runner = ModelRunner(folder, dtype="float32", num_pages=8, page_size=16)
    runner.open("a")
    with pytest.raises(KernelError, match="token id outside"):
        runner.step([StepEntry("a", [1, 999, 2], 0, [2])])
    runner.close("a")
    runner.open("b")                     # the engine stays usable
    assert runner.step([StepEntry("b", [1, 2], 0, [1])]).shape == (1, 256)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_give_the_same_tokens(tmp_path, dtype):
    """Decode steps launched before the tokens of the step before are on the host (their ids
    are taken on the device) against steps planned one by one: greedy and sampled requests
    side by side, one of them ending on an end token while the next step is under way."""
    from lockstep_b200 import Engine, Request

    folder = H.make_model_folder(tmp_path, H.TINY_B, seed=31, dtype=dtype)
    prompts = {f"a{i}": H.random_tokens(n, 500, 70 + i) for i, n in enumerate([6, 21, 40])}

    def requests(new):
        return [Request(uid=u, prompt=p, seed=5, max_new_tokens=new, temperature=0.8 if u == "a1" else 0.0,
                        top_p=0.9) for u, p in prompts.items()]

    def run(eos, **kw):
        engine = Engine(folder, dtype=dtype, num_pages=48, page_size=H.PAGE_B, max_running=4,
                        eos_token_ids=eos, **kw)
        out = engine.generate(requests(40))
        assert engine.cache.free_pages() == engine.cache.total_pages()
        return out, engine.scheduler.stats["launched_ahead"]

    one_by_one, ahead = run(None, audit=True)          # the audit after every step rules run-ahead out
    assert ahead == 0
    free, ahead = run(None)
    assert ahead > 20 and free == one_by_one
    check_tokens(folder, prompts["a0"], free["a0"], dtype)
    check_tokens(folder, prompts["a1"], free["a1"][:12], dtype,
                 sampling={"seed": 5, "uid": "a1", "top_p": 0.9, "temperature": 0.8}) if dtype == "float32" else None
    # an end token in the middle of a0's tokens
    eos = one_by_one["a0"][17]
    cut = one_by_one["a0"][:one_by_one["a0"].index(eos) + 1]
    ended, ahead = run([eos])
    assert ahead > 0 and ended["a0"] == cut
    planned, _ = run([eos], audit=True)
    assert ended == planned
