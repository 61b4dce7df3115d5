"""Generation through the Python entry point against the plain implementation."""

from __future__ import annotations

import pytest
import torch

import helpers as H
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


def check_tokens(folder, prompt, generated, dtype, sampling=None):
    """Every generated token is the plain implementation's choice on the same
    context, or (for greedy) within rounding of its best logit."""
    cfg, w = plain.read_model_folder(folder, torch.float64)
    ids = list(prompt)
    for i, tok in enumerate(generated):
        row = plain.logits(cfg, w, ids, torch.float64)[-1]
        if sampling is None:
            margin = 1e-3 if dtype == "float32" else 0.05 * (1 + float(row.abs().max()))
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
        check_tokens(folder, prompt, out[uid], dtype,
                     sampling={"seed": 77, "uid": uid, "top_p": 0.95, "temperature": 0.7})
    assert len({tuple(v) for v in out.values()}) == 3


def test_preemption_and_prefix_reuse_do_not_change_the_tokens(tmp_path):
    from lockstep_b200 import Engine, Request

    dtype = "float32"
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
    assert tight == roomy
    cached, engine = run(num_pages=64, enable_prefix_cache=True)
    again = engine.generate([Request(uid="again", prompt=prompts["p3"], max_new_tokens=24)])
    assert cached == roomy and again["again"] == roomy["p3"]
    assert any(e[1] == "cache_hit" for e in engine.scheduler.events)


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
