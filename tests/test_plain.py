"""The plain implementation against LockStep's own CPU code (committed golden files)."""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors.torch import load_file

from plain import qwen3_plain as plain

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_logits_match_lockstep_fp64_reference():
    want = load_file(str(GOLDEN / "lockstep_fp64_outputs.safetensors"))
    prompts = json.loads((GOLDEN / "prompts.json").read_text())
    cfg, w = plain.read_model_folder(GOLDEN / "tiny_model", torch.float64)
    for name, ids in prompts.items():
        hidden = plain.hidden_states(cfg, w, ids, torch.float64)
        logits = plain.logits(cfg, w, ids, torch.float64)
        assert torch.allclose(hidden, want[f"hidden_{name}"], rtol=0, atol=1e-11)
        assert torch.allclose(logits, want[f"logits_{name}"], rtol=0, atol=1e-11)


def test_float32_plain_is_close_to_float64_plain():
    prompts = json.loads((GOLDEN / "prompts.json").read_text())
    cfg, w64 = plain.read_model_folder(GOLDEN / "tiny_model", torch.float64)
    _, w32 = plain.read_model_folder(GOLDEN / "tiny_model", torch.float32)
    a = plain.logits(cfg, w64, prompts["a"], torch.float64)
    b = plain.logits(cfg, w32, prompts["a"], torch.float32)
    assert (a - b.double()).abs().max() < 2e-4


def test_sampler_matches_lockstep_draws():
    draws = json.loads((GOLDEN / "lockstep_sampler_draws.json").read_text())
    for d in draws["uniform"]:
        assert plain.uniform(d["seed"], d["uid"], d["position"]) == d["value"]
    for d in draws["philox_4x32"]:
        assert list(plain.philox_4x32(tuple(d["counter"]), tuple(d["key"]))) == d["words"]
    want = load_file(str(GOLDEN / "lockstep_fp64_outputs.safetensors"))
    row = want["logits_a"][-1]
    assert plain.sample_top_p(row, 0, "r", 0, temperature=0.0) == draws["greedy_last_row_a"]
    for d in draws["top_p"]:
        got = plain.sample_top_p(row, d["seed"], d["uid"], d["position"], p=d["p"],
                                 temperature=d["temperature"])
        assert got == d["token"]


def test_window_masks_far_keys():
    torch.manual_seed(0)
    q = torch.randn(6, 2, 8, dtype=torch.float64)
    k = torch.randn(6, 1, 8, dtype=torch.float64)
    v = torch.randn(6, 1, 8, dtype=torch.float64)
    full = plain.causal_attention(q, k, v, 0.3)
    win = plain.causal_attention(q, k, v, 0.3, window=3)
    assert torch.allclose(full[:3], win[:3])
    assert not torch.allclose(full[5], win[5])
    tail = plain.causal_attention(q[5:], k[3:], v[3:], 0.3)
    assert torch.allclose(tail[0], win[5])
