"""Tiny configurations, model folders and replay plans shared by the tests.

The two main configurations differ in every size and option: layers, width,
heads and groups, head size, feed-forward width, vocabulary, rope theta, eps,
tied or untied head, page size.  A third adds windowed layers.
"""

from __future__ import annotations

import json
import os
import random
from pathlib import Path

import torch

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 2048,
}
PAGE_A = 16

TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 80, "num_attention_heads": 4, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 200, "vocab_size": 500, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 2048,
}
PAGE_B = 8

# windowed layers (1 and 2 of 3), 6 query heads in 3 groups, head size 48
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 72, "num_attention_heads": 6, "num_key_value_heads": 3,
    "head_dim": 48, "intermediate_size": 136, "vocab_size": 311, "rope_theta": 50000.0,
    "rms_norm_eps": 3e-6, "tie_word_embeddings": False, "max_position_embeddings": 2048,
    "use_sliding_window": True, "sliding_window": 40, "max_window_layers": 1,
}
PAGE_C = 32

# The sizes the tensor-core kernels are built for, two layers deep: the layer sizes of
# Qwen3-0.6B (head size 128, groups of 2) with a vocabulary cut to a prime that still gives
# the head product one share of K, and a second one that differs in every size and option
# (head size 64, groups of 4, untied head whose product is shared out, page 8).
HOT_D = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 1024, "num_attention_heads": 16, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 3072, "vocab_size": 10007, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 2048,
}
PAGE_D = 16
HOT_E = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 512, "num_attention_heads": 8, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 1536, "vocab_size": 3001, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 2048,
}
PAGE_E = 8

CONFIGS = {"A": (TINY_A, PAGE_A), "B": (TINY_B, PAGE_B), "C": (TINY_C, PAGE_C),
           "D": (HOT_D, PAGE_D), "E": (HOT_E, PAGE_E)}
# standard deviation of the random matrices: about 1 / sqrt(width), so that no part of a layer
# drowns the others
INIT_STD = {"A": 0.3, "B": 0.3, "C": 0.3, "D": 0.04, "E": 0.06}


def make_model_folder(tmp_path: Path, config: dict, seed: int, dtype: str, init_std: float = 0.3,
                      gain_std: float = 0.1) -> Path:
    """A model folder under ``tmp_path`` written by the engine's random-weights mode."""
    from lockstep_b200.weights import write_random_model

    folder = Path(tmp_path) / f"model-{seed}-{dtype}"
    return write_random_model(folder, config, seed=seed, dtype=dtype, init_std=init_std,
                              gain_std=gain_std)


def random_tokens(n: int, vocab: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def plain_logits(folder: Path, tokens: list[int], compute=torch.float64) -> torch.Tensor:
    from plain import qwen3_plain as plain

    return plain.model_logits(folder, tokens, compute)


# ---------------------------------------------------------------------------
# replay plans: lists of steps {"entries": [(uid, tokens, want)], "end": [uid]}
# ---------------------------------------------------------------------------

def plan_whole(requests: dict[str, list[int]]):
    steps = []
    for uid, toks in requests.items():
        steps.append({"entries": [(uid, toks, list(range(len(toks))))], "end": [uid]})
    return steps


def plan_bulk_then_single(requests: dict[str, list[int]], tail: int = 32):
    steps = []
    for uid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"entries": [(uid, toks[:head], list(range(head)))], "end": []})
        for i in range(head, len(toks)):
            steps.append({"entries": [(uid, toks[i:i + 1], [0])], "end": [uid] if i == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [uid]
    return steps


SIZES_WIDE = (7, 2, 150, 17, 3, 33, 2, 5, 64, 1, 2, 100, 40, 129)   # also more than 128 tokens a portion


def plan_portions(requests: dict[str, list[int]], sizes=(7, 2, 17, 3, 33, 2, 5, 64, 1, 2)):
    steps = []
    for uid, toks in requests.items():
        i, k = 0, 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            steps.append({"entries": [(uid, toks[i:i + n], list(range(n)))],
                          "end": [uid] if i + n == len(toks) else []})
            i += n
    return steps


def plan_mixed(requests: dict[str, list[int]], prompt_fraction: float = 0.6, max_live: int = 4,
               sizes=(5, 2, 11, 3, 24, 2, 9), seed: int = 0):
    """Up to ``max_live`` requests at a time.  The first part of each request is
    fed in portions of changing size (as a prompt), the rest one token a step (as
    decoding), so steps hold portions of some beside single tokens of others.
    A finished request is ended at once and the next one starts, so that its
    pages are handed to the newcomer."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, dict] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            uid, toks = waiting.pop(0)
            live[uid] = {"toks": toks, "at": 0, "prompt": max(1, int(len(toks) * prompt_fraction)),
                         "k": rng.randrange(len(sizes))}
        entries, end = [], []
        for uid, st in list(live.items()):
            toks, at = st["toks"], st["at"]
            if rng.random() < 0.15 and len(live) > 1 and len(entries) > 0:
                continue   # this request sits the step out
            if at < st["prompt"]:
                n = min(sizes[st["k"] % len(sizes)], st["prompt"] - at)
                st["k"] += 1
            else:
                n = 1
            entries.append((uid, toks[at:at + n], list(range(n))))
            st["at"] = at + n
            if st["at"] == len(toks):
                end.append(uid)
                del live[uid]
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


def run_plan(runner, steps) -> dict[tuple[str, int], torch.Tensor]:
    """Drive ``runner.step`` through a plan; returns logits rows by (uid, position)."""
    from lockstep_b200.engine import StepEntry

    rows: dict[tuple[str, int], torch.Tensor] = {}
    live: set[str] = set()
    for step in steps:
        entries = []
        for uid, toks, want in step["entries"]:
            if uid not in live:
                runner.open(uid)
                live.add(uid)
            entries.append(StepEntry(uid=uid, tokens=list(toks), start=runner.kv_len(uid), want=list(want)))
        logits = runner.step(entries).float().cpu()
        r = 0
        for e in entries:
            for w in e.want:
                rows[(e.uid, e.start + w)] = logits[r]
                r += 1
        assert r == logits.shape[0]
        for uid in step["end"]:
            runner.close(uid)
            live.discard(uid)
    assert not live
    return rows


def plan_to_jsonl(steps) -> str:
    lines = []
    for i, step in enumerate(steps):
        lines.append(json.dumps({
            "step": i,
            "entries": [{"id": uid, "tokens": list(toks), "want": list(want)} for uid, toks, want in step["entries"]],
            "end": list(step["end"]),
        }))
    return "\n".join(lines) + "\n"


def max_live_tokens(steps, round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: dict[str, int] = {}
    worst = 0
    for step in steps:
        for uid, toks, _ in step["entries"]:
            held[uid] = held.get(uid, 0) + len(toks)
        worst = max(worst, sum(-(-n // round_to) * round_to for n in held.values()))
        for uid in step["end"]:
            held.pop(uid, None)
    return worst


# Error bounds, relative to 1 + the largest plain logit of the request: four times the
# largest error measured on a B200 for the configuration and element type (over all four ways
# of cutting), against the float64 plain run of the same weights.  In float32 that is the
# rounding of float32 sums a few hundred terms long; a product that lost mantissa bits (a
# tensor-core mode with 10 of them) would be some hundred times above it.  In bfloat16 every
# product's output and the cache are rounded to 8 bits of mantissa, a few dozen roundings deep.
MEASURED_ERROR = {
    ("A", "float32"): 1.3e-6, ("A", "bfloat16"): 1.5e-2,
    ("B", "float32"): 1.9e-6, ("B", "bfloat16"): 1.7e-2,
    ("C", "float32"): 2.3e-6, ("C", "bfloat16"): 1.8e-2,
    ("D", "float32"): 2.9e-6, ("D", "bfloat16"): 1.0e-2,
    ("E", "float32"): 2.6e-6, ("E", "bfloat16"): 1.3e-2,
}
# the bound where no figure was measured (the toy parts), and the most any configuration gets
LOOSE = {"float32": 2e-4, "bfloat16": 4e-2}


def tolerance(dtype: str, want: torch.Tensor, config: str | None = None) -> float:
    scale = 1.0 + float(want.abs().max())
    measured = MEASURED_ERROR.get((config, dtype))
    return (min(4.0 * measured, LOOSE[dtype]) if measured is not None else LOOSE[dtype]) * scale


_RECORD = os.environ.get("LOCKSTEP_TEST_RECORD_ERRORS")      # a file that gets one JSON line per comparison


def assert_rows_close(rows, plain_by_uid, dtype: str, what: str, config: str | None = None):
    worst, where, worst_rel = 0.0, None, 0.0
    first_bad = None
    for (uid, pos), got in sorted(rows.items()):
        want = plain_by_uid[uid][pos].float()
        err = float((got - want).abs().max())
        tol = tolerance(dtype, plain_by_uid[uid], config)
        worst_rel = max(worst_rel, err / (1.0 + float(plain_by_uid[uid].abs().max())))
        if err > worst:
            worst, where = err, (uid, pos)
        if err > tol and first_bad is None:
            first_bad = (uid, pos, err, tol)
    if _RECORD:
        with open(_RECORD, "a") as f:
            f.write(json.dumps({"what": what, "config": config, "dtype": dtype, "relative": worst_rel}) + "\n")
    assert first_bad is None, (
        f"{what}: first wrong row is request {first_bad[0]} position {first_bad[1]}: max abs error "
        f"{first_bad[2]:.3e} > {first_bad[3]:.3e}")
    return worst, where
