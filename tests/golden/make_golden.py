"""Writes the golden files of this folder from LockStep's own CPU code.

Run once, by hand, on a machine where the LockStep project is checked out:

    python tests/golden/make_golden.py /path/to/LockStep

It builds a tiny random Qwen3 model folder (``tiny_model/``), runs LockStep's
float64 CPU forward (``bench/fp64_reference.py``: ``Fp64Reference.hidden`` and
``logits_for``) on two prompts, and records a few draws of LockStep's sampler
(``engine/sampler/philox.py``: ``uniform``, ``greedy``, ``top_p``).  The
outputs are committed; ``tests/test_plain.py`` compares the plain
implementation under ``tests/plain/`` with them.  Nothing here is imported by
the engine.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import torch
from safetensors.torch import save_file

HERE = Path(__file__).resolve().parent

CONFIG = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "hidden_size": 40,
    "intermediate_size": 56,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "vocab_size": 96,
    "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0,
    "max_position_embeddings": 128,
    "tie_word_embeddings": False,
}

PROMPTS = {
    "a": [(7 * i * i + 3 * i + 1) % 96 for i in range(37)],
    "b": [(11 * i + 5) % 96 for i in range(9)],
}


def make_weights(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def mat(rows, cols, std=0.2):
        return torch.randn(rows, cols, generator=g) * std

    def gain(n):
        return 1.0 + 0.1 * torch.randn(n, generator=g)

    w = {"model.embed_tokens.weight": mat(v, h, 1.0), "model.norm.weight": gain(h),
         "lm_head.weight": mat(v, h)}
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}"
        w[f"{p}.input_layernorm.weight"] = gain(h)
        w[f"{p}.post_attention_layernorm.weight"] = gain(h)
        w[f"{p}.self_attn.q_proj.weight"] = mat(nq * d, h)
        w[f"{p}.self_attn.k_proj.weight"] = mat(nkv * d, h)
        w[f"{p}.self_attn.v_proj.weight"] = mat(nkv * d, h)
        w[f"{p}.self_attn.o_proj.weight"] = mat(h, nq * d)
        w[f"{p}.self_attn.q_norm.weight"] = gain(d)
        w[f"{p}.self_attn.k_norm.weight"] = gain(d)
        w[f"{p}.mlp.gate_proj.weight"] = mat(i, h)
        w[f"{p}.mlp.up_proj.weight"] = mat(i, h)
        w[f"{p}.mlp.down_proj.weight"] = mat(h, i)
    return {k: t.contiguous() for k, t in w.items()}


def main():
    lockstep = Path(sys.argv[1]).resolve()
    sys.path.insert(0, str(lockstep))
    model = HERE / "tiny_model"
    model.mkdir(exist_ok=True)
    (model / "config.json").write_text(json.dumps(CONFIG, indent=1) + "\n")
    save_file(make_weights(CONFIG, seed=1234), str(model / "model.safetensors"))

    import bench.fp64_reference as fr
    from engine.sampler import philox

    fr.ENGINE_DTYPE = torch.float32  # keep the stored float32 values
    ref = fr.Fp64Reference(model)
    out = {}
    for name, ids in PROMPTS.items():
        hidden = ref.hidden(ids)
        out[f"hidden_{name}"] = hidden.contiguous()
        out[f"logits_{name}"] = ref.logits_for(hidden).contiguous()
    save_file(out, str(HERE / "lockstep_fp64_outputs.safetensors"))

    row = out["logits_a"][-1]
    draws = {
        "uniform": [
            {"seed": s, "uid": u, "position": p, "value": philox.uniform(s, u, p)}
            for (s, u, p) in [(0, "r00", 0), (7, "r01", 3), (7, "r01", 4), (123456789, "x", 2 ** 33 + 5)]
        ],
        "philox_4x32": [
            {"counter": [1, 2, 3, 4], "key": [5, 6],
             "words": list(philox.philox_4x32((1, 2, 3, 4), (5, 6)))},
        ],
        "greedy_last_row_a": philox.greedy(row),
        "top_p": [
            {"seed": s, "uid": u, "position": pos, "p": p, "temperature": t,
             "token": philox.top_p(row, seed=s, uid=u, position=pos, p=p, temperature=t)}
            for (s, u, pos, p, t) in [
                (0, "r00", 36, 1.0, 1.0), (1, "r00", 36, 0.9, 0.7), (2, "r01", 37, 0.5, 1.3),
                (3, "r02", 38, 1.0, 0.7), (4, "r03", 39, 0.3, 1.0), (5, "r04", 40, 0.95, 2.0),
            ]
        ],
    }
    (HERE / "lockstep_sampler_draws.json").write_text(json.dumps(draws, indent=1) + "\n")
    (HERE / "prompts.json").write_text(json.dumps(PROMPTS) + "\n")
    print("wrote", sorted(p.name for p in HERE.iterdir()))


if __name__ == "__main__":
    main()
