"""Position encodings other than the engine's own half rotation, defined here and used by the
engine's attention without a change to the framework's files:

- a bias on the scores that grows with the distance of key and query (a slope per head),
- a rotation of neighbouring pairs (2i, 2i + 1) instead of the halves (i, i + dim / 2),
- both at once, the rotation over a part of the head only.

The toy architecture has a layer of each.  The plain implementation below writes the three out
in float64.  Head size 64: where there is no bias the bfloat16 engine takes its tensor-core
attention, where there is one it takes the CUDA-core kernels, which know the bias; both are
asserted by the kernels' launch counters.
"""

from __future__ import annotations

import json

import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu


def register_toys():
    from lockstep_b200.config import LayerRun, LayerSpec, ModelSpec, PartSpec, register_architecture
    from lockstep_b200.parts import PositionEncoding, register_part

    class ToyPositions(PositionEncoding):
        """``slope_base`` > 0: head h's scores get -slope_base^(h + 1) x distance.  ``dim`` > 0:
        neighbouring pairs of the first ``dim`` elements are rotated by pos x theta^(-2i/dim)."""

        graph_safe = True
        rotary_interleaved = True

        def __init__(self, dim, theta, slope_base, runtime):
            self.dim, self.slope_base, self.rt = int(dim), float(slope_base), runtime
            if self.dim:
                i = torch.arange(self.dim // 2, dtype=torch.float64)
                ang = torch.arange(runtime.max_positions, dtype=torch.float64)[:, None] * theta ** (-2 * i / self.dim)[None, :]
                self.cos = ang.cos().float().to(runtime.device).contiguous()
                self.sin = ang.sin().float().to(runtime.device).contiguous()

        def rotary(self):
            return (self.cos, self.sin, self.dim) if self.dim else None

        def score_slopes(self, num_heads):
            if not self.slope_base:
                return None
            return torch.tensor([self.slope_base ** (h + 1) for h in range(num_heads)], dtype=torch.float32,
                                device=self.rt.device)

    @register_part("position", "toy_positions")
    def build_pos(spec, runtime, **_):
        return ToyPositions(spec["dim"], spec["theta"], spec["slope_base"], runtime)

    @register_architecture("ToyPositionsForCausalLM", model_type="toy_positions")
    class ToyConfig:
        def __init__(self, raw):
            self.raw = dict(raw)

        @classmethod
        def from_dict(cls, raw):
            return cls(raw)

        def to_dict(self):
            return dict(self.raw)

        def model_spec(self):
            r = self.raw
            width, d = r["width"], r["head_dim"]
            norm = PartSpec("rmsnorm", {"width": width, "eps": r["eps"]})
            attn = PartSpec("gqa_attention", {"hidden_size": width, "num_heads": r["heads"], "num_kv_heads": r["kv_heads"],
                                              "head_dim": d, "qk_norm_eps": r["eps"], "window": 0, "scale": d ** -0.5})
            ffn = PartSpec("swiglu", {"hidden_size": width, "intermediate_size": r["ffn"]})
            layers = [LayerSpec(prefix=f"layers.{i}", block=PartSpec("pre_norm"), mixer=attn, feed_forward=ffn,
                                mixer_norm=norm, feed_forward_norm=norm,
                                position=PartSpec("toy_positions", {"dim": dim, "theta": r["theta"], "slope_base": base}))
                      for i, (dim, base) in enumerate(r["positions"])]
            return ModelSpec(architecture="ToyPositionsForCausalLM", hidden_size=width, vocab_size=r["vocab"],
                             max_positions=512,
                             embedding=PartSpec("token_embedding", {"vocab_size": r["vocab"], "width": width}),
                             final_norm=norm,
                             head=PartSpec("linear_head", {"vocab_size": r["vocab"], "width": width, "tied": True}),
                             layers=layers, schedule=[LayerRun(i, i) for i in range(len(layers))],
                             names={"embedding": "embed", "final_norm": "norm", "head": "lm_head"})


def unregister_toys():
    from lockstep_b200.config import unregister_architecture
    from lockstep_b200.parts import unregister_part

    unregister_architecture("ToyPositionsForCausalLM")
    unregister_part("position", "toy_positions")


def plain_toy(folder, tokens):
    from plain import qwen3_plain as plain
    from safetensors.torch import load_file

    r = json.loads((folder / "config.json").read_text())
    w = {k: v.double() for k, v in load_file(str(folder / "model.safetensors")).items()}
    n, d, nq, nkv = len(tokens), r["head_dim"], r["heads"], r["kv_heads"]
    h = w["embed.weight"][torch.tensor(tokens)]
    pos = torch.arange(n, dtype=torch.float64)
    distance = pos[None, :] - pos[:, None]                 # key position - query position
    causal = distance <= 0
    for i, (dim, base) in enumerate(r["positions"]):
        p = f"layers.{i}"
        y = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], r["eps"])
        q = (y @ w[f"{p}.self_attn.q_proj.weight"].T).view(n, nq, d)
        k = (y @ w[f"{p}.self_attn.k_proj.weight"].T).view(n, nkv, d)
        v = (y @ w[f"{p}.self_attn.v_proj.weight"].T).view(n, nkv, d)
        q = plain.rms_norm(q, w[f"{p}.self_attn.q_norm.weight"], r["eps"])
        k = plain.rms_norm(k, w[f"{p}.self_attn.k_norm.weight"], r["eps"])
        if dim:
            idx = torch.arange(dim // 2, dtype=torch.float64)
            ang = pos[:, None] * r["theta"] ** (-2 * idx / dim)[None, :]
            c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]

            def turn(x):
                lo, hi = x[..., 0:dim:2], x[..., 1:dim:2]
                out = x.clone()
                out[..., 0:dim:2] = lo * c - hi * s
                out[..., 1:dim:2] = hi * c + lo * s
                return out

            q, k = turn(q), turn(k)
        heads = []
        for head in range(nq):
            scores = q[:, head] @ k[:, head // (nq // nkv)].T * d ** -0.5
            if base:
                scores = scores + base ** (head + 1) * distance
            scores = scores.masked_fill(~causal, float("-inf"))
            heads.append(torch.softmax(scores, dim=-1) @ v[:, head // (nq // nkv)])
        a = torch.stack(heads, dim=1)
        h = h + a.reshape(n, nq * d) @ w[f"{p}.self_attn.o_proj.weight"].T
        y = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], r["eps"])
        h = h + plain.swiglu_mlp(y, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                                 w[f"{p}.mlp.down_proj.weight"])
    return plain.rms_norm(h, w["norm.weight"], r["eps"]) @ w["embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_score_bias_and_rotation_of_neighbouring_pairs(tmp_path, dtype):
    from lockstep_b200 import ModelRunner
    from lockstep_b200 import kernels as K
    from lockstep_b200.weights import write_random_model

    register_toys()
    try:
        raw = {"architectures": ["ToyPositionsForCausalLM"], "width": 96, "heads": 4, "kv_heads": 2, "head_dim": 64,
               "ffn": 160, "vocab": 190, "eps": 1e-5, "theta": 300.0,
               # (rotated elements, slope base) of each layer: bias alone; pairs over the whole
               # head; pairs over 48 of the 64 elements and a bias
               "positions": [[0, 0.5], [64, 0.0], [48, 0.7]]}
        folder = write_random_model(tmp_path / "toy", raw, seed=6, dtype=dtype, init_std=0.3, gain_std=0.1)
        runner = ModelRunner(folder, dtype=dtype, num_pages=64, page_size=16, max_live=3, max_seq_len=512)
        requests = {"a": H.random_tokens(300, 190, 1), "b": H.random_tokens(70, 190, 2), "c": H.random_tokens(33, 190, 3)}
        want = {u: plain_toy(folder, t) for u, t in requests.items()}
        before = K.kernel_counts()
        for plan in (H.plan_whole, H.plan_portions, lambda r: H.plan_mixed(r, max_live=3),
                     lambda r: H.plan_bulk_then_single(r, tail=24)):
            rows = H.run_plan(runner, plan(requests))
            H.assert_rows_close(rows, want, dtype, "toy positions")
        ran = {k: v - before.get(k, 0) for k, v in K.kernel_counts().items()}
        assert ran["attention_tile"] > 0                  # the layers with a bias (in float32: all layers, all rows)
        if dtype == "bfloat16":
            assert ran["attention_decode"] > 0            # decoded rows of the layers with a bias
            assert ran["attention_prefill_tc"] > 0 and ran["attention_decode_mma"] > 0   # the layer without
        assert runner.graphs.replays > 40

        # the bias matters: a far key with a huge score loses against near ones under a steep slope
        assert (want["a"][-1] - plain_toy_without_bias(folder, requests["a"])[-1]).abs().max() > 1e-2
    finally:
        unregister_toys()


def plain_toy_without_bias(folder, tokens):
    """The same model with every slope set to zero, to show that the bias is not a no-op."""
    import shutil
    import tempfile
    from pathlib import Path

    with tempfile.TemporaryDirectory() as tmp:
        copy = Path(tmp) / "m"
        shutil.copytree(folder, copy)
        raw = json.loads((copy / "config.json").read_text())
        raw["positions"] = [[dim, 0.0] for dim, _ in raw["positions"]]
        (copy / "config.json").write_text(json.dumps(raw))
        return plain_toy(copy, tokens)
