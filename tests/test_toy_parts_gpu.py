"""Parts defined here, not in the framework: a feed-forward with routing (each token goes to
the one of three small SwiGLU experts that its router scores highest, weighted by the
softmax of the router's logits) and another position encoding (rotation angles that grow
linearly with the pair's index instead of geometrically, over half of the head).  A toy
architecture puts them beside the engine's attention, norm and dense feed-forward, with
different parts in different layers, and is replayed whole, in portions and mixed."""

from __future__ import annotations

import json

import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

EXPERTS = 3


def register_toys():
    from lockstep_b200 import kernels as K
    from lockstep_b200.config import LayerRun, LayerSpec, ModelSpec, PartSpec, register_architecture
    from lockstep_b200.parts import FeedForward, PositionEncoding, WeightSpec, register_part

    class RoutedSwiGLU(FeedForward):
        """residual += p_e(x) * down_e(silu(gate_e x) * up_e x) for the expert e with the largest
        router logit (ties to the lowest index); router logits and their softmax in float32."""

        def __init__(self, width, inner, runtime):
            self.width, self.inner, self.rt = width, inner, runtime
            self.router = None
            self.experts = []

        def weight_specs(self):
            specs = {"router.weight": WeightSpec((EXPERTS, self.width))}
            for e in range(EXPERTS):
                specs[f"experts.{e}.gate_up.weight"] = WeightSpec((2 * self.inner, self.width))
                specs[f"experts.{e}.down.weight"] = WeightSpec((self.width, self.inner))
            return specs

        def bind(self, tensors):
            self.router = tensors["router.weight"].float()
            self.experts = [(tensors[f"experts.{e}.gate_up.weight"], tensors[f"experts.{e}.down.weight"])
                            for e in range(EXPERTS)]

        def forward(self, x, ctx, residual):
            logits = x.float() @ self.router.T                       # float32, a library product of 3 rows
            prob = torch.softmax(logits, dim=-1)
            choice = logits.argmax(dim=-1)
            for e, (gate_up, down) in enumerate(self.experts):
                rows = (choice == e).nonzero().flatten()
                if not rows.numel():
                    continue
                xe = x[rows].contiguous()
                act = torch.empty((rows.numel(), self.inner), dtype=x.dtype, device=x.device)
                K.gemm_nt(xe, gate_up, act, K.EPILOGUE_SILU_MUL, err=self.rt.err)     # the engine's kernels
                out = torch.zeros((rows.numel(), self.width), dtype=torch.float32, device=x.device)
                K.gemm_nt(act, down, out, K.EPILOGUE_RESIDUAL, err=self.rt.err)
                residual[rows] += out * prob[rows, e][:, None]

    class LinearAngles(PositionEncoding):
        """cos/sin of pos * (i + 1) * step for pair i, over ``dim`` dimensions of the head."""

        graph_safe = True

        def __init__(self, dim, step, runtime):
            half = dim // 2
            ang = torch.arange(runtime.max_positions, dtype=torch.float64)[:, None] * \
                (torch.arange(1, half + 1, dtype=torch.float64) * step)[None, :]
            self.dim = dim
            self.cos = ang.cos().float().to(runtime.device).contiguous()
            self.sin = ang.sin().float().to(runtime.device).contiguous()

        def rotary(self):
            return self.cos, self.sin, self.dim

    @register_part("feed_forward", "toy_routed_swiglu")
    def build_ffn(spec, runtime, **_):
        return RoutedSwiGLU(spec["width"], spec["inner"], runtime)

    @register_part("position", "toy_linear_angles")
    def build_pos(spec, runtime, **_):
        return LinearAngles(spec["dim"], spec["step"], runtime)

    @register_architecture("ToyRoutedForCausalLM", model_type="toy_routed")
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
            routed = PartSpec("toy_routed_swiglu", {"width": width, "inner": r["inner"]})
            dense = PartSpec("swiglu", {"hidden_size": width, "intermediate_size": r["ffn"]})
            linear = PartSpec("toy_linear_angles", {"dim": d // 2, "step": r["step"]})
            rotary = PartSpec("rotary", {"dim": d, "theta": 500.0})
            layers = [LayerSpec(prefix=f"layers.{i}", block=PartSpec("pre_norm"), mixer=attn,
                                feed_forward=routed if i % 2 == 0 else dense, mixer_norm=norm, feed_forward_norm=norm,
                                position=linear if i % 2 == 0 else rotary)
                      for i in range(r["layers"])]
            return ModelSpec(architecture="ToyRoutedForCausalLM", hidden_size=width, vocab_size=r["vocab"],
                             max_positions=256,
                             embedding=PartSpec("token_embedding", {"vocab_size": r["vocab"], "width": width}),
                             final_norm=norm,
                             head=PartSpec("linear_head", {"vocab_size": r["vocab"], "width": width, "tied": False}),
                             layers=layers, schedule=[LayerRun(i, i) for i in range(r["layers"])],
                             names={"embedding": "embed", "final_norm": "norm", "head": "lm_head"})


def unregister_toys():
    from lockstep_b200.config import unregister_architecture
    from lockstep_b200.parts import unregister_part

    unregister_architecture("ToyRoutedForCausalLM")
    unregister_part("feed_forward", "toy_routed_swiglu")
    unregister_part("position", "toy_linear_angles")


def plain_toy(folder, tokens, dtype):
    """The toy model written out plainly in float64, whole sequence.  The expert of a token is
    taken from the engine's own arithmetic precision only through ``dtype``: the router reads
    the normed row as the engine stores it (bfloat16 or float32)."""
    from plain import qwen3_plain as plain
    from safetensors.torch import load_file

    r = json.loads((folder / "config.json").read_text())
    w = {k: v.double() for k, v in load_file(str(folder / "model.safetensors")).items()}
    n, d, nq, nkv = len(tokens), r["head_dim"], r["heads"], r["kv_heads"]
    h = w["embed.weight"][torch.tensor(tokens)]
    pos = torch.arange(n, dtype=torch.float64)
    margins = []
    for i in range(r["layers"]):
        p = f"layers.{i}"
        y = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], r["eps"])
        q = (y @ w[f"{p}.self_attn.q_proj.weight"].T).view(n, nq, d)
        k = (y @ w[f"{p}.self_attn.k_proj.weight"].T).view(n, nkv, d)
        v = (y @ w[f"{p}.self_attn.v_proj.weight"].T).view(n, nkv, d)
        q = plain.rms_norm(q, w[f"{p}.self_attn.q_norm.weight"], r["eps"])
        k = plain.rms_norm(k, w[f"{p}.self_attn.k_norm.weight"], r["eps"])
        if i % 2 == 0:
            half = d // 4
            ang = pos[:, None] * (torch.arange(1, half + 1, dtype=torch.float64) * r["step"])[None, :]
            cos, sin, rot = ang.cos(), ang.sin(), d // 2
        else:
            cos, sin = plain.rope_tables(range(n), d, 500.0)
            rot = d
        def turn(x):
            a, b, rest = x[..., :rot // 2], x[..., rot // 2:rot], x[..., rot:]
            c, s = cos[:, None, :], sin[:, None, :]
            return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)
        a = plain.causal_attention(turn(q), turn(k), v, d ** -0.5)
        h = h + a.reshape(n, nq * d) @ w[f"{p}.self_attn.o_proj.weight"].T
        y = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], r["eps"])
        if i % 2 == 0:
            logits = y @ w[f"{p}.mlp.router.weight"].T
            top2 = logits.topk(2, dim=-1).values
            margins.append((top2[:, 0] - top2[:, 1]).min())
            prob = torch.softmax(logits, dim=-1)
            choice = logits.argmax(dim=-1)
            out = torch.zeros_like(h)
            for e in range(EXPERTS):
                gu, down = w[f"{p}.mlp.experts.{e}.gate_up.weight"], w[f"{p}.mlp.experts.{e}.down.weight"]
                g, u = y @ gu[:r["inner"]].T, y @ gu[r["inner"]:].T
                ye = (torch.nn.functional.silu(g) * u) @ down.T
                out = torch.where((choice == e)[:, None], ye * prob[:, e][:, None], out)
            h = h + out
        else:
            h = h + plain.swiglu_mlp(y, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                                     w[f"{p}.mlp.down_proj.weight"])
    return plain.rms_norm(h, w["norm.weight"], r["eps"]) @ w["lm_head.weight"].T, float(min(margins))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_another_position_encoding(tmp_path, dtype):
    from lockstep_b200 import ModelRunner
    from lockstep_b200.weights import write_random_model

    register_toys()
    try:
        raw = {"architectures": ["ToyRoutedForCausalLM"], "width": 80, "heads": 4, "kv_heads": 2, "head_dim": 32,
               "inner": 48, "ffn": 112, "vocab": 210, "layers": 3, "eps": 1e-5, "step": 0.013}
        folder = write_random_model(tmp_path / "toy", raw, seed=4, dtype=dtype, init_std=0.3, gain_std=0.1)
        runner = ModelRunner(folder, dtype=dtype, num_pages=24, page_size=8, max_live=3, max_seq_len=256)
        # the routed part reads values on the host, so it is called as it is between the recorded
        # runs of the other steps of a decode step
        assert runner.graphs is not None
        requests, want = {}, {}
        # sequences whose every token has a clear winner among the experts (a near tie may go
        # either way in reduced precision, which is a property of routing, not a fault)
        seed = 0
        while len(requests) < 4:
            seed += 1
            tokens = H.random_tokens([41, 19, 30, 11][len(requests)], 210, seed)
            logits, margin = plain_toy(folder, tokens, dtype)
            if margin > (1e-3 if dtype == "float32" else 0.05):
                uid = "abcd"[len(requests)]
                requests[uid], want[uid] = tokens, logits
        for plan in (H.plan_whole, H.plan_portions, lambda r: H.plan_mixed(r, max_live=3),
                     lambda r: H.plan_bulk_then_single({u: r[u] for u in "ac"}, tail=16)):
            rows = H.run_plan(runner, plan(requests))
            H.assert_rows_close(rows, want, dtype, "toy parts")
        assert runner.graphs.replays >= 14
        pieces = next(iter(runner.graphs.graphs.values()))[0]
        assert [graph is not None for graph, _ in pieces].count(False) == 2     # the routed parts of layers 0 and 2
    finally:
        unregister_toys()
