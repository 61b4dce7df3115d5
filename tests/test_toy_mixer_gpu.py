"""A mixer with state of its own, defined here, is registered, built and stepped
without a change to the framework's files: a toy architecture whose layers
alternate between the toy mixer (a running mean kept in a fixed-size state slot)
and the engine's attention."""

from __future__ import annotations

import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu


def register_toy():
    from lockstep_b200.config import (LayerRun, LayerSpec, ModelSpec, PartSpec, register_architecture)
    from lockstep_b200.parts import CacheNeed, Mixer, WeightSpec, register_part

    class RunningMean(Mixer):
        """out[t] = W @ mean(x[0..t]); the state slot holds the running sum and the count."""

        def __init__(self, width, runtime):
            self.width, self.rt, self.w = width, runtime, None

        def cache_need(self):
            return CacheNeed("state", state_shape=(self.width + 1,), state_dtype=torch.float32)

        def weight_specs(self):
            return {"mix.weight": WeightSpec((self.width, self.width))}

        def bind(self, tensors):
            self.w = tensors["mix.weight"]

        def forward(self, x, ctx, cache, residual):
            for slot, off, start, n in ctx.portions:
                state = cache.state[slot]
                if start == 0:
                    state.zero_()
                xs = x[off:off + n].float()
                sums = state[:self.width] + torch.cumsum(xs, dim=0)
                counts = state[self.width] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                mean = (sums / counts[:, None]).to(x.dtype)
                residual[off:off + n] += (mean @ self.w.T).float()
                if cache.writes:
                    state[:self.width] = sums[-1]
                    state[self.width] = counts[-1]

    @register_part("mixer", "toy_running_mean")
    def build_mixer(spec, runtime, **_):
        return RunningMean(spec["width"], runtime)

    @register_architecture("ToyStateForCausalLM", model_type="toy_state")
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
            width = r["width"]
            norm = PartSpec("rmsnorm", {"width": width, "eps": r["eps"]})
            attn = PartSpec("gqa_attention", {"hidden_size": width, "num_heads": r["heads"], "num_kv_heads": 1,
                                              "head_dim": r["head_dim"], "qk_norm_eps": None, "window": 0,
                                              "scale": r["head_dim"] ** -0.5})
            toy = PartSpec("toy_running_mean", {"width": width})
            ffn = PartSpec("swiglu", {"hidden_size": width, "intermediate_size": r["ffn"]})
            layers = [LayerSpec(prefix=f"blocks.{i}", block=PartSpec("pre_norm"),
                                mixer=toy if i % 2 == 0 else attn, feed_forward=ffn, mixer_norm=norm,
                                feed_forward_norm=norm,
                                position=PartSpec("rotary", {"dim": r["head_dim"], "theta": 1000.0}))
                      for i in range(r["layers"])]
            # the order of layers is data: layer 0 runs twice (on cache entries of its own)
            schedule = [LayerRun(0, 0), LayerRun(1, 1), LayerRun(2, 2), LayerRun(0, 3)]
            return ModelSpec(architecture="ToyStateForCausalLM", hidden_size=width, vocab_size=r["vocab"],
                             max_positions=256, embedding=PartSpec("token_embedding", {"vocab_size": r["vocab"], "width": width}),
                             final_norm=norm, head=PartSpec("linear_head", {"vocab_size": r["vocab"], "width": width, "tied": True}),
                             layers=layers, schedule=schedule,
                             names={"embedding": "tok", "final_norm": "out_norm", "head": "head"})


def unregister_toy():
    from lockstep_b200.config import unregister_architecture
    from lockstep_b200.parts import unregister_part

    unregister_architecture("ToyStateForCausalLM")
    unregister_part("mixer", "toy_running_mean")


def plain_toy(folder, tokens):
    """The toy model written out plainly in float64 (whole sequence, no cache)."""
    import json

    from plain import qwen3_plain as plain
    from safetensors.torch import load_file

    r = json.loads((folder / "config.json").read_text())
    w = {k: v.double() for k, v in load_file(str(folder / "model.safetensors")).items()}
    h = w["tok.weight"][torch.tensor(tokens)]
    n = len(tokens)
    cos, sin = plain.rope_tables(range(n), r["head_dim"], 1000.0)
    for layer in (0, 1, 2, 0):
        p = f"blocks.{layer}"
        y = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], r["eps"])
        if layer % 2 == 0:
            mean = torch.cumsum(y, 0) / torch.arange(1, n + 1, dtype=torch.float64)[:, None]
            h = h + mean @ w[f"{p}.self_attn.mix.weight"].T
        else:
            d, nq = r["head_dim"], r["heads"]
            q = (y @ w[f"{p}.self_attn.q_proj.weight"].T).view(n, nq, d)
            k = (y @ w[f"{p}.self_attn.k_proj.weight"].T).view(n, 1, d)
            v = (y @ w[f"{p}.self_attn.v_proj.weight"].T).view(n, 1, d)
            a = plain.causal_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v, d ** -0.5)
            h = h + a.reshape(n, nq * d) @ w[f"{p}.self_attn.o_proj.weight"].T
        y = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], r["eps"])
        h = h + plain.swiglu_mlp(y, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                                 w[f"{p}.mlp.down_proj.weight"])
    return plain.rms_norm(h, w["out_norm.weight"], r["eps"]) @ w["tok.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path, dtype):
    from lockstep_b200 import ModelRunner
    from lockstep_b200.weights import write_random_model

    register_toy()
    try:
        raw = {"architectures": ["ToyStateForCausalLM"], "width": 48, "heads": 3, "head_dim": 16,
               "ffn": 72, "vocab": 150, "layers": 3, "eps": 1e-5}
        folder = write_random_model(tmp_path / "toy", raw, seed=2, dtype=dtype, init_std=0.3, gain_std=0.1)
        runner = ModelRunner(folder, dtype=dtype, num_pages=16, page_size=16, max_live=3, max_seq_len=256)
        assert len(runner.cache.states) == 1 and len(runner.cache.paged) == 1
        assert runner.cache.states[0].entries == [0, 2, 3] and runner.cache.paged[0].entries == [1]
        requests = {"a": H.random_tokens(45, 150, 1), "b": H.random_tokens(23, 150, 2),
                    "c": H.random_tokens(31, 150, 3), "d": H.random_tokens(12, 150, 4)}
        want = {u: plain_toy(folder, t) for u, t in requests.items()}
        for plan in (H.plan_whole, H.plan_portions, lambda r: H.plan_mixed(r, max_live=3)):
            rows = H.run_plan(runner, plan(requests))
            H.assert_rows_close(rows, want, dtype, "toy")   # slot reuse: "d" takes a used slot
    finally:
        unregister_toy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_of_the_toy_model_are_recorded_around_its_mixer(tmp_path, dtype):
    """The toy mixer reads the step's portions on the host, so it cannot be part of a recorded
    step.  The steps around it can: the decode steps replay graphs of the attention layer, the
    feed-forwards and the head, call the toy mixer between them, and give the bits of a runner
    that records nothing."""
    from lockstep_b200 import ModelRunner
    from lockstep_b200.weights import write_random_model

    register_toy()
    try:
        raw = {"architectures": ["ToyStateForCausalLM"], "width": 48, "heads": 3, "head_dim": 16,
               "ffn": 72, "vocab": 150, "layers": 3, "eps": 1e-5}
        folder = write_random_model(tmp_path / "toy", raw, seed=2, dtype=dtype, init_std=0.3, gain_std=0.1)
        requests = {"a": H.random_tokens(60, 150, 1), "b": H.random_tokens(47, 150, 2)}
        want = {u: plain_toy(folder, t) for u, t in requests.items()}
        rows = {}
        for graphs in (True, False):
            runner = ModelRunner(folder, dtype=dtype, num_pages=16, page_size=16, max_live=3, max_seq_len=256,
                                 use_graphs=graphs)
            assert (runner.graphs is not None) == graphs
            rows[graphs] = H.run_plan(runner, H.plan_bulk_then_single(requests, tail=32))
            if graphs:
                assert runner.graphs.replays >= 25
                pieces = next(iter(runner.graphs.graphs.values()))[0]
                kinds = [graph is not None for graph, _ in pieces]
                # embedding | toy | ffn, attention layer, ffn | toy | ffn | toy | ffn, head
                assert kinds == [True, False, True, False, True, False, True]
        H.assert_rows_close(rows[True], want, dtype, "toy, recorded around the mixer")
        assert rows[True].keys() == rows[False].keys()
        for key in rows[True]:
            assert torch.equal(rows[True][key], rows[False][key]), key
    finally:
        unregister_toy()
