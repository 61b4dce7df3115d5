"""A block arrangement, an embedding and a norm defined here, not in the framework.

The block is a "sandwich": a norm before and a norm after the mixer, and after the
feed-forward, whose output is the sum of two branches (the layer's own feed-forward and a
second, shared one).  Its further parts come from ``LayerSpec.extra`` under names of the
block's own choosing; the norm after the mixer is a toy norm of its own kind
(centred, with a bias).  The embedding adds a learned table of absolute positions to the token
embedding, and the mixers rotate nothing: the position encoding lives outside the mixer.  A
toy architecture uses both, is replayed whole, in portions and mixed (decode steps recorded as
graphs), and compared with the same model written out plainly in float64."""

from __future__ import annotations

import json

import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu


def register_toys():
    from lockstep_b200 import kernels as K
    from lockstep_b200.config import LayerRun, LayerSpec, ModelSpec, PartSpec, register_architecture
    from lockstep_b200.parts import Block, Norm, Part, WeightSpec, build_part, register_part

    class CentredNorm(Norm):
        """y = (x - mean(x)) * rsqrt(var(x) + eps) * gain + bias, in float32, out in the engine's type."""

        graph_safe = True

        def __init__(self, width, eps, runtime):
            self.width, self.eps, self.rt = width, eps, runtime

        def weight_specs(self):
            return {"weight": WeightSpec((self.width,), "gain"), "bias": WeightSpec((self.width,))}

        def bind(self, tensors):
            self.gain, self.bias = tensors["weight"].float(), tensors["bias"].float()

        def forward(self, h, row_index=None):
            x = h if row_index is None else h[row_index.long()]
            x = x - x.mean(dim=-1, keepdim=True)
            y = x * torch.rsqrt(x.square().mean(dim=-1, keepdim=True) + self.eps) * self.gain + self.bias
            return y.to(self.rt.dtype)

    class Sandwich(Block):
        """h += post_a(mixer(pre_a(h)));  h += post_b(ffn(pre_b(h)) + shared(pre_b(h)))."""

        ORDER = ("pre_a", "mixer", "post_a", "pre_b", "ffn", "shared", "post_b")

        def __init__(self, layer, runtime):
            self.rt = runtime
            self.position = build_part("position", layer.position, runtime)
            self.parts = {
                "pre_a": build_part("norm", layer.mixer_norm, runtime),
                "mixer": build_part("mixer", layer.mixer, runtime, position=self.position),
                "post_a": build_part("norm", layer.extra["post_mixer_norm"], runtime),
                "pre_b": build_part("norm", layer.feed_forward_norm, runtime),
                "ffn": build_part("feed_forward", layer.feed_forward, runtime),
                "shared": build_part("feed_forward", layer.extra["shared_feed_forward"], runtime),
                "post_b": build_part("norm", layer.extra["post_feed_forward_norm"], runtime),
            }

        graph_safe = True           # kernels and torch ops on device tensors of the step only

        def cache_need(self):
            return self.parts["mixer"].cache_need()

        def attention_windows(self):
            return self.parts["mixer"].attention_windows()

        def weight_specs(self):
            return {f"{name}.{local}": spec for name in self.ORDER
                    for local, spec in self.parts[name].weight_specs().items()}

        def bind(self, tensors):
            for name in self.ORDER:
                self.parts[name].bind({k[len(name) + 1:]: v for k, v in tensors.items() if k.startswith(name + ".")})

        def forward(self, h, ctx, cache):
            p = self.parts
            delta = torch.zeros_like(h)                     # what the mixer adds, kept apart
            p["mixer"].forward(p["pre_a"].forward(h), ctx, cache, delta)
            h += p["post_a"].forward(delta).float()
            delta = torch.zeros_like(h)
            x = p["pre_b"].forward(h)
            p["ffn"].forward(x, ctx, delta)
            p["shared"].forward(x, ctx, delta)              # the second branch adds into the same sum
            h += p["post_b"].forward(delta).float()

    class LearnedPositions(Part):
        """h[t] = tokens[id[t]] + places[position[t]]: both rows gathered by the engine's kernel."""

        graph_safe = True

        def __init__(self, vocab, width, places, runtime):
            self.vocab, self.width, self.places, self.rt = vocab, width, places, runtime

        def weight_specs(self):
            return {"tokens.weight": WeightSpec((self.vocab, self.width), "table"),
                    "places.weight": WeightSpec((self.places, self.width), "table")}

        def bind(self, tensors):
            self.tok, self.pos = tensors["tokens.weight"], tensors["places.weight"]

        def forward(self, ctx):
            n = ctx.token_ids.numel()
            h = torch.empty((n, self.width), dtype=torch.float32, device=ctx.token_ids.device)
            place = torch.empty_like(h)
            K.embed_gather(ctx.token_ids, self.tok, h, self.rt.err)
            K.embed_gather(ctx.positions, self.pos, place, self.rt.err)
            return h.add_(place)

    @register_part("block", "toy_sandwich")
    def build_block(spec, runtime, layer_spec=None, **_):
        return Sandwich(layer_spec, runtime)

    @register_part("norm", "toy_centred_norm")
    def build_norm(spec, runtime, **_):
        return CentredNorm(spec["width"], spec["eps"], runtime)

    @register_part("embedding", "toy_learned_positions")
    def build_embedding(spec, runtime, **_):
        return LearnedPositions(spec["vocab_size"], spec["width"], spec["places"], runtime)

    @register_architecture("ToySandwichForCausalLM", model_type="toy_sandwich")
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
            centred = PartSpec("toy_centred_norm", {"width": width, "eps": r["eps"]})
            attn = PartSpec("gqa_attention", {"hidden_size": width, "num_heads": r["heads"], "num_kv_heads": r["kv_heads"],
                                              "head_dim": d, "qk_norm_eps": None, "window": 0, "scale": d ** -0.5})
            layers = [LayerSpec(prefix=f"blocks.{i}", block=PartSpec("toy_sandwich"), mixer=attn,
                                feed_forward=PartSpec("swiglu", {"hidden_size": width, "intermediate_size": r["ffn"]}),
                                mixer_norm=norm, feed_forward_norm=norm, position=PartSpec("none"),
                                extra={"post_mixer_norm": centred, "post_feed_forward_norm": norm,
                                       "shared_feed_forward": PartSpec("swiglu", {"hidden_size": width,
                                                                                  "intermediate_size": r["shared"]})})
                      for i in range(r["layers"])]
            return ModelSpec(architecture="ToySandwichForCausalLM", hidden_size=width, vocab_size=r["vocab"],
                             max_positions=r["places"],
                             embedding=PartSpec("toy_learned_positions",
                                                {"vocab_size": r["vocab"], "width": width, "places": r["places"]}),
                             final_norm=norm,
                             head=PartSpec("linear_head", {"vocab_size": r["vocab"], "width": width, "tied": False}),
                             layers=layers, schedule=[LayerRun(i, i) for i in range(r["layers"])],
                             names={"embedding": "embed", "final_norm": "norm", "head": "lm_head"})


def unregister_toys():
    from lockstep_b200.config import unregister_architecture
    from lockstep_b200.parts import unregister_part

    unregister_architecture("ToySandwichForCausalLM")
    unregister_part("block", "toy_sandwich")
    unregister_part("embedding", "toy_learned_positions")
    unregister_part("norm", "toy_centred_norm")


def plain_toy(folder, tokens):
    from plain import qwen3_plain as plain
    from safetensors.torch import load_file

    r = json.loads((folder / "config.json").read_text())
    w = {k: v.double() for k, v in load_file(str(folder / "model.safetensors")).items()}
    n, d, nq, nkv = len(tokens), r["head_dim"], r["heads"], r["kv_heads"]
    h = w["embed.tokens.weight"][torch.tensor(tokens)] + w["embed.places.weight"][:n]
    norm = lambda x, name: plain.rms_norm(x, w[name], r["eps"])

    def centred(x, name):
        x = x - x.mean(dim=-1, keepdim=True)
        return x * torch.rsqrt(x.square().mean(dim=-1, keepdim=True) + r["eps"]) * w[f"{name}.weight"] + w[f"{name}.bias"]

    for i in range(r["layers"]):
        p = f"blocks.{i}"
        y = norm(h, f"{p}.pre_a.weight")
        q = (y @ w[f"{p}.mixer.q_proj.weight"].T).view(n, nq, d)
        k = (y @ w[f"{p}.mixer.k_proj.weight"].T).view(n, nkv, d)
        v = (y @ w[f"{p}.mixer.v_proj.weight"].T).view(n, nkv, d)
        a = plain.causal_attention(q, k, v, d ** -0.5).reshape(n, nq * d) @ w[f"{p}.mixer.o_proj.weight"].T
        h = h + centred(a, f"{p}.post_a")
        y = norm(h, f"{p}.pre_b.weight")
        both = sum(plain.swiglu_mlp(y, w[f"{p}.{b}.gate_proj.weight"], w[f"{p}.{b}.up_proj.weight"],
                                    w[f"{p}.{b}.down_proj.weight"]) for b in ("ffn", "shared"))
        h = h + norm(both, f"{p}.post_b.weight")
    return norm(h, "norm.weight") @ w["lm_head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_block_with_further_parts_and_an_embedding_that_encodes_positions(tmp_path, dtype):
    from lockstep_b200 import ModelRunner
    from lockstep_b200.weights import write_random_model

    register_toys()
    try:
        raw = {"architectures": ["ToySandwichForCausalLM"], "width": 96, "heads": 6, "kv_heads": 2, "head_dim": 16,
               "ffn": 144, "shared": 40, "vocab": 190, "layers": 2, "eps": 2e-6, "places": 192}
        folder = write_random_model(tmp_path / "toy", raw, seed=9, dtype=dtype, init_std=0.3, gain_std=0.1)
        runner = ModelRunner(folder, dtype=dtype, num_pages=40, page_size=8, max_live=3, max_seq_len=192)
        assert runner.graphs is not None
        requests = {u: H.random_tokens(n, 190, 30 + i) for i, (u, n) in enumerate(zip("abcd", [57, 19, 80, 11]))}
        want = {u: plain_toy(folder, t) for u, t in requests.items()}
        for plan in (H.plan_whole, H.plan_bulk_then_single, H.plan_portions, lambda r: H.plan_mixed(r, max_live=3)):
            rows = H.run_plan(runner, plan(requests))
            H.assert_rows_close(rows, want, dtype, "toy sandwich")
        assert runner.graphs.replays > 30            # the last tokens of plan two were recorded decode steps
        assert runner.cache.free_pages() == runner.cache.total_pages()
    finally:
        unregister_toys()
