"""Each part alone, built through the registries, against the plain functions."""

from __future__ import annotations

import math

import pytest
import torch

from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def runtime(dtype, page=8, max_positions=256):
    from lockstep_b200 import kernels as K
    from lockstep_b200.parts import Runtime

    dev = torch.device("cuda:0")
    return Runtime(device=dev, dtype=dtype, page_size=page, max_positions=max_positions,
                   err=K.new_error_word(dev))


def bound(dtype, want):
    return (2e-5 if dtype == torch.float32 else 3e-2) * (1 + float(want.abs().max()))


def rand(gen, *shape, scale=1.0, dtype=torch.float32):
    return (torch.randn(*shape, generator=gen) * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from lockstep_b200.config import PartSpec
    from lockstep_b200.parts import build_part

    rt = runtime(dtype)
    g = torch.Generator().manual_seed(0)
    part = build_part("norm", PartSpec("rmsnorm", {"width": 88, "eps": 2e-5}), rt)
    assert part.weight_specs()["weight"].shape == (88,)
    gain = (1 + rand(g, 88, scale=0.2)).to(dtype)
    part.bind({"weight": gain.to(rt.device)})
    h = rand(g, 9, 88, scale=4.0)
    got = part.forward(h.to(rt.device)).cpu().double()
    want = plain.rms_norm(h.double(), gain.double(), 2e-5)
    assert got.dtype == torch.float64 and (got - want).abs().max() <= bound(dtype, want)


def test_rotary_tables_match_plain():
    from lockstep_b200.config import PartSpec
    from lockstep_b200.parts import build_part

    rt = runtime(torch.float32, max_positions=300)
    part = build_part("position", PartSpec("rotary", {"dim": 48, "theta": 50000.0}), rt)
    cos, sin, dim = part.rotary()
    c, s = plain.rope_tables(range(300), 48, 50000.0, torch.float32)
    assert dim == 48 and torch.equal(cos.cpu(), c) and torch.equal(sin.cpu(), s)
    assert build_part("position", PartSpec("none"), rt).rotary() is None


def step_context(rt, portions, page, entries=1, need=None):
    """A StepContext and cache view for hand-made portions [(uid, start, tokens)]."""
    from lockstep_b200 import kernels as K
    from lockstep_b200.cache import CacheManager
    from lockstep_b200.engine.batch import StepContext, StepEntry

    return StepContext, StepEntry, CacheManager, K.attention_split_size()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 24])
def test_attention_part_alone(dtype, window):
    """The mixer over its own cache: a prompt in two portions, then two decoded tokens."""
    from lockstep_b200.cache import CacheManager
    from lockstep_b200.config import PartSpec
    from lockstep_b200.engine.batch import StepContext, StepEntry
    from lockstep_b200 import kernels as K
    from lockstep_b200.parts import build_part

    hsz, nq, nkv, d, page = 56, 6, 2, 32, 8
    rt = runtime(dtype, page=page)
    pos = build_part("position", PartSpec("rotary", {"dim": d, "theta": 10000.0}), rt)
    spec = PartSpec("gqa_attention", {"hidden_size": hsz, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d,
                                      "qk_norm_eps": 1e-6, "window": window, "scale": 1 / math.sqrt(d)})
    mixer = build_part("mixer", spec, rt, position=pos)
    g = torch.Generator().manual_seed(3)
    w = {n: (rand(g, *s.shape, scale=0.3) if s.role == "matrix" else 1 + rand(g, *s.shape, scale=0.1)).to(dtype)
         for n, s in mixer.weight_specs().items()}
    mixer.bind({n: t.to(rt.device) for n, t in w.items()})
    cache = CacheManager([mixer.cache_need()], num_pages=12, page_size=page, max_live=2, max_seq_len=256,
                         dtype=dtype, device=rt.device)
    total = 70
    x = rand(g, total, hsz).to(dtype)
    cache.create("a")
    out = torch.zeros(total, hsz, dtype=torch.float32, device=rt.device)
    at = 0
    for n in (37, 31, 1, 1):
        cache.reserve("a", at + n)
        cache.sync()
        ctx = StepContext([StepEntry("a", [0] * n, at, [])], [cache.slots["a"]], rt.device, rt.err,
                          K.attention_split_size())
        res = torch.zeros(n, hsz, dtype=torch.float32, device=rt.device)
        mixer.forward(x[at:at + n].to(rt.device).contiguous(), ctx, cache.view(0), res)
        out[at:at + n] = res
        at += n
        cache.advance("a", at)
    K.raise_on_fault(rt.err)
    cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": d, "rms_norm_eps": 1e-6}
    cos, sin = plain.rope_tables(range(total), d, 10000.0, torch.float64)
    w64 = {f"p.{n}": t.double() for n, t in w.items()}
    want = plain.attention_block(x.double(), w64, "p", cfg, cos, sin, window=window)
    assert (out.cpu().double() - want).abs().max() <= bound(dtype, want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    from lockstep_b200.config import PartSpec
    from lockstep_b200.parts import build_part

    rt = runtime(dtype)
    g = torch.Generator().manual_seed(4)
    part = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": 72, "intermediate_size": 200}), rt)
    w = {n: rand(g, *s.shape, scale=0.2).to(dtype) for n, s in part.weight_specs().items()}
    part.bind({n: t.to(rt.device) for n, t in w.items()})
    x = rand(g, 13, 72).to(dtype)
    res = rand(g, 13, 72)
    got = res.to(rt.device).clone()
    part.forward(x.to(rt.device), None, got)
    want = res.double() + plain.swiglu_mlp(x.double(), w["gate_proj.weight"].double(),
                                           w["up_proj.weight"].double(), w["down_proj.weight"].double())
    assert (got.cpu().double() - want).abs().max() <= bound(dtype, want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    from lockstep_b200.config import PartSpec
    from lockstep_b200.parts import build_part

    rt = runtime(dtype)
    g = torch.Generator().manual_seed(5)
    emb = build_part("embedding", PartSpec("token_embedding", {"vocab_size": 301, "width": 40}), rt)
    head = build_part("head", PartSpec("linear_head", {"vocab_size": 301, "width": 40, "tied": True}), rt)
    assert head.weight_specs() == {}
    table = rand(g, 301, 40).to(dtype)
    emb.bind({"weight": table.to(rt.device)})
    head.bind({"weight": table.to(rt.device)})

    class Ctx:
        token_ids = torch.tensor([5, 300, 0, 5], dtype=torch.int32, device=rt.device)

    h = emb.forward(Ctx)
    assert torch.equal(h.cpu(), table.float()[[5, 300, 0, 5]])
    y = rand(g, 3, 40).to(dtype)
    logits = head.forward(y.to(rt.device))
    want = y.double() @ table.double().T
    assert logits.dtype == torch.float32
    assert (logits.cpu().double() - want).abs().max() <= 1e-5 * (1 + float(want.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
def test_pre_norm_block_alone(dtype):
    from lockstep_b200.cache import CacheManager
    from lockstep_b200.config import config_from_dict
    from lockstep_b200.engine.batch import StepContext, StepEntry
    from lockstep_b200 import kernels as K
    from lockstep_b200.parts import build_part
    import helpers as H

    cfg = dict(H.TINY_B)
    layer = config_from_dict(cfg).model_spec().layers[1]
    rt = runtime(dtype, page=8)
    block = build_part("block", layer.block, rt, layer_spec=layer)
    g = torch.Generator().manual_seed(6)
    w = {n: (rand(g, *s.shape, scale=0.25) if s.role == "matrix" else 1 + rand(g, *s.shape, scale=0.1)).to(dtype)
         for n, s in block.weight_specs().items()}
    assert "self_attn.q_norm.weight" in w and "mlp.down_proj.weight" in w and "input_layernorm.weight" in w
    block.bind({n: t.to(rt.device) for n, t in w.items()})
    cache = CacheManager([block.cache_need()], num_pages=8, page_size=8, max_live=2, max_seq_len=256,
                         dtype=dtype, device=rt.device)
    cache.create("a")
    n = 29
    cache.reserve("a", n)
    cache.sync()
    h0 = rand(g, n, 80)
    h = h0.to(rt.device).clone()
    ctx = StepContext([StepEntry("a", [0] * n, 0, [])], [cache.slots["a"]], rt.device, rt.err,
                      K.attention_split_size())
    block.forward(h, ctx, cache.view(0))
    K.raise_on_fault(rt.err)
    cos, sin = plain.rope_tables(range(n), 32, cfg["rope_theta"], torch.float64)
    w64 = {f"model.layers.0.{k}": t.double() for k, t in w.items()}
    want = plain.decoder_layer(h0.double(), w64, 0, cfg, cos, sin)
    assert (h.cpu().double() - want).abs().max() <= bound(dtype, want)
