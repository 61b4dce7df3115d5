"""A context of 40,000 tokens (the longest Qwen3's configuration allows is 40,960): positions far
into the rotary table, block tables of 2,500 pages, 157 splits of the keys of a decoded token, page
and row offsets beyond 2^16.  A model of one layer with head size 128, so that the rows that are
asked for can be written out plainly in float64 from all keys without the other rows' attention.
Two cuttings (portions of 4,096 and then single tokens; ragged portions of 2 to 8,192) must agree
with it, and with each other bit for bit in float32."""

from __future__ import annotations

import pytest
import torch

import helpers as H
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

CFG = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 1, "hidden_size": 256,
       "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 384,
       "vocab_size": 1009, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
       "max_position_embeddings": 40960}
N = 40000
WANTED = [0, 1, 255, 256, 4095, 4096, 20000, 32767, 32768, 39990, 39999]


def plain_rows(folder, tokens, rows):
    """Logits of the rows ``rows`` of the one-layer model: every key and value of the sequence,
    attention, feed-forward and head for these rows only."""
    cfg, w = plain.read_model_folder(folder)
    d, nq, nkv, eps = cfg["head_dim"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["rms_norm_eps"]
    n = len(tokens)
    h = plain.embed(w["model.embed_tokens.weight"], tokens)
    p = "model.layers.0"
    y = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], eps)
    q = plain.rms_norm((y @ w[f"{p}.self_attn.q_proj.weight"].T).view(n, nq, d), w[f"{p}.self_attn.q_norm.weight"], eps)
    k = plain.rms_norm((y @ w[f"{p}.self_attn.k_proj.weight"].T).view(n, nkv, d), w[f"{p}.self_attn.k_norm.weight"], eps)
    v = (y @ w[f"{p}.self_attn.v_proj.weight"].T).view(n, nkv, d)
    cos, sin = plain.rope_tables(range(n), d, cfg["rope_theta"])
    q, k = plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin)
    out = {}
    for r in rows:
        a = torch.empty(nq, d, dtype=torch.float64)
        for head in range(nq):
            kv = head // (nq // nkv)
            a[head] = torch.softmax((k[:r + 1, kv] @ q[r, head]) * d ** -0.5, 0) @ v[:r + 1, kv]
        hr = h[r] + a.reshape(-1) @ w[f"{p}.self_attn.o_proj.weight"].T
        yr = plain.rms_norm(hr[None], w[f"{p}.post_attention_layernorm.weight"], eps)
        hr = hr + plain.swiglu_mlp(yr, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"],
                                   w[f"{p}.mlp.down_proj.weight"])[0]
        out[r] = plain.rms_norm(hr[None], w["model.norm.weight"], eps)[0] @ w["model.embed_tokens.weight"].T
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_forty_thousand_tokens_in_two_cuttings(tmp_path, dtype):
    from lockstep_b200 import ModelRunner, StepEntry
    from lockstep_b200.weights import write_random_model

    folder = write_random_model(tmp_path / "m", CFG, seed=9, dtype=dtype, init_std=0.06, gain_std=0.1)
    tokens = H.random_tokens(N, CFG["vocab_size"], 5)
    want = plain_rows(folder, tokens, WANTED)
    cuttings = ([4096] * 9 + [N - 9 * 4096 - 12] + [1] * 12, [3001, 17, 8192, 2, 5000] * 3 + [N])
    got = []
    for sizes in cuttings:
        runner = ModelRunner(folder, dtype=dtype, num_pages=N // 16 + 8, page_size=16, max_live=2, max_seq_len=40960)
        runner.open("a")
        start, rows = 0, {}
        for n in sizes:
            n = min(n, N - start)
            if n <= 0:
                break
            here = [r for r in WANTED if start <= r < start + n]
            logits = runner.step([StepEntry(uid="a", tokens=tokens[start:start + n], start=start,
                                            want=[r - start for r in here])])
            for i, r in enumerate(here):
                rows[r] = logits[i].double().cpu()
            start += n
        assert start == N and runner.kv_len("a") == N
        runner.close("a")
        assert runner.cache.free_pages() == runner.cache.total_pages()
        for r in WANTED:
            bound = (2e-5 if dtype == "float32" else 4e-2) * (1 + float(want[r].abs().max()))
            assert float((rows[r] - want[r]).abs().max()) <= bound, (sizes[:2], r)
        got.append(rows)
    if dtype == "float32":
        for r in WANTED:
            assert torch.equal(got[0][r], got[1][r]), r
