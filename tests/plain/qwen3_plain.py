"""A plain, slow Qwen3 dense forward pass used only as the test oracle.

Whole sequences, no cache, one function for each part. It shares no code with
``lockstep_b200``: it reads ``config.json`` and ``model.safetensors`` on its
own, and every formula is written out from LockStep's files (cited as
``path:line`` within the LockStep project).

LockStep's own fp64 CPU forward (``bench/fp64_reference.py``) imports on the
CPU; ``tests/golden/make_golden.py`` ran it once on a tiny random model and the
outputs it wrote are compared with this file in ``tests/test_plain.py``.

Everything runs in the dtype of ``compute`` (float32 or float64) on the CPU.
The weights are used at the values the file holds (a bfloat16 file gives
bfloat16-rounded values, upcast exactly).
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors.torch import load_file


# --------------------------------------------------------------------------
# reading a model folder
# --------------------------------------------------------------------------

def read_model_folder(folder, compute=torch.float64):
    """Return (config dict, weights dict upcast to ``compute``).

    A tied head is an alias of the embedding, as in engine/model/qwen3.py:201-202.
    """
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    raw = load_file(str(folder / "model.safetensors"))
    w = {k: v.to(compute) for k, v in raw.items()}
    if cfg.get("tie_word_embeddings", False) and "lm_head.weight" not in w:
        w["lm_head.weight"] = w["model.embed_tokens.weight"]
    return cfg, w


# --------------------------------------------------------------------------
# one function for each part
# --------------------------------------------------------------------------

def embed(table, token_ids):
    """h = embed_tokens.weight[token_ids], no scaling (engine/model/qwen3.py:235)."""
    return table[torch.as_tensor(token_ids, dtype=torch.long)]


def rms_norm(x, gain, eps):
    """y = x * rsqrt(mean(x^2) + eps) * w over the last dim
    (engine/kernels/rmsnorm.py:30-38, bench/fp64_reference.py:86-90)."""
    variance = (x * x).mean(dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(variance + eps)) * gain


def rope_tables(positions, head_dim, theta, compute=torch.float64):
    """cos and sin [len, head_dim/2]: inv_freq_i = theta^(-2i/d), angle = pos*inv_freq,
    built in float64 (engine/model/qwen3.py:117-129)."""
    half = head_dim // 2
    exponent = torch.arange(0, half, dtype=torch.float64) * 2.0 / head_dim
    inv_freq = 1.0 / (float(theta) ** exponent)
    pos = torch.as_tensor(positions, dtype=torch.float64)
    ang = pos[:, None] * inv_freq[None, :]
    return ang.cos().to(compute), ang.sin().to(compute)


def apply_rope(x, cos, sin):
    """Half rotation on [T, heads, d]: out[i] = x[i]c - x[i+h]s, out[i+h] = x[i+h]c + x[i]s
    (engine/kernels/rope.py:38-56, bench/fp64_reference.py:99-104)."""
    half = x.shape[-1] // 2
    lo, hi = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1)


def causal_attention(q, k, v, scale, window=0, q_positions=None, k_positions=None):
    """Softmax attention of q [Tq, nq, d] over k, v [Tk, nkv, d].

    Query head hq reads kv head hq // (nq / nkv); a key is kept iff
    k_pos <= q_pos (engine/kernels/attention.py:91-93), and, when ``window`` > 0,
    also q_pos - k_pos < window (not in LockStep; the engine's window option).
    Softmax is the plain max-subtracted one (bench/fp64_reference.py:40-49).
    """
    tq, nq, d = q.shape
    tk, nkv, _ = k.shape
    group = nq // nkv
    if q_positions is None:
        q_positions = torch.arange(tk - tq, tk)
    if k_positions is None:
        k_positions = torch.arange(tk)
    qp = torch.as_tensor(q_positions)[:, None]
    kp = torch.as_tensor(k_positions)[None, :]
    keep = kp <= qp
    if window and window > 0:
        keep = keep & ((qp - kp) < window)
    out = torch.empty_like(q)
    for h in range(nq):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~keep, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        e = (s - m).exp()
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def swiglu_mlp(x, w_gate, w_up, w_down):
    """down(silu(gate(x)) * up(x)), no biases
    (engine/model/qwen3.py:285-287, engine/kernels/swiglu.py:25-29)."""
    g = x @ w_gate.T
    u = x @ w_up.T
    return (g * torch.sigmoid(g) * u) @ w_down.T


def layer_window(cfg, layer):
    """Window of a layer: layers at or past ``max_window_layers`` are windowed when
    ``use_sliding_window`` is set (LockStep never reads these keys; full attention
    is engine/kernels/attention.py:91-93)."""
    if cfg.get("use_sliding_window", False) and cfg.get("sliding_window"):
        if layer >= int(cfg.get("max_window_layers", 0)):
            return int(cfg["sliding_window"])
    return 0


def attention_block(x, w, prefix, cfg, cos, sin, window=0):
    """q/k/v projections, per-head q_norm/k_norm, RoPE, attention, o_proj
    (engine/model/qwen3.py:246-277)."""
    t = x.shape[0]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    q = (x @ w[f"{prefix}.q_proj.weight"].T).view(t, nq, d)
    k = (x @ w[f"{prefix}.k_proj.weight"].T).view(t, nkv, d)
    v = (x @ w[f"{prefix}.v_proj.weight"].T).view(t, nkv, d)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], cfg["rms_norm_eps"])
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], cfg["rms_norm_eps"])
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    a = causal_attention(q, k, v, 1.0 / math.sqrt(d), window=window)
    return a.reshape(t, nq * d) @ w[f"{prefix}.o_proj.weight"].T


def decoder_layer(h, w, layer, cfg, cos, sin):
    """Pre-norm block: h += attn(norm(h)); h += mlp(norm(h))
    (engine/model/qwen3.py:242-287)."""
    p = f"model.layers.{layer}"
    eps = cfg["rms_norm_eps"]
    y = rms_norm(h, w[f"{p}.input_layernorm.weight"], eps)
    h = h + attention_block(y, w, f"{p}.self_attn", cfg, cos, sin, window=layer_window(cfg, layer))
    y = rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps)
    h = h + swiglu_mlp(
        y,
        w[f"{p}.mlp.gate_proj.weight"],
        w[f"{p}.mlp.up_proj.weight"],
        w[f"{p}.mlp.down_proj.weight"],
    )
    return h


def hidden_states(cfg, w, token_ids, compute=torch.float64):
    """Final-normed hidden rows [T, H] for a whole sequence
    (engine/model/qwen3.py:226-291)."""
    h = embed(w["model.embed_tokens.weight"], token_ids).to(compute)
    cos, sin = rope_tables(range(len(token_ids)), cfg["head_dim"], cfg["rope_theta"], compute)
    for layer in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, w, layer, cfg, cos, sin)
    return rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])


def logits(cfg, w, token_ids, compute=torch.float64):
    """Logits [T, V] at every position of a whole sequence
    (engine/model/qwen3.py:291-292)."""
    return hidden_states(cfg, w, token_ids, compute) @ w["lm_head.weight"].T


def model_logits(folder, token_ids, compute=torch.float64):
    cfg, w = read_model_folder(folder, compute)
    return logits(cfg, w, token_ids, compute)


def greedy_generate(cfg, w, prompt, max_new_tokens, compute=torch.float64):
    """Argmax decoding by re-running the whole sequence each step; ties go to the
    lowest id (engine/sampler/philox.py:64-68)."""
    ids = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        row = logits(cfg, w, ids, compute)[-1]
        tok = int(torch.nonzero(row == row.max())[0].item())
        out.append(tok)
        ids.append(tok)
    return out


# --------------------------------------------------------------------------
# sampling (engine/sampler/philox.py)
# --------------------------------------------------------------------------

def philox_4x32(counter, key, rounds=10):
    """Philox-4x32 (engine/sampler/philox.py:29-48): multipliers 0xD2511F53 and
    0xCD9E8D57, Weyl increments 0x9E3779B9 and 0xBB67AE85."""
    mask = 0xFFFFFFFF
    c0, c1, c2, c3 = (x & mask for x in counter)
    k0, k1 = (x & mask for x in key)
    for r in range(rounds):
        p0 = 0xD2511F53 * c0
        p1 = 0xCD9E8D57 * c2
        hi0, lo0 = (p0 >> 32) & mask, p0 & mask
        hi1, lo1 = (p1 >> 32) & mask, p1 & mask
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & mask, lo1, (hi0 ^ c3 ^ k1) & mask, lo0
        if r < rounds - 1:
            k0 = (k0 + 0x9E3779B9) & mask
            k1 = (k1 + 0xBB67AE85) & mask
    return c0, c1, c2, c3


def uniform(seed, uid, position, index=0):
    """u in [0,1) keyed on (seed, sha256(uid)[:8], position)
    (engine/sampler/philox.py:19-61)."""
    import hashlib

    key64 = int.from_bytes(hashlib.sha256(uid.encode("utf-8")).digest()[:8], "big")
    mixed = seed ^ key64
    words = philox_4x32(
        (position & 0xFFFFFFFF, (position >> 32) & 0xFFFFFFFF, index & 0xFFFFFFFF, 0),
        (mixed & 0xFFFFFFFF, (mixed >> 32) & 0xFFFFFFFF),
    )
    return words[0] * 2.0 ** -32


def sample_top_p(row, seed, uid, position, p=1.0, temperature=1.0):
    """Nucleus sampling: softmax(logits/T) in float64, order by (-prob, id), keep the
    shortest head whose mass reaches p, inverse CDF with the Philox draw
    (engine/sampler/philox.py:71-98)."""
    if temperature <= 0:
        row = row.to(torch.float32)
        return int(torch.nonzero(row == row.max())[0].item())
    values = (row.to(torch.float32) / temperature).to(torch.float64)
    m = values.max()
    e = (values - m).exp()
    probs = e / e.sum()
    order = sorted(range(probs.numel()), key=lambda i: (-float(probs[i]), i))
    ordered = probs[order]
    cum = torch.cumsum(ordered, dim=0)
    keep = int(torch.searchsorted(cum, torch.tensor(p, dtype=torch.float64)).item()) + 1
    keep = min(keep, len(order))
    head = ordered[:keep]
    draw = uniform(seed, uid, position) * float(head.sum())
    chosen = int(torch.searchsorted(torch.cumsum(head, dim=0), torch.tensor(draw, dtype=torch.float64)).item())
    return order[min(chosen, keep - 1)]
