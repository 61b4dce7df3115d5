"""Grouped-query attention over the paged cache.

q, k, v projections without bias as one product over the row-concatenated
weights (a row of the product is the same dot product as in three separate
ones), optional per-head RMSNorm of q and k before the rotation, rotation by
the position encoding, write of k and v into the cache pages, causal softmax
attention with an optional window, output projection added into the residual
stream (LockStep: engine/model/qwen3.py:246-277, engine/kernels/attention.py).
"""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import CacheNeed, Mixer, PositionEncoding, Runtime, WeightSpec, register_part
from .norm import NormedRows


class GQAttention(Mixer):
    graph_safe = True
    accepts_normed_rows = True

    def __init__(self, hidden_size, num_heads, num_kv_heads, head_dim, scale, window, qk_norm_eps,
                 position: PositionEncoding, runtime: Runtime):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise ValueError(
                f"head_dim {head_dim} is not supported: the attention kernels take multiples of 16 up to 256")
        self.h, self.nq, self.nkv, self.d = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.scale, self.window = float(scale), int(window or 0)
        self.qk_norm_eps = qk_norm_eps
        self.position, self.rt = position, runtime
        self.w_qkv = self.w_o = self.q_gain = self.k_gain = self.slopes = None
        # in float32 every row takes the tile kernel, so that a row's bits do not
        # depend on whether it was decoded or part of a prompt
        self.exact = runtime.dtype == torch.float32

    def cache_need(self):
        return CacheNeed("paged_kv", kv_heads=self.nkv, head_dim=self.d, window=self.window)

    def attention_windows(self):
        return {self.window}

    def weight_specs(self):
        specs = {
            "q_proj.weight": WeightSpec((self.nq * self.d, self.h)),
            "k_proj.weight": WeightSpec((self.nkv * self.d, self.h)),
            "v_proj.weight": WeightSpec((self.nkv * self.d, self.h)),
            "o_proj.weight": WeightSpec((self.h, self.nq * self.d)),
        }
        if self.qk_norm_eps is not None:
            specs["q_norm.weight"] = WeightSpec((self.d,), "gain")
            specs["k_norm.weight"] = WeightSpec((self.d,), "gain")
        return specs

    def bind(self, tensors):
        self.w_qkv = torch.cat(
            [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"]
        self.slopes = self.position.score_slopes(self.nq)      # asked once: a step allocates nothing for it
        if self.qk_norm_eps is not None:
            self.q_gain, self.k_gain = tensors["q_norm.weight"], tensors["k_norm.weight"]

    def forward(self, x, ctx, cache, residual):
        nq, nkv, d = self.nq, self.nkv, self.d
        t = residual.shape[0]
        q = self.rt.rows(t, nq * d)
        rot = self.position.rotary()
        cos, sin, rot_dim = rot if rot is not None else (None, None, 0)
        heads = (q, cache.pages, self.q_gain, self.k_gain, cos, sin, ctx.positions, ctx.token_slot,
                 cache.block_table, nq, nkv, d, rot_dim, self.qk_norm_eps or 0.0, cache.writes, self.rt.err)
        interleaved = bool(rot_dim and self.position.rotary_interleaved)
        # a bias on the scores is known to the CUDA-core attention kernels only
        slopes = self.slopes
        tensor_core_attention = not self.exact and slopes is None
        # few tokens: the product finishes its heads itself (norm, rotation, cache write); else
        # the projection goes through memory and a second kernel does that
        fused = False
        if t <= K.FEW_TOKENS and not self.exact and not interleaved:
            pending = isinstance(x, NormedRows) and x.pending()
            fused = K.gemm_nt_tc_qkv_heads(None if pending else (x.materialize() if isinstance(x, NormedRows) else x),
                                           self.w_qkv, *heads,
                                           normed=(x.h, x.gain, x.eps, x.row_index) if pending else None)
        if not fused:
            qkv = self.rt.rows(t, (nq + 2 * nkv) * d)
            if isinstance(x, NormedRows):
                x.linear(self.w_qkv, qkv, K.EPILOGUE_STORE, self.rt.err)
            else:
                K.gemm_nt(x, self.w_qkv, qkv, err=self.rt.err)
            K.qk_norm_rope_store(qkv, *heads, interleaved=interleaved)
        attn = self.rt.rows(t, nq * d)
        plan, done = None, False
        if tensor_core_attention and d in (64, 128):
            plan = ctx.attention_plan(self.window, K.attention_prefill_tc_tile_tokens())
            done = not plan.n_tile or K.attention_prefill_tc(
                q, cache.pages, attn, plan.tile_work, plan.n_tile, cache.block_table, nq, nkv, d,
                self.window, self.scale, self.rt.err)
        if not done:
            plan = ctx.attention_plan(self.window)
            if plan.n_tile:
                K.attention_tile(q, cache.pages, attn, None, None, plan.tile_work, plan.n_tile,
                                 cache.block_table, nq, nkv, d, self.window, self.scale, self.rt.err, slopes)
        if plan.n_split:
            part_acc = self.rt.rows(plan.n_slots, nq, d, dtype=torch.float32)
            part_ml = self.rt.rows(plan.n_slots, nq, 2, dtype=torch.float32)
            done = False
            if tensor_core_attention:
                done = K.attention_decode_mma(q, cache.pages, part_acc, part_ml, plan.split_work,
                                              plan.n_split, cache.block_table, nq, nkv, d, self.window,
                                              self.scale, self.rt.err)
            if not done and not self.exact:
                done = K.attention_decode(q, cache.pages, part_acc, part_ml, plan.split_work,
                                          plan.n_split, cache.block_table, nq, nkv, d, self.window,
                                          self.scale, self.rt.err, slopes)
            if not done:
                K.attention_tile(q, cache.pages, None, part_acc, part_ml, plan.split_work,
                                 plan.n_split, cache.block_table, nq, nkv, d, self.window,
                                 self.scale, self.rt.err, slopes)
            K.attention_combine(part_acc, part_ml, attn, plan.combine_items, plan.n_combine, nq, d)
        K.gemm_nt(attn, self.w_o, residual, K.EPILOGUE_RESIDUAL, err=self.rt.err)


@register_part("mixer", "gqa_attention")
def _build(spec, runtime, position=None, **_):
    return GQAttention(spec["hidden_size"], spec["num_heads"], spec["num_kv_heads"], spec["head_dim"],
                       spec["scale"], spec.get("window", 0), spec.get("qk_norm_eps"), position, runtime)
