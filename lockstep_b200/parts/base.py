"""Interfaces of the parts a layer is put together from.

A part is built from a ``PartSpec`` (its sizes and constants) and a
``Runtime`` (device, element type, page size, error word).  It declares the
tensors it needs with names relative to its own prefix, receives them in
``bind``, and does its work in ``forward``.  No part knows which model it is in.

Shapes: ``x`` and the outputs of norms are [tokens, width] in the engine's
element type; the residual stream ``h`` is [tokens, hidden] float32, and a
mixer or feed-forward adds its result into it in place.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping

import torch

from ..config.spec import PartSpec


@dataclass(frozen=True)
class WeightSpec:
    """A tensor a part needs.  role: "matrix" (used in a product), "table"
    (looked up by integer id) or "gain" (a norm's scale vector)."""

    shape: tuple[int, ...]
    role: str = "matrix"


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps between steps.

    kind "paged_kv": keys and values of ``kv_heads`` x ``head_dim`` per token in
    pages; ``window`` > 0 means only the last ``window`` positions are read, so
    pages behind it can be given back.  kind "state": one tensor of
    ``state_shape`` per request, of fixed size, in a slot.
    """

    kind: str
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    state_shape: tuple[int, ...] = ()
    state_dtype: torch.dtype = torch.float32

    def group_key(self):
        if self.kind == "paged_kv":
            return ("paged_kv", self.kv_heads, self.head_dim, self.window)
        return ("state", tuple(self.state_shape), str(self.state_dtype))


@dataclass
class Runtime:
    """What every part of one model shares."""

    device: torch.device
    dtype: torch.dtype
    page_size: int
    max_positions: int
    err: torch.Tensor            # int32[2] device error word
    options: dict = field(default_factory=dict)
    # True while a step is recorded into a CUDA graph: buffers then have exactly the rows asked
    # for (they are kept for the graph's life, and their sizes never change).
    exact_sizes: bool = False

    def rows(self, rows: int, *tail: int, dtype: torch.dtype | None = None) -> torch.Tensor:
        """An uninitialised [rows, *tail] buffer of a step's activations (``dtype``: the
        engine's element type unless given).

        The number of tokens in a step changes from step to step, and with it the size of
        every activation.  torch's caching allocator keeps freed blocks by size, and a block
        of more than a few MB serves only requests of nearly its own size, so a step with a
        few more rows than any step before it asks the driver for new memory: a call that
        waits for the device, tens of milliseconds in the middle of serving.  So the buffer
        is cut from an allocation whose row count is rounded up (to 8 up to 64 rows, to 64
        above): steps of nearly equal size then ask for equal sizes, and the allocator's
        blocks are used again.  The rows beyond ``rows`` are never read or written.
        """
        dtype = self.dtype if dtype is None else dtype
        if self.exact_sizes or rows <= 8:
            return torch.empty((rows, *tail), dtype=dtype, device=self.device)
        step = 8 if rows <= 64 else 64
        return torch.empty((-(-rows // step) * step, *tail), dtype=dtype, device=self.device)[:rows]


class Part:
    """Base of all parts."""

    # True when ``forward`` only launches kernels whose arguments are device
    # tensors of the step context and shapes that depend on the batch's token
    # count alone: such a part may be recorded in a CUDA graph and replayed with
    # new contents in the same buffers.  A part that reads host-side values of the
    # context (``ctx.portions``) in ``forward`` must leave it False: it is then called as
    # it is between the recorded runs of the other parts.  Whether recorded or not, a part
    # takes token ids from ``ctx.token_ids`` (on the device) only: a decode step may be
    # launched before the host has seen the tokens it brings.
    graph_safe = False

    # True for a mixer or feed-forward whose ``forward`` takes ``x`` either as a tensor or
    # as a ``norm.NormedRows`` (rows still to be normalised), so that it can make the norm
    # inside its first product.  Parts that leave it False always get a tensor.
    accepts_normed_rows = False

    def attention_windows(self) -> set[int]:
        """Window sizes for which this part asks ``ctx.attention_plan``."""
        return set()

    def weight_specs(self) -> dict[str, WeightSpec]:
        return {}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        if tensors:
            raise ValueError(f"{type(self).__name__} takes no weights")


class Norm(Part):
    def forward(self, h: torch.Tensor, row_index: torch.Tensor | None = None) -> torch.Tensor:
        """Normalise float32 rows of ``h`` (all, or those ``row_index`` names) into
        a new tensor of the engine's element type."""
        raise NotImplementedError


class PositionEncoding(Part):
    """How a mixer learns where its tokens are.  A position encoding may do any of three
    things (an absolute table that is added to the embedding belongs to the embedding part,
    which sees ``ctx.positions``):"""

    # rotated pairs are elements (2i, 2i + 1) of a head instead of (i, i + rot_dim / 2)
    rotary_interleaved = False

    def rotary(self):
        """(cos, sin, rot_dim) tables [max_positions, rot_dim/2] for a mixer that
        rotates its queries and keys, or None."""
        return None

    def score_slopes(self, num_heads: int):
        """float32 [num_heads] on the device, or None: the score of a query at position p
        with a key at position j gets slopes[head] x (j - p) added before the softmax (a
        bias that grows with distance, in place of or beside a rotation)."""
        return None


class Mixer(Part):
    def cache_need(self) -> CacheNeed | None:
        return None

    def forward(self, x: torch.Tensor, ctx, cache, residual: torch.Tensor) -> None:
        """Mix tokens of ``x`` [tokens, hidden] (using and updating ``cache``) and
        add the result into ``residual`` [tokens, hidden] float32."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor) -> None:
        raise NotImplementedError


class Block(Part):
    def cache_need(self) -> CacheNeed | None:
        raise NotImplementedError

    def forward(self, h: torch.Tensor, ctx, cache) -> None:
        """Run the layer on the residual stream ``h`` in place."""
        raise NotImplementedError

    def steps(self) -> list[tuple[bool, Callable]]:
        """The layer's work cut into steps that run one after the other: pairs
        ``(graph_safe, fn)`` with ``fn(h, ctx, cache)`` changing ``h`` in place.  Running all
        of them is ``forward``.  A recorded decode step records runs of graph-safe steps and
        calls the others as they are, so an arrangement that names its mixer and its
        feed-forward as steps of their own keeps the one in a graph when the other cannot be."""
        return [(bool(self.graph_safe), self.forward)]


# ---------------------------------------------------------------------------
# registries: (category, kind) -> builder(spec, runtime, **extra) -> Part
# ---------------------------------------------------------------------------

CATEGORIES = ("block", "mixer", "feed_forward", "norm", "position", "embedding", "head")
_BUILDERS: dict[tuple[str, str], Callable[..., Part]] = {}


def register_part(category: str, kind: str):
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; one of {CATEGORIES}")

    def wrap(builder):
        _BUILDERS[(category, kind)] = builder
        return builder

    return wrap


def unregister_part(category: str, kind: str) -> None:
    _BUILDERS.pop((category, kind), None)


def build_part(category: str, spec: PartSpec, runtime: Runtime, **extra: Any) -> Part:
    try:
        builder = _BUILDERS[(category, spec.kind)]
    except KeyError:
        known = sorted(k for c, k in _BUILDERS if c == category)
        raise KeyError(f"no {category} part is registered as {spec.kind!r}; known: {known}") from None
    return builder(spec, runtime, **extra)


def known_parts(category: str) -> list[str]:
    return sorted(k for c, k in _BUILDERS if c == category)
