"""Decode steps recorded as CUDA graphs.

A step whose entries all bring one token launches a few hundred small kernels;
recorded once and replayed, the host's share of the step shrinks to filling one
pinned buffer.  A graph is keyed by (number of requests, capacity of the
attention work list).  More than eight requests are padded to the next multiple of
eight with rows that bring token 0 at position 0 of the cache manager's padding slot
(their keys go to the padding page, their attention work is empty, their logits are
dropped), so that a batch that shrinks as requests end does not record a graph per
size.  The capacity is rounded up to a multiple of max(CAPACITY_STEP, 4 x rows), so
that a batch records a new graph about every 1,024 decoded tokens whatever its size,
and at most MAX_GRAPHS graphs are kept (the least recently replayed one is dropped
first).  A graph holds its input
buffer (a few KB), its activations (a few hundred KB a request) and its logits
[requests, vocabulary] in float32, all from one memory pool shared by the graphs.  Everything that changes from step to step (token ids,
positions, slots, wanted rows, the attention work lists) lives in one device
buffer that is refilled before each replay; work lists are padded to the
capacity with null items, which the kernels skip.  Nothing about the
arithmetic changes: the same kernels run on the same values.

Steps that mix portions of prompts (a step that fills the token budget, say) are recorded too,
keyed by their exact number of tokens and the rounded numbers of wanted rows and split items,
when a step of the same shape comes for the third time: such steps launch some 300 kernels, and the
host is slower at enqueueing them than the device at running them.

A model whose parts are all ``graph_safe`` is one graph.  Where some are not (a mixer that
reads the step's portions on the host), the runs of graph-safe steps between them are
recorded, one graph each, and the other steps are called between the replays.
"""

from __future__ import annotations

import gc
from collections import OrderedDict

import numpy as np
import torch

from .batch import AttentionPlan, plan_attention

CAPACITY_STEP = 32      # the attention work list of a recorded step holds a multiple of this many items
MAX_GRAPHS = 24         # recorded steps kept; the least recently used one goes first
EXACT_BATCHES = 8       # up to here a step is recorded at its own size, above at the next multiple of this


def padded_batch(n: int) -> int:
    """Rows of the recorded step that serves ``n`` requests."""
    return n if n <= EXACT_BATCHES else -(-n // EXACT_BATCHES) * EXACT_BATCHES


class StaticStepContext:
    """What parts see of a recorded decode step: views into the graph's buffer."""

    def __init__(self, batch: int, capacity: int, windows: list[int], device, err, split_size: int,
                 pad_slot: int = 0):
        self.batch, self.capacity, self.windows = batch, capacity, list(windows)
        self.pad_slot = pad_slot
        self.device, self.err, self.split_size = device, err, split_size
        self.num_tokens = self.n_wanted = batch
        per_window = capacity * 8 + batch * 4
        self.size = 4 * batch + len(self.windows) * per_window
        self.host = torch.zeros(self.size, dtype=torch.int32).pin_memory()
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.size, dtype=torch.int32, device=device)
        b = batch
        self.token_ids, self.positions = self.dev[0:b], self.dev[b:2 * b]
        self.token_slot, self.wanted_rows = self.dev[2 * b:3 * b], self.dev[3 * b:4 * b]
        self._plans: dict[int, AttentionPlan] = {}
        self._offsets: dict[int, int] = {}
        off = 4 * b
        for w in self.windows:
            self._offsets[w] = off
            self._plans[w] = AttentionPlan(
                tile_work=None, n_tile=0,
                split_work=self.dev[off:off + capacity * 8].view(capacity, 8), n_split=capacity,
                combine_items=self.dev[off + capacity * 8:off + per_window].view(batch, 4),
                n_combine=batch, n_slots=capacity)
            off += per_window
        self._arange = np.arange(batch, dtype=np.int32)
        self.portions: list = []
        self.entries: list = []
        self.slots: list = []
        self.copied = torch.cuda.Event()
        self._pending = False

    def attention_plan(self, window: int, tile_tokens: int = 0) -> AttentionPlan:
        try:
            return self._plans[window]
        except KeyError:
            raise KeyError(f"a part asked for the attention plan of window {window}, which it did not "
                           "declare in attention_windows()") from None

    def fill(self, entries, slots) -> None:
        """Write this step's values into the pinned buffer and start its copy."""
        if self._pending:
            self.copied.synchronize()      # the last copy has read the pinned buffer
        b, h = self.batch, self.host_np
        n = len(entries)                   # the rows n .. b - 1 pad the step: token 0 at position 0 of the padding slot
        self.entries, self.slots = entries, slots
        start = np.zeros(b, dtype=np.int64)
        start[:n] = np.fromiter((e.start for e in entries), dtype=np.int64, count=n)
        slot = np.full(b, self.pad_slot, dtype=np.int64)
        slot[:n] = np.asarray(slots, dtype=np.int64)
        self.portions = list(zip(slots, range(n), start[:n].tolist(), [1] * n))
        h[0:b] = 0
        h[0:n] = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=n)
        h[b:2 * b] = start
        h[2 * b:3 * b] = slot
        h[3 * b:4 * b] = self._arange
        for w in self.windows:
            # one item per (entry, split): splits lo // S .. start // S of each entry, in entry order
            lo = np.maximum(0, start - w + 1) if w else np.zeros(b, dtype=np.int64)
            first, last = lo // self.split_size, start // self.split_size
            count = last - first + 1
            count[n:] = 0                  # padding rows attend to nothing: no items, an empty combine
            total = int(count.sum())
            if total > self.capacity:
                raise ValueError("the attention work list outgrew the capacity this graph was recorded for")
            base = np.cumsum(count) - count                       # first scratch slot of each entry
            owner = np.repeat(np.arange(b), count)
            split = np.arange(total) - np.repeat(base, count) + np.repeat(first, count)
            off = self._offsets[w]
            items = h[off:off + self.capacity * 8].reshape(self.capacity, 8)
            items[:total, 0] = slot[owner]
            items[:total, 1] = owner
            items[:total, 2] = 1
            items[:total, 3] = start[owner]
            items[:total, 4] = split
            items[:total, 5] = split + 1
            items[:total, 6] = np.arange(total)
            items[:total, 7] = 0
            items[total:] = 0
            comb = h[off + self.capacity * 8:off + self.capacity * 8 + b * 4].reshape(b, 4)
            comb[:, 0] = self._arange
            comb[:, 1] = base
            comb[:, 2] = 1
            comb[:, 3] = count
        self.dev.copy_(self.host, non_blocking=True)
        self.copied.record()
        self._pending = True


MIXED_MIN_TOKENS = 256   # steps of fewer tokens are not worth a graph of their own
MIXED_GRAPHS = 8         # recorded steps of mixed portions kept (least recently used goes first)
MIXED_SPLIT_STEP = 64    # the split work list of such a step holds this many items, or a power of two times as many
MIXED_PORTIONS = 4       # portions of two or more tokens such a step may hold
MIXED_SIGHTINGS = 3      # a shape is recorded when it comes for this many times
MIXED_RECORDINGS = 48    # recordings of such steps in a runner's life: a workload of ever new shapes stops recording


class StaticMixedContext:
    """What parts see of a recorded step that mixes portions of prompts and decoded tokens: the
    same fields as ``batch.StepContext``, as views into one device buffer that is refilled before
    each replay.  The number of tokens is exact (it is part of the graph's key); the wanted rows
    and the attention work lists are padded to capacities (with the first wanted row again, whose
    logits are dropped, and with null items, which the kernels skip)."""

    def __init__(self, tokens: int, wanted_cap: int, split_cap: int, max_entries: int,
                 plan_keys: list[tuple[int, int]], device, err, split_size: int):
        self.num_tokens, self.n_wanted = tokens, wanted_cap
        self.split_cap, self.max_entries = split_cap, max_entries
        self.plan_keys = sorted(plan_keys)
        self.device, self.err, self.split_size = device, err, split_size
        t = tokens
        # (a few items more than the tokens make in one portion: a launcher that chooses a kernel
        # by the number of items then sees about the real number)
        self._tile_cap = {key: t // key[1] + MIXED_PORTIONS for key in self.plan_keys}
        size = 3 * t + wanted_cap
        self._off = {}
        for key in self.plan_keys:
            self._off[key] = size
            size += 8 * self._tile_cap[key] + 8 * split_cap + 4 * max_entries
        self.size = size
        self.host = torch.zeros(size, dtype=torch.int32).pin_memory()
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(size, dtype=torch.int32, device=device)
        self.token_ids, self.positions = self.dev[0:t], self.dev[t:2 * t]
        self.token_slot, self.wanted_rows = self.dev[2 * t:3 * t], self.dev[3 * t:3 * t + wanted_cap]
        self._plans = {}
        for key in self.plan_keys:
            a = self._off[key]
            b = a + 8 * self._tile_cap[key]
            c = b + 8 * split_cap
            self._plans[key] = AttentionPlan(
                tile_work=self.dev[a:b].view(-1, 8), n_tile=self._tile_cap[key],
                split_work=self.dev[b:c].view(-1, 8) if split_cap else None, n_split=split_cap,
                combine_items=self.dev[c:c + 4 * max_entries].view(-1, 4) if split_cap else None,
                n_combine=max_entries if split_cap else 0, n_slots=split_cap)
        self.portions: list = []
        self.entries: list = []
        self.slots: list = []
        self.copied = torch.cuda.Event()
        self._pending = False
        self.wanted = 0

    def attention_plan(self, window: int, tile_tokens: int = 16) -> AttentionPlan:
        try:
            return self._plans[(window, tile_tokens)]
        except KeyError:
            raise KeyError(f"a part asked for the attention plan ({window}, {tile_tokens}), which the step "
                           "that was recorded did not ask for") from None

    def fill(self, entries, slots) -> None:
        if self._pending:
            self.copied.synchronize()
        h, t = self.host_np, self.num_tokens
        self.entries, self.slots = entries, slots
        self.portions = []
        wanted, off = [], 0
        for e, slot in zip(entries, slots):
            n = len(e.tokens)
            h[off:off + n] = e.tokens
            h[t + off:t + off + n] = np.arange(e.start, e.start + n)
            h[2 * t + off:2 * t + off + n] = slot
            wanted.extend(off + w for w in e.want)
            self.portions.append((slot, off, e.start, n))
            off += n
        if off != t or len(wanted) > self.n_wanted:
            raise ValueError("the step does not fit the recorded one")
        self.wanted = len(wanted)
        h[3 * t:3 * t + self.n_wanted] = wanted[0] if wanted else 0
        h[3 * t:3 * t + len(wanted)] = wanted
        for key in self.plan_keys:
            tile, split, combine, n_slots = plan_attention(self.portions, key[0], self.split_size, key[1])
            if len(tile) > self._tile_cap[key] or len(split) > self.split_cap or len(combine) > self.max_entries:
                raise ValueError("the step's attention work outgrew the recorded capacities")
            a = self._off[key]
            b = a + 8 * self._tile_cap[key]
            c = b + 8 * self.split_cap
            h[a:c + 4 * self.max_entries] = 0
            h[a:a + tile.size] = tile.reshape(-1)
            h[b:b + split.size] = split.reshape(-1)
            h[c:c + combine.size] = combine.reshape(-1)
        self.dev.copy_(self.host, non_blocking=True)
        self.copied.record()
        self._pending = True


def split_items(entries, windows: list[int], split_size: int) -> int:
    """The longest attention work list of a decode step over ``entries``."""
    worst = 0
    for w in windows:
        n = 0
        for e in entries:
            lo = max(0, e.start - w + 1) if w else 0
            n += e.start // split_size - lo // split_size + 1
        worst = max(worst, n)
    return worst


class DecodeGraphs:
    def __init__(self, runner, round_to: int = CAPACITY_STEP, max_graphs: int = MAX_GRAPHS):
        self.runner, self.round_to, self.max_graphs = runner, round_to, max(1, int(max_graphs))
        self.windows = sorted(set().union(*(b.attention_windows() for b in runner.model.blocks)) or {0})
        self.graphs: OrderedDict[tuple[int, int], tuple] = OrderedDict()
        self.pool = None
        self.replays = 0
        self.dropped = 0
        # steps that mix portions: recorded when a step of the same shape comes a second time
        self.mixed: OrderedDict[tuple, tuple] = OrderedDict()
        self.mixed_seen: OrderedDict[tuple, int] = OrderedDict()
        self.mixed_replays = 0
        self.mixed_recordings = 0

    def capacity_for(self, entries) -> int:
        n = split_items(entries, self.windows, self.runner.split_size)
        step = max(self.round_to, 4 * padded_batch(len(entries)))
        return -(-n // step) * step

    def key_for(self, entries) -> tuple[int, int]:
        """(rows, capacity) of the recorded step that serves ``entries``."""
        return padded_batch(len(entries)), self.capacity_for(entries)

    def ready(self, key) -> bool:
        return key in self.graphs

    def input_bytes(self) -> int:
        """Bytes that go from the host to the device before a replay of the largest recorded step."""
        return 4 * max((entry[1].size for entry in self.graphs.values()), default=0)

    def record(self, key) -> None:
        """Record the model's forward for ``key`` (nothing runs while recording).

        The program's runs of graph-safe steps become one graph each; a step that is not
        graph-safe (a part that reads host-side values of the context) is kept as it is and
        called between the replays, on the same residual stream: the buffer that the recorded
        embedding made.  Such steps are not called here, so a mixer's state is not touched by
        recording."""
        r = self.runner
        batch, capacity = key
        ctx = StaticStepContext(batch, capacity, self.windows, r.device, r.err, r.split_size,
                                pad_slot=r.cache.pad_slot)
        self.graphs[key] = self._record(ctx)
        while len(self.graphs) > self.max_graphs:
            # nothing of the dropped graph is in flight: _record() synchronised
            self.graphs.popitem(last=False)
            self.dropped += 1

    def _record(self, ctx) -> tuple:
        """(pieces, ctx, residual stream, logits or None, launches recorded) of the program on ``ctx``."""
        r = self.runner
        if self.pool is None:
            self.pool = torch.cuda.graph_pool_handle()
        torch.cuda.synchronize()
        from .. import kernels as K

        before = K.LAUNCHES[0]
        # No object may be collected while the stream is capturing: the destructor of
        # another runner's graph calls into CUDA and would invalidate the capture.
        collecting = gc.isenabled()
        gc.collect()
        gc.disable()
        r.rt.exact_sizes = True
        pieces, h, stream = [], None, None
        try:
            for safe, fns in _runs(r.program):
                if not safe:
                    pieces.append((None, fns))
                    continue
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, pool=self.pool):
                    for fn in fns:
                        h = fn(h, ctx)
                        if stream is None:
                            stream = h       # what the embedding made: the residual stream
                pieces.append((graph, None))
        finally:
            r.rt.exact_sizes = False
            if collecting:
                gc.enable()
        recorded = K.LAUNCHES[0] - before
        K.LAUNCHES[0] = before               # recording launches nothing
        # the last step's result is the logits: the graph's own buffer when that step is
        # recorded, else what the step returns at every replay
        logits = h if pieces[-1][0] is not None else None
        return pieces, ctx, stream, logits, recorded

    # -- steps that mix portions of prompts and decoded tokens --------------
    def mixed_key_for(self, entries) -> tuple | None:
        """(tokens, wanted rows, split items) of the recorded step that would serve ``entries``, the
        last two rounded up; None for steps too small to be worth recording, with more portions
        than its tile work lists are made for, or with more wanted rows than requests can be live."""
        tokens = sum(len(e.tokens) for e in entries)
        if tokens < MIXED_MIN_TOKENS or len(entries) > self.runner.cache.max_live:
            return None
        wanted = sum(len(e.want) for e in entries)
        singles = [e for e in entries if len(e.tokens) == 1]
        splits = split_items(singles, self.windows, self.runner.split_size) if singles else 0
        # the tile work lists hold what the tokens can make in up to MIXED_PORTIONS portions
        if sum(len(e.tokens) > 1 for e in entries) > MIXED_PORTIONS:
            return None
        # few classes, so that a continuous batch whose decoded rows come and go records a
        # handful of steps and not one per mix: wanted rows in sixty-fours (at most as many as requests may be live),
        # split items the next power of two
        split_cap = 0
        if splits:
            split_cap = MIXED_SPLIT_STEP
            while split_cap < splits:
                split_cap *= 2
        if wanted > self.runner.cache.max_live:
            return None
        return tokens, min(self.runner.cache.max_live, -(-max(wanted, 1) // 64) * 64), split_cap

    def mixed_ready(self, key) -> bool:
        return key in self.mixed

    def mixed_seen_again(self, key) -> bool:
        """Counts a step of this shape that ran unrecorded; True from the MIXED_SIGHTINGS-th on."""
        if self.mixed_recordings >= MIXED_RECORDINGS:
            return False
        n = self.mixed_seen.pop(key, 0) + 1
        self.mixed_seen[key] = n
        while len(self.mixed_seen) > 64:
            self.mixed_seen.popitem(last=False)
        return n >= MIXED_SIGHTINGS

    def record_mixed(self, key, plan_keys) -> None:
        tokens, wanted_cap, split_cap = key
        r = self.runner
        ctx = StaticMixedContext(tokens, wanted_cap, split_cap, r.cache.max_live, list(plan_keys), r.device,
                                 r.err, r.split_size)
        self.mixed[key] = self._record(ctx)
        self.mixed_recordings += 1
        while len(self.mixed) > MIXED_GRAPHS:
            dropped, _ = self.mixed.popitem(last=False)
            self.mixed_seen.pop(dropped, None)        # it has to come three times again
            self.dropped += 1

    def replay_mixed(self, key, entries, slots) -> torch.Tensor:
        from .. import kernels as K

        pieces, ctx, h, logits, recorded = self.mixed[key]
        self.mixed.move_to_end(key)
        ctx.fill(entries, slots)
        for graph, fns in pieces:
            if graph is not None:
                graph.replay()
            else:
                for fn in fns:
                    h = fn(h, ctx)
        K.LAUNCHES[0] += recorded
        self.mixed_replays += 1
        return (h if logits is None else logits)[:ctx.wanted]

    def replay(self, key, entries, slots, tokens_device=None) -> torch.Tensor:
        """``tokens_device`` (int32, one per entry, on the device): the step's token ids, in
        place of the entries' own: they are copied into the graph's buffer on the stream,
        after the host's values and before the replay."""
        from .. import kernels as K

        pieces, ctx, h, logits, recorded = self.graphs[key]
        self.graphs.move_to_end(key)
        ctx.fill(entries, slots)
        if tokens_device is not None:
            ctx.token_ids[:len(entries)].copy_(tokens_device, non_blocking=True)
        for graph, fns in pieces:
            if graph is not None:
                graph.replay()
            else:
                for fn in fns:
                    h = fn(h, ctx)
        K.LAUNCHES[0] += recorded
        self.replays += 1
        return (h if logits is None else logits)[:len(entries)]


def _runs(program):
    """``program`` [(graph_safe, fn)] as runs [(graph_safe, [fn, ...])] of equal safety."""
    out: list[tuple[bool, list]] = []
    for safe, fn in program:
        if out and out[-1][0] == safe:
            out[-1][1].append(fn)
        else:
            out.append((safe, [fn]))
    return out
