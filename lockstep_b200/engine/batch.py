"""One step's batch: what the step function is given and what parts see of it.

A batch is a list of entries (request, its next tokens, the position of the
first of them, the places whose logits are wanted).  Entries are packed into
one token axis.  ``StepContext`` holds the packed device arrays and builds, per
window size, the attention work lists: how rows are cut into tiles and splits
is a function of each row's own position alone (split = position //
split_size), never of the batch.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

TILE_TOKENS = 16   # query tokens of one block of the tile kernel (csrc/attention_simt.cu)


@dataclass
class StepEntry:
    uid: str
    tokens: list[int]
    start: int                       # position of tokens[0]
    want: list[int] = field(default_factory=list)   # places among ``tokens``


@dataclass
class AttentionPlan:
    tile_work: torch.Tensor | None
    n_tile: int
    split_work: torch.Tensor | None
    n_split: int
    combine_items: torch.Tensor | None
    n_combine: int
    n_slots: int


def plan_attention(portions, window: int, split_size: int, tile_tokens: int = TILE_TOKENS):
    """portions: (slot, token offset, start position, length) per entry.
    Returns numpy arrays (tile_work [n,8], split_work [n,8], combine [n,4]) and
    the number of scratch slots.  Tiles hold up to ``tile_tokens`` tokens and are
    listed longest context first, so that the heaviest start first."""
    tile, split, combine = [], [], []
    n_slots = 0
    for slot, off, start, length in portions:
        if length == 1:
            lo = max(0, start - window + 1) if window else 0
            s_lo, s_hi = lo // split_size, start // split_size
            combine.append((off, n_slots, 1, s_hi - s_lo + 1))
            for s in range(s_lo, s_hi + 1):
                split.append((slot, off, 1, start, s, s + 1, n_slots, 0))
                n_slots += 1
        else:
            for i in range(0, length, tile_tokens):
                ntok = min(tile_tokens, length - i)
                pos0 = start + i
                lo = max(0, pos0 - window + 1) if window else 0
                tile.append((slot, off + i, ntok, pos0, lo // split_size,
                             (pos0 + ntok - 1) // split_size + 1, -1, 0))
    tile.sort(key=lambda item: -(item[3] + item[2]))
    as_np = lambda rows, w: np.asarray(rows, dtype=np.int32).reshape(-1, w)
    return as_np(tile, 8), as_np(split, 8), as_np(combine, 4), n_slots


class StepContext:
    def __init__(self, entries: list[StepEntry], slots: list[int], device, err, split_size: int):
        self.entries, self.slots, self.device, self.err = entries, slots, device, err
        self.split_size = split_size
        ids, pos, tslot, wanted = [], [], [], []
        self.portions = []
        off = 0
        for e, slot in zip(entries, slots):
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"{e.uid}: an entry must bring at least one token")
            ids.extend(e.tokens)
            pos.extend(range(e.start, e.start + n))
            tslot.extend([slot] * n)
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"{e.uid}: wanted place {w} outside its {n} tokens")
                wanted.append(off + w)
            self.portions.append((slot, off, e.start, n))
            off += n
        self.num_tokens = off
        self.n_wanted = len(wanted)
        packed = np.asarray(ids + pos + tslot + wanted, dtype=np.int64)
        if packed.size and (packed.min() < -(2 ** 31) or packed.max() >= 2 ** 31):
            raise ValueError("a token id or position does not fit 32 bits")
        dev = torch.from_numpy(packed.astype(np.int32)).to(device)
        t = off
        self.token_ids = dev[0:t]
        self.positions = dev[t:2 * t]
        self.token_slot = dev[2 * t:3 * t]
        self.wanted_rows = dev[3 * t:3 * t + self.n_wanted]
        self._plans: dict[tuple[int, int], AttentionPlan] = {}

    def attention_plan(self, window: int, tile_tokens: int = TILE_TOKENS) -> AttentionPlan:
        """Work lists for attention with ``window`` (0: all keys): portions of two or
        more tokens cut into tiles of ``tile_tokens``, single tokens into one item
        per split plus a combine item."""
        plan = self._plans.get((window, tile_tokens))
        if plan is None:
            tile, split, combine, n_slots = plan_attention(self.portions, window, self.split_size, tile_tokens)
            flat = np.concatenate([tile.reshape(-1), split.reshape(-1), combine.reshape(-1)])
            dev = torch.from_numpy(flat).to(self.device) if flat.size else None
            a, b = tile.size, tile.size + split.size
            plan = AttentionPlan(
                tile_work=dev[:a].view(-1, 8) if tile.size else None, n_tile=len(tile),
                split_work=dev[a:b].view(-1, 8) if split.size else None, n_split=len(split),
                combine_items=dev[b:].view(-1, 4) if combine.size else None, n_combine=len(combine),
                n_slots=n_slots)
            self._plans[(window, tile_tokens)] = plan
        return plan
