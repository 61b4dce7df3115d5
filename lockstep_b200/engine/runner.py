"""The step function: one batch in, logits at the wanted places out.

``ModelRunner`` owns the model's parts, its weights and the cache manager.
``step`` runs only the tokens it is given, as one batch, on top of what earlier
steps left in the cache: portions of prompts beside single decoded tokens, cut
anywhere.  Generation, the scheduler and trace replay all go through it.
"""

from __future__ import annotations

from pathlib import Path

import torch

from .. import kernels as K
from ..cache import CacheManager, OutOfPages
from ..config import load_config
from ..parts import Runtime
from ..weights import load_weights
from .batch import StepContext, StepEntry
from .model import Model

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


class ModelRunner:
    def __init__(self, model_dir, dtype="bfloat16", device="cuda:0", num_pages: int = 512,
                 page_size: int = 16, max_live: int = 64, max_seq_len: int | None = None,
                 use_graphs: bool = True, poison_freed_pages: bool = False, check_exclusive: bool = False):
        K.require_cuda()
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.dtype = parse_dtype(dtype)
        self.config = load_config(model_dir)
        self.spec = self.config.model_spec()
        self.max_seq_len = int(max_seq_len or self.spec.max_positions)
        K.library("core")
        self.split_size = K.attention_split_size()
        if self.split_size % page_size or page_size <= 0:
            raise ValueError(
                f"page_size {page_size} must divide the attention split of {self.split_size} tokens "
                "and the 32- and 64-token key tiles")
        if 32 % page_size and page_size % 32:
            raise ValueError(f"page_size {page_size} is not supported (use 8, 16, 32 or 64)")
        self.page_size = int(page_size)
        self.err = K.new_error_word(self.device)
        self.rt = Runtime(device=self.device, dtype=self.dtype, page_size=self.page_size,
                          max_positions=self.max_seq_len, err=self.err)
        self.model = Model(self.spec, self.rt)
        self._cast_report: dict = {}
        tensors = load_weights(Path(model_dir), self.model.weight_specs(), self.dtype, self.device,
                               aliases=self.model.aliases(), report=self._cast_report)
        self.model.bind(tensors)
        self.cache = CacheManager(self.model.cache_needs(), num_pages=num_pages, page_size=page_size,
                                  max_live=max_live, max_seq_len=self.max_seq_len, dtype=self.dtype,
                                  device=self.device, poison_freed_pages=poison_freed_pages)
        # debugging aids: freed pages are filled with a poison value; before a step writes a
        # request's new tokens, the pages they go to are checked to be that request's alone
        self.check_exclusive = bool(check_exclusive or poison_freed_pages)
        self.steps_run = 0
        self.program = self._program()
        # decode steps are recorded as CUDA graphs: the runs of graph-safe steps of the program
        # are recorded, the other steps are called between the replays.  (The embedding has to
        # be graph-safe: what it returns is the buffer every later step works on.)
        self.graphs = None
        if use_graphs and self.program[0][0] and any(safe for safe, _ in self.program[1:]):
            from .graphs import DecodeGraphs

            self.graphs = DecodeGraphs(self)

    def weight_cast_report(self) -> dict:
        """What reading the model folder's tensors into the engine's element types cost: elements
        by stored and by kept type, how many changed in the cast, the largest absolute and
        relative error (LockStep: engine/model/qwen3.py:205-220)."""
        return dict(self._cast_report)

    # -- requests -----------------------------------------------------------
    def open(self, uid: str) -> int:
        return self.cache.create(uid)

    def close(self, uid: str) -> None:
        self.cache.release(uid)

    def kv_len(self, uid: str) -> int:
        return self.cache.lengths[uid]

    def fill_random(self, uid: str, tokens: int, seed: int = 0) -> None:
        """Give the open request ``uid`` a context of ``tokens`` positions whose keys
        and values are random numbers, without running the model (for timing decode
        steps at a long context; the values do not change a step's work)."""
        if self.cache.lengths[uid] != 0:
            raise ValueError(f"{uid} already holds tokens")
        self.cache.reserve(uid, tokens)
        gen = torch.Generator(device=self.device).manual_seed(seed)
        for group in self.cache.paged:
            ids = torch.tensor([p for p in group.seqs[uid].pages if p >= 0], device=self.device)
            shape = (group.pages.shape[0], ids.numel(), *group.pages.shape[2:])
            group.pages[:, ids] = torch.randn(shape, generator=gen, device=self.device,
                                              dtype=torch.float32).to(group.pages.dtype)
        self.cache.advance(uid, tokens)

    # -- the step -----------------------------------------------------------
    def _program(self) -> list[tuple[bool, object]]:
        """The model as steps ``(graph_safe, fn)`` that run one after the other:
        ``fn(h, ctx)`` returns the residual stream for the next step (the embedding makes
        it, the layers' steps change it in place) and the last one returns the logits."""
        model = self.model

        def embed(h, ctx):
            return model.embedding.forward(ctx)

        def layer_step(fn, run):
            def call(h, ctx):
                fn(h, ctx, self.cache.view(run.cache, run.writes_cache))
                return h
            return call

        def finish(h, ctx):
            if ctx.n_wanted:
                return model.head.forward(model.final_norm.forward(h, ctx.wanted_rows))
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)

        program = [(bool(model.embedding.graph_safe), embed)]
        for run in self.spec.schedule:
            for safe, fn in model.blocks[run.layer].steps():
                program.append((bool(safe), layer_step(fn, run)))
        program.append((bool(model.final_norm.graph_safe and model.head.graph_safe), finish))
        return program

    @torch.no_grad()
    def forward(self, ctx) -> torch.Tensor:
        """The model on one packed batch: embedding, the scheduled layers, final norm
        and head at the wanted rows.  Launches kernels only; no host synchronisation."""
        h = None
        for _, fn in self.program:
            h = fn(h, ctx)
        return h

    @torch.no_grad()
    def can_step_ahead(self, entries: list[StepEntry]) -> bool:
        """True if ``step`` can take the token ids of these single-token entries from the
        device: the step is a recorded one."""
        if self.graphs is None or not all(len(e.tokens) == 1 and e.want == [0] for e in entries):
            return False
        return self.graphs.ready(self.graphs.key_for(entries))

    @torch.no_grad()
    def step(self, entries: list[StepEntry], check: bool = True, static_logits: bool = False,
             tokens_device: torch.Tensor | None = None) -> torch.Tensor:
        """Run one batch; returns float32 logits [wanted, vocab] in the order of
        the entries and of their ``want`` lists.  Every entry's request must be
        open and ``start`` must equal the number of tokens it already holds.
        ``check=False`` skips reading the device error word (no synchronisation);
        ``static_logits=True`` lets a replayed decode step return its graph's own
        output buffer, which the next replay overwrites.  ``tokens_device``: the token
        ids of a recorded step (``can_step_ahead``), taken on the device instead of from
        the entries."""
        if not entries:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        seen = set()
        for e in entries:
            if e.uid in seen:
                raise ValueError(f"request {e.uid!r} appears twice in one step")
            seen.add(e.uid)
            have = self.cache.lengths.get(e.uid)
            if have is None:
                raise KeyError(f"request {e.uid!r} is not open")
            if e.start != have:
                raise ValueError(f"{e.uid}: portion starts at {e.start} but the cache holds {have} tokens")
            if not e.tokens:
                raise ValueError(f"{e.uid}: an entry must bring at least one token")
            if any(not 0 <= w < len(e.tokens) for w in e.want):
                raise ValueError(f"{e.uid}: a wanted place lies outside its {len(e.tokens)} tokens")
            if e.start + len(e.tokens) > self.max_seq_len:
                raise ValueError(f"{e.uid}: {e.start + len(e.tokens)} tokens exceed max_seq_len {self.max_seq_len}")
        # every entry is valid: only now are pages taken, for all entries or for none
        wants = [(e.uid, e.start + len(e.tokens)) for e in entries]
        if not self.cache.can_reserve_all(wants):
            raise OutOfPages(f"the step needs more pages than the {self.cache.free_pages()} that are free")
        for uid, total in wants:
            self.cache.reserve(uid, total)
        if self.check_exclusive:
            for e in entries:
                self.cache.assert_exclusive(e.uid, e.start, e.start + len(e.tokens) - 1)
        self.cache.sync()
        slots = [self.cache.slots[e.uid] for e in entries]
        logits = None
        if self.graphs is not None and all(len(e.tokens) == 1 and e.want == [0] for e in entries):
            key = self.graphs.key_for(entries)
            if self.graphs.ready(key):
                logits = self.graphs.replay(key, entries, slots, tokens_device)
                if not static_logits:
                    logits = logits.clone()
            elif tokens_device is not None:
                raise ValueError("token ids on the device serve recorded steps only (see can_step_ahead)")
            else:
                # this step runs eagerly (it also warms every kernel up); later ones replay
                logits = self.forward(StepContext(entries, slots, self.device, self.err, self.split_size))
                self.graphs.record(key)
        if logits is None:
            if tokens_device is not None:
                raise ValueError("token ids on the device serve recorded steps only (see can_step_ahead)")
            mixed = self.graphs.mixed_key_for(entries) if self.graphs is not None else None
            if mixed is not None and self.graphs.mixed_ready(mixed):
                logits = self.graphs.replay_mixed(mixed, entries, slots)
                if not static_logits:
                    logits = logits.clone()
            else:
                ctx = StepContext(entries, slots, self.device, self.err, self.split_size)
                logits = self.forward(ctx)
                # a step of this shape has come often enough: later ones replay a recorded one
                if mixed is not None and self.graphs.mixed_seen_again(mixed):
                    self.graphs.record_mixed(mixed, ctx._plans.keys())
        for e in entries:
            self.cache.advance(e.uid, e.start + len(e.tokens))
        self.steps_run += 1
        if check:
            K.raise_on_fault(self.err)
        return logits
