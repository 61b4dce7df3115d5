"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it
drives ``ModelRunner.step``, the step function that generation uses.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input holds one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose
logits are wanted.  ``end``: requests that are finished after this step; their
pages are given back.  For a step in which something is wanted the logits are
written to ``<out>/<step>.f32`` as little-endian float32 [wanted, vocab], in
the order of the entries and of ``want``.  After every step a line
``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder the logits are written to")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to 64)")
    p.add_argument("--page-size", type=int, default=16, help="tokens per cache page (default 16)")
    p.add_argument("--max-live", type=int, default=16, help="most requests live at a time")
    p.add_argument("--device", default="cuda:0")
    return p


def run(args, lines) -> int:
    import numpy as np

    from .batch import StepEntry
    from .runner import ModelRunner

    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    max_tokens = max(64, -(-int(args.max_tokens) // 64) * 64)
    runner = ModelRunner(args.model, dtype=args.dtype, device=args.device,
                         num_pages=-(-max_tokens // args.page_size), page_size=args.page_size,
                         max_live=args.max_live, max_seq_len=max_tokens)
    live: set[str] = set()
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            uid = str(e["id"])
            if uid not in live:
                runner.open(uid)
                live.add(uid)
            entries.append(StepEntry(uid=uid, tokens=[int(t) for t in e["tokens"]],
                                     start=runner.kv_len(uid), want=[int(w) for w in e.get("want", [])]))
        logits = runner.step(entries)
        if logits.shape[0]:
            logits.cpu().numpy().astype("<f4").tofile(str(out / f"{step}.f32"))
        for uid in rec.get("end", []):
            uid = str(uid)
            if uid in live:
                runner.close(uid)
                live.discard(uid)
        print(f"done {step}", flush=True)
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return run(args, sys.stdin)


if __name__ == "__main__":
    raise SystemExit(main())
