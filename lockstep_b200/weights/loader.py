"""Reads a model folder's tensors by name.

The tensors a model needs (name, shape, role) come from its parts.  The file's
names are compared with them before anything is copied to the device, and one
``WeightError`` lists every missing tensor, every unexpected one and every wrong
shape.  Element types: with the bfloat16 engine, matrices and tables are kept
in bfloat16 (a float32 file is rounded once, here); a norm gain that the file
stores in float32 stays float32; integer tensors become int32.  With the
float32 engine everything floating is float32 (an exact widening of bfloat16).

A tied head (``tie_word_embeddings``) takes the embedding table; if the file
also stores the head it must equal the table, as LockStep requires
(engine/model/qwen3.py:159-174).

What the rounding to the engine's element type cost is measured while loading
(``report``; LockStep: engine/model/qwen3.py:176-220): how many elements are not
exactly representable, and the largest absolute and relative error.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping

import torch

from ..parts.base import WeightSpec


class WeightError(ValueError):
    """The model folder's tensors do not match what the model needs."""


def _open_files(folder: Path):
    from safetensors import safe_open

    index = folder / "model.safetensors.index.json"
    single = folder / "model.safetensors"
    if index.is_file():
        weight_map = json.loads(index.read_text())["weight_map"]
        files = sorted(set(weight_map.values()))
    elif single.is_file():
        files = [single.name]
    else:
        raise WeightError(f"{folder} holds neither model.safetensors nor model.safetensors.index.json")
    handles = {}
    where: dict[str, str] = {}
    for f in files:
        path = folder / f
        if not path.is_file():
            raise WeightError(f"{path} is named by the index but does not exist")
        h = safe_open(str(path), framework="pt", device="cpu")
        handles[f] = h
        for name in h.keys():
            where[name] = f
    return handles, where


def engine_dtype_for(role: str, stored: torch.dtype, engine_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if engine_dtype == torch.float32:
        return torch.float32
    if role == "gain" and stored == torch.float32:
        return torch.float32
    return engine_dtype


_REPORT_CHUNK = 1 << 24      # elements compared at a time


def _cast_error(exact: torch.Tensor, cast: torch.Tensor) -> tuple[int, float, float]:
    """(elements that changed, largest absolute error, largest relative error) of a cast."""
    inexact, max_abs, max_rel = 0, 0.0, 0.0
    tiny = torch.finfo(torch.float32).tiny
    a, b = exact.reshape(-1), cast.reshape(-1)
    for start in range(0, a.numel(), _REPORT_CHUNK):
        x = a[start:start + _REPORT_CHUNK].to(torch.float32)
        diff = (x - b[start:start + _REPORT_CHUNK].to(torch.float32)).abs()
        inexact += int((diff > 0).sum())
        max_abs = max(max_abs, float(diff.max()))
        max_rel = max(max_rel, float((diff / x.abs().clamp_min(tiny)).max()))
    return inexact, max_abs, max_rel


def load_weights(folder, expected: Mapping[str, WeightSpec], engine_dtype: torch.dtype, device,
                 aliases: Mapping[str, str] | None = None, report: dict | None = None) -> dict[str, torch.Tensor]:
    """``aliases``: name -> name of an expected tensor it must equal if the file
    stores it (the tied head); such names are not "unexpected".  ``report``: a dict
    that receives what the cast to the engine's element types cost."""
    folder = Path(folder)
    handles, where = _open_files(folder)
    aliases = dict(aliases or {})

    missing = sorted(n for n in expected if n not in where)
    unexpected = sorted(n for n in where if n not in expected and n not in aliases)
    wrong = []
    for name, spec in expected.items():
        if name in where:
            shape = tuple(handles[where[name]].get_slice(name).get_shape())
            if shape != tuple(spec.shape):
                wrong.append(f"{name}: file has {list(shape)}, model needs {list(spec.shape)}")
    if missing or unexpected or wrong:
        parts = [f"{folder}: the tensors do not match the model"]
        if missing:
            parts.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            parts.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            parts.append(f"  wrong shape ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("\n".join(parts))

    for alias, target in aliases.items():
        if alias in where:
            a = handles[where[alias]].get_tensor(alias)
            b = handles[where[target]].get_tensor(target)
            if a.shape != b.shape or not torch.equal(a, b):
                raise WeightError(
                    f"{folder}: the configuration ties {alias} to {target}, but the file stores "
                    "both and they differ")

    out: dict[str, torch.Tensor] = {}
    stored: dict[str, int] = {}
    kept: dict[str, int] = {}
    elements = inexact = 0
    max_abs = max_rel = 0.0
    for name, spec in expected.items():
        t = handles[where[name]].get_tensor(name)
        dt = engine_dtype_for(spec.role, t.dtype, engine_dtype)
        if report is None:
            out[name] = t.to(dt).to(device).contiguous()
            continue
        t = t.to(device)                     # compared where the copy lives: a pass over every weight
        out[name] = t.to(dt).contiguous()
        stored[str(t.dtype)] = stored.get(str(t.dtype), 0) + t.numel()
        kept[str(dt)] = kept.get(str(dt), 0) + t.numel()
        elements += t.numel()
        if t.dtype.is_floating_point and dt != t.dtype:
            n, a, r = _cast_error(t, out[name])
            inexact, max_abs, max_rel = inexact + n, max(max_abs, a), max(max_rel, r)
    if report is not None:
        dropped = [a for a in aliases if a in where]
        report.update({
            "engine_dtype": str(engine_dtype), "stored_elements_by_dtype": stored, "kept_elements_by_dtype": kept,
            "distinct_elements": elements,
            "tied_names_dropped": dropped,
            "duplicate_elements_dropped": sum(int(torch.tensor(handles[where[a]].get_slice(a).get_shape()).prod())
                                              for a in dropped),
            "elements_not_exactly_representable": inexact, "max_abs_error": max_abs, "max_rel_error": max_rel,
        })
    return out
