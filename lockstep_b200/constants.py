"""The table of launch constants, and its digest.

Every constant that fixes how work is cut (and with it the order of a reduction)
lives in the source that uses it; each CUDA source reports its own through
``ls_constants_<source>()``.  This module gathers them, adds the host's, and
hashes the table, so that a benchmark line or a trajectory can record which
constants it ran with (LockStep keeps such a table and its sha256 in
engine/kernels/registry.py:17-177).  None of the constants depends on a batch.
"""

from __future__ import annotations

import ctypes
import hashlib
import json

_SOURCES = {
    "core": ["attention_simt", "gemm_simt", "sampling"],
    "tc": ["gemm_tc", "attention_decode_mma", "attention_prefill_tc"],
}


def _host_constants() -> dict[str, int]:
    from . import kernels as K
    from .engine import batch, graphs

    return {
        "host.few_tokens": K.FEW_TOKENS,
        "host.attention_tile_tokens": batch.TILE_TOKENS,
        "host.graph_capacity_step": graphs.CAPACITY_STEP,
        "host.graph_cache_size": graphs.MAX_GRAPHS,
    }


def table(libraries=("core", "tc")) -> dict[str, int]:
    """name -> value, sorted by name, of the libraries named (compiled at first use)."""
    from . import kernels as K

    out = dict(_host_constants())
    for lib_name in libraries:
        lib = K.library(lib_name)
        for source in _SOURCES[lib_name]:
            fn = getattr(lib, f"ls_constants_{source}")
            fn.restype, fn.argtypes = ctypes.c_char_p, []
            for item in fn().decode("ascii").split(";"):
                name, value = item.split("=")
                out[name] = int(value)
    return dict(sorted(out.items()))


def digest(libraries=("core", "tc")) -> str:
    """sha256 of the table in canonical JSON."""
    blob = json.dumps(table(libraries), sort_keys=True, separators=(",", ":")).encode("ascii")
    return hashlib.sha256(blob).hexdigest()


def describe(libraries=("core", "tc")) -> str:
    """The table on one line: ``name=value`` joined by commas."""
    return ",".join(f"{k}={v}" for k, v in table(libraries).items())
