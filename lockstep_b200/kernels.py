"""Python faces of the CUDA kernels in ``csrc/``.

Each function checks what it is given (device, element type, contiguity,
shapes), launches on torch's current stream and raises ``KernelError`` when the
launcher refuses the arguments or the launch fails.  There is no CPU path: a
tensor that is not on a CUDA device is an error, and so is a missing or
unbuildable extension.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

EPILOGUE_STORE, EPILOGUE_RESIDUAL, EPILOGUE_SILU_MUL = 0, 1, 2
FEW_TOKENS = 32      # up to here a product runs in the few-token kernel, which can also finish q/k/v heads

_REFUSALS = {
    -1: "unsupported element type combination",
    -2: "a size this kernel does not take",
    -3: "a pointer or stride that is not aligned as required",
    -4: "needs more shared memory than the device offers",
}

DEVICE_FAULTS = {
    1: "token id outside the embedding table (token index {d})",
    2: "block table names a page outside the pool (at {d})",
    3: "position outside the rotary table (token index {d})",
    4: "a bounded wait inside a kernel ran out (code {d})",
    5: "row index outside its tensor (row {d})",
}


class KernelError(RuntimeError):
    """A launcher refused its arguments, a launch failed, or a kernel recorded a fault."""


_SIGNATURES = {
    "core": {
        "ls_embed_gather": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
        "ls_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                       c_float, c_void_p, c_void_p],
        "ls_qk_norm_rope_store": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                  c_void_p, c_void_p],
        "ls_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "ls_gemm_nt_simt": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                            c_int64, c_int64, c_int64, c_int, c_void_p],
        "ls_attention_split_size": [],
        "ls_attention_tile": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                              c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_float, c_void_p, c_void_p, c_void_p],
        "ls_attention_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                c_void_p, c_void_p, c_void_p],
        "ls_attention_combine": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                 c_void_p],
        "ls_argmax": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "ls_sample": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                      c_int, c_void_p],
    },
}

_SIGNATURES["tc"] = {
    "ls_gemm_tc_token_tile": [c_int, c_int, c_int, c_int],
    "ls_gemm_tc_k_shares": [c_int, c_int],
    "ls_attention_decode_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "ls_attention_prefill_tc_tile_tokens": [],
    "ls_attention_prefill_tc": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "ls_gemm_nt_tc_qkv_heads": [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int, c_float, c_void_p,
                                c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "ls_gemm_nt_tc_rmsnorm": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int,
                              c_int, c_int, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p],
    "ls_gemm_nt_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                      c_int, c_void_p, c_void_p],
}

_libs: dict[str, ctypes.CDLL] = {}


def library(name: str = "core") -> ctypes.CDLL:
    """The loaded extension library `name` (compiled at first use)."""
    lib = _libs.get(name)
    if lib is None:
        lib = _build.load(name)
        for fn, argtypes in _SIGNATURES.get(name, {}).items():
            f = getattr(lib, fn)
            f.argtypes = argtypes
            f.restype = c_int
        _libs[name] = lib
    return lib


def set_gemm_tc_pairs(on: bool) -> None:
    """Whether tensor-core products of more than 128 tokens run on pairs of blocks that share
    a tile of 256 tokens (tcgen05 cta_group::2; the default) or on single blocks with tiles of
    128 tokens.  The sums are the same either way."""
    fn = library("tc").ls_set_gemm_tc_pairs
    fn.argtypes, fn.restype = [c_int], None
    fn(1 if on else 0)


def set_attention_prefill_pairs(mode: int) -> None:
    """How the tensor-core attention of prompt portions takes the heads of a key head: 0 one
    head a block; 1 (the default) two heads a block, sharing the key and value tiles, where the
    group size is even and the items fill the device twice over; 2 wherever the group is even."""
    fn = library("tc").ls_set_attention_prefill_pairs
    fn.argtypes, fn.restype = [c_int], None
    fn(int(mode))


def set_dependent_launch(on: bool) -> None:
    """Programmatic dependent launch of all kernels (on by default): a kernel is
    scheduled while its predecessor drains and waits for it before it touches memory."""
    for name in ("core", "tc"):
        fn = getattr(library(name), f"ls_set_dependent_launch_{name}")
        fn.argtypes, fn.restype = [c_int], None
        fn(1 if on else 0)


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError(
            "lockstep_b200 runs on a CUDA device only (sm_100a); there is no CPU fallback")


def _stream() -> int:
    """The current stream's handle (also while a graph is being captured).  Asked of torch's
    C layer directly: ``torch.cuda.current_stream()`` builds a Python object on every call,
    which was a third of the host's share of a step."""
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not supported (float32 or bfloat16)") from None


def _dev(t: torch.Tensor, name: str, dtype=None) -> int:
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device; there is no CPU fallback")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _opt(t, name, dtype=None) -> int:
    return 0 if t is None else _dev(t, name, dtype)


# bfloat16 work goes to the tensor cores unless this is cleared (a debugging aid)
USE_TENSOR_CORES = [True]

# kernel launches since the counter was last cleared: launcher calls (each is at
# least one kernel) plus, for a replayed graph, the calls that were recorded in it
LAUNCHES = [0]


def kernel_counts() -> dict[str, int]:
    """How often each kernel's launcher has launched in this process (a launch recorded into
    a graph counts once, its replays do not), over the libraries that are loaded."""
    out: dict[str, int] = {}
    library("core")
    for name, lib in list(_libs.items()):
        names_fn = getattr(lib, f"ls_kernel_names_{name}")
        names_fn.restype, names_fn.argtypes = ctypes.c_char_p, []
        names = names_fn().decode("ascii").split(",")
        counts = (ctypes.c_ulonglong * len(names))()
        fn = getattr(lib, f"ls_kernel_launches_{name}")
        fn.restype, fn.argtypes = c_int, [ctypes.POINTER(ctypes.c_ulonglong), c_int]
        fn(counts, len(names))
        for kernel, count in zip(names, counts):
            out[kernel] = out.get(kernel, 0) + int(count)
    return out


def _check(status: int, what: str) -> None:
    if status == 0:
        LAUNCHES[0] += 1
        return
    if status < 0:
        raise KernelError(f"{what}: {_REFUSALS.get(status, f'refused with code {status}')}")
    raise KernelError(f"{what}: CUDA launch failed with error {status}")


def new_error_word(device) -> torch.Tensor:
    """Two int32 on the device: the first fault a kernel recorded and its detail."""
    return torch.zeros(2, dtype=torch.int32, device=device)


def raise_on_fault(err: torch.Tensor) -> None:
    """Read the error word (synchronises) and raise if a kernel recorded a fault."""
    code, detail = err.tolist()
    if code != 0:
        err.zero_()
        raise KernelError("device fault: " + DEVICE_FAULTS.get(code, "code {d}").format(d=detail))


# ---------------------------------------------------------------------------

def attention_split_size() -> int:
    return int(library().ls_attention_split_size())


def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: torch.Tensor) -> None:
    tokens, width = out.shape
    if ids.numel() != tokens or table.shape[1] != width:
        raise KernelError("embed_gather: shapes do not agree")
    _check(library().ls_embed_gather(
        _dev(ids, "ids", torch.int32), _dev(table, "table"), _code(table),
        _dev(out, "out", torch.float32), tokens, width, table.shape[0], _dev(err, "err", torch.int32),
        _stream()), "embed_gather")


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, out: torch.Tensor, eps: float, err: torch.Tensor,
            row_index: torch.Tensor | None = None) -> None:
    rows, width = out.shape
    if x.shape[1] != width or gain.numel() != width:
        raise KernelError("rmsnorm: shapes do not agree")
    if row_index is None and x.shape[0] != rows:
        raise KernelError("rmsnorm: row counts do not agree")
    if row_index is not None and row_index.numel() != rows:
        raise KernelError("rmsnorm: row_index does not match the output rows")
    _check(library().ls_rmsnorm(
        _dev(x, "x", torch.float32), _opt(row_index, "row_index", torch.int32), _dev(gain, "gain"),
        _code(gain), _dev(out, "out"), _code(out), rows, width, x.shape[0], float(eps),
        _dev(err, "err", torch.int32), _stream()), "rmsnorm")


def qk_norm_rope_store(qkv, q_out, pages, q_gain, k_gain, cos, sin, positions, token_req,
                       block_table, nq: int, nkv: int, d: int, rot_dim: int, eps: float,
                       write_cache: bool, err, interleaved: bool = False) -> None:
    """pages: [num_pages, 2, nkv, page_size, d] of one cache layer (may be None if not written).
    ``interleaved``: a rotated pair is elements (2i, 2i + 1) of the head instead of
    (i, i + rot_dim / 2)."""
    tokens = qkv.shape[0]
    if qkv.shape[1] != (nq + 2 * nkv) * d or q_out.shape != (tokens, nq * d):
        raise KernelError("qk_norm_rope_store: shapes do not agree")
    if (q_gain is None) != (k_gain is None):
        raise KernelError("qk_norm_rope_store: q and k gains come together")
    if write_cache:
        if pages.dtype != qkv.dtype or pages.shape[1:3] != (2, nkv) or pages.shape[4] != d:
            raise KernelError("qk_norm_rope_store: cache pages do not match the projections")
        num_pages, page_size = pages.shape[0], pages.shape[3]
    else:
        num_pages, page_size = 0, 1
    half = rot_dim // 2
    if rot_dim:
        if cos.shape != sin.shape or cos.shape[1] != half:
            raise KernelError("qk_norm_rope_store: rotary tables do not match rot_dim")
    gain_code = _code(q_gain) if q_gain is not None else F32
    if q_gain is not None and (q_gain.dtype != k_gain.dtype or q_gain.numel() != d or k_gain.numel() != d):
        raise KernelError("qk_norm_rope_store: gains do not match the head size")
    _check(library().ls_qk_norm_rope_store(
        _dev(qkv, "qkv"), _dev(q_out, "q_out", qkv.dtype), _opt(pages if write_cache else None, "pages"),
        _code(qkv), _opt(q_gain, "q_gain"), _opt(k_gain, "k_gain"), gain_code,
        _opt(cos if rot_dim else None, "cos", torch.float32),
        _opt(sin if rot_dim else None, "sin", torch.float32),
        _dev(positions, "positions", torch.int32), _dev(token_req, "token_req", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[-1], tokens, nq, nkv, d,
        rot_dim, page_size, num_pages, cos.shape[0] if rot_dim else 0, float(eps),
        1 if write_cache else 0, 1 if interleaved else 0, _dev(err, "err", torch.int32), _stream()),
        "qk_norm_rope_store")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    rows, width = out.shape
    if gate_up.shape != (rows, 2 * width) or gate_up.dtype != out.dtype:
        raise KernelError("silu_mul: shapes do not agree")
    _check(library().ls_silu_mul(_dev(gate_up, "gate_up"), _dev(out, "out"), _code(out), rows, width,
                                 _stream()), "silu_mul")


def gemm_nt_simt(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPILOGUE_STORE) -> None:
    """c = a @ w.T on the CUDA cores with the chosen epilogue (see csrc/gemm_simt.cu)."""
    m, k = a.shape
    n = c.shape[1]
    rows_w = 2 * n if epilogue == EPILOGUE_SILU_MUL else n
    if w.shape != (rows_w, k) or c.shape[0] != m or a.dtype != w.dtype:
        raise KernelError(f"gemm_nt: shapes do not agree: a {tuple(a.shape)} w {tuple(w.shape)} c {tuple(c.shape)}")
    _check(library().ls_gemm_nt_simt(
        _dev(a, "a"), _dev(w, "w"), _dev(c, "c"), _code(a), _code(c), m, n, k, k, k, n, epilogue,
        _stream()), "gemm_nt_simt")


def _slopes(slopes, nq: int) -> int:
    if slopes is not None and slopes.numel() != nq:
        raise KernelError(f"a score bias needs one slope per query head: {slopes.numel()} for {nq} heads")
    return _opt(slopes, "slopes", torch.float32)


def attention_tile(q, pages, out, part_acc, part_ml, work, n_work, block_table, nq, nkv, d,
                   window, scale, err, slopes=None) -> None:
    """``slopes`` (float32 [nq] or None): slopes[head] x (key position - query position) is added
    to every score."""
    _check(library().ls_attention_tile(
        _dev(q, "q"), _dev(pages, "pages", q.dtype), _opt(out, "out", q.dtype),
        _opt(part_acc, "part_acc", torch.float32), _opt(part_ml, "part_ml", torch.float32), _code(q),
        _dev(work, "work", torch.int32), n_work, _dev(block_table, "block_table", torch.int32),
        block_table.shape[-1], nq, nkv, d, pages.shape[3], pages.shape[0], int(window), float(scale),
        _slopes(slopes, nq), _dev(err, "err", torch.int32), _stream()), "attention_tile")


def attention_decode(q, pages, part_acc, part_ml, work, n_work, block_table, nq, nkv, d, window,
                     scale, err, slopes=None) -> bool:
    """Returns False (and launches nothing) for shapes the decode kernel does not take."""
    status = library().ls_attention_decode(
        _dev(q, "q"), _dev(pages, "pages", q.dtype), _dev(part_acc, "part_acc", torch.float32),
        _dev(part_ml, "part_ml", torch.float32), _code(q), _dev(work, "work", torch.int32), n_work,
        _dev(block_table, "block_table", torch.int32), block_table.shape[-1], nq, nkv, d,
        pages.shape[3], pages.shape[0], int(window), float(scale), _slopes(slopes, nq),
        _dev(err, "err", torch.int32), _stream())
    if status == -2:
        return False
    _check(status, "attention_decode")
    return True


def attention_decode_mma(q, pages, part_acc, part_ml, work, n_work, block_table, nq, nkv, d, window,
                         scale, err) -> bool:
    """Decode attention on mma.sync with TMA-fed pages (csrc/attention_decode_mma.cu): bfloat16,
    head size 64 or 128, groups up to 16.  Returns False (nothing launched) otherwise."""
    if q.dtype != torch.bfloat16 or not USE_TENSOR_CORES[0]:
        return False
    status = library("tc").ls_attention_decode_mma(
        _dev(q, "q"), _dev(pages, "pages", q.dtype), _dev(part_acc, "part_acc", torch.float32),
        _dev(part_ml, "part_ml", torch.float32), _dev(work, "work", torch.int32), n_work,
        _dev(block_table, "block_table", torch.int32), block_table.shape[-1], nq, nkv, d,
        pages.shape[3], pages.shape[0], int(window), float(scale), _dev(err, "err", torch.int32),
        _stream())
    if status == -2:
        return False
    _check(status, "attention_decode_mma")
    return True


def attention_prefill_tc_tile_tokens() -> int:
    return int(library("tc").ls_attention_prefill_tc_tile_tokens())


def attention_prefill_tc(q, pages, out, work, n_work, block_table, nq, nkv, d, window, scale, err) -> bool:
    """Attention of prompt portions on tcgen05 (csrc/attention_prefill_tc.cu): bfloat16, head
    size 64 or 128, work items of up to 128 tokens.  Returns False (nothing launched) for
    anything else."""
    if q.dtype != torch.bfloat16 or not USE_TENSOR_CORES[0]:
        return False
    status = library("tc").ls_attention_prefill_tc(
        _dev(q, "q"), _dev(pages, "pages", q.dtype), _dev(out, "out", q.dtype), q.shape[0],
        _dev(work, "work", torch.int32), n_work, _dev(block_table, "block_table", torch.int32),
        block_table.shape[-1], nq, nkv, d, pages.shape[3], pages.shape[0], int(window), float(scale),
        _dev(err, "err", torch.int32), _stream())
    if status in (-2, -3):
        return False
    _check(status, "attention_prefill_tc")
    return True


def attention_combine(part_acc, part_ml, out, items, n_items, nq, d) -> None:
    _check(library().ls_attention_combine(
        _dev(part_acc, "part_acc", torch.float32), _dev(part_ml, "part_ml", torch.float32),
        _dev(out, "out"), _code(out), _dev(items, "items", torch.int32), n_items, nq, d, _stream()),
        "attention_combine")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    rows, vocab = logits.shape
    scratch = torch.empty(rows * 128, dtype=torch.int32, device=logits.device)
    _check(library().ls_argmax(_dev(logits, "logits", torch.float32), _dev(out, "out", torch.int32),
                               _dev(scratch, "scratch"), rows, vocab, _stream()), "argmax")


def sample_scratch_floats(rows: int, vocab: int) -> int:
    """Floats of scratch ``sample`` needs for ``rows`` rows of ``vocab`` logits (0: none)."""
    fn = library().ls_sample_scratch_floats
    fn.argtypes, fn.restype = [c_int, c_int], ctypes.c_longlong
    return int(fn(rows, vocab))


def sample(logits, probs, temperature, top_p, keys, positions, out) -> None:
    """keys, positions: [rows, 2] int32 holding the low and high 32 bits.  ``probs``: float32
    scratch of ``sample_scratch_floats(rows, vocab)`` elements, or None where that is 0."""
    rows, vocab = logits.shape
    if probs is not None and probs.numel() < rows * vocab:
        raise KernelError("sample: probs scratch does not match the logits")
    if probs is None and sample_scratch_floats(rows, vocab):
        raise KernelError("sample: this vocabulary needs a scratch for the probabilities")
    _check(library().ls_sample(
        _dev(logits, "logits", torch.float32), _opt(probs, "probs", torch.float32),
        _dev(temperature, "temperature", torch.float32), _dev(top_p, "top_p", torch.float32),
        _dev(keys, "keys", torch.int32), _dev(positions, "positions", torch.int32),
        _dev(out, "out", torch.int32), rows, vocab, _stream()), "sample")



def gemm_nt_tc(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int, err: torch.Tensor) -> bool:
    """c = a @ w.T on the tcgen05 tensor cores (csrc/gemm_tc.cu).  Returns False,
    having launched nothing, when TMA cannot address the operands (a row pitch
    that is no multiple of 16 bytes): the caller then uses the CUDA-core product."""
    m, k = a.shape
    n = c.shape[1]
    rows_w = 2 * n if epilogue == EPILOGUE_SILU_MUL else n
    if w.shape != (rows_w, k) or c.shape[0] != m or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_nt_tc: shapes or types do not agree: a {tuple(a.shape)} w {tuple(w.shape)} c {tuple(c.shape)}")
    status = library("tc").ls_gemm_nt_tc(
        _dev(a, "a"), _dev(w, "w"), _dev(c, "c"), _code(c), m, n, k, k, k, n, epilogue,
        _dev(err, "err", torch.int32), _stream())
    if status == -3:
        return False
    _check(status, "gemm_nt_tc")
    return True


def gemm_nt_tc_rmsnorm(h: torch.Tensor, gain: torch.Tensor, eps: float, w: torch.Tensor, c: torch.Tensor,
                       epilogue: int, err: torch.Tensor, row_index: torch.Tensor | None = None) -> bool:
    """c = rmsnorm(h)[rows] @ w.T with the norm made inside the product's kernel, bit for bit
    what ``rmsnorm`` followed by ``gemm_nt_tc`` gives.  h [rows, k] float32, w bfloat16.
    Returns False, having launched nothing, where the fused form does not apply (many
    tokens, a weight whose depth is not shared out, unaligned rows)."""
    if not USE_TENSOR_CORES[0] or w.dtype != torch.bfloat16:
        return False
    k = h.shape[1]
    m, n = c.shape
    rows_w = 2 * n if epilogue == EPILOGUE_SILU_MUL else n
    if w.shape != (rows_w, k) or gain.numel() != k:
        raise KernelError("gemm_nt_tc_rmsnorm: shapes do not agree")
    if row_index is None and h.shape[0] != m:
        raise KernelError("gemm_nt_tc_rmsnorm: row counts do not agree")
    status = library("tc").ls_gemm_nt_tc_rmsnorm(
        _dev(h, "h", torch.float32), _opt(row_index, "row_index", torch.int32), h.shape[0],
        _dev(gain, "gain"), _code(gain), float(eps), _dev(w, "w"), _dev(c, "c"), _code(c), m, n, k, k, n,
        epilogue, _dev(err, "err", torch.int32), _stream())
    if status in (-2, -3):
        return False
    _check(status, "gemm_nt_tc_rmsnorm")
    return True


def gemm_nt_tc_qkv_heads(x, w, q_out, pages, q_gain, k_gain, cos, sin, positions, token_req, block_table,
                         nq: int, nkv: int, d: int, rot_dim: int, head_eps: float, write_cache: bool, err,
                         normed=None) -> bool:
    """The q/k/v projection of few tokens with the work of ``qk_norm_rope_store`` done in the
    product's epilogue (same bits, one kernel).  ``x`` [tokens, k] bfloat16, or None with
    ``normed`` = (h float32 [rows, k], gain, eps, row_index or None) to make the RMSNorm of the
    rows inside the product as well.  Returns False, having launched nothing, where the fused
    form does not apply; the caller then runs the product and ``qk_norm_rope_store``."""
    if not USE_TENSOR_CORES[0] or w.dtype != torch.bfloat16 or q_out.dtype != torch.bfloat16:
        return False
    tokens = q_out.shape[0]
    k = w.shape[1]
    if w.shape[0] != (nq + 2 * nkv) * d or q_out.shape != (tokens, nq * d):
        raise KernelError("gemm_nt_tc_qkv_heads: shapes do not agree")
    if (q_gain is None) != (k_gain is None):
        raise KernelError("gemm_nt_tc_qkv_heads: q and k gains come together")
    if q_gain is not None and (q_gain.dtype != k_gain.dtype or q_gain.numel() != d or k_gain.numel() != d):
        raise KernelError("gemm_nt_tc_qkv_heads: gains do not match the head size")
    if write_cache:
        if pages.dtype != torch.bfloat16 or pages.shape[1:3] != (2, nkv) or pages.shape[4] != d:
            raise KernelError("gemm_nt_tc_qkv_heads: cache pages do not match the projections")
        num_pages, page_size = pages.shape[0], pages.shape[3]
    else:
        num_pages, page_size = 0, 1
    if rot_dim and (cos.shape != sin.shape or cos.shape[1] != rot_dim // 2):
        raise KernelError("gemm_nt_tc_qkv_heads: rotary tables do not match rot_dim")
    if normed is None:
        if x.dtype != torch.bfloat16 or x.shape != (tokens, k):
            raise KernelError("gemm_nt_tc_qkv_heads: the token operand does not match")
        xp, ldx, hp, rows_p, src_rows, gain_p, gain_code, eps = _dev(x, "x"), k, None, None, 0, None, F32, 0.0
    else:
        h, gain, eps, row_index = normed
        if h.shape[1] != k or gain.numel() != k or (row_index is None and h.shape[0] != tokens):
            raise KernelError("gemm_nt_tc_qkv_heads: the rows to norm do not match")
        xp, ldx, hp, rows_p = None, 0, _dev(h, "h", torch.float32), _opt(row_index, "row_index", torch.int32)
        src_rows, gain_p, gain_code = h.shape[0], _dev(gain, "gain"), _code(gain)
    status = library("tc").ls_gemm_nt_tc_qkv_heads(
        xp, ldx, hp, rows_p, src_rows, gain_p, gain_code, float(eps), _dev(w, "w"), k, tokens, k,
        _dev(q_out, "q_out"), _opt(pages if write_cache else None, "pages"), _opt(q_gain, "q_gain"),
        _opt(k_gain, "k_gain"), _code(q_gain) if q_gain is not None else F32,
        _opt(cos if rot_dim else None, "cos", torch.float32), _opt(sin if rot_dim else None, "sin", torch.float32),
        _dev(positions, "positions", torch.int32), _dev(token_req, "token_req", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[-1], nq, nkv, d, rot_dim, page_size,
        num_pages, cos.shape[0] if rot_dim else 0, float(head_eps), 1 if write_cache else 0,
        _dev(err, "err", torch.int32), _stream())
    if status in (-2, -3):
        return False
    _check(status, "gemm_nt_tc_qkv_heads")
    return True


_tc_err: dict = {}


def gemm_nt(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPILOGUE_STORE,
            err: torch.Tensor | None = None) -> None:
    """c = a @ w.T with float32 accumulation and the chosen epilogue.

    a [m, k] and w [n, k] (or [2n, k] for the silu-mul epilogue) share an element
    type; c is [m, n] in that type, or float32 (always for the residual epilogue,
    where the product is added into c in place).  bfloat16 operands go to the
    tensor cores, float32 operands to the CUDA cores (true 32-bit)."""
    if a.dtype == torch.bfloat16 and USE_TENSOR_CORES[0]:
        if err is None:
            err = _tc_err.get(a.device)
            if err is None:
                err = _tc_err[a.device] = new_error_word(a.device)
        if gemm_nt_tc(a, w, c, epilogue, err):
            return
    gemm_nt_simt(a, w, c, epilogue)
