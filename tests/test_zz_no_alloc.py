"""The decode-attention entry point that allocates nothing, against the ordinary one.

``ls_attention_decode_noalloc`` serves hosts that cannot call cudaMalloc where
the step function would (all device memory already given to a pool of their
own, or a loop that cannot take cudaMalloc's device-wide synchronisation).  It
keeps the split partials in a fixed 8 MiB array inside the library.  Here it
is called through its exported C symbol, twice in a row with different inputs
(the array keeps the first call's contents), and compared with
``ls_attention_decode`` + ``ls_attention_combine`` on caller-allocated scratch:
the same kernels do the same arithmetic, so the bits must be equal, and both
must agree with plain softmax attention computed in float64.  The second call
uses fewer slots than the first and much larger values, so stale partials of the
first call would show.  A call that needs more than the array holds must be
refused, one that needs exactly what it holds must run, and a work item that
names a slot outside the call's slots must be reported and skipped.

This file is collected last, so that a run that stops at the first failure has
already run every other test.
"""

from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

NOALLOC_TOO_LARGE = -10
SCRATCH_FLOATS = 2 * 1024 * 1024


def _entry():
    from lockstep_b200 import kernels as K

    fn = K.library("core").ls_attention_decode_noalloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                   c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                   c_void_p]
    return fn


def _case(seed, dtype, batch, nq, nkv, d, page, lengths, window=0, value_scale=1.0):
    """Random queries and a random paged cache for `batch` single-token rows."""
    from lockstep_b200 import kernels as K
    from lockstep_b200.engine.batch import plan_attention

    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(seed)
    max_pages = max(-(-n // page) for n in lengths)
    num_pages = batch * max_pages
    pages = torch.randn((num_pages, 2, nkv, page, d), generator=g, device=dev)
    pages[:, 1] *= value_scale
    pages = pages.to(dtype)
    perm = torch.randperm(num_pages, generator=g, device=dev).to(torch.int32)
    table = perm.view(batch, max_pages).contiguous()
    q = torch.randn((batch, nq * d), generator=g, device=dev).to(dtype)
    portions = [(i, i, lengths[i] - 1, 1) for i in range(batch)]
    _, split, combine, n_slots = plan_attention(portions, window, K.attention_split_size())
    return dict(q=q, pages=pages, table=table, work=torch.from_numpy(split).to(dev),
                combine=torch.from_numpy(combine).to(dev), n_slots=n_slots, nq=nq, nkv=nkv, d=d,
                page=page, num_pages=num_pages, scale=1 / math.sqrt(d), window=window, lengths=lengths)


def _plain(c):
    """Softmax attention of every row over its own keys, in float64, straight from the pages."""
    nq, nkv, d, page = c["nq"], c["nkv"], c["d"], c["page"]
    out = torch.empty((len(c["lengths"]), nq * d), dtype=torch.float64)
    pages, table, q = c["pages"].double().cpu(), c["table"].cpu(), c["q"].double().cpu()
    for i, n in enumerate(c["lengths"]):
        ids = table[i, : -(-n // page)].long()
        k = pages[ids, 0].permute(1, 0, 2, 3).reshape(nkv, -1, d)[:, :n]      # [nkv, n, d]
        v = pages[ids, 1].permute(1, 0, 2, 3).reshape(nkv, -1, d)[:, :n]
        lo = max(0, n - c["window"]) if c["window"] else 0
        for h in range(nq):
            kv = h // (nq // nkv)
            s = (k[kv, lo:] @ q[i, h * d:(h + 1) * d]) * c["scale"]
            out[i, h * d:(h + 1) * d] = torch.softmax(s, dim=0) @ v[kv, lo:]
    return out


def _with_caller_scratch(c):
    from lockstep_b200 import kernels as K

    dev = c["q"].device
    err = K.new_error_word(dev)
    acc = torch.empty((c["n_slots"], c["nq"], c["d"]), dtype=torch.float32, device=dev)
    ml = torch.empty((c["n_slots"], c["nq"], 2), dtype=torch.float32, device=dev)
    out = torch.empty_like(c["q"])
    assert K.attention_decode(c["q"], c["pages"], acc, ml, c["work"], len(c["work"]), c["table"],
                              c["nq"], c["nkv"], c["d"], c["window"], c["scale"], err)
    K.attention_combine(acc, ml, out, c["combine"], len(c["combine"]), c["nq"], c["d"])
    K.raise_on_fault(err)
    return out


def _without_allocating(fn, c):
    from lockstep_b200 import kernels as K

    dev = c["q"].device
    err = K.new_error_word(dev)
    out = torch.empty_like(c["q"])           # the caller's output; the entry point allocates nothing
    status = fn(c["q"].data_ptr(), c["pages"].data_ptr(), out.data_ptr(),
                0 if c["q"].dtype == torch.float32 else 1, c["work"].data_ptr(), len(c["work"]),
                c["combine"].data_ptr(), len(c["combine"]), c["n_slots"], c["table"].data_ptr(),
                c["table"].shape[1], c["nq"], c["nkv"], c["d"], c["page"], c["num_pages"], c["window"],
                c["scale"], err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return status, out, err


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_calls_in_a_row_match_the_ordinary_entry_point(dtype):
    from lockstep_b200 import kernels as K

    fn = _entry()
    first = _case(1, dtype, batch=5, nq=8, nkv=2, d=64, page=16, lengths=[700, 1, 256, 257, 90])
    # fewer slots than the first call, values a hundred times larger, and a window
    second = _case(2, dtype, batch=3, nq=8, nkv=2, d=64, page=16, lengths=[300, 513, 40], window=70,
                   value_scale=100.0)
    assert second["n_slots"] < first["n_slots"]
    for case in (first, second):
        want = _with_caller_scratch(case)
        status, got, err = _without_allocating(fn, case)
        assert status == 0
        K.raise_on_fault(err)
        assert torch.equal(got, want), "the same kernels on another scratch must give the same bits"
        plain = _plain(case)
        bound = (2e-5 if dtype == torch.float32 else 1.6e-2) * float(plain.abs().max())
        assert (got.double().cpu() - plain).abs().max().item() <= bound


def test_a_call_beyond_the_scratch_is_refused_and_the_largest_that_fits_runs():
    from lockstep_b200 import kernels as K

    fn = _entry()
    case = _case(3, torch.bfloat16, batch=2, nq=8, nkv=2, d=64, page=16, lengths=[20, 30])
    want = _with_caller_scratch(case)
    per_slot = 8 * (64 + 2)
    # (a head size is a multiple of 16, so no call needs exactly the 2^21 floats of the array)
    case["n_slots"] = SCRATCH_FLOATS // per_slot + 1
    status, _, _ = _without_allocating(fn, case)
    assert status == NOALLOC_TOO_LARGE
    case["n_slots"] = SCRATCH_FLOATS // per_slot            # the most slots that fit: the call runs
    status, got, err = _without_allocating(fn, case)
    assert status == 0
    K.raise_on_fault(err)
    assert torch.equal(got, want)


def test_a_work_item_outside_the_calls_slots_is_reported_not_written():
    """The caller says how many slots its work items use; the items live on the device, so the
    kernels check them: an item that names a slot beyond that number is recorded in the error
    word and skipped instead of writing past the call's part of the array."""
    from lockstep_b200 import kernels as K

    fn = _entry()
    case = _case(7, torch.float32, batch=3, nq=4, nkv=2, d=32, page=16, lengths=[300, 20, 600])
    assert case["n_slots"] == 6
    case["n_slots"] = 4                                       # the last request's items name slots 3..5
    status, _, err = _without_allocating(fn, case)
    assert status == 0
    with pytest.raises(K.KernelError, match="row index outside"):
        K.raise_on_fault(err)
