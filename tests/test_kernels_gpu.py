"""Each CUDA kernel alone against its plain float32/float64 reference, at sizes
other than the engine's (widths and vocabularies that are no power of two, head
sizes in steps of 16, several group sizes, page sizes 8 to 64)."""

from __future__ import annotations

import math
import random

import pytest
import torch

from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def K():
    from lockstep_b200 import kernels

    return kernels


def dev():
    return torch.device("cuda:0")


def tol(dtype):
    return 1e-5 if dtype == torch.float32 else 1.6e-2


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_gather(dtype):
    k = K()
    g = torch.Generator().manual_seed(1)
    table = torch.randn(311, 72, generator=g).to(dtype)
    ids = torch.randint(0, 311, (37,), generator=g, dtype=torch.int32)
    out = torch.empty(37, 72, dtype=torch.float32, device=dev())
    err = k.new_error_word(dev())
    k.embed_gather(ids.to(dev()), table.to(dev()), out, err)
    assert torch.equal(out.cpu(), plain.embed(table, ids.tolist()).float())
    k.raise_on_fault(err)
    bad = ids.clone()
    bad[5] = 311
    k.embed_gather(bad.to(dev()), table.to(dev()), out, err)
    with pytest.raises(k.KernelError, match="token id"):
        k.raise_on_fault(err)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [50, 1000, 4104])
def test_rmsnorm(dtype, width):
    k = K()
    g = torch.Generator().manual_seed(width)
    x = torch.randn(19, width, generator=g) * 3
    gain = (1 + 0.1 * torch.randn(width, generator=g)).to(dtype)
    err = k.new_error_word(dev())
    out = torch.empty(19, width, dtype=dtype, device=dev())
    k.rmsnorm(x.to(dev()), gain.to(dev()), out, 1e-5, err)
    want = plain.rms_norm(x.double(), gain.double(), 1e-5)
    assert (out.cpu().double() - want).abs().max() <= tol(dtype) * want.abs().max()
    rows = torch.tensor([3, 18, 0, 3], dtype=torch.int32)
    out2 = torch.empty(4, width, dtype=dtype, device=dev())
    k.rmsnorm(x.to(dev()), gain.to(dev()), out2, 1e-5, err, rows.to(dev()))
    assert torch.equal(out2.cpu(), out.cpu()[rows.long()])   # a row alone has the same bits
    k.raise_on_fault(err)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k_", [(1, 70, 45), (33, 129, 100), (130, 64, 16), (5, 500, 80), (8, 1024, 3072),
                                    (17, 300, 200), (32, 96, 64), (9, 50, 68), (40, 33, 260)])
def test_gemm_and_epilogues(dtype, m, n, k_):
    k = K()
    few_before = k.kernel_counts()["gemm_simt_few"]
    g = torch.Generator().manual_seed(m * n)
    a = torch.randn(m, k_, generator=g).to(dtype)
    w = (torch.randn(2 * n, k_, generator=g) * 0.3).to(dtype)
    ad, wd = a.to(dev()), w.to(dev())
    want = a.double() @ w[:n].double().T
    bound = tol(dtype) * float(want.abs().max()) + 1e-6
    c = torch.empty(m, n, dtype=dtype, device=dev())
    k.gemm_nt(ad, wd[:n].contiguous(), c)
    assert (c.cpu().double() - want).abs().max() <= bound
    cf = torch.empty(m, n, dtype=torch.float32, device=dev())
    k.gemm_nt(ad, wd[:n].contiguous(), cf)
    assert (cf.cpu().double() - want).abs().max() <= 1e-5 * float(want.abs().max()) + 1e-6
    res = torch.randn(m, n, generator=g)
    rd = res.to(dev()).clone()
    k.gemm_nt(ad, wd[:n].contiguous(), rd, k.EPILOGUE_RESIDUAL)
    assert (rd.cpu().double() - (res.double() + want)).abs().max() <= 1e-5 * float(want.abs().max()) + 1e-5
    up = a.double() @ w[n:].double().T
    act = torch.empty(m, n, dtype=dtype, device=dev())
    k.gemm_nt(ad, wd, act, k.EPILOGUE_SILU_MUL)
    want_act = want * torch.sigmoid(want) * up
    assert (act.cpu().double() - want_act).abs().max() <= tol(dtype) * float(want_act.abs().max()) + 1e-6
    # a row alone has the bits it has inside a larger batch
    one = torch.empty(1, n, dtype=dtype, device=dev())
    k.gemm_nt(ad[m - 1:m].contiguous(), wd[:n].contiguous(), one)
    assert torch.equal(one.cpu()[0], c.cpu()[m - 1])
    if dtype == torch.float32:
        # and among 40 rows, which the tile kernel takes whatever the depth: the few-token kernel
        # (up to 32 float32 rows of a depth that is a multiple of 4) keeps every sum's order
        many = torch.cat([ad, torch.randn(40, k_, device=dev())])
        cm = torch.empty(m + 40, n, dtype=dtype, device=dev())
        k.gemm_nt(many, wd[:n].contiguous(), cm)
        assert torch.equal(cm[:m], c)
        am = torch.empty(m + 40, n, dtype=dtype, device=dev())
        k.gemm_nt(many, wd, am, k.EPILOGUE_SILU_MUL)
        assert torch.equal(am[:m], act)
        ran = k.kernel_counts()["gemm_simt_few"] - few_before
        assert (ran > 0) == (k_ % 4 == 0), "the few-token kernel serves float32 rows of a depth in fours"


def paged_from_dense(kk, vv, page_size, num_pages, seed):
    """Scatter dense k, v [T, nkv, d] into shuffled pages; returns pages and the table row."""
    t, nkv, d = kk.shape
    need = -(-t // page_size)
    rng = random.Random(seed)
    ids = rng.sample(range(num_pages), need)
    pages = torch.full((num_pages, 2, nkv, page_size, d), float("nan"), dtype=kk.dtype)
    for pos in range(t):
        p, s = ids[pos // page_size], pos % page_size
        pages[p, 0, :, s, :] = kk[pos]
        pages[p, 1, :, s, :] = vv[pos]
    return pages, ids


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rot,page", [(6, 3, 48, 48, 8), (4, 1, 32, 16, 16), (16, 8, 128, 128, 32),
                                               (5, 1, 64, 64, 16), (3, 3, 128, 64, 8)])
def test_qk_norm_rope_store(dtype, nq, nkv, d, rot, page):
    k = K()
    g = torch.Generator().manual_seed(d)
    t = 21
    qkv = torch.randn(t, (nq + 2 * nkv) * d, generator=g).to(dtype)
    qg = (1 + 0.1 * torch.randn(d, generator=g)).to(dtype)
    kg = (1 + 0.1 * torch.randn(d, generator=g)).to(dtype)
    positions = torch.tensor([40 + i for i in range(t)], dtype=torch.int32)
    max_pos = 128
    half = rot // 2
    cos, sin = plain.rope_tables(range(max_pos), rot, 10000.0, torch.float32)
    num_pages = 16
    table = torch.full((3, 16), -1, dtype=torch.int32)
    table[2, :num_pages] = torch.tensor(random.Random(3).sample(range(num_pages), num_pages), dtype=torch.int32)
    token_req = torch.full((t,), 2, dtype=torch.int32)
    pages = torch.zeros(num_pages, 2, nkv, page, d, dtype=dtype, device=dev())
    q_out = torch.empty(t, nq * d, dtype=dtype, device=dev())
    err = k.new_error_word(dev())
    k.qk_norm_rope_store(qkv.to(dev()), q_out, pages, qg.to(dev()), kg.to(dev()), cos.to(dev()).contiguous(),
                         sin.to(dev()).contiguous(), positions.to(dev()), token_req.to(dev()),
                         table.to(dev()), nq, nkv, d, rot, 1e-6, True, err)
    k.raise_on_fault(err)
    x = qkv.double()
    q = x[:, :nq * d].view(t, nq, d)
    kk = x[:, nq * d:(nq + nkv) * d].view(t, nkv, d)
    vv = x[:, (nq + nkv) * d:].view(t, nkv, d)
    c64, s64 = cos.double()[positions.long()], sin.double()[positions.long()]

    def norm_rope(z, gain):
        z = plain.rms_norm(z, gain.double(), 1e-6)
        return torch.cat([plain.apply_rope(z[..., :rot], c64, s64), z[..., rot:]], dim=-1)

    want_q, want_k = norm_rope(q, qg), norm_rope(kk, kg)
    assert (q_out.cpu().double().view(t, nq, d) - want_q).abs().max() <= tol(dtype) * 4
    got = pages.cpu()
    for i in range(t):
        pos = int(positions[i])
        p, s = int(table[2, pos // page]), pos % page
        assert (got[p, 0, :, s, :].double() - want_k[i]).abs().max() <= tol(dtype) * 4
        assert torch.equal(got[p, 1, :, s, :], vv[i].to(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rot,page", [(6, 3, 48, 48, 8), (4, 1, 32, 16, 16), (16, 8, 128, 128, 32), (3, 3, 128, 64, 8)])
def test_qk_norm_rope_store_rotates_neighbouring_pairs(dtype, nq, nkv, d, rot, page):
    """The interleaved layout: pair i of a head is elements (2i, 2i + 1)."""
    k = K()
    g = torch.Generator().manual_seed(d + 1)
    t = 9
    qkv = torch.randn(t, (nq + 2 * nkv) * d, generator=g).to(dtype)
    qg = (1 + 0.1 * torch.randn(d, generator=g)).to(dtype)
    kg = (1 + 0.1 * torch.randn(d, generator=g)).to(dtype)
    positions = torch.tensor([3 + 5 * i for i in range(t)], dtype=torch.int32)
    cos, sin = plain.rope_tables(range(64), rot, 10000.0, torch.float32)
    table = torch.arange(8, dtype=torch.int32).flip(0).view(1, 8).contiguous()
    pages = torch.zeros(8, 2, nkv, page, d, dtype=dtype, device=dev())
    q_out = torch.empty(t, nq * d, dtype=dtype, device=dev())
    err = k.new_error_word(dev())
    k.qk_norm_rope_store(qkv.to(dev()), q_out, pages, qg.to(dev()), kg.to(dev()), cos.to(dev()).contiguous(),
                         sin.to(dev()).contiguous(), positions.to(dev()), torch.zeros(t, dtype=torch.int32, device=dev()),
                         table.to(dev()), nq, nkv, d, rot, 1e-6, True, err, interleaved=True)
    k.raise_on_fault(err)
    x = qkv.double()
    c, s_ = cos.double()[positions.long()][:, None, :], sin.double()[positions.long()][:, None, :]

    def norm_turn(z, gain):
        z = plain.rms_norm(z, gain.double(), 1e-6)
        lo, hi = z[..., 0:rot:2], z[..., 1:rot:2]
        out = z.clone()
        out[..., 0:rot:2] = lo * c - hi * s_
        out[..., 1:rot:2] = hi * c + lo * s_
        return out

    want_q = norm_turn(x[:, :nq * d].view(t, nq, d), qg)
    want_k = norm_turn(x[:, nq * d:(nq + nkv) * d].view(t, nkv, d), kg)
    assert (q_out.cpu().double().view(t, nq, d) - want_q).abs().max() <= tol(dtype) * 4
    got = pages.cpu()
    for i in range(t):
        pos = int(positions[i])
        if pos // page >= 8:
            continue
        assert (got[int(table[0, pos // page]), 0, :, pos % page, :].double() - want_k[i]).abs().max() <= tol(dtype) * 4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page", [(6, 3, 48, 8), (8, 2, 64, 16), (5, 1, 128, 32)])
def test_attention_with_a_slope_per_head_on_the_distance(dtype, nq, nkv, d, page):
    """score += slopes[head] x (key position - query position): a portion and single tokens."""
    k = K()
    g = torch.Generator().manual_seed(nq + d)
    total = 600
    q = torch.randn(total, nq, d, generator=g).to(dtype)
    kk = torch.randn(total, nkv, d, generator=g).to(dtype)
    vv = torch.randn(total, nkv, d, generator=g).to(dtype)
    slopes = torch.tensor([0.02 * (h + 1) * (-1) ** h for h in range(nq)], dtype=torch.float32)   # some favour far keys
    scale = 1 / math.sqrt(d)
    pos = torch.arange(total, dtype=torch.float64)
    distance = pos[None, :] - pos[:, None]
    want = torch.empty(total, nq, d, dtype=torch.float64)
    for h in range(nq):
        sc = q[:, h].double() @ kk[:, h // (nq // nkv)].double().T * scale + slopes[h].double() * distance
        sc = sc.masked_fill(distance > 0, float("-inf"))
        want[:, h] = torch.softmax(sc, dim=-1) @ vv[:, h // (nq // nkv)].double()
    want = want.float()
    pages, ids = paged_from_dense(kk, vv, page, 128, seed=6)
    bound = 2e-5 if dtype == torch.float32 else 2e-2
    got = run_attention(k, q[450:], pages, ids, 450, 0, scale, False, slopes=slopes)
    assert (got - want[450:]).abs().max() <= bound
    for p in [0, 1, 255, 256, 511, 512, 599]:
        for decode_kernel in (False, True):
            got = run_attention(k, q[p:p + 1], pages, ids, p, 0, scale, decode_kernel, slopes=slopes)
            assert (got[0] - want[p]).abs().max() <= bound, (p, decode_kernel)
    assert (want[599] - plain.causal_attention(q.double(), kk.double(), vv.double(), scale).float()[599]).abs().max() > 0.05


def run_attention(k, q, pages, table_row, start, window, scale, decode_kernel, slopes=None):
    """q [n, nq, d] at positions start..; returns out [n, nq, d] (float32, cpu)."""
    from lockstep_b200.engine.batch import plan_attention

    n, nq, d = q.shape
    nkv = pages.shape[2]
    split = k.attention_split_size()
    table = torch.full((2, 256), -1, dtype=torch.int32)
    table[1, :len(table_row)] = torch.tensor(table_row, dtype=torch.int32)
    prefill_tc = decode_kernel == "prefill_tc"
    tile_tokens = 128 if prefill_tc else 16
    tile, sp, comb, n_slots = plan_attention([(1, 0, start, n)], window, split, tile_tokens)
    D = dev()
    err = k.new_error_word(D)
    slopes = None if slopes is None else slopes.to(D)
    qd, pd, td = q.reshape(n, nq * d).contiguous().to(D), pages.to(D), table.to(D)
    out = torch.empty(n, nq * d, dtype=q.dtype, device=D)
    if len(tile) and prefill_tc:
        assert k.attention_prefill_tc(qd, pd, out, torch.from_numpy(tile).to(D), len(tile), td, nq, nkv, d,
                                      window, scale, err)
    elif len(tile):
        k.attention_tile(qd, pd, out, None, None, torch.from_numpy(tile).to(D), len(tile), td, nq, nkv, d,
                         window, scale, err, slopes)
    if len(sp):
        acc = torch.empty(n_slots, nq, d, dtype=torch.float32, device=D)
        ml = torch.empty(n_slots, nq, 2, dtype=torch.float32, device=D)
        w = torch.from_numpy(sp).to(D)
        done = False
        if decode_kernel == "mma":
            done = k.attention_decode_mma(qd, pd, acc, ml, w, len(sp), td, nq, nkv, d, window, scale, err)
            assert done
        elif decode_kernel and not prefill_tc:
            done = k.attention_decode(qd, pd, acc, ml, w, len(sp), td, nq, nkv, d, window, scale, err, slopes)
            assert done
        if not done:
            k.attention_tile(qd, pd, None, acc, ml, w, len(sp), td, nq, nkv, d, window, scale, err, slopes)
        k.attention_combine(acc, ml, out, torch.from_numpy(comb).to(D), len(comb), nq, d)
    k.raise_on_fault(err)
    return out.cpu().float().view(n, nq, d)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page", [(4, 2, 16, 16), (6, 3, 48, 8), (8, 1, 64, 32), (16, 8, 128, 16), (2, 2, 256, 64),
                                           (12, 1, 128, 8), (16, 1, 64, 64), (5, 5, 128, 32)])
@pytest.mark.parametrize("window", [0, 100])
def test_attention_prefix_portion_and_decode(dtype, nq, nkv, d, page, window):
    """A portion (tile kernel, serial splits) and a single token (split kernels
    and combine) over a paged cache of 700 keys, against plain attention."""
    k = K()
    g = torch.Generator().manual_seed(nq * d + window)
    total = 700
    q = torch.randn(total, nq, d, generator=g).to(dtype)
    kk = torch.randn(total, nkv, d, generator=g).to(dtype)
    vv = torch.randn(total, nkv, d, generator=g).to(dtype)
    scale = 1 / math.sqrt(d)
    want = plain.causal_attention(q.double(), kk.double(), vv.double(), scale, window=window).float()
    pages, ids = paged_from_dense(kk, vv, page, 128, seed=5)
    bound = 2e-5 if dtype == torch.float32 else 2e-2
    # the last 150 tokens as one portion (crosses the split edge at 512 and ends off a tile edge)
    got = run_attention(k, q[550:], pages, ids, 550, window, scale, False)
    assert (got - want[550:]).abs().max() <= bound
    if dtype == torch.bfloat16 and d in (64, 128):
        # the tensor-core kernel: a whole prompt, a ragged tail, two tokens at a tile's edge
        # (tcgen05, 128-token tiles)
        for kernel in ("prefill_tc",):
            for lo, hi in [(0, 700), (550, 700), (0, 1), (63, 65), (640, 642), (100, 229), (127, 130), (0, 129)]:
                got = run_attention(k, q[lo:hi], pages, ids, lo, window, scale, kernel)
                assert (got - want[lo:hi]).abs().max() <= bound, (kernel, lo, hi)
                if (nq // nkv) % 2 == 0:
                    # two heads of a key head in a block: another kernel, the same sums, the same bits
                    k.set_attention_prefill_pairs(2)
                    try:
                        paired = run_attention(k, q[lo:hi], pages, ids, lo, window, scale, kernel)
                    finally:
                        k.set_attention_prefill_pairs(1)
                    assert torch.equal(paired, got), (kernel, lo, hi)
    # single tokens at telling places: first, page edges, split edges, last
    for pos in [0, 1, page - 1, page, 255, 256, 257, 511, 512, 699]:
        sub_pages, sub_ids = pages, ids
        for decode_kernel in (False, True, "mma"):
            if decode_kernel and (nq // nkv) * d > 1024:
                continue
            if decode_kernel == "mma" and (dtype != torch.bfloat16 or d not in (64, 128)):
                continue
            got = run_attention(k, q[pos:pos + 1], sub_pages, sub_ids, pos, window, scale, decode_kernel)
            assert (got[0] - want[pos]).abs().max() <= bound, (pos, decode_kernel)
    # in float32 a decoded row has the bits of the same row inside a portion
    if dtype == torch.float32:
        whole = run_attention(k, q[500:700], pages, ids, 500, window, scale, False)
        one = run_attention(k, q[640:641], pages, ids, 640, window, scale, False)
        assert torch.equal(one[0], whole[140])


@pytest.mark.parametrize("nq,nkv,d,page,n,window", [(16, 8, 128, 16, 8192, 0), (8, 2, 64, 8, 5000, 0),
                                                     (32, 8, 128, 32, 4096, 1000), (4, 1, 128, 16, 12000, 0)])
def test_the_two_prompt_attention_kernels_agree_bit_for_bit_on_long_prompts(nq, nkv, d, page, n, window):
    """One head a block against the two heads of a key head a block, on prompts long enough that a
    launch would take the second by itself, five runs each: the same bits every time (the second
    kernel writes P over the scores it came from and relies on the order of the MMAs; a race
    would show as a run that differs)."""
    from lockstep_b200.engine.batch import plan_attention

    k = K()
    g = torch.Generator(device=dev()).manual_seed(n)
    q = torch.randn(n, nq * d, generator=g, device=dev()).bfloat16()
    num_pages = -(-n // page)
    pages = torch.randn(num_pages, 2, nkv, page, d, generator=g, device=dev()).bfloat16()
    table = torch.randperm(num_pages, generator=g, device=dev()).to(torch.int32).view(1, -1).contiguous()
    tile, _, _, _ = plan_attention([(0, 0, 0, n)], window, k.attention_split_size(), 128)
    work = torch.from_numpy(tile).to(dev())
    err = k.new_error_word(dev())
    outs = {0: [], 2: []}
    try:
        for mode in (0, 2):
            k.set_attention_prefill_pairs(mode)
            for _ in range(1 if mode == 0 else 5):
                out = torch.full_like(q, float("nan"))
                assert k.attention_prefill_tc(q, pages, out, work, len(tile), table, nq, nkv, d, window,
                                              1 / math.sqrt(d), err)
                outs[mode].append(out)
    finally:
        k.set_attention_prefill_pairs(1)
    k.raise_on_fault(err)
    assert bool(torch.isfinite(outs[0][0].float()).all())
    for out in outs[2]:
        assert torch.equal(out, outs[0][0])
    # spot rows against plain attention
    qf = q.double().cpu().view(n, nq, d)
    for r in (0, 127, 128, n // 2 + 3, n - 1):
        keys = torch.arange(max(0, r - window + 1) if window else 0, r + 1)
        want = torch.empty(nq, d, dtype=torch.float64)
        for h in range(nq):
            kv = h // (nq // nkv)
            pg, off = table[0, (keys // page).to(dev())].cpu().long(), keys % page
            kk = pages[pg, 0, kv, off].double().cpu()
            vv = pages[pg, 1, kv, off].double().cpu()
            want[h] = torch.softmax(kk @ qf[r, h] / math.sqrt(d), 0) @ vv
        assert (outs[0][0][r].double().cpu().view(nq, d) - want).abs().max() <= 2e-2, r


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [32, 128])
def test_attention_finds_one_far_key(dtype, d):
    """One key among hundreds is made to stand out for the last query; the output
    must be that key's value.  A fault in a far page, split or tile shows here."""
    k = K()
    nq, nkv, page = 4, 2, 16
    g = torch.Generator().manual_seed(9)
    total = 600
    for far in [0, 15, 16, 255, 256, 300, 511, 512, 598]:
        q = torch.randn(total, nq, d, generator=g) * 0.1
        kk = torch.randn(total, nkv, d, generator=g) * 0.1
        vv = torch.randn(total, nkv, d, generator=g)
        direction = torch.randn(d, generator=g)
        direction = direction / direction.norm()
        q[-1] = direction * 30.0
        kk[far] = direction * 30.0
        q, kk, vv = q.to(dtype), kk.to(dtype), vv.to(dtype)
        pages, ids = paged_from_dense(kk, vv, page, 64, seed=far)
        kinds = (False, True, "mma") if (dtype == torch.bfloat16 and d == 128) else (False, True)
        for decode_kernel in kinds:
            got = run_attention(k, q[-1:], pages, ids, total - 1, 0, 1.0, decode_kernel)
            for h in range(nq):
                assert (got[0, h] - vv[far, h // 2].float()).abs().max() <= 2e-2, (far, decode_kernel)


@pytest.mark.parametrize("d", [64, 128])
def test_prefill_attention_follows_rising_maxima(d):
    """Scores that grow from key tile to key tile: by less than the tensor-core kernel's lazy threshold (its
    reference maximum stays behind and P exceeds 1), by more (the row of O in tensor memory is scaled), and
    far more (the scaled part all but vanishes).  Every row sees a different prefix of the steps."""
    k = K()
    nq, nkv, page, total = 4, 2, 16, 640
    g = torch.Generator().manual_seed(d)
    direction = torch.randn(d, generator=g)
    direction = direction / direction.norm()
    # score of key j for every query: level[j] (natural units, scale 1) plus a little noise
    level = torch.zeros(total)
    level[128:256] = 3.0        # + 4.3 in powers of two: no move
    level[256:384] = 10.0       # + 10: a move
    level[384:512] = 11.0       # + 1.4: none
    level[512:] = 40.0          # + 42: what was there before counts for nothing
    q = (torch.randn(total, nq, d, generator=g) * 0.05 + direction * 2.0).to(torch.bfloat16)
    kk = (torch.randn(total, nkv, d, generator=g) * 0.05 + direction * (level / 2.0).view(-1, 1, 1)).to(torch.bfloat16)
    vv = torch.randn(total, nkv, d, generator=g).to(torch.bfloat16)
    want = plain.causal_attention(q.double(), kk.double(), vv.double(), 1.0, window=0).float()
    pages, ids = paged_from_dense(kk, vv, page, 64, seed=1)
    for lo, hi in [(0, 640), (200, 640), (500, 530)]:
        got = run_attention(k, q[lo:hi], pages, ids, lo, 0, 1.0, "prefill_tc")
        assert (got - want[lo:hi]).abs().max() <= 2e-2, (lo, hi)


def test_argmax_ties_go_to_lowest_id():
    k = K()
    logits = torch.full((3, 1001), -1.0)
    logits[0, [7, 500, 900]] = 2.5
    logits[1, 1000] = 9.0
    logits[2, :] = 0.25
    out = torch.empty(3, dtype=torch.int32, device=dev())
    k.argmax(logits.to(dev()), out)
    assert out.tolist() == [7, 1000, 0]


def test_sampling_matches_plain_on_clear_cases_and_in_distribution():
    k = K()
    from lockstep_b200.sampling import philox

    vocab = 777
    g = torch.Generator().manual_seed(4)
    rows = 64
    logits = torch.randn(rows, vocab, generator=g) * 3
    temperature = torch.tensor([0.7 if i % 2 else 1.3 for i in range(rows)])
    temperature[0] = 0.0
    top_p = torch.tensor([1.0 if i % 3 else 0.8 for i in range(rows)])
    uids = [f"req{i}" for i in range(rows)]
    positions = [17 + 3 * i for i in range(rows)]
    seed = 1234
    keys = torch.tensor([philox.key_words(seed, u) for u in uids], dtype=torch.int64)
    pos = torch.tensor([[p & 0xFFFFFFFF, p >> 32] for p in positions], dtype=torch.int64)
    as_i32 = lambda t: t.to(torch.int64).where(t < 2 ** 31, t - 2 ** 32).to(torch.int32)
    out = torch.empty(rows, dtype=torch.int32, device=dev())
    probs = torch.empty(rows, vocab, dtype=torch.float32, device=dev())
    k.sample(logits.to(dev()), probs, temperature.to(dev()), top_p.to(dev()), as_i32(keys).to(dev()),
             as_i32(pos).to(dev()), out)
    got = out.tolist()
    agree = 0
    for i in range(rows):
        want = plain.sample_top_p(logits[i], seed, uids[i], positions[i], p=float(top_p[i]),
                                  temperature=float(temperature[i]))
        agree += int(want == got[i])
    # float32 sums on the device against float64 on the host: a draw that falls
    # within rounding of a boundary may pick the neighbour
    assert got[0] == int(logits[0].argmax())
    assert agree >= rows - 2, f"only {agree} of {rows} draws agree with the plain sampler"


def test_sampling_over_a_wide_vocabulary_with_ties():
    """151,936 tokens (a row spread over the blocks of a cluster, probabilities in registers)
    against the plain sampler; rows with many equal logits, where the rank among the ties
    decides; a greedy row; a row whose mass sits on one token."""
    k = K()
    from lockstep_b200.sampling import philox

    vocab = 151936
    g = torch.Generator().manual_seed(9)
    rows = 24
    logits = torch.randn(rows, vocab, generator=g) * 4
    logits[1] = torch.randint(0, 6, (vocab,), generator=g).float()          # six values: ties everywhere
    logits[2] = 0.0                                                          # all equal: the draw picks an id
    logits[3, 77777] = 60.0                                                  # one token has all the mass
    temperature = torch.tensor([0.9 if i % 2 else 1.2 for i in range(rows)])
    temperature[0] = 0.0
    top_p = torch.tensor([1.0 if i % 3 else 0.7 for i in range(rows)])
    top_p[1], top_p[2] = 0.5, 1.0
    uids = [f"wide{i}" for i in range(rows)]
    positions = [5 + 11 * i for i in range(rows)]
    seed = 77
    keys = torch.tensor([philox.key_words(seed, u) for u in uids], dtype=torch.int64)
    pos = torch.tensor([[p & 0xFFFFFFFF, p >> 32] for p in positions], dtype=torch.int64)
    as_i32 = lambda t: t.to(torch.int64).where(t < 2 ** 31, t - 2 ** 32).to(torch.int32)
    out = torch.full((rows,), -7, dtype=torch.int32, device=dev())
    probs = torch.empty(rows, vocab, dtype=torch.float32, device=dev())
    k.sample(logits.to(dev()), probs, temperature.to(dev()), top_p.to(dev()), as_i32(keys).to(dev()),
             as_i32(pos).to(dev()), out)
    got = out.tolist()
    assert all(0 <= t < vocab for t in got)
    assert got[0] == int(logits[0].argmax()) and got[3] == 77777
    agree, near = 0, 0
    for i in range(rows):
        want = plain.sample_top_p(logits[i], seed, uids[i], positions[i], p=float(top_p[i]),
                                  temperature=float(temperature[i]))
        agree += int(want == got[i])
        # a draw within float32 rounding of a boundary may land on a neighbour in the ranking:
        # a token of the same or the next probability
        near += int(want == got[i] or abs(float(logits[i, want]) - float(logits[i, got[i]])) < 1e-3)
    assert near == rows, f"{rows - near} draws are far from the plain sampler's"
    assert agree >= rows - 4, f"only {agree} of {rows} draws agree with the plain sampler"
    # the same call twice gives the same tokens
    again = torch.empty_like(out)
    k.sample(logits.to(dev()), probs, temperature.to(dev()), top_p.to(dev()), as_i32(keys).to(dev()),
             as_i32(pos).to(dev()), again)
    assert torch.equal(out, again)
