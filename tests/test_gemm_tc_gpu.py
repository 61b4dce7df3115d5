"""The tensor-core product (tcgen05, TMA, tensor memory) alone, against float64:
token counts that fill each tile width and spill over it, widths and depths
that are no multiple of the tile, all three epilogues; and that a row's bits do
not depend on the batch it is in."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda:0")


SHAPES = [
    # tokens, out features, depth
    (1, 128, 64), (8, 256, 128), (16, 384, 1024), (17, 100, 72), (33, 500, 80), (64, 1024, 200),
    (100, 130, 136), (129, 3072, 1024), (300, 264, 328), (2048, 512, 256), (5, 1187, 40),
    # deep and narrow: K is cut into shares over a cluster (8, 6 and 5 of them)
    (8, 1024, 3072), (40, 256, 2056), (200, 1024, 2048), (3, 200, 1344), (16, 12800, 1024),
    # more than 128 tokens: one block walks the shares and keeps the running sum in registers
    (300, 256, 2048), (1000, 384, 3080), (129, 1024, 1024),
]


@pytest.mark.parametrize("t,n,k", SHAPES)
def test_tensor_core_product_and_epilogues(t, n, k):
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(t * 7 + n)
    x = torch.randn(t, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * n, k, generator=g) * 0.3).to(torch.bfloat16)
    xd, wd = x.to(dev()), w.to(dev())
    err = K.new_error_word(dev())
    want = x.double() @ w[:n].double().T
    scale = float(want.abs().max()) + 1e-6

    c = torch.empty(t, n, dtype=torch.bfloat16, device=dev())
    assert K.gemm_nt_tc(xd, wd[:n].contiguous(), c, K.EPILOGUE_STORE, err)
    K.raise_on_fault(err)
    assert (c.cpu().double() - want).abs().max() <= 1e-2 * scale

    cf = torch.empty(t, n, dtype=torch.float32, device=dev())
    assert K.gemm_nt_tc(xd, wd[:n].contiguous(), cf, K.EPILOGUE_STORE, err)
    assert (cf.cpu().double() - want).abs().max() <= 2e-5 * scale

    res = torch.randn(t, n, generator=g)
    rd = res.to(dev()).clone()
    assert K.gemm_nt_tc(xd, wd[:n].contiguous(), rd, K.EPILOGUE_RESIDUAL, err)
    assert (rd.cpu().double() - (res.double() + want)).abs().max() <= 2e-5 * scale + 1e-5

    up = x.double() @ w[n:].double().T
    want_act = want * torch.sigmoid(want) * up
    act = torch.empty(t, n, dtype=torch.bfloat16, device=dev())
    assert K.gemm_nt_tc(xd, wd, act, K.EPILOGUE_SILU_MUL, err)
    assert (act.cpu().double() - want_act).abs().max() <= 1e-2 * (float(want_act.abs().max()) + 1e-6)
    K.raise_on_fault(err)

    # the CUDA-core product of the same operands agrees to float32 rounding
    cs = torch.empty(t, n, dtype=torch.float32, device=dev())
    K.gemm_nt_simt(xd, wd[:n].contiguous(), cs)
    assert (cs - cf).abs().max().item() <= 2e-5 * scale


def test_k_shares_depend_on_the_weight_alone():
    from lockstep_b200 import kernels as K

    lib = K.library("tc")
    assert lib.ls_gemm_tc_k_shares(4096, 1024) == 4      # q, k, v of the 0.6B sizes
    assert lib.ls_gemm_tc_k_shares(1024, 2048) == 8      # o
    assert lib.ls_gemm_tc_k_shares(1024, 3072) == 8      # down
    assert lib.ls_gemm_tc_k_shares(151936, 1024) == 1    # head
    assert lib.ls_gemm_tc_k_shares(128, 64) == 1
    assert lib.ls_gemm_tc_k_shares(12288, 4096) == 1     # gate/up of the 8B sizes: 96 row tiles, one round
    assert lib.ls_gemm_tc_k_shares(2560, 4096) == 7      # o of the 4B sizes: 20 row tiles, 140 blocks
    assert lib.ls_gemm_tc_k_shares(4096, 12288) == 4     # down of the 8B sizes


@pytest.mark.parametrize("k,n", [(1024, 640), (3072, 384)])
def test_a_row_has_the_same_bits_in_every_batch(k, n):
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(5)
    x = torch.randn(300, k, generator=g).to(torch.bfloat16).to(dev())
    w = (torch.randn(n, k, generator=g) * 0.1).to(torch.bfloat16).to(dev())
    err = K.new_error_word(dev())
    full = torch.empty(300, n, dtype=torch.float32, device=dev())
    assert K.gemm_nt_tc(x, w, full, K.EPILOGUE_STORE, err)
    for lo, hi in [(0, 1), (7, 8), (5, 21), (100, 133), (0, 64), (40, 169), (299, 300)]:
        part = torch.empty(hi - lo, n, dtype=torch.float32, device=dev())
        assert K.gemm_nt_tc(x[lo:hi].contiguous(), w, part, K.EPILOGUE_STORE, err)
        assert torch.equal(part, full[lo:hi]), (lo, hi)
    K.raise_on_fault(err)


@pytest.mark.parametrize("t,n,k", [(2048, 4096, 1024), (2048, 1024, 2048), (300, 264, 328), (129, 3072, 1024),
                                   (1000, 384, 3080), (257, 130, 136), (2304, 2048, 512)])
def test_pairs_of_blocks_give_the_bits_of_single_blocks(t, n, k):
    """Tiles of 256 tokens on two blocks (cta_group::2) against tiles of 128 tokens on one, every epilogue,
    tiles of 256 and of 128 features, edges in every dimension."""
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(t + n + k)
    x = torch.randn(t, k, generator=g).to(torch.bfloat16).to(dev())
    w = (torch.randn(2 * n, k, generator=g) * 0.3).to(torch.bfloat16).to(dev())
    res = torch.randn(t, n, generator=g).to(dev())
    err = K.new_error_word(dev())
    got = {}
    try:
        for pairs in (False, True):
            K.set_gemm_tc_pairs(pairs)
            c = torch.empty(t, n, dtype=torch.bfloat16, device=dev())
            assert K.gemm_nt_tc(x, w[:n].contiguous(), c, K.EPILOGUE_STORE, err)
            cf = torch.empty(t, n, dtype=torch.float32, device=dev())
            assert K.gemm_nt_tc(x, w[:n].contiguous(), cf, K.EPILOGUE_STORE, err)
            rd = res.clone()
            assert K.gemm_nt_tc(x, w[:n].contiguous(), rd, K.EPILOGUE_RESIDUAL, err)
            act = torch.empty(t, n, dtype=torch.bfloat16, device=dev())
            assert K.gemm_nt_tc(x, w, act, K.EPILOGUE_SILU_MUL, err)
            K.raise_on_fault(err)
            got[pairs] = (c, cf, rd, act)
    finally:
        K.set_gemm_tc_pairs(True)
    for a, b in zip(got[False], got[True]):
        assert torch.equal(a, b)
    want = x.double() @ w[:n].double().T
    assert (got[True][1].double() - want).abs().max().item() <= 2e-5 * (float(want.abs().max()) + 1e-6)


def test_unaligned_depth_falls_back_to_the_cuda_cores():
    from lockstep_b200 import kernels as K

    x = torch.randn(4, 45).to(torch.bfloat16).to(dev())
    w = torch.randn(9, 45).to(torch.bfloat16).to(dev())
    c = torch.empty(4, 9, dtype=torch.float32, device=dev())
    err = K.new_error_word(dev())
    assert not K.gemm_nt_tc(x, w, c, K.EPILOGUE_STORE, err)
    K.gemm_nt(x, w, c, err=err)
    assert (c.cpu().double() - x.cpu().double() @ w.cpu().double().T).abs().max() < 1e-4


@pytest.mark.parametrize("gain_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("t,n,k", [(1, 4096, 1024), (8, 1024, 2048), (16, 384, 1024), (27, 640, 1536), (32, 256, 1024)])
def test_norm_made_inside_the_product_gives_the_same_bits(t, n, k, gain_dtype):
    """rmsnorm then product, against the product that makes the norm itself, for all epilogues."""
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(t + n)
    h = (torch.randn(t + 3, k, generator=g) * 2).to(dev())
    gain = (1 + 0.1 * torch.randn(k, generator=g)).to(gain_dtype).to(dev())
    w = (torch.randn(2 * n, k, generator=g) * 0.1).to(torch.bfloat16).to(dev())
    rows = torch.randperm(t + 3, generator=g)[:t].to(torch.int32).to(dev())
    err = K.new_error_word(dev())
    for row_index in (None, rows):
        hh = h[:t].contiguous() if row_index is None else h
        x = torch.empty(t, k, dtype=torch.bfloat16, device=dev())
        K.rmsnorm(hh, gain, x, 1e-6, err, row_index)
        for epilogue, wt, dtype in [(K.EPILOGUE_STORE, w[:n].contiguous(), torch.bfloat16),
                                    (K.EPILOGUE_STORE, w[:n].contiguous(), torch.float32),
                                    (K.EPILOGUE_RESIDUAL, w[:n].contiguous(), torch.float32),
                                    (K.EPILOGUE_SILU_MUL, w, torch.bfloat16)]:
            base = torch.randn(t, n, generator=g).to(dtype).to(dev())
            want, got = base.clone(), base.clone()
            assert K.gemm_nt_tc(x, wt, want, epilogue, err)
            assert K.gemm_nt_tc_rmsnorm(hh, gain, 1e-6, wt, got, epilogue, err, row_index), (t, n, k, epilogue)
            assert torch.equal(want, got), (epilogue, dtype, row_index is not None)
    K.raise_on_fault(err)


def test_norm_fusion_declines_where_it_does_not_apply():
    from lockstep_b200 import kernels as K

    err = K.new_error_word(dev())
    h = torch.randn(300, 1024, device=dev())
    gain = torch.ones(1024, dtype=torch.bfloat16, device=dev())
    w = torch.randn(256, 1024, device=dev()).to(torch.bfloat16)
    c = torch.empty(300, 256, dtype=torch.bfloat16, device=dev())
    assert not K.gemm_nt_tc_rmsnorm(h, gain, 1e-6, w, c, K.EPILOGUE_STORE, err)          # many tokens
    wide = torch.randn(151936 // 8, 1024, device=dev()).to(torch.bfloat16)
    c2 = torch.empty(4, wide.shape[0], dtype=torch.float32, device=dev())
    assert not K.gemm_nt_tc_rmsnorm(h[:4].contiguous(), gain, 1e-6, wide, c2, K.EPILOGUE_STORE, err)  # one share


@pytest.mark.parametrize("gain_dtype", [torch.bfloat16, torch.float32, None])
@pytest.mark.parametrize("t,nq,nkv,d,k,rot,page", [(8, 16, 8, 128, 1024, 128, 16), (1, 16, 8, 128, 1024, 128, 16),
                                                   (5, 6, 3, 64, 512, 32, 8), (32, 4, 2, 32, 1024, 32, 32),
                                                   (17, 3, 1, 128, 2056, 64, 16)])
def test_qkv_heads_finished_in_the_product_give_the_same_bits(t, nq, nkv, d, k, rot, page, gain_dtype):
    """product + qk_norm_rope_store against the product that finishes its heads, with the token
    operand given and with the RMSNorm made inside as well; the cache is written or not."""
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(t * 31 + d)
    n = (nq + 2 * nkv) * d
    h = (torch.randn(t, k, generator=g) * 2).to(dev())
    norm_gain = (1 + 0.1 * torch.randn(k, generator=g)).to(torch.bfloat16).to(dev())
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(dev())
    qg = kg = None
    if gain_dtype is not None:
        qg = (1 + 0.1 * torch.randn(d, generator=g)).to(gain_dtype).to(dev())
        kg = (1 + 0.1 * torch.randn(d, generator=g)).to(gain_dtype).to(dev())
    max_pos, num_pages = 300, 64
    ang = torch.rand(max_pos, rot // 2, generator=g) * 6.28
    cos, sin = ang.cos().to(dev()), ang.sin().to(dev())
    positions = torch.randperm(max_pos, generator=g)[:t].to(torch.int32).to(dev())     # no two tokens in one place
    token_req = torch.randint(0, 3, (t,), generator=g).to(torch.int32).to(dev())
    table = torch.stack([torch.randperm(num_pages, generator=g)[:max_pos // page + 1] for _ in range(3)]).to(torch.int32).to(dev())
    err = K.new_error_word(dev())
    x = torch.empty(t, k, dtype=torch.bfloat16, device=dev())
    K.rmsnorm(h, norm_gain, x, 1e-6, err)
    for write in (True, False):
        qkv = torch.empty(t, n, dtype=torch.bfloat16, device=dev())
        assert K.gemm_nt_tc(x, w, qkv, K.EPILOGUE_STORE, err)
        q_want = torch.zeros(t, nq * d, dtype=torch.bfloat16, device=dev())
        pages_want = torch.zeros(num_pages, 2, nkv, page, d, dtype=torch.bfloat16, device=dev())
        K.qk_norm_rope_store(qkv, q_want, pages_want, qg, kg, cos, sin, positions, token_req, table, nq, nkv, d, rot,
                             1e-5, write, err)
        for normed in (None, (h, norm_gain, 1e-6, None)):
            q_got = torch.zeros_like(q_want)
            pages_got = torch.zeros_like(pages_want)
            assert K.gemm_nt_tc_qkv_heads(None if normed else x, w, q_got, pages_got, qg, kg, cos, sin, positions,
                                          token_req, table, nq, nkv, d, rot, 1e-5, write, err, normed=normed)
            K.raise_on_fault(err)
            assert torch.equal(q_got, q_want)
            assert torch.equal(pages_got, pages_want)
            assert bool(pages_want.any()) == write


def test_qkv_heads_in_the_product_decline_what_they_do_not_cover():
    from lockstep_b200 import kernels as K

    err = K.new_error_word(dev())
    nq, nkv, d, k = 4, 2, 128, 1024
    w = torch.zeros((nq + 2 * nkv) * d, k, dtype=torch.bfloat16, device=dev())
    pages = torch.zeros(8, 2, nkv, 16, d, dtype=torch.bfloat16, device=dev())
    table = torch.zeros(1, 4, dtype=torch.int32, device=dev())
    cos = sin = torch.zeros(64, d // 2, device=dev())

    def call(t, d_=d, w_=w):
        x = torch.zeros(t, w_.shape[1], dtype=torch.bfloat16, device=dev())
        q = torch.zeros(t, nq * d_, dtype=torch.bfloat16, device=dev())
        z = torch.zeros(t, dtype=torch.int32, device=dev())
        return K.gemm_nt_tc_qkv_heads(x, w_, q, pages, None, None, cos, sin, z, z, table, nq, nkv, d_, d_, 0.0, False, err)

    assert call(8)
    assert not call(33)                      # more tokens than the few-token kernel takes
    # a weight with one share of K runs in the persistent kernel, which has no such epilogue
    shallow = torch.zeros((nq + 2 * nkv) * d, 128, dtype=torch.bfloat16, device=dev())
    assert K.library("tc").ls_gemm_tc_k_shares(shallow.shape[0], 128) == 1
    assert not call(8, w_=shallow)
