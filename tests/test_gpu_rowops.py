"""GPU parity of the row ops (RMSNorm, RoPE, SiLU*mul, add, argmax, embedding) through the C-ABI, against the CPU
oracle and, where built, the reference's CUDA ops."""
import ctypes as C

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _torch():
    import torch
    return torch


def _ulp_diff(a, b):
    """distance in fp16 representable steps (monotone integer mapping of the bit patterns)"""
    def key(x):
        u = x.view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7fff), u)
    return np.abs(key(a) - key(b))


@pytest.mark.parametrize("x_fp32,y_fp32", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("dim", [128, 1024, 5120, 17408])
def test_rms_norm(ctx, ref, dim, x_fp32, y_fp32):
    from oracle import oracle as O
    torch = _torch()
    r = H.rng(dim)
    rows = 9
    x = r.standard_normal((rows, dim)).astype(np.float32 if x_fp32 else np.float16)
    w = (1 + 0.1 * r.standard_normal(dim)).astype(np.float16)
    dx, dw = H.to_dev(x), H.to_dev(w)
    y = torch.empty(rows, dim, dtype=torch.float32 if y_fp32 else torch.float16, device="cuda")
    ctx.rms_norm(dx, dw, y, 1e-6, 0.0, 1.0)
    want = O.rms_norm(x, w, 1e-6, out_dtype=np.float32 if y_fp32 else np.float16)
    got = y.cpu().numpy()
    if y_fp32:
        assert np.allclose(got, want, rtol=2e-5, atol=1e-6)
    else:
        assert _ulp_diff(got, want).max() <= 1
    if ref is not None:
        y2 = torch.empty_like(y)
        assert ref.ref_rms_norm(H.ptr(dx), int(x_fp32), H.ptr(dw), H.ptr(y2), int(y_fp32), C.c_float(1e-6),
                                C.c_float(0.0), C.c_float(1.0), rows, dim) == 0
        torch.cuda.synchronize()
        if y_fp32:
            assert torch.allclose(y, y2, rtol=2e-5, atol=1e-6)
        else:
            assert _ulp_diff(got, y2.cpu().numpy()).max() <= 1


@pytest.mark.parametrize("x_fp32", [False, True])
def test_rms_norm_res_in(ctx, ref, x_fp32):
    from oracle import oracle as O
    torch = _torch()
    r = H.rng(5)
    rows, dim = 7, 5120
    x = r.standard_normal((rows, dim)).astype(np.float32 if x_fp32 else np.float16)
    res = r.standard_normal((rows, dim)).astype(np.float32)
    w = (1 + 0.1 * r.standard_normal(dim)).astype(np.float16)
    dx, dw, dres = H.to_dev(x), H.to_dev(w), H.to_dev(res)
    y = torch.empty(rows, dim, dtype=torch.float16, device="cuda")
    ctx.rms_norm_res_in(dx, dw, y, dres, 1e-6)
    res_want = res.copy()
    want = O.rms_norm(x, w, 1e-6, res=res_want)
    assert np.array_equal(dres.cpu().numpy(), res_want)          # r += x is a single fp32 add: exact
    assert _ulp_diff(y.cpu().numpy(), want).max() <= 1
    if ref is not None:
        dres2, y2 = H.to_dev(res), torch.empty_like(y)
        assert ref.ref_rms_norm_res_in(H.ptr(dx), int(x_fp32), H.ptr(dw), H.ptr(y2), 0, H.ptr(dres2), 1, C.c_float(1e-6),
                                       C.c_float(0.0), C.c_float(1.0), rows, dim) == 0
        torch.cuda.synchronize()
        assert torch.equal(dres, dres2)
        assert _ulp_diff(y.cpu().numpy(), y2.cpu().numpy()).max() <= 1


@pytest.mark.parametrize("with_norm", [False, True])
@pytest.mark.parametrize("mode", [2, 1])
def test_rope(ctx, ref, mode, with_norm):
    from oracle import oracle as O
    torch = _torch()
    r = H.rng(21 + mode)
    bsz, seq, nq, nk, hd = 3, 5, 16, 8, 128
    q = r.standard_normal((bsz, seq, nq, hd)).astype(np.float16)
    k = r.standard_normal((bsz, seq, nk, hd)).astype(np.float16)
    inv_freq = (1.0 / (10000.0 ** (np.arange(0, hd, 2) / hd))).astype(np.float32)
    positions = np.array([0, 17, 900], np.int32)
    qn = (1 + 0.1 * r.standard_normal(hd)).astype(np.float16) if with_norm else None
    kn = (1 + 0.1 * r.standard_normal(hd)).astype(np.float16) if with_norm else None
    dq, dk = H.to_dev(q), H.to_dev(k)
    dif, dpos = H.to_dev(inv_freq), H.to_dev(positions)
    dqn = None if qn is None else H.to_dev(qn)
    dkn = None if kn is None else H.to_dev(kn)
    ctx.rope(dq, dk, dif, 0, dpos, dqn, dkn, 1e-6, 0.0, mode, 1.0)
    wq, wk = O.rope(q, k, inv_freq, 0, positions, qn, kn, 1e-6, 0.0, mode, 1.0)
    # __sinf/__cosf on the device versus libm here: absolute error grows with the angle (positions up to ~900 rad)
    assert np.abs(dq.cpu().numpy().astype(np.float32) - wq.astype(np.float32)).max() < 2e-2
    assert np.abs(dk.cpu().numpy().astype(np.float32) - wk.astype(np.float32)).max() < 2e-2
    if ref is not None:
        dq2, dk2 = H.to_dev(q), H.to_dev(k)
        assert ref.ref_rope(H.ptr(dq2), H.ptr(dk2), H.ptr(dif), inv_freq.size, 0, H.ptr(dpos), H.ptr(dqn), H.ptr(dkn),
                            C.c_float(1e-6), C.c_float(0.0), mode, C.c_float(1.0), bsz, seq, nq, nk, hd) == 0
        torch.cuda.synchronize()
        assert _ulp_diff(dq.cpu().numpy(), dq2.cpu().numpy()).max() <= 1
        assert _ulp_diff(dk.cpu().numpy(), dk2.cpu().numpy()).max() <= 1


def test_rope_ragged_rows_match_rectangular(ctx):
    torch = _torch()
    r = H.rng(31)
    bsz, seq, nq, nk, hd = 4, 3, 8, 2, 128
    q = r.standard_normal((bsz, seq, nq, hd)).astype(np.float16)
    k = r.standard_normal((bsz, seq, nk, hd)).astype(np.float16)
    inv_freq = (1.0 / (10000.0 ** (np.arange(0, hd, 2) / hd))).astype(np.float32)
    positions = np.array([3, 40, 0, 1000], np.int32)
    dq, dk, dq2, dk2 = H.to_dev(q), H.to_dev(k), H.to_dev(q), H.to_dev(k)
    ctx.rope(dq, dk, H.to_dev(inv_freq), 0, H.to_dev(positions))
    row_pos = (positions[:, None] + np.arange(seq)[None, :]).astype(np.int32).reshape(-1)
    ctx.rope(dq2.view(1, bsz * seq, nq, hd), dk2.view(1, bsz * seq, nk, hd), H.to_dev(inv_freq), 0, None,
             row_pos=H.to_dev(row_pos))
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2)


def test_silu_mul_and_add(ctx, ref):
    from oracle import oracle as O
    torch = _torch()
    r = H.rng(41)
    x = (3 * r.standard_normal((6, 3072))).astype(np.float16)
    y = r.standard_normal((6, 3072)).astype(np.float16)
    dx, dy = H.to_dev(x), H.to_dev(y)
    z = torch.empty_like(dx)
    ctx.silu_mul(dx, dy, z)
    want = O.silu_mul(x, y)
    got = z.cpu().numpy()
    # fp16 exp/rcp on the device are hardware approximations; the oracle uses correctly rounded ones
    assert np.abs(got.astype(np.float32) - want.astype(np.float32)).max() <= 4e-3 * max(1.0, np.abs(want).max())
    if ref is not None:
        z2 = torch.empty_like(z)
        assert ref.ref_silu_mul(H.ptr(dx), H.ptr(dy), H.ptr(z2), C.c_int64(6), C.c_int64(3072)) == 0
        torch.cuda.synchronize()
        assert torch.equal(z, z2)
    s = torch.empty_like(dx)
    ctx.add(dx, dy, s)
    assert np.array_equal(s.cpu().numpy().view(np.uint16), O.add(x, y).view(np.uint16))


@pytest.mark.parametrize("fp32", [False, True])
def test_argmax(ctx, ref, fp32):
    from oracle import oracle as O
    torch = _torch()
    r = H.rng(51)
    rows, n = 5, 151936
    lg = r.standard_normal((rows, n)).astype(np.float32 if fp32 else np.float16)
    lg[1, 777] = lg[1, 99999] = 50.0          # tie: lowest index wins
    lg[2, :] = -3.0                            # all equal: index 0
    d = H.to_dev(lg)
    ids = torch.empty(rows, dtype=torch.int64, device="cuda")
    ctx.argmax_sample(d, ids)
    got = ids.cpu().numpy()
    assert np.array_equal(got, O.argmax(lg))
    assert got[1] == 777 and got[2] == 0
    if ref is not None and not fp32:
        ids2 = torch.empty(rows, 1, dtype=torch.int64, device="cuda")
        assert ref.ref_argmax_sample(H.ptr(d), H.ptr(ids2), rows, n, 0) == 0
        torch.cuda.synchronize()
        assert np.array_equal(got, ids2.cpu().numpy().reshape(-1))


def test_embed(ctx):
    from oracle import oracle as O
    torch = _torch()
    r = H.rng(61)
    table = r.standard_normal((1000, 1024)).astype(np.float16)
    ids = r.integers(0, 1000, 33).astype(np.int64)
    out = torch.empty(33, 1024, dtype=torch.float32, device="cuda")
    ctx.embed(H.to_dev(ids), H.to_dev(table), out)
    assert np.array_equal(out.cpu().numpy(), O.embed(ids, table))
