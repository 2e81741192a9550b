"""The element-wise ops and the Linear::forward policy layer that complete the reference's op surface on the decode path:
soft-cap, GELU and ReLU^2 gates, and a linear layer with input padding, bias, output trim and soft-cap."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _close_fp16(got, want, steps):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    allowed = H.fp16_ulp(want) * (steps + 0.001)
    return float((np.abs(got - want) / allowed).max())


@pytest.mark.parametrize("limit", [0.0, 1.5])
@pytest.mark.parametrize("act", ["gelu", "relu2"])
def test_gated_activations(ctx, ref, act, limit):
    import torch
    from oracle import oracle as O
    r = H.rng(11)
    x = (r.standard_normal(3 * 4096) * 2).astype(np.float16)
    y = (r.standard_normal(3 * 4096) * 2).astype(np.float16)
    dx, dy = H.to_dev(x), H.to_dev(y)
    dz = torch.empty_like(dx)
    getattr(ctx, act + "_mul")(dx, dy, dz, act_limit=limit)
    got = dz.cpu().numpy().astype(np.float64)
    want = getattr(O, act + "_mul")(x, y, limit).astype(np.float64)
    # against exact arithmetic: one fp16 step on the activation and one on the product; the GELU of the reference takes its
    # tanh from the hardware approximation (kernels/compat.cuh:22-27, relative error 2^-11), which moves the activation by
    # up to |x| / 2 * 2^-10.6 before the product
    yc = np.clip(y.astype(np.float64), -limit, limit) if limit else y.astype(np.float64)
    allowed = 2.001 * H.fp16_ulp(want) + H.fp16_ulp(want / np.where(yc == 0, 1, yc)) * np.abs(yc)
    if act == "gelu":
        allowed = allowed + 0.5 * np.abs(x.astype(np.float64)) * 2.0 ** -10.5 * np.abs(yc)
    assert (np.abs(got - want) <= allowed).all(), float((np.abs(got - want) / allowed).max())
    if ref is not None and hasattr(ref, "ref_act_mul"):
        import ctypes as C
        dz2 = torch.empty_like(dx)
        assert ref.ref_act_mul(0 if act == "gelu" else 1, H.ptr(dx), H.ptr(dy), H.ptr(dz2), C.c_float(limit), C.c_int64(3),
                               C.c_int64(4096)) == 0
        torch.cuda.synchronize()
        assert torch.equal(dz, dz2), "the same operations in the same order as the reference kernel: equal bits"


@pytest.mark.parametrize("fp32", [False, True])
def test_softcap(ctx, ref, fp32):
    import torch
    from oracle import oracle as O
    r = H.rng(12)
    x = (r.standard_normal(2 * 5000) * 40).astype(np.float32 if fp32 else np.float16)
    dx = H.to_dev(x)
    dy = torch.empty_like(dx)
    ctx.softcap(dx, dy, 30.0)
    want = O.softcap(x, 30.0)
    if fp32:
        assert np.abs(dy.cpu().numpy() - want).max() <= 1e-5 * 30
    else:
        assert _close_fp16(dy.cpu().numpy(), want, 1) <= 1.0
    if ref is not None and hasattr(ref, "ref_softcap"):
        import ctypes as C
        dy2 = torch.empty_like(dx)
        assert ref.ref_softcap(H.ptr(dx), H.ptr(dy2), C.c_float(30.0), C.c_int64(2), C.c_int64(5000), int(fp32)) == 0
        torch.cuda.synchronize()
        diff = (dy.float() - dy2.float()).abs().max().item()
        assert diff <= 2 ** -5, diff        # the reference is compiled with fast-math: its tanhf is the 2^-11 hardware approximation
    ctx.softcap(dx, dx, 30.0)                                     # in place
    assert torch.equal(dx, dy)


@pytest.mark.parametrize("rows", [1, 5, 40])
@pytest.mark.parametrize("variant", ["plain", "padded_in", "bias_trim", "softcap_head", "dense_bias"])
def test_linear_forward(ctx, rows, variant):
    import torch
    import exl3b200
    from oracle import oracle as O
    r = H.rng(rows * 7 + len(variant))
    k, n, K, cb = 640, 512, 4, 1
    in_last = 600 if variant == "padded_in" else k
    out_unp = 500 if variant in ("bias_trim", "softcap_head") else n
    trim = variant in ("bias_trim", "softcap_head")
    cap = 30.0 if variant == "softcap_head" else 0.0
    bias = (r.standard_normal(n) * 0.5).astype(np.float16) if variant in ("bias_trim", "dense_bias") else None
    x = r.standard_normal((rows, in_last)).astype(np.float16)
    L = exl3b200.LinearLayer()
    keep = []
    if variant == "dense_bias":
        w = (r.standard_normal((k, n)) * 0.05).astype(np.float16)
        dw = H.to_dev(w); keep.append(dw)
        L.w.trellis, L.dense = None, dw.data_ptr()
        want = O.linear_forward(x, K, cb, k, n, dense=w, bias=bias)
    else:
        tr, suh, svh = H.rand_trellis(r, k, n, K), H.rand_signs(r, k), H.rand_signs(r, n)
        dtr, dsuh, dsvh = H.to_dev(tr), H.to_dev(suh), H.to_dev(svh); keep += [dtr, dsuh, dsvh]
        L.w.trellis, L.w.suh, L.w.svh = dtr.data_ptr(), dsuh.data_ptr(), dsvh.data_ptr()
        want = O.linear_forward(x, K, cb, k, n, trellis=tr, suh=suh, svh=svh, bias=bias, out_unpadded=out_unp,
                                trim_padded_out=trim, softcap_factor=cap)
    L.w.k, L.w.n, L.w.K, L.w.cb = k, n, K, cb
    if bias is not None:
        db = H.to_dev(bias); keep.append(db); L.bias = db.data_ptr()
    L.in_unpadded, L.out_unpadded, L.trim_padded_out, L.softcap = in_last, out_unp, int(trim), cap
    y = torch.full((rows, out_unp if trim else n), float("nan"), dtype=torch.float16, device="cuda")
    ctx.linear_forward(L, H.to_dev(x), y)
    ctx.poll_status()
    got = y.float().cpu().numpy()
    assert got.shape == want.shape and np.isfinite(got).all()
    # the GEMM bar, with one more fp16 step for each rounded epilogue stage
    assert H.gemm_mismatch(got, want.astype(np.float32), 2e-3, True, steps=1 + (bias is not None) + 2 * (cap != 0)) <= 1.0


def test_linear_forward_rejects_wide_input(ctx):
    import torch
    import exl3b200
    L = exl3b200.LinearLayer()
    t = torch.zeros(8, 8, 64, dtype=torch.int16, device="cuda")
    L.w.trellis = t.data_ptr(); L.w.k, L.w.n, L.w.K, L.w.cb = 128, 128, 4, 0
    L.in_unpadded = L.out_unpadded = 128
    x = torch.zeros(1, 256, dtype=torch.float16, device="cuda")
    y = torch.zeros(1, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(exl3b200.Exl3Error):
        ctx.linear_forward(L, x, y)
