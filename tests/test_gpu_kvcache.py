"""GPU parity of the paged KV write path (append, quantise on write, dequantise) through the C-ABI."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _torch():
    import torch
    return torch


def _pools(pages, nkv, hd, bits):
    torch = _torch()
    groups = nkv * hd // 32
    qk = torch.zeros(pages, 256, groups * bits, dtype=torch.int32, device="cuda")
    sk = torch.zeros(pages, 256, groups, dtype=torch.float16, device="cuda")
    return qk, sk, torch.zeros_like(qk), torch.zeros_like(sk)


def test_paged_kv_update(ctx, ref):
    from oracle import oracle as O
    torch = _torch()
    r = H.rng(1)
    bsz, seq, nkv, hd = 5, 3, 8, 128
    ctxlen = np.array([0, 255, 256, 700, 1023], np.int32)
    bt, pages = H.make_paged(r, bsz, ctxlen, nkv, hd, append=seq)
    k = r.standard_normal((bsz, seq, nkv, hd)).astype(np.float16)
    v = r.standard_normal((bsz, seq, nkv, hd)).astype(np.float16)
    kc0 = r.standard_normal((pages, 256, nkv, hd)).astype(np.float16)
    vc0 = r.standard_normal((pages, 256, nkv, hd)).astype(np.float16)
    kc, vc = H.to_dev(kc0), H.to_dev(vc0)
    dbt, dsl = H.to_dev(bt), H.to_dev(ctxlen)
    ctx.paged_kv_cache_update(H.to_dev(k), H.to_dev(v), kc, vc, dbt, dsl)
    wk, wv = kc0.copy(), vc0.copy()
    O.paged_kv_update(k, v, wk, wv, bt, ctxlen)
    assert np.array_equal(kc.cpu().numpy().view(np.uint16), wk.view(np.uint16))
    assert np.array_equal(vc.cpu().numpy().view(np.uint16), wv.view(np.uint16))
    if ref is not None:
        kc2, vc2 = H.to_dev(kc0), H.to_dev(vc0)
        dk, dv = H.to_dev(k), H.to_dev(v)
        assert ref.ref_paged_kv_cache_update(H.ptr(dk), H.ptr(dv), H.ptr(kc2), H.ptr(vc2), H.ptr(dbt), H.ptr(dsl), bsz, seq,
                                             nkv, hd, pages, bt.shape[1]) == 0
        torch.cuda.synchronize()
        assert torch.equal(kc, kc2) and torch.equal(vc, vc2)


def test_paged_kv_update_ragged(ctx):
    from oracle import oracle as O
    r = H.rng(2)
    nkv, hd = 8, 128
    qlens = np.array([1, 8, 0, 256, 1], np.int32)
    cu = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)
    ctxlen = np.array([10, 300, 5, 512, 2047], np.int32)
    bt, pages = H.make_paged(r, 5, ctxlen + qlens, nkv, hd)
    rows = int(cu[-1])
    k = r.standard_normal((rows, nkv, hd)).astype(np.float16)
    v = r.standard_normal((rows, nkv, hd)).astype(np.float16)
    kc0 = np.zeros((pages, 256, nkv, hd), np.float16)
    kc, vc = H.to_dev(kc0), H.to_dev(kc0)
    ctx.paged_kv_cache_update(H.to_dev(k), H.to_dev(v), kc, vc, H.to_dev(bt), H.to_dev(ctxlen), cu_q=H.to_dev(cu))
    wk, wv = kc0.copy(), kc0.copy()
    for b in range(5):
        if qlens[b]:
            O.paged_kv_update(k[None, cu[b]:cu[b + 1]], v[None, cu[b]:cu[b + 1]], wk, wv, bt[b:b + 1], ctxlen[b:b + 1])
    assert np.array_equal(kc.cpu().numpy().view(np.uint16), wk.view(np.uint16))
    assert np.array_equal(vc.cpu().numpy().view(np.uint16), wv.view(np.uint16))


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 6, 7, 8])
def test_quant_dequant_cache_paged(ctx, ref, bits):
    """Codes and scales against the oracle (the device uses the approximate reciprocal of the reference's fast-math
    build, so a code may differ by one step where v/s*m sits on an integer boundary), bit-exact against the reference
    CUDA op; dequantised values against both."""
    from oracle import oracle as O
    torch = _torch()
    r = H.rng(70 + bits)
    bsz, seq, nkv, hd = 4, 5, 8, 128
    ctxlen = np.array([0, 254, 300, 1000], np.int32)
    bt, pages = H.make_paged(r, bsz, ctxlen, nkv, hd, append=seq)
    k = (0.5 * r.standard_normal((bsz, seq, nkv, hd))).astype(np.float16)
    v = (0.5 * r.standard_normal((bsz, seq, nkv, hd))).astype(np.float16)
    qk, sk, qv, sv = _pools(pages, nkv, hd, bits)
    dk, dv, dbt, dsl = H.to_dev(k), H.to_dev(v), H.to_dev(bt), H.to_dev(ctxlen)
    ctx.quant_cache_paged(dk, qk, sk, dv, qv, sv, dsl, dbt)
    groups = nkv * hd // 32
    oqk = np.zeros((pages, 256, groups * bits), np.uint32); osk = np.zeros((pages, 256, groups), np.float16)
    oqv = np.zeros_like(oqk); osv = np.zeros_like(osk)
    O.quant_cache_paged(k, oqk, osk, v, oqv, osv, ctxlen, bt, bits, bits)
    assert np.array_equal(sk.cpu().numpy().view(np.uint16), osk.view(np.uint16))
    assert np.array_equal(sv.cpu().numpy().view(np.uint16), osv.view(np.uint16))
    gqk = qk.cpu().numpy().view(np.uint32)
    mism = (gqk != oqk).reshape(-1, bits).any(axis=1).mean()
    assert mism < 2e-3, f"fraction of groups whose codes differ from the oracle: {mism}"
    if ref is not None:
        qk2, sk2, qv2, sv2 = _pools(pages, nkv, hd, bits)
        assert ref.ref_quant_cache_paged(H.ptr(dk), H.ptr(qk2), H.ptr(sk2), H.ptr(dv), H.ptr(qv2), H.ptr(sv2), H.ptr(dsl),
                                         H.ptr(dbt), bsz, seq, nkv, hd, pages, bt.shape[1], bits, bits) == 0
        torch.cuda.synchronize()
        assert torch.equal(qk, qk2) and torch.equal(qv, qv2) and torch.equal(sk, sk2) and torch.equal(sv, sv2)

    # dequantise what was just written (now cache_seqlens = ctx + seq), in place and compact
    newlen = (ctxlen + seq).astype(np.int32)
    dnl = H.to_dev(newlen)
    ko = torch.zeros(pages, 256, nkv, hd, dtype=torch.float16, device="cuda"); vo = torch.zeros_like(ko)
    ctx.dequant_cache_paged(qk, sk, ko, qv, sv, vo, dnl, dbt)
    wko = np.zeros((pages, 256, nkv * hd), np.float16); wvo = np.zeros_like(wko)
    O.dequant_cache_paged(gqk, sk.cpu().numpy(), wko, qv.cpu().numpy().view(np.uint32), sv.cpu().numpy(), wvo, newlen, bt,
                          bits, bits)
    got = ko.cpu().numpy().reshape(pages, 256, -1)
    assert np.abs(got.astype(np.float32) - wko.astype(np.float32)).max() <= 2e-3
    # the written rows reproduce the inputs to within the quantiser's step
    for b in range(bsz):
        for s in range(seq):
            pos = ctxlen[b] + s
            row = got[bt[b, pos // 256], pos % 256]
            err = np.abs(row.astype(np.float32) - k[b, s].reshape(-1).astype(np.float32)).max()
            assert err < 6.0 / (1 << bits), (b, s, err)
    pps = bt.shape[1]
    kw = torch.zeros(bsz * pps, 256, nkv, hd, dtype=torch.float16, device="cuda"); vw = torch.zeros_like(kw)
    ctx.dequant_cache_paged_window(qk, sk, kw, qv, sv, vw, dsl, dbt, bonus_len=seq)
    gw = kw.cpu().numpy()
    gfull = ko.cpu().numpy()
    for b in range(bsz):
        for p in range((newlen[b] + 255) // 256):
            nt = min(256, newlen[b] - p * 256)
            assert np.array_equal(gw[b * pps + p, :nt].view(np.uint16), gfull[bt[b, p], :nt].view(np.uint16))
    if ref is not None:
        ko2 = torch.zeros_like(ko); vo2 = torch.zeros_like(vo)
        assert ref.ref_dequant_cache_paged(H.ptr(qk), H.ptr(sk), H.ptr(ko2), H.ptr(qv), H.ptr(sv), H.ptr(vo2), H.ptr(dnl),
                                           H.ptr(dbt), bsz, nkv, hd, pages, pages, pps, bits, bits, 0, 0) == 0
        torch.cuda.synchronize()
        dk_ = (ko.float() - ko2.float()).abs().max().item()
        dv_ = (vo.float() - vo2.float()).abs().max().item()
        assert dk_ <= 1e-3 and dv_ <= 1e-3, (dk_, dv_, (ko != ko2).sum().item(), (vo != vo2).sum().item())


def test_quant_rejects_unsupported(ctx):
    import exl3b200
    torch = _torch()
    qk, sk, qv, sv = _pools(2, 8, 128, 4)
    k = torch.zeros(1, 1, 8, 128, dtype=torch.float16, device="cuda")
    bt = torch.zeros(1, 1, dtype=torch.int32, device="cuda")
    sl = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(exl3b200.Exl3Error):
        ctx.quant_cache_paged(k, qk, sk, k, qv, sv, sl, bt, compand_a=0.5)
    with pytest.raises(exl3b200.Exl3Error):
        ctx.quant_cache_paged(k, qk, sk, k, qv, sv, sl, bt, page_size=128)
