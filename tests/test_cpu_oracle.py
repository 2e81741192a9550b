"""CPU tests: the oracle against the golden fixtures produced by the reference's own CUDA ops
(tests/golden/golden_ref.npz, made by tests/golden/make_golden.py), plus internal consistency of the oracle."""
import os

import numpy as np
import pytest

from oracle import oracle as O
from tests import helpers as H
from tests.golden import cases

GOLD = os.path.join(os.path.dirname(cases.__file__), "golden_ref.npz")


@pytest.fixture(scope="module")
def gold():
    if not os.path.exists(GOLD):
        pytest.skip("golden fixtures not generated yet")
    return np.load(GOLD)


def test_codebooks_are_finite_and_centred():
    for cb, std in ((0, 1.244), (1, 1.244), (2, 1.0)):
        c = O.codebook(cb).astype(np.float64)
        assert np.isfinite(c).all()
        assert abs(c.mean()) < 5e-3 and abs(c.std() - std) < 5e-3


def test_reconstruct_bit_exact_vs_reference(gold):
    for name, c in cases.reconstruct_cases():
        w = O.reconstruct(c["trellis"], c["K"], c["cb"])
        assert np.array_equal(w.view(np.uint16), gold[name].view(np.uint16)), name


def test_gemm_vs_reference(gold):
    """The reference kernel keeps its cross-CTA partial sums in the fp16 output buffer, so its own result carries up to
    about one extra fp16 rounding step; the bar is 2e-3 * RMS or two fp16 steps of the value."""
    for name, c in cases.gemm_cases():
        w = O.exl3_gemm(c["A"], c["trellis"], c["suh"], c["svh"], c["K"], c["cb"]).astype(np.float64)
        g = gold[name].astype(np.float64)
        rms = np.sqrt((g * g).mean())
        allowed = np.maximum(2e-3 * rms, 2.002 * H.fp16_ulp(g))
        assert (np.abs(w - g) <= allowed).all(), name


def test_hadamard_norm_rope_silu_vs_reference(gold):
    for name, c in cases.had_cases():
        w = O.had_r_128(c["x"], c["scale"] if c["mode"] == "pre" else None, c["scale"] if c["mode"] == "post" else None)
        assert np.array_equal(w.view(np.uint16), gold[name].view(np.uint16)), name
    for name, c in cases.norm_cases():
        res = c["res"].copy()
        y = O.rms_norm(c["x"], c["w"], 1e-6, res=res)
        assert np.array_equal(res, gold[name + "_r"])
        assert np.abs(y.astype(np.float32) - gold[name + "_y"].astype(np.float32)).max() <= 2e-3
    for name, c in cases.rope_cases():
        q, k = O.rope(c["q"], c["k"], c["inv_freq"], 0, c["positions"], c["q_norm"], c["k_norm"], 1e-6, 0.0, 2, 1.0)
        # the device uses __sinf/__cosf; positions reach ~300 rad here
        assert np.abs(q.astype(np.float32) - gold[name + "_q"].astype(np.float32)).max() <= 1e-2
        assert np.abs(k.astype(np.float32) - gold[name + "_k"].astype(np.float32)).max() <= 1e-2
    for name, c in cases.silu_cases():
        z = O.silu_mul(c["x"], c["y"]).astype(np.float32)
        g = gold[name].astype(np.float32)
        assert np.abs(z - g).max() <= 4e-3 * max(1.0, np.abs(g).max())


def test_kv_codec_vs_reference(gold):
    for name, c in cases.kvquant_cases():
        bits, groups = c["bits"], c["nkv"] * c["hd"] // 32
        qk = np.zeros((c["pages"], 256, groups * bits), np.uint32); sk = np.zeros((c["pages"], 256, groups), np.float16)
        qv = np.zeros_like(qk); sv = np.zeros_like(sk)
        O.quant_cache_paged(c["k"], qk, sk, c["v"], qv, sv, c["seqlens"], c["block_table"], bits, bits)
        assert np.array_equal(sk.view(np.uint16), gold[name + "_sk"].view(np.uint16)), name
        gq = gold[name + "_qk"].view(np.uint32)
        assert (qk != gq).reshape(-1, bits).any(axis=1).mean() < 2e-3, name
        bsz, seq = c["k"].shape[:2]
        ko = np.zeros((c["pages"], 256, c["nkv"] * c["hd"]), np.float16); vo = np.zeros_like(ko)
        O.dequant_cache_paged(gq, gold[name + "_sk"], ko, gq, gold[name + "_sk"], vo, (c["seqlens"] + seq).astype(np.int32),
                              c["block_table"], bits, bits)
        rows = [ko[c["block_table"][b, (c["seqlens"][b] + s) // 256], (c["seqlens"][b] + s) % 256]
                for b in range(bsz) for s in range(seq)]
        assert np.abs(np.stack(rows).astype(np.float32) - gold[name + "_deq"].astype(np.float32)).max() <= 1e-3, name


def test_attention_vs_reference(gold):
    for name, c in cases.attn_cases():
        kc, vc = c["kc"].copy(), c["vc"].copy()
        O.paged_kv_update(c["k"], c["v"], kc, vc, c["block_table"], c["seqlens"])
        o = O.attn_paged(c["q"], kc, vc, c["block_table"], c["seqlens"])
        for mma in (0, 1):
            key = f"{name}_mma{mma}"
            if key in gold.files:
                assert H.gemm_mismatch(o, gold[key], 2e-3, True) <= 1.0, key


def test_kv_codec_round_trip_and_packing():
    r = H.rng(3)
    x = (0.5 * r.standard_normal(32 * 64)).astype(np.float16)
    for bits in range(2, 9):
        q, s = O.quant_groups(x, bits)
        y = O.dequant_groups(q, s, bits)
        assert np.abs(y.astype(np.float32) - x.astype(np.float32)).max() < 6.0 / (1 << bits)
        assert q.shape == (64, bits)


def test_gemm_equals_reconstruct_path():
    """exl3_gemm == had(post) o matmul(had(pre)(A), reconstruct(W)): the two routes of the reference's Linear
    (src/modules.rs:225-234) agree."""
    r = H.rng(4)
    A = r.standard_normal((3, 256)).astype(np.float16)
    tr = H.rand_trellis(r, 256, 384, 3)
    suh, svh = H.rand_signs(r, 256), H.rand_signs(r, 384)
    c1 = O.exl3_gemm(A, tr, suh, svh, 3, 1, c_fp32=True)
    W = O.reconstruct(tr, 3, 1)
    ah = O.had_r_128(A, pre=suh)
    c2 = O.had_r_128(O.hgemm(ah, W, c_fp32=True), post=svh)
    assert H.rel_rms_err(c1, c2) < 1e-5


def test_attention_ragged_equals_rectangular():
    r = H.rng(5)
    nq, nkv, hd = 4, 2, 128
    seqlens = np.array([10, 300], np.int32)
    bt, pages = H.make_paged(r, 2, seqlens, nkv, hd, append=3)
    q = r.standard_normal((2, 3, nq, hd)).astype(np.float16)
    kc = (0.5 * r.standard_normal((pages, 256, nkv, hd))).astype(np.float16)
    vc = (0.5 * r.standard_normal((pages, 256, nkv, hd))).astype(np.float16)
    a = O.attn_paged(q, kc, vc, bt, seqlens)
    b = O.attn_paged(q.reshape(6, nq, hd), kc, vc, bt, seqlens, cu_q=np.array([0, 3, 6], np.int32))
    assert np.array_equal(a.reshape(6, nq, hd).view(np.uint16), b.view(np.uint16))
