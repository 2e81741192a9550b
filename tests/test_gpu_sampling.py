"""Sampler-side ops (penalties over a token history, Gumbel noise and Gumbel-max sampling on the reference's Philox
stream, page permutation) and two small element-wise ops, against the oracle and, when it was built, the reference's ops."""
import ctypes as C

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu

VOCAB = 151936


def _history(r, n, vocab=VOCAB):
    past = r.integers(0, vocab, n).astype(np.int64)
    past[::7] = past[0]                       # one token many times
    past[-3:] = [11, 4097, vocab - 1]         # span borders
    return past


@pytest.mark.parametrize("fp32", [False, True])
@pytest.mark.parametrize("past_len,sustain,decay", [(1000, 256, 512), (300, 1024, 0), (50, 10, 20), (0, 10, 10)])
def test_repetition_penalty(ctx, ref, fp32, past_len, sustain, decay):
    import torch
    from oracle import oracle as O
    r = H.rng(past_len + sustain)
    logits = (r.standard_normal((1, VOCAB)) * 4).astype(np.float32 if fp32 else np.float16)
    past = _history(r, past_len) if past_len else np.zeros(0, np.int64)
    dl, dp = H.to_dev(logits), H.to_dev(past.reshape(1, -1))
    out = torch.full((1, VOCAB), float("nan"), dtype=torch.float32, device="cuda")
    ctx.apply_rep_pens(dl, out, dp, 1.3, sustain, decay)
    want = O.apply_rep_pens(logits, past, 1.3, sustain, decay)
    got = out.cpu().numpy()
    assert np.allclose(got, want, rtol=2e-6, atol=1e-6), float(np.abs(got - want).max())
    if ref is not None and hasattr(ref, "ref_apply_rep_pens") and past_len:
        out2 = torch.empty_like(out)
        assert ref.ref_apply_rep_pens(H.ptr(dl), int(fp32), H.ptr(out2), H.ptr(dp), C.c_float(1.3), sustain, decay, VOCAB, past_len) == 0
        torch.cuda.synchronize()
        assert np.allclose(got, out2.cpu().numpy(), rtol=2e-6, atol=1e-6)      # the reference divides with fast-math


@pytest.mark.parametrize("past_len,sustain,decay", [(1000, 256, 512), (300, 1024, 0), (50, 10, 20)])
def test_presence_frequency_penalty(ctx, ref, past_len, sustain, decay):
    import torch
    from oracle import oracle as O
    r = H.rng(past_len)
    logits = (r.standard_normal((1, VOCAB)) * 4).astype(np.float16)
    past = _history(r, past_len)
    dl, dp = H.to_dev(logits), H.to_dev(past.reshape(1, -1))
    out = torch.full((1, VOCAB), float("nan"), dtype=torch.float32, device="cuda")
    ctx.apply_pres_freq_pens(dl, out, dp, 0.7, 0.2, sustain, decay)
    want = O.apply_pres_freq_pens(logits, past, 0.7, 0.2, sustain, decay)
    got = out.cpu().numpy()
    # the frequency term is a sum of up to ~150 weights added in no fixed order
    assert np.allclose(got, want, rtol=1e-5, atol=2e-5), float(np.abs(got - want).max())
    if ref is not None and hasattr(ref, "ref_apply_pres_freq_pens"):
        out2 = torch.empty_like(out)
        assert ref.ref_apply_pres_freq_pens(H.ptr(dl), 0, H.ptr(out2), H.ptr(dp), C.c_float(0.7), C.c_float(0.2), sustain, decay,
                                            VOCAB, past_len) == 0
        torch.cuda.synchronize()
        assert np.allclose(got, out2.cpu().numpy(), rtol=1e-5, atol=2e-5)


def test_gumbel_noise_matches_the_reference_stream(ctx, ref):
    import torch
    from oracle import oracle as O
    r = H.rng(5)
    x = r.standard_normal(200001).astype(np.float32)
    dx = H.to_dev(x)
    out = torch.empty_like(dx)
    ctx.gumbel_noise_f32(dx, out, random=0xC0FFEE11)
    got = out.cpu().numpy()
    if ref is not None and hasattr(ref, "ref_gumbel_noise_f32"):
        out2 = torch.empty_like(dx)
        assert ref.ref_gumbel_noise_f32(H.ptr(dx), H.ptr(out2), C.c_int64(x.size), C.c_uint32(0xC0FFEE11)) == 0
        torch.cuda.synchronize()
        assert torch.equal(out, out2), "same generator, same stream, same arithmetic: equal bits"
    want = O.gumbel_noise_f32(x, 0xC0FFEE11)
    # the device takes -log(-log u) with the fast logarithm, whose absolute error of about 1e-7 is a large relative one
    # on -log u for the u next to 1: half of the values agree to 1e-6, 99.9 % to 1e-3, the rest to a few 1e-2
    err = np.abs(got - want)
    assert np.median(err) < 1e-6 and np.quantile(err, 0.999) < 1e-3 and err.max() < 0.1, (float(np.quantile(err, 0.999)), float(err.max()))
    g = got - x
    assert abs(g.mean() - 0.5772) < 0.02 and abs(g.var() - np.pi ** 2 / 6) < 0.05       # a standard Gumbel sample


@pytest.mark.parametrize("rows,n,max_logit", [(1, VOCAB, 0), (5, 32000, 0), (3, 5000, 3001), (2, 129, 0)])
def test_gumbel_sample(ctx, ref, rows, n, max_logit):
    import torch
    from oracle import oracle as O
    r = H.rng(rows + n)
    logits = (r.standard_normal((rows, n)) * 2).astype(np.float16)
    dl = H.to_dev(logits)
    ids = torch.full((rows, 1), -1, dtype=torch.int64, device="cuda")
    seed = 12345 + n
    ctx.gumbel_sample(dl, ids, max_logit=max_logit, random=seed)
    got = ids.cpu().numpy().reshape(-1)
    noisy = O.gumbel_sample_noisy(logits, seed, max_logit)
    lim = noisy.shape[1]
    assert ((got >= 0) & (got < lim)).all() and np.isfinite(noisy[np.arange(rows), got]).all()
    for i in range(rows):       # the chosen column is the oracle's maximum up to the fast logarithm's error
        assert noisy[i, got[i]] >= noisy[i].max() - 1e-3, (i, got[i], int(noisy[i].argmax()))
    # (the reference's kernel reads fp16 pairs from the start of every row, which needs an even row length as soon as
    # there is a second row: kernels/generator/sampling_basic.cu:39-62,100; odd lengths are checked against the oracle only)
    if ref is not None and hasattr(ref, "ref_gumbel_sample") and n % 2 == 0:
        ids2 = torch.full((rows, 1), -1, dtype=torch.int64, device="cuda")
        assert ref.ref_gumbel_sample(H.ptr(dl), H.ptr(ids2), rows, n, max_logit, C.c_uint32(seed)) == 0
        torch.cuda.synchronize()
        assert torch.equal(ids, ids2)
    # fp32 logits go through the same stream
    ids3 = torch.full((rows, 1), -1, dtype=torch.int64, device="cuda")
    ctx.gumbel_sample(dl.float(), ids3, max_logit=max_logit, random=seed)
    assert torch.equal(ids, ids3)


def test_cache_rotate(ctx, ref):
    import torch
    from oracle import oracle as O
    r = H.rng(8)
    pages, shape = 9, (256, 2, 24)                 # 24 KB pages of fp16
    cache = r.standard_normal((pages,) + shape).astype(np.float16)
    order = np.array([-1, 3, 3, 5, 5, 0, 0, -1, 7, 7, 2, 8, 8, 2], np.int32)     # a cycle through temp, a self-copy, an overwrite chain
    dc, do = H.to_dev(cache.copy()), H.to_dev(order)
    temp = torch.zeros(shape, dtype=torch.float16, device="cuda")
    ctx.cache_rotate(dc, do, temp)
    want = O.cache_rotate(cache.copy(), order, np.zeros(shape, np.float16))
    assert np.array_equal(dc.cpu().numpy(), want)
    if ref is not None and hasattr(ref, "ref_cache_rotate"):
        dc2 = H.to_dev(cache.copy())
        temp2 = torch.zeros(shape, dtype=torch.float16, device="cuda")
        page_bytes = int(np.prod(shape)) * 2
        assert ref.ref_cache_rotate(H.ptr(dc2), H.ptr(do), H.ptr(temp2), pages, order.size // 2, C.c_int64(page_bytes)) == 0
        torch.cuda.synchronize()
        assert torch.equal(dc, dc2) and torch.equal(temp, temp2)


def test_mul_sigmoid_and_deinterleave(ctx, ref):
    import torch
    from oracle import oracle as O
    r = H.rng(9)
    x = r.standard_normal(6 * 1024).astype(np.float16)
    y = (r.standard_normal(6 * 1024) * 3).astype(np.float16)
    dx, dy = H.to_dev(x.copy()), H.to_dev(y)
    ctx.mul_sigmoid_(dx, dy)
    got = dx.cpu().numpy().astype(np.float64)
    want = O.mul_sigmoid(x, y).astype(np.float64)
    assert (np.abs(got - want) <= 2.001 * H.fp16_ulp(want)).all()          # fp16 exp and reciprocal of the device vs exact
    if ref is not None and hasattr(ref, "ref_mul_sigmoid_"):
        dx2 = H.to_dev(x.copy())
        assert ref.ref_mul_sigmoid_(H.ptr(dx2), H.ptr(dy), C.c_int64(x.size)) == 0
        torch.cuda.synchronize()
        assert torch.equal(dx, dx2)
    rows, heads, hd = 7, 5, 64
    qg = r.standard_normal((rows, heads * 2 * hd)).astype(np.float16)
    dqg = H.to_dev(qg)
    q = torch.empty(rows, heads * hd, dtype=torch.float16, device="cuda")
    g = torch.empty_like(q)
    ctx.deinterleave_qg(dqg, q, g, hd)
    v = qg.reshape(rows, heads, 2, hd)
    assert np.array_equal(q.cpu().numpy(), v[:, :, 0].reshape(rows, -1)) and np.array_equal(g.cpu().numpy(), v[:, :, 1].reshape(rows, -1))
