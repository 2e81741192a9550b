"""exl3_gemm_noalloc: the EXL3 GEMM variant for callers that may not allocate device memory (allocator callbacks,
latency-critical loops, fixed-budget plug-ins).  It is called through the C-ABI without any context, twice in a row on
the same stream (the second call meets the scratch array as the first one left it), and must reproduce exl3_gemm.
This file sorts last so that a run stopping at the first failure has already executed every other test."""
import ctypes as C

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,k,n,K,cb,c_fp32", [(1, 5120, 17408, 4, 1, False), (8, 1024, 3072, 8, 0, True),
                                               (16, 2048, 1024, 3, 2, False)])
def test_noalloc_matches_context_gemm_twice(ctx, m, k, n, K, cb, c_fp32):
    import torch
    from exl3b200 import lib
    r = H.rng(m + k + K)
    dtr = H.to_dev(H.rand_trellis(r, k, n, K))
    dsuh, dsvh = H.to_dev(H.rand_signs(r, k)), H.to_dev(H.rand_signs(r, n))
    dt = torch.float32 if c_fp32 else torch.float16
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        dA = H.to_dev(r.standard_normal((m, k)).astype(np.float16))
        want = torch.empty(m, n, dtype=dt, device="cuda")
        ctx.exl3_gemm(dA, dtr, want, dsuh, None, dsvh, mcg=cb == 1, mul1=cb == 2)
        got = torch.full((m, n), float("nan"), dtype=dt, device="cuda")
        rc = lib().exl3_gemm_noalloc(stream, H.ptr(dA), H.ptr(dtr), H.ptr(got), H.ptr(dsuh), H.ptr(dsvh), m, k, n, K,
                                     int(c_fp32), int(cb == 1), int(cb == 2))
        assert rc == 0
        torch.cuda.synchronize()
        g, w = got.float().cpu().numpy(), want.float().cpu().numpy()
        assert np.isfinite(g).all()
        # two different kernels behind the two entry points (and different split-K factors): the usual GEMM bar applies
        assert H.gemm_mismatch(g, w, 2e-3, not c_fp32) <= 1.0, call
    assert lib().exl3_gemm_noalloc_poll_status(stream) == 0


def test_noalloc_wide_tensor_keeps_its_grid_and_allocates_nothing(ctx):
    """the 151936-column head at 16 rows: the partial sums of a grid that covers the GPU fit the fixed array (a CTA
    publishes at most two 128-column tiles whatever the column count), the result equals exl3_gemm's, the call is as
    fast as the context's small-M kernel would be (not a one-CTA crawl), and a warmed call leaves the amount of free
    device memory unchanged"""
    import torch
    from exl3b200 import lib
    m, k, n, K = 16, 5120, 151936, 4
    g = torch.Generator(device="cuda"); g.manual_seed(5)
    tr = torch.randint(-32768, 32768, (k // 16, n // 16, 16 * K), dtype=torch.int16, device="cuda", generator=g)
    suh = (torch.randint(0, 2, (k,), device="cuda", generator=g) * 2 - 1).to(torch.float16)
    svh = (torch.randint(0, 2, (n,), device="cuda", generator=g) * 2 - 1).to(torch.float16)
    A = torch.randn(m, k, device="cuda", generator=g).to(torch.float16)
    want = torch.empty(m, n, dtype=torch.float16, device="cuda")
    ctx.exl3_gemm(A, tr, want, suh, None, svh, mcg=True)
    ctx.poll_status()
    got = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = (stream, H.ptr(A), H.ptr(tr), H.ptr(got), H.ptr(suh), H.ptr(svh), m, k, n, K, 0, 1, 0)
    assert lib().exl3_gemm_noalloc(*args) == 0            # warm-up: first use of this (bits, codebook) on the device
    torch.cuda.synchronize()
    free0 = lib().exl3_cuda_free_mib()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    assert lib().exl3_gemm_noalloc(*args) == 0
    e1.record()
    torch.cuda.synchronize()
    assert lib().exl3_cuda_free_mib() == free0
    assert lib().exl3_gemm_noalloc_poll_status(stream) == 0
    assert torch.isfinite(got).all()
    assert H.gemm_mismatch(got.float().cpu().numpy(), want.float().cpu().numpy(), 2e-3, True) <= 1.0
    assert e0.elapsed_time(e1) < 5.0, "389 MB of codes at decode speed take well under a millisecond"


def test_noalloc_rejects_sizes_beyond_its_scratch():
    import torch
    from exl3b200 import lib
    a = torch.zeros(17, 128, dtype=torch.float16, device="cuda")
    tr = torch.zeros(8, 8, 64, dtype=torch.int16, device="cuda")
    c = torch.zeros(17, 128, dtype=torch.float16, device="cuda")
    rc = lib().exl3_gemm_noalloc(C.c_void_p(0), H.ptr(a), H.ptr(tr), H.ptr(c), None, None, 17, 128, 128, 4, 0, 0, 0)
    assert rc == -3      # EXL3_ERR_WORKSPACE: more rows than the fixed scratch holds
