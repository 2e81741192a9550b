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
        # same kernels; only the split-K factor may differ with the scratch size, so the usual GEMM bar applies
        assert H.gemm_mismatch(g, w, 2e-3, not c_fp32) <= 1.0, call


def test_noalloc_rejects_sizes_beyond_its_scratch():
    import torch
    from exl3b200 import lib
    a = torch.zeros(17, 128, dtype=torch.float16, device="cuda")
    tr = torch.zeros(8, 8, 64, dtype=torch.int16, device="cuda")
    c = torch.zeros(17, 128, dtype=torch.float16, device="cuda")
    rc = lib().exl3_gemm_noalloc(C.c_void_p(0), H.ptr(a), H.ptr(tr), H.ptr(c), None, None, 17, 128, 128, 4, 0, 0, 0)
    assert rc == -3      # EXL3_ERR_WORKSPACE: more rows than the fixed scratch holds
