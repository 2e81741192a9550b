"""CUDA-graph capture/replay of ops through exl3_graph_* (the reference's CudaGraph, src/ffi.rs:403-451)."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def test_capture_and_replay_decode_ops(ctx):
    import torch
    import exl3b200
    r = H.rng(5)
    m, k, n, K = 2, 1024, 3072, 4
    dA = H.to_dev(r.standard_normal((m, k)).astype(np.float16))
    dtr = H.to_dev(H.rand_trellis(r, k, n, K))
    dsuh, dsvh = H.to_dev(H.rand_signs(r, k)), H.to_dev(H.rand_signs(r, n))
    c = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    z = torch.zeros(m, n, dtype=torch.float16, device="cuda")
    want_c = torch.empty_like(c); want_z = torch.empty_like(z)
    ctx.exl3_gemm(dA, dtr, want_c, dsuh, None, dsvh, mcg=True)
    ctx.silu_mul(want_c, want_c, want_z)
    torch.cuda.synchronize()

    g = exl3b200.CudaGraph(ctx)
    side = g.side_stream()
    # warm-up on the side stream (sets the kernels' attributes outside the capture), then capture
    ctx.exl3_gemm(dA, dtr, c, dsuh, None, dsvh, mcg=True, stream=side)
    exl3b200.lib().exl3_sync_side_stream(ctx.handle)
    g.capture_begin()
    ctx.exl3_gemm(dA, dtr, c, dsuh, None, dsvh, mcg=True, stream=side)
    ctx.silu_mul(c, c, z, stream=side)
    g.capture_end()
    c.zero_(); z.zero_()
    torch.cuda.synchronize()
    for _ in range(3):
        g.replay()
    assert exl3b200.lib().exl3_sync_side_stream(ctx.handle) == 0
    assert torch.equal(c, want_c) and torch.equal(z, want_z)
    # new input values through the same pointers are picked up by the replay
    dA.copy_(H.to_dev(r.standard_normal((m, k)).astype(np.float16)))
    ctx.exl3_gemm(dA, dtr, want_c, dsuh, None, dsvh, mcg=True)
    torch.cuda.synchronize()
    g.replay()
    exl3b200.lib().exl3_sync_side_stream(ctx.handle)
    assert torch.equal(c, want_c)
    assert exl3b200.lib().exl3_cuda_free_mib() > 0
