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


def test_capture_ragged_attention_with_stream_fork(ctx):
    """A ragged attention call with decode rows and long row blocks forks its decode pass onto the context's second
    stream; captured into a graph, the replay must give exactly what the eager call gives."""
    import torch
    import exl3b200
    r = H.rng(77)
    nq, nkv, hd = 40, 8, 128
    qlens = np.array([1, 1, 256, 1, 70], np.int32)
    ctx_lens = np.array([500, 3000, 2048, 9000, 255], np.int32)
    cu = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)
    bt, pages = H.make_paged(r, len(qlens), ctx_lens + qlens, nkv, hd)
    rows = int(cu[-1])
    q = H.to_dev(r.standard_normal((rows, nq, hd)).astype(np.float16))
    k = H.to_dev((0.5 * r.standard_normal((rows, nkv, hd))).astype(np.float16))
    v = H.to_dev((0.5 * r.standard_normal((rows, nkv, hd))).astype(np.float16))
    kc = H.to_dev((0.5 * r.standard_normal((pages, 256, nkv, hd))).astype(np.float16))
    vc = H.to_dev((0.5 * r.standard_normal((pages, 256, nkv, hd))).astype(np.float16))
    dbt, dsl, dcu = H.to_dev(bt), H.to_dev(ctx_lens), H.to_dev(cu)
    want = torch.full((rows, nq, hd), float("nan"), dtype=torch.float16, device="cuda")
    ctx.bighead_attn_paged(q, k, v, kc, vc, dbt, dsl, want, cu_q=dcu, max_q_len=int(qlens.max()))
    ctx.poll_status()
    torch.cuda.synchronize()

    g = exl3b200.CudaGraph(ctx)
    side = g.side_stream()
    got = torch.full_like(want, float("nan"))
    ctx.bighead_attn_paged(q, k, v, kc, vc, dbt, dsl, got, cu_q=dcu, max_q_len=int(qlens.max()), stream=side)   # warm-up
    exl3b200.lib().exl3_sync_side_stream(ctx.handle)
    g.capture_begin()
    ctx.bighead_attn_paged(q, k, v, kc, vc, dbt, dsl, got, cu_q=dcu, max_q_len=int(qlens.max()), stream=side)
    g.capture_end()
    got.fill_(float("nan"))
    torch.cuda.synchronize()
    for _ in range(2):
        g.replay()
    assert exl3b200.lib().exl3_sync_side_stream(ctx.handle) == 0
    ctx.poll_status()
    assert torch.isfinite(got).all()
    assert torch.equal(got, want)


def test_bounded_wait_times_out_and_the_context_recovers(ctx):
    """the failure path: a device-side wait that can never be satisfied gives up after its poll limit, the status word
    carries it to the host as EXL3_ERR_DEVICE_WAIT (once), and the context keeps working"""
    import torch
    import exl3b200
    from exl3b200 import lib
    from oracle import oracle as O
    ctx.poll_status()
    assert lib().exl3_selftest_bounded_wait(ctx.handle, ctx.stream(), 1000) == 0
    with pytest.raises(exl3b200.Exl3Error, match="bounded device-side wait"):
        ctx.poll_status()
    ctx.poll_status()                                   # cleared by the report
    r = H.rng(3)
    m, k, n, K = 3, 1024, 512, 4
    A = r.standard_normal((m, k)).astype(np.float16)
    tr, suh, svh = H.rand_trellis(r, k, n, K), H.rand_signs(r, k), H.rand_signs(r, n)
    c = torch.empty(m, n, dtype=torch.float32, device="cuda")
    ctx.exl3_gemm(H.to_dev(A), H.to_dev(tr), c, H.to_dev(suh), None, H.to_dev(svh), mcg=True)
    ctx.poll_status()
    want = O.exl3_gemm(A, tr, suh, svh, K, 1, c_fp32=True)
    assert H.rel_rms_err(c.cpu().numpy(), want) < 2e-3
