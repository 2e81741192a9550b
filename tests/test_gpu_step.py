"""The whole decode step through exl3_step_forward on a small synthetic model, against the oracle composition of the
same ops: device-built descriptors, packed ragged batch, greedy tokens."""
import ctypes as C

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu


def _setup(kv_bits, K, cb, q_lens, ctx_lens, seed, n_layers=2, vocab=2048):
    import torch
    from exl3b200.step import SyntheticModel
    from oracle import oracle_model
    r = H.rng(seed)
    q_lens = np.asarray(q_lens, np.int32); ctx_lens = np.asarray(ctx_lens, np.int32)
    bt, pages = H.make_paged(r, len(q_lens), ctx_lens + q_lens, 8, 128)
    model = SyntheticModel(n_layers, 1024, 16, 8, 128, 3072, vocab, K=K, cb=cb, pages=pages, kv_bits=kv_bits, seed=seed)
    if kv_bits == 0:
        model.fill_kv()
    ids = r.integers(0, vocab, int(q_lens.sum())).astype(np.int64)
    return model, oracle_model.model_to_numpy(model), ids, q_lens, ctx_lens, bt


def test_build_descriptors(ctx):
    import torch
    from exl3b200 import lib
    q_lens = np.array([1, 8, 0, 256, 1], np.int32); seqlens = np.array([5, 100, 7, 512, 0], np.int32)
    rows = int(q_lens.sum())
    cu = torch.zeros(6, dtype=torch.int32, device="cuda"); pos = torch.zeros(rows, dtype=torch.int32, device="cuda")
    last = torch.zeros(5, dtype=torch.int32, device="cuda")
    dq, dsl = H.to_dev(q_lens), H.to_dev(seqlens)       # named: a temporary's memory would be reused at once
    rc = lib().exl3_step_build_descriptors(ctx.handle, ctx.stream(), H.ptr(dq), H.ptr(dsl), 5, rows, H.ptr(cu),
                                           H.ptr(pos), H.ptr(last))
    assert rc == 0
    wcu = np.concatenate([[0], np.cumsum(q_lens)])
    assert np.array_equal(cu.cpu().numpy(), wcu)
    wpos = np.concatenate([seqlens[b] + np.arange(q_lens[b]) for b in range(5)])
    assert np.array_equal(pos.cpu().numpy(), wpos)
    assert np.array_equal(last.cpu().numpy(), [0, 8, -1, 264, 265])


@pytest.mark.parametrize("kv_bits,K,cb", [(0, 8, 0), (0, 4, 1), (4, 4, 2)])
def test_decode_step_matches_oracle(ctx, kv_bits, K, cb):
    """Op-level reference workload: 8 decode sequences with contexts in [64, 1024] on a 0.6B-shaped layer stack."""
    from oracle import oracle_model
    r = H.rng(40 + K)
    ctx_lens = r.integers(64, 1025, 8)
    model, nm, ids, q_lens, ctx_lens, bt = _setup(kv_bits, K, cb, [1] * 8, ctx_lens, 17 + K)
    dsl = H.to_dev(ctx_lens)
    tok, logits = model.step(ctx, H.to_dev(ids), H.to_dev(q_lens), dsl, H.to_dev(bt), 1, advance=True, want_logits=True)
    ctx.poll_status()
    wtok, wlog = oracle_model.step(nm, ids, q_lens, ctx_lens, bt)
    got = logits.cpu().numpy()
    tol = 2e-2 if kv_bits else 1e-2        # a whole 2-layer stack of fp16 ops; single ops are checked at 2e-3 elsewhere
    assert H.rel_rms_err(got, wlog) < tol
    assert np.array_equal(tok.cpu().numpy(), wtok)
    assert np.array_equal(dsl.cpu().numpy(), ctx_lens + 1)


def test_ragged_step_equals_sequence_by_sequence(ctx):
    """A packed ragged step (decode + verify + prefill chunk) gives the same tokens as one call per sequence."""
    from oracle import oracle_model
    q_lens = [1, 8, 256, 1, 40]
    ctx_lens = [300, 1000, 512, 64, 0]
    model, nm, ids, q_lens, ctx_lens, bt = _setup(0, 4, 1, q_lens, ctx_lens, 99, n_layers=1)
    pools0 = [(L["k_cache"].clone(), L["v_cache"].clone()) for L in model.layers]
    tok, logits = model.step(ctx, H.to_dev(ids), H.to_dev(q_lens), H.to_dev(ctx_lens), H.to_dev(bt), int(q_lens.max()),
                             want_logits=True)
    ctx.poll_status()
    got = logits.cpu().numpy()
    wtok, wlog = oracle_model.step(nm, ids, q_lens, ctx_lens, bt)
    assert H.rel_rms_err(got, wlog) < 1e-2
    assert np.array_equal(tok.cpu().numpy(), wtok)
    # sequence by sequence on fresh pools
    for L, (k0, v0) in zip(model.layers, pools0):
        L["k_cache"].copy_(k0); L["v_cache"].copy_(v0)
    cu = np.concatenate([[0], np.cumsum(q_lens)])
    for b in range(len(q_lens)):
        t1, l1 = model.step(ctx, H.to_dev(ids[cu[b]:cu[b + 1]]), H.to_dev(q_lens[b:b + 1]), H.to_dev(ctx_lens[b:b + 1]),
                            H.to_dev(bt[b:b + 1]), int(q_lens[b]), want_logits=True)
        assert H.rel_rms_err(l1.cpu().numpy()[0], got[b]) < 5e-3
        assert int(t1[0]) == int(tok[b])


def test_fused_input_transform_equals_separate_launches(ctx):
    """From 128 rows on the norm and activation kernels of the step write the tensor-core GEMM's transformed activations
    themselves.  The fp32 butterflies run in another order than in the separate transform launch (shuffles against two
    small tensor-core products), so a transformed activation that sits on an fp16 rounding boundary may come out one
    step apart, and every later fp16 rounding of that row can then fall the other way: per sequence the two paths are
    either bit-identical or 3e-4 .. 9e-4 of the logits' RMS apart, each 9e-4 .. 1.1e-3 from the oracle.  Bars: 5e-3
    between the two, 1e-2 against the oracle for both."""
    import os
    import exl3b200
    from oracle import oracle_model
    q_lens = [1, 8, 256, 1, 40]
    ctx_lens = [300, 1000, 512, 64, 0]
    model, nm, ids, q_lens, ctx_lens, bt = _setup(0, 4, 1, q_lens, ctx_lens, 123, n_layers=2)
    pools0 = [(L["k_cache"].clone(), L["v_cache"].clone()) for L in model.layers]
    args = lambda: (H.to_dev(ids), H.to_dev(q_lens), H.to_dev(ctx_lens), H.to_dev(bt), int(q_lens.max()))  # noqa: E731
    n0 = ctx.launch_count()
    tok, logits = model.step(ctx, *args(), want_logits=True)
    fused_launches = ctx.launch_count() - n0
    ctx.poll_status()
    os.environ["EXL3_B200_NO_FUSED_TRANSFORM"] = "1"
    try:
        ctx2 = exl3b200.Ctx(0)
    finally:
        del os.environ["EXL3_B200_NO_FUSED_TRANSFORM"]
    for L, (k0, v0) in zip(model.layers, pools0):
        L["k_cache"].copy_(k0); L["v_cache"].copy_(v0)
    n0 = ctx2.launch_count()
    tok2, logits2 = model.step(ctx2, *args(), want_logits=True)
    plain_launches = ctx2.launch_count() - n0
    ctx2.poll_status()
    err = H.rel_rms_err(logits.cpu().numpy(), logits2.cpu().numpy())
    print(f"fused vs separate: relative RMS difference {err:.2e}")
    assert err < 5e-3
    wtok, wlog = oracle_model.step(nm, ids, q_lens, ctx_lens, bt)
    assert H.rel_rms_err(logits.cpu().numpy(), wlog) < 1e-2 and H.rel_rms_err(logits2.cpu().numpy(), wlog) < 1e-2
    assert np.array_equal(tok.cpu().numpy(), wtok)
    assert np.array_equal(tok.cpu().numpy(), tok2.cpu().numpy())
    assert fused_launches == plain_launches - 3 * 2           # three transform launches fewer per layer


def test_stage_profile(ctx):
    """The step runner's per-stage timer: off by default, sums device time per stage over the profiled steps, leaves the
    step's results alone and stays out of a graph capture."""
    import exl3b200
    model, nm, ids, q_lens, ctx_lens, bt = _setup(0, 4, 1, [1, 8, 40], [300, 100, 0], 321, n_layers=2)
    args = lambda: (H.to_dev(ids), H.to_dev(q_lens), H.to_dev(ctx_lens), H.to_dev(bt), int(q_lens.max()))  # noqa: E731
    pools0 = [(L["k_cache"].clone(), L["v_cache"].clone()) for L in model.layers]
    tok0, lg0 = model.step(ctx, *args(), want_logits=True)
    times, steps = ctx.stage_times(reset=True)
    assert steps == 0 and all(v == 0.0 for v in times.values())
    ctx.stage_profile(True)
    try:
        for _ in range(3):
            for L, (k0, v0) in zip(model.layers, pools0):
                L["k_cache"].copy_(k0); L["v_cache"].copy_(v0)
            tok1, lg1 = model.step(ctx, *args(), want_logits=True)
        times, steps = ctx.stage_times(reset=True)
        assert steps == 3
        assert set(times) == set(ctx.STAGES) and all(v > 0.0 for v in times.values())
        assert lg1.cpu().numpy().tobytes() == lg0.cpu().numpy().tobytes()
        assert np.array_equal(tok1.cpu().numpy(), tok0.cpu().numpy())
        # a captured step records nothing
        g = exl3b200.CudaGraph(ctx)
        import torch
        tok_static = torch.empty(len(q_lens), dtype=torch.int64, device="cuda")
        a = args()
        g.capture_begin()
        model.step(ctx, *a, stream=g.side_stream(), tokens_out=tok_static)
        g.capture_end()
        g.replay()
        torch.cuda.synchronize()
        _, steps = ctx.stage_times(reset=True)
        assert steps == 0
    finally:
        ctx.stage_profile(False)
    ctx.poll_status()


@pytest.mark.parametrize("kv_bits", [0, 4])
def test_multi_step_greedy_generation_with_page_allocator(ctx, kv_bits):
    """A continuous batch over many steps: ragged prefill of four prompts, then 20 greedy decode steps, on pools and pages
    handed out by the library's page table.  Two sequences cross a 256-token page boundary on the way (a page is
    allocated when a sequence reaches it).  The oracle composition runs the same greedy loop on its own pools.  At every
    step the device's logits must match the oracle's and its greedy tokens must be the oracle's; where the oracle's two
    best logits are closer than the fp16 noise of a two-layer stack (a coin flip on either side) the oracle's second
    choice is accepted too.  Both loops continue with the oracle's token, so their caches stay comparable."""
    import torch
    import exl3b200
    from exl3b200.step import SyntheticModel
    from oracle import oracle_model
    n_layers, vocab, steps = 2, 2048, 20
    prompts_len = [250, 40, 100, 511]
    bsz, pps, seed = len(prompts_len), 4, 7
    pool = exl3b200.Pool(0, n_layers, 16, 8, 128, kv_bits, kv_bits)
    model = SyntheticModel(n_layers, 1024, 16, 8, 128, 3072, vocab, K=4, cb=1, pages=16, kv_bits=kv_bits, seed=seed, pool=pool)
    nm = oracle_model.model_to_numpy(model)
    r = H.rng(seed)
    prompts = [r.integers(0, vocab, n).astype(np.int64) for n in prompts_len]
    blocks = [pool.alloc_prefix(p, 1)[0] for p in prompts]           # room for the prompt and the first new token
    assert [len(b) for b in blocks] == [1, 1, 1, 2]
    d_sl = torch.zeros(bsz, dtype=torch.int32, device="cuda")
    lens = np.zeros(bsz, np.int32)
    ids, q_lens = np.concatenate(prompts), np.array(prompts_len, np.int32)
    # logits of a 2-layer stack; with 4-bit KV a prefill chunk attends to its own freshly quantised keys, and the two
    # sides' codes differ at rounding ties in a fraction of a percent of the groups
    tol = 3e-2 if kv_bits else 1e-2
    exact, ties = 0, 0
    for step in range(steps + 1):
        for b in range(bsz):                                         # a page for the last position this step writes
            while (lens[b] + q_lens[b] + 255) // 256 > len(blocks[b]):
                blocks[b] += pool.alloc(1)
        bt = np.zeros((bsz, pps), np.int32)
        for b, blk in enumerate(blocks):
            bt[b, :len(blk)] = blk
        wtok, wlog = oracle_model.step(nm, ids, q_lens, lens, bt)
        tok, logits = model.step(ctx, H.to_dev(ids), H.to_dev(q_lens), d_sl, H.to_dev(bt), int(q_lens.max()), advance=True,
                                 want_logits=True)
        ctx.poll_status()
        got, glog = tok.cpu().numpy(), logits.cpu().numpy()
        assert H.rel_rms_err(glog, wlog) < tol, f"step {step}"
        order = np.argsort(wlog, axis=1)
        for b in range(bsz):
            gap = (wlog[b, order[b, -1]] - wlog[b, order[b, -2]]) / wlog[b].std()
            if got[b] == wtok[b]:
                exact += 1
            else:
                assert gap < 2 * tol and got[b] == order[b, -2], f"step {step} sequence {b}: {got[b]} vs {wtok[b]}, gap {gap:.4f}"
                ties += 1
        lens = lens + q_lens
        assert np.array_equal(d_sl.cpu().numpy(), lens)
        ids, q_lens = wtok.astype(np.int64), np.ones(bsz, np.int32)
    assert exact >= (steps + 1) * bsz - 4, f"{ties} of {(steps + 1) * bsz} tokens fell on near-ties"
    assert lens.tolist() == [p + steps + 1 - 1 for p in prompts_len] and len(blocks[0]) == 2 and len(blocks[3]) == 3
    assert pool.num_free() == 16 - sum(len(b) for b in blocks)
    for blk in blocks:
        pool.release(blk)
    assert pool.num_free() == 16
    pool.close()
