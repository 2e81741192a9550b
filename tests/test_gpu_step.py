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
