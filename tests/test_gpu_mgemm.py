"""exl3_mgemm (src/ffi.rs:28-42): products over a device table of EXL3 tensors chosen by device-resident indices, with the
optional weighted sum per token.  Checked against the oracle composition and, when it was built, the reference's own
exl3_mgemm op."""
import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu

GEMM_TOL = 2e-3


def _table(r, num_mats, k, n, K):
    import torch
    tr = [H.rand_trellis(r, k, n, K) for _ in range(num_mats)]
    suh = [H.rand_signs(r, k) for _ in range(num_mats)]
    svh = [H.rand_signs(r, n) for _ in range(num_mats)]
    dev = {"tr": [H.to_dev(t) for t in tr], "suh": [H.to_dev(t) for t in suh], "svh": [H.to_dev(t) for t in svh]}
    tabs = {key: torch.tensor([t.data_ptr() for t in dev[key]], dtype=torch.int64, device="cuda") for key in dev}
    return tr, suh, svh, dev, tabs


CASES = [
    # num_mats, bszm_in, bszm_out, m, k, n, K, cb, fp32, indices, weights, num_tokens
    (8, 1, 4, 1, 1024, 512, 4, 1, False, [5, 0, 7, 2], True, 1),          # one token routed to 4 of 8 experts
    (8, 1, 4, 1, 1024, 512, 4, 1, True, [5, -1, 7, 2], True, 1),          # one slot switched off
    (4, 4, 4, 3, 512, 384, 3, 0, False, None, False, 1),                  # plain batch: slot j uses tensor j
    (6, 8, 8, 2, 640, 256, 5, 2, False, [1, 3, -1, 0, 5, 5, 2, -1], True, 2),   # two tokens, four slots each
    (6, 8, 8, 1, 640, 256, 2, 1, True, [1, 3, 4, 0, 5, 5, 2, 1], True, 4),      # four tokens, two slots each
    (3, 1, 3, 9, 768, 256, 8, 1, False, [2, 2, 0], False, 1),             # 9 rows: the 16-row form of the kernel
    (3, 3, 3, 20, 512, 256, 4, 1, False, [0, -1, 1], False, 1),           # more than 16 rows: two passes
    (2, 1, 2, 1, 5120, 1024, 4, 1, False, [1, 0], True, 1),               # a model-sized reduction dimension
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"mats{c[0]}_in{c[1]}_out{c[2]}_m{c[3]}_K{c[6]}_cb{c[7]}_tok{c[11]}")
def test_mgemm_matches_oracle_and_reference(ctx, ref, case):
    import torch
    from oracle import oracle as O
    num_mats, bszm_in, bszm_out, m, k, n, K, cb, fp32, indices, use_w, num_tokens = case
    r = H.rng(sum(case[:8]))
    tr, suh, svh, dev, tabs = _table(r, num_mats, k, n, K)
    bszm = max(bszm_in, bszm_out)
    A = r.standard_normal((bszm_in, m, k)).astype(np.float16)
    w = (r.random(bszm) * 0.5 + 0.1).astype(np.float16) if use_w else None
    dt = torch.float32 if fp32 else torch.float16
    sentinel = r.standard_normal((bszm_out, m, n)).astype(np.float32 if fp32 else np.float16)
    dC = H.to_dev(sentinel.copy())
    dA = H.to_dev(A)
    di = None if indices is None else H.to_dev(np.array(indices, np.int64))
    dw = None if w is None else H.to_dev(w)
    ctx.exl3_mgemm(dA, tabs["tr"], dC, tabs["suh"], tabs["svh"], K, indices=di, weights=dw, mcg=cb == 1, mul1=cb == 2,
                   num_tokens=num_tokens)
    ctx.poll_status()
    got = dC.float().cpu().numpy()
    want = O.exl3_mgemm(A, tr, suh, svh, sentinel, K, cb, indices=indices, weights=w, num_tokens=num_tokens).astype(np.float32)
    assert np.isfinite(got).all()
    stride = bszm // num_tokens
    steps = 1 + (stride if use_w else 0)                       # fp16 sums of several rounded terms
    tol = GEMM_TOL * (np.sqrt(stride) if use_w else 1.0)       # ... each of which carries the single product's error
    for j in range(bszm_out):
        skipped = indices is not None and indices[j] < 0
        if skipped and not (use_w and j < num_tokens):
            assert np.array_equal(got[j], sentinel[j].astype(np.float32)), f"slot {j} is switched off and must stay untouched"
            continue
        err = H.gemm_mismatch(got[j], want[j], tol, not fp32, steps=steps)
        assert err <= 1.0, f"slot {j} vs oracle: {err} x the allowed difference"
    if ref is not None and hasattr(ref, "ref_exl3_mgemm"):
        C2 = H.to_dev(sentinel.copy())
        ah = torch.empty(bszm, m, k, dtype=torch.float16, device="cuda")
        tag = ref.ref_exl3_mgemm(H.ptr(dA), H.ptr(tabs["tr"]), H.ptr(C2), H.ptr(tabs["suh"]), H.ptr(ah), H.ptr(tabs["svh"]),
                                 H.ptr(di), H.ptr(dw), num_mats, bszm_in, bszm_out, m, k, n, K, int(fp32), int(cb == 1),
                                 int(cb == 2), num_tokens)
        torch.cuda.synchronize()
        assert tag >= 0, tag
        theirs = C2.float().cpu().numpy()
        rows = range(num_tokens) if use_w else [j for j in range(bszm_out) if indices is None or indices[j] >= 0]
        for j in rows:
            err = H.gemm_mismatch(got[j], theirs[j], 1.5 * tol, not fp32, steps=steps + 1)
            assert err <= 1.0, f"slot {j} vs reference CUDA op: {err} x the allowed difference"


def test_mgemm_rejects_bad_arguments(ctx):
    import torch
    import exl3b200
    r = H.rng(3)
    tr, suh, svh, dev, tabs = _table(r, 2, 256, 128, 4)
    a = torch.zeros(3, 1, 256, dtype=torch.float16, device="cuda")
    c = torch.zeros(4, 1, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(exl3b200.Exl3Error):          # three input slots for four output slots
        ctx.exl3_mgemm(a, tabs["tr"], c, tabs["suh"], tabs["svh"], 4)
    a = torch.zeros(1, 1, 256, dtype=torch.float16, device="cuda")
    w = torch.ones(4, dtype=torch.float16, device="cuda")
    with pytest.raises(exl3b200.Exl3Error):          # four slots do not divide among three tokens
        ctx.exl3_mgemm(a, tabs["tr"], c, tabs["suh"], tabs["svh"], 4, weights=w, num_tokens=3)
