"""GPU parity at the shapes the benchmark configurations name, through the C-ABI, against the reference's own CUDA ops
(when that library was built) and the CPU oracle:

  * EXL3 GEMM sweep: K = 5120, N = 17408, bits in {2,3,4,5,8}, M in {256, 2048} and the step's M = 1052;
  * paged attention alone: 64 sequences, contexts log-uniform in [128, 32768], 40 q / 8 kv heads, one query row, fp16 pools
    and 4-bit pools built by the quantiser;
  * the verify shape: 4 sequences x 8 draft rows, GQA 5, 4-bit KV, contexts up to 32768.

Inputs are seeded and generated on the device (the tensors are large); the oracle is run on a seeded subset that it
finishes in seconds (whole 128-column blocks of the GEMM, whole sequences of the attention)."""
import ctypes as C

import numpy as np
import pytest

from tests import helpers as H

pytestmark = pytest.mark.gpu
GEMM_TOL = 2e-3
TOL_FP16 = 2e-3
TOL_QUANT = 1e-2


def _torch():
    import torch
    return torch


def _gen(seed):
    torch = _torch()
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return g


@pytest.mark.parametrize("m,K", [(256, 2), (256, 3), (256, 4), (256, 5), (256, 8), (2048, 2), (2048, 3), (2048, 4), (2048, 5),
                                 (2048, 8), (1052, 4)])
def test_gemm_sweep_large_m(ctx, ref, m, K):
    from oracle import oracle as O
    torch = _torch()
    k, n = 5120, 17408
    g = _gen(2000 + m + K)
    tr = torch.randint(-32768, 32768, (k // 16, n // 16, 16 * K), dtype=torch.int16, device="cuda", generator=g)
    suh = (torch.randint(0, 2, (k,), device="cuda", generator=g) * 2 - 1).to(torch.float16)
    svh = (torch.randint(0, 2, (n,), device="cuda", generator=g) * 2 - 1).to(torch.float16)
    A = torch.randn(m, k, device="cuda", generator=g).to(torch.float16)
    out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    ctx.exl3_gemm(A, tr, out, suh, None, svh, mcg=True)
    ctx.poll_status()
    assert torch.isfinite(out).all()
    # oracle on two seeded 128-column blocks (the product has no terms across blocks)
    hA, hsuh = A.cpu().numpy(), suh.cpu().numpy()
    for nb in H.rng(m + K).choice(n // 128, size=2, replace=False):
        nb = int(nb)
        sub = np.ascontiguousarray(tr[:, nb * 8:nb * 8 + 8].cpu().numpy())
        want = O.exl3_gemm(hA, sub, hsuh, svh[nb * 128:nb * 128 + 128].cpu().numpy(), K, 1, c_fp32=False).astype(np.float32)
        got = out[:, nb * 128:nb * 128 + 128].float().cpu().numpy()
        assert H.gemm_mismatch(got, want, GEMM_TOL, True) <= 1.0, f"block {nb} vs oracle"
    if ref is not None:
        C2 = torch.zeros_like(out)
        ah = torch.empty(m, k, dtype=torch.float16, device="cuda")
        tag = ref.ref_exl3_gemm(H.ptr(A), H.ptr(tr), H.ptr(C2), H.ptr(suh), H.ptr(ah), H.ptr(svh), m, k, n, K, 0, 1, 0, -1)
        torch.cuda.synchronize()
        assert tag >= 0
        # the reference's partial sums pass through its fp16 output buffer: 3e-3 * RMS or two fp16 steps against it
        worst = 0.0
        for r0 in range(0, m, 256):
            worst = max(worst, H.gemm_mismatch(out[r0:r0 + 256].float().cpu().numpy(), C2[r0:r0 + 256].float().cpu().numpy(),
                                               1.5 * GEMM_TOL, True, steps=2))
        assert worst <= 1.0, f"vs reference CUDA op: {worst} x the allowed difference"


def _c3_batch(seed, bsz, lo, hi, q_len, pin=None):
    r = H.rng(seed)
    ctx_lens = np.exp(r.uniform(np.log(lo), np.log(hi), bsz)).astype(np.int32)
    if pin:
        for i, v in pin.items():
            ctx_lens[i] = v
    need = (ctx_lens + q_len + 255) // 256
    pages = int(need.sum()) + 2
    perm = r.permutation(pages).astype(np.int32)
    bt = np.zeros((bsz, int(need.max())), np.int32)
    o = 0
    for b in range(bsz):
        bt[b, :need[b]] = perm[o:o + need[b]]
        o += need[b]
    return ctx_lens, bt, pages


def _sub_pool(pool_t, bt, seqs):
    """compact copy of the pages of the chosen sequences: (numpy pool, remapped block table rows)"""
    pages = sorted({int(p) for b in seqs for p in bt[b]})
    remap = {p: i for i, p in enumerate(pages)}
    torch = _torch()
    sub = pool_t[torch.tensor(pages, device="cuda")].cpu().numpy()
    nbt = np.array([[remap[int(p)] for p in bt[b]] for b in seqs], np.int32)
    return sub, nbt


def test_attention_alone_64_sequences_fp16(ctx, ref):
    """the attention-alone configuration in full: 64 decode sequences, contexts log-uniform in [128, 32768]"""
    from oracle import oracle as O
    torch = _torch()
    bsz, nq, nkv, hd = 64, 40, 8, 128
    ctx_lens, bt, pages = _c3_batch(31, bsz, 128, 32768, 1, pin={0: 32767, 1: 128})
    g = _gen(32)
    kc = (torch.randn(pages, 256, nkv, hd, device="cuda", generator=g) * 0.5).to(torch.float16)
    vc = (torch.randn(pages, 256, nkv, hd, device="cuda", generator=g) * 0.5).to(torch.float16)
    q = torch.randn(bsz, 1, nq, hd, device="cuda", generator=g).to(torch.float16)
    kn = (torch.randn(bsz, 1, nkv, hd, device="cuda", generator=g) * 0.5).to(torch.float16)
    vn = (torch.randn(bsz, 1, nkv, hd, device="cuda", generator=g) * 0.5).to(torch.float16)
    kc2, vc2 = kc.clone(), vc.clone()
    dbt, dsl = H.to_dev(bt), H.to_dev(ctx_lens)
    o = torch.full(q.shape, float("nan"), dtype=torch.float16, device="cuda")
    ctx.bighead_attn_paged(q, kn, vn, kc, vc, dbt, dsl, o)
    ctx.poll_status()
    got = o.cpu().numpy()
    assert np.isfinite(got).all()
    if ref is not None:
        ref.ref_set_mma_attn(0)
        o2 = torch.zeros_like(o)
        assert ref.ref_bighead_attn_paged(H.ptr(q), H.ptr(kn), H.ptr(vn), H.ptr(kc2), H.ptr(vc2), H.ptr(dbt), H.ptr(dsl), H.ptr(o2),
                                          bsz, 1, 1, nq, nkv, hd, pages, bt.shape[1], 256, 1, C.c_float(0.0)) == 0
        torch.cuda.synchronize()
        assert torch.equal(kc, kc2) and torch.equal(vc, vc2), "appended rows land in the same places"
    # oracle on the longest, the shortest and two more sequences
    seqs = [0, 1, 17, 40]
    sk, nbt = _sub_pool(kc, bt, seqs)
    sv, _ = _sub_pool(vc, bt, seqs)
    want = O.attn_paged(q.cpu().numpy()[seqs], sk, sv, nbt, ctx_lens[seqs], kv_append=1)
    e_or = H.gemm_mismatch(got[seqs], want, TOL_FP16, True)
    assert e_or <= 1.0, e_or
    if ref is not None:
        # the two kernels round differently (ours rounds the softmax weights to fp16 for the tensor core, the reference's
        # decode kernel keeps them in fp32): each is held to the bar against the exact result, and to 1.25 x the bar
        # against the other over the whole batch
        rgot = o2.cpu().numpy()
        e_rr = H.gemm_mismatch(rgot[seqs], want, TOL_FP16, True)
        e_ref = H.gemm_mismatch(got, rgot, TOL_FP16, True)
        assert e_ref <= 1.25 and e_or <= max(1.0, 1.1 * e_rr), (e_or, e_ref, e_rr)


def _quantise_context(ctx, ctx_lens, bt, pages, nkv, hd, bits, seed):
    """4-bit (or other) pools holding a seeded N(0, 0.5^2) context of ctx_lens[b] tokens per sequence, written by the
    library's quantiser (ragged form, every sequence starting at position 0)."""
    torch = _torch()
    g = _gen(seed)
    groups = nkv * hd // 32
    rows = int(ctx_lens.sum())
    k_rows = (torch.randn(rows, nkv * hd, device="cuda", generator=g) * 0.5).to(torch.float16)
    v_rows = (torch.randn(rows, nkv * hd, device="cuda", generator=g) * 0.5).to(torch.float16)
    qk = torch.zeros(pages, 256, groups * bits, dtype=torch.int32, device="cuda"); qv = torch.zeros_like(qk)
    sk = torch.zeros(pages, 256, groups, dtype=torch.float16, device="cuda"); sv = torch.zeros_like(sk)
    cu = np.concatenate([[0], np.cumsum(ctx_lens)]).astype(np.int32)
    ctx.quant_cache_paged(k_rows, qk, sk, v_rows, qv, sv, H.to_dev(np.zeros(len(ctx_lens), np.int32)), H.to_dev(bt),
                          cu_q=H.to_dev(cu), seq_len=int(ctx_lens.max()))
    ctx.poll_status()
    return qk, sk, qv, sv


def _quant_attention_case(ctx, ref, bsz, q_len, lo, hi, seed, oracle_seqs, pin=None):
    from oracle import oracle as O
    torch = _torch()
    nq, nkv, hd, bits = 40, 8, 128, 4
    ctx_lens, bt, pages = _c3_batch(seed, bsz, lo, hi, q_len, pin=pin)
    qk, sk, qv, sv = _quantise_context(ctx, ctx_lens, bt, pages, nkv, hd, bits, seed + 1)
    g = _gen(seed + 2)
    q = torch.randn(bsz, q_len, nq, hd, device="cuda", generator=g).to(torch.float16)
    kn = (torch.randn(bsz, q_len, nkv, hd, device="cuda", generator=g) * 0.5).to(torch.float16)
    vn = (torch.randn(bsz, q_len, nkv, hd, device="cuda", generator=g) * 0.5).to(torch.float16)
    pools2 = [t.clone() for t in (qk, sk, qv, sv)]
    dbt, dsl = H.to_dev(bt), H.to_dev(ctx_lens)
    o = torch.full(q.shape, float("nan"), dtype=torch.float16, device="cuda")
    ctx.bighead_attn_paged_q(q, kn, vn, qk, sk, qv, sv, dbt, dsl, o, nkv)
    ctx.poll_status()
    got = o.cpu().numpy()
    assert np.isfinite(got).all()
    if ref is not None:
        o2 = torch.zeros_like(o)
        assert ref.ref_bighead_attn_paged_q(H.ptr(q), H.ptr(kn), H.ptr(vn), *[H.ptr(x) for x in pools2], H.ptr(dbt), H.ptr(dsl),
                                            H.ptr(o2), bsz, q_len, q_len, nq, nkv, hd, pages, bt.shape[1], bits, bits, 256, 1,
                                            C.c_float(0.0)) == 0
        torch.cuda.synchronize()
        assert torch.equal(qk, pools2[0]) and torch.equal(sk, pools2[1]), "fresh rows quantise to the same codes and scales"
        assert H.gemm_mismatch(got, o2.cpu().numpy(), TOL_QUANT, True) <= 1.0
    seqs = oracle_seqs
    subs = [_sub_pool(t, bt, seqs) for t in (qk, sk, qv, sv)]
    nbt = subs[0][1]
    want = O.attn_paged(q.cpu().numpy()[seqs], None, None, nbt, ctx_lens[seqs], nkv=nkv, kv_append=q_len,
                        quant=(subs[0][0].view(np.uint32), subs[1][0], subs[2][0].view(np.uint32), subs[3][0], bits))
    assert H.gemm_mismatch(got[seqs], want, TOL_QUANT, True) <= 1.0


def test_attention_alone_64_sequences_q4(ctx, ref):
    """the 4-bit variant of the attention-alone configuration, pools written by the quantiser"""
    _quant_attention_case(ctx, ref, 64, 1, 128, 32768, 51, [0, 1, 9], pin={0: 32767, 1: 128})


def test_attention_verify_shape_q4(ctx, ref):
    """4 sequences x 8 draft rows (40 packed rows per kv head) over 4-bit contexts up to 32768 tokens"""
    _quant_attention_case(ctx, ref, 4, 8, 1024, 32768, 61, [0, 2], pin={0: 32760, 1: 1024})
