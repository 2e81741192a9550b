"""Seeded inputs of the golden cases.  make_golden.py feeds them to the reference's CUDA ops and stores the outputs in
golden_ref.npz; the CPU tests feed the same inputs to the oracle and the GPU tests to this repository's kernels."""
import numpy as np


def _rng(seed):
    return np.random.default_rng(seed)


def _trellis(r, k, n, K):
    return r.integers(-32768, 32768, size=(k // 16, n // 16, 16 * K), dtype=np.int16)


def _signs(r, n):
    return (r.integers(0, 2, n) * 2 - 1).astype(np.float16)


def reconstruct_cases():
    for cb in range(3):
        for K in range(1, 9):
            r = _rng(1000 + cb * 8 + K)
            yield f"recon_K{K}_cb{cb}", dict(k=32, n=128, K=K, cb=cb, trellis=_trellis(r, 32, 128, K))


def gemm_cases():
    for cb in range(3):
        for K in (2, 3, 4, 5, 8):
            r = _rng(2000 + cb * 8 + K)
            k, n, m = 256, 256, 3
            yield f"gemm_K{K}_cb{cb}", dict(A=r.standard_normal((m, k)).astype(np.float16), n=n, K=K, cb=cb,
                                             trellis=_trellis(r, k, n, K), suh=_signs(r, k), svh=_signs(r, n))


def had_cases():
    for mode in ("plain", "pre", "post"):
        r = _rng(3000 + len(mode))
        yield f"had_{mode}", dict(x=r.standard_normal((3, 256)).astype(np.float16), mode=mode,
                                  scale=(_signs(r, 256) * np.float16(1.25)))


def norm_cases():
    r = _rng(4000)
    yield "norm_res_in", dict(x=r.standard_normal((4, 1024)).astype(np.float16),
                              res=r.standard_normal((4, 1024)).astype(np.float32),
                              w=(1 + 0.1 * r.standard_normal(1024)).astype(np.float16))


def rope_cases():
    r = _rng(5000)
    hd = 128
    yield "rope_neox_norm", dict(q=r.standard_normal((2, 3, 4, hd)).astype(np.float16),
                                 k=r.standard_normal((2, 3, 2, hd)).astype(np.float16),
                                 inv_freq=(1.0 / (10000.0 ** (np.arange(0, hd, 2) / hd))).astype(np.float32),
                                 positions=np.array([5, 300], np.int32),
                                 q_norm=(1 + 0.1 * r.standard_normal(hd)).astype(np.float16),
                                 k_norm=(1 + 0.1 * r.standard_normal(hd)).astype(np.float16))


def silu_cases():
    r = _rng(6000)
    yield "silu_mul", dict(x=(3 * r.standard_normal((4, 512))).astype(np.float16),
                           y=r.standard_normal((4, 512)).astype(np.float16))


def _paged(r, ctx_lens, append, extra=2):
    need = [(int(c) + append + 255) // 256 for c in ctx_lens]
    pps = max(max(need), 1)
    total = sum(need) + extra
    perm = r.permutation(total).astype(np.int32)
    bt = np.zeros((len(ctx_lens), pps), np.int32)
    o = 0
    for b, nd in enumerate(need):
        bt[b, :nd] = perm[o:o + nd]
        o += nd
    return bt, total


def kvquant_cases():
    for bits in (2, 3, 4, 5, 6, 7, 8):
        r = _rng(7000 + bits)
        nkv, hd, seq = 2, 128, 2
        seqlens = np.array([0, 255, 300], np.int32)
        bt, pages = _paged(r, seqlens, seq)
        yield f"kvq_b{bits}", dict(bits=bits, nkv=nkv, hd=hd, pages=pages, block_table=bt, seqlens=seqlens,
                                   k=(0.5 * r.standard_normal((3, seq, nkv, hd))).astype(np.float16),
                                   v=(0.5 * r.standard_normal((3, seq, nkv, hd))).astype(np.float16))


def attn_cases():
    """(name, q_len, nq, nkv, context lengths before the append)"""
    specs = [("attn_dec_g5", 1, 10, 2, [0, 40, 255, 256, 700]),
             ("attn_dec_g2", 1, 4, 2, [3, 513]),
             ("attn_ver_g5", 8, 10, 2, [0, 100, 600]),
             ("attn_pre_g2", 40, 4, 2, [0, 250])]
    for i, (name, q_len, nq, nkv, ctx) in enumerate(specs):
        r = _rng(8000 + i)
        hd = 128
        seqlens = np.array(ctx, np.int32)
        bt, pages = _paged(r, seqlens, q_len)
        bsz = len(ctx)
        yield name, dict(q=r.standard_normal((bsz, q_len, nq, hd)).astype(np.float16),
                         k=(0.5 * r.standard_normal((bsz, q_len, nkv, hd))).astype(np.float16),
                         v=(0.5 * r.standard_normal((bsz, q_len, nkv, hd))).astype(np.float16),
                         kc=(0.5 * r.standard_normal((pages, 256, nkv, hd))).astype(np.float16),
                         vc=(0.5 * r.standard_normal((pages, 256, nkv, hd))).astype(np.float16),
                         block_table=bt, seqlens=seqlens)
