"""Device times of the reference's own CUDA ops (oracle/_ref/libexl3ref.so) on the shapes of `bench.py --op gemm_sweep`
and `bench.py --op attn`, for the comparison columns of the tables under profiles/.  Test infrastructure: it is the one
place outside the parity tests that runs the compiled reference ops, and nothing in the library or bench.py uses it.

    python -m tests.ref_timing gemm      # EXL3 GEMM 5120 x 17408, bits x rows
    python -m tests.ref_timing attn      # paged attention: 64 decode sequences (fp16, 4-bit), 32 x 8 verify rows

Timing: CUDA events on the current stream around `reps` back-to-back calls after warm-up (the reference's GEMM picks its
kernel shape by timing candidates on first use of a shape); weights rotate through a ring larger than L2.
"""
import ctypes as C
import json
import sys

import numpy as np

from tests import helpers as H


def _time(fn, reps, warm=6):
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / reps


def gemm(ref, reps=20):
    import torch
    g = torch.Generator(device="cuda"); g.manual_seed(5)
    k, n = 5120, 17408
    for K in (2, 3, 4, 5, 8):
        ring = max(2, min(8, int(300e6 // (k * n * K / 8)) + 1))
        ws = [torch.randint(-32768, 32768, (k // 16, n // 16, 16 * K), dtype=torch.int16, device="cuda", generator=g)
              for _ in range(ring)]
        suh = (torch.randint(0, 2, (k,), device="cuda", generator=g) * 2 - 1).to(torch.float16)
        svh = (torch.randint(0, 2, (n,), device="cuda", generator=g) * 2 - 1).to(torch.float16)
        for m in (1, 4, 16, 64, 256, 2048):
            a = torch.randn(m, k, device="cuda", generator=g).to(torch.float16)
            c = torch.empty(m, n, dtype=torch.float16, device="cuda")
            ah = torch.empty(m, k, dtype=torch.float16, device="cuda")
            state = {"i": 0}

            def call():
                w = ws[state["i"] % ring]; state["i"] += 1
                ref.ref_exl3_gemm(H.ptr(a), H.ptr(w), H.ptr(c), H.ptr(suh), H.ptr(ah), H.ptr(svh), m, k, n, K, 0, 1, 0, -1)
            t = _time(call, reps * ring // 2 if m <= 256 else reps)
            print(json.dumps({"op": "reference exl3_gemm", "m": m, "k": k, "n": n, "bits": K, "us": t * 1e6}), flush=True)
        del ws


def attn(ref, reps=20):
    import torch
    g = torch.Generator(device="cuda"); g.manual_seed(5)
    nq, nkv, hd = 40, 8, 128
    for bsz, q_len, bits in ((64, 1, 0), (64, 1, 4), (32, 8, 0), (32, 8, 4)):
        r = np.random.default_rng(3)
        ctx_lens = np.exp(r.uniform(np.log(128), np.log(32768), bsz)).astype(np.int32)
        need = (ctx_lens + q_len + 255) // 256
        pages = int(need.sum()) + 1
        perm = r.permutation(pages).astype(np.int32)
        bt = np.zeros((bsz, int(need.max())), np.int32)
        o = 0
        for b in range(bsz):
            bt[b, :need[b]] = perm[o:o + need[b]]; o += need[b]
        q = torch.randn(bsz, q_len, nq, hd, device="cuda", generator=g).to(torch.float16)
        kn = (torch.randn(bsz, q_len, nkv, hd, device="cuda", generator=g) * 0.5).to(torch.float16)
        out = torch.empty_like(q)
        dbt, dsl = torch.from_numpy(bt).cuda(), torch.from_numpy(ctx_lens).cuda()
        ref.ref_set_mma_attn(1 if q_len > 1 else 0)
        if bits:
            groups = nkv * hd // 32
            qk = torch.randint(-2 ** 31, 2 ** 31 - 1, (pages, 256, groups * bits), dtype=torch.int32, device="cuda", generator=g)
            qv = torch.randint(-2 ** 31, 2 ** 31 - 1, (pages, 256, groups * bits), dtype=torch.int32, device="cuda", generator=g)
            sk = (torch.rand(pages, 256, groups, device="cuda", generator=g) * 0.05 + 0.01).to(torch.float16)
            sv = (torch.rand(pages, 256, groups, device="cuda", generator=g) * 0.05 + 0.01).to(torch.float16)

            def call():
                ref.ref_bighead_attn_paged_q(H.ptr(q), H.ptr(kn), H.ptr(kn), H.ptr(qk), H.ptr(sk), H.ptr(qv), H.ptr(sv), H.ptr(dbt),
                                             H.ptr(dsl), H.ptr(out), bsz, q_len, q_len, nq, nkv, hd, pages, bt.shape[1], bits, bits,
                                             256, 1, C.c_float(0.0))
        else:
            kc = (torch.randn(pages, 256, nkv, hd, device="cuda", generator=g) * 0.5).to(torch.float16)
            vc = (torch.randn(pages, 256, nkv, hd, device="cuda", generator=g) * 0.5).to(torch.float16)

            def call():
                ref.ref_bighead_attn_paged(H.ptr(q), H.ptr(kn), H.ptr(kn), H.ptr(kc), H.ptr(vc), H.ptr(dbt), H.ptr(dsl), H.ptr(out),
                                           bsz, q_len, q_len, nq, nkv, hd, pages, bt.shape[1], 256, 1, C.c_float(0.0))
        t = _time(call, reps)
        print(json.dumps({"op": "reference bighead_attn_paged" + ("_q" if bits else ""), "kv_bits": bits or 16, "seqs": bsz,
                          "q_len": q_len, "us": t * 1e6}), flush=True)


if __name__ == "__main__":
    lib = H.load_ref()
    if lib is None:
        sys.exit("oracle/_ref/libexl3ref.so is not built (make -C oracle ref)")
    {"gemm": gemm, "attn": attn}[sys.argv[1]](lib)
