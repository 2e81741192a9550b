"""Generate the golden fixtures in this folder by running the REFERENCE's own CUDA ops.

Needs a GPU and oracle/_ref/libexl3ref.so (built by `make -C oracle ref` from the reference checkout).  Inputs are
regenerated from fixed seeds by `cases.py` (shared with the tests); only the reference outputs are stored, as
`golden_ref.npz`.  Usage:  python tests/golden/make_golden.py <output-dir>
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from tests import helpers as H          # noqa: E402
from tests.golden import cases           # noqa: E402


def main(out_dir):
    ref = H.load_ref()
    assert ref is not None, "reference library missing"
    out = {}
    keep = []   # every device tensor stays referenced: a temporary's memory would be reused by the next allocation

    def dev(a):
        keep.append(H.to_dev(a))
        return keep[-1]

    p = H.ptr
    for name, c in cases.reconstruct_cases():
        o = torch.empty(c["k"], c["n"], dtype=torch.float16, device="cuda")
        assert ref.ref_reconstruct(p(o), p(dev(c["trellis"])), c["k"], c["n"], c["K"], int(c["cb"] == 1), int(c["cb"] == 2)) == 0
        out[name] = o.cpu().numpy()
    for name, c in cases.gemm_cases():
        m, k, n = c["A"].shape[0], c["A"].shape[1], c["n"]
        o = torch.zeros(m, n, dtype=torch.float16, device="cuda")
        ah = torch.empty(m, k, dtype=torch.float16, device="cuda")
        # force_shape_idx = 2 selects the reference's fp32-accumulating cooperative kernel without its timing autotuner
        tag = ref.ref_exl3_gemm(p(dev(c["A"])), p(dev(c["trellis"])), p(o), p(dev(c["suh"])), p(ah), p(dev(c["svh"])), m, k, n,
                                c["K"], 0, int(c["cb"] == 1), int(c["cb"] == 2), 2)
        torch.cuda.synchronize()
        assert tag >= 0, tag
        out[name] = o.cpu().numpy()
    for name, c in cases.had_cases():
        x = dev(c["x"]); y = torch.empty_like(x)
        sc = dev(c["scale"])
        assert ref.ref_had_r_128(p(x), p(y), p(sc if c["mode"] == "pre" else None), p(sc if c["mode"] == "post" else None),
                                 C.c_float(1.0), c["x"].shape[0], c["x"].shape[1], 0) == 0
        out[name] = y.cpu().numpy()
    for name, c in cases.norm_cases():
        x = dev(c["x"]); y = torch.empty(c["x"].shape, dtype=torch.float16, device="cuda")
        r = dev(c["res"])
        assert ref.ref_rms_norm_res_in(p(x), 0, p(dev(c["w"])), p(y), 0, p(r), 1, C.c_float(1e-6), C.c_float(0.0),
                                       C.c_float(1.0), c["x"].shape[0], c["x"].shape[1]) == 0
        out[name + "_y"] = y.cpu().numpy(); out[name + "_r"] = r.cpu().numpy()
    for name, c in cases.rope_cases():
        q, k = dev(c["q"]), dev(c["k"])
        bsz, seq, nq, hd = c["q"].shape
        assert ref.ref_rope(p(q), p(k), p(dev(c["inv_freq"])), c["inv_freq"].size, 0, p(dev(c["positions"])),
                            p(dev(c["q_norm"])), p(dev(c["k_norm"])), C.c_float(1e-6), C.c_float(0.0), 2, C.c_float(1.0),
                            bsz, seq, nq, c["k"].shape[2], hd) == 0
        out[name + "_q"] = q.cpu().numpy(); out[name + "_k"] = k.cpu().numpy()
    for name, c in cases.silu_cases():
        x, y = dev(c["x"]), dev(c["y"]); z = torch.empty_like(x)
        assert ref.ref_silu_mul(p(x), p(y), p(z), C.c_int64(c["x"].shape[0]), C.c_int64(c["x"].shape[1])) == 0
        out[name] = z.cpu().numpy()
    for name, c in cases.kvquant_cases():
        bits, nkv, hd = c["bits"], c["nkv"], c["hd"]
        groups = nkv * hd // 32
        pages = c["pages"]
        qk = torch.zeros(pages, 256, groups * bits, dtype=torch.int32, device="cuda"); qv = torch.zeros_like(qk)
        sk = torch.zeros(pages, 256, groups, dtype=torch.float16, device="cuda"); sv = torch.zeros_like(sk)
        bsz, seq = c["k"].shape[:2]
        dbt, dsl = dev(c["block_table"]), dev(c["seqlens"])
        assert ref.ref_quant_cache_paged(p(dev(c["k"])), p(qk), p(sk), p(dev(c["v"])), p(qv), p(sv), p(dsl), p(dbt), bsz,
                                         seq, nkv, hd, pages, c["block_table"].shape[1], bits, bits) == 0
        ko = torch.zeros(pages, 256, nkv, hd, dtype=torch.float16, device="cuda"); vo = torch.zeros_like(ko)
        dnl = dev((c["seqlens"] + seq).astype(np.int32))
        assert ref.ref_dequant_cache_paged(p(qk), p(sk), p(ko), p(qv), p(sv), p(vo), p(dnl), p(dbt), bsz, nkv, hd, pages,
                                           pages, c["block_table"].shape[1], bits, bits, 0, 0) == 0
        torch.cuda.synchronize()
        out[name + "_qk"] = qk.cpu().numpy(); out[name + "_sk"] = sk.cpu().numpy()
        # the rows written, dequantised (bsz*seq rows)
        rows = []
        g = ko.cpu().numpy()
        for b in range(bsz):
            for s in range(seq):
                pos = int(c["seqlens"][b]) + s
                rows.append(g[c["block_table"][b, pos // 256], pos % 256].reshape(-1))
        out[name + "_deq"] = np.stack(rows)
    for name, c in cases.attn_cases():
        bsz, q_len, nq, hd = c["q"].shape
        nkv = c["kc"].shape[2]
        pages = c["kc"].shape[0]
        for mma in (0, 1):
            if mma == 1 and q_len == 1:
                continue
            ref.ref_set_mma_attn(mma)
            kc, vc = dev(c["kc"]), dev(c["vc"])
            o = torch.zeros(bsz, q_len, nq, hd, dtype=torch.float16, device="cuda")
            assert ref.ref_bighead_attn_paged(p(dev(c["q"])), p(dev(c["k"])), p(dev(c["v"])), p(kc), p(vc),
                                              p(dev(c["block_table"])), p(dev(c["seqlens"])), p(o), bsz, q_len, q_len, nq,
                                              nkv, hd, pages, c["block_table"].shape[1], 256, 1, C.c_float(0.0)) == 0
            torch.cuda.synchronize()
            out[f"{name}_mma{mma}"] = o.cpu().numpy()
    os.makedirs(out_dir, exist_ok=True)
    np.savez_compressed(os.path.join(out_dir, "golden_ref.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
