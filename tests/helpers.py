"""Shared test helpers: seeded synthetic inputs, the optional reference-op library, comparison metrics."""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libexl3ref.so")

_ref = None


def load_ref():
    """ctypes handle of the compiled reference ops, or None.  Needs torch's CUDA libraries loaded first."""
    global _ref
    if _ref is None and os.path.exists(REF_SO):
        import torch  # noqa: F401  (loads libtorch/libc10 that the reference library links against)
        os.environ.setdefault("EXL3_INT8_GEMV", "0")   # keep the reference on its fp16-activation kernels
        try:
            _ref = C.CDLL(REF_SO)
        except OSError:
            _ref = None
    return _ref


def rng(seed):
    return np.random.default_rng(seed)


def rand_trellis(r, k, n, K):
    return r.integers(-32768, 32768, size=(k // 16, n // 16, 16 * K), dtype=np.int16)


def rand_signs(r, n):
    return (r.integers(0, 2, n) * 2 - 1).astype(np.float16)


def rel_rms_err(a, b):
    """max |a-b| relative to the RMS of b (the parity metric of the reference's north star)."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / (np.sqrt((b * b).mean()) + 1e-30))


def to_dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ptr(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def make_paged(r, bsz, ctx_lens, nkv, hd, extra_pages=3, append=0):
    """Random page assignment: returns (block_table [bsz,pps] int32, pages) with a seeded permutation of the pool."""
    need = [(int(c) + append + 255) // 256 for c in ctx_lens]
    pps = max(max(need), 1)
    total = sum(need) + extra_pages
    perm = r.permutation(total).astype(np.int32)
    bt = np.zeros((bsz, pps), np.int32)
    o = 0
    for b in range(bsz):
        bt[b, :need[b]] = perm[o:o + need[b]]
        o += need[b]
    return bt, total


def fp16_ulp(x):
    """spacing of binary16 numbers at |x| (normal range)"""
    ax = np.maximum(np.abs(np.asarray(x, np.float64)), 2.0 ** -14)
    return 2.0 ** (np.floor(np.log2(ax)) - 10)


def gemm_mismatch(got, want, tol, fp16_out, steps=1):
    """Worst violation of the GEMM parity bar: |got - want| <= tol * RMS(want).  For fp16 outputs a difference of one
    fp16 rounding step of the reference value is also accepted: two correct fp32 results that straddle a rounding
    boundary differ by one step, which at |value| > 2*RMS already exceeds tol * RMS.  `steps` = 2 is used against the
    reference's CUDA GEMM, whose cross-CTA partial sums pass through the fp16 output buffer, and for multi-row
    attention, where both sides round the softmax weights to fp16 before the PV product."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    rms = np.sqrt((want * want).mean()) + 1e-30
    allowed = np.full(want.shape, tol * rms)
    if fp16_out:
        allowed = np.maximum(allowed, fp16_ulp(want) * (steps + 0.001))
    return float((np.abs(got - want) / allowed).max())


_ST_DTYPES = {"float16": "F16", "float32": "F32", "int16": "I16", "int32": "I32", "int64": "I64", "uint8": "U8", "int8": "I8"}


def write_safetensors(path, tensors, metadata=None, raw_header=None):
    """A safetensors file from {name: numpy array} (bf16 as ("BF16", uint16 array)); `raw_header` replaces the JSON text
    (for malformed-header tests) while the data section is still written."""
    import json
    import struct
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, a in tensors.items():
        dt = None
        if isinstance(a, tuple):
            dt, a = a
        a = np.ascontiguousarray(a)
        b = a.tobytes()
        header[name] = {"dtype": dt or _ST_DTYPES[a.dtype.name], "shape": list(a.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    text = (raw_header if raw_header is not None else json.dumps(header, separators=(",", ":"))).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for b in blobs:
            f.write(b)
    return header
