"""On-disk checkpoints: the safetensors header reader and its validation (host only: runs without a GPU), and on a GPU
Linear::load for an EXL3 layer and a dense layer followed by the layer's forward."""
import json
import struct

import numpy as np
import pytest

from tests import helpers as H


def _open(path):
    import exl3b200
    return exl3b200.Checkpoint(str(path))


def test_header_index(tmp_path):
    r = H.rng(1)
    tensors = {
        "model.layers.0.q_proj.trellis": r.integers(-32768, 32768, (8, 16, 64), dtype=np.int16),
        "model.layers.0.q_proj.suh": H.rand_signs(r, 128),
        "model.layers.0.q_proj.svh": H.rand_signs(r, 256),
        "model.layers.0.q_proj.mcg": np.zeros(1, np.int32),
        'odd "name"\\x': np.arange(6, dtype=np.float32).reshape(2, 3),
        "empty": np.zeros((0, 4), np.float16),
    }
    p = tmp_path / "a.safetensors"
    H.write_safetensors(p, tensors, metadata={"format": "pt", "note": "{nested: [1,2]}"})
    ck = _open(p)
    assert ck.names() == list(tensors)
    for name, a in tensors.items():
        dt, shape, nbytes = ck.info(name)
        assert shape == a.shape and nbytes == a.nbytes and dt == H._ST_DTYPES[a.dtype.name]
    assert ck.has("empty") and not ck.has("model.layers.0.q_proj.mul1") and not ck.has("__metadata__")
    ck.close()


def _raw(path, header_text, data=b"", size_field=None):
    text = header_text.encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text) if size_field is None else size_field))
        f.write(text)
        f.write(data)


@pytest.mark.parametrize("case", ["tiny", "zero_header", "huge_header", "truncated_header", "not_json", "past_end", "size_mismatch",
                                  "negative_dim", "float_dim", "reversed_offsets", "one_offset", "entry_not_object", "overflow_shape"])
def test_header_validation(tmp_path, case):
    """every field that could size a read or an allocation is checked before use (src/safetensors.rs:64-112,118-138)"""
    import exl3b200
    p = tmp_path / (case + ".safetensors")
    good = {"dtype": "F16", "shape": [2, 4], "data_offsets": [0, 16]}
    data = b"\0" * 16
    if case == "tiny":
        open(p, "wb").write(b"\1\2\3")
    elif case == "zero_header":
        _raw(p, "", size_field=0)
    elif case == "huge_header":
        _raw(p, "{}", size_field=(100 << 20) + 1)
    elif case == "truncated_header":
        _raw(p, "{}", size_field=4096)
    elif case == "not_json":
        _raw(p, "[1, 2, 3]", data)
    elif case == "entry_not_object":
        _raw(p, json.dumps({"t": [1, 2]}), data)
    else:
        e = dict(good)
        if case == "past_end":
            e["data_offsets"] = [0, 32]; e["shape"] = [4, 4]
        elif case == "size_mismatch":
            e["shape"] = [2, 5]
        elif case == "negative_dim":
            e["shape"] = [-2, -4]
        elif case == "float_dim":
            e["shape"] = [2.0, 4]
        elif case == "reversed_offsets":
            e["data_offsets"] = [16, 0]
        elif case == "one_offset":
            e["data_offsets"] = [16]
        elif case == "overflow_shape":
            e["shape"] = [1 << 40, 1 << 40, 8]          # wraps to 8 elements in 64-bit arithmetic
        _raw(p, json.dumps({"t": e}), data)
    with pytest.raises(exl3b200.Exl3Error):
        _open(p)


def test_unknown_dtype_is_indexed_but_not_sized(tmp_path):
    """the reference checks the span only for dtypes it knows (src/safetensors.rs:105-110)"""
    p = tmp_path / "u.safetensors"
    _raw(p, json.dumps({"t": {"dtype": "F4_WEIRD", "shape": [3], "data_offsets": [0, 2]}}), b"ab")
    ck = _open(p)
    assert ck.info("t") == ("F4_WEIRD", (3,), 2)


@pytest.mark.gpu
@pytest.mark.parametrize("codebook", ["3inst", "mcg", "mul1"])
def test_load_exl3_layer_and_run_it(ctx, tmp_path, codebook):
    import torch
    import exl3b200
    from oracle import oracle as O
    r = H.rng(7)
    in_f, out_f, K = 600, 500, 4                       # padded to 640 x 512
    k, n = 640, 512
    tr, suh, svh = H.rand_trellis(r, k, n, K), H.rand_signs(r, k), H.rand_signs(r, n)
    bias = (r.standard_normal(out_f) * 0.5).astype(np.float16)              # shorter than the padded width
    key = "model.layers.3.mlp.up_proj"
    tensors = {key + ".trellis": tr, key + ".suh": suh, key + ".svh": svh, key + ".bias": bias,
               "filler": r.integers(0, 255, 1000, dtype=np.uint8)}
    if codebook != "3inst":
        tensors[key + "." + codebook] = np.zeros(1, np.int32)
    p = tmp_path / "m.safetensors"
    H.write_safetensors(p, tensors)
    ck = _open(p)
    layer = ck.linear("model.layers.3.mlp.up_proj_missing", in_f, out_f, alt_key=key, trim_padded_out=True)
    cb = {"3inst": 0, "mcg": 1, "mul1": 2}[codebook]
    assert (layer.w.k, layer.w.n, layer.w.K, layer.w.cb) == (k, n, K, cb) and layer.in_unpadded == in_f and layer.out_unpadded == out_f
    x = r.standard_normal((5, in_f)).astype(np.float16)
    y = torch.full((5, out_f), float("nan"), dtype=torch.float16, device="cuda")
    ctx.linear_forward(layer, H.to_dev(x), y)
    ctx.poll_status()
    bias_p = np.concatenate([bias, np.zeros(n - out_f, np.float16)])
    want = O.linear_forward(x, K, cb, k, n, trellis=tr, suh=suh, svh=svh, bias=bias_p, out_unpadded=out_f, trim_padded_out=True)
    assert H.gemm_mismatch(y.float().cpu().numpy(), want.astype(np.float32), 2e-3, True, steps=2) <= 1.0
    # the raw tensor reads back bit for bit
    back = torch.empty(tr.shape, dtype=torch.int16, device="cuda")
    ck.read(key + ".trellis", back)
    assert np.array_equal(back.cpu().numpy(), tr)
    ck.free_linear(layer)
    assert not layer.w.trellis
    ck.close()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["F16", "BF16", "F32"])
def test_load_dense_layer_and_run_it(ctx, tmp_path, dtype):
    import torch
    from oracle import oracle as O
    r = H.rng(9)
    in_f, out_f = 200, 300                              # padded to 256 x 384
    w = (r.standard_normal((out_f, in_f)) * 0.05).astype(np.float32)         # checkpoint order [out, in]
    b = (r.standard_normal(out_f) * 0.3).astype(np.float32)
    if dtype == "F16":
        tw, tb = w.astype(np.float16), b.astype(np.float16)
        w16, b16 = tw, tb
    elif dtype == "F32":
        tw, tb = w, b
        w16, b16 = w.astype(np.float16), b.astype(np.float16)
    else:
        wb = (w.view(np.uint32) >> 16).astype(np.uint16); bb = (b.view(np.uint32) >> 16).astype(np.uint16)    # truncated bf16
        tw, tb = ("BF16", wb), ("BF16", bb)
        w16 = (wb.astype(np.uint32) << 16).view(np.float32).astype(np.float16)
        b16 = (bb.astype(np.uint32) << 16).view(np.float32).astype(np.float16)
    p = tmp_path / "d.safetensors"
    H.write_safetensors(p, {"lm_head.weight": tw, "lm_head.bias": tb})
    ck = _open(p)
    layer = ck.linear("lm_head", in_f, out_f)
    assert layer.w.k == 256 and layer.w.n == 384 and not layer.w.trellis and layer.dense
    x = r.standard_normal((3, in_f)).astype(np.float16)
    y = torch.full((3, 384), float("nan"), dtype=torch.float16, device="cuda")
    ctx.linear_forward(layer, H.to_dev(x), y)
    ctx.poll_status()
    wp = np.zeros((256, 384), np.float16); wp[:in_f, :out_f] = w16.T
    bp = np.zeros(384, np.float16); bp[:out_f] = b16
    want = O.linear_forward(x, 0, 0, 256, 384, dense=wp, bias=bp)
    got = y.float().cpu().numpy()
    assert H.gemm_mismatch(got, want.astype(np.float32), 2e-3, True, steps=2) <= 1.0
    assert (got[:, out_f:] == 0).all(), "padded output columns carry neither weight nor bias"
    ck.free_linear(layer)
    ck.close()
