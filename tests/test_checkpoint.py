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


def _dump_model(model, tmp_path, shards=2, norm_dtype="F16"):
    """The tensors of a SyntheticModel under the checkpoint's key scheme (src/model.rs:262-420), spread over `shards` files"""
    c = model.cfg
    t = {}

    def vec(x):
        a = x.cpu().numpy()
        if norm_dtype == "F32":
            return a.astype(np.float32)
        if norm_dtype == "BF16":        # these values are not bf16-exact: the loader sees the truncated ones
            return ("BF16", (a.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16))
        return a

    def lin(key, L, marker=True):
        t[key + ".trellis"] = L.trellis.cpu().numpy()
        t[key + ".suh"] = L.suh.cpu().numpy()
        t[key + ".svh"] = L.svh.cpu().numpy()
        if L.cb:
            t[key + (".mcg" if L.cb == 1 else ".mul1")] = np.zeros(1, np.int32)

    t["model.embed_tokens.weight"] = model.embed.cpu().numpy()
    for i, L in enumerate(model.layers):
        k = f"model.layers.{i}"
        t[k + ".input_layernorm.weight"] = vec(L["attn_norm"])
        t[k + ".post_attention_layernorm.weight"] = vec(L["mlp_norm"])
        if L["q_norm"] is not None:
            t[k + ".self_attn.q_norm.weight"] = vec(L["q_norm"])
            t[k + ".self_attn.k_norm.weight"] = vec(L["k_norm"])
        for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
            lin(f"{k}.self_attn.{n}", L[n])
        for n in ("gate_proj", "up_proj", "down_proj"):
            lin(f"{k}.mlp.{n}", L[n])
    t["model.norm.weight"] = vec(model.final_norm)
    lin("lm_head", model.lm_head)
    names = list(t)
    paths = []
    for s in range(shards):
        part = {n: t[n] for n in names[s::shards]}
        p = tmp_path / f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        H.write_safetensors(p, part, metadata={"format": "pt"})
        paths.append(str(p))
    return paths


@pytest.mark.gpu
@pytest.mark.parametrize("kv_bits,norm_dtype", [(0, "F16"), (4, "F32")])
def test_model_from_checkpoint_steps_like_the_model_in_memory(ctx, tmp_path, kv_bits, norm_dtype):
    """a two-layer model written to two safetensors files, read back by exl3_model_load into a pool of its own, gives the
    same tokens and logits as the in-memory model over a ragged prefill step and a decode step"""
    import torch
    import exl3b200
    from exl3b200.step import LoadedModel, SyntheticModel
    n_layers, hidden, nq, nkv, hd, inter, vocab, pages = 2, 1024, 16, 8, 128, 3072, 2048, 8
    pool_a = exl3b200.Pool(0, n_layers, pages, nkv, hd, kv_bits, kv_bits)
    pool_b = exl3b200.Pool(0, n_layers, pages, nkv, hd, kv_bits, kv_bits)
    mem = SyntheticModel(n_layers, hidden, nq, nkv, hd, inter, vocab, K=4, cb=1, pages=pages, kv_bits=kv_bits, seed=3, pool=pool_a)
    paths = _dump_model(mem, tmp_path, shards=2, norm_dtype=norm_dtype)
    disk = LoadedModel(paths, pool_b, n_layers, hidden, nq, nkv, hd, inter, vocab)
    assert disk.struct.n_layers == n_layers and disk.struct.kv_bits == kv_bits and disk.struct.pages == pages
    r = H.rng(4)
    q_lens = np.array([70, 1, 300], np.int32)
    ids = r.integers(0, vocab, int(q_lens.sum())).astype(np.int64)
    bt = np.array([[0, 0], [1, 0], [2, 3]], np.int32)
    outs = []
    for model in (mem, disk):
        sl = torch.zeros(3, dtype=torch.int32, device="cuda")
        tok, logits = model.step(ctx, H.to_dev(ids), H.to_dev(q_lens), sl, H.to_dev(bt), int(q_lens.max()), advance=True, want_logits=True)
        tok2, logits2 = model.step(ctx, tok.clone(), H.to_dev(np.ones(3, np.int32)), sl, H.to_dev(bt), 1, advance=True, want_logits=True)
        ctx.poll_status()
        outs.append((tok.cpu().numpy(), logits.cpu().numpy(), tok2.cpu().numpy(), logits2.cpu().numpy()))
    a, b = outs
    # same weights and the same kernels; the rotary table is computed by two different pow() (torch's and libm's)
    # (a last-bit difference in a rotation can move a 4-bit KV code by one step, hence the wider bar there)
    scale = np.abs(a[1]).max()
    tol = (2e-3 if kv_bits == 0 else 1e-2) * scale
    assert np.abs(a[1] - b[1]).max() <= tol and np.abs(a[3] - b[3]).max() <= tol
    for t_mem, t_disk, lg in ((a[0], b[0], a[1]), (a[2], b[2], a[3])):
        for s in range(3):
            if t_mem[s] != t_disk[s]:          # allowed only on a near-tie
                assert abs(lg[s, t_mem[s]] - lg[s, t_disk[s]]) <= tol
    disk.close()
    pool_a.close(); pool_b.close()


@pytest.mark.gpu
def test_model_load_reports_what_is_missing(ctx, tmp_path):
    import exl3b200
    from exl3b200.step import LoadedModel
    p = tmp_path / "empty.safetensors"
    H.write_safetensors(p, {"model.embed_tokens.weight": np.zeros((256, 128), np.float16)})
    pool = exl3b200.Pool(0, 1, 2, 1, 128, 0, 0)
    with pytest.raises(exl3b200.Exl3Error, match="input_layernorm"):
        LoadedModel([str(p)], pool, 1, 128, 1, 1, 128, 128, 256)
    pool.close()
