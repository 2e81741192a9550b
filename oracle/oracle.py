"""numpy front end of the CPU oracle (oracle.c).  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the benchmark's CPU-baseline leg import this module; the product library never
does.  Arrays are numpy: fp16 tensors as ``np.float16``, trellis tensors as ``np.int16`` of shape
``[k/16, n/16, 16*K]``, quantised-KV codes as ``np.uint32``/``np.int32``, block tables and lengths as ``np.int32``.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")


def build(force=False):
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "oracle"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.orc_decode_state.restype = C.c_uint16
        _lib.orc_decode_state.argtypes = [C.c_int, C.c_uint32]
        _lib.orc_tile_state.restype = C.c_uint32
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a)
    assert a.dtype == dt, (a.dtype, dt)
    return a


def num_threads():
    return lib().orc_num_threads()


def set_num_threads(n):
    lib().orc_set_num_threads(C.c_int(int(n)))


def codebook(cb):
    """All 65536 decoded fp16 values of codebook cb (0 3INST, 1 MCG, 2 MUL1)."""
    L = lib()
    return np.array([L.orc_decode_state(cb, s) for s in range(65536)], dtype=np.uint16).view(np.float16)


def reconstruct(trellis, K, cb):
    trellis = _c(trellis, np.int16)
    tk, tn, w = trellis.shape
    assert w == 16 * K
    out = np.empty((tk * 16, tn * 16), np.float16)
    lib().orc_reconstruct(_p(out), _p(trellis), C.c_int(tk * 16), C.c_int(tn * 16), C.c_int(K), C.c_int(cb))
    return out


def had_r_128(x, pre=None, post=None, scale=1.0, out_dtype=None):
    """scale multiplies 1/sqrt(128) as in the reference (hadamard.cu:106)."""
    scale = float(np.float32(scale) * np.float32(0.088388347648))
    x = np.ascontiguousarray(x)
    out_dtype = out_dtype or x.dtype
    rows = int(np.prod(x.shape[:-1]))
    cols = x.shape[-1]
    y = np.empty(x.shape, out_dtype)
    pre = None if pre is None else _c(pre, np.float16)
    post = None if post is None else _c(post, np.float16)
    lib().orc_had_r_128(_p(x), _p(y), _p(pre), _p(post), C.c_float(scale), C.c_int64(rows), C.c_int64(cols),
                        C.c_int(x.dtype == np.float32), C.c_int(out_dtype == np.float32))
    return y


def exl3_gemm(A, trellis, suh, svh, K, cb, c_fp32=False):
    A = _c(A, np.float16)
    trellis = _c(trellis, np.int16)
    m = int(np.prod(A.shape[:-1]))
    k = A.shape[-1]
    n = trellis.shape[1] * 16
    assert trellis.shape[0] * 16 == k and trellis.shape[2] == 16 * K
    Cm = np.empty(A.shape[:-1] + (n,), np.float32 if c_fp32 else np.float16)
    suh = None if suh is None else _c(suh, np.float16)
    svh = None if svh is None else _c(svh, np.float16)
    lib().orc_exl3_gemm(_p(A), _p(trellis), _p(Cm), C.c_int(c_fp32), _p(suh), _p(svh), C.c_int(m), C.c_int(k),
                        C.c_int(n), C.c_int(K), C.c_int(cb))
    return Cm


def exl3_mgemm(A, trellis_list, suh_list, svh_list, C_init, K, cb, indices=None, weights=None, num_tokens=1):
    """exl3_mgemm (kernels/quant/exl3_gemm.cu:386-678, exl3_gemm_kernel.cuh:88-314 with min/max_index = -1).
    A [bszm_in, m, k] fp16; C_init [bszm, m, n] fp16 or fp32 (slots that are skipped keep their contents);
    indices int64 [bszm] or None; weights fp16 [bszm] or None.  Returns the new C."""
    A = _c(A, np.float16)
    Cm = np.array(C_init, copy=True)
    c_fp32 = Cm.dtype == np.float32
    bszm = Cm.shape[0]
    m, k = A.shape[1], A.shape[2]
    n = Cm.shape[2]
    for j in range(bszm):
        mat = j if indices is None else int(indices[j])
        if mat < 0:
            continue
        a = A[0] if A.shape[0] == 1 else A[j]
        tr = _c(trellis_list[mat], np.int16)
        out = np.empty((m, n), Cm.dtype)
        w = 1.0 if weights is None else float(np.float16(weights[j]))
        lib().orc_exl3_gemm_scaled(_p(_c(a, np.float16)), _p(tr), _p(out), C.c_int(c_fp32), _p(_c(suh_list[mat], np.float16)),
                                   _p(_c(svh_list[mat], np.float16)), C.c_int(m), C.c_int(k), C.c_int(n), C.c_int(K),
                                   C.c_int(cb), C.c_float(w))
        Cm[j] = out
    if weights is not None:
        stride = bszm // num_tokens
        for t in range(num_tokens):
            acc = np.zeros((m, n), Cm.dtype)
            for j in range(stride):
                if indices is None or int(indices[t * stride + j]) >= 0:
                    acc = (acc + Cm[t * stride + j]).astype(Cm.dtype)        # sequential adds in C's own precision
            Cm[t] = acc
    return Cm


def hgemm(A, B, c_fp32=False):
    A = _c(A, np.float16)
    B = _c(B, np.float16)
    m, k = A.shape
    n = B.shape[1]
    Cm = np.empty((m, n), np.float32 if c_fp32 else np.float16)
    lib().orc_hgemm(_p(A), _p(B), _p(Cm), C.c_int(c_fp32), C.c_int(m), C.c_int(k), C.c_int(n))
    return Cm


def rms_norm(x, w, eps, cbias=0.0, cscale=1.0, res=None, out_dtype=np.float16):
    """res (fp32, same shape) is updated in place with res += x before the norm (RES_IN)."""
    x = np.ascontiguousarray(x)
    dim = x.shape[-1]
    rows = x.size // dim
    y = np.empty(x.shape, out_dtype)
    w = None if w is None else _c(w, np.float16)
    if res is not None:
        assert res.dtype == np.float32 and res.flags.c_contiguous
    lib().orc_rms_norm(_p(x), C.c_int(x.dtype == np.float32), _p(w), _p(y), C.c_int(out_dtype == np.float32), _p(res),
                       C.c_float(eps), C.c_float(cbias), C.c_float(cscale), C.c_int(rows), C.c_int(dim))
    return y


def rope(q, k, inv_freq, position=0, positions=None, q_norm=None, k_norm=None, norm_eps=1e-6, norm_cbias=0.0,
         rope_mode=2, attn_factor=1.0):
    """q [bsz,seq,nq,hd], k [bsz,seq,nk,hd] fp16; returns rotated copies."""
    q = _c(q, np.float16).copy()
    k = None if k is None else _c(k, np.float16).copy()
    inv_freq = _c(inv_freq, np.float32)
    bsz, seq, nq, hd = q.shape
    nk = 0 if k is None else k.shape[2]
    positions = None if positions is None else _c(positions, np.int32)
    lib().orc_rope(_p(q), _p(k), _p(inv_freq), C.c_int(inv_freq.size), C.c_uint32(position), _p(positions),
                   _p(None if q_norm is None else _c(q_norm, np.float16)),
                   _p(None if k_norm is None else _c(k_norm, np.float16)), C.c_float(norm_eps), C.c_float(norm_cbias),
                   C.c_int(rope_mode), C.c_float(attn_factor), C.c_int(bsz), C.c_int(seq), C.c_int(nq), C.c_int(nk),
                   C.c_int(hd))
    return q, k


def silu_mul(x, y):
    x = _c(x, np.float16)
    y = _c(y, np.float16)
    z = np.empty_like(x)
    lib().orc_silu_mul(_p(x), _p(y), _p(z), C.c_int64(x.size))
    return z


def _act_mul(a32, y, act_limit):
    a = a32.astype(np.float16)
    y = _c(y, np.float16)
    if act_limit != 0.0:
        lim = np.float16(act_limit)
        y = np.minimum(np.maximum(y, -lim), lim)
        a = np.minimum(a, lim)
    return (a * y).astype(np.float16)              # numpy's fp16 product: fp32 product rounded once


def gelu_mul(x, y, act_limit=0.0):
    """z = gelu_tanh(x) * y (kernels/activation_kernels.cuh:40-50,142-186): the activation in fp32, rounded to fp16; the
    optional clamps and the product in fp16."""
    a = _c(x, np.float16).astype(np.float32)
    c = np.float32(0.797884560803)
    g = np.float32(0.5) * a * (np.float32(1.0) + np.tanh(c * (a + np.float32(0.044715) * a * a * a)))
    return _act_mul(g.astype(np.float32), y, act_limit)


def relu2_mul(x, y, act_limit=0.0):
    """z = relu(x)^2 * y (kernels/activation_kernels.cuh:52-58,142-186)."""
    a = np.maximum(_c(x, np.float16).astype(np.float32), np.float32(0.0))
    return _act_mul(a * a, y, act_limit)


def softcap(x, factor):
    """y = tanh(x / factor) * factor (kernels/softcap.cu:10-52): fp32 arithmetic, rounded to x's type."""
    x = np.ascontiguousarray(x)
    v = x.astype(np.float32) / np.float32(factor)
    return (np.tanh(v) * np.float32(factor)).astype(x.dtype)


def linear_forward(x, K, cb, k, n, trellis=None, suh=None, svh=None, dense=None, bias=None, out_unpadded=None,
                   trim_padded_out=False, softcap_factor=0.0):
    """Linear::forward (src/modules.rs:183-252): zero-extend x [rows, in_last] to the padded k, multiply (EXL3 tensor or a
    dense fp16 weight [k, n]), add the bias, trim to the unpadded width, soft-cap; each step rounds to fp16 like the
    tensor ops of the reference."""
    x = _c(x, np.float16)
    rows, in_last = x.shape
    if in_last < k:
        x = np.concatenate([x, np.zeros((rows, k - in_last), np.float16)], axis=1)
    y = hgemm(x, dense) if dense is not None else exl3_gemm(x, trellis, suh, svh, K, cb)
    if bias is not None:
        y = (y + _c(bias, np.float16)[None, :]).astype(np.float16)
    if trim_padded_out and out_unpadded is not None and out_unpadded < n:
        y = np.ascontiguousarray(y[:, :out_unpadded])
    if softcap_factor != 0.0:
        f = np.float16(softcap_factor)
        t = (y / f).astype(np.float16)                                   # fp16 division
        t = np.tanh(t.astype(np.float32)).astype(np.float16)
        y = (t * f).astype(np.float16)
    return y


def _history_weights(past_len, sustain, decay):
    """weight of history position i (distance past_len - i from the end): kernels/generator/rep_pen.cu:48-69"""
    dist = (past_len - np.arange(past_len)).astype(np.float32)
    if decay > 0:
        f = np.float32(1.0) - (dist - np.float32(sustain)) / np.float32(decay)
    else:
        f = np.ones(past_len, np.float32)
    f = np.clip(f, 0.0, 1.0).astype(np.float32)
    f[dist <= sustain] = 1.0
    f[np.arange(past_len) <= past_len - sustain - decay] = 0.0
    return f


def apply_rep_pens(logits, past_ids, rep_p, sustain, decay):
    """kernels/generator/rep_pen.cu:24-91: logits [1, vocab] fp16|fp32 -> fp32"""
    v = np.asarray(logits, np.float32).reshape(-1).copy()
    past = np.asarray(past_ids, np.int64).reshape(-1)
    f = np.zeros(v.size, np.float32)
    np.maximum.at(f, past, _history_weights(past.size, sustain, decay))
    w = np.where(v > 0, v / np.float32(rep_p), v * np.float32(rep_p)).astype(np.float32)
    f = f + np.float32(1e-30)
    f1 = (np.float32(1.0) - f) + np.float32(1e-30)
    return (v * f1 + w * f).astype(np.float32).reshape(1, -1)


def apply_pres_freq_pens(logits, past_ids, pres_p, freq_p, sustain, decay):
    """kernels/generator/rep_pen.cu:135-210"""
    v = np.asarray(logits, np.float32).reshape(-1).copy()
    past = np.asarray(past_ids, np.int64).reshape(-1)
    wts = _history_weights(past.size, sustain, decay)
    freq = np.zeros(v.size, np.float32)
    pres = np.zeros(v.size, np.float32)
    np.add.at(freq, past, wts * np.float32(freq_p))
    np.maximum.at(pres, past, wts * np.float32(pres_p))
    return ((v - freq) - pres).astype(np.float32).reshape(1, -1)


def philox_uniform(seed, subsequence, draw):
    """Philox4x32-10 (Salmon et al., SC'11) consumed the way kernels/generator/gumbel.cu:47-66 does through its random
    number library: key (seed, 0), counter (draw // 4, 0, subsequence, 0), word draw % 4, uniform = w * 2^-32 + 2^-33."""
    sub = np.asarray(subsequence, np.uint64)
    draw = np.broadcast_to(np.asarray(draw, np.uint64), sub.shape)
    c = [draw >> np.uint64(2), np.zeros_like(sub), sub.copy(), np.zeros_like(sub)]
    k0, k1 = np.uint64(seed & 0xFFFFFFFF), np.uint64(0)
    M0, M1, mask = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57), np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [((p1 >> np.uint64(32)) ^ c[1] ^ k0) & mask, p1 & mask, ((p0 >> np.uint64(32)) ^ c[3] ^ k1) & mask, p0 & mask]
        k0, k1 = (k0 + np.uint64(0x9E3779B9)) & mask, (k1 + np.uint64(0xBB67AE85)) & mask
    words = np.stack(c, 0)
    w = np.take_along_axis(words, (draw & np.uint64(3)).astype(np.int64)[None], 0)[0]
    return (w.astype(np.float32) * np.float32(2.3283064e-10) + np.float32(1.1641532e-10)).astype(np.float32)


def gumbel_of(u):
    u = np.minimum(u, np.float32(0.99999994))
    inner = np.maximum(-np.log(np.maximum(u, np.float32(1e-20)).astype(np.float64)), 1e-20)
    return (-np.log(inner)).astype(np.float32)


def gumbel_noise_f32(logits, seed):
    """kernels/generator/gumbel.cu:47-66: element i takes the first draw of subsequence i"""
    x = np.asarray(logits, np.float32)
    idx = np.arange(x.size, dtype=np.uint64)
    return (x.reshape(-1) + gumbel_of(philox_uniform(seed, idx, 0))).astype(np.float32).reshape(x.shape)


def gumbel_sample_noisy(logits, seed, max_logit=0):
    """kernels/generator/sampling_basic.cu:93-129: the noisy logits whose row argmax is the sample.  Column c takes draw
    2 (c // 2048) + (c & 1) of subsequence (c // 2) % 1024; every row sees the same noise."""
    x = np.asarray(logits).astype(np.float32)
    n = x.shape[1]
    lim = n if max_logit == 0 or max_logit > n else max_logit
    end = min(n, lim + 1)
    c = np.arange(end, dtype=np.uint64)
    g = gumbel_of(philox_uniform(seed, (c >> np.uint64(1)) & np.uint64(1023), np.uint64(2) * (c >> np.uint64(11)) + (c & np.uint64(1))))
    out = x[:, :end] + g[None, :]
    # the reference admits columns pair by pair (sampling_basic.cu:38-62): (c, c + 1), c even: first if c < lim - 1, second if c < lim
    ci = np.arange(end)
    bad = np.where(ci % 2 == 1, ci - 1 >= lim, ci >= lim - 1)
    out[:, bad] = -np.inf
    return out


def cache_rotate(cache, order, temp):
    """kernels/generator/cache.cu:11-85 on numpy pages, in place"""
    order = np.asarray(order, np.int32).reshape(-1, 2)
    for a, b in order:
        src = cache[b].copy() if b >= 0 else temp.copy()
        if a >= 0:
            cache[a] = src
        else:
            temp[...] = src
    return cache


def mul_sigmoid(x, y):
    """x * sigmoid(y) with every step rounded to fp16 (kernels/activation_kernels.cuh:132-139,300-315)"""
    x, y = _c(x, np.float16), _c(y, np.float16)
    e = np.exp(-y.astype(np.float64)).astype(np.float16)
    s = (np.float16(1.0) + e).astype(np.float16)
    r = (1.0 / s.astype(np.float64)).astype(np.float16)
    return (x * r).astype(np.float16)


def add(x, y):
    x = _c(x, np.float16)
    y = _c(y, np.float16)
    z = np.empty_like(x)
    lib().orc_add(_p(x), _p(y), _p(z), C.c_int64(x.size))
    return z


def argmax(logits):
    logits = np.ascontiguousarray(logits)
    rows, n = logits.shape
    ids = np.empty(rows, np.int64)
    lib().orc_argmax(_p(logits), C.c_int(logits.dtype == np.float32), _p(ids), C.c_int(rows), C.c_int(n))
    return ids


def embed(ids, table):
    ids = _c(ids, np.int64)
    table = _c(table, np.float16)
    out = np.empty((ids.size, table.shape[1]), np.float32)
    lib().orc_embed(_p(ids), _p(table), _p(out), C.c_int(ids.size), C.c_int(table.shape[1]))
    return out


def paged_kv_update(k, v, kc, vc, block_table, seqlens):
    """k,v [bsz,seq,nkv,hd]; kc,vc [pages,256,nkv,hd] updated in place."""
    k = _c(k, np.float16)
    v = _c(v, np.float16)
    bsz, seq, nkv, hd = k.shape
    bt = _c(block_table, np.int32)
    lib().orc_paged_kv_update(_p(k), _p(v), _p(kc), _p(vc), _p(bt), _p(_c(seqlens, np.int32)), C.c_int(bsz),
                              C.c_int(seq), C.c_int(nkv), C.c_int(hd), C.c_int(bt.shape[1]))


def quant_groups(x, bits):
    x = _c(x, np.float16)
    groups = x.size // 32
    q = np.empty((groups, bits), np.uint32)
    s = np.empty(groups, np.float16)
    lib().orc_quant_groups(_p(x), _p(q), _p(s), C.c_int64(groups), C.c_int(bits))
    return q, s


def dequant_groups(q, s, bits):
    q = _c(q, np.uint32)
    s = _c(s, np.float16)
    out = np.empty(s.size * 32, np.float16)
    lib().orc_dequant_groups(_p(q), _p(s), _p(out), C.c_int64(s.size), C.c_int(bits))
    return out


def quant_cache_paged(k_in, qk, sk, v_in, qv, sv, seqlens, block_table, k_bits, v_bits):
    """k_in,v_in [bsz,seq,nkv,hd]; qk/qv [pages,256,groups*bits] uint32, sk/sv [pages,256,groups] fp16, in place."""
    k_in = _c(k_in, np.float16)
    v_in = _c(v_in, np.float16)
    bsz, seq = k_in.shape[:2]
    dim = k_in.shape[2] * k_in.shape[3]
    bt = _c(block_table, np.int32)
    lib().orc_quant_cache_paged(_p(k_in), _p(qk), _p(sk), _p(v_in), _p(qv), _p(sv), _p(_c(seqlens, np.int32)), _p(bt),
                                C.c_int(bsz), C.c_int(seq), C.c_int(dim), C.c_int(bt.shape[1]), C.c_int(k_bits),
                                C.c_int(v_bits))


def dequant_cache_paged(qk, sk, k_out, qv, sv, v_out, seqlens, block_table, k_bits, v_bits, compact=False, bonus=0):
    bt = _c(block_table, np.int32)
    dim = sk.shape[-1] * 32
    lib().orc_dequant_cache_paged(_p(qk), _p(sk), _p(k_out), _p(qv), _p(sv), _p(v_out), _p(_c(seqlens, np.int32)),
                                  _p(bt), C.c_int(bt.shape[0]), C.c_int(dim), C.c_int(bt.shape[1]), C.c_int(k_bits),
                                  C.c_int(v_bits), C.c_int(compact), C.c_int(bonus))


def attn_plain(q, k, v, causal=True, sm_scale=0.0):
    """Attention over plain tensors q [bsz,q_len,nq,hd], k, v [bsz,kv_len,nkv,hd] (kernels/attention.cu:2292-2437; causal
    limit kv_len - q_len + i, :1476).  Restated through the paged form: every sequence's keys laid into pages of its own,
    all of them already in the cache."""
    q, k, v = _c(q, np.float16), _c(k, np.float16), _c(v, np.float16)
    bsz, kv_len, nkv, hd = k.shape
    pps = max(1, (kv_len + 255) // 256)
    kc = np.zeros((bsz * pps, 256, nkv, hd), np.float16)
    vc = np.zeros_like(kc)
    kc.reshape(bsz, pps * 256, nkv, hd)[:, :kv_len] = k
    vc.reshape(bsz, pps * 256, nkv, hd)[:, :kv_len] = v
    bt = np.arange(bsz * pps, dtype=np.int32).reshape(bsz, pps)
    return attn_paged(q, kc, vc, bt, np.full(bsz, kv_len, np.int32), kv_append=0, causal=causal, sm_scale=sm_scale)


def attn_paged(q, kc, vc, block_table, seqlens, kv_append=None, causal=True, sm_scale=0.0, cu_q=None, nkv=None,
               quant=None):
    """Rectangular: q [bsz,q_len,nq,hd].  Ragged: q [rows,nq,hd] with cu_q [bsz+1].
    quant = (qk, sk, qv, sv, bits) selects the quantised pools (kc/vc ignored; nkv must be given)."""
    q = _c(q, np.float16)
    bt = _c(block_table, np.int32)
    bsz = bt.shape[0]
    if cu_q is None:
        _, q_len, nq, hd = q.shape
        kv_append = q_len if kv_append is None else kv_append
    else:
        cu_q = _c(cu_q, np.int32)
        _, nq, hd = q.shape
        q_len, kv_append = 0, 0
    if quant is None:
        nkv = kc.shape[2]
        qk = sk = qv = sv = None
        bits = 0
    else:
        qk, sk, qv, sv, bits = quant
    o = np.empty_like(q)
    lib().orc_attn_paged(_p(q), _p(kc), _p(vc), _p(qk), _p(sk), _p(qv), _p(sv), C.c_int(bits), _p(bt),
                         _p(_c(seqlens, np.int32)), _p(cu_q), _p(o), C.c_int(bsz), C.c_int(q_len), C.c_int(kv_append),
                         C.c_int(nq), C.c_int(nkv), C.c_int(hd), C.c_int(bt.shape[1]), C.c_int(causal),
                         C.c_float(sm_scale))
    return o
