"""ctypes binding of libexl3b200.so with the op names and argument meaning of the reference's safe wrappers
(src/ffi.rs:209-686).  Tensors are torch CUDA tensors used only as device buffers: each wrapper checks dtype and
contiguity, derives the shapes the C-ABI needs and passes raw device pointers.  There is no fallback: if the shared
library is missing or a call returns an error code, an exception is raised.
"""
import ctypes as C
import os

import torch

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.environ.get("EXL3_B200_LIB") or os.path.join(_PKG, "libexl3b200.so")

ROPE_NONE, ROPE_GPTJ, ROPE_NEOX = 0, 1, 2   # src/ffi.rs:217-219


class Exl3Error(RuntimeError):
    pass


class Linear(C.Structure):
    """exl3_linear (include/exl3_abi.h): one EXL3 tensor of a step-level call."""
    _fields_ = [("trellis", C.c_void_p), ("suh", C.c_void_p), ("svh", C.c_void_p),
                ("k", C.c_int), ("n", C.c_int), ("K", C.c_int), ("cb", C.c_int)]


class LinearLayer(C.Structure):
    """exl3_linear_layer (include/exl3_abi.h): one linear layer with its padding, bias, trim and soft-cap policy."""
    _fields_ = [("w", Linear), ("dense", C.c_void_p), ("bias", C.c_void_p), ("in_unpadded", C.c_int),
                ("out_unpadded", C.c_int), ("trim_padded_out", C.c_int), ("softcap", C.c_float)]


_lib = None


def lib():
    """Load the shared library (built by exllamav3-rs_b200/build.py).  Raises if it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise Exl3Error(f"{LIB_PATH} not found: build it with `python exllamav3-rs_b200/build.py` "
                            "(there is no fallback implementation)")
        L = C.CDLL(LIB_PATH)
        L.exl3_version.restype = C.c_char_p
        L.exl3_last_error.restype = C.c_char_p
        L.exl3_last_error.argtypes = [C.c_void_p]
        L.exl3_ctx_create.argtypes = [C.c_int, C.c_size_t, C.POINTER(C.c_void_p)]
        L.exl3_ctx_destroy.argtypes = [C.c_void_p]
        L.exl3_pool_create.argtypes = [C.c_int] * 7 + [C.POINTER(C.c_void_p)]
        L.exl3_pool_destroy.argtypes = [C.c_void_p]
        L.exl3_pool_layer.argtypes = [C.c_void_p, C.c_int] + [C.POINTER(C.c_void_p)] * 4
        for n in ("exl3_pool_num_free", "exl3_pool_num_pages"):
            getattr(L, n).argtypes = [C.c_void_p]
        L.exl3_pool_refcount.argtypes = [C.c_void_p, C.c_int]
        L.exl3_pool_set_dedup.argtypes = [C.c_void_p, C.c_int]
        L.exl3_pool_alloc.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int32)]
        L.exl3_pool_alloc_prefix.argtypes = [C.c_void_p, C.POINTER(C.c_int64), C.c_int, C.c_int, C.POINTER(C.c_int32), C.c_int,
                                             C.POINTER(C.c_int), C.POINTER(C.c_int64)]
        L.exl3_pool_register_page_hash.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int64), C.c_int]
        L.exl3_pool_release.argtypes = [C.c_void_p, C.POINTER(C.c_int32), C.c_int]
        L.exl3_ctx_launch_count.restype = C.c_uint64
        L.exl3_ctx_launch_count.argtypes = [C.c_void_p]
        L.exl3_cuda_free_mib.restype = C.c_int64
        L.exl3_graph_new.restype = C.c_void_p
        L.exl3_graph_new.argtypes = [C.c_void_p]
        L.exl3_side_stream.restype = C.c_void_p
        L.exl3_side_stream.argtypes = [C.c_void_p]
        for n in ("exl3_graph_free", "exl3_graph_capture_begin", "exl3_graph_capture_end", "exl3_graph_replay"):
            getattr(L, n).argtypes = [C.c_void_p]
        _lib = L
    return _lib


def _ptr(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _chk(t, dtype, name):
    if t is None:
        return
    if not t.is_cuda:
        raise Exl3Error(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype not in (dtype if isinstance(dtype, tuple) else (dtype,)):
        raise Exl3Error(f"{name} has dtype {t.dtype}, expected {dtype}")
    if not t.is_contiguous():
        raise Exl3Error(f"{name} must be contiguous")


class Ctx:
    """One context per device: owns the scratch the ops share (split-K partials, counters, status word)."""

    def __init__(self, device=0, workspace_bytes=0):
        self._h = C.c_void_p()
        torch.cuda.set_device(device)
        rc = lib().exl3_ctx_create(device, workspace_bytes, C.byref(self._h))
        if rc != 0:
            raise Exl3Error(f"exl3_ctx_create failed with code {rc}")
        self.device = device

    def close(self):
        if self._h:
            lib().exl3_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    def stream(self, stream=None):
        if stream is None:
            return C.c_void_p(torch.cuda.current_stream().cuda_stream)
        if isinstance(stream, int):
            return C.c_void_p(stream)
        return C.c_void_p(stream.cuda_stream)

    def check(self, rc, what):
        if rc != 0:
            raise Exl3Error(f"{what} failed ({rc}): {lib().exl3_last_error(self._h).decode()}")

    def poll_status(self, stream=None):
        self.check(lib().exl3_ctx_poll_status(self._h, self.stream(stream)), "device status")

    def set_mma_attn(self, on):
        """src/ffi.rs set_mma_attn: True = tcgen05 attention for long row blocks (default), False = mma.sync kernels."""
        lib().exl3_set_mma_attn(self._h, int(bool(on)))

    def launch_count(self):
        return int(lib().exl3_ctx_launch_count(self._h))

    STAGES = ("descriptors + embedding", "attention norm + q/k/v", "rope + KV write + attention", "o_proj",
              "MLP norm + gate/up", "activation + down_proj", "head")

    def stage_profile(self, enable=True):
        """Per-stage device times of the step runner (the reference's EXL3_TRUNK_PROF, src/model.rs:72-116)."""
        self.check(lib().exl3_ctx_stage_profile(self._h, int(bool(enable))), "ctx_stage_profile")

    def stage_times(self, reset=True):
        """({stage name: ms per step}, profiled steps) since the last reset."""
        ms = (C.c_double * len(self.STAGES))()
        steps = C.c_int(0)
        self.check(lib().exl3_ctx_stage_times(self._h, ms, C.byref(steps), int(bool(reset))), "ctx_stage_times")
        n = max(steps.value, 1)
        return {name: ms[i] / n for i, name in enumerate(self.STAGES)}, steps.value

    # ------------------------------------------------------------------------------------------ EXL3 linear
    def exl3_gemm(self, a, trellis, c, suh, a_had, svh, mcg=False, mul1=False, stream=None):
        """src/ffi.rs:274-291.  a [..,k] fp16, trellis [k/16,n/16,16K] int16, c [..,n] fp16|fp32."""
        _chk(a, torch.float16, "a"); _chk(trellis, torch.int16, "trellis"); _chk(c, (torch.float16, torch.float32), "c")
        _chk(suh, torch.float16, "suh"); _chk(svh, torch.float16, "svh"); _chk(a_had, torch.float16, "a_had")
        k = a.shape[-1]
        m = a.numel() // k
        n = trellis.shape[1] * 16
        K = trellis.shape[2] // 16
        if trellis.shape[0] * 16 != k or c.shape[-1] != n or c.numel() // n != m:
            raise Exl3Error("exl3_gemm: shape mismatch")
        rc = lib().exl3_gemm(self._h, self.stream(stream), _ptr(a), _ptr(trellis), _ptr(c), _ptr(suh), _ptr(a_had),
                             _ptr(svh), m, k, n, K, int(c.dtype == torch.float32), int(mcg), int(mul1))
        self.check(rc, "exl3_gemm")

    def gemm_fanout(self, a, weights, outs, stream=None):
        """The same activations through up to three EXL3 tensors (the reference's back-to-back exl3_gemm calls for
        q/k/v, src/modules.rs:646-648, and gate/up, src/modules.rs:933-934).  `weights` is a list of
        (trellis, suh, svh, cb) tuples, `outs` the matching output tensors."""
        _chk(a, torch.float16, "a")
        k = a.shape[-1]
        m = a.numel() // k
        structs, keep = [], []
        for (trellis, suh, svh, cb), c in zip(weights, outs):
            _chk(trellis, torch.int16, "trellis"); _chk(suh, torch.float16, "suh"); _chk(svh, torch.float16, "svh")
            _chk(c, (torch.float16, torch.float32), "c")
            n = trellis.shape[1] * 16
            if trellis.shape[0] * 16 != k or c.shape[-1] != n or c.numel() // n != m or c.dtype != outs[0].dtype:
                raise Exl3Error("gemm_fanout: shape mismatch")
            structs.append(Linear(_ptr(trellis), _ptr(suh), _ptr(svh), k, n, trellis.shape[2] // 16, int(cb)))
        cnt = len(structs)
        if cnt != len(outs) or not 1 <= cnt <= 3:
            raise Exl3Error("gemm_fanout: 1..3 tensors and as many outputs")
        wp = (C.POINTER(Linear) * cnt)(*[C.pointer(x) for x in structs])
        cp = (C.c_void_p * cnt)(*[_ptr(c) for c in outs])
        rc = lib().exl3_gemm_fanout(self._h, self.stream(stream), _ptr(a), cnt, wp, cp, m, int(outs[0].dtype == torch.float32))
        self.check(rc, "exl3_gemm_fanout")

    def reconstruct(self, unpacked, packed, K, mcg=False, mul1=False, stream=None):
        """src/ffi.rs:611-613."""
        _chk(unpacked, torch.float16, "unpacked"); _chk(packed, torch.int16, "packed")
        k, n = packed.shape[0] * 16, packed.shape[1] * 16
        if tuple(unpacked.shape) != (k, n) or packed.shape[2] != 16 * K:
            raise Exl3Error("reconstruct: shape mismatch")
        self.check(lib().exl3_reconstruct(self._h, self.stream(stream), _ptr(unpacked), _ptr(packed), k, n, K,
                                          int(mcg), int(mul1)), "reconstruct")

    def had_r_128(self, x, out, pre_scale=None, post_scale=None, scale=1.0, stream=None):
        """src/ffi.rs:606-608."""
        _chk(x, (torch.float16, torch.float32), "x"); _chk(out, x.dtype, "out")
        _chk(pre_scale, torch.float16, "pre_scale"); _chk(post_scale, torch.float16, "post_scale")
        cols = x.shape[-1]
        rows = x.numel() // cols
        self.check(lib().exl3_had_r_128(self._h, self.stream(stream), _ptr(x), _ptr(out), _ptr(pre_scale),
                                        _ptr(post_scale), C.c_float(scale), rows, cols,
                                        int(x.dtype == torch.float32)), "had_r_128")

    def hgemm(self, a, b, c, stream=None):
        """src/ffi.rs:335-337."""
        _chk(a, torch.float16, "a"); _chk(b, torch.float16, "b"); _chk(c, (torch.float16, torch.float32), "c")
        k = a.shape[-1]
        m = a.numel() // k
        n = b.shape[1]
        if b.shape[0] != k or c.shape[-1] != n:
            raise Exl3Error("hgemm: shape mismatch")
        self.check(lib().exl3_hgemm(self._h, self.stream(stream), _ptr(a), _ptr(b), _ptr(c), m, k, n,
                                    int(c.dtype == torch.float32)), "hgemm")

    # ---------------------------------------------------------------------------------------- norm/rope/act
    def rms_norm(self, x, w, y, eps, constant_bias=0.0, constant_scale=1.0, stream=None):
        """src/ffi.rs:294-296."""
        _chk(x, (torch.float16, torch.float32), "x"); _chk(w, torch.float16, "w"); _chk(y, (torch.float16, torch.float32), "y")
        dim = x.shape[-1]
        self.check(lib().exl3_rms_norm(self._h, self.stream(stream), _ptr(x), int(x.dtype == torch.float32), _ptr(w),
                                       _ptr(y), int(y.dtype == torch.float32), C.c_float(eps), C.c_float(constant_bias),
                                       C.c_float(constant_scale), x.numel() // dim, dim), "rms_norm")

    def rms_norm_res_in(self, x, w, y, r, eps, constant_bias=0.0, constant_scale=1.0, stream=None):
        """src/ffi.rs:466-468: r += x, y = norm(r)."""
        _chk(x, (torch.float16, torch.float32), "x"); _chk(w, torch.float16, "w"); _chk(y, (torch.float16, torch.float32), "y")
        _chk(r, torch.float32, "r")
        dim = x.shape[-1]
        self.check(lib().exl3_rms_norm_res_in(self._h, self.stream(stream), _ptr(x), int(x.dtype == torch.float32),
                                              _ptr(w), _ptr(y), int(y.dtype == torch.float32), _ptr(r), C.c_float(eps),
                                              C.c_float(constant_bias), C.c_float(constant_scale), x.numel() // dim,
                                              dim), "rms_norm_res_in")

    def rope(self, q, k, inv_freq, position=0, positions=None, q_norm=None, k_norm=None, norm_eps=1e-6,
             norm_constant_bias=0.0, rope_mode=ROPE_NEOX, attn_factor=1.0, row_pos=None, out_q=None, out_k=None, stream=None):
        """src/ffi.rs:301-333; q [bsz,seq,nq,hd] and k [bsz,seq,nk,hd] are rotated into out_q/out_k, or in place when those
        are None (the reference's call passes the same tensor twice for that)."""
        _chk(q, torch.float16, "q"); _chk(k, torch.float16, "k"); _chk(inv_freq, torch.float32, "inv_freq")
        _chk(out_q, torch.float16, "out_q"); _chk(out_k, torch.float16, "out_k")
        _chk(positions, torch.int32, "positions"); _chk(row_pos, torch.int32, "row_pos")
        _chk(q_norm, torch.float16, "q_norm"); _chk(k_norm, torch.float16, "k_norm")
        bsz, seq, nq, hd = q.shape
        nk = 0 if k is None else k.shape[2]
        self.check(lib().exl3_rope(self._h, self.stream(stream), _ptr(q), _ptr(out_q), _ptr(k), _ptr(out_k), _ptr(inv_freq),
                                   inv_freq.numel(), C.c_uint32(position), _ptr(positions), _ptr(row_pos), _ptr(q_norm),
                                   _ptr(k_norm), C.c_float(norm_eps), C.c_float(norm_constant_bias), rope_mode,
                                   C.c_float(attn_factor), bsz, seq, nq, nk, hd), "rope")

    def silu_mul(self, x, y, z, act_limit=0.0, stream=None):
        """src/ffi.rs:480-482."""
        _chk(x, torch.float16, "x"); _chk(y, torch.float16, "y"); _chk(z, torch.float16, "z")
        self.check(lib().exl3_silu_mul(self._h, self.stream(stream), _ptr(x), _ptr(y), _ptr(z), C.c_float(act_limit),
                                       C.c_int64(x.numel())), "silu_mul")

    def gelu_mul(self, x, y, z, act_limit=0.0, stream=None):
        """src/ffi.rs:126."""
        _chk(x, torch.float16, "x"); _chk(y, torch.float16, "y"); _chk(z, torch.float16, "z")
        self.check(lib().exl3_gelu_mul(self._h, self.stream(stream), _ptr(x), _ptr(y), _ptr(z), C.c_float(act_limit),
                                       C.c_int64(x.numel())), "gelu_mul")

    def relu2_mul(self, x, y, z, act_limit=0.0, stream=None):
        """src/ffi.rs:127."""
        _chk(x, torch.float16, "x"); _chk(y, torch.float16, "y"); _chk(z, torch.float16, "z")
        self.check(lib().exl3_relu2_mul(self._h, self.stream(stream), _ptr(x), _ptr(y), _ptr(z), C.c_float(act_limit),
                                        C.c_int64(x.numel())), "relu2_mul")

    def softcap(self, x, y, factor, stream=None):
        """src/ffi.rs:136: y = tanh(x / factor) * factor, fp16 or fp32 (in place when y is x)."""
        _chk(x, (torch.float16, torch.float32), "x"); _chk(y, x.dtype, "y")
        self.check(lib().exl3_softcap(self._h, self.stream(stream), _ptr(x), _ptr(y), C.c_float(factor),
                                      C.c_int64(x.numel()), int(x.dtype == torch.float32)), "softcap")

    def exl3_mgemm(self, a, trellis_tab, c, suh_tab, svh_tab, K, indices=None, weights=None, mcg=False, mul1=False,
                   num_tokens=1, a_had=None, stream=None):
        """src/ffi.rs:28-42.  a [bszm_in, m, k] fp16, c [bszm_out, m, n] fp16|fp32; *_tab int64 device tensors of device
        pointers (one per tensor of the table); indices int64 [bszm] and weights fp16 [bszm] on the device, or None."""
        _chk(a, torch.float16, "a"); _chk(c, (torch.float16, torch.float32), "c")
        for t, nm in ((trellis_tab, "trellis_tab"), (suh_tab, "suh_tab"), (svh_tab, "svh_tab")):
            _chk(t, torch.int64, nm)
        if indices is not None:
            _chk(indices, torch.int64, "indices")
        if weights is not None:
            _chk(weights, torch.float16, "weights")
        bszm_in, m, k = a.shape
        bszm_out, _, n = c.shape
        self.check(lib().exl3_mgemm(self._h, self.stream(stream), _ptr(a), _ptr(trellis_tab), _ptr(c), _ptr(suh_tab),
                                    _ptr(a_had), _ptr(svh_tab), _ptr(indices), _ptr(weights), bszm_in, bszm_out, m, k, n,
                                    K, int(c.dtype == torch.float32), int(mcg), int(mul1), num_tokens), "exl3_mgemm")

    def linear_forward(self, layer, x, y, stream=None):
        """Linear::forward (src/modules.rs:183-252): x [rows, in_last] fp16 -> y [rows, out] fp16; `layer` a LinearLayer."""
        _chk(x, torch.float16, "x"); _chk(y, torch.float16, "y")
        rows, in_last = x.shape
        self.check(lib().exl3_linear_forward(self._h, self.stream(stream), C.byref(layer), _ptr(x), in_last, _ptr(y), rows),
                   "linear_forward")

    def add(self, x, y, z, stream=None):
        _chk(x, torch.float16, "x"); _chk(y, torch.float16, "y"); _chk(z, torch.float16, "z")
        self.check(lib().exl3_add(self._h, self.stream(stream), _ptr(x), _ptr(y), _ptr(z), C.c_int64(x.numel())), "add")

    def argmax_sample(self, logits, ids, max_logit=0, stream=None):
        """src/ffi.rs:560-562; logits [rows,n] fp16|fp32, ids int64 [rows] or [rows,1]."""
        _chk(logits, (torch.float16, torch.float32), "logits"); _chk(ids, torch.int64, "ids")
        rows, n = logits.shape
        self.check(lib().exl3_argmax_sample(self._h, self.stream(stream), _ptr(logits),
                                            int(logits.dtype == torch.float32), _ptr(ids), rows, n, max_logit),
                   "argmax_sample")

    def apply_rep_pens(self, in_logits, out_logits, past_ids, rep_p, sustain_range, decay_range, stream=None):
        """src/ffi.rs:513-515: in_logits [1, vocab] fp16|fp32, out_logits fp32, past_ids int64 [1, past_len]."""
        _chk(in_logits, (torch.float16, torch.float32), "in_logits"); _chk(out_logits, torch.float32, "out_logits")
        _chk(past_ids, torch.int64, "past_ids")
        self.check(lib().exl3_apply_rep_pens(self._h, self.stream(stream), _ptr(in_logits), int(in_logits.dtype == torch.float32),
                                             _ptr(out_logits), _ptr(past_ids), C.c_float(rep_p), sustain_range, decay_range,
                                             in_logits.shape[0], in_logits.shape[1], past_ids.numel()), "apply_rep_pens")

    def apply_pres_freq_pens(self, in_logits, out_logits, past_ids, pres_p, freq_p, sustain_range, decay_range, stream=None):
        """src/ffi.rs:518-520."""
        _chk(in_logits, (torch.float16, torch.float32), "in_logits"); _chk(out_logits, torch.float32, "out_logits")
        _chk(past_ids, torch.int64, "past_ids")
        self.check(lib().exl3_apply_pres_freq_pens(self._h, self.stream(stream), _ptr(in_logits),
                                                   int(in_logits.dtype == torch.float32), _ptr(out_logits), _ptr(past_ids),
                                                   C.c_float(pres_p), C.c_float(freq_p), sustain_range, decay_range,
                                                   in_logits.shape[0], in_logits.shape[1], past_ids.numel()), "apply_pres_freq_pens")

    def gumbel_sample(self, logits, ids, max_logit=0, random=0, stream=None):
        """src/ffi.rs:528-530: logits [rows, n] fp16|fp32, ids int64 [rows] or [rows, 1]."""
        _chk(logits, (torch.float16, torch.float32), "logits"); _chk(ids, torch.int64, "ids")
        rows, n = logits.shape
        self.check(lib().exl3_gumbel_sample(self._h, self.stream(stream), _ptr(logits), int(logits.dtype == torch.float32),
                                            _ptr(ids), rows, n, max_logit, C.c_uint32(random)), "gumbel_sample")

    def gumbel_noise_f32(self, logits_in, logits_out, random=0, stream=None):
        """src/ffi.rs:533-535."""
        _chk(logits_in, torch.float32, "logits_in"); _chk(logits_out, torch.float32, "logits_out")
        self.check(lib().exl3_gumbel_noise_f32(self._h, self.stream(stream), _ptr(logits_in), _ptr(logits_out),
                                               C.c_int64(logits_in.numel()), C.c_uint32(random)), "gumbel_noise_f32")

    def cache_rotate(self, cache, order, temp, stream=None):
        """src/ffi.rs:538-540: cache [pages, ...] contiguous, order int32 [2 n], temp one page of scratch."""
        _chk(order, torch.int32, "order")
        pages = cache.shape[0]
        page_bytes = cache.numel() * cache.element_size() // pages
        if temp.numel() * temp.element_size() != page_bytes:
            raise Exl3Error("cache_rotate: temp must hold exactly one page")
        self.check(lib().exl3_cache_rotate(self._h, self.stream(stream), _ptr(cache), _ptr(order), _ptr(temp), pages,
                                           order.numel() // 2, C.c_size_t(page_bytes)), "cache_rotate")

    def mul_sigmoid_(self, x, y, stream=None):
        """src/ffi.rs:616-618: x *= sigmoid(y) in place."""
        _chk(x, torch.float16, "x"); _chk(y, torch.float16, "y")
        self.check(lib().exl3_mul_sigmoid_(self._h, self.stream(stream), _ptr(x), _ptr(y), C.c_int64(x.numel())), "mul_sigmoid_")

    def deinterleave_qg(self, qg, q, g, head_dim, stream=None):
        """src/ffi.rs:622-624: qg [rows, heads * 2 * head_dim] -> q, g [rows, heads * head_dim]."""
        _chk(qg, torch.float16, "qg"); _chk(q, torch.float16, "q"); _chk(g, torch.float16, "g")
        rows = qg.shape[0]
        heads = qg.shape[-1] // (2 * head_dim)
        self.check(lib().exl3_deinterleave_qg(self._h, self.stream(stream), _ptr(qg), _ptr(q), _ptr(g), rows, heads, head_dim),
                   "deinterleave_qg")

    def embed(self, ids, table, out, stream=None):
        _chk(ids, torch.int64, "ids"); _chk(table, torch.float16, "table"); _chk(out, torch.float32, "out")
        self.check(lib().exl3_embed(self._h, self.stream(stream), _ptr(ids), _ptr(table), _ptr(out), ids.numel(),
                                    table.shape[1], table.shape[0]), "embed")

    # ------------------------------------------------------------------------------------------------ paged
    def paged_kv_cache_update(self, k, v, k_cache, v_cache, block_table, cache_seqlens, cu_q=None, stream=None):
        """src/ffi.rs:346-358.  Rectangular k,v [bsz,seq,nkv,hd]; ragged (cu_q given) k,v [rows,nkv,hd]."""
        _chk(k, torch.float16, "k"); _chk(v, torch.float16, "v"); _chk(k_cache, torch.float16, "k_cache")
        _chk(v_cache, torch.float16, "v_cache"); _chk(block_table, torch.int32, "block_table")
        _chk(cache_seqlens, torch.int32, "cache_seqlens"); _chk(cu_q, torch.int32, "cu_q")
        bsz, pps = block_table.shape
        if cu_q is None:
            seq, nkv, hd = k.shape[1:]
        else:
            seq, (nkv, hd) = k.shape[0], k.shape[1:]
        self.check(lib().exl3_paged_kv_cache_update(self._h, self.stream(stream), _ptr(k), _ptr(v), _ptr(k_cache),
                                                    _ptr(v_cache), _ptr(block_table), _ptr(cache_seqlens), _ptr(cu_q),
                                                    bsz, seq, nkv, hd, k_cache.shape[0], pps), "paged_kv_cache_update")

    def bighead_attn_paged(self, q, k, v, k_cache, v_cache, block_table, cache_seqlens, o, kv_chunk_size=256,
                           causal=True, sm_scale=0.0, cu_q=None, max_q_len=None, stream=None):
        """src/ffi.rs:361-380.  Rectangular q [bsz,q_len,nq,hd]; ragged (cu_q given) q [rows,nq,hd]."""
        _chk(q, torch.float16, "q"); _chk(k, torch.float16, "k"); _chk(v, torch.float16, "v")
        _chk(k_cache, torch.float16, "k_cache"); _chk(v_cache, torch.float16, "v_cache"); _chk(o, torch.float16, "o")
        _chk(block_table, torch.int32, "block_table"); _chk(cache_seqlens, torch.int32, "cache_seqlens")
        _chk(cu_q, torch.int32, "cu_q")
        bsz, pps = block_table.shape
        if cu_q is None:
            q_len, nq, hd = q.shape[1:]
            kv_append = 0 if k is None else k.shape[1]
        else:
            nq, hd = q.shape[1:]
            q_len = max_q_len if max_q_len is not None else q.shape[0]
            kv_append = q.shape[0]          # ragged form: total packed rows
        nkv = k_cache.shape[2]
        self.check(lib().exl3_bighead_attn_paged(self._h, self.stream(stream), _ptr(q), _ptr(k), _ptr(v), _ptr(k_cache),
                                                 _ptr(v_cache), _ptr(block_table), _ptr(cache_seqlens), _ptr(cu_q),
                                                 _ptr(o), bsz, q_len, kv_append, nq, nkv, hd, k_cache.shape[0], pps,
                                                 kv_chunk_size, int(causal), C.c_float(sm_scale)), "bighead_attn_paged")

    def bighead_attn(self, q, k, v, o, causal=True, sm_scale=0.0, kv_chunk_size=256, stream=None):
        """src/ffi.rs:458-460: attention over plain tensors q, o [bsz,q_len,nq,hd], k, v [bsz,kv_len,nkv,hd]."""
        _chk(q, torch.float16, "q"); _chk(k, torch.float16, "k"); _chk(v, torch.float16, "v"); _chk(o, torch.float16, "o")
        if q.dim() != 4 or k.dim() != 4 or v.dim() != 4 or o.dim() != 4:
            raise ValueError("bighead_attn: q, k, v, o must be rank-4")
        bsz, q_len, nq, hd = q.shape
        if k.shape[0] != bsz or v.shape != k.shape or k.shape[3] != hd or o.shape != q.shape:
            raise ValueError("bighead_attn: shape mismatch")
        self.check(lib().exl3_bighead_attn(self._h, self.stream(stream), _ptr(q), _ptr(k), _ptr(v), _ptr(o), bsz, q_len,
                                           k.shape[1], nq, k.shape[2], hd, kv_chunk_size, int(causal),
                                           C.c_float(sm_scale)), "bighead_attn")

    def bighead_attn_paged_q(self, q, k, v, qk, sk, qv, sv, block_table, cache_seqlens, o, nkv, kv_chunk_size=256,
                             causal=True, sm_scale=0.0, compand_a=0.0, cu_q=None, max_q_len=None, stream=None):
        """src/ffi.rs:383-401 against the quantised pools (qk/qv int32 [pages,256,groups*bits], sk/sv fp16)."""
        _chk(q, torch.float16, "q"); _chk(k, torch.float16, "k"); _chk(v, torch.float16, "v"); _chk(o, torch.float16, "o")
        _chk(qk, torch.int32, "qk"); _chk(qv, torch.int32, "qv"); _chk(sk, torch.float16, "sk"); _chk(sv, torch.float16, "sv")
        _chk(block_table, torch.int32, "block_table"); _chk(cache_seqlens, torch.int32, "cache_seqlens")
        _chk(cu_q, torch.int32, "cu_q")
        bsz, pps = block_table.shape
        if cu_q is None:
            q_len, nq, hd = q.shape[1:]
            kv_append = 0 if k is None else k.shape[1]
        else:
            nq, hd = q.shape[1:]
            q_len = max_q_len if max_q_len is not None else q.shape[0]
            kv_append = q.shape[0]          # ragged form: total packed rows
        groups = sk.shape[2]
        self.check(lib().exl3_bighead_attn_paged_q(self._h, self.stream(stream), _ptr(q), _ptr(k), _ptr(v), _ptr(qk),
                                                   _ptr(sk), _ptr(qv), _ptr(sv), _ptr(block_table), _ptr(cache_seqlens),
                                                   _ptr(cu_q), _ptr(o), bsz, q_len, kv_append, nq, nkv, hd, qk.shape[0],
                                                   pps, qk.shape[2] // groups, qv.shape[2] // groups, kv_chunk_size,
                                                   int(causal), C.c_float(sm_scale), C.c_float(compand_a)),
                   "bighead_attn_paged_q")

    def quant_cache_paged(self, k_in, k_out, k_out_scales, v_in, v_out, v_out_scales, cache_seqlens, block_table,
                          page_size=256, seq_len=None, compand_a=0.0, in_contiguous=True, cu_q=None, stream=None):
        """src/ffi.rs:616-637."""
        _chk(k_in, torch.float16, "k_in"); _chk(v_in, torch.float16, "v_in")
        _chk(k_out, torch.int32, "k_out"); _chk(v_out, torch.int32, "v_out")
        _chk(k_out_scales, torch.float16, "k_out_scales"); _chk(v_out_scales, torch.float16, "v_out_scales")
        _chk(cache_seqlens, torch.int32, "cache_seqlens"); _chk(block_table, torch.int32, "block_table")
        _chk(cu_q, torch.int32, "cu_q")
        bsz, pps = block_table.shape
        groups = k_out_scales.shape[2]
        dim = groups * 32
        seq = seq_len if seq_len is not None else (k_in.shape[0] if cu_q is not None else k_in.shape[1])
        self.check(lib().exl3_quant_cache_paged(self._h, self.stream(stream), _ptr(k_in), _ptr(k_out), _ptr(k_out_scales),
                                                _ptr(v_in), _ptr(v_out), _ptr(v_out_scales), _ptr(cache_seqlens),
                                                _ptr(block_table), _ptr(cu_q), bsz, seq, dim, k_out.shape[0], pps,
                                                k_out.shape[2] // groups, v_out.shape[2] // groups, page_size,
                                                C.c_float(compand_a), int(in_contiguous)), "quant_cache_paged")

    def dequant_cache_paged(self, k_in, k_in_scales, k_out, v_in, v_in_scales, v_out, cache_seqlens, block_table,
                            page_size=256, sliding_window=0, compand_a=0.0, stream=None):
        """src/ffi.rs:640-660."""
        bsz, pps = block_table.shape
        groups = k_in_scales.shape[2]
        self.check(lib().exl3_dequant_cache_paged(self._h, self.stream(stream), _ptr(k_in), _ptr(k_in_scales), _ptr(k_out),
                                                  _ptr(v_in), _ptr(v_in_scales), _ptr(v_out), _ptr(cache_seqlens),
                                                  _ptr(block_table), bsz, groups * 32, k_in.shape[0], pps,
                                                  k_in.shape[2] // groups, v_in.shape[2] // groups, page_size,
                                                  sliding_window, C.c_float(compand_a)), "dequant_cache_paged")

    def dequant_cache_paged_window(self, k_in, k_in_scales, k_out, v_in, v_in_scales, v_out, cache_seqlens, block_table,
                                   page_size=256, bonus_len=0, compand_a=0.0, stream=None):
        """src/ffi.rs:663-685."""
        bsz, pps = block_table.shape
        groups = k_in_scales.shape[2]
        self.check(lib().exl3_dequant_cache_paged_window(self._h, self.stream(stream), _ptr(k_in), _ptr(k_in_scales),
                                                         _ptr(k_out), _ptr(v_in), _ptr(v_in_scales), _ptr(v_out),
                                                         _ptr(cache_seqlens), _ptr(block_table), bsz, groups * 32,
                                                         k_in.shape[0], pps, k_in.shape[2] // groups,
                                                         v_in.shape[2] // groups, page_size, bonus_len,
                                                         C.c_float(compand_a)), "dequant_cache_paged_window")


class Pool:
    """Paged KV pools of all layers plus their page table (include/exl3_abi.h exl3_pool_*): what the reference builds from
    PagedCache / QuantPagedCache and PageTable (src/paged.rs:18-92,330-506).  n_layers = 0 gives the page table alone."""

    def __init__(self, device, n_layers, pages, nkv, hd, k_bits=0, v_bits=0):
        self._h = C.c_void_p()
        rc = lib().exl3_pool_create(device, n_layers, pages, nkv, hd, k_bits, v_bits, C.byref(self._h))
        if rc != 0:
            raise Exl3Error(f"exl3_pool_create failed with code {rc}")
        self.pages, self.n_layers = pages, n_layers

    def close(self):
        if self._h:
            lib().exl3_pool_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def layer(self, i):
        """device addresses (k, v, sk, sv) of layer i as ints; fp16 pools have sk = sv = 0"""
        p = [C.c_void_p() for _ in range(4)]
        if lib().exl3_pool_layer(self._h, i, *[C.byref(x) for x in p]) != 0:
            raise Exl3Error("exl3_pool_layer failed")
        return tuple(x.value or 0 for x in p)

    def num_free(self):
        return lib().exl3_pool_num_free(self._h)

    def refcount(self, page):
        return lib().exl3_pool_refcount(self._h, page)

    def set_dedup(self, on):
        lib().exl3_pool_set_dedup(self._h, int(bool(on)))

    def alloc(self, n):
        out = (C.c_int32 * max(n, 1))()
        if lib().exl3_pool_alloc(self._h, n, out) != 0:
            raise Exl3Error(f"page table exhausted: need {n}, {self.num_free()} free")
        return list(out)[:n]

    def alloc_prefix(self, prompt_ids, gen_reserve):
        """-> (pages, matched_tokens)"""
        import numpy as np
        ids = np.ascontiguousarray(prompt_ids, np.int64)
        cap = (len(ids) + gen_reserve + 255) // 256 + 1
        out = (C.c_int32 * cap)(); cnt = C.c_int(); matched = C.c_int64()
        rc = lib().exl3_pool_alloc_prefix(self._h, ids.ctypes.data_as(C.POINTER(C.c_int64)), len(ids), gen_reserve, out, cap,
                                          C.byref(cnt), C.byref(matched))
        if rc != 0:
            raise Exl3Error(f"alloc_prefix failed with code {rc}")
        return list(out)[:cnt.value], int(matched.value)

    def register_page_hash(self, page, prev_page, token_ids):
        import numpy as np
        ids = np.ascontiguousarray(token_ids, np.int64)
        if lib().exl3_pool_register_page_hash(self._h, page, prev_page, ids.ctypes.data_as(C.POINTER(C.c_int64)), len(ids)) != 0:
            raise Exl3Error("register_page_hash failed")

    def release(self, pages):
        arr = (C.c_int32 * max(len(pages), 1))(*pages)
        if lib().exl3_pool_release(self._h, arr, len(pages)) != 0:
            raise Exl3Error("release failed")


class Checkpoint:
    """A safetensors file opened through exl3_checkpoint_* (src/safetensors.rs): header index, tensor reads into device
    memory, and Linear::load (src/modules.rs:97-165) as `linear()`."""

    def __init__(self, path):
        L = lib()
        L.exl3_checkpoint_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
        L.exl3_checkpoint_close.argtypes = [C.c_void_p]
        L.exl3_checkpoint_error.argtypes = [C.c_void_p]; L.exl3_checkpoint_error.restype = C.c_char_p
        L.exl3_checkpoint_count.argtypes = [C.c_void_p]
        L.exl3_checkpoint_name.argtypes = [C.c_void_p, C.c_int]; L.exl3_checkpoint_name.restype = C.c_char_p
        L.exl3_checkpoint_has.argtypes = [C.c_void_p, C.c_char_p]
        L.exl3_checkpoint_info.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p, C.c_int, C.POINTER(C.c_int64), C.c_int,
                                           C.POINTER(C.c_int), C.POINTER(C.c_uint64)]
        L.exl3_checkpoint_read.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_size_t, C.c_void_p]
        L.exl3_linear_load.argtypes = [C.c_void_p, C.c_void_p, C.c_char_p, C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_float,
                                       C.POINTER(LinearLayer)]
        L.exl3_linear_free.argtypes = [C.POINTER(LinearLayer)]
        h = C.c_void_p()
        rc = L.exl3_checkpoint_open(os.fsencode(path), C.byref(h))
        self._h = h
        if rc != 0:
            msg = L.exl3_checkpoint_error(h).decode() if h else "out of memory"
            self.close()
            raise Exl3Error(f"checkpoint {path}: {msg} (code {rc})")

    def close(self):
        if getattr(self, "_h", None):
            lib().exl3_checkpoint_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc, what):
        if rc != 0:
            raise Exl3Error(f"{what}: {lib().exl3_checkpoint_error(self._h).decode()} (code {rc})")

    def names(self):
        L = lib()
        return [L.exl3_checkpoint_name(self._h, i).decode() for i in range(L.exl3_checkpoint_count(self._h))]

    def has(self, name):
        return bool(lib().exl3_checkpoint_has(self._h, name.encode()))

    def info(self, name):
        """(dtype string, shape tuple, bytes)"""
        dt = C.create_string_buffer(16)
        shape = (C.c_int64 * 8)()
        nd, nb = C.c_int(), C.c_uint64()
        self._check(lib().exl3_checkpoint_info(self._h, name.encode(), dt, 16, shape, 8, C.byref(nd), C.byref(nb)), name)
        return dt.value.decode(), tuple(shape[i] for i in range(nd.value)), nb.value

    def read(self, name, out, stream=None):
        """the tensor's bytes into the CUDA tensor `out` (same byte size)"""
        st = C.c_void_p(stream.cuda_stream if stream is not None else torch.cuda.current_stream().cuda_stream)
        self._check(lib().exl3_checkpoint_read(self._h, name.encode(), _ptr(out), out.numel() * out.element_size(), st), name)
        return out

    def linear(self, key, in_features, out_features, alt_key=None, trim_padded_out=False, softcap=0.0, stream=None):
        """Linear::load -> LinearLayer (free it with `free_linear`)."""
        layer = LinearLayer()
        st = C.c_void_p(stream.cuda_stream if stream is not None else torch.cuda.current_stream().cuda_stream)
        self._check(lib().exl3_linear_load(self._h, st, key.encode(), alt_key.encode() if alt_key else None, in_features,
                                           out_features, int(trim_padded_out), softcap, C.byref(layer)), key)
        return layer

    @staticmethod
    def free_linear(layer):
        lib().exl3_linear_free(C.byref(layer))


class CudaGraph:
    """RAII wrapper like src/ffi.rs:403-451: capture ops launched on ctx.side_stream, then replay."""

    def __init__(self, ctx):
        self.ctx = ctx
        self._g = lib().exl3_graph_new(ctx.handle)
        if not self._g:
            raise Exl3Error("exl3_graph_new failed")

    def capture_begin(self):
        if lib().exl3_graph_capture_begin(C.c_void_p(self._g)) != 0:
            raise Exl3Error("graph capture_begin failed")

    def capture_end(self):
        if lib().exl3_graph_capture_end(C.c_void_p(self._g)) != 0:
            raise Exl3Error("graph capture_end failed")

    def replay(self):
        if lib().exl3_graph_replay(C.c_void_p(self._g)) != 0:
            raise Exl3Error("graph replay failed")

    def side_stream(self):
        return int(lib().exl3_side_stream(self.ctx.handle) or 0)

    def __del__(self):
        try:
            if self._g:
                lib().exl3_graph_free(C.c_void_p(self._g))
                self._g = None
        except Exception:
            pass
