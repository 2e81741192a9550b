"""Step-level binding: ctypes mirrors of exl3_linear / exl3_layer / exl3_model / exl3_batch (include/exl3_abi.h) and
helpers that build a synthetic dense EXL3 model and paged pools on the device.  The role of the reference's
src/paged.rs pools and src/generator.rs step construction, over the C-ABI."""
import ctypes as C

import numpy as np
import torch

from .ffi import Exl3Error, Linear, lib


class Layer(C.Structure):
    _fields_ = [(n, Linear) for n in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")] + \
               [(n, C.c_void_p) for n in ("attn_norm", "mlp_norm", "q_norm", "k_norm", "k_cache", "v_cache",
                                          "qk", "sk", "qv", "sv")]


class Model(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("hidden", C.c_int), ("nq", C.c_int), ("nkv", C.c_int), ("hd", C.c_int),
                ("inter", C.c_int), ("vocab", C.c_int), ("kv_bits", C.c_int), ("pages", C.c_int),
                ("norm_eps", C.c_float), ("attn_factor", C.c_float), ("rope_mode", C.c_int), ("n_freq", C.c_int),
                ("inv_freq", C.c_void_p), ("embed", C.c_void_p), ("final_norm", C.c_void_p), ("lm_head", Linear),
                ("layers", C.POINTER(Layer))]


class Batch(C.Structure):
    _fields_ = [("ids", C.c_void_p), ("q_lens", C.c_void_p), ("cache_seqlens", C.c_void_p), ("block_table", C.c_void_p),
                ("bsz", C.c_int), ("rows", C.c_int), ("max_q_len", C.c_int), ("pages_per_seq", C.c_int),
                ("advance", C.c_int), ("all_rows", C.c_int)]


def _randint16(shape, gen, device):
    return torch.randint(-32768, 32768, shape, dtype=torch.int16, device=device, generator=gen)


class SyntheticLinear:
    """Seeded random EXL3 tensor: uniform trellis codes, +-1 sign vectors; svh is scaled by `out_scale` so that a stack of
    layers keeps activations in fp16 range (the decoded codebooks have unit-order variance)."""

    def __init__(self, k, n, K, cb, gen, device, out_scale=None):
        self.k, self.n, self.K, self.cb = k, n, K, cb
        self.trellis = _randint16((k // 16, n // 16, 16 * K), gen, device)
        self.suh = (torch.randint(0, 2, (k,), device=device, generator=gen) * 2 - 1).to(torch.float16)
        sc = (1.0 / np.sqrt(k)) if out_scale is None else out_scale
        self.svh = ((torch.randint(0, 2, (n,), device=device, generator=gen) * 2 - 1).to(torch.float32) * sc).to(torch.float16)

    def struct(self):
        return Linear(self.trellis.data_ptr(), self.suh.data_ptr(), self.svh.data_ptr(), self.k, self.n, self.K, self.cb)


class SyntheticModel:
    """Dense transformer with seeded random EXL3 weights and its paged KV pools, resident on one device."""

    def __init__(self, n_layers, hidden, nq, nkv, hd, inter, vocab, K=4, cb=1, pages=64, kv_bits=0, seed=0,
                 device="cuda", rope_theta=1e6, qk_norm=True, head_K=None, pool=None):
        """`pool` (exl3b200.Pool): the KV planes are the pool's instead of tensors allocated here"""
        self.cfg = dict(n_layers=n_layers, hidden=hidden, nq=nq, nkv=nkv, hd=hd, inter=inter, vocab=vocab, K=K, cb=cb,
                        pages=pages, kv_bits=kv_bits)
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        self.device = device
        f16 = dict(dtype=torch.float16, device=device)

        def normw(n):
            return (1.0 + 0.1 * torch.randn(n, device=device, generator=g)).to(torch.float16)

        self.embed = (torch.randn(vocab, hidden, device=device, generator=g)).to(torch.float16)
        self.final_norm = normw(hidden)
        self.lm_head = SyntheticLinear(hidden, vocab, head_K or K, cb, g, device)
        self.inv_freq = (1.0 / (rope_theta ** (torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd))).contiguous()
        self.layers = []
        groups = nkv * hd // 32
        for _ in range(n_layers):
            L = dict(q_proj=SyntheticLinear(hidden, nq * hd, K, cb, g, device),
                     k_proj=SyntheticLinear(hidden, nkv * hd, K, cb, g, device),
                     v_proj=SyntheticLinear(hidden, nkv * hd, K, cb, g, device),
                     o_proj=SyntheticLinear(nq * hd, hidden, K, cb, g, device),
                     gate_proj=SyntheticLinear(hidden, inter, K, cb, g, device),
                     up_proj=SyntheticLinear(hidden, inter, K, cb, g, device),
                     down_proj=SyntheticLinear(inter, hidden, K, cb, g, device),
                     attn_norm=normw(hidden), mlp_norm=normw(hidden),
                     q_norm=normw(hd) if qk_norm else None, k_norm=normw(hd) if qk_norm else None)
            if pool is not None:
                pass
            elif kv_bits == 0:
                L["k_cache"] = torch.zeros(pages, 256, nkv, hd, **f16)
                L["v_cache"] = torch.zeros(pages, 256, nkv, hd, **f16)
            else:
                L["qk"] = torch.zeros(pages, 256, groups * kv_bits, dtype=torch.int32, device=device)
                L["qv"] = torch.zeros(pages, 256, groups * kv_bits, dtype=torch.int32, device=device)
                L["sk"] = torch.zeros(pages, 256, groups, **f16)
                L["sv"] = torch.zeros(pages, 256, groups, **f16)
            self.layers.append(L)
        self._layer_array = (Layer * n_layers)()
        for i, L in enumerate(self.layers):
            s = self._layer_array[i]
            for n in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"):
                setattr(s, n, L[n].struct())
            for n in ("attn_norm", "mlp_norm", "q_norm", "k_norm", "k_cache", "v_cache", "qk", "sk", "qv", "sv"):
                t = L.get(n)
                setattr(s, n, None if t is None else t.data_ptr())
            if pool is not None:
                k, v, sk, sv = pool.layer(i)
                if kv_bits == 0:
                    s.k_cache, s.v_cache = k, v
                else:
                    s.qk, s.qv, s.sk, s.sv = k, v, sk, sv
        self.pool = pool
        self.struct = Model(n_layers, hidden, nq, nkv, hd, inter, vocab, kv_bits, pages, 1e-6, 1.0, 2,
                            self.inv_freq.numel(), self.inv_freq.data_ptr(), self.embed.data_ptr(),
                            self.final_norm.data_ptr(), self.lm_head.struct(), self._layer_array)
        self._scratch = None

    def fill_kv(self, std=0.5, seed=1, chunk_pages=64):
        """Fill the pools with synthetic context: N(0, std^2) values in fp16 pools; in quantised pools uniform random codes
        (every bit pattern is a valid code) with group scales uniform in [0.01, 0.06], i.e. values of the same magnitude."""
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        c = self.cfg
        for L in self.layers:
            if c["kv_bits"] == 0:
                for name in ("k_cache", "v_cache"):
                    t = L[name]
                    for p0 in range(0, c["pages"], chunk_pages):
                        sl = t[p0:p0 + chunk_pages]
                        sl.copy_((torch.randn(sl.shape, device=self.device, generator=g) * std).to(torch.float16))
            else:
                for name in ("qk", "qv"):
                    t = L[name]
                    for p0 in range(0, c["pages"], chunk_pages):
                        sl = t[p0:p0 + chunk_pages]
                        sl.copy_(torch.randint(-2 ** 31, 2 ** 31 - 1, sl.shape, dtype=torch.int32, device=self.device, generator=g))
                for name in ("sk", "sv"):
                    t = L[name]
                    for p0 in range(0, c["pages"], chunk_pages):
                        sl = t[p0:p0 + chunk_pages]
                        sl.copy_((torch.rand(sl.shape, device=self.device, generator=g) * 0.05 + 0.01).to(torch.float16))

    def weight_bytes(self):
        b = self.lm_head.trellis.numel() * 2
        for L in self.layers:
            for n in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"):
                b += L[n].trellis.numel() * 2
        return b

    def step(self, ctx, ids, q_lens, cache_seqlens, block_table, max_q_len, advance=False, want_logits=False, stream=None,
             tokens_out=None, all_rows=False):
        """ids int64 [rows], q_lens/cache_seqlens int32 [bsz], block_table int32 [bsz,pps] (device).  Returns tokens
        (int64 [bsz]) and, if asked, fp32 logits [bsz, vocab]; with `all_rows` one token (and logits row) per packed row.
        `tokens_out` (int64, device) makes the call allocation-free once the scratch exists, which is what a CUDA-graph
        capture of the step needs."""
        L = lib()
        L.exl3_step_scratch_bytes.restype = C.c_size_t
        L.exl3_step_scratch_bytes.argtypes = [C.POINTER(Model), C.c_int, C.c_int, C.c_int]
        bsz, rows = q_lens.numel(), ids.numel()
        need = L.exl3_step_scratch_bytes(C.byref(self.struct), rows, bsz, int(all_rows))
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(need, dtype=torch.uint8, device=self.device)
        n_out = rows if all_rows else bsz
        tokens = tokens_out if tokens_out is not None else torch.empty(n_out, dtype=torch.int64, device=self.device)
        logits = torch.empty(n_out, self.cfg["vocab"], dtype=torch.float32, device=self.device) if want_logits else None
        batch = Batch(ids.data_ptr(), q_lens.data_ptr(), cache_seqlens.data_ptr(), block_table.data_ptr(), bsz, rows,
                      max_q_len, block_table.shape[1], int(advance), int(all_rows))
        rc = L.exl3_step_forward(ctx.handle, ctx.stream(stream), C.byref(self.struct), C.byref(batch),
                                 C.c_void_p(self._scratch.data_ptr()), C.c_size_t(self._scratch.numel()),
                                 C.c_void_p(tokens.data_ptr()), C.c_void_p(0 if logits is None else logits.data_ptr()))
        if rc != 0:
            raise Exl3Error(f"exl3_step_forward failed ({rc}): {L.exl3_last_error(ctx.handle).decode()}")
        return tokens, logits


class LoadedModel:
    """A dense model read from safetensors files by exl3_model_load (Model::load, src/model.rs:262-420) into device memory
    owned by the library; KV planes come from `pool`.  `step` is SyntheticModel.step."""

    def __init__(self, paths, pool, n_layers, hidden, nq, nkv, hd, inter, vocab, norm_eps=1e-6, rope_theta=1e6,
                 prefix="model", device="cuda", stream=None):
        from .ffi import Checkpoint
        L = lib()
        L.exl3_model_load.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_void_p, C.c_char_p] + [C.c_int] * 7 + \
                                     [C.c_float, C.c_float, C.c_void_p, C.POINTER(C.c_void_p)]
        L.exl3_model_get.argtypes = [C.c_void_p]; L.exl3_model_get.restype = C.POINTER(Model)
        L.exl3_model_error.argtypes = [C.c_void_p]; L.exl3_model_error.restype = C.c_char_p
        L.exl3_model_free.argtypes = [C.c_void_p]
        self.device, self.pool, self._scratch, self._h = device, pool, None, None
        cks = [Checkpoint(p) for p in paths]
        try:
            arr = (C.c_void_p * len(cks))(*[c._h for c in cks])
            h = C.c_void_p()
            st = C.c_void_p(stream.cuda_stream if stream is not None else torch.cuda.current_stream().cuda_stream)
            rc = L.exl3_model_load(arr, len(cks), st, prefix.encode(), n_layers, hidden, nq, nkv, hd, inter, vocab,
                                   norm_eps, rope_theta, pool._h, C.byref(h))
            self._h = h
            if rc != 0:
                msg = L.exl3_model_error(h).decode() if h else "out of memory"
                self.close()
                raise Exl3Error(f"exl3_model_load: {msg} (code {rc})")
        finally:
            for c in cks:
                c.close()
        self.struct = L.exl3_model_get(self._h).contents
        self.cfg = dict(n_layers=n_layers, hidden=hidden, nq=nq, nkv=nkv, hd=hd, inter=inter, vocab=vocab,
                        pages=self.struct.pages, kv_bits=self.struct.kv_bits)

    def close(self):
        if self._h:
            lib().exl3_model_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    step = SyntheticModel.step

