"""The decode step composed from oracle ops in the reference's op order (src/model.rs:1171-1194,
src/modules.rs:634-789,932-940,1020-1035, src/model.rs:1038-1050).  Test infrastructure only (also the CPU-baseline leg of the benchmark)."""
import numpy as np

from oracle import oracle as O


def _np(t):
    return None if t is None else t.detach().cpu().numpy()


def model_to_numpy(model):
    """Copy a device SyntheticModel's weights and pools to numpy."""
    out = dict(cfg=dict(model.cfg), embed=_np(model.embed), final_norm=_np(model.final_norm),
               inv_freq=_np(model.inv_freq), layers=[])

    def lin(l):
        return dict(trellis=_np(l.trellis), suh=_np(l.suh), svh=_np(l.svh), K=l.K, cb=l.cb)

    out["lm_head"] = lin(model.lm_head)
    cfg = model.cfg
    for L in model.layers:
        d = {}
        for n, v in L.items():
            d[n] = lin(v) if hasattr(v, "trellis") else _np(v)
        if "k_cache" not in d and "qk" not in d:
            # planes owned by a pool object start zeroed: the same on this side
            if cfg["kv_bits"] == 0:
                d["k_cache"] = np.zeros((cfg["pages"], 256, cfg["nkv"], cfg["hd"]), np.float16)
                d["v_cache"] = np.zeros_like(d["k_cache"])
            else:
                groups = cfg["nkv"] * cfg["hd"] // 32
                d["qk"] = np.zeros((cfg["pages"], 256, groups * cfg["kv_bits"]), np.int32); d["qv"] = np.zeros_like(d["qk"])
                d["sk"] = np.zeros((cfg["pages"], 256, groups), np.float16); d["sv"] = np.zeros_like(d["sk"])
        out["layers"].append(d)
    return out


def _linear(x, w, c_fp32=False):
    return O.exl3_gemm(x, w["trellis"], w["suh"], w["svh"], w["K"], w["cb"], c_fp32=c_fp32)


def step(m, ids, q_lens, seqlens, block_table):
    """Returns (tokens [bsz], logits [bsz, vocab] fp32); updates the numpy pools in m in place."""
    cfg = m["cfg"]
    nq, nkv, hd = cfg["nq"], cfg["nkv"], cfg["hd"]
    bsz = len(q_lens)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    rows = int(cu[-1])
    row_pos = np.concatenate([seqlens[b] + np.arange(q_lens[b]) for b in range(bsz)]).astype(np.int32)
    resid = O.embed(ids, m["embed"])
    pending = None
    for L in m["layers"]:
        if pending is None:
            a_in = O.rms_norm(resid, L["attn_norm"], 1e-6)
        else:
            a_in = O.rms_norm(pending, L["attn_norm"], 1e-6, res=resid)
        q = _linear(a_in, L["q_proj"]).reshape(rows, 1, nq, hd)
        k = _linear(a_in, L["k_proj"]).reshape(rows, 1, nkv, hd)
        v = _linear(a_in, L["v_proj"]).reshape(rows, 1, nkv, hd)
        # one "sequence" per row with its own position: same arithmetic as positions[b] + t
        q, k = O.rope(q, k, m["inv_freq"], 0, row_pos, L["q_norm"], L["k_norm"], 1e-6, 0.0, 2, 1.0)
        q = q.reshape(rows, nq, hd); k = k.reshape(rows, nkv, hd); v = v.reshape(rows, nkv, hd)
        if cfg["kv_bits"] == 0:
            for b in range(bsz):
                if q_lens[b]:
                    O.paged_kv_update(k[None, cu[b]:cu[b + 1]], v[None, cu[b]:cu[b + 1]], L["k_cache"], L["v_cache"],
                                      block_table[b:b + 1], seqlens[b:b + 1])
            o = O.attn_paged(q, L["k_cache"], L["v_cache"], block_table, seqlens, cu_q=cu)
        else:
            bits = cfg["kv_bits"]
            for b in range(bsz):
                if q_lens[b]:
                    O.quant_cache_paged(k[None, cu[b]:cu[b + 1]], L["qk"].view(np.uint32), L["sk"], v[None, cu[b]:cu[b + 1]],
                                        L["qv"].view(np.uint32), L["sv"], seqlens[b:b + 1], block_table[b:b + 1], bits, bits)
            o = O.attn_paged(q, None, None, block_table, seqlens, cu_q=cu, nkv=nkv,
                             quant=(L["qk"].view(np.uint32), L["sk"], L["qv"].view(np.uint32), L["sv"], bits))
        proj = _linear(o.reshape(rows, nq * hd), L["o_proj"])
        m_in = O.rms_norm(proj, L["mlp_norm"], 1e-6, res=resid)
        act = O.silu_mul(_linear(m_in, L["gate_proj"]), _linear(m_in, L["up_proj"]))
        pending = _linear(act, L["down_proj"])
    last = np.array([cu[b + 1] - 1 for b in range(bsz)])
    r_last = np.ascontiguousarray(resid[last])
    y = O.rms_norm(np.ascontiguousarray(pending[last]), m["final_norm"], 1e-6, res=r_last)
    logits = _linear(y, m["lm_head"], c_fp32=True)
    return O.argmax(logits), logits
