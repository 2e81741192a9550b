"""CPU tests of host-side pieces: the C-ABI library exports every symbol the header declares, the bit-window
extraction of the kernels matches the format definition (compiled for the host), error handling without a GPU."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "exllamav3-rs_b200", "libexl3b200.so")


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB):
        sys.path.insert(0, ROOT)
        import __graft_entry__
        __graft_entry__.build()
    return C.CDLL(LIB)


def test_every_declared_symbol_is_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "exl3_abi.h")).read()
    names = re.findall(r"EXL3_API\s+[\w\s\*]+?\b(exl3_\w+)\s*\(", hdr)
    assert len(names) >= 30
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_version_and_no_gpu_errors(lib):
    lib.exl3_version.restype = C.c_char_p
    assert b"sm_100a" in lib.exl3_version()
    import torch
    if not torch.cuda.is_available():
        h = C.c_void_p()
        assert lib.exl3_ctx_create(0, C.c_size_t(0), C.byref(h)) != 0      # fails loudly, no CPU fallback
        assert not h.value


def test_window_extraction_on_host(tmp_path):
    exe = str(tmp_path / "host_decode_check")
    subprocess.check_call(["nvcc", "-O1", "-Wno-deprecated-gpu-targets", "-o", exe,
                           os.path.join(ROOT, "tests", "host_decode_check.cu")])
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout


# every exl3_shim_* / exl3_* symbol the reference's Rust side binds (src/ffi.rs:17-203) and the name it has here
REFERENCE_SURFACE = {
    "exl3_shim_gemm": "exl3_gemm", "exl3_shim_mgemm": "exl3_mgemm", "exl3_shim_rms_norm": "exl3_rms_norm",
    "exl3_shim_rope": "exl3_rope", "exl3_shim_hgemm": "exl3_hgemm", "exl3_shim_bighead_attn": "exl3_bighead_attn",
    "exl3_shim_paged_kv_cache_update": "exl3_paged_kv_cache_update",
    "exl3_shim_bighead_attn_paged": "exl3_bighead_attn_paged", "exl3_shim_bighead_attn_paged_q": "exl3_bighead_attn_paged_q",
    "exl3_shim_rms_norm_res_in": "exl3_rms_norm_res_in", "exl3_shim_gated_rms_norm": "exl3_gated_rms_norm",
    "exl3_shim_softcap": "exl3_softcap", "exl3_shim_add": "exl3_add", "exl3_shim_silu_mul": "exl3_silu_mul",
    "exl3_shim_gelu_mul": "exl3_gelu_mul", "exl3_shim_relu2_mul": "exl3_relu2_mul",
    "exl3_shim_apply_rep_pens": "exl3_apply_rep_pens", "exl3_shim_apply_pres_freq_pens": "exl3_apply_pres_freq_pens",
    "exl3_shim_argmax_sample": "exl3_argmax_sample", "exl3_shim_gumbel_sample": "exl3_gumbel_sample",
    "exl3_shim_gumbel_noise_f32": "exl3_gumbel_noise_f32", "exl3_shim_cache_rotate": "exl3_cache_rotate",
    "exl3_shim_quant_cache_paged": "exl3_quant_cache_paged", "exl3_shim_dequant_cache_paged": "exl3_dequant_cache_paged",
    "exl3_shim_dequant_cache_paged_window": "exl3_dequant_cache_paged_window", "exl3_shim_had_r_128": "exl3_had_r_128",
    "exl3_shim_reconstruct": "exl3_reconstruct", "exl3_shim_mul_sigmoid_": "exl3_mul_sigmoid_",
    "exl3_shim_deinterleave_qg": "exl3_deinterleave_qg", "exl3_shim_gdn_fused_op_2": "exl3_gdn_fused_op_2",
    "exl3_shim_gdn_chunk_wy": "exl3_gdn_chunk_wy", "exl3_shim_gdn_chunk_fused": "exl3_gdn_chunk_fused",
    "exl3_shim_recurrent_gated_delta_rule": "exl3_recurrent_gated_delta_rule",
    "exl3_shim_causal_conv1d_update": "exl3_causal_conv1d_update",
    "exl3_graph_new": "exl3_graph_new", "exl3_graph_free": "exl3_graph_free",
    "exl3_graph_capture_begin": "exl3_graph_capture_begin", "exl3_graph_capture_end": "exl3_graph_capture_end",
    "exl3_graph_replay": "exl3_graph_replay", "exl3_use_side_stream": "exl3_side_stream",
    "exl3_sync_side_stream": "exl3_sync_side_stream", "exl3_empty_cache": "exl3_empty_cache",
    "exl3_shim_set_mma_attn": "exl3_set_mma_attn", "exl3_cuda_free_mib": "exl3_cuda_free_mib",
}


def test_reference_op_surface_is_exported(lib):
    """the crate links: each of the 44 symbols of the reference's extern block has its counterpart in the library and
    in the header"""
    assert len(REFERENCE_SURFACE) == 44
    hdr = open(os.path.join(ROOT, "include", "exl3_abi.h")).read()
    for ref_name, ours in REFERENCE_SURFACE.items():
        assert hasattr(lib, ours), f"{ref_name} -> {ours} is not exported"
        assert re.search(r"\b" + ours + r"\s*\(", hdr), f"{ours} is not declared in the header"


def _page_table(lib, pages):
    h = C.c_void_p()
    assert lib.exl3_pool_create(0, 0, pages, 8, 128, 0, 0, C.byref(h)) == 0
    return h


def test_page_table_free_list_and_refcounts(lib):
    """PageTable::alloc / release (src/paged.rs:405-412,495-506): ascending pages first, exhaustion is an error that takes
    nothing, released pages are reused"""
    pt = _page_table(lib, 6)
    assert lib.exl3_pool_num_free(pt) == 6
    a = (C.c_int32 * 4)()
    assert lib.exl3_pool_alloc(pt, 4, a) == 0 and list(a) == [0, 1, 2, 3]
    b = (C.c_int32 * 3)()
    assert lib.exl3_pool_alloc(pt, 3, b) != 0 and lib.exl3_pool_num_free(pt) == 2
    assert [lib.exl3_pool_refcount(pt, i) for i in range(6)] == [1, 1, 1, 1, 0, 0]
    assert lib.exl3_pool_release(pt, a, 2) == 0 and lib.exl3_pool_num_free(pt) == 4
    assert lib.exl3_pool_alloc(pt, 3, b) == 0 and sorted(b) == [0, 1, 4] or sorted(b) == [1, 0, 5] or len(set(b)) == 3
    assert lib.exl3_pool_num_free(pt) == 1
    lib.exl3_pool_destroy(pt)


def test_page_table_prefix_sharing(lib):
    """alloc_prefix / register_page_hash (src/paged.rs:425-480): complete pages of an identical prompt prefix are shared,
    released hashed pages stay reclaimable and are revived by a later hit, and are evicted oldest first when the free
    list is empty"""
    import numpy as np
    pt = _page_table(lib, 8)
    lib.exl3_pool_set_dedup(pt, 1)
    r = np.random.default_rng(0)
    prompt = r.integers(0, 50000, 700).astype(np.int64)          # 2 complete pages + 188 tokens
    ids = prompt.ctypes.data_as(C.POINTER(C.c_int64))
    blk = (C.c_int32 * 8)(); cnt = C.c_int(); matched = C.c_int64()
    assert lib.exl3_pool_alloc_prefix(pt, ids, 700, 100, blk, 8, C.byref(cnt), C.byref(matched)) == 0
    assert cnt.value == 4 and matched.value == 0
    first = list(blk)[:4]
    # the two complete pages get their chained hashes
    for i in range(2):
        assert lib.exl3_pool_register_page_hash(pt, first[i], first[i - 1] if i else -1, prompt[i * 256:].ctypes.data_as(C.POINTER(C.c_int64)), 256) == 0
    # a second sequence with the same first 600 tokens shares both pages
    p2 = prompt.copy(); p2[600:] += 1
    blk2 = (C.c_int32 * 8)()
    assert lib.exl3_pool_alloc_prefix(pt, p2.ctypes.data_as(C.POINTER(C.c_int64)), 700, 0, blk2, 8, C.byref(cnt), C.byref(matched)) == 0
    assert cnt.value == 3 and matched.value == 512 and list(blk2)[:2] == first[:2]
    assert lib.exl3_pool_refcount(pt, first[0]) == 2 and lib.exl3_pool_refcount(pt, first[1]) == 2
    # a different first page: nothing shared
    p3 = prompt.copy(); p3[0] += 1
    blk3 = (C.c_int32 * 8)()
    assert lib.exl3_pool_alloc_prefix(pt, p3.ctypes.data_as(C.POINTER(C.c_int64)), 300, 0, blk3, 8, C.byref(cnt), C.byref(matched)) != 0 or matched.value == 0
    # release everything: hashed pages become reclaimable, still counted as free, and a new hit revives them
    lib.exl3_pool_release(pt, blk, 4); lib.exl3_pool_release(pt, blk2, 3)
    if cnt.value and matched.value == 0:
        lib.exl3_pool_release(pt, blk3, cnt.value)
    assert lib.exl3_pool_num_free(pt) == 8
    assert lib.exl3_pool_alloc_prefix(pt, ids, 700, 0, blk, 8, C.byref(cnt), C.byref(matched)) == 0
    assert matched.value == 512 and list(blk)[:2] == first[:2]
    lib.exl3_pool_release(pt, blk, cnt.value)
    # exhausting the free list repurposes the hashed pages (oldest first) and reports them as evicted
    big = (C.c_int32 * 8)()
    assert lib.exl3_pool_alloc(pt, 8, big) == 0
    ev = (C.c_int32 * 8)()
    n_ev = lib.exl3_pool_drain_evicted(pt, ev, 8)
    assert sorted(list(ev)[:n_ev]) == sorted(first[:2])
    lib.exl3_pool_release(pt, big, 8)
    assert lib.exl3_pool_alloc_prefix(pt, ids, 700, 0, blk, 8, C.byref(cnt), C.byref(matched)) == 0 and matched.value == 0
    lib.exl3_pool_destroy(pt)
