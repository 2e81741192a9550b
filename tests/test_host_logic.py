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
