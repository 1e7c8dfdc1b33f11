"""CPU-only checks of the C-ABI boundary: the in-tree library loads and exports every function that
include/dgen_cuda.h declares; argument validation that needs no device."""
import ctypes as C
import os
import re

import dgen_b200

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "dgen_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dgc_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(dgen_b200.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), "libdgen_cuda.so does not export " + n


def test_python_binding_covers_the_header():
    assert sorted(dgen_b200.SIGNATURES) == declared_functions()


def test_abi_version_and_null_context_errors():
    lib = dgen_b200.load()
    assert lib.dgc_abi_version() == 1
    assert lib.dgc_sync(None, 0) == -1
    assert lib.dgc_launch_count(None) == -1
    assert lib.dgc_mss_partial_floats(None) == 0
    p = dgen_b200.mss_params(16, 64000)
    hops = [s // 4 for s in (2048, 1024, 512, 256, 128, 64)]
    want = sum(2 * ((64000 + h - 1) // h) * 16 for h in hops)
    assert lib.dgc_mss_partial_floats(C.byref(p)) == want
    # windows longer than the render are skipped, as the reference's usableWindows filter does
    q = dgen_b200.mss_params(2, 100, sizes=(2048, 64))
    assert lib.dgc_mss_partial_floats(C.byref(q)) == 2 * ((100 + 15) // 16) * 2


def test_no_cpu_fallback():
    import pytest
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    with pytest.raises(dgen_b200.DgenCudaError):
        dgen_b200.Context(0)
