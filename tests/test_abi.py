"""The C-ABI library loads and exports every symbol include/orangu_b200.h declares (no GPU needed)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from orangu_b200 import build, capi

    build.build_all()
    return capi.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "orangu_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ob_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    from orangu_b200 import capi

    names = declared_symbols()
    assert len(names) >= 30
    assert set(names) == set(capi.SIGNATURES), set(names) ^ set(capi.SIGNATURES)
    for n in names:
        assert hasattr(lib, n), f"library does not export {n}"


def test_constants_without_a_device(lib):
    assert lib.ob_abi_version() == 1
    assert [lib.ob_supports_type(t) for t in (0, 8, 12, 14, 2, 6, 20)] == [1, 1, 1, 1, 1, 1, 1]
    assert [lib.ob_supports_type(t) for t in (1, 3, 7, 10, 13, 30)] == [0, 0, 0, 0, 0, 0]
    assert lib.ob_reduced_surface() is None


def test_init_without_a_device_is_a_status_not_a_crash(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    h = C.c_void_p()
    rc = lib.ob_init(0, C.byref(h))
    assert rc == -3 and not h.value
    assert b"CUDA" in lib.ob_last_error(None) or lib.ob_last_error(None)
    from orangu_b200 import CudaBackend

    assert CudaBackend.try_init_index(0) is None  # Option::None, as try_init_index returns


def test_null_arguments_are_rejected(lib):
    assert lib.ob_init(0, None) == -1
    assert lib.ob_matmul(None, None, 1, None, None) == -1
    assert lib.ob_kv_len(None) == 0
    assert lib.ob_tp_unique_id(None) == -1


def test_cpp_host_wrapper_compiles():
    """include/orangu_b200.hpp (the C++ mirror of the Backend trait) must at least compile against the C header."""
    import subprocess, tempfile

    hpp = os.path.join(ROOT, "include", "orangu_b200.hpp")
    if not os.path.exists(hpp):
        pytest.skip("no C++ wrapper")
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "t.cpp")
        open(src, "w").write('#include "orangu_b200.hpp"\nint main(){ return orangu::CudaBackend::try_init_index(0) ? 0 : 0; }\n')
        r = subprocess.run(["/usr/bin/g++", "-std=c++17", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), src], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
