"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the public header
declares, and the functions that need no GPU behave.  No compute entry point is called here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "lutgemm.h")
LIB = os.path.join(ROOT, "appmult-aware-retraining_b200", "liblutgemm_b200.so")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lutgemm_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB):
        import importlib.util
        spec = importlib.util.spec_from_file_location(
            "build_ext", os.path.join(ROOT, "appmult-aware-retraining_b200", "build_ext.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    return ctypes.CDLL(LIB)


def test_header_declares_the_expected_entry_points():
    syms = declared_symbols()
    for s in ("lutgemm_forward", "lutgemm_backward", "lutgemm_backward_scratch_bytes", "lutgemm_lut_elem_num",
              "lutgemm_bits_from_elem_num", "lutgemm_status_string", "lutgemm_version", "lutgemm_device_error",
              "lutgemm_selftest_bounded_wait", "lutgemm_conv2d_forward", "lutgemm_conv2d_backward",
              "lutgemm_conv2d_backward_scratch_bytes", "lutgemm_backward_gw_noalloc"):
        assert s in syms


def test_library_exports_every_declared_symbol(lib):
    for s in declared_symbols():
        assert hasattr(lib, s), f"{s} declared in include/lutgemm.h but not exported"


def test_geometry_functions(lib):
    lib.lutgemm_bits_from_elem_num.argtypes = [ctypes.c_long]
    assert [lib.lutgemm_lut_elem_num(b) for b in (4, 6, 7, 8)] == [1024, 5120, 17408, 66306]
    assert lib.lutgemm_lut_elem_num(5) == -2
    assert [lib.lutgemm_bits_from_elem_num(n) for n in (1024, 5120, 17408, 66306)] == [4, 6, 7, 8]
    assert lib.lutgemm_bits_from_elem_num(12345) == -2
    assert lib.lutgemm_version() >= 100


def test_status_strings(lib):
    lib.lutgemm_status_string.restype = ctypes.c_char_p
    assert lib.lutgemm_status_string(0) == b"ok"
    for code in (-1, -2, -4, -5):
        assert len(lib.lutgemm_status_string(code)) > 3


def test_bad_arguments_are_rejected_before_any_cuda_call(lib):
    vp = ctypes.c_void_p
    lib.lutgemm_forward.argtypes = [vp, vp, vp, vp] + [ctypes.c_int] * 4 + [vp]
    assert lib.lutgemm_forward(None, None, None, None, 5, 1, 1, 1, None) == -2   # bits
    assert lib.lutgemm_forward(None, None, None, None, 7, 1, 1, 1, None) == -1   # null pointers
    assert lib.lutgemm_forward(16, 16, 16, 16, 7, 0, 1, 1, None) == -1           # empty problem
    lib.lutgemm_backward.argtypes = [vp] * 7 + [ctypes.c_int] * 4 + [vp, ctypes.c_size_t, vp]
    assert lib.lutgemm_backward(None, None, None, None, None, None, None, 3, 1, 1, 1, None, 0, None) == -2
    assert lib.lutgemm_backward(None, None, None, None, None, None, None, 8, 1, 1, 1, None, 0, None) == -1
