"""CPU-side checks of the C ABI: the shared library loads, exports exactly what
include/aion_cuda.h declares, and argument errors come back as status codes (no GPU needed
for those that fail before any CUDA call)."""
import ctypes as C
import os
import re

from aion_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "aion_cuda.h")).read()
    return sorted(set(re.findall(r"AION_CUDA_API\s+[\w\s\*]+?\b(aion_cuda_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    declared = _declared_symbols()
    assert declared, "no declarations parsed"
    assert sorted(capi.SIGNATURES) == declared


def test_library_exports_every_declared_symbol():
    lib = capi.load()
    for name in _declared_symbols():
        assert hasattr(lib, name), name


def test_struct_sizes_match_the_header_layout():
    assert C.sizeof(capi.Operand) == 24
    assert C.sizeof(capi.MatMul) == 3 * 24 + 8 + 6 * 8 + 8
    assert C.sizeof(capi.MatMulNT) == 3 * 24 + 16 + 6 * 8 + 8
    assert C.sizeof(capi.Attention) == 6 * 24 + 16 + 7 * 8 + 8 + 16


def test_null_arguments_are_rejected_with_a_message():
    lib = capi.load()
    assert lib.aion_cuda_matmul(None, None) == capi.INVALID_ARGUMENT
    assert "null" in capi.last_error()
    assert lib.aion_cuda_device_create(0, None) == capi.INVALID_ARGUMENT
    assert lib.aion_cuda_sync(None) == capi.INVALID_ARGUMENT
    n = C.c_size_t()
    lib.aion_cuda_last_error(None, 0, C.byref(n))
    assert n.value > 0
