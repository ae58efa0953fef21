"""CPU-side checks of the C ABI: the shared library loads, exports exactly what
include/aion_cuda.h declares, and argument errors come back as status codes (no GPU needed
for those that fail before any CUDA call)."""
import ctypes as C
import os
import re
import subprocess

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


STRUCTS = {"AionCudaOperand": capi.Operand, "AionCudaDeviceInfo": capi.DeviceInfo, "AionCudaMatMul": capi.MatMul,
           "AionCudaMatMulPlan": capi.MatMulPlan, "AionCudaMatMulNT": capi.MatMulNT, "AionCudaAttention": capi.Attention,
           "AionCudaRMSNorm": capi.RMSNorm, "AionCudaElemwise": capi.Elemwise, "AionCudaRoPE": capi.RoPE,
           "AionCudaCast": capi.Cast, "AionCudaSequenceAppend": capi.SequenceAppend, "AionCudaGatherRows": capi.GatherRows,
           "AionCudaArgMax": capi.ArgMax, "AionCudaRMSNormPair": capi.RMSNormPair, "AionCudaRopeKVAppend": capi.RopeKVAppend,
           "AionCudaPeerFanout": capi.PeerFanout}


def test_struct_layouts_match_the_header(tmp_path):
    """Every struct the header declares, compiled by the C compiler, has the size and the field
    offsets of its ctypes mirror."""
    text = open(os.path.join(ROOT, "include", "aion_cuda.h")).read()
    declared = set(re.findall(r"typedef struct \w+ \{[^}]*\} (\w+);", text))
    assert declared == set(STRUCTS), declared ^ set(STRUCTS)
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{os.path.join(ROOT, "include", "aion_cuda.h")}"',
             "int main(void) {"]
    for name, ct in STRUCTS.items():
        lines.append(f'printf("{name} %zu\\n", sizeof({name}));')
        for field, _ in ct._fields_:
            cfield = field[:-1] if field.endswith("_") and field != "_" else field  # `in_` mirrors the C field `in`
            lines.append(f'printf("{name}.{field} %zu\\n", offsetof({name}, {cfield}));')
    lines.append("return 0; }")
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c11", "-o", str(exe), str(src)], check=True)
    out = dict(line.split() for line in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for name, ct in STRUCTS.items():
        assert int(out[name]) == C.sizeof(ct), name
        for field, _ in ct._fields_:
            assert int(out[f"{name}.{field}"]) == getattr(ct, field).offset, f"{name}.{field}"


def test_null_arguments_are_rejected_with_a_message():
    lib = capi.load()
    assert lib.aion_cuda_matmul(None, None) == capi.INVALID_ARGUMENT
    assert "null" in capi.last_error()
    assert lib.aion_cuda_device_create(0, None) == capi.INVALID_ARGUMENT
    assert lib.aion_cuda_sync(None) == capi.INVALID_ARGUMENT
    n = C.c_size_t()
    lib.aion_cuda_last_error(None, 0, C.byref(n))
    assert n.value > 0
