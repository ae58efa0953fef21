"""ctypes binding of libaion_cuda's C ABI (include/aion_cuda.h), one declaration per symbol.

The library is the product; there is no Python or CPU fallback. Loading fails loudly
when the shared object has not been built (`python -m aion_b200.build`).
"""
from __future__ import annotations

import ctypes as C
import os

OK, INVALID_ARGUMENT, OUT_OF_MEMORY, UNSUPPORTED, INTERNAL_ERROR = range(5)
STATUS_NAMES = {0: "OK", 1: "INVALID_ARGUMENT", 2: "OUT_OF_MEMORY", 3: "UNSUPPORTED", 4: "INTERNAL_ERROR"}

DTYPE_F32, DTYPE_F16, DTYPE_I8, DTYPE_Q4_0, DTYPE_Q8_0, DTYPE_I32 = range(6)
ORDER_ROW_MAJOR, ORDER_LANES4, ORDER_LANES8, ORDER_LANES16, ORDER_LANES32, ORDER_LANES32X16 = range(6)
WINDOW_UNBOUNDED = 0xFFFFFFFF
MATMUL_AUTO, MATMUL_FORCE_GENERIC, MATMUL_FORCE_GEMV, MATMUL_FORCE_GEMM, MATMUL_ONE_SM = 0, 1, 2, 4, 8
INT8_GROUP_ROWS = 64
GEMM_MIN_M = 33
KERNEL_GENERIC, KERNEL_INT8, KERNEL_GEMM = 1, 2, 3
ELEMWISE_ADD, ELEMWISE_MUL, ELEMWISE_GATE_GELU = 0, 1, 2
RECORD_LANES = 8

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libaion_cuda.so")


class Operand(C.Structure):
    _fields_ = [("handle", C.c_uint64), ("offset", C.c_uint64), ("len", C.c_uint64)]


class DeviceInfo(C.Structure):
    _fields_ = [
        ("name", C.c_char * 128),
        ("ordinal", C.c_int32),
        ("sm_count", C.c_int32),
        ("cc_major", C.c_int32),
        ("cc_minor", C.c_int32),
        ("total_bytes", C.c_uint64),
        ("l2_bytes", C.c_uint64),
    ]


class MatMul(C.Structure):
    _fields_ = [
        ("c", Operand), ("a", Operand), ("b", Operand),
        ("b_dtype", C.c_uint32), ("flags", C.c_uint32),
        ("m", C.c_uint64), ("n", C.c_uint64), ("k", C.c_uint64),
        ("lda", C.c_uint64), ("ldb", C.c_uint64), ("ldc", C.c_uint64),
        ("alpha", C.c_float), ("beta", C.c_float),
        ("a_image", Operand),
    ]


class MatMulPlan(C.Structure):
    _fields_ = [("kernel", C.c_uint32), ("tile_rows", C.c_uint32), ("tile_cols", C.c_uint32), ("k_splits", C.c_uint32),
                ("grid", C.c_uint32), ("cta_pairs", C.c_uint32), ("reserved", C.c_uint32 * 2)]


class PeerFanout(C.Structure):
    _fields_ = [("world", C.c_uint32), ("rank", C.c_uint32), ("c", Operand * 8), ("flags", Operand * 8), ("state", Operand)]


class MatMulNT(C.Structure):
    _fields_ = [
        ("c", Operand), ("a", Operand), ("b", Operand),
        ("b_dtype", C.c_uint32), ("block_order", C.c_uint32), ("flags", C.c_uint32), ("reserved", C.c_uint32),
        ("m", C.c_uint64), ("n", C.c_uint64), ("k", C.c_uint64),
        ("lda", C.c_uint64), ("ldc", C.c_uint64), ("c_off", C.c_uint64),
        ("alpha", C.c_float), ("beta", C.c_float),
        ("a_image", Operand),
    ]


ATTENTION_GENERIC = 1
ATTENTION_ROW_UNITS = 2
ATTENTION_BLOCKS = 4


class Attention(C.Structure):
    _fields_ = [
        ("out", Operand), ("q", Operand), ("k", Operand), ("v", Operand),
        ("query_positions", Operand), ("kv_lengths", Operand),
        ("q_dtype", C.c_uint32), ("k_dtype", C.c_uint32), ("v_dtype", C.c_uint32), ("rolling", C.c_uint32),
        ("batch", C.c_uint64), ("l_q", C.c_uint64), ("h_q", C.c_uint64), ("h_kv", C.c_uint64),
        ("d_k", C.c_uint64), ("d_v", C.c_uint64), ("t_cap", C.c_uint64),
        ("scale", C.c_float), ("soft_cap", C.c_float),
        ("window_left", C.c_uint32), ("window_right", C.c_uint32), ("window_chunk", C.c_uint32),
        ("flags", C.c_uint32),
        ("image", Operand), ("image_dtype", C.c_uint32), ("page_tokens", C.c_uint32),
        ("page_table", Operand), ("pool_pages", C.c_uint64),
    ]


class RMSNorm(C.Structure):
    _fields_ = [("out", Operand), ("x", Operand), ("gamma", Operand), ("beta", Operand), ("residual", Operand),
                ("rows", C.c_uint64), ("cols", C.c_uint64), ("eps", C.c_float), ("image_dtype", C.c_uint32),
                ("image", Operand)]


class Elemwise(C.Structure):
    _fields_ = [("out", Operand), ("a", Operand), ("b", Operand), ("count", C.c_uint64), ("op", C.c_uint32),
                ("reserved", C.c_uint32), ("cols", C.c_uint64), ("ld_out", C.c_uint64), ("ld_a", C.c_uint64),
                ("ld_b", C.c_uint64), ("image", Operand), ("image_dtype", C.c_uint32), ("reserved2", C.c_uint32)]


class RMSNormPair(C.Structure):
    _fields_ = [("out1", Operand), ("out2", Operand), ("x", Operand), ("gamma1", Operand), ("beta1", Operand),
                ("residual", Operand), ("gamma2", Operand), ("beta2", Operand),
                ("rows", C.c_uint64), ("cols", C.c_uint64), ("eps1", C.c_float), ("eps2", C.c_float),
                ("image", Operand), ("image_dtype", C.c_uint32), ("reserved", C.c_uint32)]


class RopeKVAppend(C.Structure):
    _fields_ = [("q_out", Operand), ("qkv", Operand), ("positions", Operand), ("end_index", Operand),
                ("k_cache", Operand), ("v_cache", Operand),
                ("batch", C.c_uint64), ("len", C.c_uint64), ("h_q", C.c_uint64), ("h_kv", C.c_uint64),
                ("head_dim", C.c_uint64), ("ld_qkv", C.c_uint64), ("t_cap", C.c_uint64),
                ("base_frequency", C.c_float), ("scale_factor", C.c_float), ("proportion", C.c_float),
                ("rolling", C.c_uint32)]


class RoPE(C.Structure):
    _fields_ = [("out", Operand), ("x", Operand), ("positions", Operand),
                ("batch", C.c_uint64), ("len", C.c_uint64), ("heads", C.c_uint64), ("head_dim", C.c_uint64),
                ("base_frequency", C.c_float), ("scale_factor", C.c_float), ("proportion", C.c_float),
                ("reserved", C.c_uint32)]


class Cast(C.Structure):
    _fields_ = [("out", Operand), ("in_", Operand), ("count", C.c_uint64), ("from_dtype", C.c_uint32),
                ("to_dtype", C.c_uint32)]


class SequenceAppend(C.Structure):
    _fields_ = [("cache", Operand), ("new_kv", Operand), ("end_index", Operand),
                ("batch", C.c_uint64), ("t_cap", C.c_uint64), ("heads", C.c_uint64), ("head_dim", C.c_uint64),
                ("new_len", C.c_uint64), ("dtype", C.c_uint32), ("rolling", C.c_uint32),
                ("page_table", Operand), ("page_tokens", C.c_uint64), ("pool_pages", C.c_uint64)]


class GatherRows(C.Structure):
    _fields_ = [("out", Operand), ("table", Operand), ("indices", Operand),
                ("table_rows", C.c_uint64), ("d", C.c_uint64), ("count", C.c_uint64),
                ("block_order", C.c_uint32), ("reserved", C.c_uint32)]


class ArgMax(C.Structure):
    _fields_ = [("out", Operand), ("in_", Operand), ("outer", C.c_uint64), ("n", C.c_uint64)]


_DEV = C.c_void_p
_OPP = C.POINTER(Operand)

# name -> (restype, argtypes); every symbol include/aion_cuda.h declares.
SIGNATURES = {
    "aion_cuda_device_count": (C.c_int32, [C.POINTER(C.c_int32)]),
    "aion_cuda_device_create": (C.c_int32, [C.c_int32, C.POINTER(_DEV)]),
    "aion_cuda_device_destroy": (None, [_DEV]),
    "aion_cuda_device_info": (C.c_int32, [_DEV, C.POINTER(DeviceInfo)]),
    "aion_cuda_quant_block_order": (C.c_uint8, [_DEV]),
    "aion_cuda_set_stream": (C.c_int32, [_DEV, C.c_void_p]),
    "aion_cuda_get_stream": (C.c_void_p, [_DEV]),
    "aion_cuda_sync": (C.c_int32, [_DEV]),
    "aion_cuda_record_begin": (C.c_int32, [_DEV]),
    "aion_cuda_record_lane": (C.c_int32, [_DEV, C.c_uint32]),
    "aion_cuda_record_join": (C.c_int32, [_DEV]),
    "aion_cuda_record_end": (C.c_int32, [_DEV, C.POINTER(C.c_void_p)]),
    "aion_cuda_program_launch": (C.c_int32, [_DEV, C.c_void_p]),
    "aion_cuda_program_destroy": (None, [_DEV, C.c_void_p]),
    "aion_cuda_debug_expire_waits": (C.c_int32, [_DEV, C.c_int32]),
    "aion_cuda_last_error": (C.c_int32, [C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "aion_cuda_memory_model": (C.c_int32, [_DEV]),
    "aion_cuda_max_binding_bytes": (C.c_uint64, [_DEV]),
    "aion_cuda_alloc": (C.c_int32, [_DEV, C.c_size_t, C.c_size_t, C.POINTER(C.c_uint64)]),
    "aion_cuda_free": (C.c_int32, [_DEV, C.c_uint64]),
    "aion_cuda_h2d": (C.c_int32, [_DEV, C.c_uint64, C.c_size_t, C.c_void_p, C.c_size_t]),
    "aion_cuda_d2h": (C.c_int32, [_DEV, C.c_void_p, C.c_uint64, C.c_size_t, C.c_size_t]),
    "aion_cuda_d2d": (C.c_int32, [_DEV, C.c_uint64, C.c_size_t, C.c_uint64, C.c_size_t, C.c_size_t]),
    "aion_cuda_memset": (C.c_int32, [_DEV, C.c_uint64, C.c_size_t, C.c_int32, C.c_size_t]),
    "aion_cuda_matmul": (C.c_int32, [_DEV, C.POINTER(MatMul)]),
    "aion_cuda_matmul_static_scratch": (C.c_int32, [_DEV, C.POINTER(MatMul)]),
    "aion_cuda_matmul_plan": (C.c_int32, [_DEV, C.POINTER(MatMul), C.POINTER(MatMulPlan)]),
    "aion_cuda_act_image_bytes": (C.c_int32, [C.c_uint64, C.c_uint64, C.POINTER(C.c_uint64)]),
    "aion_cuda_act_image": (C.c_int32, [_DEV, C.c_uint32, _OPP, C.c_uint64, C.c_uint64, C.c_uint64, _OPP]),
    "aion_cuda_matmul_nt": (C.c_int32, [_DEV, C.POINTER(MatMulNT)]),
    "aion_cuda_attention": (C.c_int32, [_DEV, C.POINTER(Attention)]),
    "aion_cuda_rms_norm": (C.c_int32, [_DEV, C.POINTER(RMSNorm)]),
    "aion_cuda_elemwise": (C.c_int32, [_DEV, C.POINTER(Elemwise)]),
    "aion_cuda_rope": (C.c_int32, [_DEV, C.POINTER(RoPE)]),
    "aion_cuda_cast": (C.c_int32, [_DEV, C.POINTER(Cast)]),
    "aion_cuda_sequence_append": (C.c_int32, [_DEV, C.POINTER(SequenceAppend)]),
    "aion_cuda_gather_rows": (C.c_int32, [_DEV, C.POINTER(GatherRows)]),
    "aion_cuda_argmax": (C.c_int32, [_DEV, C.POINTER(ArgMax)]),
    "aion_cuda_rms_norm_pair": (C.c_int32, [_DEV, C.POINTER(RMSNormPair)]),
    "aion_cuda_rope_kv_append": (C.c_int32, [_DEV, C.POINTER(RopeKVAppend)]),
    "aion_cuda_quantize": (C.c_int32, [_DEV, C.c_uint32, _OPP, C.POINTER(C.c_uint64), C.c_uint32, C.c_uint32, _OPP]),
    "aion_cuda_dequantize": (C.c_int32, [_DEV, C.c_uint32, _OPP, C.c_uint64, _OPP]),
    "aion_cuda_relayout_q8": (C.c_int32, [_DEV, C.c_uint32, C.c_uint32, C.c_uint64, C.c_uint64, _OPP, _OPP]),
    "aion_cuda_matmul_peers": (C.c_int32, [_DEV, C.POINTER(MatMul), C.POINTER(PeerFanout)]),
    "aion_cuda_peer_wait": (C.c_int32, [_DEV, _OPP, _OPP, C.c_uint32, C.c_uint32]),
    "aion_cuda_ipc_export": (C.c_int32, [_DEV, C.c_uint64, C.POINTER(C.c_uint8 * 64)]),
    "aion_cuda_ipc_import": (C.c_int32, [_DEV, C.POINTER(C.c_uint8 * 64), C.POINTER(C.c_uint64)]),
    "aion_cuda_ipc_close": (C.c_int32, [_DEV, C.c_uint64]),
    "aion_cuda_derive_kmajor_q8": (C.c_int32, [_DEV, C.c_uint32, C.c_uint64, C.c_uint64, _OPP, _OPP]),
}

_lib = None


class AionCudaError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
        self.message = message


def load() -> C.CDLL:
    """dlopen libaion_cuda.so and attach the signatures. Raises if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m aion_b200.build` (there is no fallback path)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    buf = C.create_string_buffer(1024)
    load().aion_cuda_last_error(buf, len(buf), None)
    return buf.value.decode("utf-8", "replace")


def check(status: int) -> None:
    if status != OK:
        raise AionCudaError(status, last_error())
