"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only tests/, the smoke check and the benchmark's CPU-baseline leg may import this
package. The shipped library (aion_b200) never does: it has no CPU path.

Every function takes and returns numpy arrays. dtype codes are aion's `AionDType`
values: f32 = 0, f16 = 1, q4_0 = 3, q8_0 = 4.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build as _build

F32, F16, Q4_0, Q8_0 = 0, 1, 3, 4
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34}
ORDERS = {"row_major": 0, "lanes4": 1, "lanes8": 2, "lanes16": 3, "lanes32": 4, "lanes32x16": 5}
UNBOUNDED = 0xFFFFFFFF

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(_build.build())
        _lib.aion_oracle_f32_to_f16.restype = C.c_uint16
        _lib.aion_oracle_f32_to_f16.argtypes = [C.c_float]
        _lib.aion_oracle_f16_to_f32.restype = C.c_float
        _lib.aion_oracle_f16_to_f32.argtypes = [C.c_uint16]
        _lib.aion_oracle_exp_approx.restype = C.c_float
        _lib.aion_oracle_exp_approx.argtypes = [C.c_float]
        _lib.aion_oracle_tanh_approx.restype = C.c_float
        _lib.aion_oracle_tanh_approx.argtypes = [C.c_float]
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise ValueError(f"oracle {what} failed with status {rc}")


def quantize(dtype: int, values: np.ndarray, quant_axis: int) -> np.ndarray:
    """Pack an f32 tensor into q8_0 / q4_0 blocks along `quant_axis` (row-major over block space)."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    shape = (C.c_uint64 * v.ndim)(*v.shape)
    nblocks = v.size // 32
    out = np.zeros(nblocks * BLOCK_BYTES[dtype], dtype=np.uint8)
    _check(lib().aion_oracle_quantize(dtype, _p(v), shape, v.ndim, quant_axis, _p(out)), "quantize")
    return out


def dequant(dtype: int, blocks: np.ndarray) -> np.ndarray:
    """Dequantize consecutive blocks to f32, 32 values per block, in storage order."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    n = b.size // BLOCK_BYTES[dtype]
    out = np.empty(n * 32, dtype=np.float32)
    _check(lib().aion_oracle_dequant(dtype, _p(b), C.c_uint64(n), _p(out)), "dequant")
    return out


def relayout_q8(order: str | int, n: int, k: int, src: np.ndarray, inverse: bool = False) -> np.ndarray:
    o = ORDERS[order] if isinstance(order, str) else order
    s = np.ascontiguousarray(src, dtype=np.uint8)
    dst = np.zeros_like(s)
    _check(lib().aion_oracle_relayout_q8(o, int(inverse), C.c_uint64(n), C.c_uint64(k), _p(s), _p(dst)), "relayout")
    return dst


def quantize_activation(a: np.ndarray):
    a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
    q = np.empty(a.size, dtype=np.int8)
    s = np.empty(a.size // 32, dtype=np.float32)
    _check(lib().aion_oracle_quantize_activation(_p(a), C.c_uint64(a.size), _p(q), _p(s)), "quantize_activation")
    return q, s


def matmul_q(dtype, a, b, m, n, k, *, lda=0, ldb=0, ldc=0, alpha=1.0, beta=0.0, c=None, route=0, kc=0):
    """`MatMul` with K-major quantized B, reference CPU (int8-activation) arithmetic."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.uint8)
    rows = ldc if ldc else n
    if c is None:
        c = np.zeros(m * rows, dtype=np.float32)
    else:
        c = np.array(c, dtype=np.float32).reshape(-1).copy()
    rc = lib().aion_oracle_matmul_q(
        dtype, C.c_uint64(m), C.c_uint64(n), C.c_uint64(k), C.c_uint64(lda), C.c_uint64(ldb), C.c_uint64(ldc),
        C.c_float(alpha), C.c_float(beta), _p(c), _p(a), _p(b), route, C.c_uint64(kc))
    _check(rc, "matmul_q")
    return c.reshape(m, rows)


def matmul_nt_q8(a, b, m, n, k, *, order="row_major", lda=0, ldc=0, alpha=1.0, beta=0.0, c=None):
    """`MatMulNT` with q8_0 [n, k] B in a QuantBlockOrder, reference CPU arithmetic."""
    o = ORDERS[order] if isinstance(order, str) else order
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.uint8)
    rows = ldc if ldc else n
    if c is None:
        c = np.zeros(m * rows, dtype=np.float32)
    else:
        c = np.array(c, dtype=np.float32).reshape(-1).copy()
    rc = lib().aion_oracle_matmul_nt_q8(
        o, C.c_uint64(m), C.c_uint64(n), C.c_uint64(k), C.c_uint64(lda), C.c_uint64(ldc),
        C.c_float(alpha), C.c_float(beta), _p(c), _p(a), _p(b))
    _check(rc, "matmul_nt_q8")
    return c.reshape(m, rows)


def matmul_deqf32(dtype, a, b, m, n, k, *, nt=False, lda=0, ldb=0, ldc=0, alpha=1.0, beta=0.0, c=None):
    """f32 activation x dequant(B): the host reference of the reference's GPU tests."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.uint8)
    rows = ldc if ldc else n
    if c is None:
        c = np.zeros(m * rows, dtype=np.float32)
    else:
        c = np.array(c, dtype=np.float32).reshape(-1).copy()
    rc = lib().aion_oracle_matmul_deqf32(
        dtype, int(nt), C.c_uint64(m), C.c_uint64(n), C.c_uint64(k), C.c_uint64(lda), C.c_uint64(ldb),
        C.c_uint64(ldc), C.c_float(alpha), C.c_float(beta), _p(c), _p(a), _p(b))
    _check(rc, "matmul_deqf32")
    return c.reshape(m, rows)


def _dt(a: np.ndarray) -> int:
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.float16:
        return F16
    raise TypeError(a.dtype)


def attention(q, k, v, *, scale, positions=None, kv_lengths=None, left=UNBOUNDED, right=UNBOUNDED,
              chunk=0, soft_cap=0.0, rolling=False, exact=False):
    """`Attention` step. q [B,L,Hq,Dk], k [B,T,Hkv,Dk], v [B,T,Hkv,Dv] (f16 or f32) -> f32 [B,L,Hq,Dv]."""
    q = np.ascontiguousarray(q)
    k = np.ascontiguousarray(k)
    v = np.ascontiguousarray(v)
    B, L, Hq, Dk = q.shape
    _, T, Hkv, _ = k.shape
    Dv = v.shape[3]
    out = np.zeros((B, L, Hq, Dv), dtype=np.float32)
    pos = None if positions is None else np.ascontiguousarray(positions, dtype=np.int32)
    lens = None if kv_lengths is None else np.ascontiguousarray(kv_lengths, dtype=np.int32)
    rc = lib().aion_oracle_attention(
        _p(out), _p(q), _dt(q), _p(k), _dt(k), _p(v), _dt(v), _p(pos), _p(lens),
        C.c_uint64(B), C.c_uint64(L), C.c_uint64(Hq), C.c_uint64(Hkv), C.c_uint64(Dk), C.c_uint64(Dv),
        C.c_uint64(T), C.c_float(scale), C.c_uint32(left), C.c_uint32(right), C.c_uint32(chunk),
        C.c_float(soft_cap), int(rolling), int(exact))
    _check(rc, "attention")
    return out


# ---- timed CPU baseline (threaded port of the reference kernels) ------------------------
def fast_has_vnni() -> bool:
    return bool(lib().aion_oracle_fast_has_vnni())


def fast_max_threads() -> int:
    return int(lib().aion_oracle_fast_max_threads())


def fast_matmul_q(dtype, a, b, m, n, k, *, alpha=1.0, beta=0.0, c=None, threads=0):
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.uint8)
    c = np.zeros(m * n, dtype=np.float32) if c is None else c
    rc = lib().aion_oracle_fast_matmul_q(dtype, C.c_uint64(m), C.c_uint64(n), C.c_uint64(k), C.c_float(alpha),
                                         C.c_float(beta), _p(c), _p(a), _p(b), threads)
    _check(rc, "fast_matmul_q")
    return c.reshape(m, n)


def fast_matmul_nt_q8(a, b, m, n, k, *, alpha=1.0, beta=0.0, c=None, threads=0):
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.uint8)
    c = np.zeros(m * n, dtype=np.float32) if c is None else c
    rc = lib().aion_oracle_fast_matmul_nt_q8(C.c_uint64(m), C.c_uint64(n), C.c_uint64(k), C.c_float(alpha),
                                             C.c_float(beta), _p(c), _p(a), _p(b), threads)
    _check(rc, "fast_matmul_nt_q8")
    return c.reshape(m, n)


def fast_attention(q, k, v, *, scale, positions=None, kv_lengths=None, left=UNBOUNDED, right=UNBOUNDED, chunk=0, soft_cap=0.0,
                   rolling=False, threads=0):
    """`attention` with the requests spread over host threads (same values)."""
    q = np.ascontiguousarray(q)
    k = np.ascontiguousarray(k)
    v = np.ascontiguousarray(v)
    B, L, Hq, Dk = q.shape
    _, T, Hkv, _ = k.shape
    Dv = v.shape[3]
    out = np.zeros((B, L, Hq, Dv), dtype=np.float32)
    pos = None if positions is None else np.ascontiguousarray(positions, dtype=np.int32)
    lens = None if kv_lengths is None else np.ascontiguousarray(kv_lengths, dtype=np.int32)
    rc = lib().aion_oracle_fast_attention(
        _p(out), _p(q), _dt(q), _p(k), _dt(k), _p(v), _dt(v), _p(pos), _p(lens),
        C.c_uint64(B), C.c_uint64(L), C.c_uint64(Hq), C.c_uint64(Hkv), C.c_uint64(Dk), C.c_uint64(Dv),
        C.c_uint64(T), C.c_float(scale), C.c_uint32(left), C.c_uint32(right), C.c_uint32(chunk),
        C.c_float(soft_cap), int(rolling), int(threads))
    _check(rc, "fast_attention")
    return out


# ---- decoder glue steps -----------------------------------------------------------------
ELEMWISE_ADD, ELEMWISE_MUL, ELEMWISE_GATE_GELU = 0, 1, 2


def rms_norm(x, gamma, beta, eps, residual=None):
    """RMSNorm over the last axis (+ optional residual added after normalization)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    cols = x.shape[-1]
    rows = x.size // cols
    g = np.ascontiguousarray(gamma, dtype=np.float32)
    b = np.ascontiguousarray(beta, dtype=np.float32)
    r = None if residual is None else np.ascontiguousarray(residual, dtype=np.float32)
    out = np.empty_like(x)
    _check(lib().aion_oracle_rms_norm(_p(out), _p(x), _p(g), _p(b), _p(r), C.c_uint64(rows), C.c_uint64(cols), C.c_float(eps)),
           "rms_norm")
    return out


def elemwise(op: int, a, b):
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    out = np.empty_like(a)
    _check(lib().aion_oracle_elemwise(op, _p(out), _p(a), _p(b), C.c_uint64(a.size)), "elemwise")
    return out


def rope(x, positions, base_frequency, scale_factor=1.0, proportion=1.0):
    """RoPE1D over x [B, L, H, D] f32 with positions [B, L] i32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    B, L, H, D = x.shape
    out = np.empty_like(x)
    _check(lib().aion_oracle_rope(_p(out), _p(x), _p(pos), C.c_uint64(B), C.c_uint64(L), C.c_uint64(H), C.c_uint64(D),
                                  C.c_float(base_frequency), C.c_float(scale_factor), C.c_float(proportion)), "rope")
    return out


def cast_f32_f16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    _check(lib().aion_oracle_cast_f32_f16(_p(out), _p(x), C.c_uint64(x.size)), "cast")
    return out.view(np.float16)


def sequence_append(cache, new_kv, end_index, rolling=False):
    """Returns a copy of cache [B, T, H, D] with new_kv [B, Ln, H, D] written at end_index[b] + t."""
    cache = np.ascontiguousarray(cache).copy()
    new_kv = np.ascontiguousarray(new_kv, dtype=cache.dtype)
    idx = np.ascontiguousarray(end_index, dtype=np.int32)
    B, T, H, D = cache.shape
    _check(lib().aion_oracle_sequence_append(_p(cache), _p(new_kv), _p(idx), C.c_uint64(cache.itemsize), C.c_uint64(B),
                                             C.c_uint64(T), C.c_uint64(H), C.c_uint64(D), C.c_uint64(new_kv.shape[1]),
                                             int(rolling)), "sequence_append")
    return cache


def gather_rows_q8(table, table_rows, d, indices, order="row_major"):
    table = np.ascontiguousarray(table, dtype=np.uint8)
    idx = np.ascontiguousarray(indices, dtype=np.int32)
    out = np.empty((idx.size, d), dtype=np.float32)
    o = ORDERS[order] if isinstance(order, str) else int(order)
    _check(lib().aion_oracle_gather_rows_q8(_p(out), _p(table), o, C.c_uint64(table_rows), C.c_uint64(d), _p(idx),
                                            C.c_uint64(idx.size)), "gather_rows_q8")
    return out


def argmax(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    n = x.shape[-1]
    outer = x.size // n
    out = np.empty(outer, dtype=np.int32)
    _check(lib().aion_oracle_argmax(_p(out), _p(x), C.c_uint64(outer), C.c_uint64(n)), "argmax")
    return out.reshape(x.shape[:-1])
