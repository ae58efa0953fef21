"""Helpers for the GPU parity tests: run one step through the C ABI on numpy inputs."""
from __future__ import annotations

import ctypes as C

import numpy as np

from aion_b200 import capi
from aion_b200.backend import BackendError, CudaBackend

CANARY = np.float32(-12345.678)


class DevBuf:
    """A device allocation filled from a numpy array, freed on exit."""

    def __init__(self, backend: CudaBackend, data: np.ndarray | None = None, nbytes: int | None = None, pad: int = 0):
        self.mem = backend.device_memory
        self.nbytes = int(data.nbytes if data is not None else nbytes)
        self.pad = pad
        self.handle = self.mem.alloc(max(self.nbytes + pad, 1), 64)
        if data is not None:
            self.mem.copy_h2d(self.handle, 0, np.ascontiguousarray(data))

    def operand(self, offset: int = 0, length: int | None = None) -> capi.Operand:
        return capi.Operand(self.handle, offset, self.nbytes - offset if length is None else length)

    def read(self, dtype, count: int | None = None, offset: int = 0) -> np.ndarray:
        n = (self.nbytes - offset) // np.dtype(dtype).itemsize if count is None else count
        out = np.empty(n, dtype=dtype)
        self.mem.copy_d2h(out, self.handle, offset)
        return out

    def free(self):
        if self.handle:
            self.mem.free(self.handle)
            self.handle = 0


def _raise(status: int):
    if status != capi.OK:
        raise BackendError(status, capi.last_error())


def image_bytes(m: int, k: int) -> int:
    n = C.c_uint64()
    _raise(capi.load().aion_cuda_act_image_bytes(m, k, C.byref(n)))
    return int(n.value)


def make_image(backend: CudaBackend, dtype: int, a_buf: "DevBuf", m: int, k: int, lda: int = 0) -> "DevBuf":
    """The quantized image of the f32 rows in `a_buf`, made by aion_cuda_act_image (zero-filled first)."""
    img = DevBuf(backend, np.zeros(image_bytes(m, k), dtype=np.uint8))
    a_op, i_op = a_buf.operand(), img.operand()
    _raise(backend._lib.aion_cuda_act_image(backend.handle, dtype, C.byref(a_op), m, k, lda, C.byref(i_op)))
    return img


def matmul_plan(backend: CudaBackend, dtype: int, m: int, n: int, k: int, flags=capi.MATMUL_AUTO) -> capi.MatMulPlan:
    """aion_cuda_matmul_plan for dense operands of this shape (placeholder buffers of the right sizes)."""
    bb = 18 if dtype == capi.DTYPE_Q4_0 else 34
    bufs = [DevBuf(backend, nbytes=m * k * 4), DevBuf(backend, nbytes=(k // 32) * n * bb), DevBuf(backend, nbytes=m * n * 4)]
    try:
        rec = capi.MatMul(c=bufs[2].operand(), a=bufs[0].operand(), b=bufs[1].operand(), b_dtype=dtype, flags=flags, m=m, n=n,
                          k=k, lda=0, ldb=0, ldc=0, alpha=1.0, beta=0.0)
        plan = capi.MatMulPlan()
        _raise(backend._lib.aion_cuda_matmul_plan(backend.handle, C.byref(rec), C.byref(plan)))
        return plan
    finally:
        for x in bufs:
            x.free()


def run_matmul(backend: CudaBackend, dtype: int, a: np.ndarray, b: np.ndarray, m: int, n: int, k: int, *, lda=0, ldb=0,
               ldc=0, alpha=1.0, beta=0.0, c: np.ndarray | None = None, flags=capi.MATMUL_AUTO, canary=True, image=False):
    """aion_cuda_matmul on host arrays; returns C as [m, ldc or n]. Checks a canary past the end of C.
    image: hand the step the quantized image of A (made by aion_cuda_act_image) as well."""
    width = ldc if ldc else n
    c_host = np.zeros(m * width, dtype=np.float32) if c is None else np.asarray(c, dtype=np.float32).reshape(-1).copy()
    tail = np.full(64, CANARY, dtype=np.float32)
    bufs = [DevBuf(backend, np.ascontiguousarray(a, dtype=np.float32)), DevBuf(backend, np.ascontiguousarray(b, dtype=np.uint8)),
            DevBuf(backend, np.concatenate([c_host, tail]))]
    try:
        need_c = ((m - 1) * width + n) * 4 if m else 0
        img_op = capi.Operand(0, 0, 0)
        if image:
            bufs.append(make_image(backend, dtype, bufs[0], m, k, lda))
            img_op = bufs[-1].operand()
        rec = capi.MatMul(c=bufs[2].operand(0, max(need_c, c_host.nbytes)), a=bufs[0].operand(), b=bufs[1].operand(),
                          b_dtype=dtype, flags=flags, m=m, n=n, k=k, lda=lda, ldb=ldb, ldc=ldc, alpha=alpha, beta=beta,
                          a_image=img_op)
        _raise(backend._lib.aion_cuda_matmul(backend.handle, C.byref(rec)))
        out = bufs[2].read(np.float32)
        if canary:
            assert np.array_equal(out[c_host.size:], tail), "kernel wrote past the end of C"
        return out[:c_host.size].reshape(m, width)
    finally:
        for x in bufs:
            x.free()


def run_matmul_nt(backend: CudaBackend, a: np.ndarray, b: np.ndarray, m: int, n: int, k: int, *, order=capi.ORDER_ROW_MAJOR,
                  lda=0, ldc=0, c_off=0, alpha=1.0, beta=0.0, c: np.ndarray | None = None, flags=capi.MATMUL_AUTO, image=False):
    width = ldc if ldc else n
    c_host = np.zeros(m * width, dtype=np.float32) if c is None else np.asarray(c, dtype=np.float32).reshape(-1).copy()
    tail = np.full(64, CANARY, dtype=np.float32)
    bufs = [DevBuf(backend, np.ascontiguousarray(a, dtype=np.float32)), DevBuf(backend, np.ascontiguousarray(b, dtype=np.uint8)),
            DevBuf(backend, np.concatenate([c_host, tail]))]
    try:
        img_op = capi.Operand(0, 0, 0)
        if image:
            bufs.append(make_image(backend, capi.DTYPE_Q8_0, bufs[0], m, k, lda))
            img_op = bufs[-1].operand()
        rec = capi.MatMulNT(c=bufs[2].operand(0, c_host.nbytes), a=bufs[0].operand(), b=bufs[1].operand(),
                            b_dtype=capi.DTYPE_Q8_0, block_order=order, flags=flags, m=m, n=n, k=k, lda=lda, ldc=ldc,
                            c_off=c_off, alpha=alpha, beta=beta, a_image=img_op)
        _raise(backend._lib.aion_cuda_matmul_nt(backend.handle, C.byref(rec)))
        out = bufs[2].read(np.float32)
        assert np.array_equal(out[c_host.size:], tail), "kernel wrote past the end of C"
        return out[:c_host.size].reshape(m, width)
    finally:
        for x in bufs:
            x.free()


NP_DT = {np.dtype(np.float32): capi.DTYPE_F32, np.dtype(np.float16): capi.DTYPE_F16}


def run_attention(backend: CudaBackend, q, k, v, *, scale, positions=None, kv_lengths=None, left=capi.WINDOW_UNBOUNDED,
                  right=capi.WINDOW_UNBOUNDED, chunk=0, soft_cap=0.0, rolling=False, sync=True, flags=0, page_table=None):
    """page_table (i32 [B, pages per request]): k and v are page pools [pages, page_tokens, Hkv, D]."""
    q, k, v = np.ascontiguousarray(q), np.ascontiguousarray(k), np.ascontiguousarray(v)
    B, L, Hq, Dk = q.shape
    _, T, Hkv, _ = k.shape
    Dv = v.shape[3]
    table_op, page_tokens, pool_pages = capi.Operand(0, 0, 0), 0, 0
    if page_table is not None:
        page_table = np.ascontiguousarray(page_table, dtype=np.int32)
        pool_pages, page_tokens = k.shape[0], k.shape[1]
        T = page_table.shape[1] * page_tokens
    out_n = B * L * Hq * Dv
    tail = np.full(64, CANARY, dtype=np.float32)
    bufs = [DevBuf(backend, q), DevBuf(backend, k), DevBuf(backend, v),
            DevBuf(backend, np.concatenate([np.full(out_n, np.float32(777.0)), tail]))]
    none = capi.Operand(0, 0, 0)
    pos_op, len_op = none, none
    if positions is not None:
        bufs.append(DevBuf(backend, np.ascontiguousarray(positions, dtype=np.int32)))
        pos_op = bufs[-1].operand()
    if kv_lengths is not None:
        bufs.append(DevBuf(backend, np.ascontiguousarray(kv_lengths, dtype=np.int32)))
        len_op = bufs[-1].operand()
    if page_table is not None:
        bufs.append(DevBuf(backend, page_table))
        table_op = bufs[-1].operand()
    try:
        rec = capi.Attention(out=bufs[3].operand(0, out_n * 4), q=bufs[0].operand(), k=bufs[1].operand(), v=bufs[2].operand(),
                             page_table=table_op, page_tokens=page_tokens, pool_pages=pool_pages,
                             query_positions=pos_op, kv_lengths=len_op, q_dtype=NP_DT[q.dtype], k_dtype=NP_DT[k.dtype],
                             v_dtype=NP_DT[v.dtype], rolling=int(rolling), batch=B, l_q=L, h_q=Hq, h_kv=Hkv, d_k=Dk, d_v=Dv,
                             t_cap=T, scale=scale, soft_cap=soft_cap, window_left=left, window_right=right,
                             window_chunk=chunk, flags=flags)
        _raise(backend._lib.aion_cuda_attention(backend.handle, C.byref(rec)))
        out = bufs[3].read(np.float32)  # d2h waits and reports device-side input faults
        assert np.array_equal(out[out_n:], tail), "kernel wrote past the end of out"
        return out[:out_n].reshape(B, L, Hq, Dv)
    finally:
        for x in bufs:
            x.free()
