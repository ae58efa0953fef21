"""The decode matmul entry point that never allocates.

Some hosts of this library cannot let it call cudaMalloc: they run it inside their own
memory pool, inside a capture they own, or under a fixed device-memory budget.
`aion_cuda_matmul_static_scratch` serves them with scratch compiled into the library.
This file checks, through the C ABI, that it gives what `aion_cuda_matmul` gives — on
shapes whose tiles are shared between CTAs, so the built-in scratch is really used — on
two calls in a row (all calls share the one array and its counters). The file name makes
pytest collect it after every other test.
"""
import ctypes as C

import numpy as np
import pytest

from aion_b200 import capi
from aion_b200.backend import BackendError
from tests import refdata as rd
from tests.gpu_util import DevBuf

pytestmark = pytest.mark.gpu

TIGHT = 2e-5  # rel-L2: same integer dots, only the order of f32 additions may differ


def _run(backend, entry, dtype, a, b, m, n, k, c0, alpha, beta):
    bufs = [DevBuf(backend, a), DevBuf(backend, b), DevBuf(backend, c0)]
    try:
        rec = capi.MatMul(c=bufs[2].operand(), a=bufs[0].operand(), b=bufs[1].operand(), b_dtype=dtype,
                          flags=capi.MATMUL_FORCE_GEMV, m=m, n=n, k=k, lda=0, ldb=0, ldc=0, alpha=alpha, beta=beta)
        st = getattr(backend._lib, entry)(backend.handle, C.byref(rec))
        if st != capi.OK:
            raise BackendError(st, capi.last_error())
        return bufs[2].read(np.float32).reshape(m, n)
    finally:
        for x in bufs:
            x.free()


def _quantize(backend, dtype, w):
    from aion_b200 import backend as ab

    return ab.quantize(backend, dtype, w, 0)


@pytest.mark.parametrize("dtype", [capi.DTYPE_Q4_0, capi.DTYPE_Q8_0])
def test_static_scratch_matches_the_allocating_entry_point_twice_in_a_row(backend, dtype):
    cases = [(1, 2048, 2048), (5, 1536, 4096)]  # narrow matrices: every tile is split across CTAs
    for call, (m, n, k) in enumerate(cases):
        a = rd.synth_acts(m, k, seed=10 + call)
        b = _quantize(backend, dtype, rd.synth_weights(k, n, seed=20 + call))
        c0 = rd.synth_acts(m, n, seed=30 + call)
        want = _run(backend, "aion_cuda_matmul", dtype, a, b, m, n, k, c0, 0.5, 2.0)
        got = _run(backend, "aion_cuda_matmul_static_scratch", dtype, a, b, m, n, k, c0, 0.5, 2.0)
        assert rd.rel_l2(got, want) < TIGHT
        again = _run(backend, "aion_cuda_matmul_static_scratch", dtype, a, b, m, n, k, c0, 0.5, 2.0)
        assert np.array_equal(again, got)  # the shared array carries nothing over between calls


def test_static_scratch_rejects_what_it_cannot_hold(backend):
    k, n = 64, 64
    b = _quantize(backend, capi.DTYPE_Q8_0, rd.synth_weights(k, n))
    with pytest.raises(BackendError) as e:
        _run(backend, "aion_cuda_matmul_static_scratch", capi.DTYPE_Q8_0, rd.synth_acts(9, k), b, 9, n, k,
             np.zeros((9, n), dtype=np.float32), 1.0, 0.0)
    assert e.value.name == "Unsupported" and "8 rows" in str(e.value)
    kk = 8192
    bb = _quantize(backend, capi.DTYPE_Q4_0, rd.synth_weights(kk, 64))
    with pytest.raises(BackendError) as e:
        _run(backend, "aion_cuda_matmul_static_scratch", capi.DTYPE_Q4_0, rd.synth_acts(4, kk), bb, 4, 64, kk,
             np.zeros((4, 64), dtype=np.float32), 1.0, 0.0)
    assert e.value.name == "Unsupported" and "one launch" in str(e.value)


@pytest.mark.parametrize("dtype", [capi.DTYPE_Q4_0, capi.DTYPE_Q8_0])
def test_static_scratch_does_not_disturb_the_allocating_entry_point(backend, dtype):
    """Both entry points run the same kernel for one row; the shared-memory allowance one of them
    raised must survive a smaller call through the other."""
    n = 512
    big_k, small_k = 3072, 256
    a_big, a_small = rd.synth_acts(1, big_k, seed=1), rd.synth_acts(1, small_k, seed=2)
    b_big = _quantize(backend, dtype, rd.synth_weights(big_k, n, seed=3))
    b_small = _quantize(backend, dtype, rd.synth_weights(small_k, n, seed=4))
    c0 = np.zeros((1, n), dtype=np.float32)
    first = _run(backend, "aion_cuda_matmul", dtype, a_big, b_big, 1, n, big_k, c0, 1.0, 0.0)
    _run(backend, "aion_cuda_matmul_static_scratch", dtype, a_small, b_small, 1, n, small_k, c0, 1.0, 0.0)
    again = _run(backend, "aion_cuda_matmul", dtype, a_big, b_big, 1, n, big_k, c0, 1.0, 0.0)
    assert np.array_equal(again, first)


def test_static_scratch_at_its_limits_and_leaves_device_memory_alone(backend):
    """A grid that is clamped to the built-in scratch (more units than its 512 CTA slots), the deepest K of
    one row, and no change in free device memory across a call on a shape this device has not seen."""
    import torch

    cases = [(capi.DTYPE_Q4_0, 1, 8192, 2048), (capi.DTYPE_Q8_0, 1, 256, 16384), (capi.DTYPE_Q4_0, 8, 4096, 4096)]
    for dtype, m, n, k in cases:
        a = rd.synth_acts(m, k, seed=k)
        b = _quantize(backend, dtype, rd.synth_weights(k, n, seed=n))
        c0 = np.zeros((m, n), dtype=np.float32)
        bufs = [DevBuf(backend, a), DevBuf(backend, b), DevBuf(backend, c0)]
        try:
            rec = capi.MatMul(c=bufs[2].operand(), a=bufs[0].operand(), b=bufs[1].operand(), b_dtype=dtype, flags=0, m=m, n=n, k=k,
                              lda=0, ldb=0, ldc=0, alpha=1.0, beta=0.0)
            backend.sync()
            free_before = torch.cuda.mem_get_info(0)[0]
            assert backend._lib.aion_cuda_matmul_static_scratch(backend.handle, C.byref(rec)) == capi.OK
            backend.sync()
            assert torch.cuda.mem_get_info(0)[0] == free_before
            got = bufs[2].read(np.float32).reshape(m, n)
        finally:
            for x in bufs:
                x.free()
        import oracle

        assert rd.rel_l2(got, oracle.fast_matmul_q(dtype, a, b, m, n, k)) < TIGHT
