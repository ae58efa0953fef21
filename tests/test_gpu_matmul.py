"""`MatMul` / `MatMulNT` parity: the CUDA kernels through the C ABI against the oracle
(reference CPU arithmetic, int8 activations). Tolerance for these fp32-accumulate
kernels: rel-L2 <= 1e-3 (the bound the task states); observed values are ~1e-6 because
the integer dots are exact and only the order of the f32 additions differs."""
import ctypes as C
import os

import numpy as np
import pytest

import oracle
from aion_b200 import capi
from aion_b200.backend import (BackendError, CudaBackend, DeviceStore, StepMatMul, StepMatMulNT, TensorMeta)
from tests import refdata as rd
from tests.gpu_util import run_matmul, run_matmul_nt

pytestmark = pytest.mark.gpu

TOL = 1e-3        # stated bound, rel-L2 vs the reference CPU arithmetic
TIGHT = 2e-5      # what exact integer dots + f32 accumulation should give

KERNELS = [capi.MATMUL_AUTO, capi.MATMUL_FORCE_GENERIC, capi.MATMUL_FORCE_GEMV]


# ---- the reference's own fixtures ----------------------------------------------------
def test_matvec_chunk_boundary_fixture(backend):
    # src/aion/backend/cpu/kernels/matvec_q.zig:176-219 (n = 5: the any-shape kernel)
    m, n, k, a, b = rd.matvec_q_chunk_case()
    got = run_matmul(backend, capi.DTYPE_Q8_0, a, b, m, n, k)
    np.testing.assert_allclose(got, rd.int8_reference_f64(a, b, m, n, k, nt=False), rtol=1e-5)


@pytest.mark.parametrize("order,group", [(0, 1), (1, 4), (2, 8), (3, 16), (4, 32), (5, 32)])
@pytest.mark.parametrize("m", [1, 2, 7, 10])
def test_nt_grouped_fixture_every_order(backend, order, group, m):
    # src/aion/backend/cpu/kernels/matmul_nt_q.zig:587-637
    m, n, k, a, rows = rd.nt_grouped_case(group, m)
    tile = oracle.relayout_q8(order, n, k, rows)
    got = run_matmul_nt(backend, a, tile, m, n, k, order=order)
    want = rd.int8_reference_f64(a, rows, m, n, k, nt=True)
    assert np.all(np.abs(got - want) <= 1e-4 * np.maximum(1.0, np.abs(want)))


@pytest.mark.parametrize("m", [1, 2, 3, 7, 8, 17])
@pytest.mark.parametrize("flags", KERNELS)
def test_weight_layout_arithmetic_fixture(backend, m, flags):
    # src/aion/graph/opt/test_opt.zig:1106-1175: NMSE < 1e-10 vs the f64 int8 reference
    m, n, k, a, w = rd.weight_layout_arith_case(m)
    b = oracle.quantize(oracle.Q8_0, w, 0)
    want = rd.int8_reference_f64(a, b, m, n, k, nt=False)
    got = run_matmul(backend, capi.DTYPE_Q8_0, a, b, m, n, k, flags=flags)
    assert np.sum((got - want) ** 2) / np.sum(want ** 2) < 1e-10


def test_nt_backend_fixture(backend):
    # src/aion/backend/cpu/test_cpu_backend.zig:2879-3012
    m, n, k, a, packed, c_ref = rd.nt_backend_case()
    np.testing.assert_allclose(run_matmul_nt(backend, a, packed, m, n, k), c_ref, atol=1e-4)


# ---- benchmark configurations (seeded synthetic inputs of those shapes) -----------------
def test_config1_q8_nt_gemv(backend):
    n, k = 8192, 2048
    x = rd.synth_acts(1, k)
    w = rd.synth_weights(n, k)
    b = oracle.quantize(oracle.Q8_0, w, 1)
    want = oracle.matmul_nt_q8(x, b, 1, n, k)
    for flags in KERNELS:
        got = run_matmul_nt(backend, x, b, 1, n, k, flags=flags)
        assert rd.rel_l2(got, want) < TIGHT < TOL
    # distance to the f32-activation arithmetic of the reference's device kernels (reported, not gated)
    deq = oracle.matmul_deqf32(oracle.Q8_0, x, b, 1, n, k, nt=True)
    assert rd.rel_l2(got, deq) < 2e-2


@pytest.mark.parametrize("nk", [(2048, 2048), (8192, 2048), (2048, 8192)])
@pytest.mark.parametrize("m", [1, 2, 4, 8])
def test_config2_q4_gemv_sweep(backend, nk, m):
    n, k = nk
    x = rd.synth_acts(m, k)
    b = oracle.quantize(oracle.Q4_0, rd.synth_weights(k, n), 0)
    want = oracle.matmul_q(oracle.Q4_0, x, b, m, n, k)
    got = run_matmul(backend, capi.DTYPE_Q4_0, x, b, m, n, k, flags=capi.MATMUL_FORCE_GEMV)
    assert rd.rel_l2(got, want) < TIGHT < TOL
    if m == 1:
        assert rd.rel_l2(run_matmul(backend, capi.DTYPE_Q4_0, x, b, m, n, k, flags=capi.MATMUL_FORCE_GENERIC), want) < TIGHT


@pytest.mark.parametrize("dtype", [capi.DTYPE_Q8_0, capi.DTYPE_Q4_0])
@pytest.mark.parametrize("m", [1, 3, 8, 9, 13, 16])
def test_kmajor_gemv_all_m(backend, dtype, m):
    n, k = 512, 1024
    x = rd.synth_acts(m, k, seed=m)
    b = oracle.quantize(dtype, rd.synth_weights(k, n, seed=99), 0)
    want = oracle.matmul_q(dtype, x, b, m, n, k)
    got = run_matmul(backend, dtype, x, b, m, n, k, flags=capi.MATMUL_FORCE_GEMV)
    assert rd.rel_l2(got, want) < TIGHT


# ---- edges: tails, strides, epilogue -------------------------------------------------
@pytest.mark.parametrize("dtype", [capi.DTYPE_Q8_0, capi.DTYPE_Q4_0])
@pytest.mark.parametrize("n,k", [(8, 32), (72, 96), (200, 2080), (64, 32 * 65), (1544, 288)])
def test_kmajor_tails(backend, dtype, n, k):
    m = 5
    x = rd.synth_acts(m, k, seed=n)
    b = oracle.quantize(dtype, rd.synth_weights(k, n, seed=k), 0)
    want = oracle.matmul_q(dtype, x, b, m, n, k)
    for flags in KERNELS:
        assert rd.rel_l2(run_matmul(backend, dtype, x, b, m, n, k, flags=flags), want) < TIGHT


@pytest.mark.parametrize("n,k", [(16, 256), (72, 512), (1000, 1280)])
def test_nt_tails(backend, n, k):
    m = 3
    x = rd.synth_acts(m, k, seed=n)
    b = oracle.quantize(oracle.Q8_0, rd.synth_weights(n, k, seed=k), 1)
    want = oracle.matmul_nt_q8(x, b, m, n, k)
    for flags in KERNELS:
        assert rd.rel_l2(run_matmul_nt(backend, x, b, m, n, k, flags=flags), want) < TIGHT


def test_nt_unaligned_k_takes_the_any_shape_kernel(backend):
    m, n, k = 2, 40, 96  # k/32 not a multiple of 8: rows are not 16-byte aligned
    x = rd.synth_acts(m, k)
    b = oracle.quantize(oracle.Q8_0, rd.synth_weights(n, k), 1)
    assert rd.rel_l2(run_matmul_nt(backend, x, b, m, n, k), oracle.matmul_nt_q8(x, b, m, n, k)) < TIGHT
    with pytest.raises(BackendError) as e:
        run_matmul_nt(backend, x, b, m, n, k, flags=capi.MATMUL_FORCE_GEMV)
    assert e.value.name == "Unsupported"


@pytest.mark.parametrize("dtype", [capi.DTYPE_Q8_0, capi.DTYPE_Q4_0])
@pytest.mark.parametrize("flags", KERNELS)
def test_alpha_beta_and_leading_dimensions(backend, dtype, flags):
    rng = np.random.default_rng(4)
    m, n, k = 4, 64, 256
    lda, ldb, ldc = k + 8, n + 16, n + 24
    a = rng.standard_normal((m, lda)).astype(np.float32)
    wide = oracle.quantize(dtype, rd.synth_weights(k, ldb), 0)       # [k/32][ldb] blocks; the step reads n of each row
    c0 = rng.standard_normal((m, ldc)).astype(np.float32)
    want = oracle.matmul_q(dtype, a, wide, m, n, k, lda=lda, ldb=ldb, ldc=ldc, alpha=0.75, beta=-1.5, c=c0)
    got = run_matmul(backend, dtype, a, wide, m, n, k, lda=lda, ldb=ldb, ldc=ldc, alpha=0.75, beta=-1.5, c=c0, flags=flags)
    assert rd.rel_l2(got[:, :n], want[:, :n]) < TIGHT
    assert np.array_equal(got[:, n:], c0[:, n:])  # the gap between rows of C is untouched


def test_nt_c_off_writes_one_chunk_of_c(backend):
    # One weight issued as two N-chunks of the same C (src/aion/backend/gpu/exec/matmul_nt.zig:151-160).
    m, n, k = 2, 256, 512
    x = rd.synth_acts(m, k)
    b = oracle.quantize(oracle.Q8_0, rd.synth_weights(n, k), 1)
    want = oracle.matmul_nt_q8(x, b, m, n, k)
    half = n // 2
    rows_bytes = half * (k // 32) * 34
    c = np.zeros((m, n), dtype=np.float32)
    c = run_matmul_nt(backend, x, b[:rows_bytes], m, half, k, ldc=n, c_off=0, c=c)
    c = run_matmul_nt(backend, x, b[rows_bytes:], m, half, k, ldc=n, c_off=half, c=c)
    assert rd.rel_l2(c, want) < TIGHT


def test_zero_and_degenerate_activations(backend):
    m, n, k = 3, 64, 128
    x = np.zeros((m, k), dtype=np.float32)
    x[1, 40] = 1e-30   # a tiny block max
    x[2, :32] = 65504.0
    b = oracle.quantize(oracle.Q4_0, rd.synth_weights(k, n), 0)
    want = oracle.matmul_q(oracle.Q4_0, x, b, m, n, k)
    for flags in KERNELS:
        got = run_matmul(backend, capi.DTYPE_Q4_0, x, b, m, n, k, flags=flags)
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-30)


@pytest.mark.parametrize("split", [1, 2, 4, 8])
def test_cluster_split_k_is_value_stable(split):
    """Every K split of the tiled GEMV (1 CTA, or 2/4/8 CTAs of a cluster meeting in
    distributed shared memory) gives the same answer within f32 rounding."""
    os.environ["AION_CUDA_GEMV_SPLIT"] = str(split)
    try:
        b2 = CudaBackend(0)
    finally:
        del os.environ["AION_CUDA_GEMV_SPLIT"]
    try:
        m, n, k = 4, 256, 4096
        x = rd.synth_acts(m, k)
        for dtype in (capi.DTYPE_Q4_0, capi.DTYPE_Q8_0):
            b = oracle.quantize(dtype, rd.synth_weights(k, n), 0)
            want = oracle.matmul_q(dtype, x, b, m, n, k)
            assert rd.rel_l2(run_matmul(b2, dtype, x, b, m, n, k, flags=capi.MATMUL_FORCE_GEMV), want) < TIGHT
        bn = oracle.quantize(oracle.Q8_0, rd.synth_weights(n, k), 1)
        assert rd.rel_l2(run_matmul_nt(b2, x, bn, m, n, k, flags=capi.MATMUL_FORCE_GEMV),
                         oracle.matmul_nt_q8(x, bn, m, n, k)) < TIGHT
    finally:
        b2.deinit()


def test_repeated_launches_are_bitwise_reproducible(backend):
    m, n, k = 8, 2048, 2048
    x = rd.synth_acts(m, k)
    b = oracle.quantize(oracle.Q4_0, rd.synth_weights(k, n), 0)
    first = run_matmul(backend, capi.DTYPE_Q4_0, x, b, m, n, k)
    for _ in range(3):
        assert np.array_equal(run_matmul(backend, capi.DTYPE_Q4_0, x, b, m, n, k), first)


# ---- the session interface (reference: Backend / Session / DeviceStore) -----------------
def test_session_executes_a_program(backend):
    m, n, k = 2, 128, 256
    x = rd.synth_acts(m, k)
    w = rd.synth_weights(k, n)
    store = DeviceStore(backend.device_memory)
    try:
        a_id = store.add(TensorMeta(capi.DTYPE_F32, (1, m, k)), x)
        b_id = store.add(TensorMeta(capi.DTYPE_Q4_0, (k, n), quant_axis=0), oracle.quantize(oracle.Q4_0, w, 0))
        bt_id = store.add(TensorMeta(capi.DTYPE_Q8_0, (n, k), quant_axis=1),
                          oracle.quantize(oracle.Q8_0, np.ascontiguousarray(w.T), 1))
        c_id = store.add(TensorMeta(capi.DTYPE_F32, (1, m, n)))
        d_id = store.add(TensorMeta(capi.DTYPE_F32, (1, m, n)))
        sess = backend.create_session(store)
        sess.execute([StepMatMul(c_id, a_id, b_id, 1.0, 0.0), StepMatMulNT(d_id, a_id, bt_id, 2.0, 0.0)])
        sess.retire_resources()
        assert rd.rel_l2(store.read(c_id).reshape(m, n), oracle.matmul_q(oracle.Q4_0, x, store.read(b_id), m, n, k)) < TIGHT
        assert rd.rel_l2(store.read(d_id).reshape(m, n), 2 * oracle.matmul_nt_q8(x, store.read(bt_id), m, n, k)) < TIGHT
        with pytest.raises(BackendError) as e:
            sess.execute([object()])
        assert e.value.name == "Unsupported"
    finally:
        store.deinit()


def test_argument_errors(backend):
    x = np.zeros((1, 64), dtype=np.float32)
    b = np.zeros(2 * 8 * 34, dtype=np.uint8)
    with pytest.raises(BackendError) as e:
        run_matmul(backend, capi.DTYPE_Q8_0, x, b, 1, 8, 48)       # k not a multiple of 32
    assert e.value.name == "InvalidArgument"
    with pytest.raises(BackendError) as e:
        run_matmul(backend, capi.DTYPE_F32, x, b, 1, 8, 64)        # float B is outside this backend
    assert e.value.name == "Unsupported"
    with pytest.raises(BackendError) as e:
        run_matmul(backend, capi.DTYPE_Q8_0, x, b[:100], 1, 8, 64)  # B shorter than the step needs
    assert e.value.name == "InvalidArgument"
    with pytest.raises(BackendError) as e:
        run_matmul_nt(backend, x, b, 1, 6, 64, order=capi.ORDER_LANES4)  # n does not fill groups of 4
    assert e.value.name == "InvalidArgument"
    assert backend.device_memory.model() == "discrete"
    assert backend.device_memory.max_binding_bytes() == 2**64 - 1
    assert backend.quant_block_order == capi.ORDER_ROW_MAJOR


def test_scratch_cannot_move_under_a_recorded_program():
    """A recorded program holds scratch addresses: a later, larger step must be refused, not re-allocate."""
    import ctypes as C
    backend = CudaBackend(0)  # its own device object, so its scratch starts empty whatever ran before
    try:
        lib, dev = backend._lib, backend.handle
        rng = np.random.default_rng(0)
        k, n = 64, 8
        a = rng.standard_normal((1, k)).astype(np.float32)
        b = oracle.quantize(oracle.Q4_0, (rng.standard_normal((k, n)) * 0.02).astype(np.float32), 0)
        run_matmul(backend, capi.DTYPE_Q4_0, a, b, 1, n, k, flags=capi.MATMUL_FORCE_GENERIC)  # sizes scratch for this shape
        assert lib.aion_cuda_record_begin(dev) == capi.OK
        prog = C.c_void_p()
        assert lib.aion_cuda_record_end(dev, C.byref(prog)) == capi.OK
        big_m, big_k = 512, 4096  # the any-shape kernel's activation scratch grows with m * k
        a_big = rng.standard_normal((big_m, big_k)).astype(np.float32)
        b_big = oracle.quantize(oracle.Q8_0, (rng.standard_normal((big_k, n)) * 0.02).astype(np.float32), 0)
        try:
            with pytest.raises(BackendError) as e:
                run_matmul(backend, capi.DTYPE_Q8_0, a_big, b_big, big_m, n, big_k, flags=capi.MATMUL_FORCE_GENERIC)
            assert e.value.status == capi.INVALID_ARGUMENT
        finally:
            lib.aion_cuda_program_destroy(dev, prog)
        got = run_matmul(backend, capi.DTYPE_Q8_0, a_big, b_big, big_m, n, big_k, flags=capi.MATMUL_FORCE_GENERIC)
        want = oracle.matmul_q(oracle.Q8_0, a_big, b_big, big_m, n, big_k).reshape(big_m, n)
        assert np.sum((got - want) ** 2) / np.sum(want ** 2) < 1e-10
    finally:
        backend.deinit()
