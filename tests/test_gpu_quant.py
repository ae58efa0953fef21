"""Device quantizer / dequantizer / re-layout against the oracle: byte- and bit-exact."""
import numpy as np
import pytest

import oracle
from aion_b200 import backend as ab
from aion_b200 import capi
from tests import refdata as rd
from tests.gpu_util import run_matmul, run_matmul_nt

pytestmark = pytest.mark.gpu


def test_q8_reference_vector(backend):
    vals, expect = rd.quantize_zig_q8_kn()  # src/aion/storage/quantize.zig:105-137
    assert np.array_equal(ab.quantize(backend, capi.DTYPE_Q8_0, vals, 0), expect)


@pytest.mark.parametrize("dtype", [capi.DTYPE_Q8_0, capi.DTYPE_Q4_0])
@pytest.mark.parametrize("shape,axis", [((2048, 256), 0), ((256, 2048), 1), ((3, 64, 40), 1), ((32, 1), 0)])
def test_quantize_bytes_equal_oracle(backend, dtype, shape, axis):
    rng = np.random.default_rng(sum(shape) + axis)
    w = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    w.reshape(-1)[: min(64, w.size)] = 0.0
    # exact half-way quotients and the clamp edges
    w.reshape(-1)[-1] = np.abs(w).max() * 2
    got = ab.quantize(backend, dtype, w, axis)
    assert np.array_equal(got, oracle.quantize(dtype, w, axis))


@pytest.mark.parametrize("dtype", [capi.DTYPE_Q8_0, capi.DTYPE_Q4_0])
def test_dequantize_bit_exact(backend, dtype):
    w = rd.synth_weights(512, 2048)
    packed = oracle.quantize(dtype, w, 1)
    got = ab.dequantize(backend, dtype, packed)
    want = oracle.dequant(dtype, packed)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequantize_every_code_and_scale_class(backend):
    # every q8 code and every nibble against normal, subnormal and large f16 scales
    for dtype, bb in ((capi.DTYPE_Q8_0, 34), (capi.DTYPE_Q4_0, 18)):
        blocks = bytearray()
        for sbits in (0x0001, 0x03FF, 0x0400, 0x211F, 0x3C00, 0x7BFF, 0x8001, 0xA11F):
            for base in range(0, 256, 32):
                payload = bytes((base + t) & 0xFF for t in range(bb - 2))
                blocks += int(sbits).to_bytes(2, "little") + payload
        packed = np.frombuffer(bytes(blocks), dtype=np.uint8)
        got = ab.dequantize(backend, dtype, packed)
        assert np.array_equal(got.view(np.uint32), oracle.dequant(dtype, packed).view(np.uint32))


@pytest.mark.parametrize("order", range(1, 6))
def test_relayout_matches_oracle_and_inverts(backend, order):
    n, k = 96, 256
    rows = oracle.quantize(oracle.Q8_0, rd.synth_weights(n, k), 1)
    got = ab.relayout_q8(backend, order, n, k, rows)
    assert np.array_equal(got, oracle.relayout_q8(order, n, k, rows))
    assert np.array_equal(ab.relayout_q8(backend, order, n, k, got, inverse=True), rows)


@pytest.mark.parametrize("order", range(0, 6))
@pytest.mark.parametrize("n,k", [(96, 256), (160, 2080)])
def test_derived_kmajor_weight_is_the_block_transpose(backend, order, n, k):
    """Any stored order -> the K-major layout `MatMul` reads: the same 34-byte blocks, [k/32][n]; both
    steps then give the reference's int8 arithmetic over the same blocks."""
    rows = oracle.quantize(oracle.Q8_0, rd.synth_weights(n, k), 1)
    stored = rows if order == 0 else oracle.relayout_q8(order, n, k, rows)
    got = ab.derive_kmajor_q8(backend, order, n, k, stored)
    want = rows.reshape(n, k // 32, 34).transpose(1, 0, 2)
    assert np.array_equal(got.reshape(k // 32, n, 34), want)
    a = rd.synth_acts(3, k)
    c_nt = run_matmul_nt(backend, a, stored, 3, n, k, order=order)
    c_km = run_matmul(backend, capi.DTYPE_Q8_0, a, got, 3, n, k)
    want_c = rd.int8_reference_f64(a, rows, 3, n, k, nt=True)
    assert rd.rel_l2(c_km, want_c) < 2e-5 and rd.rel_l2(c_nt, want_c) < 2e-5


@pytest.mark.parametrize("m", [4, 64])
@pytest.mark.parametrize("order", [0, 3])
def test_a_matmul_issued_right_after_the_derivation_reads_the_finished_weight(backend, order, m):
    """The matmul kernels start their weight loads without waiting for the kernel before them, so a kernel that
    writes weights must not let its successors start early: derive, then multiply, with nothing in between,
    over a matrix large enough that the derivation is still running when the matmul is issued."""
    import ctypes as C
    n, k = 8192, 2048
    rows = oracle.quantize(oracle.Q8_0, rd.synth_weights(n, k), 1)
    stored = rows if order == 0 else oracle.relayout_q8(order, n, k, rows)
    a = rd.synth_acts(m, k)
    mem, lib, dev = backend.device_memory, backend._lib, backend.handle
    nb = stored.nbytes
    hs, hd, ha, hc = mem.alloc(nb), mem.alloc(nb), mem.alloc(a.nbytes), mem.alloc(m * n * 4)
    try:
        mem.copy_h2d(hs, 0, np.ascontiguousarray(stored, dtype=np.uint8))
        mem.copy_h2d(ha, 0, a)
        mem.memset(hd, 0, 0, nb)
        backend.sync()
        so, do = capi.Operand(hs, 0, nb), capi.Operand(hd, 0, nb)
        rec = capi.MatMul(c=capi.Operand(hc, 0, m * n * 4), a=capi.Operand(ha, 0, a.nbytes), b=do, b_dtype=capi.DTYPE_Q8_0,
                          flags=capi.MATMUL_AUTO, m=m, n=n, k=k, lda=0, ldb=0, ldc=0, alpha=1.0, beta=0.0)
        for rnd in range(3):   # the first round sizes scratch (and may synchronize); the later ones run back to back
            if rnd:
                mem.memset(hd, 0, 0, nb)   # a matmul that read too early would see zero weights
            assert lib.aion_cuda_derive_kmajor_q8(dev, order, n, k, C.byref(so), C.byref(do)) == capi.OK
            assert lib.aion_cuda_matmul(dev, C.byref(rec)) == capi.OK
        backend.sync()
        got = np.empty(m * n, dtype=np.float32)
        mem.copy_d2h(got, hc, 0)
        want = oracle.matmul_nt_q8(a, rows, m, n, k)   # the reference's int8 arithmetic over the same blocks
        tol = 2e-5 if m <= 32 else 1e-2
        assert rd.rel_l2(got.reshape(m, n), want) < tol
    finally:
        for h in (hs, hd, ha, hc):
            mem.free(h)


def test_quantize_rejects_bad_arguments(backend):
    with pytest.raises(ab.BackendError) as e:
        ab.quantize(backend, capi.DTYPE_Q8_0, np.zeros((33, 4), dtype=np.float32), 0)
    assert e.value.name == "InvalidArgument"
    with pytest.raises(ab.BackendError) as e:
        ab.quantize(backend, capi.DTYPE_F16, np.zeros((32, 4), dtype=np.float32), 0)
    assert e.value.name == "Unsupported"
