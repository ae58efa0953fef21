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
from tests.gpu_util import DevBuf, image_bytes, make_image, matmul_plan, run_matmul, run_matmul_nt

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


# ---- decode batches beyond 16 rows: the same int8 arithmetic, weights streamed once per 64 rows ----
@pytest.mark.parametrize("dtype", [capi.DTYPE_Q8_0, capi.DTYPE_Q4_0])
@pytest.mark.parametrize("m", [17, 29, 32, 33, 48, 64, 65, 100, 128, 200, 512])
def test_decode_batches_keep_int8_arithmetic(backend, dtype, m):
    # 128-column tiles (two tiles and a tail of 8 columns), a K that is not whole stages
    n, k = 264, 2080
    x = rd.synth_acts(m, k, seed=m)
    b = oracle.quantize(dtype, rd.synth_weights(k, n, seed=7), 0)
    want = oracle.fast_matmul_q(dtype, x, b, m, n, k)
    # up to 32 rows the library picks this kernel itself; beyond, the flag keeps it (exact integer dots at any m)
    flags = capi.MATMUL_AUTO if m < capi.GEMM_MIN_M else capi.MATMUL_FORCE_GEMV
    plan = matmul_plan(backend, dtype, m, n, k, flags=flags)
    assert plan.kernel == capi.KERNEL_INT8 and plan.tile_cols == 128 and plan.tile_rows == (32 if m <= 32 else 64)
    got = run_matmul(backend, dtype, x, b, m, n, k, flags=flags)
    assert rd.rel_l2(got, want) < TIGHT


@pytest.mark.parametrize("m", [24, 64, 130])
def test_decode_batches_nt(backend, m):
    n, k = 328, 1024
    x = rd.synth_acts(m, k, seed=m)
    b = oracle.quantize(oracle.Q8_0, rd.synth_weights(n, k, seed=3), 1)
    want = oracle.fast_matmul_nt_q8(x, b, m, n, k)
    assert rd.rel_l2(run_matmul_nt(backend, x, b, m, n, k, flags=capi.MATMUL_FORCE_GEMV), want) < TIGHT


@pytest.mark.parametrize("dtype", [capi.DTYPE_Q8_0, capi.DTYPE_Q4_0])
def test_decode_batch_at_decoder_widths_alpha_beta_ldc(backend, dtype):
    # the synthetic decoder's gate/up projection for 64 requests, written into a wider C
    m, n, k, ldc = 64, 16384, 1536, 16384 + 8
    x = rd.synth_acts(m, k, seed=1)
    b = oracle.quantize(dtype, rd.synth_weights(k, n, seed=2), 0)
    c0 = rd.synth_acts(m, ldc, seed=3)
    want = oracle.fast_matmul_q(dtype, x, b, m, n, k)
    got = run_matmul(backend, dtype, x, b, m, n, k, ldc=ldc, alpha=0.5, beta=-2.0, c=c0, flags=capi.MATMUL_FORCE_GEMV)
    assert rd.rel_l2(got[:, :n], 0.5 * want - 2.0 * c0[:, :n]) < TIGHT
    assert np.array_equal(got[:, n:], c0[:, n:])


def test_a_row_does_not_depend_on_its_batch(backend):
    """Rows multiplied alone, in a batch of 8, of 32 and of 64. Up to 32 rows the int8 kernel runs (different
    tile variants and K splits, the same arithmetic: equal to f32 summation order). From 33 rows the tensor-core
    GEMM takes over; it multiplies the same int8-quantized activation, rounded to bf16 like the weights, so a
    row moves by the bf16 rounding only."""
    n, k = 1536, 2048
    x = rd.synth_acts(64, k, seed=9)
    b = oracle.quantize(oracle.Q4_0, rd.synth_weights(k, n, seed=10), 0)
    one = run_matmul(backend, capi.DTYPE_Q4_0, x[:1], b, 1, n, k)
    eight = run_matmul(backend, capi.DTYPE_Q4_0, x[:8], b, 8, n, k)
    thirty_two = run_matmul(backend, capi.DTYPE_Q4_0, x[:32], b, 32, n, k)
    forced = run_matmul(backend, capi.DTYPE_Q4_0, x, b, 64, n, k, flags=capi.MATMUL_FORCE_GEMV)
    assert rd.rel_l2(thirty_two[:8], eight) < TIGHT and rd.rel_l2(thirty_two[:1], one) < TIGHT
    assert rd.rel_l2(forced[:32], thirty_two) < TIGHT
    assert matmul_plan(backend, capi.DTYPE_Q4_0, 64, n, k).kernel == capi.KERNEL_GEMM
    gemm = run_matmul(backend, capi.DTYPE_Q4_0, x, b, 64, n, k)
    d = rd.rel_l2(gemm[:32], thirty_two)
    print(f"\nrows in a batch of 64 (tensor-core GEMM) against the same rows in a batch of 32 (int8 kernel): rel-L2 {d:.2e}")
    assert d < 5e-3


# ---- the quantized-activation image ---------------------------------------------------------
def _oracle_image_blocks(x, dtype):
    """(codes int8 [m, k], scales f32 [m, k/32]) of the reference activation quantizer."""
    m, k = x.shape
    q, s = oracle.quantize_activation(x)
    return q.reshape(m, k), s.reshape(m, k // 32)


def _decode_image(raw, m, k, dtype):
    """Undo the image layout (groups of rows, padded K blocks, fragment order): codes [m, k], scales [m, k/32]."""
    kb = k // 32
    kb_pad = (kb + 7) // 8 * 8
    rpg = 2 if m <= 1 else 8 if m <= 8 else 16 if m <= 16 else 32 if m <= 32 else 64
    groups = 1 if m <= 64 else (m + 63) // 64
    gbytes = kb_pad * rpg * 36
    assert raw.size == groups * gbytes
    codes = np.zeros((m, k), np.int8)
    scales = np.zeros((m, kb), np.float32)
    for g in range(groups):
        blob = raw[g * gbytes:(g + 1) * gbytes]
        cq = blob[: kb_pad * rpg * 32].view(np.int8).reshape(kb_pad, rpg, 8, 4)
        cs = blob[kb_pad * rpg * 32:].view(np.float32).reshape(kb_pad, rpg)
        for r in range(rpg):
            row = g * rpg + r
            if row >= m:
                assert not cq[:, r].any()
                if rpg == 2:  # a single-row image repeats the row's scale in its pad row
                    assert np.array_equal(cs[:, r], cs[:, 0])
                else:
                    assert not cs[:, r].any()
                continue
            assert not cq[kb:, r].any() and not cs[kb:, r].any()
            w = cq[:kb, r]  # [kb, 8 words, 4 bytes]
            if dtype == capi.DTYPE_Q8_0:
                # word 2j = codes 4j..4j+3, word 2j+1 = codes 16+4j..
                lo = w[:, 0::2].reshape(kb, 16)
                hi = w[:, 1::2].reshape(kb, 16)
                codes[row] = np.concatenate([lo, hi], axis=1).reshape(-1)
            else:
                # word 2j = elements 8j+{0,2,4,6}, word 2j+1 = elements 8j+{1,3,5,7}
                blk = np.zeros((kb, 32), np.int8)
                for j in range(4):
                    blk[:, 8 * j + 0:8 * j + 8:2] = w[:, 2 * j]
                    blk[:, 8 * j + 1:8 * j + 8:2] = w[:, 2 * j + 1]
                codes[row] = blk.reshape(-1)
            scales[row] = cs[:kb, r] * (16.0 if dtype == capi.DTYPE_Q4_0 else 1.0)
    return codes, scales


def _bf16_bits(x):
    """f32 -> bf16 bits, round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


@pytest.mark.parametrize("dtype", [capi.DTYPE_Q8_0, capi.DTYPE_Q4_0])
@pytest.mark.parametrize("m,k", [(33, 64), (40, 512), (130, 320)])
def test_act_image_for_the_gemm_holds_the_same_quantization_in_bf16(backend, dtype, m, k):
    """From 33 rows the image is what the tensor-core GEMM reads: bf16(code * scale) of the reference quantizer,
    row-major, K inside each group of 8 in the q4 unpack order for q4 weights."""
    x = rd.synth_acts(m, k, seed=m + k)
    x[1, 32:64] = 0.0
    a = DevBuf(backend, x)
    img = make_image(backend, dtype, a, m, k)
    try:
        raw = img.read(np.uint16)
        assert raw.size == m * k == image_bytes(m, k) // 2
        q, s = oracle.quantize_activation(x)
        deq = (q.reshape(m, k // 32, 32).astype(np.float32) * s.reshape(m, k // 32, 1)).reshape(m, k)
        want = _bf16_bits(deq).reshape(m, k // 8, 8)
        if dtype == capi.DTYPE_Q4_0:
            want = want[:, :, [0, 4, 1, 5, 2, 6, 3, 7]]
        assert np.array_equal(raw.reshape(m, k // 8, 8), want)
    finally:
        a.free()
        img.free()


@pytest.mark.parametrize("dtype", [capi.DTYPE_Q8_0, capi.DTYPE_Q4_0])
@pytest.mark.parametrize("m,k", [(1, 96), (5, 2080), (16, 256), (32, 512)])
def test_act_image_holds_the_reference_quantization(backend, dtype, m, k):
    x = rd.synth_acts(m, k, seed=m + k)
    x[0, :32] = 0.0  # a zero block: zero codes, zero scale
    a = DevBuf(backend, x)
    img = make_image(backend, dtype, a, m, k)
    try:
        raw = img.read(np.uint8)
        assert raw.size == image_bytes(m, k)
        codes, scales = _decode_image(raw, m, k, dtype)
        want_q, want_s = _oracle_image_blocks(x, dtype)
        assert np.array_equal(codes, want_q)
        assert np.array_equal(scales, want_s)
    finally:
        a.free()
        img.free()


@pytest.mark.parametrize("dtype", [capi.DTYPE_Q8_0, capi.DTYPE_Q4_0])
@pytest.mark.parametrize("m", [1, 5, 16, 40, 64, 130])
def test_matmul_with_image_equals_matmul_without(backend, dtype, m):
    n, k = 520, 1024
    x = rd.synth_acts(m, k, seed=m)
    b = oracle.quantize(dtype, rd.synth_weights(k, n, seed=5), 0)
    plain = run_matmul(backend, dtype, x, b, m, n, k)
    with_image = run_matmul(backend, dtype, x, b, m, n, k, image=True)   # int8 image up to 32 rows, bf16 image beyond
    if m == 1:  # alone, a single row is quantized inside the matmul and K may be split differently
        assert rd.rel_l2(with_image, plain) < TIGHT
    else:
        assert np.array_equal(with_image, plain)
    assert rd.rel_l2(with_image, oracle.fast_matmul_q(dtype, x, b, m, n, k)) < (TIGHT if m < capi.GEMM_MIN_M else 5e-3)
    if m >= capi.GEMM_MIN_M:  # the int8 kernel forced onto these rows has no use for a bf16 image and quantizes A itself
        forced = run_matmul(backend, dtype, x, b, m, n, k, image=True, flags=capi.MATMUL_FORCE_GEMV)
        assert rd.rel_l2(forced, oracle.fast_matmul_q(dtype, x, b, m, n, k)) < TIGHT


def test_matmul_nt_with_image(backend):
    m, n, k = 6, 256, 512
    x = rd.synth_acts(m, k)
    b = oracle.quantize(oracle.Q8_0, rd.synth_weights(n, k), 1)
    assert np.array_equal(run_matmul_nt(backend, x, b, m, n, k, image=True), run_matmul_nt(backend, x, b, m, n, k))


def test_image_operand_is_checked(backend):
    m, n, k = 4, 64, 128
    x = rd.synth_acts(m, k)
    b = oracle.quantize(oracle.Q8_0, rd.synth_weights(k, n), 0)
    bufs = [DevBuf(backend, x), DevBuf(backend, b), DevBuf(backend, nbytes=m * n * 4), DevBuf(backend, nbytes=image_bytes(m, k) - 16)]
    try:
        rec = capi.MatMul(c=bufs[2].operand(), a=bufs[0].operand(), b=bufs[1].operand(), b_dtype=capi.DTYPE_Q8_0, flags=0, m=m, n=n,
                          k=k, lda=0, ldb=0, ldc=0, alpha=1.0, beta=0.0, a_image=bufs[3].operand())
        assert backend._lib.aion_cuda_matmul(backend.handle, C.byref(rec)) == capi.INVALID_ARGUMENT  # image too short
    finally:
        for x_ in bufs:
            x_.free()


def test_plan_names_the_kernel(backend):
    assert matmul_plan(backend, capi.DTYPE_Q4_0, 1, 8192, 2048).kernel == capi.KERNEL_INT8
    assert matmul_plan(backend, capi.DTYPE_Q4_0, 32, 8192, 2048).kernel == capi.KERNEL_INT8
    assert matmul_plan(backend, capi.DTYPE_Q4_0, 33, 8192, 2048).kernel == capi.KERNEL_GEMM
    assert matmul_plan(backend, capi.DTYPE_Q4_0, 512, 8192, 2048, flags=capi.MATMUL_FORCE_GEMV).kernel == capi.KERNEL_INT8
    p = matmul_plan(backend, capi.DTYPE_Q4_0, 2048, 8192, 2048)
    assert p.kernel == capi.KERNEL_GEMM and p.tile_cols == 256
    assert matmul_plan(backend, capi.DTYPE_Q4_0, 3, 5, 64).kernel == capi.KERNEL_GENERIC  # n not a multiple of 8
    assert matmul_plan(backend, capi.DTYPE_Q8_0, 64, 256, 256, flags=capi.MATMUL_FORCE_GEMM).kernel == capi.KERNEL_GEMM


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


@pytest.mark.parametrize("dtype", [capi.DTYPE_Q8_0, capi.DTYPE_Q4_0])
@pytest.mark.parametrize("m", [1, 8, 16])
@pytest.mark.parametrize("nk", [(520, 1536), (328, 8192)])
def test_whole_tile_and_streaming_variants_agree_with_the_oracle(backend, dtype, m, nk):
    """A launch on a chain takes one whole tile per CTA (a deep K: ranges of eight stages); the same step
    recorded into parallel lanes takes the streaming variant. Both against the reference arithmetic."""
    n, k = nk
    lib, dev = backend._lib, backend.handle
    odt = oracle.Q8_0 if dtype == capi.DTYPE_Q8_0 else oracle.Q4_0
    xs = [rd.synth_acts(m, k, seed=11 + i) for i in range(2)]
    b = oracle.quantize(odt, rd.synth_weights(k, n), 0)
    want = [oracle.matmul_q(odt, x, b, m, n, k) for x in xs]
    for x, w in zip(xs, want):   # on a chain (not being recorded): whole tiles
        assert rd.rel_l2(run_matmul(backend, dtype, x, b, m, n, k), w) < TIGHT
    bufs = [DevBuf(backend, np.ascontiguousarray(b, dtype=np.uint8))]
    try:
        recs = []
        for x in xs:
            a_buf, c_buf = DevBuf(backend, x), DevBuf(backend, np.zeros(m * n, dtype=np.float32))
            bufs += [a_buf, c_buf]
            recs.append((capi.MatMul(c=c_buf.operand(), a=a_buf.operand(), b=bufs[0].operand(), b_dtype=dtype, flags=capi.MATMUL_AUTO,
                                     m=m, n=n, k=k, lda=0, ldb=0, ldc=0, alpha=1.0, beta=0.0), c_buf))
        for r, _ in recs:   # the run before the recording reserves scratch
            assert lib.aion_cuda_matmul(dev, C.byref(r)) == capi.OK
        assert lib.aion_cuda_record_begin(dev) == capi.OK
        for i, (r, _) in enumerate(recs):
            assert lib.aion_cuda_record_lane(dev, 1 + i) == capi.OK   # two parallel lanes: the streaming variant
            assert lib.aion_cuda_matmul(dev, C.byref(r)) == capi.OK
        prog = C.c_void_p()
        assert lib.aion_cuda_record_end(dev, C.byref(prog)) == capi.OK
        for _, c_buf in recs:
            backend.device_memory.memset(c_buf.handle, 0, 0, m * n * 4)
        assert lib.aion_cuda_program_launch(dev, prog) == capi.OK
        backend.sync()
        for (_, c_buf), w in zip(recs, want):
            assert rd.rel_l2(c_buf.read(np.float32).reshape(m, n), w) < TIGHT
        lib.aion_cuda_program_destroy(dev, prog)
    finally:
        for x in bufs:
            try:
                x.free()
            except BackendError:
                pass   # a failure inside the recording is the one to report


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


@pytest.mark.parametrize("m,tol", [(4, TIGHT), (64, 5e-3), (300, 5e-3)], ids=["int8", "tcgen05_one_sm", "tcgen05_pairs"])
def test_an_expired_wait_is_reported_and_the_device_stays_usable(m, tol):
    """Every barrier wait in the kernels is bounded. With the test hook on, a matmul leaves out a weight copy and polls
    briefly: the wait runs out, the kernel records the fault, frees what it holds (tensor memory in the GEMMs) and
    returns, the next synchronization reports it, and the same device object then computes correctly again. One case
    per matmul kernel: the int8 kernel, the one-SM tcgen05 GEMM and the GEMM on pairs of CTAs."""
    backend = CudaBackend(0)  # its own device object: the fault word of the shared one stays clean
    try:
        n, k = 512, 512
        x = rd.synth_acts(m, k)
        b = oracle.quantize(oracle.Q4_0, rd.synth_weights(k, n), 0)
        want = oracle.fast_matmul_q(oracle.Q4_0, x, b, m, n, k)
        assert rd.rel_l2(run_matmul(backend, capi.DTYPE_Q4_0, x, b, m, n, k), want) < tol
        assert backend._lib.aion_cuda_debug_expire_waits(backend.handle, 1) == capi.OK
        with pytest.raises(BackendError) as e:
            run_matmul(backend, capi.DTYPE_Q4_0, x, b, m, n, k)   # reading C back synchronizes and finds the fault
        assert e.value.name == "ExecutionFailed" and "bounded wait" in str(e.value)
        assert backend._lib.aion_cuda_debug_expire_waits(backend.handle, 0) == capi.OK
        assert rd.rel_l2(run_matmul(backend, capi.DTYPE_Q4_0, x, b, m, n, k), want) < tol
    finally:
        backend.deinit()
