"""The oracle's decoder glue steps against independent numpy float64 formulas and the
reference's stated semantics (file:line in each test)."""
import math

import numpy as np
import pytest

import oracle


def test_rms_norm_formula_and_residual():
    # src/aion/backend/cpu/exec/layernorm.zig:41-154: out = x * inv * gamma + beta (+ residual)
    rng = np.random.default_rng(1)
    x = rng.standard_normal((5, 1536)).astype(np.float32)
    g = rng.standard_normal(1536).astype(np.float32)
    b = rng.standard_normal(1536).astype(np.float32)
    res = rng.standard_normal((5, 1536)).astype(np.float32)
    x64 = x.astype(np.float64)
    want = x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + 1e-6) * g + b
    np.testing.assert_allclose(oracle.rms_norm(x, g, b, 1e-6), want, rtol=2e-6, atol=2e-6)
    np.testing.assert_allclose(oracle.rms_norm(x, g, b, 1e-6, residual=res), want + res, rtol=2e-6, atol=2e-6)
    with pytest.raises(ValueError):
        oracle.rms_norm(x, g, b, 0.0)


def test_gelu_gate_tracks_exact_gelu():
    # src/aion/backend/cpu/kernels/gelu.zig:8-14 over tanhApprox (fast_math.zig:137-141)
    a = np.linspace(-9, 9, 4001).astype(np.float32)
    b = np.full_like(a, 1.5)
    got = oracle.elemwise(oracle.ELEMWISE_GATE_GELU, a, b)
    want = np.array([0.5 * v * (1 + math.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3))) for v in a.astype(np.float64)]) * 1.5
    assert np.max(np.abs(got - want)) < 2e-4  # the polynomial exp's own error
    assert np.array_equal(oracle.elemwise(oracle.ELEMWISE_ADD, a, b), a + b)
    assert np.array_equal(oracle.elemwise(oracle.ELEMWISE_MUL, a, b), a * b)


def test_rope_pairs_halves_and_proportion():
    # src/aion/backend/cpu/kernels/rope.zig:32-97: pair i = (x[i], x[D/2 + i])
    rng = np.random.default_rng(2)
    x = rng.standard_normal((2, 3, 4, 64)).astype(np.float32)
    pos = np.array([[0, 1, 2], [7, 100, 2047]], dtype=np.int32)
    got = oracle.rope(x, pos, 10000.0)
    i = np.arange(32)
    f = 10000.0 ** (-2.0 * i / 64)
    ang = pos[..., None, None] * f
    xl, xh = x[..., :32].astype(np.float64), x[..., 32:].astype(np.float64)
    want = np.concatenate([xl * np.cos(ang) - xh * np.sin(ang), xl * np.sin(ang) + xh * np.cos(ang)], -1)
    np.testing.assert_allclose(got, want, atol=2e-3)  # f32 frequency table and angle, as in the reference
    assert np.array_equal(got[0, 0], x[0, 0])         # position 0 rotates by nothing
    half = oracle.rope(x, pos, 10000.0, proportion=0.5)
    assert np.array_equal(half[..., 16:32], x[..., 16:32]) and np.array_equal(half[..., 48:], x[..., 48:])
    np.testing.assert_array_equal(half[..., :16], got[..., :16])


def test_cast_rounds_to_nearest_even():
    x = np.array([1.0, 1.00048828125, 65504.0, 1e-8, -2.5, 70000.0], dtype=np.float32)
    assert np.array_equal(oracle.cast_f32_f16(x).view(np.uint16), x.astype(np.float16).view(np.uint16))


def test_sequence_append_plain_and_rolling():
    # src/aion/backend/cpu/exec/sequence_append.zig:12-104
    cache = np.zeros((2, 8, 2, 4), dtype=np.float16)
    new = np.arange(2 * 2 * 2 * 4, dtype=np.float16).reshape(2, 2, 2, 4)
    out = oracle.sequence_append(cache, new, [3, 6])
    assert np.array_equal(out[0, 3:5], new[0]) and np.array_equal(out[1, 6:8], new[1])
    assert out[0, :3].sum() == 0 and out[0, 5:].sum() == 0
    with pytest.raises(ValueError):
        oracle.sequence_append(cache, new, [3, 7])        # step 8 is past the end
    with pytest.raises(ValueError):
        oracle.sequence_append(cache, new, [-1, 0])
    ring = oracle.sequence_append(cache, new, [7, 17], rolling=True)
    assert np.array_equal(ring[0, 7], new[0, 0]) and np.array_equal(ring[0, 0], new[0, 1])
    assert np.array_equal(ring[1, 1], new[1, 0]) and np.array_equal(ring[1, 2], new[1, 1])


@pytest.mark.parametrize("order", ["row_major", "lanes4", "lanes32x16"])
def test_gather_rows_q8_every_index_rule(order):
    # src/aion/backend/cpu/exec/gather.zig:22-28, 57-87
    rng = np.random.default_rng(3)
    w = rng.standard_normal((64, 96)).astype(np.float32)
    rows = oracle.quantize(oracle.Q8_0, w, 1)
    table = oracle.relayout_q8(order, 64, 96, rows)
    deq = oracle.dequant(oracle.Q8_0, rows).reshape(64, 96)
    got = oracle.gather_rows_q8(table, 64, 96, [0, 63, -1, -64, 17], order=order)
    assert np.array_equal(got, deq[[0, 63, 63, 0, 17]])
    with pytest.raises(ValueError):
        oracle.gather_rows_q8(table, 64, 96, [64], order=order)
    with pytest.raises(ValueError):
        oracle.gather_rows_q8(table, 64, 96, [-65], order=order)


def test_argmax_first_maximum_and_nan():
    # src/aion/backend/cpu/exec/argmax.zig:56-82
    x = np.array([[1, 3, 3, 2], [np.nan, 5, 1, 0], [0, np.nan, 7, 7], [-np.inf, -np.inf, -np.inf, -np.inf]], dtype=np.float32)
    assert oracle.argmax(x).tolist() == [1, 0, 2, 0]
