"""Pins the CPU oracle against the reference's own test fixtures (regenerated from their
formulas in tests/refdata.py) and against independently computed "want" values."""
import numpy as np
import pytest

import oracle
from tests import refdata as rd


def test_f16_conversion_matches_ieee():
    lib = oracle.lib()
    rng = np.random.default_rng(0)
    xs = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 100.0, 3e4)])
    xs = np.concatenate([xs, np.array([0.0, -0.0, 65504, 65519.9, 65520, 2**-25, 2**-24, 2**-14, 5.96e-8],
                                      dtype=np.float32)])
    for x in xs:
        assert lib.aion_oracle_f32_to_f16(float(x)) == int(np.float32(x).astype(np.float16).view(np.uint16))
    for h in range(0, 65536, 5):
        want = np.uint16(h).view(np.float16).astype(np.float32)
        got = np.float32(lib.aion_oracle_f16_to_f32(h))
        assert (np.isnan(want) and np.isnan(got)) or want == got


def test_q8_quantizer_matches_reference_test_vector():
    # src/aion/storage/quantize.zig:105-137
    vals, expect = rd.quantize_zig_q8_kn()
    got = oracle.quantize(oracle.Q8_0, vals, 0)
    assert np.array_equal(got, expect)


@pytest.mark.parametrize("axis", [0, 1])
def test_q8_q4_quantizers_match_numpy_restatement(axis):
    rng = np.random.default_rng(7)
    w = (rng.standard_normal((64, 96)) * 0.02).astype(np.float32)
    w[0:32, 3] = 0.0  # an all-zero block along axis 0
    w[5, 32:64] = 0.0  # and one along axis 1
    for dtype, packer in ((oracle.Q8_0, rd.pack_q8_block_np), (oracle.Q4_0, rd.pack_q4_block_np)):
        got = oracle.quantize(dtype, w, axis)
        want = bytearray()
        if axis == 0:
            for kb in range(2):
                for j in range(96):
                    want += packer(w[kb * 32:(kb + 1) * 32, j])
        else:
            for r in range(64):
                for kb in range(3):
                    want += packer(w[r, kb * 32:(kb + 1) * 32])
        assert np.array_equal(got, np.frombuffer(bytes(want), dtype=np.uint8))


def test_q4_nibble_order_and_dequant():
    # even element -> low nibble, odd -> high; value = nibble - 8
    # (src/aion/backend/cpu/kernels/matmul_q_i8.zig:362-369).
    block = bytearray(np.float16(0.5).tobytes())
    block += bytes((t & 0xF) | (((15 - t) & 0xF) << 4) for t in range(16))
    out = oracle.dequant(oracle.Q4_0, np.frombuffer(bytes(block), dtype=np.uint8))
    want = np.empty(32, dtype=np.float32)
    want[0::2] = (np.arange(16) - 8) * 0.5
    want[1::2] = ((15 - np.arange(16)) - 8) * 0.5
    assert np.array_equal(out, want)


def test_dequant_is_exact_product():
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((32 * 50,)) * 0.02).astype(np.float32)
    for dtype, bb in ((oracle.Q8_0, 34), (oracle.Q4_0, 18)):
        packed = oracle.quantize(dtype, w.reshape(50, 32), 1)
        deq = oracle.dequant(dtype, packed)
        for i in range(50):
            blk = packed[i * bb:(i + 1) * bb]
            scale = np.float32(blk[:2].view(np.float16)[0])
            if dtype == oracle.Q8_0:
                q = blk[2:].view(np.int8).astype(np.float32)
            else:
                q = np.empty(32, dtype=np.float32)
                q[0::2] = (blk[2:] & 0xF).astype(np.float32) - 8
                q[1::2] = (blk[2:] >> 4).astype(np.float32) - 8
            assert np.array_equal(deq[i * 32:(i + 1) * 32], q * scale)


def test_activation_quantizer():
    rng = np.random.default_rng(5)
    a = rng.standard_normal(32 * 40).astype(np.float32)
    a[64:96] = 0.0
    a[100] = 3.5  # a half-way case somewhere is likely; the numpy restatement rounds half away too
    q, s = oracle.quantize_activation(a)
    for kb in range(40):
        wq, ws = rd.quantize_a_block_np(a[kb * 32:(kb + 1) * 32])
        assert np.array_equal(q[kb * 32:(kb + 1) * 32], wq)
        assert s[kb] == ws
    assert s[2] == 0 and not q[64:96].any()


def test_matvec_q8_chunk_boundary_case():
    # src/aion/backend/cpu/kernels/matvec_q.zig:176-219: k past the 8192 activation chunk, m = 2, rel 1e-5.
    m, n, k, a, b = rd.matvec_q_chunk_case()
    got = oracle.matmul_q(oracle.Q8_0, a, b, m, n, k)
    want = rd.int8_reference_f64(a, b, m, n, k, nt=False)
    np.testing.assert_allclose(got, want, rtol=1e-5)
    # the packed-GEMM route agrees to the same bound
    got2 = oracle.matmul_q(oracle.Q8_0, a, b, m, n, k, route=2)
    np.testing.assert_allclose(got2, want, rtol=1e-5)


@pytest.mark.parametrize("order,group", [("row_major", 1), ("lanes4", 4), ("lanes8", 8), ("lanes16", 16), ("lanes32", 32)])
@pytest.mark.parametrize("m", [1, 2, 7, 10])
def test_matmul_nt_grouped_orders(order, group, m):
    # src/aion/backend/cpu/kernels/matmul_nt_q.zig:587-637: abs 1e-4 * max(1, |want|)
    m, n, k, a, rows = rd.nt_grouped_case(group, m)
    tile = oracle.relayout_q8(order, n, k, rows)
    got = oracle.matmul_nt_q8(a, tile, m, n, k, order=order)
    want = rd.int8_reference_f64(a, rows, m, n, k, nt=True)
    assert np.all(np.abs(got - want) <= 1e-4 * np.maximum(1.0, np.abs(want)))


@pytest.mark.parametrize("order,group,chunk", [("lanes4", 4, 4), ("lanes8", 8, 4), ("lanes16", 16, 4), ("lanes32", 32, 4),
                                               ("lanes32x16", 32, 16)])
def test_relayout_byte_map(order, group, chunk):
    # src/aion/graph/opt/test_opt.zig:921-968 (the map), for every order incl. the GPU one.
    n, k = 96, 64
    w = (np.array([((i * 7 + 3) % 23) - 11 for i in range(n * k)], dtype=np.float32) * np.float32(0.07)).reshape(n, k)
    rows = oracle.quantize(oracle.Q8_0, w, 1)
    got = oracle.relayout_q8(order, n, k, rows)
    assert np.array_equal(got, rd.relayout_map_np(group, chunk, n, k, rows))
    assert np.array_equal(oracle.relayout_q8(order, n, k, got, inverse=True), rows)


@pytest.mark.parametrize("m", [1, 2, 3, 7, 8, 17])
def test_weight_layout_arithmetic_case(m):
    # src/aion/graph/opt/test_opt.zig:1106-1175: NMSE < 1e-10 vs the f64 int8 reference,
    # for the K-major MatMul and for the same weight as [N,K] NT.
    m, n, k, a, w = rd.weight_layout_arith_case(m)
    b_km = oracle.quantize(oracle.Q8_0, w, 0)
    want = rd.int8_reference_f64(a, b_km, m, n, k, nt=False)
    got = oracle.matmul_q(oracle.Q8_0, a, b_km, m, n, k)
    nmse = np.sum((got - want) ** 2) / np.sum(want ** 2)
    assert nmse < 1e-10
    b_nt = oracle.quantize(oracle.Q8_0, np.ascontiguousarray(w.T), 1)
    got_nt = oracle.matmul_nt_q8(a, b_nt, m, n, k)
    assert np.sum((got_nt - want) ** 2) / np.sum(want ** 2) < 1e-10


def test_nt_backend_case():
    # src/aion/backend/cpu/test_cpu_backend.zig:2879-3012: abs 1e-4
    m, n, k, a, packed, c_ref = rd.nt_backend_case()
    got = oracle.matmul_nt_q8(a, packed, m, n, k)
    np.testing.assert_allclose(got, c_ref, atol=1e-4)


def test_q4_matmul_against_f64_int8_reference_and_loose_f32_bound():
    # The reference's only q4 numeric test (src/aion/backend/cpu/test_cpu_kernels.zig:572-617)
    # bounds the q4 GEMM against the UNQUANTIZED f32 product by 0.8 abs on U(-1,1) inputs.
    rng = np.random.default_rng(0x9999)
    m, n, k = 8, 32, 64
    a = ((rng.random((m, k), dtype=np.float32) - 0.5) * 2).astype(np.float32)
    w = ((rng.random((k, n), dtype=np.float32) - 0.5) * 2).astype(np.float32)
    b = oracle.quantize(oracle.Q4_0, w, 0)
    got = oracle.matmul_q(oracle.Q4_0, a, b, m, n, k)
    assert np.max(np.abs(got - a @ w)) < 0.8
    want = rd.int8_reference_f64(a, b, m, n, k, nt=False, bb=18)
    np.testing.assert_allclose(got, want, rtol=2e-5, atol=1e-6)


def test_alpha_beta_ldc_epilogue():
    rng = np.random.default_rng(11)
    m, n, k = 3, 40, 96
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    c0 = rng.standard_normal((m, 48)).astype(np.float32)
    for dtype in (oracle.Q8_0, oracle.Q4_0):
        b = oracle.quantize(dtype, w, 0)
        plain = oracle.matmul_q(dtype, a, b, m, n, k)
        got = oracle.matmul_q(dtype, a, b, m, n, k, ldc=48, alpha=0.5, beta=-2.0, c=c0)
        np.testing.assert_allclose(got[:, :n], 0.5 * plain - 2.0 * c0[:, :n], rtol=1e-5, atol=1e-6)
        assert np.array_equal(got[:, n:], c0[:, n:])  # columns past n are untouched


def test_int8a_vs_deqf32_distance_is_the_documented_gap():
    # Reference: "They quantize different operands" (src/aion/backend/gpu/test_gpu_backend.zig:1004-1014).
    m, n, k = 2, 64, 2048
    a = rd.synth_acts(m, k)
    w = rd.synth_weights(k, n)
    for dtype in (oracle.Q8_0, oracle.Q4_0):
        b = oracle.quantize(dtype, w, 0)
        d = rd.rel_l2(oracle.matmul_deqf32(dtype, a, b, m, n, k), oracle.matmul_q(dtype, a, b, m, n, k))
        assert 1e-3 < d < 2e-2


def test_exp_and_tanh_approx_accuracy():
    lib = oracle.lib()
    xs = np.linspace(-20, 0, 2001, dtype=np.float32)
    err = max(abs(lib.aion_oracle_exp_approx(float(x)) - np.exp(np.float64(x))) / np.exp(np.float64(x)) for x in xs)
    assert err < 1e-4  # 4th-order Taylor on |t| <= ln2/2 (src/aion/backend/cpu/kernels/fast_math.zig:53-63)
    assert lib.aion_oracle_exp_approx(0.0) == 1.0
    ts = np.linspace(-6, 6, 1201, dtype=np.float32)
    assert max(abs(lib.aion_oracle_tanh_approx(float(x)) - np.tanh(np.float64(x))) for x in ts) < 3e-4


def test_attention_exact_known_answer():
    # src/aion/api/test_api.zig:3256-3330
    q, k, v, pos, end, kw, expected = rd.api_attention_case()
    got = oracle.attention(q, k, v, positions=pos, kv_lengths=end, **kw)
    np.testing.assert_allclose(got, expected, atol=1e-6)


def test_attention_matches_cached_gqa_reference():
    # src/aion/backend/cpu/test_cpu_backend.zig:4906-5172: max abs 8e-2 (f32), 1.5e-1 (f16 K/V).
    q, k, v, pos, end, kw = rd.gqa_case_f32()
    want = rd.cached_gqa_ref(q, k, v, pos, end, **kw)
    got = oracle.attention(q, k, v, positions=pos, kv_lengths=end, **kw)
    assert np.max(np.abs(got - want)) < 2e-3  # far inside the reference's 8e-2
    got16 = oracle.attention(q, k.astype(np.float16), v.astype(np.float16), positions=pos, kv_lengths=end, **kw)
    assert np.max(np.abs(got16 - want)) < 1.5e-1
    exact = oracle.attention(q, k, v, positions=pos, kv_lengths=end, exact=True, **kw)
    assert np.max(np.abs(exact - want)) < 1e-5


def test_attention_long_context_online_path_and_ring():
    rng = np.random.default_rng(21)
    B, Hq, Hkv, D, T = 1, 4, 1, 32, 2500
    q = rng.standard_normal((B, 1, Hq, D)).astype(np.float16)
    k = rng.standard_normal((B, T, Hkv, D)).astype(np.float16)
    v = rng.standard_normal((B, T, Hkv, D)).astype(np.float16)
    kw = dict(scale=1 / np.sqrt(D), right=0)
    pos = np.array([[T - 1]], dtype=np.int32)
    lens = np.array([T], dtype=np.int32)
    got = oracle.attention(q, k, v, positions=pos, kv_lengths=lens, **kw)        # > 2048 keys: online path
    exact = oracle.attention(q, k, v, positions=pos, kv_lengths=lens, exact=True, **kw)
    assert rd.rel_l2(got, exact) < 1e-4
    # A ring of T rows holding logical keys [300, 300+T): identical to a plain cache holding them in order.
    total = T + 300
    kl = rng.standard_normal((B, total, Hkv, D)).astype(np.float16)
    vl = rng.standard_normal((B, total, Hkv, D)).astype(np.float16)
    ring_k = np.empty_like(k)
    ring_v = np.empty_like(v)
    for t in range(300, total):
        ring_k[:, t % T] = kl[:, t]
        ring_v[:, t % T] = vl[:, t]
    ring = oracle.attention(q, ring_k, ring_v, positions=np.array([[total - 1]], dtype=np.int32),
                            kv_lengths=np.array([total], dtype=np.int32), rolling=True, **kw)
    plain = oracle.attention(q, kl[:, 300:], vl[:, 300:], positions=pos, kv_lengths=lens, **kw)
    np.testing.assert_allclose(ring, plain, rtol=1e-5, atol=1e-6)


def test_attention_empty_window_is_zero_and_bad_inputs_fail():
    q = np.ones((1, 1, 2, 4), dtype=np.float32)
    k = np.ones((1, 4, 1, 4), dtype=np.float32)
    v = np.ones((1, 4, 1, 4), dtype=np.float32)
    out = oracle.attention(q, k, v, scale=1.0, positions=np.array([[0]], dtype=np.int32),
                           kv_lengths=np.array([0], dtype=np.int32), right=0)
    assert not out.any()
    with pytest.raises(ValueError):
        oracle.attention(q, k, v, scale=1.0, kv_lengths=np.array([9], dtype=np.int32))  # beyond a non-rolling cache
    with pytest.raises(ValueError):
        oracle.attention(q, k, v, scale=0.0)
