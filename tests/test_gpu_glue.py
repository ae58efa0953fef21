"""Decoder glue steps: the CUDA kernels through `CudaSession` (C ABI) against the oracle.

Elementwise, cast, append, gather and argmax are integer / per-element work: bit-exact.
RMSNorm sums a row in a different order than the CPU's vector lanes: rel 1e-5. RoPE's
sin / cos come from the device's f64 sincos instead of the host libm: abs 1e-6."""
import numpy as np
import pytest

import oracle
from aion_b200 import capi
from aion_b200.backend import (BackendError, DeviceStore, StepArgMax, StepCast, StepElemwiseBinary, StepGatherRows,
                               StepRMSNorm, StepRMSNormPair, StepRoPE1D, StepSequenceAppend, TensorMeta, act_image_meta)
from tests import refdata as rd
from tests.gpu_util import DevBuf, make_image

pytestmark = pytest.mark.gpu

F32, F16, I32, Q8 = capi.DTYPE_F32, capi.DTYPE_F16, capi.DTYPE_I32, capi.DTYPE_Q8_0


@pytest.fixture()
def sess(backend):
    store = DeviceStore(backend.device_memory)
    s = backend.create_session(store)
    yield s, store
    store.deinit()


def put(store, arr, dtype):
    return store.add(TensorMeta(dtype, tuple(arr.shape)), arr)


# Rows of up to 4096 columns (a multiple of 4) take the register-resident kernel, two or four
# float4 chunks per thread; wider or ragged rows the element-wise one.
@pytest.mark.parametrize("rows,cols", [(1, 1536), (7, 256), (64, 1536), (3, 100), (520, 32), (5, 4096), (3, 3000), (2, 8200),
                                       (3, 1023)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rms_norm(sess, rows, cols, with_res):
    s, store = sess
    rng = np.random.default_rng(rows * 1000 + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    g = rng.standard_normal(cols).astype(np.float32)
    b = rng.standard_normal(cols).astype(np.float32)
    res = rng.standard_normal((rows, cols)).astype(np.float32) if with_res else None
    tx, tg, tb = put(store, x, F32), put(store, g, F32), put(store, b, F32)
    tr = put(store, res, F32) if with_res else None
    to = store.add(TensorMeta(F32, (rows, cols)))
    s.execute([StepRMSNorm(out=to, x=tx, gamma=tg, beta=tb, eps=1e-6, residual=tr)])
    np.testing.assert_allclose(store.read(to), oracle.rms_norm(x, g, b, 1e-6, residual=res), rtol=1e-5, atol=1e-6)


def test_rms_norm_in_place_and_bad_eps(sess):
    s, store = sess
    x = np.random.default_rng(0).standard_normal((4, 8, 256)).astype(np.float32)
    g, b = np.ones(256, np.float32), np.zeros(256, np.float32)
    tx, tg, tb = put(store, x, F32), put(store, g, F32), put(store, b, F32)
    s.execute([StepRMSNorm(out=tx, x=tx, gamma=tg, beta=tb, eps=1e-6)])
    np.testing.assert_allclose(store.read(tx), oracle.rms_norm(x, g, b, 1e-6), rtol=1e-5, atol=1e-6)
    with pytest.raises(BackendError):
        s.execute([StepRMSNorm(out=tx, x=tx, gamma=tg, beta=tb, eps=0.0)])


@pytest.mark.parametrize("op,code", [("add", 0), ("mul", 1), ("gate", 2)])
@pytest.mark.parametrize("n", [70001, 1 << 21])  # element by element; as float4s (large, aligned counts)
def test_elemwise_bit_exact(sess, op, code, n):
    s, store = sess
    rng = np.random.default_rng(code)
    a = (rng.standard_normal(n) * 4).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    a[:8] = [0.0, -0.0, 50.0, -50.0, 1e-30, 9.99, -9.99, 100.0]
    ta, tb = put(store, a, F32), put(store, b, F32)
    to = store.add(TensorMeta(F32, a.shape))
    s.execute([StepElemwiseBinary(op=op, out=to, a=ta, b=tb)])
    assert np.array_equal(store.read(to), oracle.elemwise(code, a, b))


# ---- producers that also write the quantized image of their output ---------------------------
def _image_of(backend, store, tid, rows, cols, dtype):
    """The image aion_cuda_act_image makes of a tensor's f32 values: what a fused producer must equal."""
    vals = store.read(tid).reshape(rows, cols)
    a = DevBuf(backend, vals)
    img = make_image(backend, dtype, a, rows, cols)
    try:
        return img.read(np.uint8)
    finally:
        a.free()
        img.free()


@pytest.mark.parametrize("dtype", [capi.DTYPE_Q4_0, capi.DTYPE_Q8_0])
@pytest.mark.parametrize("rows,cols", [(1, 1536), (8, 1536), (20, 256), (64, 1536), (70, 4096), (3, 2080)])
def test_rms_norm_writes_the_image_of_its_output(sess, backend, dtype, rows, cols):
    s, store = sess
    rng = np.random.default_rng(rows + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    g = rng.standard_normal(cols).astype(np.float32)
    b = rng.standard_normal(cols).astype(np.float32)
    res = rng.standard_normal((rows, cols)).astype(np.float32)
    tx, tg, tb, tr = put(store, x, F32), put(store, g, F32), put(store, b, F32), put(store, res, F32)
    to, to2 = store.add(TensorMeta(F32, (rows, cols))), store.add(TensorMeta(F32, (rows, cols)))
    ti = store.add(act_image_meta(rows, cols, dtype))
    s.execute([StepRMSNorm(out=to, x=tx, gamma=tg, beta=tb, eps=1e-6, image=ti)])
    assert np.array_equal(store.read(ti).view(np.uint8), _image_of(backend, store, to, rows, cols, dtype))
    np.testing.assert_allclose(store.read(to), oracle.rms_norm(x, g, b, 1e-6), rtol=1e-5, atol=1e-6)
    # the pair: the image is that of the second output
    s.execute([StepRMSNormPair(out1=to, out2=to2, x=tx, gamma1=tg, beta1=tb, gamma2=tg, beta2=tb, eps1=1e-6, eps2=1e-5,
                               residual=tr, image=ti)])
    assert np.array_equal(store.read(ti).view(np.uint8), _image_of(backend, store, to2, rows, cols, dtype))
    first = oracle.rms_norm(x, g, b, 1e-6, residual=res)
    np.testing.assert_allclose(store.read(to), first, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(store.read(to2), oracle.rms_norm(first, g, b, 1e-5), rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("dtype", [capi.DTYPE_Q4_0, capi.DTYPE_Q8_0])
@pytest.mark.parametrize("rows,cols", [(1, 8192), (8, 8192), (65, 512), (3, 96)])
def test_gate_writes_the_image_of_its_output(sess, backend, dtype, rows, cols):
    # the two halves of a [gate | up] matmul output, as the fused decoder reads them
    s, store = sess
    rng = np.random.default_rng(cols)
    gu = (rng.standard_normal((rows, 2 * cols)) * 3).astype(np.float32)
    tgu = put(store, gu, F32)
    ch = store.acquire_const(tgu)
    half = TensorMeta(F32, (rows, cols), row_stride=2 * cols)
    from aion_b200.backend import Chunk

    tgate = store.bind(half, Chunk(ch.handle, ch.offset, ch.len))
    tup = store.bind(half, Chunk(ch.handle, ch.offset + cols * 4, ch.len - cols * 4))
    to = store.add(TensorMeta(F32, (rows, cols)))
    ti = store.add(act_image_meta(rows, cols, dtype))
    s.execute([StepElemwiseBinary(op="gate", out=to, a=tgate, b=tup, image=ti)])
    want = oracle.elemwise(2, np.ascontiguousarray(gu[:, :cols]), np.ascontiguousarray(gu[:, cols:]))
    assert np.array_equal(store.read(to), want)
    assert np.array_equal(store.read(ti).view(np.uint8), _image_of(backend, store, to, rows, cols, dtype))


@pytest.mark.parametrize("shape,prop", [((2, 1, 8, 256), 1.0), ((3, 5, 1, 64), 1.0), ((1, 2, 4, 128), 0.25)])
def test_rope(sess, shape, prop):
    s, store = sess
    rng = np.random.default_rng(4)
    x = rng.standard_normal(shape).astype(np.float32)
    pos = rng.integers(0, 4096, size=shape[:2]).astype(np.int32)
    pos.flat[0] = 2047
    tx, tp = put(store, x, F32), put(store, pos, I32)
    to = store.add(TensorMeta(F32, shape))
    s.execute([StepRoPE1D(out=to, x=tx, positions=tp, base_frequency=10000.0, rope_proportion=prop)])
    np.testing.assert_allclose(store.read(to), oracle.rope(x, pos, 10000.0, proportion=prop), rtol=0, atol=1e-6)


def test_cast_both_ways_bit_exact(sess):
    s, store = sess
    x = (np.random.default_rng(5).standard_normal(5000) * 100).astype(np.float32)
    x[:6] = [1.00048828125, 65504.0, 1e-8, -2.5, 6.1e-5, 3.0e-8]
    tx = put(store, x, F32)
    th = store.add(TensorMeta(F16, x.shape))
    tb = store.add(TensorMeta(F32, x.shape))
    s.execute([StepCast(out=th, x=tx, to_dtype=F16), StepCast(out=tb, x=th, to_dtype=F32)])
    want = oracle.cast_f32_f16(x)
    assert np.array_equal(store.read(th).view(np.uint16), want.view(np.uint16))
    assert np.array_equal(store.read(tb), want.astype(np.float32))


@pytest.mark.parametrize("rolling", [False, True])
def test_sequence_append(sess, rolling):
    s, store = sess
    rng = np.random.default_rng(6)
    cache = rng.standard_normal((3, 16, 1, 256)).astype(np.float16)
    new = rng.standard_normal((3, 2, 1, 256)).astype(np.float16)
    idx = np.array([0, 14, 37 if rolling else 5], dtype=np.int32)
    tc = store.add(TensorMeta(F16, cache.shape, cache_policy="rolling" if rolling else "none"), cache)
    tn, ti = put(store, new, F16), put(store, idx, I32)
    s.execute([StepSequenceAppend(cache=tc, new_kv=tn, end_index=ti)])
    assert np.array_equal(store.read(tc).view(np.uint16), oracle.sequence_append(cache, new, idx, rolling=rolling).view(np.uint16))


def test_sequence_append_into_a_paged_cache_then_attention_reads_it(sess, backend):
    """New rows go to the pages the table names (byte-equal to the contiguous append gathered page by
    page), and the attention step then reads the same pool through the same table."""
    from aion_b200.backend import AttentionWindow, StepAttention
    s, store = sess
    rng = np.random.default_rng(16)
    B, T, H, D, PT, Ln = 3, 256, 2, 64, 64, 5
    per = T // PT
    pool = B * per + 2
    table = rng.permutation(pool)[: B * per].reshape(B, per).astype(np.int32)
    k0 = rng.standard_normal((B, T, H, D)).astype(np.float16)
    v0 = rng.standard_normal((B, T, H, D)).astype(np.float16)
    idx = np.array([0, 62, 200], dtype=np.int32)     # the second request's rows straddle two pages
    knew = rng.standard_normal((B, Ln, H, D)).astype(np.float16)
    vnew = rng.standard_normal((B, Ln, H, D)).astype(np.float16)

    def to_pool(c):
        p = np.zeros((pool, PT, H, D), dtype=np.float16)
        for b in range(B):
            for i in range(per):
                p[table[b, i]] = c[b, i * PT:(i + 1) * PT]
        return p

    tk = store.add(TensorMeta(F16, (pool, PT, H, D)), to_pool(k0))
    tv = store.add(TensorMeta(F16, (pool, PT, H, D)), to_pool(v0))
    tt, ti = put(store, table, I32), put(store, idx, I32)
    tkn, tvn = put(store, knew, F16), put(store, vnew, F16)
    q = rng.standard_normal((B, Ln, 4, D)).astype(np.float16)
    pos = (idx[:, None] + np.arange(Ln, dtype=np.int32)[None, :]).astype(np.int32)
    lens = (idx + Ln).astype(np.int32)
    tq, tp, tl = put(store, q, F16), put(store, pos, I32), put(store, lens, I32)
    to = store.add(TensorMeta(F32, (B, Ln, 4, D)))
    s.execute([StepSequenceAppend(cache=tk, new_kv=tkn, end_index=ti, page_table=tt),
               StepSequenceAppend(cache=tv, new_kv=tvn, end_index=ti, page_table=tt),
               StepAttention(out=to, q=tq, k=tk, v=tv, query_positions=tp, kv_lengths=tl, scale=0.125,
                             window=AttentionWindow.causal(), page_table=tt)])
    k1, v1 = oracle.sequence_append(k0, knew, idx), oracle.sequence_append(v0, vnew, idx)
    assert np.array_equal(store.read(tk).view(np.uint16), to_pool(k1).view(np.uint16))
    assert np.array_equal(store.read(tv).view(np.uint16), to_pool(v1).view(np.uint16))
    want = oracle.attention(q, k1, v1, scale=0.125, positions=pos, kv_lengths=lens, right=0)
    assert rd.rel_l2(store.read(to), want) < 1e-3


def test_sequence_append_out_of_range_is_reported(sess, backend):
    s, store = sess
    cache = np.zeros((2, 8, 1, 64), dtype=np.float16)
    new = np.ones((2, 1, 1, 64), dtype=np.float16)
    tc, tn = put(store, cache, F16), put(store, new, F16)
    ti = put(store, np.array([3, 8], dtype=np.int32), I32)
    s.execute([StepSequenceAppend(cache=tc, new_kv=tn, end_index=ti)])
    with pytest.raises(BackendError):
        backend.sync()
    got = store.read(tc)
    assert got[0, 3].sum() == 64 and got[1].sum() == 0   # the valid request was written, the bad one untouched


@pytest.mark.parametrize("order", [capi.ORDER_ROW_MAJOR, capi.ORDER_LANES8, capi.ORDER_LANES32X16])
def test_gather_rows_q8(sess, backend, order):
    s, store = sess
    rng = np.random.default_rng(7)
    V, D = 128, 1536
    w = rng.standard_normal((V, D)).astype(np.float32)
    table = oracle.relayout_q8(order, V, D, oracle.quantize(oracle.Q8_0, w, 1))
    idx = np.array([[0, 127, -1], [-128, 5, 64]], dtype=np.int32)
    tt = store.add(TensorMeta(Q8, (V, D), quant_axis=1, block_order=order), table)
    ti = put(store, idx, I32)
    to = store.add(TensorMeta(F32, (2, 3, D)))
    s.execute([StepGatherRows(out=to, table=tt, indices=ti)])
    assert np.array_equal(store.read(to).reshape(6, D), oracle.gather_rows_q8(table, V, D, idx, order=order))
    store.write(ti, np.array([[0, 128, 0], [0, 0, 0]], dtype=np.int32))
    s.execute([StepGatherRows(out=to, table=tt, indices=ti)])
    with pytest.raises(BackendError):
        backend.sync()


def test_argmax(sess):
    s, store = sess
    rng = np.random.default_rng(8)
    x = rng.standard_normal((9, 262144)).astype(np.float32)
    x[0, 100] = x[0, 200000] = 9.0           # tie: the first wins
    x[1, 0] = np.nan                         # NaN in front answers 0
    x[2, 5] = np.nan
    x[2, 262143] = 11.0                      # NaN elsewhere is skipped
    x[3, :] = -np.inf
    ta = put(store, x, F32)
    to = store.add(TensorMeta(I32, (9,)))
    s.execute([StepArgMax(out=to, a=ta)])
    got = store.read(to)
    assert np.array_equal(got, oracle.argmax(x))
    assert got[0] == 100 and got[1] == 0 and got[2] == 262143 and got[3] == 0
    small = rng.standard_normal((5, 7)).astype(np.float32)
    ts, t2 = put(store, small, F32), store.add(TensorMeta(I32, (5,)))
    s.execute([StepArgMax(out=t2, a=ts)])
    assert np.array_equal(store.read(t2), oracle.argmax(small))


# ---- fused steps against the unfused reference sequences --------------------------------
from aion_b200.backend import StepRMSNormPair, StepRopeKVAppend, Chunk  # noqa: E402


@pytest.mark.parametrize("with_res", [False, True])
def test_rms_norm_pair_equals_two_norms(sess, with_res):
    s, store = sess
    rng = np.random.default_rng(31)
    rows, cols = 9, 1536
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    res = rng.standard_normal((rows, cols)).astype(np.float32) if with_res else None
    g1, b1, g2, b2 = (rng.standard_normal(cols).astype(np.float32) for _ in range(4))
    t = {k: put(store, v, F32) for k, v in dict(x=x, g1=g1, b1=b1, g2=g2, b2=b2).items()}
    tr = put(store, res, F32) if with_res else None
    o1, o2 = store.add(TensorMeta(F32, (rows, cols))), store.add(TensorMeta(F32, (rows, cols)))
    s.execute([StepRMSNormPair(out1=o1, out2=o2, x=t["x"], gamma1=t["g1"], beta1=t["b1"], gamma2=t["g2"], beta2=t["b2"],
                               eps1=1e-6, eps2=1e-5, residual=tr)])
    want1 = oracle.rms_norm(x, g1, b1, 1e-6, residual=res)
    want2 = oracle.rms_norm(want1, g2, b2, 1e-5)
    np.testing.assert_allclose(store.read(o1), want1, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(store.read(o2), want2, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("cols", [1536, 4096, 4100])
def test_rms_norm_pair_in_place_on_the_residual(sess, cols):
    """The decoder's use: x = x + RMSNorm(o), x_norm = RMSNorm(x), with out1 and residual the same tensor."""
    s, store = sess
    rng = np.random.default_rng(cols)
    rows = 6
    o = rng.standard_normal((rows, cols)).astype(np.float32)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    g1, b1, g2, b2 = (rng.standard_normal(cols).astype(np.float32) for _ in range(4))
    t = {k: put(store, v, F32) for k, v in dict(o=o, x=x, g1=g1, b1=b1, g2=g2, b2=b2).items()}
    o2 = store.add(TensorMeta(F32, (rows, cols)))
    s.execute([StepRMSNormPair(out1=t["x"], out2=o2, x=t["o"], gamma1=t["g1"], beta1=t["b1"], gamma2=t["g2"], beta2=t["b2"],
                               eps1=1e-6, eps2=1e-6, residual=t["x"])])
    want1 = oracle.rms_norm(o, g1, b1, 1e-6, residual=x)
    want2 = oracle.rms_norm(want1, g2, b2, 1e-6)
    np.testing.assert_allclose(store.read(t["x"]), want1, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(store.read(o2), want2, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("rolling", [False, True])
def test_rope_kv_append_equals_the_six_steps(sess, rolling):
    s, store = sess
    rng = np.random.default_rng(32)
    B, L, Hq, Hkv, D, T = 3, 2, 4, 1, 64, 16
    width = (Hq + 2 * Hkv) * D
    ld = width + 32                                        # rows are slices of a wider buffer
    buf = rng.standard_normal((B * L, ld)).astype(np.float32)
    qkv = buf[:, :width]
    pos = rng.integers(0, 500, size=(B, L)).astype(np.int32)
    idx = np.array([0, 14, 33 if rolling else 7], dtype=np.int32)
    kc0 = rng.standard_normal((B, T, Hkv, D)).astype(np.float16)
    vc0 = rng.standard_normal((B, T, Hkv, D)).astype(np.float16)
    tb = put(store, buf, F32)
    ch = store.acquire_const(tb)
    tq = store.bind(TensorMeta(F32, (B, L, width), row_stride=ld), Chunk(ch.handle, ch.offset, ch.len))
    policy = "rolling" if rolling else "none"
    tk = store.add(TensorMeta(F16, kc0.shape, cache_policy=policy), kc0)
    tv = store.add(TensorMeta(F16, vc0.shape, cache_policy=policy), vc0)
    tp, ti = put(store, pos, I32), put(store, idx, I32)
    to = store.add(TensorMeta(F32, (B, L, Hq, D)))
    s.execute([StepRopeKVAppend(q_out=to, qkv=tq, positions=tp, end_index=ti, k_cache=tk, v_cache=tv, base_frequency=10000.0)])
    q = qkv[:, : Hq * D].reshape(B, L, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].reshape(B, L, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].reshape(B, L, Hkv, D)
    np.testing.assert_allclose(store.read(to), oracle.rope(q, pos, 10000.0), rtol=0, atol=1e-6)
    want_k = oracle.sequence_append(kc0, oracle.cast_f32_f16(oracle.rope(k, pos, 10000.0)), idx, rolling=rolling)
    want_v = oracle.sequence_append(vc0, oracle.cast_f32_f16(v), idx, rolling=rolling)
    got_k, got_v = store.read(tk), store.read(tv)
    assert np.array_equal(got_v.view(np.uint16), want_v.view(np.uint16))
    np.testing.assert_allclose(got_k.astype(np.float32), want_k.astype(np.float32), rtol=0, atol=2e-3)  # one f16 ulp where sincos differs


@pytest.mark.parametrize("R,F", [(5, 512), (3, 510), (520, 2048)])  # small; ragged rows; large enough for the float4 kernel
def test_gate_on_strided_halves(sess, R, F):
    s, store = sess
    rng = np.random.default_rng(33)
    gu = rng.standard_normal((R, 2 * F)).astype(np.float32)
    tg = put(store, gu, F32)
    ch = store.acquire_const(tg)
    half = TensorMeta(F32, (R, F), row_stride=2 * F)
    ta = store.bind(half, Chunk(ch.handle, ch.offset, ch.len))
    tb = store.bind(half, Chunk(ch.handle, ch.offset + F * 4, ch.len - F * 4))
    to = store.add(TensorMeta(F32, (R, F)))
    s.execute([StepElemwiseBinary(op="gate", out=to, a=ta, b=tb)])
    assert np.array_equal(store.read(to), oracle.elemwise(2, gu[:, :F], gu[:, F:]))


# ---- edge cases ----------------------------------------------------------------------------
def test_empty_steps_are_no_ops(sess, backend):
    s, store = sess
    z = store.add(TensorMeta(F32, (0, 64)))
    g = put(store, np.ones(64, np.float32), F32)
    b = put(store, np.zeros(64, np.float32), F32)
    zi = store.add(TensorMeta(I32, (0,)))
    zo = store.add(TensorMeta(I32, (0,)))
    zl = store.add(TensorMeta(F32, (0, 7)))
    s.execute([StepRMSNorm(out=z, x=z, gamma=g, beta=b, eps=1e-6), StepElemwiseBinary(op="add", out=z, a=z, b=z),
               StepArgMax(out=zo, a=zl)])
    backend.sync()
    assert store.read(z).shape == (0, 64) and zi is not None


def test_argmax_single_column_and_rope_without_rotation(sess):
    s, store = sess
    x = np.array([[3.0], [np.nan], [-np.inf]], np.float32)
    ta, to = put(store, x, F32), store.add(TensorMeta(I32, (3,)))
    s.execute([StepArgMax(out=to, a=ta)])
    assert store.read(to).tolist() == [0, 0, 0]
    q = np.random.default_rng(1).standard_normal((1, 2, 3, 32)).astype(np.float32)
    pos = np.array([[9, 1000]], np.int32)
    tq, tp = put(store, q, F32), put(store, pos, I32)
    tr = store.add(TensorMeta(F32, q.shape))
    s.execute([StepRoPE1D(out=tr, x=tq, positions=tp, base_frequency=10000.0, rope_proportion=0.0)])
    assert np.array_equal(store.read(tr), q)  # no pair rotates: a copy


def test_rms_norm_non_finite_row_is_reported(sess, backend):
    s, store = sess
    x = np.ones((2, 64), np.float32)
    x[1, 3] = np.inf
    tx = put(store, x, F32)
    g, b = put(store, np.ones(64, np.float32), F32), put(store, np.zeros(64, np.float32), F32)
    to = store.add(TensorMeta(F32, (2, 64)))
    s.execute([StepRMSNorm(out=to, x=tx, gamma=g, beta=b, eps=1e-6)])
    with pytest.raises(BackendError):   # the reference rejects a non-finite mean square (layernorm.zig:131-133)
        backend.sync()
