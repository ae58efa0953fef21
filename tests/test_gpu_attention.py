"""`Attention` step parity through the C ABI against the oracle (the reference's generic
per-row executor, with its polynomial exp). Stated bound: rel-L2 <= 1e-3; the reference's
own bound against its exact-exp test reference is max-abs 8e-2 (f32) / 1.5e-1 (f16 K/V)."""
import os

import numpy as np
import pytest

import oracle
from aion_b200 import capi
from aion_b200.backend import (AttentionWindow, BackendError, CudaBackend, DeviceStore, StepAttention, TensorMeta)
from tests import refdata as rd
from tests.gpu_util import run_attention

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _qkv(B, L, Hq, Hkv, T, Dk, Dv, qdt, kvdt, seed=0):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((B, L, Hq, Dk)).astype(qdt)
    k = rng.standard_normal((B, T, Hkv, Dk)).astype(kvdt)
    v = rng.standard_normal((B, T, Hkv, Dv)).astype(kvdt)
    return q, k, v


# ---- the reference's own fixtures ----------------------------------------------------
def test_exact_window_averages(backend):
    # src/aion/api/test_api.zig:3256-3330
    q, k, v, pos, end, kw, expected = rd.api_attention_case()
    got = run_attention(backend, q, k, v, positions=pos, kv_lengths=end, **kw)
    np.testing.assert_allclose(got, expected, atol=1e-6)


def test_cached_gqa_fixture(backend):
    # src/aion/backend/cpu/test_cpu_backend.zig:4906-5172: sliding(2,0), soft cap 1.75
    q, k, v, pos, end, kw = rd.gqa_case_f32()
    want = rd.cached_gqa_ref(q, k, v, pos, end, **kw)
    got = run_attention(backend, q, k, v, positions=pos, kv_lengths=end, **kw)
    assert np.max(np.abs(got - want)) < 1e-4            # reference bound: 8e-2
    got16 = run_attention(backend, q, k.astype(np.float16), v.astype(np.float16), positions=pos, kv_lengths=end, **kw)
    assert np.max(np.abs(got16 - want)) < 1.5e-1
    assert rd.rel_l2(got, oracle.attention(q, k, v, positions=pos, kv_lengths=end, **kw)) < TOL


def test_plain_sequence_equals_cache_with_implied_indices(backend):
    # src/aion/backend/cpu/test_cpu_backend.zig:1531: no positions / lengths = (row, T)
    q, k, v = _qkv(2, 5, 4, 2, 5, 64, 64, np.float32, np.float16, seed=4)
    kw = dict(scale=0.125, right=0)
    implied = run_attention(backend, q, k, v, **kw)
    pos = np.tile(np.arange(5, dtype=np.int32), (2, 1))
    explicit = run_attention(backend, q, k, v, positions=pos, kv_lengths=np.full(2, 5, dtype=np.int32), **kw)
    assert np.array_equal(implied, explicit)
    assert rd.rel_l2(implied, oracle.attention(q, k, v, **kw)) < TOL


# ---- benchmark configuration 4 (seeded synthetic inputs of that shape) -------------------
@pytest.mark.parametrize("B,T", [(1, 1024), (8, 1024), (64, 1024), (1, 4096), (3, 4096), (2, 16384)])
def test_config4_decode(backend, B, T):
    q, k, v = _qkv(B, 1, 8, 1, T, 256, 256, np.float16, np.float16, seed=T + B)
    pos = np.full((B, 1), T - 1, dtype=np.int32)
    lens = np.full(B, T, dtype=np.int32)
    kw = dict(scale=1.0 / 16.0, positions=pos, kv_lengths=lens, right=0)
    got = run_attention(backend, q, k, v, **kw)
    assert rd.rel_l2(got, oracle.attention(q, k, v, **kw)) < TOL
    assert rd.rel_l2(got, oracle.attention(q, k, v, exact=True, **kw)) < TOL


@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("qdt", [np.float16, np.float32])
@pytest.mark.parametrize("Hq,Hkv", [(8, 1), (4, 2), (12, 1), (16, 2), (3, 3)])
def test_head_layouts_and_q_dtypes(backend, D, qdt, Hq, Hkv):
    B, L, T = 2, 2, 300
    q, k, v = _qkv(B, L, Hq, Hkv, T, D, D, qdt, np.float16, seed=D + Hq)
    pos = np.array([[150, 299], [7, 64]], dtype=np.int32)
    lens = np.array([300, 200], dtype=np.int32)
    kw = dict(scale=float(1 / np.sqrt(D)), positions=pos, kv_lengths=lens, right=0)
    got = run_attention(backend, q, k, v, **kw)
    assert rd.rel_l2(got, oracle.attention(q, k, v, **kw)) < TOL


# ---- several query rows per request: blocks of positions share one pass over K / V ----------
@pytest.mark.parametrize("Hq,Hkv,D", [(8, 4, 256), (8, 1, 256), (4, 4, 128), (6, 2, 64), (12, 1, 128), (2, 1, 64)])
@pytest.mark.parametrize("qdt", [np.float16, np.float32])
def test_prefill_blocks_causal(backend, Hq, Hkv, D, qdt):
    """A whole prompt per request: row l sees keys 0..l. Lengths that leave ragged blocks, with the
    per-row kernel of the same library as a second witness (same arithmetic, other tiling)."""
    B, L = 2, 150
    q, k, v = _qkv(B, L, Hq, Hkv, L, D, D, qdt, np.float16, seed=Hq * D)
    kw = dict(scale=float(1 / np.sqrt(D)), right=0)
    got = run_attention(backend, q, k, v, **kw)
    want = oracle.attention(q, k, v, **kw)
    assert rd.rel_l2(got, want) < TOL
    rows = run_attention(backend, q, k, v, flags=capi.ATTENTION_ROW_UNITS, **kw)
    assert rd.rel_l2(got, rows) < 5e-4   # f16 rounding of the weights against a different running maximum
    for l in (0, 1, 63, 64, 149):   # every row on its own, the short ones too
        assert rd.rel_l2(got[:, l], want[:, l]) < TOL


@pytest.mark.parametrize("window", [dict(left=40, right=0), dict(left=64, right=0, chunk=32), dict(left=5, right=2), dict(right=0)])
@pytest.mark.parametrize("soft_cap", [0.0, 4.0])
def test_prefill_blocks_on_a_cache_with_windows(backend, window, soft_cap):
    """A chunk of new rows appended to a cache that already holds a prefix: explicit positions, ragged
    lengths per request, sliding and chunked windows whose key ranges differ inside one block."""
    B, L, T, Hq, Hkv, D = 3, 70, 600, 8, 2, 128
    q, k, v = _qkv(B, L, Hq, Hkv, T, D, D, np.float32, np.float16, seed=31)
    q *= 2.0
    starts = np.array([0, 311, 530], dtype=np.int32)
    pos = (starts[:, None] + np.arange(L, dtype=np.int32)[None, :]).astype(np.int32)
    lens = (starts + L).astype(np.int32)
    kw = dict(scale=0.11, positions=pos, kv_lengths=lens, soft_cap=soft_cap, **window)
    got = run_attention(backend, q, k, v, **kw)
    assert rd.rel_l2(got, oracle.attention(q, k, v, **kw)) < TOL


def test_prefill_block_with_split_context(backend):
    """Few rows against a long cache: the block's context is split over CTAs and merged by the last one."""
    B, L, T, Hq, Hkv, D = 1, 9, 6000, 8, 4, 256
    q, k, v = _qkv(B, L, Hq, Hkv, T, D, D, np.float32, np.float16, seed=77)
    pos = (T - L + np.arange(L, dtype=np.int32)).reshape(1, L)
    kw = dict(scale=1 / 16.0, positions=pos, kv_lengths=np.array([T], dtype=np.int32), right=0)
    want = oracle.attention(q, k, v, **kw)
    for _ in range(2):
        assert rd.rel_l2(run_attention(backend, q, k, v, **kw), want) < TOL


def test_prefill_rows_with_no_keys_write_zeros(backend):
    B, L, T, D = 1, 20, 64, 64
    q, k, v = _qkv(B, L, 4, 2, T, D, D, np.float16, np.float16, seed=3)
    pos = np.arange(L, dtype=np.int32).reshape(1, L)
    kw = dict(scale=0.2, positions=pos, kv_lengths=np.array([7], dtype=np.int32), left=2, right=0)  # rows >= 10 see nothing
    got = run_attention(backend, q, k, v, **kw)
    assert rd.rel_l2(got, oracle.attention(q, k, v, **kw)) < TOL
    assert not got[0, 10:].any() and got[0, :9].any()


# ---- paged K / V -----------------------------------------------------------------------
def _paged(k, v, page_tokens, seed):
    """Scatter contiguous [B, T, H, D] caches over a shuffled pool of pages; returns pools and the table."""
    B, T, H, D = k.shape
    per = (T + page_tokens - 1) // page_tokens
    rng = np.random.default_rng(seed)
    pool = B * per + 3
    ids = rng.permutation(pool)[: B * per].reshape(B, per).astype(np.int32)
    kp = rng.standard_normal((pool, page_tokens, H, D)).astype(k.dtype)   # unused pages hold other data
    vp = rng.standard_normal((pool, page_tokens, H, D)).astype(v.dtype)
    for b in range(B):
        for i in range(per):
            n = min(page_tokens, T - i * page_tokens)
            kp[ids[b, i], :n] = k[b, i * page_tokens: i * page_tokens + n]
            vp[ids[b, i], :n] = v[b, i * page_tokens: i * page_tokens + n]
    return kp, vp, ids


@pytest.mark.parametrize("page_tokens", [64, 256])
@pytest.mark.parametrize("B,L,T,window", [(5, 1, 1000, dict(right=0)), (2, 1, 4500, dict(left=700, right=0)),
                                           (2, 40, 500, dict(right=0)), (64, 1, 300, dict(right=0))])
def test_paged_cache_equals_contiguous(backend, page_tokens, B, L, T, window):
    Hq, Hkv, D = 8, 2, 128
    q, k, v = _qkv(B, L, Hq, Hkv, T, D, D, np.float16, np.float16, seed=T + page_tokens)
    lens = np.random.default_rng(T).integers(L, T + 1, B).astype(np.int32)
    pos = (lens[:, None] - L + np.arange(L, dtype=np.int32)[None, :]).astype(np.int32)
    kw = dict(scale=0.09, positions=pos, kv_lengths=lens, **window)
    kp, vp, table = _paged(k, v, page_tokens, seed=B)
    got = run_attention(backend, q, kp, vp, page_table=table, **kw)
    assert rd.rel_l2(got, oracle.attention(q, k, v, **kw)) < TOL
    assert rd.rel_l2(got, run_attention(backend, q, k, v, **kw)) < 5e-4   # slices start on stage multiples with a table


def test_paged_cache_argument_errors(backend):
    q, k, v = _qkv(1, 1, 8, 1, 128, 64, 64, np.float16, np.float16)
    kp, vp, table = _paged(k, v, 64, seed=0)
    with pytest.raises(BackendError) as e:   # pages that a stage would straddle
        run_attention(backend, q, kp.reshape(-1, 32, 1, 64), vp.reshape(-1, 32, 1, 64), page_table=np.zeros((1, 4), np.int32), scale=1.0)
    assert e.value.name == "InvalidArgument"
    with pytest.raises(BackendError) as e:
        run_attention(backend, q, kp, vp, page_table=table, scale=1.0, rolling=True)
    assert e.value.name == "Unsupported"
    with pytest.raises(BackendError) as e:   # the f32 any-shape kernel does not read tables
        run_attention(backend, q, kp.astype(np.float32), vp.astype(np.float32), page_table=table, scale=1.0)
    assert e.value.name == "Unsupported"


@pytest.mark.parametrize("length", [0, 1, 15, 16, 17, 63, 64, 65, 129, 1000])
def test_ragged_lengths(backend, length):
    B, T, D = 3, 1000, 128
    q, k, v = _qkv(B, 1, 8, 1, T, D, D, np.float16, np.float16, seed=length)
    lens = np.array([length, T, max(length - 1, 0)], dtype=np.int32)
    pos = np.maximum(lens - 1, 0).reshape(B, 1).astype(np.int32)
    kw = dict(scale=0.1, positions=pos, kv_lengths=lens, right=0)
    got = run_attention(backend, q, k, v, **kw)
    want = oracle.attention(q, k, v, **kw)
    assert rd.rel_l2(got, want) < TOL
    if length == 0:
        assert not got[0].any()  # an empty key range writes zeros


@pytest.mark.parametrize("window", [dict(left=100, right=0), dict(left=17, right=3), dict(left=50, right=0, chunk=64),
                                    dict(), dict(left=0, right=0)])
@pytest.mark.parametrize("soft_cap", [0.0, 5.0])
def test_windows_and_soft_cap(backend, window, soft_cap):
    B, L, T, D = 1, 4, 700, 64
    q, k, v = _qkv(B, L, 8, 2, T, D, D, np.float32, np.float16, seed=11)
    q *= 3.0  # push logits into the cap's curved range
    pos = np.array([[0, 130, 420, 699]], dtype=np.int32)
    kw = dict(scale=0.2, positions=pos, kv_lengths=np.array([700], dtype=np.int32), soft_cap=soft_cap, **window)
    got = run_attention(backend, q, k, v, **kw)
    assert rd.rel_l2(got, oracle.attention(q, k, v, **kw)) < TOL


def test_rolling_cache(backend):
    # A ring of T rows addressed t % T; only the last T logical keys are visible
    # (src/aion/backend/cpu/exec/attention.zig:1072-1075, 1150-1153).
    B, T, D = 2, 256, 128
    q, k, v = _qkv(B, 1, 8, 1, T, D, D, np.float16, np.float16, seed=5)
    lens = np.array([1000, 200], dtype=np.int32)  # one wrapped, one not yet
    pos = (lens - 1).reshape(B, 1)
    kw = dict(scale=0.09, positions=pos, kv_lengths=lens, left=511, right=0, rolling=True)
    got = run_attention(backend, q, k, v, **kw)
    assert rd.rel_l2(got, oracle.attention(q, k, v, **kw)) < TOL


@pytest.mark.parametrize("kvdt", [np.float32])
def test_f32_kv_and_odd_head_sizes_take_the_any_shape_kernel(backend, kvdt):
    for Dk, Dv in ((256, 256), (40, 24), (3, 2)):
        q, k, v = _qkv(2, 2, 4, 2, 90, Dk, Dv, np.float16, kvdt, seed=Dk)
        kw = dict(scale=0.3, right=0, positions=np.array([[10, 89], [0, 45]], dtype=np.int32),
                  kv_lengths=np.array([90, 46], dtype=np.int32))
        got = run_attention(backend, q, k, v, **kw)
        assert rd.rel_l2(got, oracle.attention(q, k, v, **kw)) < TOL


@pytest.mark.parametrize("split", [1, 2, 7, 64, 256])
def test_context_split_is_value_stable(split):
    os.environ["AION_CUDA_ATTN_SPLIT"] = str(split)
    try:
        b2 = CudaBackend(0)
    finally:
        del os.environ["AION_CUDA_ATTN_SPLIT"]
    try:
        q, k, v = _qkv(2, 1, 8, 1, 3000, 256, 256, np.float16, np.float16, seed=split)
        lens = np.array([3000, 1234], dtype=np.int32)
        kw = dict(scale=1 / 16.0, positions=(lens - 1).reshape(2, 1), kv_lengths=lens, right=0)
        want = oracle.attention(q, k, v, **kw)
        for _ in range(2):  # the arrival counters must be back at zero for the second launch
            assert rd.rel_l2(run_attention(b2, q, k, v, **kw), want) < TOL
    finally:
        b2.deinit()


def test_bad_lengths_are_reported_and_the_device_stays_usable(backend):
    q, k, v = _qkv(1, 1, 8, 1, 64, 64, 64, np.float16, np.float16)
    with pytest.raises(BackendError) as e:
        run_attention(backend, q, k, v, scale=1.0, kv_lengths=np.array([-1], dtype=np.int32))
    assert e.value.name == "InvalidArgument"
    with pytest.raises(BackendError) as e:
        run_attention(backend, q, k, v, scale=1.0, kv_lengths=np.array([65], dtype=np.int32))  # beyond a plain cache
    assert e.value.name == "InvalidArgument"
    with pytest.raises(BackendError):
        run_attention(backend, q, k, v, scale=0.0)
    with pytest.raises(BackendError):
        run_attention(backend, q, k, v, scale=1.0, soft_cap=-1.0)
    got = run_attention(backend, q, k, v, scale=1.0)
    assert rd.rel_l2(got, oracle.attention(q, k, v, scale=1.0)) < TOL


def test_session_attention_step(backend):
    B, T, D = 2, 128, 64
    q, k, v = _qkv(B, 1, 8, 1, T, D, D, np.float16, np.float16, seed=9)
    store = DeviceStore(backend.device_memory)
    try:
        ids = dict(
            q=store.add(TensorMeta(capi.DTYPE_F16, q.shape), q),
            k=store.add(TensorMeta(capi.DTYPE_F16, k.shape, cache_policy="growable"), k),
            v=store.add(TensorMeta(capi.DTYPE_F16, v.shape, cache_policy="growable"), v),
            out=store.add(TensorMeta(capi.DTYPE_F32, (B, 1, 8, D))),
            pos=store.add(TensorMeta(capi.DTYPE_I32, (B, 1)), np.array([[99], [127]], dtype=np.int32)),
            lens=store.add(TensorMeta(capi.DTYPE_I32, (B,)), np.array([100, 128], dtype=np.int32)),
        )
        sess = backend.create_session(store)
        sess.execute([StepAttention(ids["out"], ids["q"], ids["k"], ids["v"], ids["pos"], ids["lens"], scale=0.125,
                                    window=AttentionWindow.causal())])
        got = store.read(ids["out"])
        want = oracle.attention(q, k, v, scale=0.125, positions=np.array([[99], [127]]), kv_lengths=np.array([100, 128]),
                                right=0)
        assert rd.rel_l2(got, want) < TOL
    finally:
        store.deinit()


@pytest.mark.parametrize("dtype", [capi.DTYPE_Q4_0, capi.DTYPE_Q8_0])
@pytest.mark.parametrize("B,T,qdt", [(1, 48, np.float32), (8, 2048, np.float32), (70, 300, np.float16)])
def test_attention_writes_the_image_of_its_output(backend, dtype, B, T, qdt):
    """The decode kernel (one pass per row, and split contexts merged by the last CTA) also writes the
    quantized image of out [B, Hq*Dv] that the output projection reads."""
    from aion_b200.backend import act_image_meta
    from tests.gpu_util import DevBuf, make_image

    Hq, D = 8, 256
    q, k, v = _qkv(B, 1, Hq, 1, T, D, D, qdt, np.float16, seed=B)
    lens = np.random.default_rng(1).integers(1, T + 1, B).astype(np.int32)
    pos = (lens - 1).reshape(B, 1).astype(np.int32)
    store = DeviceStore(backend.device_memory)
    try:
        f = {np.float32: capi.DTYPE_F32, np.float16: capi.DTYPE_F16}
        tq = store.add(TensorMeta(f[qdt], q.shape), q)
        tk = store.add(TensorMeta(capi.DTYPE_F16, k.shape), k)
        tv = store.add(TensorMeta(capi.DTYPE_F16, v.shape), v)
        tp = store.add(TensorMeta(capi.DTYPE_I32, pos.shape), pos)
        tl = store.add(TensorMeta(capi.DTYPE_I32, lens.shape), lens)
        to = store.add(TensorMeta(capi.DTYPE_F32, (B, 1, Hq, D)))
        ti = store.add(act_image_meta(B, Hq * D, dtype))
        sess = backend.create_session(store)
        sess.execute([StepAttention(out=to, q=tq, k=tk, v=tv, query_positions=tp, kv_lengths=tl, scale=1.0 / 16.0,
                                    window=AttentionWindow.causal(), image=ti)])
        got = store.read(to)
        assert rd.rel_l2(got, oracle.attention(q, k, v, scale=1.0 / 16.0, positions=pos, kv_lengths=lens, right=0)) < TOL
        a = DevBuf(backend, got.reshape(B, Hq * D))
        img = make_image(backend, dtype, a, B, Hq * D)
        try:
            assert np.array_equal(store.read(ti).view(np.uint8), img.read(np.uint8))
        finally:
            a.free()
            img.free()
    finally:
        store.deinit()


@pytest.mark.parametrize("L", [1, 40], ids=["decode_rows", "query_blocks"])
def test_an_expired_wait_in_attention_is_reported_and_the_device_stays_usable(L):
    """With the test hook on, every CTA leaves out the K / V copies of its first stage and polls briefly: the
    consumers' wait runs out, the kernel records the fault and returns, the next synchronization reports it,
    and the same device object then computes correctly again."""
    b2 = CudaBackend(0)
    try:
        q, k, v = _qkv(2, L, 8, 2, 300, 128, 128, np.float16, np.float16, seed=L)
        pos = (300 - L + np.arange(L, dtype=np.int32))[None, :].repeat(2, 0).astype(np.int32)
        kw = dict(scale=0.09, positions=pos, kv_lengths=np.full(2, 300, np.int32), right=0)
        want = oracle.attention(q, k, v, **kw)
        assert rd.rel_l2(run_attention(b2, q, k, v, **kw), want) < TOL
        assert b2._lib.aion_cuda_debug_expire_waits(b2.handle, 1) == capi.OK
        with pytest.raises(BackendError) as e:
            run_attention(b2, q, k, v, **kw)
        assert e.value.name == "ExecutionFailed" and "bounded wait" in str(e.value)
        assert b2._lib.aion_cuda_debug_expire_waits(b2.handle, 0) == capi.OK
        assert rd.rel_l2(run_attention(b2, q, k, v, **kw), want) < TOL
    finally:
        b2.deinit()
