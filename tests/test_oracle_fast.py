"""The threaded CPU baseline computes what the exact oracle computes."""
import numpy as np
import pytest

import oracle
from tests import refdata as rd


@pytest.mark.parametrize("dtype", [oracle.Q8_0, oracle.Q4_0])
@pytest.mark.parametrize("m", [1, 5, 20])
def test_fast_matmul_matches_oracle(dtype, m):
    n, k = 200, 544
    a = rd.synth_acts(m, k)
    b = oracle.quantize(dtype, rd.synth_weights(k, n), 0)
    want = oracle.matmul_q(dtype, a, b, m, n, k)
    for threads in (1, 4):
        got = oracle.fast_matmul_q(dtype, a, b, m, n, k, threads=threads)
        assert rd.rel_l2(got, want) < 2e-6


def test_fast_matmul_nt_matches_oracle():
    m, n, k = 3, 77, 256
    a = rd.synth_acts(m, k)
    b = oracle.quantize(oracle.Q8_0, rd.synth_weights(n, k), 1)
    got = oracle.fast_matmul_nt_q8(a, b, m, n, k, threads=3)
    assert rd.rel_l2(got, oracle.matmul_nt_q8(a, b, m, n, k)) < 2e-6


def test_fast_alpha_beta():
    m, n, k = 2, 64, 512
    a = rd.synth_acts(m, k)
    b = oracle.quantize(oracle.Q4_0, rd.synth_weights(k, n), 0)
    c0 = rd.synth_acts(m, n, seed=3)
    want = oracle.matmul_q(oracle.Q4_0, a, b, m, n, k, alpha=0.5, beta=2.0, c=c0)
    got = oracle.fast_matmul_q(oracle.Q4_0, a, b, m, n, k, alpha=0.5, beta=2.0, c=c0.reshape(-1).copy())
    assert rd.rel_l2(got, want) < 2e-6


def test_fast_attention_equals_the_scalar_oracle():
    rng = np.random.default_rng(0)
    B, T, Hq, D = 5, 96, 8, 64
    q = rng.standard_normal((B, 1, Hq, D)).astype(np.float16)
    k = rng.standard_normal((B, T, 1, D)).astype(np.float16)
    v = rng.standard_normal((B, T, 1, D)).astype(np.float16)
    lens = np.array([96, 1, 40, 77, 13], np.int32)
    pos = (lens - 1).reshape(B, 1)
    kw = dict(scale=0.125, positions=pos, kv_lengths=lens, right=0)
    assert np.array_equal(oracle.fast_attention(q, k, v, threads=3, **kw), oracle.attention(q, k, v, **kw))
