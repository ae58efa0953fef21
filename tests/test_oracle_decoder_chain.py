"""How far two runs of the reference arithmetic drift apart along a decoder layer (CPU only).

Every matmul of the reference quantizes its activation to int8 per 32-block. A relative difference d
between two activations flips roughly d * |code| of those roundings, and a flipped rounding is a whole
code step, so about sqrt(d / |code|) is left behind: small differences grow by a square root at every
matmul until they reach the quantization noise itself. This test measures it on the oracle alone: the same
layer with the softmax's polynomial exp against the exact exp (a 3e-5 difference in attention's output)
ends a few 1e-3 apart. That is why the device-vs-oracle comparison of a chained decoder step is held to
2e-2 while every single op is held to 1e-5 .. 1e-3 on identical inputs.
"""
import numpy as np

import oracle
from aion_b200.decoder import DecoderConfig
from oracle.decoder_ref import OracleDecoder


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b.astype(np.float64)), 1e-30))


def test_the_oracle_chain_amplifies_small_differences_itself(monkeypatch):
    cfg = DecoderConfig(layers=1, hidden=1536, ffn=8192, heads=8, kv_heads=1, head_dim=256, vocab=2048, ctx=128)
    R = 4
    rng = np.random.default_rng(21)
    w = {f"l0.{name}": (rng.standard_normal(shape) * 0.02).astype(np.float32) for name, shape in cfg.layer_weights().items()}
    w["head"] = (rng.standard_normal((cfg.hidden, cfg.vocab)) * 0.02).astype(np.float32)
    emb = rng.standard_normal((cfg.vocab, cfg.hidden)).astype(np.float32)
    caches = rng.standard_normal((2, R, cfg.ctx, 1, cfg.head_dim)).astype(np.float16)
    tokens, pos = np.array([3, 500, 77, 1999], np.int32), np.full(R, 100, np.int32)

    def run(exact):
        ref = OracleDecoder(cfg, R, w, emb, fast=True)
        ref.k_cache[0][:], ref.v_cache[0][:] = caches[0], caches[1]
        real = oracle.attention
        monkeypatch.setattr(oracle, "attention", lambda *a, **kw: real(*a, exact=exact, **kw))
        try:
            x, logits, _ = ref.step(tokens, pos)
        finally:
            monkeypatch.setattr(oracle, "attention", real)
        return ref.trace[0]["attn"], ref.trace[0]["o"], ref.trace[0]["down"], x, logits

    a0, o0, d0, x0, l0 = run(False)
    a1, o1, d1, x1, l1 = run(True)
    d_attn, d_o, d_down, d_logits = rel_l2(a0, a1), rel_l2(o0, o1), rel_l2(d0, d1), rel_l2(l0, l1)
    print(f"\noracle vs itself (polynomial exp vs exact exp): attention {d_attn:.2e}, o {d_o:.2e}, down {d_down:.2e}, logits {d_logits:.2e}")
    assert d_attn < 2e-4                 # the two softmaxes differ by the polynomial's error
    assert d_o > 3 * d_attn              # one re-quantization later the difference has grown
    assert d_down > d_o                  # and again along gate / up and the down projection
    assert 1e-3 < d_logits < 2e-2        # the level a chained comparison can be held to
