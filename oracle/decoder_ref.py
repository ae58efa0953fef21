"""The synthetic decoder's token step composed from oracle ops on the CPU.

TEST / BENCHMARK INFRASTRUCTURE ONLY (the checker, never the product): mirrors
aion_b200.decoder.SyntheticDecoder._build_steps op for op — the decode graph of the reference's
bench (src/bench/models.zig:364-540) reduced to its dense core — with state (KV caches) kept in
numpy arrays. Weights come as f32 values (quantized here with the oracle's quantizer) or, through
`from_packed`, as the packed q4_0 / q8_0 bytes a device decoder already holds."""
import numpy as np

import oracle


class OracleDecoder:
    def __init__(self, cfg, requests, weights_f32, embedding_f32, fast=False):
        self.cfg, self.R, self.fast = cfg, requests, fast
        dt = oracle.Q4_0 if cfg.weight_dtype == 3 else oracle.Q8_0
        self.dt = dt
        self.w = {name: oracle.quantize(dt, v, 0) for name, v in weights_f32.items()}
        self.embed = oracle.quantize(oracle.Q8_0, embedding_f32, 1)
        shape = (requests, cfg.ctx, cfg.kv_heads, cfg.head_dim)
        self.k_cache = [np.zeros(shape, np.float16) for _ in range(cfg.layers)]
        self.v_cache = [np.zeros(shape, np.float16) for _ in range(cfg.layers)]
        self.gamma, self.beta = np.ones(cfg.hidden, np.float32), np.zeros(cfg.hidden, np.float32)

    @classmethod
    def from_packed(cls, cfg, requests, packed, embed_q8, fast=True):
        """`packed`: name -> packed weight bytes. A layer may hold "l{i}.wqkv" / "l{i}.wgu" (columns of
        wq | wk | wv and wg | wu side by side) instead of the separate weights: block quantization along K
        makes the concatenated weight the same bytes side by side, and every output column is its own dot."""
        self = cls.__new__(cls)
        self.cfg, self.R, self.fast = cfg, requests, fast
        self.dt = oracle.Q4_0 if cfg.weight_dtype == 3 else oracle.Q8_0
        self.w = dict(packed)
        self.embed = embed_q8
        self.embed_rows = embed_q8.size // (cfg.hidden // 32 * 34)  # the table may hold only the rows that are looked up
        shape = (requests, cfg.ctx, cfg.kv_heads, cfg.head_dim)
        self.k_cache = [np.zeros(shape, np.float16) for _ in range(cfg.layers)]
        self.v_cache = [np.zeros(shape, np.float16) for _ in range(cfg.layers)]
        self.gamma, self.beta = np.ones(cfg.hidden, np.float32), np.zeros(cfg.hidden, np.float32)
        return self

    def _mm(self, a, name, k, n):
        m = a.size // k
        if self.fast:  # the threaded port of the same kernels (tests/test_oracle_fast.py holds it to the scalar oracle)
            return oracle.fast_matmul_q(self.dt, np.ascontiguousarray(a.reshape(m, k)), self.w[name], m, n, k,
                                        threads=getattr(self, "threads", 0)).reshape(m, n)
        return oracle.matmul_q(self.dt, a.reshape(m, k), self.w[name], m, n, k).reshape(m, n)

    def step(self, tokens, positions):
        cfg, R = self.cfg, self.R
        pos = np.asarray(positions, np.int32).reshape(R, 1)
        rms = lambda v, res=None: oracle.rms_norm(v, self.gamma, self.beta, cfg.eps, residual=res)
        x = oracle.gather_rows_q8(self.embed, getattr(self, "embed_rows", cfg.vocab), cfg.hidden, np.asarray(tokens, np.int32)).reshape(R, cfg.hidden)
        self.trace = []  # per layer: the intermediate tensors of the last step, for tests that localise a difference
        for l in range(cfg.layers):
            xn = rms(x)
            if f"l{l}.wqkv" in self.w:
                qkv = self._mm(xn, f"l{l}.wqkv", cfg.hidden, cfg.q_width + 2 * cfg.kv_width)
                q, k, v = np.split(qkv, [cfg.q_width, cfg.q_width + cfg.kv_width], axis=1)
            else:
                q = self._mm(xn, f"l{l}.wq", cfg.hidden, cfg.q_width)
                k = self._mm(xn, f"l{l}.wk", cfg.hidden, cfg.kv_width)
                v = self._mm(xn, f"l{l}.wv", cfg.hidden, cfg.kv_width)
            q = np.ascontiguousarray(q).reshape(R, 1, cfg.heads, cfg.head_dim)
            k = np.ascontiguousarray(k).reshape(R, 1, cfg.kv_heads, cfg.head_dim)
            v = np.ascontiguousarray(v).reshape(R, 1, cfg.kv_heads, cfg.head_dim)
            q = oracle.rope(q, pos, cfg.rope_base)
            k = oracle.rope(k, pos, cfg.rope_base)
            self.k_cache[l] = oracle.sequence_append(self.k_cache[l], oracle.cast_f32_f16(k), pos.reshape(R))
            self.v_cache[l] = oracle.sequence_append(self.v_cache[l], oracle.cast_f32_f16(v), pos.reshape(R))
            a = oracle.attention(q, self.k_cache[l], self.v_cache[l], scale=1.0 / np.sqrt(cfg.head_dim), positions=pos,
                                 kv_lengths=(pos.reshape(R) + 1).astype(np.int32), right=0)
            o = self._mm(a.reshape(R, cfg.q_width), f"l{l}.wo", cfg.q_width, cfg.hidden)
            x = rms(o, res=x)
            h = rms(x)
            if f"l{l}.wgu" in self.w:
                gu = self._mm(h, f"l{l}.wgu", cfg.hidden, 2 * cfg.ffn)
                gate, up = np.ascontiguousarray(gu[:, :cfg.ffn]), np.ascontiguousarray(gu[:, cfg.ffn:])
            else:
                gate = self._mm(h, f"l{l}.wg", cfg.hidden, cfg.ffn)
                up = self._mm(h, f"l{l}.wu", cfg.hidden, cfg.ffn)
            act = oracle.elemwise(oracle.ELEMWISE_GATE_GELU, gate, up)
            down = self._mm(act, f"l{l}.wd", cfg.ffn, cfg.hidden)
            x = rms(down, res=x)
            self.trace.append({"q": q, "k": k, "v": v, "attn": a, "o": o, "gate": gate, "up": up, "act": act, "down": down, "x": x})
        xf = rms(x)
        logits = self._mm(xf, "head", cfg.hidden, cfg.vocab)
        return x, logits, oracle.argmax(logits)
