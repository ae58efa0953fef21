"""The synthetic q4 decoder of the decode benchmark, as a step program for `CudaSession`.

The graph shape follows the reference's decode bench (src/bench/models.zig:364-540) reduced
to the benchmark's dense core: per layer

    x_norm = RMSNorm(x)
    q, k, v = MatMul(x_norm, Wq | Wk | Wv)              q4_0 [K/32][N] weights
    q, k    = RoPE1D(q | k, positions)
    K, V    = SequenceAppend(cache, Cast(k | v -> f16), write_index)
    a       = Attention(q, K, V, positions, visible_end, scale, causal)
    x       = x + RMSNorm(MatMul(a, Wo))                 (RMSNorm with residual)
    h       = RMSNorm(x)
    x       = x + RMSNorm(MatMul(gelu(MatMul(h, Wg)) * MatMul(h, Wu), Wd))

then `ArgMax(MatMul(RMSNorm(x), Whead))`, with x gathered from a q8_0 embedding table.

`fused=True` (the default) issues the same arithmetic as fewer, fuller steps, the way a
fusion pass would rewrite the graph: one matmul against [Wq | Wk | Wv] and one against
[Wg | Wu] (column concatenation commutes with K-major block quantization, so the packed
weights are the same bytes side by side), `StepRopeKVAppend` for RoPE + cast + append, and
`StepRMSNormPair` for "x = x + RMSNorm(.)" followed by the next block's RMSNorm: 9 launches
per layer instead of 19. With `images=True` (the default) every step that produces a matmul's
activation (the norms, the GELU gate, attention) also writes its quantized image, so no matmul
launches a quantization kernel of its own; the codes are the ones the matmul would compute.
Every request is independent of the others in its batch (all ops are row-wise), which is
what lets a batch be split over GPUs with replicated weights and no exchange.

Only step records and device tensors are built here; all arithmetic runs in the library.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import Callable, Optional

import numpy as np

from . import capi
from .backend import (AttentionWindow, Chunk, CudaBackend, CudaSession, DeviceStore, StepArgMax, StepAttention, StepCast,
                      StepElemwiseBinary, StepGatherRows, StepMatMul, StepRMSNorm, StepRMSNormPair, StepRoPE1D,
                      StepRopeKVAppend, StepSequenceAppend, TensorMeta, _check, act_image_meta)

F32, F16, I32, Q4, Q8 = capi.DTYPE_F32, capi.DTYPE_F16, capi.DTYPE_I32, capi.DTYPE_Q4_0, capi.DTYPE_Q8_0


@dataclasses.dataclass
class DecoderConfig:
    layers: int = 30
    hidden: int = 1536
    ffn: int = 8192
    heads: int = 8
    kv_heads: int = 1
    head_dim: int = 256
    vocab: int = 262144
    ctx: int = 2048
    eps: float = 1e-6
    rope_base: float = 10000.0
    weight_dtype: int = Q4

    @property
    def q_width(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.kv_heads * self.head_dim

    def layer_weights(self) -> dict:
        """name -> (k, n) of one layer's matmul weights."""
        return {"wq": (self.hidden, self.q_width), "wk": (self.hidden, self.kv_width), "wv": (self.hidden, self.kv_width),
                "wo": (self.q_width, self.hidden), "wg": (self.hidden, self.ffn), "wu": (self.hidden, self.ffn),
                "wd": (self.ffn, self.hidden)}

    def weights_per_step(self) -> int:
        """Weights one token step reads (matmuls only)."""
        per_layer = sum(k * n for k, n in self.layer_weights().values())
        return self.layers * per_layer + self.hidden * self.vocab

    def weight_bytes_per_step(self) -> int:
        bb = 18 if self.weight_dtype == Q4 else 34
        return self.weights_per_step() // 32 * bb

    def kv_bytes_per_request_step(self) -> int:
        return self.layers * 2 * self.ctx * self.kv_width * 2


def quantize_on_device(backend: CudaBackend, dtype: int, src: capi.Operand, shape: tuple, quant_axis: int, dst: capi.Operand) -> None:
    """`aion_cuda_quantize` between two device operands (values f32 -> packed blocks)."""
    sh = (C.c_uint64 * len(shape))(*shape)
    _check(backend._lib.aion_cuda_quantize(backend._h, dtype, C.byref(src), sh, len(shape), quant_axis, C.byref(dst)))


class SyntheticDecoder:
    """Device tensors + step list of one decode step for `requests` concurrent requests.

    `weight_values(name, k, n)` returns the f32 [k, n] values of a matmul weight as a host
    array, or a `Chunk` of f32 already on the device; they are quantized on the device.
    `embedding_values(v0, v1)` likewise returns rows [v0, v1) of the f32 [vocab, hidden] table.
    """

    def __init__(self, backend: CudaBackend, cfg: DecoderConfig, requests: int,
                 weight_values: Callable[[str, int, int], object], embedding_values: Callable[[int, int], object],
                 store: Optional[DeviceStore] = None, fused: bool = True, images: bool = True):
        self.backend, self.cfg, self.requests, self.fused = backend, cfg, requests, fused
        # Images ride on the fused steps and on rows the register-resident norm kernel takes.
        self.images = bool(images and fused and cfg.hidden % 32 == 0 and cfg.hidden <= 4096 and cfg.ffn % 32 == 0
                           and cfg.head_dim in (64, 128, 256))
        self.store = store or DeviceStore(backend.device_memory)
        self.session: CudaSession = backend.create_session(self.store)
        self._build_weights(weight_values, embedding_values)
        self._build_state()
        self.steps = self._build_steps_fused() if fused else self._build_steps()
        self.program = None

    # ---- weights -----------------------------------------------------------------------
    def _quantized(self, values, shape: tuple, dtype: int, axis: int) -> int:
        st, mem = self.store, self.backend.device_memory
        tid = st.add(TensorMeta(dtype, shape, quant_axis=axis))
        dst = st.acquire_mut(tid).operand()
        n = int(np.prod(shape))
        if isinstance(values, Chunk):
            quantize_on_device(self.backend, dtype, values.operand(), shape, axis, dst)
            self.backend.sync()
        else:
            v = np.ascontiguousarray(values, dtype=np.float32)
            h = mem.alloc(n * 4, 256)
            try:
                mem.copy_h2d(h, 0, v)
                quantize_on_device(self.backend, dtype, capi.Operand(h, 0, n * 4), shape, axis, dst)
                self.backend.sync()
            finally:
                mem.free(h)
        return tid

    def _build_weights(self, weight_values, embedding_values) -> None:
        cfg, st = self.cfg, self.store
        self.w = []
        shapes = cfg.layer_weights()
        for layer in range(cfg.layers):
            names = {}
            if self.fused:
                # [Wq | Wk | Wv] and [Wg | Wu] as single weights; host arrays are concatenated so the
                # values stay those of the separate weights, device-side sources are asked directly.
                for fused_name, parts in (("wqkv", ("wq", "wk", "wv")), ("wgu", ("wg", "wu"))):
                    k = shapes[parts[0]][0]
                    n = sum(shapes[p][1] for p in parts)
                    first = weight_values(f"l{layer}.{parts[0]}", k, shapes[parts[0]][1])
                    if isinstance(first, Chunk):
                        vals = weight_values(f"l{layer}.{fused_name}", k, n)
                    else:
                        vals = np.concatenate([np.asarray(first, dtype=np.float32)] +
                                              [np.asarray(weight_values(f"l{layer}.{p}", k, shapes[p][1]), dtype=np.float32)
                                               for p in parts[1:]], axis=1)
                    names[fused_name] = self._quantized(vals, (k, n), cfg.weight_dtype, 0)
                for name in ("wo", "wd"):
                    k, n = shapes[name]
                    names[name] = self._quantized(weight_values(f"l{layer}.{name}", k, n), (k, n), cfg.weight_dtype, 0)
            else:
                for name, (k, n) in shapes.items():
                    names[name] = self._quantized(weight_values(f"l{layer}.{name}", k, n), (k, n), cfg.weight_dtype, 0)
            self.w.append(names)
        self.w_head = self._quantized(weight_values("head", cfg.hidden, cfg.vocab), (cfg.hidden, cfg.vocab), cfg.weight_dtype, 0)
        # q8_0 [vocab, hidden] embedding table, quantized along hidden, filled in row slabs.
        self.embed = st.add(TensorMeta(Q8, (cfg.vocab, cfg.hidden), quant_axis=1))
        ech = st.acquire_mut(self.embed)
        row_bytes = cfg.hidden // 32 * 34
        slab = max(1, min(cfg.vocab, (64 << 20) // (cfg.hidden * 4)))
        mem = self.backend.device_memory
        for v0 in range(0, cfg.vocab, slab):
            v1 = min(cfg.vocab, v0 + slab)
            vals = embedding_values(v0, v1)
            dst = capi.Operand(ech.handle, ech.offset + v0 * row_bytes, (v1 - v0) * row_bytes)
            if isinstance(vals, Chunk):
                quantize_on_device(self.backend, Q8, vals.operand(), (v1 - v0, cfg.hidden), 1, dst)
                self.backend.sync()
            else:
                v = np.ascontiguousarray(vals, dtype=np.float32)
                h = mem.alloc(v.nbytes, 256)
                try:
                    mem.copy_h2d(h, 0, v)
                    quantize_on_device(self.backend, Q8, capi.Operand(h, 0, v.nbytes), (v1 - v0, cfg.hidden), 1, dst)
                    self.backend.sync()
                finally:
                    mem.free(h)
        ones, zeros = np.ones(cfg.hidden, np.float32), np.zeros(cfg.hidden, np.float32)
        self.gamma = st.add(TensorMeta(F32, (cfg.hidden,)), ones)   # RMSNorm gamma = 1 everywhere
        self.beta = st.add(TensorMeta(F32, (cfg.hidden,)), zeros)

    # ---- per-request state and activations ----------------------------------------------
    def _view(self, tid: int, shape: tuple, dtype: Optional[int] = None) -> int:
        m, ch = self.store.meta(tid), self.store.acquire_const(tid)
        return self.store.bind(TensorMeta(m.dtype if dtype is None else dtype, shape), ch)

    def _build_state(self) -> None:
        cfg, st, R = self.cfg, self.store, self.requests
        self.tokens = st.add(TensorMeta(I32, (R, 1)), np.zeros((R, 1), np.int32))
        self.positions = st.add(TensorMeta(I32, (R, 1)), np.zeros((R, 1), np.int32))
        self.write_index = st.add(TensorMeta(I32, (R,)), np.zeros(R, np.int32))
        self.visible_end = st.add(TensorMeta(I32, (R,)), np.zeros(R, np.int32))
        self.k_cache, self.v_cache = [], []
        for _ in range(cfg.layers):
            for lst in (self.k_cache, self.v_cache):
                tid = st.add(TensorMeta(F16, (R, cfg.ctx, cfg.kv_heads, cfg.head_dim)))
                ch = st.acquire_mut(tid)
                self.backend.device_memory.memset(ch.handle, ch.offset, 0, ch.len)
                lst.append(tid)
        f = lambda *shape: st.add(TensorMeta(F32, shape))
        self.x = f(R, 1, cfg.hidden)
        self.x_norm = f(R, 1, cfg.hidden)
        self.q = f(R, 1, cfg.q_width)
        self.k = f(R, 1, cfg.kv_width)
        self.v = f(R, 1, cfg.kv_width)
        self.q4 = self._view(self.q, (R, 1, cfg.heads, cfg.head_dim))
        self.k4 = self._view(self.k, (R, 1, cfg.kv_heads, cfg.head_dim))
        self.v4 = self._view(self.v, (R, 1, cfg.kv_heads, cfg.head_dim))
        self.k16 = st.add(TensorMeta(F16, (R, 1, cfg.kv_heads, cfg.head_dim)))
        self.v16 = st.add(TensorMeta(F16, (R, 1, cfg.kv_heads, cfg.head_dim)))
        self.attn = f(R, 1, cfg.heads, cfg.head_dim)
        self.attn2 = self._view(self.attn, (R, 1, cfg.q_width))
        self.o = f(R, 1, cfg.hidden)
        self.gate = f(R, 1, cfg.ffn)
        self.up = f(R, 1, cfg.ffn)
        self.act = f(R, 1, cfg.ffn)
        self.down = f(R, 1, cfg.hidden)
        if self.fused:
            width = cfg.q_width + 2 * cfg.kv_width
            self.qkv = f(R, 1, width)
            self.q_rot = f(R, 1, cfg.heads, cfg.head_dim)
            self.gu = f(R, 1, 2 * cfg.ffn)
            ch = st.acquire_const(self.gu)
            half = TensorMeta(F32, (R, 1, cfg.ffn), row_stride=2 * cfg.ffn)
            self.gate_view = st.bind(half, Chunk(ch.handle, ch.offset, ch.len))
            self.up_view = st.bind(half, Chunk(ch.handle, ch.offset + cfg.ffn * 4, ch.len - cfg.ffn * 4))
        self.logits = f(R, 1, cfg.vocab)
        self.next_token = st.add(TensorMeta(I32, (R, 1)))
        self.img_xn = self.img_attn = self.img_act = None
        if self.images:
            self.img_xn = st.add(act_image_meta(R, cfg.hidden, cfg.weight_dtype))
            self.img_attn = st.add(act_image_meta(R, cfg.q_width, cfg.weight_dtype))
            self.img_act = st.add(act_image_meta(R, cfg.ffn, cfg.weight_dtype))

    def _build_steps(self) -> list:
        cfg = self.cfg
        g, b = self.gamma, self.beta
        scale = 1.0 / float(np.sqrt(cfg.head_dim))
        steps: list = [StepGatherRows(out=self.x, table=self.embed, indices=self.tokens)]
        for layer in range(cfg.layers):
            w = self.w[layer]
            steps += [
                StepRMSNorm(out=self.x_norm, x=self.x, gamma=g, beta=b, eps=cfg.eps),
                StepMatMul(c=self.q, a=self.x_norm, b=w["wq"]),
                StepMatMul(c=self.k, a=self.x_norm, b=w["wk"]),
                StepMatMul(c=self.v, a=self.x_norm, b=w["wv"]),
                StepRoPE1D(out=self.q4, x=self.q4, positions=self.positions, base_frequency=cfg.rope_base),
                StepRoPE1D(out=self.k4, x=self.k4, positions=self.positions, base_frequency=cfg.rope_base),
                StepCast(out=self.k16, x=self.k4, to_dtype=F16),
                StepCast(out=self.v16, x=self.v4, to_dtype=F16),
                StepSequenceAppend(cache=self.k_cache[layer], new_kv=self.k16, end_index=self.write_index),
                StepSequenceAppend(cache=self.v_cache[layer], new_kv=self.v16, end_index=self.write_index),
                StepAttention(out=self.attn, q=self.q4, k=self.k_cache[layer], v=self.v_cache[layer],
                              query_positions=self.positions, kv_lengths=self.visible_end, scale=scale,
                              window=AttentionWindow.causal()),
                StepMatMul(c=self.o, a=self.attn2, b=w["wo"]),
                StepRMSNorm(out=self.x, x=self.o, gamma=g, beta=b, eps=cfg.eps, residual=self.x),
                StepRMSNorm(out=self.x_norm, x=self.x, gamma=g, beta=b, eps=cfg.eps),
                StepMatMul(c=self.gate, a=self.x_norm, b=w["wg"]),
                StepMatMul(c=self.up, a=self.x_norm, b=w["wu"]),
                StepElemwiseBinary(op="gate", out=self.act, a=self.gate, b=self.up),
                StepMatMul(c=self.down, a=self.act, b=w["wd"]),
                StepRMSNorm(out=self.x, x=self.down, gamma=g, beta=b, eps=cfg.eps, residual=self.x),
            ]
        steps += [
            StepRMSNorm(out=self.x_norm, x=self.x, gamma=g, beta=b, eps=cfg.eps),
            StepMatMul(c=self.logits, a=self.x_norm, b=self.w_head),
            StepArgMax(out=self.next_token, a=self.logits),
        ]
        return steps

    def _build_steps_fused(self) -> list:
        cfg = self.cfg
        g, b = self.gamma, self.beta
        ixn, iat, iac = self.img_xn, self.img_attn, self.img_act
        scale = 1.0 / float(np.sqrt(cfg.head_dim))
        steps: list = [StepGatherRows(out=self.x, table=self.embed, indices=self.tokens),
                       StepRMSNorm(out=self.x_norm, x=self.x, gamma=g, beta=b, eps=cfg.eps, image=ixn)]
        for layer in range(cfg.layers):
            w = self.w[layer]
            steps += [
                StepMatMul(c=self.qkv, a=self.x_norm, b=w["wqkv"], a_image=ixn),
                StepRopeKVAppend(q_out=self.q_rot, qkv=self.qkv, positions=self.positions, end_index=self.write_index,
                                 k_cache=self.k_cache[layer], v_cache=self.v_cache[layer], base_frequency=cfg.rope_base),
                StepAttention(out=self.attn, q=self.q_rot, k=self.k_cache[layer], v=self.v_cache[layer],
                              query_positions=self.positions, kv_lengths=self.visible_end, scale=scale,
                              window=AttentionWindow.causal(), image=iat),
                StepMatMul(c=self.o, a=self.attn2, b=w["wo"], a_image=iat),
                # x = x + RMSNorm(o);  x_norm = RMSNorm(x)
                StepRMSNormPair(out1=self.x, out2=self.x_norm, x=self.o, gamma1=g, beta1=b, gamma2=g, beta2=b, eps1=cfg.eps,
                                eps2=cfg.eps, residual=self.x, image=ixn),
                StepMatMul(c=self.gu, a=self.x_norm, b=w["wgu"], a_image=ixn),
                StepElemwiseBinary(op="gate", out=self.act, a=self.gate_view, b=self.up_view, image=iac),
                StepMatMul(c=self.down, a=self.act, b=w["wd"], a_image=iac),
                # x = x + RMSNorm(down);  x_norm = RMSNorm(x): the next layer's input norm, or the final norm
                StepRMSNormPair(out1=self.x, out2=self.x_norm, x=self.down, gamma1=g, beta1=b, gamma2=g, beta2=b, eps1=cfg.eps,
                                eps2=cfg.eps, residual=self.x, image=ixn),
            ]
        steps += [StepMatMul(c=self.logits, a=self.x_norm, b=self.w_head, a_image=ixn),
                  StepArgMax(out=self.next_token, a=self.logits)]
        return steps

    # ---- running -------------------------------------------------------------------------
    def set_inputs(self, tokens, positions) -> None:
        """tokens, positions: i32 [R]. The new K/V row is written at `positions`, and keys up to
        and including it are visible."""
        R = self.requests
        tok = np.ascontiguousarray(tokens, dtype=np.int32).reshape(R, 1)
        pos = np.ascontiguousarray(positions, dtype=np.int32).reshape(R, 1)
        self.store.write(self.tokens, tok)
        self.store.write(self.positions, pos)
        self.store.write(self.write_index, pos.reshape(R))
        self.store.write(self.visible_end, (pos.reshape(R) + 1).astype(np.int32))

    def execute(self) -> None:
        """One token step, step by step (also the warm-up that sizes scratch before `record`)."""
        self.session.execute(self.steps)

    def record(self, lanes: int = capi.RECORD_LANES) -> None:
        self.program = self.session.record(self.steps, lanes=lanes)

    def launch(self) -> None:
        self.program.launch()

    def read_next_tokens(self) -> np.ndarray:
        return self.store.read(self.next_token).reshape(self.requests)

    def deinit(self) -> None:
        if self.program is not None:
            self.program.destroy()
            self.program = None
        self.store.deinit()
