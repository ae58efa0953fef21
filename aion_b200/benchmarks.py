"""Timed legs beyond the headline GEMV pass: the synthetic decoder (tokens/s), the prefill
GEMM (TFLOP/s), decode attention (GB/s) and the column-split large layer with its NCCL
all-gather. `bench.py` calls these; each returns a plain dict for its JSON line.

torch is used for what it is here for: device RNG for synthetic inputs, CUDA events on the
library's stream, and `torch.distributed` (NCCL) between ranks. All measured work runs in
libaion_cuda through the C ABI.
"""
from __future__ import annotations

import ctypes as C
import time

import numpy as np

from . import capi
from .backend import BackendError, Chunk, CudaBackend
from .decoder import DecoderConfig, SyntheticDecoder
from .sharding import column_shard, request_shard


def _chk(st):
    if st != capi.OK:
        raise BackendError(st, capi.last_error())


class _DevArray:
    """Exposes a device allocation of the library to torch (zero copy) as a flat array."""

    def __init__(self, handle: int, nbytes: int, typestr: str, itemsize: int):
        self.__cuda_array_interface__ = {"shape": (nbytes // itemsize,), "typestr": typestr, "data": (handle, False),
                                         "version": 2}


def _events(torch, backend, local_rank):
    stream = torch.cuda.ExternalStream(int(backend._lib.aion_cuda_get_stream(backend.handle)),
                                       device=torch.device("cuda", local_rank))
    return stream, torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def _max_over_ranks(torch, dist, world, value):
    if world == 1:
        return value
    t = torch.tensor([value], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _oracle_check_of_request0(dec, cfg, token0: int, position0: int, caches0, logits0, threads: int) -> dict:
    """One request of the step just executed, recomputed by the CPU oracle (the checker: the reference's
    arithmetic composed op by op) from the packed weights the device holds and the request's own cache rows.
    Returns the distance of the device's logits from the oracle's and the oracle's speed."""
    import time as _time

    from oracle.decoder_ref import OracleDecoder

    st = dec.store
    packed = {}
    for l, names in enumerate(dec.w):
        for name, tid in names.items():
            packed[f"l{l}.{name}"] = st.read(tid)
    packed["head"] = st.read(dec.w_head)
    row_bytes = cfg.hidden // 32 * 34
    ech = st.acquire_const(dec.embed)
    row = np.empty(row_bytes, dtype=np.uint8)
    dec.backend.device_memory.copy_d2h(row, ech.handle, ech.offset + token0 * row_bytes)
    ref = OracleDecoder.from_packed(cfg, 1, packed, row, fast=True)
    for l in range(cfg.layers):
        ref.k_cache[l][0], ref.v_cache[l][0] = caches0[l]
    ref.threads = threads  # explicit: the launcher of several ranks pins the OpenMP default to 1
    t0 = _time.perf_counter()
    _, logits_ref, next_ref = ref.step(np.array([0], np.int32), np.array([position0], np.int32))
    dt = _time.perf_counter() - t0
    got = np.asarray(logits0, dtype=np.float64)
    want = logits_ref.reshape(-1).astype(np.float64)
    top2 = np.sort(want)[-2:]
    return {"rel_l2_vs_oracle": float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)),
            "argmax_device": int(np.argmax(logits0)), "argmax_oracle": int(next_ref[0]),
            "oracle_top2_gap_over_max": float((top2[1] - top2[0]) / max(np.abs(want).max(), 1e-30)),
            "what": "request 0 of rank 0, all layers and the full head, device logits against the CPU oracle's on the same "
                    "packed weights and cache rows",
            "cpu_baseline": {"value": round(1.0 / dt, 3), "unit": "tokens/s", "cores": threads, "kind": "port",
                             "sample": "one request, one token step, through the oracle's decoder graph (threaded port of the "
                                       "reference's CPU kernels for the matmuls)"}}


def decode_leg(torch, dist, backend: CudaBackend, rank: int, world: int, local_rank: int, requests_total: int, steps: int,
               warmup: int, lanes: int, cfg: DecoderConfig | None = None, peak_gbs: float = 6552.3, check: bool = False,
               threads: int = 1) -> dict:
    """Decode tokens/s of the synthetic q4 decoder: `requests_total` concurrent requests at the far
    end of the context window, split evenly over the ranks (replicated weights, no exchange).
    check: on rank 0, recompute request 0 of the first step with the CPU oracle and report the distance."""
    cfg = cfg or DecoderConfig()
    mine = request_shard(requests_total, world, rank)
    R = mine.stop - mine.start
    if R == 0:
        raise ValueError("fewer requests than ranks")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234)  # every rank holds the same weights
    keep = []

    def weight_values(name, k, n):
        w = torch.randn((k, n), generator=gen, device="cuda", dtype=torch.float32) * 0.02
        torch.cuda.synchronize()
        keep[:] = [w]
        return Chunk(w.data_ptr(), 0, w.numel() * 4)

    def embedding_values(v0, v1):
        w = torch.randn((v1 - v0, cfg.hidden), generator=gen, device="cuda", dtype=torch.float32)
        torch.cuda.synchronize()
        keep[:] = [w]
        return Chunk(w.data_ptr(), 0, w.numel() * 4)

    t_build = time.perf_counter()
    dec = SyntheticDecoder(backend, cfg, R, weight_values, embedding_values)
    keep.clear()
    # Caches full of plausible keys / values: every request sits at the last position of its window.
    cgen = torch.Generator(device="cuda")
    cgen.manual_seed(11 + rank)
    for tid in dec.k_cache + dec.v_cache:
        ch = dec.store.acquire_mut(tid)
        t = torch.as_tensor(_DevArray(ch.handle + ch.offset, ch.len, "<f2", 2), device="cuda")
        t.normal_(0.0, 1.0, generator=cgen)
    torch.cuda.synchronize()
    tokens = (np.arange(mine.start, mine.stop) * 7919 + 13) % cfg.vocab
    positions = np.full(R, cfg.ctx - 1, np.int32)
    dec.set_inputs(tokens, positions)
    caches0 = None
    if check and rank == 0:
        # request 0's cache rows before the step appends to them (the oracle appends its own k, v)
        caches0 = []
        per_req = cfg.ctx * cfg.kv_width
        for l in range(cfg.layers):
            pair = []
            for tid in (dec.k_cache[l], dec.v_cache[l]):
                ch = dec.store.acquire_const(tid)
                rows = np.empty((cfg.ctx, cfg.kv_heads, cfg.head_dim), dtype=np.float16)
                backend.device_memory.copy_d2h(rows, ch.handle, ch.offset)
                pair.append(rows)
            caches0.append(tuple(pair))
    dec.execute()  # sizes scratch; also the un-recorded reference run
    backend.sync()
    first = dec.read_next_tokens().copy()
    oracle_check = None
    if caches0 is not None:
        lch = dec.store.acquire_const(dec.logits)
        logits0 = np.empty(cfg.vocab, dtype=np.float32)
        backend.device_memory.copy_d2h(logits0, lch.handle, lch.offset)
        try:
            oracle_check = _oracle_check_of_request0(dec, cfg, int(tokens[0]), int(positions[0]), caches0, logits0, threads)
        except Exception as e:  # the timing below must still run
            oracle_check = {"error": f"{type(e).__name__}: {e}"}
        caches0 = None
    dec.record(lanes=lanes)
    build_s = time.perf_counter() - t_build

    stream, ev0, ev1 = _events(torch, backend, local_rank)

    def barrier():
        backend.sync()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    for _ in range(max(warmup, 3)):
        dec.launch()
    barrier()
    replay_same = bool(np.array_equal(dec.read_next_tokens(), first))
    barrier()
    ev0.record(stream)
    for _ in range(steps):
        dec.launch()
    ev1.record(stream)
    backend.sync()
    torch.cuda.synchronize()
    ms = _max_over_ranks(torch, dist, world, ev0.elapsed_time(ev1)) / steps

    # end to end: per step the host sends token ids + positions and reads the next tokens back
    tok_host = np.ascontiguousarray(tokens, dtype=np.int32).reshape(R, 1)
    e2e_steps = max(3, min(steps, 50))
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        dec.set_inputs(tok_host, positions)
        dec.launch()
        tok_host = dec.read_next_tokens().reshape(R, 1) % cfg.vocab
    e2e_s = _max_over_ranks(torch, dist, world, time.perf_counter() - t0)

    step_bytes = cfg.weight_bytes_per_step() + R * cfg.kv_bytes_per_request_step()
    out = {
        "metric": "decode tokens/s", "value": round(requests_total / (ms * 1e-3), 1), "unit": "tokens/s",
        "ms_per_step": round(ms, 4), "requests_total": requests_total, "requests_per_gpu": R, "n_gpus": world,
        "scaling": "strong over requests (fixed total, batch-sharded, replicated weights, no collective)",
        "e2e_tokens_per_s": round(requests_total * e2e_steps / e2e_s, 1),
        "h2d_bytes_per_step": 4 * R * 4, "d2h_bytes_per_step": 4 * R,
        "hbm_bytes_per_step_per_gpu": step_bytes,
        "hbm_gbs_per_gpu": round(step_bytes / (ms * 1e-3) / 1e9, 1),
        "hbm_frac_of_measured": round(step_bytes / (ms * 1e-3) / 1e9 / peak_gbs, 4),
        "launches_per_step": len(dec.steps), "replay_matches_eager": replay_same, "build_s": round(build_s, 1),
        "matmul_kernel": ("int8 tensor-core kernel" if R < capi.GEMM_MIN_M else "tcgen05 GEMM (bf16 operands)") +
                         (", activation images written by the producing steps" if dec.images else ""),
        "config": {"layers": cfg.layers, "hidden": cfg.hidden, "ffn": cfg.ffn, "heads": cfg.heads, "kv_heads": cfg.kv_heads,
                   "head_dim": cfg.head_dim, "vocab": cfg.vocab, "ctx": cfg.ctx, "weights": "q4_0, N(0, 0.02), random init"},
    }
    if oracle_check is not None:
        out["oracle_check"] = oracle_check
    dec.deinit()
    return out


def gemm_leg(torch, backend: CudaBackend, local_rank: int, dtype: int, m: int, n: int, k: int, iters: int = 20, copies: int = 8,
             peak_tflops: float = 1622.7, nt: bool = False, kernel: str = "gemm") -> dict:
    """Prefill GEMM TFLOP/s: `copies` distinct weight matrices walked in turn, device-timed.
    nt: the `MatMulNT` step (q8_0 [n, k] row-major weights) instead of `MatMul`.
    kernel: "gemm" = the tcgen05 kernel (bf16 operands), "int8" = the int8-activation kernel, "auto" = by m."""
    flags = {"gemm": capi.MATMUL_FORCE_GEMM, "int8": capi.MATMUL_FORCE_GEMV, "auto": capi.MATMUL_AUTO}[kernel]
    lib, dev, mem = backend._lib, backend.handle, backend.device_memory
    bb = 18 if dtype == capi.DTYPE_Q4_0 else 34
    nb = (k // 32) * n * bb
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234)
    shape = (C.c_uint64 * 2)(*((n, k) if nt else (k, n)))
    hb = []
    for _ in range(copies):
        w = torch.randn((n, k) if nt else (k, n), generator=gen, device="cuda", dtype=torch.float32) * 0.02
        torch.cuda.synchronize()
        h = mem.alloc(nb, 256)
        src, dst = capi.Operand(w.data_ptr(), 0, w.numel() * 4), capi.Operand(h, 0, nb)
        _chk(lib.aion_cuda_quantize(dev, dtype, C.byref(src), shape, 2, 1 if nt else 0, C.byref(dst)))
        backend.sync()
        hb.append(h)
    a = torch.randn((m, k), generator=torch.Generator().manual_seed(5678), dtype=torch.float32).numpy()
    ha = mem.alloc(a.nbytes, 256)
    mem.copy_h2d(ha, 0, a)
    hc = mem.alloc(m * n * 4, 256)
    if nt:
        recs = [capi.MatMulNT(c=capi.Operand(hc, 0, m * n * 4), a=capi.Operand(ha, 0, a.nbytes), b=capi.Operand(h, 0, nb),
                              b_dtype=dtype, block_order=capi.ORDER_ROW_MAJOR, flags=flags, reserved=0, m=m, n=n, k=k, lda=0, ldc=0,
                              c_off=0, alpha=1.0, beta=0.0) for h in hb]
        call = lib.aion_cuda_matmul_nt
    else:
        recs = [capi.MatMul(c=capi.Operand(hc, 0, m * n * 4), a=capi.Operand(ha, 0, a.nbytes), b=capi.Operand(h, 0, nb),
                            b_dtype=dtype, flags=flags, m=m, n=n, k=k, lda=0, ldb=0, ldc=0, alpha=1.0, beta=0.0)
                for h in hb]
        call = lib.aion_cuda_matmul
    for i in range(3):
        _chk(call(dev, C.byref(recs[i % copies])))
    backend.sync()
    stream, ev0, ev1 = _events(torch, backend, local_rank)
    ev0.record(stream)
    for i in range(iters):
        _chk(call(dev, C.byref(recs[i % copies])))
    ev1.record(stream)
    backend.sync()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / iters
    tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    for h in hb + [ha, hc]:
        mem.free(h)
    return {"dtype": "q4_0" if dtype == capi.DTYPE_Q4_0 else "q8_0", "step": "MatMulNT [n,k]" if nt else "MatMul [k/32][n]",
            "kernel": kernel, "m": m, "n": n, "k": k, "ms": round(ms, 4), "tflops": round(tf, 1),
            "frac_of_measured_bf16_peak": round(tf / peak_tflops, 4),
            "includes": ("activation quantization + int8 kernel per call" if kernel == "int8" else
                         ("block permutation to K-major + " if nt else "") + "f32->bf16 activation pre-pass + GEMM kernel per call")}


def attention_leg(torch, backend: CudaBackend, local_rank: int, batch: int, t_ctx: int, iters: int = 20,
                  peak_gbs: float = 6552.3, heads: int = 8, kv_heads: int = 1, d: int = 256) -> dict:
    """Decode attention GB/s of algorithmic bytes (K + V once per request + q + out)."""
    lib, dev, mem = backend._lib, backend.handle, backend.device_memory
    # enough distinct cache sets that consecutive launches do not find K/V in L2
    kv_bytes = batch * t_ctx * kv_heads * d * 2
    copies = max(2, min(16, int((512 << 20) // max(2 * kv_bytes, 1)) + 1))
    gen = torch.Generator(device="cuda")
    gen.manual_seed(12)
    sets = []
    for _ in range(copies):
        hk, hv = mem.alloc(kv_bytes, 256), mem.alloc(kv_bytes, 256)
        for h in (hk, hv):
            torch.as_tensor(_DevArray(h, kv_bytes, "<f2", 2), device="cuda").normal_(0.0, 1.0, generator=gen)
        sets.append((hk, hv))
    torch.cuda.synchronize()
    q = torch.randn((batch, 1, heads, d), generator=torch.Generator().manual_seed(11), dtype=torch.float32).to(torch.float16).numpy()
    hq = mem.alloc(q.nbytes, 256)
    mem.copy_h2d(hq, 0, q)
    out_bytes = batch * heads * d * 4
    ho = mem.alloc(out_bytes, 256)
    pos = np.full((batch, 1), t_ctx - 1, np.int32)
    lens = np.full(batch, t_ctx, np.int32)
    hp, hl = mem.alloc(pos.nbytes, 64), mem.alloc(lens.nbytes, 64)
    mem.copy_h2d(hp, 0, pos)
    mem.copy_h2d(hl, 0, lens)
    recs = [capi.Attention(out=capi.Operand(ho, 0, out_bytes), q=capi.Operand(hq, 0, q.nbytes), k=capi.Operand(hk, 0, kv_bytes),
                           v=capi.Operand(hv, 0, kv_bytes), query_positions=capi.Operand(hp, 0, pos.nbytes),
                           kv_lengths=capi.Operand(hl, 0, lens.nbytes), q_dtype=capi.DTYPE_F16, k_dtype=capi.DTYPE_F16,
                           v_dtype=capi.DTYPE_F16, rolling=0, batch=batch, l_q=1, h_q=heads, h_kv=kv_heads, d_k=d, d_v=d,
                           t_cap=t_ctx, scale=1.0 / float(np.sqrt(d)), soft_cap=0.0, window_left=capi.WINDOW_UNBOUNDED,
                           window_right=0, window_chunk=0, flags=0) for hk, hv in sets]
    for i in range(copies):
        _chk(lib.aion_cuda_attention(dev, C.byref(recs[i])))
    backend.sync()
    # One recorded program = one launch over every cache set, so the host's per-call cost
    # (two tensor-map encodes and a launch) stays out of the device-timed region.
    _chk(lib.aion_cuda_record_begin(dev))
    for i in range(copies):
        _chk(lib.aion_cuda_attention(dev, C.byref(recs[i])))
    prog = C.c_void_p()
    _chk(lib.aion_cuda_record_end(dev, C.byref(prog)))
    for _ in range(3):
        _chk(lib.aion_cuda_program_launch(dev, prog))
    backend.sync()
    stream, ev0, ev1 = _events(torch, backend, local_rank)
    ev0.record(stream)
    for _ in range(iters):
        _chk(lib.aion_cuda_program_launch(dev, prog))
    ev1.record(stream)
    backend.sync()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / (iters * copies)
    lib.aion_cuda_program_destroy(dev, prog)
    alg = 2 * kv_bytes + q.nbytes + out_bytes
    for hk, hv in sets:
        mem.free(hk)
        mem.free(hv)
    for h in (hq, ho, hp, hl):
        mem.free(h)
    gbs = alg / (ms * 1e-3) / 1e9
    return {"batch": batch, "context": t_ctx, "ms": round(ms, 4), "gbs": round(gbs, 1), "frac_of_measured_hbm": round(gbs / peak_gbs, 4),
            "algorithmic_bytes": alg, "distinct_cache_sets": copies}


def prefill_attention_leg(torch, backend: CudaBackend, local_rank: int, batch: int, rows: int, iters: int = 10, heads: int = 8,
                          kv_heads: int = 4, d: int = 256, flags: int = 0, peak_tflops: float = 1622.7) -> dict:
    """Causal attention of a whole prompt (l_q = rows, keys 0..l per row), TFLOP/s of the two contractions
    over the visible keys only. flags: capi.ATTENTION_* (ROW_UNITS times the one-CTA-per-row tiling)."""
    lib, dev, mem = backend._lib, backend.handle, backend.device_memory
    gen = torch.Generator(device="cuda")
    gen.manual_seed(21)
    kv_bytes = batch * rows * kv_heads * d * 2
    q_bytes = batch * rows * heads * d * 2
    out_bytes = batch * rows * heads * d * 4
    hk, hv, hq, ho = mem.alloc(kv_bytes, 256), mem.alloc(kv_bytes, 256), mem.alloc(q_bytes, 256), mem.alloc(out_bytes, 256)
    for h, nb in ((hk, kv_bytes), (hv, kv_bytes), (hq, q_bytes)):
        torch.as_tensor(_DevArray(h, nb, "<f2", 2), device="cuda").normal_(0.0, 1.0, generator=gen)
    torch.cuda.synchronize()
    none = capi.Operand(0, 0, 0)
    rec = capi.Attention(out=capi.Operand(ho, 0, out_bytes), q=capi.Operand(hq, 0, q_bytes), k=capi.Operand(hk, 0, kv_bytes),
                         v=capi.Operand(hv, 0, kv_bytes), query_positions=none, kv_lengths=none, q_dtype=capi.DTYPE_F16,
                         k_dtype=capi.DTYPE_F16, v_dtype=capi.DTYPE_F16, rolling=0, batch=batch, l_q=rows, h_q=heads, h_kv=kv_heads,
                         d_k=d, d_v=d, t_cap=rows, scale=1.0 / float(np.sqrt(d)), soft_cap=0.0, window_left=capi.WINDOW_UNBOUNDED,
                         window_right=0, window_chunk=0, flags=flags)
    for _ in range(3):
        _chk(lib.aion_cuda_attention(dev, C.byref(rec)))
    backend.sync()
    stream, ev0, ev1 = _events(torch, backend, local_rank)
    ev0.record(stream)
    for _ in range(iters):
        _chk(lib.aion_cuda_attention(dev, C.byref(rec)))
    ev1.record(stream)
    backend.sync()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / iters
    for h in (hk, hv, hq, ho):
        mem.free(h)
    flops = 4.0 * batch * heads * d * rows * (rows + 1) / 2
    tf = flops / (ms * 1e-3) / 1e12
    return {"batch": batch, "rows": rows, "heads": heads, "kv_heads": kv_heads, "d": d, "ms": round(ms, 4), "tflops": round(tf, 1),
            "frac_of_measured_bf16_peak": round(tf / peak_tflops, 4),
            "tiling": "one CTA per row" if flags & capi.ATTENTION_ROW_UNITS else "blocks of positions",
            "kv_mb_streamed_once": round(2 * kv_bytes / 1e6, 1)}


def colsplit_leg(torch, dist, backend: CudaBackend, rank: int, world: int, local_rank: int, m: int, iters: int = 50,
                 n: int = 28672, k: int = 8192) -> dict:
    """The one large q4 layer column-split over the ranks: each rank computes y[:, n0:n1] straight
    into its slot of the gather buffer, then one NCCL all-gather (in place) assembles y on every rank.
    Every rank quantizes the SAME full weight (one seed) and keeps its column range of the packed blocks, so
    the assembled y can be compared with the unsplit matmul on one GPU: `max_abs_diff` below."""
    from .sharding import assemble_gathered

    lib, dev, mem = backend._lib, backend.handle, backend.device_memory
    n0, n1 = column_shard(n, world, rank)
    n_loc = n1 - n0
    bb = 18
    nb_full, nb = (k // 32) * n * bb, (k // 32) * n_loc * bb
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234)  # the same weight on every rank
    w = torch.randn((k, n), generator=gen, device="cuda", dtype=torch.float32) * 0.02
    torch.cuda.synchronize()
    h_full = mem.alloc(nb_full, 256)
    shape = (C.c_uint64 * 2)(k, n)
    src, dst = capi.Operand(w.data_ptr(), 0, w.numel() * 4), capi.Operand(h_full, 0, nb_full)
    _chk(lib.aion_cuda_quantize(dev, capi.DTYPE_Q4_0, C.byref(src), shape, 2, 0, C.byref(dst)))
    backend.sync()
    del w
    # this rank's columns of the packed [k/32][n] blocks: a strided copy on the device, block row by block row
    hw = mem.alloc(nb, 256)
    full_t = torch.as_tensor(_DevArray(h_full, nb_full, "|u1", 1), device="cuda").view(k // 32, n * bb)
    loc_t = torch.as_tensor(_DevArray(hw, nb, "|u1", 1), device="cuda").view(k // 32, n_loc * bb)
    loc_t.copy_(full_t[:, n0 * bb:n1 * bb])
    torch.cuda.synchronize()
    x = torch.randn((m, k), generator=torch.Generator().manual_seed(5678), dtype=torch.float32)
    xd = x.cuda()
    # gather buffer [world][m][n_loc]; rank r's matmul writes slot r (ldc = n_loc)
    gather = torch.zeros((world, m, n_loc), device="cuda", dtype=torch.float32)
    slot = gather[rank]
    rec = capi.MatMul(c=capi.Operand(slot.data_ptr(), 0, m * n_loc * 4), a=capi.Operand(xd.data_ptr(), 0, xd.numel() * 4),
                      b=capi.Operand(hw, 0, nb), b_dtype=capi.DTYPE_Q4_0, flags=capi.MATMUL_AUTO, m=m, n=n_loc, k=k,
                      lda=0, ldb=0, ldc=0, alpha=1.0, beta=0.0)
    stream, ev0, ev1 = _events(torch, backend, local_rank)

    def step():
        _chk(lib.aion_cuda_matmul(dev, C.byref(rec)))
        if world > 1:
            with torch.cuda.stream(stream):  # same stream as the kernel: ordered after it, no host sync
                dist.all_gather_into_tensor(gather.view(-1), slot.reshape(-1))

    for _ in range(5):
        step()
    backend.sync()
    torch.cuda.synchronize()
    # parity: the gathered y against the unsplit matmul over the full weight on this GPU
    y_full = torch.zeros((m, n), device="cuda", dtype=torch.float32)
    rec_full = capi.MatMul(c=capi.Operand(y_full.data_ptr(), 0, m * n * 4), a=capi.Operand(xd.data_ptr(), 0, xd.numel() * 4),
                           b=capi.Operand(h_full, 0, nb_full), b_dtype=capi.DTYPE_Q4_0, flags=capi.MATMUL_AUTO, m=m, n=n, k=k,
                           lda=0, ldb=0, ldc=0, alpha=1.0, beta=0.0)
    _chk(lib.aion_cuda_matmul(dev, C.byref(rec_full)))
    backend.sync()
    torch.cuda.synchronize()
    assembled = assemble_gathered(gather.cpu().numpy())
    want = y_full.cpu().numpy()
    max_abs = float(np.max(np.abs(assembled - want)))
    rel = float(np.linalg.norm(assembled.astype(np.float64) - want) / max(np.linalg.norm(want.astype(np.float64)), 1e-30))
    if world > 1:
        worst = torch.tensor([max_abs, rel], device="cuda", dtype=torch.float64)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        max_abs, rel = float(worst[0].item()), float(worst[1].item())
        dist.barrier()
    ev0.record(stream)
    for _ in range(iters):
        step()
    ev1.record(stream)
    backend.sync()
    torch.cuda.synchronize()
    ms = _max_over_ranks(torch, dist, world, ev0.elapsed_time(ev1)) / iters
    total_w = (k // 32) * n * 18
    out = {"m": m, "n": n, "k": k, "n_gpus": world, "columns_per_gpu": n_loc, "ms": round(ms, 4),
           "aggregate_weight_gbs": round(total_w / (ms * 1e-3) / 1e9, 1),
           "all_gather_bytes_per_rank": m * n_loc * 4,
           "parity": {"against": "the unsplit matmul over the full weight on one GPU, every rank checks the gathered y",
                      "max_abs_diff": max_abs, "rel_l2": rel, "pass": bool(rel <= 2e-5)}}
    if world > 1 and m <= 32:
        out["peer_stores"] = _colsplit_peer_stores(torch, dist, backend, rank, world, local_rank, m, n, k, n0, n1, hw, nb, xd, y_full, iters)
    mem.free(hw)
    mem.free(h_full)
    return out


def _colsplit_peer_stores(torch, dist, backend, rank, world, local_rank, m, n, k, n0, n1, hw, nb, xd, y_full, iters) -> dict:
    """The same layer with the exchange inside the matmul kernel: every rank's kernel stores its columns into
    every rank's y [m, n] over NVLink (peer stores from the epilogue) and announces them; a bounded wait kernel
    then finds y complete. Two y buffers alternate, since a rank may run one step ahead of a peer. One recorded
    program = two steps.

    Every rank makes the same collective calls in the same order whatever happens locally: a phase that fails
    on one rank is agreed on by all (an all-reduce of a flag after each phase), the rest of the leg is skipped
    everywhere, and the error is reported instead of a number."""
    lib, dev, mem = backend._lib, backend.handle, backend.device_memory
    y_bytes = m * n * 4
    n_loc = n1 - n0
    state = {"error": None}

    def phase(fn):
        """Runs fn on this rank unless an earlier phase failed somewhere; returns True when it worked everywhere."""
        if state["error"] is None:
            try:
                fn()
            except Exception as ex:  # noqa: BLE001 - reported in the leg's result
                state["error"] = f"{fn.__name__}: {type(ex).__name__}: {ex}"[:300]
        bad = torch.tensor([0 if state["error"] is None else 1], device="cuda", dtype=torch.int32)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()) and state["error"] is None:
            state["error"] = "another rank failed in this phase"
        return state["error"] is None

    mine, peers, opened, prog = {}, [], [], [None]
    everyone = [None] * world

    def allocate():
        for name, nbytes in (("y0", y_bytes), ("y1", y_bytes), ("flags", 32), ("state", 8)):
            mine[name] = mem.alloc(nbytes, 256)
            mem.memset(mine[name], 0, 0, nbytes)
        backend.sync()

    def export():
        exported = {}
        for name, h in mine.items():
            buf = (C.c_uint8 * 64)()
            _chk(lib.aion_cuda_ipc_export(dev, h, C.byref(buf)))
            exported[name] = bytes(buf)
        state["exported"] = exported

    phase(allocate)
    phase(export)
    dist.all_gather_object(everyone, state.get("exported"))

    def open_peers():
        for r in range(world):
            if r == rank:
                peers.append(dict(mine))
                continue
            got = {}
            for name in ("y0", "y1", "flags"):
                buf = (C.c_uint8 * 64).from_buffer_copy(everyone[r][name])
                h = C.c_uint64()
                _chk(lib.aion_cuda_ipc_import(dev, C.byref(buf), C.byref(h)))
                got[name] = h.value
                opened.append(h.value)
            peers.append(got)

    def fan_out(parity):
        key = "y1" if parity else "y0"
        c_of = lambda r: capi.Operand(peers[r][key], n0 * 4, y_bytes - n0 * 4)
        rec = capi.MatMul(c=c_of(rank), a=capi.Operand(xd.data_ptr(), 0, xd.numel() * 4), b=capi.Operand(hw, 0, nb),
                          b_dtype=capi.DTYPE_Q4_0, flags=capi.MATMUL_AUTO, m=m, n=n_loc, k=k, lda=0, ldb=0, ldc=n, alpha=1.0, beta=0.0)
        fan = capi.PeerFanout(world=world, rank=rank, state=capi.Operand(mine["state"], 0, 8))
        for r in range(world):
            fan.c[r] = c_of(r)
            fan.flags[r] = capi.Operand(peers[r]["flags"], 0, 32)
        _chk(lib.aion_cuda_matmul_peers(dev, C.byref(rec), C.byref(fan)))
        fl, st = capi.Operand(mine["flags"], 0, 32), capi.Operand(mine["state"], 0, 8)
        _chk(lib.aion_cuda_peer_wait(dev, C.byref(fl), C.byref(st), world, 0))

    result = {}

    def first_steps():
        fan_out(0)
        fan_out(1)
        backend.sync()
        got = [np.empty(m * n, np.float32), np.empty(m * n, np.float32)]
        mem.copy_d2h(got[0], mine["y0"], 0)
        mem.copy_d2h(got[1], mine["y1"], 0)
        want = y_full.cpu().numpy().reshape(-1).astype(np.float64)
        result["rel"] = max(float(np.linalg.norm(g.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30)) for g in got)

    def record():
        _chk(lib.aion_cuda_record_begin(dev))
        fan_out(0)
        fan_out(1)
        pg = C.c_void_p()
        _chk(lib.aion_cuda_record_end(dev, C.byref(pg)))
        prog[0] = pg
        for _ in range(3):
            _chk(lib.aion_cuda_program_launch(dev, pg))
        backend.sync()

    def timed():
        stream, ev0, ev1 = _events(torch, backend, local_rank)
        ev0.record(stream)
        for _ in range(iters):
            _chk(lib.aion_cuda_program_launch(dev, prog[0]))
        ev1.record(stream)
        backend.sync()
        torch.cuda.synchronize()
        result["ms_local"] = ev0.elapsed_time(ev1)

    # (each phase ends in an all-reduce: every rank's buffers are zeroed and opened everywhere before the first store)
    ok = phase(open_peers) and phase(first_steps)
    if ok:
        worst = torch.tensor([result["rel"]], device="cuda", dtype=torch.float64)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        result["rel"] = float(worst[0].item())
    ok = ok and phase(record) and phase(timed)
    if ok:
        result["ms"] = _max_over_ranks(torch, dist, world, result["ms_local"]) / (2 * iters)
    # Tear down in lockstep too: nobody closes a mapping another rank may still store into.
    try:
        backend.sync()
    except Exception:  # noqa: BLE001 - a fault recorded by a failed phase; already in the result
        pass
    dist.barrier()
    if prog[0] is not None:
        lib.aion_cuda_program_destroy(dev, prog[0])
    for h in opened:
        lib.aion_cuda_ipc_close(dev, h)
    dist.barrier()
    for h in mine.values():
        mem.free(h)
    what = "peer stores from the matmul kernel's epilogue into every rank's y + arrival words + one bounded wait kernel"
    if not ok:
        # every rank's own account, so that the rank that failed first can be told from those that waited for it
        errors = [None] * world
        dist.all_gather_object(errors, state["error"])
        return {"error": state["error"], "errors_by_rank": errors, "exchange": what}
    total_w = (k // 32) * n * 18
    ms = result["ms"]
    return {"ms": round(ms, 4), "aggregate_weight_gbs": round(total_w / (ms * 1e-3) / 1e9, 1), "exchange": what,
            "peer_bytes_per_rank": m * n_loc * 4 * (world - 1),
            "parity": {"against": "the unsplit matmul over the full weight on this GPU, both y buffers, worst rank", "rel_l2": result["rel"],
                       "pass": bool(result["rel"] <= 2e-5)}}


def matmul_leg(torch, backend: CudaBackend, local_rank: int, dtype: int, nt: bool, m: int, n: int, k: int, lanes: int = 8,
               iters: int = 20, min_bytes: int = 2400 << 20, peak_gbs: float = 6552.3) -> dict:
    """Decode-sized matmul (`MatMul` K-major or `MatMulNT` row-major q8) GB/s of algorithmic bytes over
    enough distinct weight copies (2.4 GB like the headline pass, at most 256 copies) that no launch finds its
    weights in L2 and that the lanes' drain at the end of a pass is a small part of it; one recorded program
    per pass, its independent steps spread over `lanes` parallel lanes."""
    lib, dev, mem = backend._lib, backend.handle, backend.device_memory
    bb = 18 if dtype == capi.DTYPE_Q4_0 else 34
    w_bytes = (k // 32) * n * bb
    copies = max(8, min(256, -(-min_bytes // w_bytes)))
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234)
    arena = mem.alloc(copies * w_bytes, 256)
    shape = (C.c_uint64 * 2)(*((n, k) if nt else (k, n)))
    for i in range(copies):
        w = torch.randn((n, k) if nt else (k, n), generator=gen, device="cuda", dtype=torch.float32) * 0.02
        torch.cuda.synchronize()
        src, dst = capi.Operand(w.data_ptr(), 0, w.numel() * 4), capi.Operand(arena, i * w_bytes, w_bytes)
        _chk(lib.aion_cuda_quantize(dev, dtype, C.byref(src), shape, 2, 1 if nt else 0, C.byref(dst)))
        backend.sync()
    x = torch.randn((copies, m, k), generator=torch.Generator().manual_seed(5678), dtype=torch.float32).numpy()
    hx, hy = mem.alloc(x.nbytes, 256), mem.alloc(copies * m * n * 4, 256)
    mem.copy_h2d(hx, 0, x)
    recs = []
    for i in range(copies):
        c_op, a_op = capi.Operand(hy, i * m * n * 4, m * n * 4), capi.Operand(hx, i * m * k * 4, m * k * 4)
        b_op = capi.Operand(arena, i * w_bytes, w_bytes)
        if nt:
            recs.append(capi.MatMulNT(c=c_op, a=a_op, b=b_op, b_dtype=dtype, block_order=capi.ORDER_ROW_MAJOR, flags=0, reserved=0,
                                      m=m, n=n, k=k, lda=0, ldc=0, c_off=0, alpha=1.0, beta=0.0))
        else:
            recs.append(capi.MatMul(c=c_op, a=a_op, b=b_op, b_dtype=dtype, flags=0, m=m, n=n, k=k, lda=0, ldb=0, ldc=0,
                                    alpha=1.0, beta=0.0))
    call = lib.aion_cuda_matmul_nt if nt else lib.aion_cuda_matmul

    def issue(nl):
        for i, r in enumerate(recs):
            if nl:
                _chk(lib.aion_cuda_record_lane(dev, i % nl))
            _chk(call(dev, C.byref(r)))

    issue(0)
    backend.sync()
    out = {"dtype": "q4_0" if dtype == capi.DTYPE_Q4_0 else "q8_0", "layout": "[N,K] row-major (MatMulNT)" if nt else "[K/32][N] (MatMul)",
           "m": m, "n": n, "k": k, "distinct_weight_copies": copies}
    alg = w_bytes + 4 * m * k + 4 * m * n
    stream, ev0, ev1 = _events(torch, backend, local_rank)
    for name, nl in (("lanes", lanes), ("serial", 1)):
        _chk(lib.aion_cuda_record_begin(dev))
        issue(nl)
        prog = C.c_void_p()
        _chk(lib.aion_cuda_record_end(dev, C.byref(prog)))
        for _ in range(3):
            _chk(lib.aion_cuda_program_launch(dev, prog))
        backend.sync()
        ev0.record(stream)
        for _ in range(iters):
            _chk(lib.aion_cuda_program_launch(dev, prog))
        ev1.record(stream)
        backend.sync()
        torch.cuda.synchronize()
        us = ev0.elapsed_time(ev1) * 1e3 / (iters * copies)
        gbs = alg / (us * 1e-6) / 1e9
        out[f"us_per_launch_{name}"] = round(us, 2)
        out[f"gbs_{name}"] = round(gbs, 1)
        out[f"frac_of_measured_hbm_{name}"] = round(gbs / peak_gbs, 4)
        lib.aion_cuda_program_destroy(dev, prog)
    for h in (arena, hx, hy):
        mem.free(h)
    return out


def gemv_cpu_baseline(dtype: int, nt: bool, m: int, n: int, k: int, threads: int, budget_s: float = 1.5) -> dict:
    """The reference's CPU path for a decode matmul (threaded port), walking enough distinct weight copies
    (random bytes with sane scales: the arithmetic does not care) that no cache holds them, for about `budget_s`."""
    import oracle

    bb = 18 if dtype == capi.DTYPE_Q4_0 else 34
    wb = (k // 32) * n * bb
    copies = int(max(2, min(64, (384 << 20) // wb + 1)))
    rng = np.random.default_rng(99)
    arena = rng.integers(0, 256, copies * wb, dtype=np.uint8)
    blocks = arena.reshape(-1, bb)
    blocks[:, 0] = rng.integers(0, 256, blocks.shape[0], dtype=np.uint8)
    blocks[:, 1] = 0x1F   # f16 scales around 2^-8
    a = rng.standard_normal((m, k)).astype(np.float32)
    c = np.zeros(m * n, dtype=np.float32)

    def one(i):
        w = arena[(i % copies) * wb:(i % copies + 1) * wb]
        if nt:
            oracle.fast_matmul_nt_q8(a, w, m, n, k, c=c, threads=threads)
        else:
            oracle.fast_matmul_q(dtype, a, w, m, n, k, c=c, threads=threads)

    one(0)
    t0, reps = time.perf_counter(), 0
    while time.perf_counter() - t0 < budget_s:
        one(reps)
        reps += 1
    dt = time.perf_counter() - t0
    alg = wb + 4 * m * k + 4 * m * n
    return {"value": round(alg * reps / dt / 1e9, 2), "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{reps} launches over {copies} distinct weight copies"}


def gemm_cpu_baseline(dtype: int, m: int, n: int, k: int, threads: int, sample_rows: int = 256, budget_s: float = 3.0) -> dict:
    """The reference's CPU path for the prefill GEMM (threaded port of its packed int8 GEMM) on a bounded
    sample: `sample_rows` of the m rows against the whole weight, repeated for about `budget_s`."""
    import oracle

    rows = min(m, sample_rows)
    rng = np.random.default_rng(1234)
    b = oracle.quantize(dtype, (rng.standard_normal((k, n)) * 0.02).astype(np.float32), 0)
    a = rng.standard_normal((rows, k)).astype(np.float32)
    c = np.zeros(rows * n, dtype=np.float32)
    oracle.fast_matmul_q(dtype, a, b, rows, n, k, c=c, threads=threads)
    t0, reps = time.perf_counter(), 0
    while time.perf_counter() - t0 < budget_s:
        oracle.fast_matmul_q(dtype, a, b, rows, n, k, c=c, threads=threads)
        reps += 1
    dt = time.perf_counter() - t0
    return {"value": round(2.0 * rows * n * k * reps / dt / 1e12, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"{rows} of the {m} rows against the whole {k}x{n} weight, {reps} passes, threaded port of the reference's "
                      f"packed int8 GEMM (vnni={oracle.fast_has_vnni()})"}


def attention_cpu_baseline(batch: int, t_ctx: int, threads: int, heads: int = 8, kv_heads: int = 1, d: int = 256,
                           sample_requests: int = 16, budget_s: float = 3.0) -> dict:
    """The reference's CPU path for decode attention with f16 q (its generic per-row executor, which streams K/V
    once per query head), requests over the host threads, on a bounded sample of the batch."""
    import oracle

    B = min(batch, sample_requests)
    rng = np.random.default_rng(12)
    q = rng.standard_normal((B, 1, heads, d)).astype(np.float16)
    kk = rng.standard_normal((B, t_ctx, kv_heads, d)).astype(np.float16)
    vv = rng.standard_normal((B, t_ctx, kv_heads, d)).astype(np.float16)
    pos = np.full((B, 1), t_ctx - 1, np.int32)
    lens = np.full(B, t_ctx, np.int32)
    kw = dict(scale=1.0 / float(np.sqrt(d)), positions=pos, kv_lengths=lens, right=0, threads=threads)
    oracle.fast_attention(q, kk, vv, **kw)
    t0, reps = time.perf_counter(), 0
    while time.perf_counter() - t0 < budget_s:
        oracle.fast_attention(q, kk, vv, **kw)
        reps += 1
    dt = time.perf_counter() - t0
    alg = 2 * kk.nbytes + q.nbytes + B * heads * d * 4
    return {"value": round(alg * reps / dt / 1e9, 3), "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{B} of the {batch} requests at context {t_ctx}, {reps} passes, the oracle's per-row executor with the requests "
                      "spread over the host threads"}
