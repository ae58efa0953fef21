#!/usr/bin/env python
"""Benchmark of the decode GEMV hot path (the `MatMul` step with q4_0 weights).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (the q4 GEMV of the benchmark configurations): x f32 [M=1, K=2048] ~ N(0,1),
W [K=2048, N=8192] ~ N(0,0.02) quantized to q4_0 [K/32][N] by the device quantizer
(byte-exact with the reference's q4 packer), y = x . W. One weight matrix is 9.4 MB and
would sit in the 126 MB L2, so a step walks COPIES = 256 distinct matrices (2.4 GB):
every launch reads weights that are not cached. One step = one replay of a recorded
program of 256 `aion_cuda_matmul` steps = one pass over the batch.

Metric: GB/s of algorithmic bytes (weights once + x + y per launch) — higher is better.
  value  : inputs resident in HBM, device-timed (CUDA events on the launching stream).
  e2e    : the same pass driven through the C ABI from HOST buffers (four sessions on four host
           threads, so one session's copies overlap the other's kernels): per step one
           aion_cuda_h2d of the batch's activations (pinned), the program, one
           aion_cuda_d2h of the results.
  N > 1  : replicas only (independent GEMVs share nothing): every rank runs the same
           pass on its GPU, no collective on the data path; value = sum of the ranks'
           bytes / max time.
--impl reference times the reference's CPU path for the same step (a threaded port of its
kernels: the reference is Zig and cannot be built here) on the host cores.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M, N, K = 1, 8192, 2048
COPIES = 256
W_BYTES = (K // 32) * N * 18
BYTES_PER_LAUNCH = W_BYTES + 4 * M * K + 4 * M * N
WORKLOAD = f"q4_0 GEMV (MatMul step) M={M} N={N} K={K}, {COPIES} distinct weight matrices per step"
# The same `config` in both arms (ours and --impl reference): the workload and how caches are kept out of it.
CONFIG = {"workload": WORKLOAD, "l2": "inputs larger than L2: every GEMV of a step reads a weight matrix no cache holds"}
METRIC = "q4 GEMV HBM GB/s"

# DRAM bytes per launch of the GEMV kernel from an ncu capture of this workload
# (dram__bytes_read.sum + dram__bytes_write.sum of one launch; summary under profiles/).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 9508096


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def measured_peak_tflops():
    """(burst, sustained) bf16 TFLOP/s of this pool's B200s, and which figures they are."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while a region runs (read-only NVML)."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, torch_device_index: int):
        self.samples = []
        self.stamped = []     # (time, MHz, reason mask) of every sample
        self.window = None    # (begin, end) of the timed region, when the sampler was started ahead of it
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml
            import torch

            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(torch_device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if hasattr(uuid, "encode") else uuid)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._h = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                self.samples.append(mhz)
                self.stamped.append((time.perf_counter(), mhz, mask))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.0005)

    def __enter__(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def begin_window(self):
        """The timed region starts now (the sampler thread is already running: its first reading takes a few ms)."""
        self.window = (time.perf_counter(), None)

    def end_window(self):
        self.window = (self.window[0], time.perf_counter())

    def summary(self):
        if self.window and self.window[1] is not None:
            inside = [(m, k) for t, m, k in self.stamped if self.window[0] <= t <= self.window[1]]
            if inside:
                reasons = sorted({name for _, k in inside for bit, name in self.REASONS.items() if k & bit})
                return {"sm_mhz": int(np.median([m for m, _ in inside])), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                        "samples": len(inside), "over": "the timed steps"}
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": int(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def run_ours(args):
    import torch
    import torch.distributed as dist

    from aion_b200 import capi
    from aion_b200.backend import BackendError, CudaBackend

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    backend = CudaBackend(local_rank)
    lib, dev = backend._lib, backend.handle
    mem = backend.device_memory

    def chk(st):
        if st != capi.OK:
            raise BackendError(st, capi.last_error())

    # ---- synthetic inputs, resident in HBM ------------------------------------------------
    w_arena = mem.alloc(COPIES * W_BYTES, 256)
    x_dev = mem.alloc(COPIES * M * K * 4, 256)
    y_dev = mem.alloc(COPIES * M * N * 4, 256)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234 + rank)
    shape = (C.c_uint64 * 2)(K, N)
    for i in range(COPIES):
        w = torch.randn((K, N), generator=gen, device="cuda", dtype=torch.float32) * 0.02
        torch.cuda.synchronize()
        src = capi.Operand(w.data_ptr(), 0, w.numel() * 4)
        dst = capi.Operand(w_arena, i * W_BYTES, W_BYTES)
        chk(lib.aion_cuda_quantize(dev, capi.DTYPE_Q4_0, C.byref(src), shape, 2, 0, C.byref(dst)))
        backend.sync()
    gen.manual_seed(5678 + rank)
    x_host = torch.randn((COPIES, M, K), generator=torch.Generator().manual_seed(5678 + rank), dtype=torch.float32).pin_memory()
    y_host = torch.empty((COPIES, M, N), dtype=torch.float32).pin_memory()
    chk(lib.aion_cuda_h2d(dev, x_dev, 0, C.c_void_p(x_host.data_ptr()), x_host.numel() * 4))

    steps_rec = []
    for i in range(COPIES):
        steps_rec.append(capi.MatMul(
            c=capi.Operand(y_dev, i * M * N * 4, M * N * 4), a=capi.Operand(x_dev, i * M * K * 4, M * K * 4),
            b=capi.Operand(w_arena, i * W_BYTES, W_BYTES), b_dtype=capi.DTYPE_Q4_0, flags=capi.MATMUL_AUTO,
            m=M, n=N, k=K, lda=0, ldb=0, ldc=0, alpha=1.0, beta=0.0))

    def issue_pass(lanes=0):
        for i, rec in enumerate(steps_rec):
            if lanes:
                chk(lib.aion_cuda_record_lane(dev, i % lanes))  # the steps share no tensor
            chk(lib.aion_cuda_matmul(dev, C.byref(rec)))

    issue_pass()  # first use of the kernels, outside any recording
    backend.sync()
    chk(lib.aion_cuda_record_begin(dev))
    issue_pass(args.lanes)
    prog = C.c_void_p()
    chk(lib.aion_cuda_record_end(dev, C.byref(prog)))

    stream = torch.cuda.ExternalStream(int(lib.aion_cuda_get_stream(dev)), device=torch.device("cuda", local_rank))
    ev0 = torch.cuda.Event(enable_timing=True)
    ev1 = torch.cuda.Event(enable_timing=True)

    def barrier():
        backend.sync()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    with ClockSampler(local_rank) as clocks:   # started ahead of the warm-up; only readings inside the timed region count
        for _ in range(max(args.warmup, 3)):
            chk(lib.aion_cuda_program_launch(dev, prog))
        barrier()
        clocks.begin_window()
        ev0.record(stream)
        for _ in range(args.steps):
            chk(lib.aion_cuda_program_launch(dev, prog))
        ev1.record(stream)
        backend.sync()
        torch.cuda.synchronize()
        clocks.end_window()
    elapsed_ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([elapsed_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        max_ms = float(t.item())
    else:
        max_ms = elapsed_ms
    ms_per_step = max_ms / args.steps
    bytes_per_step = COPIES * BYTES_PER_LAUNCH
    value = world * bytes_per_step / (ms_per_step * 1e-3) / 1e9

    # ---- the same pass held for about two seconds, with the clocks it ran at (sampling only) ------
    sustained = None
    if not args.no_sustained:
        n_sust = max(args.steps, int(2000.0 / max(ms_per_step, 1e-3)))
        barrier()
        with ClockSampler(local_rank) as sclocks:
            ev0.record(stream)
            for _ in range(n_sust):
                chk(lib.aion_cuda_program_launch(dev, prog))
            ev1.record(stream)
            backend.sync()
            torch.cuda.synchronize()
        s_ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([s_ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            s_ms = float(t.item())
        s_val = world * bytes_per_step * n_sust / (s_ms * 1e-3) / 1e9
        sc = sclocks.summary()
        sustained = {"value": round(s_val, 2), "unit": "GB/s", "steps": n_sust, "seconds": round(s_ms * 1e-3, 3),
                     "frac_of_peak_per_gpu": round(s_val / world / measured_peak_gbs()[0], 4), "clocks": sc,
                     "ms_per_step_times_sm_mhz": round(s_ms / n_sust * sc["sm_mhz"], 2) if sc.get("sm_mhz") else None}

    # ---- end to end from host buffers through the C ABI -------------------------------------
    e2e_steps = max(3, min(args.steps, 200))
    h2d_bytes = x_host.numel() * 4
    d2h_bytes = y_host.numel() * 4

    # Several sessions (device objects, each with its own stream, activation / result buffers
    # and recorded program over the shared weights) driven by one host thread each, the way a
    # server overlaps requests: one session's copies run under the other's kernels. Every step
    # of either session is h2d of its inputs, the program, d2h of its results.
    class E2ESession:
        def __init__(self, be, xd, yd, pg, owned):
            self.be, self.xd, self.yd, self.pg, self.owned = be, xd, yd, pg, owned
            self.y = y_host if not owned else torch.empty_like(y_host).pin_memory()

        def step(self):
            lb, dv = self.be._lib, self.be.handle
            chk(lb.aion_cuda_h2d(dv, self.xd, 0, C.c_void_p(x_host.data_ptr()), h2d_bytes))
            chk(lb.aion_cuda_program_launch(dv, self.pg))
            chk(lb.aion_cuda_d2h(dv, C.c_void_p(self.y.data_ptr()), self.yd, 0, d2h_bytes))

    sessions = [E2ESession(backend, x_dev, y_dev, prog, False)]
    for _extra in range(args.e2e_sessions - 1):
        be2 = CudaBackend(local_rank)
        x2 = be2.device_memory.alloc(COPIES * M * K * 4, 256)
        y2 = be2.device_memory.alloc(COPIES * M * N * 4, 256)
        recs2 = [capi.MatMul(c=capi.Operand(y2, i * M * N * 4, M * N * 4), a=capi.Operand(x2, i * M * K * 4, M * K * 4),
                             b=capi.Operand(w_arena, i * W_BYTES, W_BYTES), b_dtype=capi.DTYPE_Q4_0, flags=capi.MATMUL_AUTO,
                             m=M, n=N, k=K, lda=0, ldb=0, ldc=0, alpha=1.0, beta=0.0) for i in range(COPIES)]
        chk(be2._lib.aion_cuda_h2d(be2.handle, x2, 0, C.c_void_p(x_host.data_ptr()), h2d_bytes))
        for r2 in recs2:
            chk(be2._lib.aion_cuda_matmul(be2.handle, C.byref(r2)))
        be2.sync()
        chk(be2._lib.aion_cuda_record_begin(be2.handle))
        for i, r2 in enumerate(recs2):
            chk(be2._lib.aion_cuda_record_lane(be2.handle, i % args.lanes))
            chk(be2._lib.aion_cuda_matmul(be2.handle, C.byref(r2)))
        prog2 = C.c_void_p()
        chk(be2._lib.aion_cuda_record_end(be2.handle, C.byref(prog2)))
        sessions.append(E2ESession(be2, x2, y2, prog2, True))

    for sn in sessions:
        for _ in range(3):
            sn.step()
    barrier()
    per_session = max(2, e2e_steps // len(sessions))
    e2e_steps = per_session * len(sessions)
    errors = []

    def drive(sn):
        try:
            for _ in range(per_session):
                sn.step()
        except Exception as ex:  # surfaced after the join
            errors.append(ex)

    threads_ = [threading.Thread(target=drive, args=(sn,)) for sn in sessions[1:]]
    t0 = time.perf_counter()
    for th in threads_:
        th.start()
    drive(sessions[0])
    for th in threads_:
        th.join()
    for sn in sessions:
        sn.be.sync()
    e2e_s = time.perf_counter() - t0
    if errors:
        raise errors[0]
    same = True
    for sn in sessions[1:]:
        same = same and bool(torch.equal(sn.y, y_host))
        sn.be._lib.aion_cuda_program_destroy(sn.be.handle, sn.pg)
        sn.be.device_memory.free(sn.xd)
        sn.be.device_memory.free(sn.yd)
        sn.be.deinit()
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = world * bytes_per_step * e2e_steps / e2e_s / 1e9
    finite = bool(torch.isfinite(y_host).all().item()) and float(y_host.abs().sum()) > 0.0

    # ---- CPU baseline beside it (rank 0, one GPU only; bounded sample) ----------------------
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
        import oracle

        sample = 8
        wh = np.empty(sample * W_BYTES, dtype=np.uint8)
        mem.copy_d2h(wh, w_arena, 0)
        xs = x_host.numpy()
        cbuf = np.zeros(N * M, dtype=np.float32)
        threads = host_threads()
        oracle.fast_matmul_q(oracle.Q4_0, xs[0], wh[:W_BYTES], M, N, K, c=cbuf, threads=threads)
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 8.0:
            for i in range(sample):
                oracle.fast_matmul_q(oracle.Q4_0, xs[i], wh[i * W_BYTES:(i + 1) * W_BYTES], M, N, K, c=cbuf, threads=threads)
            reps += 1
        dt = time.perf_counter() - t0
        cpu_baseline = {"value": round(reps * sample * BYTES_PER_LAUNCH / dt / 1e9, 3), "unit": "GB/s", "cores": threads,
                        "kind": "port",
                        "sample": f"{sample} of the {COPIES} weight matrices, {reps} passes (~8 s), threaded port of the "
                                  f"reference's packed int8 GEMM route for q4 (vnni={oracle.fast_has_vnni()})"}

    peak, peak_kind = measured_peak_gbs()
    achieved = BYTES_PER_LAUNCH / (elapsed_ms * 1e-3 / (args.steps * COPIES)) / 1e9
    out = {
        "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x int4 -> int32, f32 scale/accumulate", "data": "synthetic",
        "config": dict(CONFIG),
        "run": {"parallelism": "replicas only" if world > 1 else "single GPU", "distinct_weight_bytes_per_step": COPIES * W_BYTES,
                "program": f"one recorded program per step; its 256 independent steps sit in {args.lanes} parallel lanes",
                "kernels_per_gemv": ("gemv_act_image_kernel + gemv_q_mma_kernel" if args.lanes > 1 else "gemv_q_mma_kernel"),
                "outputs_finite_nonzero": finite},
        "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d_bytes,
                "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps, "sessions": len(sessions),
                "how": "host threads, one per session; a step = aion_cuda_h2d + aion_cuda_program_launch + aion_cuda_d2h",
                "sessions_agree": same},
        # per GEMV of the pass: the activation-image kernel (A quantized once per launch) and the matmul kernel
        "gpu_launches": args.steps * COPIES * (2 if args.lanes > 1 else 1),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "peak_kind": f"of {peak_kind}",
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "algorithmic_bytes_per_launch": BYTES_PER_LAUNCH},
        "clocks": clocks.summary(),
    }
    if cpu_baseline is not None:
        out["cpu_baseline"] = cpu_baseline
    if sustained is not None:
        out["sustained"] = sustained
    lib.aion_cuda_program_destroy(dev, prog)
    for h in (w_arena, x_dev, y_dev):
        mem.free(h)
    from aion_b200 import benchmarks
    from aion_b200.decoder import DecoderConfig

    def leg(name, fn):
        try:
            out[name] = fn()
        except Exception as e:  # the headline line must still print
            out[name] = {"error": f"{type(e).__name__}: {e}"}

    threads = host_threads()
    if not args.no_extra_legs and world == 1:
        # The other kernels of the path, each beside its roofline and the reference's CPU path (bounded samples).
        tf_burst, tf_sust, tf_kind = measured_peak_tflops()

        def gemm_rows():
            rows = []
            for dt, m in ((capi.DTYPE_Q4_0, 512), (capi.DTYPE_Q4_0, 2048), (capi.DTYPE_Q8_0, 2048)):
                r = benchmarks.gemm_leg(torch, backend, local_rank, dt, m, 8192, 2048, iters=30, peak_tflops=tf_burst)
                r["roofline"] = {"bound": "tensor", "achieved": r["tflops"], "peak": tf_burst, "unit": "TFLOP/s",
                                 "frac": round(r["tflops"] / tf_burst, 4), "peak_kind": f"of {tf_kind} (bf16 burst)"}
                if not args.skip_cpu_baseline and dt == capi.DTYPE_Q4_0 and m == 2048:
                    r["cpu_baseline"] = benchmarks.gemm_cpu_baseline(dt, m, 8192, 2048, threads)
                rows.append(r)
            return {"metric": "prefill GEMM TFLOP/s (q4_0 / q8_0 [k/32][n] weights, k=2048, n=8192)", "rows": rows}

        def attention_rows():
            rows = []
            for b, t in ((64, 1024), (64, 4096), (8, 4096)):
                r = benchmarks.attention_leg(torch, backend, local_rank, b, t, iters=20, peak_gbs=peak)
                r["roofline"] = {"bound": "hbm", "achieved": r["gbs"], "peak": peak, "unit": "GB/s", "frac": r["frac_of_measured_hbm"],
                                 "peak_kind": f"of {peak_kind}"}
                if not args.skip_cpu_baseline and (b, t) == (64, 4096):
                    r["cpu_baseline"] = benchmarks.attention_cpu_baseline(b, t, threads)
                rows.append(r)
            return {"metric": "decode attention GB/s (8 query heads / 1 kv head, head_dim 256, f16)", "rows": rows}

        leg("gemm", gemm_rows)
        leg("attention", attention_rows)
    if not args.no_extra_legs and world > 1:
        def colsplit():
            return {"metric": "column-split q4 layer (k=8192, n=28672) + NCCL all-gather",
                    **benchmarks.colsplit_leg(torch, dist, backend, rank, world, local_rank, 1, iters=50)}

        leg("colsplit", colsplit)
    if not args.no_decode:
        # Second leg of the metric: decode tokens/s of the synthetic q4 decoder on the same GPUs.
        leg("decode", lambda: benchmarks.decode_leg(torch, dist, backend, rank, world, local_rank, args.decode_requests,
                                                    args.decode_steps, 3, args.lanes, DecoderConfig(layers=args.decode_layers), peak,
                                                    check=not args.skip_cpu_baseline, threads=threads))
    if rank == 0:
        print(json.dumps(out), flush=True)
    backend.deinit()
    if world > 1:
        dist.destroy_process_group()


def run_other(args):
    """The other workloads of the benchmark configurations, one JSON line each."""
    import torch
    import torch.distributed as dist

    from aion_b200 import benchmarks, capi
    from aion_b200.backend import CudaBackend
    from aion_b200.decoder import DecoderConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    backend = CudaBackend(local_rank)
    peak, peak_kind = measured_peak_gbs()
    with ClockSampler(local_rank) as clocks:
        if args.workload == "decode":
            out = benchmarks.decode_leg(torch, dist, backend, rank, world, local_rank, args.decode_requests, args.decode_steps,
                                        max(args.warmup, 3), args.lanes, DecoderConfig(layers=args.decode_layers), peak)
        elif args.workload == "gemm":
            dt = capi.DTYPE_Q4_0 if args.gemm_dtype == "q4" else capi.DTYPE_Q8_0
            out = {"metric": "prefill GEMM TFLOP/s", "n_gpus": 1,
                   **benchmarks.gemm_leg(torch, backend, local_rank, dt, args.gemm_m, 8192, 2048, iters=max(3, min(args.steps, 50)),
                                         kernel=args.gemm_kernel)}
        elif args.workload == "attention":
            out = {"metric": "decode attention GB/s", "n_gpus": 1,
                   **benchmarks.attention_leg(torch, backend, local_rank, args.attn_batch, args.attn_context,
                                              iters=max(3, min(args.steps, 50)), peak_gbs=peak)}
        elif args.workload == "prefill-attention":
            tf_peak = measured_peak_tflops()[0]
            legs = [benchmarks.prefill_attention_leg(torch, backend, local_rank, args.attn_batch, args.attn_rows, kv_heads=args.attn_kv_heads,
                                                     iters=max(3, min(args.steps, 20)), flags=fl, peak_tflops=tf_peak)
                    for fl in (0, capi.ATTENTION_ROW_UNITS)]
            out = {"metric": "prefill attention TFLOP/s", "n_gpus": 1, **legs[0], "one_cta_per_row": legs[1]}
        elif args.workload == "sweep":
            # The GEMV configurations of the benchmark: the single q8 NT op, then the q4 batch / shape sweep.
            rows = [benchmarks.matmul_leg(torch, backend, local_rank, capi.DTYPE_Q8_0, True, 1, 8192, 2048, lanes=args.lanes, peak_gbs=peak)]
            for (n, k) in ((2048, 2048), (8192, 2048), (2048, 8192)):
                for m in (1, 2, 4, 8):
                    rows.append(benchmarks.matmul_leg(torch, backend, local_rank, capi.DTYPE_Q4_0, False, m, n, k, lanes=args.lanes,
                                                      peak_gbs=peak))
            rows.append(benchmarks.matmul_leg(torch, backend, local_rank, capi.DTYPE_Q8_0, False, 1, 28672, 8192, lanes=args.lanes, peak_gbs=peak))
            rows.append(benchmarks.matmul_leg(torch, backend, local_rank, capi.DTYPE_Q4_0, False, 1, 28672, 8192, lanes=args.lanes, peak_gbs=peak))
            for dt in (capi.DTYPE_Q4_0, capi.DTYPE_Q8_0):
                for m in (512, 2048):
                    rows.append(benchmarks.gemm_leg(torch, backend, local_rank, dt, m, 8192, 2048))
            for m in (512, 2048):
                rows.append(benchmarks.gemm_leg(torch, backend, local_rank, capi.DTYPE_Q8_0, m, 8192, 2048, nt=True))
            if not args.skip_cpu_baseline:
                threads = host_threads()
                for r in rows:
                    dt = capi.DTYPE_Q4_0 if r["dtype"] == "q4_0" else capi.DTYPE_Q8_0
                    if "gbs_lanes" in r:
                        r["cpu_baseline"] = benchmarks.gemv_cpu_baseline(dt, r["layout"].startswith("[N,K]"), r["m"], r["n"], r["k"], threads)
                    elif r.get("step", "").startswith("MatMul ["):
                        r["cpu_baseline"] = benchmarks.gemm_cpu_baseline(dt, r["m"], r["n"], r["k"], threads, budget_s=1.5)
            for r in rows:
                print(json.dumps(r), flush=True)
            out = {"metric": "matmul sweep", "rows": len(rows)}
        else:
            out = {"metric": "column-split q4 layer + all-gather",
                   **benchmarks.colsplit_leg(torch, dist, backend, rank, world, local_rank, args.colsplit_m,
                                             iters=max(3, min(args.steps, 100)))}
    out["clocks"] = clocks.summary()
    out["data"] = "synthetic"
    if rank == 0:
        print(json.dumps(out), flush=True)
    backend.deinit()
    if world > 1:
        dist.destroy_process_group()


def host_threads() -> int:
    """Cores this process may run on. The launcher for several ranks sets OMP_NUM_THREADS=1, so the
    OpenMP default is not the answer: the CPU legs pass this count to the kernels explicitly."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def run_reference(args):
    """The reference's CPU path for the same step, on this host's cores (rank 0 only)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import oracle

    threads = host_threads()
    rng = np.random.default_rng(1234)
    base = 4
    mats = [oracle.quantize(oracle.Q4_0, (rng.standard_normal((K, N)) * 0.02).astype(np.float32), 0) for _ in range(base)]
    copies = 64  # 604 MB of distinct weight bytes: beyond any last-level cache
    arena = np.empty(copies * W_BYTES, dtype=np.uint8)
    for i in range(copies):
        arena[i * W_BYTES:(i + 1) * W_BYTES] = np.roll(mats[i % base], 18 * 8192 * (i // base))
    xs = rng.standard_normal((copies, M, K)).astype(np.float32)
    cbuf = np.zeros(M * N, dtype=np.float32)

    def gemv(i):
        oracle.fast_matmul_q(oracle.Q4_0, xs[i % copies], arena[(i % copies) * W_BYTES:(i % copies + 1) * W_BYTES], M, N, K, c=cbuf,
                             threads=threads)

    gemv(0)
    t0 = time.perf_counter()
    for i in range(8):
        gemv(i)
    t_one = (time.perf_counter() - t0) / 8
    # A step is a bounded sample of the pass: as many of its GEMVs as keep the whole run near two minutes.
    budget_s = 120.0
    total_steps = args.steps + max(args.warmup, 3)
    per_step = int(max(1, min(COPIES, budget_s / (total_steps * t_one))))
    it = 0
    for _ in range(max(args.warmup, 3)):
        for _ in range(per_step):
            gemv(it)
            it += 1
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for _ in range(per_step):
            gemv(it)
            it += 1
    dt = time.perf_counter() - t0
    value = args.steps * per_step * BYTES_PER_LAUNCH / dt / 1e9
    sample = (f"{per_step} of the pass's {COPIES} GEMVs per step over {copies} distinct matrices; threaded port of the "
              f"reference's CPU kernels (q4 takes its packed int8 GEMM route, re-packing B per call), vnni={oracle.fast_has_vnni()}")
    out = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(dt / args.steps * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int4 -> int32, f32 scale/accumulate",
        "data": "synthetic", "config": dict(CONFIG), "run": {"sample": sample, "distinct_weight_bytes": copies * W_BYTES},
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--lanes", type=int, default=8, help="parallel lanes the independent steps are recorded into (1..8)")
    ap.add_argument("--skip-cpu-baseline", action="store_true", help="leave the CPU leg out (profiling runs)")
    ap.add_argument("--workload", default="gemv", choices=["gemv", "decode", "gemm", "attention", "prefill-attention", "colsplit", "sweep"],
                    help="gemv: the headline pass (default; its line also carries the decode leg). The others print "
                         "their own line: decode tokens/s, prefill GEMM TFLOP/s, decode attention GB/s, the "
                         "column-split layer with its all-gather")
    ap.add_argument("--no-decode", action="store_true", help="gemv workload: leave the decoder leg out")
    ap.add_argument("--no-sustained", action="store_true", help="gemv workload: leave out the two-second run of the same pass")
    ap.add_argument("--no-extra-legs", action="store_true",
                    help="gemv workload: leave out the prefill GEMM / attention legs (1 GPU) and the column-split leg (several GPUs)")
    ap.add_argument("--e2e-sessions", type=int, default=4, choices=[1, 2, 3, 4],
                    help="sessions (device objects + host threads) the end-to-end leg drives concurrently")
    ap.add_argument("--decode-requests", type=int, default=512, help="concurrent requests in total, split over the GPUs")
    ap.add_argument("--decode-steps", type=int, default=20)
    ap.add_argument("--decode-layers", type=int, default=30)
    ap.add_argument("--gemm-m", type=int, default=2048)
    ap.add_argument("--gemm-dtype", default="q4", choices=["q4", "q8"])
    ap.add_argument("--gemm-kernel", default="gemm", choices=["gemm", "int8", "auto"],
                    help="gemm workload: the tcgen05 kernel (bf16 operands), the int8-activation kernel, or the library's own choice")
    ap.add_argument("--attn-batch", type=int, default=64)
    ap.add_argument("--attn-context", type=int, default=4096)
    ap.add_argument("--attn-rows", type=int, default=2048, help="prefill-attention workload: prompt rows per request (set --attn-batch too)")
    ap.add_argument("--attn-kv-heads", type=int, default=4, help="prefill-attention workload: kv heads under the 8 query heads")
    ap.add_argument("--colsplit-m", type=int, default=1)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "gemv":
        run_ours(args)
    else:
        run_other(args)


if __name__ == "__main__":
    main()
