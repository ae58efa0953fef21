"""Host-side logic that needs no GPU: tensor sizes of strided views, the decoder's step list,
and the lane assignment of `CudaSession.record` (driven through a stand-in library object that
only logs calls)."""
import numpy as np

from aion_b200 import capi
from aion_b200.backend import (Chunk, CudaSession, DeviceStore, StepElemwiseBinary, StepMatMul, StepRMSNorm, TensorMeta)
from aion_b200.decoder import DecoderConfig

F32, Q4 = capi.DTYPE_F32, capi.DTYPE_Q4_0


def test_tensor_meta_sizes():
    assert TensorMeta(F32, (3, 5)).nbytes() == 60
    assert TensorMeta(Q4, (64, 8), quant_axis=0).nbytes() == 64 * 8 // 32 * 18
    assert TensorMeta(capi.DTYPE_Q8_0, (8, 64), quant_axis=1).nbytes() == 8 * 64 // 32 * 34
    # rows of 4 elements inside rows of 10: the last row ends after its own 4 elements
    assert TensorMeta(F32, (3, 1, 4), row_stride=10).nbytes() == (2 * 10 + 4) * 4


def test_decoder_config_byte_counts():
    cfg = DecoderConfig()
    # the figures the benchmark's roofline uses (weights once per step, K + V per request)
    assert cfg.weights_per_step() == 30 * 44826624 + 402653184
    assert cfg.weight_bytes_per_step() == 982941696
    assert cfg.kv_bytes_per_request_step() == 62914560


class _Log:
    """Stands in for the loaded C library: every entry point returns OK and is logged."""

    def __init__(self):
        self.calls = []

    def __getattr__(self, name):
        def fn(*args):
            self.calls.append((name, args[1] if name == "aion_cuda_record_lane" else None))
            return capi.OK
        return fn


class _Mem:
    def __init__(self):
        self.next = 4096

    def alloc(self, nbytes, alignment=64):
        h = self.next
        self.next += (nbytes + 255) // 256 * 256 + 256
        return h

    def free(self, h):
        pass

    def copy_h2d(self, *a):
        pass


class _Backend:
    def __init__(self):
        self._lib = _Log()
        self._h = 1
        self.device_memory = _Mem()


def _lanes(calls):
    out, lane = [], None
    for name, arg in calls:
        if name == "aion_cuda_record_lane":
            lane = arg
        elif name == "aion_cuda_record_join":
            out.append("join")
        elif name in ("aion_cuda_matmul", "aion_cuda_rms_norm", "aion_cuda_elemwise"):
            out.append((name.replace("aion_cuda_", ""), lane))
    return out


def test_record_puts_independent_steps_in_parallel_lanes_and_orders_dependent_ones():
    be = _Backend()
    store = DeviceStore(be.device_memory)
    sess = CudaSession(be, store)
    R, H, N = 2, 64, 32
    x = store.add(TensorMeta(F32, (R, H)))
    g = store.add(TensorMeta(F32, (H,)))
    b = store.add(TensorMeta(F32, (H,)))
    xn = store.add(TensorMeta(F32, (R, H)))
    w1 = store.add(TensorMeta(Q4, (H, N), quant_axis=0))
    w2 = store.add(TensorMeta(Q4, (H, N), quant_axis=0))
    y1 = store.add(TensorMeta(F32, (R, N)))
    y2 = store.add(TensorMeta(F32, (R, N)))
    z = store.add(TensorMeta(F32, (R, N)))
    steps = [StepRMSNorm(out=xn, x=x, gamma=g, beta=b, eps=1e-6),      # lane 0
             StepMatMul(c=y1, a=xn, b=w1),                              # reads xn: same lane as the norm
             StepMatMul(c=y2, a=xn, b=w2),                              # reads xn too: same lane (one writer)
             StepElemwiseBinary(op="mul", out=z, a=y1, b=y2)]           # joins what wrote y1 and y2
    sess.record(steps, lanes=4)
    got = _lanes(be._lib.calls)
    assert got[0] == ("rms_norm", 0)
    assert got[1] == ("matmul", 0) and got[2] == ("matmul", 0)
    assert got[3] == ("elemwise", 0)
    # two unrelated chains go to different lanes
    be._lib.calls.clear()
    a2, c2 = store.add(TensorMeta(F32, (R, H))), store.add(TensorMeta(F32, (R, N)))
    sess.record([StepMatMul(c=y1, a=xn, b=w1), StepMatMul(c=c2, a=a2, b=w2)], lanes=4)
    got = _lanes(be._lib.calls)
    assert got[0][1] != got[1][1]


def test_views_of_one_buffer_are_seen_as_the_same_memory():
    be = _Backend()
    store = DeviceStore(be.device_memory)
    sess = CudaSession(be, store)
    R, F = 2, 16
    gu = store.add(TensorMeta(F32, (R, 2 * F)))
    ch = store.acquire_const(gu)
    half = TensorMeta(F32, (R, F), row_stride=2 * F)
    gate = store.bind(half, Chunk(ch.handle, ch.offset, ch.len))
    up = store.bind(half, Chunk(ch.handle, ch.offset + F * 4, ch.len - F * 4))
    x = store.add(TensorMeta(F32, (R, 32)))
    w = store.add(TensorMeta(Q4, (32, 2 * F), quant_axis=0))
    act = store.add(TensorMeta(F32, (R, F)))
    sess.record([StepMatMul(c=gu, a=x, b=w), StepElemwiseBinary(op="gate", out=act, a=gate, b=up)], lanes=4)
    got = _lanes(be._lib.calls)
    assert got[0][1] == got[1][1], "the gate reads the matmul's output through views: it must follow it in the same lane"


def test_cpu_legs_use_the_hosts_cores_whatever_the_launcher_sets(monkeypatch):
    """The multi-rank launcher exports OMP_NUM_THREADS=1; bench.py's CPU legs must still pass the
    cores this process may run on to the threaded oracle port, explicitly."""
    import os
    import bench
    monkeypatch.setenv("OMP_NUM_THREADS", "1")
    want = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    assert bench.host_threads() == max(1, want)
