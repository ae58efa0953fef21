"""Column-split layer with the exchange done by the matmul kernel itself: every rank's int8 kernel stores its
columns into every rank's y and announces them; a bounded wait then finds y complete. Here the ranks are
device objects on ONE GPU and are issued one after the other (a kernel never waits for a kernel that has
not finished), so what is tested is the data path, the arrival words and the epoch; the processes-on-several-
GPUs form runs in `bench.py --gpus N` (its `colsplit` leg checks the same parity)."""
import ctypes as C

import numpy as np
import pytest

import oracle
from aion_b200 import capi
from aion_b200.backend import BackendError, CudaBackend
from aion_b200.sharding import column_shard
from tests import refdata as rd
from tests.gpu_util import DevBuf, run_matmul

pytestmark = pytest.mark.gpu


def _raise(st):
    if st != capi.OK:
        raise BackendError(st, capi.last_error())


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("m", [1, 5])
def test_fan_out_assembles_y_on_every_rank(world, m):
    n, k = 64 * 8 * 6, 1024
    rng = np.random.default_rng(world * 10 + m)
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    a = rng.standard_normal((m, k)).astype(np.float32)
    packed = oracle.quantize(oracle.Q4_0, w, 0).reshape(k // 32, n, 18)
    ranks = [CudaBackend(0) for _ in range(world)]
    bufs = []
    try:
        ys = [[DevBuf(b, np.full(m * n, np.float32(777.0))) for _ in range(2)] for b in ranks]      # two parities
        flags = [DevBuf(b, np.zeros(8, np.uint32)) for b in ranks]
        states = [DevBuf(b, np.zeros(2, np.uint32)) for b in ranks]
        acts = [DevBuf(b, a) for b in ranks]
        slices, shards = [], []
        for r, b in enumerate(ranks):
            n0, n1 = column_shard(n, world, r)
            shards.append((n0, n1))
            slices.append(DevBuf(b, np.ascontiguousarray(packed[:, n0:n1]).reshape(-1)))
        bufs = [x for pair in ys for x in pair] + flags + states + acts + slices
        want = run_matmul(ranks[0], capi.DTYPE_Q4_0, a, packed.reshape(-1), m, n, k)
        for step in range(3):
            par = step & 1
            for r, b in enumerate(ranks):
                n0, n1 = shards[r]
                c_of = lambda q: capi.Operand(ys[q][par].handle, n0 * 4, (m * n - n0) * 4)
                rec = capi.MatMul(c=c_of(r), a=acts[r].operand(), b=slices[r].operand(), b_dtype=capi.DTYPE_Q4_0, flags=0, m=m, n=n1 - n0,
                                  k=k, lda=0, ldb=0, ldc=n, alpha=1.0, beta=0.0)
                fan = capi.PeerFanout(world=world, rank=r, state=states[r].operand())
                for q in range(world):
                    fan.c[q] = c_of(q)
                    fan.flags[q] = flags[q].operand()
                _raise(b._lib.aion_cuda_matmul_peers(b.handle, C.byref(rec), C.byref(fan)))
            for b in ranks:
                b.sync()
            for r, b in enumerate(ranks):   # every arrival is already there: the waits return at once
                _raise(b._lib.aion_cuda_peer_wait(b.handle, C.byref(flags[r].operand()), C.byref(states[r].operand()), world, 1000))
            for r, b in enumerate(ranks):
                b.sync()
                got = ys[r][par].read(np.float32).reshape(m, n)
                assert rd.rel_l2(got, want) < 1e-6, (step, r)
                assert states[r].read(np.uint32)[0] == step + 1            # the epoch advanced
                assert np.all(flags[r].read(np.uint32)[:world] == step + 1)  # every rank's arrival word
    finally:
        for x in bufs:
            x.free()
        for b in ranks:
            b.deinit()


def test_a_rank_that_never_arrives_is_reported_and_the_device_stays_usable(backend):
    """A wait on an arrival word that nothing writes runs out after its poll limit (no trap, no endless loop):
    the status word says so, the epoch does not move, and the device computes on."""
    flags = DevBuf(backend, np.zeros(8, np.uint32))
    state = DevBuf(backend, np.zeros(2, np.uint32))
    try:
        _raise(backend._lib.aion_cuda_peer_wait(backend.handle, C.byref(flags.operand()), C.byref(state.operand()), 2, 2000))
        with pytest.raises(BackendError) as e:
            backend.sync()
        assert e.value.name == "ExecutionFailed"
        assert state.read(np.uint32)[0] == 0
        a = rd.synth_acts(2, 256)
        b = oracle.quantize(oracle.Q8_0, rd.synth_weights(256, 64), 0)
        got = run_matmul(backend, capi.DTYPE_Q8_0, a, b, 2, 64, 256)
        assert rd.rel_l2(got, oracle.matmul_q(oracle.Q8_0, a, b, 2, 64, 256).reshape(2, 64)) < 2e-5
    finally:
        flags.free()
        state.free()


def test_fan_out_argument_errors(backend):
    a = DevBuf(backend, np.zeros(40 * 64, np.float32))
    try:
        rec = capi.MatMul(c=a.operand(), a=a.operand(), b=a.operand(), b_dtype=capi.DTYPE_Q4_0, flags=0, m=40, n=64, k=64, lda=0, ldb=0, ldc=0,
                          alpha=1.0, beta=0.0)
        fan = capi.PeerFanout(world=2, rank=0, state=a.operand())
        for q in range(2):
            fan.c[q], fan.flags[q] = a.operand(), a.operand()
        assert backend._lib.aion_cuda_matmul_peers(backend.handle, C.byref(rec), C.byref(fan)) == capi.UNSUPPORTED   # m > 32
        fan.world = 9
        assert backend._lib.aion_cuda_matmul_peers(backend.handle, C.byref(rec), C.byref(fan)) == capi.INVALID_ARGUMENT
    finally:
        a.free()
