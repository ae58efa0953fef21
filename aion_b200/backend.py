"""Host-side mirror of aion's backend seam over libaion_cuda.

aion's backends implement three Zig vtables; this module gives the same three roles in
Python (the reference toolchain, Zig, is not available here), with the reference's
names and argument meaning, so a test reads like the reference's own backend tests:

  * `DeviceMemory`  - src/aion/runtime/device_memory.zig:36-112
  * `DeviceStore`   - src/aion/runtime/device_store.zig:24-93 (TensorId -> meta + chunk)
  * `CudaBackend` / `CudaSession` - src/aion/backend/backend.zig:24-107

and the three step records of the hot path (src/aion/runtime/executable.zig:27,
105-115, 217-223). `CudaSession.execute(program)` walks the steps exactly as
`GpuSession.execute` does (src/aion/backend/gpu/backend.zig:551-662) and issues one C
call per step. Errors surface as the reference's error names.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
from typing import Optional, Sequence

import numpy as np

from . import capi

# types.BackendKind (src/aion/backend/types.zig:4-11)
BACKEND_KIND_CUDA = "cuda"

DTYPE_BYTES = {capi.DTYPE_F32: 4, capi.DTYPE_F16: 2, capi.DTYPE_I8: 1, capi.DTYPE_I32: 4}
BLOCK_BYTES = {capi.DTYPE_Q4_0: 18, capi.DTYPE_Q8_0: 34}
ORDER_NAMES = ["row_major", "lanes4", "lanes8", "lanes16", "lanes32", "lanes32x16"]


class BackendError(RuntimeError):
    """`BackendError || StoreError` (src/aion/backend/types.zig:27, src/aion/runtime/tensor_store.zig:7)."""

    NAMES = {1: "InvalidArgument", 2: "OutOfMemory", 3: "Unsupported", 4: "ExecutionFailed"}

    def __init__(self, status: int, message: str):
        self.status = status
        self.name = self.NAMES.get(status, f"status{status}")
        super().__init__(f"{self.name}: {message}")


def _check(status: int) -> None:
    if status != capi.OK:
        raise BackendError(status, capi.last_error())


class CudaBackend:
    """One B200 behind `Backend.VTable` {kind, name, caps, deinit, createSession}."""

    def __init__(self, ordinal: int = 0):
        self._lib = capi.load()
        h = C.c_void_p()
        _check(self._lib.aion_cuda_device_create(ordinal, C.byref(h)))
        self._h = h
        info = capi.DeviceInfo()
        _check(self._lib.aion_cuda_device_info(self._h, C.byref(info)))
        self.info = info
        self.device_memory = DeviceMemory(self)

    # -- Backend.VTable ----------------------------------------------------------
    def kind(self) -> str:
        return BACKEND_KIND_CUDA

    def name(self) -> str:
        return f"cuda:{self.info.ordinal} {self.info.name.decode()}"

    def caps(self) -> dict:
        # BackendCaps (src/aion/backend/types.zig:13-25)
        return {"simd": True, "threads": True, "fp16": True, "int8": True, "quant_q4": True, "quant_q8": True,
                "strided_copy": False}

    @property
    def quant_block_order(self) -> int:
        """The order the weight_layout pass should re-lay q8 [N,K] weights into."""
        return int(self._lib.aion_cuda_quant_block_order(self._h))

    def create_session(self, store: "DeviceStore") -> "CudaSession":
        return CudaSession(self, store)

    def deinit(self) -> None:
        if self._h:
            self._lib.aion_cuda_device_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.deinit()
        except Exception:
            pass

    # -- stream plumbing (no reference counterpart) -------------------------------
    def set_stream(self, cuda_stream: int | None) -> None:
        _check(self._lib.aion_cuda_set_stream(self._h, C.c_void_p(cuda_stream or 0)))

    def sync(self) -> None:
        _check(self._lib.aion_cuda_sync(self._h))

    @property
    def handle(self):
        return self._h


class DeviceMemory:
    """`DeviceMemory.VTable`: model, alloc, free, copyH2D, copyD2H, copyD2HMany, copyD2D, maxBindingBytes."""

    def __init__(self, backend: CudaBackend):
        self._b = backend
        self._lib = backend._lib

    def model(self) -> str:
        return "discrete" if self._lib.aion_cuda_memory_model(self._b._h) == 0 else "unified"

    def max_binding_bytes(self) -> int:
        return int(self._lib.aion_cuda_max_binding_bytes(self._b._h))

    def alloc(self, nbytes: int, alignment: int = 64) -> int:
        h = C.c_uint64()
        _check(self._lib.aion_cuda_alloc(self._b._h, nbytes, alignment, C.byref(h)))
        return int(h.value)

    def free(self, handle: int) -> None:
        _check(self._lib.aion_cuda_free(self._b._h, handle))

    def copy_h2d(self, handle: int, dst_offset: int, src: np.ndarray) -> None:
        src = np.ascontiguousarray(src)
        _check(self._lib.aion_cuda_h2d(self._b._h, handle, dst_offset, src.ctypes.data_as(C.c_void_p), src.nbytes))

    def copy_d2h(self, dst: np.ndarray, handle: int, src_offset: int = 0) -> None:
        assert dst.flags.c_contiguous and dst.flags.writeable
        _check(self._lib.aion_cuda_d2h(self._b._h, dst.ctypes.data_as(C.c_void_p), handle, src_offset, dst.nbytes))

    def copy_d2h_many(self, regions: Sequence[tuple[np.ndarray, int, int]]) -> None:
        for dst, handle, off in regions:
            self.copy_d2h(dst, handle, off)

    def copy_d2d(self, dst: int, dst_offset: int, src: int, src_offset: int, nbytes: int) -> None:
        _check(self._lib.aion_cuda_d2d(self._b._h, dst, dst_offset, src, src_offset, nbytes))

    def memset(self, handle: int, offset: int, value: int, nbytes: int) -> None:
        _check(self._lib.aion_cuda_memset(self._b._h, handle, offset, value, nbytes))


@dataclasses.dataclass
class TensorMeta:
    """`TensorMeta` (src/aion/runtime/tensor_store.zig:22-32) plus the quant axis storage keeps beside it."""

    dtype: int
    shape: tuple
    quant_axis: int = 0
    block_order: int = capi.ORDER_ROW_MAJOR
    # SequenceCachePolicyKind (src/aion/runtime/tensor_store.zig:9-13): "none" | "growable" | "rolling"
    cache_policy: str = "none"
    # Elements between consecutive rows (rows = all leading dims folded) of a view whose rows
    # are slices of a wider buffer; 0 = dense. Only the steps that say so accept such views.
    row_stride: int = 0
    # For a quantized-activation image (an i8 byte buffer made by `act_image_meta`): the weight
    # dtype it is laid out for; None for ordinary tensors.
    image_for: Optional[int] = None

    @property
    def rank(self) -> int:
        return len(self.shape)

    def nbytes(self) -> int:
        n = int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1
        if self.row_stride and self.shape:
            cols = int(self.shape[-1])
            n = (n // cols - 1) * self.row_stride + cols
        if self.dtype in BLOCK_BYTES:
            return n // 32 * BLOCK_BYTES[self.dtype]
        return n * DTYPE_BYTES[self.dtype]


@dataclasses.dataclass
class Chunk:
    """`Chunk{handle, offset, len}` (src/aion/runtime/device_store.zig:14-22)."""

    handle: int
    offset: int
    len: int

    def operand(self) -> capi.Operand:
        return capi.Operand(self.handle, self.offset, self.len)


def act_image_meta(m: int, k: int, weight_dtype: int) -> TensorMeta:
    """Meta of the quantized image of an [m, k] activation for a matmul against `weight_dtype` weights
    (`aion_cuda_act_image_bytes`): a zero-filled byte buffer a producing step writes and the matmul reads."""
    n = C.c_uint64()
    _check(capi.load().aion_cuda_act_image_bytes(m, k, C.byref(n)))
    return TensorMeta(capi.DTYPE_I8, (int(n.value),), image_for=weight_dtype)


class DeviceStore:
    """A minimal tensor table: TensorId -> (meta, device chunk). Owns what it allocates."""

    def __init__(self, memory: DeviceMemory):
        self.memory = memory
        self._meta: dict[int, TensorMeta] = {}
        self._chunk: dict[int, Chunk] = {}
        self._owned: list[int] = []
        self._next = 0

    def add(self, meta: TensorMeta, data: Optional[np.ndarray] = None) -> int:
        """Allocate a tensor on the device (optionally filled from host bytes); returns its TensorId."""
        nbytes = meta.nbytes()
        h = self.memory.alloc(max(nbytes, 1), 64)
        self._owned.append(h)
        if data is not None:
            data = np.ascontiguousarray(data)
            if data.nbytes != nbytes:
                raise BackendError(capi.INVALID_ARGUMENT, f"tensor holds {nbytes} bytes, data has {data.nbytes}")
            self.memory.copy_h2d(h, 0, data)
        elif meta.image_for is not None:
            self.memory.memset(h, 0, 0, max(nbytes, 1))  # an image's padding must read as zeros
        return self.bind(meta, Chunk(h, 0, nbytes))

    def bind(self, meta: TensorMeta, chunk: Chunk) -> int:
        """Register memory the caller owns (a torch tensor's data_ptr, a slice of an arena)."""
        tid = self._next
        self._next += 1
        self._meta[tid] = meta
        self._chunk[tid] = chunk
        return tid

    def meta(self, tid: int) -> TensorMeta:
        if tid not in self._meta:
            raise BackendError(capi.INVALID_ARGUMENT, f"unknown TensorId {tid}")
        return self._meta[tid]

    def acquire_const(self, tid: int) -> Chunk:
        self.meta(tid)
        return self._chunk[tid]

    acquire_mut = acquire_const

    def sequence_cache_policy_info(self, tid: int) -> str:
        return self.meta(tid).cache_policy

    def read(self, tid: int) -> np.ndarray:
        """Read a tensor back to the host (waits for the stream)."""
        meta, ch = self.meta(tid), self._chunk[tid]
        if meta.dtype in BLOCK_BYTES:
            out = np.empty(meta.nbytes(), dtype=np.uint8)
        else:
            np_dt = {capi.DTYPE_F32: np.float32, capi.DTYPE_F16: np.float16, capi.DTYPE_I8: np.int8,
                     capi.DTYPE_I32: np.int32}[meta.dtype]
            if meta.row_stride:
                cols = int(meta.shape[-1])
                rows = int(np.prod(meta.shape)) // cols
                raw = np.empty((rows - 1) * meta.row_stride + cols, dtype=np_dt)
                self.memory.copy_d2h(raw, ch.handle, ch.offset)
                idx = (np.arange(rows)[:, None] * meta.row_stride + np.arange(cols)[None, :]).reshape(-1)
                return raw[idx].reshape(meta.shape)
            out = np.empty(meta.shape, dtype=np_dt)
        self.memory.copy_d2h(out, ch.handle, ch.offset)
        return out

    def write(self, tid: int, data: np.ndarray) -> None:
        ch = self._chunk[tid]
        self.memory.copy_h2d(ch.handle, ch.offset, data)

    def deinit(self) -> None:
        for h in self._owned:
            self.memory.free(h)
        self._owned.clear()


# ---- step records (src/aion/runtime/executable.zig) ----------------------------------

@dataclasses.dataclass
class StepMatMul:
    c: int
    a: int
    b: int
    alpha: float = 1.0
    beta: float = 0.0
    flags: int = capi.MATMUL_AUTO
    # TensorId of the quantized image of A that the producing step wrote (no counterpart in the
    # reference; see `ActImage`), or None.
    a_image: Optional[int] = None


@dataclasses.dataclass
class StepMatMulNT:
    c: int
    a: int
    b: int
    alpha: float = 1.0
    beta: float = 0.0
    flags: int = capi.MATMUL_AUTO
    a_image: Optional[int] = None


@dataclasses.dataclass
class AttentionWindow:
    """src/aion/graph/graph.zig:130-167."""

    left: int = capi.WINDOW_UNBOUNDED
    right: int = capi.WINDOW_UNBOUNDED
    chunk: int = 0

    @staticmethod
    def causal() -> "AttentionWindow":
        return AttentionWindow(right=0)

    @staticmethod
    def sliding(n: int, m: int) -> "AttentionWindow":
        return AttentionWindow(left=n, right=m)

    @staticmethod
    def chunked(size: int, n: int) -> "AttentionWindow":
        return AttentionWindow(left=n, right=0, chunk=size)


@dataclasses.dataclass
class StepAttention:
    out: int
    q: int
    k: int
    v: int
    query_positions: Optional[int] = None
    kv_lengths: Optional[int] = None
    scale: float = 1.0
    window: AttentionWindow = dataclasses.field(default_factory=AttentionWindow)
    attn_logits_soft_cap: float = 0.0
    image: Optional[int] = None       # also write the quantized image of `out` (see `ActImage`)
    # Paged K / V: k and v are pools [pages, page_tokens, Hkv, D] and page_table is i32 [B, pages per request];
    # key t of request b is row t % page_tokens of page page_table[b, t // page_tokens].
    page_table: Optional[int] = None
    flags: int = 0                    # capi.ATTENTION_*


@dataclasses.dataclass
class StepRMSNorm:
    """src/aion/runtime/executable.zig:94-101."""
    out: int
    x: int
    gamma: int
    beta: int
    eps: float
    residual: Optional[int] = None
    image: Optional[int] = None


@dataclasses.dataclass
class StepElemwiseBinary:
    """src/aion/runtime/executable.zig:42-51; identical shapes only; op in {"add", "mul", "gate"} (gate act = gelu)."""
    op: str
    out: int
    a: int
    b: int
    image: Optional[int] = None


@dataclasses.dataclass
class StepRMSNormPair:
    """Fusion of StepRMSNorm(out1, x, gamma1, beta1, eps1, residual) and StepRMSNorm(out2, out1, gamma2, beta2, eps2)."""
    out1: int
    out2: int
    x: int
    gamma1: int
    beta1: int
    gamma2: int
    beta2: int
    eps1: float
    eps2: float
    residual: Optional[int] = None
    image: Optional[int] = None       # the quantized image of out2


@dataclasses.dataclass
class StepRopeKVAppend:
    """Fusion of RoPE1D(q), RoPE1D(k), Cast(k, v -> f16) and SequenceAppend of both, reading q | k | v
    from one [B, L, (h_q + 2 h_kv) * head_dim] matmul output (possibly a strided view)."""
    q_out: int
    qkv: int
    positions: int
    end_index: int
    k_cache: int
    v_cache: int
    base_frequency: float
    scale_factor: float = 1.0
    rope_proportion: float = 1.0


@dataclasses.dataclass
class StepRoPE1D:
    """src/aion/runtime/executable.zig:163-170."""
    out: int
    x: int
    positions: int
    base_frequency: float
    scale_factor: float = 1.0
    rope_proportion: float = 1.0


@dataclasses.dataclass
class StepCast:
    """src/aion/runtime/executable.zig:209."""
    out: int
    x: int
    to_dtype: int


@dataclasses.dataclass
class StepSequenceAppend:
    """src/aion/runtime/executable.zig:199-206."""
    cache: int
    new_kv: int
    end_index: int
    page_table: Optional[int] = None   # paged cache: `cache` is the pool [pages, page_tokens, H, D]


@dataclasses.dataclass
class StepGatherRows:
    """src/aion/runtime/executable.zig:155; q8_0 table dequantized on read."""
    out: int
    table: int
    indices: int


@dataclasses.dataclass
class StepArgMax:
    """src/aion/runtime/executable.zig:140; last axis only."""
    out: int
    a: int
    axis: int = -1


def _rows_of(shape: tuple) -> int:
    """Leading dims folded into M (src/aion/backend/cpu/exec/matmul.zig:333-338)."""
    m = 1
    for d in shape[:-1]:
        m *= d
    return m


class CudaSession:
    """`Session.VTable` {execute, retireResources, deinit} bound to one `DeviceStore`."""

    def __init__(self, backend: CudaBackend, store: DeviceStore):
        self.backend = backend
        self.store = store
        self._lib = backend._lib

    def execute(self, program: Sequence[object]) -> None:
        """Run the steps in order; asynchronous, like the reference's device path."""
        for step in program:
            if isinstance(step, StepMatMul):
                self._matmul(step)
            elif isinstance(step, StepMatMulNT):
                self._matmul_nt(step)
            elif isinstance(step, StepAttention):
                self._attention(step)
            elif type(step) in self._GLUE:
                getattr(self, self._GLUE[type(step)])(step)
            else:
                # An unsupported step never falls back to the host
                # (src/aion/runtime/executable.zig:355-357).
                raise BackendError(capi.UNSUPPORTED, f"step {type(step).__name__} is outside this backend")

    @staticmethod
    def _touches(step) -> tuple[set, set]:
        """(tensors read, tensors written) of a step, by TensorId."""
        img = lambda t: {t} if t is not None else set()
        if isinstance(step, (StepMatMul, StepMatMulNT)):
            reads = {step.a, step.b} | ({step.c} if step.beta != 0.0 else set()) | img(step.a_image)
            return reads, {step.c}
        if isinstance(step, StepAttention):
            reads = {step.q, step.k, step.v}
            reads |= {t for t in (step.query_positions, step.kv_lengths, step.page_table) if t is not None}
            return reads, {step.out} | img(step.image)
        if isinstance(step, StepRMSNorm):
            reads = {step.x, step.gamma, step.beta} | ({step.residual} if step.residual is not None else set())
            return reads, {step.out} | img(step.image)
        if isinstance(step, StepElemwiseBinary):
            return {step.a, step.b}, {step.out} | img(step.image)
        if isinstance(step, StepRMSNormPair):
            reads = {step.x, step.gamma1, step.beta1, step.gamma2, step.beta2}
            reads |= {step.residual} if step.residual is not None else set()
            return reads, {step.out1, step.out2} | img(step.image)
        if isinstance(step, StepRopeKVAppend):
            return ({step.qkv, step.positions, step.end_index, step.k_cache, step.v_cache},
                    {step.q_out, step.k_cache, step.v_cache})
        if isinstance(step, StepRoPE1D):
            return {step.x, step.positions}, {step.out}
        if isinstance(step, StepCast):
            return {step.x}, {step.out}
        if isinstance(step, StepSequenceAppend):
            return {step.new_kv, step.end_index, step.cache} | img(step.page_table), {step.cache}
        if isinstance(step, StepGatherRows):
            return {step.table, step.indices}, {step.out}
        if isinstance(step, StepArgMax):
            return {step.a}, {step.out}
        return set(), set()

    def _span(self, tid: int) -> tuple:
        """The device bytes a tensor occupies: views of one buffer must be seen as the same memory."""
        ch = self.store.acquire_const(tid)
        return (ch.handle, ch.offset, ch.offset + max(ch.len, 1))

    def record(self, program: Sequence[object], lanes: int = capi.RECORD_LANES) -> "RecordedProgram":
        """Record the steps once into a replayable device program (one launch per replay).

        Steps that share no tensor are issued into parallel lanes, so the device may overlap
        them; a step that depends on earlier ones follows them in the same lane, or after a
        join when they sit in several lanes. Steps that need scratch must have executed once
        before (run `execute` first)."""
        lib, h = self._lib, self.backend._h
        lanes = max(1, min(int(lanes), capi.RECORD_LANES))
        _check(lib.aion_cuda_record_begin(h))
        prog = C.c_void_p()
        try:
            writers: list[tuple] = []              # (span, lane) written since the last join
            readers: list[tuple] = []              # (span, lane) read since the last join
            next_lane = 0

            def overlaps(a, b):
                return a[0] == b[0] and a[1] < b[2] and b[1] < a[2]

            for step in program:
                reads, writes = self._touches(step)
                rspans = [self._span(t) for t in reads]
                wspans = [self._span(t) for t in writes]
                clash = {ln for sp, ln in writers for q in rspans + wspans if overlaps(sp, q)}
                clash |= {ln for sp, ln in readers for q in wspans if overlaps(sp, q)}
                if not clash:
                    lane = next_lane
                    next_lane = (next_lane + 1) % lanes
                elif len(clash) == 1:
                    lane = next(iter(clash))
                else:
                    _check(lib.aion_cuda_record_join(h))
                    writers.clear()
                    readers.clear()
                    lane, next_lane = 0, 1 % lanes
                _check(lib.aion_cuda_record_lane(h, lane))
                self.execute([step])
                writers.extend((sp, lane) for sp in wspans)
                readers.extend((sp, lane) for sp in rspans)
        finally:
            st = lib.aion_cuda_record_end(h, C.byref(prog))
        _check(st)
        return RecordedProgram(self.backend, prog)

    def retire_resources(self) -> None:
        self.backend.sync()

    def _image(self, tid: Optional[int], what: str) -> tuple:
        """(operand, weight dtype) of an optional activation image."""
        if tid is None:
            return capi.Operand(0, 0, 0), 0
        m = self.store.meta(tid)
        if m.image_for is None:
            raise BackendError(capi.INVALID_ARGUMENT, f"{what}: tensor {tid} is not an activation image")
        return self.store.acquire_mut(tid).operand(), m.image_for

    def deinit(self) -> None:
        self.retire_resources()

    # ---------------------------------------------------------------------------
    def _matmul(self, s: StepMatMul) -> None:
        st = self.store
        am, bm, cm = st.meta(s.a), st.meta(s.b), st.meta(s.c)
        if am.dtype != capi.DTYPE_F32 or cm.dtype != capi.DTYPE_F32:
            raise BackendError(capi.INVALID_ARGUMENT, "matmul: A and C must be f32")
        if bm.rank != 2 or (bm.dtype in BLOCK_BYTES and bm.quant_axis != 0):
            raise BackendError(capi.INVALID_ARGUMENT, "matmul: B must be [k, n] quantized along axis 0")
        k, n = bm.shape
        m = _rows_of(cm.shape)
        if am.shape[-1] != k or cm.shape[-1] != n or _rows_of(am.shape) != m:
            raise BackendError(capi.INVALID_ARGUMENT, "matmul: shapes do not agree")
        img, img_dt = self._image(s.a_image, "matmul.a_image")
        if s.a_image is not None and img_dt != bm.dtype:
            raise BackendError(capi.INVALID_ARGUMENT, "matmul: the image of A was laid out for another weight dtype")
        rec = capi.MatMul(c=st.acquire_mut(s.c).operand(), a=st.acquire_const(s.a).operand(),
                          b=st.acquire_const(s.b).operand(), b_dtype=bm.dtype, flags=s.flags, m=m, n=n, k=k,
                          lda=0, ldb=0, ldc=0, alpha=s.alpha, beta=s.beta, a_image=img)
        _check(self._lib.aion_cuda_matmul(self.backend._h, C.byref(rec)))

    def _matmul_nt(self, s: StepMatMulNT) -> None:
        st = self.store
        am, bm, cm = st.meta(s.a), st.meta(s.b), st.meta(s.c)
        if am.dtype != capi.DTYPE_F32 or cm.dtype != capi.DTYPE_F32:
            raise BackendError(capi.INVALID_ARGUMENT, "matmul_nt: A and C must be f32")
        # src/aion/runtime/executable.zig:210-216: B rank 2, quant_axis 1.
        if bm.rank != 2 or (bm.dtype in BLOCK_BYTES and bm.quant_axis != 1):
            raise BackendError(capi.INVALID_ARGUMENT, "matmul_nt: B must be [n, k] quantized along axis 1")
        n, k = bm.shape
        m = _rows_of(cm.shape)
        if am.shape[-1] != k or cm.shape[-1] != n:
            raise BackendError(capi.INVALID_ARGUMENT, "matmul_nt: shapes do not agree")
        img, img_dt = self._image(s.a_image, "matmul_nt.a_image")
        if s.a_image is not None and img_dt != bm.dtype:
            raise BackendError(capi.INVALID_ARGUMENT, "matmul_nt: the image of A was laid out for another weight dtype")
        rec = capi.MatMulNT(c=st.acquire_mut(s.c).operand(), a=st.acquire_const(s.a).operand(),
                            b=st.acquire_const(s.b).operand(), b_dtype=bm.dtype, block_order=bm.block_order,
                            flags=s.flags, m=m, n=n, k=k, lda=0, ldc=0, c_off=0, alpha=s.alpha, beta=s.beta, a_image=img)
        _check(self._lib.aion_cuda_matmul_nt(self.backend._h, C.byref(rec)))

    def _attention(self, s: StepAttention) -> None:
        st = self.store
        qm, km, vm, om = st.meta(s.q), st.meta(s.k), st.meta(s.v), st.meta(s.out)
        # src/aion/backend/cpu/exec/attention.zig:1461-1500
        if qm.rank != 4 or km.rank != 4 or vm.rank != 4 or om.rank != 4:
            raise BackendError(capi.INVALID_ARGUMENT, "attention: q, k, v, out must be rank 4")
        if om.dtype != capi.DTYPE_F32:
            raise BackendError(capi.INVALID_ARGUMENT, "attention: out must be f32")
        B, L, Hq, Dk = qm.shape
        _, T, Hkv, _ = km.shape
        Dv = vm.shape[3]
        none = capi.Operand(0, 0, 0)
        table, page_tokens, pool_pages = none, 0, 0
        if s.page_table is not None:
            tm = st.meta(s.page_table)
            if tm.dtype != capi.DTYPE_I32 or tm.rank != 2 or tm.shape[0] != B:
                raise BackendError(capi.INVALID_ARGUMENT, "attention: page_table must be i32 [B, pages per request]")
            if tuple(vm.shape[:3]) != tuple(km.shape[:3]) or km.shape[3] != Dk:
                raise BackendError(capi.INVALID_ARGUMENT, "attention: q/k/v shapes do not agree")
            pool_pages, page_tokens = km.shape[0], km.shape[1]
            T = tm.shape[1] * page_tokens
            table = st.acquire_const(s.page_table).operand()
        elif km.shape[0] != B or vm.shape[0] != B or km.shape[3] != Dk or vm.shape[1] != T or vm.shape[2] != Hkv:
            raise BackendError(capi.INVALID_ARGUMENT, "attention: q/k/v shapes do not agree")
        if tuple(om.shape) != (B, L, Hq, Dv):
            raise BackendError(capi.INVALID_ARGUMENT, "attention: out shape")
        pos = none
        if s.query_positions is not None:
            pm = st.meta(s.query_positions)
            if pm.dtype != capi.DTYPE_I32 or tuple(pm.shape) != (B, L):
                raise BackendError(capi.INVALID_ARGUMENT, "attention: query_positions must be i32 [B, L]")
            pos = st.acquire_const(s.query_positions).operand()
        lens = none
        if s.kv_lengths is not None:
            lm = st.meta(s.kv_lengths)
            if lm.dtype != capi.DTYPE_I32 or tuple(lm.shape) != (B,):
                raise BackendError(capi.INVALID_ARGUMENT, "attention: kv_lengths must be i32 [B]")
            lens = st.acquire_const(s.kv_lengths).operand()
        rolling = 1 if st.sequence_cache_policy_info(s.k) == "rolling" else 0
        img, img_dt = self._image(s.image, "attention.image")
        rec = capi.Attention(image=img, image_dtype=img_dt, out=st.acquire_mut(s.out).operand(), q=st.acquire_const(s.q).operand(),
                             k=st.acquire_const(s.k).operand(), v=st.acquire_const(s.v).operand(),
                             query_positions=pos, kv_lengths=lens, q_dtype=qm.dtype, k_dtype=km.dtype,
                             v_dtype=vm.dtype, rolling=rolling, batch=B, l_q=L, h_q=Hq, h_kv=Hkv, d_k=Dk, d_v=Dv,
                             t_cap=T, scale=s.scale, soft_cap=s.attn_logits_soft_cap,
                             window_left=s.window.left, window_right=s.window.right, window_chunk=s.window.chunk,
                             flags=s.flags, page_table=table, page_tokens=page_tokens, pool_pages=pool_pages)
        _check(self._lib.aion_cuda_attention(self.backend._h, C.byref(rec)))


    # ---- decoder glue steps -------------------------------------------------------
    def _need(self, tid: int, dtype: int, what: str) -> TensorMeta:
        m = self.store.meta(tid)
        if m.dtype != dtype:
            raise BackendError(capi.INVALID_ARGUMENT, f"{what}: dtype {m.dtype}, expected {dtype}")
        return m

    def _rms_norm(self, s: StepRMSNorm) -> None:
        st = self.store
        om = st.meta(s.out)
        if om.dtype == capi.DTYPE_F16:
            raise BackendError(capi.UNSUPPORTED, "rms_norm: f16 tensors are outside this backend")
        for t in (s.out, s.x, s.gamma, s.beta):
            self._need(t, capi.DTYPE_F32, "rms_norm")
        gm = st.meta(s.gamma)
        # src/aion/backend/cpu/exec/layernorm.zig:74-79: gamma's shape is the trailing dims of out.
        if gm.rank == 0 or gm.rank > om.rank or tuple(om.shape[om.rank - gm.rank:]) != tuple(gm.shape):
            raise BackendError(capi.INVALID_ARGUMENT, "rms_norm: gamma must match the trailing dims of out")
        cols = int(np.prod(gm.shape))
        rows = int(np.prod(om.shape)) // cols
        none = capi.Operand(0, 0, 0)
        res = none
        if s.residual is not None:
            self._need(s.residual, capi.DTYPE_F32, "rms_norm.residual")
            res = st.acquire_const(s.residual).operand()
        img, img_dt = self._image(s.image, "rms_norm.image")
        rec = capi.RMSNorm(out=st.acquire_mut(s.out).operand(), x=st.acquire_const(s.x).operand(),
                           gamma=st.acquire_const(s.gamma).operand(), beta=st.acquire_const(s.beta).operand(),
                           residual=res, rows=rows, cols=cols, eps=s.eps, image_dtype=img_dt, image=img)
        _check(self._lib.aion_cuda_rms_norm(self.backend._h, C.byref(rec)))

    def _elemwise(self, s: StepElemwiseBinary) -> None:
        st = self.store
        ops = {"add": capi.ELEMWISE_ADD, "mul": capi.ELEMWISE_MUL, "gate": capi.ELEMWISE_GATE_GELU}
        if s.op not in ops:
            raise BackendError(capi.UNSUPPORTED, f"elemwise: op {s.op!r} is outside this backend")
        om = self._need(s.out, capi.DTYPE_F32, "elemwise")
        metas = [om]
        for t in (s.a, s.b):
            m = self._need(t, capi.DTYPE_F32, "elemwise")
            if tuple(m.shape) != tuple(om.shape):
                raise BackendError(capi.UNSUPPORTED, "elemwise: only identical shapes are covered")
            metas.append(m)
        strided = any(m.row_stride for m in metas)
        img, img_dt = self._image(s.image, "elemwise.image")
        cols = int(om.shape[-1]) if (strided or s.image is not None) else 0
        rec = capi.Elemwise(out=st.acquire_mut(s.out).operand(), a=st.acquire_const(s.a).operand(),
                            b=st.acquire_const(s.b).operand(), count=int(np.prod(om.shape)), op=ops[s.op], reserved=0,
                            cols=cols, ld_out=metas[0].row_stride, ld_a=metas[1].row_stride, ld_b=metas[2].row_stride,
                            image=img, image_dtype=img_dt, reserved2=0)
        _check(self._lib.aion_cuda_elemwise(self.backend._h, C.byref(rec)))

    def _rms_norm_pair(self, s: StepRMSNormPair) -> None:
        st = self.store
        for t in (s.out1, s.out2, s.x, s.gamma1, s.beta1, s.gamma2, s.beta2):
            self._need(t, capi.DTYPE_F32, "rms_norm_pair")
        om, gm = st.meta(s.out1), st.meta(s.gamma1)
        if gm.rank == 0 or gm.rank > om.rank or tuple(om.shape[om.rank - gm.rank:]) != tuple(gm.shape) or \
                tuple(st.meta(s.gamma2).shape) != tuple(gm.shape) or tuple(st.meta(s.out2).shape) != tuple(om.shape):
            raise BackendError(capi.INVALID_ARGUMENT, "rms_norm_pair: shapes do not agree")
        cols = int(np.prod(gm.shape))
        rows = int(np.prod(om.shape)) // cols
        res = capi.Operand(0, 0, 0)
        if s.residual is not None:
            self._need(s.residual, capi.DTYPE_F32, "rms_norm_pair.residual")
            res = st.acquire_const(s.residual).operand()
        op = lambda t: st.acquire_const(t).operand()
        img, img_dt = self._image(s.image, "rms_norm_pair.image")
        rec = capi.RMSNormPair(out1=op(s.out1), out2=op(s.out2), x=op(s.x), gamma1=op(s.gamma1), beta1=op(s.beta1), residual=res,
                               gamma2=op(s.gamma2), beta2=op(s.beta2), rows=rows, cols=cols, eps1=s.eps1, eps2=s.eps2,
                               image=img, image_dtype=img_dt, reserved=0)
        _check(self._lib.aion_cuda_rms_norm_pair(self.backend._h, C.byref(rec)))

    def _rope_kv_append(self, s: StepRopeKVAppend) -> None:
        st = self.store
        qm = self._need(s.q_out, capi.DTYPE_F32, "rope_kv_append.q_out")
        xm = self._need(s.qkv, capi.DTYPE_F32, "rope_kv_append.qkv")
        pm = self._need(s.positions, capi.DTYPE_I32, "rope_kv_append.positions")
        self._need(s.end_index, capi.DTYPE_I32, "rope_kv_append.end_index")
        km, vm = self._need(s.k_cache, capi.DTYPE_F16, "rope_kv_append.k_cache"), self._need(s.v_cache, capi.DTYPE_F16, "rope_kv_append.v_cache")
        if qm.rank != 4 or km.rank != 4 or tuple(km.shape) != tuple(vm.shape) or tuple(pm.shape) != tuple(qm.shape[:2]):
            raise BackendError(capi.INVALID_ARGUMENT, "rope_kv_append: q_out [B, L, Hq, D], caches [B, T, Hkv, D], positions [B, L]")
        B, L, Hq, D = qm.shape
        _, T, Hkv, Dc = km.shape
        if km.shape[0] != B or Dc != D or xm.shape[-1] != (Hq + 2 * Hkv) * D or int(np.prod(xm.shape[:-1])) != B * L:
            raise BackendError(capi.INVALID_ARGUMENT, "rope_kv_append: qkv must hold q | k | v per (b, l)")
        policy = st.sequence_cache_policy_info(s.k_cache)
        if policy == "growable":
            raise BackendError(capi.UNSUPPORTED, "rope_kv_append: growable caches are settled by the storage layer, not here")
        op = lambda t: st.acquire_const(t).operand()
        rec = capi.RopeKVAppend(q_out=op(s.q_out), qkv=op(s.qkv), positions=op(s.positions), end_index=op(s.end_index),
                                k_cache=op(s.k_cache), v_cache=op(s.v_cache), batch=B, len=L, h_q=Hq, h_kv=Hkv, head_dim=D,
                                ld_qkv=xm.row_stride, t_cap=T, base_frequency=s.base_frequency, scale_factor=s.scale_factor,
                                proportion=s.rope_proportion, rolling=1 if policy == "rolling" else 0)
        _check(self._lib.aion_cuda_rope_kv_append(self.backend._h, C.byref(rec)))

    def _rope(self, s: StepRoPE1D) -> None:
        st = self.store
        xm = self._need(s.x, capi.DTYPE_F32, "rope")
        om = self._need(s.out, capi.DTYPE_F32, "rope")
        pm = self._need(s.positions, capi.DTYPE_I32, "rope.positions")
        if xm.rank != 4 or tuple(om.shape) != tuple(xm.shape) or tuple(pm.shape) != tuple(xm.shape[:2]):
            raise BackendError(capi.INVALID_ARGUMENT, "rope: x, out [B, L, N, H] and positions [B, L]")
        B, L, N, H = xm.shape
        rec = capi.RoPE(out=st.acquire_mut(s.out).operand(), x=st.acquire_const(s.x).operand(),
                        positions=st.acquire_const(s.positions).operand(), batch=B, len=L, heads=N, head_dim=H,
                        base_frequency=s.base_frequency, scale_factor=s.scale_factor, proportion=s.rope_proportion,
                        reserved=0)
        _check(self._lib.aion_cuda_rope(self.backend._h, C.byref(rec)))

    def _cast(self, s: StepCast) -> None:
        st = self.store
        xm, om = st.meta(s.x), st.meta(s.out)
        if om.dtype != s.to_dtype or int(np.prod(xm.shape)) != int(np.prod(om.shape)):
            raise BackendError(capi.INVALID_ARGUMENT, "cast: out does not match to_dtype / element count")
        rec = capi.Cast(out=st.acquire_mut(s.out).operand(), in_=st.acquire_const(s.x).operand(),
                        count=int(np.prod(xm.shape)), from_dtype=xm.dtype, to_dtype=om.dtype)
        _check(self._lib.aion_cuda_cast(self.backend._h, C.byref(rec)))

    def _sequence_append(self, s: StepSequenceAppend) -> None:
        st = self.store
        cm, nm = st.meta(s.cache), st.meta(s.new_kv)
        im = self._need(s.end_index, capi.DTYPE_I32, "sequence_append.end_index")
        # src/aion/backend/cpu/exec/sequence_append.zig:25-37
        if cm.rank != 4 or nm.rank != 4 or im.rank != 1 or cm.dtype != nm.dtype:
            raise BackendError(capi.INVALID_ARGUMENT, "sequence_append: ranks / dtypes")
        paged = s.page_table is not None
        if (not paged and cm.shape[0] != nm.shape[0]) or cm.shape[2] != nm.shape[2] or cm.shape[3] != nm.shape[3] or im.shape[0] != nm.shape[0]:
            raise BackendError(capi.INVALID_ARGUMENT, "sequence_append: shapes do not agree")
        policy = st.sequence_cache_policy_info(s.cache)
        if policy == "growable":
            raise BackendError(capi.UNSUPPORTED, "sequence_append: growable caches are settled by the storage layer, not here")
        B, T, H, D = cm.shape
        table, page_tokens, pool_pages = capi.Operand(0, 0, 0), 0, 0
        if paged:
            tm = self._need(s.page_table, capi.DTYPE_I32, "sequence_append.page_table")
            if tm.rank != 2 or tm.shape[0] != nm.shape[0]:
                raise BackendError(capi.INVALID_ARGUMENT, "sequence_append: page_table must be i32 [B, pages per request]")
            pool_pages, page_tokens = cm.shape[0], cm.shape[1]
            B, T = nm.shape[0], tm.shape[1] * page_tokens
            table = st.acquire_const(s.page_table).operand()
        rec = capi.SequenceAppend(cache=st.acquire_mut(s.cache).operand(), new_kv=st.acquire_const(s.new_kv).operand(),
                                  end_index=st.acquire_const(s.end_index).operand(), batch=B, t_cap=T, heads=H, head_dim=D,
                                  new_len=nm.shape[1], dtype=cm.dtype, rolling=1 if policy == "rolling" else 0,
                                  page_table=table, page_tokens=page_tokens, pool_pages=pool_pages)
        _check(self._lib.aion_cuda_sequence_append(self.backend._h, C.byref(rec)))

    def _gather_rows(self, s: StepGatherRows) -> None:
        st = self.store
        tm, om = st.meta(s.table), self._need(s.out, capi.DTYPE_F32, "gather_rows.out")
        im = self._need(s.indices, capi.DTYPE_I32, "gather_rows.indices")
        if tm.dtype != capi.DTYPE_Q8_0 or tm.rank != 2 or tm.quant_axis != 1:
            raise BackendError(capi.UNSUPPORTED, "gather_rows: only q8_0 [V, D] tables quantized along axis 1 are covered")
        V, D = tm.shape
        count = int(np.prod(im.shape))
        if om.shape[-1] != D or int(np.prod(om.shape)) != count * D:
            raise BackendError(capi.INVALID_ARGUMENT, "gather_rows: out must be indices.shape + [D]")
        rec = capi.GatherRows(out=st.acquire_mut(s.out).operand(), table=st.acquire_const(s.table).operand(),
                              indices=st.acquire_const(s.indices).operand(), table_rows=V, d=D, count=count,
                              block_order=tm.block_order, reserved=0)
        _check(self._lib.aion_cuda_gather_rows(self.backend._h, C.byref(rec)))

    def _argmax(self, s: StepArgMax) -> None:
        st = self.store
        am = self._need(s.a, capi.DTYPE_F32, "argmax")
        om = self._need(s.out, capi.DTYPE_I32, "argmax.out")
        if s.axis not in (-1, am.rank - 1):
            raise BackendError(capi.UNSUPPORTED, "argmax: only the last axis is covered")
        n = am.shape[-1]
        outer = int(np.prod(am.shape)) // n
        if int(np.prod(om.shape)) != outer:
            raise BackendError(capi.INVALID_ARGUMENT, "argmax: out shape")
        rec = capi.ArgMax(out=st.acquire_mut(s.out).operand(), in_=st.acquire_const(s.a).operand(), outer=outer, n=n)
        _check(self._lib.aion_cuda_argmax(self.backend._h, C.byref(rec)))

    _GLUE = {StepRMSNormPair: "_rms_norm_pair", StepRopeKVAppend: "_rope_kv_append",
             StepRMSNorm: "_rms_norm", StepElemwiseBinary: "_elemwise", StepRoPE1D: "_rope", StepCast: "_cast",
             StepSequenceAppend: "_sequence_append", StepGatherRows: "_gather_rows", StepArgMax: "_argmax"}


class RecordedProgram:
    """A recorded step list (a CUDA graph) bound to the buffers it was recorded with."""

    def __init__(self, backend: CudaBackend, handle):
        self.backend = backend
        self._h = handle

    def launch(self) -> None:
        _check(self.backend._lib.aion_cuda_program_launch(self.backend._h, self._h))

    def destroy(self) -> None:
        if self._h:
            self.backend._lib.aion_cuda_program_destroy(self.backend._h, self._h)
            self._h = None


# ---- storage-level helpers (Context.quantize / weight_layout on the device) -----------

def quantize(backend: CudaBackend, dtype: int, values: np.ndarray, quant_axis: int) -> np.ndarray:
    """Quantize an f32 host tensor on the device; returns the packed bytes (host)."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    mem = backend.device_memory
    nblocks = v.size // 32
    out_bytes = nblocks * BLOCK_BYTES.get(dtype, 34)  # an unknown dtype is rejected by the library
    hv, ho = mem.alloc(max(v.nbytes, 1)), mem.alloc(max(out_bytes, 1))
    try:
        mem.copy_h2d(hv, 0, v)
        shape = (C.c_uint64 * v.ndim)(*v.shape)
        vo, oo = capi.Operand(hv, 0, v.nbytes), capi.Operand(ho, 0, out_bytes)
        _check(backend._lib.aion_cuda_quantize(backend._h, dtype, C.byref(vo), shape, v.ndim, quant_axis, C.byref(oo)))
        out = np.empty(out_bytes, dtype=np.uint8)
        mem.copy_d2h(out, ho, 0)
        return out
    finally:
        mem.free(hv)
        mem.free(ho)


def dequantize(backend: CudaBackend, dtype: int, blocks: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    nblocks = b.size // BLOCK_BYTES[dtype]
    mem = backend.device_memory
    hb, ho = mem.alloc(max(b.nbytes, 1)), mem.alloc(max(nblocks * 128, 1))
    try:
        mem.copy_h2d(hb, 0, b)
        bo, oo = capi.Operand(hb, 0, b.nbytes), capi.Operand(ho, 0, nblocks * 128)
        _check(backend._lib.aion_cuda_dequantize(backend._h, dtype, C.byref(bo), nblocks, C.byref(oo)))
        out = np.empty(nblocks * 32, dtype=np.float32)
        mem.copy_d2h(out, ho, 0)
        return out
    finally:
        mem.free(hb)
        mem.free(ho)


def relayout_q8(backend: CudaBackend, order: int, n: int, k: int, src: np.ndarray, inverse: bool = False) -> np.ndarray:
    s = np.ascontiguousarray(src, dtype=np.uint8)
    mem = backend.device_memory
    hs, hd = mem.alloc(max(s.nbytes, 1)), mem.alloc(max(s.nbytes, 1))
    try:
        mem.copy_h2d(hs, 0, s)
        so, do = capi.Operand(hs, 0, s.nbytes), capi.Operand(hd, 0, s.nbytes)
        _check(backend._lib.aion_cuda_relayout_q8(backend._h, order, int(inverse), n, k, C.byref(so), C.byref(do)))
        out = np.empty(s.nbytes, dtype=np.uint8)
        mem.copy_d2h(out, hd, 0)
        return out
    finally:
        mem.free(hs)
        mem.free(hd)


def derive_kmajor_q8(backend: CudaBackend, order: int, n: int, k: int, src: np.ndarray) -> np.ndarray:
    """The K-major [k/32][n] derived weight of a q8_0 [n, k] tensor stored in `order` (bytes in, bytes out)."""
    s = np.ascontiguousarray(src, dtype=np.uint8)
    mem = backend.device_memory
    hs, hd = mem.alloc(max(s.nbytes, 1)), mem.alloc(max(s.nbytes, 1))
    try:
        mem.copy_h2d(hs, 0, s)
        so, do = capi.Operand(hs, 0, s.nbytes), capi.Operand(hd, 0, s.nbytes)
        _check(backend._lib.aion_cuda_derive_kmajor_q8(backend._h, order, n, k, C.byref(so), C.byref(do)))
        out = np.empty(s.nbytes, dtype=np.uint8)
        mem.copy_d2h(out, hd, 0)
        return out
    finally:
        mem.free(hs)
        mem.free(hd)
