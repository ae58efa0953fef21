"""Reader of the weights of an `.aion` model file (format version 16), for feeding a converted
model's tensors straight to the CUDA backend.

The file is aion's own container (src/aion/storage/aion_file/types.zig:15-26):

    header (72 bytes)   magic "AION", version u32, section count u32, reserved u32,
                        directory offset u64, file size u64, flags u64, 32 reserved bytes
                        (src/aion/storage/aion_file/write.zig:607-617)
    directory           per section: type u32, flags u32 (bit 0 = required), offset u64, size u64
                        (src/aion/storage/aion_file/parse.zig:175-196)
    sections            strings, tensors, values, nodes, signatures, graph_meta, ... back to back;
                        the tensors section and every payload inside it start on a 64-byte boundary,
                        so a mapped file's payload is usable as a tensor's bytes in place
                        (types.zig:19-26, parse.zig:329-381)

Only what the weight path needs is decoded: strings, the tensors section (each initializer with
its plain dtype or its `QuantizedEncoding{scheme, block_elems, block_bytes, quant_axis}`,
types.zig:85-98), values (dtype, shape, which initializer backs them), signatures, debug names and
metadata. Graph nodes stay opaque bytes: compiling the graph is the reference's job. Errors follow
the reference's `PackageError` names (types.zig:31-38).

All integers are little-endian. Payloads are returned as memoryviews of the mapped file: nothing is
copied until a tensor is uploaded.
"""
from __future__ import annotations

import dataclasses
import mmap
import struct
from typing import Optional, Union

MAGIC = b"AION"
VERSION = 16
PAYLOAD_ALIGNMENT = 64
HEADER_SIZE = 72
SECTION_DESC_SIZE = 24
INVALID_INDEX = 0xFFFFFFFF

# SectionType (types.zig:40-54)
SECTIONS = {1: "strings", 2: "tensors", 3: "values", 4: "nodes", 5: "signatures", 6: "graph_meta", 7: "dim_symbols",
            8: "dim_exprs", 9: "metadata", 10: "debug_names", 11: "regions", 12: "io_aliases", 13: "input_roles"}
REQUIRED = ("strings", "tensors", "values", "nodes", "signatures", "graph_meta")
SECTION_REQUIRED_FLAG = 1

# DType codes (src/aion/backend/types.zig:29-39)
DTYPE_NAMES = ["f32", "f16", "i8", "q4_0", "q8_0", "i32"]
# (block elements, block bytes) per dtype (types.zig:40-56)
DTYPE_BLOCK = {0: (1, 4), 1: (1, 2), 2: (1, 1), 3: (32, 18), 4: (32, 34), 5: (1, 4)}
SCHEME_DTYPE = {"q4_0": 3, "q8_0": 4}


class PackageError(Exception):
    """The reference's `PackageError` set; `.name` is the error name."""

    def __init__(self, name: str, message: str = ""):
        self.name = name
        super().__init__(f"{name}: {message}" if message else name)


def _invalid(msg: str) -> PackageError:
    return PackageError("InvalidFormat", msg)


class _Cursor:
    """Bounds-checked little-endian reads over a bytes-like view (parse.zig:849-871)."""

    def __init__(self, view: memoryview, pos: int = 0):
        self.view, self.pos = view, pos

    def take(self, n: int) -> memoryview:
        if n < 0 or self.pos + n > len(self.view):
            raise _invalid("read past the end of a section")
        out = self.view[self.pos:self.pos + n]
        self.pos += n
        return out

    def u8(self) -> int:
        return self.take(1)[0]

    def u32(self) -> int:
        return struct.unpack("<I", self.take(4))[0]

    def i32(self) -> int:
        return struct.unpack("<i", self.take(4))[0]

    def u64(self) -> int:
        return struct.unpack("<Q", self.take(8))[0]

    def done(self) -> bool:
        return self.pos == len(self.view)


@dataclasses.dataclass
class Initializer:
    """One tensor payload (types.zig:100-104). `dtype` is the storage dtype code: the plain dtype, or
    q4_0 / q8_0 for a quantized encoding with that scheme."""

    quantized: bool
    dtype: int
    logical_dtype: Optional[int]
    scheme: Optional[str]
    block_elems: int
    block_bytes: int
    quant_axis: int
    params: bytes
    data: memoryview
    file_offset: int  # of the payload: a multiple of 64


@dataclasses.dataclass
class ValueRecord:
    """types.zig:131-137. A shape entry is an int (a constant) or ("expr", index) for a symbolic dimension."""

    dtype: int
    rank: int
    source: int  # 0 public input, 1 initializer, 2 produced
    shape: list
    initializer_index: Optional[int]


@dataclasses.dataclass
class Weight:
    """An initializer seen through the value it backs."""

    value: int
    name: Optional[str]
    dtype: int
    shape: tuple
    quant_axis: int
    data: memoryview

    @property
    def dtype_name(self) -> str:
        return DTYPE_NAMES[self.dtype]


@dataclasses.dataclass
class Package:
    version: int
    strings: list
    initializers: list
    values: list
    inputs: list      # (name, value id)
    outputs: list
    debug_names: dict  # value id -> name
    metadata: dict
    sections: dict     # name -> (offset, size, flags)
    nodes_raw: memoryview
    _mapping: object = None

    def weights(self) -> list:
        """Every value backed by an initializer whose shape is all constants."""
        out = []
        for vid, v in enumerate(self.values):
            if v.source != 1 or v.initializer_index is None:
                continue
            init = self.initializers[v.initializer_index]
            if not all(isinstance(d, int) for d in v.shape):
                continue
            out.append(Weight(vid, self.debug_names.get(vid), init.dtype, tuple(v.shape), init.quant_axis if init.quantized else 0,
                              init.data))
        return out

    def close(self) -> None:
        m, self._mapping = self._mapping, None
        if m is not None:
            for init in self.initializers:
                init.data.release()
            self.nodes_raw.release()
            try:
                m.close()
            except BufferError:  # a caller still holds a view of a payload
                pass


def _parse_strings(view: memoryview) -> list:
    c = _Cursor(view)
    out = []
    for _ in range(c.u32()):
        n = c.u32()
        out.append(bytes(c.take(n)).decode("utf-8"))
    if not c.done():
        raise _invalid("strings section has trailing bytes")
    return out


def _parse_tensors(view: memoryview, strings: list, section_offset: int) -> list:
    # parse.zig:329-381
    c = _Cursor(view)
    out = []
    for _ in range(c.u32()):
        kind, plain_dtype, logical_dtype, _pad = c.u8(), c.u8(), c.u8(), c.u8()
        scheme_idx, block_elems, block_bytes, quant_axis = c.u32(), c.u32(), c.u32(), c.i32()
        params_len, data_len = c.u32(), c.u64()
        params = bytes(c.take(params_len))
        c.take(-c.pos % PAYLOAD_ALIGNMENT)  # the payload starts on a 64-byte boundary of the section
        file_offset = section_offset + c.pos
        data = c.take(data_len)
        if kind == 0:
            if plain_dtype >= len(DTYPE_NAMES):
                raise _invalid(f"dtype code {plain_dtype}")
            be, bb = DTYPE_BLOCK[plain_dtype]
            out.append(Initializer(False, plain_dtype, None, None, be, bb, 0, params, data, file_offset))
        elif kind == 1:
            if scheme_idx == INVALID_INDEX or scheme_idx >= len(strings):
                raise _invalid("quantized tensor without a scheme name")
            if logical_dtype >= len(DTYPE_NAMES):
                raise _invalid(f"logical dtype code {logical_dtype}")
            scheme = strings[scheme_idx]
            if scheme not in SCHEME_DTYPE:
                raise PackageError("UnsupportedFeature", f"quantization scheme {scheme!r}")
            dt = SCHEME_DTYPE[scheme]
            if (block_elems, block_bytes) != DTYPE_BLOCK[dt]:
                raise _invalid(f"{scheme} with blocks of {block_elems} elements in {block_bytes} bytes")
            if data_len % block_bytes != 0:
                raise _invalid("quantized payload is not a whole number of blocks")
            out.append(Initializer(True, dt, logical_dtype, scheme, block_elems, block_bytes, quant_axis, params, data, file_offset))
        else:
            raise _invalid(f"tensor encoding kind {kind}")
    if not c.done():
        raise _invalid("tensors section has trailing bytes")
    return out


def _parse_values(view: memoryview) -> list:
    # parse.zig:383-408, shape terms :827-836
    c = _Cursor(view)
    out = []
    for _ in range(c.u32()):
        dtype, rank, source, _pad = c.u8(), c.u8(), c.u8(), c.u8()
        if dtype >= len(DTYPE_NAMES) or source > 2:
            raise _invalid("value record")
        init_raw, terms = c.u32(), c.u32()
        shape = []
        for _ in range(terms):
            kind = c.u8()
            c.take(7)
            payload = c.u64()
            if kind == 0:
                shape.append(int(payload))
            elif kind == 1:
                shape.append(("expr", int(payload)))
            else:
                raise _invalid("shape term kind")
        out.append(ValueRecord(dtype, rank, source, shape, None if init_raw == INVALID_INDEX else init_raw))
    if not c.done():
        raise _invalid("values section has trailing bytes")
    return out


def _parse_named(c: _Cursor, strings: list, count: int) -> list:
    out = []
    for _ in range(count):
        idx = c.u32()
        if idx >= len(strings):
            raise _invalid("string index")
        out.append((strings[idx], c.u32()))
    return out


def parse(data: Union[bytes, bytearray, memoryview, mmap.mmap]) -> Package:
    """Decode a file image (parse.zig:51-158 for the sections read here)."""
    view = memoryview(data)
    if len(view) < HEADER_SIZE or bytes(view[0:4]) != MAGIC:
        raise _invalid("not an .aion file")
    version, section_count, _res, dir_offset, file_size, _flags = struct.unpack("<IIIQQQ", view[4:40])
    if version != VERSION:
        raise PackageError("UnsupportedVersion", f"file version {version}, this reader takes {VERSION}")
    if file_size != len(view):
        raise _invalid("header file size does not match the file")
    c = _Cursor(view, dir_offset)
    sections = {}
    seen_required = set()
    for _ in range(section_count):
        stype, flags, offset, size = c.u32(), c.u32(), c.u64(), c.u64()
        if offset > len(view) or size > len(view) - offset:
            raise _invalid("section outside the file")
        name = SECTIONS.get(stype)
        if name is None:
            if flags & SECTION_REQUIRED_FLAG:
                raise PackageError("UnsupportedFeature", f"required section of unknown type {stype}")
            continue
        if name in sections:
            raise _invalid(f"section {name} twice")
        sections[name] = (offset, size, flags)
        if flags & SECTION_REQUIRED_FLAG:
            seen_required.add(name)
    for name in REQUIRED:
        if name not in sections or name not in seen_required:
            raise _invalid(f"required section {name} is missing")

    def body(name):
        off, size, _ = sections[name]
        return view[off:off + size]

    strings = _parse_strings(body("strings"))
    t_off = sections["tensors"][0]
    if t_off % PAYLOAD_ALIGNMENT != 0:
        raise _invalid("tensors section is not 64-byte aligned")
    initializers = _parse_tensors(body("tensors"), strings, t_off)
    values = _parse_values(body("values"))
    sc = _Cursor(body("signatures"))
    n_in, n_out = sc.u32(), sc.u32()
    inputs = _parse_named(sc, strings, n_in)
    outputs = _parse_named(sc, strings, n_out)
    if not sc.done():
        raise _invalid("signatures section has trailing bytes")
    debug_names = {}
    if "debug_names" in sections:
        dc = _Cursor(body("debug_names"))
        for _ in range(dc.u32()):
            value, idx = dc.u32(), dc.u32()
            if idx >= len(strings):
                raise _invalid("string index")
            debug_names[value] = strings[idx]
        if not dc.done():
            raise _invalid("debug_names section has trailing bytes")
    metadata = {}
    if "metadata" in sections:
        mc = _Cursor(body("metadata"))
        for _ in range(mc.u32()):
            k, v = mc.u32(), mc.u32()
            if k >= len(strings) or v >= len(strings):
                raise _invalid("string index")
            metadata[strings[k]] = strings[v]
        if not mc.done():
            raise _invalid("metadata section has trailing bytes")
    # graph_meta repeats the counts (parse.zig:750-773, checked as in :211-224)
    gm = struct.unpack("<8I", body("graph_meta")[:32])
    if gm[0] != len(values) or gm[3] != len(initializers) or gm[4] != len(inputs) or gm[5] != len(outputs):
        raise _invalid("graph_meta counts do not match the sections")
    for vid, v in enumerate(values):
        if v.source == 1:
            if v.initializer_index is None or v.initializer_index >= len(initializers):
                raise _invalid(f"value {vid} names no initializer")
            init = initializers[v.initializer_index]
            if all(isinstance(d, int) for d in v.shape):
                n = 1
                for d in v.shape:
                    n *= d
                be, bb = init.block_elems, init.block_bytes
                if n % be != 0 or n // be * bb != len(init.data):
                    raise _invalid(f"value {vid}: payload of {len(init.data)} bytes does not hold shape {v.shape}")
    return Package(version, strings, initializers, values, inputs, outputs, debug_names, metadata, sections, body("nodes"))


def open_file(path: str) -> Package:
    """Map a file read-only and decode it; payload views stay valid until `Package.close()`."""
    with open(path, "rb") as f:
        m = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    try:
        pkg = parse(m)
    except Exception:
        m.close()
        raise
    pkg._mapping = m
    return pkg


def upload_weights(pkg: Package, store, select=None) -> dict:
    """Put the package's weights on the device: value id -> TensorId in `store` (a `DeviceStore`), each with
    the meta (dtype, shape, quant axis) the matmul steps read. `select(weight) -> bool` filters."""
    import numpy as np

    from .backend import TensorMeta

    out = {}
    for w in pkg.weights():
        if select is not None and not select(w):
            continue
        meta = TensorMeta(w.dtype, w.shape, quant_axis=w.quant_axis)
        out[w.value] = store.add(meta, np.frombuffer(w.data, dtype=np.uint8))
    return out
