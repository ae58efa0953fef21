"""Authors a tiny `.aion` v16 file for the reader's tests, the way the reference's own Python tests build
their models at test time (bindings/python/tests/conftest.py:1-73) — there through the reference's
`Builder`, which needs its Zig runtime; here by laying the sections out by hand exactly as its writer does
(src/aion/storage/aion_file/write.zig:36-91, 607-625). Test infrastructure only."""
import struct

ALIGN = 64
REQUIRED = 1


def _strings(table):
    out = struct.pack("<I", len(table))
    for s in table:
        b = s.encode()
        out += struct.pack("<I", len(b)) + b
    return out


def author(tensors, metadata=None, version=16, unknown_required_section=False):
    """tensors: list of dicts {name, dtype (code), shape, data (bytes), scheme (None | "q8_0" | "q4_0"), quant_axis}.
    Every tensor becomes an initializer backing one value; there are no nodes, inputs or outputs. Returns bytes."""
    metadata = metadata or {}
    table = []

    def intern(s):
        if s not in table:
            table.append(s)
        return table.index(s)

    for t in tensors:
        intern(t["name"])
        if t.get("scheme"):
            intern(t["scheme"])
    for k, v in metadata.items():
        intern(k), intern(v)

    # tensors section: a 36-byte record, params, zero padding to 64, payload (write.zig:100-140)
    tsec = struct.pack("<I", len(tensors))
    for t in tensors:
        q = t.get("scheme")
        be, bb = {None: (0, 0), "q8_0": (32, 34), "q4_0": (32, 18)}[q]
        tsec += struct.pack("<BBBBIIIiIQ", 1 if q else 0, 0 if q else t["dtype"], 0, 0, intern(q) if q else 0xFFFFFFFF, be, bb,
                            t.get("quant_axis", 0) if q else 0, 0, len(t["data"]))
        tsec += b"\0" * (-len(tsec) % ALIGN)
        tsec += bytes(t["data"])
    vsec = struct.pack("<I", len(tensors))
    for i, t in enumerate(tensors):
        vsec += struct.pack("<BBBBII", t["dtype"], len(t["shape"]), 1, 0, i, len(t["shape"]))
        for d in t["shape"]:
            vsec += struct.pack("<B7xQ", 0, d)
    nsec = struct.pack("<I", 0)
    ssec = struct.pack("<II", 0, 0)
    msec = struct.pack("<I", len(metadata)) + b"".join(struct.pack("<II", intern(k), intern(v)) for k, v in metadata.items())
    dsec = struct.pack("<I", len(tensors)) + b"".join(struct.pack("<II", i, intern(t["name"])) for i, t in enumerate(tensors))
    gsec = struct.pack("<11I", len(tensors), 0, 0, len(tensors), 0, 0, 0, 0, len(metadata), len(tensors), 0)
    sections = [(1, REQUIRED, _strings(table)), (2, REQUIRED, tsec), (3, REQUIRED, vsec), (4, REQUIRED, nsec), (5, REQUIRED, ssec),
                (6, REQUIRED, gsec), (9, 0, msec), (10, 0, dsec)]
    if unknown_required_section:
        sections.append((77, REQUIRED, b"xyz"))
    at = 72 + 24 * len(sections)
    offsets = []
    for stype, _, body in sections:
        if stype == 2:
            at += -at % ALIGN
        offsets.append(at)
        at += len(body)
    out = bytearray(b"AION" + struct.pack("<IIIQQQ", version, len(sections), 0, 72, at, 0) + b"\0" * 32)
    for (stype, flags, body), off in zip(sections, offsets):
        out += struct.pack("<IIQQ", stype, flags, off, len(body))
    for (_, _, body), off in zip(sections, offsets):
        out += b"\0" * (off - len(out))
        out += body
    assert len(out) == at
    return bytes(out)
