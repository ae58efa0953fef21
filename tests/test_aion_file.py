"""The `.aion` v16 weights reader against files authored at test time (CPU), and a model's quantized weights
going from the file to the device and through the matmul step (GPU)."""
import struct

import numpy as np
import pytest

import oracle
from aion_b200 import aion_file
from tests import refdata as rd
from tests.aion_file_author import author

F32, Q4, Q8 = 0, 3, 4


def _model():
    k, n = 64, 24
    w = rd.synth_weights(k, n, seed=3)
    wt = np.ascontiguousarray(w.T)
    bias = np.arange(n, dtype=np.float32)
    return k, n, w, [
        {"name": "fc.weight.q8", "dtype": Q8, "shape": (k, n), "data": oracle.quantize(oracle.Q8_0, w, 0).tobytes(), "scheme": "q8_0", "quant_axis": 0},
        {"name": "fc.bias", "dtype": F32, "shape": (n,), "data": bias.tobytes()},
        {"name": "fc.weight.q4", "dtype": Q4, "shape": (k, n), "data": oracle.quantize(oracle.Q4_0, w, 0).tobytes(), "scheme": "q4_0", "quant_axis": 0},
        {"name": "head.weight", "dtype": Q8, "shape": (n, k), "data": oracle.quantize(oracle.Q8_0, wt, 1).tobytes(), "scheme": "q8_0", "quant_axis": 1},
    ]


def test_reads_what_was_written(tmp_path):
    k, n, w, tensors = _model()
    path = tmp_path / "tiny.aion"
    path.write_bytes(author(tensors, metadata={"arch": "test-tiny"}))
    pkg = aion_file.open_file(str(path))
    try:
        assert pkg.version == 16 and pkg.metadata == {"arch": "test-tiny"}
        ws = pkg.weights()
        assert [x.name for x in ws] == [t["name"] for t in tensors]
        for x, t in zip(ws, tensors):
            assert x.shape == tuple(t["shape"]) and x.dtype == t["dtype"] and bytes(x.data) == t["data"]
            assert x.quant_axis == t.get("quant_axis", 0)
        for init in pkg.initializers:
            assert init.file_offset % 64 == 0           # usable in place from a mapping
        q8 = pkg.initializers[0]
        assert (q8.scheme, q8.block_elems, q8.block_bytes, q8.quantized) == ("q8_0", 32, 34, True)
        # the payload is the reference quantizer's bytes: dequantized, it is the weight to q8 accuracy
        deq = oracle.dequant(oracle.Q8_0, np.frombuffer(ws[0].data, dtype=np.uint8)).reshape(k // 32, n, 32)
        assert np.max(np.abs(deq.transpose(0, 2, 1).reshape(k, n) - w)) < 0.02 / 127 * 6
    finally:
        pkg.close()


def test_rejects_what_the_reference_rejects():
    _, _, _, tensors = _model()
    good = author(tensors)
    aion_file.parse(good)
    with pytest.raises(aion_file.PackageError) as e:
        aion_file.parse(author(tensors, version=15))
    assert e.value.name == "UnsupportedVersion"
    with pytest.raises(aion_file.PackageError) as e:
        aion_file.parse(b"NOPE" + good[4:])
    assert e.value.name == "InvalidFormat"
    with pytest.raises(aion_file.PackageError) as e:
        aion_file.parse(good[:-1])                      # the header's file size no longer matches
    assert e.value.name == "InvalidFormat"
    with pytest.raises(aion_file.PackageError) as e:
        aion_file.parse(author(tensors, unknown_required_section=True))
    assert e.value.name == "UnsupportedFeature"
    bad = bytearray(good)
    struct.pack_into("<Q", bad, 72 + 24 + 8, len(good) + 1000)   # the tensors section's offset, outside the file
    with pytest.raises(aion_file.PackageError) as e:
        aion_file.parse(bytes(bad))
    assert e.value.name == "InvalidFormat"
    short = [dict(tensors[0], data=tensors[0]["data"][:-34])]   # a payload one block short of its shape
    with pytest.raises(aion_file.PackageError) as e:
        aion_file.parse(author(short))
    assert e.value.name == "InvalidFormat"
    with pytest.raises(aion_file.PackageError) as e:
        aion_file.parse(good[:60])                      # shorter than a header
    assert e.value.name == "InvalidFormat"


@pytest.mark.gpu
def test_weights_go_from_the_file_to_the_matmul_step(backend, tmp_path):
    from aion_b200.backend import DeviceStore, StepMatMul, StepMatMulNT, TensorMeta
    from aion_b200 import capi

    k, n, w, tensors = _model()
    path = tmp_path / "tiny.aion"
    path.write_bytes(author(tensors))
    pkg = aion_file.open_file(str(path))
    store = DeviceStore(backend.device_memory)
    try:
        ids = aion_file.upload_weights(pkg, store, select=lambda x: x.dtype in (Q4, Q8))
        by_name = {x.name: ids[x.value] for x in pkg.weights() if x.value in ids}
        x = rd.synth_acts(3, k)
        tx = store.add(TensorMeta(capi.DTYPE_F32, (3, k)), x)
        outs = {name: store.add(TensorMeta(capi.DTYPE_F32, (3, n))) for name in ("q8", "q4", "nt")}
        sess = backend.create_session(store)
        sess.execute([StepMatMul(c=outs["q8"], a=tx, b=by_name["fc.weight.q8"]), StepMatMul(c=outs["q4"], a=tx, b=by_name["fc.weight.q4"]),
                      StepMatMulNT(c=outs["nt"], a=tx, b=by_name["head.weight"])])
        assert rd.rel_l2(store.read(outs["q8"]), oracle.matmul_q(oracle.Q8_0, x, np.frombuffer(tensors[0]["data"], np.uint8), 3, n, k)) < 2e-5
        assert rd.rel_l2(store.read(outs["q4"]), oracle.matmul_q(oracle.Q4_0, x, np.frombuffer(tensors[2]["data"], np.uint8), 3, n, k)) < 2e-5
        assert rd.rel_l2(store.read(outs["nt"]), oracle.matmul_nt_q8(x, np.frombuffer(tensors[3]["data"], np.uint8), 3, n, k)) < 2e-5
    finally:
        store.deinit()
        pkg.close()
