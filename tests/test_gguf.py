"""GGUF container: writer -> reader round trips (the reference's own test strategy for the format is a
write/read round trip, xn-core/tests/quantized_tests.rs), header versions, value types, alignment."""
import io
import struct

import numpy as np
import pytest

from xn_b200 import gguf, synth
from xn_b200.dtypes import GgmlDType as D
from xn_b200.quantized import QTensor


def _tensors():
    out = []
    for i, (dt, n, k) in enumerate([(D.Q4_0, 6, 64), (D.Q8_0, 5, 96), (D.Q4K, 4, 512), (D.Q6K, 3, 256)]):
        out.append((f"blk.{i}.weight", QTensor(synth.make_weight(dt, n, k, seed=60 + i), (n, k), dt)))
    return out


def test_round_trip_of_metadata_and_quantized_tensors(tmp_path):
    V = gguf.Value
    meta = [("general.architecture", V(gguf.STRING, "llama")), ("llama.block_count", V(gguf.U32, 32)), ("a.u8", V(gguf.U8, 200)),
            ("a.i8", V(gguf.I8, -5)), ("a.u16", V(gguf.U16, 65535)), ("a.i16", V(gguf.I16, -300)), ("a.i32", V(gguf.I32, -7)),
            ("a.f32", V(gguf.F32, 0.5)), ("a.bool", V(gguf.BOOL, True)), ("a.u64", V(gguf.U64, 2 ** 40)), ("a.i64", V(gguf.I64, -2 ** 40)),
            ("a.f64", V(gguf.F64, 1e-300)), ("tokens", V(gguf.ARRAY, [V(gguf.STRING, "a"), V(gguf.STRING, "bc")])),
            ("nested", V(gguf.ARRAY, [V(gguf.ARRAY, [V(gguf.I32, 1), V(gguf.I32, 2)])]))]
    tensors = _tensors()
    path = tmp_path / "model.gguf"
    with open(path, "wb") as f:
        gguf.write(f, meta, tensors)
    c = gguf.Content.read(str(path))                   # memory-mapped
    assert c.version == 3 and c.tensor_data_offset % 32 == 0
    assert {k: v for k, v in c.metadata.items()} == dict(meta)
    for name, t in tensors:
        info = c.tensor_infos[name]
        assert info.ggml_dtype == t.dtype() and info.shape == tuple(t.shape()) and info.offset % 32 == 0
        back = c.tensor(name)
        assert np.array_equal(back.data(), t.data()) and back.shape() == t.shape()
        n, k = t.shape()
        rows = c.tensor_bytes(name, 1, 2)              # a row range is a view of the same bytes
        rb = t.dtype().row_bytes(k)
        assert np.array_equal(rows, np.asarray(t.data()).reshape(-1)[rb:3 * rb])
    with pytest.raises(KeyError, match="cannot find tensor info"):
        c.tensor("missing")
    with pytest.raises(ValueError):
        c.tensor_bytes(tensors[0][0], 5, 4)


def _v1_file():
    """Version 1: 32-bit counts, string lengths and dimensions."""
    name, key, sval = b"w", b"general.name", b"tiny\0"
    blocks = synth.make_weight(D.Q8_0, 2, 32, seed=1)
    b = struct.pack("<IIII", 0x46554747, 1, 1, 1)
    b += struct.pack("<I", len(key)) + key + struct.pack("<II", gguf.STRING, len(sval)) + sval
    b += struct.pack("<I", len(name)) + name + struct.pack("<III", 2, 32, 2) + struct.pack("<IQ", int(D.Q8_0), 0)
    b += b"\0" * (-len(b) % 32)
    return b + np.asarray(blocks).tobytes(), blocks


def test_version_1_header_and_trailing_nul_in_strings():
    raw, blocks = _v1_file()
    c = gguf.Content.read(raw)
    assert c.version == 1 and c.metadata["general.name"].value == "tiny"      # the NUL is dropped
    assert c.tensor_infos["w"].shape == (2, 32)                              # stored innermost first
    assert np.array_equal(c.tensor_bytes("w"), np.asarray(blocks).reshape(-1))


def test_alignment_key_bad_magic_and_bad_version():
    V = gguf.Value
    f = io.BytesIO()
    gguf.write(f, [("general.alignment", V(gguf.U32, 32))], _tensors()[:1])
    assert gguf.Content.read(f.getvalue()).tensor_data_offset % 32 == 0
    with pytest.raises(ValueError, match="unknown magic"):
        gguf.Content.read(b"GGML" + b"\0" * 32)
    with pytest.raises(ValueError, match="unsupported magic/version"):
        gguf.Content.read(struct.pack("<II", 0x46554747, 9) + b"\0" * 32)
    with pytest.raises(ValueError, match="empty array"):
        gguf.write(io.BytesIO(), [("x", V(gguf.ARRAY, []))], [])
    bad = gguf.TensorInfo(D.Q4K, (3, 100), 0)
    with pytest.raises(ValueError, match="not divisible by the block size"):
        bad.nbytes()
