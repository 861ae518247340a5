"""GGUF files in and out of device weight handles.

Reader and writer for the container the quantized weights come in
(xn-core/src/quantized/gguf_file.rs:57-76 tensor read, 389-453 header, 493-541 writer): versions 1-3,
all thirteen metadata value types, dimensions stored innermost-first, tensor data aligned to
``general.alignment`` (default 32). The reference reads every tensor into a fresh host ``Vec``, re-wraps
it per dtype (``ggml_file.rs:114-126``) and, for CUDA, splits it again on the host (``q8.rs:78-85``).
Here the file is memory-mapped, a tensor is a zero-copy view of the mapping, and an N-shard is uploaded
from the byte range of its rows only, so a rank never touches the rows it does not hold.
"""
from __future__ import annotations

import dataclasses
import mmap
import struct
from typing import Any, BinaryIO, Iterable, Optional, Union

import numpy as np

from .dtypes import GgmlDType

DEFAULT_ALIGNMENT = 32
_MAGICS = (0x46554747, 0x47475546)

# value type ids (gguf_file.rs:349-386)
U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
_SCALAR = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}


@dataclasses.dataclass
class Value:
    """A typed metadata value; arrays hold a list of ``Value`` of one type."""
    type: int
    value: Any

    def __post_init__(self):
        if self.type == ARRAY and any(not isinstance(v, Value) for v in self.value):
            raise TypeError("an ARRAY holds Value items")


@dataclasses.dataclass
class TensorInfo:
    ggml_dtype: GgmlDType
    shape: tuple[int, ...]   # outermost first, the way xn's Shape holds it
    offset: int              # from the start of the tensor-data section

    def nbytes(self) -> int:
        elems = int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1
        bs = self.ggml_dtype.block_size
        if elems % bs:
            raise ValueError(f"the number of elements {elems} is not divisible by the block size {bs}")  # gguf_file.rs:63-68
        return elems // bs * self.ggml_dtype.type_size


class _Reader:
    def __init__(self, buf, version_hint: int = 3):
        self.buf, self.pos, self.version = buf, 0, version_hint

    def take(self, fmt: str):
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += struct.calcsize(fmt)
        return v

    def length(self) -> int:
        return self.take("<I") if self.version == 1 else self.take("<Q")

    def string(self) -> str:
        n = self.length()
        raw = bytes(self.buf[self.pos:self.pos + n])
        if len(raw) != n:
            raise ValueError("gguf: truncated string")
        self.pos += n
        return raw.rstrip(b"\0").decode("utf-8", "replace")   # trailing NULs and invalid utf-8 occur in the wild (gguf_file.rs:95-101)

    def value(self, vtype: int) -> Value:
        if vtype in _SCALAR:
            v = self.take(_SCALAR[vtype])
            if vtype == BOOL:
                if v not in (0, 1):
                    raise ValueError(f"gguf: unexpected bool value {v}")
                v = bool(v)
            return Value(vtype, v)
        if vtype == STRING:
            return Value(STRING, self.string())
        if vtype == ARRAY:
            item_type = self.take("<I")
            n = self.length()
            return Value(ARRAY, [self.value(item_type) for _ in range(n)])
        raise ValueError(f"unrecognized value-type {vtype:#08x}")


class Content:
    """The parsed header of a GGUF file plus access to its tensors (``gguf_file.rs`` ``Content``)."""

    def __init__(self, version: int, metadata: dict[str, Value], tensor_infos: dict[str, TensorInfo], tensor_data_offset: int, buf):
        self.version, self.metadata, self.tensor_infos, self.tensor_data_offset = version, metadata, tensor_infos, tensor_data_offset
        self._buf = buf

    # -- reading ---------------------------------------------------------------------------------
    @classmethod
    def read(cls, source: Union[str, bytes, bytearray, memoryview]) -> "Content":
        """``source`` is a path (memory-mapped, read-only) or the bytes of a file."""
        if isinstance(source, str):
            with open(source, "rb") as f:
                buf = memoryview(mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ))
        else:
            buf = memoryview(source)
        r = _Reader(buf)
        magic = r.take("<I")
        if magic not in _MAGICS:
            raise ValueError(f"unknown magic 0x{magic:08x}")
        version = r.take("<I")
        if version not in (1, 2, 3):
            raise ValueError(f"gguf: unsupported magic/version Gguf/{version}")
        r.version = version
        tensor_count, kv_count = r.length(), r.length()
        metadata = {}
        for _ in range(kv_count):
            key = r.string()
            metadata[key] = r.value(r.take("<I"))
        infos = {}
        for _ in range(tensor_count):
            name = r.string()
            nd = r.take("<I")
            dims = [r.take("<I") if version == 1 else r.take("<Q") for _ in range(nd)]
            dtype = GgmlDType(r.take("<I"))
            infos[name] = TensorInfo(dtype, tuple(reversed(dims)), r.take("<Q"))
        a = metadata.get("general.alignment")
        alignment = a.value if a is not None and a.type in (U8, U16, U32, I8, I16, I32) and a.value >= 0 else DEFAULT_ALIGNMENT
        data_offset = -(-r.pos // alignment) * alignment if alignment else r.pos
        return cls(version, metadata, infos, data_offset, buf)

    def _info(self, name: str) -> TensorInfo:
        if name not in self.tensor_infos:
            raise KeyError(f"cannot find tensor info for {name}")   # gguf_file.rs:478-481
        return self.tensor_infos[name]

    def tensor_bytes(self, name: str, row0: int = 0, n_rows: Optional[int] = None) -> np.ndarray:
        """A zero-copy uint8 view of a tensor's blocks (or of rows ``[row0, row0 + n_rows)`` of a 2-d tensor)."""
        info = self._info(name)
        start, nbytes = self.tensor_data_offset + info.offset, info.nbytes()
        if n_rows is not None or row0:
            if len(info.shape) != 2:
                raise ValueError(f"row ranges need a 2-d tensor, {name} is {info.shape}")
            n, k = info.shape
            n_rows = n - row0 if n_rows is None else n_rows
            if row0 < 0 or n_rows < 0 or row0 + n_rows > n:
                raise ValueError(f"rows [{row0}, {row0 + n_rows}) are outside {name} with {n} rows")
            rb = info.ggml_dtype.row_bytes(k)
            start, nbytes = start + row0 * rb, n_rows * rb
        if start + nbytes > len(self._buf):
            raise ValueError(f"gguf: tensor {name} runs past the end of the file")
        return np.frombuffer(self._buf, np.uint8, nbytes, start)

    def tensor(self, name: str):
        """The tensor as a host ``QTensor`` (``Content::tensor``, gguf_file.rs:473-483)."""
        from .quantized import QTensor
        info = self._info(name)
        return QTensor(self.tensor_bytes(name), info.shape, info.ggml_dtype)

    def upload(self, name: str, device="cuda:0", shard_rank: int = 0, shard_count: int = 1):
        """A 2-d quantized tensor straight from the mapping to the device; with ``shard_count > 1`` only the
        rank's rows are read from the file."""
        from .parallel import shard_rows
        from .quantized import QCudaTensor
        info = self._info(name)
        if len(info.shape) != 2:
            raise ValueError(f"cuda quantized: expected a 2-d weight, got shape {info.shape}")
        n, k = info.shape
        r0, r1 = shard_rows(n, shard_rank, shard_count)
        return QCudaTensor.from_rows(info.ggml_dtype, self.tensor_bytes(name, r0, r1 - r0), n, k, r0, r1 - r0, device)


def _write_string(w: BinaryIO, s: str) -> None:
    b = s.encode("utf-8")
    w.write(struct.pack("<Q", len(b)))
    w.write(b)


def _write_value(w: BinaryIO, v: Value) -> None:
    if v.type in _SCALAR:
        w.write(struct.pack(_SCALAR[v.type], int(v.value) if v.type == BOOL else v.value))
    elif v.type == STRING:
        _write_string(w, v.value)
    elif v.type == ARRAY:
        if not v.value:
            raise ValueError("gguf: an empty array has no element type to write")   # gguf_file.rs:326-333
        item = v.value[0].type
        if any(e.type != item for e in v.value):
            raise ValueError("gguf: array elements of different types")
        w.write(struct.pack("<IQ", item, len(v.value)))
        for e in v.value:
            _write_value(w, e)
    else:
        raise ValueError(f"unrecognized value-type {v.type:#08x}")


def write(w: BinaryIO, metadata: Iterable[tuple[str, Value]], tensors: Iterable[tuple[str, Any]]) -> None:
    """Version-3 file (``gguf_file.rs:493-541``). A tensor is anything with ``dtype()``, ``shape()`` and ``data()``
    (canonical block bytes): a host ``QTensor`` or a device ``QCudaTensor``, whose blocks come back from the
    device in GGUF order whatever its device layout."""
    metadata, tensors = list(metadata), list(tensors)
    w.write(struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(metadata)))
    for key, value in metadata:
        _write_string(w, key)
        w.write(struct.pack("<I", value.type))
        _write_value(w, value)
    offset, blobs = 0, []
    for name, t in tensors:
        data = np.ascontiguousarray(t.data()).view(np.uint8).reshape(-1)
        _write_string(w, name)
        dims = tuple(t.shape())
        w.write(struct.pack("<I", len(dims)))
        for d in reversed(dims):
            w.write(struct.pack("<Q", d))
        w.write(struct.pack("<IQ", int(t.dtype()), offset))
        blobs.append(data)
        offset += -(-data.size // DEFAULT_ALIGNMENT) * DEFAULT_ALIGNMENT
    w.write(b"\0" * (-w.tell() % DEFAULT_ALIGNMENT))
    for data in blobs:
        w.write(data.tobytes())
        w.write(b"\0" * (-data.size % DEFAULT_ALIGNMENT))
