"""GGUF tensor directory reader and the weights view that hands tensors to the backend.

Host-side mirror of the reference's loader for this path: `gguf.parse`
(inference/src/formats/gguf.zig:305-412) and `weights.View`
(inference/src/runtime/weights.zig:8-31). Only what the matmul path needs is kept:
the header, the metadata keys (values of scalar and string kinds; arrays are skipped
with their length recorded), the tensor directory with the reference's checks, and
views of a tensor's bytes as a `Matrix` or an `ExpertMatrix`.

Rules restated from the reference, with the same error names:
  * magic "GGUF" (0x46554747 little endian), version 3 only (gguf.zig:316-318);
  * `general.alignment` must be a `uint32` power of two, default 32 (gguf.zig:325-337);
  * a tensor has rank 1..4, no zero dimension, a known encoding, and an offset that is a
    multiple of the alignment (gguf.zig:347-372); its byte length follows from the block
    layout: dimension 0 (the columns) must be a whole number of blocks (encoding.zig:15-24);
  * the data section starts at the directory's end rounded up to the alignment
    (gguf.zig:382-384); tensors must lie inside the file and must not overlap (gguf.zig:389-398);
  * GGUF dimension 0 is the column count K, dimension 1 the row count N, dimension 2 the
    expert count (weights.zig:16-30).

The file is memory-mapped read-only; tensor bytes are views of the mapping (no copy until
`Backend.wrap` uploads them).
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass, field

import numpy as np

from . import encoding as enc
from .backend import Backend, Buffer, ExpertMatrix, Matrix

MAGIC = 0x46554747
# GGUF metadata value kinds (gguf.zig:21-39)
UINT8, INT8, UINT16, INT16, UINT32, INT32, FLOAT32, BOOL, STRING, ARRAY, UINT64, INT64, FLOAT64 = range(13)
_SCALAR = {UINT8: "<B", INT8: "<b", UINT16: "<H", INT16: "<h", UINT32: "<I", INT32: "<i", FLOAT32: "<f", UINT64: "<Q", INT64: "<q", FLOAT64: "<d"}


class GgufError(ValueError):
    """A rejected file; `name` is the reference's error name (gguf.zig:156-172)."""

    def __init__(self, name: str, detail: str = ""):
        super().__init__(f"{name}: {detail}" if detail else name)
        self.name = name


@dataclass
class Tensor:
    name: str
    dimensions: tuple[int, ...]
    encoding_id: int
    offset: int      # relative to Document.data_offset
    bytes: int
    elements: int


@dataclass
class Document:
    version: int
    file_bytes: int
    directory_bytes: int
    data_offset: int
    alignment: int
    metadata: dict = field(default_factory=dict)
    tensors: list[Tensor] = field(default_factory=list)

    def tensor(self, name: str) -> Tensor:
        for t in self.tensors:
            if t.name == name:
                return t
        raise KeyError(name)


class _Cursor:
    def __init__(self, data, limit: int):
        self.data, self.pos, self.limit = data, 0, limit

    def take(self, n: int) -> bytes:
        if n < 0 or self.pos + n > self.limit:
            raise GgufError("EndOfStream", f"needs {n} bytes at {self.pos}")
        out = self.data[self.pos:self.pos + n]
        self.pos += n
        return out

    def int(self, fmt: str):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def string(self) -> str:
        n = self.int("<Q")
        if n > 1 << 20:
            raise GgufError("LimitExceeded", "string longer than 1 MiB")
        return bytes(self.take(n)).decode("utf-8", errors="strict")

    def value(self, kind: int):
        if kind in _SCALAR:
            return self.int(_SCALAR[kind])
        if kind == BOOL:
            b = self.int("<B")
            if b > 1:
                raise GgufError("InvalidBoolean")
            return bool(b)
        if kind == STRING:
            return self.string()
        if kind == ARRAY:
            item = self.int("<I")
            count = self.int("<Q")
            if item == ARRAY:
                raise GgufError("UnsupportedNestedArray")
            if item in _SCALAR or item == BOOL:
                self.take(count * (1 if item == BOOL else struct.calcsize(_SCALAR[item])))
            elif item == STRING:
                for _ in range(count):
                    self.take(self.int("<Q"))
            else:
                raise GgufError("InvalidMetadataType", f"array of kind {item}")
            return ("array", item, count)
        raise GgufError("InvalidMetadataType", f"kind {kind}")


def tensor_bytes(encoding_id: int, dimensions) -> int:
    """`Layout.byteCount` (encoding.zig:15-24): dimension 0 in whole blocks, times the other dimensions."""
    try:
        _, elements, size = enc.layout(encoding_id)
    except Exception:
        raise GgufError("UnsupportedTensorType", f"encoding {encoding_id}")
    if dimensions[0] % elements != 0:
        raise GgufError("InvalidShape", f"{dimensions[0]} columns are no whole number of {elements}-element blocks")
    total = dimensions[0] // elements * size
    for d in dimensions[1:]:
        total *= d
    if total >= 1 << 63:
        raise GgufError("Overflow")
    return total


def parse(data, file_bytes: int | None = None, max_tensors: int = 1 << 20, max_metadata: int = 1 << 20) -> Document:
    """Parses the directory of a GGUF image (`bytes`, `mmap` or a uint8 array) with the reference's checks."""
    file_bytes = len(data) if file_bytes is None else file_bytes
    c = _Cursor(data, file_bytes)
    if c.int("<I") != MAGIC:
        raise GgufError("InvalidMagic")
    version = c.int("<I")
    if version != 3:
        raise GgufError("UnsupportedVersion", str(version))
    tensor_count, metadata_count = c.int("<Q"), c.int("<Q")
    if tensor_count > max_tensors or metadata_count > max_metadata:
        raise GgufError("LimitExceeded")
    metadata, alignment = {}, 32
    for _ in range(metadata_count):
        key = c.string()
        if not key or len(key) > 65535:
            raise GgufError("InvalidName")
        if key in metadata:
            raise GgufError("DuplicateMetadata", key)
        kind = c.int("<I")
        value = c.value(kind)
        metadata[key] = value
        if key == "general.alignment":
            if kind != UINT32 or value == 0 or value & (value - 1):
                raise GgufError("InvalidAlignment", str(value))
            alignment = value
    tensors, names = [], set()
    for _ in range(tensor_count):
        name = c.string()
        if not name or len(name) > 65535:
            raise GgufError("InvalidName")
        if name in names:
            raise GgufError("DuplicateTensor", name)
        names.add(name)
        rank = c.int("<I")
        if rank == 0 or rank > 4:
            raise GgufError("InvalidShape", f"{name}: rank {rank}")
        dims = tuple(c.int("<Q") for _ in range(rank))
        encoding_id = c.int("<I")
        elements = 1
        for d in dims:
            if d == 0:
                raise GgufError("InvalidShape", f"{name}: zero dimension")
            elements *= d
            if elements >= 1 << 64:
                raise GgufError("Overflow", name)
        nbytes = tensor_bytes(encoding_id, dims)
        offset = c.int("<Q")
        if offset % alignment != 0:
            raise GgufError("InvalidAlignment", f"{name}: offset {offset}")
        tensors.append(Tensor(name, dims, encoding_id, offset, nbytes, elements))
    data_offset = c.pos + (alignment - c.pos % alignment) % alignment
    if data_offset > file_bytes:
        raise GgufError("EndOfStream")
    previous_end = 0
    for t in sorted(tensors, key=lambda t: t.offset):
        if t.offset > file_bytes - data_offset or t.bytes > file_bytes - data_offset - t.offset:
            raise GgufError("TensorOutOfBounds", t.name)
        if t.offset < previous_end:
            raise GgufError("OverlappingTensors", t.name)
        previous_end = t.offset + t.bytes
    return Document(version, file_bytes, c.pos, data_offset, alignment, metadata, tensors)


class View:
    """`weights.View`: a mapped file and its directory; tensors as borrowed byte ranges and matrices."""

    def __init__(self, path: str):
        self._file = open(path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        self.document = parse(self._map)
        self._bytes = np.frombuffer(self._map, dtype=np.uint8)

    def close(self) -> None:
        self._bytes = None
        try:
            self._map.close()
        except BufferError:
            pass  # a caller still holds a view of the mapping; the mapping goes with it
        self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def bytes(self, tensor: Tensor) -> np.ndarray:
        start = self.document.data_offset + tensor.offset
        if start > self._bytes.size or tensor.bytes > self._bytes.size - start:
            raise GgufError("TensorOutOfBounds", tensor.name)
        return self._bytes[start:start + tensor.bytes]

    def matrix(self, tensor: Tensor) -> tuple[Matrix, np.ndarray]:
        """A 2-D tensor as `[rows][columns]` (GGUF dimensions `[columns, rows]`) and its bytes."""
        if len(tensor.dimensions) != 2:
            raise GgufError("InvalidShape", f"{tensor.name}: rank {len(tensor.dimensions)}")
        data = self.bytes(tensor)
        return Matrix(tensor.encoding_id, tensor.dimensions[1], tensor.dimensions[0], data.size), data

    def expert_matrix(self, tensor: Tensor) -> tuple[ExpertMatrix, np.ndarray]:
        """A 3-D tensor `[experts][rows][columns]` (GGUF dimensions `[columns, rows, experts]`)."""
        if len(tensor.dimensions) != 3:
            raise GgufError("InvalidShape", f"{tensor.name}: rank {len(tensor.dimensions)}")
        data = self.bytes(tensor)
        return ExpertMatrix(tensor.encoding_id, tensor.dimensions[2], tensor.dimensions[1], tensor.dimensions[0], data.size), data

    def upload(self, backend: Backend, tensor: Tensor, prepare: bool | str = True) -> tuple[Buffer, Matrix]:
        """Wraps a 2-D tensor into device memory (uploaded once, cached by address, as `Backend.wrap` does) and, for
        the encodings whose GGUF rows the specialized kernels cannot address (Q6_K, Q8_0, Q5_0, Q5_1, Q4_0, IQ4_NL, IQ4_XS, Q2_K, Q3_K), re-lays it planar.
        ``prepare="host"`` re-lays on the host instead (`planar.relay`: the same bytes) and uploads the result: the device
        then never holds the tensor twice, which matters for a model that fills the memory."""
        m, data = self.matrix(tensor)
        if prepare == "host":
            from . import planar
            laid, layout = planar.relay(m.encoding, data, m.rows, m.columns)
            buf = backend.create(laid.size)
            buf.write(laid)
            return buf, Matrix(m.encoding, m.rows, m.columns, m.bytes, layout)
        buf = backend.wrap(data)
        if prepare and m.encoding in (enc.Q6_K, enc.Q8_0, enc.Q5_0, enc.Q5_1, enc.Q4_0, enc.IQ4_NL, enc.IQ4_XS, enc.Q2_K, enc.Q3_K) and m.rows % 16 == 0 and m.columns % 256 == 0:
            planar, m = backend.prepare(buf, m)
            backend.unwrap(data)
            buf = planar
        return buf, m


def write(path: str, tensors: list[tuple[str, tuple[int, ...], int, np.ndarray]], metadata: dict | None = None, alignment: int = 32) -> None:
    """Writes a GGUF v3 file (fixtures and synthetic models): tensors as (name, GGUF dimensions, encoding, bytes).
    Metadata values may be int (uint32), float (float32), bool or str."""
    meta = dict(metadata or {})
    alignment = meta.setdefault("general.alignment", alignment)

    def s(text: str) -> bytes:
        raw = text.encode("utf-8")
        return struct.pack("<Q", len(raw)) + raw

    head = struct.pack("<IIQQ", MAGIC, 3, len(tensors), len(meta))
    for key, value in meta.items():
        head += s(key)
        if isinstance(value, bool):
            head += struct.pack("<IB", BOOL, int(value))
        elif isinstance(value, int):
            head += struct.pack("<II", UINT32, value)
        elif isinstance(value, float):
            head += struct.pack("<If", FLOAT32, value)
        else:
            head += struct.pack("<I", STRING) + s(str(value))
    offsets, cursor = [], 0
    for name, dims, encoding_id, data in tensors:
        if tensor_bytes(encoding_id, dims) != data.size:
            raise GgufError("InvalidShape", f"{name}: {data.size} bytes for dimensions {dims}")
        offsets.append(cursor)
        cursor += data.size
        cursor += (alignment - cursor % alignment) % alignment
    for (name, dims, encoding_id, data), offset in zip(tensors, offsets):
        head += s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", encoding_id, offset)
    head += b"\0" * ((alignment - len(head) % alignment) % alignment)
    with open(path, "wb") as f:
        f.write(head)
        for (name, dims, encoding_id, data), offset in zip(tensors, offsets):
            f.write(np.ascontiguousarray(data, dtype=np.uint8).tobytes())
            f.write(b"\0" * ((alignment - data.size % alignment) % alignment))
