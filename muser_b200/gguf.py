"""GGUF container parser and weight loader: the step in front of `Weight` (repack), mirroring the reference's

    crates/muser-engine/src/gguf/parser.rs:12-120     GgufFile::parse        -> GgufFile.parse / parse_path
    crates/muser-engine/src/gguf/metadata.rs:22-76    read_metadata_value    -> _read_value
    crates/muser-engine/src/gguf/types.rs:75-127      block_size / _elements -> BLOCK_BYTES / BLOCK_ELEMENTS
    crates/muser-engine/src/weights.rs:171-373        MuseWeights::{open, view, view_2d, layout, contains}

Same container rules and the same refusals: bounded counts, duplicate keys and tensor names rejected, alignment a
non-zero power of two (default 32), every tensor inside the file; NVFP4 tensors bind their companion tensors
`<name>.nvfp4_scale` (F8_E4M3FN [n_in/16, n_out], no NaN codes), `<name>.nvfp4_scale2` (scalar F32 > 0) and, when
the file says `muser.activation_precision = nvfp4`, `<name>.nvfp4_input_scale_inv`.  Views are zero-copy slices of
one memory map (the reference's ownership model); `MuseWeights.load` hands a view to the repack entry point and
returns the device image.
"""
from __future__ import annotations

import io
import mmap
import struct
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np

GGUF_MAGIC = 0x46554747  # "GGUF" little endian
MAX_METADATA_ITEMS, MAX_TENSORS, MAX_TENSOR_DIMS = 100_000, 1_000_000, 32
MAX_ARRAY_ITEMS, MAX_NESTING, MAX_STRING_BYTES = 1_000_000, 32, 16 * 1024 * 1024

NVFP4_SCALE_SUFFIX, NVFP4_SCALE2_SUFFIX, NVFP4_INPUT_SCALE_INV_SUFFIX = ".nvfp4_scale", ".nvfp4_scale2", ".nvfp4_input_scale_inv"

# GgmlType discriminants (gguf/types.rs:9-39) and their block geometry (types.rs:75-127)
F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 2, 3, 6, 7, 8, 10, 11, 12, 13, 14, 30
NVFP4_E2M1, F8_E4M3FN = 1000, 1001
BLOCK_BYTES = {F32: 4, F16: 2, Q4_0: 18, Q4_1: 20, Q5_0: 22, Q5_1: 24, Q8_0: 34, Q2_K: 84, Q3_K: 110, Q4_K: 144, Q5_K: 176,
               Q6_K: 210, 16: 66, 17: 74, 18: 98, 19: 50, 20: 18, 21: 110, 22: 82, 23: 136, 29: 56, BF16: 2, 138: 110,
               NVFP4_E2M1: 1, F8_E4M3FN: 1}
BLOCK_ELEMENTS = {t: 256 for t in BLOCK_BYTES}
BLOCK_ELEMENTS.update({F32: 1, F16: 1, BF16: 1, F8_E4M3FN: 1, NVFP4_E2M1: 2, Q4_0: 32, Q4_1: 32, Q5_0: 32, Q5_1: 32, Q8_0: 32, 20: 32})


class GgufError(ValueError):
    """`kind` carries the reference's GgufError variant name."""

    def __init__(self, kind: str, detail: str = ""):
        super().__init__(f"{kind}: {detail}" if detail else kind)
        self.kind = kind


class MuseConfigError(ValueError):
    def __init__(self, kind: str, detail: str = ""):
        super().__init__(f"{kind}: {detail}" if detail else kind)
        self.kind, self.detail = kind, detail


@dataclass
class TensorInfo:
    name: str
    shape: list
    dtype: int
    offset: int

    def byte_size(self) -> int:
        elements = max(1, int(np.prod(self.shape, dtype=object))) if self.shape else 1
        be = BLOCK_ELEMENTS[self.dtype]
        return (elements + be - 1) // be * BLOCK_BYTES[self.dtype]


@dataclass
class GgufFile:
    version: int
    metadata: dict = field(default_factory=dict)  # key -> (type tag, value)
    tensors: list = field(default_factory=list)
    data_offset: int = 0

    def meta_str(self, key: str):
        v = self.metadata.get(key)
        return v[1] if v and v[0] == 8 else None

    def meta_u32(self, key: str):
        v = self.metadata.get(key)
        return v[1] if v and v[0] == 4 else None

    @classmethod
    def parse_path(cls, path) -> "GgufFile":
        with open(path, "rb") as f:
            return cls.parse(f)

    @classmethod
    def parse(cls, r) -> "GgufFile":
        """Header, metadata and tensor descriptors of a seekable binary stream (no tensor data is read)."""
        start = r.tell()
        file_end = r.seek(0, io.SEEK_END)
        r.seek(start)
        magic = _u32(r)
        if magic != GGUF_MAGIC:
            raise GgufError("BadMagic", hex(magic))
        version = _u32(r)
        if not 2 <= version <= 3:
            raise GgufError("UnsupportedVersion", str(version))
        raw_tensors, raw_kv = _u64(r), _u64(r)
        _bounded(raw_tensors, MAX_TENSORS, "tensor entries")
        _bounded(raw_kv, MAX_METADATA_ITEMS, "metadata entries")
        _fits(r, file_end, raw_kv, 12, "metadata entries")
        metadata = {}
        for _ in range(raw_kv):
            key = _string(r)
            tag = _u32(r)
            value = _read_value(r, tag, 0)
            if key in metadata:
                raise GgufError("DuplicateMetadataKey", key)
            metadata[key] = (tag, value)
        _fits(r, file_end, raw_tensors, 24, "tensor entries")
        tensors, names = [], set()
        for _ in range(raw_tensors):
            name = _string(r)
            if name in names:
                raise GgufError("DuplicateTensorName", name)
            names.add(name)
            n_dims = _u32(r)
            _bounded(n_dims, MAX_TENSOR_DIMS, "tensor dimensions")
            shape = [_u64(r) for _ in range(n_dims)]
            dtype = _u32(r)
            if dtype not in BLOCK_BYTES:
                raise GgufError("UnsupportedType", str(dtype))
            tensors.append(TensorInfo(name, shape, dtype, _u64(r)))
        align = metadata.get("general.alignment")
        alignment = align[1] if align and align[0] == 4 else 32
        if alignment == 0 or alignment & (alignment - 1):
            raise GgufError("InvalidAlignment", str(alignment))
        data_offset = (r.tell() + alignment - 1) // alignment * alignment
        for t in tensors:
            if data_offset + t.offset + t.byte_size() > file_end:
                raise GgufError("TensorOutOfBounds", t.name)
        return cls(version, metadata, tensors, data_offset)


def _read(r, n: int) -> bytes:
    b = r.read(n)
    if len(b) != n:
        raise GgufError("Io", "unexpected end of file")
    return b


def _u32(r) -> int:
    return struct.unpack("<I", _read(r, 4))[0]


def _u64(r) -> int:
    return struct.unpack("<Q", _read(r, 8))[0]


def _string(r) -> str:
    n = _u64(r)
    if n > MAX_STRING_BYTES:
        raise GgufError("Io", "GGUF string exceeds the bounded parser limit")
    return _read(r, n).decode("utf-8")


def _bounded(raw: int, limit: int, what: str) -> None:
    if raw > limit:
        raise GgufError("LimitExceeded", f"{what}: {raw} > {limit}")


def _fits(r, file_end: int, count: int, bytes_per_item: int, what: str) -> None:
    remaining = max(0, file_end - r.tell())
    if count > remaining // bytes_per_item:
        raise GgufError("LimitExceeded", f"{what}: {count} cannot fit in the {remaining} bytes left")


_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 10: "<Q", 11: "<q", 12: "<d"}


def _read_value(r, tag: int, depth: int):
    if tag in _SCALARS:
        fmt = _SCALARS[tag]
        return struct.unpack(fmt, _read(r, struct.calcsize(fmt)))[0]
    if tag == 7:
        return _read(r, 1)[0] != 0
    if tag == 8:
        return _string(r)
    if tag == 9:
        if depth >= MAX_NESTING:
            raise GgufError("LimitExceeded", "metadata nesting")
        elem, n = _u32(r), _u64(r)
        _bounded(n, MAX_ARRAY_ITEMS, "metadata array items")
        return [_read_value(r, elem, depth + 1) for _ in range(n)]
    raise GgufError("UnsupportedMetadataType", str(tag))


@dataclass(frozen=True)
class TensorLayout:
    """weights.rs:45-61: where a tensor and its NVFP4 companions sit in the file."""
    file_offset: int
    byte_len: int
    dtype: int
    n_in: int
    n_out: int
    nvfp4_scale_offset: int | None
    nvfp4_scale_len: int
    nvfp4_scale2: float
    nvfp4_input_scale_inv: float | None


class MuseWeights:
    """Name -> zero-copy view over one read-only memory map of the model file (weights.rs:165-373)."""

    def __init__(self, path, gguf: GgufFile):
        self.path = Path(path)
        try:
            self._file = open(self.path, "rb")
            self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        except (OSError, ValueError) as e:
            raise MuseConfigError("Geometry", f"open {self.path}: {e}") from e
        self._bytes = np.frombuffer(self._map, dtype=np.uint8)
        self.index = {}
        for t in gguf.tensors:
            start, length = gguf.data_offset + t.offset, t.byte_size()
            if start + length > self._bytes.size:
                raise MuseConfigError("Geometry", f"tensor {t.name} runs past end of file ({start} + {length} > {self._bytes.size})")
            self.index[t.name] = (start, length, t.dtype, list(t.shape))
        precision = gguf.meta_str("muser.activation_precision") or "f16"
        if precision not in ("f16", "nvfp4"):
            raise MuseConfigError("Geometry", f"unsupported muser.activation_precision={precision}")
        for t in gguf.tensors:
            if t.dtype == NVFP4_E2M1:
                *_, isi = self._nvfp4_aux(t.name, t.shape)
                if (precision == "nvfp4") != (isi is not None):
                    raise MuseConfigError("Geometry", f"NVFP4 tensor {t.name} does not match muser.activation_precision={precision}")

    @classmethod
    def open(cls, path) -> "MuseWeights":
        return cls(path, GgufFile.parse_path(path))

    def close(self) -> None:
        self._bytes = None
        try:
            self._map.close()
        except BufferError:
            pass  # a view handed out earlier is still alive; the map goes when it does
        self._file.close()

    def contains(self, name: str) -> bool:
        return name in self.index

    def _entry(self, name: str):
        if name not in self.index:
            raise MuseConfigError("MissingTensor", name)
        return self.index[name]

    def _scalar_f32(self, name: str, what: str) -> float:
        start, length, dtype, shape = self.index[name]
        if dtype != F32 or shape != [1] or length != 4:
            raise MuseConfigError("Geometry", f"NVFP4 {what} {name} must be scalar F32")
        value = float(self._bytes[start:start + 4].view("<f4")[0])
        if not np.isfinite(value) or value <= 0.0:
            raise MuseConfigError("Geometry", f"NVFP4 {what} {name} must be finite and positive")
        return value

    def _nvfp4_aux(self, name: str, shape):
        n_in = shape[0] if len(shape) > 0 else 0
        n_out = shape[1] if len(shape) > 1 else 0
        if len(shape) != 2 or n_in == 0 or n_out == 0 or n_in % 16:
            raise MuseConfigError("Geometry", f"NVFP4 tensor {name} must be a nonempty 2-D matrix with n_in divisible by 16")
        s_start, s_len, s_dtype, s_shape = self._entry(name + NVFP4_SCALE_SUFFIX)
        if s_dtype != F8_E4M3FN or s_shape != [n_in // 16, n_out]:
            raise MuseConfigError("Geometry", f"NVFP4 scale tensor {name + NVFP4_SCALE_SUFFIX} must be F8_E4M3FN {[n_in // 16, n_out]}, got {s_dtype} {s_shape}")
        scales = self._bytes[s_start:s_start + s_len]
        if np.any((scales & 0x7F) == 0x7F):
            raise MuseConfigError("Geometry", f"NVFP4 scale tensor {name + NVFP4_SCALE_SUFFIX} contains E4M3FN NaN")
        self._entry(name + NVFP4_SCALE2_SUFFIX)
        scale2 = self._scalar_f32(name + NVFP4_SCALE2_SUFFIX, "tensor scale")
        isi_name = name + NVFP4_INPUT_SCALE_INV_SUFFIX
        isi = self._scalar_f32(isi_name, "activation scale") if isi_name in self.index else None
        return s_start, s_len, scale2, isi

    def view(self, name: str):
        """`TensorView` of one tensor (weights.rs:293-317): n_in = shape[0] (contiguous), n_out = shape[1]."""
        from .operator import TensorView
        start, length, dtype, shape = self._entry(name)
        n_in = shape[0] if len(shape) > 0 else 1
        n_out = shape[1] if len(shape) > 1 else 1
        raw = self._bytes[start:start + length]
        if dtype == NVFP4_E2M1:
            s_start, s_len, scale2, isi = self._nvfp4_aux(name, shape)
            return TensorView(raw.reshape(n_out, n_in // 2), dtype, n_in, n_out,
                              self._bytes[s_start:s_start + s_len].reshape(n_out, n_in // 16), scale2, isi)
        return TensorView(raw, dtype, n_in, n_out)

    def view_2d(self, name: str, n_in: int, n_out: int):
        """A tensor of any rank as a row-major [n_out][n_in] matrix, after checking its element count (weights.rs:327-348)."""
        *_, shape = self._entry(name)
        if int(np.prod(shape, dtype=object)) != n_in * n_out:
            raise MuseConfigError("Geometry", f"tensor {name} has shape {shape}, cannot reinterpret as [{n_in}, {n_out}]")
        v = self.view(name)
        v.n_in, v.n_out = n_in, n_out
        return v

    def layout(self, name: str) -> TensorLayout:
        start, length, dtype, shape = self._entry(name)
        if dtype == NVFP4_E2M1:
            s_off, s_len, scale2, isi = self._nvfp4_aux(name, shape)
        else:
            s_off, s_len, scale2, isi = None, 0, 1.0, None
        return TensorLayout(start, length, dtype, shape[0] if shape else 1, shape[1] if len(shape) > 1 else 1, s_off, s_len, scale2, isi)

    def load(self, ctx, name: str, shard=None):
        """The tensor as a repacked device image (`muser_cuda_weight_repack`), straight from the mapped file."""
        from .operator import Weight
        return Weight(ctx, self.view(name), shard=shard)


# ------------------------------------------------------------------------------------------ writer (fixtures, tools)
def write_gguf(path, tensors: dict, metadata: dict | None = None, alignment: int = 32, version: int = 3) -> None:
    """Writes a GGUF file: `tensors` maps name -> (dtype, shape, bytes-like), `metadata` key -> (type tag, value).
    The counterpart of the parser above, used to build loader fixtures; tensor data is aligned like llama.cpp does."""
    metadata = dict(metadata or {})
    if alignment != 32:
        metadata["general.alignment"] = (4, alignment)
    out = bytearray()
    out += struct.pack("<IIQQ", GGUF_MAGIC, version, len(tensors), len(metadata))

    def put_string(s: str):
        b = s.encode("utf-8")
        out.extend(struct.pack("<Q", len(b)))
        out.extend(b)

    def put_value(tag: int, value):
        if tag in _SCALARS:
            out.extend(struct.pack(_SCALARS[tag], value))
        elif tag == 7:
            out.append(1 if value else 0)
        elif tag == 8:
            put_string(value)
        elif tag == 9:
            elem, items = value
            out.extend(struct.pack("<IQ", elem, len(items)))
            for it in items:
                put_value(elem, it)
        else:
            raise GgufError("UnsupportedMetadataType", str(tag))

    for key, (tag, value) in metadata.items():
        put_string(key)
        out.extend(struct.pack("<I", tag))
        put_value(tag, value)
    offset, blobs = 0, []
    for name, (dtype, shape, data) in tensors.items():
        blob = bytes(memoryview(np.ascontiguousarray(data)).cast("B")) if not isinstance(data, (bytes, bytearray)) else bytes(data)
        put_string(name)
        out.extend(struct.pack("<I", len(shape)))
        for d in shape:
            out.extend(struct.pack("<Q", d))
        out.extend(struct.pack("<IQ", dtype, offset))
        blobs.append((offset, blob))
        offset = (offset + len(blob) + alignment - 1) // alignment * alignment
    out.extend(b"\0" * ((len(out) + alignment - 1) // alignment * alignment - len(out)))
    data_start = len(out)
    for off, blob in blobs:
        out.extend(b"\0" * (data_start + off - len(out)))
        out.extend(blob)
    Path(path).write_bytes(bytes(out))
