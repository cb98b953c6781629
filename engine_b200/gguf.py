"""GGUF v3 files over the C ABI: the directory reader and the staged upload of encoded tensors.

Host-side mirror of `GgufFile`, `TensorInfo` and `TensorDataReader` (crates/gguf/src/lib.rs:87-505 of the reference
project) and of `CudaWeightStore::materialize_quantized` (crates/nvidia/src/cuda.rs:321-387).  Parsing, bounds and
error classes live in libribn_b200.so (csrc/gguf.cu); this file only shapes them into the reference's object model.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from . import _lib
from .sharding import split_even

# ribn_gguf_status -> the reference's GgufError variant
ERROR_KINDS = {
    100: "Io", 101: "InvalidMagic", 102: "UnsupportedVersion", 103: "UnexpectedEof", 104: "InvalidUtf8", 105: "InvalidValueType",
    106: "InvalidBool", 107: "InvalidLength", 108: "ArrayNestingTooDeep", 109: "DuplicateMetadata", 110: "InvalidDimensionCount",
    111: "InvalidAlignment", 112: "Truncated", 113: "TensorOffsetOutOfBounds", 114: "MissingMetadata", 115: "MetadataTypeMismatch",
    116: "MissingTensor", 117: "UnsupportedTensorType", 118: "ElementCountOverflow", 119: "TensorByteLengthOverflow",
    120: "QuantizationBlockMismatch", 121: "QuantizationDimensionMismatch",
    _lib.RIBN_E_INVALID_WEIGHT: "InvalidWeight", _lib.RIBN_E_OUTPUT_LENGTH: "OutputLength", _lib.RIBN_E_INVALID_ARGUMENT: "InvalidArgument",
    _lib.RIBN_E_DRIVER: "Driver",
}


class GgufError(Exception):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status
        self.kind = ERROR_KINDS.get(status, f"status {status}")


@dataclass(frozen=True)
class TensorInfo:
    """lib.rs:87-118."""

    name: str
    dimensions: tuple[int, ...]
    value_type: int
    offset: int


class TensorDataReader:
    """lib.rs:400-505: a bounded sequential reader over one tensor's encoding.  It holds no file descriptor between
    reads, so opening one per tensor of a large checkpoint is free."""

    def __init__(self, file: "GgufFile", info: TensorInfo, length: int):
        self._file, self.info, self._offset, self._length = file, info, 0, length

    def remaining(self) -> int:
        return self._length - self._offset

    def read(self, size: int = -1) -> bytes:
        want = self.remaining() if size is None or size < 0 else min(size, self.remaining())
        if want == 0:
            return b""
        buffer = (ctypes.c_ubyte * want)()
        got = ctypes.c_uint64()
        self._file._check(self._file._lib.ribn_gguf_read_tensor(self._file._handle, self.info.name.encode(), self._offset, buffer, want,
                                                                ctypes.byref(got)))
        self._offset += got.value
        return bytes(buffer[:got.value])


class GgufFile:
    """lib.rs:165-397."""

    def __init__(self, path: str):
        self._lib = _lib.load()
        self.path = str(path)
        handle = ctypes.c_void_p()
        status = self._lib.ribn_gguf_open(self.path.encode(), ctypes.byref(handle))
        if status != _lib.RIBN_OK:
            raise GgufError(status, self._lib.ribn_gguf_last_error(None).decode(errors="replace"))
        self._handle = handle

    @classmethod
    def open(cls, path: str) -> "GgufFile":
        return cls(path)

    def close(self) -> None:
        if getattr(self, "_handle", None):
            self._lib.ribn_gguf_close(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, status: int) -> None:
        if status != _lib.RIBN_OK:
            raise GgufError(status, self._lib.ribn_gguf_last_error(self._handle).decode(errors="replace"))

    def version(self) -> int:
        return self._lib.ribn_gguf_version(self._handle)

    def tensor_count(self) -> int:
        return self._lib.ribn_gguf_tensor_count(self._handle)

    def tensor_data_offset(self) -> int:
        return self._lib.ribn_gguf_tensor_data_offset(self._handle)

    # -- metadata ----------------------------------------------------------------------------------
    def metadata_keys(self) -> list[str]:
        return [self._lib.ribn_gguf_metadata_key(self._handle, i).decode() for i in range(self._lib.ribn_gguf_metadata_count(self._handle))]

    def _element(self, key: bytes, value_type: int, index: int):
        lib, h = self._lib, self._handle
        if value_type in (0, 2, 4, 10):
            out = ctypes.c_uint64()
            self._check(lib.ribn_gguf_metadata_u64(h, key, index, ctypes.byref(out)))
            return out.value
        if value_type in (1, 3, 5, 11):
            out = ctypes.c_int64()
            self._check(lib.ribn_gguf_metadata_i64(h, key, index, ctypes.byref(out)))
            return out.value
        if value_type in (6, 12):
            out = ctypes.c_double()
            self._check(lib.ribn_gguf_metadata_f64(h, key, index, ctypes.byref(out)))
            return out.value
        if value_type == 7:
            out = ctypes.c_int()
            self._check(lib.ribn_gguf_metadata_bool(h, key, index, ctypes.byref(out)))
            return bool(out.value)
        if value_type == 8:
            data, length = ctypes.c_void_p(), ctypes.c_uint64()
            self._check(lib.ribn_gguf_metadata_string(h, key, index, ctypes.byref(data), ctypes.byref(length)))
            return ctypes.string_at(data, length.value).decode()
        raise GgufError(115, f"GGUF metadata key {key.decode()!r} has an unexpected type")   # nested arrays stay opaque here

    def metadata(self, key: str):
        """The value of a key as a Python object (arrays as lists), or None when the key is absent."""
        value_type, element_type, count = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint64()
        status = self._lib.ribn_gguf_metadata_type(self._handle, key.encode(), ctypes.byref(value_type), ctypes.byref(element_type), ctypes.byref(count))
        if status == 114:
            return None
        self._check(status)
        if value_type.value == 9:
            return [self._element(key.encode(), element_type.value, i) for i in range(count.value)]
        return self._element(key.encode(), value_type.value, _lib.RIBN_GGUF_SCALAR)

    # -- tensors -----------------------------------------------------------------------------------
    def tensors(self) -> list[TensorInfo]:
        out = []
        for i in range(self.tensor_count()):
            raw = _lib.GgufTensor()
            self._check(self._lib.ribn_gguf_tensor_info(self._handle, i, ctypes.byref(raw)))
            out.append(TensorInfo(raw.name.decode(), tuple(raw.dims[:raw.n_dims]), raw.value_type, raw.offset))
        return out

    def tensor(self, name: str) -> TensorInfo | None:
        index = ctypes.c_uint64()
        if self._lib.ribn_gguf_find_tensor(self._handle, name.encode(), ctypes.byref(index)) != _lib.RIBN_OK:
            return None
        raw = _lib.GgufTensor()
        self._check(self._lib.ribn_gguf_tensor_info(self._handle, index.value, ctypes.byref(raw)))
        return TensorInfo(raw.name.decode(), tuple(raw.dims[:raw.n_dims]), raw.value_type, raw.offset)

    def tensor_data_range(self, name: str) -> range:
        begin, end = ctypes.c_uint64(), ctypes.c_uint64()
        self._check(self._lib.ribn_gguf_tensor_data_range(self._handle, name.encode(), ctypes.byref(begin), ctypes.byref(end)))
        return range(begin.value, end.value)

    def open_tensor(self, name: str) -> TensorDataReader:
        extent = self.tensor_data_range(name)
        return TensorDataReader(self, self.tensor(name), len(extent))

    def shard_bytes(self, name: str, axis: int, begin: int, end: int) -> tuple[int, int, int]:
        """(encoded bytes, K, N) of a shard; axis is _lib.RIBN_SHARD_ROWS (rows) or RIBN_SHARD_INPUT (super-blocks)."""
        size, k, n = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
        self._check(self._lib.ribn_gguf_shard_bytes(self._handle, name.encode(), axis, begin, end, ctypes.byref(size), ctypes.byref(k), ctypes.byref(n)))
        return size.value, k.value, n.value


def materialize_quantized(store, file: GgufFile, name: str, shard: str | None = None, world: int = 1, rank: int = 0, multiple: int = 1,
                          store_as: str | None = None):
    """Upload tensor `name` of `file` into `store` (a CudaWeightStore) through the staged copy of the library.

    `shard` None uploads the whole tensor; "rows" this rank's output rows (boundaries on multiples of `multiple`, e.g. the
    head size); "input" this rank's super-blocks of every row, packed -- the arithmetic of sharding.py.  Returns the
    CudaQuantizedWeight, whose dimensions are the shard's [K, N]."""
    import torch

    from .quantized import CudaQuantizedWeight, WeightTensorSpec

    info = file.tensor(name)
    if info is None:
        raise GgufError(116, f"GGUF tensor {name!r} was not found")
    axis, begin, end = _lib.RIBN_SHARD_NONE, 0, 0
    if shard is None:
        size, dims = len(file.tensor_data_range(name)), info.dimensions
    else:
        if len(info.dimensions) != 2:
            raise GgufError(_lib.RIBN_E_INVALID_WEIGHT, "invalid quantized weight: a shard needs a tensor of dimensions [input, output]")
        k, n = info.dimensions
        if shard == "rows":
            if n % multiple:
                raise ValueError(f"N={n} is not a multiple of {multiple}")
            b, e = split_even(n // multiple, world, rank)
            axis, begin, end = _lib.RIBN_SHARD_ROWS, b * multiple, e * multiple
        elif shard == "input":
            if k % 256:
                raise ValueError(f"K={k} is not a multiple of 256")
            begin, end = split_even(k // 256, world, rank)
            axis = _lib.RIBN_SHARD_INPUT
        else:
            raise ValueError(f"unknown shard kind {shard!r}")
        size, k_local, n_local = file.shard_bytes(name, axis, begin, end)
        dims = (k_local, n_local)
    context = store.context
    with torch.cuda.device(context.device):
        device = torch.empty(size, dtype=torch.uint8, device=context.device)
    # the allocation above came from torch's current stream; the copy runs on the context's
    device.record_stream(context.stream)
    context.stream.wait_stream(torch.cuda.current_stream(context.device))
    file._check(file._lib.ribn_materialize_quantized(context.handle, file._handle, name.encode(), axis, begin, end, device.data_ptr(), size))
    return store.adopt(WeightTensorSpec.new(store_as or name, dims), info.value_type, device)


def write_gguf(path: str, metadata: list[tuple[str, int, object]], tensors: list[tuple[str, tuple[int, ...], int, bytes]], alignment: int | None = None,
               version: int = 3) -> None:
    """A minimal GGUF writer for tests and synthetic checkpoints: metadata as (key, value type, value) -- arrays as
    (element type, list) -- and tensors as (name, dimensions, GGML type, encoded bytes), laid out in order with every
    payload aligned."""
    import struct

    def string(s) -> bytes:
        raw = s if isinstance(s, bytes) else s.encode()
        return struct.pack("<Q", len(raw)) + raw

    def value(value_type: int, v) -> bytes:
        formats = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}
        if value_type in formats:
            return struct.pack(formats[value_type], v)
        if value_type == 8:
            return string(v)
        if value_type == 9:
            element_type, items = v
            return struct.pack("<IQ", element_type, len(items)) + b"".join(value(element_type, item) for item in items)
        raise ValueError(f"value type {value_type}")

    align_to = alignment if alignment is not None else 32
    out = bytearray(struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(metadata)))
    for key, value_type, v in metadata:
        out += string(key) + struct.pack("<I", value_type) + value(value_type, v)
    offset, offsets = 0, []
    for _, _, _, data in tensors:
        offsets.append(offset)
        offset += (len(data) + align_to - 1) // align_to * align_to
    for (name, dims, value_type, _), at in zip(tensors, offsets):
        out += string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", value_type, at)
    out += b"\0" * (-len(out) % align_to)
    for (_, _, _, data), at in zip(tensors, offsets):
        out += bytes(data) + b"\0" * (-len(data) % align_to)
    with open(path, "wb") as f:
        f.write(out)
