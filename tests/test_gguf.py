"""The GGUF v3 reader of the library (csrc/gguf.cu through engine_b200/gguf.py) on files written by the test: the
reference's own fixture (crates/gguf/src/lib.rs:1219-1276 of the reference project, restated field by field) and one
malformed file per error class of its parser (:191-280, :1085-1156, :139-163).  No GPU is involved."""
import os
import struct

import numpy as np
import pytest

from engine_b200 import gguf, synth

MAGIC, VERSION = 0x46554747, 3


def s(text) -> bytes:
    raw = text if isinstance(text, bytes) else text.encode()
    return struct.pack("<Q", len(raw)) + raw


def reference_fixture() -> bytes:
    """One F16 tensor [4, 8] at offset 0, three metadata entries, 256 zero bytes behind the directory."""
    out = struct.pack("<IIQQ", MAGIC, VERSION, 1, 3)
    out += s("general.architecture") + struct.pack("<I", 8) + s("qwen3")
    out += s("general.alignment") + struct.pack("<II", 4, 32)
    out += s("test.array") + struct.pack("<IIQII", 9, 4, 2, 1, 0)
    out += s("token_embd.weight") + struct.pack("<IQQIQ", 2, 4, 8, 1, 0)
    return out + bytes(256)


def write(tmp_path, data: bytes, name="f.gguf") -> str:
    path = os.path.join(tmp_path, name)
    with open(path, "wb") as f:
        f.write(data)
    return path


def test_parses_metadata_and_tensor_directory_without_loading_tensor_data(tmp_path):
    parsed = gguf.GgufFile.open(write(tmp_path, reference_fixture()))
    assert parsed.version() == 3 and parsed.tensor_count() == 1
    assert parsed.metadata("general.architecture") == "qwen3"
    assert parsed.metadata("general.alignment") == 32
    assert parsed.metadata("test.array") == [1, 0]
    assert parsed.metadata("absent") is None
    info = parsed.tensors()[0]
    assert (info.name, info.dimensions, info.value_type, info.offset) == ("token_embd.weight", (4, 8), 1, 0)
    extent = parsed.tensor_data_range("token_embd.weight")
    assert len(extent) == 64 and extent.start == parsed.tensor_data_offset() and extent.start % 32 == 0


def test_streams_only_the_selected_tensor_payload(tmp_path):
    payload_a, payload_b = bytes(range(64)), bytes(range(100, 164))
    path = os.path.join(tmp_path, "two.gguf")
    gguf.write_gguf(path, [("general.architecture", 8, "qwen3")], [("a", (4, 8), 1, payload_a), ("b", (32,), 1, payload_b)])
    parsed = gguf.GgufFile.open(path)
    reader = parsed.open_tensor("a")
    assert reader.read() == payload_a and reader.remaining() == 0 and reader.read(1) == b""
    chunks, reader = [], parsed.open_tensor("b")
    while True:
        chunk = reader.read(7)
        if not chunk:
            break
        chunks.append(chunk)
    assert b"".join(chunks) == payload_b and all(len(c) == 7 for c in chunks[:-1])


def test_opening_readers_costs_no_descriptor_until_they_are_read(tmp_path):
    parsed = gguf.GgufFile.open(write(tmp_path, reference_fixture()))
    before = len(os.listdir("/proc/self/fd"))
    readers = [parsed.open_tensor("token_embd.weight") for _ in range(512)]
    assert len(os.listdir("/proc/self/fd")) <= before + 4
    assert len(readers[0].read()) == 64
    assert len(os.listdir("/proc/self/fd")) <= before + 4


def test_every_value_type_round_trips(tmp_path):
    path = os.path.join(tmp_path, "values.gguf")
    entries = [("u8", 0, 200), ("i8", 1, -100), ("u16", 2, 60000), ("i16", 3, -30000), ("u32", 4, 4000000000), ("i32", 5, -2000000000),
               ("f32", 6, 1.5), ("yes", 7, 1), ("no", 7, 0), ("text", 8, "grüß"), ("u64", 10, 2 ** 63 + 5), ("i64", 11, -2 ** 62), ("f64", 12, 2.0 ** -40),
               ("words", 9, (8, ["a", "", "ccc"])), ("ints", 9, (5, [-1, 2, -3])), ("flags", 9, (7, [1, 0])), ("empty", 9, (4, []))]
    gguf.write_gguf(path, entries, [])
    parsed = gguf.GgufFile.open(path)
    assert parsed.metadata_keys() == sorted(key for key, _, _ in entries)
    expected = {"u8": 200, "i8": -100, "u16": 60000, "i16": -30000, "u32": 4000000000, "i32": -2000000000, "f32": 1.5, "yes": True, "no": False,
                "text": "grüß", "u64": 2 ** 63 + 5, "i64": -2 ** 62, "f64": 2.0 ** -40, "words": ["a", "", "ccc"], "ints": [-1, 2, -3],
                "flags": [True, False], "empty": []}
    for key, want in expected.items():
        assert parsed.metadata(key) == want, key
    assert parsed.tensor_count() == 0


def header(tensors=0, metadata=0, magic=MAGIC, version=VERSION) -> bytes:
    return struct.pack("<IIQQ", magic, version, tensors, metadata)


def nested_arrays(depth: int) -> bytes:
    out = s("deep") + struct.pack("<I", 9)
    for _ in range(depth):
        out += struct.pack("<IQ", 9, 1)
    return out + struct.pack("<IQ", 4, 0)


MALFORMED = {
    "InvalidMagic": header(magic=0x46554746),
    "UnsupportedVersion": header(version=2),
    "UnexpectedEof": header(tensors=1)[:20],
    "InvalidLength": header(metadata=1) + struct.pack("<Q", 16 * 1024 * 1024 + 1),
    "InvalidUtf8": header(metadata=1) + s(b"\xff\xfe") + struct.pack("<II", 4, 0),
    "InvalidValueType": header(metadata=1) + s("k") + struct.pack("<I", 13),
    "InvalidBool": header(metadata=1) + s("k") + struct.pack("<IB", 7, 2),
    "ArrayNestingTooDeep": header(metadata=1) + nested_arrays(18),
    "DuplicateMetadata": header(metadata=2) + (s("k") + struct.pack("<II", 4, 1)) * 2,
    "InvalidDimensionCount": header(tensors=1) + s("t") + struct.pack("<I", 17),
    "InvalidAlignment": header(metadata=1) + s("general.alignment") + struct.pack("<II", 4, 24),
    "TensorOffsetOutOfBounds": header(tensors=1) + s("t") + struct.pack("<IQIQ", 1, 32, 0, 4096) + bytes(64),
}


@pytest.mark.parametrize("kind", list(MALFORMED))
def test_malformed_files_are_refused_with_the_reference_error_class(tmp_path, kind):
    with pytest.raises(gguf.GgufError) as e:
        gguf.GgufFile.open(write(tmp_path, MALFORMED[kind]))
    assert e.value.kind == kind, str(e.value)


def test_too_many_items_and_missing_file(tmp_path):
    with pytest.raises(gguf.GgufError) as e:
        gguf.GgufFile.open(write(tmp_path, header(metadata=1) + s("k") + struct.pack("<IIQ", 9, 4, 1000001)))
    assert e.value.kind == "InvalidLength"
    with pytest.raises(gguf.GgufError) as e:
        gguf.GgufFile.open(write(tmp_path, header(tensors=10000001)))
    assert e.value.kind == "InvalidLength"
    with pytest.raises(gguf.GgufError) as e:
        gguf.GgufFile.open(os.path.join(tmp_path, "absent.gguf"))
    assert e.value.kind == "Io"
    assert gguf.GgufFile.open(write(tmp_path, header(metadata=1) + nested_arrays(16) + bytes(64), "deep_ok.gguf")).metadata_keys() == ["deep"]


def test_tensor_layout_checks(tmp_path):
    """TensorInfo::byte_len (lib.rs:139-163): the first dimension and the element count must be whole blocks; an unknown
    type parses but has no byte length; a range that ends past the file is refused when it is asked for."""
    path = os.path.join(tmp_path, "layout.gguf")
    gguf.write_gguf(path, [], [("ok", (256, 3), 12, bytes(3 * 144)), ("ragged", (100, 3), 12, bytes(64)), ("unknown", (32,), 999, bytes(32)),
                               ("scalar", (), 0, bytes(32)), ("short", (256, 1000), 12, bytes(144))])
    parsed = gguf.GgufFile.open(path)
    assert len(parsed.tensor_data_range("ok")) == 3 * 144
    for name, kind in (("ragged", "QuantizationDimensionMismatch"), ("unknown", "UnsupportedTensorType"), ("scalar", "InvalidDimensionCount"),
                       ("short", "TensorOffsetOutOfBounds"), ("absent", "MissingTensor")):
        with pytest.raises(gguf.GgufError) as e:
            parsed.tensor_data_range(name)
        assert e.value.kind == kind, name
    assert parsed.tensor("unknown").value_type == 999 and parsed.tensor("absent") is None


def test_shard_sizes_follow_the_sharding_arithmetic(tmp_path):
    from engine_b200 import _lib, sharding

    k, n = 1024, 24
    path = os.path.join(tmp_path, "shards.gguf")
    tensors = [(f"w{vt}", (k, n), vt, synth.random_weight(vt, k, n, seed=vt).tobytes()) for vt in (8, 12, 13, 14)]
    gguf.write_gguf(path, [], tensors)
    parsed = gguf.GgufFile.open(path)
    for name, _, vt, data in tensors:
        encoded = np.frombuffer(data, np.uint8)
        for world in (1, 3, 8):
            for rank in range(world):
                rows, (_, n_local) = sharding.shard_rows(encoded, vt, k, n, world, rank)
                r0, r1 = sharding.row_range(n, world, rank)
                assert parsed.shard_bytes(name, _lib.RIBN_SHARD_ROWS, r0, r1) == (rows.size, k, n_local)
                cols, (k_local, _), (k0, k1) = sharding.shard_k(encoded, vt, k, n, world, rank)
                assert parsed.shard_bytes(name, _lib.RIBN_SHARD_INPUT, k0 // 256, k1 // 256) == (cols.size, k_local, n)
    with pytest.raises(gguf.GgufError):
        parsed.shard_bytes("w12", _lib.RIBN_SHARD_INPUT, 0, 5)
    with pytest.raises(gguf.GgufError):
        parsed.shard_bytes("w12", _lib.RIBN_SHARD_ROWS, 3, 25)
