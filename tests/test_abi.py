"""The C-ABI library loads, exports every symbol include/ribn_b200.h declares, and its host-only
entry points behave like the reference's validation layer.  No GPU, no compute calls."""
import ctypes
import os
import re

import pytest

import engine_b200
from engine_b200 import _lib

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ribn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ribn_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    # and the Python binding table covers the same set
    assert sorted(_lib.SIGNATURES) == names


def test_header_is_plain_c():
    """The boundary is plain C: the header compiles as C99 on its own."""
    import subprocess
    import tempfile

    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "t.c")
        with open(src, "w") as f:
            f.write('#include "ribn_b200.h"\nint main(void){ribn_qweight w; (void)w; return RIBN_ABI_VERSION - 1;}\n')
        subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c", src, "-o",
                        os.path.join(tmp, "t.o")], check=True)


def test_status_strings():
    lib = _lib.load()
    seen = {lib.ribn_status_string(code).decode() for code in range(10)}
    assert len(seen) == 10 and "unknown status" not in seen
    assert lib.ribn_status_string(1234).decode() == "unknown status"


# crates/gguf/src/lib.rs:1051-1083
def test_tensor_layout_table():
    assert engine_b200.tensor_layout(8) == (32, 34)
    assert engine_b200.tensor_layout(12) == (256, 144)
    assert engine_b200.tensor_layout(13) == (256, 176)
    assert engine_b200.tensor_layout(14) == (256, 210)
    assert engine_b200.tensor_layout(0) == (1, 4)
    with pytest.raises(engine_b200.CudaQuantizedKernelError) as e:
        engine_b200.tensor_layout(99)
    assert e.value.kind == "UnsupportedValueType"


# crates/nvidia/src/quantized.rs:1755-1804
def test_validate_quantized_geometry():
    v = engine_b200.validate_geometry_raw
    assert v(12, [4096, 4096], 9437184) == (4096, 4096)
    assert v(14, [12288, 4096], 41287680, 14) == (12288, 4096)
    assert v(8, [64, 3], 6 * 34, 8) == (64, 3)

    def kind(*args):
        with pytest.raises(engine_b200.CudaQuantizedKernelError) as e:
            v(*args)
        return e.value.kind

    assert kind(13, [256, 2], 352, 12) == "UnsupportedValueType"   # kernel object of another family
    assert kind(12, [256], 144, 12) == "InvalidWeight"             # rank 1
    assert kind(12, [256, 2, 1], 288, 12) == "InvalidWeight"       # rank 3
    assert kind(12, [128, 2], 144, 12) == "InvalidWeight"          # K not a multiple of the block
    assert kind(12, [0, 2], 0, 12) == "InvalidWeight"
    assert kind(12, [256, 0], 0, 12) == "InvalidWeight"
    assert kind(12, [256, 2], 287, 12) == "InvalidWeight"          # encoded length
    assert kind(12, [256, 2], 289, 12) == "InvalidWeight"
    assert kind(11, [256, 2], 220, 0) == "InvalidWeight"           # Q3_K has no kernel here
    assert kind(12, [256 * (1 << 40), 1 << 30], 0, 12) == "ShapeOverflow"
    assert kind(12, [1 << 32, 1], (1 << 24) * 144, 12) == "ShapeOverflow"  # dimension over i32::MAX


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    """No silent fallback: without the shared library the binding raises and says how to build."""
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libribn_b200.so"))
    with pytest.raises(ImportError, match="engine_b200.build"):
        _lib.load()


def test_product_never_imports_the_oracle():
    """The oracle is test infrastructure; nothing under engine_b200/ may reference it."""
    for base, _, files in os.walk(os.path.join(ROOT, "engine_b200")):
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(base, name)).read()
                assert "import oracle" not in text and "from oracle" not in text and "ribn_oracle" not in text, name


def test_create_without_gpu_is_an_error():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    handle = ctypes.c_void_p()
    assert _lib.load().ribn_create(0, None, ctypes.byref(handle)) == _lib.RIBN_E_DRIVER
    assert not handle.value
