"""CPU oracle for the GGUF quantized-matmul path.  TEST INFRASTRUCTURE ONLY.

`ribn_oracle.c` restates the reference's host algorithms in plain C;
`oracle_np.py` is an independent vectorised numpy twin.  Only the test-suite,
the smoke check and the benchmark's CPU-baseline leg may import this package;
the shipped library never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libribn_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ribn_oracle.c with gcc (see Makefile); returns the .so path."""
    src = os.path.join(_HERE, "ribn_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "-s"], check=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        u8p, f32p, f64p = (ctypes.POINTER(t) for t in (ctypes.c_uint8, ctypes.c_float, ctypes.c_double))
        u64 = ctypes.c_uint64
        _lib.ribn_oracle_tensor_layout.argtypes = [ctypes.c_uint32, ctypes.POINTER(u64), ctypes.POINTER(u64)]
        _lib.ribn_oracle_f16_to_f32.argtypes = [ctypes.c_uint16]
        _lib.ribn_oracle_f16_to_f32.restype = ctypes.c_float
        _lib.ribn_oracle_q4_k_scales.argtypes = [u8p, u8p, u8p]
        _lib.ribn_oracle_q4_k_scales.restype = None
        _lib.ribn_oracle_dequantize_block.argtypes = [ctypes.c_uint32, u8p, u64, f32p]
        _lib.ribn_oracle_dequantize.argtypes = [ctypes.c_uint32, u8p, u64, u64, f32p, ctypes.c_int]
        _lib.ribn_oracle_gemv_f32.argtypes = [ctypes.c_uint32, u8p, u64, u64, f32p, u64, f32p, ctypes.c_int]
        _lib.ribn_oracle_gemv_f64.argtypes = [ctypes.c_uint32, u8p, u64, u64, f32p, u64, f64p, ctypes.c_int]
        _lib.ribn_oracle_gemv_scale.argtypes = [ctypes.c_uint32, u8p, u64, u64, f32p, u64, f64p, ctypes.c_int]
        _lib.ribn_oracle_rms_norm.argtypes = [f32p, f32p, u64, ctypes.c_float, f32p]
        _lib.ribn_oracle_rms_norm.restype = None
        _lib.ribn_oracle_rms_norm_batch.argtypes = [f32p, f32p, u64, u64, ctypes.c_float, f32p]
        _lib.ribn_oracle_rms_norm_batch.restype = None
        _lib.ribn_oracle_silu_mul.argtypes = [f32p, f32p, u64, f32p]
        _lib.ribn_oracle_silu_mul.restype = None
        _lib.ribn_oracle_f32_to_bf16.argtypes = [ctypes.c_float]
        _lib.ribn_oracle_f32_to_bf16.restype = ctypes.c_uint16
    return _lib


class OracleError(Exception):
    """status 1 = unsupported tensor type, 2 = invalid block length, 3 = invalid shape
    (the reference's GgufError::UnsupportedTensorType / InvalidTensorBlockLength)."""

    def __init__(self, status: int):
        super().__init__({1: "unsupported tensor type", 2: "invalid tensor block length",
                          3: "invalid shape"}.get(status, f"status {status}"))
        self.status = status


def _ptr(a: np.ndarray, ctype):
    return a.ctypes.data_as(ctypes.POINTER(ctype))


def _bytes(data) -> np.ndarray:
    return np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.reshape(-1).view(np.uint8))


def tensor_layout(value_type: int) -> tuple[int, int]:
    e, b = ctypes.c_uint64(), ctypes.c_uint64()
    status = lib().ribn_oracle_tensor_layout(value_type, ctypes.byref(e), ctypes.byref(b))
    if status:
        raise OracleError(status)
    return e.value, b.value


def f16_to_f32(bits: int) -> np.float32:
    return np.float32(lib().ribn_oracle_f16_to_f32(bits))


def dequantize_block(value_type: int, encoded) -> np.ndarray:
    raw = _bytes(encoded)
    try:
        elements, _ = tensor_layout(value_type)
    except OracleError:
        elements = 1
    out = np.empty(elements, np.float32)
    status = lib().ribn_oracle_dequantize_block(value_type, _ptr(raw, ctypes.c_uint8), raw.size, _ptr(out, ctypes.c_float))
    if status:
        raise OracleError(status)
    return out


def dequantize(value_type: int, data, k: int, n: int) -> np.ndarray:
    raw = _bytes(data)
    out = np.empty((n, k), np.float32)
    status = lib().ribn_oracle_dequantize(value_type, _ptr(raw, ctypes.c_uint8), k, n, _ptr(out, ctypes.c_float),
                                          os.cpu_count() or 1)
    if status:
        raise OracleError(status)
    return out


def _gemv(fn, out_dtype, ctype, value_type, data, k, n, x, threads):
    raw = _bytes(data)
    x = np.ascontiguousarray(np.asarray(x, dtype=np.float32).reshape(-1, k))
    y = np.empty((x.shape[0], n), out_dtype)
    status = fn(value_type, _ptr(raw, ctypes.c_uint8), k, n, _ptr(x, ctypes.c_float), x.shape[0], _ptr(y, ctype), threads)
    if status:
        raise OracleError(status)
    return y


def gemv_f32(value_type: int, data, k: int, n: int, x, threads: int = 1) -> np.ndarray:
    """Reference host path: dequantise a row, sequential f32 dot. x [members, K] -> [members, N]."""
    return _gemv(lib().ribn_oracle_gemv_f32, np.float32, ctypes.c_float, value_type, data, k, n, x, threads)


def gemv_f64(value_type: int, data, k: int, n: int, x, threads: int = 0) -> np.ndarray:
    return _gemv(lib().ribn_oracle_gemv_f64, np.float64, ctypes.c_double, value_type, data, k, n, x,
                 threads or (os.cpu_count() or 1))


def gemv_scale(value_type: int, data, k: int, n: int, x, threads: int = 0) -> np.ndarray:
    return _gemv(lib().ribn_oracle_gemv_scale, np.float64, ctypes.c_double, value_type, data, k, n, x,
                 threads or (os.cpu_count() or 1))


def rms_norm(x, weight, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
    w = np.ascontiguousarray(np.asarray(weight, dtype=np.float32))
    length = x.shape[-1]
    members = x.size // length
    out = np.empty_like(x)
    lib().ribn_oracle_rms_norm_batch(_ptr(x, ctypes.c_float), _ptr(w, ctypes.c_float), members, length,
                                     ctypes.c_float(eps), _ptr(out, ctypes.c_float))
    return out


def silu_mul(gate, up) -> np.ndarray:
    g = np.ascontiguousarray(np.asarray(gate, dtype=np.float32))
    u = np.ascontiguousarray(np.asarray(up, dtype=np.float32))
    out = np.empty_like(g)
    lib().ribn_oracle_silu_mul(_ptr(g, ctypes.c_float), _ptr(u, ctypes.c_float), g.size, _ptr(out, ctypes.c_float))
    return out


def max_rel_error(y, y_ref, scale) -> float:
    """The parity metric: max |y - y_ref| / max(|y_ref|, scale), with `scale` the per-output
    sqrt(sum (w*x)^2) from gemv_scale.  The floor keeps outputs that happen to cancel to ~0
    from dominating a relative measure; it is the magnitude a dot product of that row has."""
    y = np.asarray(y, dtype=np.float64)
    y_ref = np.asarray(y_ref, dtype=np.float64)
    den = np.maximum(np.abs(y_ref), np.asarray(scale, dtype=np.float64))
    den = np.where(den == 0.0, 1.0, den)
    return float(np.max(np.abs(y - y_ref) / den))


STRICT_EPSILON = 1e-3


def row_norms(value_type: int, data, k: int, n: int) -> np.ndarray:
    """||w_row||_2 of every dequantised row, float64 [N]."""
    w = dequantize(value_type, data, k, n).astype(np.float64)
    return np.sqrt(np.sum(w * w, axis=1))


def max_rel_error_strict(y, y_ref, weight_row_norms, x, epsilon: float = STRICT_EPSILON) -> float:
    """max |y - y_ref| / max(|y_ref|, epsilon * ||w_row||_2 * ||x||_2): the relative error of every output
    against itself, with a floor that only protects outputs below epsilon (1e-3) of the Cauchy-Schwarz bound
    of their dot product.  For K = 4096 random data that floor is about 6 % of a typical output magnitude."""
    y = np.asarray(y, dtype=np.float64)
    y_ref = np.asarray(y_ref, dtype=np.float64)
    x_norm = np.sqrt(np.sum(np.asarray(x, dtype=np.float64) ** 2, axis=-1)).reshape(-1, 1)
    floor = epsilon * x_norm * np.asarray(weight_row_norms, dtype=np.float64).reshape(1, -1)
    den = np.maximum(np.abs(y_ref), floor)
    den = np.where(den == 0.0, 1.0, den)
    return float(np.max(np.abs(y - y_ref) / den))
