"""ctypes binding of libribn_b200.so (the C ABI declared in include/ribn_b200.h).

There is no fallback: if the shared library is missing or does not export a declared symbol,
importing fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libribn_b200.so")

RIBN_OK = 0
RIBN_E_DRIVER = 1
RIBN_E_INVALID_WEIGHT = 2
RIBN_E_UNSUPPORTED_TYPE = 3
RIBN_E_SHAPE_OVERFLOW = 4
RIBN_E_INPUT_LENGTH = 5
RIBN_E_OUTPUT_LENGTH = 6
RIBN_E_CONTEXT_MISMATCH = 7
RIBN_E_TIMEOUT = 8
RIBN_E_INVALID_ARGUMENT = 9

RIBN_F32 = 0
RIBN_BF16 = 1
MAX_GEMV_MEMBERS = 64


class QWeight(ctypes.Structure):
    """struct ribn_qweight"""

    _fields_ = [
        ("data", ctypes.c_void_p),
        ("encoded_bytes", ctypes.c_uint64),
        ("value_type", ctypes.c_uint32),
        ("rank", ctypes.c_uint32),
        ("dimensions", ctypes.c_uint64 * 4),
    ]


class Attention(ctypes.Structure):
    """struct ribn_attention"""

    _fields_ = [
        ("members", ctypes.c_uint32),
        ("q_heads", ctypes.c_uint32),
        ("kv_heads", ctypes.c_uint32),
        ("head_dim", ctypes.c_uint32),
        ("rot_dims", ctypes.c_uint32),
        ("rope_base", ctypes.c_float),
        ("eps", ctypes.c_float),
        ("q_norm", ctypes.c_void_p),
        ("k_norm", ctypes.c_void_p),
        ("positions", ctypes.c_void_p),
        ("k_cache", ctypes.c_void_p),
        ("v_cache", ctypes.c_void_p),
        ("max_context", ctypes.c_uint64),
        ("active_context", ctypes.c_uint64),
        ("shared_cache", ctypes.c_uint32),
        ("out_dtype", ctypes.c_uint32),
    ]


class GgufTensor(ctypes.Structure):
    """struct ribn_gguf_tensor"""

    _fields_ = [
        ("name", ctypes.c_char_p),
        ("value_type", ctypes.c_uint32),
        ("n_dims", ctypes.c_uint32),
        ("dims", ctypes.c_uint64 * 16),
        ("offset", ctypes.c_uint64),
    ]


class GemvJob(ctypes.Structure):
    """struct ribn_gemv_job"""

    _fields_ = [
        ("expected_type", ctypes.c_uint32),
        ("weight", ctypes.POINTER(QWeight)),
        ("y_device", ctypes.c_void_p),
        ("y_dtype", ctypes.c_int),
        ("y_len", ctypes.c_uint64),
        ("accumulate", ctypes.c_int),
        ("split_rows", ctypes.c_uint64),
        ("y2_device", ctypes.c_void_p),
    ]


RIBN_FUSED_SWIGLU = 1
RIBN_SHARD_NONE, RIBN_SHARD_ROWS, RIBN_SHARD_INPUT = 0, 1, 2
RIBN_GGUF_SCALAR = 2 ** 64 - 1

_u64p = ctypes.POINTER(ctypes.c_uint64)
_vp = ctypes.c_void_p
_qwp = ctypes.POINTER(QWeight)
_attp = ctypes.POINTER(Attention)

# name -> (restype, argtypes); one entry per declaration in include/ribn_b200.h
SIGNATURES = {
    "ribn_create": (ctypes.c_int, [ctypes.c_int, _vp, ctypes.POINTER(_vp)]),
    "ribn_destroy": (None, [_vp]),
    "ribn_synchronize": (ctypes.c_int, [_vp]),
    "ribn_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "ribn_last_error": (ctypes.c_char_p, [_vp]),
    "ribn_last_error_detail": (None, [_vp, _u64p, _u64p]),
    "ribn_set_option": (ctypes.c_int, [_vp, ctypes.c_char_p, ctypes.c_int64]),
    "ribn_tensor_layout": (ctypes.c_int, [ctypes.c_uint32, _u64p, _u64p]),
    "ribn_validate_quantized_geometry": (ctypes.c_int, [_qwp, ctypes.c_uint32, _u64p, _u64p]),
    "ribn_dequantize": (ctypes.c_int, [_vp, _qwp, _vp, ctypes.c_uint64]),
    "ribn_gemv": (ctypes.c_int, [_vp, ctypes.c_uint32, _qwp, _vp, ctypes.c_int, ctypes.c_uint64, _vp, ctypes.c_int,
                                 ctypes.c_uint64, ctypes.c_uint32]),
    "ribn_rms_norm_gemv": (ctypes.c_int, [_vp, ctypes.c_uint32, _qwp, _vp, ctypes.c_int, ctypes.c_uint64, _vp, ctypes.c_uint64,
                                          ctypes.c_float, _vp, ctypes.c_int, ctypes.c_uint64, ctypes.c_uint32]),
    "ribn_gemm": (ctypes.c_int, [_vp, ctypes.c_uint32, _qwp, _vp, ctypes.c_uint64, _vp, ctypes.c_int, ctypes.c_uint64,
                                 ctypes.c_uint64]),
    "ribn_reserve_staging": (ctypes.c_int, [_vp, ctypes.c_uint64]),
    "ribn_gemv_host": (ctypes.c_int, [_vp, ctypes.c_uint32, _qwp, _vp, ctypes.c_int, ctypes.c_uint64, _vp,
                                      ctypes.c_int, ctypes.c_uint64, ctypes.c_uint32]),
    "ribn_gemv_host_async": (ctypes.c_int, [_vp, ctypes.c_uint32, _qwp, _vp, ctypes.c_int, ctypes.c_uint64, _vp,
                                      ctypes.c_int, ctypes.c_uint64, ctypes.c_uint32]),
    "ribn_gemv_noalloc": (ctypes.c_int, [ctypes.c_int, _vp, _qwp, _vp, ctypes.c_int, ctypes.c_uint64, _vp, ctypes.c_int,
                                         ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int, ctypes.c_char_p, ctypes.c_uint64]),
    "ribn_noalloc_status": (ctypes.c_int, [ctypes.c_int, _vp]),
    "ribn_selftest_bounded_wait": (ctypes.c_int, [_vp, ctypes.c_uint32]),
    "ribn_gemv_fused": (ctypes.c_int, [_vp, ctypes.POINTER(GemvJob), ctypes.c_uint32, _vp, ctypes.c_int, ctypes.c_uint64, _vp, ctypes.c_uint64,
                                       ctypes.c_float, ctypes.c_uint32, ctypes.c_uint32]),
    "ribn_embedding": (ctypes.c_int, [_vp, _qwp, _vp, ctypes.c_uint32, _vp, ctypes.c_uint64]),
    "ribn_qk_norm_rope_append": (ctypes.c_int, [_vp, _attp, _vp, _vp, _vp]),
    "ribn_attention_decode": (ctypes.c_int, [_vp, _attp, _vp, _vp]),
    "ribn_quantize_q8_1": (ctypes.c_int, [_vp, _vp, ctypes.c_uint64, _vp, ctypes.c_uint64]),
    "ribn_gemv_q8_1": (ctypes.c_int, [_vp, ctypes.c_uint32, ctypes.POINTER(QWeight), _vp, ctypes.c_uint64, _vp, ctypes.c_uint64, ctypes.c_uint32]),
    "ribn_silu_mul": (ctypes.c_int, [_vp, _vp, _vp, _vp, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_uint64]),
    "ribn_silu_mul_typed": (ctypes.c_int, [_vp, _vp, _vp, _vp, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_uint64]),
    "ribn_residual_add": (ctypes.c_int, [_vp, _vp, _vp, ctypes.c_uint64]),
    "ribn_argmax": (ctypes.c_int, [_vp, _vp, ctypes.c_uint32, ctypes.c_uint64, _vp]),
    "ribn_tp_create": (ctypes.c_int, [_vp, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint64, _vp, ctypes.POINTER(_vp)]),
    "ribn_tp_destroy": (None, [_vp]),
    "ribn_tp_last_error": (ctypes.c_char_p, [_vp]),
    "ribn_tp_block_bytes": (ctypes.c_uint64, [ctypes.c_uint64]),
    "ribn_tp_export": (ctypes.c_int, [_vp, _vp]),
    "ribn_tp_connect": (ctypes.c_int, [_vp, _vp]),
    "ribn_tp_connect_pointers": (ctypes.c_int, [_vp, ctypes.POINTER(_vp)]),
    "ribn_tp_set_wait": (ctypes.c_int, [_vp, ctypes.c_uint64]),
    "ribn_tp_partial": (ctypes.c_int, [_vp, ctypes.c_uint32, ctypes.POINTER(_vp)]),
    "ribn_tp_allreduce_residual": (ctypes.c_int, [_vp, _vp, ctypes.c_uint32, _vp, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int]),
    "ribn_tp_select_tokens": (ctypes.c_int, [_vp, _vp, _vp, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_uint32, _vp]),
    "ribn_context_stream": (ctypes.c_int, [_vp, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(_vp)]),
    "ribn_gguf_open": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(_vp)]),
    "ribn_gguf_close": (None, [_vp]),
    "ribn_gguf_last_error": (ctypes.c_char_p, [_vp]),
    "ribn_gguf_version": (ctypes.c_uint32, [_vp]),
    "ribn_gguf_tensor_count": (ctypes.c_uint64, [_vp]),
    "ribn_gguf_metadata_count": (ctypes.c_uint64, [_vp]),
    "ribn_gguf_tensor_data_offset": (ctypes.c_uint64, [_vp]),
    "ribn_gguf_metadata_key": (ctypes.c_char_p, [_vp, ctypes.c_uint64]),
    "ribn_gguf_metadata_type": (ctypes.c_int, [_vp, ctypes.c_char_p, ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_uint32), _u64p]),
    "ribn_gguf_metadata_u64": (ctypes.c_int, [_vp, ctypes.c_char_p, ctypes.c_uint64, _u64p]),
    "ribn_gguf_metadata_i64": (ctypes.c_int, [_vp, ctypes.c_char_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_int64)]),
    "ribn_gguf_metadata_f64": (ctypes.c_int, [_vp, ctypes.c_char_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_double)]),
    "ribn_gguf_metadata_bool": (ctypes.c_int, [_vp, ctypes.c_char_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_int)]),
    "ribn_gguf_metadata_string": (ctypes.c_int, [_vp, ctypes.c_char_p, ctypes.c_uint64, ctypes.POINTER(_vp), _u64p]),
    "ribn_gguf_tensor_info": (ctypes.c_int, [_vp, ctypes.c_uint64, ctypes.POINTER(GgufTensor)]),
    "ribn_gguf_find_tensor": (ctypes.c_int, [_vp, ctypes.c_char_p, _u64p]),
    "ribn_gguf_tensor_data_range": (ctypes.c_int, [_vp, ctypes.c_char_p, _u64p, _u64p]),
    "ribn_gguf_read_tensor": (ctypes.c_int, [_vp, ctypes.c_char_p, ctypes.c_uint64, _vp, ctypes.c_uint64, _u64p]),
    "ribn_gguf_shard_bytes": (ctypes.c_int, [_vp, ctypes.c_char_p, ctypes.c_int, ctypes.c_uint64, ctypes.c_uint64, _u64p, _u64p, _u64p]),
    "ribn_materialize_quantized": (ctypes.c_int, [_vp, _vp, ctypes.c_char_p, ctypes.c_int, ctypes.c_uint64, ctypes.c_uint64, _vp, ctypes.c_uint64]),
    "ribn_rms_norm": (ctypes.c_int, [_vp, _vp, ctypes.c_int, ctypes.c_uint64, _vp, ctypes.c_uint64, _vp, ctypes.c_int,
                                     ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_float]),
}

_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing. Build it with `python -m engine_b200.build` (needs nvcc; the library "
            "targets sm_100a only and has no CPU or PyTorch fallback)."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise ImportError(f"{LIB_PATH} does not export {name}; rebuild with `python -m engine_b200.build --force`") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib
