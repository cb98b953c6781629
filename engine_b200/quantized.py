"""Host-side mirror of the reference's kernel wrapper objects, over the C ABI.

The names, argument meaning and error behaviour follow the reference project's
`crates/nvidia/src/quantized.rs` (Cuda{Q4K,Q5K,Q6K,Q8_0}Gemv, :1366-1753),
`staging.rs` (QwenGemvKernel, :90-217), `cuda.rs` (CudaWeightStore / CudaQuantizedWeight,
:157-387) and `model_ops.rs` (CudaQwen35Ops::rms_norm{,_batch}, :1714-1824), so that parity
tests read like the reference's own tests.  torch supplies device memory and streams only;
every computation goes through libribn_b200.so.  There is no fallback path.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from ._lib import QWeight

_KIND = {
    _lib.RIBN_E_DRIVER: "Driver",
    _lib.RIBN_E_INVALID_WEIGHT: "InvalidWeight",
    _lib.RIBN_E_UNSUPPORTED_TYPE: "UnsupportedValueType",
    _lib.RIBN_E_SHAPE_OVERFLOW: "ShapeOverflow",
    _lib.RIBN_E_INPUT_LENGTH: "InputLength",
    _lib.RIBN_E_OUTPUT_LENGTH: "OutputLength",
    _lib.RIBN_E_CONTEXT_MISMATCH: "ContextMismatch",
    _lib.RIBN_E_TIMEOUT: "Timeout",
    _lib.RIBN_E_INVALID_ARGUMENT: "InvalidArgument",
}


class CudaQuantizedKernelError(Exception):
    """quantized.rs:90-100.  `kind` is the enum variant name; `expected` / `actual` are filled for
    UnsupportedValueType, InputLength and OutputLength."""

    def __init__(self, status: int, message: str, expected: int = 0, actual: int = 0):
        super().__init__(message or _lib.load().ribn_status_string(status).decode())
        self.status = status
        self.kind = _KIND.get(status, f"status{status}")
        self.expected = expected
        self.actual = actual


def tensor_layout(value_type: int) -> tuple[int, int]:
    """crates/gguf/src/lib.rs:1051-1083."""
    e, b = ctypes.c_uint64(), ctypes.c_uint64()
    status = _lib.load().ribn_tensor_layout(value_type, ctypes.byref(e), ctypes.byref(b))
    if status != _lib.RIBN_OK:
        raise CudaQuantizedKernelError(status, f"unsupported tensor type {value_type}")
    return e.value, b.value


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _lib.RIBN_F32
    if t.dtype == torch.bfloat16:
        return _lib.RIBN_BF16
    raise TypeError(f"activations must be float32 or bfloat16, got {t.dtype}")


class RibnContext:
    """One (device, stream) owner: `ribn_ctx`.  Not thread-safe, like the reference's kernel
    objects (one mutable execution owner per model, adapter.rs:16)."""

    def __init__(self, device: int | torch.device = 0, stream: torch.cuda.Stream | None = None):
        self._lib = _lib.load()
        index = torch.device(device).index if not isinstance(device, int) else device
        self.device = torch.device("cuda", index or 0)
        with torch.cuda.device(self.device):
            torch.cuda.init()
            self.stream = stream if stream is not None else torch.cuda.current_stream(self.device)
        handle = ctypes.c_void_p()
        status = self._lib.ribn_create(self.device.index, ctypes.c_void_p(self.stream.cuda_stream), ctypes.byref(handle))
        if status != _lib.RIBN_OK:
            raise CudaQuantizedKernelError(status, "ribn_create failed (an sm_100 GPU is required)")
        self.handle = handle

    def close(self) -> None:
        if getattr(self, "handle", None):
            self._lib.ribn_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, status: int) -> None:
        if status == _lib.RIBN_OK:
            return
        expected, actual = ctypes.c_uint64(), ctypes.c_uint64()
        self._lib.ribn_last_error_detail(self.handle, ctypes.byref(expected), ctypes.byref(actual))
        message = self._lib.ribn_last_error(self.handle).decode()
        raise CudaQuantizedKernelError(status, message, expected.value, actual.value)

    def synchronize(self) -> None:
        self.check(self._lib.ribn_synchronize(self.handle))

    def selftest_bounded_wait(self, polls: int = 1000) -> None:
        """Launches a kernel whose bounded wait runs out by design; the next synchronize() must raise kind 'Timeout'."""
        self.check(self._lib.ribn_selftest_bounded_wait(self.handle, polls))

    def set_option(self, name: str, value: int) -> None:
        self.check(self._lib.ribn_set_option(self.handle, name.encode(), value))

    def reserve_staging(self, nbytes: int) -> None:
        self.check(self._lib.ribn_reserve_staging(self.handle, nbytes))


@dataclass(frozen=True)
class WeightTensorSpec:
    """crates/core/src/weights.rs:16-82: a name and GGML-order dimensions ([K, N] for a matrix)."""

    name: str
    dimensions: tuple[int, ...]

    @staticmethod
    def new(name: str, dimensions) -> "WeightTensorSpec":
        return WeightTensorSpec(name, tuple(int(d) for d in dimensions))


class CudaQuantizedWeight:
    """cuda.rs:157-183: opaque GGUF-encoded bytes resident on the device, never dequantised on the host."""

    def __init__(self, spec: WeightTensorSpec, value_type: int, encoded: torch.Tensor):
        if encoded.dtype != torch.uint8 or not encoded.is_cuda or not encoded.is_contiguous():
            raise TypeError("encoded weight must be a contiguous CUDA uint8 tensor")
        self._spec = spec
        self._value_type = int(value_type)
        self._encoded = encoded
        self._descriptor = None

    def spec(self) -> WeightTensorSpec:
        return self._spec

    def value_type(self) -> int:
        return self._value_type

    def encoded_bytes(self) -> int:
        return self._encoded.numel()

    def encoded_data(self) -> torch.Tensor:
        return self._encoded

    def descriptor(self) -> QWeight:
        if self._descriptor is None:   # the bytes never move or change once resident, so neither does their description
            dims = (ctypes.c_uint64 * 4)(*(list(self._spec.dimensions)[:4] + [0] * (4 - min(4, len(self._spec.dimensions)))))
            self._descriptor = QWeight(self._encoded.data_ptr(), self._encoded.numel(), self._value_type,
                                       len(self._spec.dimensions), dims)
        return self._descriptor


class CudaWeightStore:
    """cuda.rs:321-387: uploads encoded tensors as opaque bytes and hands them out by name."""

    def __init__(self, context: RibnContext):
        self.context = context
        self._weights: dict[str, CudaQuantizedWeight] = {}

    def materialize_quantized(self, spec: WeightTensorSpec, value_type: int, byte_len: int, reader) -> WeightTensorSpec:
        data = reader.read(byte_len) if hasattr(reader, "read") else reader
        host = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.reshape(-1).view(np.uint8)
        if host.size != byte_len:
            raise CudaQuantizedKernelError(_lib.RIBN_E_INVALID_WEIGHT,
                                           f"invalid quantized weight: encoded length is {host.size}, expected {byte_len}")
        if spec.name in self._weights:
            raise CudaQuantizedKernelError(_lib.RIBN_E_INVALID_WEIGHT, f"duplicate weight {spec.name}")
        with torch.cuda.device(self.context.device), torch.cuda.stream(self.context.stream):
            device = torch.from_numpy(np.ascontiguousarray(host)).to(self.context.device)
        self._weights[spec.name] = CudaQuantizedWeight(spec, value_type, device)
        return spec

    def adopt(self, spec: WeightTensorSpec, value_type: int, encoded: torch.Tensor) -> CudaQuantizedWeight:
        """Register bytes that are already on the device (random-init models generated in place)."""
        weight = CudaQuantizedWeight(spec, value_type, encoded)
        self._weights[spec.name] = weight
        return weight

    def quantized_tensor(self, name: str) -> CudaQuantizedWeight:
        return self._weights[name]

    def copy_quantized_to_host(self, name: str) -> bytes:
        return self._weights[name].encoded_data().cpu().numpy().tobytes()


class _CudaQuantizedGemv:
    """Shared body of the four kernel objects (quantized.rs:143-488)."""

    VALUE_TYPE = 0
    LABEL = ""

    def __init__(self, context: RibnContext):
        self.context = context

    @classmethod
    def from_context(cls, context: RibnContext):
        return cls(context)

    def value_type(self) -> int:
        return self.VALUE_TYPE

    def _run(self, weight: CudaQuantizedWeight, x: torch.Tensor, y: torch.Tensor, members: int) -> None:
        ctx = self.context
        descriptor = weight.descriptor()
        ctx.check(ctx._lib.ribn_gemv(ctx.handle, self.VALUE_TYPE, ctypes.byref(descriptor), x.data_ptr(), _dtype_code(x),
                                     x.numel(), y.data_ptr(), _dtype_code(y), y.numel(), members))

    def execute(self, weight: CudaQuantizedWeight, input: torch.Tensor, output: torch.Tensor) -> None:
        """quantized.rs:1612: one matrix-vector product; asynchronous on the context's stream."""
        self._run(weight, input, output, 1)

    def execute_warp(self, weight: CudaQuantizedWeight, input: torch.Tensor, output: torch.Tensor) -> None:
        """quantized.rs:1629.  The reference keeps a scalar and a warp kernel; here both names reach
        the same kernel."""
        self._run(weight, input, output, 1)

    def execute_warp_batch(self, weight: CudaQuantizedWeight, input: torch.Tensor, output: torch.Tensor, members: int) -> None:
        """quantized.rs:1645: `members` activation rows [members][K] -> [members][N], weights read once."""
        self._run(weight, input, output, members)

    def execute_rms_norm(self, weight: CudaQuantizedWeight, input: torch.Tensor, norm_weight: torch.Tensor, epsilon: float,
                         output: torch.Tensor, members: int) -> None:
        """rms_norm(_batch) followed by the GEMV (decode.rs:582-609) as one call: ribn_rms_norm_gemv."""
        ctx = self.context
        descriptor = weight.descriptor()
        if norm_weight.dtype != torch.float32:
            raise TypeError("RMSNorm weights are float32")
        ctx.check(ctx._lib.ribn_rms_norm_gemv(ctx.handle, self.VALUE_TYPE, ctypes.byref(descriptor), input.data_ptr(),
                                              _dtype_code(input), input.numel(), norm_weight.data_ptr(), norm_weight.numel(),
                                              ctypes.c_float(epsilon), output.data_ptr(), _dtype_code(output), output.numel(),
                                              members))

    def execute_host(self, weight: CudaQuantizedWeight, input: np.ndarray | torch.Tensor, output: np.ndarray | torch.Tensor,
                     members: int, wait: bool = True) -> None:
        """Host activations in, host outputs out (copies inside); needs context.reserve_staging().  With wait=False
        the call only enqueues (ribn_gemv_host_async): `output` is valid after context.synchronize(), and `input`
        must stay untouched (and, for the copies to be asynchronous, pinned) until then."""
        ctx = self.context
        descriptor = weight.descriptor()
        x_ptr, x_code, x_len = _host_view(input)
        y_ptr, y_code, y_len = _host_view(output)
        entry = ctx._lib.ribn_gemv_host if wait else ctx._lib.ribn_gemv_host_async
        ctx.check(entry(ctx.handle, self.VALUE_TYPE, ctypes.byref(descriptor), x_ptr, x_code, x_len, y_ptr, y_code, y_len, members))


def _host_view(t):
    if isinstance(t, torch.Tensor):
        if t.is_cuda:
            raise TypeError("execute_host takes host tensors")
        return t.data_ptr(), _dtype_code(t), t.numel()
    if t.dtype == np.float32:
        return t.ctypes.data, _lib.RIBN_F32, t.size
    if t.dtype == np.uint16:  # bf16 bit patterns
        return t.ctypes.data, _lib.RIBN_BF16, t.size
    raise TypeError(f"unsupported host dtype {t.dtype}")


class CudaQ8_0Gemv(_CudaQuantizedGemv):
    VALUE_TYPE, LABEL = 8, "Q8_0"


class CudaQ4KGemv(_CudaQuantizedGemv):
    VALUE_TYPE, LABEL = 12, "Q4_K"


class CudaQ5KGemv(_CudaQuantizedGemv):
    VALUE_TYPE, LABEL = 13, "Q5_K"


class CudaQ6KGemv(_CudaQuantizedGemv):
    VALUE_TYPE, LABEL = 14, "Q6_K"


class QwenGemvKernel:
    """staging.rs:90-217: picks the kernel object from a tensor's value type."""

    _BY_TYPE = {8: CudaQ8_0Gemv, 12: CudaQ4KGemv, 13: CudaQ5KGemv, 14: CudaQ6KGemv}

    def __init__(self, inner: _CudaQuantizedGemv):
        self.inner = inner

    @classmethod
    def from_value_type(cls, value_type: int, context: RibnContext) -> "QwenGemvKernel":
        if value_type not in cls._BY_TYPE:
            raise CudaQuantizedKernelError(_lib.RIBN_E_INVALID_WEIGHT,
                                           f"no quantized GEMV kernel for GGML value type {value_type}")
        return cls(cls._BY_TYPE[value_type](context))

    def value_type(self) -> int:
        return self.inner.value_type()

    def execute(self, weight, input, output) -> None:
        self.inner.execute(weight, input, output)

    def execute_warp(self, weight, input, output) -> None:
        self.inner.execute_warp(weight, input, output)

    def execute_warp_batch(self, weight, input, output, members: int) -> None:
        self.inner.execute_warp_batch(weight, input, output, members)


class CudaQwen35Ops:
    """The slice of model_ops.rs on the path: rms_norm / rms_norm_batch (:1714-1824)."""

    def __init__(self, context: RibnContext):
        self.context = context

    @classmethod
    def from_context(cls, context: RibnContext):
        return cls(context)

    def rms_norm(self, input: torch.Tensor, weight: torch.Tensor, output: torch.Tensor, epsilon: float) -> None:
        self.rms_norm_batch(input, weight, output, input.numel(), epsilon)

    def rms_norm_batch(self, input: torch.Tensor, weight: torch.Tensor, output: torch.Tensor, length: int,
                       epsilon: float) -> None:
        ctx = self.context
        members = input.numel() // length if length else 0
        if length and members * length != input.numel():
            raise CudaQuantizedKernelError(_lib.RIBN_E_INPUT_LENGTH,
                                           f"RMSNorm input has {input.numel()} values, not a multiple of {length}",
                                           length, input.numel())
        if weight.dtype != torch.float32:
            raise TypeError("RMSNorm weights are float32")
        ctx.check(ctx._lib.ribn_rms_norm(ctx.handle, input.data_ptr(), _dtype_code(input), input.numel(),
                                         weight.data_ptr(), weight.numel(), output.data_ptr(), _dtype_code(output),
                                         output.numel(), members, length, ctypes.c_float(epsilon)))


class CudaQ8_1Quantizer:
    """CudaQ8_1Quantizer (crates/nvidia/src/activation.rs:15-88): f32 values -> the reference's Q8_1 words, nine per
    block of 32, bit-identical to its quantize_q8_1 kernel."""

    def __init__(self, context: RibnContext):
        self.context = context

    def execute(self, input: torch.Tensor, output: torch.Tensor) -> None:
        if input.dtype != torch.float32 or output.dtype not in (torch.int32, torch.uint32):
            raise TypeError("the Q8_1 packer takes float32 values and writes 32-bit words")
        ctx = self.context
        ctx.check(ctx._lib.ribn_quantize_q8_1(ctx.handle, input.data_ptr(), input.numel(), output.data_ptr(), output.numel()))


class CudaQ8_1Gemv:
    """The integer-dot GEMV family over Q8_1 activations: CudaQ4KQ8_1Gemv (crates/nvidia/src/q4_q8_1.rs) and its
    Q5_K / Q6_K / Q8_0 twins, `execute` for one packed vector and `execute_batch` for up to eight."""

    def __init__(self, context: RibnContext, value_type: int):
        self.context, self.value_type = context, value_type

    def execute(self, weight: CudaQuantizedWeight, packed: torch.Tensor, output: torch.Tensor) -> None:
        self.execute_batch(weight, packed, output, 1)

    def execute_batch(self, weight: CudaQuantizedWeight, packed: torch.Tensor, output: torch.Tensor, members: int) -> None:
        if output.dtype != torch.float32:
            raise TypeError("the integer-dot GEMV writes float32")
        ctx = self.context
        descriptor = weight.descriptor()
        ctx.check(ctx._lib.ribn_gemv_q8_1(ctx.handle, self.value_type, ctypes.byref(descriptor), packed.data_ptr(), packed.numel(),
                                          output.data_ptr(), output.numel(), members))


def gemm(context: RibnContext, weight: CudaQuantizedWeight, input: torch.Tensor, output: torch.Tensor,
         expected_type: int = 0) -> None:
    """Prefill GEMM on the tensor cores: input bf16 [tokens, K] -> output bf16/f32 [tokens, N] (ribn_gemm)."""
    if input.dtype != torch.bfloat16:
        raise TypeError("the tensor-core GEMM takes bfloat16 activations")
    k = weight.spec().dimensions[0] if weight.spec().dimensions else 0
    tokens = input.numel() // k if k else 0
    descriptor = weight.descriptor()
    context.check(context._lib.ribn_gemm(context.handle, expected_type, ctypes.byref(descriptor), input.data_ptr(),
                                         input.numel(), output.data_ptr(), _dtype_code(output), output.numel(), tokens))


def dequantize(context: RibnContext, weight: CudaQuantizedWeight, output: torch.Tensor) -> None:
    """Device twin of engine_gguf::dequantize_block over a whole tensor -> f32 [N, K]."""
    if output.dtype != torch.float32:
        raise TypeError("dequantize writes float32")
    descriptor = weight.descriptor()
    context.check(context._lib.ribn_dequantize(context.handle, ctypes.byref(descriptor), output.data_ptr(), output.numel()))


def validate_quantized_geometry(weight: CudaQuantizedWeight, value_type: int = 0) -> tuple[int, int]:
    """quantized.rs:1755-1804; pure host code (no GPU needed).  Returns (input_size, output_size)."""
    lib = _lib.load()
    k, n = ctypes.c_uint64(), ctypes.c_uint64()
    descriptor = weight.descriptor()
    status = lib.ribn_validate_quantized_geometry(ctypes.byref(descriptor), value_type, ctypes.byref(k), ctypes.byref(n))
    if status != _lib.RIBN_OK:
        raise CudaQuantizedKernelError(status, lib.ribn_status_string(status).decode())
    return k.value, n.value


def validate_geometry_raw(value_type: int, dimensions, encoded_bytes: int, expected_type: int = 0) -> tuple[int, int]:
    """Same check on a bare descriptor (no device buffer involved)."""
    lib = _lib.load()
    dims = list(dimensions)
    descriptor = QWeight(None, encoded_bytes, value_type, len(dims), (ctypes.c_uint64 * 4)(*(dims[:4] + [0] * (4 - min(4, len(dims))))))
    k, n = ctypes.c_uint64(), ctypes.c_uint64()
    status = lib.ribn_validate_quantized_geometry(ctypes.byref(descriptor), expected_type, ctypes.byref(k), ctypes.byref(n))
    if status != _lib.RIBN_OK:
        raise CudaQuantizedKernelError(status, lib.ribn_status_string(status).decode())
    return k.value, n.value
