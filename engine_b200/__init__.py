"""engine_b200: B200 (sm_100a) kernels for the GGUF block-quantized matmul path behind a C ABI.

`include/ribn_b200.h` is the product boundary; this package is the Python host mirror of the
reference's kernel wrapper objects over that boundary, plus the build recipe.
"""
from . import _lib
from .quantized import (
    CudaQ4KGemv,
    CudaQ5KGemv,
    CudaQ6KGemv,
    CudaQ8_0Gemv,
    CudaQ8_1Gemv,
    CudaQ8_1Quantizer,
    CudaQuantizedKernelError,
    CudaQuantizedWeight,
    CudaQwen35Ops,
    CudaWeightStore,
    QwenGemvKernel,
    RibnContext,
    WeightTensorSpec,
    dequantize,
    gemm,
    tensor_layout,
    validate_geometry_raw,
    validate_quantized_geometry,
)

__all__ = [
    "CudaQ4KGemv", "CudaQ5KGemv", "CudaQ6KGemv", "CudaQ8_0Gemv", "CudaQ8_1Gemv", "CudaQ8_1Quantizer", "CudaQuantizedKernelError",
    "CudaQuantizedWeight", "CudaQwen35Ops", "CudaWeightStore", "QwenGemvKernel", "RibnContext",
    "WeightTensorSpec", "dequantize", "gemm", "tensor_layout", "validate_geometry_raw",
    "validate_quantized_geometry",
]
