"""Runs the reference project's own CUDA kernels (compiled by build_ref.py into oracle/_ref/) on this GPU.

TEST / BASELINE INFRASTRUCTURE ONLY: the shipped library never loads these cubins.  The launch
geometry is the reference host code's:

    q*_gemv_warp         one warp per weight row, 4 warps per block        (quantized.rs:395-425)
    q*_gemv_warp_batch   one warp per MAX_BATCH_ROWS = 2 rows, 4 warps per block, members <= 8
                         (quantized.rs:268-318, :445-487); larger batches are served the way the
                         reference's prefill does it, eight members per launch (decode.rs:1953-1977)
    rms_norm             one block of 256 threads per vector                (model_ops.rs:1714-1768)

Inputs and outputs are f32 torch tensors on the current CUDA device; launches go to torch's current
stream, so they can be captured into a CUDA graph and timed with CUDA events like our own kernels.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
QUANTIZED_CUBIN = os.path.join(_HERE, "_ref", "ref_quantized.cubin")
MODEL_OPS_CUBIN = os.path.join(_HERE, "_ref", "ref_model_ops.cubin")

FAMILY = {8: "q8_0", 12: "q4_k", 13: "q5_k", 14: "q6_k"}
MAX_BATCH_MEMBERS = 8
MAX_BATCH_ROWS = 2


def available() -> bool:
    return os.path.exists(QUANTIZED_CUBIN)


def _check(result):
    code = result[0]
    if int(code) != 0:
        raise RuntimeError(f"CUDA driver call failed with {code}")
    return result[1] if len(result) == 2 else result[1:]


class ReferenceKernels:
    """The reference's GEMV kernels, loaded from the cubin with the driver API."""

    def __init__(self):
        import torch
        from cuda.bindings import driver

        if not available():
            raise FileNotFoundError(f"{QUANTIZED_CUBIN} is missing: run oracle/build_ref.py where the reference tree is mounted")
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # make torch's primary context current
        self._driver = driver
        self._torch = torch
        with open(QUANTIZED_CUBIN, "rb") as f:
            image = f.read()
        self._image = image  # keep alive
        self._module = _check(driver.cuModuleLoadData(image))
        self._functions = {}

    def _function(self, name: str):
        if name not in self._functions:
            self._functions[name] = _check(self._driver.cuModuleGetFunction(self._module, name.encode()))
        return self._functions[name]

    def _launch(self, name, blocks, threads, pointers, ints):
        driver = self._driver
        stream = self._torch.cuda.current_stream().cuda_stream
        arguments = (tuple(pointers) + tuple(ints), (ctypes.c_void_p,) * len(pointers) + (ctypes.c_int,) * len(ints))
        _check(driver.cuLaunchKernel(self._function(name), blocks, 1, 1, threads, 1, 1, 0, stream, arguments, 0))

    def gemv_warp(self, value_type: int, weights, x, y, k: int, n: int) -> None:
        """y[n] = W x with the reference's default decode kernel (one member)."""
        self._launch(f"{FAMILY[value_type]}_gemv_warp", (n + 3) // 4, 128, [weights.data_ptr(), x.data_ptr(), y.data_ptr()], [k, n])

    def gemv_warp_batch(self, value_type: int, weights, x, y, k: int, n: int, members: int) -> None:
        """y[m][n] for any member count: eight members per launch, as the reference's prefill loop does."""
        warps = (n + MAX_BATCH_ROWS - 1) // MAX_BATCH_ROWS
        for first in range(0, members, MAX_BATCH_MEMBERS):
            count = min(MAX_BATCH_MEMBERS, members - first)
            self._launch(f"{FAMILY[value_type]}_gemv_warp_batch", (warps + 3) // 4, 128,
                         [weights.data_ptr(), x.data_ptr() + first * k * 4, y.data_ptr() + first * n * 4], [k, n, count])

    def gemv(self, value_type: int, weights, x, y, k: int, n: int, members: int) -> None:
        """What the reference's decode calls for this batch (decode.rs:1480-1558): warp kernel for one member, batch kernel otherwise."""
        if members == 1:
            self.gemv_warp(value_type, weights, x, y, k, n)
        else:
            self.gemv_warp_batch(value_type, weights, x, y, k, n, members)


def launches_for(members: int) -> int:
    return 1 if members == 1 else (members + MAX_BATCH_MEMBERS - 1) // MAX_BATCH_MEMBERS


def as_numpy(t) -> np.ndarray:
    return t.detach().cpu().numpy()
