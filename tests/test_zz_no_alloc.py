"""ribn_gemv_noalloc, the entry point for callers that may not allocate device memory (a serving loop
that owns all of HBM, a latency-critical section, a plug-in in someone else's process).  It runs the
same kernels as ribn_gemv with its scratch in a fixed device array inside the library, so its output
must equal ribn_gemv's; two calls in a row (different inputs) check that nothing stale survives in
the shared scratch.  Collected last on purpose: a failure here cannot hide any other test."""
import ctypes

import numpy as np
import pytest
import torch

import engine_b200
import oracle
from engine_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def call_noalloc(weight, x, y, members, wait=1):
    lib = _lib.load()
    message = ctypes.create_string_buffer(256)
    descriptor = weight.descriptor()
    code = lambda t: _lib.RIBN_BF16 if t.dtype == torch.bfloat16 else _lib.RIBN_F32
    status = lib.ribn_gemv_noalloc(x.device.index, ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream),
                                   ctypes.byref(descriptor), x.data_ptr(), code(x), x.numel(), y.data_ptr(), code(y),
                                   y.numel(), members, wait, message, len(message))
    return status, message.value.decode()


@pytest.mark.parametrize("vt", [12, 14])
def test_matches_ribn_gemv_on_two_calls_in_a_row(vt):
    device = torch.device("cuda", 0)
    torch.cuda.synchronize()
    k, n = 4096, 1536
    w_host = synth.random_weight(vt, k, n, seed=vt)
    w = torch.from_numpy(w_host).to(device)
    weight = engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new("w", [k, n]), vt, w)
    ctx = engine_b200.RibnContext(0)
    try:
        # ribn_gemv on the integer-dot kernel, the one the no-allocation entry point runs
        ctx.set_option("mma_gemv", 0)
        kernel = engine_b200.QwenGemvKernel.from_value_type(vt, ctx)
        for call, (members, dtype) in enumerate([(4, torch.float32), (1, torch.bfloat16)]):
            x = torch.from_numpy(synth.random_activations(members, k, seed=10 + call)).to(device).to(dtype)
            want = torch.full((members, n), float("nan"), device=device)
            kernel.execute_warp_batch(weight, x, want, members)
            ctx.synchronize()
            got = torch.full((members, n), float("nan"), device=device)
            status, message = call_noalloc(weight, x, got, members)
            assert status == _lib.RIBN_OK, message
            # same kernels, same arithmetic: the tolerance of the GEMV tests (2e-3 relative) is met with equality
            assert torch.equal(got, want)
            # and against the CPU oracle's f64 product, with the GEMV tests' bound
            seen = x.float().cpu().numpy()
            error = oracle.max_rel_error(got.cpu().numpy(), oracle.gemv_f64(vt, w_host, k, n, seen), oracle.gemv_scale(vt, w_host, k, n, seen))
            assert error <= 2e-3, error
    finally:
        ctx.close()


def test_refuses_sizes_beyond_the_fixed_scratch():
    device = torch.device("cuda", 0)
    k, n = 32768, 8
    w = torch.from_numpy(synth.random_weight(12, k, n, seed=1)).to(device)
    weight = engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new("w", [k, n]), 12, w)
    x = torch.zeros((4, k), device=device)
    y = torch.full((4, n), 7.0, device=device)
    status, message = call_noalloc(weight, x, y, 4)
    assert status == _lib.RIBN_E_SHAPE_OVERFLOW and "exceeds the fixed scratch" in message
    status, _ = call_noalloc(weight, x[:1], y, 5)
    assert status == _lib.RIBN_E_INVALID_WEIGHT
    torch.cuda.synchronize()
    assert torch.all(y == 7.0)


def test_refuses_buffers_that_are_not_device_memory():
    """A host pointer handed to the kernels would fault the GPU: it is refused before anything is enqueued."""
    device = torch.device("cuda", 0)
    k, n = 512, 32
    w = torch.from_numpy(synth.random_weight(12, k, n, seed=2)).to(device)
    weight = engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new("w", [k, n]), 12, w)
    y = torch.full((n,), 7.0, device=device)
    host_x = torch.zeros(k).pin_memory()
    lib = _lib.load()
    message = ctypes.create_string_buffer(256)
    descriptor = weight.descriptor()
    status = lib.ribn_gemv_noalloc(0, ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream), ctypes.byref(descriptor),
                                   host_x.data_ptr(), _lib.RIBN_F32, k, y.data_ptr(), _lib.RIBN_F32, n, 1, 1, message, len(message))
    assert status == _lib.RIBN_E_CONTEXT_MISMATCH, message.value
    torch.cuda.synchronize()
    assert torch.all(y == 7.0)


def test_status_reader_after_an_enqueue_only_call():
    device = torch.device("cuda", 0)
    k, n = 1024, 64
    w = torch.from_numpy(synth.random_weight(12, k, n, seed=3)).to(device)
    weight = engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new("w", [k, n]), 12, w)
    x = torch.randn(2, k, device=device)
    y = torch.full((2, n), float("nan"), device=device)
    status, message = call_noalloc(weight, x, y, 2, wait=0)
    assert status == _lib.RIBN_OK, message
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    assert _lib.load().ribn_noalloc_status(0, stream) == _lib.RIBN_OK
    assert torch.isfinite(y).all()
