"""RMSNorm on the GPU, through the C ABI, against the host equation
(crates/nvidia/src/qwen_reference.rs:550-556 of the reference project).  Tolerance 1e-5 absolute on
O(1) values, the bound of the reference's own device test (tests/cuda_reference.rs:969-987); a bf16
output adds one bf16 unit roundoff (2^-8 relative)."""
import numpy as np
import pytest
import torch

import engine_b200
import oracle

pytestmark = pytest.mark.gpu


def run(ctx, x, w, eps, length, x_dtype=torch.float32, y_dtype=torch.float32):
    ops = engine_b200.CudaQwen35Ops.from_context(ctx)
    xd = torch.from_numpy(x).to(ctx.device).to(x_dtype).contiguous()
    wd = torch.from_numpy(w).to(ctx.device)
    yd = torch.full(xd.shape, float("nan"), dtype=y_dtype, device=ctx.device)
    if xd.numel() == length:
        ops.rms_norm(xd.reshape(-1), wd, yd.reshape(-1), eps)
    else:
        ops.rms_norm_batch(xd, wd, yd, length, eps)
    ctx.synchronize()
    return yd.float().cpu().numpy(), xd.float().cpu().numpy()


def test_known_answer(ctx, golden):
    y, _ = run(ctx, golden["rms_input"], golden["rms_weight"], float(golden["rms_eps"][0]), 4)
    assert np.max(np.abs(y - golden["rms_expect"])) < 1e-5


@pytest.mark.parametrize("length", [1, 3, 4, 5, 127, 4096, 5120, 8192, 8200, 20000])
@pytest.mark.parametrize("members", [1, 2, 64])
def test_against_host_equation(ctx, length, members):
    rng = np.random.default_rng(length + members)
    x = rng.standard_normal((members, length)).astype(np.float32) * 3.0
    w = (1.0 + 0.02 * rng.standard_normal(length)).astype(np.float32)
    y, x_seen = run(ctx, x, w, 1e-6, length)
    want = oracle.rms_norm(x_seen, w, 1e-6)
    assert np.max(np.abs(y - want)) < 1e-5 * max(1.0, float(np.max(np.abs(want))))


@pytest.mark.parametrize("x_dtype,y_dtype", [(torch.bfloat16, torch.float32), (torch.float32, torch.bfloat16),
                                             (torch.bfloat16, torch.bfloat16)])
def test_bf16_variants(ctx, x_dtype, y_dtype):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((8, 4096)).astype(np.float32)
    w = (1.0 + 0.02 * rng.standard_normal(4096)).astype(np.float32)
    y, x_seen = run(ctx, x, w, 1e-6, 4096, x_dtype, y_dtype)
    want = oracle.rms_norm(x_seen, w, 1e-6)
    tol = 1e-5 + (2.0 ** -8 if y_dtype == torch.bfloat16 else 0.0)
    assert np.max(np.abs(y - want) / np.maximum(np.abs(want), 1.0)) < tol


def test_rejections(ctx):
    ops = engine_b200.CudaQwen35Ops.from_context(ctx)
    x = torch.ones(8, device=ctx.device)
    w = torch.ones(4, device=ctx.device)
    y = torch.full((8,), 7.0, device=ctx.device)

    def kind(call):
        with pytest.raises(engine_b200.CudaQuantizedKernelError) as e:
            call()
        return e.value.kind

    assert kind(lambda: ops.rms_norm(x, w, y, 1e-6)) == "InputLength"          # weight length != vector length
    assert kind(lambda: ops.rms_norm_batch(x, w, y[:4], 4, 1e-6)) == "OutputLength"
    assert kind(lambda: ops.rms_norm_batch(x[:6], w, y[:6], 4, 1e-6)) == "InputLength"
    assert kind(lambda: ops.rms_norm_batch(x, w, y, 0, 1e-6)) == "InputLength"
    ctx.synchronize()
    assert torch.all(y == 7.0)
