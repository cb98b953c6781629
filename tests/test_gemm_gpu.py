"""Tensor-core quantized GEMM (tcgen05) on the GPU, through the C ABI, against the CPU oracle.

Tolerance: max relative error 2e-3 against an f64 host product of the exactly-dequantised weights
and the bf16 activations, measured as in test_gemv_gpu (|y - ref| / max(|ref|, sqrt(sum (w*x)^2)));
a bf16 output adds one bf16 unit roundoff, 2^-8.
"""
import numpy as np
import pytest
import torch

import engine_b200
import oracle
from engine_b200 import synth

pytestmark = pytest.mark.gpu

TOL = 2e-3
BF16_ROUNDOFF = 2.0 ** -8


@pytest.fixture(params=[0, 1], ids=["f16-normalised", "gemm-kernel"], autouse=True)
def tc_kernel(request, ctx):
    """Batches of up to 64 tokens have two tensor-core kernels (the decode kernel, whose f16 operand tile is normalised
    per super-block, and the prefill GEMM, which accumulates over the whole K range in tensor memory); every test runs
    with each.  Larger batches always use the second."""
    ctx.set_option("tc_split_operands", request.param)
    yield request.param
    ctx.set_option("tc_split_operands", 0)


def upload(ctx, vt, encoded, k, n):
    store = engine_b200.CudaWeightStore(ctx)
    raw = np.ascontiguousarray(np.asarray(encoded).reshape(-1).view(np.uint8))
    store.materialize_quantized(engine_b200.WeightTensorSpec.new("w", [k, n]), vt, raw.size, raw)
    return store.quantized_tensor("w")


def run(ctx, weight, x_host, n, y_dtype=torch.float32):
    x = torch.from_numpy(x_host).to(ctx.device).to(torch.bfloat16).contiguous()
    y = torch.full((x.shape[0], n), float("nan"), dtype=y_dtype, device=ctx.device)
    engine_b200.gemm(ctx, weight, x, y)
    ctx.synchronize()
    return y.float().cpu().numpy().astype(np.float64), x.float().cpu().numpy()


def check(vt, w, k, n, y, x_seen, y_bf16=False):
    ref = oracle.gemv_f64(vt, w, k, n, x_seen)
    scale = oracle.gemv_scale(vt, w, k, n, x_seen)
    assert np.all(np.isfinite(y)), "kernel left outputs unwritten"
    err = oracle.max_rel_error(y, ref, scale)
    bound = TOL + (BF16_ROUNDOFF if y_bf16 else 0.0)
    assert err <= bound, f"max rel err {err:.3e} > {bound:.3e}"
    return err


@pytest.mark.parametrize("vt", [12, 13, 14, 8])
@pytest.mark.parametrize("n,k,m", [(128, 256, 16), (128, 512, 1), (256, 1024, 5), (100, 768, 33), (384, 2048, 64),
                                   (130, 256, 17), (512, 1024, 129), (256, 512, 300)])
def test_small_shapes(ctx, vt, n, k, m):
    w = synth.random_weight(vt, k, n, seed=vt * 31 + n + k + m)
    weight = upload(ctx, vt, w, k, n)
    x = synth.random_activations(m, k, seed=m)
    y, x_seen = run(ctx, weight, x, n)
    check(vt, w, k, n, y, x_seen)


@pytest.mark.parametrize("vt", [12, 13, 14, 8])
def test_per_row_copy_variant(ctx, vt):
    """The kernel variant that fetches raw rows with bulk copies (used when rows are not 16-byte aligned)."""
    k, n, m = 1024, 200, 24
    w = synth.random_weight(vt, k, n, seed=vt)
    weight = upload(ctx, vt, w, k, n)
    x = synth.random_activations(m, k, seed=3)
    try:
        ctx.set_option("tc_row_copies", 1)
        y, x_seen = run(ctx, weight, x, n)
    finally:
        ctx.set_option("tc_row_copies", 0)
    check(vt, w, k, n, y, x_seen)


@pytest.mark.parametrize("k", [256, 1280, 5120])
def test_q6_k_rows_that_are_not_16_byte_aligned(ctx, k):
    """210-byte blocks: K/256 not a multiple of 8 gives rows that start on 2-, 4- or 8-byte boundaries,
    and a tensor whose byte length is not a multiple of 16."""
    n, m = 131, 20
    w = synth.random_weight(14, k, n, seed=k)
    weight = upload(ctx, 14, w, k, n)
    x = synth.random_activations(m, k, seed=5)
    y, x_seen = run(ctx, weight, x, n)
    check(14, w, k, n, y, x_seen)


@pytest.mark.parametrize("ksplit", [1, 2, 3, 8])
def test_split_k_factors_agree(ctx, ksplit):
    k, n, m = 4096, 640, 48
    w = synth.random_weight(12, k, n, seed=77)
    weight = upload(ctx, 12, w, k, n)
    x = synth.random_activations(m, k, seed=7)
    try:
        ctx.set_option("tc_ksplit", ksplit)
        y, x_seen = run(ctx, weight, x, n)
        again, _ = run(ctx, weight, x, n)
    finally:
        ctx.set_option("tc_ksplit", 0)
    check(12, w, k, n, y, x_seen)
    assert np.array_equal(y, again), "split-K reduction must be deterministic and leave its tickets at zero"


def test_reference_fixture_blocks(ctx, golden):
    """The structured fixtures of the reference's tests as 5 x 768 matrices, through the GEMM."""
    for name, vt in (("q4_k", 12), ("q5_k", 13), ("q6_k", 14), ("q8_0", 8)):
        w = golden[f"struct_{name}"].reshape(-1)
        k, n = 768, 5
        x = np.array([[((i * 17 + 3 + t) % 101 - 50) * 0.0137 for i in range(k)] for t in range(9)], np.float32)
        weight = upload(ctx, vt, w, k, n)
        y, x_seen = run(ctx, weight, x, n)
        check(vt, w, k, n, y, x_seen)


# configuration 3: prefill, 12288 x 4096 Q4_K and 4096 x 12288 Q6_K, M = 512 and 2048, bf16 in and out
@pytest.mark.parametrize("vt,n,k", [(12, 12288, 4096), (14, 4096, 12288)])
@pytest.mark.parametrize("m", [512, 2048])
def test_config3_prefill(ctx, vt, n, k, m):
    w = synth.random_weight(vt, k, n, seed=vt + m)
    weight = upload(ctx, vt, w, k, n)
    x = synth.random_activations(m, k, seed=m)
    y, x_seen = run(ctx, weight, x, n, y_dtype=torch.bfloat16)
    # the f64 host reference over all output rows of a sample of tokens: every 37th, the rows either side of each
    # 256-token tile boundary, the last token, and one whole token tile (the last 128 tokens)
    edges = np.array([t for b in range(256, m, 256) for t in (b - 1, b)] + [m - 1])
    sample = np.unique(np.concatenate([np.arange(0, m, 37), edges, np.arange(m - 128, m)]))
    check(vt, w, k, n, y[sample], x_seen[sample], y_bf16=True)


def test_rejections_leave_output_untouched(ctx):
    k, n = 512, 128
    w = synth.random_weight(12, k, n, seed=1)
    weight = upload(ctx, 12, w, k, n)
    x = torch.zeros((4, k), dtype=torch.bfloat16, device=ctx.device)
    y = torch.full((4, n), 7.0, device=ctx.device)

    def kind(call):
        with pytest.raises(engine_b200.CudaQuantizedKernelError) as e:
            call()
        return e.value.kind

    assert kind(lambda: engine_b200.gemm(ctx, weight, x[:3], y)) == "OutputLength"
    assert kind(lambda: engine_b200.gemm(ctx, weight, x, y[:3])) == "OutputLength"
    assert kind(lambda: engine_b200.gemm(ctx, weight, x, y, expected_type=13)) == "UnsupportedValueType"
    q8 = synth.random_weight(8, 96, 4, seed=2)
    odd = upload(ctx, 8, q8, 96, 4)
    assert kind(lambda: engine_b200.gemm(ctx, odd, torch.zeros((2, 96), dtype=torch.bfloat16, device=ctx.device),
                                         torch.zeros((2, 4), device=ctx.device))) == "InvalidWeight"
    ctx.synchronize()
    assert torch.all(y == 7.0)
