"""Our GEMV against the reference project's own CUDA kernels on the same GPU and the same bytes.

The reference kernels are the cubins that oracle/build_ref.py compiles from the mounted reference tree
(q*_gemv_warp and q*_gemv_warp_batch of crates/nvidia/src/kernels/quantized/*.cu); where they were not
built the tests skip.  Both sides must agree with the f64 oracle within the bound of the path, and with
each other within twice that bound.
"""
import numpy as np
import pytest
import torch

import engine_b200
import oracle
from engine_b200 import synth
from oracle import ref_cuda

pytestmark = pytest.mark.gpu

TOL = 2e-3


@pytest.fixture(scope="module")
def reference():
    if not ref_cuda.available():
        pytest.skip("reference cubins not built (oracle/build_ref.py needs the reference tree)")
    return ref_cuda.ReferenceKernels()


@pytest.mark.parametrize("vt", [8, 12, 13, 14])
@pytest.mark.parametrize("members", [1, 3, 8, 16])
def test_gemv_matches_reference_kernels(ctx, reference, vt, members):
    k, n = 2048, 515
    w = synth.random_weight(vt, k, n, seed=vt * 7 + members)
    x = synth.random_activations(members, k, seed=members)
    wd = torch.from_numpy(w).to(ctx.device)
    xd = torch.from_numpy(x).to(ctx.device)
    weight = engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new("w", [k, n]), vt, wd)

    y_ref = torch.full((members, n), float("nan"), device=ctx.device)
    reference.gemv(vt, wd, xd, y_ref, k, n, members)
    torch.cuda.synchronize()

    y = torch.full((members, n), float("nan"), device=ctx.device)
    kernel = engine_b200.QwenGemvKernel.from_value_type(vt, ctx)
    if members == 1:
        kernel.execute_warp(weight, xd.reshape(-1), y.reshape(-1))
    else:
        kernel.execute_warp_batch(weight, xd, y, members)
    ctx.synchronize()

    exact = oracle.gemv_f64(vt, w, k, n, x)
    scale = oracle.gemv_scale(vt, w, k, n, x)
    ours = y.cpu().numpy().astype(np.float64)
    theirs = y_ref.cpu().numpy().astype(np.float64)
    assert np.all(np.isfinite(theirs)), "the reference kernel left outputs unwritten"
    assert oracle.max_rel_error(theirs, exact, scale) <= TOL
    assert oracle.max_rel_error(ours, exact, scale) <= TOL
    assert oracle.max_rel_error(ours, theirs, scale) <= 2 * TOL


def test_dequantize_matches_reference_gemv_on_unit_vectors(ctx, reference):
    """The reference has no device dequantiser; its GEMV against unit vectors reads single weights back."""
    vt, k, n = 12, 256, 64
    w = synth.random_weight(vt, k, n, seed=5)
    wd = torch.from_numpy(w).to(ctx.device)
    weight = engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new("w", [k, n]), vt, wd)
    out = torch.empty(n * k, device=ctx.device)
    engine_b200.dequantize(ctx, weight, out)
    ctx.synchronize()
    ours = out.cpu().numpy().reshape(n, k)
    for column in (0, 31, 32, 100, 255):
        x = torch.zeros(k, device=ctx.device)
        x[column] = 1.0
        y = torch.empty(n, device=ctx.device)
        reference.gemv_warp(vt, wd, x, y, k, n)
        torch.cuda.synchronize()
        assert np.array_equal(y.cpu().numpy(), ours[:, column])


# ---- the reference's decode step, composed from its own kernels (oracle/ref_decode.py), against ours on the same model
@pytest.mark.parametrize("members", [1, 3])
def test_decode_step_matches_the_reference_kernels_composition(members):
    from engine_b200 import decode
    from oracle import ref_decode

    if not ref_cuda.available():
        pytest.skip("reference cubins not built (oracle/build_ref.py needs the reference tree)")
    stream = torch.cuda.Stream()
    context = engine_b200.RibnContext(0, stream=stream)
    try:
        geometry = decode.DenseGeometry(hidden=1024, layers=2, q_heads=8, kv_heads=2, head_dim=128, intermediate=1536, vocabulary=777)
        weights = decode.random_weights(context, geometry, seed=5)
        ours = decode.CudaDenseDecode(context, geometry, weights, members, 16)
        theirs = ref_decode.ReferenceDenseDecode(geometry, weights, members, 16, context.device)
        token = 123
        for position in range(4):
            ours.tokens.fill_(token)
            ours.positions.fill_(position)
            ours.run_step()
            context.synchronize()
            with torch.cuda.stream(stream):
                theirs.step(token, position)
            torch.cuda.synchronize()
            a, b = ours.logits.cpu().numpy(), theirs.logits.cpu().numpy()
            scale = np.max(np.abs(b))
            assert np.max(np.abs(a - b)) <= 2e-3 * scale, (position, float(np.max(np.abs(a - b)) / scale))
            assert np.array_equal(ours.next_tokens.cpu().numpy(), theirs.selected.cpu().numpy())
            token = int(theirs.selected[0])
    finally:
        context.close()
