"""The Q8_1 compatibility mode on the device, through the C ABI: the packer against the reference's byte known-answers
(crates/nvidia/tests/cuda_activation.rs:14-70) and the host packer model, the integer-dot GEMV against the packed host
arithmetic within the reference tests' own allowances (crates/nvidia/tests/q4_q8_1.rs:255-296, :353-410 and twins)."""
import numpy as np
import pytest
import torch

import engine_b200
from engine_b200 import synth
from oracle import q8_1_np
from test_q8_1 import FORMATS, GOLDEN, INPUTS, ROWS, activations, check_kat_words, kat_values

pytestmark = pytest.mark.gpu


def dev(ctx, array):
    return torch.from_numpy(np.ascontiguousarray(array)).to(ctx.device)


def pack_on_device(ctx, values: np.ndarray, fill: int = -1) -> np.ndarray:
    out = torch.full((values.size // 32 * 9,), fill, dtype=torch.int32, device=ctx.device)
    engine_b200.CudaQ8_1Quantizer(ctx).execute(dev(ctx, values.reshape(-1)), out)
    ctx.synchronize()
    return out.cpu().numpy().view(np.uint32)


def test_packs_q8_1_layout_rounding_and_partial_launch(ctx):
    words = pack_on_device(ctx, kat_values())
    check_kat_words(words)
    assert np.array_equal(pack_on_device(ctx, kat_values()), words)          # scratch reuse on the same stream


def test_packer_is_bit_identical_to_the_host_model(ctx):
    rng = np.random.default_rng(3)
    cases = [activations(True), activations(False), np.zeros(INPUTS, np.float32),
             (rng.standard_normal(32 * 4099) * np.exp(rng.standard_normal(32 * 4099))).astype(np.float32),    # many CTAs, a partial last one
             np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5] + [127.0] + [0.0] * 25, np.float32)]                  # ties round away from zero
    for values in cases:
        assert np.array_equal(pack_on_device(ctx, values), q8_1_np.pack_q8_1(values))


def test_rejects_invalid_q8_1_storage_before_launch(ctx):
    quantizer = engine_b200.CudaQ8_1Quantizer(ctx)
    words = lambda n: torch.zeros(n, dtype=torch.int32, device=ctx.device)
    for count, out, kind in ((31, 9, "InputLength"), (32, 8, "OutputLength"), (0, 9, "InputLength")):
        with pytest.raises(engine_b200.CudaQuantizedKernelError) as e:
            quantizer.execute(torch.zeros(count, device=ctx.device), words(out))
        assert e.value.kind == kind


def weight_of(ctx, name):
    vt = FORMATS[name]
    return engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new(name, [INPUTS, ROWS]), vt, dev(ctx, GOLDEN[f"struct_{name}"]))


@pytest.mark.parametrize("name", list(FORMATS))
def test_integer_dot_matches_packed_host_arithmetic_and_float_error_bound(ctx, name):
    vt, weight = FORMATS[name], weight_of(ctx, name)
    kernel = engine_b200.CudaQ8_1Gemv(ctx, vt)
    for values in (activations(True), activations(False), np.zeros(INPUTS, np.float32)):
        packed = pack_on_device(ctx, values)
        y = torch.full((ROWS,), 7.0, device=ctx.device)
        kernel.execute(weight, dev(ctx, packed.view(np.int32)), y)
        ctx.synchronize()
        want = q8_1_np.gemv_q8_1(vt, GOLDEN[f"struct_{name}"], INPUTS, ROWS, values, packed)
        got = y.cpu().numpy().astype(np.float64)
        rounding = q8_1_np.rounding_allowance(want["arithmetic_magnitude"][0])
        assert np.all(np.abs(got - want["packed_output"][0]) <= rounding)
        assert np.all(np.abs(got - want["float_output"][0]) <= want["packing_error_bound"][0] + rounding)


@pytest.mark.parametrize("name", list(FORMATS))
def test_batch_matches_per_member_host_arithmetic(ctx, name):
    vt, weight = FORMATS[name], weight_of(ctx, name)
    members = [activations(True), activations(False), np.zeros(INPUTS, np.float32)]
    packed = pack_on_device(ctx, np.concatenate(members))                      # one linear stream covers the batch
    y = torch.zeros(len(members) * ROWS, device=ctx.device)
    engine_b200.CudaQ8_1Gemv(ctx, vt).execute_batch(weight, dev(ctx, packed.view(np.int32)), y, len(members))
    ctx.synchronize()
    got = y.cpu().numpy().astype(np.float64).reshape(len(members), ROWS)
    for m, values in enumerate(members):
        words = packed.reshape(len(members), -1)[m]
        assert np.array_equal(words, q8_1_np.pack_q8_1(values))
        want = q8_1_np.gemv_q8_1(vt, GOLDEN[f"struct_{name}"], INPUTS, ROWS, values, words)
        rounding = q8_1_np.rounding_allowance(want["arithmetic_magnitude"][0])
        assert np.all(np.abs(got[m] - want["packed_output"][0]) <= rounding)
        assert np.all(np.abs(got[m] - want["float_output"][0]) <= want["packing_error_bound"][0] + rounding)


@pytest.mark.parametrize("vt,k,n,members", [(12, 4096, 1000, 8), (13, 1024, 77, 5), (14, 2048, 130, 8), (8, 4096 + 32, 65, 3), (14, 256, 1, 1)])
def test_random_weights_all_member_counts(ctx, vt, k, n, members):
    rng = np.random.default_rng(vt + members)
    encoded = synth.random_weight(vt, k, n, seed=vt)
    weight = engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new("w", [k, n]), vt, dev(ctx, encoded))
    x = rng.standard_normal((members, k)).astype(np.float32)
    packed = pack_on_device(ctx, x)
    y = torch.zeros(members * n, device=ctx.device)
    engine_b200.CudaQ8_1Gemv(ctx, vt).execute_batch(weight, dev(ctx, packed.view(np.int32)), y, members)
    ctx.synchronize()
    want = q8_1_np.gemv_q8_1(vt, encoded, k, n, x, packed)
    got = y.cpu().numpy().astype(np.float64).reshape(members, n)
    assert np.all(np.abs(got - want["packed_output"]) <= q8_1_np.rounding_allowance(want["arithmetic_magnitude"]))


def test_rejects_invalid_storage(ctx):
    weight = engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new("q4", [256, 1]), 12, dev(ctx, GOLDEN["struct_q4_k"].reshape(-1)[:144]))
    kernel = engine_b200.CudaQ8_1Gemv(ctx, 12)
    words = lambda n: torch.zeros(n, dtype=torch.int32, device=ctx.device)
    y = torch.tensor([1.0, 2.0], device=ctx.device)
    for packed, out, members, kind in ((words(71), y[:1], 1, "InputLength"), (words(72), y, 1, "OutputLength"), (words(144), y, 0, "InputLength"),
                                       (words(144), y, 9, "InvalidWeight"), (words(143), y, 2, "InputLength"),
                                       (words(144), torch.zeros(3, device=ctx.device), 2, "OutputLength")):
        with pytest.raises(engine_b200.CudaQuantizedKernelError) as e:
            kernel.execute_batch(weight, packed, out, members)
        assert e.value.kind == kind
    with pytest.raises(engine_b200.CudaQuantizedKernelError) as e:
        engine_b200.CudaQ8_1Gemv(ctx, 8).execute(weight, words(72), y[:1])
    assert e.value.kind == "UnsupportedValueType"
    ctx.synchronize()
    assert y.cpu().tolist() == [1.0, 2.0]
