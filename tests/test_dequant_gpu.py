"""Bit-exact dequantisation on the GPU, through the C ABI, against the CPU oracle and the golden
fixtures of the reference's tests."""
import numpy as np
import pytest
import torch

import engine_b200
import oracle
from engine_b200 import synth

pytestmark = pytest.mark.gpu

TYPES = {"q8_0": 8, "q4_k": 12, "q5_k": 13, "q6_k": 14}


def bits(a):
    return np.asarray(a, np.float32).view(np.uint32)


def device_dequant(ctx, vt, encoded, k, n):
    store = engine_b200.CudaWeightStore(ctx)
    spec = engine_b200.WeightTensorSpec.new("w", [k, n])
    raw = np.ascontiguousarray(np.asarray(encoded).reshape(-1).view(np.uint8))
    store.materialize_quantized(spec, vt, raw.size, raw)
    out = torch.full((n, k), float("nan"), dtype=torch.float32, device=ctx.device)
    engine_b200.dequantize(ctx, store.quantized_tensor("w"), out)
    ctx.synchronize()
    return out.cpu().numpy()


def test_known_answer_blocks(ctx, golden):
    q8 = device_dequant(ctx, 8, golden["kat_q8_0"], 32, 1)[0]
    assert np.array_equal(bits(q8[:2]), bits(golden["kat_q8_0_expect_head"]))
    q4 = device_dequant(ctx, 12, golden["kat_q4_k"], 256, 1)[0]
    assert np.array_equal(bits([q4[0], q4[32]]), bits(golden["kat_q4_k_expect"]))
    q5 = device_dequant(ctx, 13, golden["kat_q5_k"], 256, 1)[0]
    assert np.array_equal(bits([q5[0], q5[32]]), bits(golden["kat_q5_k_expect"]))
    q6 = device_dequant(ctx, 14, golden["kat_q6_k"], 256, 1)[0]
    assert np.all(bits(q6) == bits(golden["kat_q6_k_expect_all"])[0])


@pytest.mark.parametrize("name", list(TYPES))
def test_structured_fixtures_exact(ctx, golden, name):
    vt = TYPES[name]
    blocks = golden[f"struct_{name}"]
    elements, _ = engine_b200.tensor_layout(vt)
    got = device_dequant(ctx, vt, blocks, elements, len(blocks))
    assert np.array_equal(bits(got), bits(golden[f"struct_{name}_expect"]))


@pytest.mark.parametrize("name", list(TYPES))
def test_gemv_fixture_blocks_exact(ctx, golden, name):
    vt = TYPES[name]
    k, n = (int(v) for v in golden[f"gemv_{name}_shape"])
    got = device_dequant(ctx, vt, golden[f"gemv_{name}"], k, n)
    assert np.array_equal(bits(got), bits(golden[f"gemv_{name}_dequant"]))


@pytest.mark.parametrize("vt", [8, 12, 13, 14])
@pytest.mark.parametrize("k,n", [(256, 1), (768, 5), (4096, 33), (5120, 7)])
def test_synthetic_bit_exact(ctx, vt, k, n):
    w = synth.random_weight(vt, k, n, seed=1000 * vt + k + n)
    want = oracle.dequantize(vt, w, k, n)
    got = device_dequant(ctx, vt, w, k, n)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("k,n", [(32, 1), (64, 3), (96, 5), (288, 4), (4128, 3)])
def test_q8_0_rows_that_end_inside_a_super_block(ctx, k, n):
    w = synth.random_weight(8, k, n, seed=k)
    assert np.array_equal(bits(device_dequant(ctx, 8, w, k, n)), bits(oracle.dequantize(8, w, k, n)))


@pytest.mark.parametrize("vt", [8, 12, 13, 14])
def test_random_bytes_bit_exact_where_finite(ctx, vt):
    """Arbitrary bytes, including negative, subnormal, infinite and NaN f16 scales: identical bits
    wherever the reference value is not NaN, NaN exactly where it is NaN."""
    elements, block_bytes = engine_b200.tensor_layout(vt)
    rows = 512
    per_row = 4 if vt != 8 else 8
    data = np.random.default_rng(77 + vt).integers(0, 256, size=rows * per_row * block_bytes, dtype=np.uint8)
    k = per_row * elements
    want = oracle.dequantize(vt, data, k, rows)
    got = device_dequant(ctx, vt, data, k, rows)
    nan = np.isnan(want)
    assert np.array_equal(nan, np.isnan(got))
    assert np.array_equal(bits(got)[~nan], bits(want)[~nan])


def test_full_size_config_shape_matches_oracle(ctx):
    """Config-1 shape: 4096 x 4096 Q4_K, seed 0, every one of the 16.7 M weights bit-exact."""
    w = synth.random_weight(12, 4096, 4096, seed=0)
    want = oracle.dequantize(12, w, 4096, 4096)
    got = device_dequant(ctx, 12, w, 4096, 4096)
    assert np.array_equal(bits(got), bits(want))


def test_rejections_leave_output_untouched(ctx):
    store = engine_b200.CudaWeightStore(ctx)
    w = synth.random_weight(12, 256, 2, seed=5)
    store.materialize_quantized(engine_b200.WeightTensorSpec.new("w", [256, 2]), 12, w.size, w)
    weight = store.quantized_tensor("w")
    out = torch.full((3, 256), 7.0, dtype=torch.float32, device=ctx.device)
    with pytest.raises(engine_b200.CudaQuantizedKernelError) as e:
        engine_b200.dequantize(ctx, weight, out)
    assert e.value.kind == "OutputLength" and (e.value.expected, e.value.actual) == (512, 768)
    bad = engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new("b", [256, 3]), 12, weight.encoded_data())
    with pytest.raises(engine_b200.CudaQuantizedKernelError) as e:
        engine_b200.dequantize(ctx, bad, out)
    assert e.value.kind == "InvalidWeight"
    ctx.synchronize()
    assert torch.all(out == 7.0)
