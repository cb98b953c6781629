"""Pins the CPU oracle (oracle/ribn_oracle.c and its numpy twin) to the fixtures the reference's own
tests hold for the path.  No GPU.  Citations are file:line inside the reference project."""
import numpy as np
import pytest

import oracle
from oracle import oracle_np

TYPES = {"q8_0": 8, "q4_k": 12, "q5_k": 13, "q6_k": 14}


def bits(a):
    return np.asarray(a, np.float32).view(np.uint32)


# crates/gguf/src/lib.rs:1369-1455
def test_known_answer_blocks(golden):
    q8 = oracle.dequantize_block(8, golden["kat_q8_0"])
    assert len(q8) == 32 and np.array_equal(bits(q8[:2]), bits(golden["kat_q8_0_expect_head"]))
    q4 = oracle.dequantize_block(12, golden["kat_q4_k"])
    assert len(q4) == 256 and np.array_equal(bits([q4[0], q4[32]]), bits(golden["kat_q4_k_expect"]))
    q5 = oracle.dequantize_block(13, golden["kat_q5_k"])
    assert len(q5) == 256 and np.array_equal(bits([q5[0], q5[32]]), bits(golden["kat_q5_k_expect"]))
    q6 = oracle.dequantize_block(14, golden["kat_q6_k"])
    assert len(q6) == 256 and np.all(bits(q6) == bits(golden["kat_q6_k_expect_all"])[0])
    f32 = oracle.dequantize_block(0, np.array([1.5], np.float32).view(np.uint8))
    assert bits(f32)[0] == bits([1.5])[0]
    f16 = oracle.dequantize_block(1, np.array([0x3C00], np.uint16).view(np.uint8))
    assert bits(f16)[0] == bits([1.0])[0]


# crates/gguf/src/lib.rs:1457-1472
def test_rejects_invalid_blocks():
    with pytest.raises(oracle.OracleError) as short:
        oracle.dequantize_block(12, np.zeros(143, np.uint8))
    assert short.value.status == 2
    with pytest.raises(oracle.OracleError) as unsupported:
        oracle.dequantize_block(22, np.zeros(82, np.uint8))
    assert unsupported.value.status == 1
    with pytest.raises(oracle.OracleError):
        oracle.tensor_layout(99)


# crates/gguf/src/lib.rs:1474-1514 and the size table :1051-1083
def test_block_size_table():
    assert oracle.tensor_layout(8) == (32, 34)
    assert oracle.tensor_layout(12) == (256, 144)
    assert oracle.tensor_layout(13) == (256, 176)
    assert oracle.tensor_layout(14) == (256, 210)
    assert oracle.tensor_layout(23) == (256, 136)
    assert oracle.tensor_layout(21) == (256, 110)
    for vt, layout in oracle_np.BLOCK_LAYOUT.items():
        assert oracle.tensor_layout(vt) == layout
    # a [128, 2] Q4_K tensor does not split into whole blocks (QuantizationDimensionMismatch)
    with pytest.raises(oracle.OracleError):
        oracle.gemv_f32(12, np.zeros(144, np.uint8), 128, 2, np.zeros((1, 128), np.float32))


# crates/nvidia/tests/q4_q8_1.rs:205-228 and the q5/q6/q8_0 twins: decoder == closed form, exactly
@pytest.mark.parametrize("name", list(TYPES))
def test_structured_fixtures_exact(golden, name):
    vt = TYPES[name]
    blocks = golden[f"struct_{name}"]
    expect = golden[f"struct_{name}_expect"]
    elements, _ = oracle.tensor_layout(vt)
    for i, block in enumerate(blocks):
        got = oracle.dequantize_block(vt, block)
        assert np.array_equal(bits(got), bits(expect[i])), (name, i)
    got_np = oracle_np.dequantize_blocks(vt, blocks.reshape(-1))
    assert np.array_equal(bits(got_np), bits(expect))
    whole = oracle.dequantize(vt, blocks.reshape(-1), elements, len(blocks))
    assert np.array_equal(bits(whole), bits(expect))


# crates/nvidia/tests/cuda_reference.rs:750-960: sum of decoded weight * x, tolerance 1e-3 absolute
@pytest.mark.parametrize("name", list(TYPES))
def test_gemv_fixtures(golden, name):
    vt = TYPES[name]
    k, n = (int(v) for v in golden[f"gemv_{name}_shape"])
    encoded, x = golden[f"gemv_{name}"], golden[f"gemv_{name}_input"]
    assert np.array_equal(bits(oracle.dequantize(vt, encoded, k, n)), bits(golden[f"gemv_{name}_dequant"]))
    y32 = oracle.gemv_f32(vt, encoded, k, n, x[None, :])[0]
    y64 = oracle.gemv_f64(vt, encoded, k, n, x[None, :])[0]
    assert np.max(np.abs(y32 - golden[f"gemv_{name}_expect"])) < 1e-3
    assert np.allclose(y64, golden[f"gemv_{name}_expect"], rtol=1e-12, atol=1e-12)


# crates/nvidia/tests/cuda_reference.rs:969-987
def test_rms_norm_known_answer(golden):
    got = oracle.rms_norm(golden["rms_input"], golden["rms_weight"], float(golden["rms_eps"][0]))
    assert np.max(np.abs(got - golden["rms_expect"])) < 1e-5
    got_np = oracle_np.rms_norm(golden["rms_input"], golden["rms_weight"], float(golden["rms_eps"][0]))
    assert np.array_equal(bits(got), bits(got_np))


# crates/nvidia/src/model_ops_tests.rs:3-58: every binary16 pattern
def test_f16_exhaustive():
    patterns = np.arange(65536, dtype=np.uint16)
    mine = np.array([oracle.f16_to_f32(int(p)) for p in patterns], np.float32)
    want = patterns.view(np.float16).astype(np.float32)
    finite = ~np.isnan(want)
    assert np.array_equal(bits(mine[finite]), bits(want[finite]))
    assert np.all(bits(mine[~finite]) == 0x7FC00000)  # every NaN becomes the canonical quiet NaN


def test_scale_unpack_roundtrip():
    from engine_b200 import synth

    rng = np.random.default_rng(3)
    scales = rng.integers(0, 64, (64, 8), dtype=np.uint8)
    minima = rng.integers(0, 64, (64, 8), dtype=np.uint8)
    packed = synth.pack_q4_k_scales(scales, minima)
    s2, m2 = oracle_np.q4_k_scales(packed)
    assert np.array_equal(s2, scales) and np.array_equal(m2, minima)


@pytest.mark.parametrize("vt", [8, 12, 13, 14])
def test_c_oracle_matches_numpy_twin_on_random_bytes(vt):
    elements, block_bytes = oracle.tensor_layout(vt)
    rng = np.random.default_rng(vt)
    data = rng.integers(0, 256, size=(4096, block_bytes), dtype=np.uint8)
    a = oracle.dequantize(vt, data, elements, 4096)
    b = oracle_np.dequantize(vt, data, elements, 4096)
    nan = np.isnan(a)
    assert np.array_equal(nan, np.isnan(b))
    assert np.array_equal(bits(a)[~nan], bits(b)[~nan])


@pytest.mark.parametrize("vt", [8, 12, 13, 14])
def test_gemv_oracles_agree_on_synthetic(vt):
    from engine_b200 import synth

    k, n = 1024, 96
    w = synth.random_weight(vt, k, n, seed=vt)
    x = synth.random_activations(3, k, seed=100 + vt)
    y32 = oracle.gemv_f32(vt, w, k, n, x)
    y32_mt = oracle.gemv_f32(vt, w, k, n, x, threads=4)
    y64 = oracle.gemv_f64(vt, w, k, n, x)
    scale = oracle.gemv_scale(vt, w, k, n, x)
    assert np.array_equal(bits(y32), bits(y32_mt))  # the row split does not change any row's arithmetic
    assert np.allclose(y64, oracle_np.gemv_f64(vt, w, k, n, x), rtol=1e-12, atol=1e-12)
    assert np.allclose(scale, oracle_np.gemv_scale(vt, w, k, n, x), rtol=1e-12)
    assert oracle.max_rel_error(y32, y64, scale) < 1e-4  # sequential f32 over K=1024


def test_synthetic_distributions():
    """The generators follow the benchmark configurations: 6-bit scales/minima uniform in 0..63,
    Q6_K scales in -64..63, f16 d = |N(0,1)| * sigma."""
    from engine_b200 import synth

    blocks = synth.random_blocks(12, 20000, np.random.default_rng(0))
    sc, mn = oracle_np.q4_k_scales(blocks[:, 4:16])
    assert sc.min() == 0 and sc.max() == 63 and mn.min() == 0 and mn.max() == 63
    d = oracle_np.f16_bits_to_f32(blocks[:, 0].astype(np.uint16) | (blocks[:, 1].astype(np.uint16) << 8))
    assert np.all(d >= 0) and abs(float(d.mean()) - 0.01 * np.sqrt(2 / np.pi)) < 3e-4
    q6 = synth.random_blocks(14, 20000, np.random.default_rng(1))
    s6 = q6[:, 192:208].view(np.int8)
    assert s6.min() == -64 and s6.max() == 63
    assert synth.encoded_bytes(12, 4096, 4096) == 9437184
    assert synth.encoded_bytes(14, 12288, 4096) == 41287680
    with pytest.raises(ValueError):
        synth.encoded_bytes(12, 128, 2)
