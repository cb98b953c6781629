"""The reference-compatible Q8_1 activation format: CPU pins of the restatement (oracle/q8_1_np.py) against the
reference's byte known-answers (crates/nvidia/tests/cuda_activation.rs:14-40) and the exact / lossy identities of
crates/nvidia/tests/q4_q8_1.rs:205-252 and its q5 / q6 / q8_0 twins, on the fixtures of those files."""
import os

import numpy as np
import pytest

from oracle import q8_1_np

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))
FORMATS = {"q4_k": 12, "q5_k": 13, "q6_k": 14, "q8_0": 8}
INPUTS, ROWS = 768, 5


def kat_values() -> np.ndarray:
    """Five blocks; powers of two make the half scale and sum independent of a decoder (cuda_activation.rs:14-26)."""
    values = np.zeros(160, np.float32)
    for block, scale in enumerate([0.0, 1.0, 0.5, 2.0, 0.25]):
        if block == 0:
            continue
        values[block * 32:block * 32 + 6] = np.array([127.0, -127.0, 0.5, -0.5, 1.5, -1.5], np.float32) * scale
        values[block * 32 + 31] = 2.0 * scale
    return values


KAT_HEADERS = [0x40003C00, 0x3C003800, 0x44004000, 0x38003400]


def check_kat_words(words: np.ndarray) -> None:
    words = np.asarray(words, np.uint32).reshape(5, 9)
    assert not words[0].any()
    for block, header in enumerate(KAT_HEADERS):
        row = words[block + 1]
        assert row[0] == header
        assert row[1] == 0xFF01817F and row[2] == 0x0000FE02          # 127, -127, round(.5)=1, -1 | round(1.5)=2, -2
        assert not row[3:8].any() and row[8] == 0x02000000


def activations(exact: bool) -> np.ndarray:
    """q4_q8_1.rs:90-105 (the same generator in all four files)."""
    index = np.arange(INPUTS)
    if exact:
        integer = np.where(index % 32 == 0, 127, np.where(index % 32 == 1, -127, (index * 7) % 17 - 8))
        return (integer * np.array([0.25, 0.125, 0.0625])[(index // 32) % 3]).astype(np.float32)
    return (((index * 17 + 3) % 101 - 50).astype(np.float32) * np.float32(0.0137)).astype(np.float32)


def test_packer_known_answers():
    check_kat_words(q8_1_np.pack_q8_1(kat_values()))


def test_packer_round_trip_fields():
    x = activations(False)
    scale, total, q = q8_1_np.unpack_q8_1(q8_1_np.pack_q8_1(x))
    blocks = x.reshape(-1, 32)
    assert np.all(np.abs(q).max(axis=1) == 127)
    assert np.allclose(scale, np.abs(blocks).max(axis=1) / 127.0, rtol=2 ** -11)
    assert np.allclose(total, blocks.sum(axis=1), rtol=2 ** -10, atol=1e-3)
    assert np.max(np.abs(scale[:, None] * q - blocks)) <= 0.5 * scale.max() * (1 + 2 ** -10)


@pytest.mark.parametrize("name", list(FORMATS))
def test_exact_activations_match_float_arithmetic(name):
    vt = FORMATS[name]
    result = q8_1_np.gemv_q8_1(vt, GOLDEN[f"struct_{name}"], INPUTS, ROWS, activations(True))
    assert not result["packing_error_bound"].any()
    assert np.array_equal(result["packed_output"], result["float_output"])


@pytest.mark.parametrize("name", list(FORMATS))
def test_lossy_activations_have_an_explicit_float_error_bound(name):
    vt = FORMATS[name]
    result = q8_1_np.gemv_q8_1(vt, GOLDEN[f"struct_{name}"], INPUTS, ROWS, activations(False))
    error = np.abs(result["packed_output"] - result["float_output"])
    assert (error > 1e-4).any()
    assert np.all(error <= result["packing_error_bound"] + 1e-10)
    assert np.all(result["packing_error_bound"] > 0)


@pytest.mark.parametrize("name", list(FORMATS))
def test_float_output_is_the_f64_gemv_of_the_block_decoder(name):
    from oracle import oracle_np

    vt = FORMATS[name]
    x = activations(False)
    result = q8_1_np.gemv_q8_1(vt, GOLDEN[f"struct_{name}"], INPUTS, ROWS, x)
    assert np.allclose(result["float_output"], oracle_np.gemv_f64(vt, GOLDEN[f"struct_{name}"], INPUTS, ROWS, x[None]), rtol=1e-12, atol=1e-9)
