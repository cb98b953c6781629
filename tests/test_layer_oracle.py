"""CPU checks of the decoder-layer restatement (oracle/layer_np.py) against closed forms and the reference's
known-answer test for RMSNorm (tests/cuda_reference.rs:969-987 of the reference project)."""
import numpy as np

from oracle import layer_np


def test_rms_norm_known_answer():
    x = np.array([1.0, -2.0, 3.0, -4.0], np.float32)
    w = np.array([1.0, 0.5, 2.0, -1.0], np.float32)
    inverse = 1.0 / np.sqrt(30.0 / 4.0 + 1e-5)
    assert np.allclose(layer_np.rms_norm_raw(x, w, 1e-5), x * inverse * w, atol=1e-6)


def test_rope_is_a_rotation_of_half_split_pairs():
    rng = np.random.default_rng(0)
    heads = rng.standard_normal((3, 128)).astype(np.float32)
    assert np.array_equal(layer_np.rope_neox(heads, 0, 128, 1e6), heads)           # angle 0
    rotated = layer_np.rope_neox(heads, 5, 64, 1e4)
    assert np.array_equal(rotated[:, 64:], heads[:, 64:])                            # beyond rot_dims: untouched
    assert np.allclose(rotated[:, :32] ** 2 + rotated[:, 32:64] ** 2, heads[:, :32] ** 2 + heads[:, 32:64] ** 2, rtol=1e-5)
    theta0 = 5.0                                                                      # pair 0: base^0
    assert np.allclose(rotated[:, 0], heads[:, 0] * np.cos(theta0) - heads[:, 32] * np.sin(theta0), atol=1e-5)


def test_attention_closed_forms():
    rng = np.random.default_rng(1)
    q = rng.standard_normal((4, 128)).astype(np.float32)
    keys = rng.standard_normal((1, 2, 128)).astype(np.float32)
    values = rng.standard_normal((1, 2, 128)).astype(np.float32)
    out = layer_np.attention(q, keys, values)
    assert np.allclose(out[0], values[0, 0]) and np.allclose(out[3], values[0, 1])  # one token: its value, per KV group
    keys = np.zeros((5, 2, 128), np.float32)                                         # equal scores: the mean of the values
    values = rng.standard_normal((5, 2, 128)).astype(np.float32)
    assert np.allclose(layer_np.attention(q, keys, values)[1], values[:, 0].mean(0), atol=1e-6)


def test_argmax_rules_and_silu():
    assert layer_np.argmax(np.array([1.0, 5.0, 5.0, np.nan], np.float32)) == 1
    assert layer_np.argmax(np.array([np.nan, np.nan], np.float32)) == 0
    assert np.allclose(layer_np.silu_mul(np.array([0.0, 2.0], np.float32), np.array([3.0, 3.0], np.float32)), [0.0, 3 * 2 / (1 + np.exp(-2.0))])


def test_dense_model_cache_grows_and_is_deterministic():
    rng = np.random.default_rng(2)
    hidden, heads, kv, d, inter, vocab = 256, 2, 1, 128, 256, 50
    w = {"token_embd": rng.standard_normal((vocab, hidden)).astype(np.float32), "output": rng.standard_normal((vocab, hidden)).astype(np.float32),
         "output_norm": np.ones(hidden, np.float32)}
    for name, shape in (("attn_q", (heads * d, hidden)), ("attn_k", (kv * d, hidden)), ("attn_v", (kv * d, hidden)),
                        ("attn_output", (hidden, heads * d)), ("ffn_gate", (inter, hidden)), ("ffn_up", (inter, hidden)), ("ffn_down", (hidden, inter))):
        w[f"blk.0.{name}"] = (rng.standard_normal(shape) * 0.05).astype(np.float32)
    for name, n in (("attn_norm", hidden), ("ffn_norm", hidden), ("attn_q_norm", d), ("attn_k_norm", d)):
        w[f"blk.0.{name}"] = np.ones(n, np.float32)
    a = layer_np.DenseModel(w, 1, heads, kv, d, 1e6, 1e-6)
    b = layer_np.DenseModel(w, 1, heads, kv, d, 1e6, 1e-6)
    for position, token in enumerate([3, 7, 7]):
        assert np.array_equal(a.step(token, position), b.step(token, position))
    assert a.keys[0].shape == (3, kv, d)


def _golden():
    import os

    return np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))


def test_rope_matches_the_reference_device_test_expectation():
    """Input and host replay of executes_rope_sigmoid_against_host_equations (tests/cuda_reference.rs:1996-2038
    of the reference project), with that test's tolerance."""
    g = _golden()
    rot, position, base = g["rope_params"]
    out = layer_np.rope_neox(g["rope_input"], int(position), int(rot), float(base))
    assert np.abs(out - g["rope_expect"]).max() < 1e-5
    assert np.array_equal(out[:, int(rot):], g["rope_input"][:, int(rot):])


def test_attention_matches_the_reference_device_test_expectation():
    """executes_attn_score_gqa_against_host_equations (tests/cuda_reference.rs:2062-2160): grouped heads over an
    f16 cache; the reference kernel's output gate is applied outside the restated function."""
    g = _golden()
    keys, values = layer_np.to_f16(g["attn_keys"]), layer_np.to_f16(g["attn_values"])
    assert np.array_equal(keys, g["attn_keys"]) and np.array_equal(values, g["attn_values"])     # eighths are exact in f16
    out = layer_np.attention(g["attn_q"], keys, values)
    assert np.abs(out - g["attn_expect_ungated"]).max() < 1e-3
    d = out.shape[1]
    gated = out * (1.0 / (1.0 + np.exp(-g["attn_gate"][:, d:])))
    assert np.abs(gated - g["attn_expect"]).max() < 1e-3


def test_cache_rounding_matches_the_reference_device_test_expectation():
    """executes_kv_append_f16_against_host_rounding (tests/cuda_reference.rs:3435-3500): the appended rows hold the
    binary16 pattern of each value, composed there without a half type; untouched rows stay zero."""
    g = _golden()
    bits = g["append_key_cache_bits"]
    rounded = layer_np.to_f16(g["append_keys"]).astype(np.float16).view(np.uint16)
    assert np.array_equal(bits[0], rounded) and np.array_equal(bits[3], rounded)
    assert not bits[[1, 2, 4]].any()
