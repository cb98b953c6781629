"""Regenerates tests/golden/golden.npz: the fixtures the reference's own tests hold for this path.

Run from the repository root:  python tests/golden/make_golden.py

The reference is Rust and cannot be executed here, so nothing in this file runs reference code.
Each fixture below restates the *inputs* a reference test builds (cited by file:line inside the
reference project) and derives the expected values the way that test does: either the literal
values the test asserts, or a closed form in float64 that the test requires the decoder to match
exactly.  The C oracle and the CUDA kernels are then checked against this file.

  kat_*      crates/gguf/src/lib.rs:1369-1455   dequantizes_supported_scalar_and_quantized_blocks
  struct_*   crates/nvidia/tests/q4_q8_1.rs:15-49 (+ q5_q8_1.rs, q6_q8_1.rs, q8_0_q8_1.rs twins),
             expected = d*sc*q - dmin*m in float64, required exact (q4_q8_1.rs:205-228)
  gemv_*     crates/nvidia/tests/cuda_reference.rs:312-425 fixture blocks, input
             x[i] = (i % 17) * 0.125 - 1, expected = sum of decoded weight * x (:750-960), 1e-3 abs
  rms_*      crates/nvidia/tests/cuda_reference.rs:969-987
"""
from __future__ import annotations

import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def half(bits: int) -> float:
    return float(np.array([bits], np.uint16).view(np.float16)[0])


def put_u16(block: np.ndarray, offset: int, bits: int) -> None:
    block[offset] = bits & 0xFF
    block[offset + 1] = bits >> 8


# ---------------------------------------------------------------- known-answer blocks
def kat_blocks():
    out = {}
    q8 = np.zeros(34, np.uint8)
    put_u16(q8, 0, 0x3C00)
    q8[2], q8[3] = 0x80, 0x7F
    out["kat_q8_0"] = q8
    out["kat_q8_0_expect_head"] = np.array([-128.0, 127.0], np.float32)  # decoded[0], decoded[1]

    q4 = np.zeros(144, np.uint8)
    put_u16(q4, 0, 0x3C00)
    q4[4:8] = 1
    q4[16] = 0x10
    out["kat_q4_k"] = q4
    out["kat_q4_k_expect"] = np.array([0.0, 1.0], np.float32)  # decoded[0], decoded[32]

    q5 = np.zeros(176, np.uint8)
    put_u16(q5, 0, 0x3C00)
    q5[4:8] = 1
    q5[16] = 1
    q5[48] = 0x10
    out["kat_q5_k"] = q5
    out["kat_q5_k_expect"] = np.array([16.0, 1.0], np.float32)  # decoded[0], decoded[32]

    q6 = np.zeros(210, np.uint8)
    q6[192:208] = 1
    put_u16(q6, 208, 0x3C00)
    out["kat_q6_k"] = q6
    out["kat_q6_k_expect_all"] = np.array([-32.0], np.float32)  # every element
    return out


# ---------------------------------------------------------------- structured fixtures (15 blocks / family)
SCALES = [1, 17, 33, 63, 32, 47, 62, 48]
MINIMA = [63, 32, 17, 1, 47, 48, 33, 62]
D_BITS = [0x2C00, 0x3000, 0x3400]
DMIN_BITS = [0x2800, 0x2C00, 0x3000]


def pack_scales(block: np.ndarray) -> None:
    for g in range(4):
        block[4 + g] = SCALES[g] | ((SCALES[g + 4] >> 4) << 6)
        block[8 + g] = MINIMA[g] | ((MINIMA[g + 4] >> 4) << 6)
        block[12 + g] = (SCALES[g + 4] & 15) | ((MINIMA[g + 4] & 15) << 4)


def structured_q4_k():
    blocks, expect = [], []
    for seed in range(15):
        b = np.zeros(144, np.uint8)
        put_u16(b, 0, D_BITS[seed % 3])
        put_u16(b, 2, DMIN_BITS[seed % 3])
        pack_scales(b)
        q = np.array([(i * 7 + seed * 3 + i // 32) % 16 for i in range(256)], np.uint8)
        for g in range(8):
            b[16 + (g // 2) * 32:16 + (g // 2) * 32 + 32] |= q[g * 32:(g + 1) * 32] << ((g % 2) * 4)
        d, dm = half(D_BITS[seed % 3]), half(DMIN_BITS[seed % 3])
        expect.append([d * SCALES[i // 32] * float(q[i]) - dm * MINIMA[i // 32] for i in range(256)])
        blocks.append(b)
    return np.stack(blocks), np.array(expect, np.float64)


def structured_q5_k():
    blocks, expect = [], []
    for seed in range(15):
        b = np.zeros(176, np.uint8)
        put_u16(b, 0, D_BITS[seed % 3])
        put_u16(b, 2, DMIN_BITS[seed % 3])
        pack_scales(b)
        q = np.array([(i * 7 + seed * 3 + i // 32) % 32 for i in range(256)], np.uint8)
        for g in range(8):
            for i in range(32):
                v = int(q[g * 32 + i])
                b[48 + (g // 2) * 32 + i] |= (v & 15) << ((g % 2) * 4)
                b[16 + i] |= ((v >> 4) & 1) << g
        d, dm = half(D_BITS[seed % 3]), half(DMIN_BITS[seed % 3])
        expect.append([d * SCALES[i // 32] * float(q[i]) - dm * MINIMA[i // 32] for i in range(256)])
        blocks.append(b)
    return np.stack(blocks), np.array(expect, np.float64)


Q6_SCALES = [3, -5, 11, -13, 19, -23, 29, -31, 7, -9, 15, -17, 21, -25, 27, -2]


def structured_q6_k():
    blocks, expect = [], []
    for seed in range(15):
        b = np.zeros(210, np.uint8)
        q = np.array([(i * 7 + seed * 3 + i // 32) % 64 - 32 for i in range(256)], np.int16)
        for g in range(8):
            low_base = (g // 4) * 64 + (g % 2) * 32
            low_shift = 0 if g % 4 < 2 else 4
            high_base = 128 + (g // 4) * 32
            high_shift = (g % 4) * 2
            for i in range(32):
                u = int(q[g * 32 + i]) + 32
                b[low_base + i] |= (u & 15) << low_shift
                b[high_base + i] |= ((u >> 4) & 3) << high_shift
        b[192:208] = np.array(Q6_SCALES, np.int8).view(np.uint8)
        put_u16(b, 208, D_BITS[seed % 3])
        d = half(D_BITS[seed % 3])
        expect.append([d * Q6_SCALES[i // 16] * float(q[i]) for i in range(256)])
        blocks.append(b)
    return np.stack(blocks), np.array(expect, np.float64)


def structured_q8_0():
    blocks, expect = [], []
    for seed in range(5 * (768 // 32)):
        b = np.zeros(34, np.uint8)
        put_u16(b, 0, D_BITS[seed % 3])
        q = np.array([(i * 11 + seed * 5) % 61 - 30 for i in range(32)], np.int8)
        b[2:34] = q.view(np.uint8)
        d = half(D_BITS[seed % 3])
        expect.append([d * float(v) for v in q])
        blocks.append(b)
    return np.stack(blocks), np.array(expect, np.float64)


# ---------------------------------------------------------------- GEMV fixtures
def gemv_q4_k_block(seed: int) -> np.ndarray:
    b = np.zeros(144, np.uint8)
    put_u16(b, 0, 0x3C00)
    put_u16(b, 2, 0x3800)
    for i in range(4):
        b[4 + i] = ((1 + seed + i) | ((i & 3) << 6)) & 0xFF
        b[8 + i] = ((1 + i) | (((i + 1) & 3) << 6)) & 0xFF
        b[12 + i] = ((5 + seed + i) | ((2 + i) << 4)) & 0xFF
    for i in range(128):
        pattern = (i + seed * 5) % 16
        low = (pattern * 3) & 0x0F
        high = (15 - pattern * 3) & 0x0F
        b[16 + i] = low | (high << 4)
    return b


def gemv_q5_k_block(seed: int) -> np.ndarray:
    b = np.zeros(176, np.uint8)
    b[:144] = gemv_q4_k_block(seed)
    rot = ((0x55 << seed) | (0x55 >> (8 - seed))) & 0xFF if seed else 0x55
    b[16:48] = rot
    for i in range(128):
        pattern = (i + seed * 7) % 16
        low = (pattern * 5) & 0x0F
        high = (15 - pattern * 5) & 0x0F
        b[48 + i] = low | (high << 4)
    return b


def gemv_q6_k_block(seed: int) -> np.ndarray:
    b = np.zeros(210, np.uint8)
    for i in range(128):
        b[i] = (i * 7 + seed * 11) % 256
    for i in range(64):
        b[128 + i] = (i * 13 + seed * 5) % 256
    for i in range(16):
        b[192 + i] = np.array([(i + seed * 3) % 17 - 8], np.int8).view(np.uint8)[0]
    put_u16(b, 208, 0x3C00)
    return b


def gemv_q8_0_block(seed: int) -> np.ndarray:
    b = np.zeros(34, np.uint8)
    put_u16(b, 0, 0x3C00)
    for i in range(32):
        b[2 + i] = np.array([(i + seed * 3) % 31 - 15], np.int8).view(np.uint8)[0]
    return b


def gemv_input(k: int) -> np.ndarray:
    return np.array([(i % 17) * 0.125 - 1.0 for i in range(k)], np.float32)


def lcg_eighths(state: int, count: int) -> tuple[np.ndarray, int]:
    """The reference tests' value generator (crates/nvidia/tests/cuda_reference.rs:1669-1673): a 32-bit
    linear congruential step, then bits 16..21 as multiples of 0.125 in [-4, 4) - exact in f16."""
    values = np.empty(count, np.float32)
    for i in range(count):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        values[i] = np.float32(((state >> 16) & 0x3F) * 0.125 - 4.0)
    return values, state


def layer_fixtures() -> dict[str, np.ndarray]:
    """Inputs and host-replay expectations of three reference device tests, restated with sequential
    float32 arithmetic as the tests' own host loops do:
      rope        cuda_reference.rs:1996-2038  4 heads x 256 dims, 64 rotary dims, base 1e7, position 3, tolerance 1e-5
      attention   cuda_reference.rs:2062-2160  6 q heads over 2 kv heads, head size 32, 3 cached tokens, sigmoid output gate
                                                read from the second half of each 2*head_dim slice, tolerance 1e-3
      kv append   cuda_reference.rs:3435-3500  4 kv heads x 256 dims appended at tokens 0 and 3 of a 5-token f16 cache
    """
    f32 = np.float32
    out: dict[str, np.ndarray] = {}
    heads, head_dim, rot, base, position = 4, 256, 64, f32(1.0e7), 3
    x = np.array([f32(i % 97) * f32(0.03) - f32(1.4) for i in range(heads * head_dim)], np.float32)
    expect = x.copy()
    for head in range(heads):
        for pair in range(rot // 2):
            exponent = -(f32(2.0) * f32(pair)) / f32(rot)
            theta = f32(position) * f32(np.power(base, exponent, dtype=np.float32))
            sin, cos = f32(np.sin(theta)), f32(np.cos(theta))
            x0, x1 = expect[head * head_dim + pair], expect[head * head_dim + rot // 2 + pair]
            expect[head * head_dim + pair] = x0 * cos - x1 * sin
            expect[head * head_dim + rot // 2 + pair] = x0 * sin + x1 * cos
    out["rope_input"], out["rope_expect"] = x.reshape(heads, head_dim), expect.reshape(heads, head_dim)
    out["rope_params"] = np.array([rot, position, 1.0e7], np.float64)

    q_heads, kv_heads, d, tokens = 6, 2, 32, 3
    state = 12345
    q, state = lcg_eighths(state, q_heads * d)
    gate, state = lcg_eighths(state, q_heads * 2 * d)
    keys, state = lcg_eighths(state, tokens * kv_heads * d)
    values, state = lcg_eighths(state, tokens * kv_heads * d)
    scale = f32(1.0) / f32(np.sqrt(f32(d)))
    plain = np.zeros(q_heads * d, np.float32)
    gated = np.zeros(q_heads * d, np.float32)
    for head in range(q_heads):
        kv = head // (q_heads // kv_heads)
        scores = []
        for token in range(tokens):
            start = (token * kv_heads + kv) * d
            total = f32(0.0)
            for i in range(d):
                total = f32(total + q[head * d + i] * keys[start + i])
            scores.append(f32(total * scale))
        top = max(scores)
        exps = [f32(np.exp(f32(s - top))) for s in scores]
        denom = f32(0.0)
        for e in exps:
            denom = f32(denom + e)
        for dim in range(d):
            acc = f32(0.0)
            for token, e in enumerate(exps):
                acc = f32(acc + f32(e / denom) * values[(token * kv_heads + kv) * d + dim])
            g = gate[head * 2 * d + d + dim]
            plain[head * d + dim] = acc
            gated[head * d + dim] = f32(acc * f32(f32(1.0) / f32(f32(1.0) + f32(np.exp(-g)))))
    out["attn_q"] = q.reshape(q_heads, d)
    out["attn_gate"] = gate.reshape(q_heads, 2 * d)
    out["attn_keys"] = keys.reshape(tokens, kv_heads, d)
    out["attn_values"] = values.reshape(tokens, kv_heads, d)
    out["attn_expect_ungated"] = plain.reshape(q_heads, d)
    out["attn_expect"] = gated.reshape(q_heads, d)

    kv_heads, d, tokens = 4, 256, 5
    state = 909
    keys, state = lcg_eighths(state, kv_heads * d)
    values, state = lcg_eighths(state, kv_heads * d)
    cache = np.zeros((tokens, kv_heads * d), np.uint16)
    bits = f16_bits_of_eighths(keys)
    cache[0], cache[3] = bits, bits
    out["append_keys"], out["append_values"] = keys.reshape(kv_heads, d), values.reshape(kv_heads, d)
    out["append_key_cache_bits"] = cache.reshape(tokens, kv_heads, d)
    return out


def f16_bits_of_eighths(values: np.ndarray) -> np.ndarray:
    """Binary16 patterns of multiples of 0.125 below 4 in magnitude, composed from sign, exponent and
    fraction without a half-precision type (cuda_reference.rs:1679-1703)."""
    bits = np.zeros(values.shape, np.uint16)
    for i, value in enumerate(values):
        if value == 0.0:
            continue
        magnitude, exponent = abs(float(value)), 0
        while magnitude >= 2.0:
            magnitude, exponent = magnitude * 0.5, exponent + 1
        while magnitude < 1.0:
            magnitude, exponent = magnitude * 2.0, exponent - 1
        bits[i] = (0x8000 if value < 0 else 0) | ((exponent + 15) * 1024 + int((magnitude - 1.0) * 1024.0))
    return bits


def main() -> None:
    import sys

    sys.path.insert(0, os.path.join(HERE, "..", ".."))
    from oracle import oracle_np

    out = dict(kat_blocks())
    for name, (blocks, expect), vt in (("q4_k", structured_q4_k(), 12), ("q5_k", structured_q5_k(), 13),
                                       ("q6_k", structured_q6_k(), 14), ("q8_0", structured_q8_0(), 8)):
        out[f"struct_{name}"] = blocks
        # the closed form is exactly representable in float32 (the reference test asserts equality
        # after widening the decoder's f32 to f64), so the f32 cast below loses nothing
        as_f32 = expect.astype(np.float32)
        assert np.array_equal(as_f32.astype(np.float64), expect), name
        out[f"struct_{name}_expect"] = as_f32
    for name, make, count, vt, (k, n) in (("q4_k", gemv_q4_k_block, 4, 12, (512, 2)), ("q5_k", gemv_q5_k_block, 4, 13, (512, 2)),
                                          ("q6_k", gemv_q6_k_block, 4, 14, (512, 2)), ("q8_0", gemv_q8_0_block, 6, 8, (64, 3))):
        encoded = np.concatenate([make(seed) for seed in range(count)])
        x = gemv_input(k)
        out[f"gemv_{name}"] = encoded
        out[f"gemv_{name}_shape"] = np.array([k, n], np.int64)
        out[f"gemv_{name}_input"] = x
        # independent numpy decode, float64 dot: the reference test accepts 1e-3 absolute around
        # its own f32 sum of the same products
        out[f"gemv_{name}_expect"] = oracle_np.gemv_f64(vt, encoded, k, n, x[None, :])[0]
        out[f"gemv_{name}_dequant"] = oracle_np.dequantize(vt, encoded, k, n)
    x = np.array([1.0, -2.0, 3.0, -4.0], np.float32)
    w = np.array([1.0, 0.5, 2.0, -1.0], np.float32)
    inv = 1.0 / np.sqrt(np.float64((x.astype(np.float64) ** 2).sum() / 4.0 + 1e-5))
    out["rms_input"], out["rms_weight"] = x, w
    out["rms_eps"] = np.array([1e-5], np.float32)
    out["rms_expect"] = (x.astype(np.float64) * inv * w.astype(np.float64))
    out.update(layer_fixtures())
    path = os.path.join(HERE, "golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
