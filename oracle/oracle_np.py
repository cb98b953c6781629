"""Vectorised numpy twin of the C oracle.  TEST INFRASTRUCTURE ONLY.

An independent second restatement of the reference's block decoders
(crates/gguf/src/lib.rs:551-661 of the reference project), written over whole
arrays of blocks so that tests can decode millions of blocks in seconds and
cross-check the C oracle.  Nothing in the shipped package imports it.

Every function returns float32 and performs the same float32 operations in the
same order as the reference: one multiply for the group scale, one multiply by
the quant, one subtract (Q4_K/Q5_K).  numpy never fuses multiply and add.
"""
from __future__ import annotations

import numpy as np

# crates/gguf/src/lib.rs:1051-1083 (the value types on the path)
BLOCK_LAYOUT = {8: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210)}
TYPE_NAMES = {8: "Q8_0", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K"}


def tensor_layout(value_type: int) -> tuple[int, int]:
    if value_type not in BLOCK_LAYOUT:
        raise ValueError(f"unsupported tensor type {value_type}")
    return BLOCK_LAYOUT[value_type]


def f16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """crates/gguf/src/lib.rs:551-563: exact widening; NaN -> canonical NaN."""
    bits = np.asarray(bits, dtype=np.uint16)
    out = bits.view(np.float16).astype(np.float32)
    nan = np.isnan(out)
    if nan.any():
        out = out.copy()
        out[nan] = np.float32(np.nan)
    return out


def _u16(blocks: np.ndarray, offset: int) -> np.ndarray:
    return blocks[:, offset].astype(np.uint16) | (blocks[:, offset + 1].astype(np.uint16) << 8)


def q4_k_scales(packed: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """crates/gguf/src/lib.rs:573-587 over [blocks, 12] uint8 -> two [blocks, 8] uint8."""
    s = packed.astype(np.uint8)
    scales = np.empty((s.shape[0], 8), np.uint8)
    minima = np.empty((s.shape[0], 8), np.uint8)
    scales[:, :4] = s[:, 0:4] & 0x3F
    minima[:, :4] = s[:, 4:8] & 0x3F
    scales[:, 4:] = (s[:, 8:12] & 0x0F) | ((s[:, 0:4] >> 2) & 0x30)
    minima[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 2) & 0x30)
    return scales, minima


def _as_blocks(data, value_type: int) -> np.ndarray:
    _, block_bytes = tensor_layout(value_type)
    raw = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.reshape(-1)
    if raw.size % block_bytes:
        raise ValueError(f"encoded length {raw.size} is not a whole number of {block_bytes}-byte blocks")
    return raw.reshape(-1, block_bytes)


def dequantize_blocks(value_type: int, data) -> np.ndarray:
    """Decode every block of `data`; returns [blocks, elements] float32."""
    b = _as_blocks(data, value_type)
    if value_type == 8:  # lib.rs:589-594
        d = f16_bits_to_f32(_u16(b, 0))
        q = b[:, 2:34].view(np.int8).astype(np.float32)
        return d[:, None] * q
    if value_type in (12, 13):  # lib.rs:596-633
        d = f16_bits_to_f32(_u16(b, 0))
        dmin = f16_bits_to_f32(_u16(b, 2))
        scales, minima = q4_k_scales(b[:, 4:16])
        group_scale = d[:, None] * scales.astype(np.float32)
        group_min = dmin[:, None] * minima.astype(np.float32)
        nib = b[:, 16:144] if value_type == 12 else b[:, 48:176]
        nib = nib.reshape(-1, 4, 32)
        q = np.empty((b.shape[0], 8, 32), np.uint8)
        q[:, 0::2, :] = nib & 0x0F
        q[:, 1::2, :] = nib >> 4
        if value_type == 13:
            qh = b[:, 16:48]
            for group in range(8):
                q[:, group, :] |= ((qh >> group) & 1) << 4
        w = group_scale[:, :, None] * q.astype(np.float32) - group_min[:, :, None]
        return w.reshape(-1, 256)
    if value_type == 14:  # lib.rs:635-661
        ql = b[:, 0:128].reshape(-1, 2, 2, 32)       # [block, chunk, variant%2, p]
        qh = b[:, 128:192].reshape(-1, 2, 32)        # [block, chunk, p]
        sc = b[:, 192:208].view(np.int8).astype(np.float32)  # [block, 16]
        d = f16_bits_to_f32(_u16(b, 208))
        q = np.empty((b.shape[0], 8, 32), np.int16)
        for group in range(8):
            chunk, variant = divmod(group, 4)
            low = ql[:, chunk, variant % 2, :]
            low = (low & 0x0F) if variant < 2 else (low >> 4)
            high = (qh[:, chunk, :] >> (2 * variant)) & 0x03
            q[:, group, :] = (low | (high << 4)).astype(np.int16) - 32
        group_scale = (d[:, None] * sc).reshape(-1, 8, 2)  # scale index = 2*group + p//16
        w = np.repeat(group_scale, 16, axis=2) * q.astype(np.float32)
        return w.reshape(-1, 256)
    raise ValueError(f"unsupported tensor type {value_type}")


def dequantize(value_type: int, data, k: int, n: int) -> np.ndarray:
    """Whole tensor, GGML dims [K, N] -> float32 [N, K]."""
    elements, block_bytes = tensor_layout(value_type)
    if k <= 0 or k % elements:
        raise ValueError(f"input size {k} must be a positive multiple of {elements}")
    raw = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.reshape(-1)
    if raw.size != (k // elements) * n * block_bytes:
        raise ValueError(f"encoded length is {raw.size}, expected {(k // elements) * n * block_bytes}")
    return dequantize_blocks(value_type, raw).reshape(n, k)


def gemv_f64(value_type: int, data, k: int, n: int, x: np.ndarray) -> np.ndarray:
    """f64 dot of the exactly-dequantised f32 weights with x [members, K]; returns [members, N]."""
    w = dequantize(value_type, data, k, n).astype(np.float64)
    x = np.asarray(x, dtype=np.float32).reshape(-1, k).astype(np.float64)
    return x @ w.T


def gemv_scale(value_type: int, data, k: int, n: int, x: np.ndarray) -> np.ndarray:
    """sqrt(sum_k (w*x)^2) per output: the floor of the relative-error denominator."""
    w = dequantize(value_type, data, k, n).astype(np.float64)
    x = np.asarray(x, dtype=np.float32).reshape(-1, k).astype(np.float64)
    return np.sqrt((x * x) @ (w * w).T)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """crates/nvidia/src/qwen_reference.rs:550-556 per row of x [members, n] (f32, sequential sum)."""
    x = np.asarray(x, dtype=np.float32)
    x2 = x.reshape(-1, x.shape[-1])
    out = np.empty_like(x2)
    count = np.float32(x2.shape[1])
    for m in range(x2.shape[0]):
        total = np.float32(0.0)
        for v in x2[m]:
            total = np.float32(total + np.float32(v * v))
        inv = np.float32(1.0) / np.sqrt(np.float32(total / count + np.float32(eps)), dtype=np.float32)
        out[m] = x2[m] * inv * weight.astype(np.float32)
    return out.reshape(x.shape)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (uint16)."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = np.isnan(np.asarray(x, dtype=np.float32))
    if nan.any():
        rounded = np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), rounded)
    return rounded


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
