"""CPU restatement of the reference's Q8_1 activation format and of its integer-dot GEMV arithmetic.
TEST INFRASTRUCTURE ONLY: imported by tests/ and by the benchmark's CPU legs, never by the product path.

Follows, in the reference project:
    quantize_q8_1                crates/nvidia/src/activation.cu:3-28 (one warp per block of 32 values: header word
                                 half(max/127) | half(sum) << 16, then eight words of four signed bytes)
    pack_host                    crates/nvidia/tests/q4_q8_1.rs:107-148 (the host model of that kernel, including the
                                 pairwise xor tree of the sum)
    reference()                  crates/nvidia/tests/q4_q8_1.rs:157-203, q5_q8_1.rs, q6_q8_1.rs:156-208,
                                 q8_0_q8_1.rs:135-174: packed arithmetic in f64, the float result, the packing-error
                                 bound and the arithmetic magnitude the device tests accept results against
    q*_q8_1_gemv{,_batch}        crates/nvidia/src/kernels/quantized/q4_k_q8_1.cu:40-144 and the q5_k / q6_k / q8_0 twins
Pinned by tests/test_q8_1.py against the byte known-answers of crates/nvidia/tests/cuda_activation.rs:14-40 and the
exact-fixture identities of the q*_q8_1.rs files.
"""
from __future__ import annotations

import numpy as np

from . import oracle_np

WORDS_PER_BLOCK = 9


def pack_q8_1(x: np.ndarray) -> np.ndarray:
    """float32 [..., multiple of 32] -> uint32 [blocks * 9], blocks in linear order (a batch packs as one stream)."""
    blocks = np.asarray(x, np.float32).reshape(-1, 32)
    maximum = np.abs(blocks).max(axis=1)
    scale = (maximum / np.float32(127.0)).astype(np.float32)
    sums = blocks.copy()
    lanes = np.arange(32)
    for offset in (16, 8, 4, 2, 1):                     # the warp's xor shuffles: lane 0 ends with this exact f32 tree
        sums = (sums + sums[:, lanes ^ offset]).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        ratio = (blocks / scale[:, None]).astype(np.float32)
    rounded = np.where(ratio >= 0, np.floor(ratio + np.float32(0.5)), np.ceil(ratio - np.float32(0.5)))    # roundf: ties away from zero
    q = np.where(maximum[:, None] == 0, 0, np.clip(np.nan_to_num(rounded), -127, 127)).astype(np.int8)
    words = np.empty((blocks.shape[0], WORDS_PER_BLOCK), np.uint32)
    header_scale = scale.astype(np.float16).view(np.uint16).astype(np.uint32)            # cvt.rn.f16.f32
    header_sum = sums[:, 0].astype(np.float16).view(np.uint16).astype(np.uint32)
    words[:, 0] = header_scale | (header_sum << 16)
    words[:, 1:] = q.view(np.uint8).reshape(-1, 8, 4).astype(np.uint32) @ np.array([1, 1 << 8, 1 << 16, 1 << 24], np.uint32)
    return words.reshape(-1)


def unpack_q8_1(words: np.ndarray) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """uint32 [blocks * 9] -> (scale f64 [blocks], sum f64 [blocks], q int8 [blocks, 32])."""
    w = np.asarray(words, np.uint32).reshape(-1, WORDS_PER_BLOCK)
    scale = (w[:, 0] & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float64)
    total = (w[:, 0] >> 16).astype(np.uint16).view(np.float16).astype(np.float64)
    q = np.ascontiguousarray(w[:, 1:]).view(np.uint8).view(np.int8).reshape(-1, 32)
    return scale, total, q


def weight_fields(value_type: int, data, k: int, n: int) -> dict:
    """Integer fields of every row: `q` int [n, k], `a` f64 [n, k/16] (the factor of each run of 16 quants) and, for
    the affine formats, `b` f64 [n, k/32] (the offset of each group of 32)."""
    b = oracle_np._as_blocks(data, value_type)
    if value_type == 8:
        d = oracle_np.f16_bits_to_f32(oracle_np._u16(b, 0)).astype(np.float64)
        q = b[:, 2:34].view(np.int8).astype(np.int32)
        return {"q": q.reshape(n, k), "a": np.repeat(d, 2).reshape(n, k // 16), "b": None}
    if value_type in (12, 13):
        d = oracle_np.f16_bits_to_f32(oracle_np._u16(b, 0)).astype(np.float64)
        dmin = oracle_np.f16_bits_to_f32(oracle_np._u16(b, 2)).astype(np.float64)
        scales, minima = oracle_np.q4_k_scales(b[:, 4:16])
        nib = (b[:, 16:144] if value_type == 12 else b[:, 48:176]).reshape(-1, 4, 32)
        q = np.empty((b.shape[0], 8, 32), np.int32)
        q[:, 0::2, :] = nib & 0x0F
        q[:, 1::2, :] = nib >> 4
        if value_type == 13:
            for group in range(8):
                q[:, group, :] |= ((b[:, 16:48].astype(np.int32) >> group) & 1) << 4
        a = d[:, None] * scales.astype(np.float64)
        return {"q": q.reshape(n, k), "a": np.repeat(a, 2, axis=1).reshape(n, k // 16), "b": (dmin[:, None] * minima.astype(np.float64)).reshape(n, k // 32)}
    if value_type == 14:
        ql, qh = b[:, 0:128].reshape(-1, 2, 2, 32), b[:, 128:192].reshape(-1, 2, 32)
        sc = b[:, 192:208].view(np.int8).astype(np.float64)
        d = oracle_np.f16_bits_to_f32(oracle_np._u16(b, 208)).astype(np.float64)
        q = np.empty((b.shape[0], 8, 32), np.int32)
        for group in range(8):
            chunk, variant = divmod(group, 4)
            low = ql[:, chunk, variant % 2, :]
            low = (low & 0x0F) if variant < 2 else (low >> 4)
            q[:, group, :] = (low | (((qh[:, chunk, :] >> (2 * variant)) & 3) << 4)).astype(np.int32) - 32
        return {"q": q.reshape(n, k), "a": (d[:, None] * sc).reshape(n, k // 16), "b": None}
    raise ValueError(f"unsupported tensor type {value_type}")


def gemv_q8_1(value_type: int, data, k: int, n: int, x: np.ndarray, packed: np.ndarray | None = None) -> dict:
    """The four quantities of the reference tests' host model, each [members, n] float64:
    `packed_output` (what the integer-dot kernel computes, in exact arithmetic), `float_output` (the float GEMV),
    `packing_error_bound` (how far the two may differ) and `arithmetic_magnitude` (scales the accepted f32 rounding:
    magnitude * 2^-23 * 32 + 1e-5)."""
    x = np.asarray(x, np.float32).reshape(-1, k)
    members = x.shape[0]
    packed = pack_q8_1(x) if packed is None else np.asarray(packed, np.uint32)
    scale, total, q = unpack_q8_1(packed)
    scale, total = scale.reshape(members, k // 32), total.reshape(members, k // 32)
    qa = q.reshape(members, k // 16, 16).astype(np.int64)
    f = weight_fields(value_type, data, k, n)
    qw = f["q"].reshape(n, k // 16, 16).astype(np.int64)
    a = f["a"]                                                                     # [n, k/16]
    out = {name: np.zeros((members, n)) for name in ("packed_output", "float_output", "packing_error_bound", "arithmetic_magnitude")}
    x64 = x.astype(np.float64).reshape(members, k // 16, 16)
    for m in range(members):
        run_scale = np.repeat(scale[m], 2)                                         # [k/16]
        dots = (qw * qa[m][None]).sum(axis=2)                                       # exact integers, [n, k/16]
        dequantised = run_scale[None, :, None] * qa[m][None].astype(np.float64)   # what the packed bytes stand for
        out["float_output"][m] = (a[:, :, None] * qw * x64[m][None]).sum(axis=(1, 2))
        out["packing_error_bound"][m] = (np.abs(a)[:, :, None] * np.abs(qw) * np.abs(dequantised - x64[m][None])).sum(axis=(1, 2))
        if value_type == 14:
            # the kernel dots unsigned (q + 32) bytes and removes the bias through the packed half sums; in exact
            # arithmetic that is the signed dot, and the magnitude counts the elementwise terms and the combined one
            out["packed_output"][m] = (a * run_scale[None] * dots).sum(axis=1)
            out["arithmetic_magnitude"][m] = (np.abs(a[:, :, None] * qw * dequantised).sum(axis=(1, 2)) + np.abs(a * run_scale[None] * dots).sum(axis=1))
        elif value_type == 8:
            block_dots = dots.reshape(n, k // 32, 2).sum(axis=2)
            d = a[:, ::2]
            out["packed_output"][m] = (d * scale[m][None] * block_dots).sum(axis=1)
            out["arithmetic_magnitude"][m] = (np.abs(a[:, :, None] * qw * dequantised).sum(axis=(1, 2)) + np.abs(d * scale[m][None] * block_dots).sum(axis=1))
        else:
            group_dots = dots.reshape(n, k // 32, 2).sum(axis=2)
            group_a, b = a[:, ::2], f["b"]
            out["packed_output"][m] = (group_a * scale[m][None] * group_dots - b * total[m][None]).sum(axis=1)
            group_sum = x64[m].reshape(k // 32, 32).sum(axis=1)
            out["float_output"][m] -= (b * group_sum[None]).sum(axis=1)
            out["packing_error_bound"][m] += (np.abs(b) * np.abs(total[m] - group_sum)[None]).sum(axis=1)
            out["arithmetic_magnitude"][m] = (np.abs(a[:, :, None] * qw * dequantised).sum(axis=(1, 2)) + np.abs(b * total[m][None]).sum(axis=1))
    return out


def rounding_allowance(magnitude: np.ndarray) -> np.ndarray:
    """The f32-accumulation slack the reference device tests grant around `packed_output` (q4_q8_1.rs:283-284)."""
    return magnitude * float(np.finfo(np.float32).eps) * 32.0 + 1e-5
