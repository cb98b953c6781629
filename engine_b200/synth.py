"""Seeded synthetic GGUF blocks with the value distributions the benchmark configurations state.

Q4_K  (144 B): d, dmin = f16(|N(0,1)| * 0.01); the 12-byte field packs 8 scales and 8 minima, each
               uniform in 0..63 (layout: crates/gguf/src/lib.rs:573-587 of the reference project);
               128 uniform random quant bytes.
Q5_K  (176 B): as Q4_K plus a uniform random qh[32] high-bit plane.
Q6_K  (210 B): ql[128], qh[64] uniform random bytes; int8 scales uniform in -64..63;
               d = f16(|N(0,1)| * 0.005).
Q8_0  (34 B):  d = f16(|N(0,1)| * 0.01); 32 int8 quants uniform in -128..127.

A tensor is GGML dims [K, N]: N rows of K/block_elements consecutive blocks
(crates/nvidia/src/quantized.rs:138-142).  The numpy generators are the ones parity tests use (the
same bytes go to the CPU checker and to the GPU); the torch generator fills large random-init model
weights directly in device memory.
"""
from __future__ import annotations

import numpy as np

Q8_0, Q4_K, Q5_K, Q6_K = 8, 12, 13, 14
BLOCK_LAYOUT = {Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}
TYPE_NAMES = {Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K"}
_D_OFFSETS = {Q8_0: ((0, 0.01),), Q4_K: ((0, 0.01), (2, 0.01)), Q5_K: ((0, 0.01), (2, 0.01)), Q6_K: ((208, 0.005),)}


def encoded_bytes(value_type: int, k: int, n: int) -> int:
    elements, block_bytes = BLOCK_LAYOUT[value_type]
    if k <= 0 or k % elements:
        raise ValueError(f"K={k} must be a positive multiple of {elements}")
    return (k // elements) * n * block_bytes


def pack_q4_k_scales(scales: np.ndarray, minima: np.ndarray) -> np.ndarray:
    """Inverse of the 6-bit unpack: [blocks, 8] scales + minima (0..63) -> [blocks, 12] bytes."""
    s = scales.astype(np.uint8)
    m = minima.astype(np.uint8)
    out = np.empty((s.shape[0], 12), np.uint8)
    out[:, 0:4] = s[:, 0:4] | ((s[:, 4:8] >> 4) << 6)
    out[:, 4:8] = m[:, 0:4] | ((m[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (s[:, 4:8] & 0x0F) | ((m[:, 4:8] & 0x0F) << 4)
    return out


def random_blocks(value_type: int, blocks: int, rng: np.random.Generator) -> np.ndarray:
    """[blocks, block_bytes] uint8 with the distributions in the module docstring."""
    _, block_bytes = BLOCK_LAYOUT[value_type]
    out = rng.integers(0, 256, size=(blocks, block_bytes), dtype=np.uint8)
    if value_type in (Q4_K, Q5_K):
        scales = rng.integers(0, 64, size=(blocks, 8), dtype=np.uint8)
        minima = rng.integers(0, 64, size=(blocks, 8), dtype=np.uint8)
        out[:, 4:16] = pack_q4_k_scales(scales, minima)
    if value_type == Q6_K:
        out[:, 192:208] = rng.integers(-64, 64, size=(blocks, 16), dtype=np.int8).view(np.uint8)
    for offset, sigma in _D_OFFSETS[value_type]:
        d = (np.abs(rng.standard_normal(blocks)) * sigma).astype(np.float16)
        out[:, offset:offset + 2] = d.view(np.uint8).reshape(blocks, 2)
    return out


def random_weight(value_type: int, k: int, n: int, seed: int) -> np.ndarray:
    """Encoded bytes of one [K, N] tensor, flat uint8, from numpy default_rng(seed)."""
    elements, _ = BLOCK_LAYOUT[value_type]
    encoded_bytes(value_type, k, n)
    rng = np.random.default_rng(seed)
    return random_blocks(value_type, (k // elements) * n, rng).reshape(-1)


def random_activations(members: int, k: int, seed: int) -> np.ndarray:
    """float32 N(0,1) [members, K]."""
    return np.random.default_rng(seed).standard_normal((members, k)).astype(np.float32)


def random_weight_device(value_type: int, k: int, n: int, seed: int, device):
    """Same distributions, generated in device memory with torch (for multi-GB random-init models).
    Returns a flat uint8 torch tensor.  Uniform random bytes already give uniform 6-bit scales/minima
    in the 12-byte field; Q6_K scales are an arithmetic shift of a random int8 (uniform in -64..63)."""
    import torch

    elements, block_bytes = BLOCK_LAYOUT[value_type]
    blocks = encoded_bytes(value_type, k, n) // block_bytes
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out = torch.empty((blocks, block_bytes), dtype=torch.uint8, device=device)
    chunk = max(1, (256 << 20) // block_bytes)
    for start in range(0, blocks, chunk):
        stop = min(blocks, start + chunk)
        out[start:stop] = torch.randint(0, 256, (stop - start, block_bytes), dtype=torch.uint8, device=device,
                                        generator=gen)
    if value_type == Q6_K:
        sc = out[:, 192:208].contiguous().view(torch.int8)
        out[:, 192:208] = (sc >> 1).view(torch.uint8)
    for offset, sigma in _D_OFFSETS[value_type]:
        d = (torch.randn(blocks, device=device, generator=gen).abs() * sigma).to(torch.float16)
        out[:, offset:offset + 2] = d.view(torch.uint8).reshape(blocks, 2)
    return out.reshape(-1)
