"""Tensor-parallel sharding of GGUF-encoded weights (host-side logic, pure numpy).

The reference has no multi-GPU code.  The path shards the way dense transformer layers do:

  * output-row split (attn q/k/v, ffn gate/up, output head): rank r keeps a contiguous range of the
    N rows -- a contiguous byte range of the encoded tensor, no repacking, no communication;
  * input-K split (attn o_proj, ffn_down): rank r keeps a contiguous range of the K/256 super-block
    columns of every row -- a strided gather of block ranges at load time -- consumes the matching
    slice of the activation and produces a full-length partial output; one all-reduce (sum) follows.

K shards are whole super-blocks (a Q8_0 tensor is sharded in units of eight 32-blocks), so shards
may be uneven: 100 super-blocks over 8 ranks is 13,13,13,13,12,12,12,12.  Row shards can be forced
to a multiple (e.g. the head dimension, so that a shard holds whole attention heads).
"""
from __future__ import annotations

import numpy as np

from .synth import BLOCK_LAYOUT

SUPER_BLOCK = 256


def split_even(total: int, world: int, rank: int) -> tuple[int, int]:
    """[begin, end) of `rank`'s share when `total` units are dealt as evenly as possible, larger shares first."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def row_range(n: int, world: int, rank: int, multiple: int = 1) -> tuple[int, int]:
    """Rows [begin, end) of an output-row shard; boundaries fall on multiples of `multiple`."""
    if n % multiple:
        raise ValueError(f"N={n} is not a multiple of {multiple}")
    begin, end = split_even(n // multiple, world, rank)
    return begin * multiple, end * multiple


def k_range(k: int, world: int, rank: int) -> tuple[int, int]:
    """Input elements [begin, end) of an input-K shard: whole 256-element super-blocks."""
    if k % SUPER_BLOCK:
        raise ValueError(f"K={k} is not a multiple of {SUPER_BLOCK}")
    begin, end = split_even(k // SUPER_BLOCK, world, rank)
    return begin * SUPER_BLOCK, end * SUPER_BLOCK


def _row_bytes(value_type: int, k: int) -> int:
    elements, block_bytes = BLOCK_LAYOUT[value_type]
    if k % elements:
        raise ValueError(f"K={k} is not a multiple of the block size {elements}")
    return (k // elements) * block_bytes


def shard_rows(encoded: np.ndarray, value_type: int, k: int, n: int, world: int, rank: int, multiple: int = 1):
    """Output-row shard: (bytes, [K, rows]) -- a contiguous slice (a view, nothing is copied)."""
    row_bytes = _row_bytes(value_type, k)
    raw = encoded.reshape(-1)
    if raw.size != row_bytes * n:
        raise ValueError(f"encoded length is {raw.size}, expected {row_bytes * n}")
    begin, end = row_range(n, world, rank, multiple)
    return raw[begin * row_bytes:end * row_bytes], (k, end - begin)


def shard_k(encoded: np.ndarray, value_type: int, k: int, n: int, world: int, rank: int):
    """Input-K shard: (bytes, [k_local, N], (k_begin, k_end)) -- every row's blocks of the K range, packed."""
    elements, block_bytes = BLOCK_LAYOUT[value_type]
    row_bytes = _row_bytes(value_type, k)
    raw = encoded.reshape(-1)
    if raw.size != row_bytes * n:
        raise ValueError(f"encoded length is {raw.size}, expected {row_bytes * n}")
    k_begin, k_end = k_range(k, world, rank)
    b0, b1 = k_begin // elements * block_bytes, k_end // elements * block_bytes
    shard = np.ascontiguousarray(raw.reshape(n, row_bytes)[:, b0:b1]).reshape(-1)
    return shard, (k_end - k_begin, n), (k_begin, k_end)
