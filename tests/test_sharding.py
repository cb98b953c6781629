"""Tensor-parallel sharding of encoded weights, on CPU.  The single-process tests check the shard
arithmetic; the two-rank test runs the sharded GEMV as real `torch.distributed` ranks over gloo
(row shards concatenated with all_gather, K shards summed with all_reduce) against the unsharded
oracle result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from engine_b200 import sharding, synth


def test_split_even_and_ranges():
    assert [sharding.split_even(100, 8, r) for r in range(8)] == [(0, 13), (13, 26), (26, 39), (39, 52), (52, 64), (64, 76), (76, 88), (88, 100)]
    assert sharding.k_range(25600, 8, 0) == (0, 13 * 256) and sharding.k_range(25600, 8, 7) == (88 * 256, 25600)
    assert sharding.row_range(8192, 8, 3, multiple=128) == (3072, 4096)     # 64 q heads of 128 over 8 ranks
    assert sharding.row_range(1024, 8, 7, multiple=128) == (896, 1024)      # 8 kv heads: one per rank
    with pytest.raises(ValueError):
        sharding.row_range(1000, 8, 0, multiple=128)
    with pytest.raises(ValueError):
        sharding.k_range(4000, 2, 0)
    with pytest.raises(ValueError):
        sharding.split_even(10, 2, 2)
    # empty shards are legal (more ranks than units)
    assert sharding.split_even(2, 4, 3) == (2, 2)


@pytest.mark.parametrize("vt", [8, 12, 13, 14])
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_shards_reassemble_the_product(vt, world):
    k, n = 2304, 40          # 9 super-blocks: uneven K shards for every world size > 1
    w = synth.random_weight(vt, k, n, seed=vt)
    x = synth.random_activations(2, k, seed=1)
    full = oracle.gemv_f64(vt, w, k, n, x)
    rows = []
    for rank in range(world):
        part, (kk, nn) = sharding.shard_rows(w, vt, k, n, world, rank, multiple=8)
        rows.append(oracle.gemv_f64(vt, part, kk, nn, x) if nn else np.zeros((2, 0)))
    assert np.array_equal(np.concatenate(rows, axis=1), full)
    total = np.zeros_like(full)
    for rank in range(world):
        part, (kk, nn), (k0, k1) = sharding.shard_k(w, vt, k, n, world, rank)
        if kk:
            total += oracle.gemv_f64(vt, part, kk, nn, np.ascontiguousarray(x[:, k0:k1]))
    assert np.allclose(total, full, rtol=1e-12, atol=1e-12)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        vt, k, n = 12, 1280, 48
        w = synth.random_weight(vt, k, n, seed=3)            # every rank holds the same seed, keeps its shard
        x = synth.random_activations(3, k, seed=4)
        # row-parallel projection followed by a K-parallel one, as in attention (q -> o) or the FFN (up -> down)
        part, (kk, nn) = sharding.shard_rows(w, vt, k, n, world, rank, multiple=8)
        local = torch.from_numpy(oracle.gemv_f64(vt, part, kk, nn, x))
        gathered = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(gathered, local)
        row_result = torch.cat(gathered, dim=1).numpy()
        part, (kk, nn), (k0, k1) = sharding.shard_k(w, vt, k, n, world, rank)
        partial = torch.from_numpy(oracle.gemv_f64(vt, part, kk, nn, np.ascontiguousarray(x[:, k0:k1])))
        dist.all_reduce(partial, op=dist.ReduceOp.SUM)
        if rank == 0:
            full = oracle.gemv_f64(vt, w, k, n, x)
            queue.put((bool(np.array_equal(row_result, full)), bool(np.allclose(partial.numpy(), full, rtol=1e-12, atol=1e-12))))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_result():
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    assert queue.get(timeout=10) == (True, True)
