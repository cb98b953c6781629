"""Tensor-parallel decode on two GPUs (NCCL) against the single-GPU decoder on the same weights.

Needs two CUDA devices; skipped otherwise.  Each rank is a child process that keeps the shard
engine_b200.decode.local_shapes assigns to it (cut from the same host-side encoded tensors with
engine_b200.sharding), all-reduces after o_proj and ffn_down inside the captured CUDA graph, and chooses
tokens from the per-rank logit slices; rank 0 also runs the unsharded decoder and compares.
"""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

GEOMETRY = dict(hidden=512, layers=2, q_heads=4, kv_heads=2, head_dim=128, intermediate=1024, vocabulary=1000)


def encoded_model(seed):
    from engine_b200 import decode
    g = decode.DenseGeometry(**GEOMETRY)
    tensors, vectors = decode.host_model(g, seed)
    return g, tensors, vectors


def shard_weights(context, g, tensors, vectors, world, rank):
    from engine_b200 import decode
    return decode.shard_host_model(context, g, tensors, vectors, world, rank)


def _rank_main(rank, world, port, members, queue, path="nccl"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    import engine_b200
    from engine_b200 import decode
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        g, tensors, vectors = encoded_model(seed=members)
        context = engine_b200.RibnContext(rank, stream=torch.cuda.Stream(device=rank))
        link, partial_dtype = None, torch.float32
        if path != "nccl":
            # the exchanges over peer memory: one kernel per rank instead of an NCCL all-reduce plus a residual_add
            from engine_b200 import tp
            partial_dtype = torch.bfloat16 if path == "link-bf16" else torch.float32
            link = tp.PeerLink(context, rank, world, members * g.hidden * 4)
            link.connect_group(dist.group.WORLD)
        sharded = decode.CudaDenseDecode(context, g, shard_weights(context, g, tensors, vectors, world, rank), members, 64,
                                         process_group=dist.group.WORLD, world=world, rank=rank, peer_link=link, partial_dtype=partial_dtype)
        single = None
        if rank == 0:
            single = decode.CudaDenseDecode(context, g, shard_weights(context, g, tensors, vectors, 1, 0), members, 64)
        tokens = torch.tensor([(17 * m + 3) % g.vocabulary for m in range(members)], dtype=torch.int32)
        for decoder in (sharded, single):
            if decoder is not None:
                decoder.tokens.copy_(tokens)
        torch.cuda.synchronize()
        sharded.capture()
        sharded.k_cache.zero_()
        sharded.v_cache.zero_()
        torch.cuda.synchronize()
        ok = True
        for step in range(5):
            sharded.replay()
            context.synchronize()
            slices = [torch.empty(members, decode.local_shapes(g, world, r)["vocab_end"] - decode.local_shapes(g, world, r)["vocab_begin"],
                                  device=context.device) for r in range(world)]
            dist.all_gather(slices, sharded.logits)
            if rank == 0:
                single.run_step()
                context.synchronize()
                full = single.logits.cpu().numpy()
                got = torch.cat(slices, dim=1).cpu().numpy()
                scale = np.abs(full).max()
                ok &= bool(np.max(np.abs(got - full)) <= 2e-2 * scale)
                top = np.sort(full, axis=1)[:, -2:]
                clear = (top[:, 1] - top[:, 0]) > 4e-2 * scale
                ok &= bool(np.all(sharded.next_tokens.cpu().numpy()[clear] == single.next_tokens.cpu().numpy()[clear]))
                # keep the two decoders on the same token stream
                sharded_next = single.next_tokens.clone()
            else:
                sharded_next = torch.empty(members, dtype=torch.int32, device=context.device)
            dist.broadcast(sharded_next, src=0)
            sharded.tokens.copy_(sharded_next)
            sharded.positions.add_(1)
            if rank == 0:
                single.tokens.copy_(sharded_next)
                single.positions.add_(1)
            torch.cuda.synchronize()
        if rank == 0:
            queue.put(ok)
        # Release the captured graph (it holds NCCL kernels) before the communicator goes away.
        del sharded, single
        torch.cuda.synchronize()
        dist.barrier()      # nobody unmaps a block a peer's kernel may still read
        if link is not None:
            link.close()
        context.close()
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("path", ["nccl", "link-f32", "link-bf16"])
@pytest.mark.parametrize("members", [2, 6])
def test_two_gpus_decode_like_one(members, path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, members, queue, path)) for r in range(2)]
    for p in procs:
        p.start()
    result = queue.get(timeout=240)      # rank 0 reports before teardown; a stuck rank must not hold the suite
    for p in procs:
        p.join(timeout=60)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:
        p.terminate()
    assert result is True
    assert not stuck, "a rank did not exit"
    assert all(p.exitcode == 0 for p in procs)
