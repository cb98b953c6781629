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
    """Full encoded tensors (numpy bytes) and norm vectors, generated on the host so that every rank sees the same."""
    from engine_b200 import decode, synth
    g = decode.DenseGeometry(**GEOMETRY)
    shapes = decode.local_shapes(g, 1, 0)
    rng = np.random.default_rng(seed)
    tensors, vectors = {}, {}
    kinds = ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")
    for name, kind, salt in [("token_embd", "token_embd", 1), ("output", "output", 2)] + [
            (f"blk.{i}.{kind}", kind, 10 + 8 * i + j) for i in range(g.layers) for j, kind in enumerate(kinds)]:
        k, n = shapes[kind]
        tensors[name] = (decode.VALUE_TYPES[kind], k, n, synth.random_weight(decode.VALUE_TYPES[kind], k, n, seed=seed * 100 + salt))
    for name, length in [("output_norm", g.hidden)] + [(f"blk.{i}.{v}", n) for i in range(g.layers)
                                                      for v, n in (("attn_norm", g.hidden), ("ffn_norm", g.hidden),
                                                                   ("attn_q_norm", g.head_dim), ("attn_k_norm", g.head_dim))]:
        vectors[name] = (1 + 0.02 * rng.standard_normal(length)).astype(np.float32)
    return g, tensors, vectors


def shard_weights(context, g, tensors, vectors, world, rank):
    import engine_b200
    from engine_b200 import decode, sharding
    weights = decode.DenseWeights()
    put = lambda name, vt, k, n, data: weights.matrices.__setitem__(
        name, engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new(name, [k, n]), vt, torch.from_numpy(np.ascontiguousarray(data)).to(context.device)))
    for name, (vt, k, n, data) in tensors.items():
        kind = name.split(".")[-1]
        if kind == "token_embd":
            put(name, vt, k, n, data)
        elif kind in ("attn_q", "attn_k", "attn_v"):
            part, (kk, nn) = sharding.shard_rows(data, vt, k, n, world, rank, multiple=g.head_dim)
            put(name, vt, kk, nn, part)
        elif kind == "output":
            part, (kk, nn) = sharding.shard_rows(data, vt, k, n, world, rank)
            put(name, vt, kk, nn, part)
        elif kind in ("attn_output", "ffn_down"):
            part, (kk, nn), _ = sharding.shard_k(data, vt, k, n, world, rank)
            put(name, vt, kk, nn, part)
        elif kind == "ffn_gate":
            up_vt, _, _, up = tensors[name.replace("ffn_gate", "ffn_up")]
            gate_part, (kk, nn) = sharding.shard_rows(data, vt, k, n, world, rank, multiple=256)
            up_part, _ = sharding.shard_rows(up, up_vt, k, n, world, rank, multiple=256)
            put(name.replace("ffn_gate", "ffn_gate_up"), vt, kk, 2 * nn, np.concatenate([gate_part, up_part]))
    for name, v in vectors.items():
        weights.vectors[name] = torch.from_numpy(v).to(context.device)
    return weights


def _rank_main(rank, world, port, members, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    import engine_b200
    from engine_b200 import decode
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        g, tensors, vectors = encoded_model(seed=members)
        context = engine_b200.RibnContext(rank, stream=torch.cuda.Stream(device=rank))
        sharded = decode.CudaDenseDecode(context, g, shard_weights(context, g, tensors, vectors, world, rank), members, 64,
                                         process_group=dist.group.WORLD, world=world, rank=rank)
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
        context.close()
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("members", [2, 6])
def test_two_gpus_decode_like_one(members):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, members, queue)) for r in range(2)]
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
