"""A tensor-parallel decode step as two real `torch.distributed` ranks over gloo, on CPU.

Each rank keeps the shard that engine_b200.decode.local_shapes assigns to it (whole heads of q/k/v, whole
256-column blocks of ffn_down, a contiguous range of the vocabulary), runs the layer arithmetic of the host
model (oracle/layer_np.py) on its shard, and all-reduces the partial outputs of o_proj and ffn_down -- the two
collectives of the GPU path.  The result must equal the unsharded step, and the token chosen from the
per-rank logit slices must be the global argmax.
"""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from engine_b200 import decode
from engine_b200.sharding import split_even
from oracle import layer_np

GEOMETRY = decode.DenseGeometry(hidden=256, layers=2, q_heads=4, kv_heads=2, head_dim=128, intermediate=768, vocabulary=101)


def full_weights(seed=0):
    g, rng, w = GEOMETRY, np.random.default_rng(seed), {}
    d = g.head_dim
    w["token_embd"] = rng.standard_normal((g.vocabulary, g.hidden)).astype(np.float32)
    w["output"] = (rng.standard_normal((g.vocabulary, g.hidden)) * 0.1).astype(np.float32)
    w["output_norm"] = (1 + 0.02 * rng.standard_normal(g.hidden)).astype(np.float32)
    for i in range(g.layers):
        for name, shape in (("attn_q", (g.q_heads * d, g.hidden)), ("attn_k", (g.kv_heads * d, g.hidden)), ("attn_v", (g.kv_heads * d, g.hidden)),
                            ("attn_output", (g.hidden, g.q_heads * d)), ("ffn_gate", (g.intermediate, g.hidden)),
                            ("ffn_up", (g.intermediate, g.hidden)), ("ffn_down", (g.hidden, g.intermediate))):
            w[f"blk.{i}.{name}"] = (rng.standard_normal(shape) * 0.05).astype(np.float32)
        for name, n in (("attn_norm", g.hidden), ("ffn_norm", g.hidden), ("attn_q_norm", d), ("attn_k_norm", d)):
            w[f"blk.{i}.{name}"] = (1 + 0.02 * rng.standard_normal(n)).astype(np.float32)
    return w


def shard(w, world, rank):
    """Rows of q/k/v/gate/up/output and columns of attn_output/ffn_down that `rank` keeps."""
    g, d = GEOMETRY, GEOMETRY.head_dim
    q0, q1 = split_even(g.q_heads, world, rank)
    kv0, kv1 = split_even(g.kv_heads, world, rank)
    i0, i1 = (v * 256 for v in split_even(g.intermediate // 256, world, rank))
    v0, v1 = split_even(g.vocabulary, world, rank)
    local = {k: v for k, v in w.items() if v.ndim == 1}
    local["token_embd"] = w["token_embd"]
    local["output"] = w["output"][v0:v1]
    for i in range(g.layers):
        local[f"blk.{i}.attn_q"] = w[f"blk.{i}.attn_q"][q0 * d:q1 * d]
        local[f"blk.{i}.attn_k"] = w[f"blk.{i}.attn_k"][kv0 * d:kv1 * d]
        local[f"blk.{i}.attn_v"] = w[f"blk.{i}.attn_v"][kv0 * d:kv1 * d]
        local[f"blk.{i}.attn_output"] = w[f"blk.{i}.attn_output"][:, q0 * d:q1 * d]
        local[f"blk.{i}.ffn_gate"] = w[f"blk.{i}.ffn_gate"][i0:i1]
        local[f"blk.{i}.ffn_up"] = w[f"blk.{i}.ffn_up"][i0:i1]
        local[f"blk.{i}.ffn_down"] = w[f"blk.{i}.ffn_down"][:, i0:i1]
    return local, (q1 - q0, kv1 - kv0, v0)


def test_shard_plan_matches_the_decoder():
    for world in (1, 2):
        for rank in range(world):
            local, (q_heads, kv_heads, v0) = shard(full_weights(), world, rank)
            shapes = decode.local_shapes(GEOMETRY, world, rank)
            assert (shapes["q_heads"], shapes["kv_heads"], shapes["vocab_begin"]) == (q_heads, kv_heads, v0)
            for kind in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down", "output"):
                name = kind if kind == "output" else f"blk.0.{kind}"
                assert local[name].shape == (shapes[kind][1], shapes[kind][0])       # [N rows, K columns]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class ShardedModel(layer_np.DenseModel):
    """The host model on one rank's shard: partial outputs of the column-split projections are all-reduced."""

    @staticmethod
    def _matvec(matrix, x):
        return layer_np.DenseModel._matvec(matrix, x)

    def layer(self, i, hidden, position):
        w, d = self.w, self.head_dim
        x = layer_np.rms_norm_raw(hidden, w[f"blk.{i}.attn_norm"], self.eps)
        q = self._matvec(w[f"blk.{i}.attn_q"], x).reshape(self.q_heads, d)
        k = self._matvec(w[f"blk.{i}.attn_k"], x).reshape(self.kv_heads, d)
        v = self._matvec(w[f"blk.{i}.attn_v"], x).reshape(self.kv_heads, d)
        q = layer_np.rope_neox(layer_np.rms_norm_raw(q, w[f"blk.{i}.attn_q_norm"], self.eps), position, self.rot_dims, self.rope_base)
        k = layer_np.rope_neox(layer_np.rms_norm_raw(k, w[f"blk.{i}.attn_k_norm"], self.eps), position, self.rot_dims, self.rope_base)
        self.keys[i] = np.concatenate([self.keys[i], layer_np.to_f16(k)[None]], axis=0)
        self.values[i] = np.concatenate([self.values[i], layer_np.to_f16(v)[None]], axis=0)
        attended = layer_np.attention(q, self.keys[i], self.values[i]).reshape(-1)
        partial = torch.from_numpy(self._matvec(w[f"blk.{i}.attn_output"], attended))
        dist.all_reduce(partial)
        hidden = hidden + partial.numpy()
        x = layer_np.rms_norm_raw(hidden, w[f"blk.{i}.ffn_norm"], self.eps)
        act = layer_np.silu_mul(self._matvec(w[f"blk.{i}.ffn_gate"], x), self._matvec(w[f"blk.{i}.ffn_up"], x))
        partial = torch.from_numpy(self._matvec(w[f"blk.{i}.ffn_down"], act))
        dist.all_reduce(partial)
        return (hidden + partial.numpy()).astype(np.float32)


def _rank_main(rank, world, port, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = GEOMETRY
        w = full_weights()
        local, (q_heads, kv_heads, v0) = shard(w, world, rank)
        model = ShardedModel(local, g.layers, q_heads, kv_heads, g.head_dim, g.rope_base, g.eps)
        reference = layer_np.DenseModel(w, g.layers, g.q_heads, g.kv_heads, g.head_dim, g.rope_base, g.eps)
        ok, token = True, 5
        for position in range(4):
            logits = model.step(token, position)                   # this rank's slice of the vocabulary
            full = reference.step(token, position)
            ok &= bool(np.allclose(logits, full[v0:v0 + len(logits)], rtol=2e-5, atol=2e-5))
            # token selection as the GPU path does it: local argmax, then the best (value, index) over the ranks
            best = layer_np.argmax(logits)
            pairs = [None] * world
            dist.all_gather_object(pairs, (float(logits[best]), best + v0))
            values = [p[0] for p in pairs]
            token = pairs[int(np.argmax(values))][1]
            ok &= token == layer_np.argmax(full)
        if rank == 0:
            queue.put(ok)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_decode_like_one():
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
        assert p.exitcode == 0
    assert queue.get(timeout=10) is True
