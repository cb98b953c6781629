"""The tensor-parallel exchange kernels (csrc/tp.cu through engine_b200/tp.py) on ONE GPU: the peer's side of the
protocol -- its partial, its flag, its token candidates -- is written into its block by the host before the launch, so
no kernel ever waits for another kernel.  The bounded wait is exercised with a flag that nobody sets."""
import numpy as np
import pytest
import torch

import engine_b200
from engine_b200 import tp

pytestmark = pytest.mark.gpu

FLAGS, SELECT_FLAGS, PAIRS = 0, 16, 32        # word offsets in the tail of a block (include/ribn_b200.h)


def two_links(ctx, slot_bytes):
    blocks = [torch.zeros(tp.PeerLink.block_bytes(slot_bytes), dtype=torch.uint8, device=ctx.device) for _ in range(2)]
    links = [tp.PeerLink(ctx, rank, 2, slot_bytes, local_block=blocks[rank]) for rank in range(2)]
    for link in links:
        link.connect_pointers([b.data_ptr() for b in blocks])
    tails = [b[2 * links[0].slot_bytes:].view(torch.int32) for b in blocks]
    return links, tails


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_exchange_adds_the_partials_in_rank_order(ctx, dtype):
    members, hidden = 5, 1024
    links, tails = two_links(ctx, members * hidden * 4)
    rng = np.random.default_rng(0)
    residual = rng.standard_normal((members, hidden)).astype(np.float32)
    state = torch.from_numpy(residual.copy()).to(ctx.device)
    for exchange in (1, 2, 3):
        slot = (exchange - 1) & 1
        parts = [torch.from_numpy(rng.standard_normal((members, hidden)).astype(np.float32)).to(ctx.device).to(dtype) for _ in range(2)]
        for rank in range(2):
            links[rank].partial(slot, members, hidden, dtype).copy_(parts[rank])
        tails[0][FLAGS + 1] = exchange                  # what rank 1 would have published in rank 0's block
        before = state.clone()
        links[0].allreduce_residual(slot, state, members, hidden, dtype)
        ctx.synchronize()
        expect = (before + parts[0].float()) + parts[1].float()
        assert torch.equal(state, expect)
        assert int(tails[1][FLAGS + 0]) == exchange     # and rank 0 has published in rank 1's block


def test_a_peer_that_never_arrives_times_out_and_leaves_the_state_alone(ctx):
    members, hidden = 2, 512
    links, tails = two_links(ctx, members * hidden * 4)
    links[0].set_wait(2000)                              # 2 ms
    state = torch.ones(members, hidden, device=ctx.device)
    links[0].allreduce_residual(0, state, members, hidden, torch.float32)
    with pytest.raises(engine_b200.CudaQuantizedKernelError) as e:
        ctx.synchronize()
    assert e.value.kind == "Timeout"
    assert torch.equal(state, torch.ones_like(state))
    # the context and the link stay usable: the exchange counter has moved on, the late peer publishes it and the next one
    tails[0][FLAGS + 1] = 2
    links[1].partial(1, members, hidden, torch.float32).fill_(2.0)
    links[0].partial(1, members, hidden, torch.float32).fill_(0.5)
    links[0].allreduce_residual(1, state, members, hidden, torch.float32)
    ctx.synchronize()
    assert torch.equal(state, torch.full_like(state, 3.5))


def ordered_key(values: np.ndarray) -> np.ndarray:
    bits = values.astype(np.float32).view(np.uint32)
    return np.where(bits >> 31, ~bits, bits ^ np.uint32(0x80000000)).astype(np.uint32)


def test_token_selection_follows_the_argmax_rules_across_ranks(ctx):
    members, local_vocab = 6, 777
    links, tails = two_links(ctx, 4096)
    rng = np.random.default_rng(1)
    mine = rng.standard_normal((members, local_vocab)).astype(np.float32)
    theirs = rng.standard_normal((members, local_vocab)).astype(np.float32)
    mine[1, 5] = theirs[1, 9] = 9.0                      # a tie across ranks: the lower token wins
    mine[2] = np.nan                                      # one rank all NaN: the other rank's best wins
    mine[3] = np.nan
    theirs[3] = np.nan                                    # NaN everywhere: token 0
    theirs[4, 100] = np.inf
    mine[5, 700] = 50.0
    mine[5, 3] = np.nan
    # rank 1's candidates, as its kernel would leave them (generation 1 = first selection)
    best = np.array([0 if np.all(np.isnan(r)) else int(np.nanargmax(r)) for r in theirs])
    keys = np.array([0 if np.all(np.isnan(r)) else ordered_key(r[b:b + 1])[0] for r, b in zip(theirs, best)], np.uint32)
    pairs = np.stack([keys, (local_vocab + best).astype(np.uint32)], axis=1).reshape(-1)
    offset = PAIRS + 1 * 64 * 2
    tails[1][offset:offset + pairs.size] = torch.from_numpy(pairs.view(np.int32)).to(ctx.device)
    tails[0][SELECT_FLAGS + 1] = 1
    out = torch.full((members,), -1, dtype=torch.int32, device=ctx.device)
    links[0].select_tokens(torch.from_numpy(mine).to(ctx.device), members, 0, out)
    ctx.synchronize()
    joined = np.concatenate([mine, theirs], axis=1)
    expect = [0 if np.all(np.isnan(r)) else int(np.nanargmax(r)) for r in joined]
    assert out.cpu().tolist() == expect
    assert expect[1] == 5 and expect[2] >= local_vocab and expect[3] == 0 and expect[4] == local_vocab + 100 and expect[5] == 700


def test_a_single_rank_link_is_a_residual_add_and_an_argmax(ctx):
    members, hidden = 3, 256
    link = tp.PeerLink(ctx, 0, 1, members * hidden * 4)
    state = torch.arange(members * hidden, dtype=torch.float32, device=ctx.device).view(members, hidden)
    link.partial(0, members, hidden, torch.float32).fill_(1.0)
    link.allreduce_residual(0, state, members, hidden, torch.float32)
    logits = torch.randn(members, 1000, device=ctx.device)
    out = torch.zeros(members, dtype=torch.int32, device=ctx.device)
    link.select_tokens(logits, members, 0, out)
    ctx.synchronize()
    assert torch.equal(state, torch.arange(members * hidden, dtype=torch.float32, device=ctx.device).view(members, hidden) + 1)
    assert out.cpu().tolist() == logits.argmax(dim=1).cpu().tolist()
    assert len(link.export_handle()) == 64
