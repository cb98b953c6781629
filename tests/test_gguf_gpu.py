"""Staged upload of GGUF tensors to the device (ribn_materialize_quantized), whole and as tensor-parallel shards, on a
synthetic GGUF v3 file written by the test; the uploaded bytes must be the file's, shards must equal the host-side
shard arithmetic (engine_b200/sharding.py), and a GEMV over an uploaded tensor must equal the one over a torch copy."""
import os

import numpy as np
import pytest
import torch

import engine_b200
import oracle
from engine_b200 import gguf, sharding, synth

pytestmark = pytest.mark.gpu

K, N = 1024, 40
BIG_K, BIG_N = 4096, 5000          # 11.5 MiB of Q4_K: more than one staging piece, a ragged last one


@pytest.fixture(scope="module")
def checkpoint(tmp_path_factory):
    path = os.path.join(tmp_path_factory.mktemp("gguf"), "synthetic.gguf")
    tensors = {f"blk.0.w{vt}": (vt, K, N, synth.random_weight(vt, K, N, seed=vt)) for vt in (8, 12, 13, 14)}
    tensors["big"] = (12, BIG_K, BIG_N, synth.random_weight(12, BIG_K, BIG_N, seed=99))
    gguf.write_gguf(path, [("general.architecture", 8, "qwen3"), ("qwen3.block_count", 4, 1)],
                    [(name, (k, n), vt, data.tobytes()) for name, (vt, k, n, data) in tensors.items()])
    return gguf.GgufFile.open(path), tensors


def test_whole_tensors_arrive_byte_for_byte(ctx, checkpoint):
    file, tensors = checkpoint
    store = engine_b200.CudaWeightStore(ctx)
    for name, (vt, k, n, data) in tensors.items():
        weight = gguf.materialize_quantized(store, file, name)
        ctx.synchronize()
        assert weight.value_type() == vt and weight.spec().dimensions == (k, n)
        assert np.array_equal(weight.encoded_data().cpu().numpy(), data.reshape(-1))
        assert store.quantized_tensor(name) is weight


@pytest.mark.parametrize("world", [2, 3, 8])
def test_shards_equal_the_host_arithmetic(ctx, checkpoint, world):
    file, tensors = checkpoint
    for name, (vt, k, n, data) in tensors.items():
        if name == "big" and world != 3:
            continue
        for rank in range(world):
            store = engine_b200.CudaWeightStore(ctx)
            rows = gguf.materialize_quantized(store, file, name, shard="rows", world=world, rank=rank, store_as="rows")
            want_rows, dims_rows = sharding.shard_rows(data, vt, k, n, world, rank)
            want_cols, dims_cols, _ = sharding.shard_k(data, vt, k, n, world, rank)
            if want_cols.size == 0:       # four super-blocks over eight ranks: the last ranks hold nothing, which an upload refuses
                with pytest.raises(gguf.GgufError) as e:
                    gguf.materialize_quantized(store, file, name, shard="input", world=world, rank=rank, store_as="cols")
                assert e.value.kind == "InvalidWeight"
            else:
                cols = gguf.materialize_quantized(store, file, name, shard="input", world=world, rank=rank, store_as="cols")
                ctx.synchronize()
                assert cols.spec().dimensions == dims_cols
                assert np.array_equal(cols.encoded_data().cpu().numpy(), want_cols)
            ctx.synchronize()
            assert rows.spec().dimensions == dims_rows
            assert np.array_equal(rows.encoded_data().cpu().numpy(), want_rows)


def test_gemv_over_an_uploaded_shard(ctx, checkpoint):
    file, tensors = checkpoint
    vt, k, n, data = tensors["blk.0.w14"]
    store = engine_b200.CudaWeightStore(ctx)
    world = 2
    x = np.random.default_rng(0).standard_normal(k).astype(np.float32)
    total = np.zeros(n)
    for rank in range(world):
        shard = gguf.materialize_quantized(store, file, "blk.0.w14", shard="input", world=world, rank=rank, store_as=f"r{rank}")
        k0, k1 = sharding.k_range(k, world, rank)
        y = torch.zeros(n, device=ctx.device)
        engine_b200.QwenGemvKernel.from_value_type(vt, ctx).execute(shard, torch.from_numpy(x[k0:k1].copy()).to(ctx.device), y)
        ctx.synchronize()
        total += y.cpu().numpy().astype(np.float64)
    ref = oracle.gemv_f64(vt, data, k, n, x[None])[0]
    assert oracle.max_rel_error(total, ref, oracle.gemv_scale(vt, data, k, n, x[None])[0]) <= 2e-3


def test_upload_rejections(ctx, checkpoint, tmp_path):
    file, tensors = checkpoint
    lib, handle = ctx._lib, ctx.handle
    size = tensors["blk.0.w12"][3].size
    dst = torch.zeros(size + 16, dtype=torch.uint8, device=ctx.device)
    status = lib.ribn_materialize_quantized(handle, file._handle, b"blk.0.w12", 0, 0, 0, dst.data_ptr(), size - 1)
    assert status == engine_b200._lib.RIBN_E_OUTPUT_LENGTH
    status = lib.ribn_materialize_quantized(handle, file._handle, b"absent", 0, 0, 0, dst.data_ptr(), size)
    assert gguf.ERROR_KINDS[status] == "MissingTensor"
    # a file cut short after it was opened: the source ends early
    path = os.path.join(tmp_path, "cut.gguf")
    gguf.write_gguf(path, [], [("w", (K, N), 12, tensors["blk.0.w12"][3].tobytes())])
    cut = gguf.GgufFile.open(path)
    extent = cut.tensor_data_range("w")
    os.truncate(path, extent.start + 1000)
    status = lib.ribn_materialize_quantized(handle, cut._handle, b"w", 0, 0, 0, dst.data_ptr(), size)
    assert gguf.ERROR_KINDS[status] == "UnexpectedEof"
    ctx.synchronize()
