"""Decode loop of a dense grouped-query-attention transformer over the C ABI.

Host-side mirror of the reference's `CudaQwen35Decode::run_step` / `full_attention_layer` /
`run_output_head` (crates/nvidia/src/decode.rs:544-632, :929-1052, :678-696) and their batch twins
(`run_step_batch`, :1990-2140), restricted to dense-attention layers: the order of launches is the
reference's (norm, q/k/v projections, head norms, rope, cache append, attention, output projection,
residual, norm, gate/up, silu_mul, down, residual; final norm, output head, argmax), every launch goes
through libribn_b200.so, and torch only owns device memory, the stream, the CUDA graph and -- for
tensor-parallel runs -- the NCCL process group.

Tensor parallelism (the reference has none): q/k/v/gate/up and the output head are split by output rows,
attention runs on the local heads, o_proj and ffn_down are split by input columns and followed by an
all-reduce (sum) of the partial [members][hidden] outputs; norms and the embedding are replicated.
See sharding.py for the shard arithmetic.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib, synth
from .quantized import CudaQuantizedWeight, CudaQwen35Ops, QwenGemvKernel, RibnContext, WeightTensorSpec, gemm
from .sharding import split_even

Q4_K, Q6_K = 12, 14


@dataclass(frozen=True)
class DenseGeometry:
    hidden: int
    layers: int
    q_heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocabulary: int
    rope_base: float = 1.0e6
    eps: float = 1.0e-6

    @staticmethod
    def qwen3_8b(layers: int = 36) -> "DenseGeometry":
        return DenseGeometry(4096, layers, 32, 8, 128, 12288, 151936)

    @staticmethod
    def qwen3_32b(layers: int = 64) -> "DenseGeometry":
        return DenseGeometry(5120, layers, 64, 8, 128, 25600, 151936)


# The Q4_K_M mix named by the benchmark configuration: attn_v, ffn_down and the output head in Q6_K,
# every other matrix in Q4_K.
VALUE_TYPES = {"attn_q": Q4_K, "attn_k": Q4_K, "attn_v": Q6_K, "attn_output": Q4_K, "ffn_gate": Q4_K, "ffn_up": Q4_K, "ffn_gate_up": Q4_K,
               "ffn_down": Q6_K, "token_embd": Q4_K, "output": Q6_K}


class CudaDenseOps:
    """The layer operators between the GEMVs (CudaQwen35Ops of model_ops.rs, CudaQ4KEmbedding of quantized.rs:913-1161)."""

    def __init__(self, context: RibnContext):
        self.context = context
        self._lib = context._lib

    def embedding(self, weight: CudaQuantizedWeight, tokens: torch.Tensor, output: torch.Tensor) -> None:
        descriptor = weight.descriptor()
        self.context.check(self._lib.ribn_embedding(self.context.handle, ctypes.byref(descriptor), tokens.data_ptr(), tokens.numel(),
                                                    output.data_ptr(), output.numel()))

    def qk_norm_rope_append(self, attention: "_lib.Attention", q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
        self.context.check(self._lib.ribn_qk_norm_rope_append(self.context.handle, ctypes.byref(attention), q.data_ptr(), k.data_ptr(),
                                                              v.data_ptr()))

    def attention_decode(self, attention: "_lib.Attention", q: torch.Tensor, output: torch.Tensor) -> None:
        self.context.check(self._lib.ribn_attention_decode(self.context.handle, ctypes.byref(attention), q.data_ptr(), output.data_ptr()))

    def silu_mul(self, gate: torch.Tensor, up: torch.Tensor, output: torch.Tensor, members: int, length: int, input_row_stride: int) -> None:
        dtype = _lib.RIBN_F32 if output.dtype == torch.float32 else _lib.RIBN_BF16
        self.context.check(self._lib.ribn_silu_mul_typed(self.context.handle, gate.data_ptr(), up.data_ptr(), output.data_ptr(), dtype, members,
                                                         length, input_row_stride))

    def residual_add(self, accumulator: torch.Tensor, addend: torch.Tensor) -> None:
        self.context.check(self._lib.ribn_residual_add(self.context.handle, accumulator.data_ptr(), addend.data_ptr(), accumulator.numel()))

    def argmax(self, logits: torch.Tensor, members: int, output: torch.Tensor) -> None:
        self.context.check(self._lib.ribn_argmax(self.context.handle, logits.data_ptr(), members, logits.numel() // members, output.data_ptr()))


def gemv_fused(context: RibnContext, jobs, x: torch.Tensor, members: int, norm: torch.Tensor | None = None, eps: float = 0.0,
               swiglu: bool = False) -> None:
    """ribn_gemv_fused: `jobs` is a list of (weight, output, accumulate[, second output]); one activation pre-pass serves
    them all.  With a second output the weight holds two projections one after the other (split_rows of the C struct)."""
    array = (_lib.GemvJob * len(jobs))()
    descriptors = [job[0].descriptor() for job in jobs]   # kept alive until the call returns
    for slot, descriptor, job in zip(array, descriptors, jobs):
        weight, y, accumulate = job[:3]
        second = job[3] if len(job) > 3 else None   # a weight that holds two projections: the second one's output
        slot.expected_type = 0
        slot.weight = ctypes.pointer(descriptor)
        slot.y_device = y.data_ptr()
        slot.y_dtype = _lib.RIBN_F32 if y.dtype == torch.float32 else _lib.RIBN_BF16
        slot.y_len = y.numel() + (second.numel() if second is not None else 0)
        slot.accumulate = 1 if accumulate else 0
        slot.split_rows = y.numel() // members if second is not None else 0
        slot.y2_device = second.data_ptr() if second is not None else None
    context.check(context._lib.ribn_gemv_fused(context.handle, array, len(jobs), x.data_ptr(),
                                               _lib.RIBN_F32 if x.dtype == torch.float32 else _lib.RIBN_BF16, x.numel(),
                                               norm.data_ptr() if norm is not None else None, norm.numel() if norm is not None else 0, eps,
                                               members, _lib.RIBN_FUSED_SWIGLU if swiglu else 0))


def attention_descriptor(geometry: DenseGeometry, members: int, q_heads: int, kv_heads: int, q_norm, k_norm, positions, k_cache, v_cache,
                         max_context: int, active_context: int) -> "_lib.Attention":
    return _lib.Attention(members, q_heads, kv_heads, geometry.head_dim, geometry.head_dim, geometry.rope_base, geometry.eps,
                          q_norm.data_ptr() if q_norm is not None else None, k_norm.data_ptr() if k_norm is not None else None,
                          positions.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), max_context, active_context)


class DenseWeights:
    """Encoded matrices and f32 norm vectors of this rank's shard, on the device."""

    def __init__(self):
        self.matrices: dict[str, CudaQuantizedWeight] = {}
        self.vectors: dict[str, torch.Tensor] = {}

    def bytes_per_step(self) -> int:
        """Encoded weight bytes one decode step streams: every matrix once, except the embedding (one row per member)."""
        # attn_qk holds the bytes attn_q and attn_k are views of
        return sum(w.encoded_bytes() for name, w in self.matrices.items() if name != "token_embd" and not name.endswith(".attn_qk"))


def local_shapes(geometry: DenseGeometry, world: int, rank: int) -> dict:
    """[K, N] of each matrix on `rank`: output-row splits on whole heads, input-column splits on whole super-blocks."""
    d = geometry.head_dim
    if geometry.kv_heads % world or geometry.q_heads % world:
        raise ValueError(f"{world} ranks do not divide {geometry.q_heads} query / {geometry.kv_heads} key-value heads")
    q0, q1 = split_even(geometry.q_heads, world, rank)
    kv0, kv1 = split_even(geometry.kv_heads, world, rank)
    i0, i1 = split_even(geometry.intermediate // 256, world, rank)   # whole super-blocks; shares may differ by one
    v0, v1 = split_even(geometry.vocabulary, world, rank)
    local_q, local_kv, local_inter = (q1 - q0) * d, (kv1 - kv0) * d, (i1 - i0) * 256
    return {
        "q_heads": q1 - q0, "kv_heads": kv1 - kv0, "intermediate": local_inter, "vocab_begin": v0, "vocab_end": v1,
        "attn_q": (geometry.hidden, local_q), "attn_k": (geometry.hidden, local_kv), "attn_v": (geometry.hidden, local_kv),
        "attn_output": (local_q, geometry.hidden), "ffn_gate": (geometry.hidden, local_inter), "ffn_up": (geometry.hidden, local_inter),
        "ffn_gate_up": (geometry.hidden, 2 * local_inter),   # rows: this rank's gate rows, then its up rows
        "ffn_down": (local_inter, geometry.hidden), "token_embd": (geometry.hidden, geometry.vocabulary),
        "output": (geometry.hidden, v1 - v0),
    }


def random_weights(context: RibnContext, geometry: DenseGeometry, seed: int = 0, world: int = 1, rank: int = 0) -> DenseWeights:
    """Random-init shard generated on the device (no checkpoint exists for the benchmark configurations):
    block scales and quants as the synthetic GEMV weights, norm vectors 1 + N(0, 0.02)."""
    shapes = local_shapes(geometry, world, rank)
    weights = DenseWeights()
    generator = torch.Generator(device=context.device)
    generator.manual_seed(seed)

    def matrix(name: str, kind: str, salt: int) -> None:
        k, n = shapes[kind]
        vt = VALUE_TYPES[kind]
        shard = 0 if kind == "token_embd" else rank   # the embedding is replicated: every rank generates the same bytes
        data = synth.random_weight_device(vt, k, n, seed=(seed * 7919 + salt * 104729 + shard * 15485863) & 0x7FFFFFFF, device=context.device)
        weights.matrices[name] = CudaQuantizedWeight(WeightTensorSpec.new(name, [k, n]), vt, data)

    def vector(name: str, length: int) -> None:
        weights.vectors[name] = (1.0 + 0.02 * torch.randn(length, device=context.device, generator=generator)).float()

    matrix("token_embd", "token_embd", 1)
    matrix("output", "output", 2)
    vector("output_norm", geometry.hidden)
    for i in range(geometry.layers):
        # ffn_gate and ffn_up are stored as one matrix (gate rows, then up rows): one GEMV writes [gate | up]
        for j, kind in enumerate(("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate_up", "ffn_down")):
            matrix(f"blk.{i}.{kind}", kind, 10 + i * 8 + j)
        vector(f"blk.{i}.attn_norm", geometry.hidden)
        vector(f"blk.{i}.ffn_norm", geometry.hidden)
        vector(f"blk.{i}.attn_q_norm", geometry.head_dim)
        vector(f"blk.{i}.attn_k_norm", geometry.head_dim)
    return weights


def host_model(geometry: DenseGeometry, seed: int = 0):
    """Full (unsharded) encoded tensors and norm vectors generated on the host with numpy, so that every rank of a
    tensor-parallel run -- and the single-GPU run it is compared with -- starts from the same bytes.
    Returns ({name: (value_type, K, N, bytes)}, {name: float32 vector}); gate and up are separate tensors here."""
    import numpy as np

    shapes = local_shapes(geometry, 1, 0)
    rng = np.random.default_rng(seed)
    tensors, vectors = {}, {}
    kinds = ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")
    for name, kind, salt in [("token_embd", "token_embd", 1), ("output", "output", 2)] + [
            (f"blk.{i}.{kind}", kind, 10 + 8 * i + j) for i in range(geometry.layers) for j, kind in enumerate(kinds)]:
        k, n = shapes[kind]
        tensors[name] = (VALUE_TYPES[kind], k, n, synth.random_weight(VALUE_TYPES[kind], k, n, seed=seed * 100 + salt))
    for name, length in [("output_norm", geometry.hidden)] + [(f"blk.{i}.{v}", n) for i in range(geometry.layers)
                                                              for v, n in (("attn_norm", geometry.hidden), ("ffn_norm", geometry.hidden),
                                                                           ("attn_q_norm", geometry.head_dim), ("attn_k_norm", geometry.head_dim))]:
        vectors[name] = (1 + 0.02 * rng.standard_normal(length)).astype(np.float32)
    return tensors, vectors


def shard_host_model(context: RibnContext, geometry: DenseGeometry, tensors: dict, vectors: dict, world: int, rank: int) -> DenseWeights:
    """Rank `rank`'s shard of a host_model, uploaded: q/k/v by whole heads, the output head by rows, o_proj and ffn_down by
    input super-blocks, gate and up by rows of whole super-blocks and stored as one [gate | up] matrix (sharding.py)."""
    import numpy as np

    from . import sharding

    weights = DenseWeights()

    def put(name, vt, k, n, data):
        weights.matrices[name] = CudaQuantizedWeight(WeightTensorSpec.new(name, [k, n]), vt, torch.from_numpy(np.ascontiguousarray(data)).to(context.device))

    for name, (vt, k, n, data) in tensors.items():
        kind = name.split(".")[-1]
        if kind == "token_embd":
            put(name, vt, k, n, data)
        elif kind in ("attn_q", "attn_k", "attn_v"):
            part, (kk, nn) = sharding.shard_rows(data, vt, k, n, world, rank, multiple=geometry.head_dim)
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


class CudaDenseDecode:
    """One decode step for `members` sequences (one new token each), replayable as a CUDA graph.

    `process_group` (a torch.distributed NCCL group) makes it one rank of a tensor-parallel run; weights
    must then be that rank's shard (see local_shapes)."""

    def __init__(self, context: RibnContext, geometry: DenseGeometry, weights: DenseWeights, members: int, max_context: int,
                 process_group=None, world: int = 1, rank: int = 0, peer_link=None, partial_dtype: torch.dtype = torch.float32):
        self.context, self.geometry, self.weights, self.members, self.max_context = context, geometry, weights, members, max_context
        self.group, self.world, self.rank = process_group, world, rank
        # peer_link (engine_b200.tp.PeerLink, connected): the sums after o_proj / ffn_down and the token choice run as
        # one kernel each over peer memory instead of NCCL collectives plus elementwise launches
        self.link, self.partial_dtype = peer_link, partial_dtype
        self.skip_exchange = False   # timing aid: leave the exchanges out of a captured step (results are then wrong)
        self.shapes = local_shapes(geometry, world, rank)
        self.ops = CudaDenseOps(context)
        self.kernels = {vt: QwenGemvKernel.from_value_type(vt, context) for vt in (Q4_K, Q6_K)}
        dev, g, s, m = context.device, geometry, self.shapes, members
        f32 = dict(dtype=torch.float32, device=dev)
        self.tokens = torch.zeros(m, dtype=torch.int32, device=dev)       # u32 on the device side
        self.positions = torch.zeros(m, dtype=torch.int32, device=dev)
        self.hidden = torch.zeros(m, g.hidden, **f32)
        # q and k projections of the same format are stored as one matrix (q rows, then k rows) and run as one GEMV:
        # for one sequence [q | k] is contiguous in the output; batches name the second output (split_rows).
        # attn_q and attn_k stay available as views of the joined bytes (the prefill GEMM uses them).
        q_dim, k_dim = s["q_heads"] * g.head_dim, s["kv_heads"] * g.head_dim
        self.qk_weights = {}
        for i in range(g.layers):
            wq, wk = weights.matrices.get(f"blk.{i}.attn_q"), weights.matrices.get(f"blk.{i}.attn_k")
            joined = weights.matrices.get(f"blk.{i}.attn_qk")
            if joined is None and wq is not None and wk is not None and wq.value_type() == wk.value_type() and q_dim % 128 == 0:
                data = torch.cat([wq.encoded_data(), wk.encoded_data()])
                joined = CudaQuantizedWeight(WeightTensorSpec.new(f"blk.{i}.attn_qk", [g.hidden, q_dim + k_dim]), wq.value_type(), data)
                weights.matrices[f"blk.{i}.attn_qk"] = joined
                q_bytes = wq.encoded_bytes()
                weights.matrices[f"blk.{i}.attn_q"] = CudaQuantizedWeight(wq.spec(), wq.value_type(), data[:q_bytes])
                weights.matrices[f"blk.{i}.attn_k"] = CudaQuantizedWeight(wk.spec(), wk.value_type(), data[q_bytes:])
            if joined is not None:
                self.qk_weights[i] = joined
        self.qk = torch.zeros(m, q_dim + k_dim, **f32)
        self.q = self.qk[:, :q_dim] if m == 1 else torch.zeros(m, q_dim, **f32)
        self.k = self.qk[:, q_dim:] if m == 1 else torch.zeros(m, k_dim, **f32)
        self.v = torch.zeros(m, s["kv_heads"] * g.head_dim, **f32)
        self.attended = torch.zeros(m, s["q_heads"] * g.head_dim, **f32)
        self.projected = torch.zeros(m, g.hidden, **f32)
        self.gate_up = torch.zeros(m, 2 * s["intermediate"], **f32)
        self.logits = torch.zeros(m, s["vocab_end"] - s["vocab_begin"], **f32)
        self.next_tokens = torch.zeros(m, dtype=torch.int32, device=dev)
        cache_shape = (g.layers, m, s["kv_heads"], max_context, g.head_dim)
        self.k_cache = torch.zeros(cache_shape, dtype=torch.float16, device=dev)
        self.v_cache = torch.zeros(cache_shape, dtype=torch.float16, device=dev)
        self.active_context = max_context
        self.prefill_scratch: dict | None = None
        self.graph = None
        self.launches_per_step = 0
        if members > 4:
            # Batches go to the tensor-core kernel, which rounds the f32 activations to f16 (inside the 2e-3 bound).
            context.set_option("tc_f32_activations", 1)

    # -- building blocks -------------------------------------------------------------------------
    def _fused(self, names_outputs, x: torch.Tensor, norm: torch.Tensor | None = None, swiglu: bool = False, accumulate: bool = False) -> None:
        jobs = [(self.weights.matrices[name], y, accumulate) for name, y in names_outputs]
        gemv_fused(self.context, jobs, x, self.members, norm, self.geometry.eps, swiglu)
        # one launch per projection, plus the activation pre-pass where one runs (from three members on, for wide
        # two-member inputs, for gated inputs, and whenever several projections share a normalised input)
        shared = len(jobs) > 1 and norm is not None and self.members >= 2
        prepass = self.members >= 3 or shared or swiglu or x.shape[-1] // 256 > 24
        self.launches_per_step += len(jobs) + (1 if prepass else 0)

    def _all_reduce(self, t: torch.Tensor) -> None:
        if not self.skip_exchange:
            torch.distributed.all_reduce(t, group=self.group)
            self.launches_per_step += 1

    def _exchange(self, slot: int) -> None:
        if not self.skip_exchange:
            self.link.allreduce_residual(slot, self.hidden, self.members, self.geometry.hidden, self.partial_dtype)
            self.launches_per_step += 1

    def _layer(self, i: int) -> None:
        g, s, w = self.geometry, self.shapes, self.weights
        parallel = self.group is not None and self.world > 1
        if i in self.qk_weights:
            qk_job = (self.qk_weights[i], self.qk, False) if self.members == 1 else (self.qk_weights[i], self.q, False, self.k)
            gemv_fused(self.context, [qk_job, (w.matrices[f"blk.{i}.attn_v"], self.v, False)], self.hidden, self.members,
                       w.vectors[f"blk.{i}.attn_norm"], g.eps, False)
            # one row: every CTA normalises and converts it itself; from two rows on one pre-pass serves the launches,
            # and only the batch kernel (nine rows and more) writes q and k from one launch
            self.launches_per_step += 2 if self.members == 1 else (3 if self.members >= 9 else 4)
        else:
            self._fused([(f"blk.{i}.attn_q", self.q), (f"blk.{i}.attn_k", self.k), (f"blk.{i}.attn_v", self.v)], self.hidden,
                        norm=w.vectors[f"blk.{i}.attn_norm"])
        attention = attention_descriptor(g, self.members, s["q_heads"], s["kv_heads"], w.vectors[f"blk.{i}.attn_q_norm"],
                                         w.vectors[f"blk.{i}.attn_k_norm"], self.positions, self.k_cache[i], self.v_cache[i],
                                         self.max_context, self.active_context)
        self.ops.qk_norm_rope_append(attention, self.q, self.k, self.v)
        self.ops.attention_decode(attention, self.q, self.attended)
        self.launches_per_step += 3   # head norm + rope + cache append; split-KV attention; merge of the splits
        if parallel and self.link is not None:
            # partial sums of the column-split projection go straight into the link's slot; one kernel pulls the peers'
            self._fused([(f"blk.{i}.attn_output", self.link.partial(0, self.members, g.hidden, self.partial_dtype))], self.attended)
            self._exchange(0)
        elif parallel:
            # partial sums of the column-split projection: all-reduce, then the residual
            self._fused([(f"blk.{i}.attn_output", self.projected)], self.attended)
            self._all_reduce(self.projected)
            self.ops.residual_add(self.hidden, self.projected)
            self.launches_per_step += 1
        else:
            self._fused([(f"blk.{i}.attn_output", self.hidden)], self.attended, accumulate=True)      # hidden += W attended
        self._fused([(f"blk.{i}.ffn_gate_up", self.gate_up)], self.hidden, norm=w.vectors[f"blk.{i}.ffn_norm"])
        if parallel and self.link is not None:
            self._fused([(f"blk.{i}.ffn_down", self.link.partial(1, self.members, g.hidden, self.partial_dtype))], self.gate_up, swiglu=True)
            self._exchange(1)
        elif parallel:
            self._fused([(f"blk.{i}.ffn_down", self.projected)], self.gate_up, swiglu=True)
            self._all_reduce(self.projected)
            self.ops.residual_add(self.hidden, self.projected)
            self.launches_per_step += 1
        else:
            self._fused([(f"blk.{i}.ffn_down", self.hidden)], self.gate_up, swiglu=True, accumulate=True)

    def _forward(self) -> None:
        self.launches_per_step = 0
        self.ops.embedding(self.weights.matrices["token_embd"], self.tokens, self.hidden)
        for i in range(self.geometry.layers):
            self._layer(i)
        self._fused([("output", self.logits)], self.hidden, norm=self.weights.vectors["output_norm"])
        self.launches_per_step += 1
        if self.world == 1:
            self.ops.argmax(self.logits, self.members, self.next_tokens)
            self.launches_per_step += 1

    def _select_tokens_tensor_parallel(self, logits: torch.Tensor | None = None, out: torch.Tensor | None = None) -> None:
        """Each rank holds a slice of the logits: local argmax, then the best (value, index) over the ranks."""
        logits = self.logits if logits is None else logits
        out = self.next_tokens if out is None else out
        rows = logits.shape[0]
        if self.link is not None and out.data_ptr() % 16 == 0 and logits.data_ptr() % 16 == 0:
            self.link.select_tokens(logits, rows, self.shapes["vocab_begin"], out)
            self.launches_per_step += 1
            return
        local = torch.empty(rows, dtype=torch.int32, device=self.context.device)
        self.ops.argmax(logits, rows, local)
        values = logits.gather(1, local.long().unsqueeze(1)).squeeze(1)
        gathered_values = [torch.empty_like(values) for _ in range(self.world)]
        gathered_indices = [torch.empty_like(local) for _ in range(self.world)]
        torch.distributed.all_gather(gathered_values, values, group=self.group)
        torch.distributed.all_gather(gathered_indices, local + self.shapes["vocab_begin"], group=self.group)
        all_values = torch.stack(gathered_values)            # [world][members]
        # the rules of ribn_argmax across ranks: NaN never wins (a rank whose slice is all NaN reports its first index with
        # a NaN value), and argmax returns the first of equal maxima, i.e. the lowest rank = the lowest token index
        all_values = torch.where(torch.isnan(all_values), torch.full_like(all_values, float("-inf")), all_values)
        best = all_values.argmax(dim=0)
        out.copy_(torch.stack(gathered_indices).gather(0, best.unsqueeze(0)).squeeze(0))

    # -- prefill ------------------------------------------------------------------------------------
    def _prefill_buffers(self, chunk: int) -> dict:
        if self.prefill_scratch is not None and self.prefill_scratch["chunk"] >= chunk:
            return self.prefill_scratch
        g, s, dev = self.geometry, self.shapes, self.context.device
        f32, bf16 = dict(dtype=torch.float32, device=dev), dict(dtype=torch.bfloat16, device=dev)
        q_dim, kv_dim = s["q_heads"] * g.head_dim, s["kv_heads"] * g.head_dim
        self.prefill_scratch = {
            "chunk": chunk, "tokens": torch.zeros(chunk, dtype=torch.int32, device=dev), "positions": torch.zeros(chunk, dtype=torch.int32, device=dev),
            "hidden": torch.zeros(chunk, g.hidden, **f32), "normed": torch.zeros(chunk, g.hidden, **bf16),
            "q": torch.zeros(chunk, q_dim, **f32), "k": torch.zeros(chunk, kv_dim, **f32), "v": torch.zeros(chunk, kv_dim, **f32),
            "attended": torch.zeros(chunk, q_dim, **bf16), "projected": torch.zeros(chunk, g.hidden, **f32),
            "gate_up": torch.zeros(chunk, 2 * s["intermediate"], **f32), "activated": torch.zeros(chunk, s["intermediate"], **bf16),
        }
        return self.prefill_scratch

    def _prefill_chunk(self, tokens: torch.Tensor, sequence: int, start: int) -> torch.Tensor:
        """One chunk of consecutive prompt tokens of one sequence through every layer (run_prefill_chunk,
        decode.rs:2149-2267; attention per token over the shared cache, :2945-3021).  The projections are
        ribn_gemm over the whole chunk instead of eight-row GEMVs.  Returns the chunk's hidden rows."""
        g, s, w, ctx = self.geometry, self.shapes, self.weights, self.context
        count = tokens.numel()
        b = self._prefill_buffers(count)
        rows = lambda name: b[name][:count]                                        # leading rows: contiguous
        norms = CudaQwen35Ops(ctx)
        parallel = self.group is not None and self.world > 1
        b["tokens"][:count].copy_(tokens)
        torch.arange(start, start + count, dtype=torch.int32, device=ctx.device, out=b["positions"][:count])
        hidden, normed, projected, gate_up = rows("hidden"), rows("normed"), rows("projected"), rows("gate_up")
        self.ops.embedding(w.matrices["token_embd"], b["tokens"][:count], hidden)
        for i in range(g.layers):
            norms.rms_norm_batch(hidden, w.vectors[f"blk.{i}.attn_norm"], normed, g.hidden, g.eps)
            for name, out in (("attn_q", rows("q")), ("attn_k", rows("k")), ("attn_v", rows("v"))):
                gemm(ctx, w.matrices[f"blk.{i}.{name}"], normed, out)
            attention = attention_descriptor(g, count, s["q_heads"], s["kv_heads"], w.vectors[f"blk.{i}.attn_q_norm"],
                                             w.vectors[f"blk.{i}.attn_k_norm"], b["positions"], self.k_cache[i][sequence],
                                             self.v_cache[i][sequence], self.max_context, start + count)
            attention.shared_cache, attention.out_dtype = 1, _lib.RIBN_BF16
            self.ops.qk_norm_rope_append(attention, rows("q"), rows("k"), rows("v"))
            self.ops.attention_decode(attention, rows("q"), rows("attended"))
            gemm(ctx, w.matrices[f"blk.{i}.attn_output"], rows("attended"), projected)
            if parallel:
                torch.distributed.all_reduce(projected, group=self.group)
            self.ops.residual_add(hidden, projected)
            norms.rms_norm_batch(hidden, w.vectors[f"blk.{i}.ffn_norm"], normed, g.hidden, g.eps)
            gemm(ctx, w.matrices[f"blk.{i}.ffn_gate_up"], normed, gate_up)
            inter = s["intermediate"]
            self.ops.silu_mul(gate_up[:, :inter], gate_up[:, inter:], rows("activated"), count, inter, 2 * inter)
            gemm(ctx, w.matrices[f"blk.{i}.ffn_down"], rows("activated"), projected)
            if parallel:
                torch.distributed.all_reduce(projected, group=self.group)
            self.ops.residual_add(hidden, projected)
        return hidden

    def prefill(self, tokens, sequence: int = 0, start: int = 0, chunk: int = 512) -> None:
        """Fill the KV cache of `sequence` from prompt `tokens` at positions start.. (run_prefill_chunks,
        crates/nvidia/src/serving.rs:136 over decode.rs:1953-1977), `chunk` tokens per pass.  Afterwards the
        sequence is ready for run_step: positions[sequence] is the first free slot and tokens[sequence] the
        token chosen from the last prompt token's logits (also left in next_tokens[sequence])."""
        tokens = torch.as_tensor(tokens, dtype=torch.int32).to(self.context.device)
        if tokens.numel() == 0:
            raise ValueError("a prompt needs at least one token")
        if start + tokens.numel() > self.max_context:
            raise ValueError(f"prompt end {start + tokens.numel()} exceeds the cache of {self.max_context} tokens")
        with torch.cuda.stream(self.context.stream):
            for begin in range(0, tokens.numel(), chunk):
                part = tokens[begin:begin + chunk]
                hidden = self._prefill_chunk(part, sequence, start + begin)
            last = hidden[part.numel() - 1:part.numel()]
            logits = self.logits[sequence:sequence + 1]
            if logits.data_ptr() % 16:                                # a row of an odd vocabulary: go through an aligned row
                logits = torch.empty_like(logits)
            gemv_fused(self.context, [(self.weights.matrices["output"], logits, False)], last, 1, self.weights.vectors["output_norm"],
                       self.geometry.eps)
            chosen = self._prefill_buffers(1)["tokens"][:1]          # an aligned word of its own: entry points want 16-byte alignment
            if self.world > 1:
                self._select_tokens_tensor_parallel(logits, chosen)
            else:
                self.ops.argmax(logits, 1, chosen)
            if logits.data_ptr() != self.logits[sequence:sequence + 1].data_ptr():
                self.logits[sequence:sequence + 1].copy_(logits)
            self.next_tokens[sequence:sequence + 1].copy_(chosen)
            self.tokens[sequence:sequence + 1].copy_(chosen)
            self.positions[sequence:sequence + 1].fill_(start + tokens.numel())

    # -- public ------------------------------------------------------------------------------------
    def run_step(self) -> None:
        """tokens, positions -> next_tokens (all device resident); appends to the KV cache at `positions`."""
        with torch.cuda.stream(self.context.stream):
            self._forward()
            if self.world > 1:
                self._select_tokens_tensor_parallel()

    def capture(self, advance: bool = False) -> None:
        """Record run_step into a CUDA graph (positions and tokens are read from device memory at replay).
        With `advance` the graph also feeds the chosen tokens back and increments the positions, so that
        one replay is one generated token per sequence."""
        self.run_step()   # first launches set kernel attributes, which a capture must not contain
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=self.context.stream):
            self._forward()
            if self.world > 1:
                self._select_tokens_tensor_parallel()
            if advance:
                self.tokens.copy_(self.next_tokens)
                self.positions.add_(1)
        self.graph = graph

    def fill_context(self, tokens_in_context: int, seed: int = 0) -> None:
        """Stand-in for a prompt of `tokens_in_context` random tokens: the cache positions below it get random
        f16 keys and values (what a random prompt leaves there, at none of the prefill cost), positions point
        at the next free slot and every sequence starts from a random token."""
        generator = torch.Generator(device=self.context.device)
        generator.manual_seed(seed + self.rank)
        with torch.cuda.stream(self.context.stream):
            for cache in (self.k_cache, self.v_cache):
                for layer in range(self.geometry.layers):
                    view = cache[layer][:, :, :tokens_in_context]
                    view.copy_(torch.randn(view.shape, device=self.context.device, generator=generator, dtype=torch.float32).to(torch.float16))
            self.positions.fill_(tokens_in_context)
            token_generator = torch.Generator(device=self.context.device)
            token_generator.manual_seed(seed)   # the same tokens on every rank
            self.tokens.copy_(torch.randint(0, self.geometry.vocabulary, (self.members,), device=self.context.device, generator=token_generator,
                                            dtype=torch.int32))
        torch.cuda.synchronize()

    def replay(self) -> None:
        with torch.cuda.stream(self.context.stream):
            self.graph.replay()

    def advance(self) -> None:
        """Feed the chosen tokens back and move every sequence one position on (device-side, graph-safe)."""
        with torch.cuda.stream(self.context.stream):
            self.tokens.copy_(self.next_tokens)
            self.positions.add_(1)
