"""The reference project's own CUDA decode step at a dense Qwen3 geometry, composed from its unmodified kernels.

TEST / BASELINE INFRASTRUCTURE ONLY: the shipped library never loads these cubins.  The reference's layer
forward is Rust host code that cannot be built here; what it does per token is a fixed sequence of kernel
launches, restated below launch for launch from

    crates/nvidia/src/decode.rs:544-632     run_step: embedding, per layer rms_norm -> attention -> rms_norm -> FFN
    crates/nvidia/src/decode.rs:929-1052    full_attention_layer: q, head norm, k, head norm, v, rope x2, kv_append,
                                            attn_score_gqa, o projection, residual_add
    crates/nvidia/src/decode.rs:678-696     run_output_head: rms_norm, output projection, argmax
    crates/nvidia/src/decode.rs:1990-2140, :2868-3036   the batched twins (members <= 8): *_batch kernels, one
                                            kv_append + attn_score_gqa launch per member

with the launch geometry of crates/nvidia/src/model_ops.rs (rms_norm 1 x 256, strided_rms_norm ceil(heads/64) x 64,
rope_neox ceil(pairs/64) x 64, kv_append_f16 ceil(total/256) x 256, attn_score_gqa one warp per (row, q head) in
blocks of four warps, silu_mul / residual_add ceil(n/256) x 256, argmax 1 x 1024) and of
crates/nvidia/src/quantized.rs (gemv_warp ceil(N/4) x 128; gemv_warp_batch ceil(ceil(N/2)/4) x 128).

Substitutions, because the reference's attention is the Qwen3.5 gated variant and its model is a hybrid:
  * q head norm: `strided_rms_norm` (the generic per-head norm) in place of `q_gate_norm`, which expects the
    q projection to carry a gate half per head;
  * `attn_score_gqa` multiplies its output by sigmoid(gate): it gets a constant gate buffer of +88.0, for which
    sigmoid is exactly 1.0f;
  * gate and up projections are two launches over the two halves of one stored [gate | up] matrix;
  * token and position are kernel arguments in the reference (the host passes them every step); a replayed CUDA
    graph keeps the values it was captured with, so the timed steps all run at one position (the middle of the
    generated range), write the same cache slot and embed the same token.  Launch count and bytes moved per
    step are those of a real step at that position.
"""
from __future__ import annotations

import ctypes

from . import ref_cuda


class ReferenceModelOps:
    """The kernels of the CUDA source string embedded in model_ops.rs (compiled by build_ref.py), plus the GEMV and
    embedding kernels of the quantized families."""

    def __init__(self):
        import torch
        from cuda.bindings import driver

        self._torch = torch
        self._driver = driver
        self.gemv = ref_cuda.ReferenceKernels()
        with open(ref_cuda.MODEL_OPS_CUBIN, "rb") as f:
            self._image = f.read()
        self._module = ref_cuda._check(driver.cuModuleLoadData(self._image))
        self._functions = {}
        self.launches = 0

    def _function(self, name):
        if name not in self._functions:
            self._functions[name] = ref_cuda._check(self._driver.cuModuleGetFunction(self._module, name.encode()))
        return self._functions[name]

    def launch(self, name, blocks, threads, args, module_function=None):
        """args: list of (ctype, value)."""
        stream = self._torch.cuda.current_stream().cuda_stream
        values = tuple(v for _, v in args)
        types = tuple(t for t, _ in args)
        function = module_function if module_function is not None else self._function(name)
        ref_cuda._check(self._driver.cuLaunchKernel(function, blocks, 1, 1, threads, 1, 1, 0, stream, (values, types), 0))
        self.launches += 1


P, I, F, L, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_uint


class ReferenceDenseDecode:
    """One decode step of a dense model with the reference's kernels.  `weights` is an engine_b200.decode.DenseWeights
    of an unsharded model (gate and up stored as one matrix)."""

    def __init__(self, geometry, weights, members: int, max_context: int, device):
        import torch

        if members not in (1,) and not (2 <= members <= ref_cuda.MAX_BATCH_MEMBERS):
            raise ValueError("the reference's batch kernels serve at most eight members")
        self.ops = ReferenceModelOps()
        self.g, self.w, self.members, self.max_context = geometry, weights, members, max_context
        g, m = geometry, members
        f32 = dict(dtype=torch.float32, device=device)
        self.hidden = torch.zeros(m, g.hidden, **f32)
        self.normed = torch.zeros(m, g.hidden, **f32)
        self.q_raw = torch.zeros(m, g.q_heads * g.head_dim, **f32)
        self.q_packed = torch.zeros_like(self.q_raw)
        self.k_raw = torch.zeros(m, g.kv_heads * g.head_dim, **f32)
        self.k_normed = torch.zeros_like(self.k_raw)
        self.v_raw = torch.zeros_like(self.k_raw)
        self.attn_out = torch.zeros(m, g.q_heads * g.head_dim, **f32)
        self.incr = torch.zeros(m, g.hidden, **f32)
        self.gate = torch.zeros(m, g.intermediate, **f32)
        self.up = torch.zeros(m, g.intermediate, **f32)
        self.act = torch.zeros(m, g.intermediate, **f32)
        self.logits = torch.zeros(m, g.vocabulary, **f32)
        self.selected = torch.zeros(m, dtype=torch.int32, device=device)
        self.tokens = torch.zeros(m, dtype=torch.int32, device=device)
        self.positions64 = torch.zeros(m, dtype=torch.int64, device=device)
        # the sigmoid gate of attn_score_gqa reads [q_heads][2 * head_dim] and uses the second half of each slice
        self.gate_one = torch.full((g.q_heads * 2 * g.head_dim,), 88.0, **f32)
        self.scores = torch.zeros(m, g.q_heads * max_context, **f32)
        # reference cache layout: [token][kv_head][dim] f16, one pair per (layer, member)
        shape = (g.layers, m, max_context, g.kv_heads, g.head_dim)
        self.k_cache = torch.zeros(shape, dtype=torch.float16, device=device)
        self.v_cache = torch.zeros(shape, dtype=torch.float16, device=device)

    def fill_context(self, tokens_in_context: int, seed: int = 0) -> None:
        torch = self.ops._torch
        generator = torch.Generator(device=self.hidden.device)
        generator.manual_seed(seed)
        for cache in (self.k_cache, self.v_cache):
            for layer in range(self.g.layers):
                view = cache[layer][:, :tokens_in_context]
                view.copy_(torch.randn(view.shape, device=view.device, generator=generator, dtype=torch.float32).to(torch.float16))

    # -- the reference's wrappers, batch-1 or batched -------------------------------------------------------------
    def _gemv(self, weight, x, y, row_begin=0, rows=None):
        k, n = weight.spec().dimensions[0], weight.spec().dimensions[1]
        rows = n if rows is None else rows
        data = weight.encoded_data()
        row_bytes = data.numel() // n
        view = data[row_begin * row_bytes:(row_begin + rows) * row_bytes]
        self.ops.gemv.gemv(weight.value_type(), view, x, y, k, rows, self.members)
        self.ops.launches += ref_cuda.launches_for(self.members)

    def _rms_norm(self, x, weight, y):
        g, m = self.g, self.members
        if m == 1:
            self.ops.launch("rms_norm", 1, 256, [(P, x.data_ptr()), (P, weight.data_ptr()), (P, y.data_ptr()), (I, g.hidden), (F, g.eps)])
        else:
            self.ops.launch("rms_norm_batch", m, 256, [(P, x.data_ptr()), (P, weight.data_ptr()), (P, y.data_ptr()), (I, g.hidden), (F, g.eps)])

    def _head_norm(self, x, weight, y, heads):
        g, m = self.g, self.members
        if m == 1:
            self.ops.launch("strided_rms_norm", (heads + 63) // 64, 64,
                            [(P, x.data_ptr()), (P, weight.data_ptr()), (P, y.data_ptr()), (I, heads), (I, g.head_dim), (F, g.eps)])
        else:
            self.ops.launch("strided_rms_norm_batch", (heads * m + 63) // 64, 64,
                            [(P, x.data_ptr()), (P, weight.data_ptr()), (P, y.data_ptr()), (I, heads), (I, g.head_dim), (F, g.eps), (I, m)])

    def _rope(self, values, heads, position):
        g, m = self.g, self.members
        pairs = g.head_dim // 2
        if m == 1:
            self.ops.launch("rope_neox", (heads * pairs + 63) // 64, 64,
                            [(P, values.data_ptr()), (L, position), (I, heads), (I, g.head_dim), (I, pairs), (F, g.rope_base)])
        else:
            self.ops.launch("rope_neox_batch", (m * heads * pairs + 63) // 64, 64,
                            [(P, values.data_ptr()), (P, self.positions64.data_ptr()), (I, heads), (I, g.head_dim), (I, pairs), (F, g.rope_base), (I, m)])

    def _elementwise(self, name, length, pointers):
        self.ops.launch(name, (length + 255) // 256, 256, [(P, p.data_ptr()) for p in pointers] + [(I, length)])

    def step(self, token: int, position: int) -> None:
        """Launches one decode step for every member at `position` (the same token and position for all members)."""
        g, w, m = self.g, self.w, self.members
        mats, vecs = w.matrices, w.vectors
        embed = mats["token_embd"]
        if m == 1:
            self.ops.launch("q4_k_embedding", (g.hidden + 255) // 256, 256,
                            [(P, embed.encoded_data().data_ptr()), (U, token), (P, self.hidden.data_ptr()), (I, g.hidden), (I, g.vocabulary)],
                            module_function=self.ops.gemv._function("q4_k_embedding"))
        else:
            self.tokens.fill_(token)
            self.positions64.fill_(position)
            self.ops.launch("q4_k_embedding_batch", (m * g.hidden + 255) // 256, 256,
                            [(P, embed.encoded_data().data_ptr()), (P, self.tokens.data_ptr()), (P, self.hidden.data_ptr()), (I, g.hidden),
                             (I, g.vocabulary), (I, m)], module_function=self.ops.gemv._function("q4_k_embedding_batch"))
        kv_total = g.kv_heads * g.head_dim
        for i in range(g.layers):
            self._rms_norm(self.hidden, vecs[f"blk.{i}.attn_norm"], self.normed)
            self._gemv(mats[f"blk.{i}.attn_q"], self.normed, self.q_raw)
            self._head_norm(self.q_raw, vecs[f"blk.{i}.attn_q_norm"], self.q_packed, g.q_heads)
            self._gemv(mats[f"blk.{i}.attn_k"], self.normed, self.k_raw)
            self._head_norm(self.k_raw, vecs[f"blk.{i}.attn_k_norm"], self.k_normed, g.kv_heads)
            self._gemv(mats[f"blk.{i}.attn_v"], self.normed, self.v_raw)
            self._rope(self.q_packed, g.q_heads, position)
            self._rope(self.k_normed, g.kv_heads, position)
            for member in range(m):
                keys, values = self.k_cache[i, member], self.v_cache[i, member]
                self.ops.launch("kv_append_f16", (kv_total + 127) // 128, 128,
                                [(P, self.k_normed[member].data_ptr()), (P, self.v_raw[member].data_ptr()), (P, keys.data_ptr()), (P, values.data_ptr()),
                                 (I, position), (I, g.kv_heads), (I, g.head_dim)])
                self.ops.launch("attn_score_gqa", (g.q_heads + 3) // 4, 128,
                                [(P, self.q_packed[member].data_ptr()), (P, keys.data_ptr()), (P, values.data_ptr()), (P, self.gate_one.data_ptr()),
                                 (P, self.scores[member].data_ptr()), (P, self.attn_out[member].data_ptr()), (I, position + 1), (I, 1),
                                 (I, self.max_context), (I, g.q_heads), (I, g.kv_heads), (I, g.head_dim)])
            self._gemv(mats[f"blk.{i}.attn_output"], self.attn_out, self.incr)
            self._elementwise("residual_add", m * g.hidden, [self.hidden, self.incr])
            self._rms_norm(self.hidden, vecs[f"blk.{i}.ffn_norm"], self.normed)
            gate_up = mats[f"blk.{i}.ffn_gate_up"]
            self._gemv(gate_up, self.normed, self.gate, 0, g.intermediate)
            self._gemv(gate_up, self.normed, self.up, g.intermediate, g.intermediate)
            self._elementwise("silu_mul", m * g.intermediate, [self.gate, self.up, self.act])
            self._gemv(mats[f"blk.{i}.ffn_down"], self.act, self.incr)
            self._elementwise("residual_add", m * g.hidden, [self.hidden, self.incr])
        self._rms_norm(self.hidden, vecs["output_norm"], self.normed)
        self._gemv(mats["output"], self.normed, self.logits)
        if m == 1:
            self.ops.launch("argmax", 1, 1024, [(P, self.logits.data_ptr()), (P, self.selected.data_ptr()), (I, g.vocabulary)])
        else:
            self.ops.launch("argmax_batch", m, 1024, [(P, self.logits.data_ptr()), (P, self.selected.data_ptr()), (I, g.vocabulary), (I, m)])
