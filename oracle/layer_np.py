"""CPU restatement of the reference's host model of a dense-attention decoder layer.  TEST INFRASTRUCTURE ONLY.

Follows crates/nvidia/src/qwen_reference.rs of the reference project:
    rms_norm_raw                      :550-556
    host_full_attn_ar_step_traced     :368-470  (per-head Q/K RMSNorm, NEOX rope, cache append, GQA attention);
                                      the Qwen3.5 output gate of that function is not part of the dense layer
    host_ffn_step                     :523-539  down(silu(gate x) * (up x))
and the order of operations of CudaQwen35Decode::run_step / full_attention_layer
(crates/nvidia/src/decode.rs:544-632, :929-1052): embedding, per layer [norm, q/k/v, head norms, rope,
append, attention, o_proj, residual, norm, FFN, residual], final norm, output head, argmax.

Weights are dequantised once with the block decoders of the oracle; arithmetic is numpy float32 with
float64 dot products (the tolerance of the path absorbs the difference to the reference's sequential f32
sums).  K and V are rounded to f16 when they enter the cache, as kv_append_f16 does
(crates/nvidia/src/model_ops.rs:1256-1275).
"""
from __future__ import annotations

import numpy as np


def rms_norm_raw(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    x = np.asarray(x, np.float32)
    mean = np.mean(x.astype(np.float64) ** 2, axis=-1, keepdims=True)
    inverse = (1.0 / np.sqrt(mean + eps)).astype(np.float32)
    return (x * inverse * np.asarray(weight, np.float32)).astype(np.float32)


def rope_neox(values: np.ndarray, position: int, rot_dims: int, base: float) -> np.ndarray:
    """values [heads, head_dim]; pairs (p, p + rot_dims/2) of the first rot_dims dims, the rest passes through."""
    out = np.array(values, np.float32, copy=True)
    half = rot_dims // 2
    pair = np.arange(half, dtype=np.float32)
    theta = np.float32(position) * np.power(np.float32(base), -(np.float32(2.0) * pair) / np.float32(rot_dims)).astype(np.float32)
    sin, cos = np.sin(theta).astype(np.float32), np.cos(theta).astype(np.float32)
    x0, x1 = out[:, :half].copy(), out[:, half:rot_dims].copy()
    out[:, :half] = x0 * cos - x1 * sin
    out[:, half:rot_dims] = x0 * sin + x1 * cos
    return out


def to_f16(values: np.ndarray) -> np.ndarray:
    return np.asarray(values, np.float32).astype(np.float16).astype(np.float32)


def attention(q: np.ndarray, keys: np.ndarray, values: np.ndarray) -> np.ndarray:
    """q [q_heads, d]; keys, values [tokens, kv_heads, d] (already f16-rounded) -> [q_heads, d]."""
    q_heads, d = q.shape
    kv_heads = keys.shape[1]
    group = q_heads // kv_heads
    scale = 1.0 / np.sqrt(np.float32(d))
    out = np.zeros((q_heads, d), np.float32)
    for head in range(q_heads):
        kv = head // group
        scores = (keys[:, kv, :].astype(np.float64) @ q[head].astype(np.float64)) * scale
        weights = np.exp(scores - scores.max())
        weights /= weights.sum()
        out[head] = (weights @ values[:, kv, :].astype(np.float64)).astype(np.float32)
    return out


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    gate = np.asarray(gate, np.float32)
    return ((gate / (1.0 + np.exp(-gate))) * np.asarray(up, np.float32)).astype(np.float32)


def argmax(logits: np.ndarray) -> int:
    """First occurrence of the largest non-NaN value; 0 for a row of NaNs (model_ops.rs:201-258)."""
    logits = np.asarray(logits, np.float32)
    finite = ~np.isnan(logits)
    if not finite.any():
        return 0
    masked = np.where(finite, logits, -np.inf)
    return int(np.argmax(masked))


class DenseModel:
    """Dequantised weights of a dense GQA transformer and its decode step.

    `weights` maps names to float32 matrices [N, K] (rows = outputs) or vectors:
        token_embd [vocab, hidden]; output [vocab, hidden]; output_norm [hidden];
        blk.{i}.attn_norm, blk.{i}.ffn_norm [hidden]; blk.{i}.attn_q_norm, blk.{i}.attn_k_norm [head_dim];
        blk.{i}.attn_q [q_heads*d, hidden], attn_k / attn_v [kv_heads*d, hidden], attn_output [hidden, q_heads*d];
        blk.{i}.ffn_gate / ffn_up [inter, hidden], ffn_down [hidden, inter].
    """

    def __init__(self, weights: dict, layers: int, q_heads: int, kv_heads: int, head_dim: int, rope_base: float, eps: float,
                 rot_dims: int | None = None):
        self.w = weights
        # True models a prefill chunk on the tensor-core GEMM, whose activation operands are bf16: the inputs of the
        # seven projections are rounded to bf16 (the reference computes prefill in f32 like decode)
        self.bf16_activations = False
        self.layers, self.q_heads, self.kv_heads, self.head_dim = layers, q_heads, kv_heads, head_dim
        self.rope_base, self.eps = rope_base, eps
        self.rot_dims = head_dim if rot_dims is None else rot_dims
        self.keys = [np.zeros((0, kv_heads, head_dim), np.float32) for _ in range(layers)]
        self.values = [np.zeros((0, kv_heads, head_dim), np.float32) for _ in range(layers)]

    @staticmethod
    def _matvec(matrix: np.ndarray, x: np.ndarray) -> np.ndarray:
        return (matrix.astype(np.float64) @ x.astype(np.float64)).astype(np.float32)

    def _operand(self, x: np.ndarray) -> np.ndarray:
        if not self.bf16_activations:
            return x
        bits = np.asarray(x, np.float32).view(np.uint32).astype(np.uint64)
        rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16 << 16).astype(np.uint32)      # round to nearest even on the top 16 bits
        return rounded.view(np.float32).reshape(np.shape(x))

    def layer(self, i: int, hidden: np.ndarray, position: int) -> np.ndarray:
        w, d = self.w, self.head_dim
        x = self._operand(rms_norm_raw(hidden, w[f"blk.{i}.attn_norm"], self.eps))
        q = self._matvec(w[f"blk.{i}.attn_q"], x).reshape(self.q_heads, d)
        k = self._matvec(w[f"blk.{i}.attn_k"], x).reshape(self.kv_heads, d)
        v = self._matvec(w[f"blk.{i}.attn_v"], x).reshape(self.kv_heads, d)
        q = rope_neox(rms_norm_raw(q, w[f"blk.{i}.attn_q_norm"], self.eps), position, self.rot_dims, self.rope_base)
        k = rope_neox(rms_norm_raw(k, w[f"blk.{i}.attn_k_norm"], self.eps), position, self.rot_dims, self.rope_base)
        self.keys[i] = np.concatenate([self.keys[i], to_f16(k)[None]], axis=0)
        self.values[i] = np.concatenate([self.values[i], to_f16(v)[None]], axis=0)
        attended = self._operand(attention(q, self.keys[i], self.values[i]).reshape(-1))
        hidden = hidden + self._matvec(w[f"blk.{i}.attn_output"], attended)
        x = self._operand(rms_norm_raw(hidden, w[f"blk.{i}.ffn_norm"], self.eps))
        act = self._operand(silu_mul(self._matvec(w[f"blk.{i}.ffn_gate"], x), self._matvec(w[f"blk.{i}.ffn_up"], x)))
        return (hidden + self._matvec(w[f"blk.{i}.ffn_down"], act)).astype(np.float32)

    def step(self, token: int, position: int) -> np.ndarray:
        """Logits after feeding `token` at `position` (positions must come in order 0, 1, 2, ...)."""
        hidden = np.array(self.w["token_embd"][token], np.float32)
        for i in range(self.layers):
            hidden = self.layer(i, hidden, position)
        return self._matvec(self.w["output"], rms_norm_raw(hidden, self.w["output_norm"], self.eps))
