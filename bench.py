#!/usr/bin/env python
"""Benchmark of the GGUF quantized-GEMV hot path on B200.

Workload (`config.workload` = "gemv_sweep"): the batched decode GEMV sweep of the benchmark
configuration list -- Q4_K / Q5_K / Q6_K weights of N x K in {4096x4096, 1024x4096, 12288x4096,
4096x12288}, members M in {1, 4, 16, 64}, bf16 N(0,1) activations, f32 outputs -- 48 GEMVs per step.
Synthetic seeded blocks stand in for model weights (no datasets or checkpoints are involved).

metric  = algorithmic bytes moved per second over a whole step: for each GEMV the encoded weight
          bytes + M*K*2 activation bytes + M*N*4 output bytes, counted once.
L2      = every (format, shape) has a ring of distinct weight copies larger than 2x the 126 MB L2
          and each launch uses the next copy, so no launch finds its weights in cache.
value   = device-resident inputs, CUDA-event timed on the launching stream.
e2e     = the same sweep through ribn_gemv_host_async + one ribn_synchronize per step: pinned host activations in, host outputs out,
          copies inside the timed region.
cases   = every (format, shape, members) timed on its own (bursts over its cold ring), with the fraction of the
          measured HBM peak; `sustained` repeats the step for about a second so that the clock sampler sees it.
parity  = largest error observed in this run, per kernel path, against the CPU checker (computed in the CPU-baseline leg).
--impl reference = the CPU restatement of the reference's host path (dequantise a row, sequential
          f32 dot; oracle/ribn_oracle.c) on all host threads, on a bounded sample (a row range) of every GEMV of the sweep.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FORMATS = [12, 13, 14]
SHAPES = [(4096, 4096), (1024, 4096), (12288, 4096), (4096, 12288)]  # (N, K)
MEMBERS = [1, 4, 16, 64]
L2_BYTES = 126 << 20
NOMINAL_HBM_GBS = 6650.0  # fallback when MEASURED_PEAKS.json is absent


def case_bytes(vt: int, n: int, k: int, m: int) -> int:
    from engine_b200 import synth

    return synth.encoded_bytes(vt, k, n) + m * k * 2 + m * n * 4


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return NOMINAL_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, smax, reasons = [], [], set()
        for parts in self.samples:
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        # under load: samples at or above 90 % of the highest clock seen are the ones taken while kernels ran
        busy = [v for v in sm if v >= 0.9 * max(sm)] if sm else []
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm), "sm_mhz_all_median": float(np.median(sm)) if sm else None}


def run_reference(args, rank: int, world: int) -> None:
    """The reference's host path for the same metric, on this box's cores."""
    if rank != 0:
        return
    import oracle
    from oracle import oracle_np
    from engine_b200 import synth

    threads = os.cpu_count() or 1
    # Every GEMV of the sweep, on a range of its rows sized so that one step is about a second of CPU work:
    # rows / members (at least 64), i.e. the same number of multiply-adds per case.
    cases = []
    step_bytes = 0
    for vt in FORMATS:
        for n, k in SHAPES:
            w = synth.random_weight(vt, k, max(64, n // 4), seed=vt * 100 + n // 1024 + k // 1024)
            for m in MEMBERS:
                rows = max(64, n // (4 * m))
                x = oracle_np.bf16_bits_to_f32(oracle_np.f32_to_bf16_bits(synth.random_activations(m, k, seed=m)))
                sub = w[:synth.encoded_bytes(vt, k, rows)]
                cases.append((vt, rows, k, m, sub, x))
                step_bytes += case_bytes(vt, rows, k, m)

    def step():
        for vt, rows, k, m, w, x in cases:
            oracle.gemv_f32(vt, w, k, rows, x, threads=threads)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    elapsed = time.perf_counter() - t0
    value = step_bytes * args.steps / elapsed / 1e9
    sample = (f"all {len(cases)} GEMVs of the sweep, each on its first max(64, N / (4 M)) rows; all {threads} host threads, rows split over threads; "
              "GB/s counts the algorithmic bytes of the rows computed")
    line = {
        "impl": "reference", "metric": "qgemv_algorithmic_GBps", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "gemv_sweep", "formats": ["Q4_K", "Q5_K", "Q6_K"], "shapes_NxK": SHAPES,
                   "members": MEMBERS, "activations": "bf16", "outputs": "f32"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# DRAM bytes moved per algorithmic byte by the batch kernel (weights unpacked into tensor memory), from an ncu capture
# of one launch (dram__bytes_read.sum + dram__bytes_write.sum = 28.56 MB over 28.44 MB of encoded weights, activations
# and outputs for Q4_K 12288x4096 with 16 member rows; profiles/qgemv_tmem_q4k_12288x4096_m16.md).  The kernel reads
# every weight byte once whatever the shape, so the ratio is applied to the sweep's mean call.
TC_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.004


def roofline(step_gbps, step_bytes, dominant, peak, peak_kind):
    source = f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback 6.65 TB/s"
    if dominant is None:   # a run restricted to calls of up to eight member rows
        return {"bound": "hbm", "achieved": step_gbps, "peak": peak, "unit": "GB/s", "frac": step_gbps / peak, "traffic": None,
                "peak_source": source, "kernel": "gemv_imma_kernel / gemv_mma_kernel (+ activation pre-pass from three rows on), all calls of the step",
                "bytes_per_step": step_bytes}
    achieved, us_per_call, bytes_per_call = dominant
    traffic = None if TC_TRAFFIC_PER_ALGORITHMIC_BYTE is None else TC_TRAFFIC_PER_ALGORITHMIC_BYTE * bytes_per_call
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
            "peak_source": source, "kernel": "qgemv_tmem_kernel + its activation pre-pass (calls of 16 and 64 member rows)",
            "us_per_call": us_per_call, "algorithmic_bytes_per_call": bytes_per_call,
            "whole_step": {"achieved": step_gbps, "frac": step_gbps / peak, "bytes_per_step": step_bytes}}


def attention_profile(spec: str) -> None:
    """One layer's decode attention (ribn_attention_decode: split-KV kernel + merge) on random f16 KV entries, five calls;
    prints the mean device time and the KV bytes per second.  For profiler captures of attention_split_kernel."""
    import torch

    import engine_b200
    from engine_b200 import _lib, decode

    fields = [int(v) for v in spec.split(":")]
    members, context = fields[0], fields[1]
    q_heads, kv_heads = (fields[2], fields[3]) if len(fields) >= 4 else (32, 8)
    stream = torch.cuda.Stream()
    ctx = engine_b200.RibnContext(0, stream=stream)
    ops = decode.CudaDenseOps(ctx)
    with torch.cuda.stream(stream):
        k_cache = torch.randn(members, kv_heads, context, 128, device=ctx.device).to(torch.float16)
        v_cache = torch.randn(members, kv_heads, context, 128, device=ctx.device).to(torch.float16)
        q = torch.randn(members, q_heads * 128, device=ctx.device)
        out = torch.empty(members, q_heads * 128, device=ctx.device)
        positions = torch.full((members,), context - 1, dtype=torch.int32, device=ctx.device)
        attention = _lib.Attention(members, q_heads, kv_heads, 128, 128, 1e6, 1e-6, None, None, positions.data_ptr(), k_cache.data_ptr(),
                                   v_cache.data_ptr(), context, context)
        ops.attention_decode(attention, q, out)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(5):
            ops.attention_decode(attention, q, out)
        b.record(stream)
    ctx.synchronize()
    us = a.elapsed_time(b) / 5 * 1e3
    kv_bytes = 2 * k_cache.numel() * 2
    print(json.dumps({"attention_profile": {"members": members, "context": context, "q_heads": q_heads, "kv_heads": kv_heads, "us_per_call": us,
                                            "kv_bytes": kv_bytes, "GBps": kv_bytes / us / 1e3, "frac_of_peak": kv_bytes / us / 1e3 / measured_peak()[0],
                                            "note": "back-to-back calls over the same cache: a cache of more than 126 MB is re-read from HBM"}}))


def prefill_leg(ctx, device, stream):
    """ribn_gemm on the two configuration-3 matrices, 512 and 2048 tokens, bf16 in and out: TFLOP/s and the fraction of
    the measured dense bf16 throughput (the call's f16 conversion pre-pass of the activations is inside the timed region)."""
    import torch

    import engine_b200
    from engine_b200 import synth

    try:
        peaks = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")))
        tensor_peak, source = float(peaks["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    except Exception:
        tensor_peak, source = 1590.0, "fallback 1.59 PFLOP/s"
    results = {"peak_tflops": tensor_peak, "peak_source": source}
    try:
        for vt, n, k in ((12, 12288, 4096), (14, 4096, 12288)):
            data = synth.random_weight_device(vt, k, n, seed=vt, device=device)
            weight = engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new("w", [k, n]), vt, data)
            for tokens in (512, 2048):
                x = torch.randn(tokens, k, device=device).to(torch.bfloat16)
                y = torch.empty(tokens, n, dtype=torch.bfloat16, device=device)
                with torch.cuda.stream(stream):
                    for _ in range(3):
                        engine_b200.gemm(ctx, weight, x, y)
                    torch.cuda.synchronize()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                    reps = 10
                    for _ in range(reps):
                        engine_b200.gemm(ctx, weight, x, y)
                    b.record(stream)
                torch.cuda.synchronize()
                ms = a.elapsed_time(b) / reps
                tflops = 2.0 * tokens * n * k / (ms * 1e-3) / 1e12
                results[f"{synth.TYPE_NAMES[vt]}_{n}x{k}_M{tokens}"] = {"ms": ms, "tflops": tflops, "frac_of_peak": tflops / tensor_peak}
    except Exception as exc:
        results["error"] = f"{type(exc).__name__}: {exc}"
    return results


def time_decode(decoder, generated, world, device, stream):
    """Replays the captured step `generated - 3` times after three warm-up replays; device time, max over the ranks."""
    import torch
    import torch.distributed as dist

    for _ in range(3):
        decoder.replay()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(generated - 3):
        decoder.replay()
    b.record(stream)
    torch.cuda.synchronize()
    ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def decode_entry(decoder, geometry, weights, members, context_tokens, generated, ms, peak, world, data):
    steps = generated - 3
    step_ms = ms / steps
    weight_bytes = weights.bytes_per_step()   # this rank's shard
    kv_bytes = geometry.layers * members * decoder.shapes["kv_heads"] * geometry.head_dim * 2 * 2 * (context_tokens + generated // 2)
    return {
        "tokens_per_s": members * steps / (ms * 1e-3), "ms_per_token_step": step_ms, "members": members,
        "context": context_tokens, "generated": generated, "layers": geometry.layers, "launches_per_step": decoder.launches_per_step,
        "weight_bytes_per_step_per_gpu": weight_bytes, "kv_bytes_per_step_per_gpu": kv_bytes,
        "hbm_GBps_per_gpu": (weight_bytes + kv_bytes) / (step_ms * 1e-3) / 1e9,
        "hbm_frac_of_peak": (weight_bytes + kv_bytes) / (step_ms * 1e-3) / 1e9 / peak,
        "data": data, "n_gpus": world,
    }


def tp_parity_leg(ctx, rank, world, link_factory):
    """Two layers of a reduced geometry, weights generated on the host and cut with engine_b200/sharding.py: the
    tensor-parallel decoder (exchanges over peer memory) against the unsharded decoder on rank 0, five steps."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from engine_b200 import decode

    geometry = decode.DenseGeometry(hidden=1024, layers=2, q_heads=16, kv_heads=8, head_dim=128, intermediate=2048, vocabulary=4096)
    members = 4
    tensors, vectors = decode.host_model(geometry, seed=3)
    out = {}
    for label, partial_dtype in (("f32_partials", torch.float32), ("bf16_partials", torch.bfloat16)):
        link = link_factory(members * geometry.hidden * 4)
        sharded = decode.CudaDenseDecode(ctx, geometry, decode.shard_host_model(ctx, geometry, tensors, vectors, world, rank), members, 32,
                                         process_group=dist.group.WORLD, world=world, rank=rank, peer_link=link, partial_dtype=partial_dtype)
        single = decode.CudaDenseDecode(ctx, geometry, decode.shard_host_model(ctx, geometry, tensors, vectors, 1, 0), members, 32) if rank == 0 else None
        tokens = torch.tensor([(17 * m + 3) % geometry.vocabulary for m in range(members)], dtype=torch.int32)
        worst, equal, compared = 0.0, 0, 0
        for decoder in (sharded, single):
            if decoder is not None:
                decoder.tokens.copy_(tokens)
        for _ in range(5):
            sharded.run_step()
            ctx.synchronize()
            slices = [torch.empty(members, decode.local_shapes(geometry, world, r)["vocab_end"] - decode.local_shapes(geometry, world, r)["vocab_begin"],
                                  device=ctx.device) for r in range(world)]
            dist.all_gather(slices, sharded.logits)
            following = torch.empty(members, dtype=torch.int32, device=ctx.device)
            if rank == 0:
                single.run_step()
                ctx.synchronize()
                full, got = single.logits.cpu().numpy(), torch.cat(slices, dim=1).cpu().numpy()
                worst = max(worst, float(np.max(np.abs(got - full)) / np.abs(full).max()))
                equal += int((sharded.next_tokens == single.next_tokens).sum().item())
                compared += members
                following.copy_(single.next_tokens)
            dist.broadcast(following, src=0)
            for decoder in (sharded, single):
                if decoder is not None:
                    decoder.tokens.copy_(following)
                    decoder.positions.add_(1)
            torch.cuda.synchronize()
        out[label] = {"logits_max_rel_err": worst, "tokens_equal": equal, "tokens_compared": compared}
        del sharded, single
        torch.cuda.synchronize()
        dist.barrier()
        link.close()
    out["geometry"] = "hidden 1024, 2 layers, 16 query / 8 key-value heads, intermediate 2048, vocabulary 4096; 4 sequences, 5 steps"
    return out


def decode_leg(args, ctx, device, rank, world, peak):
    """Decode tok/s.  One GPU: Qwen3-8B shape, Q4_K_M mix, 2048 tokens of context, 256 generated, batch 1 and 32, and
    the Qwen3-32B shape at batch 64 with 4096 tokens of context (the one-GPU point of the tensor-parallel curve).
    Several GPUs: the Qwen3-32B shape tensor parallel over all ranks, once with the exchanges over peer memory
    (ribn_tp_*: one kernel per exchange) and once with NCCL all-reduces, each also with the exchanges left out of the
    captured step to show their share of it.  Weights are random-init on the device; the one-GPU 8B contexts are real
    prompts run through the prefill path, the 32B contexts random KV entries (what a random prompt leaves behind)."""
    import torch
    import torch.distributed as dist

    from engine_b200 import decode, tp

    results = {}
    generated = 256
    try:
        if world == 1:
            geometry = decode.DenseGeometry.qwen3_8b(args.decode_layers or 36)
            weights = decode.random_weights(ctx, geometry, seed=1)
            for name, members, context_tokens in [("qwen3_8b_batch1", 1, 2048), ("qwen3_8b_batch32", 32, 2048)]:
                decoder = decode.CudaDenseDecode(ctx, geometry, weights, members, context_tokens + generated + 8)
                # the context is a real prompt: random tokens through the prefill path (tensor-core GEMM, shared-cache
                # attention), which leaves the KV entries and the first generated token of every sequence
                prompt_generator = torch.Generator(device="cpu")
                prompt_generator.manual_seed(members)
                prompts = torch.randint(0, geometry.vocabulary, (members, context_tokens), generator=prompt_generator, dtype=torch.int32)
                # warm-up with one full chunk: first launches load their kernels, set attributes and allocate the chunk's buffers
                decoder.prefill(prompts[0][:512], sequence=0)
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(ctx.stream)
                for m in range(members):
                    decoder.prefill(prompts[m], sequence=m)
                b.record(ctx.stream)
                ctx.synchronize()
                prefill_ms = a.elapsed_time(b)
                decoder.capture(advance=True)            # its eager step writes slot `context_tokens` again and advances nothing
                ms = time_decode(decoder, generated, 1, device, ctx.stream)
                results[name] = decode_entry(decoder, geometry, weights, members, context_tokens, generated, ms, peak, 1,
                                             "random-init weights (Q4_K_M mix), context prefilled from random prompt tokens, greedy decoding")
                results[name]["prefill"] = {"tokens_per_s": members * context_tokens / (prefill_ms * 1e-3), "ms": prefill_ms, "chunk": 512,
                                            "prompt_tokens": members * context_tokens}
                del decoder
                torch.cuda.empty_cache()
            results["reference_cuda_decode"] = reference_decode_leg(ctx, geometry, weights, device)
            del weights
            torch.cuda.empty_cache()
        # ---- the Qwen3-32B shape at batch 64 x 4096: every rank count runs it, so that the curve has its one-GPU point
        geometry = decode.DenseGeometry.qwen3_32b(args.decode_layers or 64)
        members, context_tokens, steps32 = 64, 4096, 67
        data32 = "random-init weights (Q4_K_M mix), random KV context, greedy decoding"
        group = dist.group.WORLD if world > 1 else None
        weights = decode.random_weights(ctx, geometry, seed=1, world=world, rank=rank)
        name = f"qwen3_32b_tp{world}_batch64"
        paths = [("peer_memory", True)] + ([("nccl", False)] if world > 1 else [])
        for label, fused in (paths if world > 1 else [("single", False)]):
            link = None
            if fused:
                link = tp.PeerLink(ctx, rank, world, members * geometry.hidden * 4)
                link.connect_group(group)
            decoder = decode.CudaDenseDecode(ctx, geometry, weights, members, context_tokens + generated + 8, process_group=group, world=world, rank=rank,
                                             peer_link=link, partial_dtype=torch.bfloat16)
            decoder.fill_context(context_tokens)
            decoder.capture(advance=True)
            decoder.fill_context(context_tokens)   # the eager step inside capture() advanced nothing but wrote one cache slot
            ms = time_decode(decoder, steps32, world, device, ctx.stream)
            entry = decode_entry(decoder, geometry, weights, members, context_tokens, steps32, ms, peak, world, data32)
            if world > 1:
                # the same step captured without its exchanges: what is left is GEMVs, attention and elementwise launches
                decoder.skip_exchange = True
                decoder.capture(advance=True)
                decoder.fill_context(context_tokens)
                bare = time_decode(decoder, steps32, world, device, ctx.stream)
                decoder.skip_exchange = False
                entry["ms_per_step_without_exchanges"] = bare / (steps32 - 3)
                entry["exchange_share_of_step"] = 1.0 - bare / ms
                entry["exchanges_per_step"] = 2 * geometry.layers
                entry["exchange"] = ("one kernel per exchange over peer memory (bf16 partials, residual folded in), token choice in one kernel"
                                     if fused else "ncclAllReduce of f32 partials + residual_add, token choice by all-gathers")
            results[name if label in ("peer_memory", "single") else f"{name}_{label}"] = entry
            del decoder
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            if link is not None:
                link.close()
            torch.cuda.empty_cache()
        if world > 1:
            results["tp_parity"] = tp_parity_leg(ctx, rank, world, lambda slot: _connected_link(ctx, rank, world, slot, group))
            # the one-GPU point, measured in this very run on every rank's own GPU (no communication): rank 0's figure
            del weights
            torch.cuda.empty_cache()
            solo_weights = decode.random_weights(ctx, geometry, seed=1)
            solo = decode.CudaDenseDecode(ctx, geometry, solo_weights, members, context_tokens + generated + 8)
            solo.fill_context(context_tokens)
            solo.capture(advance=True)
            solo.fill_context(context_tokens)
            ms = time_decode(solo, 35, 1, device, ctx.stream)
            one = decode_entry(solo, geometry, solo_weights, members, context_tokens, 35, ms, peak, 1, data32)
            results["qwen3_32b_tp1_batch64"] = one
            results["tp_efficiency"] = {"tokens_per_s": results[name]["tokens_per_s"], "tp1_tokens_per_s": one["tokens_per_s"],
                                        "speedup": results[name]["tokens_per_s"] / one["tokens_per_s"],
                                        "efficiency": results[name]["tokens_per_s"] / one["tokens_per_s"] / world, "n_gpus": world}
            del solo, solo_weights
            torch.cuda.empty_cache()
    except Exception as exc:   # the sweep line must still be printed
        import traceback

        results["error"] = f"{type(exc).__name__}: {exc}"
        results["traceback"] = traceback.format_exc()[-1500:]
    return results


def _connected_link(ctx, rank, world, slot_bytes, group):
    from engine_b200 import tp

    link = tp.PeerLink(ctx, rank, world, slot_bytes)
    link.connect_group(group)
    return link


def reference_decode_leg(ctx, geometry, weights, device):
    """The reference's own decode step on this GPU: its unmodified kernels in its launch order (oracle/ref_decode.py,
    which also lists the substitutions), one CUDA graph per step, Qwen3-8B shape, 2048 tokens of context, batch 1 and 8
    (its batch kernels serve at most eight members)."""
    import torch
    from oracle import ref_cuda, ref_decode

    if not ref_cuda.available() or not os.path.exists(ref_cuda.MODEL_OPS_CUBIN):
        return {"unavailable": "reference cubins not built here (oracle/build_ref.py needs the reference tree)"}
    out = {"substitutions": "strided_rms_norm for the q head norm (q_gate_norm expects a gated q projection); a constant gate buffer of +88 so that "
                            "attn_score_gqa's sigmoid gate is exactly 1; gate and up as two launches over one stored matrix; every timed step "
                            "runs at one position (the middle of the generated range) because token and position are kernel arguments",
           "source": "the reference's .cu sources compiled with nvcc for sm_100a, launched in the order of decode.rs:544-632, :929-1052, :678-696 "
                     "(batch: :1990-2140, :2868-3036) with the geometry of model_ops.rs / quantized.rs"}
    context_tokens, generated = 2048, 256
    try:
        for members in (1, 8):
            reference = ref_decode.ReferenceDenseDecode(geometry, weights, members, context_tokens + generated + 8, device)
            reference.fill_context(context_tokens + generated // 2)
            position = context_tokens + generated // 2
            with torch.cuda.stream(ctx.stream):
                reference.step(7, position)
            torch.cuda.synchronize()
            launches = reference.ops.launches
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=ctx.stream):
                reference.step(7, position)
            with torch.cuda.stream(ctx.stream):
                for _ in range(2):
                    graph.replay()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(ctx.stream)
                steps = 20
                for _ in range(steps):
                    graph.replay()
                b.record(ctx.stream)
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / steps
            out[f"batch{members}"] = {"tokens_per_s": members / (ms * 1e-3), "ms_per_step": ms, "launches_per_step": launches, "members": members,
                                      "context": context_tokens, "position": position, "cuda_graph": True}
            del reference, graph
            torch.cuda.empty_cache()
    except Exception as exc:
        out["error"] = f"{type(exc).__name__}: {exc}"
    return out


def time_reference_cuda(cases, rings, acts, outs, capture, stream, step_bytes, reps):
    """GB/s of the sweep when the reference project's own GEMV kernels serve it (cubins from oracle/build_ref.py)."""
    import torch
    from oracle import ref_cuda

    if not ref_cuda.available():
        return {"unavailable": "reference cubins not built here (oracle/build_ref.py needs the reference tree)"}
    try:
        kernels = ref_cuda.ReferenceKernels()
        x32 = {key: t.float() for key, t in acts.items()}
        cursor = {key: 0 for key in rings}

        def step():
            for vt, n, k, m in cases:
                ring = rings[(vt, n, k)]
                weight = ring[cursor[(vt, n, k)] % len(ring)]
                cursor[(vt, n, k)] += 1
                kernels.gemv(vt, weight.encoded_data(), x32[(k, m)], outs[(n, m)], k, n, m)

        with torch.cuda.stream(stream):
            step()
        torch.cuda.synchronize()
        graph = capture(step)
        with torch.cuda.stream(stream):
            replay = (lambda: graph.replay()) if graph is not None else step
            for _ in range(3):
                replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(reps):
                replay()
            b.record(stream)
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / reps
        launches = sum(ref_cuda.launches_for(m) for _, _, _, m in cases)
        # the same per member count: the reference serves 16 and 64 rows as two and eight launches that re-read the weights
        by_members = {}
        for members in sorted({m for _, _, _, m in cases}):
            subset = [c for c in cases if c[3] == members]

            def sub_step(subset=subset):
                for vt, n, k, m in subset:
                    ring = rings[(vt, n, k)]
                    weight = ring[cursor[(vt, n, k)] % len(ring)]
                    cursor[(vt, n, k)] += 1
                    kernels.gemv(vt, weight.encoded_data(), x32[(k, m)], outs[(n, m)], k, n, m)

            sub_graph = capture(sub_step)
            with torch.cuda.stream(stream):
                sub_replay = (lambda g=sub_graph: g.replay()) if sub_graph is not None else sub_step
                for _ in range(3):
                    sub_replay()
                torch.cuda.synchronize()
                c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                c0.record(stream)
                for _ in range(reps):
                    sub_replay()
                c1.record(stream)
            torch.cuda.synchronize()
            sub_ms = c0.elapsed_time(c1) / reps
            sub_bytes = sum(case_bytes(*c) for c in subset)
            by_members[str(members)] = {"GBps": round(sub_bytes / (sub_ms * 1e-3) / 1e9, 1), "us_per_call": round(sub_ms * 1e3 / len(subset), 2)}
        return {"value": step_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms, "launches_per_step": launches,
                "by_members": by_members,
                "kernels": "q{4,5,6}_k_gemv_warp (1 member row), q{4,5,6}_k_gemv_warp_batch (8 member rows per launch)",
                "activations": "f32 (the reference has no bf16 input)", "cuda_graph": graph is not None,
                "source": "the reference's .cu files compiled with nvcc for sm_100a, launched with the reference's geometry"}
    except Exception as exc:  # the comparison is optional; the benchmark line must still be printed
        return {"unavailable": f"{type(exc).__name__}: {exc}"}


def cpu_baseline_leg(ctx=None):
    """Bounded CPU sample for the main arm: the M=1 GEMV of every (format, shape), reference host
    arithmetic, once single-threaded (the reference's host path is single-threaded) and once on all cores.
    The CPU results double as the checker of this run's GPU results: `parity` holds the largest error observed
    per kernel path -- task metric |y - ref| / max(|ref|, sqrt(sum (w x)^2)) against the f64 product, the same
    against the reference's sequential f32 product, and the strict metric of oracle.max_rel_error_strict."""
    import oracle
    from engine_b200 import synth

    threads = os.cpu_count() or 1
    total = 0
    t1 = tn = 0.0
    parity = {}

    def observe(path, vt, n, k, w, x_seen, y, f32_reference=None, norms=None):
        ref = oracle.gemv_f64(vt, w, k, n, x_seen)
        scale = oracle.gemv_scale(vt, w, k, n, x_seen)
        entry = parity.setdefault(path, {"max_rel_err_vs_f64": 0.0, "max_rel_err_strict": 0.0, "cases": 0})
        entry["max_rel_err_vs_f64"] = max(entry["max_rel_err_vs_f64"], oracle.max_rel_error(y, ref, scale))
        if norms is None:
            norms = oracle.row_norms(vt, w, k, n)
        entry["max_rel_err_strict"] = max(entry["max_rel_err_strict"], oracle.max_rel_error_strict(y, ref, norms, x_seen))
        if f32_reference is not None:
            entry["max_rel_err_vs_reference_f32"] = max(entry.get("max_rel_err_vs_reference_f32", 0.0),
                                                        oracle.max_rel_error(y, f32_reference, scale))
        entry["cases"] += 1

    def gpu_gemv(vt, w, k, n, x, dtype, options=()):
        import torch

        import engine_b200

        for name, value in options:
            ctx.set_option(name, value)
        try:
            data = torch.from_numpy(np.ascontiguousarray(w)).to(ctx.device)
            weight = engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new("parity", [k, n]), vt, data)
            xd = torch.from_numpy(x).to(ctx.device).to(dtype).contiguous()
            yd = torch.full((x.shape[0], n), float("nan"), device=ctx.device)
            engine_b200.QwenGemvKernel.from_value_type(vt, ctx).execute_warp_batch(weight, xd, yd, x.shape[0])
            ctx.synchronize()
            return yd.cpu().numpy().astype(np.float64), xd.float().cpu().numpy()
        finally:
            for name, _ in options:
                ctx.set_option(name, {"mma_gemv": 1, "gemv_path": 0, "tmem_gemv": 1, "imma_gemv": 1}[name])

    for vt in FORMATS:
        for n, k in SHAPES:
            w = synth.random_weight(vt, k, n, seed=1)
            x = synth.random_activations(1, k, seed=1)
            total += case_bytes(vt, n, k, 1)
            t0 = time.perf_counter()
            oracle.gemv_f32(vt, w, k, n, x, threads=1)
            t1 += time.perf_counter() - t0
            t0 = time.perf_counter()
            y32 = oracle.gemv_f32(vt, w, k, n, x, threads=threads)
            tn += time.perf_counter() - t0
            if ctx is not None and not (n == 12288 or k == 12288):   # the two smaller shapes of every format
                import torch

                norms = oracle.row_norms(vt, w, k, n)
                y, seen = gpu_gemv(vt, w, k, n, x, torch.float32)
                observe("integer mma (1 row, f32 in)", vt, n, k, w, seen, y, f32_reference=y32, norms=norms)
                x4 = synth.random_activations(4, k, seed=4)
                y, seen = gpu_gemv(vt, w, k, n, x4, torch.bfloat16)
                observe("integer mma (4 rows, bf16 in)", vt, n, k, w, seen, y, norms=norms)
                y, seen = gpu_gemv(vt, w, k, n, x, torch.float32, options=(("imma_gemv", 0),))
                observe("f16 mma, two planes (1 row, f32 in; imma_gemv = 0)", vt, n, k, w, seen, y, norms=norms)
                x16 = synth.random_activations(16, k, seed=16)
                y, seen = gpu_gemv(vt, w, k, n, x16, torch.bfloat16)
                observe("tcgen05_weights_in_tmem (16 rows, bf16 in)", vt, n, k, w, seen, y, norms=norms)
                y, seen = gpu_gemv(vt, w, k, n, x16, torch.bfloat16, options=(("tmem_gemv", 0),))
                observe("tcgen05_f16_tile (16 rows, bf16 in; tmem_gemv = 0)", vt, n, k, w, seen, y, norms=norms)
                y, seen = gpu_gemv(vt, w, k, n, x, torch.float32, options=(("mma_gemv", 0),))
                observe("integer_dot (1 row, f32 in)", vt, n, k, w, seen, y, norms=norms)
                y, seen = gpu_gemv(vt, w, k, n, x, torch.float32, options=(("gemv_path", 1),))
                observe("f32_cuda_core (1 row, f32 in)", vt, n, k, w, seen, y, norms=norms)
    result = {"value": total / tn / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
              "sample": "M=1 GEMV of all 12 (format, shape) pairs, one pass; rows split over all host threads",
              "single_thread_value": total / t1 / 1e9}
    return result, (parity if parity else None)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=300)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--variant", type=int, default=0, help="GEMV tuning variant")
    parser.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                        help="library tuning option passed to ribn_set_option (measurement runs only)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-reference-cuda", action="store_true", help="skip timing the reference's own CUDA kernels")
    parser.add_argument("--no-prefill", action="store_true", help="skip the prefill GEMM measurements")
    parser.add_argument("--no-decode", action="store_true", help="skip the decode-loop measurements")
    parser.add_argument("--decode-layers", type=int, default=0, help="layer count of the decode models (0 = the full 36 / 64)")
    parser.add_argument("--no-graph", action="store_true", help="time plain launches instead of a captured CUDA graph")
    parser.add_argument("--cases", action="store_true", help="(kept for older command lines: the per-case table is now always produced)")
    parser.add_argument("--no-cases", action="store_true", help="skip the per-case table and the Q8_0 leg")
    parser.add_argument("--members", default="", help="comma-separated member counts replacing 1,4,16,64 (measurement runs, not the benchmark line)")
    parser.add_argument("--formats", default="", help="comma-separated formats (Q8_0,Q4_K,Q5_K,Q6_K) replacing the sweep's three")
    parser.add_argument("--attention", default="", metavar="MEMBERS:CONTEXT[:Q_HEADS:KV_HEADS]",
                        help="profiling run, not the benchmark: five calls of the decode attention of one layer (random KV), then exit")
    parser.add_argument("--only", default="", help="restrict the sweep to one case FORMAT:NxK:M (e.g. Q4_K:4096x4096:1); "
                        "a small run for profiler captures, not a benchmark line")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    global FORMATS, SHAPES, MEMBERS
    names = {"Q8_0": 8, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14}
    if args.members:
        MEMBERS = [int(v) for v in args.members.split(",")]
    if args.formats:
        FORMATS = [names[v] for v in args.formats.split(",")]
    if args.only:
        fmt, shape, m = args.only.split(":")
        FORMATS = [{"Q8_0": 8, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14}[fmt]]
        SHAPES = [tuple(int(v) for v in shape.split("x"))]
        MEMBERS = [int(m)]

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    import engine_b200
    from engine_b200 import synth

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    if args.attention:
        attention_profile(args.attention)
        return
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    # The library launches on its context's stream; a dedicated stream lets the step be captured
    # into a CUDA graph, so the timed region measures the GPU and not the Python launch loop.
    stream = torch.cuda.Stream(device=device)
    ctx = engine_b200.RibnContext(local_rank, stream=stream)
    ctx.set_option("gemv_variant", args.variant)
    for item in args.option:
        name, value = item.split("=")
        ctx.set_option(name, int(value))
    kernels = {vt: engine_b200.QwenGemvKernel.from_value_type(vt, ctx) for vt in FORMATS}
    store = engine_b200.CudaWeightStore(ctx)

    # Rings of distinct weight copies, each ring larger than 2x L2.
    rings = {}
    for vt in FORMATS:
        for n, k in SHAPES:
            nbytes = synth.encoded_bytes(vt, k, n)
            copies = (2 * L2_BYTES + nbytes - 1) // nbytes + 1
            ring = []
            for c in range(copies):
                name = f"{synth.TYPE_NAMES[vt]}.{n}x{k}.{c}"
                data = synth.random_weight_device(vt, k, n, seed=(rank * 1000003 + vt * 4099 + n + k + c) & 0x7FFFFFFF, device=device)
                ring.append(store.adopt(engine_b200.WeightTensorSpec.new(name, [k, n]), vt, data))
            rings[(vt, n, k)] = ring
    acts = {(k, m): torch.randn(m, k, device=device).to(torch.bfloat16) for _, k in SHAPES for m in MEMBERS}
    outs = {(n, m): torch.empty(m, n, dtype=torch.float32, device=device) for n, _ in SHAPES for m in MEMBERS}
    cursor = {key: 0 for key in rings}
    # One batch size at a time through every matrix, the way a decode step meets them.
    cases = [(vt, n, k, m) for m in MEMBERS for vt in FORMATS for n, k in SHAPES]
    step_bytes = sum(case_bytes(*c) for c in cases)
    # Launches per call: one for up to two member rows over at most 24 super-blocks (the kernel converts its activations
    # itself), otherwise an activation pre-pass and the GEMV kernel.
    launches_per_step = sum(1 if (m <= 2 and k // 256 <= 24) else 2 for _, _, k, m in cases)

    def launch(vt, n, k, m):
        ring = rings[(vt, n, k)]
        weight = ring[cursor[(vt, n, k)] % len(ring)]
        cursor[(vt, n, k)] += 1
        kernels[vt].execute_warp_batch(weight, acts[(k, m)], outs[(n, m)], m)

    def step():
        for c in cases:
            launch(*c)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def capture(fn):
        """Record fn's launches into a CUDA graph on the library's stream; None if capture is refused."""
        if args.no_graph:
            return None
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                fn()
            return graph
        except Exception as exc:  # fall back to plain launches, and say so in the output
            sys.stderr.write(f"CUDA graph capture failed ({exc}); timing eager launches\n")
            torch.cuda.synchronize()
            return None

    torch.cuda.synchronize()
    step()  # first launches set per-kernel attributes, which must not happen inside a capture
    torch.cuda.synchronize()
    step_graph = capture(step)

    def run_step():
        if step_graph is not None:
            with torch.cuda.stream(stream):
                step_graph.replay()
        else:
            step()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        run_step()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(ctx.stream)
    for _ in range(args.steps):
        run_step()
    stop.record(ctx.stream)
    barrier()
    ctx.synchronize()
    ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    value = step_bytes * world / (ms_per_step * 1e-3) / 1e9

    # ---- the same step repeated for about a second and a half, so that the clock sampler (20 ms period) sees it under load
    sustained = None
    if not args.only:
        reps = max(args.steps, int(1500.0 / max(ms_per_step, 1e-3)))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(ctx.stream)
        for _ in range(reps):
            run_step()
        b.record(ctx.stream)
        barrier()
        sustained_ms = a.elapsed_time(b)
        sustained = {"steps": reps, "seconds": sustained_ms * 1e-3, "value": step_bytes * world * reps / (sustained_ms * 1e-3) / 1e9, "unit": "GB/s"}

    # ---- end to end: host activations in, host outputs out, through ribn_gemv_host
    max_stage = max(m * k * 2 + 256 + m * n * 4 for _, n, k, m in cases)
    ctx.reserve_staging(max_stage + 4096)
    host_x = {key: t.cpu().pin_memory() for key, t in acts.items()}
    host_y = {key: torch.empty(t.shape, dtype=t.dtype).pin_memory() for key, t in outs.items()}

    def e2e_step():
        for vt, n, k, m in cases:
            ring = rings[(vt, n, k)]
            weight = ring[cursor[(vt, n, k)] % len(ring)]
            cursor[(vt, n, k)] += 1
            kernels[vt].inner.execute_host(weight, host_x[(k, m)], host_y[(n, m)], m, wait=False)
        ctx.synchronize()   # the step's results are in host memory from here on

    e2e_steps = max(3, min(args.steps, 10))
    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = step_bytes * world * e2e_steps / e2e_s / 1e9
    h2d = sum(m * k * 2 for _, _, k, m in cases)
    d2h = sum(m * n * 4 for _, n, _, m in cases)

    # ---- roofline of the dominant kernel: the tensor-core decode kernel (batches of 5..64 member rows) takes
    # most of the step; its calls are timed on their own (same graph replay, same cold weight rings).
    dominant = [c for c in cases if c[3] >= 9]
    dominant_roofline = None
    if dominant:
        def dominant_step():
            for c in dominant:
                launch(*c)

        graph = capture(dominant_step)
        replay = (lambda: graph.replay()) if graph is not None else dominant_step
        reps = max(3, min(args.steps, 50))
        with torch.cuda.stream(stream):
            for _ in range(3):
                replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(ctx.stream)
            for _ in range(reps):
                replay()
            b.record(ctx.stream)
        torch.cuda.synchronize()
        dominant_ms = a.elapsed_time(b) / reps
        dominant_bytes = sum(case_bytes(*c) for c in dominant)
        dominant_roofline = (dominant_bytes / (dominant_ms * 1e-3) / 1e9, dominant_ms * 1e3 / len(dominant), dominant_bytes / len(dominant))

    # ---- the reference's own CUDA kernels on this GPU, same sweep, same cold weight rings, same graph protocol.
    # They take f32 activations only and at most eight member rows per launch, so 16 and 64 member rows are
    # two and eight launches, the way the reference's prefill loop serves them.
    reference_cuda = None
    if rank == 0 and world == 1 and not args.no_reference_cuda:
        reference_cuda = time_reference_cuda(cases, rings, acts, outs, capture, stream, step_bytes, max(3, min(args.steps, 20)))

    # ---- prefill GEMM (BASELINE configuration 3): tensor-core TFLOP/s against the measured dense bf16 peak
    prefill_results = None
    if rank == 0 and world == 1 and not args.no_prefill and not args.only:
        prefill_results = prefill_leg(ctx, device, stream)

    # ---- decode loop: tokens per second of a random-init dense model (second half of the metric)
    decode_results = None
    if not args.no_decode and not args.only:
        decode_results = decode_leg(args, ctx, device, rank, world, peak=measured_peak()[0])

    breakdown = None
    peak_now = measured_peak()[0]
    if rank == 0 and not args.no_cases:
        breakdown = {}
        for c in cases:
            reps = 2 * len(rings[(c[0], c[1], c[2])])  # two trips round the ring of cold copies

            def burst(c=c, reps=reps):
                for _ in range(reps):
                    launch(*c)

            graph = capture(burst)
            replay = (lambda g=graph: g.replay()) if graph is not None else burst
            with torch.cuda.stream(stream):
                replay()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(ctx.stream)
                replay()
                b.record(ctx.stream)
            torch.cuda.synchronize()
            us = a.elapsed_time(b) / reps * 1e3
            vt, n, k, m = c
            gbps = case_bytes(*c) / us / 1e3
            breakdown[f"{synth.TYPE_NAMES[vt]}_{n}x{k}_M{m}"] = {"us": round(us, 2), "GBps": round(gbps, 1), "frac_of_peak": round(gbps / peak_now, 3)}

    # ---- Q8_0 (not part of the headline sweep): the same per-case protocol on two shapes
    q8_0 = None
    if rank == 0 and world == 1 and not args.no_cases and not args.only:
        q8_0 = {}
        try:
            kernel8 = engine_b200.QwenGemvKernel.from_value_type(8, ctx)
            for n, k in ((4096, 4096), (12288, 4096)):
                nbytes = synth.encoded_bytes(8, k, n)
                copies = (2 * L2_BYTES + nbytes - 1) // nbytes + 1
                ring8 = [store.adopt(engine_b200.WeightTensorSpec.new(f"Q8_0.{n}x{k}.{c}", [k, n]), 8,
                                     synth.random_weight_device(8, k, n, seed=8000 + c, device=device)) for c in range(copies)]
                for m in (1, 4, 16, 64):
                    x8 = torch.randn(m, k, device=device).to(torch.bfloat16)
                    y8 = torch.empty(m, n, dtype=torch.float32, device=device)

                    def burst8(ring8=ring8, x8=x8, y8=y8, m=m):
                        for _ in range(2):
                            for wgt in ring8:
                                kernel8.execute_warp_batch(wgt, x8, y8, m)

                    burst8()
                    torch.cuda.synchronize()
                    graph = capture(burst8)
                    replay = (lambda g=graph: g.replay()) if graph is not None else burst8
                    with torch.cuda.stream(stream):
                        replay()
                        torch.cuda.synchronize()
                        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        a.record(ctx.stream)
                        replay()
                        b.record(ctx.stream)
                    torch.cuda.synchronize()
                    us = a.elapsed_time(b) / (2 * len(ring8)) * 1e3
                    gbps = case_bytes(8, n, k, m) / us / 1e3
                    q8_0[f"Q8_0_{n}x{k}_M{m}"] = {"us": round(us, 2), "GBps": round(gbps, 1), "frac_of_peak": round(gbps / peak_now, 3)}
                del ring8
                torch.cuda.empty_cache()
        except Exception as exc:
            q8_0["error"] = f"{type(exc).__name__}: {exc}"

    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        peak, peak_kind = measured_peak()
        cpu_baseline = parity = None
        if not args.no_cpu_baseline and world == 1:
            cpu_baseline, parity = cpu_baseline_leg(ctx)
        line = {
            "metric": "qgemv_algorithmic_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "gemv_sweep" if not args.only else f"single case {args.only} (profiling run, not the benchmark)",
                       "formats": [synth.TYPE_NAMES[v] for v in FORMATS], "shapes_NxK": SHAPES,
                       "members": MEMBERS, "activations": "bf16", "outputs": "f32",
                       "l2": "ring of distinct weight copies > 2x L2 per (format, shape); inputs larger than L2",
                       "order": "one member count at a time through all 12 (format, shape) matrices, as a decode step meets them",
                       "parallelism": "replicas" if world > 1 else "single", "gemv_variant": args.variant, "options": args.option,
                       "cuda_graph": step_graph is not None},
            "roofline": roofline(value / world, step_bytes, dominant_roofline, peak, peak_kind),
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if sustained is not None:
            line["sustained"] = sustained
        if breakdown is not None:
            line["cases"] = breakdown
        if q8_0 is not None:
            line["q8_0"] = q8_0
        if parity is not None:
            line["parity"] = parity
        if reference_cuda is not None:
            line["reference_cuda"] = reference_cuda
        if decode_results is not None:
            line["decode"] = decode_results
            # the tensor-parallel curve, at the top level: tok/s of the Qwen3-32B shape on this many GPUs (strong scaling:
            # one model, one batch) and, from two GPUs on, its ratio to the one-GPU point measured in the same run
            key = f"qwen3_32b_tp{world}_batch64"
            if key in decode_results:
                line["tp"] = {"metric": "decode_tokens_per_s", "model": "Qwen3-32B shape, Q4_K_M mix, batch 64, 4096 context", "n_gpus": world,
                              "scaling": "strong", "tokens_per_s": decode_results[key]["tokens_per_s"],
                              "exchange_share_of_step": decode_results[key].get("exchange_share_of_step"),
                              "nccl_tokens_per_s": decode_results.get(key + "_nccl", {}).get("tokens_per_s"),
                              "tp1_tokens_per_s": decode_results.get("tp_efficiency", {}).get("tp1_tokens_per_s"),
                              "efficiency": decode_results.get("tp_efficiency", {}).get("efficiency"),
                              "parity": decode_results.get("tp_parity")}
        if prefill_results is not None:
            line["prefill"] = prefill_results
        if cpu_baseline is not None:
            line["cpu_baseline"] = cpu_baseline
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
