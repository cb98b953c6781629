"""Dequant-fused GEMV on the GPU, through the C ABI, against the CPU oracle.

Tolerance (stated by the task): max relative error 2e-3 with f32 accumulation against an f64 host
dot product of the exactly-dequantised weights.  "Relative" is |y - y_ref| / max(|y_ref|, s) with
s = sqrt(sum_k (w*x)^2) of that output (oracle.max_rel_error): outputs that cancel to almost zero
are measured against the size a dot product of that row has.  A bf16 output adds its own rounding,
one unit roundoff 2^-8.  The reference's own fixture tests use 1e-3 absolute
(crates/nvidia/tests/cuda_reference.rs:750-960) and are replayed with that bound.
"""
import numpy as np
import pytest
import torch

import engine_b200
import oracle
from engine_b200 import synth

pytestmark = pytest.mark.gpu

TOL = 2e-3
BF16_ROUNDOFF = 2.0 ** -8
KERNELS = {8: engine_b200.CudaQ8_0Gemv, 12: engine_b200.CudaQ4KGemv, 13: engine_b200.CudaQ5KGemv, 14: engine_b200.CudaQ6KGemv}
NAMES = {"q8_0": 8, "q4_k": 12, "q5_k": 13, "q6_k": 14}


@pytest.fixture(params=[0, 1, 2], ids=["auto", "f32-kernel", "integer-dot"], autouse=True)
def gemv_path(request, ctx):
    """Every test runs three times: with the default kernel choice (half2-unpack + mma.sync kernel for up to
    eight members per launch where it serves the shape), with the f32 CUDA-core kernel forced, and with the
    mma kernel switched off, which leaves 1..4 member rows to the integer-dot kernel."""
    ctx.set_option("gemv_path", 1 if request.param == 1 else 0)
    ctx.set_option("mma_gemv", 0 if request.param == 2 else 1)
    yield request.param
    ctx.set_option("gemv_path", 0)
    ctx.set_option("mma_gemv", 1)


def upload(ctx, vt, encoded, k, n, name="w"):
    store = engine_b200.CudaWeightStore(ctx)
    raw = np.ascontiguousarray(np.asarray(encoded).reshape(-1).view(np.uint8))
    store.materialize_quantized(engine_b200.WeightTensorSpec.new(name, [k, n]), vt, raw.size, raw)
    return store.quantized_tensor(name)


def run_gemv(ctx, vt, weight, x_host, n, x_dtype=torch.float32, y_dtype=torch.float32):
    """x_host float32 [members, K].  Returns (y as float64 numpy, x actually seen by the kernel as float32)."""
    members = x_host.shape[0]
    x = torch.from_numpy(x_host).to(ctx.device).to(x_dtype).contiguous()
    y = torch.full((members, n), float("nan"), dtype=y_dtype, device=ctx.device)
    kernel = KERNELS[vt].from_context(ctx)
    if members == 1:
        kernel.execute_warp(weight, x.reshape(-1), y.reshape(-1))
    else:
        kernel.execute_warp_batch(weight, x, y, members)
    ctx.synchronize()
    return y.float().cpu().numpy().astype(np.float64), x.float().cpu().numpy()


def check(vt, w, k, n, y, x_seen, y_bf16=False, strict=False):
    """Task metric |y - ref| / max(|ref|, sqrt(sum (w x)^2)) <= 2e-3 against the f64 product.  `strict` also asks for the
    stricter denominator max(|ref|, 1e-3 * ||w_row|| * ||x||) (oracle.max_rel_error_strict): it holds on every path that
    keeps f32-class arithmetic; the two tcgen05 batch kernels round weights to f16 and exceed it on cancelling outputs,
    which is why their tests do not pass strict=True."""
    ref = oracle.gemv_f64(vt, w, k, n, x_seen)
    scale = oracle.gemv_scale(vt, w, k, n, x_seen)
    err = oracle.max_rel_error(y, ref, scale)
    bound = TOL + (BF16_ROUNDOFF if y_bf16 else 0.0)
    assert np.all(np.isfinite(y)), "kernel left outputs unwritten"
    assert err <= bound, f"max rel err {err:.3e} > {bound:.3e}"
    if strict:
        tight = oracle.max_rel_error_strict(y, ref, oracle.row_norms(vt, w, k, n), x_seen)
        print(f"observed max rel err {err:.2e} (task metric), {tight:.2e} (strict metric)")
        assert tight <= bound, f"strict max rel err {tight:.3e} > {bound:.3e}"
    return err


# ---- the reference's own GEMV fixtures (cuda_reference.rs:312-425, :750-960), 1e-3 absolute
@pytest.mark.parametrize("name", list(NAMES))
def test_reference_fixture(ctx, golden, name):
    vt = NAMES[name]
    k, n = (int(v) for v in golden[f"gemv_{name}_shape"])
    weight = upload(ctx, vt, golden[f"gemv_{name}"], k, n, f"{name}.fixture")
    y, _ = run_gemv(ctx, vt, weight, golden[f"gemv_{name}_input"][None, :], n)
    assert np.max(np.abs(y[0] - golden[f"gemv_{name}_expect"])) < 1e-3


# ---- structured fixtures of tests/q*_q8_1.rs as 5 x 768 matrices, float activations
@pytest.mark.parametrize("name", list(NAMES))
def test_structured_fixture_matrix(ctx, golden, name):
    vt = NAMES[name]
    w = golden[f"struct_{name}"].reshape(-1)
    k, n = 768, 5
    x = np.array([[((i * 17 + 3) % 101 - 50) * 0.0137 for i in range(k)]], np.float32)
    weight = upload(ctx, vt, w, k, n)
    y, x_seen = run_gemv(ctx, vt, weight, x, n)
    check(vt, w, k, n, y, x_seen)


# ---- configuration 1: Q4_K 4096 x 4096, M = 1, f32 activations, seed 0
def test_config1_q4_k_4096(ctx):
    k = n = 4096
    w = synth.random_weight(12, k, n, seed=0)
    x = synth.random_activations(1, k, seed=0)
    weight = upload(ctx, 12, w, k, n)
    y, x_seen = run_gemv(ctx, 12, weight, x, n)
    check(12, w, k, n, y, x_seen)
    # and against the reference host path itself (sequential f32 dot), same bound
    y32 = oracle.gemv_f32(12, w, k, n, x_seen, threads=8)
    assert oracle.max_rel_error(y, y32, oracle.gemv_scale(12, w, k, n, x_seen)) <= TOL


# ---- configuration 2 sweep: formats x shapes x members, bf16 activations
SWEEP_SHAPES = [(4096, 4096), (1024, 4096), (12288, 4096), (4096, 12288)]  # (N, K)


@pytest.mark.parametrize("vt", [12, 13, 14])
@pytest.mark.parametrize("n,k", SWEEP_SHAPES)
def test_config2_sweep_bf16(ctx, vt, n, k):
    w = synth.random_weight(vt, k, n, seed=vt * 10 + SWEEP_SHAPES.index((n, k)))
    weight = upload(ctx, vt, w, k, n)
    for members in (1, 4, 16, 64):
        x = synth.random_activations(members, k, seed=members)
        y, x_seen = run_gemv(ctx, vt, weight, x, n, x_dtype=torch.bfloat16, y_dtype=torch.float32)
        check(vt, w, k, n, y, x_seen)
    x = synth.random_activations(4, k, seed=99)
    y, x_seen = run_gemv(ctx, vt, weight, x, n, x_dtype=torch.bfloat16, y_dtype=torch.bfloat16)
    check(vt, w, k, n, y, x_seen, y_bf16=True)


@pytest.mark.parametrize("n,k", [(4096, 4096), (1024, 4096)])
@pytest.mark.parametrize("members", [1, 8])
def test_q8_0_shapes(ctx, n, k, members):
    w = synth.random_weight(8, k, n, seed=8)
    weight = upload(ctx, 8, w, k, n)
    x = synth.random_activations(members, k, seed=members)
    y, x_seen = run_gemv(ctx, 8, weight, x, n)
    check(8, w, k, n, y, x_seen)


# ---- edges: tiny and ragged shapes, every member count the register tiles distinguish
@pytest.mark.parametrize("vt", [8, 12, 13, 14])
@pytest.mark.parametrize("n,k", [(1, 256), (2, 512), (3, 768), (5, 768), (7, 2304), (31, 256), (33, 5120), (300, 1024)])
def test_small_and_ragged_shapes(ctx, vt, n, k):
    w = synth.random_weight(vt, k, n, seed=n * 7 + k)
    weight = upload(ctx, vt, w, k, n)
    for members in (1, 2, 3, 5, 8, 9):
        x = synth.random_activations(members, k, seed=members + n)
        y, x_seen = run_gemv(ctx, vt, weight, x, n)
        check(vt, w, k, n, y, x_seen)


@pytest.mark.parametrize("k,n", [(32, 1), (64, 3), (96, 7), (288, 9), (4128, 5)])
def test_q8_0_input_sizes_that_are_not_multiples_of_256(ctx, k, n):
    w = synth.random_weight(8, k, n, seed=k + n)
    weight = upload(ctx, 8, w, k, n)
    for members in (1, 3):
        x = synth.random_activations(members, k, seed=members)
        y, x_seen = run_gemv(ctx, 8, weight, x, n)
        check(8, w, k, n, y, x_seen)


# ---- the mma kernel's two ways of getting its activations (converted inside the kernel / pre-pass image), every
# member count, f32 (two f16 planes) and bf16 (one) inputs; and members of one launch do not influence each other:
# a row's result is the same bits whatever the batch around it (the reference asserts the same of its batch
# kernels, crates/nvidia/tests/cuda_reference.rs:5243-5337)
@pytest.mark.parametrize("vt", [12, 13, 14])
@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("integer_kernel", [1, 0], ids=["imma", "f16-mma"])
def test_mma_kernel_modes_and_batch_identity(ctx, gemv_path, vt, x_dtype, integer_kernel):
    """The K-quants run on the integer tensor-core kernel by default and on the f16 kernel with imma_gemv = 0."""
    if gemv_path != 0:
        pytest.skip("the mma kernels are the default path only")
    ctx.set_option("imma_gemv", integer_kernel)
    k, n = 4096, 528
    w = synth.random_weight(vt, k, n, seed=vt)
    weight = upload(ctx, vt, w, k, n)
    x = synth.random_activations(8, k, seed=5)
    x[2, 256:512] = 0.0            # an all-zero K slice
    x[3, 1024:1280] *= 3e5         # slices of one row far apart in magnitude
    x[3, 1280:1536] *= 1e-6
    results = {}
    try:
        for image_members in (1, 9):
            ctx.set_option("mma_image_members", image_members)
            for members in range(1, 9):
                y, x_seen = run_gemv(ctx, vt, weight, x[:members], n, x_dtype=x_dtype)
                check(vt, w, k, n, y, x_seen, strict=True)
                results[(image_members, members)] = y
    finally:
        ctx.set_option("mma_image_members", 3)
        ctx.set_option("imma_gemv", 1)
    full = results[(1, 8)]
    for (image_members, members), y in results.items():
        assert np.array_equal(y, full[:members]), (image_members, members)


@pytest.mark.parametrize("vt", [12, 13, 14])
def test_batch_size_contract_beyond_the_reference_cap(ctx, gemv_path, vt):
    """The reference requires a row's result not to depend on its batch (tests/cuda_reference.rs:5243-5337 of the
    reference project, batches of 1..8, its cap).  Here that holds bit for bit for 1..8 rows of either dtype (the test
    above) and for f32 batches of any size (served eight rows per launch); bf16 batches of nine or more rows run on the
    f16-tile tensor-core kernel, whose rounding differs: those rows agree with their small-batch value within the 2e-3
    parity bound, not bit for bit."""
    if gemv_path != 0:
        pytest.skip("routing by batch size is the default path's")
    k, n = 4096, 528
    w = synth.random_weight(vt, k, n, seed=vt)
    weight = upload(ctx, vt, w, k, n)
    x = synth.random_activations(16, k, seed=6)
    one, _ = run_gemv(ctx, vt, weight, x[:1], n)
    wide, _ = run_gemv(ctx, vt, weight, x, n)
    nine, _ = run_gemv(ctx, vt, weight, x[:9], n)
    assert np.array_equal(wide[:1], one) and np.array_equal(wide[:9], nine)
    eight, x_seen = run_gemv(ctx, vt, weight, x[:8], n, x_dtype=torch.bfloat16)
    nine, _ = run_gemv(ctx, vt, weight, x[:9], n, x_dtype=torch.bfloat16)
    scale = oracle.gemv_scale(vt, w, k, n, x_seen)
    drift = oracle.max_rel_error(nine[:8], eight, scale)
    print(f"bf16 rows 0..7, batch of 9 against batch of 8: max rel difference {drift:.2e}")
    assert 0 < drift <= 2e-3


@pytest.mark.parametrize("nsb", [1, 2, 3, 4, 5, 13, 25, 50, 100])
def test_q6_k_batches_when_rows_do_not_start_on_16_byte_boundaries(ctx, gemv_path, nsb):
    """Q6_K rows are 210 * K/256 bytes: unless K/256 is a multiple of eight most rows start off the 16-byte boundary
    tiled TMA needs (the Qwen3-32B shape's ffn_down, K = 25600, and every input-column shard of it).  The batch kernel
    then reads the matrix as 2, 4 or 8 interleaved matrices; 300 rows leave a ragged last tile."""
    if gemv_path != 0:
        pytest.skip("the batch kernel is on the default path only")
    k, n = 256 * nsb, 300
    w = synth.random_weight(14, k, n, seed=nsb)
    weight = upload(ctx, 14, w, k, n)
    for members in (9, 64):
        x = synth.random_activations(members, k, seed=members + nsb)
        y, x_seen = run_gemv(ctx, 14, weight, x, n, x_dtype=torch.bfloat16)
        check(14, w, k, n, y, x_seen)


def test_q6_k_full_range_scales(ctx):
    """Q6_K scales over the whole int8 range: sc * (q - 32) reaches 4096, beyond the integers f16 holds exactly."""
    k, n = 2048, 64
    w = np.array(synth.random_weight(14, k, n, seed=77)).reshape(-1).view(np.uint8).copy()
    blocks = w.reshape(-1, 210)
    rng = np.random.default_rng(3)
    blocks[:, 192:208] = rng.integers(0, 256, size=(blocks.shape[0], 16), dtype=np.uint8)
    blocks[::7, 192:208] = 0x80    # -128 everywhere in some blocks
    weight = upload(ctx, 14, w, k, n)
    for members in (1, 8):
        x = synth.random_activations(members, k, seed=members)
        y, x_seen = run_gemv(ctx, 14, weight, x, n)
        check(14, w, k, n, y, x_seen)


def test_every_tuning_variant_agrees(ctx, gemv_path):
    if gemv_path != 1:
        pytest.skip("variants are tile geometries of the f32 kernel")
    k, n = 2048, 777
    try:
        for vt in (8, 12, 13, 14):
            w = synth.random_weight(vt, k, n, seed=vt)
            weight = upload(ctx, vt, w, k, n)
            for variant in (0, 1, 2, 3):
                ctx.set_option("gemv_variant", variant)
                for members in (1, 4):
                    x = synth.random_activations(members, k, seed=variant)
                    y, x_seen = run_gemv(ctx, vt, weight, x, n, x_dtype=torch.bfloat16)
                    check(vt, w, k, n, y, x_seen)
    finally:
        ctx.set_option("gemv_variant", 0)


def test_results_are_deterministic(ctx):
    k, n = 4096, 4096
    w = synth.random_weight(14, k, n, seed=3)
    weight = upload(ctx, 14, w, k, n)
    x = synth.random_activations(4, k, seed=1)
    first, _ = run_gemv(ctx, 14, weight, x, n)
    for _ in range(3):
        again, _ = run_gemv(ctx, 14, weight, x, n)
        assert np.array_equal(first, again)


# ---- batch members see the same weights: a batched call equals the per-member calls closely
# (the reference asserts bit identity between its batch and batch-1 kernels, cuda_reference.rs:5243-5337;
# here the single-row kernel applies group scales after the 4-term dot, so identity is to rounding)
def test_batched_matches_single(ctx):
    k, n = 1024, 64
    w = synth.random_weight(12, k, n, seed=4)
    weight = upload(ctx, 12, w, k, n)
    x = synth.random_activations(8, k, seed=2)
    batched, _ = run_gemv(ctx, 12, weight, x, n)
    scale = oracle.gemv_scale(12, w, k, n, x)
    for m in range(8):
        single, _ = run_gemv(ctx, 12, weight, x[m:m + 1], n)
        assert oracle.max_rel_error(single[0], batched[m], scale[m]) < 1e-5


# ---- host-buffer entry point
def test_host_buffers(ctx):
    k, n, members = 4096, 1024, 4
    w = synth.random_weight(13, k, n, seed=6)
    weight = upload(ctx, 13, w, k, n)
    x = synth.random_activations(members, k, seed=3)
    y = np.full((members, n), np.nan, np.float32)
    own = engine_b200.RibnContext(0)  # a context of its own: staging starts unreserved
    try:
        weight = upload(own, 13, w, k, n)
        kernel = engine_b200.CudaQ5KGemv.from_context(own)
        with pytest.raises(engine_b200.CudaQuantizedKernelError) as e:
            kernel.execute_host(weight, x, y, members)  # nothing reserved yet
        assert e.value.kind == "InvalidArgument"
        own.reserve_staging(1 << 20)
        kernel.execute_host(weight, x, y, members)
        check(13, w, k, n, y.astype(np.float64), x)
        # enqueue-only variant: eleven calls back to back (the four staging slots are reused), one synchronisation
        xs = [torch.from_numpy(synth.random_activations(members, k, seed=10 + i)).pin_memory() for i in range(11)]
        ys = [torch.full((members, n), float("nan")).pin_memory() for _ in range(11)]
        for xi, yi in zip(xs, ys):
            kernel.execute_host(weight, xi, yi, members, wait=False)
        own.synchronize()
        for xi, yi in zip(xs, ys):
            check(13, w, k, n, yi.numpy().astype(np.float64), xi.numpy())
    finally:
        own.close()


# ---- rejections happen before the launch and leave the output untouched (tests/q4_q8_1.rs:298-349)
def test_rejections_leave_output_untouched(ctx):
    k, n = 512, 2
    w = synth.random_weight(12, k, n, seed=9)
    weight = upload(ctx, 12, w, k, n)
    kernel = engine_b200.CudaQ4KGemv.from_context(ctx)
    x = torch.zeros(k, device=ctx.device)
    y = torch.full((n,), 7.0, device=ctx.device)

    def kind(call):
        with pytest.raises(engine_b200.CudaQuantizedKernelError) as e:
            call()
        return e.value

    e = kind(lambda: engine_b200.CudaQ5KGemv.from_context(ctx).execute_warp(weight, x, y))
    assert e.kind == "UnsupportedValueType" and (e.expected, e.actual) == (13, 12)
    e = kind(lambda: kernel.execute_warp(weight, x[:-1], y))
    assert e.kind == "InputLength" and (e.expected, e.actual) == (512, 511)
    e = kind(lambda: kernel.execute_warp(weight, x, torch.full((3,), 7.0, device=ctx.device)))
    assert e.kind == "OutputLength" and (e.expected, e.actual) == (2, 3)
    e = kind(lambda: kernel.execute_warp_batch(weight, x, y, 0))
    assert e.kind == "InputLength" and (e.expected, e.actual) == (1, 0)
    e = kind(lambda: kernel.execute_warp_batch(weight, x, y, 65))
    assert e.kind == "InvalidWeight"
    e = kind(lambda: kernel.execute_warp_batch(weight, x, y, 2))
    assert e.kind == "InputLength" and (e.expected, e.actual) == (1024, 512)
    wrong_rank = engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new("r", [512, 2, 1]), 12, weight.encoded_data())
    assert kind(lambda: kernel.execute_warp(wrong_rank, x, y)).kind == "InvalidWeight"
    short = engine_b200.CudaQuantizedWeight(engine_b200.WeightTensorSpec.new("s", [512, 2]), 12, weight.encoded_data()[:-1])
    assert kind(lambda: kernel.execute_warp(short, x, y)).kind == "InvalidWeight"
    host_x = torch.zeros(k)
    assert kind(lambda: kernel.execute_warp(weight, host_x, y)).kind == "ContextMismatch"
    assert kind(lambda: kernel.execute_warp(weight, torch.zeros(k + 1, device=ctx.device)[1:], y)).kind == "InvalidArgument"
    ctx.synchronize()
    assert torch.all(y == 7.0)


def test_qwen_gemv_kernel_dispatches_on_value_type(ctx):
    k, n = 512, 9
    for vt in (8, 12, 13, 14):
        w = synth.random_weight(vt, k, n, seed=vt)
        weight = upload(ctx, vt, w, k, n)
        kernel = engine_b200.QwenGemvKernel.from_value_type(vt, ctx)
        assert kernel.value_type() == vt
        x = torch.from_numpy(synth.random_activations(1, k, seed=1)).to(ctx.device)
        y = torch.empty(n, device=ctx.device)
        kernel.execute_warp(weight, x.reshape(-1), y)
        ctx.synchronize()
        check(vt, w, k, n, y.cpu().numpy()[None, :].astype(np.float64), x.cpu().numpy())
    with pytest.raises(engine_b200.CudaQuantizedKernelError):
        engine_b200.QwenGemvKernel.from_value_type(11, ctx)


# ---- fused RMSNorm -> GEMV: same result contract as the two calls
@pytest.mark.parametrize("vt", [8, 12, 13, 14])
@pytest.mark.parametrize("members,x_dtype", [(1, torch.float32), (2, torch.bfloat16), (4, torch.float32), (7, torch.float32),
                                             (8, torch.bfloat16), (33, torch.bfloat16)])
def test_fused_rms_norm_gemv(ctx, vt, members, x_dtype):
    k, n = 4096, 513
    w = synth.random_weight(vt, k, n, seed=vt + members)
    weight = upload(ctx, vt, w, k, n)
    rng = np.random.default_rng(members)
    x = torch.from_numpy((rng.standard_normal((members, k)) * 2.5).astype(np.float32)).to(ctx.device).to(x_dtype)
    gain_host = (1.0 + 0.02 * rng.standard_normal(k)).astype(np.float32)
    gain = torch.from_numpy(gain_host).to(ctx.device)
    y = torch.full((members, n), float("nan"), device=ctx.device)
    KERNELS[vt].from_context(ctx).execute_rms_norm(weight, x, gain, 1e-6, y, members)
    ctx.synchronize()
    normed = oracle.rms_norm(x.float().cpu().numpy(), gain_host, 1e-6)
    check(vt, w, k, n, y.cpu().numpy().astype(np.float64), normed)


# ---- f32 batches reach the tensor-core kernel only on request (its operands are f16)
@pytest.mark.parametrize("vt", [8, 12, 13, 14])
@pytest.mark.parametrize("fused", [False, True])
def test_f32_batches_on_the_tensor_core_kernel(ctx, vt, fused):
    k, n, members = 2048, 300, 9
    w = synth.random_weight(vt, k, n, seed=vt)
    weight = upload(ctx, vt, w, k, n)
    rng = np.random.default_rng(vt)
    x_host = (rng.standard_normal((members, k)) * np.float32(3.0)).astype(np.float32)
    x_host[3] *= np.float32(1e-6)     # rows far apart in magnitude: every row has its own power-of-two factor
    x_host[5] *= np.float32(3e5)
    gain_host = (1.0 + 0.02 * rng.standard_normal(k)).astype(np.float32)
    x = torch.from_numpy(x_host).to(ctx.device)
    y = torch.full((members, n), float("nan"), device=ctx.device)
    ctx.set_option("tc_f32_activations", 1)
    try:
        if fused:
            KERNELS[vt].from_context(ctx).execute_rms_norm(weight, x, torch.from_numpy(gain_host).to(ctx.device), 1e-6, y, members)
        else:
            KERNELS[vt].from_context(ctx).execute_warp_batch(weight, x, y, members)
        ctx.synchronize()
    finally:
        ctx.set_option("tc_f32_activations", 0)
    seen = oracle.rms_norm(x_host, gain_host, 1e-6) if fused else x_host
    check(vt, w, k, n, y.cpu().numpy().astype(np.float64), seen)


# ---- calls of 1..4 rows can pack their activations inside the integer-dot kernel (option dp4a_prepass = 0)
@pytest.mark.parametrize("vt", [8, 12, 13, 14])
@pytest.mark.parametrize("members,x_dtype,fused", [(1, torch.float32, False), (3, torch.bfloat16, False), (4, torch.float32, True), (2, torch.bfloat16, True)])
def test_activations_packed_inside_the_kernel(ctx, vt, members, x_dtype, fused):
    k, n = 2304, 333
    w = synth.random_weight(vt, k, n, seed=vt + members)
    weight = upload(ctx, vt, w, k, n)
    rng = np.random.default_rng(members)
    x = torch.from_numpy((rng.standard_normal((members, k)) * 2.0).astype(np.float32)).to(ctx.device).to(x_dtype)
    gain_host = (1.0 + 0.02 * rng.standard_normal(k)).astype(np.float32)
    y = torch.full((members, n), float("nan"), device=ctx.device)
    ctx.set_option("dp4a_prepass", 0)
    ctx.set_option("mma_gemv", 0)
    try:
        if fused:
            KERNELS[vt].from_context(ctx).execute_rms_norm(weight, x, torch.from_numpy(gain_host).to(ctx.device), 1e-6, y, members)
        else:
            KERNELS[vt].from_context(ctx).execute_warp_batch(weight, x, y, members)
        ctx.synchronize()
    finally:
        ctx.set_option("dp4a_prepass", 1)
        ctx.set_option("mma_gemv", 1)
    seen = x.float().cpu().numpy()
    check(vt, w, k, n, y.cpu().numpy().astype(np.float64), oracle.rms_norm(seen, gain_host, 1e-6) if fused else seen)


def test_fused_rejections(ctx):
    k, n = 512, 4
    w = synth.random_weight(12, k, n, seed=1)
    weight = upload(ctx, 12, w, k, n)
    x = torch.zeros(k, device=ctx.device)
    y = torch.full((n,), 7.0, device=ctx.device)
    with pytest.raises(engine_b200.CudaQuantizedKernelError) as e:
        engine_b200.CudaQ4KGemv.from_context(ctx).execute_rms_norm(weight, x, torch.ones(k - 1, device=ctx.device), 1e-6, y, 1)
    assert e.value.kind == "InputLength"
    ctx.synchronize()
    assert torch.all(y == 7.0)


def test_non_finite_activations_reach_the_output(ctx):
    k, n = 512, 8
    w = synth.random_weight(12, k, n, seed=2)
    weight = upload(ctx, 12, w, k, n)
    x = synth.random_activations(1, k, seed=1)
    x[0, 100] = np.inf
    xd = torch.from_numpy(x).to(ctx.device)
    yd = torch.zeros(n, device=ctx.device)
    engine_b200.CudaQ4KGemv.from_context(ctx).execute_warp(weight, xd.reshape(-1), yd)
    ctx.synchronize()
    assert not torch.isfinite(yd).any()
