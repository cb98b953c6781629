// C ABI of the library: context, validation, error reporting, dispatch.
//
// Host-side twin of the reference's kernel wrapper layer
// (crates/nvidia/src/quantized.rs:143-488, :1755-1804 and
// crates/nvidia/src/model_ops.rs:1714-1824 of the reference project): every
// check that layer performs before a launch is performed here, in the same
// order, with the same error classes and message wording.
#include <cuda_runtime.h>

#include <cinttypes>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <limits>
#include <new>
#include <string>

#include "../../include/ribn_b200.h"
#include "internal.h"

struct ribn_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    int* device_status = nullptr;   // one word, written by kernels whose bounded waits ran out
    void* staging = nullptr;        // device scratch for the host-buffer entry points: kStagingSlots slots of staging_bytes
    uint64_t staging_bytes = 0;
    // Host-buffer calls overlap: uploads run on `in_stream`, downloads on `out_stream`, the GEMVs on the context's stream,
    // tied together per staging slot by events, so that the copies of one call hide behind the compute of its neighbours.
    cudaStream_t in_stream = nullptr, out_stream = nullptr;
    cudaEvent_t in_done[4] = {}, compute_done[4] = {}, out_done[4] = {};
    bool slot_used[4] = {};
    uint64_t host_calls = 0;
    int variant = 0;                // GEMV tuning variant (ribn_set_option)
    int gemv_path = 0;              // 0 = choose per shape, 1 = f32 CUDA-core kernel only, 2 = integer-dot kernel only
    void* workspace = nullptr;      // device scratch owned by the context (packed activations, split-K partial tiles)
    uint64_t workspace_bytes = 0;
    unsigned int* tickets = nullptr;  // split-K tile counters of the tensor-core GEMM, zero between launches
    int tc_ksplit = 0;              // 0 = choose the split-K factor per shape
    int tc_split_operands = 0;      // 1 = bf16 batches <= 64 use the prefill GEMM kernel instead of the f16 decode kernel
    int tc_trace = 0;               // builds with -DRIBN_TRACE: 1 = kernels record pipeline clock stamps in the workspace tail
    int tc_row_copies = 0;          // 1 = force the per-row bulk-copy variant of the tensor-core kernel
    int dp4a_prepass = 1;           // 0 = calls of 1..4 rows pack their activations inside the GEMV kernel (measured slower: see the header)
    int tc_f32_activations = 0;     // 1 = f32 activation batches may use the tensor-core kernel too (they are rounded to f16)
    int64_t tc_four_row_bytes = 8 << 20;   // batches of four rows use the tensor-core kernel too when the weights are at least this large
    int tc_min_members = 9;         // batches of at least this many rows go to the tcgen05 decode kernel
    int tmem_gemv = 1;              // 1 = Q4_K / Q5_K batches of nine or more rows use the kernel that unpacks the weights into tensor memory
    int mma_gemv = 1;               // 1 = batches of up to eight rows use the half2-unpack + mma.sync kernel where it serves the shape
    int imma_gemv = 1;              // 1 = up to imma_max_members rows of a K-quant use the integer tensor-core kernel (gemv_imma.cu)
    int imma_max_members = 8;
    int mma_image_members = 3;      // launches of at least this many rows convert their activations in a pre-pass, fewer inside the kernel
    int mma_stages = 0;             // ring depth of that kernel, 0 = as many stages as fit
    int mma_resident = 0;           // CTAs per SM its shared-memory plan allows for, 0 = up to three
    int mma_ctas = 0;               // CTAs per SM its grid is sized for, 0 = min(resident, 2)
    std::string message;
    uint64_t expected = 0, actual = 0;
};

namespace ribn {
void context_internals(const ribn_ctx* ctx, int* device, void** stream, int* sm_count, int** status) {
    *device = ctx->device;
    *stream = ctx->stream;
    *sm_count = ctx->sm_count;
    *status = ctx->device_status;
}
}  // namespace ribn

namespace {

using ribn::GemvArgs;

constexpr int kTicketCount = 16384;
constexpr int kStagingSlots = 4;
constexpr uint64_t kTraceBytes = 64 << 10;

struct Layout {
    uint64_t elements, bytes;
};

// crates/gguf/src/lib.rs:1051-1083
bool tensor_layout(uint32_t t, Layout* out) {
    switch (t) {
        case 0: case 26: *out = {1, 4}; return true;
        case 1: case 25: case 30: *out = {1, 2}; return true;
        case 2: case 20: *out = {32, 18}; return true;
        case 3: *out = {32, 20}; return true;
        case 6: *out = {32, 22}; return true;
        case 7: *out = {32, 24}; return true;
        case 8: *out = {32, 34}; return true;
        case 9: *out = {32, 36}; return true;
        case 10: *out = {256, 84}; return true;
        case 11: case 21: *out = {256, 110}; return true;
        case 12: *out = {256, 144}; return true;
        case 13: *out = {256, 176}; return true;
        case 14: *out = {256, 210}; return true;
        case 15: *out = {256, 292}; return true;
        case 16: case 35: *out = {256, 66}; return true;
        case 17: *out = {256, 74}; return true;
        case 18: *out = {256, 98}; return true;
        case 19: *out = {256, 50}; return true;
        case 22: *out = {256, 82}; return true;
        case 23: *out = {256, 136}; return true;
        case 24: *out = {1, 1}; return true;
        case 27: case 28: *out = {1, 8}; return true;
        case 29: *out = {256, 56}; return true;
        case 34: *out = {256, 54}; return true;
        case 39: *out = {32, 17}; return true;
        case 40: *out = {64, 36}; return true;
        case 41: *out = {128, 18}; return true;
        case 42: *out = {64, 18}; return true;
        default: return false;
    }
}

const char* type_label(uint32_t t) {
    switch (t) {
        case RIBN_TYPE_Q8_0: return "Q8_0";
        case RIBN_TYPE_Q4_K: return "Q4_K";
        case RIBN_TYPE_Q5_K: return "Q5_K";
        case RIBN_TYPE_Q6_K: return "Q6_K";
        default: return "?";
    }
}

bool supported_type(uint32_t t) {
    return t == RIBN_TYPE_Q8_0 || t == RIBN_TYPE_Q4_K || t == RIBN_TYPE_Q5_K || t == RIBN_TYPE_Q6_K;
}

// A failed check: status + message + the two numbers some classes carry.
struct Failure {
    int status = RIBN_OK;
    std::string message;
    uint64_t expected = 0, actual = 0;
};

Failure fail(int status, std::string message, uint64_t expected = 0, uint64_t actual = 0) {
    Failure f;
    f.status = status;
    f.message = std::move(message);
    f.expected = expected;
    f.actual = actual;
    return f;
}

std::string fmt(const char* pattern, ...) {
    char buffer[256];
    va_list args;
    va_start(args, pattern);
    vsnprintf(buffer, sizeof buffer, pattern, args);
    va_end(args);
    return buffer;
}

bool mul_overflows(uint64_t a, uint64_t b, uint64_t* out) { return __builtin_mul_overflow(a, b, out); }

// validate_quantized_geometry, crates/nvidia/src/quantized.rs:1755-1804, check for check.
Failure validate_geometry(const ribn_qweight* w, uint32_t expected_type, uint64_t* k_out, uint64_t* n_out) {
    if (w == nullptr) return fail(RIBN_E_INVALID_ARGUMENT, "null weight descriptor");
    uint32_t type = expected_type;
    if (type == 0) {
        // QwenGemvKernel::from_value_type (staging.rs:108-140): the kernel follows the weight's type.
        type = w->value_type;
        if (!supported_type(type))
            return fail(RIBN_E_INVALID_WEIGHT, fmt("no quantized GEMV kernel for GGML value type %u", type));
    } else if (!supported_type(type)) {
        return fail(RIBN_E_INVALID_WEIGHT, fmt("no quantized GEMV kernel for GGML value type %u", type));
    }
    if (w->value_type != type)
        return fail(RIBN_E_UNSUPPORTED_TYPE,
                    fmt("quantized GEMV requires GGML value type %u, got %u", type, w->value_type), type, w->value_type);
    if (w->rank != 2) return fail(RIBN_E_INVALID_WEIGHT, fmt("invalid quantized weight: expected rank-2 tensor, got rank %u", w->rank));
    Layout layout{};
    tensor_layout(type, &layout);
    const uint64_t k = w->dimensions[0], n = w->dimensions[1];
    if (k == 0 || n == 0 || k % layout.elements != 0)
        return fail(RIBN_E_INVALID_WEIGHT,
                    fmt("invalid quantized weight: %s shape is %" PRIu64 "x%" PRIu64
                        "; input size must be a positive multiple of %" PRIu64,
                        type_label(type), k, n, layout.elements));
    uint64_t blocks = 0, expected_bytes = 0;
    if (mul_overflows(k / layout.elements, n, &blocks) || mul_overflows(blocks, layout.bytes, &expected_bytes))
        return fail(RIBN_E_SHAPE_OVERFLOW, "quantized GEMV shape does not fit CUDA launch arguments");
    if (w->encoded_bytes != expected_bytes)
        return fail(RIBN_E_INVALID_WEIGHT,
                    fmt("invalid quantized weight: encoded length is %" PRIu64 ", expected %" PRIu64, w->encoded_bytes,
                        expected_bytes));
    // The reference's kernels index with 32-bit ints, so it refuses blocks > i32::MAX / block_bytes
    // and dims > i32::MAX.  These kernels index bytes with 64 bits; only the dimension limit is kept.
    const uint64_t i32_max = static_cast<uint64_t>(std::numeric_limits<int32_t>::max());
    if (k > i32_max || n > i32_max)
        return fail(RIBN_E_SHAPE_OVERFLOW, "quantized GEMV shape does not fit CUDA launch arguments");
    if (k_out) *k_out = k;
    if (n_out) *n_out = n;
    return Failure{};
}

int record(ribn_ctx* ctx, const Failure& f) {
    if (ctx != nullptr) {
        ctx->message = f.message;
        ctx->expected = f.expected;
        ctx->actual = f.actual;
    }
    return f.status;
}

int record_cuda(ribn_ctx* ctx, cudaError_t e, const char* what) {
    return record(ctx, fail(RIBN_E_DRIVER, fmt("CUDA driver error: %s: %s", what, cudaGetErrorString(e))));
}

bool valid_dtype(int d) { return d == RIBN_F32 || d == RIBN_BF16; }
uint64_t dtype_bytes(int d) { return d == RIBN_BF16 ? 2 : 4; }

// ContextMismatch (quantized.rs:326-331): every buffer must be device memory of the context's GPU.
Failure check_device_pointer(const ribn_ctx* ctx, const void* p, const char* what) {
    if (p == nullptr) return fail(RIBN_E_INVALID_ARGUMENT, fmt("%s pointer is null", what));
    if (reinterpret_cast<uintptr_t>(p) % 16 != 0)
        return fail(RIBN_E_INVALID_ARGUMENT, fmt("%s pointer is not 16-byte aligned", what));
    cudaPointerAttributes attr{};
    const cudaError_t e = cudaPointerGetAttributes(&attr, p);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(RIBN_E_CONTEXT_MISMATCH, "quantized GEMV buffers and stream belong to different CUDA contexts");
    }
    if ((attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged) || attr.device != ctx->device)
        return fail(RIBN_E_CONTEXT_MISMATCH, "quantized GEMV buffers and stream belong to different CUDA contexts");
    return Failure{};
}

struct DeviceGuard {
    int previous = -1;
    explicit DeviceGuard(int device) {
        cudaGetDevice(&previous);
        if (previous != device) cudaSetDevice(device);
    }
    ~DeviceGuard() {
        int now = -1;
        cudaGetDevice(&now);
        if (previous >= 0 && now != previous) cudaSetDevice(previous);
    }
};

// Everything ribn_gemv checks before launching, shared with the host-buffer variant.
Failure validate_gemv(const ribn_qweight* w, uint32_t expected_type, int x_dtype, uint64_t x_len, int y_dtype,
                      uint64_t y_len, uint32_t members, uint64_t* k, uint64_t* n) {
    if (!valid_dtype(x_dtype) || !valid_dtype(y_dtype)) return fail(RIBN_E_INVALID_ARGUMENT, "unknown activation dtype");
    // quantized.rs:458-469: members == 0 and members over the cap are refused before geometry.
    if (members == 0)
        return fail(RIBN_E_INPUT_LENGTH, "quantized GEMV input has 0 values, expected 1", 1, 0);
    if (members > RIBN_MAX_GEMV_MEMBERS)
        return fail(RIBN_E_INVALID_WEIGHT,
                    fmt("invalid quantized weight: batch variant supports at most %u members", RIBN_MAX_GEMV_MEMBERS));
    Failure f = validate_geometry(w, expected_type, k, n);
    if (f.status != RIBN_OK) return f;
    uint64_t expected_in = 0, expected_out = 0;
    if (mul_overflows(*k, members, &expected_in) || mul_overflows(*n, members, &expected_out))
        return fail(RIBN_E_SHAPE_OVERFLOW, "quantized GEMV shape does not fit CUDA launch arguments");
    if (x_len != expected_in)
        return fail(RIBN_E_INPUT_LENGTH,
                    fmt("quantized GEMV input has %" PRIu64 " values, expected %" PRIu64, x_len, expected_in), expected_in,
                    x_len);
    if (y_len != expected_out)
        return fail(RIBN_E_OUTPUT_LENGTH,
                    fmt("quantized GEMV output has %" PRIu64 " values, expected %" PRIu64, y_len, expected_out),
                    expected_out, y_len);
    return Failure{};
}

struct TcExtras {
    bool swiglu = false;        // x rows are [gate | up]
    bool skip_prepass = false;  // reuse the f16 activations the previous call of the group left in the workspace
    bool accumulate = false;    // y += W x
};

int enqueue_tc(ribn_ctx* ctx, const ribn_qweight* w, uint64_t k, uint64_t n, const void* x, int x_dtype, void* y, int y_dtype,
               uint64_t members, const float* norm_weight = nullptr, float eps = 0.0f, TcExtras extras = TcExtras{}) {
    ribn::TcArgs t{};
    t.weights = static_cast<const uint8_t*>(w->data);
    t.weight_bytes = w->encoded_bytes;
    t.value_type = w->value_type;
    t.k = static_cast<int>(k);
    t.n = static_cast<int>(n);
    t.m = static_cast<int>(members);
    t.x = x;
    t.x_bf16 = x_dtype == RIBN_BF16;
    t.norm_weight = norm_weight;
    t.eps = eps;
    t.swiglu = extras.swiglu;
    t.skip_prepass = extras.skip_prepass;
    t.accumulate = extras.accumulate;
    t.y = y;
    t.y_bf16 = y_dtype == RIBN_BF16;
    t.scratch = ctx->workspace;
    t.scratch_bytes = ctx->workspace_bytes;
    t.tickets = ctx->tickets;
    t.ticket_count = kTicketCount;
    t.force_ksplit = ctx->tc_ksplit;
    t.force_row_copies = ctx->tc_row_copies;
    t.trace = nullptr;
    if (ctx->tc_trace != 0) {
        // the last 64 KiB of the workspace; split-K partial tiles use the front
        t.trace = reinterpret_cast<long long*>(static_cast<uint8_t*>(ctx->workspace) + ctx->workspace_bytes - kTraceBytes);
        t.scratch_bytes -= kTraceBytes;
    }
    t.device_status = ctx->device_status;
    t.sm_count = ctx->sm_count;
    t.stream = ctx->stream;
    // Decode batches: one f16 tile per step, normalised per super-block, accumulated in registers.  Prefill:
    // split bf16 operands accumulated in TMEM over the whole K range (hundreds of tokens per tile do not
    // fit the registers of the accumulate warps).
    const bool decode = members <= 64 && (ctx->tc_split_operands == 0 || !t.x_bf16 || norm_weight != nullptr || extras.swiglu ||
                                          extras.skip_prepass || extras.accumulate);
    const cudaError_t e = decode ? ribn::launch_qgemv_tc(t) : ribn::launch_qgemm_tc(t);
    if (e != cudaSuccess) return record_cuda(ctx, e, "tensor-core GEMM launch");
    return RIBN_OK;
}

// The tcgen05 kernel with the weight operand in tensor memory.
bool tmem_serves(const ribn_ctx* ctx, const ribn_qweight* w, uint64_t k, uint64_t n, uint32_t members, int x_dtype) {
    // Batches of nine or more rows (tc_min_members) of Q4_K / Q5_K: weights unpacked into tensor memory.  f32 batches
    // come here only on request, like the f16-tile kernel (their default keeps every row bit-identical to a batch of one).
    if (ctx->tmem_gemv == 0 || ctx->gemv_path != 0 || members < static_cast<uint32_t>(ctx->tc_min_members)) return false;
    if (x_dtype != RIBN_BF16 && ctx->tc_f32_activations == 0) return false;
    return ribn::qgemv_tmem_supports(w->value_type, static_cast<int>(k), static_cast<int>(n), static_cast<int>(members), x_dtype == RIBN_BF16,
                                     w->data);
}

int enqueue_tmem(ribn_ctx* ctx, const ribn_qweight* w, uint64_t k, uint64_t n, const void* x, int x_dtype, int mode, const float* norm_weight,
                 float eps, void* y, int y_dtype, uint32_t members, bool accumulate, bool image_ready = false, void* y2 = nullptr,
                 uint64_t n_first = 0) {
    ribn::TmemGemvArgs a{};
    a.weights = static_cast<const uint8_t*>(w->data);
    a.value_type = w->value_type;
    a.k = static_cast<int>(k);
    a.n = static_cast<int>(n);
    a.x = x;
    a.x_bf16 = x_dtype == RIBN_BF16;
    a.mode = mode;
    a.norm_weight = norm_weight;
    a.eps = eps;
    a.y = y;
    a.y2 = y2;
    a.n_first = static_cast<int>(n_first);
    a.y_bf16 = y_dtype == RIBN_BF16;
    a.accumulate = accumulate;
    a.members = static_cast<int>(members);
    a.scratch = ctx->workspace;
    a.scratch_bytes = ctx->workspace_bytes;
    a.tickets = ctx->tickets;
    a.ticket_count = kTicketCount;
    a.force_ksplit = ctx->tc_ksplit;
    a.stages = ctx->mma_stages;
    a.image_ready = image_ready;
    a.trace = ctx->tc_trace != 0 ? reinterpret_cast<long long*>(static_cast<uint8_t*>(ctx->workspace) + ctx->workspace_bytes - kTraceBytes) : nullptr;
    if (a.trace != nullptr) a.scratch_bytes -= kTraceBytes;
    a.device_status = ctx->device_status;
    a.sm_count = ctx->sm_count;
    a.stream = ctx->stream;
    const cudaError_t e = ribn::launch_qgemv_tmem(a);
    if (e != cudaSuccess) return record_cuda(ctx, e, "GEMV launch");
    return RIBN_OK;
}

// The half2-unpack + mma.sync kernel, eight member rows per launch.  mode: 0 plain, 1 RMSNorm, 2 silu(gate) * up.
// `image_ready` = the activation images of this x are already in the workspace (an earlier projection of the
// same fused call made them).
bool mma_serves(const ribn_ctx* ctx, const ribn_qweight* w, uint64_t k, uint64_t n, uint32_t members) {
    if (ctx->mma_gemv == 0 || ctx->gemv_path != 0) return false;
    const int per_launch = members < 8 ? static_cast<int>(members) : 8;
    return ribn::gemv_mma_supports(w->value_type, static_cast<int>(k), static_cast<int>(n), per_launch, w->data);
}

// `images_made` (fused calls: shared by the projections of one input): bit 0 = the f16 image of this x is in the
// workspace, bit 1 = the int8 image is (the two narrow kernels keep different images, side by side).
int enqueue_mma(ribn_ctx* ctx, const ribn_qweight* w, uint64_t k, uint64_t n, const void* x, int x_dtype, int mode, const float* norm_weight,
                float eps, void* y, int y_dtype, uint32_t members, bool accumulate, unsigned* images_made, bool shared_image = false) {
    const bool x_bf16 = x_dtype == RIBN_BF16;
    const uint64_t x_row_bytes = k * (mode == 2 ? 2 : 1) * dtype_bytes(x_dtype);
    unsigned none_made = 0;
    if (images_made == nullptr) images_made = &none_made;
    // The integer tensor-core kernel, eight rows per launch (quants go to the instruction as 8-bit operands).
    const uint32_t per_launch = members < 8 ? members : 8;
    if (ctx->imma_gemv != 0 && (members <= static_cast<uint32_t>(ctx->imma_max_members) || members > 8) &&
        ribn::gemv_imma_supports(w->value_type, static_cast<int>(k), static_cast<int>(n), static_cast<int>(per_launch), w->data)) {
        // its images follow the ones the f16 kernel would keep for the same call
        uint64_t offset = static_cast<uint64_t>((members + 7) / 8) * ribn::gemv_mma_image_bytes(static_cast<int>(per_launch), static_cast<int>(k), 2);
        for (uint32_t m0 = 0; m0 < members; m0 += 8) {
            ribn::MmaGemvArgs a{};
            a.weights = static_cast<const uint8_t*>(w->data);
            a.value_type = w->value_type;
            a.k = static_cast<int>(k);
            a.n = static_cast<int>(n);
            a.members = static_cast<int>(members - m0 < 8 ? members - m0 : 8);
            a.x = static_cast<const uint8_t*>(x) + static_cast<uint64_t>(m0) * x_row_bytes;
            a.x_bf16 = x_bf16;
            a.mode = mode;
            a.norm_weight = norm_weight;
            a.eps = eps;
            a.y = static_cast<uint8_t*>(y) + static_cast<uint64_t>(m0) * n * dtype_bytes(y_dtype);
            a.y_bf16 = y_dtype == RIBN_BF16;
            a.accumulate = accumulate;
            a.stages = ctx->mma_stages;
            a.resident = ctx->mma_resident;
            a.grid_ctas = ctx->mma_ctas;
            a.device_status = ctx->device_status;
            a.sm_count = ctx->sm_count;
            a.stream = ctx->stream;
            const bool wide = a.members >= ctx->mma_image_members || (a.members <= 2 && ctx->mma_image_members <= 3 && a.k / 256 > 24) ||
                              (shared_image && a.members >= 2 && ctx->mma_image_members <= 8) || (mode == 2 && ctx->mma_image_members <= 8);
            const uint64_t image_bytes = ribn::gemv_imma_image_bytes(a.members, a.k);
            if (wide && offset + image_bytes <= ctx->workspace_bytes) {
                void* image = static_cast<uint8_t*>(ctx->workspace) + offset;
                offset += image_bytes;
                if ((*images_made & 2u) == 0) {
                    const cudaError_t e = ribn::launch_gemv_imma_image(a, image);
                    if (e != cudaSuccess) return record_cuda(ctx, e, "activation image launch");
                }
                a.image = image;
            }
            const cudaError_t e = ribn::launch_gemv_imma(a);
            if (e != cudaSuccess) return record_cuda(ctx, e, "GEMV launch");
        }
        *images_made |= 2u;
        return RIBN_OK;
    }
    const bool image_ready = (*images_made & 1u) != 0;
    uint64_t image_offset = 0;
    for (uint32_t m0 = 0; m0 < members; m0 += 8) {
        ribn::MmaGemvArgs a{};
        a.weights = static_cast<const uint8_t*>(w->data);
        a.value_type = w->value_type;
        a.k = static_cast<int>(k);
        a.n = static_cast<int>(n);
        a.members = static_cast<int>(members - m0 < 8 ? members - m0 : 8);
        a.x = static_cast<const uint8_t*>(x) + static_cast<uint64_t>(m0) * x_row_bytes;
        a.x_bf16 = x_bf16;
        a.mode = mode;
        a.norm_weight = norm_weight;
        a.eps = eps;
        a.y = static_cast<uint8_t*>(y) + static_cast<uint64_t>(m0) * n * dtype_bytes(y_dtype);
        a.y_bf16 = y_dtype == RIBN_BF16;
        a.accumulate = accumulate;
        a.planes = ribn::gemv_mma_planes(a.value_type, a.k, a.members, x_bf16);
        a.stages = ctx->mma_stages;
        a.resident = ctx->mma_resident;
        a.grid_ctas = ctx->mma_ctas;
        a.device_status = ctx->device_status;
        a.sm_count = ctx->sm_count;
        a.trace = ctx->tc_trace != 0 ? reinterpret_cast<long long*>(static_cast<uint8_t*>(ctx->workspace) + ctx->workspace_bytes - kTraceBytes) : nullptr;
        a.stream = ctx->stream;
        const uint64_t image_bytes = ribn::gemv_mma_image_bytes(a.members, a.k, a.planes);
        // Narrow launches convert their activations inside the kernel (no second launch on the critical path); from
        // about four slices per warp on, the conversion is worth a launch of its own (measured: one and two rows over
        // K = 12288, where every CTA would otherwise convert 48 slices before its first multiply).
        // Several projections of one normalised or gated input of two rows or more share the image: the norm /
        // activation runs once (one row is cheaper converted by every CTA than waited for).
        const bool wide = a.members >= ctx->mma_image_members || (a.members <= 2 && ctx->mma_image_members <= 3 && a.k / 256 > 24) ||
                          (shared_image && a.members >= 2 && ctx->mma_image_members <= 8) ||
                          (mode == 2 && ctx->mma_image_members <= 8);   // silu(gate) * up once, not once per CTA (measured: K = 12288, one row)
        if (wide && image_offset + image_bytes <= ctx->workspace_bytes) {
            void* image = static_cast<uint8_t*>(ctx->workspace) + image_offset;
            image_offset += image_bytes;
            if (!image_ready) {
                const cudaError_t e = ribn::launch_gemv_mma_image(a, image);
                if (e != cudaSuccess) return record_cuda(ctx, e, "activation image launch");
            }
            a.image = image;
        }
        const cudaError_t e = ribn::launch_gemv_mma(a);
        if (e != cudaSuccess) return record_cuda(ctx, e, "GEMV launch");
    }
    if (image_offset != 0) *images_made |= 1u;
    return RIBN_OK;
}

int enqueue_gemv(ribn_ctx* ctx, const ribn_qweight* w, uint64_t k, uint64_t n, const void* x, int x_dtype, void* y,
                 int y_dtype, uint32_t members, const float* norm_weight = nullptr, float eps = 0.0f) {
    GemvArgs a{};
    a.weights = static_cast<const uint8_t*>(w->data);
    a.weight_bytes = w->encoded_bytes;
    a.value_type = w->value_type;
    a.k = static_cast<int>(k);
    a.n = static_cast<int>(n);
    a.x_bf16 = x_dtype == RIBN_BF16;
    a.y_bf16 = y_dtype == RIBN_BF16;
    a.device_status = ctx->device_status;
    a.sm_count = ctx->sm_count;
    a.variant = ctx->variant;
    a.trace = ctx->tc_trace != 0 ? reinterpret_cast<long long*>(static_cast<uint8_t*>(ctx->workspace) + ctx->workspace_bytes - kTraceBytes) : nullptr;
    a.stream = ctx->stream;
    // Path 0: tensor-core decode kernel for batches (RMSNorm, when asked for, is applied in f32 by its
    // activation pre-pass).  Its operands are f16: bf16 activations convert exactly and the weights'
    // rounding (2^-12) is below the one the caller applied to the activations (2^-9); f32 activations
    // would lose 13 bits, so they take it only on request.  Its scratch is the f16 copy of the activations.
    // (Measured: a 16-token tile of the tensor-core kernel beats the integer-dot kernel's four rows from ~8 MB of weights up.)
    if (tmem_serves(ctx, w, k, n, members, x_dtype))
        return enqueue_tmem(ctx, w, k, n, x, x_dtype, norm_weight != nullptr ? 1 : 0, norm_weight, eps, y, y_dtype, members, false);
    const bool mma = mma_serves(ctx, w, k, n, members);
    const bool tc_batch = members >= static_cast<uint32_t>(ctx->tc_min_members) ||
                          (!mma && (members >= 5 || (members == 4 && static_cast<int64_t>(w->encoded_bytes) >= ctx->tc_four_row_bytes)));
    if (ctx->gemv_path == 0 && (a.x_bf16 || ctx->tc_f32_activations != 0) && tc_batch && ribn::qgemm_tc_supports(a.value_type, a.k) &&
        members * k * 2 + (1u << 20) <= ctx->workspace_bytes)
        return enqueue_tc(ctx, w, k, n, x, x_dtype, y, y_dtype, members, norm_weight, eps);
    // Up to eight rows per launch (and wider f32 batches, in groups of eight): half2 unpack + mma.sync.
    if (mma)
        return enqueue_mma(ctx, w, k, n, x, x_dtype, norm_weight != nullptr ? 1 : 0, norm_weight, eps, y, y_dtype, members, false, nullptr);
    // Path 1: integer-dot kernel.  The activations (normalised first when norm_weight is given) are
    // packed once into the context workspace, then consumed four member rows per launch (the
    // weights stay in L2 between the launches of one call).
    const int members_per_launch = members < 4 ? static_cast<int>(members) : 4;
    const uint64_t stride = ribn::packed_activation_stride(ribn::padded_k(a.k));
    if (ctx->gemv_path != 1 && ribn::gemv_dp4a_fits(a.value_type, a.k, members_per_launch) &&
        stride * members <= ctx->workspace_bytes) {
        if (members <= 4 && ctx->dp4a_prepass == 0) {
            // Up to four member rows: the kernel packs the activations itself (no pre-pass launch, no dependency on it).
            a.members = static_cast<int>(members);
            a.x = x;
            a.y = y;
            a.pack_mode = norm_weight != nullptr ? 2 : 1;
            a.norm_weight = norm_weight;
            a.eps = eps;
            bool handled = false;
            const cudaError_t e = ribn::launch_gemv_dp4a(a, &handled);
            if (e != cudaSuccess) return record_cuda(ctx, e, "GEMV launch");
            if (!handled) return record(ctx, fail(RIBN_E_DRIVER, "integer-dot GEMV refused a shape it had accepted"));
            return RIBN_OK;
        }
        cudaError_t e = ribn::launch_quantize_activations(x, a.x_bf16, norm_weight, eps, ctx->workspace,
                                                          static_cast<int>(members), a.k, ctx->stream);
        if (e != cudaSuccess) return record_cuda(ctx, e, "activation packing launch");
        for (uint32_t m0 = 0; m0 < members; m0 += 4) {
            a.members = static_cast<int>(members - m0 < 4 ? members - m0 : 4);
            a.x = static_cast<const uint8_t*>(ctx->workspace) + static_cast<uint64_t>(m0) * stride;
            a.y = static_cast<uint8_t*>(y) + static_cast<uint64_t>(m0) * n * dtype_bytes(y_dtype);
            bool handled = false;
            e = ribn::launch_gemv_dp4a(a, &handled);
            if (e != cudaSuccess) return record_cuda(ctx, e, "GEMV launch");
            if (!handled) return record(ctx, fail(RIBN_E_DRIVER, "integer-dot GEMV refused a shape it had accepted"));
        }
        return RIBN_OK;
    }
    if (ctx->gemv_path == 2)
        return record(ctx, fail(RIBN_E_INVALID_ARGUMENT, "integer-dot GEMV cannot stage these activations in shared memory"));
    // Path 2: f32 CUDA-core kernel, eight member rows per launch.
    const void* x_in = x;
    bool x_in_bf16 = a.x_bf16;
    if (norm_weight != nullptr) {
        const uint64_t need = static_cast<uint64_t>(members) * k * sizeof(float);
        if (need > ctx->workspace_bytes)
            return record(ctx, fail(RIBN_E_SHAPE_OVERFLOW, "RMSNorm+GEMV intermediate does not fit the context workspace"));
        const cudaError_t e = ribn::launch_rms_norm(x, a.x_bf16, norm_weight, ctx->workspace, false,
                                                    static_cast<int>(members), a.k, eps, ctx->stream);
        if (e != cudaSuccess) return record_cuda(ctx, e, "RMSNorm launch");
        x_in = ctx->workspace;
        x_in_bf16 = false;
    }
    a.x_bf16 = x_in_bf16;
    for (uint32_t m0 = 0; m0 < members; m0 += 8) {
        a.members = static_cast<int>(members - m0 < 8 ? members - m0 : 8);
        a.x = static_cast<const uint8_t*>(x_in) + static_cast<uint64_t>(m0) * k * (x_in_bf16 ? 2 : 4);
        a.y = static_cast<uint8_t*>(y) + static_cast<uint64_t>(m0) * n * dtype_bytes(y_dtype);
        const cudaError_t e = ribn::launch_gemv(a);
        if (e != cudaSuccess) return record_cuda(ctx, e, "GEMV launch");
    }
    return RIBN_OK;
}

}  // namespace

namespace {
// One activation pre-pass, then one GEMV launch per job (see ribn_gemv_fused).  Every job was validated.
int enqueue_fused(ribn_ctx* ctx, const ribn_gemv_job* jobs, uint32_t job_count, const uint64_t* ns, uint64_t k, const void* x,
                  int x_dtype, const float* norm_weight, float eps, uint32_t members, bool swiglu) {
    const bool x_bf16 = x_dtype == RIBN_BF16;
    bool all_tc = true, all_dp4a = true;
    const int members_per_launch = members < 4 ? static_cast<int>(members) : 4;
    for (uint32_t j = 0; j < job_count; ++j) {
        all_tc = all_tc && ribn::qgemm_tc_supports(jobs[j].weight->value_type, static_cast<int>(k));
        all_dp4a = all_dp4a && ribn::gemv_dp4a_fits(jobs[j].weight->value_type, static_cast<int>(k), members_per_launch);
    }
    bool all_tmem = true, any_split = false;
    for (uint32_t j = 0; j < job_count; ++j) {
        all_tmem = all_tmem && tmem_serves(ctx, jobs[j].weight, k, ns[j], members, x_dtype);
        any_split = any_split || jobs[j].split_rows != 0;
    }
    if (any_split && !all_tmem) {
        // Only the batch kernel writes two outputs from one launch; elsewhere the two projections of such a weight run as
        // two jobs over its two row ranges (contiguous byte ranges of the encoded tensor).
        ribn_gemv_job parts[2 * RIBN_MAX_FUSED_JOBS];
        ribn_qweight views[2 * RIBN_MAX_FUSED_JOBS];
        uint64_t part_ns[2 * RIBN_MAX_FUSED_JOBS];
        uint32_t count = 0;
        for (uint32_t j = 0; j < job_count; ++j) {
            if (jobs[j].split_rows == 0) {
                parts[count] = jobs[j];
                part_ns[count++] = ns[j];
                continue;
            }
            const uint64_t row_bytes = jobs[j].weight->encoded_bytes / ns[j];
            for (int half = 0; half < 2; ++half) {
                const uint64_t first = half == 0 ? 0 : jobs[j].split_rows, rows = half == 0 ? jobs[j].split_rows : ns[j] - jobs[j].split_rows;
                views[count] = *jobs[j].weight;
                views[count].data = static_cast<const uint8_t*>(jobs[j].weight->data) + first * row_bytes;
                views[count].encoded_bytes = rows * row_bytes;
                views[count].dimensions[1] = rows;
                parts[count] = jobs[j];
                parts[count].weight = &views[count];
                parts[count].y_device = half == 0 ? jobs[j].y_device : jobs[j].y2_device;
                parts[count].y_len = rows * members;
                parts[count].split_rows = 0;
                parts[count].y2_device = nullptr;
                part_ns[count++] = rows;
            }
        }
        return enqueue_fused(ctx, parts, count, part_ns, k, x, x_dtype, norm_weight, eps, members, swiglu);
    }
    if (all_tmem) {
        const int mode = swiglu ? 2 : (norm_weight != nullptr ? 1 : 0);
        for (uint32_t j = 0; j < job_count; ++j) {
            const int rc = enqueue_tmem(ctx, jobs[j].weight, k, ns[j], x, x_dtype, mode, norm_weight, eps, jobs[j].y_device, jobs[j].y_dtype, members,
                                        jobs[j].accumulate != 0, /*image_ready=*/j > 0, jobs[j].split_rows != 0 ? jobs[j].y2_device : nullptr,
                                        jobs[j].split_rows);
            if (rc != RIBN_OK) return rc;
        }
        return RIBN_OK;
    }
    int64_t smallest = INT64_MAX;
    bool all_mma = true;
    for (uint32_t j = 0; j < job_count; ++j) {
        smallest = std::min<int64_t>(smallest, static_cast<int64_t>(jobs[j].weight->encoded_bytes));
        all_mma = all_mma && mma_serves(ctx, jobs[j].weight, k, ns[j], members);
    }
    const bool tc_batch = members >= static_cast<uint32_t>(ctx->tc_min_members) ||
                          (!all_mma && (members >= 5 || (members == 4 && smallest >= ctx->tc_four_row_bytes)));
    if (ctx->gemv_path == 0 && (x_bf16 || ctx->tc_f32_activations != 0) && tc_batch && all_tc &&
        members * k * 2 + (1u << 20) <= ctx->workspace_bytes) {
        for (uint32_t j = 0; j < job_count; ++j) {
            TcExtras extras;
            extras.swiglu = swiglu;
            extras.skip_prepass = j > 0;
            extras.accumulate = jobs[j].accumulate != 0;
            const int rc = enqueue_tc(ctx, jobs[j].weight, k, ns[j], x, x_dtype, jobs[j].y_device, jobs[j].y_dtype, members, norm_weight, eps,
                                      extras);
            if (rc != RIBN_OK) return rc;
        }
        return RIBN_OK;
    }
    if (all_mma) {
        const int mode = swiglu ? 2 : (norm_weight != nullptr ? 1 : 0);
        unsigned images_made = 0;
        for (uint32_t j = 0; j < job_count; ++j) {
            const int rc = enqueue_mma(ctx, jobs[j].weight, k, ns[j], x, x_dtype, mode, norm_weight, eps, jobs[j].y_device, jobs[j].y_dtype, members,
                                       jobs[j].accumulate != 0, &images_made, job_count > 1 && mode != 0);
            if (rc != RIBN_OK) return rc;
        }
        return RIBN_OK;
    }
    const uint64_t stride = ribn::packed_activation_stride(ribn::padded_k(static_cast<int>(k)));
    if (ctx->gemv_path == 1 || !all_dp4a || stride * members > ctx->workspace_bytes)
        return record(ctx, fail(RIBN_E_INVALID_ARGUMENT, "the fused call needs a shape the packed-activation kernels serve"));
    const bool in_kernel = members <= 4 && ctx->dp4a_prepass == 0;
    if (!in_kernel) {
        const cudaError_t e = ribn::launch_quantize_activations(x, x_bf16, norm_weight, eps, ctx->workspace, static_cast<int>(members),
                                                                static_cast<int>(k), ctx->stream, swiglu);
        if (e != cudaSuccess) return record_cuda(ctx, e, "activation packing launch");
    }
    cudaError_t e = cudaSuccess;
    for (uint32_t j = 0; j < job_count; ++j) {
        GemvArgs a{};
        a.weights = static_cast<const uint8_t*>(jobs[j].weight->data);
        a.weight_bytes = jobs[j].weight->encoded_bytes;
        a.value_type = jobs[j].weight->value_type;
        a.k = static_cast<int>(k);
        a.n = static_cast<int>(ns[j]);
        a.x_bf16 = x_bf16;
        a.y_bf16 = jobs[j].y_dtype == RIBN_BF16;
        a.accumulate = jobs[j].accumulate != 0;
        a.device_status = ctx->device_status;
        a.sm_count = ctx->sm_count;
        a.variant = ctx->variant;
        a.trace = nullptr;
        a.stream = ctx->stream;
        for (uint32_t m0 = 0; m0 < members; m0 += 4) {
            a.members = static_cast<int>(members - m0 < 4 ? members - m0 : 4);
            a.x = static_cast<const uint8_t*>(ctx->workspace) + static_cast<uint64_t>(m0) * stride;
            if (in_kernel) {
                a.x = x;
                a.pack_mode = swiglu ? 3 : (norm_weight != nullptr ? 2 : 1);
                a.norm_weight = norm_weight;
                a.eps = eps;
            }
            a.y = static_cast<uint8_t*>(jobs[j].y_device) + static_cast<uint64_t>(m0) * ns[j] * dtype_bytes(jobs[j].y_dtype);
            bool handled = false;
            e = ribn::launch_gemv_dp4a(a, &handled);
            if (e != cudaSuccess) return record_cuda(ctx, e, "GEMV launch");
            if (!handled) return record(ctx, fail(RIBN_E_DRIVER, "integer-dot GEMV refused a shape it had accepted"));
        }
    }
    return RIBN_OK;
}



Failure validate_attention(const ribn_attention* a) {
    if (a == nullptr) return fail(RIBN_E_INVALID_ARGUMENT, "null attention descriptor");
    if (a->members == 0 || a->q_heads == 0 || a->kv_heads == 0)
        return fail(RIBN_E_INPUT_LENGTH, "attention needs at least one member and one head", 1, 0);
    if (a->head_dim != 128)
        return fail(RIBN_E_INVALID_ARGUMENT, fmt("attention head size is %u, this build serves 128", a->head_dim));
    if (a->q_heads % a->kv_heads != 0 || a->q_heads / a->kv_heads > 8)
        return fail(RIBN_E_INVALID_ARGUMENT, "query heads must be 1..8 times the key/value heads");
    if (a->rot_dims > a->head_dim || (a->rot_dims & 1u) != 0) return fail(RIBN_E_INVALID_ARGUMENT, "rotary dims must be even and at most the head size");
    if (a->max_context == 0 || a->active_context == 0 || a->active_context > a->max_context)
        return fail(RIBN_E_INVALID_ARGUMENT, "the active context must be 1..max_context");
    if (a->max_context > (1ull << 31)) return fail(RIBN_E_SHAPE_OVERFLOW, "context does not fit CUDA launch arguments");
    if (a->shared_cache > 1) return fail(RIBN_E_INVALID_ARGUMENT, "shared_cache is 0 or 1");
    if (a->members > 65535) return fail(RIBN_E_SHAPE_OVERFLOW, "at most 65535 members per attention call");
    if (!valid_dtype(static_cast<int>(a->out_dtype))) return fail(RIBN_E_INVALID_ARGUMENT, "unknown attention output dtype");
    return Failure{};
}

ribn::LayerAttentionArgs attention_args(const ribn_ctx* ctx, const ribn_attention* a, float* q, const float* k, const float* v) {
    ribn::LayerAttentionArgs r{};
    r.q = q;
    r.k = k;
    r.v = v;
    r.q_norm = a->q_norm;
    r.k_norm = a->k_norm;
    r.eps = a->eps;
    r.positions = a->positions;
    r.members = static_cast<int>(a->members);
    r.q_heads = static_cast<int>(a->q_heads);
    r.kv_heads = static_cast<int>(a->kv_heads);
    r.head_dim = static_cast<int>(a->head_dim);
    r.rot_dims = static_cast<int>(a->rot_dims);
    r.rope_base = a->rope_base;
    r.k_cache = a->k_cache;
    r.v_cache = a->v_cache;
    r.max_context = static_cast<long long>(a->max_context);
    r.active_context = static_cast<long long>(a->active_context);
    r.shared_cache = a->shared_cache == 1;
    r.device_status = ctx->device_status;
    r.stream = ctx->stream;
    return r;
}

}  // namespace

extern "C" {

int ribn_create(int device, void* cuda_stream, ribn_ctx** out) {
    if (out == nullptr) return RIBN_E_INVALID_ARGUMENT;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || device < 0 || device >= count) {
        cudaGetLastError();
        return RIBN_E_DRIVER;
    }
    DeviceGuard guard(device);
    cudaDeviceProp prop{};
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return RIBN_E_DRIVER;
    // The kernels are built for sm_100a only and there is no fallback path.
    if (prop.major != 10) return RIBN_E_DRIVER;
    ribn_ctx* ctx = new (std::nothrow) ribn_ctx();
    if (ctx == nullptr) return RIBN_E_DRIVER;
    ctx->device = device;
    ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    ctx->sm_count = prop.multiProcessorCount;
    e = cudaMalloc(&ctx->device_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(ctx->device_status, 0, sizeof(int));
    // Scratch for fused-op intermediates, allocated once here so that no later call allocates.
    ctx->workspace_bytes = 96ull << 20;   // the f16 copy of 2048 token rows of 12288 values takes half of it
    if (e == cudaSuccess) e = cudaMalloc(&ctx->workspace, ctx->workspace_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->tickets, kTicketCount * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(ctx->tickets, 0, kTicketCount * sizeof(unsigned int));
    if (e != cudaSuccess) {
        if (ctx->device_status != nullptr) cudaFree(ctx->device_status);
        if (ctx->workspace != nullptr) cudaFree(ctx->workspace);
        if (ctx->tickets != nullptr) cudaFree(ctx->tickets);
        delete ctx;
        return RIBN_E_DRIVER;
    }
    *out = ctx;
    return RIBN_OK;
}

void ribn_destroy(ribn_ctx* ctx) {
    if (ctx == nullptr) return;
    DeviceGuard guard(ctx->device);
    if (ctx->staging != nullptr) cudaFree(ctx->staging);
    for (int i = 0; i < kStagingSlots; ++i) {
        if (ctx->in_done[i] != nullptr) cudaEventDestroy(ctx->in_done[i]);
        if (ctx->compute_done[i] != nullptr) cudaEventDestroy(ctx->compute_done[i]);
        if (ctx->out_done[i] != nullptr) cudaEventDestroy(ctx->out_done[i]);
    }
    if (ctx->in_stream != nullptr) cudaStreamDestroy(ctx->in_stream);
    if (ctx->out_stream != nullptr) cudaStreamDestroy(ctx->out_stream);
    if (ctx->workspace != nullptr) cudaFree(ctx->workspace);
    if (ctx->tickets != nullptr) cudaFree(ctx->tickets);
    if (ctx->device_status != nullptr) cudaFree(ctx->device_status);
    delete ctx;
}

int ribn_context_stream(const ribn_ctx* ctx, int* device, void** cuda_stream) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    if (device != nullptr) *device = ctx->device;
    if (cuda_stream != nullptr) *cuda_stream = ctx->stream;
    return RIBN_OK;
}

int ribn_synchronize(ribn_ctx* ctx) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess && ctx->out_stream != nullptr) e = cudaStreamSynchronize(ctx->out_stream);   // downloads of host-buffer calls
    if (e != cudaSuccess) return record_cuda(ctx, e, "stream synchronize");
    int status = 0;
    e = cudaMemcpy(&status, ctx->device_status, sizeof status, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return record_cuda(ctx, e, "status readback");
    if (status != ribn::kDeviceOk) {
        cudaMemset(ctx->device_status, 0, sizeof(int));
        if (status == ribn::kDeviceScaleRange)
            return record(ctx, fail(RIBN_E_INVALID_WEIGHT,
                                    "invalid quantized weight: a super-block scale of 32 or more cannot be folded into f16 weights; results of this "
                                    "stream are invalid (set option tmem_gemv to 0 for such tensors)"));
        if (status == ribn::kDevicePositionOutOfRange)
            return record(ctx, fail(RIBN_E_INVALID_ARGUMENT,
                                    "a KV-cache position read from device memory lay outside the cache; nothing was stored there and the "
                                    "attention of that member is invalid"));
        return record(ctx, fail(RIBN_E_TIMEOUT, "a bounded device-side wait ran out; results of this stream are invalid"));
    }
    return RIBN_OK;
}

int ribn_selftest_bounded_wait(ribn_ctx* ctx, uint32_t polls) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    if (polls == 0 || polls > 65536) return record(ctx, fail(RIBN_E_INVALID_ARGUMENT, "polls must be 1..65536"));
    DeviceGuard guard(ctx->device);
    const cudaError_t e = ribn::launch_bounded_wait_selftest(ctx->device_status, polls, ctx->stream);
    if (e != cudaSuccess) return record_cuda(ctx, e, "self-test launch");
    return RIBN_OK;
}

const char* ribn_status_string(int status) {
    switch (status) {
        case RIBN_OK: return "ok";
        case RIBN_E_DRIVER: return "CUDA driver error";
        case RIBN_E_INVALID_WEIGHT: return "invalid quantized weight";
        case RIBN_E_UNSUPPORTED_TYPE: return "unsupported GGML value type for this kernel";
        case RIBN_E_SHAPE_OVERFLOW: return "quantized GEMV shape does not fit CUDA launch arguments";
        case RIBN_E_INPUT_LENGTH: return "input length mismatch";
        case RIBN_E_OUTPUT_LENGTH: return "output length mismatch";
        case RIBN_E_CONTEXT_MISMATCH: return "quantized GEMV buffers and stream belong to different CUDA contexts";
        case RIBN_E_TIMEOUT: return "bounded device wait timed out";
        case RIBN_E_INVALID_ARGUMENT: return "invalid argument";
        default: return "unknown status";
    }
}

const char* ribn_last_error(const ribn_ctx* ctx) { return ctx == nullptr ? "" : ctx->message.c_str(); }

void ribn_last_error_detail(const ribn_ctx* ctx, uint64_t* expected, uint64_t* actual) {
    if (expected) *expected = ctx ? ctx->expected : 0;
    if (actual) *actual = ctx ? ctx->actual : 0;
}

int ribn_set_option(ribn_ctx* ctx, const char* name, int64_t value) {
    if (ctx == nullptr || name == nullptr) return RIBN_E_INVALID_ARGUMENT;
    if (std::strcmp(name, "gemv_variant") == 0) {
        ctx->variant = static_cast<int>(value);
        return RIBN_OK;
    }
    if (std::strcmp(name, "tc_ksplit") == 0 && value >= 0 && value <= 64) {
        ctx->tc_ksplit = static_cast<int>(value);
        return RIBN_OK;
    }
    if (std::strcmp(name, "tc_split_operands") == 0 && (value == 0 || value == 1)) {
        ctx->tc_split_operands = static_cast<int>(value);
        return RIBN_OK;
    }
#ifdef RIBN_TRACE
    if (std::strcmp(name, "tc_trace") == 0 && (value == 0 || value == 1)) {
        ctx->tc_trace = static_cast<int>(value);
        return RIBN_OK;
    }
#endif
    if (std::strcmp(name, "tc_row_copies") == 0 && (value == 0 || value == 1)) {
        ctx->tc_row_copies = static_cast<int>(value);
        return RIBN_OK;
    }
    if (std::strcmp(name, "dp4a_prepass") == 0 && (value == 0 || value == 1)) {
        ctx->dp4a_prepass = static_cast<int>(value);
        return RIBN_OK;
    }
    if (std::strcmp(name, "pdl") == 0 && value >= 0 && value <= 2) {
        ribn::pdl_switch() = static_cast<int>(value);   // process-wide
        return RIBN_OK;
    }
    if (std::strcmp(name, "tc_f32_activations") == 0 && (value == 0 || value == 1)) {
        ctx->tc_f32_activations = static_cast<int>(value);
        return RIBN_OK;
    }
    if (std::strcmp(name, "tc_four_row_bytes") == 0 && value >= 0) {
        ctx->tc_four_row_bytes = value;
        return RIBN_OK;
    }
    if (std::strcmp(name, "tc_min_members") == 0 && value >= 1) {
        ctx->tc_min_members = static_cast<int>(value);
        return RIBN_OK;
    }
    if (std::strcmp(name, "tmem_gemv") == 0 && (value == 0 || value == 1)) {
        ctx->tmem_gemv = static_cast<int>(value);
        return RIBN_OK;
    }
    if (std::strcmp(name, "imma_gemv") == 0 && (value == 0 || value == 1)) {
        ctx->imma_gemv = static_cast<int>(value);
        return RIBN_OK;
    }
    if (std::strcmp(name, "imma_max_members") == 0 && value >= 1 && value <= 8) {
        ctx->imma_max_members = static_cast<int>(value);
        return RIBN_OK;
    }
    if (std::strcmp(name, "mma_gemv") == 0 && (value == 0 || value == 1)) {
        ctx->mma_gemv = static_cast<int>(value);
        return RIBN_OK;
    }
    if (std::strcmp(name, "mma_image_members") == 0 && value >= 1 && value <= 9) {
        ctx->mma_image_members = static_cast<int>(value);
        return RIBN_OK;
    }
    if (std::strcmp(name, "mma_stages") == 0 && value >= 0 && value <= 8) {
        ctx->mma_stages = static_cast<int>(value);
        return RIBN_OK;
    }
    if (std::strcmp(name, "mma_resident") == 0 && value >= 0 && value <= 3) {
        ctx->mma_resident = static_cast<int>(value);
        return RIBN_OK;
    }
    if (std::strcmp(name, "mma_ctas") == 0 && value >= 0 && value <= 3) {
        ctx->mma_ctas = static_cast<int>(value);
        return RIBN_OK;
    }
    if (std::strcmp(name, "gemv_path") == 0 && value >= 0 && value <= 2) {
        ctx->gemv_path = static_cast<int>(value);
        return RIBN_OK;
    }
    return record(ctx, fail(RIBN_E_INVALID_ARGUMENT, fmt("unknown option %s", name)));
}

int ribn_tensor_layout(uint32_t value_type, uint64_t* block_elements, uint64_t* block_bytes) {
    Layout layout{};
    if (!tensor_layout(value_type, &layout)) return RIBN_E_UNSUPPORTED_TYPE;
    if (block_elements) *block_elements = layout.elements;
    if (block_bytes) *block_bytes = layout.bytes;
    return RIBN_OK;
}

int ribn_validate_quantized_geometry(const ribn_qweight* weight, uint32_t expected_type, uint64_t* input_size,
                                     uint64_t* output_size) {
    return validate_geometry(weight, expected_type, input_size, output_size).status;
}

int ribn_dequantize(ribn_ctx* ctx, const ribn_qweight* weight, float* out_device, uint64_t out_len) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    uint64_t k = 0, n = 0;
    Failure f = validate_geometry(weight, 0, &k, &n);
    if (f.status != RIBN_OK) return record(ctx, f);
    uint64_t expected = 0;
    if (mul_overflows(k, n, &expected)) return record(ctx, fail(RIBN_E_SHAPE_OVERFLOW, "tensor element count overflows"));
    if (out_len != expected)
        return record(ctx, fail(RIBN_E_OUTPUT_LENGTH,
                                fmt("dequantize output has %" PRIu64 " values, expected %" PRIu64, out_len, expected),
                                expected, out_len));
    DeviceGuard guard(ctx->device);
    f = check_device_pointer(ctx, weight->data, "weight");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, out_device, "output");
    if (f.status != RIBN_OK) return record(ctx, f);
    const cudaError_t e = ribn::launch_dequantize(static_cast<const uint8_t*>(weight->data), weight->value_type, k, n,
                                                  out_device, ctx->sm_count, ctx->stream);
    if (e != cudaSuccess) return record_cuda(ctx, e, "dequantize launch");
    return RIBN_OK;
}

int ribn_gemv(ribn_ctx* ctx, uint32_t expected_type, const ribn_qweight* weight, const void* x_device, int x_dtype,
              uint64_t x_len, void* y_device, int y_dtype, uint64_t y_len, uint32_t members) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    uint64_t k = 0, n = 0;
    Failure f = validate_gemv(weight, expected_type, x_dtype, x_len, y_dtype, y_len, members, &k, &n);
    if (f.status != RIBN_OK) return record(ctx, f);
    DeviceGuard guard(ctx->device);
    f = check_device_pointer(ctx, weight->data, "weight");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, x_device, "input");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, y_device, "output");
    if (f.status != RIBN_OK) return record(ctx, f);
    return enqueue_gemv(ctx, weight, k, n, x_device, x_dtype, y_device, y_dtype, members);
}

int ribn_rms_norm_gemv(ribn_ctx* ctx, uint32_t expected_type, const ribn_qweight* weight, const void* x_device,
                       int x_dtype, uint64_t x_len, const float* norm_weight_device, uint64_t norm_weight_len, float eps,
                       void* y_device, int y_dtype, uint64_t y_len, uint32_t members) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    uint64_t k = 0, n = 0;
    Failure f = validate_gemv(weight, expected_type, x_dtype, x_len, y_dtype, y_len, members, &k, &n);
    if (f.status != RIBN_OK) return record(ctx, f);
    if (norm_weight_len != k)
        return record(ctx, fail(RIBN_E_INPUT_LENGTH,
                                fmt("RMSNorm weight has %" PRIu64 " values, expected %" PRIu64, norm_weight_len, k), k,
                                norm_weight_len));
    DeviceGuard guard(ctx->device);
    f = check_device_pointer(ctx, weight->data, "weight");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, x_device, "input");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, norm_weight_device, "norm weight");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, y_device, "output");
    if (f.status != RIBN_OK) return record(ctx, f);
    return enqueue_gemv(ctx, weight, k, n, x_device, x_dtype, y_device, y_dtype, members, norm_weight_device, eps);
}

int ribn_gemm(ribn_ctx* ctx, uint32_t expected_type, const ribn_qweight* weight, const void* x_device, uint64_t x_len,
              void* y_device, int y_dtype, uint64_t y_len, uint64_t tokens) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    if (!valid_dtype(y_dtype)) return record(ctx, fail(RIBN_E_INVALID_ARGUMENT, "unknown output dtype"));
    if (tokens == 0) return record(ctx, fail(RIBN_E_INPUT_LENGTH, "quantized GEMM input has 0 values, expected 1", 1, 0));
    uint64_t k = 0, n = 0;
    Failure f = validate_geometry(weight, expected_type, &k, &n);
    if (f.status != RIBN_OK) return record(ctx, f);
    uint64_t expected_in = 0, expected_out = 0;
    if (tokens > static_cast<uint64_t>(std::numeric_limits<int32_t>::max()) || mul_overflows(k, tokens, &expected_in) ||
        mul_overflows(n, tokens, &expected_out))
        return record(ctx, fail(RIBN_E_SHAPE_OVERFLOW, "quantized GEMM shape does not fit CUDA launch arguments"));
    if (x_len != expected_in)
        return record(ctx, fail(RIBN_E_INPUT_LENGTH,
                                fmt("quantized GEMM input has %" PRIu64 " values, expected %" PRIu64, x_len, expected_in),
                                expected_in, x_len));
    if (y_len != expected_out)
        return record(ctx, fail(RIBN_E_OUTPUT_LENGTH,
                                fmt("quantized GEMM output has %" PRIu64 " values, expected %" PRIu64, y_len, expected_out),
                                expected_out, y_len));
    if (!ribn::qgemm_tc_supports(weight->value_type, static_cast<int>(k)))
        return record(ctx, fail(RIBN_E_INVALID_WEIGHT,
                                "invalid quantized weight: the tensor-core GEMM needs an input size that is a multiple of 256"));
    DeviceGuard guard(ctx->device);
    f = check_device_pointer(ctx, weight->data, "weight");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, x_device, "input");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, y_device, "output");
    if (f.status != RIBN_OK) return record(ctx, f);
    // The kernel reads an f16 copy of the activations from the workspace: token rows go through in chunks whose copy takes at
    // most half of it (a multiple of the 256-token tile; the weights of a later chunk come from L2 or HBM again).
    uint64_t chunk = (ctx->workspace_bytes / 2) / (k * 2);
    chunk = chunk >= 256 ? chunk / 256 * 256 : (chunk > 0 ? chunk : 1);
    for (uint64_t first = 0; first < tokens; first += chunk) {
        const uint64_t rows = tokens - first < chunk ? tokens - first : chunk;
        const int rc = enqueue_tc(ctx, weight, k, n, static_cast<const uint8_t*>(x_device) + first * k * 2, RIBN_BF16,
                                  static_cast<uint8_t*>(y_device) + first * n * dtype_bytes(y_dtype), y_dtype, rows);
        if (rc != RIBN_OK) return rc;
    }
    return RIBN_OK;
}

#ifdef RIBN_TRACE
// Diagnostics build only (not declared in the public header): copies the stamps the kernels recorded in the last
// 64 KiB of the workspace (option "tc_trace" = 1) to the host.
int ribn_debug_read_trace(ribn_ctx* ctx, void* host_dst, uint64_t bytes) {
    if (ctx == nullptr || host_dst == nullptr || bytes > kTraceBytes) return RIBN_E_INVALID_ARGUMENT;
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess)
        e = cudaMemcpy(host_dst, static_cast<uint8_t*>(ctx->workspace) + ctx->workspace_bytes - kTraceBytes, bytes, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return record_cuda(ctx, e, "trace readback");
    return RIBN_OK;
}
#endif

int ribn_reserve_staging(ribn_ctx* ctx, uint64_t bytes) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    if (bytes <= ctx->staging_bytes) return RIBN_OK;
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess && ctx->out_stream != nullptr) e = cudaStreamSynchronize(ctx->out_stream);
    if (e != cudaSuccess) return record_cuda(ctx, e, "stream synchronize");
    if (ctx->staging != nullptr) cudaFree(ctx->staging);
    ctx->staging = nullptr;
    ctx->staging_bytes = 0;
    bytes = (bytes + 255) & ~255ull;
    e = cudaMalloc(&ctx->staging, bytes * kStagingSlots);
    if (e != cudaSuccess) return record_cuda(ctx, e, "staging allocation");
    ctx->staging_bytes = bytes;
    if (ctx->in_stream == nullptr) {
        e = cudaStreamCreateWithFlags(&ctx->in_stream, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->out_stream, cudaStreamNonBlocking);
        for (int i = 0; i < kStagingSlots && e == cudaSuccess; ++i) {
            e = cudaEventCreateWithFlags(&ctx->in_done[i], cudaEventDisableTiming);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->compute_done[i], cudaEventDisableTiming);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->out_done[i], cudaEventDisableTiming);
        }
        if (e != cudaSuccess) return record_cuda(ctx, e, "copy streams");
    }
    for (bool& used : ctx->slot_used) used = false;
    return RIBN_OK;
}

int ribn_gemv_host(ribn_ctx* ctx, uint32_t expected_type, const ribn_qweight* weight, const void* x_host, int x_dtype,
                   uint64_t x_len, void* y_host, int y_dtype, uint64_t y_len, uint32_t members) {
    const int status = ribn_gemv_host_async(ctx, expected_type, weight, x_host, x_dtype, x_len, y_host, y_dtype, y_len, members);
    if (status != RIBN_OK) return status;
    return ribn_synchronize(ctx);   // also reports a bounded device wait that ran out
}

int ribn_gemv_host_async(ribn_ctx* ctx, uint32_t expected_type, const ribn_qweight* weight, const void* x_host, int x_dtype,
                         uint64_t x_len, void* y_host, int y_dtype, uint64_t y_len, uint32_t members) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    uint64_t k = 0, n = 0;
    Failure f = validate_gemv(weight, expected_type, x_dtype, x_len, y_dtype, y_len, members, &k, &n);
    if (f.status != RIBN_OK) return record(ctx, f);
    if (x_host == nullptr || y_host == nullptr) return record(ctx, fail(RIBN_E_INVALID_ARGUMENT, "host pointer is null"));
    DeviceGuard guard(ctx->device);
    f = check_device_pointer(ctx, weight->data, "weight");
    if (f.status != RIBN_OK) return record(ctx, f);
    const uint64_t x_bytes = x_len * dtype_bytes(x_dtype);
    const uint64_t y_bytes = y_len * dtype_bytes(y_dtype);
    const uint64_t y_offset = (x_bytes + 255) & ~255ull;
    if (y_offset + y_bytes > ctx->staging_bytes)
        return record(ctx, fail(RIBN_E_INVALID_ARGUMENT,
                                fmt("staging buffer holds %" PRIu64 " bytes, this call needs %" PRIu64
                                    " (ribn_reserve_staging)",
                                    ctx->staging_bytes, y_offset + y_bytes)));
    // slot of this call; its previous user's download must have left it before the upload overwrites it
    const int slot = static_cast<int>(ctx->host_calls++ % kStagingSlots);
    uint8_t* x_dev = static_cast<uint8_t*>(ctx->staging) + static_cast<uint64_t>(slot) * ctx->staging_bytes;
    uint8_t* y_dev = x_dev + y_offset;
    cudaError_t e = cudaSuccess;
    if (ctx->slot_used[slot]) e = cudaStreamWaitEvent(ctx->in_stream, ctx->out_done[slot], 0);
    if (e == cudaSuccess) e = cudaMemcpyAsync(x_dev, x_host, x_bytes, cudaMemcpyHostToDevice, ctx->in_stream);
    if (e == cudaSuccess) e = cudaEventRecord(ctx->in_done[slot], ctx->in_stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->stream, ctx->in_done[slot], 0);
    if (e != cudaSuccess) return record_cuda(ctx, e, "activation upload");
    const int status = enqueue_gemv(ctx, weight, k, n, x_dev, x_dtype, y_dev, y_dtype, members);
    // whatever happened, the slot's chain of events stays complete: the next user of the slot waits on out_done
    e = cudaEventRecord(ctx->compute_done[slot], ctx->stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->out_stream, ctx->compute_done[slot], 0);
    if (e == cudaSuccess && status == RIBN_OK) e = cudaMemcpyAsync(y_host, y_dev, y_bytes, cudaMemcpyDeviceToHost, ctx->out_stream);
    if (e == cudaSuccess) e = cudaEventRecord(ctx->out_done[slot], ctx->out_stream);
    ctx->slot_used[slot] = true;
    if (status != RIBN_OK) return status;
    if (e != cudaSuccess) return record_cuda(ctx, e, "output download");
    return RIBN_OK;
}

int ribn_rms_norm(ribn_ctx* ctx, const void* x_device, int x_dtype, uint64_t x_len, const float* weight_device,
                  uint64_t weight_len, void* y_device, int y_dtype, uint64_t y_len, uint32_t members, uint32_t length,
                  float eps) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    if (!valid_dtype(x_dtype) || !valid_dtype(y_dtype))
        return record(ctx, fail(RIBN_E_INVALID_ARGUMENT, "unknown activation dtype"));
    // CudaQwen35Ops::rms_norm_batch (model_ops.rs:1770-1824): zero-sized shapes and length
    // mismatches are refused before the launch.
    if (members == 0 || length == 0)
        return record(ctx, fail(RIBN_E_INPUT_LENGTH, "RMSNorm needs at least one vector of at least one value", 1, 0));
    const uint64_t expected = static_cast<uint64_t>(members) * length;
    if (x_len != expected)
        return record(ctx, fail(RIBN_E_INPUT_LENGTH,
                                fmt("RMSNorm input has %" PRIu64 " values, expected %" PRIu64, x_len, expected), expected,
                                x_len));
    if (weight_len != length)
        return record(ctx, fail(RIBN_E_INPUT_LENGTH,
                                fmt("RMSNorm weight has %" PRIu64 " values, expected %u", weight_len, length), length,
                                weight_len));
    if (y_len != expected)
        return record(ctx, fail(RIBN_E_OUTPUT_LENGTH,
                                fmt("RMSNorm output has %" PRIu64 " values, expected %" PRIu64, y_len, expected), expected,
                                y_len));
    if (length > static_cast<uint32_t>(std::numeric_limits<int32_t>::max()))
        return record(ctx, fail(RIBN_E_SHAPE_OVERFLOW, "RMSNorm length does not fit CUDA launch arguments"));
    DeviceGuard guard(ctx->device);
    Failure f = check_device_pointer(ctx, x_device, "input");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, weight_device, "weight");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, y_device, "output");
    if (f.status != RIBN_OK) return record(ctx, f);
    const cudaError_t e = ribn::launch_rms_norm(x_device, x_dtype == RIBN_BF16, weight_device, y_device,
                                                y_dtype == RIBN_BF16, static_cast<int>(members),
                                                static_cast<int>(length), eps, ctx->stream);
    if (e != cudaSuccess) return record_cuda(ctx, e, "RMSNorm launch");
    return RIBN_OK;
}

// ---------------------------------------------------------------- the reference's Q8_1 activation format

int ribn_quantize_q8_1(ribn_ctx* ctx, const float* x_device, uint64_t x_len, uint32_t* packed_device, uint64_t packed_len) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    // CudaQ8_1Quantizer::execute (activation.rs:43-69): empty and partial blocks, then the output size, then the
    // 32-bit indexing limit of the device side.
    if (x_len == 0 || x_len % 32 != 0) {
        const uint64_t expected = ((x_len == 0 ? 1 : x_len) + 31) / 32 * 32;
        return record(ctx, fail(RIBN_E_INPUT_LENGTH, fmt("Q8_1 input has %" PRIu64 " values, expected %" PRIu64, x_len, expected), expected, x_len));
    }
    const uint64_t blocks = x_len / 32;
    if (packed_len != blocks * 9)
        return record(ctx, fail(RIBN_E_OUTPUT_LENGTH, fmt("Q8_1 output has %" PRIu64 " words, expected %" PRIu64, packed_len, blocks * 9),
                                blocks * 9, packed_len));
    if (x_len > std::numeric_limits<uint32_t>::max()) return record(ctx, fail(RIBN_E_SHAPE_OVERFLOW, "Q8_1 input does not fit 32-bit indexing"));
    DeviceGuard guard(ctx->device);
    Failure f = check_device_pointer(ctx, x_device, "input");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, packed_device, "output");
    if (f.status != RIBN_OK) return record(ctx, f);
    const cudaError_t e = ribn::launch_quantize_q8_1(x_device, packed_device, blocks, ctx->sm_count, ctx->stream);
    if (e != cudaSuccess) return record_cuda(ctx, e, "Q8_1 packer launch");
    return RIBN_OK;
}

int ribn_gemv_q8_1(ribn_ctx* ctx, uint32_t expected_type, const ribn_qweight* weight, const uint32_t* packed_device, uint64_t packed_len,
                   float* y_device, uint64_t y_len, uint32_t members) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    // CudaQ4KQ8_1Gemv::execute_batch and its twins: members == 0 is an input-length error, more than eight an
    // invalid-weight error, both before geometry (tests/q4_q8_1.rs:412-445).
    if (members == 0) return record(ctx, fail(RIBN_E_INPUT_LENGTH, "quantized GEMV input has 0 values, expected 1", 1, 0));
    if (members > 8) return record(ctx, fail(RIBN_E_INVALID_WEIGHT, "invalid quantized weight: batch variant supports at most 8 members"));
    uint64_t k = 0, n = 0;
    Failure f = validate_geometry(weight, expected_type, &k, &n);
    if (f.status != RIBN_OK) return record(ctx, f);
    const uint64_t expected_in = k / 32 * 9 * members, expected_out = n * members;
    if (packed_len != expected_in)
        return record(ctx, fail(RIBN_E_INPUT_LENGTH, fmt("packed GEMV input has %" PRIu64 " words, expected %" PRIu64, packed_len, expected_in),
                                expected_in, packed_len));
    if (y_len != expected_out)
        return record(ctx, fail(RIBN_E_OUTPUT_LENGTH, fmt("quantized GEMV output has %" PRIu64 " values, expected %" PRIu64, y_len, expected_out),
                                expected_out, y_len));
    if (k > static_cast<uint64_t>(std::numeric_limits<int32_t>::max()) || n > static_cast<uint64_t>(std::numeric_limits<int32_t>::max()) / 8)
        return record(ctx, fail(RIBN_E_SHAPE_OVERFLOW, "quantized GEMV shape does not fit CUDA launch arguments"));
    DeviceGuard guard(ctx->device);
    f = check_device_pointer(ctx, weight->data, "weight");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, packed_device, "input");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, y_device, "output");
    if (f.status != RIBN_OK) return record(ctx, f);
    if ((reinterpret_cast<uintptr_t>(weight->data) & 15u) != 0)
        return record(ctx, fail(RIBN_E_INVALID_ARGUMENT, "weight data must be 16-byte aligned"));
    const cudaError_t e = ribn::launch_gemv_q8_1(weight->value_type, static_cast<const uint8_t*>(weight->data), packed_device, y_device,
                                                 static_cast<int>(k), static_cast<int>(n), static_cast<int>(members), weight->encoded_bytes / n,
                                                 ctx->stream);
    if (e != cudaSuccess) return record_cuda(ctx, e, "packed GEMV launch");
    return RIBN_OK;
}

// ---------------------------------------------------------------- decoder-layer operators between the GEMVs

int ribn_embedding(ribn_ctx* ctx, const ribn_qweight* weight, const uint32_t* tokens_device, uint32_t members, float* out_device,
                   uint64_t out_len) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    uint64_t k = 0, n = 0;
    Failure f = validate_geometry(weight, 0, &k, &n);   // [hidden, vocabulary]: one encoded row per token
    if (f.status != RIBN_OK) return record(ctx, f);
    if (members == 0) return record(ctx, fail(RIBN_E_INPUT_LENGTH, "embedding needs at least one token", 1, 0));
    if (k % 256 != 0)
        return record(ctx, fail(RIBN_E_INVALID_WEIGHT, "invalid quantized weight: the embedding needs a hidden size that is a multiple of 256"));
    uint64_t expected = 0;
    if (mul_overflows(k, members, &expected)) return record(ctx, fail(RIBN_E_SHAPE_OVERFLOW, "embedding shape does not fit CUDA launch arguments"));
    if (out_len != expected)
        return record(ctx, fail(RIBN_E_OUTPUT_LENGTH, fmt("embedding output has %" PRIu64 " values, expected %" PRIu64, out_len, expected),
                                expected, out_len));
    DeviceGuard guard(ctx->device);
    f = check_device_pointer(ctx, weight->data, "weight");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, tokens_device, "tokens");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, out_device, "output");
    if (f.status != RIBN_OK) return record(ctx, f);
    const cudaError_t e = ribn::launch_embedding(static_cast<const uint8_t*>(weight->data), weight->value_type, static_cast<int>(k),
                                                 static_cast<unsigned int>(n), tokens_device, static_cast<int>(members), out_device,
                                                 ctx->stream);
    if (e != cudaSuccess) return record_cuda(ctx, e, "embedding launch");
    return RIBN_OK;
}


int ribn_qk_norm_rope_append(ribn_ctx* ctx, const ribn_attention* attention, float* q_device, const float* k_device,
                             const float* v_device) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    Failure f = validate_attention(attention);
    if (f.status != RIBN_OK) return record(ctx, f);
    DeviceGuard guard(ctx->device);
    f = check_device_pointer(ctx, q_device, "query");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, k_device, "key");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, v_device, "value");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, attention->positions, "positions");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, attention->k_cache, "key cache");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, attention->v_cache, "value cache");
    if (f.status != RIBN_OK) return record(ctx, f);
    const cudaError_t e = ribn::launch_qk_norm_rope_append(attention_args(ctx, attention, q_device, k_device, v_device));
    if (e != cudaSuccess) return record_cuda(ctx, e, "head norm / rope / cache append launch");
    return RIBN_OK;
}

int ribn_attention_decode(ribn_ctx* ctx, const ribn_attention* attention, const float* q_device, void* out_device) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    Failure f = validate_attention(attention);
    if (f.status != RIBN_OK) return record(ctx, f);
    DeviceGuard guard(ctx->device);
    f = check_device_pointer(ctx, q_device, "query");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, out_device, "output");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, attention->positions, "positions");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, attention->k_cache, "key cache");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, attention->v_cache, "value cache");
    if (f.status != RIBN_OK) return record(ctx, f);
    const ribn::LayerAttentionArgs args = attention_args(ctx, attention, const_cast<float*>(q_device), nullptr, nullptr);
    int splits = ribn::attention_splits(args.members, args.kv_heads, args.active_context, ctx->sm_count);
    while (splits > 1 && ribn::attention_scratch_bytes(args.members, args.q_heads, splits) > ctx->workspace_bytes) --splits;
    if (ribn::attention_scratch_bytes(args.members, args.q_heads, splits) > ctx->workspace_bytes)
        return record(ctx, fail(RIBN_E_SHAPE_OVERFLOW, "attention partial results do not fit the context workspace"));
    const cudaError_t e = ribn::launch_attention_decode(args, out_device, attention->out_dtype == RIBN_BF16, ctx->workspace, splits);
    if (e != cudaSuccess) return record_cuda(ctx, e, "attention launch");
    return RIBN_OK;
}

int ribn_silu_mul(ribn_ctx* ctx, const float* gate_device, const float* up_device, float* out_device, uint32_t members,
                  uint64_t length, uint64_t input_row_stride) {
    return ribn_silu_mul_typed(ctx, gate_device, up_device, out_device, RIBN_F32, members, length, input_row_stride);
}

int ribn_silu_mul_typed(ribn_ctx* ctx, const float* gate_device, const float* up_device, void* out_device, int out_dtype, uint32_t members,
                        uint64_t length, uint64_t input_row_stride) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    if (!valid_dtype(out_dtype)) return record(ctx, fail(RIBN_E_INVALID_ARGUMENT, "unknown output dtype"));
    if (members == 0 || length == 0) return record(ctx, fail(RIBN_E_INPUT_LENGTH, "silu_mul needs at least one value", 1, 0));
    if (input_row_stride < length) return record(ctx, fail(RIBN_E_INVALID_ARGUMENT, "input rows overlap"));
    DeviceGuard guard(ctx->device);
    Failure f = check_device_pointer(ctx, gate_device, "gate");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, up_device, "up");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, out_device, "output");
    if (f.status != RIBN_OK) return record(ctx, f);
    const cudaError_t e = ribn::launch_silu_mul(gate_device, up_device, out_device, out_dtype == RIBN_BF16, members, length, input_row_stride, ctx->sm_count, ctx->stream);
    if (e != cudaSuccess) return record_cuda(ctx, e, "silu_mul launch");
    return RIBN_OK;
}

int ribn_residual_add(ribn_ctx* ctx, float* y_device, const float* x_device, uint64_t length) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    if (length == 0) return record(ctx, fail(RIBN_E_INPUT_LENGTH, "residual_add needs at least one value", 1, 0));
    DeviceGuard guard(ctx->device);
    Failure f = check_device_pointer(ctx, y_device, "accumulator");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, x_device, "addend");
    if (f.status != RIBN_OK) return record(ctx, f);
    const cudaError_t e = ribn::launch_residual_add(y_device, x_device, length, ctx->sm_count, ctx->stream);
    if (e != cudaSuccess) return record_cuda(ctx, e, "residual_add launch");
    return RIBN_OK;
}

int ribn_argmax(ribn_ctx* ctx, const float* logits_device, uint32_t members, uint64_t length, uint32_t* out_device) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    if (members == 0 || length == 0) return record(ctx, fail(RIBN_E_INPUT_LENGTH, "argmax needs at least one value", 1, 0));
    if (length > (1ull << 32)) return record(ctx, fail(RIBN_E_SHAPE_OVERFLOW, "argmax indices do not fit 32 bits"));
    DeviceGuard guard(ctx->device);
    Failure f = check_device_pointer(ctx, logits_device, "logits");
    if (f.status == RIBN_OK) f = check_device_pointer(ctx, out_device, "output");
    if (f.status != RIBN_OK) return record(ctx, f);
    const cudaError_t e = ribn::launch_argmax(logits_device, static_cast<int>(members), length, out_device, ctx->stream);
    if (e != cudaSuccess) return record_cuda(ctx, e, "argmax launch");
    return RIBN_OK;
}

int ribn_gemv_fused(ribn_ctx* ctx, const ribn_gemv_job* jobs, uint32_t job_count, const void* x_device, int x_dtype, uint64_t x_len,
                    const float* norm_weight_device, uint64_t norm_weight_len, float eps, uint32_t members, uint32_t flags) {
    if (ctx == nullptr) return RIBN_E_INVALID_ARGUMENT;
    if (jobs == nullptr || job_count == 0 || job_count > RIBN_MAX_FUSED_JOBS)
        return record(ctx, fail(RIBN_E_INVALID_ARGUMENT, fmt("a fused call takes 1..%u projections", RIBN_MAX_FUSED_JOBS)));
    const bool swiglu = (flags & RIBN_FUSED_SWIGLU) != 0;
    if ((flags & ~RIBN_FUSED_SWIGLU) != 0) return record(ctx, fail(RIBN_E_INVALID_ARGUMENT, "unknown flag"));
    if (swiglu && norm_weight_device != nullptr)
        return record(ctx, fail(RIBN_E_INVALID_ARGUMENT, "RMSNorm and silu_mul cannot both be fused in front of one projection"));
    uint64_t ns[RIBN_MAX_FUSED_JOBS];
    uint64_t k = 0;
    // Every projection is validated before anything is launched, with the reference's checks.
    for (uint32_t j = 0; j < job_count; ++j) {
        if (jobs[j].weight == nullptr) return record(ctx, fail(RIBN_E_INVALID_ARGUMENT, "null weight"));
        uint64_t kj = 0;
        uint64_t x_expected = x_len;
        if (swiglu) {
            if (x_len % 2 != 0) return record(ctx, fail(RIBN_E_INPUT_LENGTH, "a [gate | up] input has an even number of values", x_len + 1, x_len));
            x_expected = x_len / 2;
        }
        Failure f = validate_gemv(jobs[j].weight, jobs[j].expected_type, x_dtype, x_expected, jobs[j].y_dtype, jobs[j].y_len, members, &kj,
                                  &ns[j]);
        if (f.status != RIBN_OK) return record(ctx, f);
        if (jobs[j].split_rows != 0 && (jobs[j].split_rows % 128 != 0 || jobs[j].split_rows >= ns[j] || jobs[j].y2_device == nullptr))
            return record(ctx, fail(RIBN_E_INVALID_ARGUMENT,
                                    fmt("projection %u: split_rows must be a multiple of 128 below N = %" PRIu64 " with a second output", j, ns[j])));
        if (j == 0) k = kj;
        if (kj != k)
            return record(ctx, fail(RIBN_E_INPUT_LENGTH, fmt("projection %u has input size %" PRIu64 ", the first has %" PRIu64, j, kj, k), k, kj));
    }
    if (norm_weight_device != nullptr && norm_weight_len != k)
        return record(ctx, fail(RIBN_E_INPUT_LENGTH, fmt("RMSNorm weight has %" PRIu64 " values, expected %" PRIu64, norm_weight_len, k), k,
                                norm_weight_len));
    DeviceGuard guard(ctx->device);
    Failure f = check_device_pointer(ctx, x_device, "input");
    if (f.status == RIBN_OK && norm_weight_device != nullptr) f = check_device_pointer(ctx, norm_weight_device, "norm weight");
    for (uint32_t j = 0; j < job_count && f.status == RIBN_OK; ++j) {
        f = check_device_pointer(ctx, jobs[j].weight->data, "weight");
        if (f.status == RIBN_OK) f = check_device_pointer(ctx, jobs[j].y_device, "output");
        if (f.status == RIBN_OK && jobs[j].split_rows != 0) f = check_device_pointer(ctx, jobs[j].y2_device, "second output");
    }
    if (f.status != RIBN_OK) return record(ctx, f);
    return enqueue_fused(ctx, jobs, job_count, ns, k, x_device, x_dtype, norm_weight_device, eps, members, swiglu);
}

}  // extern "C"
