// Internal launch interfaces between the C-ABI layer (api.cu) and the kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace ribn {

// Programmatic dependent launch.  The kernels of the GEMV path call griddepcontrol.launch_dependents at
// their start and griddepcontrol.wait before their first access to anything an earlier kernel of the
// stream may have written (activations, scratch) or may still read (scratch, outputs); launched with the
// attribute below, a kernel's launch latency, prologue and weight prefetch overlap its predecessor's tail.
// Weights are never written by a kernel, so reading them before the wait is safe.
inline int& pdl_switch() {
    static int enabled = 2;
    return enabled;
}

// pdl_switch(): 0 = off, 1 = every kernel of the path, 2 = the GEMV kernels and their pre-passes only (default;
// measured on the decode loop: 233 tok/s off, 266 with every kernel, 274 with the GEMV kernels only -- the small
// layer operators gain nothing from starting early and hold SM slots while they wait).
template <typename... KernelArgs, typename... Args>
cudaError_t launch_kernel_if(bool dependent, void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
    cudaLaunchConfig_t config{};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = dependent ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

template <typename... KernelArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    return launch_kernel_if(pdl_switch() != 0, kernel, grid, block, smem, stream, args...);
}

// Device status word values written by kernels whose bounded waits ran out.
constexpr int kDeviceOk = 0;
constexpr int kDeviceWaitTimeout = 1;
constexpr int kDeviceScaleRange = 3;           // a super-block scale of 32 or more met the kernel that folds it into f16 weights
constexpr int kDevicePositionOutOfRange = 2;   // a KV-cache position read from device memory lay outside the cache (or the planned context)

struct GemvArgs {
    const uint8_t* weights;   // GGUF blocks, 16-byte aligned
    uint64_t weight_bytes;
    uint32_t value_type;
    int k;                    // input size
    int n;                    // output rows
    const void* x;            // [members][k]
    bool x_bf16;
    void* y;                  // [members][n]
    bool y_bf16;
    int members;              // 1..8 per launch
    bool accumulate;          // y += W x instead of y = W x (integer-dot kernel only)
    // Integer-dot kernel: pack_mode 0 -> x is packed activations (quantize.cu); 1 / 2 / 3 -> x is the raw rows and the
    // kernel packs them itself (plain / RMSNorm with norm_weight, eps / silu(gate) * up of [gate | up] rows).
    int pack_mode;
    const float* norm_weight;
    float eps;
    int* device_status;
    int sm_count;
    int variant;              // tuning variant, 0 = default
    long long* trace;         // diagnostics: wall-clock stamps of one CTA of the integer-dot kernel, or null
    cudaStream_t stream;
};

cudaError_t launch_gemv(const GemvArgs& args);

// Packed activations for the integer-dot GEMV.  Each member row of K values (padded with zeros to
// kpad, a whole number of 256-element super-blocks) becomes, contiguously:
//   q1[kpad] int8 | q2[kpad] int8 | dq[kpad/32] f32 | sum[kpad/32] f32
// with x ~= dq * (256*q1 + q2) per block of 32 and sum the f32 sum of the block.
__host__ __device__ inline unsigned long long packed_activation_stride(int kpad) {
    return static_cast<unsigned long long>(kpad) * 2 + static_cast<unsigned long long>(kpad / 32) * 8;
}
inline int padded_k(int k) { return (k + 255) / 256 * 256; }

// x [members][k] (f32 or bf16) -> packed rows; with norm_weight != nullptr the row is RMS-normalised
// and scaled first (y = x * rsqrt(mean(x^2)+eps) * norm_weight), i.e. RMSNorm fused into the packer.  With
// swiglu the input rows are [gate | up] (2k values) and silu(gate) * up is what gets packed.
cudaError_t launch_quantize_activations(const void* x, bool x_bf16, const float* norm_weight, float eps, void* packed,
                                        int members, int k, cudaStream_t stream, bool swiglu = false);

// Integer-dot GEMV for 1..4 members over packed activations (args.x = packed rows).  *handled is
// false when the shape does not fit (activations too large for shared memory); nothing was launched
// then and the caller takes another path.
cudaError_t launch_gemv_dp4a(const GemvArgs& args, bool* handled);
bool gemv_dp4a_fits(uint32_t value_type, int k, int members);

// Half2-unpack + mma.sync GEMV for 1..8 members (gemv_mma.cu).  Serves Q4_K / Q5_K / Q6_K tensors whose rows are
// 16-byte aligned (a tiled TMA box streams them) and whose activation image fits shared memory.
struct MmaGemvArgs {
    const uint8_t* weights;
    uint32_t value_type;
    int k, n;
    const void* x;            // [members][k] f32 or bf16 (mode 2: [members][2k])
    bool x_bf16;
    int mode;                 // 0 plain, 1 RMSNorm with norm_weight / eps first, 2 silu(gate) * up of [gate | up] rows
    const float* norm_weight;
    float eps;
    const void* image;        // activation image made by launch_gemv_mma_image (then x is not read), or null
    void* y;                  // [members][n]
    bool y_bf16;
    bool accumulate;          // y += W x
    int members;              // 1..8
    int planes;               // gemv_mma_planes(): f16 planes the activations are kept in
    int stages;               // 0 = as many as fit
    int resident;             // CTAs per SM the shared-memory plan allows for, 0 = up to three
    int grid_ctas;            // CTAs per SM the grid is sized for, 0 = min(resident, 2)
    int* device_status;
    int sm_count;
    long long* trace;         // diagnostics buffer (builds with -DRIBN_TRACE), or null
    cudaStream_t stream;
};
bool gemv_mma_supports(uint32_t value_type, int k, int n, int members, const void* weights);
int gemv_mma_planes(uint32_t value_type, int k, int members, bool x_bf16);
size_t gemv_mma_image_bytes(int members, int k, int planes);
cudaError_t launch_gemv_mma_image(const MmaGemvArgs& args, void* image);
cudaError_t launch_gemv_mma(const MmaGemvArgs& args);

// The same call on the integer tensor-core instruction (gemv_imma.cu): K-quants, 1..8 member rows; `planes` is unused.
bool gemv_imma_supports(uint32_t value_type, int k, int n, int members, const void* weights);
size_t gemv_imma_image_bytes(int members, int k);
cudaError_t launch_gemv_imma_image(const MmaGemvArgs& args, void* image);
cudaError_t launch_gemv_imma(const MmaGemvArgs& args);

// tcgen05 GEMV with the weight operand unpacked into tensor memory (qgemv_tmem.cu): Q4_K / Q5_K, up to 8 f32 or
// 16 bf16 member rows per launch.
struct TmemGemvArgs {
    const uint8_t* weights;
    uint32_t value_type;
    int k, n;
    const void* x;            // [members][k] f32 or bf16 (mode 2: [members][2k])
    bool x_bf16;
    int mode;                 // 0 plain, 1 RMSNorm with norm_weight / eps first, 2 silu(gate) * up of [gate | up] rows
    const float* norm_weight;
    float eps;
    void* y;                  // [members][n], or with y2: rows below n_first as [members][n_first]
    void* y2;                 // null, or where rows n_first.. go, as [members][n - n_first] (n_first a multiple of 128)
    int n_first;
    bool y_bf16;
    bool accumulate;          // y += W x
    int members;
    void* scratch;            // the activation tiles, then split-K partial tiles
    size_t scratch_bytes;
    unsigned int* tickets;    // zero-initialised counters, one per row tile
    int ticket_count;
    int force_ksplit;         // 0 = choose
    int stages;               // raw ring depth, 0 = as deep as fits
    bool image_ready;         // the activation tiles of this x are in the scratch already (an earlier projection of the same call)
    long long* trace;         // diagnostics buffer (builds with -DRIBN_TRACE), or null
    int* device_status;
    int sm_count;
    cudaStream_t stream;
};
bool qgemv_tmem_supports(uint32_t value_type, int k, int n, int members, bool x_bf16, const void* weights);
cudaError_t launch_qgemv_tmem(const TmemGemvArgs& args);

// Tensor-core GEMM (tcgen05): Y[m][n] = sum_k dequant(W[n][k]) * X[m][k], X bf16.
struct TcArgs {
    const uint8_t* weights;
    uint64_t weight_bytes;
    uint32_t value_type;
    int k, n, m;
    const void* x;            // [m][k], 16-byte aligned; bf16 or f32 (x_bf16)
    bool x_bf16;
    const float* norm_weight; // launch_qgemv_tc only: RMSNorm weight applied to x first, or null
    float eps;
    bool swiglu;              // launch_qgemv_tc only: x rows are [gate | up], the operand is silu(gate) * up
    bool skip_prepass;        // launch_qgemv_tc only: the f16 activations of the previous call are still in the scratch
    bool accumulate;          // launch_qgemv_tc only: y += W x
    void* y;                  // [m][n]
    bool y_bf16;
    void* scratch;            // the f16 activations and their factors, then split-K partial tiles
    size_t scratch_bytes;
    unsigned int* tickets;    // zero-initialised counters, one per output tile
    int ticket_count;
    int force_ksplit;         // 0 = choose
    long long* trace;         // diagnostics buffer of the decode kernel (see TcParams), or null
    int force_row_copies;     // 1 = per-row bulk copies even where one tiled TMA box per stage would do
    int* device_status;
    int sm_count;
    cudaStream_t stream;
};
bool qgemm_tc_supports(uint32_t value_type, int k);
cudaError_t launch_qgemm_tc(const TcArgs& args);
// Decode batches (1..64 members): one f16 operand tile per step, normalised per super-block; takes
// f32 or bf16 activations and can apply RMSNorm to them in its conversion pre-pass.
cudaError_t launch_qgemv_tc(const TcArgs& args);
// The conversion pre-pass of both tensor-core kernels: row r of x (f32 or bf16, [gate | up] rows with swiglu, RMSNorm first
// when norm_weight is given) times the power of two that brings its largest magnitude to at most 2^14, as f16 [m][k];
// factor[r] = the inverse of that power.
cudaError_t launch_convert_activations_f16(const void* x, bool x_bf16, bool swiglu, const float* norm_weight, float eps, void* x16, float* factor,
                                           int m, int k, cudaStream_t stream);

cudaError_t launch_dequantize(const uint8_t* weights, uint32_t value_type, uint64_t k, uint64_t n, float* out,
                              int sm_count, cudaStream_t stream);

// What the tensor-parallel exchange (tp.cu) needs of a context: its device, stream, SM count and status word.
}  // namespace ribn
struct ribn_ctx;
namespace ribn {
void context_internals(const ribn_ctx* ctx, int* device, void** stream, int* sm_count, int** status);

// The reference's Q8_1 activation format and the integer-dot GEMV over it (q8_1.cu).
cudaError_t launch_quantize_q8_1(const float* input, uint32_t* output, uint64_t blocks, int sm_count, cudaStream_t stream);
cudaError_t launch_gemv_q8_1(uint32_t value_type, const uint8_t* weights, const uint32_t* packed, float* output, int k, int n, int members,
                             uint64_t row_bytes, cudaStream_t stream);

// Decoder-layer operators between the GEMVs (layer_ops.cu).  KV cache: [member][kv_head][max_context][head_dim] f16.
struct LayerAttentionArgs {
    float* q;                 // [members][q_heads * head_dim], rewritten in place by the norm/rope step
    const float* k;           // [members][kv_heads * head_dim]
    const float* v;
    const float* q_norm;      // [head_dim] or null
    const float* k_norm;
    float eps;
    const int* positions;     // device, one per member: index of the token being appended
    int members, q_heads, kv_heads, head_dim;
    int rot_dims;             // rotary dims per head (even, <= head_dim)
    float rope_base;
    void* k_cache;
    void* v_cache;
    long long max_context;    // tokens the cache holds per (member, head)
    long long active_context; // upper bound on positions + 1 in this call (plans the KV splits)
    bool shared_cache;        // the members are consecutive tokens of ONE sequence (a prefill chunk): all use cache slot 0
    int* device_status;       // status word of the context: kernels report positions outside the cache here
    cudaStream_t stream;
};
cudaError_t launch_embedding(const uint8_t* weights, uint32_t value_type, int k, unsigned int vocabulary, const uint32_t* tokens,
                             int members, float* out, cudaStream_t stream);
cudaError_t launch_qk_norm_rope_append(const LayerAttentionArgs& args);
int attention_splits(int members, int kv_heads, long long active_context, int sm_count);
size_t attention_scratch_bytes(int members, int q_heads, int splits);
cudaError_t launch_attention_decode(const LayerAttentionArgs& args, void* out, bool out_bf16, void* scratch, int splits);
cudaError_t launch_silu_mul(const float* gate, const float* up, void* out, bool out_bf16, uint64_t members, uint64_t length, uint64_t in_stride,
                            int sm_count, cudaStream_t stream);
cudaError_t launch_residual_add(float* y, const float* x, uint64_t total, int sm_count, cudaStream_t stream);
cudaError_t launch_argmax(const float* logits, int members, uint64_t length, uint32_t* out, cudaStream_t stream);

// One CTA polls an mbarrier nobody arrives at, at most `polls` times, then records kDeviceWaitTimeout in *status.
cudaError_t launch_bounded_wait_selftest(int* status, uint32_t polls, cudaStream_t stream);

cudaError_t launch_rms_norm(const void* x, bool x_bf16, const float* weight, void* y, bool y_bf16, int members,
                            int length, float eps, cudaStream_t stream);

}  // namespace ribn
