// Internal launch interfaces between the C-ABI layer (api.cu) and the kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace ribn {

// Device status word values written by kernels whose bounded waits ran out.
constexpr int kDeviceOk = 0;
constexpr int kDeviceWaitTimeout = 1;

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
    int* device_status;
    int sm_count;
    int variant;              // tuning variant, 0 = default
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
// and scaled first (y = x * rsqrt(mean(x^2)+eps) * norm_weight), i.e. RMSNorm fused into the packer.
cudaError_t launch_quantize_activations(const void* x, bool x_bf16, const float* norm_weight, float eps, void* packed,
                                        int members, int k, cudaStream_t stream);

// Integer-dot GEMV for 1..4 members over packed activations (args.x = packed rows).  *handled is
// false when the shape does not fit (activations too large for shared memory); nothing was launched
// then and the caller takes another path.
cudaError_t launch_gemv_dp4a(const GemvArgs& args, bool* handled);
bool gemv_dp4a_fits(uint32_t value_type, int k, int members);

// Tensor-core GEMM (tcgen05): Y[m][n] = sum_k dequant(W[n][k]) * X[m][k], X bf16.
struct TcArgs {
    const uint8_t* weights;
    uint64_t weight_bytes;
    uint32_t value_type;
    int k, n, m;
    const void* x;            // [m][k], 16-byte aligned; bf16 for launch_qgemm_tc, bf16 or f32 (x_bf16) for launch_qgemv_tc
    bool x_bf16;
    const float* norm_weight; // launch_qgemv_tc only: RMSNorm weight applied to x first, or null
    float eps;
    void* y;                  // [m][n]
    bool y_bf16;
    void* scratch;            // split-K partial tiles
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

cudaError_t launch_dequantize(const uint8_t* weights, uint32_t value_type, uint64_t k, uint64_t n, float* out,
                              int sm_count, cudaStream_t stream);

cudaError_t launch_rms_norm(const void* x, bool x_bf16, const float* weight, void* y, bool y_bf16, int members,
                            int length, float eps, cudaStream_t stream);

}  // namespace ribn
