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

cudaError_t launch_dequantize(const uint8_t* weights, uint32_t value_type, uint64_t k, uint64_t n, float* out,
                              int sm_count, cudaStream_t stream);

cudaError_t launch_rms_norm(const void* x, bool x_bf16, const float* weight, void* y, bool y_bf16, int members,
                            int length, float eps, cudaStream_t stream);

}  // namespace ribn
