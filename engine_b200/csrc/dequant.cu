// Whole-tensor dequantisation GGUF blocks -> f32, the bit-exactness gate.
//
// Device twin of dequantize_block applied block by block
// (crates/gguf/src/lib.rs:520-547, :589-661 of the reference project): one warp
// per super-block of 256 weights, the same lane mapping and decoders as the
// GEMV kernels (formats.cuh), 128-bit stores.  HBM-bound on the f32 output
// (4 bytes per weight written against 0.56-1.06 read).
#include "formats.cuh"
#include "internal.h"

namespace ribn {
namespace {

template <uint32_t FMT>
__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t* __restrict__ w, float* __restrict__ out,
                                                         unsigned long long k, unsigned long long n,
                                                         unsigned long long row_bytes, int nsb) {
    using F = Format<FMT>;
    const int lane = threadIdx.x & 31;
    const unsigned long long warps = (static_cast<unsigned long long>(gridDim.x) * blockDim.x) >> 5;
    const unsigned long long total = n * static_cast<unsigned long long>(nsb);
    int off_a, off_b;
    F::offsets(lane, off_a, off_b);
    for (unsigned long long unit = (static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
         unit < total; unit += warps) {
        const unsigned long long row = unit / nsb;
        const int sb = static_cast<int>(unit - row * nsb);
        const long long valid = static_cast<long long>(k) - static_cast<long long>(sb) * kSuperBlock;
        if (FMT == kQ8_0 && off_a >= valid) continue;  // a Q8_0 row may end inside a super-block
        const uint8_t* blk = w + row * row_bytes + static_cast<unsigned long long>(sb) * F::kBytes;
        float qa[4], qb[4], sa, ma, sb_scale, mb;
        F::quants(blk, lane, qa, qb);
        F::direct_scales(blk, lane, sa, ma, sb_scale, mb);
        float* dst = out + row * k + static_cast<unsigned long long>(sb) * kSuperBlock;
        float4 va, vb;
        va.x = dequant_value(sa, qa[0], ma);
        va.y = dequant_value(sa, qa[1], ma);
        va.z = dequant_value(sa, qa[2], ma);
        va.w = dequant_value(sa, qa[3], ma);
        vb.x = dequant_value(sb_scale, qb[0], mb);
        vb.y = dequant_value(sb_scale, qb[1], mb);
        vb.z = dequant_value(sb_scale, qb[2], mb);
        vb.w = dequant_value(sb_scale, qb[3], mb);
        *reinterpret_cast<float4*>(dst + off_a) = va;
        *reinterpret_cast<float4*>(dst + off_b) = vb;
    }
}

template <uint32_t FMT>
cudaError_t launch(const uint8_t* w, uint64_t k, uint64_t n, float* out, int sm_count, cudaStream_t stream) {
    const int nsb = static_cast<int>((k + kSuperBlock - 1) / kSuperBlock);
    const unsigned long long row_bytes = FMT == kQ8_0 ? (k / 32) * 34ull : (k / kSuperBlock) * Format<FMT>::kBytes;
    const unsigned long long units = n * static_cast<unsigned long long>(nsb);
    unsigned long long blocks = (units + 7) / 8;  // 8 warps per CTA
    const unsigned long long cap = static_cast<unsigned long long>(sm_count) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    dequantize_kernel<FMT><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(w, out, k, n, row_bytes, nsb);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_dequantize(const uint8_t* weights, uint32_t value_type, uint64_t k, uint64_t n, float* out,
                              int sm_count, cudaStream_t stream) {
    switch (value_type) {
        case kQ4_K: return launch<kQ4_K>(weights, k, n, out, sm_count, stream);
        case kQ5_K: return launch<kQ5_K>(weights, k, n, out, sm_count, stream);
        case kQ6_K: return launch<kQ6_K>(weights, k, n, out, sm_count, stream);
        case kQ8_0: return launch<kQ8_0>(weights, k, n, out, sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ribn
