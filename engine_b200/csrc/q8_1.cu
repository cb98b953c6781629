// The reference's Q8_1 activation format and integer-dot GEMV, as a compatibility mode.
//
//   quantize_q8_1   crates/nvidia/src/activation.cu:3-28 -- per block of 32 values one header word
//                   half(max|x| / 127) | half(sum x) << 16 and eight words of four signed bytes.  The packer here
//                   reproduces that kernel bit for bit: the same IEEE division and roundf, the same xor-shuffle
//                   tree for the sum, cvt.rn for both halves.
//   GEMV            crates/nvidia/src/kernels/quantized/q4_k_q8_1.cu:40-144 and the q5_k / q6_k / q8_0 twins:
//                     Q4_K, Q5_K   y += d*scale[g] * act_d * dot(q, qa) - dmin*min[g] * act_sum   per group of 32
//                     Q6_K         y += d*scale[h] * act_d * (dot(q + 32, qa) - 32 * sum(qa))      per run of 16
//                     Q8_0         y += d * act_d * dot(q, qa)                                     per block of 32
//                   integer dots are exact (dp4a); the f32 accumulation order differs from the reference's, which its
//                   tests allow for (magnitude * 2^-23 * 32 + 1e-5).
//
// The product's own integer-dot path (two int8 planes, f32 scales) is the more accurate design; this file exists so
// that a host which already holds Q8_1-packed activations, or wants the reference's exact lossy arithmetic, gets it.
//
// Layout of the GEMV: one warp per output row, eight rows per CTA.  Lane = (group of 32 values = lane / 4, quarter of
// the group = lane % 4): every lane owns eight consecutive weights and the two activation words that face them, so a
// warp covers one super-block of 256 per iteration with each byte loaded once.  Members share the decoded weights.
#include <cuda_fp16.h>

#include "formats.cuh"
#include "internal.h"
#include "pipeline.cuh"

namespace ribn {
namespace {

constexpr int kPackWarps = 8;
constexpr int kRowsPerCta = 8;
constexpr int kMaxMembers = 8;

__global__ void __launch_bounds__(kPackWarps * 32) quantize_q8_1_kernel(const float* __restrict__ input, uint32_t* __restrict__ output,
                                                                       unsigned long long blocks) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const unsigned int lane = threadIdx.x & 31u;
    for (unsigned long long block = static_cast<unsigned long long>(blockIdx.x) * kPackWarps + (threadIdx.x >> 5); block < blocks;
         block += static_cast<unsigned long long>(gridDim.x) * kPackWarps) {
        const float x = input[block * 32 + lane];
        float maximum = fabsf(x);
        float sum = x;
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, offset));
            sum += __shfl_xor_sync(0xffffffffu, sum, offset);
        }
        const float d = __fdiv_rn(maximum, 127.0f);
        const int q = maximum == 0.0f ? 0 : static_cast<int>(roundf(__fdiv_rn(x, d)));
        uint32_t packed = static_cast<uint32_t>(q & 255);
        packed |= __shfl_down_sync(0xffffffffu, packed, 1) << 8;
        packed |= __shfl_down_sync(0xffffffffu, packed, 2) << 16;
        if ((lane & 3u) == 0u) output[block * 9 + 1 + lane / 4] = packed;
        if (lane == 0u) {
            const uint32_t dh = __half_as_ushort(__float2half_rn(d));
            const uint32_t sh = __half_as_ushort(__float2half_rn(sum));
            output[block * 9] = dh | (sh << 16);
        }
    }
}

// What a lane holds of one super-block (or, for Q8_0, of eight blocks): two words of four quants each, the factor of
// its integer dot, and -- first quarter of a group in the affine formats -- the factor of the activation sum.
struct LaneWeights {
    uint32_t q0, q1;
    float dot_factor;
    float sum_factor;   // Q4_K / Q5_K only, 0 elsewhere
};

template <uint32_t FMT>
__device__ __forceinline__ LaneWeights load_weights(const uint8_t* __restrict__ block, int group, int quarter) {
    LaneWeights w{};
    if constexpr (FMT == kQ4_K || FMT == kQ5_K) {
        const uint32_t header = ld_u32(block);
        const float d = f16_bits_to_f32(header & 0xffffu);
        const float dmin = f16_bits_to_f32(header >> 16);
        uint32_t sc_lo, sc_hi, m_lo, m_hi;
        unpack_k_scales(ld_u32(block + 4), ld_u32(block + 8), ld_u32(block + 12), sc_lo, sc_hi, m_lo, m_hi);
        const int shift = 8 * (group & 3);
        const float scale = static_cast<float>(((group < 4 ? sc_lo : sc_hi) >> shift) & 0xffu);
        const float minimum = static_cast<float>(((group < 4 ? m_lo : m_hi) >> shift) & 0xffu);
        const int quants_at = (FMT == kQ4_K ? 16 : 48) + (group >> 1) * 32 + quarter * 8;
        const uint2 packed = *reinterpret_cast<const uint2*>(block + quants_at);
        const int nibble = 4 * (group & 1);
        w.q0 = (packed.x >> nibble) & 0x0f0f0f0fu;
        w.q1 = (packed.y >> nibble) & 0x0f0f0f0fu;
        if constexpr (FMT == kQ5_K) {
            const uint2 high = *reinterpret_cast<const uint2*>(block + 16 + quarter * 8);
            w.q0 |= ((high.x >> group) & 0x01010101u) << 4;
            w.q1 |= ((high.y >> group) & 0x01010101u) << 4;
        }
        w.dot_factor = d * scale;
        w.sum_factor = quarter == 0 ? dmin * minimum : 0.0f;
    } else if constexpr (FMT == kQ6_K) {
        const int chunk = group >> 2, variant = group & 3;
        const uint8_t* low = block + chunk * 64 + (variant & 1) * 32 + quarter * 8;
        const uint8_t* high = block + 128 + chunk * 32 + quarter * 8;
        const int low_shift = variant < 2 ? 0 : 4;
        const int high_shift = 2 * variant;
        w.q0 = ((ld_u32_a2(low) >> low_shift) & 0x0f0f0f0fu) | (((ld_u32_a2(high) >> high_shift) & 0x03030303u) << 4);
        w.q1 = ((ld_u32_a2(low + 4) >> low_shift) & 0x0f0f0f0fu) | (((ld_u32_a2(high + 4) >> high_shift) & 0x03030303u) << 4);
        const float d = f16_bits_to_f32(ld_u16(block + 208));
        const float scale = static_cast<float>(static_cast<signed char>(block[192 + group * 2 + (quarter >> 1)]));
        w.dot_factor = d * scale;
    } else {
        const uint8_t* b = block + group * 34;
        w.q0 = ld_u32_a2(b + 2 + quarter * 8);
        w.q1 = ld_u32_a2(b + 6 + quarter * 8);
        w.dot_factor = f16_bits_to_f32(ld_u16(b));
    }
    return w;
}

// input: [members][k / 32 * 9] words; output [members][n].  `blocks32` = k / 32; a warp iteration covers eight of them.
template <uint32_t FMT>
__global__ void __launch_bounds__(kRowsPerCta * 32) gemv_q8_1_kernel(const uint8_t* __restrict__ weights, const uint32_t* __restrict__ input,
                                                                     float* __restrict__ output, int blocks32, int n, int members,
                                                                     unsigned long long row_bytes) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int row = blockIdx.x * kRowsPerCta + (threadIdx.x >> 5);
    if (row >= n) return;
    const int lane = threadIdx.x & 31;
    const int group = lane >> 2, quarter = lane & 3;
    constexpr int kUnitBytes = FMT == kQ4_K ? 144 : FMT == kQ5_K ? 176 : FMT == kQ6_K ? 210 : 8 * 34;
    const uint8_t* row_base = weights + static_cast<unsigned long long>(row) * row_bytes;
    const unsigned long long packed_stride = static_cast<unsigned long long>(blocks32) * 9ull;
    float acc[kMaxMembers];
#pragma unroll
    for (int m = 0; m < kMaxMembers; ++m) acc[m] = 0.0f;
    for (int unit = 0; unit * 8 < blocks32; ++unit) {
        const int block32 = unit * 8 + group;
        if (FMT == kQ8_0 && block32 >= blocks32) continue;      // K need only be a multiple of 32 there
        const LaneWeights w = load_weights<FMT>(row_base + static_cast<unsigned long long>(unit) * kUnitBytes, group, quarter);
#pragma unroll
        for (int m = 0; m < kMaxMembers; ++m) {
            if (m < members) {
                const uint32_t* activation = input + m * packed_stride + static_cast<unsigned long long>(block32) * 9ull;
                const uint32_t header = activation[0];
                const uint32_t a0 = activation[1 + 2 * quarter], a1 = activation[2 + 2 * quarter];
                int dot = __dp4a(static_cast<int>(w.q0), static_cast<int>(a0), 0);
                dot = __dp4a(static_cast<int>(w.q1), static_cast<int>(a1), dot);
                if constexpr (FMT == kQ6_K) {
                    // the stored quants carry a bias of 32: remove it through the sum of the facing activation bytes
                    int bias = __dp4a(0x01010101, static_cast<int>(a0), 0);
                    bias = __dp4a(0x01010101, static_cast<int>(a1), bias);
                    dot -= 32 * bias;
                }
                const float activation_scale = f16_bits_to_f32(header & 0xffffu);
                acc[m] = fmaf(w.dot_factor * activation_scale, static_cast<float>(dot), acc[m]);
                if constexpr (FMT == kQ4_K || FMT == kQ5_K) acc[m] = fmaf(-w.sum_factor, f16_bits_to_f32(header >> 16), acc[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < kMaxMembers; ++m) {
        if (m < members) {
            float total = acc[m];
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1) total += __shfl_xor_sync(0xffffffffu, total, offset);
            if (lane == 0) output[static_cast<unsigned long long>(m) * n + row] = total;
        }
    }
}

}  // namespace

cudaError_t launch_quantize_q8_1(const float* input, uint32_t* output, uint64_t blocks, int sm_count, cudaStream_t stream) {
    unsigned long long ctas = (blocks + kPackWarps - 1) / kPackWarps;
    const unsigned long long cap = static_cast<unsigned long long>(sm_count) * 16;
    if (ctas > cap) ctas = cap;
    return launch_kernel_if(pdl_switch() == 1, quantize_q8_1_kernel, dim3(static_cast<unsigned>(ctas ? ctas : 1)), dim3(kPackWarps * 32), 0, stream, input,
                            output, static_cast<unsigned long long>(blocks));
}

cudaError_t launch_gemv_q8_1(uint32_t value_type, const uint8_t* weights, const uint32_t* packed, float* output, int k, int n, int members,
                             uint64_t row_bytes, cudaStream_t stream) {
    if (members < 1 || members > kMaxMembers) return cudaErrorInvalidValue;
    const dim3 grid((n + kRowsPerCta - 1) / kRowsPerCta), block(kRowsPerCta * 32);
    const int blocks32 = k / 32;
    const unsigned long long stride = row_bytes;
    switch (value_type) {
        case kQ4_K: return launch_kernel_if(pdl_switch() == 1, gemv_q8_1_kernel<kQ4_K>, grid, block, 0, stream, weights, packed, output, blocks32, n, members, stride);
        case kQ5_K: return launch_kernel_if(pdl_switch() == 1, gemv_q8_1_kernel<kQ5_K>, grid, block, 0, stream, weights, packed, output, blocks32, n, members, stride);
        case kQ6_K: return launch_kernel_if(pdl_switch() == 1, gemv_q8_1_kernel<kQ6_K>, grid, block, 0, stream, weights, packed, output, blocks32, n, members, stride);
        case kQ8_0: return launch_kernel_if(pdl_switch() == 1, gemv_q8_1_kernel<kQ8_0>, grid, block, 0, stream, weights, packed, output, blocks32, n, members, stride);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ribn
