// Activation packer for the integer-dot GEMV, with the RMSNorm that precedes
// the projections optionally fused in.
//
//   (x [members][K], f32 or bf16)  ->  per member: q1[kpad] | q2[kpad] | dq[kpad/32] | sum[kpad/32]
//
// Per block of 32 values: d = the power of two at or above max|x|/127,
// q1 = round(x/d), q2 = round((x - q1*d) * 256/d), dq = d/256, so that
// x ~= dq * (256*q1 + q2) with an error of at most d/512 <= max|x|/32512.
// A power-of-two step makes the split exact whenever the values carry at most
// ~14 bits below the block maximum: bf16 activations near the block maximum and
// every fixture built from dyadic values reproduce exactly.  `sum` is the f32
// sum of the block's values (the multiplier of the Q4_K / Q5_K group minimum).
//
// Role in the reference: the counterpart of CudaQ8_1Quantizer / quantize_q8_1
// (crates/nvidia/src/activation.cu:3-28, activation.rs:15-88), which packs one
// int8 plane with f16 scale and sum and is lossy at the 1e-2 level; this packer
// keeps two planes and f32 scale and sum.  With norm_weight it also replaces
// the rms_norm launch in front (crates/nvidia/src/model_ops.rs:106-199): one CTA
// per row reduces sum(x^2), then packs x * inv_rms * norm_weight.
#include <cuda_bf16.h>

#include "internal.h"
#include "pipeline.cuh"

namespace ribn {
namespace {

constexpr int kPackThreads = 512;

template <typename XT>
__device__ __forceinline__ void load_x8(const XT* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load_x8<float>(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load_x8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 t = *reinterpret_cast<const uint4*>(p);
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
    v[4] = __uint_as_float(t.z << 16); v[5] = __uint_as_float(t.z & 0xffff0000u);
    v[6] = __uint_as_float(t.w << 16); v[7] = __uint_as_float(t.w & 0xffff0000u);
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (static_cast<uint32_t>(a) & 0xffu) | ((static_cast<uint32_t>(b) & 0xffu) << 8) |
           ((static_cast<uint32_t>(c) & 0xffu) << 16) | (static_cast<uint32_t>(d) << 24);
}

// One CTA per member row.  Thread t owns the 8-element chunks t, t + 512, ...; four consecutive
// threads share a block of 32 and combine their maxima and sums with two shuffles.
// MODE 0: the row as it is; 1: RMSNorm first; 2: the row is [gate | up], 2k values, and silu(gate) * up is packed
// (silu_mul of the reference, model_ops.rs:316-328, fused in front of the down projection).
template <typename XT, int MODE>
__global__ void __launch_bounds__(kPackThreads) quantize_activations_kernel(const XT* __restrict__ x,
                                                                            const float* __restrict__ norm_weight, float eps,
                                                                            uint8_t* __restrict__ packed, int k, int kpad) {
    __shared__ float partial[kPackThreads / 32];
    pdl_launch_dependents();
    pdl_wait_prior();   // x may be the previous kernel's output; the packed rows may still be read by it
    constexpr bool NORM = MODE == 1;
    const XT* xr = x + static_cast<size_t>(blockIdx.x) * k * (MODE == 2 ? 2 : 1);
    uint8_t* out = packed + static_cast<size_t>(blockIdx.x) * packed_activation_stride(kpad);
    int8_t* q1 = reinterpret_cast<int8_t*>(out);
    int8_t* q2 = q1 + kpad;
    float* dq = reinterpret_cast<float*>(out + 2 * static_cast<size_t>(kpad));
    float* xsum = dq + kpad / 32;
    const int chunks = kpad / 8;  // a multiple of 32: whole warps enter and leave the loops together

    float inv = 1.0f;
    if (NORM) {
        float acc = 0.0f;
        for (int c = threadIdx.x; c < chunks; c += kPackThreads) {
            if (c * 8 < k) {
                float v[8];
                load_x8<XT>(xr + c * 8, v);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc += v[j] * v[j];
            }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, offset);
        if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = acc;
        __syncthreads();
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < kPackThreads / 32; ++w) total += partial[w];
        inv = 1.0f / sqrtf(total / static_cast<float>(k) + eps);
    }

    for (int c = threadIdx.x; c < chunks; c += kPackThreads) {
        float v[8];
        if (c * 8 < k) {
            load_x8<XT>(xr + c * 8, v);
            if (MODE == 2) {
                float u[8];
                load_x8<XT>(xr + k + c * 8, u);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = (v[j] / (1.0f + expf(-v[j]))) * u[j];
            }
            if (NORM) {
                float g[8];
                load_x8<float>(norm_weight + c * 8, g);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = v[j] * inv * g[j];
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.0f;
        }
        float amax = 0.0f, sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            amax = fmaxf(amax, fabsf(v[j]));
            sum += v[j];
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        // Power of two at or above amax/127 (never below 2^-100, so that 1/d stays finite).
        const float t = fmaxf(amax * (1.0f / 127.0f), 7.888609052210118e-31f);
        const float d = __uint_as_float((__float_as_uint(t) + 0x007fffffu) & 0x7f800000u);
        const float inv_d = 1.0f / d;
        int a[8], b[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float r1 = fminf(fmaxf(rintf(v[j] * inv_d), -127.0f), 127.0f);
            const float rem = fmaf(-r1, d, v[j]);
            const float r2 = fminf(fmaxf(rintf(rem * inv_d * 256.0f), -127.0f), 127.0f);
            a[j] = static_cast<int>(r1);
            b[j] = static_cast<int>(r2);
        }
        *reinterpret_cast<uint2*>(q1 + c * 8) = make_uint2(pack4(a[0], a[1], a[2], a[3]), pack4(a[4], a[5], a[6], a[7]));
        *reinterpret_cast<uint2*>(q2 + c * 8) = make_uint2(pack4(b[0], b[1], b[2], b[3]), pack4(b[4], b[5], b[6], b[7]));
        if ((c & 3) == 0) {
            // A non-finite activation makes the block scale NaN, so it still reaches the output.
            const bool finite = (amax - amax == 0.0f) && (sum - sum == 0.0f);
            dq[c >> 2] = finite ? d * (1.0f / 256.0f) : __int_as_float(0x7fc00000);
            xsum[c >> 2] = sum;
        }
    }
}

template <typename XT>
cudaError_t launch(const void* x, const float* norm_weight, float eps, void* packed, int members, int k, int kpad,
                   bool swiglu, cudaStream_t stream) {
    if (swiglu)
        return launch_kernel(quantize_activations_kernel<XT, 2>, dim3(members), dim3(kPackThreads), 0, stream,
                             static_cast<const XT*>(x), norm_weight, eps, static_cast<uint8_t*>(packed), k, kpad);
    if (norm_weight != nullptr)
        return launch_kernel(quantize_activations_kernel<XT, 1>, dim3(members), dim3(kPackThreads), 0, stream,
                             static_cast<const XT*>(x), norm_weight, eps, static_cast<uint8_t*>(packed), k, kpad);
    return launch_kernel(quantize_activations_kernel<XT, 0>, dim3(members), dim3(kPackThreads), 0, stream,
                         static_cast<const XT*>(x), norm_weight, eps, static_cast<uint8_t*>(packed), k, kpad);
}

}  // namespace

cudaError_t launch_quantize_activations(const void* x, bool x_bf16, const float* norm_weight, float eps, void* packed,
                                        int members, int k, cudaStream_t stream, bool swiglu) {
    const int kpad = padded_k(k);
    return x_bf16 ? launch<__nv_bfloat16>(x, norm_weight, eps, packed, members, k, kpad, swiglu, stream)
                  : launch<float>(x, norm_weight, eps, packed, members, k, kpad, swiglu, stream);
}

}  // namespace ribn
