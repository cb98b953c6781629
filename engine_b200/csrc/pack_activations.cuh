// Packing of one activation row for the integer-dot GEMV (layout and arithmetic: see quantize.cu), as a device
// function that a CTA -- or a part of one, with its own barrier -- calls cooperatively.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

#include "internal.h"

namespace ribn {


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

// Row cursors: a typed pointer, or a pointer whose element type (f32 / bf16) is only known at run time.
__device__ __forceinline__ void load_row8(const float* p, float (&v)[8]) { load_x8<float>(p, v); }
__device__ __forceinline__ void load_row8(const __nv_bfloat16* p, float (&v)[8]) { load_x8<__nv_bfloat16>(p, v); }
struct AnyRow {
    const uint8_t* p;
    int bf16;
    __device__ AnyRow operator+(int elements) const { return AnyRow{p + static_cast<size_t>(elements) * (bf16 ? 2 : 4), bf16}; }
};
__device__ __forceinline__ void load_row8(AnyRow r, float (&v)[8]) {
    if (r.bf16) {
        load_x8<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(r.p), v);
    } else {
        load_x8<float>(reinterpret_cast<const float*>(r.p), v);
    }
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (static_cast<uint32_t>(a) & 0xffu) | ((static_cast<uint32_t>(b) & 0xffu) << 8) |
           ((static_cast<uint32_t>(c) & 0xffu) << 16) | (static_cast<uint32_t>(d) << 24);
}

// Thread t owns the 8-element chunks t, t + THREADS, ...; four consecutive threads share a block of 32 and combine
// their maxima and sums with two shuffles.
// mode 0: the row as it is; 1: RMSNorm first; 2: the row is [gate | up], 2k values, and silu(gate) * up is packed
// (silu_mul of the reference, model_ops.rs:316-328, fused in front of the down projection).
// `xr` points at the row, `out` at its packed image; THREADS threads (a multiple of 32) with indices tid = 0..THREADS-1
// take part, `partial` is THREADS / 32 floats of shared memory and `sync` a barrier over exactly these threads.
template <int THREADS, typename Row, typename Sync>
__device__ __forceinline__ void pack_activation_row(Row xr, int mode, const float* __restrict__ norm_weight, float eps,
                                                    uint8_t* __restrict__ out, int k, int kpad, float* partial, int tid, Sync sync) {
    const bool NORM = mode == 1;
    int8_t* q1 = reinterpret_cast<int8_t*>(out);
    int8_t* q2 = q1 + kpad;
    float* dq = reinterpret_cast<float*>(out + 2 * static_cast<size_t>(kpad));
    float* xsum = dq + kpad / 32;
    const int chunks = kpad / 8;  // a multiple of 32: whole warps enter and leave the loops together

    float inv = 1.0f;
    if (NORM) {
        float acc = 0.0f;
        for (int c = tid; c < chunks; c += THREADS) {
            if (c * 8 < k) {
                float v[8];
                load_row8(xr + c * 8, v);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc += v[j] * v[j];
            }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, offset);
        if ((tid & 31) == 0) partial[tid >> 5] = acc;
        sync();
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < THREADS / 32; ++w) total += partial[w];
        sync();   // `partial` may be reused for the next row
        inv = 1.0f / sqrtf(total / static_cast<float>(k) + eps);
    }

    for (int c = tid; c < chunks; c += THREADS) {
        float v[8];
        if (c * 8 < k) {
            load_row8(xr + c * 8, v);
            if (mode == 2) {
                float u[8];
                load_row8(xr + (k + c * 8), u);
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

}  // namespace ribn
