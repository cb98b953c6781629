// RMSNorm: y[m][i] = x[m][i] * rsqrt(mean_i(x[m]^2) + eps) * weight[i].
//
// Replaces rms_norm / rms_norm_batch of the reference
// (crates/nvidia/src/model_ops.rs:106-199; host equation
// crates/nvidia/src/qwen_reference.rs:550-556).  One CTA per activation row;
// the row is read once from memory with 128-bit loads and kept in registers
// between the reduction and the scaling pass (a row of 4096..8192 floats fits
// the register file of one CTA), so the op moves each byte once.
#include <cuda_bf16.h>

#include "internal.h"
#include "pipeline.cuh"

namespace ribn {
namespace {

constexpr int kNormThreads = 256;
constexpr int kNormVecPerThread = 8;  // 8 x 4 floats x 256 threads = 8192 elements held in registers

template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
    return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(t.x << 16), __uint_as_float(t.x & 0xffff0000u), __uint_as_float(t.y << 16),
                       __uint_as_float(t.y & 0xffff0000u));
}
template <typename T>
__device__ __forceinline__ float load1(const T* p);
template <>
__device__ __forceinline__ float load1<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load1<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__device__ __forceinline__ void store4(T* p, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 t;
    t.x = *reinterpret_cast<const uint32_t*>(&lo);
    t.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = t;
}
template <typename T>
__device__ __forceinline__ void store1(T* p, float v);
template <>
__device__ __forceinline__ void store1<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store1<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) total += scratch[w];  // fixed order: deterministic
    return total;
}

template <typename XT, typename YT>
__global__ void __launch_bounds__(kNormThreads) rms_norm_kernel(const XT* __restrict__ x, const float* __restrict__ weight,
                                                                 YT* __restrict__ y, int length, int vecs, float eps) {
    __shared__ float scratch[kNormThreads / 32];
    const XT* xr = x + static_cast<size_t>(blockIdx.x) * length;
    YT* yr = y + static_cast<size_t>(blockIdx.x) * length;
    // `vecs` groups of four elements go through 128-bit accesses; the host passes 0 when rows
    // are not 16-byte aligned (length not a multiple of four), and everything is then scalar.
    const int tail = vecs << 2;             // first element not covered by a group
    float4 held[kNormVecPerThread];
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < kNormVecPerThread; ++j) {
        const int v = threadIdx.x + j * kNormThreads;
        if (v < vecs) {
            held[j] = load4<XT>(xr + 4 * v);
            sum += held[j].x * held[j].x + held[j].y * held[j].y + held[j].z * held[j].z + held[j].w * held[j].w;
        }
    }
    // Rows longer than the register window, and the ragged last 1..3 elements, are re-read.
    for (int v = threadIdx.x + kNormVecPerThread * kNormThreads; v < vecs; v += kNormThreads) {
        const float4 t = load4<XT>(xr + 4 * v);
        sum += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
    }
    for (int i = tail + threadIdx.x; i < length; i += kNormThreads) {
        const float t = load1<XT>(xr + i);
        sum += t * t;
    }
    const float total = block_sum(sum, scratch);
    const float inv = 1.0f / sqrtf(total / static_cast<float>(length) + eps);
#pragma unroll
    for (int j = 0; j < kNormVecPerThread; ++j) {
        const int v = threadIdx.x + j * kNormThreads;
        if (v < vecs) {
            const float4 w = *reinterpret_cast<const float4*>(weight + 4 * v);
            const float4 h = held[j];
            store4<YT>(yr + 4 * v, make_float4(h.x * inv * w.x, h.y * inv * w.y, h.z * inv * w.z, h.w * inv * w.w));
        }
    }
    for (int v = threadIdx.x + kNormVecPerThread * kNormThreads; v < vecs; v += kNormThreads) {
        const float4 t = load4<XT>(xr + 4 * v);
        const float4 w = *reinterpret_cast<const float4*>(weight + 4 * v);
        store4<YT>(yr + 4 * v, make_float4(t.x * inv * w.x, t.y * inv * w.y, t.z * inv * w.z, t.w * inv * w.w));
    }
    for (int i = tail + threadIdx.x; i < length; i += kNormThreads)
        store1<YT>(yr + i, load1<XT>(xr + i) * inv * weight[i]);
}

}  // namespace

cudaError_t launch_rms_norm(const void* x, bool x_bf16, const float* weight, void* y, bool y_bf16, int members,
                            int length, float eps, cudaStream_t stream) {
    const int vecs = (length % 4 == 0) ? length / 4 : 0;
    if (x_bf16 && y_bf16)
        rms_norm_kernel<__nv_bfloat16, __nv_bfloat16><<<members, kNormThreads, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(x), weight, static_cast<__nv_bfloat16*>(y), length, vecs, eps);
    else if (x_bf16)
        rms_norm_kernel<__nv_bfloat16, float><<<members, kNormThreads, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(x), weight, static_cast<float*>(y), length, vecs, eps);
    else if (y_bf16)
        rms_norm_kernel<float, __nv_bfloat16><<<members, kNormThreads, 0, stream>>>(
            static_cast<const float*>(x), weight, static_cast<__nv_bfloat16*>(y), length, vecs, eps);
    else
        rms_norm_kernel<float, float><<<members, kNormThreads, 0, stream>>>(static_cast<const float*>(x), weight,
                                                                              static_cast<float*>(y), length, vecs, eps);
    return cudaGetLastError();
}

namespace {
__global__ void bounded_wait_selftest_kernel(int* status, uint32_t polls) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
        bool arrived = false;
        for (uint32_t spin = 0; spin < polls && !arrived; ++spin) arrived = mbar_try_wait(&bar, 0);
        if (!arrived) atomicExch(status, kDeviceWaitTimeout);
    }
}
}  // namespace

cudaError_t launch_bounded_wait_selftest(int* status, uint32_t polls, cudaStream_t stream) {
    bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(status, polls);
    return cudaGetLastError();
}

}  // namespace ribn
