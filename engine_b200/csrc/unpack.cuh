// Register-level primitives shared by the kernels that expand packed GGUF quants with half2 arithmetic:
// shared-memory loads by 32-bit address, one-instruction logic ops, packed f16 arithmetic on raw registers,
// and the "magic number" conversions (a small integer ORed into the mantissa of the half 1024.0 is 1024 + it).
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

#include "formats.cuh"

namespace ribn {

constexpr uint32_t kMagic = 0x64006400u;       // half2 (1024, 1024)
constexpr uint32_t kMagicBytes = 0x64646464u;

__device__ __forceinline__ uint32_t half2_bits(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}


__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
template <int OFFSET>
__device__ __forceinline__ uint2 lds64_at(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(a), "n"(OFFSET));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
    uint32_t v;
    asm volatile("{ .reg .u16 t; ld.shared.u16 t, [%1]; cvt.u32.u16 %0, t; }" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ int lds_s8(uint32_t a) {
    int v;
    asm volatile("{ .reg .s8 t; ld.shared.s8 t, [%1]; cvt.s32.s8 %0, t; }" : "=r"(v) : "r"(a));
    return v;
}
// (a & b) | c in one logic instruction (the integer pipe issues at half rate on this GPU, so every logic op counts twice)
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// half2 (lo, lo) / (hi, hi) of a packed pair
__device__ __forceinline__ uint32_t dup_low(uint32_t pair) {
    const __half2 h = __low2half2(*reinterpret_cast<const __half2*>(&pair));
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t dup_high(uint32_t pair) {
    const __half2 h = __high2half2(*reinterpret_cast<const __half2*>(&pair));
    return *reinterpret_cast<const uint32_t*>(&h);
}


// Scale pairs of Q4_K / Q5_K as f16: bytes (lo, lo + 1) of `packed` -> half2 (b_lo, b_lo+1), exactly.
__device__ __forceinline__ uint32_t byte_pair_half2(uint32_t packed, bool upper) {
    return hsub2(__byte_perm(packed, kMagicBytes, upper ? 0x4342u : 0x4140u), kMagic);
}

__device__ __forceinline__ uint4 lds128_unaligned(uint32_t a) {
    const uint32_t base = a & ~15u;
    const uint32_t word = (a >> 2) & 3u;
    const uint32_t shift = (a & 2u) * 8u;
    const uint4 lo = lds128(base), hi = lds128(base + 16);
    uint4 r;
    switch (word) {   // uniform across the warp
        case 0:
            r.x = __funnelshift_r(lo.x, lo.y, shift); r.y = __funnelshift_r(lo.y, lo.z, shift);
            r.z = __funnelshift_r(lo.z, lo.w, shift); r.w = __funnelshift_r(lo.w, hi.x, shift);
            break;
        case 1:
            r.x = __funnelshift_r(lo.y, lo.z, shift); r.y = __funnelshift_r(lo.z, lo.w, shift);
            r.z = __funnelshift_r(lo.w, hi.x, shift); r.w = __funnelshift_r(hi.x, hi.y, shift);
            break;
        case 2:
            r.x = __funnelshift_r(lo.z, lo.w, shift); r.y = __funnelshift_r(lo.w, hi.x, shift);
            r.z = __funnelshift_r(hi.x, hi.y, shift); r.w = __funnelshift_r(hi.y, hi.z, shift);
            break;
        default:
            r.x = __funnelshift_r(lo.w, hi.x, shift); r.y = __funnelshift_r(hi.x, hi.y, shift);
            r.z = __funnelshift_r(hi.y, hi.z, shift); r.w = __funnelshift_r(hi.z, hi.w, shift);
            break;
    }
    return r;
}

// The four 6-bit quants of one (group v, word i), as bytes shifted left by two: (q << 2) in every byte.
template <int V>
__device__ __forceinline__ uint32_t q6_bytes(uint32_t la, uint32_t lb, uint32_t h) {
    if (V == 0) return and_or(la << 2, 0x3c3c3c3cu, (h << 6) & 0xc0c0c0c0u);
    if (V == 1) return and_or(lb << 2, 0x3c3c3c3cu, (h << 4) & 0xc0c0c0c0u);
    if (V == 2) return and_or(la >> 2, 0x3c3c3c3cu, (h << 2) & 0xc0c0c0c0u);
    return and_or(lb >> 2, 0x3c3c3c3cu, h & 0xc0c0c0c0u);
}


}  // namespace ribn
