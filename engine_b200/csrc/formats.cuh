// GGUF block formats as seen by one warp lane.
//
// Everything here works on a "super-block" of 256 weights: one Q4_K / Q5_K /
// Q6_K block (144 / 176 / 210 bytes) or eight consecutive Q8_0 blocks
// (8 x 34 = 272 bytes).  A warp covers a super-block with every lane owning two
// runs of four consecutive weights (run A and run B); the run positions are
// chosen per format so that the lane's quant bytes are one 32-bit word of each
// bit plane.
//
// Layout authority: crates/gguf/src/lib.rs:573-661 of the reference project.
// The decoders here are shared by the dequantize kernel (whose output is
// compared bit for bit with the reference decoder) and by the GEMV kernels, so
// the bit-exactness test covers the GEMV's decode as well.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace ribn {

constexpr uint32_t kQ8_0 = 8, kQ4_K = 12, kQ5_K = 13, kQ6_K = 14;
constexpr int kSuperBlock = 256;

// IEEE binary16 -> binary32, exact (one cvt.f32.f16); reference twin:
// crates/gguf/src/lib.rs:551-563.
__device__ __forceinline__ float f16_bits_to_f32(uint32_t bits) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(bits)));
}

__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) {
    return *reinterpret_cast<const uint16_t*>(p);
}
// 32-bit word from an address that is only 2-byte aligned (Q6_K and Q8_0 block
// strides are 210 and 34 bytes).
__device__ __forceinline__ uint32_t ld_u32_a2(const uint8_t* p) {
    return ld_u16(p) | (ld_u16(p + 2) << 16);
}
__device__ __forceinline__ uint32_t ld_u32(const uint8_t* p) {
    return *reinterpret_cast<const uint32_t*>(p);
}

// Byte `i` of `packed` (an unsigned 0..255 value) as float, minus `bias`.
// prmt drops the byte into the mantissa of 2^23, so the float is 8388608 + b
// exactly; the subtraction is exact as well.
template <int I>
__device__ __forceinline__ float byte_to_float(uint32_t packed, float bias) {
#ifdef RIBN_CVT_I2F
    return static_cast<float>((packed >> (8 * I)) & 0xffu) - bias;
#else
    return __uint_as_float(__byte_perm(packed, 0x4B000000u, 0x7650u + I)) - (8388608.0f + bias);
#endif
}

__device__ __forceinline__ void bytes_to_float4(uint32_t packed, float bias, float (&out)[4]) {
    out[0] = byte_to_float<0>(packed, bias);
    out[1] = byte_to_float<1>(packed, bias);
    out[2] = byte_to_float<2>(packed, bias);
    out[3] = byte_to_float<3>(packed, bias);
}

// The 6-bit scale/min unpack of Q4_K and Q5_K on packed words
// (crates/gguf/src/lib.rs:573-587): s0 = bytes 0..3, s1 = bytes 4..7,
// s2 = bytes 8..11 of the 12-byte field.  Byte j of sc_lo / m_lo is scale / min
// of group j, byte j of sc_hi / m_hi that of group j + 4.
__device__ __forceinline__ void unpack_k_scales(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t& sc_lo,
                                                uint32_t& sc_hi, uint32_t& m_lo, uint32_t& m_hi) {
    sc_lo = s0 & 0x3f3f3f3fu;
    m_lo = s1 & 0x3f3f3f3fu;
    sc_hi = (s2 & 0x0f0f0f0fu) | ((s0 >> 2) & 0x30303030u);
    m_hi = ((s2 >> 4) & 0x0f0f0f0fu) | ((s1 >> 2) & 0x30303030u);
}

__device__ __forceinline__ float byte_of(uint32_t packed, int i) {
    return static_cast<float>((packed >> (8 * i)) & 0xffu);
}

// Per-lane view of a super-block.  For each format:
//   kBytes              bytes per super-block
//   kScaleFloats        floats in the pre-decoded scale table of one super-block
//   offsets(lane,a,b)   element offsets (0..255) of the lane's run A and run B
//   quants(blk,lane,qa,qb)  the 8 quants as floats (signed where the format is)
//   decode_table(blk,t) scale table for the whole super-block (run by one lane)
//   scales(t,lane,...)  the lane's (scale, min) for run A and run B from a table
//   weight = scale * quant - min     (min = 0 for Q6_K / Q8_0)
template <uint32_t FMT>
struct Format;

template <>
struct Format<kQ4_K> {
    static constexpr int kBytes = 144;
    static constexpr int kScaleFloats = 16;
    static constexpr bool kHasMin = true;
    // lane = 8*j + i: run A = group 2j, positions 4i..4i+3; run B = group 2j+1.
    __device__ static void offsets(int lane, int& a, int& b) {
        a = (lane >> 3) * 64 + (lane & 7) * 4;
        b = a + 32;
    }
    __device__ static void quants(const uint8_t* blk, int lane, float (&qa)[4], float (&qb)[4]) {
        const uint32_t w = ld_u32(blk + 16 + 4 * lane);
        bytes_to_float4(w & 0x0f0f0f0fu, 0.0f, qa);
        bytes_to_float4((w >> 4) & 0x0f0f0f0fu, 0.0f, qb);
    }
    // table[4*j + {0,1,2,3}] = {d*sc[2j], dmin*m[2j], d*sc[2j+1], dmin*m[2j+1]}
    __device__ static void decode_table(const uint8_t* blk, float* table) {
        const uint4 h = *reinterpret_cast<const uint4*>(blk);
        const float d = f16_bits_to_f32(h.x & 0xffffu);
        const float dmin = f16_bits_to_f32(h.x >> 16);
        uint32_t sc_lo, sc_hi, m_lo, m_hi;
        unpack_k_scales(h.y, h.z, h.w, sc_lo, sc_hi, m_lo, m_hi);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const float sc = byte_of(g < 4 ? sc_lo : sc_hi, g & 3);
            const float mn = byte_of(g < 4 ? m_lo : m_hi, g & 3);
            table[(g >> 1) * 4 + (g & 1) * 2 + 0] = d * sc;
            table[(g >> 1) * 4 + (g & 1) * 2 + 1] = dmin * mn;
        }
    }
    __device__ static void scales(const float* table, int lane, float& sa, float& ma, float& sb, float& mb) {
        const float4 t = *reinterpret_cast<const float4*>(table + (lane >> 3) * 4);
        sa = t.x; ma = t.y; sb = t.z; mb = t.w;
    }
    // The lane's scales straight from the block header (no shared table).
    __device__ static void direct_scales(const uint8_t* blk, int lane, float& sa, float& ma, float& sb, float& mb) {
        const uint4 h = *reinterpret_cast<const uint4*>(blk);
        const float d = f16_bits_to_f32(h.x & 0xffffu);
        const float dmin = f16_bits_to_f32(h.x >> 16);
        uint32_t sc_lo, sc_hi, m_lo, m_hi;
        unpack_k_scales(h.y, h.z, h.w, sc_lo, sc_hi, m_lo, m_hi);
        const int j = lane >> 3;  // groups 2j and 2j+1
        const uint32_t sc = j < 2 ? sc_lo : sc_hi;
        const uint32_t mn = j < 2 ? m_lo : m_hi;
        const int b = (2 * j) & 3;
        sa = d * byte_of(sc, b);
        ma = dmin * byte_of(mn, b);
        sb = d * byte_of(sc, b + 1);
        mb = dmin * byte_of(mn, b + 1);
    }
};

template <>
struct Format<kQ5_K> {
    static constexpr int kBytes = 176;
    static constexpr int kScaleFloats = 16;
    static constexpr bool kHasMin = true;
    __device__ static void offsets(int lane, int& a, int& b) { Format<kQ4_K>::offsets(lane, a, b); }
    __device__ static void quants(const uint8_t* blk, int lane, float (&qa)[4], float (&qb)[4]) {
        const uint32_t w = ld_u32(blk + 48 + 4 * lane);
        // qh byte p carries, in bit g, the fifth bit of element g*32 + p.
        const uint32_t h = ld_u32(blk + 16 + 4 * (lane & 7));
        const int g = (lane >> 3) * 2;
        const uint32_t lo = (w & 0x0f0f0f0fu) | (((h >> g) & 0x01010101u) << 4);
        const uint32_t hi = ((w >> 4) & 0x0f0f0f0fu) | (((h >> (g + 1)) & 0x01010101u) << 4);
        bytes_to_float4(lo, 0.0f, qa);
        bytes_to_float4(hi, 0.0f, qb);
    }
    __device__ static void decode_table(const uint8_t* blk, float* table) { Format<kQ4_K>::decode_table(blk, table); }
    __device__ static void direct_scales(const uint8_t* blk, int lane, float& sa, float& ma, float& sb, float& mb) {
        Format<kQ4_K>::direct_scales(blk, lane, sa, ma, sb, mb);
    }
    __device__ static void scales(const float* table, int lane, float& sa, float& ma, float& sb, float& mb) {
        Format<kQ4_K>::scales(table, lane, sa, ma, sb, mb);
    }
};

template <>
struct Format<kQ6_K> {
    static constexpr int kBytes = 210;
    static constexpr int kScaleFloats = 16;
    static constexpr bool kHasMin = false;
    // lane = 16*chunk + 8*h + i: ql word 4*lane holds, in its low nibbles, group
    // 4*chunk + h (run A) and, in its high nibbles, group 4*chunk + h + 2 (run B),
    // positions 4i..4i+3 of each.
    __device__ static void offsets(int lane, int& a, int& b) {
        a = ((lane >> 4) * 4 + ((lane >> 3) & 1)) * 32 + (lane & 7) * 4;
        b = a + 64;
    }
    __device__ static void quants(const uint8_t* blk, int lane, float (&qa)[4], float (&qb)[4]) {
        const uint32_t l = ld_u32_a2(blk + 4 * lane);
        const uint32_t h = ld_u32_a2(blk + 128 + (lane >> 4) * 32 + (lane & 7) * 4);
        const int v = (lane >> 3) & 1;  // variant of run A; run B is variant v + 2
        const uint32_t lo = (l & 0x0f0f0f0fu) | (((h >> (2 * v)) & 0x03030303u) << 4);
        const uint32_t hi = ((l >> 4) & 0x0f0f0f0fu) | (((h >> (2 * v + 4)) & 0x03030303u) << 4);
        bytes_to_float4(lo, 32.0f, qa);
        bytes_to_float4(hi, 32.0f, qb);
    }
    // table[s] = d * scales[s], s = 2*group + position/16
    __device__ static void decode_table(const uint8_t* blk, float* table) {
        const float d = f16_bits_to_f32(ld_u16(blk + 208));
#pragma unroll
        for (int s = 0; s < 16; s += 2) {
            const uint32_t pair = ld_u16(blk + 192 + s);
            table[s] = d * static_cast<float>(static_cast<int8_t>(pair & 0xffu));
            table[s + 1] = d * static_cast<float>(static_cast<int8_t>(pair >> 8));
        }
    }
    __device__ static void scales(const float* table, int lane, float& sa, float& ma, float& sb, float& mb) {
        const int g = (lane >> 4) * 4 + ((lane >> 3) & 1);
        const int half = (lane & 7) >> 2;
        sa = table[2 * g + half];
        sb = table[2 * g + 4 + half];
        ma = 0.0f;
        mb = 0.0f;
    }
    __device__ static void direct_scales(const uint8_t* blk, int lane, float& sa, float& ma, float& sb, float& mb) {
        const float d = f16_bits_to_f32(ld_u16(blk + 208));
        const int s = 2 * ((lane >> 4) * 4 + ((lane >> 3) & 1)) + ((lane & 7) >> 2);
        sa = d * static_cast<float>(static_cast<int8_t>(blk[192 + s]));
        sb = d * static_cast<float>(static_cast<int8_t>(blk[192 + s + 4]));
        ma = 0.0f;
        mb = 0.0f;
    }
};

template <>
struct Format<kQ8_0> {
    static constexpr int kBytes = 272;  // eight 34-byte blocks
    static constexpr int kScaleFloats = 8;
    static constexpr bool kHasMin = false;
    // lane = 4*block + i: eight consecutive int8 of block `lane >> 2`.
    __device__ static void offsets(int lane, int& a, int& b) {
        a = lane * 8;
        b = a + 4;
    }
    __device__ static void quants(const uint8_t* blk, int lane, float (&qa)[4], float (&qb)[4]) {
        const uint8_t* q = blk + (lane >> 2) * 34 + 2 + (lane & 3) * 8;
        // int8 -> unsigned by flipping the sign bit, then remove the 128 again as float
        bytes_to_float4(ld_u32_a2(q) ^ 0x80808080u, 128.0f, qa);
        bytes_to_float4(ld_u32_a2(q + 4) ^ 0x80808080u, 128.0f, qb);
    }
    __device__ static void decode_table(const uint8_t* blk, float* table) {
#pragma unroll
        for (int b = 0; b < 8; ++b) table[b] = f16_bits_to_f32(ld_u16(blk + 34 * b));
    }
    __device__ static void scales(const float* table, int lane, float& sa, float& ma, float& sb, float& mb) {
        sa = table[lane >> 2];
        sb = sa;
        ma = 0.0f;
        mb = 0.0f;
    }
    __device__ static void direct_scales(const uint8_t* blk, int lane, float& sa, float& ma, float& sb, float& mb) {
        sa = f16_bits_to_f32(ld_u16(blk + 34 * (lane >> 2)));
        sb = sa;
        ma = 0.0f;
        mb = 0.0f;
    }
};

// weight = scale*quant - min with a single rounding: scale*quant is exact in
// binary32 for every format (<= 24 significant bits), so the fused form gives
// the same bits as the reference's multiply-then-subtract.
__device__ __forceinline__ float dequant_value(float scale, float quant, float minimum) {
    return fmaf(scale, quant, -minimum);
}

}  // namespace ribn
