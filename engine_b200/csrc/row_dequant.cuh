// Row-wise dequantisation of GGUF super-blocks into K-major tensor-core operand tiles.
//
// One thread owns one weight row and one half (h = 0/1) of a 64-wide K step; the raw bytes of the
// row's super-block are in shared memory.  The arithmetic per weight is the one of the reference's
// dequantisers (crates/gguf/src/lib.rs:724-884): d * scale * q - dmin * min in f32, optionally
// multiplied by a power of two (`prescale`, exact) before it is encoded for the tensor cores.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "formats.cuh"

namespace ribn {

__device__ __forceinline__ uint4 raw16(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint4 raw16_a2(const uint8_t* p) {
    uint4 v;
    v.x = ld_u32_a2(p);
    v.y = ld_u32_a2(p + 4);
    v.z = ld_u32_a2(p + 8);
    v.w = ld_u32_a2(p + 12);
    return v;
}

// Operand encodings.  An encoder turns eight f32 weights into one 16-byte chunk of a K-major tile
// (or one chunk per plane).
//
// SplitBf16: w_high = bf16(w) and w_low = bf16(w - w_high), two tiles, together 16 significant bits.
struct SplitBf16 {
    static constexpr bool kFoldOffset = false;   // 16 significant bits: keep the exact two-step dequantisation
    struct Chunk {
        uint4 high, low;
    };
    __device__ static void pair(float w0, float w1, uint32_t& high, uint32_t& low) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(w0, w1);
        high = *reinterpret_cast<const uint32_t*>(&h);
        const float h0 = __uint_as_float(high << 16);
        const float h1 = __uint_as_float(high & 0xffff0000u);
        const __nv_bfloat162 l = __floats2bfloat162_rn(w0 - h0, w1 - h1);
        low = *reinterpret_cast<const uint32_t*>(&l);
    }
    __device__ static Chunk encode(const float (&a)[4], const float (&b)[4]) {
        Chunk out;
        pair(a[0], a[1], out.high.x, out.low.x);
        pair(a[2], a[3], out.high.y, out.low.y);
        pair(b[0], b[1], out.high.z, out.low.z);
        pair(b[2], b[3], out.high.w, out.low.w);
        return out;
    }
    __device__ static Chunk zero() {
        Chunk out;
        out.high = out.low = make_uint4(0, 0, 0, 0);
        return out;
    }
};

// SingleF16: one f16 tile (11 significant bits); the caller keeps the values in f16 range by
// pre-scaling each super-block (see RowDequant::magnitude_bound).
struct SingleF16 {
    static constexpr bool kFoldOffset = true;
    struct Chunk {
        uint4 high;
    };
    __device__ static uint32_t pair(float w0, float w1) {
        const __half2 h = __floats2half2_rn(w0, w1);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    __device__ static Chunk encode(const float (&a)[4], const float (&b)[4]) {
        Chunk out;
        out.high = make_uint4(pair(a[0], a[1]), pair(a[2], a[3]), pair(b[0], b[1]), pair(b[2], b[3]));
        return out;
    }
    __device__ static Chunk zero() {
        Chunk out;
        out.high = make_uint4(0, 0, 0, 0);
        return out;
    }
};

// Byte I of `packed` (0..127) as the float 128 + byte: prmt drops it into the top mantissa bits of 128.0f.
template <int I>
__device__ __forceinline__ float byte_plus_128(uint32_t packed) {
    return __uint_as_float(__byte_perm(packed, 0x43000000u, 0x7054u + (I << 8)));
}

// Eight weights (two packed words of four byte-sized quants) -> one chunk (pair).
template <class Enc>
__device__ __forceinline__ typename Enc::Chunk chunk_from_bytes(uint32_t q0, uint32_t q1, float bias, float scale, float minimum) {
    float a[4], b[4];
    if (Enc::kFoldOffset && bias < 100.0f) {
        // Quants below 128 (every K-quant): w = scale * (128 + q) - (scale * (128 + bias) + minimum), one prmt and one
        // FMA per weight.  The folded constant is rounded at the magnitude of 160 * scale, 2^-17 of a quant step: far
        // below the f16 rounding that follows (the exact two-step form is kept where results must be bit-exact).
        const float offset = -fmaf(scale, 128.0f + bias, minimum);
        a[0] = fmaf(scale, byte_plus_128<0>(q0), offset);
        a[1] = fmaf(scale, byte_plus_128<1>(q0), offset);
        a[2] = fmaf(scale, byte_plus_128<2>(q0), offset);
        a[3] = fmaf(scale, byte_plus_128<3>(q0), offset);
        b[0] = fmaf(scale, byte_plus_128<0>(q1), offset);
        b[1] = fmaf(scale, byte_plus_128<1>(q1), offset);
        b[2] = fmaf(scale, byte_plus_128<2>(q1), offset);
        b[3] = fmaf(scale, byte_plus_128<3>(q1), offset);
        return Enc::encode(a, b);
    }
    bytes_to_float4(q0, bias, a);
    bytes_to_float4(q1, bias, b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        a[i] = dequant_value(scale, a[i], minimum);
        b[i] = dequant_value(scale, b[i], minimum);
    }
    return Enc::encode(a, b);
}

// One thread owns one weight row and one half (h = 0/1) of every 64-wide K step.  Per step it
// produces four 16-byte chunks (32 weights); chunk c of a row covers K offsets 8c .. 8c+7.
//   K-quants: chunks 2h, 2h+1 (first group of the step) and 4+2h, 4+2h+1 (second group)
//   Q8_0:     chunks 4h .. 4h+3 (block 2t+h of the super-block)
template <uint32_t FMT, class Enc>
struct RowDequant;

template <class Enc>
struct RowDequant<kQ4_K, Enc> {
    using Chunk = typename Enc::Chunk;
    // Largest |weight| the super-block can hold: |d| * 63 * 15 + |dmin| * 63.
    __device__ static float magnitude_bound(const uint8_t* blk) {
        const uint32_t h = ld_u32_a2(blk);
        return fabsf(f16_bits_to_f32(h & 0xffffu)) * 945.0f + fabsf(f16_bits_to_f32(h >> 16)) * 63.0f;
    }
    struct Scales { float a[8], b[8]; };
    __device__ static void load_scales(const uint8_t* blk, Scales& s, float prescale) {
        const uint4 h = raw16(blk);
        const float d = f16_bits_to_f32(h.x & 0xffffu) * prescale;
        const float dmin = f16_bits_to_f32(h.x >> 16) * prescale;
        uint32_t sc_lo, sc_hi, m_lo, m_hi;
        unpack_k_scales(h.y, h.z, h.w, sc_lo, sc_hi, m_lo, m_hi);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            s.a[g] = d * byte_of(g < 4 ? sc_lo : sc_hi, g & 3);
            s.b[g] = dmin * byte_of(g < 4 ? m_lo : m_hi, g & 3);
        }
    }
    __device__ static int chunk_index(int h, int c) { return (c >> 1) * 4 + 2 * h + (c & 1); }
    // The four values one K step needs, for callers whose step index is only known at run time (an array of all
    // sixteen indexed dynamically would live in local memory): scale and minimum of groups 2t and 2t+1.
    struct StepScales { float v[4]; };
    __device__ static void load_step_scales(const uint8_t* blk, int t, float prescale, StepScales& ss) {
        const uint4 h = raw16(blk);
        const float d = f16_bits_to_f32(h.x & 0xffffu) * prescale;
        const float dmin = f16_bits_to_f32(h.x >> 16) * prescale;
        uint32_t sc_lo, sc_hi, m_lo, m_hi;
        unpack_k_scales(h.y, h.z, h.w, sc_lo, sc_hi, m_lo, m_hi);
        const uint32_t sc = t < 2 ? sc_lo : sc_hi;
        const uint32_t mn = t < 2 ? m_lo : m_hi;
        const int shift = (t & 1) * 16;
        ss.v[0] = d * static_cast<float>((sc >> shift) & 0xffu);
        ss.v[1] = dmin * static_cast<float>((mn >> shift) & 0xffu);
        ss.v[2] = d * static_cast<float>((sc >> (shift + 8)) & 0xffu);
        ss.v[3] = dmin * static_cast<float>((mn >> (shift + 8)) & 0xffu);
    }
    __device__ static void step_with(const uint8_t* blk, int t, int h, float a0, float b0, float a1, float b1, Chunk (&out)[4]) {
        const uint4 w = raw16(blk + 16 + 32 * t + 16 * h);
        out[0] = chunk_from_bytes<Enc>(w.x & 0x0f0f0f0fu, w.y & 0x0f0f0f0fu, 0.0f, a0, b0);
        out[1] = chunk_from_bytes<Enc>(w.z & 0x0f0f0f0fu, w.w & 0x0f0f0f0fu, 0.0f, a0, b0);
        out[2] = chunk_from_bytes<Enc>((w.x >> 4) & 0x0f0f0f0fu, (w.y >> 4) & 0x0f0f0f0fu, 0.0f, a1, b1);
        out[3] = chunk_from_bytes<Enc>((w.z >> 4) & 0x0f0f0f0fu, (w.w >> 4) & 0x0f0f0f0fu, 0.0f, a1, b1);
    }
    __device__ static void step(const uint8_t* blk, const Scales& s, int t, int h, Chunk (&out)[4]) {
        step_with(blk, t, h, s.a[2 * t], s.b[2 * t], s.a[2 * t + 1], s.b[2 * t + 1], out);
    }
    __device__ static void step(const uint8_t* blk, const StepScales& ss, int t, int h, Chunk (&out)[4]) {
        step_with(blk, t, h, ss.v[0], ss.v[1], ss.v[2], ss.v[3], out);
    }
};

template <class Enc>
struct RowDequant<kQ5_K, Enc> {
    using Chunk = typename Enc::Chunk;
    // Largest |weight| the super-block can hold: |d| * 63 * 31 + |dmin| * 63.
    __device__ static float magnitude_bound(const uint8_t* blk) {
        const uint32_t h = ld_u32_a2(blk);
        return fabsf(f16_bits_to_f32(h & 0xffffu)) * 1953.0f + fabsf(f16_bits_to_f32(h >> 16)) * 63.0f;
    }
    using Scales = typename RowDequant<kQ4_K, Enc>::Scales;
    __device__ static void load_scales(const uint8_t* blk, Scales& s, float prescale) { RowDequant<kQ4_K, Enc>::load_scales(blk, s, prescale); }
    __device__ static int chunk_index(int h, int c) { return RowDequant<kQ4_K, Enc>::chunk_index(h, c); }
    __device__ static uint32_t lo5(uint32_t w, uint32_t hb, int g) { return (w & 0x0f0f0f0fu) | (((hb >> g) & 0x01010101u) << 4); }
    __device__ static uint32_t hi5(uint32_t w, uint32_t hb, int g) {
        return ((w >> 4) & 0x0f0f0f0fu) | (((hb >> g) & 0x01010101u) << 4);
    }
    __device__ static void step_with(const uint8_t* blk, int t, int h, float a0, float b0, float a1, float b1, Chunk (&out)[4]) {
        const uint4 w = raw16(blk + 48 + 32 * t + 16 * h);
        const uint4 hb = raw16(blk + 16 + 16 * h);
        const int g = 2 * t;
        out[0] = chunk_from_bytes<Enc>(lo5(w.x, hb.x, g), lo5(w.y, hb.y, g), 0.0f, a0, b0);
        out[1] = chunk_from_bytes<Enc>(lo5(w.z, hb.z, g), lo5(w.w, hb.w, g), 0.0f, a0, b0);
        out[2] = chunk_from_bytes<Enc>(hi5(w.x, hb.x, g + 1), hi5(w.y, hb.y, g + 1), 0.0f, a1, b1);
        out[3] = chunk_from_bytes<Enc>(hi5(w.z, hb.z, g + 1), hi5(w.w, hb.w, g + 1), 0.0f, a1, b1);
    }
    using StepScales = typename RowDequant<kQ4_K, Enc>::StepScales;
    __device__ static void load_step_scales(const uint8_t* blk, int t, float prescale, StepScales& ss) {
        RowDequant<kQ4_K, Enc>::load_step_scales(blk, t, prescale, ss);
    }
    __device__ static void step(const uint8_t* blk, const Scales& s, int t, int h, Chunk (&out)[4]) {
        step_with(blk, t, h, s.a[2 * t], s.b[2 * t], s.a[2 * t + 1], s.b[2 * t + 1], out);
    }
    __device__ static void step(const uint8_t* blk, const StepScales& ss, int t, int h, Chunk (&out)[4]) {
        step_with(blk, t, h, ss.v[0], ss.v[1], ss.v[2], ss.v[3], out);
    }
};

template <class Enc>
struct RowDequant<kQ6_K, Enc> {
    using Chunk = typename Enc::Chunk;
    // Largest |weight| the super-block can hold: |d| * 128 * 32.
    __device__ static float magnitude_bound(const uint8_t* blk) { return fabsf(f16_bits_to_f32(ld_u16(blk + 208))) * 4096.0f; }
    struct Scales { float a[16]; };
    __device__ static void load_scales(const uint8_t* blk, Scales& s, float prescale) {
        const float d = f16_bits_to_f32(ld_u16(blk + 208)) * prescale;
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
            const uint32_t pair = ld_u16(blk + 192 + i);
            s.a[i] = d * static_cast<float>(static_cast<int8_t>(pair & 0xffu));
            s.a[i + 1] = d * static_cast<float>(static_cast<int8_t>(pair >> 8));
        }
    }
    __device__ static int chunk_index(int h, int c) { return RowDequant<kQ4_K, Enc>::chunk_index(h, c); }
    // Step t covers groups 2t and 2t+1 = variants v, v+1 of chunk c = t/2 with v = 2*(t%2):
    // group 2t reads ql[c*64 + p], group 2t+1 reads ql[c*64 + 32 + p], low nibble when t is even,
    // high nibble when odd; both take two bits of qh[c*32 + p], at shifts 2v and 2v+2.
    __device__ static uint32_t q6(uint32_t l, uint32_t hb, int nib, int shift) {
        return ((l >> nib) & 0x0f0f0f0fu) | (((hb >> shift) & 0x03030303u) << 4);
    }
    struct StepScales { float v[4]; };   // d * scales[4t .. 4t+3]
    __device__ static void load_step_scales(const uint8_t* blk, int t, float prescale, StepScales& ss) {
        const float d = f16_bits_to_f32(ld_u16(blk + 208)) * prescale;
        const uint32_t lo = ld_u16(blk + 192 + 4 * t), hi = ld_u16(blk + 194 + 4 * t);
        ss.v[0] = d * static_cast<float>(static_cast<int8_t>(lo & 0xffu));
        ss.v[1] = d * static_cast<float>(static_cast<int8_t>(lo >> 8));
        ss.v[2] = d * static_cast<float>(static_cast<int8_t>(hi & 0xffu));
        ss.v[3] = d * static_cast<float>(static_cast<int8_t>(hi >> 8));
    }
    __device__ static void step(const uint8_t* blk, const Scales& s, int t, int h, Chunk (&out)[4]) {
        step_with(blk, t, h, h ? s.a[4 * t + 1] : s.a[4 * t], h ? s.a[4 * t + 3] : s.a[4 * t + 2], out);
    }
    __device__ static void step(const uint8_t* blk, const StepScales& ss, int t, int h, Chunk (&out)[4]) {
        step_with(blk, t, h, h ? ss.v[1] : ss.v[0], h ? ss.v[3] : ss.v[2], out);
    }
    __device__ static void step_with(const uint8_t* blk, int t, int h, float s0, float s1, Chunk (&out)[4]) {
        const int c = t >> 1;
        const int nib = (t & 1) * 4;
        const int v2 = (t & 1) * 4;  // 2 * variant of the first group
        const uint4 l0 = raw16_a2(blk + c * 64 + 16 * h);
        const uint4 l1 = raw16_a2(blk + c * 64 + 32 + 16 * h);
        const uint4 hb = raw16_a2(blk + 128 + c * 32 + 16 * h);
        out[0] = chunk_from_bytes<Enc>(q6(l0.x, hb.x, nib, v2), q6(l0.y, hb.y, nib, v2), 32.0f, s0, 0.0f);
        out[1] = chunk_from_bytes<Enc>(q6(l0.z, hb.z, nib, v2), q6(l0.w, hb.w, nib, v2), 32.0f, s0, 0.0f);
        out[2] = chunk_from_bytes<Enc>(q6(l1.x, hb.x, nib, v2 + 2), q6(l1.y, hb.y, nib, v2 + 2), 32.0f, s1, 0.0f);
        out[3] = chunk_from_bytes<Enc>(q6(l1.z, hb.z, nib, v2 + 2), q6(l1.w, hb.w, nib, v2 + 2), 32.0f, s1, 0.0f);
    }
};

template <class Enc>
struct RowDequant<kQ8_0, Enc> {
    using Chunk = typename Enc::Chunk;
    // Largest |weight| the super-block (eight 32-blocks) can hold.
    __device__ static float magnitude_bound(const uint8_t* blk) {
        float d = 0.0f;
#pragma unroll
        for (int b = 0; b < 8; ++b) d = fmaxf(d, fabsf(f16_bits_to_f32(ld_u16(blk + 34 * b))));
        return d * 128.0f;
    }
    struct Scales { float d[8]; };
    __device__ static void load_scales(const uint8_t* blk, Scales& s, float prescale) {
#pragma unroll
        for (int b = 0; b < 8; ++b) s.d[b] = f16_bits_to_f32(ld_u16(blk + 34 * b)) * prescale;
    }
    __device__ static int chunk_index(int h, int c) { return 4 * h + c; }
    struct StepScales { float v[4]; };   // d of blocks 2t and 2t+1
    __device__ static void load_step_scales(const uint8_t* blk, int t, float prescale, StepScales& ss) {
        ss.v[0] = f16_bits_to_f32(ld_u16(blk + 34 * (2 * t))) * prescale;
        ss.v[1] = f16_bits_to_f32(ld_u16(blk + 34 * (2 * t + 1))) * prescale;
        ss.v[2] = ss.v[3] = 0.0f;
    }
    __device__ static void step(const uint8_t* blk, const Scales& s, int t, int h, Chunk (&out)[4]) {
        step_with(blk, t, h, h ? s.d[2 * t + 1] : s.d[2 * t], out);
    }
    __device__ static void step(const uint8_t* blk, const StepScales& ss, int t, int h, Chunk (&out)[4]) {
        step_with(blk, t, h, h ? ss.v[1] : ss.v[0], out);
    }
    __device__ static void step_with(const uint8_t* blk, int t, int h, float d, Chunk (&out)[4]) {
        const uint8_t* q = blk + 34 * (2 * t + h) + 2;
        const uint4 w0 = raw16_a2(q);
        const uint4 w1 = raw16_a2(q + 16);
        out[0] = chunk_from_bytes<Enc>(w0.x ^ 0x80808080u, w0.y ^ 0x80808080u, 128.0f, d, 0.0f);
        out[1] = chunk_from_bytes<Enc>(w0.z ^ 0x80808080u, w0.w ^ 0x80808080u, 128.0f, d, 0.0f);
        out[2] = chunk_from_bytes<Enc>(w1.x ^ 0x80808080u, w1.y ^ 0x80808080u, 128.0f, d, 0.0f);
        out[3] = chunk_from_bytes<Enc>(w1.z ^ 0x80808080u, w1.w ^ 0x80808080u, 128.0f, d, 0.0f);
    }
};

}  // namespace ribn
