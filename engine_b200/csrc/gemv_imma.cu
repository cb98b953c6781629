// Dequant-fused GEMV for 1..8 activation rows per launch on the integer tensor-core instruction
// (mma.sync m16n8k32 u8 x s8 for Q4_K and Q5_K, m16n8k16 s8 x s8 for Q6_K; s32 accumulate).
//
//   y[m][n] = sum_k dequant(W[n][k]) * x[m][k]
//
// Why a second narrow kernel.  The f16 kernel of gemv_mma.cu turns every pair of quants into a half2 with one
// logic op and one HFMA2 and is bound by instruction issue (about 3.8 thread instructions per weight, the logic
// pipe half busy) at half of the HBM rate.  Here the packed nibbles ARE the operand: (word & 0x0f0f0f0f) is four
// unsigned 8-bit quants, so a weight costs 3/8 of a logic instruction, and nothing is multiplied before the
// tensor core.  What makes that possible:
//   * the activations are 22-bit integers X = rint(x * 2^e) per (member, super-block), 2^e the power of two
//     that brings the largest of the 256 magnitudes into [2^20, 2^21), stored as three 8-bit planes
//     X = 2^14 p2 + 2^7 p1 + p0 (p2 signed, p1 and p0 in 0..127).  The planes of a member are COLUMNS of the
//     same instruction (a column group is two members x [p0 p1 p2 0]), so two members cost one mma per
//     sub-block of 32 weights and eight members four;
//   * one m16n8k32 covers exactly one sub-block (the K order inside it is free, the activations are stored in
//     the order the bytes come in), so its s32 result is multiplied by the 6-bit sub-block scale as an
//     INTEGER (one IMAD per accumulator, on the pipe the unpacking does not use) and the sums over the eight
//     sub-blocks stay exact; d * 2^-e is applied in f32 once per super-block and row;
//   * the minima term (dmin * m_j * sum of the sub-block's activations) is one f16 mma per super-block, as in
//     the f16 kernel: A = the eight minima, B = the block sums as f16 hi + lo.
// Q6_K: scales cover 16 weights, so the instruction is the k16 one; a quant is six bits from two places
// (a nibble and two bits, merged with three logic ops per four weights), and q - 32 is made a signed byte in two
// more (set the top bit, subtract 32 without a borrow between bytes, clear the top bit again), which needs no
// block sums.  Super-blocks are 210 bytes: every second one starts two bytes off a word boundary, and its words
// are funnel-shifted out of two aligned loads.
// Rounding: the weights are exact; an activation carries 2^-22 of its super-block's largest magnitude, all
// integer sums are exact, and a row's result does not depend on the rows launched with it.
//
// Reference counterparts: q*_gemv_warp / _warp_batch (crates/nvidia/src/kernels/quantized/q4_k.cu:103-258,
// q5_k.cu) for the contract; rms_norm (crates/nvidia/src/model_ops.rs:106-147) and silu_mul
// (model_ops.rs:316-328) for the fused prologues.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "formats.cuh"
#include "internal.h"
#include "pack_activations.cuh"
#include "pipeline.cuh"
#include "tc_host.h"
#include "tcgen05.cuh"
#include "unpack.cuh"

namespace ribn {
namespace {

constexpr int kWarps = 8;                      // consumer warps = super-blocks per stage
constexpr int kConsumers = kWarps * 32;
constexpr int kThreads = kConsumers + 32;      // + the producer warp
constexpr int kTileRows = 16;                  // weight rows per tile (the M of m16n8k32)
constexpr int kMaxStages = 8;
constexpr int kMaxMembers = 8;                 // four column groups of two members
constexpr int kSliceBytes = 768;               // image bytes per (member, super-block): 8 sub-blocks x 3 planes x 32
constexpr int kZeroBytes = 1024;               // zeros the fourth column of every member (and absent members) read

template <uint32_t FMT>
struct ImmaPlan {
    static constexpr int kSbBytes = Format<FMT>::kBytes;
    // Super-blocks per TMA box.  Q4_K / Q5_K: two, a row pitch of 288 / 352 bytes = 8 or 24 (mod 32) words, so that the
    // 64-bit loads of four rows x four lanes fall on 32 different banks.  Q6_K: eight (1680 bytes, the smallest multiple of
    // 210 that is a multiple of 16) = 4 (mod 32) words: the 32-bit loads of eight rows x four lanes fall on 32 banks.
    static constexpr int kBoxSb = FMT == kQ6_K ? 8 : 2;
    static constexpr int kBoxes = kWarps / kBoxSb;
    static constexpr int kRowPitch = kBoxSb * kSbBytes;
    static constexpr int kBoxBytes = kTileRows * kRowPitch;
    static constexpr int kStageBytes = kBoxes * kBoxBytes;
    static_assert(kRowPitch % 16 == 0 && kBoxBytes % 128 == 0, "TMA box: 16-byte rows, 128-byte aligned destination");
    static_assert((kSbBytes * kBoxSb / 8) % 2 == 0, "TMA x coordinate of every box on a 16-byte boundary");
};

struct ImmaParams {
    const void* x;              // [members][k] (swiglu: [members][2k]) f32 or bf16; unused when `image` is set
    int x_bf16;
    int mode;                   // 0 plain, 1 RMSNorm first, 2 silu(gate) * up
    const float* norm_weight;
    float eps;
    const uint8_t* image;       // activation image made by the pre-pass (layout below), or null: convert here
    void* y;
    int y_bf16;
    int accumulate;
    int k, n, nsb, members, stages;
    int* status;
};

// ---------------------------------------------------------------- activation image
// Per call, in shared memory (and in global memory when a pre-pass makes it):
//   planes [members][nsb][8 sub-blocks][p0 32 B | p1 32 B | p2 32 B] int8, bytes in element order.  The 64-bit
//          fragment loads of a half-warp (one member: three planes and the zero column, four lanes each) then
//          cover 96 contiguous bytes plus 32 bytes of the zero area placed 96 bytes further on: 32 banks;
//   sums   [members][nsb][16] f16: (sum of the sub-block's 32 integers) / 2^11 as f16 hi (8 values) then f16 lo (8);
//   scale  [nsb][8] f32: 2^-e per (super-block, member), 0 for an all-zero slice, NaN when it holds a non-finite value.
__host__ __device__ inline size_t image_plane_bytes(int members, int nsb) { return static_cast<size_t>(members) * nsb * kSliceBytes; }
__host__ __device__ inline size_t image_sums_bytes(int members, int nsb) { return static_cast<size_t>(members) * nsb * 32; }
__host__ __device__ inline size_t image_scale_bytes(int nsb) { return static_cast<size_t>(nsb) * 32; }
__host__ __device__ inline size_t image_bytes(int members, int nsb) {
    return image_plane_bytes(members, nsb) + image_sums_bytes(members, nsb) + image_scale_bytes(nsb);
}

// Lane `lane` of a warp loads elements 8 lane .. 8 lane + 7 of super-block sb of member row m, prologue applied.
__device__ __forceinline__ void load_slice(const ImmaParams& p, int m, int sb, int lane, float inv_rms, float (&v)[8]) {
    const int k0 = sb * kSuperBlock + lane * 8;
    const size_t row_elements = static_cast<size_t>(p.k) * (p.mode == 2 ? 2 : 1);
    const AnyRow row{static_cast<const uint8_t*>(p.x) + static_cast<size_t>(m) * row_elements * (p.x_bf16 ? 2 : 4), p.x_bf16};
    load_row8(row + k0, v);
    if (p.mode == 2) {
        float u[8];
        load_row8(row + (p.k + k0), u);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (v[j] / (1.0f + expf(-v[j]))) * u[j];
    } else if (p.mode == 1) {
        float g[8];
        load_x8<float>(p.norm_weight + k0, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = v[j] * inv_rms * g[j];
    }
}

// The warp's 256 values -> three int8 planes, block sums and the slice's factor (generic pointers: shared or global).
__device__ __forceinline__ void store_slice(int m, int sb, int lane, float (&v)[8], uint8_t* planes_row, __half* sums_row, float* scale) {
    // Largest magnitude in one warp reduction: non-negative floats order like their bit patterns, and infinities
    // and NaNs (0x7f800000 and above) come out on top, which is how they are detected.
    uint32_t biggest = 0u;
#pragma unroll
    for (int j = 0; j < 8; ++j) biggest = max(biggest, __float_as_uint(fabsf(v[j])));
    biggest = __reduce_max_sync(0xffffffffu, biggest);
    const bool bad = biggest >= 0x7f800000u;
    // amax * 2^e in [2^20, 2^21); e clamped so that both 2^e and 2^-e are normal numbers
    int e = 20 - (static_cast<int>(biggest >> 23) - 127);
    e = max(-100, min(100, e));
    float down = __uint_as_float(static_cast<uint32_t>(127 + e) << 23);
    float up = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
    if (biggest == 0u) up = 0.0f;
    if (bad) {
        down = 0.0f;
        up = __int_as_float(0x7fc00000);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.0f;
    }
    int xi[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        xi[j] = max(-2097151, min(2097151, __float2int_rn(v[j] * down)));
        sum += xi[j];
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    const int j = lane >> 2, t = lane & 3;
    uint8_t* slot = planes_row + static_cast<size_t>(sb) * kSliceBytes + j * 96 + 8 * t;
    *reinterpret_cast<uint2*>(slot) = make_uint2(pack4(xi[0] & 127, xi[1] & 127, xi[2] & 127, xi[3] & 127),
                                                 pack4(xi[4] & 127, xi[5] & 127, xi[6] & 127, xi[7] & 127));
    *reinterpret_cast<uint2*>(slot + 32) = make_uint2(pack4((xi[0] >> 7) & 127, (xi[1] >> 7) & 127, (xi[2] >> 7) & 127, (xi[3] >> 7) & 127),
                                                      pack4((xi[4] >> 7) & 127, (xi[5] >> 7) & 127, (xi[6] >> 7) & 127, (xi[7] >> 7) & 127));
    *reinterpret_cast<uint2*>(slot + 64) = make_uint2(pack4(xi[0] >> 14, xi[1] >> 14, xi[2] >> 14, xi[3] >> 14),
                                                      pack4(xi[4] >> 14, xi[5] >> 14, xi[6] >> 14, xi[7] >> 14));
    if (t == 0) {
        const float s = static_cast<float>(sum) * 0.00048828125f;   // 2^-11: below the f16 range's top
        const __half hi = __float2half_rn(s);
        sums_row[sb * 16 + j] = hi;
        sums_row[sb * 16 + 8 + j] = __float2half_rn(s - __half2float(hi));
    }
    if (lane == 0) scale[sb * 8 + m] = up;
}

// sum of squares of member row m over the whole K range, by `threads` threads with index tid; the caller reduces.
__device__ __forceinline__ float partial_square_sum(const ImmaParams& p, int m, int tid, int threads) {
    const AnyRow row{static_cast<const uint8_t*>(p.x) + static_cast<size_t>(m) * p.k * (p.x_bf16 ? 2 : 4), p.x_bf16};
    float acc = 0.0f;
    for (int c = tid; c < p.k / 8; c += threads) {
        float v[8];
        load_row8(row + c * 8, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc = fmaf(v[j], v[j], acc);
    }
    return acc;
}

// D = A(16x32, u8, row) * B(32x8, s8, col), s32.  Lane (g = lane / 4, t = lane % 4) holds
//   a0: row g, K slots 4t..4t+3     a1: row g+8, same slots     a2: row g, K slots 16+4t..     a3: row g+8
//   b0: column g, K slots 4t..4t+3  b1: column g, K slots 16+4t..
//   c0,c1: row g, columns 2t,2t+1   c2,c3: row g+8, columns 2t,2t+1
__device__ __forceinline__ void imma_zero(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void hmma_zero(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// D = A(16x16, s8, row) * B(16x8, s8, col), s32.  Lane (g, t): a0 row g, a1 row g+8, K slots 4t..4t+3; b0 column g, the same slots.
__device__ __forceinline__ void imma16_zero(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// A 32-bit word of shared memory at `address`, which is two bytes past a word boundary when ODD.
template <bool ODD>
__device__ __forceinline__ uint32_t lds32_shifted(uint32_t address) {
    if (!ODD) return lds32(address);
    return __funnelshift_r(lds32(address - 2), lds32(address + 2), 16);
}

// Per-lane shared addresses at the super-block the warp works on.  Column g of column group q is plane g & 3 of
// member 2q + (g >> 2); the fourth plane and members the launch does not have are read from the zero area.
template <int GROUPS>
struct LaneX {
    uint32_t x[GROUPS];      // the lane's 8 bytes of sub-block j in group q: x[q] + 96 j
    uint32_t step[GROUPS];   // bytes from one super-block to the next (0 for lanes that read zeros)
    uint32_t sums;           // block sums of member g (the minima instruction has one column per member)
    uint32_t scale;          // the eight factors of the super-block

    __device__ __forceinline__ void advance(int superblocks) {
#pragma unroll
        for (int q = 0; q < GROUPS; ++q) x[q] += static_cast<uint32_t>(superblocks) * step[q];
        sums += static_cast<uint32_t>(superblocks * 32);
        scale += static_cast<uint32_t>(superblocks * 32);
    }
};

template <int J>
__device__ __forceinline__ uint32_t scale_byte(uint32_t lo, uint32_t hi) {
    return __byte_perm(J < 4 ? lo : hi, 0u, 0x4440u + (J & 3));
}

// Fifth bit of sub-block J from the lane's fifth-bit word (bit J of every byte) into bit 4 of every byte of `nibbles`.
template <int J>
__device__ __forceinline__ uint32_t with_fifth(uint32_t nibbles, uint32_t h) {
    const uint32_t moved = J < 4 ? (h << (4 - J)) : (h >> (J - 4));
    return and_or(moved, 0x10101010u, nibbles);
}

// One sub-block: the four A words are ready; multiply by every column group, then fold the 6-bit scales in as integers.
template <int J, int GROUPS>
__device__ __forceinline__ void subblock(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, const LaneX<GROUPS>& lx, uint32_t sc_lo0,
                                         uint32_t sc_hi0, uint32_t sc_lo1, uint32_t sc_hi1, int (&total)[GROUPS][4]) {
    const int s0 = static_cast<int>(scale_byte<J>(sc_lo0, sc_hi0)), s1 = static_cast<int>(scale_byte<J>(sc_lo1, sc_hi1));
#pragma unroll
    for (int q = 0; q < GROUPS; ++q) {
        const uint2 b = lds64_at<96 * J>(lx.x[q]);
        int c[4];
        imma_zero(c, a0, a1, a2, a3, b.x, b.y);
        total[q][0] += s0 * c[0];
        total[q][1] += s0 * c[1];
        total[q][2] += s1 * c[2];
        total[q][3] += s1 * c[3];
    }
}

// One super-block of rows g (at p0) and g + 8 (at p1).
//   acc[q][0], acc[q][1]: rows g, g + 8 of member 2q + (t >> 1), the share of planes p0, p1 (t even) or of plane p2 (t odd);
//   mins[0..3]: the minima term of members 2t, 2t + 1 for row g, then for row g + 8.
template <uint32_t FMT, int GROUPS>
__device__ __forceinline__ void superblock(uint32_t p0, uint32_t p1, const LaneX<GROUPS>& lx, int t, float (&acc)[GROUPS][2], float (&mins)[4]) {
    constexpr uint32_t kQuantOffset = FMT == kQ4_K ? 16 : 48;   // Q5_K: 32 fifth-bit bytes between the header and the nibbles
    const uint4 h0 = lds128(p0), h1 = lds128(p1);   // d | dmin, 12 scale bytes
    uint32_t sc_lo0, sc_hi0, m_lo0, m_hi0, sc_lo1, sc_hi1, m_lo1, m_hi1;
    unpack_k_scales(h0.y, h0.z, h0.w, sc_lo0, sc_hi0, m_lo0, m_hi0);
    unpack_k_scales(h1.y, h1.z, h1.w, sc_lo1, sc_hi1, m_lo1, m_hi1);
    float cm[4];
    {
        // minimum term: A = the eight 6-bit minima, twice (K slots 0..7 and 8..15); B = column g: member g's block
        // sums, f16 hi in slots 0..7 and f16 lo in slots 8..15
        const uint32_t a0 = byte_pair_half2((t & 2) ? m_hi0 : m_lo0, (t & 1) != 0);
        const uint32_t a1 = byte_pair_half2((t & 2) ? m_hi1 : m_lo1, (t & 1) != 0);
        const uint32_t b0 = lds32(lx.sums + t * 4);
        const uint32_t b1 = lds32(lx.sums + 16 + t * 4);
        hmma_zero(cm, a0, a1, a0, a1, b0, b1);
    }
    uint2 f0 = make_uint2(0u, 0u), f1 = f0;
    if (FMT == kQ5_K) {
        f0 = lds64(p0 + 16 + 8 * t);
        f1 = lds64(p1 + 16 + 8 * t);
    }
    int total[GROUPS][4];
#pragma unroll
    for (int q = 0; q < GROUPS; ++q)
#pragma unroll
        for (int i = 0; i < 4; ++i) total[q][i] = 0;
#define RIBN_IMMA_PAIR(G)                                                                                                      \
    {                                                                                                                          \
        const uint2 q0 = lds64(p0 + kQuantOffset + 32 * (G) + 8 * t), q1 = lds64(p1 + kQuantOffset + 32 * (G) + 8 * t);  \
        uint32_t a0 = q0.x & 0x0f0f0f0fu, a1 = q1.x & 0x0f0f0f0fu, a2 = q0.y & 0x0f0f0f0fu, a3 = q1.y & 0x0f0f0f0fu;           \
        if (FMT == kQ5_K) {                                                                                                    \
            a0 = with_fifth<2 * (G)>(a0, f0.x);                                                                                \
            a1 = with_fifth<2 * (G)>(a1, f1.x);                                                                                \
            a2 = with_fifth<2 * (G)>(a2, f0.y);                                                                                \
            a3 = with_fifth<2 * (G)>(a3, f1.y);                                                                                \
        }                                                                                                                      \
        subblock<2 * (G), GROUPS>(a0, a1, a2, a3, lx, sc_lo0, sc_hi0, sc_lo1, sc_hi1, total);                                  \
        a0 = (q0.x >> 4) & 0x0f0f0f0fu;                                                                                        \
        a1 = (q1.x >> 4) & 0x0f0f0f0fu;                                                                                        \
        a2 = (q0.y >> 4) & 0x0f0f0f0fu;                                                                                        \
        a3 = (q1.y >> 4) & 0x0f0f0f0fu;                                                                                        \
        if (FMT == kQ5_K) {                                                                                                    \
            a0 = with_fifth<2 * (G) + 1>(a0, f0.x);                                                                            \
            a1 = with_fifth<2 * (G) + 1>(a1, f1.x);                                                                            \
            a2 = with_fifth<2 * (G) + 1>(a2, f0.y);                                                                            \
            a3 = with_fifth<2 * (G) + 1>(a3, f1.y);                                                                            \
        }                                                                                                                      \
        subblock<2 * (G) + 1, GROUPS>(a0, a1, a2, a3, lx, sc_lo0, sc_hi0, sc_lo1, sc_hi1, total);                              \
    }
    RIBN_IMMA_PAIR(0)
    RIBN_IMMA_PAIR(1)
    RIBN_IMMA_PAIR(2)
    RIBN_IMMA_PAIR(3)
#undef RIBN_IMMA_PAIR
    const float d0 = f16_bits_to_f32(h0.x & 0xffffu), dm0 = f16_bits_to_f32(h0.x >> 16);
    const float d1 = f16_bits_to_f32(h1.x & 0xffffu), dm1 = f16_bits_to_f32(h1.x >> 16);
    // Columns 2t, 2t+1 of a group: planes (p0, p1) of its first or second member for t = 0, 2; (p2, zeros) for t = 1, 3.
    const float weight = (t & 1) ? 16384.0f : 1.0f;
#pragma unroll
    for (int q = 0; q < GROUPS; ++q) {
        const float xs = __uint_as_float(lds32(lx.scale + 8 * q + 4 * (t >> 1))) * weight;
        const float v0 = fmaf(128.0f, static_cast<float>(total[q][1]), static_cast<float>(total[q][0]));
        const float v1 = fmaf(128.0f, static_cast<float>(total[q][3]), static_cast<float>(total[q][2]));
        acc[q][0] = fmaf(d0 * xs, v0, acc[q][0]);
        acc[q][1] = fmaf(d1 * xs, v1, acc[q][1]);
    }
    // the minima instruction: columns 2t, 2t+1 = members 2t, 2t+1; its sums were divided by 2^11
    const uint2 xm = lds64(lx.scale + 8 * t);
    const float xa = __uint_as_float(xm.x) * -2048.0f, xb = __uint_as_float(xm.y) * -2048.0f;
    mins[0] = fmaf(dm0 * xa, cm[0], mins[0]);
    mins[1] = fmaf(dm0 * xb, cm[1], mins[1]);
    mins[2] = fmaf(dm1 * xa, cm[2], mins[2]);
    mins[3] = fmaf(dm1 * xb, cm[3], mins[3]);
}

// ---- Q6_K.  Block b = 8 n2 + 2 v + h of the sixteen 16-weight blocks: positions 128 n2 + 32 v + 16 h .. + 15, low nibbles
// in ql byte 64 n2 + 32 (v & 1) + 16 h + l (the low half of the byte for v < 2, the high half above), two more bits in
// qh byte 32 n2 + 16 h + l at bit 2 v; lane t takes l = 4t .. 4t + 3 of every block, one word of each.
template <int V>
__device__ __forceinline__ uint32_t q6_signed_bytes(uint32_t ql_word, uint32_t qh_word) {
    // 128 + nibble in every byte, then bits 4..5 from qh: 128 + q; minus 32 without a borrow between bytes; top bit off again
    const uint32_t nibbles = and_or(V < 2 ? ql_word : (ql_word >> 4), 0x0f0f0f0fu, 0x80808080u);
    const uint32_t moved = V == 0 ? (qh_word << 4) : V == 1 ? (qh_word << 2) : V == 2 ? qh_word : (qh_word >> 2);
    return (and_or(moved, 0x30303030u, nibbles) - 0x20202020u) ^ 0x80808080u;
}

// Byte I of `word` as a sign-extended integer: prmt with the replicate-sign bit of the selector set for the three upper
// bytes (the __byte_perm intrinsic keeps only the byte index of a selector nibble).
template <int I>
__device__ __forceinline__ int signed_byte(uint32_t word) {
    int value;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(value) : "r"(word), "r"(0u), "n"(I | ((I | 8) << 4) | ((I | 8) << 8) | ((I | 8) << 12)));
    return value;
}

template <int B, int GROUPS>
__device__ __forceinline__ void block_q6(uint32_t a0, uint32_t a1, const LaneX<GROUPS>& lx, uint32_t scales0, uint32_t scales1,
                                         int (&total)[GROUPS][4]) {
    const int s0 = signed_byte<B & 3>(scales0), s1 = signed_byte<B & 3>(scales1);
#pragma unroll
    for (int q = 0; q < GROUPS; ++q) {
        uint32_t b0;
        asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(b0) : "r"(lx.x[q]), "n"(96 * (B >> 1) + 16 * (B & 1)));
        int c[4];
        imma16_zero(c, a0, a1, b0);
        total[q][0] += s0 * c[0];
        total[q][1] += s0 * c[1];
        total[q][2] += s1 * c[2];
        total[q][3] += s1 * c[3];
    }
}

// The two blocks that share the ql word (N2, VLOW, H): block B = 8 N2 + 2 VLOW + H from its low nibbles, block B + 4 from
// its high nibbles.
template <int N2, int H, int VLOW, int GROUPS, bool ODD>
__device__ __forceinline__ void blocks_q6(uint32_t p0, uint32_t p1, uint32_t qh0, uint32_t qh1, uint32_t lane_bytes, const LaneX<GROUPS>& lx,
                                          const uint32_t (&sc0)[4], const uint32_t (&sc1)[4], int (&total)[GROUPS][4]) {
    constexpr int B = 8 * N2 + 2 * VLOW + H;
    const uint32_t ql0 = lds32_shifted<ODD>(p0 + 64 * N2 + 32 * VLOW + 16 * H + lane_bytes);
    const uint32_t ql1 = lds32_shifted<ODD>(p1 + 64 * N2 + 32 * VLOW + 16 * H + lane_bytes);
    block_q6<B, GROUPS>(q6_signed_bytes<VLOW>(ql0, qh0), q6_signed_bytes<VLOW>(ql1, qh1), lx, sc0[B >> 2], sc1[B >> 2], total);
    block_q6<B + 4, GROUPS>(q6_signed_bytes<VLOW + 2>(ql0, qh0), q6_signed_bytes<VLOW + 2>(ql1, qh1), lx, sc0[(B + 4) >> 2], sc1[(B + 4) >> 2],
                            total);
}

// The four blocks that share the qh word (N2, H).
template <int N2, int H, int GROUPS, bool ODD>
__device__ __forceinline__ void quarter_q6(uint32_t p0, uint32_t p1, uint32_t lane_bytes, const LaneX<GROUPS>& lx, const uint32_t (&sc0)[4],
                                           const uint32_t (&sc1)[4], int (&total)[GROUPS][4]) {
    const uint32_t qh0 = lds32_shifted<ODD>(p0 + 128 + 32 * N2 + 16 * H + lane_bytes);
    const uint32_t qh1 = lds32_shifted<ODD>(p1 + 128 + 32 * N2 + 16 * H + lane_bytes);
    blocks_q6<N2, H, 0, GROUPS, ODD>(p0, p1, qh0, qh1, lane_bytes, lx, sc0, sc1, total);
    blocks_q6<N2, H, 1, GROUPS, ODD>(p0, p1, qh0, qh1, lane_bytes, lx, sc0, sc1, total);
}

// One Q6_K super-block of rows g (at p0) and g + 8 (at p1); ODD: the super-block starts two bytes past a word boundary.
template <int GROUPS, bool ODD>
__device__ __forceinline__ void superblock_q6(uint32_t p0, uint32_t p1, const LaneX<GROUPS>& lx, int t, float (&acc)[GROUPS][2]) {
    int total[GROUPS][4];
#pragma unroll
    for (int q = 0; q < GROUPS; ++q)
#pragma unroll
        for (int i = 0; i < 4; ++i) total[q][i] = 0;
    const uint32_t lane_bytes = 4u * static_cast<uint32_t>(t);
    // the sixteen scale bytes of each row: word i holds blocks 4i .. 4i + 3
    uint32_t sc0[4], sc1[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        sc0[i] = lds32_shifted<ODD>(p0 + 192 + 4 * i);
        sc1[i] = lds32_shifted<ODD>(p1 + 192 + 4 * i);
    }
    quarter_q6<0, 0, GROUPS, ODD>(p0, p1, lane_bytes, lx, sc0, sc1, total);
    quarter_q6<0, 1, GROUPS, ODD>(p0, p1, lane_bytes, lx, sc0, sc1, total);
    quarter_q6<1, 0, GROUPS, ODD>(p0, p1, lane_bytes, lx, sc0, sc1, total);
    quarter_q6<1, 1, GROUPS, ODD>(p0, p1, lane_bytes, lx, sc0, sc1, total);
    const float d0 = f16_bits_to_f32(lds_u16(p0 + 208)), d1 = f16_bits_to_f32(lds_u16(p1 + 208));
    const float weight = (t & 1) ? 16384.0f : 1.0f;
#pragma unroll
    for (int q = 0; q < GROUPS; ++q) {
        const float xs = __uint_as_float(lds32(lx.scale + 8 * q + 4 * (t >> 1))) * weight;
        const float v0 = fmaf(128.0f, static_cast<float>(total[q][1]), static_cast<float>(total[q][0]));
        const float v1 = fmaf(128.0f, static_cast<float>(total[q][3]), static_cast<float>(total[q][2]));
        acc[q][0] = fmaf(d0 * xs, v0, acc[q][0]);
        acc[q][1] = fmaf(d1 * xs, v1, acc[q][1]);
    }
}

// ---------------------------------------------------------------- the kernel
// Shared-memory plan: [ring: stages x stage][zeros 1 KiB][image: planes | sums | scale][red: 2 x 8 warps x 128 f32]
//                     [norm: 9 x 8 f32][barriers]
__host__ __device__ inline size_t imma_fixed_bytes(int members, int nsb) {
    return 128 /*alignment*/ + kZeroBytes + image_bytes(members, nsb) + 2 * kWarps * 128 * 4 + (kWarps + 1) * kMaxMembers * 4 + (2 * kMaxStages + 2) * 8;
}

template <uint32_t FMT, int GROUPS>
__global__ void __launch_bounds__(kThreads, 2) gemv_imma_kernel(const __grid_constant__ CUtensorMap wmap, const ImmaParams p) {
    using P = ImmaPlan<FMT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((128u - (smem_addr(smem_raw) & 127u)) & 127u);
    uint8_t* ring = smem;
    uint8_t* zeros = ring + static_cast<size_t>(p.stages) * P::kStageBytes;
    uint8_t* image = zeros + kZeroBytes;
    uint8_t* planes = image;
    __half* sums = reinterpret_cast<__half*>(planes + image_plane_bytes(p.members, p.nsb));
    float* scale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sums) + image_sums_bytes(p.members, p.nsb));
    float* red = scale + static_cast<size_t>(p.nsb) * 8;
    float* norm = red + 2 * kWarps * 128;
    uint64_t* full = reinterpret_cast<uint64_t*>(norm + (kWarps + 1) * kMaxMembers);
    uint64_t* empty = full + kMaxStages;
    uint64_t* image_bar = empty + kMaxStages;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int stages = p.stages;
    pdl_launch_dependents();
    // The producer warp initialises the barriers and goes straight on to request weights; the consumers only
    // need to know that the barriers exist before their first wait (named barrier 2: they sync, the producer arrives).
    if (warp == kWarps) {
        if (lane == 0) {
            tma_prefetch_descriptor(&wmap);
            for (int s = 0; s < stages; ++s) {
                mbar_init(&full[s], 1);
                mbar_init(&empty[s], kWarps);
            }
            mbar_init(image_bar, 1);
            mbar_fence_init();
        }
        __syncwarp();
        asm volatile("bar.arrive 2, %0;" ::"n"(kThreads) : "memory");
    }

    const int tiles_total = (p.n + kTileRows - 1) / kTileRows;
    const int tile_begin = static_cast<int>(static_cast<long long>(tiles_total) * blockIdx.x / gridDim.x);
    const int tile_end = static_cast<int>(static_cast<long long>(tiles_total) * (blockIdx.x + 1) / gridDim.x);
    const int tiles = tile_end - tile_begin;
    const int chunks = (p.nsb + kWarps - 1) / kWarps;
    const int total = tiles * chunks;
    bool ok = true;

    if (warp == kWarps) {
        // ---------------- producer warp: the weight stream does not depend on the activations ----------------
        if (lane == 0) {
            bool image_requested = p.image == nullptr;
            const int prefetch = min(total, stages);
            auto request_image = [&]() {
                // The image is the previous kernel's output; the first ring-full of weights is requested before it.
                pdl_wait_prior();
                const uint32_t bytes = static_cast<uint32_t>(image_bytes(p.members, p.nsb));
                mbar_arrive_expect_tx(image_bar, bytes);
                uint32_t done = 0;
                while (done < bytes) {
                    const uint32_t part = min(bytes - done, 32768u);
                    bulk_copy_g2s(image + done, p.image + done, part, image_bar);
                    done += part;
                }
                image_requested = true;
            };
            if (total == 0 && !image_requested) request_image();
#pragma unroll 1
            for (int it = 0; it < total; ++it) {
                const int s = it % stages;
                const int use = it / stages;
                if (use > 0 && !mbar_wait_bounded_hint(&empty[s], (use - 1) & 1, 2000u)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    break;
                }
                const int tile = it / chunks;
                const int chunk = it - tile * chunks;
                const int row0 = (tile_begin + tile) * kTileRows;
                const int sbs = min(kWarps, p.nsb - chunk * kWarps);
                const int boxes = (sbs + P::kBoxSb - 1) / P::kBoxSb;
                mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(boxes * P::kBoxBytes));
                for (int b = 0; b < boxes; ++b)
                    tma_load_2d(ring + static_cast<size_t>(s) * P::kStageBytes + b * P::kBoxBytes, &wmap,
                                (chunk * kWarps + b * P::kBoxSb) * P::kSbBytes / 8, row0, &full[s]);
                if (it == prefetch - 1 && !image_requested) request_image();
            }
        }
    } else {
        // ---------------- consumers ----------------
        const int g = lane >> 2, t = lane & 3;
        named_barrier_sync(2, kThreads);
        // 256 consumers x 4 bytes = the zero area, in place (and visible to every warp) before the wait for the previous
        // kernel ends: after that wait a warp only needs what it converts itself
        reinterpret_cast<uint32_t*>(zeros)[threadIdx.x] = 0u;
        named_barrier_sync(1, kConsumers);
        pdl_wait_prior();   // the activations may be the previous kernel's output, and y may still be read by it
        const int owned_slices = p.nsb > warp ? (p.nsb - warp + kWarps - 1) / kWarps : 0;
        if (p.image == nullptr && p.mode == 1 && p.members == 1 && p.nsb <= 2 * kWarps) {
            // One row of at most sixteen super-blocks to normalise (a decode step's projections): every lane keeps its
            // share of the warp's one or two slices in registers, so the row and the norm weights are read once -- one
            // round trip to memory instead of three.  Sums run in the order of the general path below (same bits).
            const AnyRow row{static_cast<const uint8_t*>(p.x), p.x_bf16};
            float v[2][8], gain[2][8];
            float part = 0.0f;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (i < owned_slices) {
                    const int k0 = (warp + i * kWarps) * kSuperBlock + lane * 8;
                    load_row8(row + k0, v[i]);
                    load_x8<float>(p.norm_weight + k0, gain[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
                if (i < owned_slices)
#pragma unroll
                    for (int j = 0; j < 8; ++j) part = fmaf(v[i][j], v[i][j], part);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            if (lane == 0) norm[warp * kMaxMembers] = part;
            named_barrier_sync(1, kConsumers);
            float totalsq = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) totalsq += norm[w * kMaxMembers];
            const float inv_rms = 1.0f / sqrtf(totalsq / static_cast<float>(p.k) + p.eps);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (i < owned_slices) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[i][j] = v[i][j] * inv_rms * gain[i][j];
                    store_slice(0, warp + i * kWarps, lane, v[i], planes, sums, scale);
                }
            }
            __syncwarp();   // a warp reads only the super-blocks it converted itself
        } else if (p.image == nullptr) {
            // norm[64 + m] = 1 / rms of member row m when RMSNorm is asked for
            if (p.mode == 1) {
                for (int m = 0; m < p.members; ++m) {
                    float part = partial_square_sum(p, m, static_cast<int>(threadIdx.x), kConsumers);
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                    if (lane == 0) norm[warp * kMaxMembers + m] = part;
                }
                named_barrier_sync(1, kConsumers);
                if (threadIdx.x < kMaxMembers) {
                    float totalsq = 0.0f;
#pragma unroll
                    for (int w = 0; w < kWarps; ++w) totalsq += norm[w * kMaxMembers + threadIdx.x];
                    norm[kWarps * kMaxMembers + threadIdx.x] = 1.0f / sqrtf(totalsq / static_cast<float>(p.k) + p.eps);
                }
                named_barrier_sync(1, kConsumers);
            }
            // The warp's slices (super-blocks warp, warp + 8, ... of every member), two loads in flight.
            const float* inv_rms = norm + kWarps * kMaxMembers;
            const int slices = owned_slices * p.members;
#pragma unroll 1
            for (int i = 0; i < slices; i += 2) {
                const int sb0 = warp + (i / p.members) * kWarps, m0 = i % p.members;
                const bool second = i + 1 < slices;
                const int i1 = second ? i + 1 : i;
                const int sb1 = warp + (i1 / p.members) * kWarps, m1 = i1 % p.members;
                float v0[8], v1[8];
                load_slice(p, m0, sb0, lane, p.mode == 1 ? inv_rms[m0] : 1.0f, v0);
                load_slice(p, m1, sb1, lane, p.mode == 1 ? inv_rms[m1] : 1.0f, v1);
                store_slice(m0, sb0, lane, v0, planes + static_cast<size_t>(m0) * p.nsb * kSliceBytes, sums + static_cast<size_t>(m0) * p.nsb * 16, scale);
                if (second)
                    store_slice(m1, sb1, lane, v1, planes + static_cast<size_t>(m1) * p.nsb * kSliceBytes, sums + static_cast<size_t>(m1) * p.nsb * 16,
                                scale);
            }
            __syncwarp();   // a warp reads only the super-blocks it converted itself
        } else if (!mbar_wait_bounded(image_bar, 0)) {
            atomicExch(p.status, kDeviceWaitTimeout);
            ok = false;
        }

        LaneX<GROUPS> lx;
        {
#pragma unroll
            for (int q = 0; q < GROUPS; ++q) {
                const int member = 2 * q + (g >> 2), plane = g & 3;
                const bool real = member < p.members && plane < 3;
                // the lane's share of a block: 8 bytes of a 32-weight sub-block (Q4_K / Q5_K), 4 bytes of a 16-weight block (Q6_K)
                const uint32_t lane_bytes = (FMT == kQ6_K ? 4u : 8u) * t;
                lx.x[q] = real ? smem_addr(planes) + static_cast<uint32_t>(member) * static_cast<uint32_t>(p.nsb) * kSliceBytes + plane * 32u + lane_bytes
                               : smem_addr(zeros) + 96u + lane_bytes;
                lx.step[q] = real ? static_cast<uint32_t>(kSliceBytes) : 0u;
            }
            const uint32_t sums_member = g < p.members ? static_cast<uint32_t>(g) : 0u;
            lx.sums = smem_addr(sums) + sums_member * static_cast<uint32_t>(p.nsb) * 32u;
            lx.scale = smem_addr(scale);
            lx.advance(warp);   // the warp's super-block of the first chunk
        }
        const uint32_t ring_addr = smem_addr(ring);
        // This warp's super-block inside a stage: box warp / kBoxSb, position warp % kBoxSb, rows g and g + 8.
        const uint32_t lane_off = static_cast<uint32_t>((warp / P::kBoxSb) * P::kBoxBytes + (warp % P::kBoxSb) * P::kSbBytes + g * P::kRowPitch);

#pragma unroll 1
        for (int tile = 0; tile < tiles; ++tile) {
            float acc[GROUPS][2], mins[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int q = 0; q < GROUPS; ++q) acc[q][0] = acc[q][1] = 0.0f;
#pragma unroll 1
            for (int chunk = 0; chunk < chunks; ++chunk) {
                const int it = tile * chunks + chunk;
                const int s = it % stages;
                if (ok && !mbar_wait_bounded_hint(&full[s], (it / stages) & 1, 2000u)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    ok = false;
                }
                const int sb = chunk * kWarps + warp;
                if (sb < p.nsb) {
                    const uint32_t p0 = ring_addr + static_cast<uint32_t>(s) * P::kStageBytes + lane_off;
                    if constexpr (FMT == kQ6_K) {
                        // 210-byte super-blocks: the warp's one starts on a word boundary when its position in the box is even
                        if (warp & 1) superblock_q6<GROUPS, true>(p0, p0 + 8 * P::kRowPitch, lx, t, acc);
                        else superblock_q6<GROUPS, false>(p0, p0 + 8 * P::kRowPitch, lx, t, acc);
                    } else {
                        superblock<FMT, GROUPS>(p0, p0 + 8 * P::kRowPitch, lx, t, acc, mins);
                    }
                }
                lx.advance(kWarps);
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }
            lx.advance(-chunks * kWarps);
            // Tile end: a member's two plane shares sit in neighbouring lanes; then the eight warps' partial sums
            // (each 16 rows x 8 members) meet in shared memory, the minima terms added by the lanes that hold them.
            float* buf = red + (tile & 1) * (kWarps * 128) + warp * 128;
#pragma unroll
            for (int q = 0; q < GROUPS; ++q) {
                const float v0 = acc[q][0] + __shfl_xor_sync(0xffffffffu, acc[q][0], 1);
                const float v1 = acc[q][1] + __shfl_xor_sync(0xffffffffu, acc[q][1], 1);
                if ((t & 1) == 0) {
                    buf[g * 8 + 2 * q + (t >> 1)] = v0;
                    buf[(g + 8) * 8 + 2 * q + (t >> 1)] = v1;
                }
            }
            __syncwarp();
            if (2 * t < 2 * GROUPS) {
                buf[g * 8 + 2 * t] += mins[0];
                buf[g * 8 + 2 * t + 1] += mins[1];
                buf[(g + 8) * 8 + 2 * t] += mins[2];
                buf[(g + 8) * 8 + 2 * t + 1] += mins[3];
            }
            named_barrier_sync(1, kConsumers);
            if (threadIdx.x < 128) {
                const int row = static_cast<int>(threadIdx.x) >> 3, m = static_cast<int>(threadIdx.x) & 7;
                const long long out_row = static_cast<long long>(tile_begin + tile) * kTileRows + row;
                if (m < p.members && out_row < p.n) {
                    const float* all = red + (tile & 1) * (kWarps * 128);
                    float v = all[threadIdx.x];
#pragma unroll
                    for (int w = 1; w < kWarps; ++w) v += all[w * 128 + threadIdx.x];
                    const size_t o = static_cast<size_t>(m) * p.n + static_cast<size_t>(out_row);
                    if (p.y_bf16) {
                        if (p.accumulate) v += __bfloat162float(static_cast<const __nv_bfloat16*>(p.y)[o]);
                        static_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(v);
                    } else {
                        if (p.accumulate) v += static_cast<const float*>(p.y)[o];
                        static_cast<float*>(p.y)[o] = v;
                    }
                }
            }
        }
    }
    // Common exit: after a wait that ran out, copies may still be in flight into this CTA's shared memory;
    // give them time to land before the memory is handed to another CTA.
    __syncthreads();
    if (*reinterpret_cast<volatile int*>(p.status) != kDeviceOk) {
        for (int spin = 0; spin < 64; ++spin) __nanosleep(1000);
    }
}

// ---------------------------------------------------------------- pre-pass: the activation image in global memory
// grid (ceil(nsb / 8), members): warp w of CTA (c, m) converts super-block 8c + w of member row m.
__global__ void __launch_bounds__(256) gemv_imma_image_kernel(const ImmaParams p, uint8_t* image) {
    __shared__ float partial[8];
    pdl_launch_dependents();
    pdl_wait_prior();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = blockIdx.y;
    float inv_rms = 1.0f;
    if (p.mode == 1) {
        float part = partial_square_sum(p, m, static_cast<int>(threadIdx.x), 256);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (lane == 0) partial[warp] = part;
        __syncthreads();
        float totalsq = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) totalsq += partial[w];
        inv_rms = 1.0f / sqrtf(totalsq / static_cast<float>(p.k) + p.eps);
    }
    __half* sums = reinterpret_cast<__half*>(image + image_plane_bytes(p.members, p.nsb));
    float* scale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sums) + image_sums_bytes(p.members, p.nsb));
    const int sb = blockIdx.x * 8 + warp;
    if (sb < p.nsb) {
        float v[8];
        load_slice(p, m, sb, lane, inv_rms, v);
        store_slice(m, sb, lane, v, image + static_cast<size_t>(m) * p.nsb * kSliceBytes, sums + static_cast<size_t>(m) * p.nsb * 16, scale);
    }
}

constexpr size_t kSmemLimit = 227 * 1024;

template <uint32_t FMT, int GROUPS>
cudaError_t launch_groups(const MmaGemvArgs& a) {
    using P = ImmaPlan<FMT>;
    auto kernel = gemv_imma_kernel<FMT, GROUPS>;
    const int nsb = a.k / kSuperBlock;
    const size_t fixed = imma_fixed_bytes(a.members, nsb);
    // Two CTAs per SM when each then has at least two stages, else one.
    auto share = [](int ctas) { return (kSmemLimit - 1024 * static_cast<size_t>(ctas)) / static_cast<size_t>(ctas); };
    int resident = fixed + 2 * static_cast<size_t>(P::kStageBytes) <= share(2) ? 2 : 1;
    if (a.resident > 0 && a.resident < resident) resident = a.resident;
    const size_t budget = share(resident);
    int stages = static_cast<int>((budget - fixed) / P::kStageBytes);
    if (stages > kMaxStages) stages = kMaxStages;
    if (a.stages > 0 && a.stages < stages) stages = a.stages;
    if (stages < 2) return cudaErrorInvalidConfiguration;
    const size_t smem = fixed + static_cast<size_t>(stages) * P::kStageBytes;
    static int configured_device = -1;
    int device = 0;
    cudaGetDevice(&device);
    if (configured_device != device) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemLimit));
        if (e != cudaSuccess) return e;
        configured_device = device;
    }
    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) return cudaErrorNotSupported;
    const unsigned long long row_bytes = static_cast<unsigned long long>(nsb) * P::kSbBytes;
    CUtensorMap wmap;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes / 8), static_cast<cuuint64_t>(a.n)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(P::kRowPitch / 8), static_cast<cuuint32_t>(kTileRows)};
    const cuuint32_t elem[2] = {1, 1};
    if (encode(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t*>(a.weights), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    ImmaParams p{};
    p.x = a.x;
    p.x_bf16 = a.x_bf16 ? 1 : 0;
    p.mode = a.mode;
    p.norm_weight = a.norm_weight;
    p.eps = a.eps;
    p.image = static_cast<const uint8_t*>(a.image);
    p.y = a.y;
    p.y_bf16 = a.y_bf16 ? 1 : 0;
    p.accumulate = a.accumulate ? 1 : 0;
    p.k = a.k;
    p.n = a.n;
    p.nsb = nsb;
    p.members = a.members;
    p.stages = stages;
    p.status = a.device_status;
    const int tiles = (a.n + kTileRows - 1) / kTileRows;
    int per_sm = resident;
    if (a.grid_ctas > 0) per_sm = a.grid_ctas < resident ? a.grid_ctas : resident;
    int grid = a.sm_count * per_sm;
    if (grid > tiles) grid = tiles;
    return launch_kernel(kernel, dim3(grid), dim3(kThreads), smem, a.stream, wmap, p);
}

template <uint32_t FMT>
cudaError_t launch_format(const MmaGemvArgs& a) {
    switch ((a.members + 1) / 2) {
        case 1: return launch_groups<FMT, 1>(a);
        case 2: return launch_groups<FMT, 2>(a);
        case 3: return launch_groups<FMT, 3>(a);
        default: return launch_groups<FMT, 4>(a);
    }
}

}  // namespace

bool gemv_imma_supports(uint32_t value_type, int k, int n, int members, const void* weights) {
    if (value_type != kQ4_K && value_type != kQ5_K && value_type != kQ6_K) return false;
    if (members < 1 || members > kMaxMembers || k <= 0 || k % kSuperBlock != 0 || n < kTileRows) return false;
    const int block_bytes = value_type == kQ4_K ? 144 : value_type == kQ5_K ? 176 : 210;
    const unsigned long long row_bytes = static_cast<unsigned long long>(k / kSuperBlock) * block_bytes;
    if (row_bytes % 16 != 0 || reinterpret_cast<uintptr_t>(weights) % 16 != 0) return false;   // Q6_K: K / 256 a multiple of eight
    const size_t stage = value_type == kQ4_K ? ImmaPlan<kQ4_K>::kStageBytes : value_type == kQ5_K ? ImmaPlan<kQ5_K>::kStageBytes
                                                                                                  : ImmaPlan<kQ6_K>::kStageBytes;
    return imma_fixed_bytes(members, k / kSuperBlock) + 2 * stage <= kSmemLimit - 1024;
}

size_t gemv_imma_image_bytes(int members, int k) { return (image_bytes(members, k / kSuperBlock) + 255) & ~static_cast<size_t>(255); }

cudaError_t launch_gemv_imma_image(const MmaGemvArgs& a, void* image) {
    ImmaParams p{};
    p.x = a.x;
    p.x_bf16 = a.x_bf16 ? 1 : 0;
    p.mode = a.mode;
    p.norm_weight = a.norm_weight;
    p.eps = a.eps;
    p.k = a.k;
    p.nsb = a.k / kSuperBlock;
    p.members = a.members;
    return launch_kernel(gemv_imma_image_kernel, dim3((p.nsb + 7) / 8, a.members), dim3(256), 0, a.stream, p, static_cast<uint8_t*>(image));
}

cudaError_t launch_gemv_imma(const MmaGemvArgs& a) {
    switch (a.value_type) {
        case kQ4_K: return launch_format<kQ4_K>(a);
        case kQ5_K: return launch_format<kQ5_K>(a);
        case kQ6_K: return launch_format<kQ6_K>(a);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ribn
