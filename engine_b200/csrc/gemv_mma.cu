// Dequant-fused GEMV for 1..8 activation rows per launch: packed quants are expanded in registers with
// half2 arithmetic and multiplied on the warp-level tensor-core instruction (mma.sync m16n8k16, f32
// accumulate), optionally with the RMSNorm or silu(gate)*up that feeds it fused into the prologue.
//
//   y[m][n] = sum_k dequant(W[n][k]) * x[m][k]
//
// Why this shape.  The path is bound by HBM: on B200 a 4.5-bit weight arrives every ~0.025 SM clocks, which
// leaves about three thread instructions per weight.  A kernel that converts every quant to f32 and issues an
// FMA per weight and member cannot keep up, and neither can one that writes a dequantised tile to shared
// memory for the tcgen05 pipe (2 bytes written and 2 read per weight against 0.56 streamed).  Here
//   * the raw super-blocks go from HBM to a shared-memory ring as tiled TMA boxes (16 rows x 4 or 8
//     super-blocks per request), never through registers on the way in;
//   * a lane reads its share with 128-bit loads and turns two quants at a time into an f16 pair with one
//     logic op and one HFMA2: (q | 0x6400) is the half 1024 + q, and (1024 + q) * sc - 1024 * sc = q * sc is
//     exact in f16 for every Q4_K / Q5_K value (q * sc <= 1953 < 2048); Q6_K's sc * (q - 32) <= 4096 rounds
//     at 2^-12 for its largest products only;
//   * those pairs ARE the A fragment of mma.m16n8k16 (16 weight rows x 16 K elements per warp), so the
//     multiply-adds of up to eight member rows cost one instruction per 256 weights and the dequantised
//     values never leave the register file.  K positions inside a fragment are a free permutation: the
//     activations are stored in shared memory in the order the unpacking produces;
//   * the super-block scale d (and dmin times the block sums of the activations, itself one extra mma)
//     is applied in f32 once per super-block and row.
// Activations are converted to f16 per (member, super-block) with a power-of-two factor that brings the
// largest magnitude of the 256 values into [512, 1024): exact for bf16 inputs, 2^-12 relative for f32.
// The conversion runs inside this kernel (each warp converts the K slices it owns; no second launch on the
// critical path) or, for wider batches, in a pre-pass whose image is bulk-copied into shared memory.
//
// Reference counterparts: q*_gemv_warp / _warp_batch (crates/nvidia/src/kernels/quantized/q4_k.cu:103-258,
// q5_k.cu, q6_k.cu) for the contract; rms_norm (crates/nvidia/src/model_ops.rs:106-147) and silu_mul
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
constexpr int kMmaThreads = kConsumers + 32;   // + the producer warp
constexpr int kTileRows = 16;                  // weight rows per tile (the M of m16n8k16)
constexpr int kMaxStages = 8;
constexpr int kMaxMembers = 8;                 // the N of m16n8k16

template <uint32_t FMT>
struct MmaGeometry;
template <>
struct MmaGeometry<kQ4_K> {
    static constexpr int kBoxSb = 4;           // row pitch 576 B = 144 words = 16 (mod 32): rows alternate bank halves
    static constexpr int kBoxes = 2;
};
template <>
struct MmaGeometry<kQ5_K> {
    static constexpr int kBoxSb = 4;           // 704 B = 176 words = 16 (mod 32)
    static constexpr int kBoxes = 2;
};
template <>
struct MmaGeometry<kQ6_K> {
    static constexpr int kBoxSb = 8;           // 1680 B: the smallest multiple of 210 that is a multiple of 16
    static constexpr int kBoxes = 1;
};

template <uint32_t FMT>
struct MmaPlan {
    using G = MmaGeometry<FMT>;
    static constexpr int kSbBytes = Format<FMT>::kBytes;
    static constexpr int kRowPitch = G::kBoxSb * kSbBytes;
    static constexpr int kBoxBytes = kTileRows * kRowPitch;
    static constexpr int kStageBytes = G::kBoxes * kBoxBytes;
    static_assert(G::kBoxSb * G::kBoxes == kWarps, "a warp owns one super-block of every stage");
    static_assert(kRowPitch % 16 == 0 && kBoxBytes % 128 == 0, "TMA box: 16-byte rows, 128-byte aligned destination");
    static_assert(kRowPitch / 8 <= 256, "TMA box dimension limit (8-byte elements)");
};

struct MmaParams {
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
    int planes;                 // f16 planes per activation: 1 (bf16 inputs are exact in one) or 2 (f32 inputs: hi + lo)
    int* status;
    long long* trace;           // diagnostics (builds with -DRIBN_TRACE): wall-clock stamps of the first and the last CTA, or null
};

// trace[slot * 64 + event] = globaltimer (ns); slot 0 = first CTA, 1 = last CTA.  Compiled in with -DRIBN_TRACE only.
__device__ __forceinline__ void wall_stamp(const MmaParams& p, int event) {
#ifdef RIBN_TRACE
    if (p.trace != nullptr && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1) && event < 64) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.trace[(blockIdx.x == 0 ? 0 : 64) + event] = static_cast<long long>(t);
    }
#else
    (void)p;
    (void)event;
#endif
}

// ---------------------------------------------------------------- activation image
// Per call, in shared memory (and in global memory when a pre-pass makes it):
//   x16   [planes][members][k] f16, scaled per (member, super-block): plane 0 = f16(v), plane 1 = f16(v - plane 0)
//         (kept for f32 inputs only, so that the activations carry ~22 bits; bf16 inputs are exact in plane 0);
//         within a row the 4-element group that holds elements 4j..4j+3 sits at group index
//         (j ^ swz(j)) ^ (member & 3)  in the order [e0, e2, e1, e3]  (swz flips bit 3 of j when bits 4 and 5 of
//         j differ): the B-fragment loads of a half-warp, four member rows x four lanes 16 or 64 or 128 elements
//         apart, then fall on 32 different banks;
//   sums  [members][nsb][16] f16: the sum of each of the eight blocks of 32 scaled values (multiplier of the
//         Q4_K/Q5_K minimum) as f16 hi (8 values) then f16 lo (8 values);
//   scale [nsb][8] f32: 2^-e per (super-block, member), NaN when the slice holds a non-finite value.
__host__ __device__ inline size_t image_plane_bytes(int members, int k) { return static_cast<size_t>(members) * k * 2; }
__host__ __device__ inline size_t image_x16_bytes(int members, int k, int planes) { return image_plane_bytes(members, k) * planes; }
__host__ __device__ inline size_t image_sums_bytes(int members, int nsb) { return static_cast<size_t>(members) * nsb * 32; }
__host__ __device__ inline size_t image_scale_bytes(int nsb) { return static_cast<size_t>(nsb) * 32; }
__host__ __device__ inline size_t image_bytes(int members, int k, int planes) {
    const int nsb = k / kSuperBlock;
    return image_x16_bytes(members, k, planes) + image_sums_bytes(members, nsb) + image_scale_bytes(nsb);
}

__device__ __forceinline__ uint32_t group_index(uint32_t j, uint32_t member) {
    return (j ^ ((((j >> 4) ^ (j >> 5)) & 1u) << 3)) ^ (member & 3u);
}

// One warp converts super-block `sb` of member row `m` (256 values, eight per lane) and writes its part of the
// image at `x16_row` (the member's row), `sums_row`, `scale` (generic pointers: shared or global memory).
// The two halves of the conversion are separate so that a warp can have the loads of several slices in flight
// before it works on the first (one memory latency per batch instead of one per slice).
__device__ __forceinline__ void load_slice(const MmaParams& p, int m, int sb, int lane, float inv_rms, float (&v)[8]) {
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

__device__ __forceinline__ void store_slice(const MmaParams& p, int m, int sb, int lane, float (&v)[8], uint8_t* x16_row, size_t plane_bytes,
                                            __half* sums_row, float* scale) {
    const int k0 = sb * kSuperBlock + lane * 8;
    // Largest magnitude of the warp's 256 values in one warp reduction: non-negative floats order like their bit
    // patterns, and infinities and NaNs (0x7f800000 and above) come out on top, which is how they are detected.
    uint32_t biggest = 0u;
#pragma unroll
    for (int j = 0; j < 8; ++j) biggest = max(biggest, __float_as_uint(fabsf(v[j])));
    biggest = __reduce_max_sync(0xffffffffu, biggest);
    const bool bad = biggest >= 0x7f800000u;
    const float amax = __uint_as_float(biggest);
    // amax * 2^e in [512, 1024); e clamped so that both 2^e and 2^-e are normal numbers
    int e = 9 - (static_cast<int>(__float_as_uint(amax) >> 23) - 127);
    e = max(-100, min(100, e));
    float down = __uint_as_float(static_cast<uint32_t>(127 + e) << 23);
    float up = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
    if (amax == 0.0f) up = 0.0f;
    if (bad) {
        down = 0.0f;
        up = __int_as_float(0x7fc00000);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.0f;
    }
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        v[j] *= down;
        sum += v[j];
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    const uint32_t j0 = static_cast<uint32_t>(k0) >> 2;
    const uint32_t ga = group_index(j0, m) * 8, gb = group_index(j0 + 1, m) * 8;
    *reinterpret_cast<uint2*>(x16_row + ga) = make_uint2(half2_bits(v[0], v[2]), half2_bits(v[1], v[3]));
    *reinterpret_cast<uint2*>(x16_row + gb) = make_uint2(half2_bits(v[4], v[6]), half2_bits(v[5], v[7]));
    if (p.planes == 2) {
        float lo[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) lo[j] = v[j] - __half2float(__float2half_rn(v[j]));
        *reinterpret_cast<uint2*>(x16_row + plane_bytes + ga) = make_uint2(half2_bits(lo[0], lo[2]), half2_bits(lo[1], lo[3]));
        *reinterpret_cast<uint2*>(x16_row + plane_bytes + gb) = make_uint2(half2_bits(lo[4], lo[6]), half2_bits(lo[5], lo[7]));
    }
    if ((lane & 3) == 0) {
        const __half hi = __float2half_rn(sum);
        sums_row[sb * 16 + (lane >> 2)] = hi;
        sums_row[sb * 16 + 8 + (lane >> 2)] = __float2half_rn(sum - __half2float(hi));
    }
    if (lane == 0) scale[sb * 8 + m] = up;
}

__device__ __forceinline__ void convert_slice(const MmaParams& p, int m, int sb, int lane, float inv_rms, uint8_t* x16_row,
                                              size_t plane_bytes, __half* sums_row, float* scale) {
    float v[8];
    load_slice(p, m, sb, lane, inv_rms, v);
    store_slice(p, m, sb, lane, v, x16_row, plane_bytes, sums_row, scale);
}

// Raw bytes of one slice share of a lane (plain rows and rows to be RMS-normalised): loaded without being looked
// at, so that the loads of a whole batch are in flight together.
template <bool BF16>
struct RawSlice {
    uint4 a, b;   // bf16: a only
};
template <bool BF16>
__device__ __forceinline__ RawSlice<BF16> load_raw(const MmaParams& p, int m, int sb, int lane) {
    const size_t element = static_cast<size_t>(m) * p.k + static_cast<size_t>(sb) * kSuperBlock + lane * 8;
    RawSlice<BF16> r;
    if (BF16) {
        r.a = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.x) + element * 2);
        r.b = make_uint4(0u, 0u, 0u, 0u);
    } else {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.x) + element * 4);
        r.a = src[0];
        r.b = src[1];
    }
    return r;
}
template <bool BF16>
__device__ __forceinline__ void unpack_raw(const RawSlice<BF16>& r, float (&v)[8]) {
    if (BF16) {
        v[0] = __uint_as_float(r.a.x << 16); v[1] = __uint_as_float(r.a.x & 0xffff0000u);
        v[2] = __uint_as_float(r.a.y << 16); v[3] = __uint_as_float(r.a.y & 0xffff0000u);
        v[4] = __uint_as_float(r.a.z << 16); v[5] = __uint_as_float(r.a.z & 0xffff0000u);
        v[6] = __uint_as_float(r.a.w << 16); v[7] = __uint_as_float(r.a.w & 0xffff0000u);
    } else {
        v[0] = __uint_as_float(r.a.x); v[1] = __uint_as_float(r.a.y); v[2] = __uint_as_float(r.a.z); v[3] = __uint_as_float(r.a.w);
        v[4] = __uint_as_float(r.b.x); v[5] = __uint_as_float(r.b.y); v[6] = __uint_as_float(r.b.z); v[7] = __uint_as_float(r.b.w);
    }
}

// A warp's slices (super-blocks warp, warp + warps, ... of every member) for modes 0 and 1, four per batch of loads.
template <bool BF16>
__device__ __forceinline__ void convert_owned(const MmaParams& p, int warp, int warps, int lane, const float* inv_rms, uint8_t* x16,
                                              size_t plane_bytes, __half* sums, float* scale) {
    const int owned = p.nsb > warp ? (p.nsb - warp + warps - 1) / warps : 0;
    int sb = warp, m = 0;   // slice cursor: members vary fastest
#pragma unroll 1
    for (int left = owned * p.members; left > 0; left -= 4) {
        RawSlice<BF16> raw[4];
        int sbs[4], ms[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            sbs[u] = sb;
            ms[u] = m;
            raw[u] = load_raw<BF16>(p, m, sb, lane);   // past the last slice: the last one again, loaded and ignored
            if (u + 1 < left) {
                if (++m == p.members) {
                    m = 0;
                    sb += warps;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (u < left) {
                float v[8];
                unpack_raw<BF16>(raw[u], v);
                if (p.mode == 1) {
                    float g[8];
                    load_x8<float>(p.norm_weight + sbs[u] * kSuperBlock + lane * 8, g);
                    const float inv = inv_rms[ms[u]];
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = v[j] * inv * g[j];
                }
                store_slice(p, ms[u], sbs[u], lane, v, x16 + static_cast<size_t>(ms[u]) * p.k * 2, plane_bytes,
                            sums + static_cast<size_t>(ms[u]) * p.nsb * 16, scale);
            }
        }
    }
}

// sum of squares of member row m over the whole K range, by `threads` threads with index tid; the caller reduces.
__device__ __forceinline__ float partial_square_sum(const MmaParams& p, int m, int tid, int threads) {
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

// D += A(16x16, f16, row) * B(16x8, f16, col), f32 accumulate.  Lane (g = lane / 4, t = lane % 4) holds
//   a0: row g, K slots 2t,2t+1     a1: row g+8, same slots     a2: row g, K slots 2t+8,2t+9     a3: row g+8
//   b0: column g, K slots 2t,2t+1  b1: column g, K slots 2t+8,2t+9
//   c0,c1: row g, columns 2t,2t+1  c2,c3: row g+8, columns 2t,2t+1
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Per-lane constants of the B-fragment addressing (byte offsets inside one member row's super-block).
// The same with a zero accumulator going in: D = A * B.
__device__ __forceinline__ void mma16816_zero(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// Lane (g, t) reads the B fragments of member g.  Lanes whose member the launch does not have read member 0
// instead: their column of the result is never stored, so its content does not matter and no branch is needed.
struct LaneX {
    // Shared address of the group (i ^ (g & 3)) of the lane's member row in plane 0 at the super-block the warp
    // works on, with the lane's share of the position folded in, for the two values q of the swizzled group bit
    // (see group_index): xa[q][i].  The kernel moves them from super-block to super-block.
    uint32_t xa[2][4];
    uint32_t sums;       // shared address of the member's block sums of that super-block
    uint32_t scale;      // shared address of that super-block's eight scale factors
    uint32_t plane;      // bytes from plane 0 to plane 1

    __device__ __forceinline__ void advance(int superblocks) {
#pragma unroll
        for (int q = 0; q < 2; ++q)
#pragma unroll
            for (int i = 0; i < 4; ++i) xa[q][i] += static_cast<uint32_t>(superblocks * 512);
        sums += static_cast<uint32_t>(superblocks * 32);
        scale += static_cast<uint32_t>(superblocks * 32);
    }
};

// The B fragment of one step (both planes when the activations have two) and its multiply-adds.
template <int PLANES, int OFFSET, bool FIRST = false>
__device__ __forceinline__ void mma_step(float (&c)[4], uint32_t x_addr, uint32_t plane, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
    const uint2 b = lds64_at<OFFSET>(x_addr);
    if (FIRST) mma16816_zero(c, a0, a1, a2, a3, b.x, b.y);
    else mma16816(c, a0, a1, a2, a3, b.x, b.y);
    if (PLANES == 2) {
        const uint2 bl = lds64_at<OFFSET>(x_addr + plane);
        mma16816(c, a0, a1, a2, a3, bl.x, bl.y);
    }
}

template <uint32_t FMT>
struct MmaFormat;

// ---- Q4_K.  Lane t of a quad owns, per row, the 16-byte chunks t and t + 4 of the 128 quant bytes: chunk c
// holds positions 16(c&1)..+15 of the sub-block pair c >> 1 (low nibbles: sub-block 2(c>>1), high nibbles the next).
// Step (r, s, i): chunk t + 4r, word i, nibble plane s -> the lane's K elements are
//   256 sb + 128 r + 64 (t >> 1) + 32 s + 16 (t & 1) + 4 i + {0, 2, 1, 3}.
template <>
struct MmaFormat<kQ4_K> {
    static constexpr uint32_t kQuantOffset = 16;
    __device__ static void fifth_bits(uint32_t, uint32_t, int, uint4&, uint4&) {}
    template <int S>
    __device__ static uint32_t merge(uint32_t v, const uint4&, int, int, int) { return v; }
};

template <uint32_t FMT, int PLANES>
__device__ __forceinline__ void superblock_q45(uint32_t p0, uint32_t p1, const LaneX& lx, int t, float (&acc)[4]) {
    using MF = MmaFormat<FMT>;
    const uint4 h0 = lds128(p0), h1 = lds128(p1);   // d | dmin, 12 scale bytes
    uint32_t sc_lo0, sc_hi0, m_lo0, m_hi0, sc_lo1, sc_hi1, m_lo1, m_hi1;
    unpack_k_scales(h0.y, h0.z, h0.w, sc_lo0, sc_hi0, m_lo0, m_hi0);
    unpack_k_scales(h1.y, h1.z, h1.w, sc_lo1, sc_hi1, m_lo1, m_hi1);
    float cq[4], cm[4];
    {
        // minimum term: A = the eight 6-bit minima, twice (K slots 0..7 and 8..15); B = the members' block sums,
        // f16 hi in slots 0..7 and f16 lo in slots 8..15
        const uint32_t a0 = byte_pair_half2((t & 2) ? m_hi0 : m_lo0, (t & 1) != 0);
        const uint32_t a1 = byte_pair_half2((t & 2) ? m_hi1 : m_lo1, (t & 1) != 0);
        const uint32_t b0 = lds32(lx.sums + t * 4);
        const uint32_t b1 = lds32(lx.sums + 16 + t * 4);
        mma16816_zero(cm, a0, a1, a0, a1, b0, b1);
    }
    // B-fragment addresses: the swizzled group bit of step (r, s) is (s ^ r) ^ (t >> 1), folded into lx.xa[s ^ r]
    uint4 f0 = make_uint4(0u, 0u, 0u, 0u), f1 = f0;
    MF::fifth_bits(p0, p1, t, f0, f1);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        constexpr int kStepBytes = 256;   // chunk t + 4 r: 128 elements further on
        const uint4 q0 = lds128(p0 + MF::kQuantOffset + 16 * (t + 4 * r));
        const uint4 q1 = lds128(p1 + MF::kQuantOffset + 16 * (t + 4 * r));
        // scales of sub-blocks 2j, 2j+1 with j = (t >> 1) + 2r: bytes 2(t>>1), +1 of sc_lo (r = 0) or sc_hi (r = 1)
        const uint32_t s0 = byte_pair_half2(r ? sc_hi0 : sc_lo0, (t >> 1) != 0);
        const uint32_t s1 = byte_pair_half2(r ? sc_hi1 : sc_lo1, (t >> 1) != 0);
        const uint32_t mul_a0 = dup_low(s0), mul_b0 = dup_high(s0);
        const uint32_t mul_a1 = dup_low(s1), mul_b1 = dup_high(s1);
        const uint32_t add_a0 = hmul2(mul_a0, 0xe400e400u);    // -1024 * sc
        const uint32_t add_a1 = hmul2(mul_a1, 0xe400e400u);
        const uint32_t add_b0 = hmul2(mul_b0, 0xd400d400u);    // -64 * sc:  (1024 + 16 q) * sc/16 - 64 sc = q sc
        const uint32_t add_b1 = hmul2(mul_b1, 0xd400d400u);
        const uint32_t mul_bh0 = hmul2(mul_b0, 0x2c002c00u);   // sc / 16
        const uint32_t mul_bh1 = hmul2(mul_b1, 0x2c002c00u);
        const int shift = 2 * ((t >> 1) + 2 * r);              // Q5_K: bit of sub-block 2j in the fifth-bit bytes
        const uint32_t q0w[4] = {q0.x, q0.y, q0.z, q0.w};
        const uint32_t q1w[4] = {q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w0 = q0w[i], w1 = q1w[i];
            const uint32_t w0s = w0 >> 8, w1s = w1 >> 8;
            {
                const uint32_t a0 = hfma2(MF::template merge<0>(and_or(w0, 0x000f000fu, kMagic), f0, i, shift, 0), mul_a0, add_a0);
                const uint32_t a1 = hfma2(MF::template merge<0>(and_or(w1, 0x000f000fu, kMagic), f1, i, shift, 0), mul_a1, add_a1);
                const uint32_t a2 = hfma2(MF::template merge<0>(and_or(w0s, 0x000f000fu, kMagic), f0, i, shift, 1), mul_a0, add_a0);
                const uint32_t a3 = hfma2(MF::template merge<0>(and_or(w1s, 0x000f000fu, kMagic), f1, i, shift, 1), mul_a1, add_a1);
                if (r == 0 && i == 0) mma_step<PLANES, 0, true>(cq, lx.xa[0][i], lx.plane, a0, a1, a2, a3);
                else if (r == 0) mma_step<PLANES, 0>(cq, lx.xa[0][i], lx.plane, a0, a1, a2, a3);
                else mma_step<PLANES, kStepBytes>(cq, lx.xa[1][i], lx.plane, a0, a1, a2, a3);
            }
            {
                const uint32_t a0 = hfma2(MF::template merge<1>(and_or(w0, 0x00f000f0u, kMagic), f0, i, shift, 0), mul_bh0, add_b0);
                const uint32_t a1 = hfma2(MF::template merge<1>(and_or(w1, 0x00f000f0u, kMagic), f1, i, shift, 0), mul_bh1, add_b1);
                const uint32_t a2 = hfma2(MF::template merge<1>(and_or(w0s, 0x00f000f0u, kMagic), f0, i, shift, 1), mul_bh0, add_b0);
                const uint32_t a3 = hfma2(MF::template merge<1>(and_or(w1s, 0x00f000f0u, kMagic), f1, i, shift, 1), mul_bh1, add_b1);
                if (r == 0) mma_step<PLANES, 0>(cq, lx.xa[1][i], lx.plane, a0, a1, a2, a3);
                else mma_step<PLANES, kStepBytes>(cq, lx.xa[0][i], lx.plane, a0, a1, a2, a3);
            }
        }
    }
    const float d0 = f16_bits_to_f32(h0.x & 0xffffu), dm0 = f16_bits_to_f32(h0.x >> 16);
    const float d1 = f16_bits_to_f32(h1.x & 0xffffu), dm1 = f16_bits_to_f32(h1.x >> 16);
    const uint2 xs = lds64(lx.scale + t * 8);
    const float xa = __uint_as_float(xs.x), xb = __uint_as_float(xs.y);
    acc[0] = fmaf(d0 * xa, cq[0], acc[0]);
    acc[0] = fmaf(-(dm0 * xa), cm[0], acc[0]);
    acc[1] = fmaf(d0 * xb, cq[1], acc[1]);
    acc[1] = fmaf(-(dm0 * xb), cm[1], acc[1]);
    acc[2] = fmaf(d1 * xa, cq[2], acc[2]);
    acc[2] = fmaf(-(dm1 * xa), cm[2], acc[2]);
    acc[3] = fmaf(d1 * xb, cq[3], acc[3]);
    acc[3] = fmaf(-(dm1 * xb), cm[3], acc[3]);
}

// ---- Q5_K: Q4_K plus one bit per weight.  Byte p of the 32 fifth-bit bytes carries, in bit b, the fifth bit of
// position p of sub-block b.  The lane's positions are 16(t&1)..+15 in both of its chunks: one 16-byte load per row.
template <>
struct MmaFormat<kQ5_K> {
    static constexpr uint32_t kQuantOffset = 48;
    __device__ static void fifth_bits(uint32_t p0, uint32_t p1, int t, uint4& f0, uint4& f1) {
        f0 = lds128(p0 + 16 + 16 * (t & 1));
        f1 = lds128(p1 + 16 + 16 * (t & 1));
    }
    // S = 0: low-nibble plane (sub-block 2j, unit = bit 0, fifth bit -> bit 4); S = 1: high-nibble plane (sub-block
    // 2j+1, unit = bit 4, fifth bit -> bit 8).  odd = 0: positions in bytes 0 and 2 of the word, 1: bytes 1 and 3.
    template <int S>
    __device__ static uint32_t merge(uint32_t v, const uint4& f, int i, int shift, int odd) {
        const uint32_t word = i == 0 ? f.x : i == 1 ? f.y : i == 2 ? f.z : f.w;
        const uint32_t bits = word >> shift;   // bit 0 of every byte: sub-block 2j, bit 1: sub-block 2j+1
        if (S == 0) return and_or(odd ? (bits >> 4) : (bits << 4), 0x00100010u, v);
        return and_or(odd ? (bits >> 1) : (bits << 7), 0x01000100u, v);
    }
};

// ---- Q6_K.  Lane t: half n2 = t >> 1 of the super-block, positions 16(t&1)..+15 of its four 32-element groups
// v = 0..3 (low nibbles of ql bytes 64 n2 + 16 h and 64 n2 + 32 + 16 h, then their high nibbles; the two upper bits
// from qh bytes 32 n2 + 16 h, bit pairs 2v).  Step (v, i): K elements 256 sb + 128 n2 + 32 v + 16 h + 4 i + {0,2,1,3}.
// Super-blocks are 210 bytes, so a lane's 16-byte chunks start on 2-byte boundaries: two aligned 16-byte loads and
// a funnel shift by the (warp-uniform) misalignment.
template <int PLANES>
__device__ __forceinline__ void superblock_q6(uint32_t p0, uint32_t p1, const LaneX& lx, int t, float (&acc)[4]) {
    const uint32_t n2 = static_cast<uint32_t>(t >> 1), h = static_cast<uint32_t>(t & 1);
    const uint4 la0 = lds128_unaligned(p0 + 64 * n2 + 16 * h), lb0 = lds128_unaligned(p0 + 64 * n2 + 32 + 16 * h);
    const uint4 qh0 = lds128_unaligned(p0 + 128 + 32 * n2 + 16 * h);
    const uint4 la1 = lds128_unaligned(p1 + 64 * n2 + 16 * h), lb1 = lds128_unaligned(p1 + 64 * n2 + 32 + 16 * h);
    const uint4 qh1 = lds128_unaligned(p1 + 128 + 32 * n2 + 16 * h);
    const uint32_t la0w[4] = {la0.x, la0.y, la0.z, la0.w}, lb0w[4] = {lb0.x, lb0.y, lb0.z, lb0.w}, qh0w[4] = {qh0.x, qh0.y, qh0.z, qh0.w};
    const uint32_t la1w[4] = {la1.x, la1.y, la1.z, la1.w}, lb1w[4] = {lb1.x, lb1.y, lb1.z, lb1.w}, qh1w[4] = {qh1.x, qh1.y, qh1.z, qh1.w};
    float cq[4];
    // B-fragment addresses: the swizzled group bit of step v is ((v & 1) ^ (v >> 1)) ^ n2, folded into lx.xa; v >> 1 adds 64 elements
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        // scale of group v of this lane: index 8 n2 + 2 v + h.  A = (1024 + 4 q) * sc/4 - 288 sc = sc * (q - 32)
        const float s0 = static_cast<float>(lds_s8(p0 + 192 + 8 * n2 + 2 * v + h));
        const float s1 = static_cast<float>(lds_s8(p1 + 192 + 8 * n2 + 2 * v + h));
        const uint32_t mul0 = half2_bits(s0 * 0.25f, s0 * 0.25f), add0 = half2_bits(s0 * -288.0f, s0 * -288.0f);
        const uint32_t mul1 = half2_bits(s1 * 0.25f, s1 * 0.25f), add1 = half2_bits(s1 * -288.0f, s1 * -288.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t b0, b1;
            if (v == 0) { b0 = q6_bytes<0>(la0w[i], lb0w[i], qh0w[i]); b1 = q6_bytes<0>(la1w[i], lb1w[i], qh1w[i]); }
            else if (v == 1) { b0 = q6_bytes<1>(la0w[i], lb0w[i], qh0w[i]); b1 = q6_bytes<1>(la1w[i], lb1w[i], qh1w[i]); }
            else if (v == 2) { b0 = q6_bytes<2>(la0w[i], lb0w[i], qh0w[i]); b1 = q6_bytes<2>(la1w[i], lb1w[i], qh1w[i]); }
            else { b0 = q6_bytes<3>(la0w[i], lb0w[i], qh0w[i]); b1 = q6_bytes<3>(la1w[i], lb1w[i], qh1w[i]); }
            const uint32_t a0 = hfma2(__byte_perm(b0, kMagicBytes, 0x4240), mul0, add0);   // positions 0, 2
            const uint32_t a1 = hfma2(__byte_perm(b1, kMagicBytes, 0x4240), mul1, add1);
            const uint32_t a2 = hfma2(__byte_perm(b0, kMagicBytes, 0x4341), mul0, add0);   // positions 1, 3
            const uint32_t a3 = hfma2(__byte_perm(b1, kMagicBytes, 0x4341), mul1, add1);
            if (v == 0 && i == 0) mma_step<PLANES, 0, true>(cq, lx.xa[0][i], lx.plane, a0, a1, a2, a3);
            else if (v < 2) mma_step<PLANES, 0>(cq, lx.xa[v & 1][i], lx.plane, a0, a1, a2, a3);
            else mma_step<PLANES, 128>(cq, lx.xa[(v & 1) ^ 1][i], lx.plane, a0, a1, a2, a3);
        }
    }
    const float d0 = f16_bits_to_f32(lds_u16(p0 + 208)), d1 = f16_bits_to_f32(lds_u16(p1 + 208));
    const uint2 xs = lds64(lx.scale + t * 8);
    const float xa = __uint_as_float(xs.x), xb = __uint_as_float(xs.y);
    acc[0] = fmaf(d0 * xa, cq[0], acc[0]);
    acc[1] = fmaf(d0 * xb, cq[1], acc[1]);
    acc[2] = fmaf(d1 * xa, cq[2], acc[2]);
    acc[3] = fmaf(d1 * xb, cq[3], acc[3]);
}

template <uint32_t FMT, int PLANES>
__device__ __forceinline__ void superblock(uint32_t p0, uint32_t p1, const LaneX& lx, int t, float (&acc)[4]) {
    if constexpr (FMT == kQ6_K) {
        superblock_q6<PLANES>(p0, p1, lx, t, acc);
    } else {
        superblock_q45<FMT, PLANES>(p0, p1, lx, t, acc);
    }
}

// ---------------------------------------------------------------- the kernel
// Shared-memory plan: [ring: stages x stage][64 B slack][image: x16 | sums | scale][red: 2 x 8 warps x 128 f32]
//                     [norm: 8 warps x 8 f32][barriers]
__host__ __device__ inline size_t mma_fixed_bytes(int members, int k, int planes) {
    return 128 /*alignment*/ + 64 + image_bytes(members, k, planes) + 2 * kWarps * 128 * 4 + (kWarps + 1) * kMaxMembers * 4 + (2 * kMaxStages + 2) * 8;
}

template <uint32_t FMT, int PLANES, int MIN_CTAS>
__global__ void __launch_bounds__(kMmaThreads, MIN_CTAS) gemv_mma_kernel(const __grid_constant__ CUtensorMap wmap, const MmaParams p) {
    using P = MmaPlan<FMT>;
    using G = MmaGeometry<FMT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((128u - (smem_addr(smem_raw) & 127u)) & 127u);
    uint8_t* ring = smem;
    uint8_t* image = ring + static_cast<size_t>(p.stages) * P::kStageBytes + 64;
    uint8_t* x16 = image;
    const size_t plane_bytes = image_plane_bytes(p.members, p.k);
    __half* sums = reinterpret_cast<__half*>(x16 + image_x16_bytes(p.members, p.k, PLANES));
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
    if (threadIdx.x == 0) wall_stamp(p, 0);
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
        asm volatile("bar.arrive 2, %0;" ::"n"(kMmaThreads) : "memory");
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
                const uint32_t bytes = static_cast<uint32_t>(image_bytes(p.members, p.k, PLANES));
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
                const int boxes = (sbs + G::kBoxSb - 1) / G::kBoxSb;
                mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(boxes * P::kBoxBytes));
                for (int b = 0; b < boxes; ++b)
                    tma_load_2d(ring + static_cast<size_t>(s) * P::kStageBytes + b * P::kBoxBytes, &wmap,
                                (chunk * kWarps + b * G::kBoxSb) * P::kSbBytes / 8, row0, &full[s]);
                if (it == prefetch - 1) wall_stamp(p, 1);
                if (it == prefetch - 1 && !image_requested) request_image();
            }
            wall_stamp(p, 2);
        }
    } else {
        // ---------------- consumers ----------------
        const int g = lane >> 2, t = lane & 3;
        named_barrier_sync(2, kMmaThreads);
        if (threadIdx.x == 0) wall_stamp(p, 3);
        pdl_wait_prior();   // the activations may be the previous kernel's output, and y may still be read by it
        if (threadIdx.x == 0) wall_stamp(p, 4);
        if (p.image == nullptr) {
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
            // Members the launch does not have: their scale stays zero (columns that are never stored).
            if (lane >= p.members && lane < kMaxMembers)
                for (int sb = warp; sb < p.nsb; sb += kWarps) scale[sb * 8 + lane] = 0.0f;
            if (p.mode == 2) {
#pragma unroll 1
                for (int sb = warp; sb < p.nsb; sb += kWarps)
#pragma unroll 1
                    for (int m = 0; m < p.members; ++m)
                        convert_slice(p, m, sb, lane, 1.0f, x16 + static_cast<size_t>(m) * p.k * 2, plane_bytes, sums + static_cast<size_t>(m) * p.nsb * 16,
                                      scale);
            } else if (p.x_bf16) {
                convert_owned<true>(p, warp, kWarps, lane, norm + kWarps * kMaxMembers, x16, plane_bytes, sums, scale);
            } else {
                convert_owned<false>(p, warp, kWarps, lane, norm + kWarps * kMaxMembers, x16, plane_bytes, sums, scale);
            }
            __syncwarp();
        } else if (!mbar_wait_bounded(image_bar, 0)) {
            atomicExch(p.status, kDeviceWaitTimeout);
            ok = false;
        }

        if (threadIdx.x == 0) wall_stamp(p, 5);
        LaneX lx;
        {
            const uint32_t member = g < p.members ? static_cast<uint32_t>(g) : 0u;
            // the lane's share of a step's position: Q4_K / Q5_K 64 (t >> 1) + 16 (t & 1), Q6_K 128 (t >> 1) + 16 (t & 1) elements
            const uint32_t lane_groups = (FMT == kQ6_K ? 32u : 16u) * (t >> 1) + 4u * (t & 1);
            const uint32_t row = smem_addr(x16) + member * static_cast<uint32_t>(p.k) * 2u + lane_groups * 8u;
#pragma unroll
            for (int q = 0; q < 2; ++q)
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    lx.xa[q][i] = row + 64u * (static_cast<uint32_t>(q) ^ static_cast<uint32_t>(t >> 1)) + static_cast<uint32_t>((i ^ (member & 3)) * 8);
            lx.sums = smem_addr(sums) + member * static_cast<uint32_t>(p.nsb) * 32u;
            lx.scale = smem_addr(scale);
            lx.plane = static_cast<uint32_t>(plane_bytes);
            lx.advance(warp);   // the warp's super-block of the first chunk
        }
        const uint32_t ring_addr = smem_addr(ring);
        // This warp's super-block inside a stage: box warp / kBoxSb, position warp % kBoxSb, rows g and g + 8.
        const uint32_t lane_off = static_cast<uint32_t>((warp / G::kBoxSb) * P::kBoxBytes + (warp % G::kBoxSb) * P::kSbBytes + g * P::kRowPitch);

#pragma unroll 1
        for (int tile = 0; tile < tiles; ++tile) {
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
            for (int chunk = 0; chunk < chunks; ++chunk) {
                const int it = tile * chunks + chunk;
                const int s = it % stages;
                if (ok && !mbar_wait_bounded_hint(&full[s], (it / stages) & 1, 2000u)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    ok = false;
                }
                if (threadIdx.x == 0) wall_stamp(p, 8 + 2 * min(it, 20));
                const int sb = chunk * kWarps + warp;
                if (sb < p.nsb) {
                    const uint32_t p0 = ring_addr + static_cast<uint32_t>(s) * P::kStageBytes + lane_off;
                    superblock<FMT, PLANES>(p0, p0 + 8 * P::kRowPitch, lx, t, acc);
                }
                lx.advance(kWarps);
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                if (threadIdx.x == 0) wall_stamp(p, 9 + 2 * min(it, 20));
            }
            lx.advance(-chunks * kWarps);
            // Tile end: the eight warps' partial sums (each 16 rows x 8 members) meet in shared memory.
            float* buf = red + (tile & 1) * (kWarps * 128);
            *reinterpret_cast<float2*>(buf + warp * 128 + g * 8 + 2 * t) = make_float2(acc[0], acc[1]);
            *reinterpret_cast<float2*>(buf + warp * 128 + (g + 8) * 8 + 2 * t) = make_float2(acc[2], acc[3]);
            named_barrier_sync(1, kConsumers);
            if (threadIdx.x < 128) {
                const int row = static_cast<int>(threadIdx.x) >> 3, m = static_cast<int>(threadIdx.x) & 7;
                const long long out_row = static_cast<long long>(tile_begin + tile) * kTileRows + row;
                if (m < p.members && out_row < p.n) {
                    float v = buf[threadIdx.x];
#pragma unroll
                    for (int w = 1; w < kWarps; ++w) v += buf[w * 128 + threadIdx.x];
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
    if (threadIdx.x == 0) wall_stamp(p, 6);
    // Common exit: after a wait that ran out, copies may still be in flight into this CTA's shared memory;
    // give them time to land before the memory is handed to another CTA.
    __syncthreads();
    if (*reinterpret_cast<volatile int*>(p.status) != kDeviceOk) {
        for (int spin = 0; spin < 64; ++spin) __nanosleep(1000);
    }
}

// ---------------------------------------------------------------- pre-pass: the activation image in global memory
// grid (ceil(nsb / 8), members): warp w of CTA (c, m) converts super-block 8c + w of member row m.
__global__ void __launch_bounds__(256) gemv_mma_image_kernel(const MmaParams p, uint8_t* image) {
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
    uint8_t* x16 = image;
    __half* sums = reinterpret_cast<__half*>(x16 + image_x16_bytes(p.members, p.k, p.planes));
    float* scale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sums) + image_sums_bytes(p.members, p.nsb));
    const int sb = blockIdx.x * 8 + warp;
    if (sb < p.nsb) {
        if (m == 0 && lane >= p.members && lane < kMaxMembers) scale[sb * 8 + lane] = 0.0f;
        convert_slice(p, m, sb, lane, inv_rms, x16 + static_cast<size_t>(m) * p.k * 2, image_plane_bytes(p.members, p.k),
                      sums + static_cast<size_t>(m) * p.nsb * 16, scale);
    }
}

constexpr size_t kSmemLimit = 227 * 1024;

template <uint32_t FMT, int PLANES, int MIN_CTAS>
cudaError_t launch_planes(const MmaGemvArgs& a) {
    using P = MmaPlan<FMT>;
    auto kernel = gemv_mma_kernel<FMT, PLANES, MIN_CTAS>;
    const size_t fixed = mma_fixed_bytes(a.members, a.k, PLANES);
    // CTAs an SM can hold (MIN_CTAS by registers): as many as leave each at least two stages.
    auto share = [](int ctas) { return (kSmemLimit - 1024 * static_cast<size_t>(ctas)) / static_cast<size_t>(ctas); };
    int resident = 1;
    for (int c = MIN_CTAS; c >= 2; --c)
        if (fixed + 2 * static_cast<size_t>(P::kStageBytes) <= share(c)) {
            resident = c;
            break;
        }
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
    const unsigned long long row_bytes = static_cast<unsigned long long>(a.k / kSuperBlock) * P::kSbBytes;
    CUtensorMap wmap;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes / 8), static_cast<cuuint64_t>(a.n)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(P::kRowPitch / 8), static_cast<cuuint32_t>(kTileRows)};
    const cuuint32_t elem[2] = {1, 1};
    if (encode(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t*>(a.weights), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    MmaParams p{};
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
    p.nsb = a.k / kSuperBlock;
    p.members = a.members;
    p.stages = stages;
    p.planes = PLANES;
    p.status = a.device_status;
    p.trace = a.trace;
    const int tiles = (a.n + kTileRows - 1) / kTileRows;
    int per_sm = resident;
    if (a.grid_ctas > 0) per_sm = a.grid_ctas < resident ? a.grid_ctas : resident;
    int grid = a.sm_count * per_sm;
    if (grid > tiles) grid = tiles;
    return launch_kernel(kernel, dim3(grid), dim3(kMmaThreads), smem, a.stream, wmap, p);
}

template <uint32_t FMT>
cudaError_t launch_format(const MmaGemvArgs& a) {
    // resident = 3: the variant compiled for three CTAs per SM (72 registers per thread instead of 96)
    if (a.resident == 3) return a.planes == 2 ? launch_planes<FMT, 2, 3>(a) : launch_planes<FMT, 1, 3>(a);
    return a.planes == 2 ? launch_planes<FMT, 2, 2>(a) : launch_planes<FMT, 1, 2>(a);
}

size_t stage_bytes(uint32_t value_type) {
    return value_type == kQ4_K ? MmaPlan<kQ4_K>::kStageBytes : value_type == kQ5_K ? MmaPlan<kQ5_K>::kStageBytes : MmaPlan<kQ6_K>::kStageBytes;
}

}  // namespace

// Planes the activations of a call are kept in: two for f32 inputs when both fit next to a two-stage ring, else one.
int gemv_mma_planes(uint32_t value_type, int k, int members, bool x_bf16) {
    if (x_bf16) return 1;
    return mma_fixed_bytes(members, k, 2) + 2 * stage_bytes(value_type) <= kSmemLimit ? 2 : 1;
}

bool gemv_mma_supports(uint32_t value_type, int k, int n, int members, const void* weights) {
    if (value_type != kQ4_K && value_type != kQ5_K && value_type != kQ6_K) return false;
    if (members < 1 || members > kMaxMembers || k <= 0 || k % kSuperBlock != 0 || n < kTileRows) return false;
    const int block_bytes = value_type == kQ4_K ? 144 : value_type == kQ5_K ? 176 : 210;
    const unsigned long long row_bytes = static_cast<unsigned long long>(k / kSuperBlock) * block_bytes;
    if (row_bytes % 16 != 0 || reinterpret_cast<uintptr_t>(weights) % 16 != 0) return false;
    return mma_fixed_bytes(members, k, 1) + 2 * stage_bytes(value_type) <= kSmemLimit;
}

size_t gemv_mma_image_bytes(int members, int k, int planes) { return (image_bytes(members, k, planes) + 255) & ~static_cast<size_t>(255); }

cudaError_t launch_gemv_mma_image(const MmaGemvArgs& a, void* image) {
    MmaParams p{};
    p.x = a.x;
    p.x_bf16 = a.x_bf16 ? 1 : 0;
    p.mode = a.mode;
    p.norm_weight = a.norm_weight;
    p.eps = a.eps;
    p.k = a.k;
    p.nsb = a.k / kSuperBlock;
    p.members = a.members;
    p.planes = a.planes;
    return launch_kernel(gemv_mma_image_kernel, dim3((p.nsb + 7) / 8, a.members), dim3(256), 0, a.stream, p, static_cast<uint8_t*>(image));
}

cudaError_t launch_gemv_mma(const MmaGemvArgs& a) {
    switch (a.value_type) {
        case kQ4_K: return launch_format<kQ4_K>(a);
        case kQ5_K: return launch_format<kQ5_K>(a);
        case kQ6_K: return launch_format<kQ6_K>(a);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ribn
