// Decode-batch quantized GEMV on the tensor cores with the block scales applied AFTER the
// contraction ("group-scaled"): members 1..64, bf16 activations.
//
//   y[m][n] = sum_g  a[n][g] * ( sum_{k in g} q[n][k] * x[m][k] )  -  c[n][g] * ( sum_{k in g} x[m][k] )
//
// where g runs over the quantisation groups of a row (32 weights; 16 for Q6_K), q are the raw
// integer quants and a, c come from the block scales.  The reference computes the same sum one
// weight at a time on CUDA cores (crates/nvidia/src/kernels/quantized/q4_k.cu:103-258 and twins).
//
// Why this shape.  Dequantising every weight to a float before the product costs ~6-11 issued
// instructions per weight on B200, several times what the weight stream allows.  The quants
// themselves are small integers, exactly representable in bf16, and turning a nibble into the bf16
// number 128+q is one byte permute and one logic op per PAIR of weights.  So the tensor core
// contracts raw quants with the activations group by group,
//     D_g[n][m] = sum_{k in g} (128 + q[n][k]) * x[m][k]        (exact products, f32 accumulate)
//     S_g[m]    = sum_{k in g} x[m][k]                            (CUDA cores, from the activation tile)
// into a ring of TMEM buffers (one buffer = the groups of a 64-wide K step, one tcgen05.commit per
// step), and the accumulate warps (thread = weight row) read each finished group with tcgen05.ld and apply  acc[m] += a_g * D_g[m] - c_g * S_g[m],  c_g = min_g + 128 a_g
// (the 128 and Q6_K's -32 are folded into c).  Per weight that is ~1.2 instructions of unpacking
// plus 2M/32 FMAs, against one conversion, one FMA and a bf16 split per weight before.
// Precision is that of an f32-accumulate dot product of the exact weights: nothing is rounded to
// bf16 except the activations, which already are bf16.
//
// Structure of a CTA (896 threads): 128 weight rows x NT tokens (NT in {16, 32, 64}) x a K range.
//   warp 0        weight producer: one tiled TMA box of raw weight bytes per super-block (or per-row
//                 bulk copies when rows are not 16-byte aligned)
//   warp 26       activation producer: one tiled TMA box of activations per 64-wide K step (128-byte
//                 swizzle, rows past M read as zero) into a ring of its own, deep enough that the
//                 L2 latency of these small loads never sits on the critical path
//   warps 1, 27   issue tcgen05.mma (M=128, N=NT, K=16), one thread each, alternate K steps (issuing
//                 costs ~70 clocks per instruction and thread, more than these small MMAs take to run);
//                 tcgen05.commit per step
//   warps 2..     accumulate warps, two or four per TMEM lane quadrant (8 or 16 of the 24 worker warps): work items (group, 16-token chunk)
//                 are dealt round-robin to the four, so that several tcgen05.ld round trips are in
//                 flight per quadrant; group scales from the raw block headers, FMAs, then a
//                 fixed-order sum of the four partial accumulators through shared memory
//   ..25          unpack warps, four or two per group of 32 rows taking K steps in turn: raw bytes ->
//                 bf16 quants in the K-major 128-byte-swizzle A tile
// Every mbarrier wait is bounded; on expiry the status word is set and all warps still reach the
// teardown that frees TMEM.
#include <cuda_bf16.h>

#include "formats.cuh"
#include "internal.h"
#include "tc_host.h"
#include "tcgen05.cuh"

namespace ribn {
namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kSub = kSuperBlock / kBK;
// 24 worker warps, split between accumulate and unpack warps by the token tile (see GsGeometry),
// + weight producer, two MMA issuers, activation producer.
constexpr int kWorkerWarps = 24;
constexpr int kGsThreads = (4 + kWorkerWarps) * 32;
constexpr int kActivationWarp = 2 + kWorkerWarps;
constexpr int kSecondMmaWarp = kActivationWarp + 1;

__device__ __forceinline__ uint4 raw16(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint4 raw16_a2(const uint8_t* p) {
    uint4 v;
    v.x = ld_u32_a2(p);
    v.y = ld_u32_a2(p + 4);
    v.z = ld_u32_a2(p + 8);
    v.w = ld_u32_a2(p + 12);
    return v;
}

// Bytes b0 b1 b2 b3 of `w` spread to the low bytes of 16-bit lanes: [b0,0,b1,0] and [b2,0,b3,0].
__device__ __forceinline__ uint32_t spread01(uint32_t w) { return __byte_perm(w, 0u, 0x4140u); }
__device__ __forceinline__ uint32_t spread23(uint32_t w) { return __byte_perm(w, 0u, 0x4342u); }

// A 7-bit unsigned integer v in the low bits of each 16-bit lane -> bf16x2 of (128 + v):
// 0x4300 is 128.0 in bf16 and its seven mantissa bits count in steps of one.
constexpr uint32_t kMagic128 = 0x43004300u;

// Eight 4-bit quants (low nibbles of the bytes of u0 and u1) -> one 16-byte chunk of bf16 (128+q).
__device__ __forceinline__ uint4 chunk_low_nibbles(uint32_t u0, uint32_t u1) {
    uint4 c;
    c.x = (spread01(u0) & 0x000f000fu) | kMagic128;
    c.y = (spread23(u0) & 0x000f000fu) | kMagic128;
    c.z = (spread01(u1) & 0x000f000fu) | kMagic128;
    c.w = (spread23(u1) & 0x000f000fu) | kMagic128;
    return c;
}

// Per format:
//   kGroup        weights per scale group (the contraction length of one TMEM buffer)
//   kUsesSum      whether the epilogue needs S_g (an offset or a minimum to remove)
//   step()        one thread's 32 weights of a 64-wide K step as four 16-byte chunks of bf16 integers;
//                 chunk_index(h, c) says which of the row's eight chunks each is
//   group_scales  a[g], c[g] of one super-block for the accumulate warps
template <uint32_t FMT>
struct Quants;

template <>
struct Quants<kQ4_K> {
    static constexpr int kGroup = 32;
    static constexpr bool kUsesSum = true;
    static constexpr int kGroupsPerSb = 8;
    static constexpr bool kStoresCoef = true;   // c_g depends on the block minimum
    __device__ static int chunk_index(int h, int c) { return (c >> 1) * 4 + 2 * h + (c & 1); }
    __device__ static void step(const uint8_t* blk, int t, int h, uint4 (&out)[4]) {
        const uint4 w = raw16(blk + 16 + 32 * t + 16 * h);
        out[0] = chunk_low_nibbles(w.x, w.y);
        out[1] = chunk_low_nibbles(w.z, w.w);
        out[2] = chunk_low_nibbles(w.x >> 4, w.y >> 4);
        out[3] = chunk_low_nibbles(w.z >> 4, w.w >> 4);
    }
    __device__ static void group_scales(const uint8_t* blk, float (&a)[8], float (&c)[8]) {
        const uint4 h = raw16(blk);
        const float d = f16_bits_to_f32(h.x & 0xffffu);
        const float dmin = f16_bits_to_f32(h.x >> 16);
        uint32_t sc_lo, sc_hi, m_lo, m_hi;
        unpack_k_scales(h.y, h.z, h.w, sc_lo, sc_hi, m_lo, m_hi);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            a[g] = d * byte_of(g < 4 ? sc_lo : sc_hi, g & 3);
            c[g] = fmaf(128.0f, a[g], dmin * byte_of(g < 4 ? m_lo : m_hi, g & 3));
        }
    }
};

template <>
struct Quants<kQ5_K> {
    static constexpr int kGroup = 32;
    static constexpr bool kUsesSum = true;
    static constexpr int kGroupsPerSb = 8;
    static constexpr bool kStoresCoef = true;   // c_g depends on the block minimum
    __device__ static int chunk_index(int h, int c) { return Quants<kQ4_K>::chunk_index(h, c); }
    // Low nibbles of u plus the fifth bit (bit `bit` of the matching byte of hb), as bf16 (128+q).
    __device__ static uint32_t pair(uint32_t u_spread, uint32_t hb_spread, int bit) {
        return ((u_spread & 0x000f000fu) | (((hb_spread >> bit) & 0x00010001u) << 4)) | kMagic128;
    }
    __device__ static uint4 chunk(uint32_t u0, uint32_t u1, uint32_t h0, uint32_t h1, int bit) {
        uint4 c;
        c.x = pair(spread01(u0), spread01(h0), bit);
        c.y = pair(spread23(u0), spread23(h0), bit);
        c.z = pair(spread01(u1), spread01(h1), bit);
        c.w = pair(spread23(u1), spread23(h1), bit);
        return c;
    }
    __device__ static void step(const uint8_t* blk, int t, int h, uint4 (&out)[4]) {
        const uint4 w = raw16(blk + 48 + 32 * t + 16 * h);
        const uint4 hb = raw16(blk + 16 + 16 * h);
        out[0] = chunk(w.x, w.y, hb.x, hb.y, 2 * t);
        out[1] = chunk(w.z, w.w, hb.z, hb.w, 2 * t);
        out[2] = chunk(w.x >> 4, w.y >> 4, hb.x, hb.y, 2 * t + 1);
        out[3] = chunk(w.z >> 4, w.w >> 4, hb.z, hb.w, 2 * t + 1);
    }
    __device__ static void group_scales(const uint8_t* blk, float (&a)[8], float (&c)[8]) {
        Quants<kQ4_K>::group_scales(blk, a, c);
    }
};

template <>
struct Quants<kQ6_K> {
    static constexpr int kGroup = 16;   // one int8 scale per 16 weights
    static constexpr bool kUsesSum = true;
    static constexpr int kGroupsPerSb = 16;
    static constexpr bool kStoresCoef = false;  // c_g = 160 a_g
    __device__ static int chunk_index(int h, int c) { return Quants<kQ4_K>::chunk_index(h, c); }
    // 4 low bits from ql (nibble `nib`), 2 high bits from qh (at `shift`): 0..63, as bf16 (128+q).
    __device__ static uint32_t pair(uint32_t l_spread, uint32_t h_spread, int nib, int shift) {
        return (((l_spread >> nib) & 0x000f000fu) | (((h_spread >> shift) & 0x00030003u) << 4)) | kMagic128;
    }
    __device__ static uint4 chunk(uint32_t l0, uint32_t l1, uint32_t h0, uint32_t h1, int nib, int shift) {
        uint4 c;
        c.x = pair(spread01(l0), spread01(h0), nib, shift);
        c.y = pair(spread23(l0), spread23(h0), nib, shift);
        c.z = pair(spread01(l1), spread01(h1), nib, shift);
        c.w = pair(spread23(l1), spread23(h1), nib, shift);
        return c;
    }
    // Step t = groups-of-32 2t and 2t+1 (see qgemm_tc.cu): ql chunk c = t/2, low nibble for even t,
    // qh shifts 4*(t%2) and 4*(t%2)+2.
    __device__ static void step(const uint8_t* blk, int t, int h, uint4 (&out)[4]) {
        const int c = t >> 1;
        const int nib = (t & 1) * 4;
        const int v2 = (t & 1) * 4;
        const uint4 l0 = raw16_a2(blk + c * 64 + 16 * h);
        const uint4 l1 = raw16_a2(blk + c * 64 + 32 + 16 * h);
        const uint4 hb = raw16_a2(blk + 128 + c * 32 + 16 * h);
        out[0] = chunk(l0.x, l0.y, hb.x, hb.y, nib, v2);
        out[1] = chunk(l0.z, l0.w, hb.z, hb.w, nib, v2);
        out[2] = chunk(l1.x, l1.y, hb.x, hb.y, nib, v2 + 2);
        out[3] = chunk(l1.z, l1.w, hb.z, hb.w, nib, v2 + 2);
    }
    // w = a * (q6 - 32) and the tile holds 128 + q6: c = 160 a.
    __device__ static void group_scales(const uint8_t* blk, float (&a)[16], float (&c)[16]) {
        const float d = f16_bits_to_f32(ld_u16(blk + 208));
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
            const uint32_t pair = ld_u16(blk + 192 + i);
            a[i] = d * static_cast<float>(static_cast<int8_t>(pair & 0xffu));
            a[i + 1] = d * static_cast<float>(static_cast<int8_t>(pair >> 8));
            c[i] = 160.0f * a[i];
            c[i + 1] = 160.0f * a[i + 1];
        }
    }
};

template <>
struct Quants<kQ8_0> {
    static constexpr int kGroup = 32;
    static constexpr bool kUsesSum = false;  // int8 quants convert exactly, no offset to remove
    static constexpr int kGroupsPerSb = 8;
    static constexpr bool kStoresCoef = false;  // no offset
    __device__ static int chunk_index(int h, int c) { return 4 * h + c; }
    __device__ static uint32_t pair(float lo, float hi) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);  // |q| <= 128: exact in bf16
        return *reinterpret_cast<const uint32_t*>(&v);
    }
    __device__ static uint4 chunk(uint32_t u0, uint32_t u1) {
        float a[4], b[4];
        bytes_to_float4(u0 ^ 0x80808080u, 128.0f, a);
        bytes_to_float4(u1 ^ 0x80808080u, 128.0f, b);
        return make_uint4(pair(a[0], a[1]), pair(a[2], a[3]), pair(b[0], b[1]), pair(b[2], b[3]));
    }
    __device__ static void step(const uint8_t* blk, int t, int h, uint4 (&out)[4]) {
        const uint8_t* q = blk + 34 * (2 * t + h) + 2;
        const uint4 w0 = raw16_a2(q);
        const uint4 w1 = raw16_a2(q + 16);
        out[0] = chunk(w0.x, w0.y);
        out[1] = chunk(w0.z, w0.w);
        out[2] = chunk(w1.x, w1.y);
        out[3] = chunk(w1.z, w1.w);
    }
    __device__ static void group_scales(const uint8_t* blk, float (&a)[8], float (&c)[8]) {
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            a[b] = f16_bits_to_f32(ld_u16(blk + 34 * b));
            c[b] = 0.0f;
        }
    }
};


// Diagnostics (see TcParams::trace): one stamp per (role, step, event) from CTA (0,0,0).
__device__ __forceinline__ void stamp(const TcParams& p, int role, int step, int event) {
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && step < 64)
        p.trace[(role * 64 + step) * 8 + event] = clock64();
}

template <uint32_t FMT, int NT, bool RAWTMA>
struct GsGeometry {
    using F = Format<FMT>;
    using Q = Quants<FMT>;
    static constexpr int kAbStages = 4;
    // 64 tokens make eight work items per K step for the accumulate warps: four of them per TMEM lane
    // quadrant and two unpack slots; smaller tiles need the warps on the unpack side instead.
    static constexpr int kAccSlots = NT >= 64 ? 4 : 2;             // accumulate warps per TMEM lane quadrant
    static constexpr int kAccWarps = 4 * kAccSlots;
    static constexpr int kUnpackSlots = (kWorkerWarps - kAccWarps) / 4;   // K steps in flight per group of 32 rows
    static constexpr int kUnpackWarps = 4 * kUnpackSlots;          // one thread per weight row and slot
    static constexpr int kFirstUnpackThread = (2 + kAccWarps) * 32;
    static_assert(kUnpackSlots == 2 || kUnpackSlots == 4, "unpack slots take K steps modulo a power of two");
    static constexpr int kGroupsPerStep = kBK / Q::kGroup;      // 2, or 4 for Q6_K
    static constexpr int kMmasPerGroup = Q::kGroup / 16;        // 2, or 1 for Q6_K
    static constexpr int kChunks = NT / 16;                     // 16-token chunks
    // TMEM: a ring of step buffers, each holding the D_g of the groups of one 64-wide K step.
    static constexpr int kStepCols = kGroupsPerStep * NT;
    static constexpr int kStepBuffers = 512 / kStepCols < 4 ? 512 / kStepCols : 4;
    static constexpr int kTmemColumns = kStepBuffers * kStepCols < 32 ? 32 : kStepBuffers * kStepCols;
    static constexpr int kBoxBytes = FMT == kQ6_K ? 240 : F::kBytes;
    static constexpr int kSlot = RAWTMA ? kBoxBytes : ((F::kBytes + 15) / 16) * 16 + 16;
    static constexpr int kRawStageBytes = kBM * kSlot;
    static constexpr int kATileBytes = kBM * kBK * 2;
    static constexpr int kBTileBytes = NT * kBK * 2;
    static constexpr int kSumBytes = kStepBuffers * kGroupsPerStep * NT * 4;   // S_g[m] ring, f32
    static constexpr int kScaleStages = 2;                       // super-blocks of decoded group scales kept
    static constexpr int kScaleRow = (Q::kStoresCoef ? 2 : 1) * Q::kGroupsPerSb;   // floats per row: a[g], then c[g] if stored
    static constexpr int kScaleBytes = kScaleStages * kBM * kScaleRow * 4;
    static constexpr int kBGroups = NT >= 64 ? 2 : 3;           // activation tiles are recycled a super-block (4 tiles) at a time
    static constexpr int kBStages = kBGroups * kSub;
    static constexpr int kTilesBytes = kAbStages * kATileBytes + kBStages * kBTileBytes;
    static constexpr int kBarrierBytes = 512;
    static constexpr int kFixedBytes = 1024 + kTilesBytes + kSumBytes + kScaleBytes + kBarrierBytes;
    // Raw stages fill what is left of shared memory (at most 8): the bytes in flight per SM must
    // cover the DRAM latency, about 100 KB at 43 GB/s per SM and ~2 us.
    static constexpr int kRawFit = (227 * 1024 - kFixedBytes) / kRawStageBytes;
    static constexpr int kRawStages = kRawFit > 8 ? 8 : kRawFit;
    static constexpr int kRawBytes = kRawStages * kRawStageBytes;
    static constexpr int kSmemBytes = kFixedBytes + kRawBytes;
    static_assert(kAccSlots % kChunks == 0, "a slot must always see the same token chunk");
    static_assert(kAccSlots * kBM * 16 * 4 <= kAbStages * kATileBytes, "the final partial sums reuse the A tiles");
    static_assert(kRawStages >= 2, "tile plan exceeds shared memory");
    static_assert(kTmemColumns <= 512 && (kTmemColumns & (kTmemColumns - 1)) == 0, "TMEM columns must be a power of two <= 512");
};

template <uint32_t FMT, int NT, bool RAWTMA>
__global__ void __launch_bounds__(kGsThreads, 1)
qgemv_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const TcParams p) {
    using G = GsGeometry<FMT, NT, RAWTMA>;
    using F = Format<FMT>;
    using Q = Quants<FMT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    uint8_t* a_tiles = smem;
    uint8_t* b_tiles = a_tiles + G::kAbStages * G::kATileBytes;
    float* s_ring = reinterpret_cast<float*>(b_tiles + G::kBStages * G::kBTileBytes);   // [step buffer][group][token]
    float* scale_ring = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(s_ring) + G::kSumBytes);   // [stage][row][a.., c..]
    uint8_t* raw = reinterpret_cast<uint8_t*>(scale_ring) + G::kScaleBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(raw + G::kRawBytes);
    uint64_t* raw_full = bars;                        // [kRawStages]
    uint64_t* raw_empty = raw_full + 8;               // [kRawStages], every warp that reads the raw stage
    uint64_t* b_full = raw_empty + 8;                 // [kBStages], activation tile landed (TMA bytes)
    uint64_t* b_empty = b_full + 12;                  // [kBGroups], one tcgen05.commit from each MMA issuer
    uint64_t* ab_full = b_empty + 12;                 // [kAbStages], the four unpack warps of the step
    uint64_t* ab_empty = ab_full + G::kAbStages;      // [kAbStages], tcgen05.commit
    uint64_t* d_full = ab_empty + G::kAbStages;       // [kStepBuffers], tcgen05.commit
    uint64_t* d_empty = d_full + 4;                   // [kStepBuffers], all accumulate warps
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(d_empty + 4);
    uint32_t* last_flag = tmem_holder + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kBM;
    const int m0 = blockIdx.y * NT;
    const int sb_begin = static_cast<int>(static_cast<long long>(p.nsb) * blockIdx.z / p.ksplit);
    const int sb_end = static_cast<int>(static_cast<long long>(p.nsb) * (blockIdx.z + 1) / p.ksplit);
    const int nsb_local = sb_end - sb_begin;
    const int steps = nsb_local * kSub;

    if (threadIdx.x == 0) {
        for (int s = 0; s < G::kRawStages; ++s) {
            mbar_init(&raw_full[s], RAWTMA ? 1 : 32);
            mbar_init(&raw_empty[s], G::kUnpackWarps);
        }
        for (int s = 0; s < G::kAbStages; ++s) {
            mbar_init(&ab_full[s], 4);
            mbar_init(&ab_empty[s], 1);
        }
        for (int s = 0; s < G::kBStages; ++s) mbar_init(&b_full[s], 1);
        for (int s = 0; s < G::kBGroups; ++s) mbar_init(&b_empty[s], 2);
        for (int s = 0; s < G::kStepBuffers; ++s) {
            mbar_init(&d_full[s], 1);
            mbar_init(&d_empty[s], G::kAccWarps);
        }
        mbar_fence_init();
        tma_prefetch_descriptor(&xmap);
        if (RAWTMA) tma_prefetch_descriptor(&wmap);
    }
    if (warp == 1) tmem_alloc(tmem_holder, G::kTmemColumns);
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        // ---------------- producer ----------------
        const unsigned long long safe_end = p.w_bytes & ~15ull;
        bool ok = true;
        for (int i = 0; i < nsb_local && ok; ++i) {
            const int rs = i % G::kRawStages;
            if (i >= G::kRawStages && !mbar_wait_bounded(&raw_empty[rs], ((i / G::kRawStages) - 1) & 1)) {
                atomicExch(p.status, kDeviceWaitTimeout);
                ok = false;
                break;
            }
            if (RAWTMA) {
                if (lane == 0) {
                    const unsigned long long byte_x = (static_cast<unsigned long long>(sb_begin + i) * F::kBytes) & ~15ull;
                    mbar_arrive_expect_tx(&raw_full[rs], kBM * G::kBoxBytes);
                    tma_load_2d(raw + rs * G::kRawStageBytes, &wmap, static_cast<int>(byte_x >> 1), n0, &raw_full[rs]);
                    stamp(p, 3, i, 0);
                }
            } else {
                // Rows that do not start on 16-byte boundaries: four bulk copies per lane, each from
                // the boundary below its block; the last bytes of the tensor by plain loads.
                unsigned long long a0[4];
                uint32_t bytes[4];
                uint32_t total = 0;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int r = lane + 32 * q;
                    const long long row = static_cast<long long>(n0) + r;
                    bytes[q] = 0;
                    a0[q] = 0;
                    if (row < p.n) {
                        const unsigned long long g0 = static_cast<unsigned long long>(row) * p.row_bytes +
                                                      static_cast<unsigned long long>(sb_begin + i) * F::kBytes;
                        const unsigned long long g1 = g0 + F::kBytes;
                        a0[q] = g0 & ~15ull;
                        unsigned long long a1 = (g1 + 15ull) & ~15ull;
                        if (a1 > safe_end) {
                            const unsigned long long bulk_end = safe_end > a0[q] ? safe_end : a0[q];
                            uint8_t* dst = raw + rs * G::kRawStageBytes + r * G::kSlot;
                            for (unsigned long long o = bulk_end; o < g1; ++o) dst[o - a0[q]] = p.w[o];
                            a1 = bulk_end;
                        }
                        bytes[q] = static_cast<uint32_t>(a1 - a0[q]);
                        total += bytes[q];
                    }
                }
                if (total > 0) {
                    mbar_arrive_expect_tx(&raw_full[rs], total);
                } else {
                    mbar_arrive(&raw_full[rs]);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    if (bytes[q] > 0)
                        bulk_copy_g2s(raw + rs * G::kRawStageBytes + (lane + 32 * q) * G::kSlot, p.w + a0[q], bytes[q], &raw_full[rs]);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
    } else if (warp == kActivationWarp) {
        // ---------------- activation producer ----------------
        if (lane == 0) {
            for (int i = 0; i < nsb_local; ++i) {
                const int g = i % G::kBGroups;
                if (i >= G::kBGroups && !mbar_wait_bounded(&b_empty[g], ((i / G::kBGroups) - 1) & 1)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    break;
                }
                for (int t = 0; t < kSub; ++t) {
                    const int bs = g * kSub + t;
                    mbar_arrive_expect_tx(&b_full[bs], G::kBTileBytes);
                    tma_load_2d(b_tiles + bs * G::kBTileBytes, &xmap, (sb_begin + i) * kSuperBlock + t * kBK, m0, &b_full[bs]);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == kSecondMmaWarp) {
        // ---------------- MMA issuers: all groups of a K step, then the commits ----------------
        // The unpack warps have already waited for the activation tile and for the TMEM step buffer
        // before they arrive on ab_full, so one wait covers all three conditions.
        if (lane == 0) {
            constexpr uint32_t idesc = umma_instr_desc(kBM, NT, /*A bf16*/ 1, /*B bf16*/ 1);
            const int first = warp == 1 ? 0 : 1;
            for (int j = first; j < steps; j += 2) {
                const int as = j % G::kAbStages;
                const int bs = j % G::kBStages;
                const int sbuf = j % G::kStepBuffers;
                if (!mbar_wait_bounded(&ab_full[as], (j / G::kAbStages) & 1)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    break;
                }
                tcgen05_fence_after_sync();
                stamp(p, 0, j, 0);
                const uint64_t desc_a = umma_smem_desc_sw128(smem_addr(a_tiles + as * G::kATileBytes));
                const uint64_t desc_b = umma_smem_desc_sw128(smem_addr(b_tiles + bs * G::kBTileBytes));
#pragma unroll
                for (int gg = 0; gg < G::kGroupsPerStep; ++gg) {
                    const uint32_t d_addr = tmem_base + sbuf * G::kStepCols + gg * NT;
#pragma unroll
                    for (int kk = 0; kk < G::kMmasPerGroup; ++kk) {
                        const int k16 = gg * G::kMmasPerGroup + kk;  // 32 bytes along the swizzled row per K=16
                        umma_f16(d_addr, desc_a + 2 * k16, desc_b + 2 * k16, idesc, kk > 0);
                    }
                }
                umma_commit(&d_full[sbuf]);
                umma_commit(&ab_empty[as]);
                // the last two steps of a super-block (one per issuer) release its four activation tiles
                if ((j & (kSub - 1)) >= kSub - 2) umma_commit(&b_empty[(j / kSub) % G::kBGroups]);
                stamp(p, 0, j, 1);
            }
        }
        __syncwarp();
    }
    else if (warp >= 2 + G::kAccWarps && warp < kActivationWarp) {
        // ---------------- unpack warps: raw bytes -> bf16 quants; group sums of the activations ----------------
        const int r = (threadIdx.x - G::kFirstUnpackThread) & (kBM - 1);    // one thread per weight row and slot
        const int unpack_slot = (threadIdx.x - G::kFirstUnpackThread) >> 7;  // this warp takes K steps j with j % slots == slot
        const long long row = static_cast<long long>(n0) + r;
        const bool row_ok = row < p.n;
        const uint32_t row_off = (r >> 3) * 1024 + (r & 7) * 128;
        const uint32_t sw = r & 7;
        bool ok = true;
        for (int i = 0; i < nsb_local && ok; ++i) {
            const int rs = i % G::kRawStages;
            if (!mbar_wait_bounded(&raw_full[rs], (i / G::kRawStages) & 1)) {
                atomicExch(p.status, kDeviceWaitTimeout);
                ok = false;
                break;
            }
            const unsigned long long g0 = (RAWTMA ? 0ull : static_cast<unsigned long long>(row) * p.row_bytes) +
                                          static_cast<unsigned long long>(sb_begin + i) * F::kBytes;
            const uint8_t* blk = raw + rs * G::kRawStageBytes + r * G::kSlot + static_cast<uint32_t>(g0 & 15ull);
            if (r == 0 && unpack_slot == 0) stamp(p, 3, i, 1);
#pragma unroll
            for (int t = 0; t < kSub; ++t) {
                if ((t & (G::kUnpackSlots - 1)) != unpack_slot) continue;
                const int j = i * kSub + t;
                const int as = j % G::kAbStages;
                const int sbuf = j % G::kStepBuffers;
                if (j >= G::kAbStages && !mbar_wait_bounded(&ab_empty[as], ((j / G::kAbStages) - 1) & 1)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    ok = false;
                    break;
                }
                if (r == 0) stamp(p, 1, j, 0);
                uint8_t* tile = a_tiles + as * G::kATileBytes + row_off;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint4 out[4];
                    if (row_ok) {
                        Q::step(blk, t, h, out);
                    } else {
#pragma unroll
                        for (int c = 0; c < 4; ++c) out[c] = make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        *reinterpret_cast<uint4*>(tile + ((static_cast<uint32_t>(Q::chunk_index(h, c)) ^ sw) << 4)) = out[c];
                }
                if (r == 0) stamp(p, 1, j, 1);
                // The MMA of this step needs the activation tile and a free TMEM step buffer as well; waiting
                // for both here lets the issuer wait on ab_full alone.
                const int bs = j % G::kBStages;
                if (!mbar_wait_bounded(&b_full[bs], (j / G::kBStages) & 1) ||
                    (j >= G::kStepBuffers && !mbar_wait_bounded(&d_empty[sbuf], ((j / G::kStepBuffers) - 1) & 1))) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    ok = false;
                    break;
                }
                if (t == 0 && unpack_slot == 0) {
                    // Group scales of this row for the accumulate warps.  Entry i % 2 was last read for super-block
                    // i - 2, which the accumulate warps finished before this warp could get here: its wait for the
                    // TMEM buffer of this step follows the accumulation of step 4(i-1), the first of super-block i-1.
                    float ga[Q::kGroupsPerSb], gcoef[Q::kGroupsPerSb];
                    if (row_ok) {
                        Q::group_scales(blk, ga, gcoef);
                    } else {
#pragma unroll
                        for (int g = 0; g < Q::kGroupsPerSb; ++g) ga[g] = gcoef[g] = 0.0f;
                    }
                    float* dst = scale_ring + ((i % G::kScaleStages) * kBM + r) * G::kScaleRow;
#pragma unroll
                    for (int g = 0; g < Q::kGroupsPerSb; g += 4) {
                        *reinterpret_cast<float4*>(dst + g) = make_float4(ga[g], ga[g + 1], ga[g + 2], ga[g + 3]);
                        if (Q::kStoresCoef)
                            *reinterpret_cast<float4*>(dst + Q::kGroupsPerSb + g) = make_float4(gcoef[g], gcoef[g + 1], gcoef[g + 2], gcoef[g + 3]);
                    }
                }
                if (Q::kUsesSum) {
                    // S_g[m] = sum over the group's K range of x[m][k], from the activation tile: a thread sums
                    // one 16-byte chunk (8 values), the chunks of a group are combined across neighbouring lanes.
                    if (r == 0) stamp(p, 1, j, 2);
                    const uint8_t* btile = b_tiles + bs * G::kBTileBytes;
                    float* sums = s_ring + sbuf * G::kGroupsPerStep * NT;
                    constexpr int kChunksPerGroup = Q::kGroup / 8;   // 4, or 2 for Q6_K
#pragma unroll
                    for (int task = r; task < NT * 8; task += kBM) {
                        const int m = task >> 3;
                        const int ck = task & 7;
                        const uint4 v = *reinterpret_cast<const uint4*>(btile + (m >> 3) * 1024 + (m & 7) * 128 + ((ck ^ (m & 7)) << 4));
                        float part = ((__uint_as_float(v.x << 16) + __uint_as_float(v.x & 0xffff0000u)) +
                                      (__uint_as_float(v.y << 16) + __uint_as_float(v.y & 0xffff0000u))) +
                                     ((__uint_as_float(v.z << 16) + __uint_as_float(v.z & 0xffff0000u)) +
                                      (__uint_as_float(v.w << 16) + __uint_as_float(v.w & 0xffff0000u)));
                        part += __shfl_xor_sync(0xffffffffu, part, 1);
                        if (kChunksPerGroup == 4) part += __shfl_xor_sync(0xffffffffu, part, 2);
                        if ((ck & (kChunksPerGroup - 1)) == 0) sums[(ck / kChunksPerGroup) * NT + m] = part;
                    }
                }
                if (r == 0) stamp(p, 1, j, 3);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ab_full[as]);
                if (r == 0) stamp(p, 1, j, 4);
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(&raw_empty[rs]);
            ok = __all_sync(0xffffffffu, ok);
        }
    } else {
        // ---------------- accumulate warps: acc[m] += a_g * D_g[m] - c_g * S_g[m] ----------------
        // Work item = (group, chunk of 16 tokens), numbered group-major; item `it` belongs to slot
        // it % 4 of each quadrant.  kChunks divides 4, so a slot always holds the same token chunk.
        const int q = warp & 3;                        // TMEM lanes 32*(warp % 4) .. +31
        const int slot = (warp - 2) >> 2;
        const int chunk = slot % G::kChunks;
        const int rrow = q * 32 + lane;
        const long long row = static_cast<long long>(n0) + rrow;
        const bool row_ok = row < p.n;
        float acc[16];
#pragma unroll
        for (int m = 0; m < 16; ++m) acc[m] = 0.0f;
        bool ok = true;
        for (int i = 0; i < nsb_local && ok; ++i) {
            const float* scales = scale_ring + ((i % G::kScaleStages) * kBM + rrow) * G::kScaleRow;
#pragma unroll
            for (int t = 0; t < kSub; ++t) {
                const int j = i * kSub + t;
                const int sbuf = j % G::kStepBuffers;
                if (!mbar_wait_bounded(&d_full[sbuf], (j / G::kStepBuffers) & 1)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    ok = false;
                    break;
                }
                tcgen05_fence_after_sync();
                if (warp == 2 && lane == 0) stamp(p, 2, j, 0);
#pragma unroll
                for (int gg = 0; gg < G::kGroupsPerStep; ++gg) {
                    const int item = (j * G::kGroupsPerStep + gg) * G::kChunks + chunk;
                    if ((item & (G::kAccSlots - 1)) != slot) continue;
                    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + sbuf * G::kStepCols + gg * NT + chunk * 16;
                    uint32_t dv[16];
                    tmem_ld16(taddr, dv);
                    float sv[16];
                    if (Q::kUsesSum) {
                        const float4* sp = reinterpret_cast<const float4*>(s_ring + (sbuf * G::kGroupsPerStep + gg) * NT + chunk * 16);
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float4 f = sp[u];
                            sv[4 * u] = f.x; sv[4 * u + 1] = f.y; sv[4 * u + 2] = f.z; sv[4 * u + 3] = f.w;
                        }
                    }
                    tmem_ld_wait();
                    const float a_g = scales[t * G::kGroupsPerStep + gg];
                    const float c_g = Q::kStoresCoef ? -scales[Q::kGroupsPerSb + t * G::kGroupsPerStep + gg] : -160.0f * a_g;
#pragma unroll
                    for (int jj = 0; jj < 16; ++jj) {
                        float v = fmaf(a_g, __uint_as_float(dv[jj]), acc[jj]);
                        if (Q::kUsesSum) v = fmaf(c_g, sv[jj], v);
                        acc[jj] = v;
                    }
                }
                // this warp is done with the step buffer (TMEM columns and the S ring entry)
                tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&d_empty[sbuf]);
                if (warp == 2 && lane == 0) stamp(p, 2, j, 1);
            }
            ok = __all_sync(0xffffffffu, ok);
        }
        if (!ok) atomicExch(p.status, kDeviceWaitTimeout);

        // ---------------- sum the four slots of each quadrant in a fixed order ----------------
        // Every MMA has been consumed once all accumulate warps are here, so the A tiles are free.
        named_barrier_sync(2, G::kAccWarps * 32);
        float* red = reinterpret_cast<float*>(a_tiles);   // [slot][row][16]
#pragma unroll
        for (int jj = 0; jj < 16; jj += 4)
            *reinterpret_cast<float4*>(red + (slot * kBM + rrow) * 16 + jj) = make_float4(acc[jj], acc[jj + 1], acc[jj + 2], acc[jj + 3]);
        named_barrier_sync(2, G::kAccWarps * 32);
        const bool owner = slot < G::kChunks;             // this thread finishes (row, token chunk `slot`)
        const bool split = p.ksplit > 1;
        float* part = split ? p.partial + static_cast<size_t>(blockIdx.z) * p.m * p.n : nullptr;
        if (owner && row_ok) {
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) {
                float total = acc[jj];
                for (int s2 = slot + G::kChunks; s2 < G::kAccSlots; s2 += G::kChunks) total += red[(s2 * kBM + rrow) * 16 + jj];
                const int m = m0 + slot * 16 + jj;
                if (m < p.m) {
                    const size_t o = static_cast<size_t>(m) * p.n + row;
                    if (split) {
                        part[o] = total;
                    } else if (p.y_bf16) {
                        static_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(total);
                    } else {
                        static_cast<float*>(p.y)[o] = total;
                    }
                }
            }
        }
        if (split) {
            // The CTA that draws the last ticket of its tile adds the partial tiles in K order.
            __threadfence();
            named_barrier_sync(2, G::kAccWarps * 32);
            if (threadIdx.x == 64) {
                unsigned int* ticket = p.tickets + blockIdx.y * gridDim.x + blockIdx.x;
                const unsigned int drawn = atomicAdd(ticket, 1u);
                const bool last = drawn == static_cast<unsigned int>(p.ksplit - 1);
                if (last) *ticket = 0;  // ready for the next launch
                *last_flag = last ? 1u : 0u;
            }
            named_barrier_sync(2, G::kAccWarps * 32);
            if (*last_flag != 0 && row_ok) {
                __threadfence();
                // all sixteen warps share the tile: slot s takes tokens m0 + 4s .. +3, then strides of 16
                const size_t plane = static_cast<size_t>(p.m) * p.n;
                const int m_end = min(m0 + NT, p.m);
                for (int m = m0 + 4 * slot; m < m_end; m += 4 * G::kAccSlots) {
                    float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    size_t o[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) o[u] = static_cast<size_t>(min(m + u, m_end - 1)) * p.n + row;
#pragma unroll 4
                    for (int z = 0; z < p.ksplit; ++z) {
#pragma unroll
                        for (int u = 0; u < 4; ++u) sum[u] += __ldcg(p.partial + z * plane + o[u]);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (m + u < m_end) {
                            if (p.y_bf16) {
                                static_cast<__nv_bfloat16*>(p.y)[o[u]] = __float2bfloat16_rn(sum[u]);
                            } else {
                                static_cast<float*>(p.y)[o[u]] = sum[u];
                            }
                        }
                    }
                }
            }
        }
    }

    // ---------------- teardown ----------------
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, G::kTmemColumns);
}

template <uint32_t FMT, int NT, bool RAWTMA>
cudaError_t launch_tile(const TcArgs& a) {
    using G = GsGeometry<FMT, NT, RAWTMA>;
    auto kernel = qgemv_tc_kernel<FMT, NT, RAWTMA>;
    static int configured_device = -1;
    int device = 0;
    cudaGetDevice(&device);
    if (configured_device != device) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G::kSmemBytes);
        if (e != cudaSuccess) return e;
        configured_device = device;
    }
    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) return cudaErrorNotSupported;
    CUtensorMap map;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.k), static_cast<cuuint64_t>(a.m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.k) * 2};
    const cuuint32_t box[2] = {kBK, NT};
    const cuuint32_t elem[2] = {1, 1};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a.x), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    TcParams p;
    p.w = a.weights;
    p.w_bytes = a.weight_bytes;
    p.row_bytes = a.value_type == kQ8_0 ? static_cast<unsigned long long>(a.k / 32) * 34
                                        : static_cast<unsigned long long>(a.k / kSuperBlock) * Format<FMT>::kBytes;
    CUtensorMap wmap = map;  // unused unless RAWTMA
    if (RAWTMA) {
        const cuuint64_t wdims[2] = {static_cast<cuuint64_t>(p.row_bytes / 2), static_cast<cuuint64_t>(a.n)};
        const cuuint64_t wstrides[1] = {static_cast<cuuint64_t>(p.row_bytes)};
        const cuuint32_t wbox[2] = {G::kBoxBytes / 2, kBM};
        if (encode(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<uint8_t*>(a.weights), wdims, wstrides, wbox, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    p.y = a.y;
    p.partial = static_cast<float*>(a.scratch);
    p.tickets = a.tickets;
    p.k = a.k;
    p.n = a.n;
    p.m = a.m;
    p.nsb = a.k / kSuperBlock;
    p.y_bf16 = a.y_bf16 ? 1 : 0;
    p.status = a.device_status;
    p.trace = a.trace;
    const int n_tiles = (a.n + kBM - 1) / kBM;
    const int m_tiles = (a.m + NT - 1) / NT;
    p.ksplit = choose_ksplit(n_tiles * m_tiles, p.nsb, a.sm_count, static_cast<size_t>(a.m) * a.n * sizeof(float),
                             a.scratch_bytes, a.ticket_count);
    if (a.force_ksplit > 0 && a.force_ksplit <= p.nsb &&
        static_cast<size_t>(a.m) * a.n * sizeof(float) * a.force_ksplit <= a.scratch_bytes && n_tiles * m_tiles <= a.ticket_count)
        p.ksplit = a.force_ksplit;
    const dim3 grid(n_tiles, m_tiles, p.ksplit);
    kernel<<<grid, kGsThreads, G::kSmemBytes, a.stream>>>(map, wmap, p);
    return cudaGetLastError();
}

template <uint32_t FMT, bool RAWTMA>
cudaError_t launch_tokens(const TcArgs& a) {
    if (a.m <= 16) return launch_tile<FMT, 16, RAWTMA>(a);
    if (a.m <= 32) return launch_tile<FMT, 32, RAWTMA>(a);
    return launch_tile<FMT, 64, RAWTMA>(a);
}

template <uint32_t FMT>
cudaError_t launch_format(const TcArgs& a) {
    const unsigned long long row_bytes = a.value_type == kQ8_0 ? static_cast<unsigned long long>(a.k / 32) * 34
                                                               : static_cast<unsigned long long>(a.k / kSuperBlock) * Format<FMT>::kBytes;
    if (row_bytes % 16 == 0 && a.force_row_copies == 0) return launch_tokens<FMT, true>(a);
    return launch_tokens<FMT, false>(a);
}

}  // namespace

// Members 1..64 (larger batches tile over blockIdx.y in steps of 64), bf16 activations, K a multiple of 256.
cudaError_t launch_qgemv_tc(const TcArgs& a) {
    switch (a.value_type) {
        case kQ4_K: return launch_format<kQ4_K>(a);
        case kQ5_K: return launch_format<kQ5_K>(a);
        case kQ6_K: return launch_format<kQ6_K>(a);
        case kQ8_0: return launch_format<kQ8_0>(a);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ribn
