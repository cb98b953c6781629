// Quantized GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) with the
// dequantisation fused into the operand producer.
//
//   Y[m][n] = sum_k dequant(W[n][k]) * X[m][k]      X bf16 [M][K], f32 accumulate
//
// The reference has no such kernel: its prefill runs the batched GEMV eight
// tokens at a time (crates/nvidia/src/decode.rs:1953-1977, :2149-2267 over
// q4_k.cu:161-258 and twins), and batches above eight are not served at all
// (crates/nvidia/src/quantized.rs:464-469).  This kernel serves every batch the
// CUDA-core GEMV kernels do not: members 5..64 of ribn_gemv and ribn_gemm.
//
// Shape of one CTA: 128 weight rows (the UMMA M dimension, one TMEM lane per
// row) x NT tokens (the UMMA N dimension, NT in {16,32,64,128,256}) x a range
// of K.  Per 64-wide K step:
//   A = 128 x 64 dequantised weights as two bf16 tiles (high and low part, see
//       below), K-major, 128-byte swizzle, written to shared memory by eight
//       dequant warps from the raw GGUF bytes that a producer warp streams in
//       with untiled bulk copies (one per row and super-block, completion on
//       mbarriers);
//   B = NT x 64 activations, bf16, brought by one tiled TMA load in the same
//       swizzled layout (rows past M read as zero);
//   D (TMEM, f32) += A_high * B + A_low * B  with eight tcgen05.mma (K = 16
//       each) issued by one thread; tcgen05.commit releases the stage.
// The epilogue reads D with tcgen05.ld (thread = weight row, registers =
// tokens) and stores Y.  With split-K the partial tiles go to a scratch buffer
// and the last CTA of a tile (an atomic ticket, no spinning) adds them in a
// fixed order, so results are deterministic.
//
// Precision: a single bf16 rounding of the weights (2^-9 relative) does not
// meet the 2e-3 bound of the path over millions of outputs.  Each exact f32
// weight is therefore split into w_high = bf16(w) and w_low = bf16(w - w_high)
// (together 16 significant bits, 2^-17 relative); both operands of every MMA
// are bf16, the activations are used as they are, and the extra MMA is free
// where the kernel is bound by the weight stream.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets the status
// word, and every warp still reaches the common teardown that frees TMEM.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "formats.cuh"
#include "internal.h"
#include "tc_host.h"
#include "tcgen05.cuh"

namespace ribn {
namespace {

constexpr int kBM = 128;            // weight rows per CTA
constexpr int kBK = 64;             // K elements per UMMA stage (one 128-byte swizzled row)
constexpr int kSub = kSuperBlock / kBK;  // stages per super-block
constexpr float kPreScale = 1.0f;   // weights are not pre-scaled: bf16 has the f32 exponent range
constexpr int kDequantWarps = 8;
constexpr int kTcThreads = (2 + kDequantWarps) * 32;

__device__ __forceinline__ uint4 raw16(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint4 raw16_a2(const uint8_t* p) {
    uint4 v;
    v.x = ld_u32_a2(p);
    v.y = ld_u32_a2(p + 4);
    v.z = ld_u32_a2(p + 8);
    v.w = ld_u32_a2(p + 12);
    return v;
}

// Two f32 weights -> a word of their bf16 high parts and a word of the bf16 remainders.
__device__ __forceinline__ void split_pair(float w0, float w1, uint32_t& high, uint32_t& low) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(w0, w1);
    high = *reinterpret_cast<const uint32_t*>(&h);
    const float h0 = __uint_as_float(high << 16);
    const float h1 = __uint_as_float(high & 0xffff0000u);
    const __nv_bfloat162 l = __floats2bfloat162_rn(w0 - h0, w1 - h1);
    low = *reinterpret_cast<const uint32_t*>(&l);
}

// A 16-byte chunk (eight weights) of the high tile and the matching chunk of the low tile.
struct ChunkPair {
    uint4 high, low;
};

// Eight weights (two packed words of four byte-sized quants) -> one chunk pair.
__device__ __forceinline__ ChunkPair chunk_from_bytes(uint32_t q0, uint32_t q1, float bias, float scale, float minimum) {
    float a[4], b[4];
    bytes_to_float4(q0, bias, a);
    bytes_to_float4(q1, bias, b);
    ChunkPair out;
    split_pair(dequant_value(scale, a[0], minimum), dequant_value(scale, a[1], minimum), out.high.x, out.low.x);
    split_pair(dequant_value(scale, a[2], minimum), dequant_value(scale, a[3], minimum), out.high.y, out.low.y);
    split_pair(dequant_value(scale, b[0], minimum), dequant_value(scale, b[1], minimum), out.high.z, out.low.z);
    split_pair(dequant_value(scale, b[2], minimum), dequant_value(scale, b[3], minimum), out.high.w, out.low.w);
    return out;
}

// One thread owns one weight row and one half (h = 0/1) of every 64-wide K step.  Per step it
// produces four 16-byte chunks (32 weights); chunk c of a row covers K offsets 8c .. 8c+7.
//   K-quants: chunks 2h, 2h+1 (first group of the step) and 4+2h, 4+2h+1 (second group)
//   Q8_0:     chunks 4h .. 4h+3 (block 2t+h of the super-block)
template <uint32_t FMT>
struct RowDequant;

template <>
struct RowDequant<kQ4_K> {
    struct Scales { float a[8], b[8]; };
    __device__ static void load_scales(const uint8_t* blk, Scales& s) {
        const uint4 h = raw16(blk);
        const float d = f16_bits_to_f32(h.x & 0xffffu) * kPreScale;
        const float dmin = f16_bits_to_f32(h.x >> 16) * kPreScale;
        uint32_t sc_lo, sc_hi, m_lo, m_hi;
        unpack_k_scales(h.y, h.z, h.w, sc_lo, sc_hi, m_lo, m_hi);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            s.a[g] = d * byte_of(g < 4 ? sc_lo : sc_hi, g & 3);
            s.b[g] = dmin * byte_of(g < 4 ? m_lo : m_hi, g & 3);
        }
    }
    __device__ static int chunk_index(int h, int c) { return (c >> 1) * 4 + 2 * h + (c & 1); }
    __device__ static void step(const uint8_t* blk, const Scales& s, int t, int h, ChunkPair (&out)[4]) {
        const uint4 w = raw16(blk + 16 + 32 * t + 16 * h);
        out[0] = chunk_from_bytes(w.x & 0x0f0f0f0fu, w.y & 0x0f0f0f0fu, 0.0f, s.a[2 * t], s.b[2 * t]);
        out[1] = chunk_from_bytes(w.z & 0x0f0f0f0fu, w.w & 0x0f0f0f0fu, 0.0f, s.a[2 * t], s.b[2 * t]);
        out[2] = chunk_from_bytes((w.x >> 4) & 0x0f0f0f0fu, (w.y >> 4) & 0x0f0f0f0fu, 0.0f, s.a[2 * t + 1], s.b[2 * t + 1]);
        out[3] = chunk_from_bytes((w.z >> 4) & 0x0f0f0f0fu, (w.w >> 4) & 0x0f0f0f0fu, 0.0f, s.a[2 * t + 1], s.b[2 * t + 1]);
    }
};

template <>
struct RowDequant<kQ5_K> {
    using Scales = RowDequant<kQ4_K>::Scales;
    __device__ static void load_scales(const uint8_t* blk, Scales& s) { RowDequant<kQ4_K>::load_scales(blk, s); }
    __device__ static int chunk_index(int h, int c) { return RowDequant<kQ4_K>::chunk_index(h, c); }
    __device__ static uint32_t lo5(uint32_t w, uint32_t hb, int g) { return (w & 0x0f0f0f0fu) | (((hb >> g) & 0x01010101u) << 4); }
    __device__ static uint32_t hi5(uint32_t w, uint32_t hb, int g) {
        return ((w >> 4) & 0x0f0f0f0fu) | (((hb >> g) & 0x01010101u) << 4);
    }
    __device__ static void step(const uint8_t* blk, const Scales& s, int t, int h, ChunkPair (&out)[4]) {
        const uint4 w = raw16(blk + 48 + 32 * t + 16 * h);
        const uint4 hb = raw16(blk + 16 + 16 * h);
        const int g = 2 * t;
        out[0] = chunk_from_bytes(lo5(w.x, hb.x, g), lo5(w.y, hb.y, g), 0.0f, s.a[g], s.b[g]);
        out[1] = chunk_from_bytes(lo5(w.z, hb.z, g), lo5(w.w, hb.w, g), 0.0f, s.a[g], s.b[g]);
        out[2] = chunk_from_bytes(hi5(w.x, hb.x, g + 1), hi5(w.y, hb.y, g + 1), 0.0f, s.a[g + 1], s.b[g + 1]);
        out[3] = chunk_from_bytes(hi5(w.z, hb.z, g + 1), hi5(w.w, hb.w, g + 1), 0.0f, s.a[g + 1], s.b[g + 1]);
    }
};

template <>
struct RowDequant<kQ6_K> {
    struct Scales { float a[16]; };
    __device__ static void load_scales(const uint8_t* blk, Scales& s) {
        const float d = f16_bits_to_f32(ld_u16(blk + 208)) * kPreScale;
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
            const uint32_t pair = ld_u16(blk + 192 + i);
            s.a[i] = d * static_cast<float>(static_cast<int8_t>(pair & 0xffu));
            s.a[i + 1] = d * static_cast<float>(static_cast<int8_t>(pair >> 8));
        }
    }
    __device__ static int chunk_index(int h, int c) { return RowDequant<kQ4_K>::chunk_index(h, c); }
    // Step t covers groups 2t and 2t+1 = variants v, v+1 of chunk c = t/2 with v = 2*(t%2):
    // group 2t reads ql[c*64 + p], group 2t+1 reads ql[c*64 + 32 + p], low nibble when t is even,
    // high nibble when odd; both take two bits of qh[c*32 + p], at shifts 2v and 2v+2.
    __device__ static uint32_t q6(uint32_t l, uint32_t hb, int nib, int shift) {
        return ((l >> nib) & 0x0f0f0f0fu) | (((hb >> shift) & 0x03030303u) << 4);
    }
    __device__ static void step(const uint8_t* blk, const Scales& s, int t, int h, ChunkPair (&out)[4]) {
        const int c = t >> 1;
        const int nib = (t & 1) * 4;
        const int v2 = (t & 1) * 4;  // 2 * variant of the first group
        const uint4 l0 = raw16_a2(blk + c * 64 + 16 * h);
        const uint4 l1 = raw16_a2(blk + c * 64 + 32 + 16 * h);
        const uint4 hb = raw16_a2(blk + 128 + c * 32 + 16 * h);
        const float s0 = h ? s.a[4 * t + 1] : s.a[4 * t];      // scale index 2*group + position/16
        const float s1 = h ? s.a[4 * t + 3] : s.a[4 * t + 2];
        out[0] = chunk_from_bytes(q6(l0.x, hb.x, nib, v2), q6(l0.y, hb.y, nib, v2), 32.0f, s0, 0.0f);
        out[1] = chunk_from_bytes(q6(l0.z, hb.z, nib, v2), q6(l0.w, hb.w, nib, v2), 32.0f, s0, 0.0f);
        out[2] = chunk_from_bytes(q6(l1.x, hb.x, nib, v2 + 2), q6(l1.y, hb.y, nib, v2 + 2), 32.0f, s1, 0.0f);
        out[3] = chunk_from_bytes(q6(l1.z, hb.z, nib, v2 + 2), q6(l1.w, hb.w, nib, v2 + 2), 32.0f, s1, 0.0f);
    }
};

template <>
struct RowDequant<kQ8_0> {
    struct Scales { float d[8]; };
    __device__ static void load_scales(const uint8_t* blk, Scales& s) {
#pragma unroll
        for (int b = 0; b < 8; ++b) s.d[b] = f16_bits_to_f32(ld_u16(blk + 34 * b)) * kPreScale;
    }
    __device__ static int chunk_index(int h, int c) { return 4 * h + c; }
    __device__ static void step(const uint8_t* blk, const Scales& s, int t, int h, ChunkPair (&out)[4]) {
        const uint8_t* q = blk + 34 * (2 * t + h) + 2;
        const uint4 w0 = raw16_a2(q);
        const uint4 w1 = raw16_a2(q + 16);
        const float d = h ? s.d[2 * t + 1] : s.d[2 * t];
        out[0] = chunk_from_bytes(w0.x ^ 0x80808080u, w0.y ^ 0x80808080u, 128.0f, d, 0.0f);
        out[1] = chunk_from_bytes(w0.z ^ 0x80808080u, w0.w ^ 0x80808080u, 128.0f, d, 0.0f);
        out[2] = chunk_from_bytes(w1.x ^ 0x80808080u, w1.y ^ 0x80808080u, 128.0f, d, 0.0f);
        out[3] = chunk_from_bytes(w1.z ^ 0x80808080u, w1.w ^ 0x80808080u, 128.0f, d, 0.0f);
    }
};


// RAWTMA: the raw weight bytes of a stage (128 rows x one super-block) arrive as ONE tiled TMA box
// instead of 128 bulk copies of 144..272 bytes (small bulk copies cost about as much per request
// as large ones, and 128 of them per 18 KB starve the pipeline).  The box is 2-D over the tensor
// viewed as [N rows][row_bytes] of 16-bit elements; it needs row_bytes to be a multiple of 16.
// Q6_K super-blocks (210 bytes) start on 2-byte boundaries: the box starts at the 16-byte
// boundary below and is 240 bytes wide, and the remainder is an offset in shared memory.
template <uint32_t FMT, int NT, bool RAWTMA>
struct TcGeometry {
    using F = Format<FMT>;
    static constexpr int kBoxBytes = FMT == kQ6_K ? 240 : F::kBytes;
    static constexpr int kAbStages = NT >= 256 ? 2 : 3;
    static constexpr int kRawStages = 2;
    // bytes per row in a raw stage: the TMA box width, or a bulk copy from the 16-byte boundary below the block
    static constexpr int kSlot = RAWTMA ? kBoxBytes : ((F::kBytes + 15) / 16) * 16 + 16;
    static constexpr int kRawStageBytes = kBM * kSlot;
    static constexpr int kAPartBytes = kBM * kBK * 2;        // one bf16 tile
    static constexpr int kATileBytes = 2 * kAPartBytes;      // high part, then low part
    static constexpr int kBTileBytes = NT * kBK * 2;
    static constexpr int kTilesBytes = kAbStages * (kATileBytes + kBTileBytes);
    static constexpr int kRawBytes = kRawStages * kRawStageBytes;
    static constexpr int kBarrierBytes = 256;
    static constexpr int kSmemBytes = 1024 + kTilesBytes + kRawBytes + kBarrierBytes;  // 1024: alignment slack
    static constexpr int kTmemColumns = NT < 32 ? 32 : NT;
    static_assert(kSmemBytes <= 227 * 1024, "tile plan exceeds shared memory");
};

template <uint32_t FMT, int NT, bool RAWTMA>
__global__ void __launch_bounds__(kTcThreads, 1)
qgemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const TcParams p) {
    using G = TcGeometry<FMT, NT, RAWTMA>;
    using F = Format<FMT>;
    using R = RowDequant<FMT>;
    extern __shared__ uint8_t smem_raw[];
    // The swizzled tiles need a 1024-byte aligned base.
    uint8_t* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    uint8_t* a_tiles = smem;
    uint8_t* b_tiles = a_tiles + G::kAbStages * G::kATileBytes;
    uint8_t* raw = b_tiles + G::kAbStages * G::kBTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(raw + G::kRawBytes);
    uint64_t* raw_full = bars;                       // [kRawStages], 32 producer lanes
    uint64_t* raw_empty = raw_full + G::kRawStages;  // [kRawStages], 8 dequant warps
    uint64_t* ab_full = raw_empty + G::kRawStages;   // [kAbStages], 8 dequant warps + 1 TMA issuer
    uint64_t* ab_empty = ab_full + G::kAbStages;     // [kAbStages], 1 tcgen05.commit
    uint64_t* acc_full = ab_empty + G::kAbStages;    // 1 tcgen05.commit
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_full + 1);
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
            mbar_init(&raw_empty[s], kDequantWarps);
        }
        for (int s = 0; s < G::kAbStages; ++s) {
            mbar_init(&ab_full[s], kDequantWarps + 1);
            mbar_init(&ab_empty[s], 1);
        }
        mbar_init(acc_full, 1);
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
        // ---------------- producer: raw weight bytes (bulk copies) and activation tiles (TMA) ----------------
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
                }
            } else {
            // Each lane brings four rows of the stage: one arrive with the byte total, then the copies.
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
                        // Last bytes of a tensor whose length is not a multiple of 16: plain loads.
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
            // Activation tiles of the four K steps of this super-block.
            if (lane == 0) {
                for (int t = 0; t < kSub; ++t) {
                    const int j = i * kSub + t;
                    const int as = j % G::kAbStages;
                    if (j >= G::kAbStages && !mbar_wait_bounded(&ab_empty[as], ((j / G::kAbStages) - 1) & 1)) {
                        atomicExch(p.status, kDeviceWaitTimeout);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&ab_full[as], G::kBTileBytes);
                    tma_load_2d(b_tiles + as * G::kBTileBytes, &xmap, (sb_begin + i) * kSuperBlock + t * kBK, m0, &ab_full[as]);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: one thread ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_instr_desc(kBM, NT, /*A bf16*/ 1, /*B bf16*/ 1);
            for (int j = 0; j < steps; ++j) {
                const int as = j % G::kAbStages;
                if (!mbar_wait_bounded(&ab_full[as], (j / G::kAbStages) & 1)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    break;
                }
                tcgen05_fence_after_sync();
                const uint64_t desc_high = umma_smem_desc_sw128(smem_addr(a_tiles + as * G::kATileBytes));
                const uint64_t desc_low = umma_smem_desc_sw128(smem_addr(a_tiles + as * G::kATileBytes + G::kAPartBytes));
                const uint64_t desc_b = umma_smem_desc_sw128(smem_addr(b_tiles + as * G::kBTileBytes));
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk) {
                    // 16 K elements = 32 bytes further along the swizzled row: +2 in the address field
                    umma_f16(tmem_base, desc_high + 2 * kk, desc_b + 2 * kk, idesc, j > 0 || kk > 0);
                    umma_f16(tmem_base, desc_low + 2 * kk, desc_b + 2 * kk, idesc, true);
                }
                umma_commit(&ab_empty[as]);
            }
            umma_commit(acc_full);
        }
        __syncwarp();
    } else {
        // ---------------- dequant warps: raw bytes -> f16 A tiles ----------------
        const int t256 = threadIdx.x - 64;
        const int r = t256 & (kBM - 1);
        const int h = t256 >> 7;
        const long long row = static_cast<long long>(n0) + r;
        const bool row_ok = row < p.n;
        // Swizzled position of chunk c of row r: (r/8)*1024 + (r%8)*128 + ((c ^ (r%8)) * 16)
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
            // With the TMA box rows are 16-byte aligned, so only the block's offset inside its row counts.
            const unsigned long long g0 = (RAWTMA ? 0ull : static_cast<unsigned long long>(row) * p.row_bytes) +
                                          static_cast<unsigned long long>(sb_begin + i) * F::kBytes;
            const uint8_t* blk = raw + rs * G::kRawStageBytes + r * G::kSlot + static_cast<uint32_t>(g0 & 15ull);
            typename R::Scales scales;
            if (row_ok) R::load_scales(blk, scales);
#pragma unroll
            for (int t = 0; t < kSub; ++t) {
                const int j = i * kSub + t;
                const int as = j % G::kAbStages;
                if (j >= G::kAbStages && !mbar_wait_bounded(&ab_empty[as], ((j / G::kAbStages) - 1) & 1)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    ok = false;
                    break;
                }
                uint8_t* tile = a_tiles + as * G::kATileBytes + row_off;
                ChunkPair out[4];
                if (row_ok) {
                    R::step(blk, scales, t, h, out);
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c) out[c].high = out[c].low = make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t chunk_off = (static_cast<uint32_t>(R::chunk_index(h, c)) ^ sw) << 4;
                    *reinterpret_cast<uint4*>(tile + chunk_off) = out[c].high;
                    *reinterpret_cast<uint4*>(tile + G::kAPartBytes + chunk_off) = out[c].low;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ab_full[as]);
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(&raw_empty[rs]);
            ok = __all_sync(0xffffffffu, ok);
        }
    }

    // ---------------- epilogue: TMEM -> registers -> Y (or split-K partials) ----------------
    if (warp >= 2 && warp < 6) {
        const int q = warp & 3;                 // a warp may only read TMEM lanes 32*(warp%4) .. +31
        const long long row = static_cast<long long>(n0) + q * 32 + lane;
        const bool ok = mbar_wait_bounded(acc_full, 0);
        if (!ok) atomicExch(p.status, kDeviceWaitTimeout);
        tcgen05_fence_after_sync();
        const bool split = p.ksplit > 1;
        float* part = split ? p.partial + static_cast<size_t>(blockIdx.z) * p.m * p.n : nullptr;
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < NT; c0 += 16) {
                if (m0 + c0 >= p.m) break;
                uint32_t v[16];
                tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c0, v);
                tmem_ld_wait();
                if (row < p.n) {
#pragma unroll
                    for (int jj = 0; jj < 16; ++jj) {
                        const int m = m0 + c0 + jj;
                        if (m < p.m) {
                            const float value = __uint_as_float(v[jj]) * (1.0f / kPreScale);
                            const size_t o = static_cast<size_t>(m) * p.n + row;
                            if (split) {
                                part[o] = value;
                            } else if (p.y_bf16) {
                                static_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(value);
                            } else {
                                static_cast<float*>(p.y)[o] = value;
                            }
                        }
                    }
                }
            }
        }
    }

    // ---------------- split-K: the CTA that draws the last ticket of its tile adds the partial tiles ----------------
    if (p.ksplit > 1 && warp >= 2) {
        // All eight dequant warps take part (they are idle by now): 256 threads, two per weight row.
        __threadfence();
        named_barrier_sync(2, kDequantWarps * 32);
        if (threadIdx.x == 64) {
            unsigned int* ticket = p.tickets + blockIdx.y * gridDim.x + blockIdx.x;
            const unsigned int drawn = atomicAdd(ticket, 1u);
            const bool last = drawn == static_cast<unsigned int>(p.ksplit - 1);
            if (last) *ticket = 0;  // ready for the next launch
            *last_flag = last ? 1u : 0u;
        }
        named_barrier_sync(2, kDequantWarps * 32);
        const int t256 = threadIdx.x - 64;
        const long long row = static_cast<long long>(n0) + (t256 & (kBM - 1));
        if (*last_flag != 0 && row < p.n) {
            __threadfence();
            const size_t plane = static_cast<size_t>(p.m) * p.n;
            const int m_end = min(m0 + NT, p.m);
            // Four tokens at a time, so that four independent loads per K slice are in flight;
            // the slices are added in index order whatever the arrival order was.
            for (int m = m0 + 4 * (t256 >> 7); m < m_end; m += 8) {
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

    // ---------------- teardown: every warp arrives here, then TMEM is released ----------------
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, G::kTmemColumns);
}

template <uint32_t FMT, int NT, bool RAWTMA>
cudaError_t launch_tile(const TcArgs& a) {
    using G = TcGeometry<FMT, NT, RAWTMA>;
    auto kernel = qgemm_tc_kernel<FMT, NT, RAWTMA>;
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
    p.trace = nullptr;
    const int n_tiles = (a.n + kBM - 1) / kBM;
    const int m_tiles = (a.m + NT - 1) / NT;
    p.ksplit = choose_ksplit(n_tiles * m_tiles, p.nsb, a.sm_count, static_cast<size_t>(a.m) * a.n * sizeof(float),
                             a.scratch_bytes, a.ticket_count);
    if (a.force_ksplit > 0 && a.force_ksplit <= p.nsb &&
        static_cast<size_t>(a.m) * a.n * sizeof(float) * a.force_ksplit <= a.scratch_bytes && n_tiles * m_tiles <= a.ticket_count)
        p.ksplit = a.force_ksplit;
    const dim3 grid(n_tiles, m_tiles, p.ksplit);
    kernel<<<grid, kTcThreads, G::kSmemBytes, a.stream>>>(map, wmap, p);
    return cudaGetLastError();
}

template <uint32_t FMT, bool RAWTMA>
cudaError_t launch_tokens(const TcArgs& a) {
    if (a.m <= 16) return launch_tile<FMT, 16, RAWTMA>(a);
    if (a.m <= 32) return launch_tile<FMT, 32, RAWTMA>(a);
    if (a.m <= 64) return launch_tile<FMT, 64, RAWTMA>(a);
    if (a.m <= 128) return launch_tile<FMT, 128, RAWTMA>(a);
    return launch_tile<FMT, 256, RAWTMA>(a);
}

template <uint32_t FMT>
cudaError_t launch_format(const TcArgs& a) {
    // The tiled box needs 16-byte aligned rows; only Q6_K rows can fail that (210-byte blocks).
    const unsigned long long row_bytes = a.value_type == kQ8_0 ? static_cast<unsigned long long>(a.k / 32) * 34
                                                               : static_cast<unsigned long long>(a.k / kSuperBlock) * Format<FMT>::kBytes;
    if (row_bytes % 16 == 0 && a.force_row_copies == 0) return launch_tokens<FMT, true>(a);
    return launch_tokens<FMT, false>(a);
}

}  // namespace

bool qgemm_tc_supports(uint32_t value_type, int k) {
    // Whole 256-element super-blocks only (a Q8_0 row may end inside one; those go to the GEMV kernels).
    return k % kSuperBlock == 0 && (value_type == kQ4_K || value_type == kQ5_K || value_type == kQ6_K || value_type == kQ8_0);
}

cudaError_t launch_qgemm_tc(const TcArgs& a) {
    switch (a.value_type) {
        case kQ4_K: return launch_format<kQ4_K>(a);
        case kQ5_K: return launch_format<kQ5_K>(a);
        case kQ6_K: return launch_format<kQ6_K>(a);
        case kQ8_0: return launch_format<kQ8_0>(a);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ribn
