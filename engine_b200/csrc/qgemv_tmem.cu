// Quantized GEMV / skinny GEMM on the 5th-generation tensor cores with the weight operand unpacked straight
// into tensor memory.
//
//   Y[m][n] = sum_k dequant(W[n][k]) * X[m][k]          m = 1..16 member rows per launch
//
// The path is bound by HBM: a 4.5-bit weight arrives every ~0.025 SM clocks, which leaves about three thread
// instructions per weight, and the integer pipe -- where the bit manipulation of the unpacking runs -- issues
// at half rate.  Two things decide whether a kernel keeps up: instructions per weight, and where the
// dequantised operand lives.  Writing an f16 tile to shared memory for the tensor pipe costs 2 bytes written
// and 2 read per weight against 0.56 streamed; the warp-level mma.sync keeps the operand in registers but makes
// every thread unpack for a 2-row x 4-element fragment and fetch its own B fragment (about three instructions
// per weight).  Here
//   * a thread owns one weight row (one TMEM lane).  It reads the row's raw super-block bytes from the
//     shared-memory ring (tiled TMA boxes of 128 rows x one super-block) and expands two quants at a time
//     with one logic op and one HFMA2:  (q | 0x6400) is the half 1024 + q, and (1024 + q) * sc - 1024 * sc
//     = q * sc is exact in f16 for Q4_K / Q5_K (q * sc <= 1953 < 2048);
//   * the expanded values go to tensor memory with tcgen05.st (32 K elements per instruction and row) and are
//     the A operand of tcgen05.mma (M = 128 rows, K = 16 per instruction, N = 16 columns), so they never
//     pass through shared memory;
//   * the B operand -- the activations as f16, two planes (hi + lo) for f32 inputs -- is a small K-major
//     tile set in shared memory that the CTA converts for its own K range only (CTAs split K), scaled by a
//     power of two per (member, super-block);
//   * the super-block scale d, and dmin times the activations' block sums (one more MMA with the eight
//     6-bit minima as A), are applied in f32 once per super-block and row when the accumulator is read back.
// About 1.3 thread instructions per weight, 0.7 of them on the integer pipe.
//
// CTA = 128 rows x a K range; grid = row tiles x K splits.  Warps 0..7 are workers (thread = row; warps 0..3
// expand the first 128 weights of every super-block, warps 4..7 the second 128, and each half reads back
// half of the accumulator columns), warp 8 streams the raw weights, warp 9 issues the MMAs and owns the TMEM
// allocation.  Partial results of K splits meet in global scratch: the CTA that draws the last ticket of a
// row tile adds them in split order (deterministic).
//
// Every wait on an mbarrier is bounded; a wait that runs out sets the status word and every warp still
// reaches the teardown that frees TMEM.
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

constexpr int kRows = 128;                 // weight rows per CTA = UMMA M = TMEM lanes
constexpr int kWorkerWarps = 8;
constexpr int kWorkers = kWorkerWarps * 32;
constexpr int kProducerWarp = 8;
constexpr int kIssuerWarp = 9;
constexpr int kTmemThreads = 320;
constexpr int kNT = 16;                    // accumulator columns (UMMA N)
constexpr int kPairs = 4;                  // 64-weight pairs of sub-blocks per super-block = A slots in TMEM
constexpr int kPairColumns = 32;           // TMEM columns of one pair: 64 halves per row
constexpr int kDBuffers = 2;
constexpr int kMaxLocalSb = 16;            // super-blocks of one CTA's K range (its B tiles stay resident: 8 KB each)
constexpr int kMaxRawStages = 4;

// TMEM columns: [A pairs: 4 x 32][A minima: 2 x 8][D: 2 buffers x (16 main + 16 minimum term)]
constexpr int kColAMin = kPairs * kPairColumns;
constexpr int kColD = kColAMin + kDBuffers * 8;
constexpr int kTmemColumns = 256;
static_assert(kColD + kDBuffers * 2 * kNT <= kTmemColumns, "TMEM plan");

struct TmemParams {
    const void* x;              // [members][k] (swiglu: [members][2k]) f32 or bf16
    int x_bf16;
    int mode;                   // 0 plain, 1 RMSNorm first, 2 silu(gate) * up
    const float* norm_weight;
    float eps;
    void* y;
    int y_bf16;
    int accumulate;
    float* partial;             // split-K scratch [ksplit][members][n]
    unsigned int* tickets;      // one zero-initialised counter per row tile
    int k, n, nsb, members, planes, ksplit, raw_stages;
    int b_sb;                   // super-blocks the resident B tiles are laid out for (the largest K range of a CTA)
    int* status;
    long long* trace;           // diagnostics (builds with -DRIBN_TRACE): SM clock stamps of CTA 0, or null
};

// trace[(warp * 16 + superblock) * 16 + event] = clock64(), CTA (0,0), lane 0.  Compiled in with -DRIBN_TRACE only.
__device__ __forceinline__ void stamp(const TmemParams& p, int warp, int sb, int event) {
#ifdef RIBN_TRACE
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && (threadIdx.x & 31) == 0 && sb < 16 && event < 16)
        p.trace[(warp * 16 + sb) * 16 + event] = clock64();
#else
    (void)p;
    (void)warp;
    (void)sb;
    (void)event;
#endif
}

template <uint32_t FMT>
struct TmemPlan {
    static constexpr int kSbBytes = Format<FMT>::kBytes;
    static constexpr int kRawStageBytes = kRows * kSbBytes;
    static constexpr int kBTileBytes = kNT * 128;            // 16 columns x 64 K elements, f16
    static_assert(kSbBytes % 16 == 0, "rows of a raw stage must stay 16-byte aligned");
    // shared memory: [raw ring][B tiles: 4 per super-block][sum tiles: 1 per 4 super-blocks][scale: f32 [sb][16]]
    //                [norm scratch][barriers]
    __host__ __device__ static constexpr size_t b_bytes(int local_sb) { return static_cast<size_t>(local_sb) * 4 * kBTileBytes; }
    __host__ __device__ static constexpr size_t sums_bytes(int local_sb) { return static_cast<size_t>((local_sb + 3) / 4) * kBTileBytes; }
    __host__ __device__ static constexpr size_t smem_bytes(int raw_stages, int local_sb) {
        return 1024 + static_cast<size_t>(raw_stages) * kRawStageBytes + b_bytes(local_sb) + sums_bytes(local_sb) +
               static_cast<size_t>(local_sb) * kNT * 4 + (kWorkerWarps + 1) * 16 * 4 + 256;
    }
};

// 16-byte chunk c (0..7) of row r of a K-major tile with the 128-byte swizzle: rows are 128 bytes, groups of
// eight rows 1024 bytes, chunk index XORed with the row's position in its group.
__device__ __forceinline__ uint32_t swizzled_chunk(uint32_t row, uint32_t chunk) {
    return (row >> 3) * 1024u + (row & 7u) * 128u + ((chunk ^ (row & 7u)) << 4);
}

// ---------------------------------------------------------------- tensor-memory primitives
// 32 lanes x 16 (or 8) consecutive 32-bit columns: thread i of the warp writes TMEM lane (base lane + i).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]),
                 "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]: 128 rows x 16 K elements from tensor memory (lane = row, 8 columns), B as a
// shared-memory descriptor; issued by the elected lane of a converged warp.
__device__ __forceinline__ void umma_f16_tmem_a_elected(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred pa, pe;\n\t"
        ".reg .b32 leader;\n\t"
        "elect.sync leader|pe, 0xffffffff;\n\t"
        "setp.ne.b32 pa, %4, 0;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, pa;\n\t"
        "}"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// ---------------------------------------------------------------- activations -> B tiles (this CTA's K range)
// One warp converts super-block `sb` (global index) of member row m: 256 values, eight per lane, scaled by a
// power of two that brings the largest magnitude into [512, 1024) and rounded to f16 (plane 0; plane 1 holds
// the remainder for f32 inputs).  Column of plane p of member m: p * 8 + m.  Within a group of four K
// elements the tile holds them in the order [e0, e2, e1, e3], the order the weight unpacking produces.
struct BTiles {
    uint8_t* tiles;     // [local sb][4][kNT x 128 B]
    uint8_t* sums;      // [local sb / 4][kNT x 128 B]: per column 4 x (8 block sums hi | 8 block sums lo)
    float* scale;       // [local sb][kNT]
};

__device__ __forceinline__ void convert_to_tiles(const TmemParams& p, const float (&raw)[8], int m, int local_sb, int lane, const BTiles& b) {
    float v[8];
    float amax = 0.0f;
    bool bad = false;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        v[j] = raw[j];
        const float a = fabsf(v[j]);
        bad = bad || !(a <= 3.0e38f);
        amax = fmaxf(amax, a);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    bad = __any_sync(0xffffffffu, bad);
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
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= down;
    // lane's eight elements: chunk (lane & 7) of K step (lane >> 3) of the super-block
    const uint32_t tile = static_cast<uint32_t>(local_sb * 4 + (lane >> 3)) * (kNT * 128);
    const uint32_t sum_tile = static_cast<uint32_t>(local_sb >> 2) * (kNT * 128);
    const uint32_t sum_chunk = static_cast<uint32_t>(local_sb & 3) * 2;
#pragma unroll
    for (int plane = 0; plane < 2; ++plane) {
        if (plane == 1 && p.planes == 1) break;
        const uint32_t column = static_cast<uint32_t>(plane * 8 + m);
        float h[8];
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            h[j] = __half2float(__float2half_rn(v[j]));
            sum += h[j];
            v[j] -= h[j];   // what plane 1 holds
        }
        *reinterpret_cast<uint4*>(b.tiles + tile + swizzled_chunk(column, lane & 7)) =
            make_uint4(half2_bits(h[0], h[2]), half2_bits(h[1], h[3]), half2_bits(h[4], h[6]), half2_bits(h[5], h[7]));
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((lane & 3) == 0) {
            const __half hi = __float2half_rn(sum);
            const __half lo = __float2half_rn(sum - __half2float(hi));
            uint8_t* base = b.sums + sum_tile;
            *reinterpret_cast<__half*>(base + swizzled_chunk(column, sum_chunk) + (lane >> 2) * 2) = hi;
            *reinterpret_cast<__half*>(base + swizzled_chunk(column, sum_chunk + 1) + (lane >> 2) * 2) = lo;
        }
        if (lane == 0) b.scale[local_sb * kNT + column] = up;
    }
}

__device__ __forceinline__ void load_activation_slice(const TmemParams& p, int m, int sb, int lane, float inv_rms, float (&v)[8]) {
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

// ---------------------------------------------------------------- weight unpacking: one row, one pair of sub-blocks
// A pair is 32 quant bytes: the low nibbles are sub-block 2j (32 weights), the high nibbles sub-block 2j+1.
// out_lo / out_hi: 16 registers = 32 halves each, K order [e0, e2, e1, e3] within every group of four.
template <uint32_t FMT>
__device__ __forceinline__ void unpack_pair(uint32_t quant_addr, uint32_t fifth_addr, int j, uint32_t scale_pair, uint32_t (&out_lo)[16],
                                            uint32_t (&out_hi)[16]) {
    const uint32_t mul_a = dup_low(scale_pair), mul_b = dup_high(scale_pair);
    const uint32_t add_a = hmul2(mul_a, 0xe400e400u);    // -1024 * sc
    const uint32_t add_b = hmul2(mul_b, 0xd400d400u);    // -64 * sc:  (1024 + 16 q) * sc/16 - 64 sc = q sc
    const uint32_t mul_bh = hmul2(mul_b, 0x2c002c00u);   // sc / 16
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const uint4 q = lds128(quant_addr + 16 * half);
        uint4 f = make_uint4(0u, 0u, 0u, 0u);
        if (FMT == kQ5_K) f = lds128(fifth_addr + 16 * half);
        const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
        const uint32_t fw[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w = qw[i], ws = w >> 8;
            uint32_t a0 = and_or(w, 0x000f000fu, kMagic), a1 = and_or(ws, 0x000f000fu, kMagic);
            uint32_t b0 = and_or(w, 0x00f000f0u, kMagic), b1 = and_or(ws, 0x00f000f0u, kMagic);
            if (FMT == kQ5_K) {
                // byte p of the fifth-bit bytes carries, in bit s, the fifth bit of position p of sub-block s
                const uint32_t bits = fw[i] >> (2 * j);
                a0 = and_or(bits << 4, 0x00100010u, a0);
                a1 = and_or(bits >> 4, 0x00100010u, a1);
                b0 = and_or(bits << 7, 0x01000100u, b0);
                b1 = and_or(bits >> 1, 0x01000100u, b1);
            }
            out_lo[half * 8 + i * 2 + 0] = hfma2(a0, mul_a, add_a);
            out_lo[half * 8 + i * 2 + 1] = hfma2(a1, mul_a, add_a);
            out_hi[half * 8 + i * 2 + 0] = hfma2(b0, mul_bh, add_b);
            out_hi[half * 8 + i * 2 + 1] = hfma2(b1, mul_bh, add_b);
        }
    }
}

// ---------------------------------------------------------------- the kernel
template <uint32_t FMT>
__global__ void __launch_bounds__(kTmemThreads, 2) qgemv_tmem_kernel(const __grid_constant__ CUtensorMap wmap, const TmemParams p) {
    using P = TmemPlan<FMT>;
    constexpr uint32_t kQuantOffset = FMT == kQ5_K ? 48 : 16;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    const int sb_begin = static_cast<int>(static_cast<long long>(p.nsb) * blockIdx.y / p.ksplit);
    const int sb_end = static_cast<int>(static_cast<long long>(p.nsb) * (blockIdx.y + 1) / p.ksplit);
    const int local_sb = sb_end - sb_begin;
    // B tiles first: they need the 1024-byte alignment
    BTiles b;
    b.tiles = smem;
    b.sums = b.tiles + P::b_bytes(p.b_sb);
    uint8_t* raw = b.sums + P::sums_bytes(p.b_sb);
    b.scale = reinterpret_cast<float*>(raw + static_cast<size_t>(p.raw_stages) * P::kRawStageBytes);
    float* norm = b.scale + p.b_sb * kNT;
    uint64_t* bars = reinterpret_cast<uint64_t*>(norm + (kWorkerWarps + 1) * 16);
    uint64_t* raw_full = bars;
    uint64_t* raw_empty = raw_full + kMaxRawStages;
    uint64_t* a_full = raw_empty + kMaxRawStages;
    uint64_t* a_empty = a_full + kPairs;
    uint64_t* d_full = a_empty + kPairs;
    uint64_t* d_empty = d_full + kDBuffers;
    uint64_t* b_ready = d_empty + kDBuffers;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(b_ready + 1);
    uint32_t* last_flag = tmem_holder + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kRows;
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.raw_stages; ++s) {
            mbar_init(&raw_full[s], 1);
            mbar_init(&raw_empty[s], kWorkerWarps);
        }
        for (int j = 0; j < kPairs; ++j) {
            mbar_init(&a_full[j], 4);      // the four warps of the half that writes the pair
            mbar_init(&a_empty[j], 1);     // tcgen05.commit
        }
        for (int d = 0; d < kDBuffers; ++d) {
            mbar_init(&d_full[d], 1);
            mbar_init(&d_empty[d], kWorkerWarps);
        }
        mbar_init(b_ready, kWorkerWarps);
        mbar_fence_init();
        tma_prefetch_descriptor(&wmap);
    }
    if (warp == kIssuerWarp) tmem_alloc(tmem_holder, kTmemColumns);
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == kProducerWarp) {
        // ---------------- raw weights: one tiled TMA box (128 rows x one super-block) per stage ----------------
        if (lane == 0) {
            for (int i = 0; i < local_sb; ++i) {
                const int s = i % p.raw_stages;
                if (i >= p.raw_stages && !mbar_wait_bounded(&raw_empty[s], ((i / p.raw_stages) - 1) & 1)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    break;
                }
                mbar_arrive_expect_tx(&raw_full[s], P::kRawStageBytes);
                tma_load_2d(raw + static_cast<size_t>(s) * P::kRawStageBytes, &wmap, (sb_begin + i) * (P::kSbBytes / 2), n0, &raw_full[s]);
            }
        }
        __syncwarp();
    } else if (warp == kIssuerWarp) {
        // ---------------- MMA issuer: the warp runs converged, an elected lane issues ----------------
        constexpr uint32_t idesc = umma_instr_desc(kRows, kNT, /*A f16*/ 0, /*B f16*/ 0);
        const uint64_t desc_b0 = umma_smem_desc_sw128(smem_addr(b.tiles));
        const uint64_t desc_s0 = umma_smem_desc_sw128(smem_addr(b.sums));
        bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(b_ready, 0));
        for (int i = 0; i < local_sb && ok; ++i) {
            const int buf = i % kDBuffers;
            if (i >= kDBuffers) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&d_empty[buf], ((i / kDBuffers) - 1) & 1));
            if (!ok) break;
            const uint32_t d_main = tmem_base + kColD + buf * 2 * kNT;
            for (int j = 0; j < kPairs && ok; ++j) {
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(&a_full[j], i & 1));
                if (!ok) break;
                tcgen05_fence_after_sync();
                stamp(p, warp, i, j * 2);
                // pair j = K step j of the super-block (64 elements): B tile i * 4 + j, four K slices of 16
                const uint64_t desc_b = desc_b0 + static_cast<uint64_t>((i * 4 + j) * (P::kBTileBytes >> 4));
#pragma unroll
                for (int slice = 0; slice < 4; ++slice)
                    umma_f16_tmem_a_elected(d_main, tmem_base + j * kPairColumns + slice * 8, desc_b + 2 * slice, idesc,
                                            (j > 0 || slice > 0) ? 1u : 0u);
                umma_commit_elected(&a_empty[j]);
                stamp(p, warp, i, j * 2 + 1);
            }
            if (!ok) break;
            // minimum term: A = the eight 6-bit minima twice, B = block sums hi | lo of this super-block
            umma_f16_tmem_a_elected(d_main + kNT, tmem_base + kColAMin + buf * 8,
                                    desc_s0 + static_cast<uint64_t>((i >> 2) * (P::kBTileBytes >> 4)) + 2 * (i & 3), idesc, 0u);
            umma_commit_elected(&d_full[buf]);
        }
        if (!ok && lane == 0) atomicExch(p.status, kDeviceWaitTimeout);
        __syncwarp();
    } else {
        // ---------------- workers ----------------
        const int half = warp >> 2;                      // which 128 weights of every super-block this thread expands
        const int quadrant = warp & 3;                   // a warp reaches TMEM lanes 32 * (warp % 4) .. + 31
        const int row_in_tile = quadrant * 32 + lane;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quadrant * 32) << 16);
        bool ok = true;

        // B tiles of this CTA's K range: the activations may be the previous kernel's output
        pdl_wait_prior();
        if (p.mode == 1) {
            for (int m = 0; m < p.members; ++m) {
                const AnyRow row{static_cast<const uint8_t*>(p.x) + static_cast<size_t>(m) * p.k * (p.x_bf16 ? 2 : 4), p.x_bf16};
                float part = 0.0f;
                for (int c = threadIdx.x; c < p.k / 8; c += kWorkers) {
                    float v[8];
                    load_row8(row + c * 8, v);
#pragma unroll
                    for (int j = 0; j < 8; ++j) part = fmaf(v[j], v[j], part);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                if (lane == 0) norm[warp * 16 + m] = part;
            }
            named_barrier_sync(1, kWorkers);
            if (threadIdx.x < 16) {
                float total = 0.0f;
#pragma unroll
                for (int w = 0; w < kWorkerWarps; ++w) total += norm[w * 16 + threadIdx.x];
                norm[kWorkerWarps * 16 + threadIdx.x] = 1.0f / sqrtf(total / static_cast<float>(p.k) + p.eps);
            }
            named_barrier_sync(1, kWorkers);
        }
        {
            const int slices = local_sb * p.members;
#pragma unroll 1
            for (int first = warp; first < slices; first += 2 * kWorkerWarps) {
                // two slices per trip so that their loads are in flight together
                const int second = first + kWorkerWarps;
                float v0[8], v1[8];
                const int m0 = first % p.members, s0 = first / p.members;
                load_activation_slice(p, m0, sb_begin + s0, lane, p.mode == 1 ? norm[kWorkerWarps * 16 + m0] : 1.0f, v0);
                const int m1 = second < slices ? second % p.members : m0, s1 = second < slices ? second / p.members : s0;
                load_activation_slice(p, m1, sb_begin + s1, lane, p.mode == 1 ? norm[kWorkerWarps * 16 + m1] : 1.0f, v1);
                convert_to_tiles(p, v0, m0, s0, lane, b);
                if (second < slices) convert_to_tiles(p, v1, m1, s1, lane, b);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(b_ready);
        }
        // every worker reads the scale factors the others wrote
        named_barrier_sync(1, kWorkers);

        float acc[kNT / 2];
#pragma unroll
        for (int c = 0; c < kNT / 2; ++c) acc[c] = 0.0f;
        float d_prev = 0.0f, dmin_prev = 0.0f;
        const uint32_t raw_addr = smem_addr(raw) + static_cast<uint32_t>(row_in_tile) * P::kSbBytes;
        const uint32_t column0 = static_cast<uint32_t>(half * (kNT / 2));

        auto read_back = [&](int i, float d, float dmin) {
            // acc[c] += scale[c] * (d * D[c] - dmin * Dmin[c]) for this thread's row and this half's columns
            const int buf = i % kDBuffers;
            if (ok && !mbar_wait_bounded(&d_full[buf], (i / kDBuffers) & 1)) {
                atomicExch(p.status, kDeviceWaitTimeout);
                ok = false;
            }
            tcgen05_fence_after_sync();
            uint32_t dm[8], dn[8];
            const uint32_t taddr = lane_base + kColD + buf * 2 * kNT + column0;
            tmem_ld8(taddr, dm);
            tmem_ld8(taddr + kNT, dn);
            tmem_ld_wait();
            const float4 s0 = *reinterpret_cast<const float4*>(b.scale + i * kNT + column0);
            const float4 s1 = *reinterpret_cast<const float4*>(b.scale + i * kNT + column0 + 4);
            const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float t = fmaf(d, __uint_as_float(dm[c]), -(dmin * __uint_as_float(dn[c])));
                acc[c] = fmaf(sc[c], t, acc[c]);
            }
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&d_empty[buf]);
        };

#pragma unroll 1
        for (int i = 0; i < local_sb; ++i) {
            const int s = i % p.raw_stages;
            if (ok && !mbar_wait_bounded(&raw_full[s], (i / p.raw_stages) & 1)) {
                atomicExch(p.status, kDeviceWaitTimeout);
                ok = false;
            }
            stamp(p, warp, i, 0);
            const uint32_t blk = raw_addr + static_cast<uint32_t>(s) * P::kRawStageBytes;
            const uint4 header = lds128(blk);   // d | dmin, 12 scale bytes
            uint32_t sc_lo, sc_hi, m_lo, m_hi;
            unpack_k_scales(header.y, header.z, header.w, sc_lo, sc_hi, m_lo, m_hi);
            const uint32_t sc_word = half ? sc_hi : sc_lo;   // scales of sub-blocks 4 half .. 4 half + 3
            if (half == 0) {
                // the eight minima as f16, twice: K slots 0..7 meet the block sums' hi parts, 8..15 their lo parts
                uint32_t mins[8];
                mins[0] = byte_pair_half2(m_lo, false);
                mins[1] = byte_pair_half2(m_lo, true);
                mins[2] = byte_pair_half2(m_hi, false);
                mins[3] = byte_pair_half2(m_hi, true);
                mins[4] = mins[0]; mins[5] = mins[1]; mins[6] = mins[2]; mins[7] = mins[3];
                // the buffer was last read by the minimum MMA of super-block i - 2, whose accumulator this thread has read back
                tmem_st8(lane_base + kColAMin + (i % kDBuffers) * 8, mins);
            }
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const int j = half * 2 + jj;
                if (i > 0 && ok && !mbar_wait_bounded(&a_empty[j], (i - 1) & 1)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    ok = false;
                }
                tcgen05_fence_after_sync();
                stamp(p, warp, i, 1 + 4 * jj);
                uint32_t out_lo[16], out_hi[16];
                unpack_pair<FMT>(blk + kQuantOffset + 32 * j, blk + 16, j, byte_pair_half2(sc_word, jj != 0), out_lo, out_hi);
                stamp(p, warp, i, 2 + 4 * jj);
                tmem_st16(lane_base + j * kPairColumns, out_lo);
                tmem_st16(lane_base + j * kPairColumns + 16, out_hi);
                stamp(p, warp, i, 3 + 4 * jj);
                tmem_st_wait();
                stamp(p, warp, i, 4 + 4 * jj);
                tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[j]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&raw_empty[s]);
            stamp(p, warp, i, 9);
            if (i > 0) read_back(i - 1, d_prev, dmin_prev);
            stamp(p, warp, i, 10);
            d_prev = f16_bits_to_f32(header.x & 0xffffu);
            dmin_prev = f16_bits_to_f32(header.x >> 16);
        }
        if (local_sb > 0) read_back(local_sb - 1, d_prev, dmin_prev);

        // ---------------- output: columns -> members (plane 1 of member m is column 8 + m) through shared memory ----------------
        named_barrier_sync(1, kWorkers);   // every raw stage has been read: the ring is free
        float* tile = reinterpret_cast<float*>(raw);   // [kNT][kRows]
#pragma unroll
        for (int c = 0; c < kNT / 2; ++c) tile[(column0 + c) * kRows + row_in_tile] = ok ? acc[c] : 0.0f;
        named_barrier_sync(1, kWorkers);
        const bool split = p.ksplit > 1;
        float* part = split ? p.partial + static_cast<size_t>(blockIdx.y) * p.members * p.n : nullptr;
        for (int idx = threadIdx.x; idx < p.members * kRows; idx += kWorkers) {
            const int m = idx >> 7;
            const long long row = static_cast<long long>(n0) + (idx & (kRows - 1));
            if (row < p.n) {
                float value = tile[m * kRows + (idx & (kRows - 1))];
                if (p.planes == 2) value += tile[(8 + m) * kRows + (idx & (kRows - 1))];
                const size_t o = static_cast<size_t>(m) * p.n + row;
                if (split) {
                    part[o] = value;
                } else if (p.y_bf16) {
                    const float old = p.accumulate ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.y)[o]) : 0.0f;
                    static_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(value + old);
                } else {
                    const float old = p.accumulate ? static_cast<const float*>(p.y)[o] : 0.0f;
                    static_cast<float*>(p.y)[o] = value + old;
                }
            }
        }
        // ---------------- split-K: the CTA that draws the last ticket of its row tile adds the partial tiles ----------------
        if (split) {
            __threadfence();
            named_barrier_sync(1, kWorkers);
            if (threadIdx.x == 0) {
                unsigned int* ticket = p.tickets + blockIdx.x;
                const unsigned int drawn = atomicAdd(ticket, 1u);
                const bool last = drawn == static_cast<unsigned int>(p.ksplit - 1);
                if (last) *ticket = 0;   // ready for the next launch
                *last_flag = last ? 1u : 0u;
            }
            named_barrier_sync(1, kWorkers);
            if (*last_flag != 0) {
                __threadfence();
                const size_t plane = static_cast<size_t>(p.members) * p.n;
                for (int idx = threadIdx.x; idx < p.members * kRows; idx += kWorkers) {
                    const int m = idx >> 7;
                    const long long row = static_cast<long long>(n0) + (idx & (kRows - 1));
                    if (row < p.n) {
                        const size_t o = static_cast<size_t>(m) * p.n + row;
                        float sum = 0.0f;
                        for (int z = 0; z < p.ksplit; ++z) sum += __ldcg(p.partial + z * plane + o);
                        if (p.y_bf16) {
                            if (p.accumulate) sum += __bfloat162float(static_cast<const __nv_bfloat16*>(p.y)[o]);
                            static_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(sum);
                        } else {
                            if (p.accumulate) sum += static_cast<const float*>(p.y)[o];
                            static_cast<float*>(p.y)[o] = sum;
                        }
                    }
                }
            }
        }
    }

    // ---------------- teardown: every warp arrives here, then TMEM is released ----------------
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == kIssuerWarp) tmem_dealloc(tmem_base, kTmemColumns);
}

constexpr size_t kSmemLimit = 227 * 1024;

// K splits: enough CTAs to fill two per SM, no CTA with more super-blocks than its resident B tiles hold.
int choose_splits(int tiles, int nsb, int sm_count, int members, size_t scratch_bytes, int n, int max_tickets) {
    // the largest split count whose CTAs still fit one wave of two per SM; more splits only where a CTA's K range
    // would not fit its resident B tiles otherwise
    int ks = (2 * sm_count) / tiles;
    const int needed = (nsb + kMaxLocalSb - 1) / kMaxLocalSb;
    if (ks < needed) ks = needed;
    if (ks > nsb) ks = nsb;
    if (ks < 1) ks = 1;
    if (ks > 1 && (static_cast<size_t>(ks) * members * n * sizeof(float) > scratch_bytes || tiles > max_tickets)) return 0;
    return ks;
}

template <uint32_t FMT>
cudaError_t launch_format(const TmemGemvArgs& a) {
    using P = TmemPlan<FMT>;
    auto kernel = qgemv_tmem_kernel<FMT>;
    const int nsb = a.k / kSuperBlock;
    const int tiles = (a.n + kRows - 1) / kRows;
    int ksplit = choose_splits(tiles, nsb, a.sm_count, a.members, a.scratch_bytes, a.n, a.ticket_count);
    if (a.force_ksplit > 0 && a.force_ksplit <= nsb && (nsb + a.force_ksplit - 1) / a.force_ksplit <= kMaxLocalSb) ksplit = a.force_ksplit;
    if (ksplit == 0) return cudaErrorInvalidConfiguration;
    const int b_sb = (nsb + ksplit - 1) / ksplit;
    // raw ring: as deep as two CTAs per SM allow (one CTA per SM when the resident B tiles leave less than two stages)
    int raw_stages = kMaxRawStages;
    while (raw_stages > 2 && P::smem_bytes(raw_stages, b_sb) > (kSmemLimit - 2048) / 2) --raw_stages;
    if (a.stages > 0 && a.stages < raw_stages) raw_stages = a.stages < 2 ? 2 : a.stages;
    const size_t smem = P::smem_bytes(raw_stages, b_sb);
    if (smem > kSmemLimit) return cudaErrorInvalidConfiguration;
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
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes / 2), static_cast<cuuint64_t>(a.n)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(P::kSbBytes / 2), static_cast<cuuint32_t>(kRows)};
    const cuuint32_t elem[2] = {1, 1};
    if (encode(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<uint8_t*>(a.weights), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    TmemParams p{};
    p.x = a.x;
    p.x_bf16 = a.x_bf16 ? 1 : 0;
    p.mode = a.mode;
    p.norm_weight = a.norm_weight;
    p.eps = a.eps;
    p.y = a.y;
    p.y_bf16 = a.y_bf16 ? 1 : 0;
    p.accumulate = a.accumulate ? 1 : 0;
    p.partial = static_cast<float*>(a.scratch);
    p.tickets = a.tickets;
    p.k = a.k;
    p.n = a.n;
    p.nsb = nsb;
    p.members = a.members;
    p.planes = a.x_bf16 ? 1 : 2;
    p.ksplit = ksplit;
    p.raw_stages = raw_stages;
    p.b_sb = b_sb;
    p.trace = a.trace;
    p.status = a.device_status;
    return launch_kernel(kernel, dim3(tiles, ksplit), dim3(kTmemThreads), smem, a.stream, wmap, p);
}

}  // namespace

bool qgemv_tmem_supports(uint32_t value_type, int k, int n, int members, bool x_bf16, const void* weights) {
    if (value_type != kQ4_K && value_type != kQ5_K) return false;
    if (members < 1 || members > (x_bf16 ? 16 : 8) || k <= 0 || k % kSuperBlock != 0 || n < 1) return false;
    return reinterpret_cast<uintptr_t>(weights) % 16 == 0;
}

cudaError_t launch_qgemv_tmem(const TmemGemvArgs& a) {
    switch (a.value_type) {
        case kQ4_K: return launch_format<kQ4_K>(a);
        case kQ5_K: return launch_format<kQ5_K>(a);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ribn
