// Quantized skinny GEMM (9..64 member rows) on the 5th-generation tensor cores with the weight operand unpacked
// straight into tensor memory.
//
//   Y[m][n] = sum_k dequant(W[n][k]) * X[m][k]          Q4_K / Q5_K / Q6_K, up to 64 member rows per launch
//
// The path is bound by HBM: a 4.5-bit weight arrives every ~0.025 SM clocks, which leaves about three thread
// instructions per weight, and the integer pipe -- where the bit manipulation of the unpacking runs -- issues
// at half rate.  Two things decide whether a kernel keeps up: instructions per weight, and where the
// dequantised operand lives.  Writing an f16 tile to shared memory for the tensor pipe costs 2 bytes written
// and 2 read per weight against 0.56 streamed; the warp-level mma.sync keeps the operand in registers but pays
// its issue rate per eight member rows.  Here
//   * a thread owns one weight row (one TMEM lane).  It reads the row's raw super-block bytes from the
//     shared-memory ring (tiled TMA boxes of 128 rows x one super-block) and expands two quants at a time
//     with one logic op and one HFMA2:  (q | 0x6400) is the half 1024 + q, and with s = f16(d * sc)
//     (1024 + q) * s - 1024 * s = q * s in one rounding;
//   * the expanded values -- the complete weight d * sc * q, so that every super-block accumulates into the
//     same accumulator -- go to tensor memory with tcgen05.st (32 K elements per instruction and row) and are
//     the A operand of tcgen05.mma (M = 128 rows, K = 16 per instruction, N = 16 / 32 / 64 columns); they never
//     pass through shared memory.  The minimum term -dmin * m[g] * sum_g(x) is one more MMA per super-block with
//     the eight products -dmin * m[g] as A and the activations' block sums as B;
//   * the B operand -- the activations as f16, scaled by one power of two per member row -- is made once per
//     call by a pre-pass in exactly the swizzled K-major tiles the MMA reads, and streamed from L2 into a
//     shared-memory ring with bulk copies next to the weights;
//   * the accumulator is read back once, at the end of the CTA's K range.
// About 1.5 thread instructions per weight whatever the number of member rows.
//
// Q6_K (210-byte super-blocks, no minima): the quant under the magic byte is 1024 + 4 q; minus 1152 it is 4 (q - 32)
// exactly, and one HMUL2 with f16(d * sc / 4) makes the weight.  A TMA box must start on a 16-byte boundary, so its
// boxes are 240 bytes wide from the boundary below each super-block and the lanes read at the (uniform) remainder.
//
// Range: f16(d * sc) and 1024 * f16(d * sc) must be finite, i.e. |d| * 63 < 64.  Rows whose super-block scale
// is larger (up to 32) take a second multiply per pair; beyond that the context's status word reports it.
// Super-block scales below 1e-6 lose bits to f16 subnormals (the product d * sc * q itself is an f16).
//
// CTA = 128 rows x a K range; grid = row tiles x K splits.  Warps 0..7 are workers (thread = row; warps 0..3
// expand the first 128 weights of every super-block, warps 4..7 the second 128), warp 8 streams the raw
// weights and the activation tiles, warp 9 issues the MMAs and owns the TMEM allocation.  Partial results of
// K splits meet in global scratch: the CTA that draws the last ticket of a row tile adds them in split order
// (deterministic).
//
// Every wait on an mbarrier is bounded; a wait that runs out sets the status word and every warp still
// reaches the teardown that frees TMEM.
//
// Reference counterparts: q*_gemv_warp_batch (crates/nvidia/src/kernels/quantized/q4_k.cu:161-258, q5_k.cu)
// for the contract -- the reference serves wider batches as several launches of eight rows
// (crates/nvidia/src/decode.rs:1953-1977); rms_norm (crates/nvidia/src/model_ops.rs:106-147) and silu_mul
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

// Upper bound of one suspended poll of an mbarrier wait: a waiting thread wakes when the phase completes, and until then
// takes no issue slots from the threads that unpack.
constexpr uint32_t kWaitHintNs = 1000u;

constexpr int kRows = 128;                 // weight rows per CTA = UMMA M = TMEM lanes
constexpr int kWorkerWarps = 8;
constexpr int kWorkers = kWorkerWarps * 32;
// Worker sets: with 64 accumulator columns one CTA owns the SM (shared memory), and eight worker warps leave the issue slots
// two thirds idle while they wait on shared memory, tensor memory and barriers; a second set of eight takes the odd
// super-blocks (its own A slots and minimum buffer: the A operand is double-buffered there anyway).
template <int NT>
struct Roles {
    static constexpr int kSets = NT >= 64 ? 2 : 1;
    static constexpr int kProducerWarp = kSets * kWorkerWarps;
    static constexpr int kIssuerWarp = kProducerWarp + 1;    // pairs 0 and 1 of every super-block and the minimum term, accumulator 0; owns TMEM
    static constexpr int kIssuerWarp2 = kProducerWarp + 2;   // pairs 2 and 3, accumulator 1
    static constexpr int kThreads = (kProducerWarp + 3) * 32;
};
constexpr int kPairs = 4;                  // 64-weight pairs of sub-blocks per super-block = A slots in TMEM
constexpr int kPairColumns = 32;           // TMEM columns of one pair: 64 halves per row
constexpr int kMaxStages = 4;

// Tiled TMA wants a 16-byte aligned base and row pitch.  A Q6_K matrix whose rows are 210 * nsb bytes with nsb not a
// multiple of eight has neither for most rows, but rows n, n + P, n + 2 P, ... (P = 16 / gcd(row bytes, 16)) are P * row
// bytes apart -- a multiple of 16 -- so the matrix is P interleaved matrices, one tensor map each, whose bases are rounded
// down to 16 bytes; a row tile is then P boxes of 128 / P rows, and tile row r = c * (128 / P) + j is matrix row
// n0 + j * P + c.
struct WeightMaps {
    CUtensorMap map[8];
};

struct TmemParams {
    const void* x;              // [members][k] (swiglu: [members][2k]) f32 or bf16
    int x_bf16;
    int mode;                   // 0 plain, 1 RMSNorm first, 2 silu(gate) * up
    const float* norm_weight;
    float eps;
    uint8_t* image;             // the activations as MMA tiles (layout below), written by the pre-pass
    void* y;                    // rows below n_first: [members][n_first]
    void* y2;                   // rows from n_first on: [members][n - n_first] (n_first = n: unused)
    int n_first;
    int y_bf16;
    int accumulate;
    float* partial;             // split-K scratch [ksplit][members][n]
    unsigned int* tickets;      // zero-initialised counters: [row tile] arrivals, [ticket_stride + row tile] departures
    int ticket_stride;
    int cooperative;            // every CTA of the grid is resident at once: the CTAs of a row tile share the sum of its partial tiles
    int k, n, nsb, members, planes, ksplit, raw_stages, b_stages;
    int row_classes;            // 1, or for Q6_K rows that do not start on 16-byte boundaries 2 / 4 / 8: rows n0 + j * classes + c share class c
    unsigned int row_bytes;
    int* status;
    long long* trace;           // diagnostics (builds with -DRIBN_TRACE): wall-clock stamps of CTA (0, 0), or null
};

// Where output (member m, matrix row `row`) lives: a call may deliver its first n_first rows and the rest to two
// buffers (two projections stored as one matrix).  n_first is a multiple of four, so groups of four rows stay together.
__device__ __forceinline__ void* output_slot(const TmemParams& p, int m, long long row, size_t& index) {
    if (row < p.n_first) {
        index = static_cast<size_t>(m) * p.n_first + row;
        return p.y;
    }
    index = static_cast<size_t>(m) * (p.n - p.n_first) + (row - p.n_first);
    return p.y2;
}

// trace[role * 32 + event] = globaltimer (ns) of CTA (0, 0); roles: 0 producer, 1 issuer, 2 worker warp 0, 3 worker warp 4.
__device__ __forceinline__ void stamp(const TmemParams& p, int role, int event) {
#ifdef RIBN_TRACE
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && (threadIdx.x & 31) == 0 && event < 32) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.trace[role * 32 + event] = static_cast<long long>(t);
    }
#else
    (void)p;
    (void)role;
    (void)event;
#endif
}

// Activation image, per super-block one stage of five K-major tiles of NT rows (columns of the product) x 128 bytes
// with the 128-byte swizzle: four tiles of 64 K elements each, then a tile whose first 32 bytes per row hold the
// eight block sums (sum of 32 scaled values) as f16 hi parts, then their f16 lo parts (unused by Q6_K, which has no minima).  Member m of plane p is
// row 2 m + p (one plane: row m).  Behind the stages: float up[NT], the inverse of each row's scale factor.
template <int NT, int TILES>
struct ImagePlan {
    static constexpr int kTileBytes = NT * 128;
    static constexpr int kStageBytes = TILES * kTileBytes;
    __host__ __device__ static constexpr size_t scales_offset(int nsb) { return static_cast<size_t>(nsb) * kStageBytes; }
    __host__ __device__ static constexpr size_t bytes(int nsb) { return scales_offset(nsb) + NT * sizeof(float); }
};

template <uint32_t FMT, int NT>
struct TmemPlan {
    using I = ImagePlan<NT, 5>;
    static constexpr int kSbBytes = Format<FMT>::kBytes;
    // Q6_K super-blocks are 210 bytes: a TMA box must start on a 16-byte boundary and be a multiple of 16 bytes wide, so
    // the box is 240 bytes from the boundary below the super-block; the data starts (sb * 210) % 16 bytes into every row
    static constexpr int kRowPitch = FMT == kQ6_K ? 240 : kSbBytes;
    static constexpr int kRawStageBytes = kRows * kRowPitch;
    // A operand: one or two sets of four pair slots; two when the accumulator leaves room and one CTA owns the SM anyway
    static constexpr int kABuffers = NT >= 64 ? 2 : 1;
    static constexpr int kColAMin = kABuffers * kPairs * kPairColumns;
    static constexpr int kColD = kColAMin + 2 * 8;
    // two accumulators, one per issuing warp (MMAs of different threads into one accumulator are not ordered)
    static constexpr int kColumnsUsed = kColD + 2 * NT;
    static constexpr int kTmemColumns = kColumnsUsed <= 256 ? 256 : 512;
    static_assert(kColumnsUsed <= 512, "TMEM plan");
    static_assert(kRowPitch % 16 == 0 && kRawStageBytes % 128 == 0, "rows of a raw stage stay 16-byte aligned, stages 128-byte aligned");
    __host__ __device__ static constexpr size_t smem_bytes(int raw_stages, int b_stages) {
        return 1024 + static_cast<size_t>(b_stages) * I::kStageBytes + static_cast<size_t>(raw_stages) * kRawStageBytes + NT * 4 + 512;
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


// The four MMAs of one pair (64 K elements): A slices 8 TMEM columns apart, B slices 32 bytes apart along the swizzled
// rows (+2 in the descriptor's address field); one election for the four.  `accumulate_first` = 0 makes the first
// slice overwrite D.
__device__ __forceinline__ void umma_f16_tmem_a_pair_elected(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate_first) {
    asm volatile(
        "{\n\t"
        ".reg .pred pf, pt, pe;\n\t"
        ".reg .b64 b1, b2, b3;\n\t"
        ".reg .b32 a1, a2, a3, leader;\n\t"
        "elect.sync leader|pe, 0xffffffff;\n\t"
        "setp.ne.b32 pf, %4, 0;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "add.u32 a1, %1, 8;\n\t"
        "add.u32 a2, %1, 16;\n\t"
        "add.u32 a3, %1, 24;\n\t"
        "add.s64 b1, %2, 2;\n\t"
        "add.s64 b2, %2, 4;\n\t"
        "add.s64 b3, %2, 6;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, pf;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, pt;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %3, pt;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %3, pt;\n\t"
        "}"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate_first)
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

// ---------------------------------------------------------------- pre-pass: activations -> MMA tiles in global memory
// grid (members), 256 threads.  One sweep over the member's row in global memory: the values (x, or silu(gate) * up) go
// to a shared-memory copy of the row while their sum of squares (fused RMSNorm) and largest magnitude are gathered; the
// normalisation, the largest magnitude of what enters the product and the conversion then work on the copy.  Every value
// is multiplied by the power of two that brings that magnitude into [512, 1024) and stored as f16 (plane 0; for two
// planes also the f16 of what plane 0 lost).  Within a group of four K elements the tiles hold [e0, e2, e1, e3], the order
// the weight unpacking produces.  Rows longer than the copy can hold (`cached` = 0) are re-read from global memory.
constexpr int kImageCacheFloats = 50 * 1024;   // 200 KB

template <int NT>
// 8 to 32 warps per CTA (chosen by the launcher from the row length): a warp owns the super-blocks sb = warp (mod warps)
// and has two of them in flight per trip, so up to 64 super-blocks are read in one round trip to memory.
__global__ void __launch_bounds__(1024) tmem_image_kernel(const TmemParams p, int cached) {
    using I = ImagePlan<NT, 5>;
    extern __shared__ __align__(16) float row_copy[];
    __shared__ float red[32];
    __shared__ uint32_t red_bits[32];
    pdl_launch_dependents();
    pdl_wait_prior();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = static_cast<int>(blockDim.x >> 5);
    const int m = blockIdx.x;
    const size_t row_elements = static_cast<size_t>(p.k) * (p.mode == 2 ? 2 : 1);
    const AnyRow row{static_cast<const uint8_t*>(p.x) + static_cast<size_t>(m) * row_elements * (p.x_bf16 ? 2 : 4), p.x_bf16};
    // what the first sweep reads of super-block sb: x (modes 0, 1) or silu(gate) * up (mode 2)
    auto read_slice = [&](int sb, float (&v)[8]) {
        const int k0 = sb * kSuperBlock + lane * 8;
        load_row8(row + k0, v);
        if (p.mode == 2) {
            float u[8];
            load_row8(row + (p.k + k0), u);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (v[j] / (1.0f + expf(-v[j]))) * u[j];
        }
    };
    auto keep = [&](int sb, const float (&v)[8]) {
        float4* dst = reinterpret_cast<float4*>(row_copy + sb * kSuperBlock + lane * 8);
        dst[0] = make_float4(v[0], v[1], v[2], v[3]);
        dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    };
    auto kept = [&](int sb, float (&v)[8]) {
        const float4* src = reinterpret_cast<const float4*>(row_copy + sb * kSuperBlock + lane * 8);
        const float4 a = src[0], b = src[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    };
    // non-negative floats order like their bit patterns; infinities and NaNs (0x7f800000 and above) come out on top
    uint32_t biggest = 0u;
    float part = 0.0f;
    for (int sb = warp; sb < p.nsb; sb += 2 * warps) {   // two slices per trip: their loads are in flight together
        float v0[8], v1[8];
        const bool second = sb + warps < p.nsb;
        read_slice(sb, v0);
        if (second) read_slice(sb + warps, v1);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            part = fmaf(v0[j], v0[j], part);
            biggest = max(biggest, __float_as_uint(fabsf(v0[j])));
        }
        if (cached) keep(sb, v0);
        if (second) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                part = fmaf(v1[j], v1[j], part);
                biggest = max(biggest, __float_as_uint(fabsf(v1[j])));
            }
            if (cached) keep(sb + warps, v1);
        }
    }
    float inv_rms = 1.0f;
    if (p.mode == 1) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (lane == 0) red[warp] = part;
        __syncthreads();
        float total = 0.0f;
        for (int w = 0; w < warps; ++w) total += red[w];
        inv_rms = 1.0f / sqrtf(total / static_cast<float>(p.k) + p.eps);
        // the normalised values, in the order of operations of rms_norm (x * inv_rms * weight), and their largest magnitude
        biggest = 0u;
        for (int sb = warp; sb < p.nsb; sb += warps) {
            float v[8], g[8];
            if (cached) kept(sb, v);
            else read_slice(sb, v);
            load_x8<float>(p.norm_weight + sb * kSuperBlock + lane * 8, g);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = v[j] * inv_rms * g[j];
                biggest = max(biggest, __float_as_uint(fabsf(v[j])));
            }
            if (cached) keep(sb, v);
        }
    }
    biggest = __reduce_max_sync(0xffffffffu, biggest);
    if (lane == 0) red_bits[warp] = biggest;
    __syncthreads();
    for (int w = 0; w < warps; ++w) biggest = max(biggest, red_bits[w]);
    const bool bad = biggest >= 0x7f800000u;
    const float amax = __uint_as_float(biggest);
    int e = 9 - (static_cast<int>(biggest >> 23) - 127);
    e = max(-100, min(100, e));
    float down = __uint_as_float(static_cast<uint32_t>(127 + e) << 23);
    float up = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
    if (amax == 0.0f) up = 0.0f;
    if (bad) {
        down = 0.0f;
        up = __int_as_float(0x7fc00000);
    }
    float* scales = reinterpret_cast<float*>(p.image + I::scales_offset(p.nsb));
    for (int sb = warp; sb < p.nsb; sb += warps) {
        float v[8];
        if (cached) {
            kept(sb, v);   // a warp reads back what it wrote itself
        } else {
            read_slice(sb, v);
            if (p.mode == 1) {
                float g[8];
                load_x8<float>(p.norm_weight + sb * kSuperBlock + lane * 8, g);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = v[j] * inv_rms * g[j];
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = bad ? 0.0f : v[j] * down;
        uint8_t* stage = p.image + static_cast<size_t>(sb) * I::kStageBytes;
        // lane's eight elements: chunk (lane & 7) of K step (lane >> 3) of the super-block
        uint8_t* tile = stage + (lane >> 3) * I::kTileBytes;
        uint8_t* sums = stage + 4 * I::kTileBytes;
#pragma unroll
        for (int plane = 0; plane < 2; ++plane) {
            if (plane == 1 && p.planes == 1) break;
            const uint32_t column = static_cast<uint32_t>(p.planes == 2 ? 2 * m + plane : m);
            float h[8];
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                h[j] = __half2float(__float2half_rn(v[j]));
                sum += h[j];
                v[j] -= h[j];   // what plane 1 holds
            }
            *reinterpret_cast<uint4*>(tile + swizzled_chunk(column, lane & 7)) =
                make_uint4(half2_bits(h[0], h[2]), half2_bits(h[1], h[3]), half2_bits(h[4], h[6]), half2_bits(h[5], h[7]));
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if ((lane & 3) == 0) {
                const __half hi = __float2half_rn(sum);
                const __half lo = __float2half_rn(sum - __half2float(hi));
                *reinterpret_cast<__half*>(sums + swizzled_chunk(column, 0) + (lane >> 2) * 2) = hi;
                *reinterpret_cast<__half*>(sums + swizzled_chunk(column, 1) + (lane >> 2) * 2) = lo;
            }
        }
    }
    if (threadIdx.x == 0) scales[m] = up;   // per member
}

// ---------------------------------------------------------------- weight unpacking: one row, one pair of sub-blocks
// A pair is 32 quant bytes: the low nibbles are sub-block 2j (32 weights), the high nibbles sub-block 2j+1.
// out_lo / out_hi: 16 registers = 32 halves each, K order [e0, e2, e1, e3] within every group of four.
// mul_a / mul_b: the factor of each sub-block as a half pair; every quant is brought to the low mantissa bits of the
// half 1024, so that one HFMA2 with -1024 * factor as addend leaves q * factor.
template <uint32_t FMT>
__device__ __forceinline__ void unpack_pair(uint32_t quant_addr, uint32_t fifth_addr, int j, uint32_t mul_a, uint32_t mul_b, uint32_t (&out_lo)[16],
                                            uint32_t (&out_hi)[16]) {
    const uint32_t add_a = hmul2(mul_a, 0xe400e400u);    // -1024 * factor
    const uint32_t add_b = hmul2(mul_b, 0xe400e400u);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const uint4 q = lds128(quant_addr + 16 * half);
        uint4 f = make_uint4(0u, 0u, 0u, 0u);
        if (FMT == kQ5_K) f = lds128(fifth_addr + 16 * half);
        const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
        const uint32_t fw[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w = qw[i];
            uint32_t a0 = and_or(w, 0x000f000fu, kMagic), a1 = and_or(w >> 8, 0x000f000fu, kMagic);
            uint32_t b0 = and_or(w >> 4, 0x000f000fu, kMagic), b1 = and_or(w >> 12, 0x000f000fu, kMagic);
            if (FMT == kQ5_K) {
                // byte p of the fifth-bit bytes carries, in bit s, the fifth bit of position p of sub-block s
                const uint32_t bits = fw[i] >> (2 * j);
                a0 = and_or(bits << 4, 0x00100010u, a0);
                a1 = and_or(bits >> 4, 0x00100010u, a1);
                b0 = and_or(bits << 3, 0x00100010u, b0);
                b1 = and_or(bits >> 5, 0x00100010u, b1);
            }
            out_lo[half * 8 + i * 2 + 0] = hfma2(a0, mul_a, add_a);
            out_lo[half * 8 + i * 2 + 1] = hfma2(a1, mul_a, add_a);
            out_hi[half * 8 + i * 2 + 0] = hfma2(b0, mul_b, add_b);
            out_hi[half * 8 + i * 2 + 1] = hfma2(b1, mul_b, add_b);
        }
    }
}

// Q6_K: one group pair of a 128-weight chunk.  `la`, `lb`: the chunk's two runs of 32 low-nibble bytes, `qh` its 32
// two-bit bytes (all at 2-byte alignment); V0 / V0 + 1 are the groups that go to out_lo / out_hi.  A quant byte
// (q << 2) under the magic byte is the half 1024 + 4 q; minus 1152 that is 4 (q - 32), exactly; times f16(factor / 4) it is
// the weight with one rounding relative to its own size (folding the offset into the addend of one HFMA2 would round
// relative to 4 q, twice as coarse at the centre of the range, and 1152 f is not exact).
template <int V0>
__device__ __forceinline__ void unpack_pair_q6(uint32_t la, uint32_t lb, uint32_t qh, const float (&factor)[4], uint32_t (&out_lo)[16],
                                               uint32_t (&out_hi)[16]) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const uint4 a = lds128_unaligned(la + 16 * half), b = lds128_unaligned(lb + 16 * half), h = lds128_unaligned(qh + 16 * half);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w}, hw[4] = {h.x, h.y, h.z, h.w};
        const float f0 = factor[half], f1 = factor[2 + half];      // the scale of each run of 16 weights
        const uint32_t mul0 = half2_bits(f0 * 0.25f, f0 * 0.25f);
        const uint32_t mul1 = half2_bits(f1 * 0.25f, f1 * 0.25f);
        constexpr uint32_t kCentre = 0x64806480u;   // 1152 = 1024 + 4 * 32
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t b0 = q6_bytes<V0>(aw[i], bw[i], hw[i]), b1 = q6_bytes<V0 + 1>(aw[i], bw[i], hw[i]);
            out_lo[half * 8 + i * 2 + 0] = hmul2(hsub2(__byte_perm(b0, kMagicBytes, 0x4240), kCentre), mul0);   // positions 0, 2
            out_lo[half * 8 + i * 2 + 1] = hmul2(hsub2(__byte_perm(b0, kMagicBytes, 0x4341), kCentre), mul0);   // positions 1, 3
            out_hi[half * 8 + i * 2 + 0] = hmul2(hsub2(__byte_perm(b1, kMagicBytes, 0x4240), kCentre), mul1);
            out_hi[half * 8 + i * 2 + 1] = hmul2(hsub2(__byte_perm(b1, kMagicBytes, 0x4341), kCentre), mul1);
        }
    }
}

// ---------------------------------------------------------------- the kernel
template <uint32_t FMT, int NT>
__global__ void __launch_bounds__(Roles<NT>::kThreads, NT >= 64 ? 1 : 2) qgemv_tmem_kernel(const __grid_constant__ WeightMaps wmaps, const TmemParams p) {
    using P = TmemPlan<FMT, NT>;
    using I = typename P::I;
    using R = Roles<NT>;
    constexpr int kProducerWarp = R::kProducerWarp, kIssuerWarp = R::kIssuerWarp, kIssuerWarp2 = R::kIssuerWarp2, kSets = R::kSets;
    constexpr uint32_t kQuantOffset = FMT == kQ5_K ? 48 : 16;
    constexpr int AB = P::kABuffers;
    static_assert(kSets == 1 || AB == kSets, "a worker set owns one buffer of the A operand");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    const int sb_begin = static_cast<int>(static_cast<long long>(p.nsb) * blockIdx.y / p.ksplit);
    const int sb_end = static_cast<int>(static_cast<long long>(p.nsb) * (blockIdx.y + 1) / p.ksplit);
    const int local_sb = sb_end - sb_begin;
    uint8_t* b_ring = smem;                                                          // 1024-byte aligned stages
    uint8_t* raw = b_ring + static_cast<size_t>(p.b_stages) * I::kStageBytes;
    float* up = reinterpret_cast<float*>(raw + static_cast<size_t>(p.raw_stages) * P::kRawStageBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(up + NT);
    uint64_t* raw_full = bars;
    uint64_t* raw_empty = raw_full + kMaxStages;
    uint64_t* b_full = raw_empty + kMaxStages;
    uint64_t* b_empty = b_full + kMaxStages;
    uint64_t* a_full = b_empty + kMaxStages;          // [AB * 4]
    uint64_t* a_empty = a_full + 2 * kPairs;
    uint64_t* min_full = a_empty + 2 * kPairs;        // [2]
    uint64_t* min_empty = min_full + 2;
    uint64_t* d_full = min_empty + 2;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(d_full + 1);
    uint32_t* last_flag = tmem_holder + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kRows;
    pdl_launch_dependents();
    if (warp == 0) stamp(p, 2, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&raw_full[s], 1);
            mbar_init(&raw_empty[s], kWorkerWarps);
            mbar_init(&b_full[s], 1);
            mbar_init(&b_empty[s], 2);            // tcgen05.commit of both issuing warps
        }
        for (int j = 0; j < 2 * kPairs; ++j) {
            mbar_init(&a_full[j], 4);              // the four warps of the half that writes the pair
            mbar_init(&a_empty[j], 1);             // tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&min_full[b], 4);
            mbar_init(&min_empty[b], 1);
        }
        mbar_init(d_full, 2);
        mbar_fence_init();
        for (int c = 0; c < p.row_classes; ++c) tma_prefetch_descriptor(&wmaps.map[c]);
    }
    if (warp == kIssuerWarp) tmem_alloc(tmem_holder, P::kTmemColumns);
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    if (warp == 0) stamp(p, 2, 1);

    if (warp == kProducerWarp) {
        // ---------------- one lane streams both rings; the weights do not depend on the kernel before this one ----------------
        if (lane == 0) {
            bool ok = true;
            auto issue_raw = [&](int i) {
                const int s = i % p.raw_stages;
                if (i >= p.raw_stages && !mbar_wait_bounded_hint(&raw_empty[s], ((i / p.raw_stages) - 1) & 1, kWaitHintNs)) return false;
                mbar_arrive_expect_tx(&raw_full[s], P::kRawStageBytes);
                if constexpr (FMT == kQ6_K) {
                    // x in 16-bit elements: the super-block's first byte within the class's rows, rounded down to 16 bytes
                    const int rows = kRows / p.row_classes;
                    for (int c = 0; c < p.row_classes; ++c) {
                        const unsigned int delta = (static_cast<unsigned int>(c) * p.row_bytes) & 15u;
                        const int x = static_cast<int>((delta + static_cast<unsigned int>(sb_begin + i) * 210u) & ~15u) / 2;
                        tma_load_2d(raw + static_cast<size_t>(s) * P::kRawStageBytes + static_cast<size_t>(c) * rows * P::kRowPitch, &wmaps.map[c], x,
                                    n0 / p.row_classes, &raw_full[s]);
                    }
                } else {
                    tma_load_2d(raw + static_cast<size_t>(s) * P::kRawStageBytes, &wmaps.map[0], (sb_begin + i) * (P::kSbBytes / 2), n0, &raw_full[s]);
                }
                return true;
            };
            auto issue_b = [&](int i) {
                const int s = i % p.b_stages;
                if (i >= p.b_stages && !mbar_wait_bounded_hint(&b_empty[s], ((i / p.b_stages) - 1) & 1, kWaitHintNs)) return false;
                mbar_arrive_expect_tx(&b_full[s], I::kStageBytes);
                const uint8_t* src = p.image + static_cast<size_t>(sb_begin + i) * I::kStageBytes;
                uint8_t* dst = b_ring + static_cast<size_t>(s) * I::kStageBytes;
#pragma unroll 1
                for (uint32_t done = 0; done < static_cast<uint32_t>(I::kStageBytes); done += 10240u)
                    bulk_copy_g2s(dst + done, src + done, min(10240u, static_cast<uint32_t>(I::kStageBytes) - done), &b_full[s]);
                return true;
            };
            int raw_i = 0, b_i = 0;
            stamp(p, 0, 0);
            for (; raw_i < min(p.raw_stages, local_sb) && ok; ++raw_i) ok = issue_raw(raw_i);
            stamp(p, 0, 1);
            pdl_wait_prior();   // the activation tiles are the pre-pass's output
            stamp(p, 0, 2);
            for (; b_i < min(p.b_stages, local_sb) && ok; ++b_i) ok = issue_b(b_i);
            stamp(p, 0, 3);
            while (ok && (raw_i < local_sb || b_i < local_sb)) {
                if (b_i < local_sb) ok = issue_b(b_i++);
                if (ok && raw_i < local_sb) ok = issue_raw(raw_i++);
            }
            stamp(p, 0, 4);
            if (!ok) atomicExch(p.status, kDeviceWaitTimeout);
        }
        __syncwarp();
    } else if (warp == kIssuerWarp || warp == kIssuerWarp2) {
        // ---------------- MMA issuers: each warp runs converged, an elected lane issues ----------------
        // Issuing is the serial part of the pipeline (about 50 clocks per instruction for one thread), so two warps share
        // it: the first takes pairs 0, 1 and the minimum term, the second pairs 2, 3, each into its own accumulator.
        constexpr uint32_t idesc = umma_instr_desc(kRows, NT, /*A f16*/ 0, /*B f16*/ 0);
        const int which = warp == kIssuerWarp ? 0 : 1;
        const uint32_t d_tmem = tmem_base + P::kColD + which * NT;
        bool ok = true;
        for (int i = 0; i < local_sb && ok; ++i) {
            const int bs = i % p.b_stages;
            ok = __all_sync(0xffffffffu, mbar_wait_bounded_hint(&b_full[bs], (i / p.b_stages) & 1, kWaitHintNs));
            if (!ok) break;
            if (i < 4 && which == 0) stamp(p, 1, i * 4);
            const uint64_t desc_b0 = umma_smem_desc_sw128(smem_addr(b_ring + static_cast<size_t>(bs) * I::kStageBytes));
            const int abuf = i % AB;
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const int j = which * 2 + jj;
                ok = ok && __all_sync(0xffffffffu, mbar_wait_bounded_hint(&a_full[abuf * kPairs + j], (i / AB) & 1, kWaitHintNs));
                if (!ok) break;
                if (i < 4 && which == 0) stamp(p, 1, i * 4 + 1 + jj);
                tcgen05_fence_after_sync();
                // pair j = K step j of the super-block (64 elements): tile j of the stage, four K slices of 16
                umma_f16_tmem_a_pair_elected(d_tmem, tmem_base + (abuf * kPairs + j) * kPairColumns, desc_b0 + static_cast<uint64_t>(j * (I::kTileBytes >> 4)),
                                             idesc, (i > 0 || jj > 0) ? 1u : 0u);
                umma_commit_elected(&a_empty[abuf * kPairs + j]);
            }
            if (!ok) break;
            if (FMT != kQ6_K && which == 0) {
                // minimum term: A = -dmin * m[g] twice (K slots 0..7 meet the block sums' hi parts, 8..15 their lo parts)
                ok = __all_sync(0xffffffffu, mbar_wait_bounded_hint(&min_full[i & 1], (i >> 1) & 1, kWaitHintNs));
                if (!ok) break;
                tcgen05_fence_after_sync();
                umma_f16_tmem_a_elected(d_tmem, tmem_base + P::kColAMin + (i & 1) * 8, desc_b0 + static_cast<uint64_t>(4 * (I::kTileBytes >> 4)), idesc, 1u);
                umma_commit_elected(&min_empty[i & 1]);
            }
            umma_commit_elected(&b_empty[bs]);
            if (i < 4 && which == 0) stamp(p, 1, i * 4 + 3);
        }
        if (ok) umma_commit_elected(d_full);
        if (which == 0) stamp(p, 1, 16);
        if (!ok && lane == 0) atomicExch(p.status, kDeviceWaitTimeout);
        __syncwarp();
    } else {
        // ---------------- workers ----------------
        const int set = warp / kWorkerWarps;             // set s expands super-blocks s, s + kSets, ...
        const int half = (warp % kWorkerWarps) >> 2;     // which 128 weights of every super-block this thread expands
        const int quadrant = warp & 3;                   // a warp reaches TMEM lanes 32 * (warp % 4) .. + 31
        const int row_in_tile = quadrant * 32 + lane;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quadrant * 32) << 16);
        const uint32_t raw_addr = smem_addr(raw) + static_cast<uint32_t>(row_in_tile) * P::kRowPitch;
        bool ok = true;

#pragma unroll 1
        for (int i = set; i < local_sb; i += kSets) {
            const int s = i % p.raw_stages;
            if (ok && !mbar_wait_bounded_hint(&raw_full[s], (i / p.raw_stages) & 1, kWaitHintNs)) {
                atomicExch(p.status, kDeviceWaitTimeout);
                ok = false;
            }
            if (i < 4 && quadrant == 0 && set == 0) stamp(p, 2 + half, 2 + i * 4);
            const int abuf = i % AB;
            if constexpr (FMT == kQ6_K) {
                const uint32_t row_class = static_cast<uint32_t>(row_in_tile) / static_cast<uint32_t>(kRows / p.row_classes);
                const uint32_t blk = raw_addr + static_cast<uint32_t>(s) * P::kRawStageBytes +
                                     ((((row_class * p.row_bytes) & 15u) + static_cast<uint32_t>(sb_begin + i) * 210u) & 15u);
                const float d = f16_bits_to_f32(lds_u16(blk + 208));
                const bool wide = !(fabsf(d) <= 1.0f);   // kept symmetrical with the other formats: beyond it d multiplies afterwards
                if (!(fabsf(d) < 32.0f)) atomicExch(p.status, kDeviceScaleRange);
                const uint32_t d2 = half2_bits(d, d);
                const float fd = wide ? 1.0f : d;
                // this half's chunk of 128 weights: 64 low-nibble bytes, 32 two-bit bytes, eight int8 scales
                const uint32_t la = blk + 64 * half, lb = la + 32, qh = blk + 128 + 32 * half, sc = blk + 192 + 8 * half;
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const int j = half * 2 + jj;
                    const int slot = abuf * kPairs + j;
                    // groups 2 jj and 2 jj + 1 of the chunk; factor[0..1]: the two runs of 16 of the first, [2..3]: of the second
                    float factor[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r) factor[r] = fd * static_cast<float>(lds_s8(sc + 4 * jj + r));
                    uint32_t out_lo[16], out_hi[16];
                    if (jj == 0) unpack_pair_q6<0>(la, lb, qh, factor, out_lo, out_hi);
                    else unpack_pair_q6<2>(la, lb, qh, factor, out_lo, out_hi);
                    if (wide) {
#pragma unroll
                        for (int r = 0; r < 16; ++r) {
                            out_lo[r] = hmul2(out_lo[r], d2);
                            out_hi[r] = hmul2(out_hi[r], d2);
                        }
                    }
                    if (i >= AB && ok && !mbar_wait_bounded_hint(&a_empty[slot], ((i / AB) - 1) & 1, kWaitHintNs)) {
                        atomicExch(p.status, kDeviceWaitTimeout);
                        ok = false;
                    }
                    tcgen05_fence_after_sync();
                    tmem_st16(lane_base + slot * kPairColumns, out_lo);
                    tmem_st16(lane_base + slot * kPairColumns + 16, out_hi);
                    tmem_st_wait();
                    tcgen05_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&a_full[slot]);
                }
            } else {
            const uint32_t blk = raw_addr + static_cast<uint32_t>(s) * P::kRawStageBytes;
            const uint4 header = lds128(blk);   // d | dmin, 12 scale bytes
            uint32_t sc_lo, sc_hi, m_lo, m_hi;
            unpack_k_scales(header.y, header.z, header.w, sc_lo, sc_hi, m_lo, m_hi);
            const uint32_t sc_word = half ? sc_hi : sc_lo;   // scales of sub-blocks 4 half .. 4 half + 3
            const float d = f16_bits_to_f32(header.x & 0xffffu);
            const float dmin = f16_bits_to_f32(header.x >> 16);
            // 1024 * f16(d * sc) must stay finite: beyond |d| = 1 the pair is expanded without d and multiplied afterwards
            const bool wide = !(fabsf(d) <= 1.0f);
            if (!(fabsf(d) < 32.0f)) atomicExch(p.status, kDeviceScaleRange);
            const uint32_t d2 = half2_bits(d, d);
            if (half == 0) {
                const float nd = -dmin;
                uint32_t mins[8];
                mins[0] = half2_bits(nd * byte_of(m_lo, 0), nd * byte_of(m_lo, 1));
                mins[1] = half2_bits(nd * byte_of(m_lo, 2), nd * byte_of(m_lo, 3));
                mins[2] = half2_bits(nd * byte_of(m_hi, 0), nd * byte_of(m_hi, 1));
                mins[3] = half2_bits(nd * byte_of(m_hi, 2), nd * byte_of(m_hi, 3));
                mins[4] = mins[0]; mins[5] = mins[1]; mins[6] = mins[2]; mins[7] = mins[3];
                if (i >= 2 && ok && !mbar_wait_bounded_hint(&min_empty[i & 1], ((i >> 1) - 1) & 1, kWaitHintNs)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    ok = false;
                }
                tcgen05_fence_after_sync();
                tmem_st8(lane_base + P::kColAMin + (i & 1) * 8, mins);
                tmem_st_wait();
                tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&min_full[i & 1]);
            }
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const int j = half * 2 + jj;
                const int slot = abuf * kPairs + j;
                const float scale_a = byte_of(sc_word, 2 * jj), scale_b = byte_of(sc_word, 2 * jj + 1);
                const float fa = wide ? scale_a : scale_a * d, fb = wide ? scale_b : scale_b * d;
                uint32_t out_lo[16], out_hi[16];
                unpack_pair<FMT>(blk + kQuantOffset + 32 * j, blk + 16, j, half2_bits(fa, fa), half2_bits(fb, fb), out_lo, out_hi);
                if (wide) {
#pragma unroll
                    for (int r = 0; r < 16; ++r) {
                        out_lo[r] = hmul2(out_lo[r], d2);
                        out_hi[r] = hmul2(out_hi[r], d2);
                    }
                }
                if (i >= AB && ok && !mbar_wait_bounded_hint(&a_empty[slot], ((i / AB) - 1) & 1, kWaitHintNs)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    ok = false;
                }
                tcgen05_fence_after_sync();
                tmem_st16(lane_base + slot * kPairColumns, out_lo);
                tmem_st16(lane_base + slot * kPairColumns + 16, out_hi);
                tmem_st_wait();
                tcgen05_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[slot]);
            }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&raw_empty[s]);
            if (i < 4 && quadrant == 0 && set == 0) stamp(p, 2 + half, 3 + i * 4);
        }
        if (quadrant == 0 && set == 0) stamp(p, 2 + half, 20);

        // ---------------- the accumulators, once (first worker set): a thread holds its row's columns of this half ----------------
        if (set == 0) {
        pdl_wait_prior();   // the scale factors (and y, when it is accumulated into) come from earlier kernels
        if (threadIdx.x < NT) up[threadIdx.x] = reinterpret_cast<const float*>(p.image + I::scales_offset(p.nsb))[threadIdx.x];
        if (ok && !mbar_wait_bounded_hint(d_full, 0, kWaitHintNs)) {
            atomicExch(p.status, kDeviceWaitTimeout);
            ok = false;
        }
        tcgen05_fence_after_sync();
        if (quadrant == 0) stamp(p, 2 + half, 21);
        named_barrier_sync(1, kWorkers);   // the scale factors are in place
        const bool split = p.ksplit > 1;
        float* part = split ? p.partial + static_cast<size_t>(blockIdx.y) * p.members * p.n : nullptr;
        // tile row -> matrix row (interleaved classes for unaligned Q6_K rows, the identity otherwise)
        const int rows_per_class = kRows / p.row_classes;
        const long long row = static_cast<long long>(n0) + (row_in_tile % rows_per_class) * p.row_classes + row_in_tile / rows_per_class;
        const int column0 = half * (NT / 2);
#pragma unroll
        for (int c8 = 0; c8 < NT / 16; ++c8) {
            uint32_t d0[8], d1[8];
            tmem_ld8(lane_base + P::kColD + column0 + c8 * 8, d0);
            tmem_ld8(lane_base + P::kColD + NT + column0 + c8 * 8, d1);
            tmem_ld_wait();
            float v[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) v[c] = ok ? __uint_as_float(d0[c]) + __uint_as_float(d1[c]) : 0.0f;
            const int per_member = p.planes;   // columns per member
#pragma unroll
            for (int c = 0; c < 8; c += 1) {
                if (per_member == 2 && (c & 1)) continue;
                const int column = column0 + c8 * 8 + c;
                const int m = per_member == 2 ? column >> 1 : column;
                if (m < p.members && row < p.n) {
                    const float value = (per_member == 2 ? v[c] + v[c + 1 < 8 ? c + 1 : c] : v[c]) * up[m];
                    if (split) {
                        part[static_cast<size_t>(m) * p.n + row] = value;
                    } else {
                        size_t o;
                        void* y = output_slot(p, m, row, o);
                        if (p.y_bf16) {
                            const float old = p.accumulate ? __bfloat162float(static_cast<const __nv_bfloat16*>(y)[o]) : 0.0f;
                            static_cast<__nv_bfloat16*>(y)[o] = __float2bfloat16_rn(value + old);
                        } else {
                            const float old = p.accumulate ? static_cast<const float*>(y)[o] : 0.0f;
                            static_cast<float*>(y)[o] = value + old;
                        }
                    }
                }
            }
        }
        tcgen05_fence_before_sync();
        if (quadrant == 0) stamp(p, 2 + half, 23);
        // ---------------- split-K: the partial tiles of a row tile are added in split order ----------------
        // When the whole grid is resident at once (the launcher knows), every CTA of the row tile waits for the others'
        // partial tiles (bounded) and adds its own share of the tile: the sum is spread over `ksplit` SMs.  Otherwise the
        // CTA that draws the last ticket adds the whole tile (a CTA must not wait for one that may not have started).
        if (split) {
            __threadfence();
            named_barrier_sync(1, kWorkers);
            unsigned int* ticket = p.tickets + blockIdx.x;
            unsigned int* departed = p.tickets + p.ticket_stride + blockIdx.x;
            int first_item = 0, last_item = p.members * (kRows / 4);
            if (threadIdx.x == 0) {
                if (p.cooperative) {
                    atomicAdd(ticket, 1u);
                    unsigned long long start;
                    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(start));
                    bool all = true;
                    unsigned int spins = 0;
                    while (*reinterpret_cast<volatile unsigned int*>(ticket) < static_cast<unsigned int>(p.ksplit)) {
                        if ((++spins & 255u) == 0u) {
                            unsigned long long now;
                            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
                            if (now - start > 1000000000ull) {
                                all = false;
                                break;
                            }
                        }
                    }
                    if (!all) atomicExch(p.status, kDeviceWaitTimeout);
                    *last_flag = all ? 1u : 0u;
                } else {
                    const unsigned int drawn = atomicAdd(ticket, 1u);
                    const bool last = drawn == static_cast<unsigned int>(p.ksplit - 1);
                    if (last) *ticket = 0;   // ready for the next launch
                    *last_flag = last ? 1u : 0u;
                }
            }
            named_barrier_sync(1, kWorkers);
            if (p.cooperative) {
                const int items = p.members * (kRows / 4);
                first_item = static_cast<int>(static_cast<long long>(items) * blockIdx.y / p.ksplit);
                last_item = static_cast<int>(static_cast<long long>(items) * (blockIdx.y + 1) / p.ksplit);
            }
            if (*last_flag != 0) {
                __threadfence();
                const size_t plane = static_cast<size_t>(p.members) * p.n;
                const bool vector = (p.n & 3) == 0;
                for (int idx = first_item + static_cast<int>(threadIdx.x); idx < last_item; idx += kWorkers) {
                    const int m = idx / (kRows / 4);
                    const long long row = static_cast<long long>(n0) + (idx % (kRows / 4)) * 4;
                    if (row >= p.n) continue;
                    const size_t o = static_cast<size_t>(m) * p.n + row;
                    float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    if (vector) {
                        int z = 0;
                        for (; z + 4 <= p.ksplit; z += 4) {   // four loads in flight, added in split order
                            const float4 a = __ldcg(reinterpret_cast<const float4*>(p.partial + (z + 0) * plane + o));
                            const float4 b = __ldcg(reinterpret_cast<const float4*>(p.partial + (z + 1) * plane + o));
                            const float4 c = __ldcg(reinterpret_cast<const float4*>(p.partial + (z + 2) * plane + o));
                            const float4 e = __ldcg(reinterpret_cast<const float4*>(p.partial + (z + 3) * plane + o));
                            sum[0] = (((sum[0] + a.x) + b.x) + c.x) + e.x;
                            sum[1] = (((sum[1] + a.y) + b.y) + c.y) + e.y;
                            sum[2] = (((sum[2] + a.z) + b.z) + c.z) + e.z;
                            sum[3] = (((sum[3] + a.w) + b.w) + c.w) + e.w;
                        }
                        for (; z < p.ksplit; ++z) {
                            const float4 a = __ldcg(reinterpret_cast<const float4*>(p.partial + z * plane + o));
                            sum[0] += a.x; sum[1] += a.y; sum[2] += a.z; sum[3] += a.w;
                        }
                    } else {
                        for (int z = 0; z < p.ksplit; ++z)
                            for (int r = 0; r < 4; ++r)
                                if (row + r < p.n) sum[r] += __ldcg(p.partial + z * plane + o + r);
                    }
                    size_t out;
                    void* y = output_slot(p, m, row, out);
                    for (int r = 0; r < 4; ++r) {
                        if (row + r >= p.n) break;
                        if (p.y_bf16) {
                            if (p.accumulate) sum[r] += __bfloat162float(static_cast<const __nv_bfloat16*>(y)[out + r]);
                            static_cast<__nv_bfloat16*>(y)[out + r] = __float2bfloat16_rn(sum[r]);
                        } else {
                            if (p.accumulate) sum[r] += static_cast<const float*>(y)[out + r];
                            static_cast<float*>(y)[out + r] = sum[r];
                        }
                    }
                }
            }
            if (p.cooperative) {
                // the last CTA to leave resets both counters: by then every CTA of the row tile has passed its wait
                named_barrier_sync(1, kWorkers);
                if (threadIdx.x == 0 && atomicAdd(departed, 1u) == static_cast<unsigned int>(p.ksplit - 1)) {
                    *departed = 0;
                    *ticket = 0;
                }
            }
        }
        }   // first worker set
    }

    // ---------------- teardown: every warp arrives here, then TMEM is released ----------------
    if (warp == 0) stamp(p, 2, 24);
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == kIssuerWarp) tmem_dealloc(tmem_base, P::kTmemColumns);
    if (warp == 0) stamp(p, 2, 25);
}

constexpr size_t kSmemLimit = 227 * 1024;

// K splits by a cost model in units of super-blocks: waves of CTAs x (super-blocks per CTA + a fixed cost per CTA).
int choose_splits(int tiles, int nsb, int ctas_per_wave, int members, size_t scratch_bytes, int n, int max_tickets) {
    max_tickets /= 2;   // arrivals and departures
    constexpr double kFixedCost = 5.0;
    int best = 1;
    double best_cost = 1e30;
    for (int ks = 1; ks <= nsb && ks <= 32; ++ks) {
        if (ks > 1 && (static_cast<size_t>(ks) * members * n * sizeof(float) > scratch_bytes || tiles > max_tickets)) break;
        const int waves = (tiles * ks + ctas_per_wave - 1) / ctas_per_wave;
        // the last CTA of a row tile reads ks partial tiles of members x 128 floats: about one super-block time per 32 KB
        // one wave: the CTAs of a row tile share the sum (each reads members x 128 floats in all); more: the last one reads all
        const double reduce = ks <= 1 ? 0.0 : (waves == 1 ? 1.0 + members * 512.0 / 32768.0 : 1.0 + ks * members * 512.0 / 32768.0);
        const double cost = waves * ((nsb + ks - 1) / ks + kFixedCost + reduce);
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = ks;
        }
    }
    return best;
}

template <uint32_t FMT, int NT>
cudaError_t launch_format(const TmemGemvArgs& a) {
    using P = TmemPlan<FMT, NT>;
    using I = typename P::I;
    auto kernel = qgemv_tmem_kernel<FMT, NT>;
    const int nsb = a.k / kSuperBlock;
    const int tiles = (a.n + kRows - 1) / kRows;
    // scratch: [activation image][split-K partial tiles]
    const size_t image_bytes = (I::bytes(nsb) + 1023) / 1024 * 1024;
    if (image_bytes > a.scratch_bytes) return cudaErrorInvalidConfiguration;
    uint8_t* image = static_cast<uint8_t*>(a.scratch);
    float* partial = reinterpret_cast<float*>(image + image_bytes);
    const size_t partial_bytes = a.scratch_bytes - image_bytes;
    // rings: two CTAs per SM for the narrow accumulators, one for 64 columns
    const int resident = NT >= 64 ? 1 : 2;
    const size_t budget = (kSmemLimit - 1024 * resident) / resident;
    int raw_stages = kMaxStages, b_stages = 3;
    while (P::smem_bytes(raw_stages, b_stages) > budget && (raw_stages > 2 || b_stages > 2)) {
        if (raw_stages > b_stages || b_stages == 2) --raw_stages;
        else --b_stages;
    }
    if (a.stages > 0 && a.stages < raw_stages) raw_stages = a.stages < 2 ? 2 : a.stages;
    const size_t smem = P::smem_bytes(raw_stages, b_stages);
    if (smem > kSmemLimit) return cudaErrorInvalidConfiguration;
    int ksplit = choose_splits(tiles, nsb, resident * a.sm_count, a.members, partial_bytes, a.n, a.ticket_count);
    if (a.force_ksplit > 0 && a.force_ksplit <= nsb && static_cast<size_t>(a.force_ksplit) * a.members * a.n * sizeof(float) <= partial_bytes &&
        tiles <= a.ticket_count)
        ksplit = a.force_ksplit;
    const bool cooperative = ksplit > 1 && tiles * ksplit <= resident * a.sm_count && 2 * tiles <= a.ticket_count;
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
    int classes = 1;
    while ((row_bytes * classes) % 16 != 0) classes *= 2;   // 1 for Q4_K / Q5_K; up to 8 for Q6_K
    WeightMaps wmaps{};
    for (int c = 0; c < classes; ++c) {
        const unsigned long long first = static_cast<unsigned long long>(c) * row_bytes, delta = first & 15ull;
        const unsigned long long class_rows = (static_cast<unsigned long long>(a.n) - c + classes - 1) / classes;
        if (static_cast<unsigned long long>(a.n) <= static_cast<unsigned long long>(c)) {
            wmaps.map[c] = wmaps.map[0];   // fewer rows than classes: never addressed with a valid row
            continue;
        }
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>((delta + row_bytes) / 2), static_cast<cuuint64_t>(class_rows)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes * classes)};
        const cuuint32_t box[2] = {static_cast<cuuint32_t>(P::kRowPitch / 2), static_cast<cuuint32_t>(kRows / classes)};
        const cuuint32_t elem[2] = {1, 1};
        if (encode(&wmaps.map[c], CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<uint8_t*>(a.weights) + (first - delta), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    TmemParams p{};
    p.x = a.x;
    p.x_bf16 = a.x_bf16 ? 1 : 0;
    p.mode = a.mode;
    p.norm_weight = a.norm_weight;
    p.eps = a.eps;
    p.image = image;
    p.y = a.y;
    p.y2 = a.y2;
    p.n_first = a.y2 != nullptr ? a.n_first : a.n;
    p.y_bf16 = a.y_bf16 ? 1 : 0;
    p.accumulate = a.accumulate ? 1 : 0;
    p.partial = partial;
    p.tickets = a.tickets;
    p.ticket_stride = a.ticket_count / 2;
    p.cooperative = cooperative ? 1 : 0;
    p.k = a.k;
    p.n = a.n;
    p.nsb = nsb;
    p.members = a.members;
    // f32 activations reach this kernel only on request (option tc_f32_activations), as values rounded to f16 under the
    // member row's power-of-two factor: one plane, like bf16.  (The image and the read-back also serve two planes, hi + lo.)
    p.planes = 1;
    p.ksplit = ksplit;
    p.raw_stages = raw_stages;
    p.b_stages = b_stages;
    p.row_classes = classes;
    p.row_bytes = static_cast<unsigned int>(row_bytes);
    p.status = a.device_status;
    p.trace = a.trace;
    if (!a.image_ready) {
        const int cached = a.k <= kImageCacheFloats ? 1 : 0;
        static int image_device = -1;
        if (image_device != device) {
            const cudaError_t attribute = cudaFuncSetAttribute(tmem_image_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                               static_cast<int>(kImageCacheFloats * sizeof(float)));
            if (attribute != cudaSuccess) return attribute;
            image_device = device;
        }
        // two super-blocks per warp and trip: as many warps as that takes, between 8 and 32
        int image_warps = (nsb + 1) / 2;
        image_warps = image_warps < 8 ? 8 : image_warps > 32 ? 32 : image_warps;
        const cudaError_t e = launch_kernel(tmem_image_kernel<NT>, dim3(a.members), dim3(32 * image_warps), cached ? static_cast<size_t>(a.k) * sizeof(float) : 0,
                                            a.stream, p, cached);
        if (e != cudaSuccess) return e;
    }
    return launch_kernel(kernel, dim3(tiles, ksplit), dim3(Roles<NT>::kThreads), smem, a.stream, wmaps, p);
}

template <uint32_t FMT>
cudaError_t launch_columns(const TmemGemvArgs& a) {
    const int columns = a.members;
    if (columns <= 16) return launch_format<FMT, 16>(a);
    if (columns <= 32) return launch_format<FMT, 32>(a);
    return launch_format<FMT, 64>(a);
}

}  // namespace

bool qgemv_tmem_supports(uint32_t value_type, int k, int n, int members, bool x_bf16, const void* weights) {
    if (value_type != kQ4_K && value_type != kQ5_K && value_type != kQ6_K) return false;
    (void)x_bf16;
    if (members < 1 || members > 64 || k <= 0 || k % kSuperBlock != 0 || n < 1) return false;
    if (value_type == kQ6_K && static_cast<unsigned long long>(k / kSuperBlock) * 210ull > 0xffffffffull) return false;
    return reinterpret_cast<uintptr_t>(weights) % 16 == 0;
}

cudaError_t launch_qgemv_tmem(const TmemGemvArgs& a) {
    switch (a.value_type) {
        case kQ4_K: return launch_columns<kQ4_K>(a);
        case kQ5_K: return launch_columns<kQ5_K>(a);
        case kQ6_K: return launch_columns<kQ6_K>(a);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ribn
