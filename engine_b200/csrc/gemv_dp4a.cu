// Dequant-fused GEMV for 1..4 activation rows on the integer dot-product pipe,
// optionally with the RMSNorm that feeds it fused into the prologue.
//
//   y[m][n] = sum_k dequant(W[n][k]) * x[m][k]
//
// Same operation, boundary and data movement as gemv.cu (bulk-copy ring, equal
// row ranges per CTA, per-warp scale tables, fixed-order reduction); what
// changes is the arithmetic.  On B200 a 4.5-bit weight arrives every ~0.024 SM
// clocks, so a kernel that converts each quant to f32 and issues one FMA per
// weight is bound by instruction issue at a fraction of HBM speed (measured:
// ~80 warp instructions per 256 weights against a budget of ~25).  Here the
// quants stay packed four to a register and meet the activations in dp4a:
//
//   * the activation rows arrive packed by quantize.cu as two int8 planes per
//     block of 32:  x = d * (q1 + q2/256), d a power of two >= max|x|/127 --
//     14-15 bits of the block maximum, an error below 3.1e-5 of the block
//     maximum per element against the 2e-3 the path allows (one int8 plane, as
//     in the reference's optional Q8_1 mode, would not do), and exact for
//     activations that have few significant bits, bf16 among them; the f32 sum
//     of each block is kept for the "minimum" term of Q4_K/Q5_K.  The producer
//     warp bulk-copies the packed rows into shared memory once per CTA;
//   * a lane owns 16 consecutive quant bytes: 32 weights of Q4_K/Q5_K/Q6_K (16
//     of each of two groups) or 16 of Q8_0; it unpacks them with word-wide
//     logic ops and issues 4 dp4a per plane and group;
//   * per lane and group one integer->float conversion and three FMAs apply
//     weight scale x activation scale and the group minimum.
//
// Reference counterparts: q*_gemv_warp / _warp_batch
// (crates/nvidia/src/kernels/quantized/q4_k.cu:103-258 and twins) for the
// contract, q*_q8_1_gemv (q4_k_q8_1.cu:40-144 and twins) for the idea of an
// integer dot, rms_norm (crates/nvidia/src/model_ops.rs:106-147) for the fused
// prologue.
#include "formats.cuh"
#include "internal.h"
#include "pack_activations.cuh"
#include "pipeline.cuh"

namespace ribn {
namespace {

constexpr int kWR = 2;             // row groups per CTA
constexpr int kWK = 4;             // K slices per CTA.  Measured against kWK = 1 (a warp owns its rows over the whole K range and a
                                   // tile ends without the CTA-wide exchange; 8 x 2 rows per tile, 8 super-blocks per stage): within
                                   // 5 % on the 12288-row shapes, 20-30 % slower on 1024 rows, where a CTA has too few rows for
                                   // eight row-owning warps
constexpr int kRW = 4;             // rows per warp
constexpr int kConsumerWarps = kWR * kWK;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kRows = kWR * kRW;   // rows per tile
constexpr int kKB = 16;            // super-blocks per row per stage

struct Dp4aParams {
    const uint8_t* w;
    unsigned long long w_bytes;
    unsigned long long row_bytes;
    const uint8_t* xq;             // packed activations (quantize.cu), `x_stride` bytes per member; used when pack_mode < 0
    unsigned long long x_stride;
    // pack_mode >= 0: the kernel packs the activations itself (every CTA its own copy in shared memory: a few thousand
    // values, cheaper than a separate launch and the dependency on it).  0 plain, 1 RMSNorm first, 2 silu(gate) * up.
    int pack_mode;
    const void* x_raw;             // [members][k] (mode 2: [members][2k]) f32 or bf16
    int x_raw_bf16;
    const float* norm_weight;
    float eps;
    void* y;
    int k;
    int n;
    int nsb;
    int members;
    int y_bf16;
    int accumulate;                // y += W x
    int stages;
    int* status;
    long long* trace;              // diagnostics (builds with -DRIBN_TRACE): wall-clock stamps of CTA 0, or null
};

// Diagnostics, compiled in with -DRIBN_TRACE only: trace[event] = globaltimer, CTA 0.
__device__ __forceinline__ void wall_stamp(const Dp4aParams& p, int event) {
#ifdef RIBN_TRACE
    if (p.trace != nullptr && blockIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.trace[event] = static_cast<long long>(t);
    }
#else
    (void)p;
    (void)event;
#endif
}

// Lanes per super-block and the geometry of a lane's 16 quant bytes.
template <uint32_t FMT>
struct LaneMap {
    static constexpr int kLanesPerSb = FMT == kQ8_0 ? 16 : 8;
    static constexpr int kSbPerIter = 32 / kLanesPerSb;  // super-blocks a warp covers per iteration
};

__device__ __forceinline__ uint4 lds128(const void* p) { return *reinterpret_cast<const uint4*>(p); }

// 16 bytes from a shared address that is only 2-byte aligned.
__device__ __forceinline__ uint4 lds128_a2(const uint8_t* p) {
    uint4 v;
    v.x = ld_u32_a2(p);
    v.y = ld_u32_a2(p + 4);
    v.z = ld_u32_a2(p + 8);
    v.w = ld_u32_a2(p + 12);
    return v;
}

__device__ __forceinline__ int dot16(const uint4& a, const uint4& b) {
    int s = __dp4a(static_cast<int>(a.x), static_cast<int>(b.x), 0);
    s = __dp4a(static_cast<int>(a.y), static_cast<int>(b.y), s);
    s = __dp4a(static_cast<int>(a.z), static_cast<int>(b.z), s);
    return __dp4a(static_cast<int>(a.w), static_cast<int>(b.w), s);
}

// Activation planes of one member for the lane's two 16-element runs.
struct XRun {
    uint4 q1a, q2a, q1b, q2b;
    float da, db;  // d/256 of the 32-blocks the runs belong to
    float sa, sb;  // f32 block sums, non-zero only in the lane that applies the minimum term
};

template <uint32_t FMT>
struct Dp4aFormat;

// Q4_K: lane l8 of a super-block: pair j = l8 >> 1 (groups 2j, 2j+1), half h = l8 & 1 (bytes 16h..16h+15 of
// the pair's 32 nibble bytes).  Run A = low nibbles (group 2j), run B = high nibbles (group 2j+1).
template <>
struct Dp4aFormat<kQ4_K> {
    __device__ static void runs(int l, int& ka, int& kb) {
        ka = (l >> 1) * 64 + (l & 1) * 16;
        kb = ka + 32;
    }
    __device__ static bool owns_minimum(int l) { return (l & 1) == 0; }
    __device__ static void quants(const uint8_t* blk, int l, uint4& qa, uint4& qb) {
        const uint4 w = lds128(blk + 16 + (l >> 1) * 32 + (l & 1) * 16);
        qa = make_uint4(w.x & 0x0f0f0f0fu, w.y & 0x0f0f0f0fu, w.z & 0x0f0f0f0fu, w.w & 0x0f0f0f0fu);
        qb = make_uint4((w.x >> 4) & 0x0f0f0f0fu, (w.y >> 4) & 0x0f0f0f0fu, (w.z >> 4) & 0x0f0f0f0fu,
                        (w.w >> 4) & 0x0f0f0f0fu);
    }
    __device__ static void scales(const float* table, int l, float& sa, float& ma, float& sb, float& mb) {
        const float4 t = *reinterpret_cast<const float4*>(table + (l >> 1) * 4);
        sa = t.x; ma = t.y; sb = t.z; mb = t.w;
    }
};

template <>
struct Dp4aFormat<kQ5_K> {
    __device__ static void runs(int l, int& ka, int& kb) { Dp4aFormat<kQ4_K>::runs(l, ka, kb); }
    __device__ static bool owns_minimum(int l) { return (l & 1) == 0; }
    __device__ static void quants(const uint8_t* blk, int l, uint4& qa, uint4& qb) {
        const uint4 w = lds128(blk + 48 + (l >> 1) * 32 + (l & 1) * 16);
        const uint4 h = lds128(blk + 16 + (l & 1) * 16);  // fifth bits of positions 16h..16h+15, bit g = group g
        const int g = (l >> 1) * 2;
        qa.x = (w.x & 0x0f0f0f0fu) | (((h.x >> g) & 0x01010101u) << 4);
        qa.y = (w.y & 0x0f0f0f0fu) | (((h.y >> g) & 0x01010101u) << 4);
        qa.z = (w.z & 0x0f0f0f0fu) | (((h.z >> g) & 0x01010101u) << 4);
        qa.w = (w.w & 0x0f0f0f0fu) | (((h.w >> g) & 0x01010101u) << 4);
        qb.x = ((w.x >> 4) & 0x0f0f0f0fu) | (((h.x >> (g + 1)) & 0x01010101u) << 4);
        qb.y = ((w.y >> 4) & 0x0f0f0f0fu) | (((h.y >> (g + 1)) & 0x01010101u) << 4);
        qb.z = ((w.z >> 4) & 0x0f0f0f0fu) | (((h.z >> (g + 1)) & 0x01010101u) << 4);
        qb.w = ((w.w >> 4) & 0x0f0f0f0fu) | (((h.w >> (g + 1)) & 0x01010101u) << 4);
    }
    __device__ static void scales(const float* table, int l, float& sa, float& ma, float& sb, float& mb) {
        Dp4aFormat<kQ4_K>::scales(table, l, sa, ma, sb, mb);
    }
};

// Q6_K: lane l8: chunk c = l8 >> 2, h = (l8 >> 1) & 1, half p = l8 & 1: ql bytes c*64 + h*32 + 16p .. +15;
// run A = low nibbles = group 4c + h, run B = high nibbles = group 4c + h + 2, positions 16p..16p+15 of each.
template <>
struct Dp4aFormat<kQ6_K> {
    __device__ static void runs(int l, int& ka, int& kb) {
        ka = ((l >> 2) * 4 + ((l >> 1) & 1)) * 32 + (l & 1) * 16;
        kb = ka + 64;
    }
    __device__ static bool owns_minimum(int) { return false; }
    __device__ static uint32_t q6(uint32_t low, uint32_t high) {
        // 0..63 -> signed -32..31, bytewise
        return __vsub4(low | (high << 4), 0x20202020u);
    }
    __device__ static void quants(const uint8_t* blk, int l, uint4& qa, uint4& qb) {
        const uint4 lo = lds128_a2(blk + (l >> 2) * 64 + ((l >> 1) & 1) * 32 + (l & 1) * 16);
        const uint4 hi = lds128_a2(blk + 128 + (l >> 2) * 32 + (l & 1) * 16);
        const int s = ((l >> 1) & 1) * 2;  // shift of run A's two high bits; run B's are 4 further up
        qa.x = q6(lo.x & 0x0f0f0f0fu, (hi.x >> s) & 0x03030303u);
        qa.y = q6(lo.y & 0x0f0f0f0fu, (hi.y >> s) & 0x03030303u);
        qa.z = q6(lo.z & 0x0f0f0f0fu, (hi.z >> s) & 0x03030303u);
        qa.w = q6(lo.w & 0x0f0f0f0fu, (hi.w >> s) & 0x03030303u);
        qb.x = q6((lo.x >> 4) & 0x0f0f0f0fu, (hi.x >> (s + 4)) & 0x03030303u);
        qb.y = q6((lo.y >> 4) & 0x0f0f0f0fu, (hi.y >> (s + 4)) & 0x03030303u);
        qb.z = q6((lo.z >> 4) & 0x0f0f0f0fu, (hi.z >> (s + 4)) & 0x03030303u);
        qb.w = q6((lo.w >> 4) & 0x0f0f0f0fu, (hi.w >> (s + 4)) & 0x03030303u);
    }
    __device__ static void scales(const float* table, int l, float& sa, float& ma, float& sb, float& mb) {
        const int g = (l >> 2) * 4 + ((l >> 1) & 1);
        sa = table[2 * g + (l & 1)];
        sb = table[2 * g + 4 + (l & 1)];
        ma = 0.0f;
        mb = 0.0f;
    }
};

// Q8_0 (eight 34-byte blocks per super-block): lane l16: block b = l16 >> 1, half h = l16 & 1;
// run A = 16 int8 of that half; there is no run B.
template <>
struct Dp4aFormat<kQ8_0> {
    __device__ static void runs(int l, int& ka, int& kb) {
        ka = l * 16;
        kb = ka;
    }
    __device__ static bool owns_minimum(int) { return false; }
    __device__ static void quants(const uint8_t* blk, int l, uint4& qa, uint4& qb) {
        qa = lds128_a2(blk + (l >> 1) * 34 + 2 + (l & 1) * 16);
        qb = make_uint4(0, 0, 0, 0);
    }
    __device__ static void scales(const float* table, int l, float& sa, float& ma, float& sb, float& mb) {
        sa = table[l >> 1];
        sb = 0.0f;
        ma = 0.0f;
        mb = 0.0f;
    }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

// Shared-memory plan (all offsets multiples of 16):
//   ring      stages x kRows x slot
//   tables    consumer warps x (kRW * kKB / kWK) x 16 floats
//   red       2 x kWK x kRows x MT floats
//   packed x  MT x (2*kpad int8 + 2*(kpad/32) floats)      (kpad = nsb * 256)
//   barriers
template <uint32_t FMT, int MT>
struct Dp4aPlan {
    using F = Format<FMT>;
    static constexpr int kSlot = ((kKB * F::kBytes + 15) / 16) * 16 + 16;
    static constexpr int kStageBytes = kRows * kSlot;
    static constexpr int kTableFloats = kRW * (kKB / kWK) * 16;
    static constexpr int kTableBytes = kConsumerWarps * kTableFloats * 4;
    static constexpr int kRedBytes = ((2 * kWK * kRows * MT * 4 + 15) / 16) * 16;
    static constexpr int kMaxStages = 8;
    __host__ __device__ static size_t x_bytes(int kpad) { return static_cast<size_t>(MT) * packed_activation_stride(kpad); }
    __host__ __device__ static size_t fixed_bytes(int kpad) {
        return kTableBytes + kRedBytes + x_bytes(kpad) + (2 * kMaxStages + 3) * 8;
    }
};

template <uint32_t FMT, int MT>
__global__ void __launch_bounds__(kThreads) gemv_dp4a_kernel(const Dp4aParams p) {
    using P = Dp4aPlan<FMT, MT>;
    using F = Format<FMT>;
    using D = Dp4aFormat<FMT>;
    using L = LaneMap<FMT>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int kpad = p.nsb * kSuperBlock;
    const int blocks32 = kpad / 32;
    uint8_t* ring = smem;
    uint8_t* cursor = smem + static_cast<size_t>(p.stages) * P::kStageBytes;
    float* tables = reinterpret_cast<float*>(cursor);
    cursor += P::kTableBytes;
    float* red = reinterpret_cast<float*>(cursor);
    cursor += P::kRedBytes;
    const uint8_t* xs = cursor;  // packed activations, member m at m * x_stride
    cursor += P::x_bytes(kpad);
    uint64_t* full = reinterpret_cast<uint64_t*>(cursor);
    uint64_t* empty = full + P::kMaxStages;
    uint64_t* red_bar = empty + P::kMaxStages;
    uint64_t* x_bar = red_bar + 2;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int stages = p.stages;
    pdl_launch_dependents();
    if (threadIdx.x == 0) wall_stamp(p, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full[s], 32);
            mbar_init(&empty[s], kConsumerWarps);
        }
        mbar_init(&red_bar[0], kConsumerWarps);
        mbar_init(&red_bar[1], kConsumerWarps);
        mbar_init(x_bar, 1);
        mbar_fence_init();
    }
    __syncthreads();

    const long long row_begin = static_cast<long long>(p.n) * blockIdx.x / gridDim.x;
    const long long row_end = static_cast<long long>(p.n) * (blockIdx.x + 1) / gridDim.x;
    const int tiles = static_cast<int>((row_end - row_begin + kRows - 1) / kRows);
    const int chunks = (p.nsb + kKB - 1) / kKB;
    const int total = tiles * chunks;

    if (warp == kConsumerWarps) {
        // ---------------- producer warp: the weight stream does not depend on the activations ----------------
        const unsigned long long safe_end = p.w_bytes & ~15ull;
        // The first ring-full of weight stages is requested before the packed activations: those come from the
        // previous kernel of the stream, which this one may overlap.
        const int prefetch = min(total, stages);
        auto request_activations = [&]() {
            if (lane == 0) wall_stamp(p, 1);
            if (p.pack_mode >= 0) return;   // the consumers pack the activations themselves
            pdl_wait_prior();
            if (lane == 0) wall_stamp(p, 2);
            if (lane == 0) {
                // Packed activations of this launch's members: one bulk copy (a multiple of 576 bytes).
                const uint32_t bytes = static_cast<uint32_t>(static_cast<unsigned long long>(min(p.members, MT)) * p.x_stride);
                mbar_arrive_expect_tx(x_bar, bytes);
                bulk_copy_g2s(const_cast<uint8_t*>(xs), p.xq, bytes, x_bar);
            }
        };
        if (total == 0) request_activations();
        for (int it = 0; it < total; ++it) {
            const int s = it % stages;
            const int use = it / stages;
            if (use > 0 && !mbar_wait_bounded(&empty[s], (use - 1) & 1)) {
                atomicExch(p.status, kDeviceWaitTimeout);
                return;
            }
            const int tile = it / chunks;
            const int chunk = it - tile * chunks;
            const long long row = row_begin + static_cast<long long>(tile) * kRows + lane;
            const int sb0 = chunk * kKB;
            const int nsbs = min(kKB, p.nsb - sb0);
            if (lane < kRows && row < row_end) {
                const unsigned long long g0 = static_cast<unsigned long long>(row) * p.row_bytes +
                                              static_cast<unsigned long long>(sb0) * F::kBytes;
                const unsigned long long g1 = min(g0 + static_cast<unsigned long long>(nsbs) * F::kBytes,
                                                  static_cast<unsigned long long>(row + 1) * p.row_bytes);
                const unsigned long long a0 = g0 & ~15ull;
                const unsigned long long a1 = (g1 + 15ull) & ~15ull;
                uint8_t* dst = ring + static_cast<size_t>(s) * P::kStageBytes + lane * P::kSlot;
                if (a1 <= safe_end) {
                    const uint32_t bytes = static_cast<uint32_t>(a1 - a0);
                    mbar_arrive_expect_tx(&full[s], bytes);
                    bulk_copy_g2s(dst, p.w + a0, bytes, &full[s]);
                } else {
                    const unsigned long long bulk_end = safe_end > a0 ? safe_end : a0;
                    for (unsigned long long o = bulk_end; o < g1; ++o) dst[o - a0] = p.w[o];
                    const uint32_t bytes = static_cast<uint32_t>(bulk_end - a0);
                    if (bytes > 0) {
                        mbar_arrive_expect_tx(&full[s], bytes);
                        bulk_copy_g2s(dst, p.w + a0, bytes, &full[s]);
                    } else {
                        mbar_arrive(&full[s]);
                    }
                }
            } else {
                mbar_arrive(&full[s]);
            }
            if (it == prefetch - 1) request_activations();
        }
        return;
    }

    // ---------------- consumers: the packed activations, fetched or made here ----------------
    if (p.pack_mode >= 0) {
        pdl_wait_prior();   // the raw activations may be the previous kernel's output
        const int rows = min(p.members, MT);
        const size_t row_elements = static_cast<size_t>(p.k) * (p.pack_mode == 2 ? 2 : 1);
        for (int m = 0; m < rows; ++m) {
            const AnyRow row{static_cast<const uint8_t*>(p.x_raw) + m * row_elements * (p.x_raw_bf16 ? 2 : 4), p.x_raw_bf16};
            pack_activation_row<kConsumerThreads>(row, p.pack_mode, p.norm_weight, p.eps, const_cast<uint8_t*>(xs) + m * p.x_stride, p.k, kpad,
                                                  red, static_cast<int>(threadIdx.x), [] { named_barrier_sync(1, kConsumerThreads); });
        }
        named_barrier_sync(1, kConsumerThreads);
    } else if (!mbar_wait_bounded(x_bar, 0)) {
        atomicExch(p.status, kDeviceWaitTimeout);
        return;
    }
    if (threadIdx.x == 0) wall_stamp(p, 3);

    // ---------------- consumers: main loop ----------------
    const int wr = warp / kWK;
    const int wk = warp % kWK;
    const int sub = lane / L::kLanesPerSb;   // which super-block of the iteration's group
    const int l = lane % L::kLanesPerSb;     // position inside the super-block
    int ka, kb;
    D::runs(l, ka, kb);
    const bool owner = D::owns_minimum(l);
    float* table = tables + warp * P::kTableFloats;
    constexpr int kSbPerWarp = kKB / kWK;                  // super-blocks per warp per stage
    constexpr int kIters = kSbPerWarp / L::kSbPerIter;     // iterations per stage

    for (int tile = 0; tile < tiles; ++tile) {
        float acc[kRW][MT];
#pragma unroll
        for (int r = 0; r < kRW; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;
        const long long row_base = row_begin + static_cast<long long>(tile) * kRows + wr * kRW;

        for (int chunk = 0; chunk < chunks; ++chunk) {
            const int it = tile * chunks + chunk;
            const int s = it % stages;
            const int sb0 = chunk * kKB;
            const int nsbs = min(kKB, p.nsb - sb0);
            if (!mbar_wait_bounded(&full[s], (it / stages) & 1)) {
                atomicExch(p.status, kDeviceWaitTimeout);
                return;
            }
            if (threadIdx.x == 0 && it < 12) wall_stamp(p, 8 + 2 * it);
            const uint8_t* stage = ring + static_cast<size_t>(s) * P::kStageBytes + wr * kRW * P::kSlot;

            // Scale tables: one lane per (row, super-block) of this warp's share of the stage.
            // The warp's super-blocks are wk*kSbPerWarp .. +kSbPerWarp-1 of the stage.
            for (int e = lane; e < kRW * kSbPerWarp; e += 32) {
                const int r = e / kSbPerWarp;
                const int sbl = wk * kSbPerWarp + (e % kSbPerWarp);
                const long long row = row_base + r;
                if (sbl < nsbs && row < row_end) {
                    const uint32_t off = (F::kBytes % 16 == 0 && FMT != kQ8_0)
                                             ? 0u
                                             : static_cast<uint32_t>((static_cast<unsigned long long>(row) * p.row_bytes +
                                                                      static_cast<unsigned long long>(sb0) * F::kBytes) & 15ull);
                    F::decode_table(stage + r * P::kSlot + off + sbl * F::kBytes, table + e * 16);
                }
            }
            __syncwarp();

#pragma unroll
            for (int i = 0; i < kIters; ++i) {
                const int sbw = i * L::kSbPerIter + sub;       // index within the warp's share
                const int sbl = wk * kSbPerWarp + sbw;         // index within the stage
                // Whole super-blocks past the end of K (stage tail) and, for Q8_0, the part of the last
                // super-block past K contribute nothing.
                const int kbase = (sb0 + sbl) * kSuperBlock;
                const bool lane_ok = sbl < nsbs && (FMT != kQ8_0 || kbase + ka < p.k);
                XRun xr[MT];
                if (lane_ok) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const uint8_t* xm = xs + static_cast<size_t>(m) * p.x_stride;
                        const uint8_t* q1m = xm + kbase;
                        const uint8_t* q2m = xm + kpad + kbase;
                        const float* dq = reinterpret_cast<const float*>(xm + 2 * static_cast<size_t>(kpad));
                        const float* xsum = dq + blocks32;
                        xr[m].q1a = lds128(q1m + ka);
                        xr[m].q2a = lds128(q2m + ka);
                        const int ba = (kbase + ka) >> 5;
                        xr[m].da = dq[ba];
                        xr[m].sa = owner ? xsum[ba] : 0.0f;
                        if (FMT != kQ8_0) {
                            xr[m].q1b = lds128(q1m + kb);
                            xr[m].q2b = lds128(q2m + kb);
                            const int bb = (kbase + kb) >> 5;
                            xr[m].db = dq[bb];
                            xr[m].sb = owner ? xsum[bb] : 0.0f;
                        }
                    }
#pragma unroll
                    for (int r = 0; r < kRW; ++r) {
                        const long long row = row_base + r;
                        if (row < row_end) {
                            const uint32_t off = (F::kBytes % 16 == 0 && FMT != kQ8_0)
                                                     ? 0u
                                                     : static_cast<uint32_t>((static_cast<unsigned long long>(row) * p.row_bytes +
                                                                              static_cast<unsigned long long>(sb0) * F::kBytes) & 15ull);
                            const uint8_t* blk = stage + r * P::kSlot + off + sbl * F::kBytes;
                            uint4 qa, qb;
                            float sa, ma, sb, mb;
                            D::quants(blk, l, qa, qb);
                            D::scales(table + (r * kSbPerWarp + sbw) * 16, l, sa, ma, sb, mb);
#pragma unroll
                            for (int m = 0; m < MT; ++m) {
                                // sum q_w * (256*q1 + q2) fits 32 bits: 16 * 127 * 127 * 257 < 2^27
                                const int ia = dot16(qa, xr[m].q1a) * 256 + dot16(qa, xr[m].q2a);
                                float t = fmaf(sa * xr[m].da, static_cast<float>(ia), acc[r][m]);
                                if (Format<FMT>::kHasMin) t = fmaf(-ma, xr[m].sa, t);
                                if (FMT != kQ8_0) {
                                    const int ib = dot16(qb, xr[m].q1b) * 256 + dot16(qb, xr[m].q2b);
                                    t = fmaf(sb * xr[m].db, static_cast<float>(ib), t);
                                    if (Format<FMT>::kHasMin) t = fmaf(-mb, xr[m].sb, t);
                                }
                                acc[r][m] = t;
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            if (threadIdx.x == 0 && it < 12) wall_stamp(p, 9 + 2 * it);
        }

        if (kWK == 1) {
            // The warp holds the complete sums of its rows: lane (r * MT + m) keeps and stores output (r, m).
            float mine = 0.0f;
#pragma unroll
            for (int r = 0; r < kRW; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const float v = warp_sum(acc[r][m]);
                    if (lane == r * MT + m) mine = v;
                }
            const int r = lane / MT;
            const int m = lane % MT;
            const long long row = row_base + r;
            if (lane < kRW * MT && row < row_end && m < p.members) {
                const size_t o = static_cast<size_t>(m) * p.n + row;
                if (p.y_bf16) {
                    if (p.accumulate) mine += __bfloat162float(static_cast<const __nv_bfloat16*>(p.y)[o]);
                    static_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(mine);
                } else {
                    if (p.accumulate) mine += static_cast<const float*>(p.y)[o];
                    static_cast<float*>(p.y)[o] = mine;
                }
            }
            continue;
        }
        float* red_buf = red + (tile & 1) * (kWK * kRows * MT);
#pragma unroll
        for (int r = 0; r < kRW; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const float v = warp_sum(acc[r][m]);
                if (lane == 0) red_buf[(wk * kRows + wr * kRW + r) * MT + m] = v;
            }
        __syncwarp();
        if (lane == 0) mbar_arrive(&red_bar[tile & 1]);
        if (!mbar_wait_bounded(&red_bar[tile & 1], (tile >> 1) & 1)) {
            atomicExch(p.status, kDeviceWaitTimeout);
            return;
        }
        for (int e = threadIdx.x; e < kRows * MT; e += kConsumerThreads) {
            const int rr = e / MT;
            const int m = e % MT;
            const long long row = row_begin + static_cast<long long>(tile) * kRows + rr;
            if (row < row_end && m < p.members) {
                float v = red_buf[rr * MT + m];
#pragma unroll
                for (int q = 1; q < kWK; ++q) v += red_buf[(q * kRows + rr) * MT + m];
                const size_t o = static_cast<size_t>(m) * p.n + row;
                if (p.y_bf16) {
                    if (p.accumulate) v += __bfloat162float(static_cast<const __nv_bfloat16*>(p.y)[o]);
                    static_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(v);
                } else {
                    if (p.accumulate) v += static_cast<const float*>(p.y)[o];
                    static_cast<float*>(p.y)[o] = v;
                }
            }
        }
        if (threadIdx.x == 0 && tile < 8) wall_stamp(p, 40 + tile);
    }
    if (threadIdx.x == 0) wall_stamp(p, 4);
}

constexpr size_t kSmemLimit = 227 * 1024;

template <uint32_t FMT, int MT>
cudaError_t launch(const GemvArgs& a, bool* handled) {
    using P = Dp4aPlan<FMT, MT>;
    auto kernel = gemv_dp4a_kernel<FMT, MT>;
    const int nsb = (a.k + kSuperBlock - 1) / kSuperBlock;
    const int kpad = nsb * kSuperBlock;
    const size_t fixed = P::fixed_bytes(kpad);
    // Prefer two CTAs per SM (half the shared memory each) when at least three stages still fit.
    // Four members need ~150 registers per thread, which already limits an SM to one CTA.
    const size_t half = (kSmemLimit - 2048) / 2;
    int ctas = 2;
    size_t budget = half;
    if (MT == 4 || fixed + 3 * static_cast<size_t>(P::kStageBytes) > half) {
        ctas = 1;
        budget = kSmemLimit;
    }
    if (fixed + 2 * static_cast<size_t>(P::kStageBytes) > budget) {
        *handled = false;  // activations too large to stage in shared memory: the caller uses the f32 kernel
        return cudaSuccess;
    }
    // Tuning variants 4 and 5 (option "gemv_variant"): three or four CTAs per SM with shorter rings -- a CTA of the
    // sweep's shapes consumes only a handful of stages, so residency may matter more than ring depth.
    if (MT != 4 && (a.variant == 4 || a.variant == 5)) {
        const int want = a.variant == 4 ? 3 : 4;
        const size_t share = (kSmemLimit - 1024 * want) / want;
        if (fixed + 2 * static_cast<size_t>(P::kStageBytes) <= share) {
            ctas = want;
            budget = share;
        }
    }
    int stages = static_cast<int>((budget - fixed) / P::kStageBytes);
    if (stages > 6) stages = 6;
    const size_t smem = fixed + static_cast<size_t>(stages) * P::kStageBytes;
    static int configured_device = -1;
    int device = 0;
    cudaGetDevice(&device);
    if (configured_device != device) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemLimit));
        if (e != cudaSuccess) return e;
        configured_device = device;
    }
    Dp4aParams p;
    p.w = a.weights;
    p.w_bytes = a.weight_bytes;
    p.row_bytes = a.value_type == kQ8_0 ? static_cast<unsigned long long>(a.k / 32) * 34
                                        : static_cast<unsigned long long>(a.k / kSuperBlock) * Format<FMT>::kBytes;
    p.xq = static_cast<const uint8_t*>(a.x);
    p.pack_mode = a.pack_mode - 1;
    p.x_raw = a.x;
    p.x_raw_bf16 = a.x_bf16 ? 1 : 0;
    p.norm_weight = a.norm_weight;
    p.eps = a.eps;
    p.x_stride = packed_activation_stride(kpad);
    p.y = a.y;
    p.k = a.k;
    p.n = a.n;
    p.nsb = nsb;
    p.members = a.members;
    p.y_bf16 = a.y_bf16 ? 1 : 0;
    p.accumulate = a.accumulate ? 1 : 0;
    p.stages = stages;
    p.status = a.device_status;
    p.trace = a.trace;
    int grid = a.sm_count * ctas;
    if (grid > a.n) grid = a.n;
    *handled = true;
    return launch_kernel(kernel, dim3(grid), dim3(kThreads), smem, a.stream, p);
}

template <uint32_t FMT>
cudaError_t launch_members(const GemvArgs& a, bool* handled) {
    if (a.members == 1) return launch<FMT, 1>(a, handled);
    if (a.members == 2) return launch<FMT, 2>(a, handled);
    return launch<FMT, 4>(a, handled);
}

}  // namespace

bool gemv_dp4a_fits(uint32_t value_type, int k, int members) {
    const int kpad = (k + kSuperBlock - 1) / kSuperBlock * kSuperBlock;
    const size_t mt = members == 1 ? 1 : members == 2 ? 2 : 4;
    size_t stage = 0;
    switch (value_type) {
        case kQ4_K: stage = Dp4aPlan<kQ4_K, 1>::kStageBytes; break;
        case kQ5_K: stage = Dp4aPlan<kQ5_K, 1>::kStageBytes; break;
        case kQ6_K: stage = Dp4aPlan<kQ6_K, 1>::kStageBytes; break;
        case kQ8_0: stage = Dp4aPlan<kQ8_0, 1>::kStageBytes; break;
        default: return false;
    }
    // conservative: fixed part of the four-member plan plus two stages
    const size_t fixed = Dp4aPlan<kQ4_K, 4>::kTableBytes + Dp4aPlan<kQ4_K, 4>::kRedBytes + mt * packed_activation_stride(kpad) + 256;
    return members >= 1 && members <= 4 && fixed + 2 * stage <= kSmemLimit;
}

// `a.x` points at packed activations (quantize.cu) of a.members rows.
cudaError_t launch_gemv_dp4a(const GemvArgs& a, bool* handled) {
    *handled = false;
    if (a.members < 1 || a.members > 4) return cudaSuccess;
    switch (a.value_type) {
        case kQ4_K: return launch_members<kQ4_K>(a, handled);
        case kQ5_K: return launch_members<kQ5_K>(a, handled);
        case kQ6_K: return launch_members<kQ6_K>(a, handled);
        case kQ8_0: return launch_members<kQ8_0>(a, handled);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ribn
