// Quantized GEMV for decode batches (5..64 member rows) on the 5th-generation tensor cores:
// one f16 operand tile per K step, normalised per super-block.
//
//   Y[m][n] = sum_k dequant(W[n][k]) * X[m][k]
//
// The reference serves batches of up to eight members with its CUDA-core GEMV
// (crates/nvidia/src/quantized.rs:445-487 over q4_k.cu:161-258 and twins).  Here a batch shares one
// pass over the weights, and the tensor pipe does the multiply-adds.
//
// A tcgen05.mma of 128 rows x 16 K costs the pipe about 54 cycles however few tokens it has (measured
// for N <= 64), so the number of MMAs per weight decides the ceiling: this kernel issues one per 16 K
// elements (the dequantised-operand GEMM of qgemm_tc.cu, which splits every weight into two bf16
// parts, needs two), and it keeps the per-weight ALU work to the dequantisation itself.
//
// Operand encoding.  f16 has 11 significant bits (2^-12 relative rounding, inside the 2e-3 bound of
// the path; a bf16 tile would not be) but only five exponent bits.  Range is handled exactly:
//   * every (row, super-block) is multiplied by a power of two that brings the largest magnitude its
//     header allows (e.g. |d|*63*15 + |dmin|*63 for Q4_K) to at most 1024; the MMAs of one
//     super-block accumulate into a TMEM buffer of their own, and the accumulate warps add
//     s * D_superblock to f32 registers (s = the inverse power of two), once per 256 K elements;
//   * every activation row is multiplied by a power of two that brings its largest magnitude to at most
//     2^14 when it is converted to f16 (a pre-pass, convert_activations_f16 below, which can also
//     apply RMSNorm first); the epilogue multiplies the result by the inverse.
// Both scalings are exact, so the only roundings are the one of each weight and each activation to f16.
//
// Shape of one CTA: 128 weight rows x NT tokens (16, 32 or 64) x a range of K; 23 warps (27 for 64 tokens):
//   warp 0        raw weight bytes of one super-block x 128 rows per stage (one tiled TMA box, or
//                 per-row bulk copies for rows that are not 16-byte aligned);
//   warp 1        MMA issuer: the warp runs its loop converged and the elect.sync lane issues four tcgen05.mma per
//                 64-wide K step, one tcgen05.commit to free a group of steps, one to publish the super-block's
//                 TMEM buffer after its last step;
//   warps 2..17   dequantisation: four slots of 128 threads (one per row); slot s converts K step s of
//                 every super-block into the swizzled K-major A tile, so four steps are in flight;
//   warps 18..    accumulate: thread = weight row (TMEM lane), registers = tokens; one warp per TMEM lane quadrant,
//                 two for 64 tokens (32 accumulators per thread either way);
//   last warp     activation tiles (tiled TMA, 128-byte swizzle), one per K step.
// The ring of A/B tiles is deeper than the four slots, so dequantising step j+4 overlaps the MMAs of
// step j.  Split-K as in qgemm_tc.cu: partial tiles and an atomic ticket, the last CTA of a tile adds
// them in index order.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets the status word, and every warp
// still reaches the common teardown that frees TMEM.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "formats.cuh"
#include "internal.h"
#include "pack_activations.cuh"
#include "row_dequant.cuh"
#include "tc_host.h"
#include "tcgen05.cuh"

namespace ribn {
namespace {

constexpr int kBM = 128;                 // weight rows per CTA
constexpr int kBK = 64;                  // K elements per step (one 128-byte swizzled row of f16)
constexpr int kSub = kSuperBlock / kBK;  // steps per super-block
constexpr int kSlots = 4;                // K steps being dequantised at once
constexpr int kDequantWarps = 4 * kSlots;
constexpr int kFirstAccWarp = 2 + kDequantWarps;
// Accumulate warps: one per TMEM lane quadrant, two for 64 tokens (32 accumulators per thread either way).
constexpr int acc_warps(int nt) { return nt >= 64 ? 8 : 4; }
constexpr int activation_warp(int nt) { return kFirstAccWarp + acc_warps(nt); }
constexpr int threads(int nt) { return (activation_warp(nt) + 1) * 32; }
constexpr int kAccBuffers = 4;           // super-blocks whose products may wait in TMEM
static_assert(kSlots == kSub, "slot s owns K step s of every super-block");

// Diagnostics (see TcParams::trace), compiled in with -DRIBN_TRACE only: one stamp per (role, step, event) from CTA (0,0,0).
__device__ __forceinline__ void stamp(const TcParams& p, int role, int step, int event) {
#ifdef RIBN_TRACE
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && step < 64)
        p.trace[(role * 64 + step) * 8 + event] = clock64();
#else
    (void)p;
    (void)role;
    (void)step;
    (void)event;
#endif
}

// Wall-clock stamps (ns) of one CTA's phases: trace[(3 * 64 + 63) * 8 + event], CTA (0,0,0).
__device__ __forceinline__ void wall_stamp(const TcParams& p, int event) {
#ifdef RIBN_TRACE
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.trace[(3 * 64 + 63) * 8 + event] = static_cast<long long>(t);
    }
#else
    (void)p;
    (void)event;
#endif
}

template <uint32_t FMT, int NT, bool RAWTMA>
struct Geometry {
    using F = Format<FMT>;
    static constexpr int kBoxBytes = FMT == kQ6_K ? 240 : F::kBytes;
    static constexpr int kSlot = RAWTMA ? kBoxBytes : ((F::kBytes + 15) / 16) * 16 + 16;
    static constexpr int kRawStageBytes = kBM * kSlot;
    static constexpr int kATileBytes = kBM * kBK * 2;
    static constexpr int kBTileBytes = NT * kBK * 2;
    // The tiles form two groups of consecutive K steps.  A group is handed to the MMA issuer, and handed
    // back, as a whole: one wait, 4 MMAs per step back to back, one commit -- a wait or a commit costs the
    // issuing thread as much as several MMAs.  While the tensor pipe reads one group the slots fill the other.
    static constexpr int kGroupSteps = (NT >= 64 || FMT == kQ8_0) ? 3 : 4;   // as many as shared memory holds
    static constexpr int kGroups = 2;
    static constexpr int kStages = kGroups * kGroupSteps;
    static constexpr int kTilesBytes = kStages * (kATileBytes + kBTileBytes);
    static constexpr int kScaleBytes = kAccBuffers * kBM * 4;   // s per (buffer, row)
    static constexpr int kBarrierBytes = 512;
    static constexpr int kFixedBytes = 1024 + kTilesBytes + kScaleBytes + kBarrierBytes;   // 1024: alignment slack
    static constexpr int kRawFit = (227 * 1024 - kFixedBytes) / kRawStageBytes;
    static constexpr int kRawStages = kRawFit > 6 ? 6 : kRawFit;
    static constexpr int kRawBytes = kRawStages * kRawStageBytes;
    static constexpr int kSmemBytes = kFixedBytes + kRawBytes;
    static constexpr int kTmemColumns = kAccBuffers * NT < 32 ? 32 : kAccBuffers * NT;
    static_assert(kRawStages >= 2, "tile plan exceeds shared memory");
    static_assert(kStages >= kSlots, "a waiter may be at most one barrier phase behind");
    static constexpr int kGroupArrivals = kGroupSteps * (4 + 1);   // per step: the slot's four warps + the activation tile
    static_assert((kTmemColumns & (kTmemColumns - 1)) == 0 && kTmemColumns <= 512, "TMEM columns: a power of two <= 512");
    static_assert((2 * kRawStages + 2 * kGroups + 2 * kAccBuffers) * 8 + 16 <= kBarrierBytes, "barrier block too small");
};

// s = 2^e with bound * 2^-e in (512, 1024]; inverse = 2^-e.  A zero bound (all-zero block) gives 0, 0.
__device__ __forceinline__ void normaliser(float bound, float& inverse, float& s) {
    const uint32_t bits = __float_as_uint(bound);
    const int exponent = static_cast<int>(bits >> 23) - 127;    // bound in [2^exponent, 2^(exponent+1))
    int e = exponent + 1 - 10;                                   // bound * 2^-e < 1024
    e = max(-100, min(100, e));
    const bool usable = bound > 0.0f && bound < 3.0e38f;
    inverse = usable ? __uint_as_float(static_cast<uint32_t>(127 - e) << 23) : 0.0f;
    s = usable ? __uint_as_float(static_cast<uint32_t>(127 + e) << 23) : 0.0f;
}

template <uint32_t FMT, int NT, bool RAWTMA>
__global__ void __launch_bounds__(threads(NT), 1)
qgemv_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const TcParams p) {
    using G = Geometry<FMT, NT, RAWTMA>;
    using F = Format<FMT>;
    using R = RowDequant<FMT, SingleF16>;
    constexpr int kAccWarps = acc_warps(NT);
    constexpr int kActivationWarp = activation_warp(NT);
    constexpr int kAccColumns = NT / (kAccWarps / 4);   // tokens per accumulate thread
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    uint8_t* a_tiles = smem;
    uint8_t* b_tiles = a_tiles + G::kStages * G::kATileBytes;
    float* scale_ring = reinterpret_cast<float*>(b_tiles + G::kStages * G::kBTileBytes);   // [buffer][row]
    uint8_t* raw = reinterpret_cast<uint8_t*>(scale_ring) + G::kScaleBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(raw + G::kRawBytes);
    uint64_t* raw_full = bars;                        // [kRawStages]  TMA bytes (or 32 producer lanes)
    uint64_t* raw_empty = raw_full + G::kRawStages;   // [kRawStages]  16 dequant warps
    uint64_t* g_full = raw_empty + G::kRawStages;     // [kGroups]     per step of the group: the slot's 4 warps + the activation tile
    uint64_t* g_empty = g_full + G::kGroups;          // [kGroups]     tcgen05.commit
    uint64_t* d_full = g_empty + G::kGroups;          // [kAccBuffers] tcgen05.commit after a super-block's last MMA
    uint64_t* d_empty = d_full + kAccBuffers;         // [kAccBuffers] 4 accumulate warps
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(d_empty + kAccBuffers);
    uint32_t* last_flag = tmem_holder + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kBM;
    const int m0 = blockIdx.y * NT;
    const int sb_begin = static_cast<int>(static_cast<long long>(p.nsb) * blockIdx.z / p.ksplit);
    const int sb_end = static_cast<int>(static_cast<long long>(p.nsb) * (blockIdx.z + 1) / p.ksplit);
    const int nsb_local = sb_end - sb_begin;
    const int steps = nsb_local * kSub;
    pdl_launch_dependents();
    if (threadIdx.x == 0) wall_stamp(p, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < G::kRawStages; ++s) {
            mbar_init(&raw_full[s], RAWTMA ? 1 : 32);
            mbar_init(&raw_empty[s], kDequantWarps);
        }
        for (int s = 0; s < G::kGroups; ++s) {
            mbar_init(&g_full[s], G::kGroupArrivals);
            mbar_init(&g_empty[s], 1);
        }
        for (int s = 0; s < kAccBuffers; ++s) {
            mbar_init(&d_full[s], 1);
            mbar_init(&d_empty[s], kAccWarps);
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
    if (threadIdx.x == 0) wall_stamp(p, 1);

    if (warp == 0) {
        // ---------------- raw weight bytes ----------------
        const unsigned long long safe_end = p.w_bytes & ~15ull;
        for (int i = 0; i < nsb_local; ++i) {
            const int rs = i % G::kRawStages;
            if (i >= G::kRawStages && !mbar_wait_bounded(&raw_empty[rs], ((i / G::kRawStages) - 1) & 1)) {
                atomicExch(p.status, kDeviceWaitTimeout);
                break;
            }
            if (lane == 0) stamp(p, 3, i, 0);
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
        }
    } else if (warp == kActivationWarp) {
        // ---------------- activation tiles ----------------
        // The f16 activations come from the pre-pass, the kernel before this one in the stream; the raw weight
        // stream and the dequantisation run ahead of this wait.
        pdl_wait_prior();
        if (lane == 0) wall_stamp(p, 2);
        if (lane == 0) {
            for (int j = 0; j < steps; ++j) {
                const int as = j % G::kStages;
                const int g = as / G::kGroupSteps;
                if (j >= G::kStages && !mbar_wait_bounded(&g_empty[g], ((j / G::kStages) - 1) & 1)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    break;
                }
                mbar_arrive_expect_tx(&g_full[g], G::kBTileBytes);
                tma_load_2d(b_tiles + as * G::kBTileBytes, &xmap, sb_begin * kSuperBlock + j * kBK, m0, &g_full[g]);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer: the whole warp runs this loop converged, an elected lane issues ----------------
        constexpr uint32_t idesc = umma_instr_desc(kBM, NT, /*A f16*/ 0, /*B f16*/ 0);
        const uint64_t desc_a0 = umma_smem_desc_sw128(smem_addr(a_tiles));
        const uint64_t desc_b0 = umma_smem_desc_sw128(smem_addr(b_tiles));
        const int groups = (steps + G::kGroupSteps - 1) / G::kGroupSteps;
        const int missing = groups * G::kGroupSteps - steps;
        bool ok = true;
        for (int gi = 0; gi < groups && ok; ++gi) {
            const int g = gi % G::kGroups;
            if (gi == groups - 1 && lane == 0) {
                // The last group may be short: the issuer stands in for the arrivals of the steps it lacks
                // (now, when the barrier's earlier phases are over).
                for (int u = 0; u < missing * (4 + 1); ++u) mbar_arrive(&g_full[g]);
            }
            __syncwarp();
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(&g_full[g], (gi / G::kGroups) & 1));
            if (!ok) break;
            if (lane == 0) stamp(p, 0, gi, 0);
            if (lane == 0 && gi == 0) wall_stamp(p, 3);
            if (lane == 0 && gi == groups - 1) wall_stamp(p, 4);
            __syncwarp();
            tcgen05_fence_after_sync();
#pragma unroll
            for (int u = 0; u < G::kGroupSteps; ++u) {
                const int j = gi * G::kGroupSteps + u;
                if (j >= steps) break;
                const int i = j / kSub;
                const int t = j % kSub;
                const int buf = i % kAccBuffers;
                if (t == 0 && i >= kAccBuffers) {
                    ok = __all_sync(0xffffffffu, mbar_wait_bounded(&d_empty[buf], ((i / kAccBuffers) - 1) & 1));
                    if (!ok) break;
                    tcgen05_fence_after_sync();
                }
                const int as = g * G::kGroupSteps + u;
                umma_f16_step4_elected(tmem_base + buf * NT, desc_a0 + static_cast<uint64_t>(as * (G::kATileBytes >> 4)),
                                       desc_b0 + static_cast<uint64_t>(as * (G::kBTileBytes >> 4)), idesc, t > 0 ? 1u : 0u);
                if (t == kSub - 1) umma_commit_elected(&d_full[buf]);
            }
            if (!ok) break;
            umma_commit_elected(&g_empty[g]);
            if (lane == 0) stamp(p, 0, gi, 1);
            __syncwarp();
        }
        if (!ok && lane == 0) atomicExch(p.status, kDeviceWaitTimeout);
        __syncwarp();
    } else if (warp < kFirstAccWarp) {
        // ---------------- dequantisation: raw bytes -> f16 A tiles ----------------
        const int worker = threadIdx.x - 64;
        const int r = worker & (kBM - 1);
        const int slot = worker >> 7;
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
            if (r == 0 && slot == 0) stamp(p, 3, i, 1);
            // With the TMA box rows are 16-byte aligned, so only the block's offset inside its row counts.
            const unsigned long long g0 = (RAWTMA ? 0ull : static_cast<unsigned long long>(row) * p.row_bytes) +
                                          static_cast<unsigned long long>(sb_begin + i) * F::kBytes;
            const uint8_t* blk = raw + rs * G::kRawStageBytes + r * G::kSlot + static_cast<uint32_t>(g0 & 15ull);
            float inverse = 0.0f, s = 0.0f;
            // The slot's K step is a run-time index: one copy of the dequantiser serves the four slots (four unrolled
            // copies measured slower: the kernel stalls on instruction fetch), and only the step's own scales are decoded.
            typename R::StepScales scales;
            if (row_ok) {
                normaliser(R::magnitude_bound(blk), inverse, s);
                R::load_step_scales(blk, slot, inverse, scales);
            }
            const int j = i * kSub + slot;
            const int as = j % G::kStages;
            const int g = as / G::kGroupSteps;
            if (j >= G::kStages && !mbar_wait_bounded(&g_empty[g], ((j / G::kStages) - 1) & 1)) {
                atomicExch(p.status, kDeviceWaitTimeout);
                ok = false;
                break;
            }
            if (r == 0) stamp(p, 1, j, 0);
            uint8_t* tile = a_tiles + as * G::kATileBytes + row_off;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                typename R::Chunk out[4];
                if (row_ok) {
                    R::step(blk, scales, slot, h, out);
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c) out[c] = SingleF16::zero();
                }
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    *reinterpret_cast<uint4*>(tile + ((static_cast<uint32_t>(R::chunk_index(h, c)) ^ sw) << 4)) = out[c].high;
            }
            if (r == 0) stamp(p, 1, j, 1);
            if (slot == 0) {
                // The super-block's factor for the accumulate warps.  Entry i % 4 was last read for super-block
                // i - 4; waiting for that TMEM buffer's release covers the entry too.
                const int buf = i % kAccBuffers;
                if (i >= kAccBuffers && !mbar_wait_bounded(&d_empty[buf], ((i / kAccBuffers) - 1) & 1)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    ok = false;
                    break;
                }
                scale_ring[buf * kBM + r] = s;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&g_full[g]);
                mbar_arrive(&raw_empty[rs]);
            }
            if (r == 0) stamp(p, 1, j, 2);
            ok = __all_sync(0xffffffffu, ok);
        }
    }

    // ---------------- accumulate warps: acc[m] += s * D_superblock[m]; then the epilogue ----------------
    if (warp >= kFirstAccWarp && warp < kActivationWarp) {
        const int q = warp & 3;                 // a warp may only read TMEM lanes 32*(warp%4) .. +31
        const int half = (warp - kFirstAccWarp) >> 2;   // which kAccColumns tokens of the tile
        const int rrow = q * 32 + lane;
        const int col0 = half * kAccColumns;
        float acc[kAccColumns];
#pragma unroll
        for (int m = 0; m < kAccColumns; ++m) acc[m] = 0.0f;
        bool ok = true;
        for (int i = 0; i < nsb_local && ok; ++i) {
            const int buf = i % kAccBuffers;
            if (!mbar_wait_bounded(&d_full[buf], (i / kAccBuffers) & 1)) {
                atomicExch(p.status, kDeviceWaitTimeout);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (rrow == 0 && half == 0) stamp(p, 2, i, 0);
            tcgen05_fence_after_sync();
            const float s = scale_ring[buf * kBM + rrow];
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * NT + col0;
            uint32_t v0[16], v1[16];
            tmem_ld16(taddr, v0);
            if (kAccColumns > 16) tmem_ld16(taddr + 16, v1);
            tmem_ld_wait();
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) acc[jj] = fmaf(s, __uint_as_float(v0[jj]), acc[jj]);
            if (kAccColumns > 16) {
#pragma unroll
                for (int jj = 0; jj < 16; ++jj) acc[16 + jj] = fmaf(s, __uint_as_float(v1[jj]), acc[16 + jj]);
            }
            tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&d_empty[buf]);
            if (rrow == 0 && half == 0) stamp(p, 2, i, 1);
        }
        if (rrow == 0 && half == 0) wall_stamp(p, 5);
        pdl_wait_prior();   // the per-row factors are the pre-pass's too (long done by now: the MMAs needed its tiles)
        // The scaled tile goes through shared memory (the A tiles are free by now: every MMA has completed), so
        // that all worker warps can store it: one thread per row storing its tokens one after the other
        // took several microseconds.  Lane l fetches the factor of token col0 + l.
        const float factor_lane = (lane < kAccColumns && m0 + col0 + lane < p.m) ? __ldg(p.x_scale + m0 + col0 + lane) : 0.0f;
        float* tile = reinterpret_cast<float*>(a_tiles);   // [NT][kBM]
#pragma unroll
        for (int jj = 0; jj < kAccColumns; ++jj) {
            const float factor = __shfl_sync(0xffffffffu, factor_lane, jj);
            tile[(col0 + jj) * kBM + rrow] = ok ? acc[jj] * factor : 0.0f;
        }
    }
    if (warp >= 2 && warp < kActivationWarp) {
        constexpr int kWriters = (kDequantWarps + kAccWarps) * 32;
        named_barrier_sync(3, kWriters);
        const float* tile = reinterpret_cast<const float*>(a_tiles);
        const bool split = p.ksplit > 1;
        float* part = split ? p.partial + static_cast<size_t>(blockIdx.z) * p.m * p.n : nullptr;
        for (int idx = threadIdx.x - 64; idx < NT * kBM; idx += kWriters) {
            const int m = m0 + (idx >> 7);
            const long long row = static_cast<long long>(n0) + (idx & (kBM - 1));
            if (m < p.m && row < p.n) {
                const float value = tile[idx];
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
    }

    // ---------------- split-K: the CTA that draws the last ticket of its tile adds the partial tiles ----------------
    if (p.ksplit > 1 && warp >= 2 && warp < kActivationWarp) {
        // Dequant and accumulate warps take part (all idle by now): five threads per weight row.
        constexpr int kReducers = (kDequantWarps + kAccWarps) * 32;
        __threadfence();
        named_barrier_sync(2, kReducers);
        if (threadIdx.x == 64) {
            unsigned int* ticket = p.tickets + blockIdx.y * gridDim.x + blockIdx.x;
            const unsigned int drawn = atomicAdd(ticket, 1u);
            const bool last = drawn == static_cast<unsigned int>(p.ksplit - 1);
            if (last) *ticket = 0;  // ready for the next launch
            *last_flag = last ? 1u : 0u;
        }
        named_barrier_sync(2, kReducers);
        const int worker = threadIdx.x - 64;
        const long long row = static_cast<long long>(n0) + (worker & (kBM - 1));
        if (*last_flag != 0 && row < p.n) {
            __threadfence();
            const size_t plane = static_cast<size_t>(p.m) * p.n;
            const int m_end = min(m0 + NT, p.m);
            // Four tokens at a time, so that four independent loads per K slice are in flight;
            // the slices are added in index order whatever the arrival order was.
            for (int m = m0 + 4 * (worker >> 7); m < m_end; m += 4 * (kReducers / kBM)) {
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
                            if (p.accumulate) sum[u] += __bfloat162float(static_cast<const __nv_bfloat16*>(p.y)[o[u]]);
                            static_cast<__nv_bfloat16*>(p.y)[o[u]] = __float2bfloat16_rn(sum[u]);
                        } else {
                            if (p.accumulate) sum[u] += static_cast<const float*>(p.y)[o[u]];
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
    if (threadIdx.x == 0) wall_stamp(p, 6);
    if (warp == 1) tmem_dealloc(tmem_base, G::kTmemColumns);
}

// ---------------- activation pre-pass: x (f32 or bf16) -> f16 rows with a power-of-two factor per row ----------------
// One CTA per member row.  With norm_weight the row is RMS-normalised first (model_ops.cu rms_norm:
// y = x * rsqrt(mean(x^2) + eps) * weight, f32 arithmetic).  The row is then multiplied by 2^-e, e chosen so
// that its largest magnitude lands in (2^13, 2^14], and rounded to f16; factor[m] = 2^e.
constexpr int kConvertThreads = 512;

// Eight consecutive elements of member row `member` starting at i; with swiglu the row is [gate | up] (2k values)
// and the elements are silu(gate) * up (silu_mul of the reference, model_ops.rs:316-328).
__device__ __forceinline__ void load_activation8(const void* x, int bf16, int swiglu, size_t member, int k, int i, float (&v)[8]) {
    const AnyRow row{static_cast<const uint8_t*>(x) + member * static_cast<size_t>(k) * (swiglu ? 2 : 1) * (bf16 ? 2 : 4), bf16};
    load_row8(row + i, v);
    if (swiglu != 0) {
        float u[8];
        load_row8(row + (k + i), u);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (v[j] / (1.0f + expf(-v[j]))) * u[j];
    }
}

__global__ void __launch_bounds__(kConvertThreads)
convert_activations_f16(const void* x, int x_bf16, int swiglu, const float* norm_weight, float eps, __half* out, float* factor, int k) {
    pdl_launch_dependents();
    pdl_wait_prior();   // x may be the previous kernel's output; `out` may still be read by it
    __shared__ float red_sum[kConvertThreads / 32];
    __shared__ float red_max[kConvertThreads / 32];
    __shared__ float broadcast[2];
    const size_t base = static_cast<size_t>(blockIdx.x) * k;
    float sum = 0.0f, biggest = 0.0f;
    // k is a multiple of 256 on this path: chunks of eight elements, 16- or 32-byte loads.
    for (int i = threadIdx.x * 8; i < k; i += kConvertThreads * 8) {
        float v[8];
        load_activation8(x, x_bf16, swiglu, blockIdx.x, k, i, v);
        float g[8];
        if (norm_weight != nullptr) load_x8<float>(norm_weight + i, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            sum = fmaf(v[j], v[j], sum);
            biggest = fmaxf(biggest, fabsf(norm_weight != nullptr ? v[j] * g[j] : v[j]));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
        biggest = fmaxf(biggest, __shfl_xor_sync(0xffffffffu, biggest, o));
    }
    if ((threadIdx.x & 31) == 0) {
        red_sum[threadIdx.x >> 5] = sum;
        red_max[threadIdx.x >> 5] = biggest;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        sum = threadIdx.x < kConvertThreads / 32 ? red_sum[threadIdx.x] : 0.0f;
        biggest = threadIdx.x < kConvertThreads / 32 ? red_max[threadIdx.x] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
            biggest = fmaxf(biggest, __shfl_xor_sync(0xffffffffu, biggest, o));
        }
        if (threadIdx.x == 0) {
            const float inv_rms = norm_weight != nullptr ? rsqrtf(sum / static_cast<float>(k) + eps) : 1.0f;
            broadcast[0] = inv_rms;
            broadcast[1] = biggest * inv_rms;
        }
    }
    __syncthreads();
    const float inv_rms = broadcast[0];
    const float amax = broadcast[1];
    float down = 1.0f, up = 1.0f;   // 2^-e, 2^e
    if (amax > 0.0f && amax < 3.0e38f) {
        int e = static_cast<int>(__float_as_uint(amax) >> 23) - 127 + 1 - 14;   // amax * 2^-e in [2^13, 2^14)
        e = max(-100, min(100, e));
        down = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
        up = __uint_as_float(static_cast<uint32_t>(127 + e) << 23);
    }
    if (threadIdx.x == 0) factor[blockIdx.x] = up;
    for (int i = threadIdx.x * 8; i < k; i += kConvertThreads * 8) {
        float v[8];
        load_activation8(x, x_bf16, swiglu, blockIdx.x, k, i, v);
        if (norm_weight != nullptr) {
            float g[8];
            load_x8<float>(norm_weight + i, g);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = v[j] * inv_rms * g[j];
        }
        uint4 packed;
        __half2 h;
        h = __floats2half2_rn(v[0] * down, v[1] * down); packed.x = *reinterpret_cast<const uint32_t*>(&h);
        h = __floats2half2_rn(v[2] * down, v[3] * down); packed.y = *reinterpret_cast<const uint32_t*>(&h);
        h = __floats2half2_rn(v[4] * down, v[5] * down); packed.z = *reinterpret_cast<const uint32_t*>(&h);
        h = __floats2half2_rn(v[6] * down, v[7] * down); packed.w = *reinterpret_cast<const uint32_t*>(&h);
        *reinterpret_cast<uint4*>(out + base + i) = packed;
    }
}

template <uint32_t FMT, int NT, bool RAWTMA>
cudaError_t launch_tile(const TcArgs& a) {
    using G = Geometry<FMT, NT, RAWTMA>;
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

    // Scratch: [f16 activations][one factor per member row][split-K partial tiles].
    const size_t x16_bytes = (static_cast<size_t>(a.m) * a.k * sizeof(__half) + 1023) & ~static_cast<size_t>(1023);
    const size_t factor_bytes = (static_cast<size_t>(a.m) * sizeof(float) + 255) & ~static_cast<size_t>(255);
    if (x16_bytes + factor_bytes > a.scratch_bytes) return cudaErrorMemoryAllocation;
    __half* x16 = static_cast<__half*>(a.scratch);
    float* factor = reinterpret_cast<float*>(static_cast<uint8_t*>(a.scratch) + x16_bytes);
    float* partial = reinterpret_cast<float*>(static_cast<uint8_t*>(a.scratch) + x16_bytes + factor_bytes);
    const size_t partial_bytes = a.scratch_bytes - x16_bytes - factor_bytes;

    static int prepass_device = -1;
    if (prepass_device != device) {
        // Same shared-memory carve-out as the main kernel, so that the two can follow each other on an SM
        // without a reconfiguration in between.
        cudaFuncSetAttribute(convert_activations_f16, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        prepass_device = device;
    }
    if (!a.skip_prepass) {
        cudaError_t launched = launch_kernel(convert_activations_f16, dim3(a.m), dim3(kConvertThreads), 0, a.stream, a.x, a.x_bf16 ? 1 : 0,
                                             a.swiglu ? 1 : 0, a.norm_weight, a.eps, x16, factor, a.k);
        if (launched != cudaSuccess) return launched;
    }

    CUtensorMap map;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.k), static_cast<cuuint64_t>(a.m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.k) * 2};
    const cuuint32_t box[2] = {kBK, NT};
    const cuuint32_t elem[2] = {1, 1};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x16, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
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
    p.partial = partial;
    p.x_scale = factor;
    p.tickets = a.tickets;
    p.k = a.k;
    p.n = a.n;
    p.m = a.m;
    p.nsb = a.k / kSuperBlock;
    p.y_bf16 = a.y_bf16 ? 1 : 0;
    p.accumulate = a.accumulate ? 1 : 0;
    p.status = a.device_status;
    p.trace = a.trace;
    const int n_tiles = (a.n + kBM - 1) / kBM;
    const int m_tiles = (a.m + NT - 1) / NT;
    const size_t plane_bytes = static_cast<size_t>(a.m) * a.n * sizeof(float);
    p.ksplit = choose_ksplit_decode(n_tiles * m_tiles, p.nsb, a.sm_count, plane_bytes, partial_bytes, a.ticket_count, NT);
    if (a.force_ksplit > 0 && a.force_ksplit <= p.nsb && plane_bytes * a.force_ksplit <= partial_bytes && n_tiles * m_tiles <= a.ticket_count)
        p.ksplit = a.force_ksplit;
    const dim3 grid(n_tiles, m_tiles, p.ksplit);
    return launch_kernel(kernel, grid, dim3(threads(NT)), G::kSmemBytes, a.stream, map, wmap, p);
}

template <uint32_t FMT, bool RAWTMA>
cudaError_t launch_tokens(const TcArgs& a) {
    if (a.m <= 16) return launch_tile<FMT, 16, RAWTMA>(a);
    if (a.m <= 32) return launch_tile<FMT, 32, RAWTMA>(a);
    return launch_tile<FMT, 64, RAWTMA>(a);
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

cudaError_t launch_convert_activations_f16(const void* x, bool x_bf16, bool swiglu, const float* norm_weight, float eps, void* x16, float* factor,
                                           int m, int k, cudaStream_t stream) {
    return launch_kernel(convert_activations_f16, dim3(m), dim3(kConvertThreads), 0, stream, x, x_bf16 ? 1 : 0, swiglu ? 1 : 0, norm_weight, eps,
                         static_cast<__half*>(x16), factor, k);
}

cudaError_t launch_qgemv_tc(const TcArgs& a) {
    if (a.m < 1 || a.m > 64) return cudaErrorInvalidValue;
    switch (a.value_type) {
        case kQ4_K: return launch_format<kQ4_K>(a);
        case kQ5_K: return launch_format<kQ5_K>(a);
        case kQ6_K: return launch_format<kQ6_K>(a);
        case kQ8_0: return launch_format<kQ8_0>(a);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ribn
