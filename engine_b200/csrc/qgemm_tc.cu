// Quantized GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) with the
// dequantisation fused into the operand producer.
//
//   Y[m][n] = sum_k dequant(W[n][k]) * X[m][k]      X bf16 (or f32) [M][K], f32 accumulate
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
//   A = 128 x 64 dequantised weights as one f16 tile, K-major, 128-byte
//       swizzle, written to shared memory by sixteen dequant warps from the raw
//       GGUF bytes that a producer warp streams in as tiled TMA boxes (bulk
//       copies per row where rows are not 16-byte aligned), completion on
//       mbarriers;
//   B = NT x 64 activations as f16: a conversion pre-pass multiplies every token
//       row by a power of two (largest magnitude at most 2^14) and the epilogue
//       by its inverse; one tiled TMA load per step brings the tile in the same
//       swizzled layout (rows past M read as zero);
//   D (TMEM, f32) += A * B  with four tcgen05.mma (K = 16 each) issued by one
//       thread; tcgen05.commit releases the stage.
// The epilogue reads D with tcgen05.ld (thread = weight row, registers =
// tokens) and stores Y.  With split-K the partial tiles go to a scratch buffer
// and the last CTA of a tile (an atomic ticket, no spinning) adds them in a
// fixed order, so results are deterministic.
//
// Precision: a single bf16 rounding of the weights (2^-9 relative) does not
// meet the 2e-3 bound of the path over millions of outputs; an f16 rounding
// (2^-12 relative, what the decode batch kernels apply) does, with one MMA per
// K step where a split of every weight into two bf16 parts needed two.  Both
// operands of kind::f16 must have the same format (an f16 A operand with a
// bf16 B operand is an illegal instruction), hence the f16 copy of the
// activations; bf16 activations convert exactly.  Weights beyond the f16 range
// (|w| > 65504: super-block scales no checkpoint has) come out as infinities.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets the status
// word, and every warp still reaches the common teardown that frees TMEM.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "formats.cuh"
#include "internal.h"
#include "row_dequant.cuh"
#include "tc_host.h"
#include "tcgen05.cuh"

namespace ribn {
namespace {

constexpr int kBM = 128;            // weight rows per CTA
constexpr int kBK = 64;             // K elements per UMMA stage (one 128-byte swizzled row)
constexpr int kSub = kSuperBlock / kBK;  // stages per super-block
constexpr int kSlots = 4;            // K steps being dequantised at once: slot s fills tile s of the ring
constexpr int kDequantWarps = 4 * kSlots;   // one thread per (weight row, slot)
constexpr int kSecondIssuerWarp = 2 + kDequantWarps;
constexpr int kActivationWarp = 3 + kDequantWarps;
constexpr int kTcThreads = (4 + kDequantWarps) * 32;


// RAWTMA: the raw weight bytes of a stage (128 rows x one super-block) arrive as ONE tiled TMA box
// instead of 128 bulk copies of 144..272 bytes (small bulk copies cost about as much per request
// as large ones, and 128 of them per 18 KB starve the pipeline).  The box is 2-D over the tensor
// viewed as [N rows][row_bytes] of 16-bit elements; it needs row_bytes to be a multiple of 16.
// Q6_K super-blocks (210 bytes) start on 2-byte boundaries: the box starts at the 16-byte
// boundary below and is 240 bytes wide, and the remainder is an offset in shared memory.
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

// TT = token tiles per CTA: with two, a dequantised weight tile is multiplied with 2 x NT tokens (issuer t owns token tile
// t and its accumulator), which halves the dequantisation per output.
template <uint32_t FMT, int NT, bool RAWTMA, int TT>
struct TcGeometry {
    using F = Format<FMT>;
    static constexpr int kBoxBytes = FMT == kQ6_K ? 240 : F::kBytes;
    // Four stages keep all four slots busy; the widest tiles leave room for three, two token tiles for two (the slots
    // then share a stage: two halves of the K step each).
    static constexpr int kAbStages = TT == 2 ? 2 : NT >= 256 ? 3 : 4;
    // bytes per row in a raw stage: the TMA box width, or a bulk copy from the 16-byte boundary below the block
    static constexpr int kSlot = RAWTMA ? kBoxBytes : ((F::kBytes + 15) / 16) * 16 + 16;
    static constexpr int kRawStageBytes = kBM * kSlot;
    static constexpr int kATileBytes = kBM * kBK * 2;        // one f16 tile
    static constexpr int kBTileBytes = NT * kBK * 2;         // one token tile
    static constexpr int kBStageBytes = TT * kBTileBytes;
    static constexpr int kTilesBytes = kAbStages * (kATileBytes + kBStageBytes);
    static constexpr int kBarrierBytes = 256;
    // Raw stages fill what is left of shared memory, between two and six.
    static constexpr int kRawFit = (227 * 1024 - 1024 - kTilesBytes - kBarrierBytes) / kRawStageBytes;
    static constexpr int kRawStages = kRawFit > 6 ? 6 : kRawFit;
    static_assert(kRawStages >= 2, "tile plan exceeds shared memory");
    static_assert(kAbStages <= kSlots, "every tile of the ring needs a slot");
    static constexpr int kRawBytes = kRawStages * kRawStageBytes;
    static constexpr int kSmemBytes = 1024 + kTilesBytes + kRawBytes + kBarrierBytes;  // 1024: alignment slack
    // Two accumulators.  One token tile: the K steps of the ring's even tiles are issued by one thread into the first,
    // those of its odd tiles by another into the second (an issue costs its thread far longer than the tensor pipe needs for so few
    // tokens); the epilogue adds them.
    static constexpr int kTmemColumns = 2 * NT < 32 ? 32 : 2 * NT;
    static_assert(kSmemBytes <= 227 * 1024, "tile plan exceeds shared memory");
};

template <uint32_t FMT, int NT, bool RAWTMA, int TT>
__global__ void __launch_bounds__(kTcThreads, 1)
qgemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const TcParams p) {
    using G = TcGeometry<FMT, NT, RAWTMA, TT>;
    using F = Format<FMT>;
    using R = RowDequant<FMT, SingleF16>;
    extern __shared__ uint8_t smem_raw[];
    // The swizzled tiles need a 1024-byte aligned base.
    uint8_t* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    uint8_t* a_tiles = smem;
    uint8_t* b_tiles = a_tiles + G::kAbStages * G::kATileBytes;
    uint8_t* raw = b_tiles + G::kAbStages * G::kBStageBytes;
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
    const int m0 = blockIdx.y * (TT * NT);
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
            mbar_init(&ab_full[s], (TT == 2 ? 8 : 4) + 1);   // the warps of the step's slot (two slots) + the activation tiles
            mbar_init(&ab_empty[s], TT);                      // tcgen05.commit of every issuer that reads the stage
        }
        mbar_init(acc_full, 2);
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
        // ---------------- activation tiles (TMA), one per K step; a warp of its own so that waiting for a
        // free tile never delays the raw weight stream ----------------
        if (lane == 0) {
            for (int j = 0; j < steps; ++j) {
                const int as = j % G::kAbStages;
                if (j >= G::kAbStages && !mbar_wait_bounded(&ab_empty[as], ((j / G::kAbStages) - 1) & 1)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    break;
                }
                mbar_arrive_expect_tx(&ab_full[as], G::kBStageBytes);
#pragma unroll
                for (int tt = 0; tt < TT; ++tt)   // a token tile past the last token reads as zeros
                    tma_load_2d(b_tiles + as * G::kBStageBytes + tt * G::kBTileBytes, &xmap, sb_begin * kSuperBlock + j * kBK, m0 + tt * NT,
                                &ab_full[as]);
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == kSecondIssuerWarp) {
        // ---------------- MMA issuers: one thread for the even tiles of the ring, one for the odd ones ----------------
        // (a tile always belongs to the same issuer, so that its waits on the tile's barrier follow one another phase by
        // phase, which the one-bit parity needs whether the ring has three tiles or four)
        if (lane == 0) {
            constexpr uint32_t idesc = umma_instr_desc(kBM, NT, /*A f16*/ 0, /*B f16*/ 0);
            const int first = warp == 1 ? 0 : 1;
            const uint32_t acc = tmem_base + first * NT;
            for (int j = TT == 2 ? 0 : first; j < steps; ++j) {
                const int as = j % G::kAbStages;
                if (TT == 1 && (as & 1) != first) continue;   // two token tiles: every step, this issuer's token tile
                if (!mbar_wait_bounded(&ab_full[as], (j / G::kAbStages) & 1)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    break;
                }
                stamp(p, 0, j, 0);
                tcgen05_fence_after_sync();
                const uint64_t desc_a = umma_smem_desc_sw128(smem_addr(a_tiles + as * G::kATileBytes));
                const uint64_t desc_b = umma_smem_desc_sw128(smem_addr(b_tiles + as * G::kBStageBytes + (TT == 2 ? first * G::kBTileBytes : 0)));
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk) {
                    // 16 K elements = 32 bytes further along the swizzled row: +2 in the address field
                    umma_f16(acc, desc_a + 2 * kk, desc_b + 2 * kk, idesc, j > (TT == 2 ? 0 : first) || kk > 0);
                }
                umma_commit(&ab_empty[as]);
                stamp(p, 0, j, 1);
            }
            umma_commit(acc_full);
        }
        __syncwarp();
    } else {
        // ---------------- dequant warps: raw bytes -> f16 A tiles ----------------
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
            // With the TMA box rows are 16-byte aligned, so only the block's offset inside its row counts.
            const unsigned long long g0 = (RAWTMA ? 0ull : static_cast<unsigned long long>(row) * p.row_bytes) +
                                          static_cast<unsigned long long>(sb_begin + i) * F::kBytes;
            const uint8_t* blk = raw + rs * G::kRawStageBytes + r * G::kSlot + static_cast<uint32_t>(g0 & 15ull);
            if (r == 0 && slot == 0) stamp(p, 3, i, 1);
            typename R::Scales scales;
            if (row_ok) R::load_scales(blk, scales, 1.0f);
#pragma unroll
            for (int t = 0; t < kSub; ++t) {
                // A slot owns one tile of the ring (slots beyond the ring idle): its waits on that tile's
                // barriers then follow one another phase by phase, which the one-bit parity needs.
                const int j = i * kSub + t;
                const int as = j % G::kAbStages;
                if (as != (TT == 2 ? (slot & 1) : slot)) continue;
                if (j >= G::kAbStages && !mbar_wait_bounded(&ab_empty[as], ((j / G::kAbStages) - 1) & 1)) {
                    atomicExch(p.status, kDeviceWaitTimeout);
                    ok = false;
                    break;
                }
                if (r == 0) stamp(p, 1, j, 0);
                uint8_t* tile = a_tiles + as * G::kATileBytes + row_off;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (TT == 2 && h != (slot >> 1)) continue;   // two slots share the stage: one half of the K step each
                    typename R::Chunk out[4];
                    if (row_ok) {
                        R::step(blk, scales, t, h, out);
                    } else {
#pragma unroll
                        for (int c = 0; c < 4; ++c) out[c] = SingleF16::zero();
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint32_t chunk_off = (static_cast<uint32_t>(R::chunk_index(h, c)) ^ sw) << 4;
                        *reinterpret_cast<uint4*>(tile + chunk_off) = out[c].high;
                    }
                }
                if (r == 0) stamp(p, 1, j, 1);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ab_full[as]);
                if (r == 0) stamp(p, 1, j, 2);
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
            // One token tile: the two accumulators hold the even and the odd share of the K steps and are added.  Two token
            // tiles: accumulator t holds token tile t, columns c0 run over both.
#pragma unroll 1
            for (int c0 = 0; c0 < TT * NT; c0 += 16) {
                if (m0 + c0 >= p.m) break;
                uint32_t v[16];
                tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c0, v);
                if (TT == 1) {
                    uint32_t odd[16];
                    tmem_ld16(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + NT + c0, odd);
                    tmem_ld_wait();
#pragma unroll
                    for (int jj = 0; jj < 16; ++jj) v[jj] = __float_as_uint(__uint_as_float(v[jj]) + __uint_as_float(odd[jj]));
                } else {
                    tmem_ld_wait();
                }
                if (row < p.n) {
#pragma unroll
                    for (int jj = 0; jj < 16; ++jj) {
                        const int m = m0 + c0 + jj;
                        if (m < p.m) {
                            const float value = __uint_as_float(v[jj]) * __ldg(p.x_scale + m);   // the token row's factor, undone
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
    if (p.ksplit > 1 && warp >= 2 && warp < 2 + kDequantWarps) {
        // All dequant warps take part (they are idle by now): four threads per weight row.
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
        const int worker = threadIdx.x - 64;
        const long long row = static_cast<long long>(n0) + (worker & (kBM - 1));
        if (*last_flag != 0 && row < p.n) {
            __threadfence();
            const size_t plane = static_cast<size_t>(p.m) * p.n;
            const int m_end = min(m0 + TT * NT, p.m);
            // Four tokens at a time, so that four independent loads per K slice are in flight;
            // the slices are added in index order whatever the arrival order was.
            for (int m = m0 + 4 * (worker >> 7); m < m_end; m += 4 * kSlots) {
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

template <uint32_t FMT, int NT, bool RAWTMA, int TT = 1>
cudaError_t launch_tile(const TcArgs& a) {
    using G = TcGeometry<FMT, NT, RAWTMA, TT>;
    auto kernel = qgemm_tc_kernel<FMT, NT, RAWTMA, TT>;
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
    // Scratch: [f16 activations][one factor per token row][split-K partial tiles].
    const size_t x16_bytes = (static_cast<size_t>(a.m) * a.k * sizeof(__half) + 1023) & ~static_cast<size_t>(1023);
    const size_t factor_bytes = (static_cast<size_t>(a.m) * sizeof(float) + 255) & ~static_cast<size_t>(255);
    if (x16_bytes + factor_bytes > a.scratch_bytes) return cudaErrorMemoryAllocation;
    void* x16 = a.scratch;
    float* factor = reinterpret_cast<float*>(static_cast<uint8_t*>(a.scratch) + x16_bytes);
    float* partial = reinterpret_cast<float*>(static_cast<uint8_t*>(a.scratch) + x16_bytes + factor_bytes);
    const size_t partial_bytes = a.scratch_bytes - x16_bytes - factor_bytes;
    if (!a.skip_prepass) {
        const cudaError_t converted = launch_convert_activations_f16(a.x, a.x_bf16, false, nullptr, 0.0f, x16, factor, a.m, a.k, a.stream);
        if (converted != cudaSuccess) return converted;
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
    p.accumulate = 0;
    p.status = a.device_status;
    p.trace = a.trace;
    const int n_tiles = (a.n + kBM - 1) / kBM;
    const int m_tiles = (a.m + TT * NT - 1) / (TT * NT);
    p.ksplit = choose_ksplit(n_tiles * m_tiles, p.nsb, a.sm_count, static_cast<size_t>(a.m) * a.n * sizeof(float), partial_bytes, a.ticket_count);
    // Hundreds of tokens: a partial tile is megabytes, written and read once more per split (192 tiles of 512 tokens: 127 us
    // unsplit, 160 us split in two).  K is split then only where the tiles leave more than half of the SMs idle.
    if (a.m > 256 && 2 * n_tiles * m_tiles > a.sm_count) p.ksplit = 1;
    if (a.force_ksplit > 0 && a.force_ksplit <= p.nsb &&
        static_cast<size_t>(a.m) * a.n * sizeof(float) * a.force_ksplit <= partial_bytes && n_tiles * m_tiles <= a.ticket_count)
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
    // From 257 tokens on a CTA takes two tiles of 256 (Q8_0's 272-byte super-blocks leave no room for the second).
    if constexpr (FMT == kQ8_0) {
        return launch_tile<FMT, 256, RAWTMA>(a);
    } else {
        // ... when CTAs of 512 tokens still cover most SMs (measured: 96 CTAs of two tiles lose to 192 of one, 128 win over 256)
        const long long wide_ctas = static_cast<long long>((a.n + kBM - 1) / kBM) * ((a.m + 511) / 512);
        if (a.m <= 256 || wide_ctas * 5 < static_cast<long long>(a.sm_count) * 4) return launch_tile<FMT, 256, RAWTMA>(a);
        return launch_tile<FMT, 256, RAWTMA, 2>(a);
    }
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
