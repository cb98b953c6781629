// Dequant-fused GEMV for GGUF block formats, CUDA-core path (members 1..8).
//
//   y[m][n] = sum_k dequant(W[n][k]) * x[m][k]          f32 accumulation
//
// Replaces q{4,5,6}_k_gemv_warp / q8_0_gemv_warp and the *_gemv_warp_batch
// kernels of the reference (crates/nvidia/src/kernels/quantized/q4_k.cu:103-258
// and the q5_k / q6_k / q8_0 twins).  Not a port: the reference gives one warp
// one row and reads the weights with 32-bit global loads; here
//
//   * the weight stream never passes through registers on its way in: a
//     producer warp issues untiled bulk copies (TMA, cp.async.bulk) of whole
//     row segments into a shared-memory ring, completion counted on mbarriers,
//     so the bytes in flight per SM are set by the ring depth and not by
//     occupancy or by the unpack code;
//   * rows are dealt to CTAs in equal contiguous ranges (the grid is a multiple
//     of the SM count), so every SM streams the same number of bytes;
//   * a consumer warp owns RW rows x a slice of the K range: the activation
//     values it holds in registers are reused for RW rows, which keeps the
//     activation reads (L1) well below the weight stream;
//   * the 6-bit scale/min fields are decoded once per super-block per warp into
//     a small shared table (one lane per super-block), not once per lane;
//   * the K slices of a row are summed across warps in shared memory in a fixed
//     order: results are deterministic, no atomics.
//
// Bulk copies need 16-byte aligned sources.  Q6_K rows (210-byte blocks) are
// only 2-byte aligned, so a segment is copied from its address rounded down to
// 16 bytes and indexed from the remainder in shared memory; the last few bytes
// of a tensor whose length is not a multiple of 16 are fetched with plain loads.
#include "formats.cuh"
#include "internal.h"
#include "pipeline.cuh"

namespace ribn {
namespace {

struct GemvParams {
    const uint8_t* w;
    unsigned long long w_bytes;
    const void* x;
    void* y;
    int k;
    int n;
    int nsb;       // super-blocks per row (the last one of a Q8_0 row may be partial)
    unsigned long long row_bytes;
    int members;
    int y_bf16;
    int* status;
};

template <typename XT>
__device__ __forceinline__ void load_x4(const XT* p, float (&v)[4]);

template <>
__device__ __forceinline__ void load_x4<float>(const float* p, float (&v)[4]) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}

template <>
__device__ __forceinline__ void load_x4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 t = __ldg(reinterpret_cast<const uint2*>(p));
    v[0] = __uint_as_float(t.x << 16);
    v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16);
    v[3] = __uint_as_float(t.y & 0xffff0000u);
}

// Byte offset of super-block `sb` of row `row` inside the tensor, and how far that is from
// the 16-byte boundary below it (the bulk copy starts at the boundary).
template <typename F>
__device__ __forceinline__ unsigned long long segment_offset(const GemvParams& p, long long row, int sb) {
    return static_cast<unsigned long long>(row) * p.row_bytes + static_cast<unsigned long long>(sb) * F::kBytes;
}

template <typename F>
__device__ __forceinline__ uint32_t segment_misalignment(const GemvParams& p, long long row, int sb) {
    if (F::kBytes == 144 || F::kBytes == 176) return 0;  // Q4_K / Q5_K blocks are whole 16-byte units
    return static_cast<uint32_t>(segment_offset<F>(p, row, sb) & 15ull);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

// Compile-time geometry of one kernel variant.
//   WR x WK consumer warps: WR row groups of RW rows, WK slices of the K range
//   KB      super-blocks per row per pipeline stage (a multiple of WK)
//   STAGES  depth of the shared-memory ring
template <uint32_t FMT, int MT, int WR, int WK, int RW, int KB, int STAGES>
struct GemvGeometry {
    using F = Format<FMT>;
    static constexpr int kConsumerWarps = WR * WK;
    static constexpr int kThreads = (kConsumerWarps + 1) * 32;
    static constexpr int kRows = WR * RW;                 // rows per tile
    static constexpr int kKBW = KB / WK;                  // super-blocks per warp per stage
    static constexpr int kSlot = ((KB * F::kBytes + 15) / 16) * 16 + 16;
    static constexpr int kStageBytes = kRows * kSlot;
    static constexpr int kTableFloats = RW * kKBW * 16;   // per consumer warp
    static constexpr int kRingBytes = STAGES * kStageBytes;
    static constexpr int kTableBytes = kConsumerWarps * kTableFloats * 4;
    static constexpr int kRedBytes = 2 * WK * kRows * MT * 4;
    static constexpr int kBarrierBytes = (2 * STAGES + 2) * 8;
    static constexpr int kSmemBytes = kRingBytes + kTableBytes + ((kRedBytes + 15) / 16) * 16 + kBarrierBytes;
    static_assert(KB % WK == 0, "stage super-blocks must split evenly over K slices");
    static_assert(kRows <= 32, "one producer lane per row");
};

template <uint32_t FMT, int MT, typename XT, int WR, int WK, int RW, int KB, int STAGES>
__global__ void __launch_bounds__(GemvGeometry<FMT, MT, WR, WK, RW, KB, STAGES>::kThreads)
gemv_kernel(const GemvParams p) {
    using G = GemvGeometry<FMT, MT, WR, WK, RW, KB, STAGES>;
    using F = Format<FMT>;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    float* tables = reinterpret_cast<float*>(smem + G::kRingBytes);
    float* red = reinterpret_cast<float*>(smem + G::kRingBytes + G::kTableBytes);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + G::kRingBytes + G::kTableBytes + ((G::kRedBytes + 15) / 16) * 16);
    uint64_t* empty = full + STAGES;
    uint64_t* red_bar = empty + STAGES;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 32);
            mbar_init(&empty[s], G::kConsumerWarps);
        }
        mbar_init(&red_bar[0], G::kConsumerWarps);
        mbar_init(&red_bar[1], G::kConsumerWarps);
        mbar_fence_init();
    }
    __syncthreads();

    // Equal contiguous row ranges per CTA.
    const long long row_begin = static_cast<long long>(p.n) * blockIdx.x / gridDim.x;
    const long long row_end = static_cast<long long>(p.n) * (blockIdx.x + 1) / gridDim.x;
    const int tiles = static_cast<int>((row_end - row_begin + G::kRows - 1) / G::kRows);
    const int chunks = (p.nsb + KB - 1) / KB;
    const int total = tiles * chunks;

    if (warp == G::kConsumerWarps) {
        // ---------------- producer warp: one lane per row of the tile ----------------
        const unsigned long long safe_end = p.w_bytes & ~15ull;
        for (int it = 0; it < total; ++it) {
            const int s = it % STAGES;
            const int use = it / STAGES;
            if (use > 0 && !mbar_wait_bounded(&empty[s], (use - 1) & 1)) {
                atomicExch(p.status, kDeviceWaitTimeout);
                return;
            }
            const int tile = it / chunks;
            const int chunk = it - tile * chunks;
            const long long row = row_begin + static_cast<long long>(tile) * G::kRows + lane;
            const int sb0 = chunk * KB;
            const int nsbs = min(KB, p.nsb - sb0);
            if (lane < G::kRows && row < row_end) {
                const unsigned long long g0 = segment_offset<F>(p, row, sb0);
                const unsigned long long g1 = min(g0 + static_cast<unsigned long long>(nsbs) * F::kBytes,
                                                  static_cast<unsigned long long>(row + 1) * p.row_bytes);
                const unsigned long long a0 = g0 & ~15ull;
                const unsigned long long a1 = (g1 + 15ull) & ~15ull;
                uint8_t* dst = ring + s * G::kStageBytes + lane * G::kSlot;
                if (a1 <= safe_end) {
                    const uint32_t bytes = static_cast<uint32_t>(a1 - a0);
                    mbar_arrive_expect_tx(&full[s], bytes);
                    bulk_copy_g2s(dst, p.w + a0, bytes, &full[s]);
                } else {
                    // Last bytes of a tensor whose length is not a multiple of 16.
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
        }
        return;
    }

    // ---------------- consumer warps ----------------
    pdl_wait_prior();   // the activations may be the previous kernel's output (the weight stream is already running)
    const int wr = warp / WK;
    const int wk = warp % WK;
    int off_a, off_b;
    F::offsets(lane, off_a, off_b);
    float* table = tables + warp * G::kTableFloats;
    const XT* x = static_cast<const XT*>(p.x);

    for (int tile = 0; tile < tiles; ++tile) {
        float acc[RW][MT];
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;
        const long long row_base = row_begin + static_cast<long long>(tile) * G::kRows + wr * RW;

        for (int chunk = 0; chunk < chunks; ++chunk) {
            const int it = tile * chunks + chunk;
            const int s = it % STAGES;
            const int sb0 = chunk * KB;
            const int nsbs = min(KB, p.nsb - sb0);
            if (!mbar_wait_bounded(&full[s], (it / STAGES) & 1)) {
                atomicExch(p.status, kDeviceWaitTimeout);
                return;
            }
            const uint8_t* stage = ring + s * G::kStageBytes + wr * RW * G::kSlot;

            // Scale tables: one lane per (row, super-block) of this warp's share.
            for (int e = lane; e < RW * G::kKBW; e += 32) {
                const int r = e / G::kKBW;
                const int sbl = wk + (e % G::kKBW) * WK;
                const long long row = row_base + r;
                if (sbl < nsbs && row < row_end) {
                    const uint32_t off = segment_misalignment<F>(p, row, sb0);
                    F::decode_table(stage + r * G::kSlot + off + sbl * F::kBytes, table + e * 16);
                }
            }
            __syncwarp();

#pragma unroll 1
            for (int i = 0; i < G::kKBW; ++i) {
                const int sbl = wk + i * WK;
                if (sbl >= nsbs) break;
                const int k0 = (sb0 + sbl) * kSuperBlock;
                // Only a Q8_0 row can end inside a super-block (K is a multiple of 32 there).
                const bool lane_ok = F::kBytes != Format<kQ8_0>::kBytes || off_a < p.k - k0;
                float xa[MT][4], xb[MT][4], sum_a[MT], sum_b[MT];
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const XT* xm = x + static_cast<size_t>(min(m, p.members - 1)) * p.k + k0;
                    if (lane_ok) {
                        load_x4<XT>(xm + off_a, xa[m]);
                        load_x4<XT>(xm + off_b, xb[m]);
                    }
                    if (MT == 1 && F::kHasMin) {
                        sum_a[m] = (xa[m][0] + xa[m][1]) + (xa[m][2] + xa[m][3]);
                        sum_b[m] = (xb[m][0] + xb[m][1]) + (xb[m][2] + xb[m][3]);
                    }
                }
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    const long long row = row_base + r;
                    if (row < row_end && lane_ok) {
                        const uint32_t off = segment_misalignment<F>(p, row, sb0);
                        const uint8_t* blk = stage + r * G::kSlot + off + sbl * F::kBytes;
                        float qa[4], qb[4], sa, ma, sb, mb;
                        F::quants(blk, lane, qa, qb);
                        F::scales(table + (r * G::kKBW + i) * 16, lane, sa, ma, sb, mb);
                        if (MT == 1) {
                            // One activation row: apply the group scale to the 4-term dot,
                            // and the group minimum to the sum of the activations.
                            float da = qa[0] * xa[0][0];
                            float db = qb[0] * xb[0][0];
#pragma unroll
                            for (int j = 1; j < 4; ++j) {
                                da = fmaf(qa[j], xa[0][j], da);
                                db = fmaf(qb[j], xb[0][j], db);
                            }
                            float t = fmaf(sa, da, acc[r][0]);
                            t = fmaf(sb, db, t);
                            if (F::kHasMin) {
                                t = fmaf(-ma, sum_a[0], t);
                                t = fmaf(-mb, sum_b[0], t);
                            }
                            acc[r][0] = t;
                        } else {
                            float wa[4], wb[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                wa[j] = dequant_value(sa, qa[j], ma);
                                wb[j] = dequant_value(sb, qb[j], mb);
                            }
#pragma unroll
                            for (int m = 0; m < MT; ++m) {
                                float t = acc[r][m];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    t = fmaf(wa[j], xa[m][j], t);
                                    t = fmaf(wb[j], xb[m][j], t);
                                }
                                acc[r][m] = t;
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }

        // Sum the lanes of each warp, then the K slices in a fixed order.
        float* red_buf = red + (tile & 1) * (WK * G::kRows * MT);
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const float v = warp_sum(acc[r][m]);
                if (lane == 0) red_buf[(wk * G::kRows + wr * RW + r) * MT + m] = v;
            }
        __syncwarp();
        if (lane == 0) mbar_arrive(&red_bar[tile & 1]);
        if (!mbar_wait_bounded(&red_bar[tile & 1], (tile >> 1) & 1)) {
            atomicExch(p.status, kDeviceWaitTimeout);
            return;
        }
        for (int e = threadIdx.x; e < G::kRows * MT; e += G::kConsumerWarps * 32) {
            const int rr = e / MT;
            const int m = e % MT;
            const long long row = row_begin + static_cast<long long>(tile) * G::kRows + rr;
            if (row < row_end && m < p.members) {
                float v = red_buf[rr * MT + m];
#pragma unroll
                for (int q = 1; q < WK; ++q) v += red_buf[(q * G::kRows + rr) * MT + m];
                const size_t o = static_cast<size_t>(m) * p.n + row;
                if (p.y_bf16) {
                    static_cast<__nv_bfloat16*>(p.y)[o] = __float2bfloat16_rn(v);
                } else {
                    static_cast<float*>(p.y)[o] = v;
                }
            }
        }
    }
}

template <uint32_t FMT, int MT, typename XT, int WR, int WK, int RW, int KB, int STAGES>
cudaError_t launch_variant(const GemvArgs& a, int ctas_per_sm) {
    using G = GemvGeometry<FMT, MT, WR, WK, RW, KB, STAGES>;
    auto kernel = gemv_kernel<FMT, MT, XT, WR, WK, RW, KB, STAGES>;
    static int configured_device = -1;  // per instantiation; the attribute is per device and function
    int device = 0;
    cudaGetDevice(&device);
    if (configured_device != device) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G::kSmemBytes);
        if (e != cudaSuccess) return e;
        configured_device = device;
    }
    GemvParams p;
    p.w = a.weights;
    p.w_bytes = a.weight_bytes;
    p.x = a.x;
    p.y = a.y;
    p.k = a.k;
    p.n = a.n;
    p.nsb = (a.k + kSuperBlock - 1) / kSuperBlock;
    p.row_bytes = a.value_type == kQ8_0 ? static_cast<unsigned long long>(a.k / 32) * 34
                                        : static_cast<unsigned long long>(a.k / kSuperBlock) * G::F::kBytes;
    p.members = a.members;
    p.y_bf16 = a.y_bf16 ? 1 : 0;
    p.status = a.device_status;
    int grid = a.sm_count * ctas_per_sm;
    // Never more CTAs than rows: a CTA without rows would only burn a launch slot.
    if (grid > a.n) grid = a.n;
    return launch_kernel(kernel, dim3(grid), dim3(G::kThreads), G::kSmemBytes, a.stream, p);
}

template <uint32_t FMT, int MT, typename XT>
cudaError_t launch_for_variant(const GemvArgs& a) {
    switch (a.variant) {
        case 1: return launch_variant<FMT, MT, XT, 4, 2, 4, 4, 6>(a, 2);
        case 2: return launch_variant<FMT, MT, XT, 1, 8, 4, 8, 6>(a, 2);
        case 3: return launch_variant<FMT, MT, XT, 2, 4, 4, 8, 4>(a, 3);
        default: return launch_variant<FMT, MT, XT, 2, 4, 4, 8, 6>(a, 2);
    }
}

template <uint32_t FMT, typename XT>
cudaError_t launch_for_members(const GemvArgs& a) {
    if (a.members == 1) return launch_for_variant<FMT, 1, XT>(a);
    if (a.members == 2) return launch_for_variant<FMT, 2, XT>(a);
    if (a.members <= 4) return launch_for_variant<FMT, 4, XT>(a);
    return launch_for_variant<FMT, 8, XT>(a);
}

template <uint32_t FMT>
cudaError_t launch_for_format(const GemvArgs& a) {
    return a.x_bf16 ? launch_for_members<FMT, __nv_bfloat16>(a) : launch_for_members<FMT, float>(a);
}

}  // namespace

cudaError_t launch_gemv(const GemvArgs& a) {
    if (a.members < 1 || a.members > 8) return cudaErrorInvalidValue;
    switch (a.value_type) {
        case kQ4_K: return launch_for_format<kQ4_K>(a);
        case kQ5_K: return launch_for_format<kQ5_K>(a);
        case kQ6_K: return launch_for_format<kQ6_K>(a);
        case kQ8_0: return launch_for_format<kQ8_0>(a);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ribn
