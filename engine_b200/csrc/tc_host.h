// Host-side helpers shared by the tensor-core kernels: kernel parameter block, tensor-map encoding
// through the runtime's driver entry point, split-K choice.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ribn {

struct TcParams {
    const uint8_t* w;
    unsigned long long w_bytes;
    unsigned long long row_bytes;
    void* y;                 // [m][n] f32 or bf16
    float* partial;          // split-K scratch: [ksplit][m][n] f32
    const float* x_scale;    // decode kernel: power-of-two factor per member row (activations were divided by it)
    unsigned int* tickets;   // one counter per (n tile, m tile), zero between launches
    int k, n, m;
    int nsb;                 // super-blocks per row
    int ksplit;
    int y_bf16;
    int accumulate;          // decode kernel: add to y instead of overwriting it
    int* status;
    // Diagnostics: when non-null, CTA (0,0,0) of the decode kernel records SM clock stamps of its
    // pipeline events here: trace[(role * 64 + step) * 8 + event], 4 roles x 64 steps x 8 events.
    long long* trace;
};

// cuTensorMapEncodeTiled through the runtime's driver entry point (the library does not link libcuda).
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// Waves x (K work per CTA + a fixed cost of about one and a half super-blocks for pipeline fill,
// TMEM allocation and the epilogue), minimised over the split factor.
inline int choose_ksplit(int tiles, int nsb, int sm_count, size_t plane_bytes, size_t scratch_bytes, int max_tickets) {
    if (tiles > max_tickets) return 1;
    int best = 1;
    double best_cost = 1e30;
    const int limit = nsb < 16 ? nsb : 16;
    for (int ks = 1; ks <= limit; ++ks) {
        if (ks > 1 && plane_bytes * ks > scratch_bytes) break;
        const int waves = (tiles * ks + sm_count - 1) / sm_count;
        const double per_cta = static_cast<double>((nsb + ks - 1) / ks) + 1.5 + (ks > 1 ? 0.5 : 0.0);
        const double cost = waves * per_cta;
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = ks;
        }
    }
    return best;
}

// The decode kernel's split factor, fitted to measurements on B200 (times in units of one 128-row super-block,
// ~1.45 us): a CTA costs its K share plus ~5 units of launch, pipeline fill and epilogue; every split adds a partial
// tile the last CTA of the tile has to add, ~0.33 units per 16 tokens.  Ties go to the smaller factor.
inline int choose_ksplit_decode(int tiles, int nsb, int sm_count, size_t plane_bytes, size_t scratch_bytes, int max_tickets,
                                int tokens_per_tile) {
    if (tiles > max_tickets) return 1;
    int best = 1;
    double best_cost = 1e30;
    const int limit = nsb < 16 ? nsb : 16;
    for (int ks = 1; ks <= limit; ++ks) {
        if (ks > 1 && plane_bytes * ks > scratch_bytes) break;
        const int waves = (tiles * ks + sm_count - 1) / sm_count;
        const double per_cta = static_cast<double>((nsb + ks - 1) / ks) + 5.0;
        const double reduce = ks > 1 ? ks * 0.33 * (tokens_per_tile / 16.0) : 0.0;
        const double cost = waves * per_cta + reduce;
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = ks;
        }
    }
    return best;
}

}  // namespace ribn
