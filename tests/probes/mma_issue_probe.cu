// Measurement probe (not part of the library): what a tcgen05.mma (M=128, K=16, bf16, f32 accumulate in TMEM)
// costs its issuing thread and the tensor pipe for N = 16 and 64, under three ways of issuing it
//   variant 0: a one-lane branch, descriptors computed per instruction;
//   variant 1: a one-lane branch, four MMAs per asm block with precomputed descriptors;
//   variant 2: the elected lane of a converged warp (every lane runs the loop);
// and with other warps of the CTA busy (bg = 1: FMA loops, bg = 2: shared-memory stores).  Every wait is bounded.
// Build and run:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I engine_b200/csrc -o /tmp/mma_issue_probe tests/probes/mma_issue_probe.cu
//   /tmp/mma_issue_probe
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include "tcgen05.cuh"
using namespace ribn;

template <int NT>
__global__ void __launch_bounds__(736, 1) probe(long long* out, int reps, int issuers, int* status, int bg_mode, float* sink, int fill, int spread, int variant) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    uint8_t* a_tile = smem;                 // 8 x 16 KB
    uint8_t* b_tile = smem + 8 * 16384;     // 8 x 64 x 128 B
    uint64_t* bars = reinterpret_cast<uint64_t*>(b_tile + 8 * 8192);
    uint32_t* holder = reinterpret_cast<uint32_t*>(bars + 4);
    for (int i = threadIdx.x; i < (8 * 16384 + 8 * 8192) / 16; i += blockDim.x) { const uint32_t w = fill ? (0x3c003c00u ^ ((i * 2654435761u) & 0x03ff03ffu)) : 0u; reinterpret_cast<uint4*>(smem)[i] = make_uint4(w, w, w, w); }
    if (threadIdx.x == 0) { mbar_init(&bars[0], 1); mbar_init(&bars[1], 1); mbar_init(&bars[3], 1); mbar_fence_init(); }
    fence_proxy_async_smem();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) tmem_alloc(holder, 512);
    tcgen05_fence_before_sync();
    __syncthreads();
    tcgen05_fence_after_sync();
    const uint32_t tmem_base = *holder;
    __shared__ volatile int stop_flag;
    __shared__ uint4 scratch[22 * 32];
    if (threadIdx.x == 0) stop_flag = 0;
    __syncthreads();
    if (warp >= 2 && bg_mode != 0) {
        // background load until the issuer is done
        float a = threadIdx.x, b = 1.0001f;
        uint4 v = make_uint4(threadIdx.x, 1, 2, 3);
        long long spins = 0;
        while (stop_flag == 0 && spins < (1 << 22)) {
            if (bg_mode == 1) {
#pragma unroll
                for (int u = 0; u < 64; ++u) a = fmaf(a, b, 0.5f);
            } else if (bg_mode == 2) {
#pragma unroll
                for (int u = 0; u < 16; ++u) { scratch[(warp - 2) * 32 + lane] = v; v.x += u; }
            } else if (bg_mode == 3) {
#pragma unroll
                for (int u = 0; u < 16; ++u) { v.y += scratch[(warp - 2) * 32 + ((lane + u) & 31)].x; }
            } else if (bg_mode == 4) {
                // poll a barrier phase that never completes
#pragma unroll
                for (int u = 0; u < 8; ++u) { if (mbar_try_wait(&bars[3], 0)) a += 1.0f; }
            }
            ++spins;
        }
        if (a == 12345.678f || v.y == 0xdeadbeef) sink[0] = a + v.x;
    }
    if (variant == 2 && warp == 0) {
        constexpr uint32_t idesc = umma_instr_desc(128, NT, 1, 1);
        const uint64_t da = umma_smem_desc_sw128(smem_addr(a_tile));
        const uint64_t db = umma_smem_desc_sw128(smem_addr(b_tile));
        const uint32_t acc = tmem_base;
        const long long t0 = clock64();
        for (int r = 0; r < reps; r += 16) {
#pragma unroll
            for (int st = 0; st < 4; ++st) {
                const uint64_t a0 = da + st * (16384 >> 4), b0 = db + st * (8192 >> 4);
                asm volatile(
                    "{\n\t.reg .pred pf, pt, pe;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t.reg .b32 tmp;\n\t"
                    "elect.sync tmp|pe, 0xffffffff;\n\t"
                    "setp.ne.b32 pf, %4, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
                    "add.s64 a1, %1, 2;\n\tadd.s64 a2, %1, 4;\n\tadd.s64 a3, %1, 6;\n\t"
                    "add.s64 b1, %2, 2;\n\tadd.s64 b2, %2, 4;\n\tadd.s64 b3, %2, 6;\n\t"
                    "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
                    "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, pt;\n\t"
                    "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, pt;\n\t"
                    "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, pt;\n\t}"
                    :: "r"(acc), "l"(a0), "l"(b0), "r"(idesc), "r"(st) : "memory");
            }
        }
        const long long t1 = clock64();
        bool ok = true;
        if (lane == 0) { umma_commit(&bars[0]); }
        __syncwarp();
        ok = mbar_wait_bounded(&bars[0], 0);
        const long long t2 = clock64();
        if (!ok) atomicExch(status, 1);
        if (blockIdx.x == 0 && lane == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
        if (lane == 0) stop_flag = 1;
    } else if (warp < issuers && lane == 0) {
        constexpr uint32_t idesc = umma_instr_desc(128, NT, 1, 1);
        const uint64_t da = umma_smem_desc_sw128(smem_addr(a_tile));
        const uint64_t db = umma_smem_desc_sw128(smem_addr(b_tile));
        const uint32_t acc = tmem_base + warp * 256;
        const long long t0 = clock64();
        if (variant == 0) {
            for (int r = 0; r < reps; ++r) { const int st = spread ? ((r >> 2) & 7) : 0; umma_f16(acc, da + 2 * (r & 3) + st * (16384 >> 4), db + 2 * (r & 3) + st * (8192 >> 4), idesc, (r & 15) != 0); }
        } else if (variant == 1) {
            // 16 MMAs per iteration, descriptors precomputed, constant predicates
            uint64_t a4[4], b4[4];
            for (int st = 0; st < 4; ++st) { a4[st] = da + st * (16384 >> 4); b4[st] = db + st * (8192 >> 4); }
            for (int r = 0; r < reps; r += 16) {
#pragma unroll
                for (int st = 0; st < 4; ++st) {
                    asm volatile(
                        "{\n\t.reg .pred pf, pt;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
                        "setp.ne.b32 pf, %4, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
                        "add.s64 a1, %1, 2;\n\tadd.s64 a2, %1, 4;\n\tadd.s64 a3, %1, 6;\n\t"
                        "add.s64 b1, %2, 2;\n\tadd.s64 b2, %2, 4;\n\tadd.s64 b3, %2, 6;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, pt;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, pt;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, pt;\n\t}"
                        :: "r"(acc), "l"(a4[st]), "l"(b4[st]), "r"(idesc), "r"(st) : "memory");
                }
            }
        }
        const long long t1 = clock64();
        umma_commit(&bars[warp]);
        const bool ok = mbar_wait_bounded(&bars[warp], 0);
        const long long t2 = clock64();
        if (!ok) atomicExch(status, 1);
        if (blockIdx.x == 0) { out[warp * 2] = t1 - t0; out[warp * 2 + 1] = t2 - t0; }
        stop_flag = 1;
    }
    tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, 512);
}

template <int NT> void run(int reps, int issuers, int grid, long long* out, int* status, int bg_mode = 0, int threads = 128, int fill = 0, int spread = 0, int variant = 0) {
    static float* sink = nullptr; if (!sink) cudaMalloc(&sink, 64);
    const size_t smem = 1024 + 8 * 16384 + 8 * 8192 + 64;
    cudaFuncSetAttribute(probe<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    probe<NT><<<grid, threads, smem>>>(out, reps, issuers, status, bg_mode, sink, fill, spread, variant);
    cudaDeviceSynchronize();
    probe<NT><<<grid, threads, smem>>>(out, reps, issuers, status, bg_mode, sink, fill, spread, variant);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[4]; int st;
    cudaMemcpy(h, out, sizeof h, cudaMemcpyDeviceToHost); cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
    printf("variant=%d fill=%d spread=%d bg=%d thr=%d N=%3d reps=%d issuers=%d grid=%3d: issue %.1f cyc/mma, complete %.1f cyc/mma (2nd issuer: %.1f / %.1f) status=%d %s\n", variant, fill, spread, bg_mode, threads, NT, reps, issuers, grid,
           (double)h[0] / reps, (double)h[1] / reps, issuers > 1 ? (double)h[2] / reps : 0.0, issuers > 1 ? (double)h[3] / reps : 0.0, st, cudaGetErrorString(e));
}

int main() {
    long long* out; int* status;
    cudaMalloc(&out, 64); cudaMalloc(&status, 4); cudaMemset(status, 0, 4); cudaMemset(out, 0, 64);
    for (int variant = 0; variant <= 2; ++variant) {
        run<16>(512, 1, 148, out, status, 0, 128, 1, 1, variant);
        run<16>(512, 1, 148, out, status, 1, 736, 1, 1, variant);
        run<16>(512, 1, 148, out, status, 2, 736, 1, 1, variant);
        run<64>(512, 1, 148, out, status, 1, 736, 1, 1, variant);
    }
    return 0;
}
