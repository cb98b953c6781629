// Measurement probe (not part of the library): how fast one producer warp per CTA pulls weight bytes into a
// shared-memory ring with (a) tiled TMA boxes of 128 rows x W bytes, (b) per-row bulk copies of W bytes, no
// consumer at all.  Every wait is bounded.
// Build and run:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I engine_b200/csrc -o /tmp/tma_box_probe tests/probes/tma_box_probe.cu
//   /tmp/tma_box_probe
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "tcgen05.cuh"

using namespace ribn;

struct P { const uint8_t* w; unsigned long long row_bytes; int rows; int nsb; int box_bytes; int stages; int mode; int* status; };

__global__ void __launch_bounds__(128, 1) probe(const __grid_constant__ CUtensorMap wmap, const P p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint8_t* ring = smem + 1024;
    const int stage_bytes = 128 * p.box_bytes;
    if (threadIdx.x == 0) { for (int s = 0; s < p.stages; ++s) mbar_init(&full[s], p.mode == 0 ? 1 : 32); mbar_fence_init(); }
    __syncthreads();
    const int tiles = p.rows / 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp != 0) return;
    // each CTA walks tiles blockIdx.x, +gridDim.x ...; within a tile all super-blocks
    int it = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        for (int sb = 0; sb < p.nsb; ++sb, ++it) {
            const int s = it % p.stages;
            if (it >= p.stages) { if (!mbar_wait_bounded(&full[s], ((it / p.stages) - 1) & 1)) { atomicExch(p.status, 1); return; } }
            if (p.mode == 0) {
                if (lane == 0) {
                    mbar_arrive_expect_tx(&full[s], stage_bytes);
                    tma_load_2d(ring + s * stage_bytes, &wmap, sb * p.box_bytes / 2, tile * 128, &full[s]);
                }
            } else {
                // per-row bulk copies: 4 rows per lane
                mbar_arrive_expect_tx(&full[s], 4 * p.box_bytes);
                for (int q = 0; q < 4; ++q) {
                    const int r = lane + 32 * q;
                    bulk_copy_g2s(ring + s * stage_bytes + r * p.box_bytes,
                                  p.w + (unsigned long long)(tile * 128 + r) * p.row_bytes + (unsigned long long)sb * p.box_bytes, p.box_bytes, &full[s]);
                }
            }
            __syncwarp();
        }
    }
    // drain
    for (int d = 0; d < p.stages && d < it; ++d) {
        const int k = it - 1 - d; const int s = k % p.stages;
        if (!mbar_wait_bounded(&full[s], (k / p.stages) & 1)) { atomicExch(p.status, 2); return; }
    }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int main() {
    void* sym = nullptr; cudaDriverEntryPointQueryResult qr;
    cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qr);
    auto encode = (EncodeTiledFn)sym;
    const int rows = 12288 * 8, nsb_total = 16;  // 8 matrices of 12288x4096 Q4_K back to back = 226 MB (> L2)
    const unsigned long long row_bytes = 2304;
    uint8_t* w; cudaMalloc(&w, (size_t)rows * row_bytes); cudaMemset(w, 1, (size_t)rows * row_bytes);
    int* status; cudaMalloc(&status, 4); cudaMemset(status, 0, 4);
    cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    struct Cfg { int mode, box, stages, grid; };
    std::vector<Cfg> cfgs = {{0,144,4,148},{0,144,8,148},{0,144,8,296},{0,576,2,148},{0,576,4,148},{0,2304,1,148},
                             {1,144,8,148},{1,576,4,148},{1,1152,1,148},{1,1152,1,296},{1,1152,1,148},{0,144,11,148},{0,288,5,148}};
    for (auto c : cfgs) {
        const int nsb = (int)(row_bytes / c.box);
        CUtensorMap map;
        cuuint64_t dims[2] = {row_bytes / 2, (cuuint64_t)rows}; cuuint64_t strides[1] = {row_bytes};
        cuuint32_t box[2] = {(cuuint32_t)c.box / 2 > 256 ? 256u : (cuuint32_t)c.box / 2, 128}; cuuint32_t el[2] = {1, 1};
        int box_bytes = box[0] * 2;
        if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, w, dims, strides, box, el, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) { printf("encode fail\n"); continue; }
        P p{w, row_bytes, rows, (int)(row_bytes / box_bytes), box_bytes, c.stages, c.mode, status};
        size_t smem = 2048 + (size_t)c.stages * 128 * box_bytes;
        if (smem > 227 * 1024) { printf("skip smem\n"); continue; }
        int grid = c.grid; if (c.grid == 296 && smem > 113 * 1024) grid = 148;
        cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
        probe<<<grid, 128, smem>>>(map, p); cudaDeviceSynchronize();
        cudaEventRecord(a); probe<<<grid, 128, smem>>>(map, p); cudaEventRecord(b); cudaDeviceSynchronize();
        float ms; cudaEventElapsedTime(&ms, a, b);
        int st; cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
        printf("mode=%s box=%4d stages=%2d grid=%3d inflight/CTA=%6.1fKB : %.1f us  %.0f GB/s  status=%d err=%s\n", c.mode ? "bulk-rows" : "tiled-box",
               box_bytes, c.stages, grid, c.stages * 128 * box_bytes / 1024.0, ms * 1e3, (double)rows * row_bytes / ms / 1e6, st, cudaGetErrorString(cudaGetLastError()));
        (void)nsb; (void)nsb_total;
    }
    return 0;
}
