// The operators of a dense-attention decoder layer that sit between the quantized GEMVs.
//
// They replace, for decode, these kernels of the reference (crates/nvidia/src/model_ops.rs and
// kernels/quantized/q4_k.cu):
//   q4_k_embedding{,_batch}   q4_k.cu:1-67          -> embedding_kernel (any of the four block formats)
//   strided_rms_norm          model_ops.rs:660-684  \
//   rope_neox                 model_ops.rs:393-422   > qk_norm_rope_append_kernel (one launch per token batch)
//   kv_append_f16             model_ops.rs:1256-1275 /
//   attn_score_gqa            model_ops.rs:439-562  -> attention_split_kernel + attention_combine_kernel
//   silu_mul                  model_ops.rs:316-328  -> silu_mul_kernel
//   residual_add              model_ops.rs:600-610  -> residual_add_kernel
//   argmax{,_batch}           model_ops.rs:201-314  -> argmax_kernel
// The arithmetic follows the reference's host model of the layer
// (crates/nvidia/src/qwen_reference.rs:368-470): per-head RMSNorm with raw weights, NEOX half-split
// rotary pairs (p, p + rot/2) with theta = pos * base^(-2p/rot), scores scaled by 1/sqrt(head_dim),
// softmax over all cached tokens, f32 accumulation; K and V are cached as f16.
//
// Layout of the KV cache (ours; the reference's is [token][kv_head][dim]):
//   [member][kv_head][token][dim] f16, max_context tokens per (member, head),
// so that one CTA streams the contiguous tokens of one head, shared by the query heads of its group.
//
// Positions are read from device memory (one int per member), so that a captured CUDA graph can be
// replayed for every decode step.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "formats.cuh"
#include "internal.h"
#include "pipeline.cuh"

namespace ribn {
namespace {

// ---------------------------------------------------------------- embedding
template <uint32_t FMT>
__global__ void __launch_bounds__(256) embedding_kernel(const uint8_t* __restrict__ w, const uint32_t* __restrict__ tokens,
                                                        float* __restrict__ out, int k, unsigned int vocabulary,
                                                        unsigned long long row_bytes, int nsb) {
    pdl_launch_dependents();
    pdl_wait_prior();   // inputs come from the kernels before this one in the stream
    using F = Format<FMT>;
    const int lane = threadIdx.x & 31;
    const int sb = blockIdx.x * 8 + (threadIdx.x >> 5);
    const unsigned int token = tokens[blockIdx.y];
    if (sb >= nsb || token >= vocabulary) return;   // as the reference: an out-of-range token leaves its row untouched
    int off_a, off_b;
    F::offsets(lane, off_a, off_b);
    const uint8_t* blk = w + static_cast<unsigned long long>(token) * row_bytes + static_cast<unsigned long long>(sb) * F::kBytes;
    float qa[4], qb[4], sa, ma, sb_scale, mb;
    F::quants(blk, lane, qa, qb);
    F::direct_scales(blk, lane, sa, ma, sb_scale, mb);
    float* dst = out + static_cast<size_t>(blockIdx.y) * k + static_cast<size_t>(sb) * kSuperBlock;
    *reinterpret_cast<float4*>(dst + off_a) = make_float4(dequant_value(sa, qa[0], ma), dequant_value(sa, qa[1], ma),
                                                          dequant_value(sa, qa[2], ma), dequant_value(sa, qa[3], ma));
    *reinterpret_cast<float4*>(dst + off_b) = make_float4(dequant_value(sb_scale, qb[0], mb), dequant_value(sb_scale, qb[1], mb),
                                                          dequant_value(sb_scale, qb[2], mb), dequant_value(sb_scale, qb[3], mb));
}

// ---------------------------------------------------------------- head norm + rope + cache append
// grid (q_heads + 2 kv_heads, members), head_dim threads.  Blocks [0, q_heads) rewrite a query head in
// place; [q_heads, q_heads + kv_heads) normalise and rotate a key head into the f16 cache; the rest
// convert a value head into the cache.
__global__ void __launch_bounds__(256) qk_norm_rope_append_kernel(float* __restrict__ q, const float* __restrict__ k,
                                                                  const float* __restrict__ v, const float* __restrict__ q_norm,
                                                                  const float* __restrict__ k_norm, float eps,
                                                                  const int* __restrict__ positions, int q_heads, int kv_heads,
                                                                  int head_dim, int rot_pairs, float base, __half* __restrict__ k_cache,
                                                                  __half* __restrict__ v_cache, long long max_context, int shared_cache,
                                                                  int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait_prior();   // inputs come from the kernels before this one in the stream
    __shared__ float values[256];
    __shared__ float warp_sums[8];
    const int member = blockIdx.y;
    const int t = threadIdx.x;
    const int position = positions[member];
    int head = blockIdx.x;
    const float* source;
    const float* norm = nullptr;
    bool rotate = true;
    __half* cache = nullptr;
    float* in_place = nullptr;
    if (head < q_heads) {
        in_place = q + (static_cast<size_t>(member) * q_heads + head) * head_dim;
        source = in_place;
        norm = q_norm;
    } else if (head < q_heads + kv_heads) {
        head -= q_heads;
        source = k + (static_cast<size_t>(member) * kv_heads + head) * head_dim;
        norm = k_norm;
        cache = k_cache;
    } else {
        head -= q_heads + kv_heads;
        source = v + (static_cast<size_t>(member) * kv_heads + head) * head_dim;
        rotate = false;
        cache = v_cache;
    }
    float x = source[t];
    if (norm != nullptr) {
        float sum = x * x;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if ((t & 31) == 0) warp_sums[t >> 5] = sum;
        __syncthreads();
        float total = 0.0f;
        for (int wi = 0; wi < (head_dim + 31) / 32; ++wi) total += warp_sums[wi];
        const float inverse = rsqrtf(total / static_cast<float>(head_dim) + eps);
        x = x * inverse * norm[t];
    }
    if (rotate && rot_pairs > 0) {
        values[t] = x;
        __syncthreads();
        if (t < 2 * rot_pairs) {
            const int pair = t < rot_pairs ? t : t - rot_pairs;
            const float theta = static_cast<float>(position) * powf(base, -(2.0f * static_cast<float>(pair)) / (2.0f * static_cast<float>(rot_pairs)));
            const float sin_theta = sinf(theta);
            const float cos_theta = cosf(theta);
            const float x0 = values[pair];
            const float x1 = values[pair + rot_pairs];
            x = t < rot_pairs ? x0 * cos_theta - x1 * sin_theta : x0 * sin_theta + x1 * cos_theta;
        }
    }
    if (in_place != nullptr) {
        in_place[t] = x;
    } else if (position >= 0 && position < max_context) {
        // a prefill chunk: the members are consecutive tokens of one sequence and append to the same cache
        const long long sequence = shared_cache ? 0 : member;
        cache[((sequence * kv_heads + head) * max_context + position) * head_dim + t] = __float2half_rn(x);
    } else if (t == 0) {
        // The position comes from device memory (a replayed graph advances it): outside the cache nothing is
        // stored and the context's status word says so.
        atomicExch(status, kDevicePositionOutOfRange);
    }
}

// ---------------------------------------------------------------- attention, one new token per member
// Split-KV ("flash decoding") on the warp-level tensor-core instruction: grid (kv_heads, members, splits), four warps.
// The query heads that share a KV head (up to eight) are the rows of one m16n8k16 A operand, so a K / V tile is read from
// shared memory once for the whole group (a kernel that lets every head read the tile with its own loads is bound by
// shared-memory bandwidth at 1/8 of what HBM delivers).  The CTA walks its token range in tiles of 64: cp.async brings K
// and V rows into padded shared-memory rows (272 bytes: ldmatrix of eight rows touches every bank once), warp w owns
// tokens 16 w .. 16 w + 15 of every tile and keeps its own running maximum, sum and 16 x 128 output accumulator; the four
// warps are merged through shared memory at the end.  The reference computes in f32 over the f16 cache
// (model_ops.rs:439-562); to stay at that accuracy the f32 queries and the probabilities enter the MMAs as two f16 parts
// each (hi + lo: about 22 bits), with f32 accumulation.
constexpr int kAttnTile = 64;
constexpr int kAttnHeadDim = 128;
constexpr int kAttnKStride = kAttnHeadDim + 8;   // halves; rows 272 bytes apart
constexpr int kAttnMaxGroup = 8;
constexpr int kAttnWarps = 4;
constexpr int kAttnTileBytes = kAttnTile * kAttnKStride * 2;
constexpr int kAttnSmemBytes = 4 * kAttnTileBytes;   // two stages of K and V; reused for the merge of the warps

__device__ __forceinline__ void ldmatrix_x4(uint32_t address, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t address, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// (lo, hi) as f16 pair, and the f16 pair of what that rounding lost
__device__ __forceinline__ void split_half2(float lo, float hi, uint32_t& main, uint32_t& rest) {
    const __half2 h = __floats2half2_rn(lo, hi);
    const float2 back = __half22float2(h);
    main = *reinterpret_cast<const uint32_t*>(&h);
    rest = pack_half2(lo - back.x, hi - back.y);
}

__global__ void __launch_bounds__(kAttnWarps * 32, 3) attention_split_kernel(const float* __restrict__ q, const __half* __restrict__ k_cache,
                                                                             const __half* __restrict__ v_cache,
                                                                             const int* __restrict__ positions, float* __restrict__ part_o,
                                                                             float* __restrict__ part_ml, int q_heads, int kv_heads,
                                                                             long long max_context, int chunk, float scale, int active_context,
                                                                             int shared_cache, int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait_prior();   // inputs come from the kernels before this one in the stream
    extern __shared__ __align__(128) uint8_t attn_smem[];
    const int kv_head = blockIdx.x;
    const int member = blockIdx.y;
    const int split = blockIdx.z;
    const int splits = gridDim.z;
    const int group = q_heads / kv_heads;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;   // fragment coordinates: row g (and g + 8), column pair t
    // positions[] is device memory: the walk is clamped to the context the splits were planned for (at most the
    // cache size), and a position outside it is reported through the status word
    int tokens = positions[member] + 1;
    if (tokens < 1 || tokens > active_context) {
        if (threadIdx.x == 0 && split == 0 && kv_head == 0) atomicExch(status, kDevicePositionOutOfRange);
        tokens = max(0, min(tokens, active_context));
    }
    const int begin = split * chunk;
    const int end = min(tokens, begin + chunk);

    const long long sequence = shared_cache ? 0 : member;
    const __half* k_base = k_cache + (sequence * kv_heads + kv_head) * max_context * kAttnHeadDim;
    const __half* v_base = v_cache + (sequence * kv_heads + kv_head) * max_context * kAttnHeadDim;
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(attn_smem));

    // Tile loads: 64 tokens x 128 halves of K and of V, 16 bytes per request; rows past the range are zero-filled.
    auto request_tile = [&](int buffer, int t0) {
        const int valid = min(kAttnTile, end - t0);
        for (int i = threadIdx.x; i < kAttnTile * (kAttnHeadDim / 8); i += blockDim.x) {
            const int row = i / (kAttnHeadDim / 8);
            const int piece = i % (kAttnHeadDim / 8);
            const uint32_t kd = smem_base + (2 * buffer) * kAttnTileBytes + (row * kAttnKStride + 8 * piece) * 2;
            const uint32_t vd = kd + kAttnTileBytes;
            if (row < valid) {
                const __half* ks = k_base + static_cast<long long>(t0 + row) * kAttnHeadDim + 8 * piece;
                const __half* vs = v_base + static_cast<long long>(t0 + row) * kAttnHeadDim + 8 * piece;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(kd), "l"(ks) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vd), "l"(vs) : "memory");
            } else {
                asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(kd), "r"(0) : "memory");
                asm volatile("st.shared.v4.b32 [%0], {%1,%1,%1,%1};" ::"r"(vd), "r"(0) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (begin < end) request_tile(0, begin);   // in flight while the queries are fetched and split below

    // The group's queries as A fragments, times scale * log2(e) (the softmax runs on exp2), hi and lo parts: rows = heads
    // (rows from `group` on are zero), eight K steps of 16 dims.
    uint32_t q_hi[8][4], q_lo[8][4];
    {
        const float factor = scale * 1.4426950408889634f;
        const float* q_group = q + (static_cast<size_t>(member) * q_heads + static_cast<size_t>(kv_head) * group) * kAttnHeadDim;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
            for (int part = 0; part < 4; ++part) {
                const int row = g + 8 * (part & 1), column = 16 * ks + 2 * t + 8 * (part >> 1);
                float2 v = make_float2(0.0f, 0.0f);
                if (row < group) v = *reinterpret_cast<const float2*>(q_group + row * kAttnHeadDim + column);
                split_half2(v.x * factor, v.y * factor, q_hi[ks][part], q_lo[ks][part]);
            }
        }
    }

    float out[16][4];   // rows g, g + 8; dims 8 n + 2 t, + 1
#pragma unroll
    for (int n = 0; n < 16; ++n) out[n][0] = out[n][1] = out[n][2] = out[n][3] = 0.0f;
    float running_max[2] = {-INFINITY, -INFINITY}, running_sum[2] = {0.0f, 0.0f};
    // ldmatrix row addresses of this lane inside a tile: K as B operand (not transposed), V as B operand (transposed)
    const uint32_t k_lane = ((16 * warp + (lane & 7) + 8 * (lane >> 4)) * kAttnKStride + 8 * ((lane >> 3) & 1)) * 2;
    const uint32_t v_lane = ((16 * warp + (lane & 7) + 8 * ((lane >> 3) & 1)) * kAttnKStride + 8 * (lane >> 4)) * 2;

    int buffer = 0;
    for (int t0 = begin; t0 < end; t0 += kAttnTile, buffer ^= 1) {
        if (t0 + kAttnTile < end) {
            request_tile(buffer ^ 1, t0 + kAttnTile);   // its previous contents were consumed before the barrier that ended the last round
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();   // this tile has landed for every thread
        const int first = t0 + 16 * warp;    // this warp's sixteen tokens
        if (first < end) {
            const uint32_t k_tile = smem_base + (2 * buffer) * kAttnTileBytes, v_tile = k_tile + kAttnTileBytes;
            // scores: S[16 heads][16 tokens] = Q K^T, two n-tiles of eight tokens
            float s[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t b[4];   // (tokens 0-7: dims lo, hi), (tokens 8-15: dims lo, hi) of this K step
                ldmatrix_x4(k_tile + k_lane + 32 * ks, b);
                mma_f16(s[0], q_hi[ks], b[0], b[1]);
                mma_f16(s[1], q_hi[ks], b[2], b[3]);
                mma_f16(s[0], q_lo[ks], b[0], b[1]);
                mma_f16(s[1], q_lo[ks], b[2], b[3]);
            }
            // mask the tokens past the range, then the online softmax of rows g and g + 8
            const int valid = end - first;
#pragma unroll
            for (int n = 0; n < 2; ++n) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    if (8 * n + 2 * t + (c & 1) >= valid) s[n][c] = -INFINITY;
            }
            uint32_t p_hi[4], p_lo[4];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float tile_max = fmaxf(fmaxf(s[0][2 * r], s[0][2 * r + 1]), fmaxf(s[1][2 * r], s[1][2 * r + 1]));
                tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
                tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
                const float new_max = fmaxf(running_max[r], tile_max);   // finite: the warp has at least one valid token
                const float rescale = exp2f(running_max[r] - new_max);   // 0 the first time round
                running_max[r] = new_max;
                const float p0 = exp2f(s[0][2 * r] - new_max), p1 = exp2f(s[0][2 * r + 1] - new_max);
                const float p2 = exp2f(s[1][2 * r] - new_max), p3 = exp2f(s[1][2 * r + 1] - new_max);
                running_sum[r] = running_sum[r] * rescale + ((p0 + p1) + (p2 + p3));   // this lane's share; lanes are added at the end
#pragma unroll
                for (int n = 0; n < 16; ++n) {
                    out[n][2 * r] *= rescale;
                    out[n][2 * r + 1] *= rescale;
                }
                // A fragment of P: a[r] = tokens 2t, 2t+1 of row g + 8 r; a[2 + r] = tokens 8 + 2t, + 1
                split_half2(p0, p1, p_hi[r], p_lo[r]);
                split_half2(p2, p3, p_hi[2 + r], p_lo[2 + r]);
            }
            // O += P V: one K step of sixteen tokens, sixteen n-tiles of eight dims
#pragma unroll
            for (int pair = 0; pair < 8; ++pair) {
                uint32_t b[4];   // dims 16 pair .. + 7: (tokens 0-7, 8-15), dims 16 pair + 8 .. + 15: (tokens 0-7, 8-15)
                ldmatrix_x4_trans(v_tile + v_lane + 32 * pair, b);
                mma_f16(out[2 * pair], p_hi, b[0], b[1]);
                mma_f16(out[2 * pair + 1], p_hi, b[2], b[3]);
                mma_f16(out[2 * pair], p_lo, b[0], b[1]);
                mma_f16(out[2 * pair + 1], p_lo, b[2], b[3]);
            }
        }
        __syncthreads();   // every warp is done with this buffer before the next round refills it
    }

    // merge the four warps: [warp][row] maximum and sum, [warp][row][dim] output, in the tile buffers
    float* merge_o = reinterpret_cast<float*>(attn_smem);                        // [4][8][128]
    float* merge_m = merge_o + kAttnWarps * kAttnMaxGroup * kAttnHeadDim;         // [4][8]
    float* merge_l = merge_m + kAttnWarps * kAttnMaxGroup;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        running_sum[r] += __shfl_xor_sync(0xffffffffu, running_sum[r], 1);
        running_sum[r] += __shfl_xor_sync(0xffffffffu, running_sum[r], 2);
    }
    if (g < kAttnMaxGroup) {   // rows g + 8 are padding: at most eight heads share a KV head
        if (t == 0) {
            merge_m[warp * kAttnMaxGroup + g] = running_max[0];
            merge_l[warp * kAttnMaxGroup + g] = running_sum[0];
        }
#pragma unroll
        for (int n = 0; n < 16; ++n)
            *reinterpret_cast<float2*>(merge_o + (warp * kAttnMaxGroup + g) * kAttnHeadDim + 8 * n + 2 * t) = make_float2(out[n][0], out[n][1]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < group * kAttnHeadDim; i += blockDim.x) {
        const int row = i / kAttnHeadDim, dim = i % kAttnHeadDim;
        float top = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) top = fmaxf(top, merge_m[w * kAttnMaxGroup + row]);
        float total = 0.0f, value = 0.0f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float m = merge_m[w * kAttnMaxGroup + row];
            const float weight = m == -INFINITY ? 0.0f : exp2f(m - top);
            total = fmaf(merge_l[w * kAttnMaxGroup + row], weight, total);
            value = fmaf(merge_o[(w * kAttnMaxGroup + row) * kAttnHeadDim + dim], weight, value);
        }
        const size_t slot = (static_cast<size_t>(member) * q_heads + static_cast<size_t>(kv_head) * group + row) * splits + split;
        part_o[slot * kAttnHeadDim + dim] = value;
        if (dim == 0) {
            part_ml[slot * 2] = top * 0.6931471805599453f;   // back to natural-log units for the merge of the splits
            part_ml[slot * 2 + 1] = total;
        }
    }
}

// grid (q_heads, members), 128 threads: merges the splits of one query head.  Lane s of every warp holds split s (at most 32
// splits): the maximum, the sum and the weights come out of two warp reductions, and a thread then has sixteen partial rows
// of its output dimension in flight at a time.
template <bool OUT_BF16>
__global__ void __launch_bounds__(kAttnHeadDim) attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                                         void* __restrict__ out, int q_heads, int splits) {
    pdl_launch_dependents();
    pdl_wait_prior();   // inputs come from the kernels before this one in the stream
    const int lane = threadIdx.x & 31;
    const size_t base = (static_cast<size_t>(blockIdx.y) * q_heads + blockIdx.x) * splits;
    float m = -INFINITY, l = 0.0f;
    if (lane < splits) {
        const float2 ml = *reinterpret_cast<const float2*>(part_ml + (base + lane) * 2);
        m = ml.x;
        l = ml.y;
    }
    float global_max = m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) global_max = fmaxf(global_max, __shfl_xor_sync(0xffffffffu, global_max, o));
    const float weight = m == -INFINITY ? 0.0f : expf(m - global_max);
    float total = l * weight;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    const float* column = part_o + base * kAttnHeadDim + threadIdx.x;
    float value = 0.0f;
    for (int s0 = 0; s0 < splits; s0 += 16) {
        float part[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) part[u] = s0 + u < splits ? column[static_cast<size_t>(s0 + u) * kAttnHeadDim] : 0.0f;
#pragma unroll
        for (int u = 0; u < 16; ++u) value = fmaf(part[u], __shfl_sync(0xffffffffu, weight, (s0 + u) & 31), value);
    }
    const size_t index = (static_cast<size_t>(blockIdx.y) * q_heads + blockIdx.x) * kAttnHeadDim + threadIdx.x;
    if constexpr (OUT_BF16) static_cast<__nv_bfloat16*>(out)[index] = __float2bfloat16_rn(value / total);
    else static_cast<float*>(out)[index] = value / total;
}

// ---------------------------------------------------------------- elementwise
// out[m][i] = silu(gate[m][i]) * up[m][i]; gate and up rows are `in_stride` floats apart (they may be the two
// halves of one [members][2 * length] GEMV output), out rows are `length` apart.
template <bool OUT_BF16>
__global__ void __launch_bounds__(256) silu_mul_kernel(const float* __restrict__ gate, const float* __restrict__ up, void* __restrict__ out,
                                                       unsigned long long length, unsigned long long in_stride, unsigned long long total) {
    pdl_launch_dependents();
    pdl_wait_prior();   // inputs come from the kernels before this one in the stream
    for (unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
        const unsigned long long member = i / length;
        const unsigned long long column = i - member * length;
        const float value = gate[member * in_stride + column];
        const float product = (value / (1.0f + expf(-value))) * up[member * in_stride + column];
        if constexpr (OUT_BF16) static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(product);
        else static_cast<float*>(out)[i] = product;
    }
}

__global__ void __launch_bounds__(256) residual_add_kernel(float* __restrict__ y, const float* __restrict__ x, unsigned long long total) {
    pdl_launch_dependents();
    pdl_wait_prior();   // inputs come from the kernels before this one in the stream
    for (unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<unsigned long long>(gridDim.x) * blockDim.x)
        y[i] += x[i];
}

// ---------------------------------------------------------------- argmax
// One CTA per member.  NaN never wins, ties go to the lowest index, a row of NaNs gives 0 -- the reference's
// rules (model_ops.rs:201-258).  Keys are the monotone unsigned image of the floats.
__device__ __forceinline__ unsigned int logit_key(float value) {
    const unsigned int bits = __float_as_uint(value);
    return (bits >> 31) ? ~bits : (bits ^ 0x80000000u);
}

__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, unsigned int* __restrict__ out, unsigned long long length) {
    pdl_launch_dependents();
    pdl_wait_prior();   // inputs come from the kernels before this one in the stream
    __shared__ unsigned int keys[32];
    __shared__ unsigned int indices[32];
    const float* row = logits + static_cast<size_t>(blockIdx.x) * length;
    unsigned int key = 0u, index = 0u;
    for (unsigned long long i = threadIdx.x; i < length; i += blockDim.x) {
        const float candidate = row[i];
        const unsigned int candidate_key = logit_key(candidate);
        if (candidate == candidate && candidate_key > key) {
            key = candidate_key;
            index = static_cast<unsigned int>(i);
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned int other_key = __shfl_down_sync(0xffffffffu, key, o);
        const unsigned int other_index = __shfl_down_sync(0xffffffffu, index, o);
        if (other_key > key || (other_key == key && other_index < index)) {
            key = other_key;
            index = other_index;
        }
    }
    if (lane == 0) {
        keys[warp] = key;
        indices[warp] = index;
    }
    __syncthreads();
    if (warp == 0) {
        key = lane < static_cast<int>(blockDim.x >> 5) ? keys[lane] : 0u;
        index = lane < static_cast<int>(blockDim.x >> 5) ? indices[lane] : 0u;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned int other_key = __shfl_down_sync(0xffffffffu, key, o);
            const unsigned int other_index = __shfl_down_sync(0xffffffffu, index, o);
            if (other_key > key || (other_key == key && other_index < index)) {
                key = other_key;
                index = other_index;
            }
        }
        if (lane == 0) out[blockIdx.x] = index;
    }
}

}  // namespace

cudaError_t launch_embedding(const uint8_t* weights, uint32_t value_type, int k, unsigned int vocabulary, const uint32_t* tokens,
                             int members, float* out, cudaStream_t stream) {
    const int nsb = k / kSuperBlock;
    const dim3 grid((nsb + 7) / 8, members);
    const unsigned long long blocks_per_row = value_type == kQ8_0 ? k / 32 : nsb;
    switch (value_type) {
        case kQ4_K: return launch_kernel_if(pdl_switch() == 1, embedding_kernel<kQ4_K>, grid, dim3(256), 0, stream, weights, tokens, out, k, vocabulary, blocks_per_row * 144ull, nsb);
        case kQ5_K: return launch_kernel_if(pdl_switch() == 1, embedding_kernel<kQ5_K>, grid, dim3(256), 0, stream, weights, tokens, out, k, vocabulary, blocks_per_row * 176ull, nsb);
        case kQ6_K: return launch_kernel_if(pdl_switch() == 1, embedding_kernel<kQ6_K>, grid, dim3(256), 0, stream, weights, tokens, out, k, vocabulary, blocks_per_row * 210ull, nsb);
        case kQ8_0: return launch_kernel_if(pdl_switch() == 1, embedding_kernel<kQ8_0>, grid, dim3(256), 0, stream, weights, tokens, out, k, vocabulary, blocks_per_row * 34ull, nsb);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_qk_norm_rope_append(const LayerAttentionArgs& a) {
    const dim3 grid(a.q_heads + 2 * a.kv_heads, a.members);
    return launch_kernel_if(pdl_switch() == 1, qk_norm_rope_append_kernel, grid, dim3(a.head_dim), 0, a.stream, a.q, a.k, a.v, a.q_norm, a.k_norm, a.eps, a.positions,
                         a.q_heads, a.kv_heads, a.head_dim, a.rot_dims / 2, a.rope_base, static_cast<__half*>(a.k_cache),
                         static_cast<__half*>(a.v_cache), a.max_context, a.shared_cache ? 1 : 0, a.device_status);
}

int attention_splits(int members, int kv_heads, long long active_context, int sm_count) {
    // About eight CTAs per SM: a CTA walks its tiles one after the other, so the memory latency is hidden by
    // the CTAs that share its SM.
    int splits = (8 * sm_count) / (members * kv_heads);
    if (splits < 1) splits = 1;
    if (splits > 32) splits = 32;
    const long long tiles = (active_context + kAttnTile - 1) / kAttnTile;
    if (splits > tiles) splits = static_cast<int>(tiles < 1 ? 1 : tiles);
    return splits;
}

size_t attention_scratch_bytes(int members, int q_heads, int splits) {
    return static_cast<size_t>(members) * q_heads * splits * (kAttnHeadDim + 2) * sizeof(float);
}

cudaError_t launch_attention_decode(const LayerAttentionArgs& a, void* out, bool out_bf16, void* scratch, int splits) {
    if (a.head_dim != kAttnHeadDim || a.q_heads % a.kv_heads != 0 || a.q_heads / a.kv_heads > kAttnMaxGroup) return cudaErrorInvalidValue;
    const int group = a.q_heads / a.kv_heads;
    long long chunk = (a.active_context + splits - 1) / splits;
    chunk = (chunk + kAttnTile - 1) / kAttnTile * kAttnTile;
    float* part_o = static_cast<float*>(scratch);
    float* part_ml = part_o + static_cast<size_t>(a.members) * a.q_heads * splits * kAttnHeadDim;
    const float scale = 1.0f / sqrtf(static_cast<float>(a.head_dim));
    static int configured_device = -1;
    int device = 0;
    cudaGetDevice(&device);
    if (configured_device != device) {
        const cudaError_t attribute = cudaFuncSetAttribute(attention_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmemBytes);
        if (attribute != cudaSuccess) return attribute;
        configured_device = device;
    }
    cudaError_t e = launch_kernel_if(pdl_switch() == 1, attention_split_kernel, dim3(a.kv_heads, a.members, splits), dim3(kAttnWarps * 32), kAttnSmemBytes, a.stream,
                                  static_cast<const float*>(a.q), static_cast<const __half*>(a.k_cache), static_cast<const __half*>(a.v_cache),
                                  a.positions, part_o, part_ml, a.q_heads, a.kv_heads, a.max_context, static_cast<int>(chunk), scale,
                                  static_cast<int>(a.active_context), a.shared_cache ? 1 : 0, a.device_status);
    if (e != cudaSuccess) return e;
    if (out_bf16)
        return launch_kernel_if(pdl_switch() == 1, attention_combine_kernel<true>, dim3(a.q_heads, a.members), dim3(kAttnHeadDim), 0, a.stream,
                                static_cast<const float*>(part_o), static_cast<const float*>(part_ml), out, a.q_heads, splits);
    return launch_kernel_if(pdl_switch() == 1, attention_combine_kernel<false>, dim3(a.q_heads, a.members), dim3(kAttnHeadDim), 0, a.stream,
                            static_cast<const float*>(part_o), static_cast<const float*>(part_ml), out, a.q_heads, splits);
}

cudaError_t launch_silu_mul(const float* gate, const float* up, void* out, bool out_bf16, uint64_t members, uint64_t length, uint64_t in_stride,
                            int sm_count, cudaStream_t stream) {
    const unsigned long long total = members * length;
    unsigned long long blocks = (total + 255) / 256;
    if (blocks > static_cast<unsigned long long>(sm_count) * 8) blocks = static_cast<unsigned long long>(sm_count) * 8;
    const dim3 grid(static_cast<unsigned>(blocks ? blocks : 1));
    if (out_bf16)
        return launch_kernel_if(pdl_switch() == 1, silu_mul_kernel<true>, grid, dim3(256), 0, stream, gate, up, out,
                                static_cast<unsigned long long>(length), static_cast<unsigned long long>(in_stride), total);
    return launch_kernel_if(pdl_switch() == 1, silu_mul_kernel<false>, grid, dim3(256), 0, stream, gate, up, out,
                            static_cast<unsigned long long>(length), static_cast<unsigned long long>(in_stride), total);
}

cudaError_t launch_residual_add(float* y, const float* x, uint64_t total, int sm_count, cudaStream_t stream) {
    unsigned long long blocks = (total + 255) / 256;
    if (blocks > static_cast<unsigned long long>(sm_count) * 8) blocks = static_cast<unsigned long long>(sm_count) * 8;
    return launch_kernel_if(pdl_switch() == 1, residual_add_kernel, dim3(static_cast<unsigned>(blocks ? blocks : 1)), dim3(256), 0, stream, y, x,
                         static_cast<unsigned long long>(total));
}

cudaError_t launch_argmax(const float* logits, int members, uint64_t length, uint32_t* out, cudaStream_t stream) {
    return launch_kernel_if(pdl_switch() == 1, argmax_kernel, dim3(members), dim3(1024), 0, stream, logits, out, static_cast<unsigned long long>(length));
}

}  // namespace ribn
