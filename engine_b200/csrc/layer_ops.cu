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
// Split-KV ("flash decoding"): grid (kv_heads, members, splits); warp w of the CTA owns query head
// kv_head * group + w.  The CTA walks its token range in tiles of 32: the K and V tiles go through shared
// memory once for the whole group; lane = token for the scores, lane = 4 output dims for P.V.
constexpr int kAttnTile = 32;
constexpr int kAttnHeadDim = 128;
constexpr int kAttnKStride = kAttnHeadDim + 8;   // halves; rows 272 bytes apart: the 16-byte loads of eight lanes cover all banks once
constexpr int kAttnMaxGroup = 8;

__global__ void __launch_bounds__(kAttnMaxGroup * 32) attention_split_kernel(const float* __restrict__ q, const __half* __restrict__ k_cache,
                                                                             const __half* __restrict__ v_cache,
                                                                             const int* __restrict__ positions, float* __restrict__ part_o,
                                                                             float* __restrict__ part_ml, int q_heads, int kv_heads,
                                                                             long long max_context, int chunk, float scale, int active_context,
                                                                             int shared_cache, int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait_prior();   // inputs come from the kernels before this one in the stream
    // Two tiles of each: the next one streams in (cp.async) while the warps work on the current one.
    __shared__ __align__(16) __half k_tiles[2][kAttnTile * kAttnKStride];
    __shared__ __align__(16) __half v_tiles[2][kAttnTile * kAttnHeadDim];
    __shared__ __align__(16) float q_rows[kAttnMaxGroup * kAttnHeadDim];
    const int kv_head = blockIdx.x;
    const int member = blockIdx.y;
    const int split = blockIdx.z;
    const int splits = gridDim.z;
    const int group = q_heads / kv_heads;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int q_head = kv_head * group + warp;
    // positions[] is device memory: the walk is clamped to the context the splits were planned for (at most the
    // cache size), and a position outside it is reported through the status word
    int tokens = positions[member] + 1;
    if (tokens < 1 || tokens > active_context) {
        if (threadIdx.x == 0 && split == 0 && kv_head == 0) atomicExch(status, kDevicePositionOutOfRange);
        tokens = max(0, min(tokens, active_context));
    }
    const int begin = split * chunk;
    const int end = min(tokens, begin + chunk);

    for (int i = threadIdx.x; i < group * kAttnHeadDim; i += blockDim.x)
        q_rows[i] = q[(static_cast<size_t>(member) * q_heads + kv_head * group) * kAttnHeadDim + i];

    const long long sequence = shared_cache ? 0 : member;
    const __half* k_base = k_cache + (sequence * kv_heads + kv_head) * max_context * kAttnHeadDim;
    const __half* v_base = v_cache + (sequence * kv_heads + kv_head) * max_context * kAttnHeadDim;
    float running_max = -INFINITY, running_sum = 0.0f;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};

    // Tile loads: 32 tokens x 128 halves each, 16 bytes per request; rows past the range are zero-filled.
    auto request_tile = [&](int buffer, int t0) {
        const int valid = min(kAttnTile, end - t0);
        for (int i = threadIdx.x; i < kAttnTile * (kAttnHeadDim / 8); i += blockDim.x) {
            const int row = i / (kAttnHeadDim / 8);
            const int chunk = i % (kAttnHeadDim / 8);
            __half* kd = k_tiles[buffer] + row * kAttnKStride + 8 * chunk;
            __half* vd = v_tiles[buffer] + row * kAttnHeadDim + 8 * chunk;
            if (row < valid) {
                const __half* ks = k_base + static_cast<long long>(t0 + row) * kAttnHeadDim + 8 * chunk;
                const __half* vs = v_base + static_cast<long long>(t0 + row) * kAttnHeadDim + 8 * chunk;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(kd))), "l"(ks) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(vd))), "l"(vs) : "memory");
            } else {
                *reinterpret_cast<uint4*>(kd) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(vd) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (begin < end) request_tile(0, begin);

    int buffer = 0;
    for (int t0 = begin; t0 < end; t0 += kAttnTile, buffer ^= 1) {
        const int valid = min(kAttnTile, end - t0);
        if (t0 + kAttnTile < end) {
            request_tile(buffer ^ 1, t0 + kAttnTile);   // its previous contents were consumed before the barrier that ended the last round
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();   // this tile has landed for every thread (and q_rows is written, first time round)
        const __half* k_tile = k_tiles[buffer];
        const __half* v_tile = v_tiles[buffer];
        if (warp < group) {
            // scores: lane = token of the tile
            const float* qv = q_rows + warp * kAttnHeadDim;
            const __half* kr = k_tile + lane * kAttnKStride;
            float dot = 0.0f;
#pragma unroll 4
            for (int d = 0; d < kAttnHeadDim; d += 8) {
                const uint4 raw = *reinterpret_cast<const uint4*>(kr + d);
                const float4 q0 = *reinterpret_cast<const float4*>(qv + d);
                const float4 q1 = *reinterpret_cast<const float4*>(qv + d + 4);
                const float2 k01 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                const float2 k23 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                const float2 k45 = __half22float2(*reinterpret_cast<const __half2*>(&raw.z));
                const float2 k67 = __half22float2(*reinterpret_cast<const __half2*>(&raw.w));
                dot = fmaf(q0.x, k01.x, dot);
                dot = fmaf(q0.y, k01.y, dot);
                dot = fmaf(q0.z, k23.x, dot);
                dot = fmaf(q0.w, k23.y, dot);
                dot = fmaf(q1.x, k45.x, dot);
                dot = fmaf(q1.y, k45.y, dot);
                dot = fmaf(q1.z, k67.x, dot);
                dot = fmaf(q1.w, k67.y, dot);
            }
            const float score = lane < valid ? dot * scale : -INFINITY;
            float tile_max = score;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, o));
            const float new_max = fmaxf(running_max, tile_max);
            const float p = lane < valid ? expf(score - new_max) : 0.0f;
            float tile_sum = p;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tile_sum += __shfl_xor_sync(0xffffffffu, tile_sum, o);
            const float rescale = running_max == -INFINITY ? 0.0f : expf(running_max - new_max);
            running_sum = running_sum * rescale + tile_sum;
            running_max = new_max;
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] *= rescale;
            // P.V: lane = output dims 4*lane .. 4*lane+3
            for (int tk = 0; tk < valid; ++tk) {
                const float pt = __shfl_sync(0xffffffffu, p, tk);
                const uint2 raw = *reinterpret_cast<const uint2*>(v_tile + tk * kAttnHeadDim + 4 * lane);
                const float2 v01 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                const float2 v23 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                acc[0] = fmaf(pt, v01.x, acc[0]);
                acc[1] = fmaf(pt, v01.y, acc[1]);
                acc[2] = fmaf(pt, v23.x, acc[2]);
                acc[3] = fmaf(pt, v23.y, acc[3]);
            }
        }
        __syncthreads();   // every warp is done with this buffer before the next round refills it
    }
    if (warp < group) {
        const size_t slot = (static_cast<size_t>(member) * q_heads + q_head) * splits + split;
        *reinterpret_cast<float4*>(part_o + slot * kAttnHeadDim + 4 * lane) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        if (lane == 0) {
            part_ml[slot * 2] = running_max;
            part_ml[slot * 2 + 1] = running_sum;
        }
    }
}

// grid (q_heads, members), 128 threads: merges the splits of one query head.
template <bool OUT_BF16>
__global__ void __launch_bounds__(kAttnHeadDim) attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                                         void* __restrict__ out, int q_heads, int splits) {
    pdl_launch_dependents();
    pdl_wait_prior();   // inputs come from the kernels before this one in the stream
    const size_t base = (static_cast<size_t>(blockIdx.y) * q_heads + blockIdx.x) * splits;
    float global_max = -INFINITY;
    for (int s = 0; s < splits; ++s) global_max = fmaxf(global_max, part_ml[(base + s) * 2]);
    float total = 0.0f, value = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float m = part_ml[(base + s) * 2];
        const float weight = m == -INFINITY ? 0.0f : expf(m - global_max);
        total = fmaf(part_ml[(base + s) * 2 + 1], weight, total);
        value = fmaf(part_o[(base + s) * kAttnHeadDim + threadIdx.x], weight, value);
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
    cudaError_t e = launch_kernel_if(pdl_switch() == 1, attention_split_kernel, dim3(a.kv_heads, a.members, splits), dim3(group * 32), 0, a.stream,
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
