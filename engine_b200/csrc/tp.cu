// Tensor-parallel exchange steps of the decode loop over peer memory (NVLink), one launch each:
//
//   ribn_tp_allreduce_residual   hidden[m][h] += sum over ranks of partial_r[m][h]
//       replaces, after the column-split projections (o_proj, ffn_down), an all-reduce of the partial outputs and the
//       residual_add that follows it (crates/nvidia/src/model_ops.rs:600-610 of the reference project; the reference
//       runs on one GPU and has no counterpart of the exchange);
//   ribn_tp_select_tokens        the argmax of every member row over all ranks' slices of the vocabulary
//       with the rules of argmax / argmax_batch (model_ops.rs:201-314): NaN never wins, ties go to the lowest index.
//
// Every rank owns one block of device memory that its peers map (CUDA IPC between processes, plain peer pointers inside
// one process):
//   [partial slot 0][partial slot 1]   written by this rank's GEMV (it is the GEMV's output buffer), read by every rank
//   [flags: world words]               flags[p] = the last exchange rank p has published; written by rank p, polled here
//   [selection flags: world words]     the same for token selection
//   [selection pairs: 2 x 64 x (value bits, index)]
// and a few words only this rank touches (the exchange counters and the ticket of the last CTA).
//
// Protocol of one exchange e (a counter kept in device memory, so that a replayed CUDA graph advances it): a rank stores e
// into flags[rank] of every peer with a release at system scope -- its partial was written by the kernel before this one
// in the stream -- polls its own flags until every peer has published e (acquire; bounded: after `wait_ns` the kernel
// records a timeout in the context's status word, leaves `hidden` untouched and returns), then pulls each peer's partial
// with plain loads over NVLink, adds them in rank order (every rank computes bit-identical sums, so the replicated
// hidden state never drifts apart) and adds the residual.  Consecutive exchanges alternate between the two slots: a rank
// can be at most one exchange ahead of a peer (it needs the peer's flag for e + 1, which the peer stores only after its
// exchange e has completed), so a slot is never rewritten while somebody still reads it.
//
// No collective library, no switch-side reduction and no bulk-copy engine is involved: ordinary loads and stores on mapped
// peer memory.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstring>
#include <new>
#include <string>

#include "../../include/ribn_b200.h"
#include "internal.h"
#include "pipeline.cuh"

namespace {

constexpr uint32_t kMaxWorld = 8;
constexpr uint32_t kMaxSelectMembers = 64;
constexpr uint64_t kTailBytes = 4096;   // flags, pairs and counters behind the two slots

struct Tail {
    uint32_t flags[16];                        // written by the peers
    uint32_t select_flags[16];                 // written by the peers
    uint32_t pairs[2][kMaxSelectMembers][2];   // this rank's (value bits, global index) per member, two generations
    uint32_t epoch;                            // exchanges completed (local)
    uint32_t select_epoch;
    uint32_t ticket;
    uint32_t select_ticket;
};
static_assert(sizeof(Tail) <= kTailBytes, "tail layout");

struct Peers {
    uint8_t* block[kMaxWorld];
};

__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 load_peer16(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint2 load_peer8(const void* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long wall_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// One lane waits until every peer has published `epoch` in `flags` (this rank's own memory); false after wait_ns.
__device__ __forceinline__ bool wait_for_peers(const uint32_t* flags, uint32_t world, uint32_t rank, uint32_t epoch, unsigned long long wait_ns) {
    const unsigned long long start = wall_ns();
    for (uint32_t p = 0; p < world; ++p) {
        if (p == rank) continue;
        uint32_t spins = 0;
        while (static_cast<int32_t>(load_acquire_sys(flags + p) - epoch) < 0) {
            if ((++spins & 63u) == 0u && wall_ns() - start > wait_ns) return false;
        }
    }
    return true;
}

__device__ __forceinline__ unsigned int logit_key(float value) {
    const unsigned int bits = __float_as_uint(value);
    return (bits >> 31) ? ~bits : (bits ^ 0x80000000u);
}

// grid: CTAs of 256 threads over `total` = members * length values, four per thread and trip.
template <bool PARTIAL_BF16>
__global__ void __launch_bounds__(256) tp_allreduce_residual_kernel(Peers peers, uint32_t rank, uint32_t world, uint64_t slot_offset, uint64_t tail_offset,
                                                                    float* __restrict__ hidden, unsigned long long total, unsigned long long wait_ns,
                                                                    int* __restrict__ status) {
    ribn::pdl_launch_dependents();
    ribn::pdl_wait_prior();   // this rank's partial is the output of the kernel before this one
    __shared__ int arrived;
    Tail* tail = reinterpret_cast<Tail*>(peers.block[rank] + tail_offset);
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(&tail->epoch) + 1u;
    if (blockIdx.x == 0 && threadIdx.x < world && threadIdx.x != rank) {
        __threadfence_system();
        store_release_sys(&reinterpret_cast<Tail*>(peers.block[threadIdx.x] + tail_offset)->flags[rank], epoch);
    }
    if (threadIdx.x == 0) arrived = wait_for_peers(tail->flags, world, rank, epoch, wait_ns) ? 1 : 0;
    __syncthreads();
    if (arrived != 0) {
        const unsigned long long quads = total / 4;
        for (unsigned long long q = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x; q < quads;
             q += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
            float4 sum = reinterpret_cast<const float4*>(hidden)[q];
            // every load is issued before the first add; the adds run in rank order on every rank
            uint4 raw[kMaxWorld];
#pragma unroll
            for (uint32_t p = 0; p < kMaxWorld; ++p) {
                if (p >= world) break;
                const uint8_t* slot = peers.block[p] + slot_offset;
                if (PARTIAL_BF16) {
                    const uint2 half = load_peer8(slot + q * 8);
                    raw[p] = make_uint4(half.x, half.y, 0u, 0u);
                } else {
                    raw[p] = load_peer16(slot + q * 16);
                }
            }
#pragma unroll
            for (uint32_t p = 0; p < kMaxWorld; ++p) {
                if (p >= world) break;
                if (PARTIAL_BF16) {
                    sum.x += __uint_as_float(raw[p].x << 16);
                    sum.y += __uint_as_float(raw[p].x & 0xffff0000u);
                    sum.z += __uint_as_float(raw[p].y << 16);
                    sum.w += __uint_as_float(raw[p].y & 0xffff0000u);
                } else {
                    sum.x += __uint_as_float(raw[p].x);
                    sum.y += __uint_as_float(raw[p].y);
                    sum.z += __uint_as_float(raw[p].z);
                    sum.w += __uint_as_float(raw[p].w);
                }
            }
            reinterpret_cast<float4*>(hidden)[q] = sum;
        }
    } else if (threadIdx.x == 0) {
        atomicExch(status, ribn::kDeviceWaitTimeout);
    }
    // the last CTA to get here closes the exchange: every CTA has read the counter by then
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&tail->ticket, 1u) == gridDim.x - 1) {
            tail->ticket = 0u;
            *reinterpret_cast<volatile uint32_t*>(&tail->epoch) = epoch;
        }
    }
}

// grid: one CTA of 1024 threads per member.  The CTA finds the best (value, index) of its member over this rank's logits
// and leaves it in the rank's block; the last CTA to do so publishes the generation to the peers; every CTA then waits for
// the peers' generations and picks the winner of its member among the ranks' pairs, in rank order.
__global__ void __launch_bounds__(1024) tp_select_tokens_kernel(Peers peers, uint32_t rank, uint32_t world, uint64_t tail_offset,
                                                                const float* __restrict__ logits, unsigned long long length, unsigned int index_base,
                                                                unsigned int* __restrict__ out, unsigned long long wait_ns, int* __restrict__ status) {
    ribn::pdl_launch_dependents();
    ribn::pdl_wait_prior();
    __shared__ unsigned int keys[32];
    __shared__ unsigned int indices[32];
    __shared__ int arrived;
    Tail* tail = reinterpret_cast<Tail*>(peers.block[rank] + tail_offset);
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(&tail->select_epoch) + 1u;
    const uint32_t generation = epoch & 1u;
    const uint32_t member = blockIdx.x;
    const float* row = logits + static_cast<size_t>(member) * length;
    unsigned int key = 0u, index = 0u;   // key 0 is below every number's key: a row of NaNs keeps (0, first index)
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
    if (threadIdx.x == 0) {
        for (int w = 1; w < 32; ++w)
            if (keys[w] > key || (keys[w] == key && indices[w] < index)) {
                key = keys[w];
                index = indices[w];
            }
        volatile uint32_t* pair = tail->pairs[generation][member];
        pair[0] = key;
        pair[1] = index_base + index;
        __threadfence_system();
        if (atomicAdd(&tail->select_ticket, 1u) == gridDim.x - 1) {
            tail->select_ticket = 0u;
            __threadfence_system();   // the other CTAs' pairs, observed through the ticket, go out before the flag
            for (uint32_t p = 0; p < world; ++p)
                if (p != rank) store_release_sys(&reinterpret_cast<Tail*>(peers.block[p] + tail_offset)->select_flags[rank], epoch);
            store_release_sys(&tail->select_flags[rank], epoch);   // this rank's own CTAs wait for it too
        }
        // every rank, this one included, must have published the generation
        const unsigned long long start = wall_ns();
        bool ok = true;
        for (uint32_t p = 0; p < world && ok; ++p) {
            uint32_t spins = 0;
            while (static_cast<int32_t>(load_acquire_sys(tail->select_flags + p) - epoch) < 0) {
                if ((++spins & 63u) == 0u && wall_ns() - start > wait_ns) {
                    ok = false;
                    break;
                }
            }
        }
        if (ok) {
            unsigned int best_key = 0u, best_index = 0u;
            bool first = true;
            for (uint32_t p = 0; p < world; ++p) {
                const uint2 pair_p = load_peer8(reinterpret_cast<Tail*>(peers.block[p] + tail_offset)->pairs[generation][member]);
                if (first || pair_p.x > best_key || (pair_p.x == best_key && pair_p.y < best_index)) {
                    best_key = pair_p.x;
                    best_index = pair_p.y;
                    first = false;
                }
            }
            // a member whose logits are NaN on every rank: index 0, as on one GPU
            out[member] = best_key == 0u ? 0u : best_index;
        } else {
            atomicExch(status, ribn::kDeviceWaitTimeout);
        }
        arrived = ok ? 1 : 0;
    }
    __syncthreads();
    // the last CTA closes the generation; CTAs count twice on the ticket's upper half to keep the two phases apart
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&tail->select_ticket, 0x10000u) == ((gridDim.x - 1) << 16)) {
            tail->select_ticket = 0u;
            *reinterpret_cast<volatile uint32_t*>(&tail->select_epoch) = epoch;
        }
    }
}

}  // namespace

struct ribn_tp {
    int device = 0;
    uint32_t rank = 0, world = 1;
    uint64_t slot_bytes = 0, block_bytes = 0;
    uint8_t* block = nullptr;      // this rank's
    bool owns_block = false;
    Peers peers{};
    bool opened[kMaxWorld] = {};   // peers mapped through IPC handles (to be closed)
    bool connected = false;
    uint64_t wait_ns = 1000000000ull;
    std::string message;
};

extern "C" {

int ribn_tp_create(ribn_ctx* ctx, uint32_t rank, uint32_t world, uint64_t slot_bytes, void* local_block, ribn_tp** out) {
    if (ctx == nullptr || out == nullptr) return RIBN_E_INVALID_ARGUMENT;
    *out = nullptr;
    if (world < 1 || world > kMaxWorld || rank >= world || slot_bytes == 0 || slot_bytes % 256 != 0) return RIBN_E_INVALID_ARGUMENT;
    ribn_tp* tp = new (std::nothrow) ribn_tp();
    if (tp == nullptr) return RIBN_E_DRIVER;
    void* stream = nullptr;
    ribn_context_stream(ctx, &tp->device, &stream);
    tp->rank = rank;
    tp->world = world;
    tp->slot_bytes = slot_bytes;
    tp->block_bytes = 2 * slot_bytes + kTailBytes;
    int previous = 0;
    cudaGetDevice(&previous);
    cudaSetDevice(tp->device);
    cudaError_t e = cudaSuccess;
    if (local_block != nullptr) {
        tp->block = static_cast<uint8_t*>(local_block);   // caller's memory (same-process peers, tests): block_bytes of it, 256-byte aligned
        if ((reinterpret_cast<uintptr_t>(local_block) & 255u) != 0) e = cudaErrorInvalidValue;
    } else {
        e = cudaMalloc(reinterpret_cast<void**>(&tp->block), tp->block_bytes);   // a whole allocation: exportable through IPC
        tp->owns_block = e == cudaSuccess;
    }
    if (e == cudaSuccess) e = cudaMemset(tp->block, 0, tp->block_bytes);
    cudaSetDevice(previous);
    if (e != cudaSuccess) {
        if (tp->owns_block) cudaFree(tp->block);
        delete tp;
        return RIBN_E_DRIVER;
    }
    tp->peers.block[rank] = tp->block;
    tp->connected = world == 1;
    *out = tp;
    return RIBN_OK;
}

void ribn_tp_destroy(ribn_tp* tp) {
    if (tp == nullptr) return;
    int previous = 0;
    cudaGetDevice(&previous);
    cudaSetDevice(tp->device);
    for (uint32_t p = 0; p < tp->world; ++p)
        if (tp->opened[p]) cudaIpcCloseMemHandle(tp->peers.block[p]);
    if (tp->owns_block) cudaFree(tp->block);
    cudaSetDevice(previous);
    delete tp;
}

const char* ribn_tp_last_error(const ribn_tp* tp) { return tp != nullptr ? tp->message.c_str() : ""; }

uint64_t ribn_tp_block_bytes(uint64_t slot_bytes) { return 2 * slot_bytes + kTailBytes; }

int ribn_tp_export(ribn_tp* tp, void* handle_out) {
    if (tp == nullptr || handle_out == nullptr) return RIBN_E_INVALID_ARGUMENT;
    if (!tp->owns_block) {
        tp->message = "a caller-supplied block is connected by pointers, not by handles";
        return RIBN_E_INVALID_ARGUMENT;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == RIBN_TP_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t handle;
    int previous = 0;
    cudaGetDevice(&previous);
    cudaSetDevice(tp->device);
    const cudaError_t e = cudaIpcGetMemHandle(&handle, tp->block);
    cudaSetDevice(previous);
    if (e != cudaSuccess) {
        tp->message = std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e);
        return RIBN_E_DRIVER;
    }
    std::memcpy(handle_out, &handle, sizeof handle);
    return RIBN_OK;
}

int ribn_tp_connect(ribn_tp* tp, const void* handles) {
    if (tp == nullptr || handles == nullptr) return RIBN_E_INVALID_ARGUMENT;
    int previous = 0;
    cudaGetDevice(&previous);
    cudaSetDevice(tp->device);
    int result = RIBN_OK;
    for (uint32_t p = 0; p < tp->world && result == RIBN_OK; ++p) {
        if (p == tp->rank || tp->opened[p]) continue;
        cudaIpcMemHandle_t handle;
        std::memcpy(&handle, static_cast<const uint8_t*>(handles) + static_cast<size_t>(p) * RIBN_TP_HANDLE_BYTES, sizeof handle);
        void* mapped = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&mapped, handle, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            tp->message = std::string("cudaIpcOpenMemHandle (rank ") + std::to_string(p) + "): " + cudaGetErrorString(e);
            result = RIBN_E_DRIVER;
        } else {
            tp->peers.block[p] = static_cast<uint8_t*>(mapped);
            tp->opened[p] = true;
        }
    }
    cudaSetDevice(previous);
    tp->connected = result == RIBN_OK;
    return result;
}

int ribn_tp_connect_pointers(ribn_tp* tp, void* const* blocks) {
    if (tp == nullptr || blocks == nullptr) return RIBN_E_INVALID_ARGUMENT;
    for (uint32_t p = 0; p < tp->world; ++p) {
        if (p == tp->rank) continue;
        if (blocks[p] == nullptr) return RIBN_E_INVALID_ARGUMENT;
        tp->peers.block[p] = static_cast<uint8_t*>(blocks[p]);
    }
    tp->connected = true;
    return RIBN_OK;
}

int ribn_tp_set_wait(ribn_tp* tp, uint64_t microseconds) {
    if (tp == nullptr || microseconds == 0 || microseconds > 10000000ull) return RIBN_E_INVALID_ARGUMENT;
    tp->wait_ns = microseconds * 1000ull;
    return RIBN_OK;
}

int ribn_tp_partial(ribn_tp* tp, uint32_t slot, void** device_pointer) {
    if (tp == nullptr || device_pointer == nullptr || slot > 1) return RIBN_E_INVALID_ARGUMENT;
    *device_pointer = tp->block + static_cast<uint64_t>(slot) * tp->slot_bytes;
    return RIBN_OK;
}

int ribn_tp_allreduce_residual(ribn_ctx* ctx, ribn_tp* tp, uint32_t slot, float* hidden_device, uint32_t members, uint64_t length,
                               int partial_dtype) {
    if (ctx == nullptr || tp == nullptr || hidden_device == nullptr || slot > 1) return RIBN_E_INVALID_ARGUMENT;
    if (!tp->connected) {
        tp->message = "peers are not connected";
        return RIBN_E_INVALID_ARGUMENT;
    }
    if (partial_dtype != RIBN_F32 && partial_dtype != RIBN_BF16) return RIBN_E_INVALID_ARGUMENT;
    const uint64_t total = static_cast<uint64_t>(members) * length;
    if (total == 0 || total % 4 != 0 || total * (partial_dtype == RIBN_BF16 ? 2 : 4) > tp->slot_bytes ||
        (reinterpret_cast<uintptr_t>(hidden_device) & 15u) != 0) {
        tp->message = "members * length must be a positive multiple of four that fits a slot, hidden 16-byte aligned";
        return RIBN_E_INVALID_ARGUMENT;
    }
    int device = 0, sm_count = 0;
    void* stream = nullptr;
    int* status = nullptr;
    ribn::context_internals(ctx, &device, &stream, &sm_count, &status);
    int previous = 0;
    cudaGetDevice(&previous);
    cudaSetDevice(device);
    // One group of four values per thread where the grid allows it: all of a rank's loads from its peers are then in flight
    // in one round trip over NVLink (no CTA waits for another CTA of this launch, so the grid may exceed what is resident).
    unsigned long long ctas = (total / 4 + 255) / 256;
    if (ctas > 4ull * static_cast<unsigned long long>(sm_count)) ctas = 4ull * static_cast<unsigned long long>(sm_count);
    const dim3 grid(static_cast<unsigned>(ctas));
    const uint64_t slot_offset = static_cast<uint64_t>(slot) * tp->slot_bytes, tail_offset = 2 * tp->slot_bytes;
    cudaError_t e;
    if (partial_dtype == RIBN_BF16)
        e = ribn::launch_kernel(tp_allreduce_residual_kernel<true>, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), tp->peers, tp->rank, tp->world,
                                slot_offset, tail_offset, hidden_device, static_cast<unsigned long long>(total),
                                static_cast<unsigned long long>(tp->wait_ns), status);
    else
        e = ribn::launch_kernel(tp_allreduce_residual_kernel<false>, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), tp->peers, tp->rank, tp->world,
                                slot_offset, tail_offset, hidden_device, static_cast<unsigned long long>(total),
                                static_cast<unsigned long long>(tp->wait_ns), status);
    cudaSetDevice(previous);
    if (e != cudaSuccess) {
        tp->message = std::string("exchange launch: ") + cudaGetErrorString(e);
        return RIBN_E_DRIVER;
    }
    return RIBN_OK;
}

int ribn_tp_select_tokens(ribn_ctx* ctx, ribn_tp* tp, const float* logits_device, uint32_t members, uint64_t length, uint32_t index_base,
                          uint32_t* tokens_device) {
    if (ctx == nullptr || tp == nullptr || logits_device == nullptr || tokens_device == nullptr) return RIBN_E_INVALID_ARGUMENT;
    if (!tp->connected || members == 0 || members > kMaxSelectMembers || length == 0 || length > 0xffffffffull) {
        tp->message = "token selection serves 1..64 members over connected peers";
        return RIBN_E_INVALID_ARGUMENT;
    }
    int device = 0, sm_count = 0;
    void* stream = nullptr;
    int* status = nullptr;
    ribn::context_internals(ctx, &device, &stream, &sm_count, &status);
    if (static_cast<int>(members) > sm_count) return RIBN_E_INVALID_ARGUMENT;   // every CTA must be resident: they wait for the last one
    int previous = 0;
    cudaGetDevice(&previous);
    cudaSetDevice(device);
    const cudaError_t e = ribn::launch_kernel(tp_select_tokens_kernel, dim3(members), dim3(1024), 0, static_cast<cudaStream_t>(stream), tp->peers, tp->rank,
                                              tp->world, 2 * tp->slot_bytes, logits_device, static_cast<unsigned long long>(length), index_base, tokens_device,
                                              static_cast<unsigned long long>(tp->wait_ns), status);
    cudaSetDevice(previous);
    if (e != cudaSuccess) {
        tp->message = std::string("token selection launch: ") + cudaGetErrorString(e);
        return RIBN_E_DRIVER;
    }
    return RIBN_OK;
}

}  // extern "C"
