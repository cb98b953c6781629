// tcgen05 / TMEM / tiled-TMA primitives for sm_100a as inline PTX.
//
// Descriptor bit layouts follow the public CUTLASS/CuTe sm100 headers
// (cute/arch/mma_sm100_desc.hpp): the shared-memory matrix descriptor and the
// 32-bit instruction descriptor of kind::f16.
#pragma once

#include <cuda.h>
#include <stdint.h>

#include "pipeline.cuh"

namespace ribn {

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes
// (64 16-bit elements) stored with the 128-byte swizzle: rows of one 8-row
// group are 128 bytes apart, groups are 1024 bytes apart (SBO), and the 16-byte
// chunk index inside a row is XORed with (row % 8).  The tile base must be
// 1024-byte aligned.
//   bits [0,14)  start address >> 4        bits [32,46) stride byte offset >> 4
//   bits [16,30) leading byte offset >> 4 (unused for swizzled K-major, 1)
//   bits [46,48) descriptor version = 1    bits [61,64) layout type, 2 = SWIZZLE_128B
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t smem_byte_addr) {
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((smem_byte_addr & 0x3ffffu) >> 4);
    desc |= static_cast<uint64_t>(1) << 16;
    desc |= static_cast<uint64_t>(1024 >> 4) << 32;
    desc |= static_cast<uint64_t>(1) << 46;
    desc |= static_cast<uint64_t>(2) << 61;
    return desc;
}

// Instruction descriptor, kind::f16, f32 accumulate, both operands K-major.
//   bits [4,6)  D format: 1 = f32          bits [7,10)  A format: 0 = f16, 1 = bf16
//   bits [10,13) B format                   bit 15 / 16  A / B major: 0 = K
//   bits [17,23) N >> 3                     bits [24,29) M >> 4
__host__ __device__ constexpr uint32_t umma_instr_desc(int m, int n, int a_format, int b_format) {
    return (1u << 4) | (static_cast<uint32_t>(a_format) << 7) | (static_cast<uint32_t>(b_format) << 10) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
    const uint32_t acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
        : "memory");
}

// The MMAs of one 64-wide K step (four K slices of 16 elements, 32 bytes apart along the swizzled rows,
// i.e. +2 in the descriptors' address field), issued by the elected lane of a CONVERGED warp: every lane
// executes this, so that the operands stay warp-uniform; issued from inside a one-lane branch instead,
// each tcgen05.mma costs its thread about twice as long (measured: ~80 cycles against ~40, and up to 125
// when other warps keep the ALUs busy).  `accumulate_first` = 0 makes the first slice overwrite D.
__device__ __forceinline__ void umma_f16_step4_elected(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                       uint32_t accumulate_first) {
    asm volatile(
        "{\n\t"
        ".reg .pred pf, pt, pe;\n\t"
        ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
        ".reg .b32 leader;\n\t"
        "elect.sync leader|pe, 0xffffffff;\n\t"
        "setp.ne.b32 pf, %4, 0;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "add.s64 a1, %1, 2;\n\t"
        "add.s64 a2, %1, 4;\n\t"
        "add.s64 a3, %1, 6;\n\t"
        "add.s64 b1, %2, 2;\n\t"
        "add.s64 b2, %2, 4;\n\t"
        "add.s64 b3, %2, 6;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, pt;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, pt;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, pt;\n\t"
        "}"
        :
        : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate_first)
        : "memory");
}

// tcgen05.commit by the elected lane of a converged warp (the lane that issued the MMAs above).
__device__ __forceinline__ void umma_commit_elected(uint64_t* bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred pe;\n\t"
        ".reg .b32 leader;\n\t"
        "elect.sync leader|pe, 0xffffffff;\n\t"
        "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}" ::"r"(smem_addr(bar))
        : "memory");
}

// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
                 : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Make generic-proxy writes to shared memory visible to the async proxy (UMMA / TMA reads).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// TMEM allocation: whole warp, `columns` a power of two >= 32; the base address lands in *holder (shared).
__device__ __forceinline__ void tmem_alloc(uint32_t* holder, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(holder)), "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns: thread i of the warp reads TMEM lane (base lane + i).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Tiled TMA load of a 2-D box into this CTA's shared memory, completion in bytes on `bar`.
__device__ __forceinline__ void tma_load_2d(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_addr(dst_smem)),
        "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

}  // namespace ribn
