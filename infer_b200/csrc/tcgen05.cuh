// tcgen05 (5th-generation tensor core) helpers: tensor-memory allocation, shared-memory matrix descriptors,
// instruction descriptors, MMA issue / commit, and TMEM loads.  Single-CTA forms only (cta_group::1).
#pragma once

#include <stdint.h>

#include "tma.cuh"

namespace fth {
namespace umma {

// ---- tensor memory ------------------------------------------------------------------------------------
// Executed by one full warp.  `columns` is a power of two in [32, 512]; the base address is written to smem.
__device__ __forceinline__ void TmemAlloc(uint32_t* smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(smem_result)), "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void TmemDealloc(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void FenceBeforeThreadSync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void FenceAfterThreadSync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- descriptors ----------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle (tile bases are 1024-byte aligned):
//   bits  0..13  start address >> 4        bits 16..29  leading-dimension byte offset >> 4
//   bits 32..45  stride byte offset >> 4   bits 46..47  descriptor version (1 on sm_100)
//   bits 61..63  layout type (2 = SWIZZLE_128B)
//
// K-major operand ([rows][128 bytes of K], the TMA box {128, rows}): 8-row groups are 1024 bytes apart
// (stride offset); the leading offset is unused.  Successive K = 32 slices advance the start address by 32 bytes.
// MN-major operand ([k rows][128 bytes of M or N], the TMA box {128, k rows}): one k row holds 128 consecutive
// M/N elements; 8 k rows form a 1024-byte group (stride offset); further 128-element M/N blocks lie
// `leading` bytes away.  Successive K = 32 slices advance the start address by 32 rows = 4096 bytes.
// The same descriptor for a 64-byte swizzle (layout type 4): rows of 64 bytes, 8-row groups 512 bytes apart.
__device__ __forceinline__ uint64_t SmemDescSw64(uint32_t smem_addr, uint32_t leading_bytes, uint32_t stride_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>((leading_bytes >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3fffu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(4) << 61;
    return d;
}

__device__ __forceinline__ uint64_t SmemDesc(uint32_t smem_addr, uint32_t leading_bytes, uint32_t stride_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>((leading_bytes >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3fffu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Instruction descriptor (32 bits): D format at bits 4..5 (1 = F32, 2 = S32), A format bits 7..9, B format
// bits 10..12 (f8f6f4: 0 = E4M3, 1 = E5M2; i8: 1 = signed), A major bit 15, B major bit 16 (0 = K, 1 = MN),
// N >> 3 at bits 17..22, M >> 4 at bits 24..28.
__host__ __device__ inline uint32_t InstrDesc(uint32_t d_format, uint32_t a_format, uint32_t b_format, bool a_mn_major,
                                              bool b_mn_major, uint32_t m, uint32_t n) {
    return (d_format << 4) | (a_format << 7) | (b_format << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
           (static_cast<uint32_t>(b_mn_major) << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---- MMA issue (one thread) --------------------------------------------------------------------------------
template <bool INT8>
__device__ __forceinline__ void Mma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (INT8) {
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
            ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}"
            ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
// Makes the barrier track completion of every MMA this thread issued so far (one arrival).
__device__ __forceinline__ void Commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(SmemAddr(bar)) : "memory");
}

// ---- CTA-pair forms (cta_group::2): one MMA spans the two CTAs of a cluster pair --------------------------------
// Allocation and release are executed by one warp of EACH CTA of the pair; both receive the same address.
__device__ __forceinline__ void TmemAllocPair(uint32_t* smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(smem_result)), "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void TmemDeallocPair(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
// Issued by one thread of the leader CTA (even rank).  M = 256: rows 0..127 come from the leader's A tile, rows
// 128..255 from the peer's tile at the same shared-memory offset; the N columns of B are split the same way
// (first half in the leader's shared memory, second half in the peer's).  Each CTA's tensor memory receives its
// 128 rows of D.
template <bool INT8>
__device__ __forceinline__ void MmaPair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (INT8) {
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n}"
            ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n}"
            ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
// One arrival on the barrier at the same shared-memory offset in every CTA named by `cta_mask`, once all MMAs this
// thread issued so far have completed.
__device__ __forceinline__ void CommitPair(uint64_t* bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(SmemAddr(bar)), "h"(cta_mask) : "memory");
}

// ---- TMEM → registers: 32 lanes x 16 consecutive 32-bit columns per warp --------------------------------------
__device__ __forceinline__ void TmemLoad16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// 4 consecutive columns (the folded split-K epilogue reads a few activation rows of many accumulators)
__device__ __forceinline__ void TmemLoad4(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void TmemLoadWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace umma
}  // namespace fth
