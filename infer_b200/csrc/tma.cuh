// TMA (cp.async.bulk.tensor) and mbarrier helpers, plus host-side tensor-map creation.
//
// Every wait in this file is bounded: a spin that does not complete within its iteration budget records
// a code in the device status word and returns false, and callers unwind (free TMEM, stop issuing copies)
// instead of hanging the GPU.  No load here uses cluster multicast.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fth {

// ---- device status word ------------------------------------------------------------------------------
// One int per device, 0 = ok.  A bounded wait that gives up stores (site << 16) | detail with atomicCAS from
// 0, so the first failure is kept.  Kernels receive its device address as a parameter (DeviceStatusPtr());
// the host reads and clears it through fth_b200_device_status().
int* DeviceStatusPtr();

__device__ __forceinline__ void ReportTimeout(int* status, int site, int detail) {
    if (status != nullptr) atomicCAS(status, 0, (site << 16) | (detail & 0xffff));
}

// ---- shared-memory addresses and barriers ---------------------------------------------------------------
__device__ __forceinline__ uint32_t SmemAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void MbarInit(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count));
}
__device__ __forceinline__ void FenceBarrierInit() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void FenceProxyAsync() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void MbarExpectTx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void MbarArrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SmemAddr(bar)) : "memory");
}
__device__ __forceinline__ bool MbarTryWait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(SmemAddr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Waits for the phase with the given parity.  After a short fast spin the loop backs off with nanosleep and
// watches the global nanosecond timer; one second after the first miss it reports (site, detail) in the
// status word and returns false.
constexpr uint64_t kWaitBudgetNs = 1000ull * 1000ull * 1000ull;
__device__ __forceinline__ uint64_t GlobalTimerNs() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool MbarWait(uint64_t* bar, uint32_t parity, int* status, int site, int detail) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i) {
        if (MbarTryWait(bar, parity)) return true;
    }
    const uint64_t start = GlobalTimerNs();
#pragma unroll 1
    for (;;) {
        if (MbarTryWait(bar, parity)) return true;
        __nanosleep(64);
        if (GlobalTimerNs() - start > kWaitBudgetNs) break;
    }
    ReportTimeout(status, site, detail);
    return false;
}

// ---- thread-block clusters: ranks, barrier, distributed shared memory ------------------------------------
__device__ __forceinline__ uint32_t ClusterRank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t ClusterSize() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
// Second use of the cluster barrier in a kernel that only needs "every CTA has got this far" (no data is handed over):
// no release fence, so the stores before it are not waited for.
__device__ __forceinline__ void ClusterArriveRelaxed() { asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory"); }
// Kernel parameters are read through the constant cache, and the first touch of each line costs a round trip to L2
// (about a microsecond here).  Reads one word of every 32 bytes of `params` so that a kernel launched ahead of its
// producer has all of them cached by the time the producer finishes.
template <typename T>
__device__ __forceinline__ void TouchConstantLines(const T& params) {
    const uint32_t* words = reinterpret_cast<const uint32_t*>(&params);
#pragma unroll
    for (int i = 0; i < static_cast<int>(sizeof(T) / 4); i += 8) asm volatile("" ::"r"(words[i]));
    asm volatile("" ::"r"(words[sizeof(T) / 4 - 1]));
}
__device__ __forceinline__ void ClusterArrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void ClusterWait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
// Address of this CTA's shared-memory location `smem_addr` inside CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t MapToRank(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
// 16-byte store into a peer CTA's shared memory that adds its 16 bytes to the transaction count of a barrier in
// the same peer: the receiver waits on that barrier and needs no other synchronisation with the sender.
__device__ __forceinline__ void StoreClusterAsync4(uint32_t addr, uint32_t bar, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar) : "memory");
}
// One arrival on a barrier in a peer CTA's shared memory (`bar` is a shared::cluster address).
__device__ __forceinline__ void MbarArriveRemote(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}

// ---- TMA loads (no multicast) -----------------------------------------------------------------------------
// x is the innermost coordinate; x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void TmaLoad2D(void* smem_dst, const CUtensorMap* map, int32_t x, int32_t y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(SmemAddr(smem_dst)), "l"(map), "r"(SmemAddr(bar)), "r"(x), "r"(y)
        : "memory");
}
// Load issued by either CTA of a pair into its own shared memory; the bytes are reported to `bar_cluster_addr`, a
// shared::cluster address that may name a barrier of the other CTA of the pair.  No multicast.
__device__ __forceinline__ void TmaLoad2DPair(void* smem_dst, const CUtensorMap* map, int32_t x, int32_t y, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(SmemAddr(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void TmaLoad4D(void* smem_dst, const CUtensorMap* map, int32_t c0, int32_t c1, int32_t c2,
                                          int32_t c3, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(SmemAddr(smem_dst)), "l"(map), "r"(SmemAddr(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// Tile store from shared memory (dense rows of the box's width, no swizzle) to global memory, this GPU's or a peer's;
// the part of the box outside the tensor is not written.  Stores of one thread are grouped with BulkCommitGroup;
// BulkWaitGroupRead0 returns when every committed group has read its shared memory (the buffer may be overwritten),
// BulkWaitGroup0 when their writes are complete.
__device__ __forceinline__ void TmaStore2D(const CUtensorMap* map, const void* smem_src, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(SmemAddr(smem_src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void BulkCommitGroup() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void BulkWaitGroupRead0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void BulkWaitGroup0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// 16 bytes to a multicast address (NVLS): the switch delivers the store to every GPU bound to the mapping.
__device__ __forceinline__ void MulticastStore16(void* multicast_addr, uint4 v) {
    asm volatile("multimem.st.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(multicast_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void TmaPrefetchDescriptor(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- host: tensor maps ---------------------------------------------------------------------------------------
enum class TmaSwizzle { kNone, k32B, k64B, k128B };

// rank-2 uint8 tensor [rows][cols] with a row pitch in bytes; box = box_cols x box_rows.
// Returns false if the driver entry point is unavailable or the encode fails (bad alignment).
bool MakeTensorMap2D(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t row_pitch_bytes,
                     uint32_t box_cols, uint32_t box_rows, TmaSwizzle swizzle);
// rank-4 uint8 tensor, dims listed innermost first; strides_bytes has 3 entries (dims 1..3).
bool MakeTensorMap4D(CUtensorMap* map, const void* base, const uint64_t dims[4], const uint64_t strides_bytes[3],
                     const uint32_t box[4], TmaSwizzle swizzle);

}  // namespace fth
