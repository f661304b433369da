// Shared by the tensor-core linear kernels (linear_tc_swapped.cu, linear_tc_pair.cu, linear_tc_cluster.cu) and their
// dispatcher (linear_tcgen05.cu): launch parameters, tile geometry, and the epilogue helpers every kernel uses.
#pragma once

#include "common.cuh"
#include "linear_internal.h"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace fth {
namespace tc {

constexpr int kBlockP = 128;
constexpr int kBlockK = 128;  // bytes of K per ring stage = one 128-byte swizzle row
constexpr int kPBytes = kBlockP * kBlockK;

struct TcParams {
    LinearArgs args;
    int swap;
    int64_t p_total, q_total;  // extents along TMEM lanes / accumulator columns
    int64_t p_tiles, q_tiles;
    int split;                 // K chunks per tile
    int64_t chunk_blocks;      // 128-byte K blocks per chunk
    int ring_stages;           // cluster kernel: weight ring depth of this launch
    int64_t k_blocks;          // ceil(K / 128)
    int tiles_per_cta;         // cluster kernel: weight tiles per CTA (1 or 2)
    int second_tile_offset;    // the second tile: 0 = the same tile of the second weight (fusion.w2), else tile + this of the same weight
    int64_t units;             // p_tiles * q_tiles * split (folded: p_tiles * q_tiles)
    int fold;                  // persistent swapped kernel: one CTA runs all K chunks of a tile and adds them itself (no reduce pass)
    uint32_t idesc;
    int e4m3;                  // FP8 format of operands and output (1 = E4M3, 0 = E5M2)
    int fast;                  // 1: no bias, alpha = beta = 1, native output dtype → vectorised epilogue
    int fast4;                 // same for the four-channel epilogue, which also covers a fused output Cast (FP8)
    int decoder;               // cluster kernel: the decoder-block form (BF16 -> FP8 product -> BF16, per-tensor scales, one GPU)
    float a_inv, out_inv;      // exact reciprocals of the activation / output scale (powers of two), else 0
    void* scratch;             // [split][q_total][p_pad] partial accumulators
    int64_t p_pad;
    int* status;
};

// Tensor maps of the output block in this GPU's buffer ([0]) and in the peers' replicas, for the CTA-pair kernel's tile
// stores (count 0: the epilogue stores from registers instead).
struct OutMaps {
    CUtensorMap map[kMaxPeers + 1];
    int count;
    uint8_t* multicast;  // the output block in a multicast mapping of all ranks' buffers (then `map` is unused), or null
    int64_t ldo;         // its row pitch
};

constexpr int kClusterQBlocks = 8;  // K blocks of activations the cluster kernel keeps resident per CTA

struct TcGeometry {
    bool swap;
    int bq;
    int split;
    int64_t chunk_blocks, k_blocks, p_total, q_total, p_tiles, q_tiles, units, p_pad;
    int cluster;  // > 0: single-launch cluster kernel with this many CTAs per weight tile
    int tiles_per_cta, second_tile_offset;  // cluster kernel: see TcParams
};


// ---- launchers, one per kernel family (each in its own translation unit) ------------------------------------------
// M <= 128, several waves of work: persistent swapped kernel (+ the split-K reduce pass when g.split > 1).
int LaunchSwapped(bool int8, const TcGeometry& g, bool weights_mn, const CUtensorMap& map_p, const CUtensorMap& map_q, const TcParams& p,
                  const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream);
// M > 128: CTA pairs.  map_a: activations, box {128 B of K, 128 rows}; map_w: weights, box of 128 columns.
int LaunchPair(bool int8, bool weights_mn, const CUtensorMap& map_a, const CUtensorMap& map_w, const OutMaps& out_maps, const TcParams& p,
               const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream);
// M <= 32, one wave: single-launch cluster kernel.
int LaunchCluster(bool int8, const TcGeometry& g, bool weights_mn, const CUtensorMap& map_p, const CUtensorMap& map_p2, const CUtensorMap& map_q,
                  const TcParams& p, const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream);

// ---- device helpers ---------------------------------------------------------------------------------------------------
template <int THREADS>
__device__ __forceinline__ void EpilogueBarrier() { asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory"); }

// Generic (slow) store of one finished accumulator through the shared epilogue helpers: every bias mode,
// Gemm alpha / beta and fused Cast / DequantizeLinear output.
template <bool INT8>
__device__ __forceinline__ void StoreOne(const Fp8Epilogue& fe, const Int8Epilogue& ie, int e4m3, int64_t m, int64_t n,
                                         uint32_t raw) {
    if constexpr (INT8) {
        StoreInt8Result(ie, m, n, static_cast<int32_t>(raw), 0, 0);
    } else {
        if (e4m3) StoreFp8Result<FTH_B200_FP8E4M3>(fe, m, n, __uint_as_float(raw));
        else StoreFp8Result<FTH_B200_FP8E5M2>(fe, m, n, __uint_as_float(raw));
    }
}

// Inf / NaN inputs of EncodePair: the software encoder, whose special codes are the reference's.  Kept out of line: the
// callers sit on latency-bound paths that run once per CTA, where every instruction fetched counts.
static __device__ __noinline__ uint32_t EncodePairSpecial(int e4m3, float y0, float y1) {
    if (e4m3) return Encode<FTH_B200_FP8E4M3>(y0) | (static_cast<uint32_t>(Encode<FTH_B200_FP8E4M3>(y1)) << 8);
    return Encode<FTH_B200_FP8E5M2>(y0) | (static_cast<uint32_t>(Encode<FTH_B200_FP8E5M2>(y1)) << 8);
}
// Encodes y0, y1 (already divided by the output scale) into two FP8 codes: low byte = y0, high byte = y1.
__device__ __forceinline__ uint32_t EncodePair(int e4m3, float y0, float y1) {
    const bool special = ((__float_as_uint(y0) & 0x7f800000u) == 0x7f800000u) || ((__float_as_uint(y1) & 0x7f800000u) == 0x7f800000u);
    if (special) return EncodePairSpecial(e4m3, y0, y1);
    uint16_t packed;
    if (e4m3) asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(packed) : "f"(y1), "f"(y0));
    else asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(packed) : "f"(y1), "f"(y0));
    return packed;
}

// ---- fused greedy selection (argmax over each output row) ---------------------------------------------------
// A candidate is one 64-bit key: the value mapped to an order-preserving 32-bit pattern in the high word, the
// complemented column in the low word — the largest key is the largest value and, among equals, the lowest column.
// Key 0 means "no candidate" (a NaN code).  -0 counts as +0, as a floating-point comparison would have it.
template <bool INT8>
__device__ __forceinline__ unsigned long long ArgmaxKey(int e4m3, uint32_t code, int64_t column) {
    float v;
    if constexpr (INT8) v = static_cast<float>(static_cast<int8_t>(code));
    else v = e4m3 ? Decode<FTH_B200_FP8E4M3>(static_cast<uint8_t>(code)) : Decode<FTH_B200_FP8E5M2>(static_cast<uint8_t>(code));
    if (v != v) return 0ull;
    if (v == 0.0f) v = 0.0f;
    const uint32_t bits = __float_as_uint(v);
    const uint32_t ordered = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    return (static_cast<unsigned long long>(ordered) << 32) | (0xffffffffu - static_cast<uint32_t>(column));
}
// Called by all 32 lanes of a warp: row < 0 marks a lane without a candidate.  Lanes of one row are combined with
// shuffles so that a warp costs one atomic; a warp that straddles rows falls back to one atomic per lane.
__device__ __forceinline__ void ArgmaxUpdate(unsigned long long* keys, int row, unsigned long long key) {
    const int top = __reduce_max_sync(0xffffffffu, row);
    const bool one_row = __all_sync(0xffffffffu, row == top || row < 0);
    if (one_row) {
        if (row < 0) key = 0ull;
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, offset);
            key = other > key ? other : key;
        }
        if ((threadIdx.x & 31) == 0 && top >= 0 && key != 0ull) atomicMax(&keys[top], key);
    } else if (row >= 0 && key != 0ull) {
        atomicMax(&keys[row], key);
    }
}

// Stores `value` at `dst` and at the same place in every peer replica of the output.
template <typename T>
__device__ __forceinline__ void StoreWithPeers(const PeerOut& peers, T* dst, T value) {
    *dst = value;
    for (int r = 0; r < peers.count; ++r) *reinterpret_cast<T*>(reinterpret_cast<uint8_t*>(dst) + peers.delta[r]) = value;
}

// ---- gather step signalling inside a kernel ---------------------------------------------------------------------
// The step this launch works on.  Read after griddepcontrol.wait: the launch in front writes the counter at its very end.
__device__ __forceinline__ uint32_t GatherStep(const GatherSignal& g) {
    uint32_t s;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(s) : "l"(g.flags[g.rank] + g.world) : "memory");
    s += 1;
    return s == 0 ? 1u : s;
}
// Called by the threads 0 .. world-1 of a group (index `r`): waits, for at most one second, until rank r has published
// step - 1 in this rank's array.  Stores into the peers' buffers of this step may only follow.
__device__ __forceinline__ void GatherWaitPrevious(const GatherSignal& g, int r, uint32_t step, int* status) {
    const uint32_t* slot = g.flags[g.rank] + r;
    const uint32_t want = step - 1;
    uint64_t start = 0;
    for (int spin = 0;; ++spin) {
        // A relaxed load is enough: nothing the peer wrote is read here.  The flag only says that the peer's stream has
        // passed its reads of the buffers this launch is about to overwrite (it publishes a step from a kernel that its
        // stream orders behind those reads), and the stores below depend on the value through the branch.
        uint32_t seen;
        asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(slot) : "memory");
        if (static_cast<int32_t>(seen - want) >= 0) return;
        if (spin == 64) start = GlobalTimerNs();
        if (spin > 64) {
            __nanosleep(100);
            if (GlobalTimerNs() - start > kWaitBudgetNs) { ReportTimeout(status, 41, r); return; }
        }
    }
}
// Called by ONE thread of every thread block of the launch, after a block-wide barrier behind the block's output
// stores.  The barrier orders the other threads' stores before this thread; its fence and arrival are a release at GPU
// scope (all blocks of the launch are on this GPU), the last block's read of the counter and its system-scope fence
// acquire every arrival and release, cumulatively, all blocks' stores to the other GPUs before the flags below.  Only
// that one fence has to wait for the peers to acknowledge the stores: a system-scope fence in every block cost 5 us
// per step on eight GPUs (15.0 -> 10.2 us), all blocks draining their own stores at the same time.  The last block
// advances the step counter and publishes the step in every rank's array.
__device__ __forceinline__ void GatherArriveAndPublish(const GatherSignal& g, uint32_t step, unsigned blocks) {
    uint32_t* mine = g.flags[g.rank];
    __threadfence();
    const unsigned arrived = atomicAdd(mine + g.world + 1, 1u);
    if (arrived != blocks - 1) return;
    __threadfence_system();  // the other blocks' stores (ordered before their arrivals) before the flags below
    mine[g.world + 1] = 0;
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(mine + g.world), "r"(step) : "memory");
    for (int r = 0; r < g.world; ++r)  // one fence above, then plain system-scope stores: none of them waits for the others
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(g.flags[r] + g.rank), "r"(step) : "memory");
}

// Epilogue of one output (activation row q, channel n) from its complete accumulator.
// Returns the output code on the direct path (read by the fused argmax).
template <bool INT8>
__device__ __forceinline__ uint32_t FinishOne(const TcParams& p, const Fp8Epilogue& fe, const Int8Epilogue& ie, int64_t q, int64_t n,
                                              uint32_t raw) {
    if (!p.fast4) { StoreOne<INT8>(fe, ie, p.e4m3, q, n, raw); return 0; }
    if constexpr (INT8) {
        const double sd = static_cast<double>(ie.a_scale) * static_cast<double>(ie.w_scales[ie.per_channel ? n : 0]);
        const double so_d = static_cast<double>(ie.out_scale);
        const double md = sd / so_d;
        const int8_t r = RequantFast(static_cast<int32_t>(raw), static_cast<float>(md), md, sd, so_d, ie.out_zp);
        StoreWithPeers(p.args.peers, static_cast<int8_t*>(ie.out) + q * ie.ldo + n, r);
        return static_cast<uint8_t>(r);
    } else {
        const float mult = fe.w_channel_scales ? fe.ab_scale * fe.w_channel_scales[n] : fe.ab_scale;
        const float t = __fmul_rn(__uint_as_float(raw), mult);
        const float y = p.out_inv != 0.0f ? __fmul_rn(t, p.out_inv) : __fdiv_rn(t, fe.out_scale);
        const uint8_t code = p.e4m3 ? Encode<FTH_B200_FP8E4M3>(y) : Encode<FTH_B200_FP8E5M2>(y);
        const int64_t o = q * fe.ldo + n;
        if (fe.out_dtype == 0) { StoreWithPeers(p.args.peers, static_cast<uint8_t*>(fe.out) + o, code); return code; }
        // fused Cast behind the MatMul: the decoded code times the output scale, as BF16 or FP32
        const float d = p.e4m3 ? Decode<FTH_B200_FP8E4M3>(code) : Decode<FTH_B200_FP8E5M2>(code);
        const float v = __fmul_rn(d, fe.out_scale);
        if (fe.out_dtype == FTH_B200_BF16) {
            StoreWithPeers(p.args.peers, static_cast<uint16_t*>(fe.out) + o, EncodeBf16Cast(v));
        } else {
            StoreWithPeers(p.args.peers, static_cast<float*>(fe.out) + o, v);
        }
        return code;
    }
}

}  // namespace tc
}  // namespace fth
