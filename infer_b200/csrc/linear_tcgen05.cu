// Tensor-core linear kernels: tcgen05.mma (kind::f8f6f4 / kind::i8) with accumulators in tensor memory, operands
// staged by TMA into 128-byte-swizzled shared memory, fused scale / bias / requant / encode epilogues.
// Weights are consumed in the layout Feather stores them: [K,N] tiles are MN-major operands, [N,K] tiles K-major
// operands — no repacking pass, no second copy of the weights.  Three kernels, chosen by shape:
//
//   LinearPairKernel     M > 128: 256 x 256 output tiles on CTA pairs (cta_group::2), activations on the TMEM lanes.
//   LinearTcgen05Kernel  M <= 128, more than one wave of work: operands swapped — weights on the 128 TMEM lanes,
//                        activations on a 16..128-wide UMMA N — so a decode-sized M pads only the narrow dimension and
//                        the weight stream fills all lanes.  One or two persistent CTAs per SM, warp-specialised
//                        (warp 0 TMA producer, warp 1 TMEM allocation + MMA issue, warps 2-5 epilogue draining one of
//                        2-4 accumulator buffers while the next unit's MMAs run).  K is split into S chunks (S depends
//                        on K and M only) so that a 28672-column weight gives ~1800 work units; partial accumulators
//                        go to a scratch buffer with coalesced stores and SplitReduceKernel adds the S partials of
//                        every output in chunk order and runs the epilogue.  (A single-kernel hand-off through fences
//                        and arrival counters was measured first: the gpu-scope fence per work unit stalled the
//                        epilogue warps behind the streaming loads and cost more than the extra launch.)
//   LinearClusterKernel  M <= 32, one wave of work: the same split, inside a thread-block cluster, in one launch.
#include <cmath>

#include "common.cuh"
#include "linear_internal.h"
#include "tcgen05.cuh"
#include "tma.cuh"

// Optional phase timeline of CTA 0 in SM clocks (development aid, compiled out unless FTH_B200_TRACE is defined).
#ifdef FTH_B200_TRACE
__device__ unsigned long long g_trace[32];
#define FTH_TRACE(i) do { if (blockIdx.x == 0) g_trace[i] = static_cast<unsigned long long>(clock64()); } while (0)
extern "C" int fth_b200_trace_read(unsigned long long* out) {
    return cudaMemcpyFromSymbol(out, g_trace, sizeof(g_trace)) == cudaSuccess ? 0 : -1;
}
#else
#define FTH_TRACE(i) do {} while (0)
#endif

namespace fth {
namespace {

constexpr int kBlockP = 128;
constexpr int kBlockK = 128;  // bytes of K per ring stage = one 128-byte swizzle row
constexpr int kPBytes = kBlockP * kBlockK;
constexpr size_t kSmemBudget = 200 * 1024;

struct TcParams {
    LinearArgs args;
    int swap;
    int64_t p_total, q_total;  // extents along TMEM lanes / accumulator columns
    int64_t p_tiles, q_tiles;
    int split;                 // K chunks per tile
    int64_t chunk_blocks;      // 128-byte K blocks per chunk
    int ring_stages;           // cluster kernel: weight ring depth of this launch
    int64_t k_blocks;          // ceil(K / 128)
    int64_t units;             // p_tiles * q_tiles * split
    uint32_t idesc;
    int e4m3;                  // FP8 format of operands and output (1 = E4M3, 0 = E5M2)
    int fast;                  // 1: no bias, alpha = beta = 1, native output dtype → vectorised epilogue
    int fast4;                 // same for the four-channel epilogue, which also covers a fused output Cast (FP8)
    float a_inv, out_inv;      // exact reciprocals of the activation / output scale (powers of two), else 0
    void* scratch;             // [split][q_total][p_pad] partial accumulators
    int64_t p_pad;
    int* status;
};

template <int BQ>
struct Cfg {
    static constexpr int kQBytes = BQ * kBlockK;
    static constexpr int kStageBytes = kPBytes + kQBytes;
    // Decode-sized tiles (BQ <= 32) run two CTAs per SM with half the ring each: two independent epilogue
    // warpgroups hide the split-K hand-off latency.  Larger tiles take the whole SM.
    static constexpr int kCtasPerSm = BQ <= 32 ? 2 : 1;
    static constexpr size_t kBudget = kCtasPerSm == 2 ? 100 * 1024 : 200 * 1024;
    static constexpr int kStagesRaw = static_cast<int>(kBudget / kStageBytes);
    static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
    // accumulator buffers in tensor memory (512 columns per SM shared by the resident CTAs)
    static constexpr int kAccBuffers = BQ <= 32 ? 4 : 2;
    static constexpr uint32_t kTmemColsRaw = kAccBuffers * BQ;
    static constexpr uint32_t kTmemCols = kTmemColsRaw < 32 ? 32 : kTmemColsRaw;
    static constexpr int kEpilogueThreads = 128;
    static constexpr int kThreads = 64 + kEpilogueThreads;
    static constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
};

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

// Encodes y0, y1 (already divided by the output scale) into two FP8 codes: low byte = y0, high byte = y1.
__device__ __forceinline__ uint32_t EncodePair(int e4m3, float y0, float y1) {
    const bool special = ((__float_as_uint(y0) & 0x7f800000u) == 0x7f800000u) || ((__float_as_uint(y1) & 0x7f800000u) == 0x7f800000u);
    if (special) {
        if (e4m3) return Encode<FTH_B200_FP8E4M3>(y0) | (static_cast<uint32_t>(Encode<FTH_B200_FP8E4M3>(y1)) << 8);
        return Encode<FTH_B200_FP8E5M2>(y0) | (static_cast<uint32_t>(Encode<FTH_B200_FP8E5M2>(y1)) << 8);
    }
    uint16_t packed;
    if (e4m3) asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(packed) : "f"(y1), "f"(y0));
    else asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(packed) : "f"(y1), "f"(y0));
    return packed;
}

template <bool INT8, bool P_MN, int BQ>
__global__ void __launch_bounds__(Cfg<BQ>::kThreads, Cfg<BQ>::kCtasPerSm)
LinearTcgen05Kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, TcParams p,
                    Fp8Epilogue fe, Int8Epilogue ie) {
    using C = Cfg<BQ>;
    constexpr int kAcc = C::kAccBuffers;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(C::kStages) * C::kStageBytes);
    uint64_t* empty = full + C::kStages;
    uint64_t* tmem_full = empty + C::kStages;      // [kAcc]
    uint64_t* tmem_empty = tmem_full + kAcc;       // [kAcc]
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + kAcc);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) { MbarInit(&full[s], 1); MbarInit(&empty[s], 1); }
        for (int b = 0; b < kAcc; ++b) { MbarInit(&tmem_full[b], 1); MbarInit(&tmem_empty[b], 4); }
        FenceBarrierInit();
    }
    if (warp == 1) umma::TmemAlloc(tmem_base_slot, C::kTmemCols);
    umma::FenceBeforeThreadSync();
    __syncthreads();
    umma::FenceAfterThreadSync();
    const uint32_t tmem_base = *tmem_base_slot;
    // Lets a dependent grid (the split-K reduce pass) be scheduled while this one runs; it still waits for this
    // grid to finish before it reads anything.  No effect when launched without programmatic serialization.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // Everything above (barriers, tensor memory) overlapped the tail of the previous kernel in the stream; the
    // operands may be that kernel's output, so nothing is read before it has completed.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // unit → (p tile, q tile, K chunk).  [K,N] weights walk the column tiles fastest (chunk-major): the CTAs running
    // together then read whole contiguous weight rows of one K range, which keeps DRAM pages open; with [N,K]
    // weights the chunks of one tile are the contiguous direction, so the chunk index varies fastest instead.
    auto decode_unit = [&](int64_t u, int64_t* pt, int64_t* qt, int* s) {
        int64_t t;
        if (P_MN) {
            const int64_t tiles = p.p_tiles * p.q_tiles;
            *s = static_cast<int>(u / tiles);
            t = u % tiles;
        } else {
            *s = static_cast<int>(u % p.split);
            t = u / p.split;
        }
        *qt = t % p.q_tiles;
        *pt = t / p.q_tiles;
    };
    auto blocks_of = [&](int s) -> int64_t {
        const int64_t begin = static_cast<int64_t>(s) * p.chunk_blocks;
        const int64_t left = p.k_blocks - begin;
        return left < p.chunk_blocks ? left : p.chunk_blocks;
    };

    if (warp == 0) {
        // ================================ TMA producer ================================
        if (lane == 0) {
            TmaPrefetchDescriptor(&map_p);
            TmaPrefetchDescriptor(&map_q);
            int stage = 0;
            uint32_t phase = 0;
            bool failed = false;
            for (int64_t u = blockIdx.x; u < p.units && !failed; u += gridDim.x) {
                int64_t pt, qt; int s;
                decode_unit(u, &pt, &qt, &s);
                const int64_t nb = blocks_of(s);
                for (int64_t kb = 0; kb < nb; ++kb) {
                    if (!MbarWait(&empty[stage], phase ^ 1u, p.status, 10, stage)) { failed = true; break; }
                    const int32_t k0 = static_cast<int32_t>((static_cast<int64_t>(s) * p.chunk_blocks + kb) * kBlockK);
                    const int32_t p0 = static_cast<int32_t>(pt * kBlockP);
                    const int32_t q0 = static_cast<int32_t>(qt * BQ);
                    uint8_t* ps = ring + static_cast<size_t>(stage) * C::kStageBytes;
                    uint8_t* qs = ps + kPBytes;
                    MbarExpectTx(&full[stage], C::kStageBytes);
                    if constexpr (P_MN) TmaLoad2D(ps, &map_p, p0, k0, &full[stage]);
                    else TmaLoad2D(ps, &map_p, k0, p0, &full[stage]);
                    TmaLoad2D(qs, &map_q, k0, q0, &full[stage]);
                    if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ================================ MMA issuer ================================
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool failed = false;
            int64_t iter = 0;
            for (int64_t u = blockIdx.x; u < p.units && !failed; u += gridDim.x, ++iter) {
                int64_t pt, qt; int s;
                decode_unit(u, &pt, &qt, &s);
                const int64_t nb = blocks_of(s);
                const int acc = static_cast<int>(iter % kAcc);
                const uint32_t acc_phase = static_cast<uint32_t>((iter / kAcc) & 1);
                if (!MbarWait(&tmem_empty[acc], acc_phase ^ 1u, p.status, 11, acc)) { failed = true; break; }
                umma::FenceAfterThreadSync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BQ);
                for (int64_t kb = 0; kb < nb; ++kb) {
                    if (!MbarWait(&full[stage], phase, p.status, 12, stage)) { failed = true; break; }
                    umma::FenceAfterThreadSync();
                    const uint32_t ps = SmemAddr(ring + static_cast<size_t>(stage) * C::kStageBytes);
                    const uint32_t qs = ps + kPBytes;
#pragma unroll
                    for (int ks = 0; ks < kBlockK / 32; ++ks) {
                        const uint64_t a_desc = P_MN ? umma::SmemDesc(ps + ks * 4096, 16384, 1024) : umma::SmemDesc(ps + ks * 32, 16, 1024);
                        const uint64_t b_desc = umma::SmemDesc(qs + ks * 32, 16, 1024);
                        umma::Mma<INT8>(d_tmem, a_desc, b_desc, p.idesc, (kb > 0 || ks > 0) ? 1u : 0u);
                    }
                    umma::Commit(&empty[stage]);  // the stage is free once these MMAs have read it
                    if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                }
                if (!failed) umma::Commit(&tmem_full[acc]);
            }
        }
    } else {
        // ================================ epilogue ================================
        const int et = threadIdx.x - 64;            // 0 .. kEpilogueThreads-1
        const int lane_group = warp & 3;            // TMEM lanes 32*lane_group .. +31 belong to this warp
        const int row = lane_group * 32 + lane;     // row inside the P tile
        const double so_d = static_cast<double>(ie.out_scale);
        // One double divide per thread; scale * so_inv is within 2^-52 of scale / out_scale, which the error bounds of
        // the two estimate stages of RequantFast absorb.
        const double so_inv = INT8 ? 1.0 / so_d : 0.0;
        const float so_f = fe.out_scale;
        const int64_t ldo = INT8 ? ie.ldo : fe.ldo;
        uint8_t* out8 = static_cast<uint8_t*>(INT8 ? ie.out : fe.out);
        bool failed = false;
        int64_t iter = 0;

        for (int64_t u = blockIdx.x; u < p.units; u += gridDim.x, ++iter) {
            int64_t pt, qt; int s;
            decode_unit(u, &pt, &qt, &s);
            const int acc = static_cast<int>(iter % kAcc);
            const uint32_t acc_phase = static_cast<uint32_t>((iter / kAcc) & 1);
            const int64_t pg = pt * kBlockP + row;
            const bool row_ok = pg < p.p_total;
            const int64_t q_begin = qt * BQ;
            const int64_t q_left = p.q_total - q_begin;
            const int q_count = static_cast<int>(q_left < BQ ? q_left : BQ);

            // ---- scale constants of this lane's output channel ----
            double row_scale_d = 0.0, row_mult_d = 0.0;
            float row_mult = 0.0f;
            if (p.fast && row_ok) {
                if constexpr (INT8) {
                    row_scale_d = static_cast<double>(ie.a_scale) * static_cast<double>(ie.w_scales[ie.per_channel ? pg : 0]);
                    row_mult_d = row_scale_d * so_inv;
                    row_mult = static_cast<float>(row_mult_d);
                } else {
                    row_mult = fe.w_channel_scales ? fe.ab_scale * fe.w_channel_scales[pg] : fe.ab_scale;
                }
            }

            // Turns 16 finished accumulators (columns c0 .. c0+cnt-1 of this thread's row) into output.
            auto finish = [&](const uint32_t (&v)[16], int c0, int cnt) {
                if (!p.fast) {
                    if (row_ok) {
                        for (int j = 0; j < cnt; ++j) {
                            const int64_t qg = q_begin + c0 + j;
                            StoreOne<INT8>(fe, ie, p.e4m3, qg, pg, v[j]);
                        }
                    }
                    return;
                }
                uint32_t b[16];  // one output byte each
                if constexpr (INT8) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (j >= cnt) break;  // uniform: a decode-sized M leaves most columns unused
                        b[j] = static_cast<uint8_t>(RequantFast(static_cast<int32_t>(v[j]), row_mult, row_mult_d, row_scale_d, so_d, ie.out_zp));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        if (j >= cnt) break;  // uniform; unused columns would only feed the divider zeros (its slow path)
                        const float y0 = __fdiv_rn(__fmul_rn(__uint_as_float(v[j]), row_mult), so_f);
                        const float y1 = __fdiv_rn(__fmul_rn(__uint_as_float(v[j + 1]), row_mult), so_f);
                        const uint32_t pair = EncodePair(p.e4m3, y0, y1);
                        b[j] = pair & 0xffu;
                        b[j + 1] = pair >> 8;
                    }
                }
                // lanes are consecutive output channels: four neighbouring lanes pack one 32-bit store
                const int64_t base_pg = pg - (lane & 3);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (j >= cnt) break;  // uniform
                    const uint32_t other1 = __shfl_xor_sync(0xffffffffu, b[j], 1);
                    const uint32_t pair = (lane & 1) ? (other1 | (b[j] << 8)) : (b[j] | (other1 << 8));
                    const uint32_t other2 = __shfl_xor_sync(0xffffffffu, pair, 2);
                    const uint32_t word = (lane & 2) ? (other2 | (pair << 16)) : (pair | (other2 << 16));
                    uint8_t* dst = out8 + (q_begin + c0 + j) * ldo + base_pg;
                    const bool group_ok = base_pg + 3 < p.p_total && (reinterpret_cast<uintptr_t>(dst) & 3) == 0;
                    if (group_ok) {
                        if ((lane & 3) == 0) *reinterpret_cast<uint32_t*>(dst) = word;
                    } else if (row_ok) {
                        dst[lane & 3] = static_cast<uint8_t>(b[j]);
                    }
                }
            };

            if (!failed && !MbarWait(&tmem_full[acc], acc_phase, p.status, 13, acc)) failed = true;
            umma::FenceAfterThreadSync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + static_cast<uint32_t>(acc * BQ);
#pragma unroll 1
            for (int c0 = 0; c0 < BQ; c0 += 16) {
                if (c0 >= q_count) break;  // uniform across the warp
                uint32_t v[16];
                umma::TmemLoad16(taddr + c0, v);
                umma::TmemLoadWait();
                const int cnt = q_count - c0 < 16 ? q_count - c0 : 16;
                if (p.split == 1) {
                    finish(v, c0, cnt);
                } else if (row_ok) {
                    uint32_t* part = static_cast<uint32_t*>(p.scratch);
                    for (int j = 0; j < cnt; ++j) part[(static_cast<int64_t>(s) * p.q_total + q_begin + c0 + j) * p.p_pad + pg] = v[j];
                }
            }
            // accumulator buffer drained: hand it back to the MMA warp
            umma::FenceBeforeThreadSync();
            __syncwarp();
            if (lane == 0) MbarArrive(&tmem_empty[acc]);

        }
    }

    umma::FenceBeforeThreadSync();
    __syncthreads();
    if (warp == 1) {
        umma::FenceAfterThreadSync();
        umma::TmemDealloc(tmem_base, C::kTmemCols);
    }
}


// ---------------------------------------------------------------------------------------------------------
// Dense tiles on CTA pairs (M > 128): tcgen05.mma.cta_group::2.
//
// With one CTA per 128 x 256 tile every MMA reads 4 KB of A and 8 KB of B from shared memory, and that read
// bandwidth (measured 77 % busy) is what holds the tensor pipe at ~72 %.  A pair of CTAs on neighbouring SMs works
// on a 256 x 256 tile instead: each CTA stages its own 128 rows of A and its own 128 of the 256 B columns, the
// leader issues M = 256 MMAs that read both CTAs' shared memory, and each CTA's tensor memory receives its 128 rows
// of D.  Per MMA a CTA now reads 4 KB + 4 KB, and pulls a third less through L2 as well.  No multicast loads: each
// CTA fetches exactly the bytes it stages.
//
//   warp 0 (each CTA)   TMA producer for the CTA's own A / B halves; bytes are reported to the LEADER's full barrier
//   warp 1 (leader)     MMA issue; tcgen05.commit multicast frees the stage in both CTAs / publishes the accumulator
//   warps 2-9 (each)    epilogue of the CTA's own 128 rows; buffers are handed back on the leader's barrier
// ---------------------------------------------------------------------------------------------------------
struct PairCfg {
    static constexpr int kTileN = 256;
    static constexpr int kHalfN = 128;                          // B columns staged by one CTA
    static constexpr int kStageBytes = kPBytes + kHalfN * kBlockK;  // 32 KB
    static constexpr int kStages = 6;
    static constexpr uint32_t kTmemCols = 512;                  // two 256-column accumulator buffers
    static constexpr int kEpilogueThreads = 256;
    static constexpr int kThreads = 64 + kEpilogueThreads;
    static constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageBytes + 1024 + 256 + kTileN * 24;
};

template <bool INT8, bool Q_MN>
__global__ void __launch_bounds__(PairCfg::kThreads, 1)
LinearPairKernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, TcParams p,
                 Fp8Epilogue fe, Int8Epilogue ie) {
    using C = PairCfg;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(C::kStages) * C::kStageBytes);
    uint64_t* empty = full + C::kStages;
    uint64_t* tmem_full = empty + C::kStages;      // [2]
    uint64_t* tmem_empty = tmem_full + 2;          // [2], used in the leader only
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    double* col_scale = reinterpret_cast<double*>(reinterpret_cast<uint8_t*>(full) + 256);
    double* col_multd = col_scale + C::kTileN;
    float* col_mult = reinterpret_cast<float*>(col_multd + C::kTileN);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t rank = ClusterRank();           // 0 = leader
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) { MbarInit(&full[s], 1); MbarInit(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { MbarInit(&tmem_full[b], 1); MbarInit(&tmem_empty[b], 2 * 8); }  // 8 epilogue warps per CTA
        FenceBarrierInit();
    }
    if (warp == 1) umma::TmemAllocPair(tmem_base_slot, C::kTmemCols);
    umma::FenceBeforeThreadSync();
    __syncthreads();
    umma::FenceAfterThreadSync();
    const uint32_t tmem_base = *tmem_base_slot;
    // both CTAs' barriers and tensor memory exist before either touches the other's
    ClusterArrive();
    ClusterWait();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int64_t m_pairs = (p.p_total + 255) / 256;
    const int64_t units = m_pairs * p.q_tiles;
    const int64_t pair_id = blockIdx.x / 2, pairs = gridDim.x / 2;
    bool failed = false;

    if (warp == 0) {
        // ================================ TMA producer (both CTAs) ================================
        if (lane == 0) {
            TmaPrefetchDescriptor(&map_p);
            TmaPrefetchDescriptor(&map_q);
            int stage = 0;
            uint32_t phase = 0;
            for (int64_t u = pair_id; u < units && !failed; u += pairs) {
                const int64_t mt = u % m_pairs, nt = u / m_pairs;  // row tiles fastest: the pairs running together share weights in L2
                const int32_t p0 = static_cast<int32_t>(mt * 256 + rank * 128);
                const int32_t q0 = static_cast<int32_t>(nt * C::kTileN + rank * C::kHalfN);
                for (int64_t kb = 0; kb < p.k_blocks; ++kb) {
                    if (!MbarWait(&empty[stage], phase ^ 1u, p.status, 30, stage)) { failed = true; break; }
                    const int32_t k0 = static_cast<int32_t>(kb * kBlockK);
                    uint8_t* ps = ring + static_cast<size_t>(stage) * C::kStageBytes;
                    uint8_t* qs = ps + kPBytes;
                    // the leader's barrier counts the bytes of both CTAs
                    if (leader) MbarExpectTx(&full[stage], 2 * C::kStageBytes);
                    const uint32_t bar = MapToRank(SmemAddr(&full[stage]), 0);
                    TmaLoad2DPair(ps, &map_p, k0, p0, bar);
                    if constexpr (Q_MN) TmaLoad2DPair(qs, &map_q, q0, k0, bar);
                    else TmaLoad2DPair(qs, &map_q, k0, q0, bar);
                    if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ================================ MMA issuer (leader only) ================================
        if (lane == 0 && leader) {
            int stage = 0;
            uint32_t phase = 0;
            int64_t iter = 0;
            for (int64_t u = pair_id; u < units && !failed; u += pairs, ++iter) {
                const int acc = static_cast<int>(iter & 1);
                const uint32_t acc_phase = static_cast<uint32_t>((iter >> 1) & 1);
                if (!MbarWait(&tmem_empty[acc], acc_phase ^ 1u, p.status, 31, acc)) { failed = true; break; }
                umma::FenceAfterThreadSync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * C::kTileN);
                for (int64_t kb = 0; kb < p.k_blocks; ++kb) {
                    if (!MbarWait(&full[stage], phase, p.status, 32, stage)) { failed = true; break; }
                    umma::FenceAfterThreadSync();
                    const uint32_t ps = SmemAddr(ring + static_cast<size_t>(stage) * C::kStageBytes);
                    const uint32_t qs = ps + kPBytes;
#pragma unroll
                    for (int ks = 0; ks < kBlockK / 32; ++ks) {
                        const uint64_t a_desc = umma::SmemDesc(ps + ks * 32, 16, 1024);
                        const uint64_t b_desc = Q_MN ? umma::SmemDesc(qs + ks * 4096, 16384, 1024) : umma::SmemDesc(qs + ks * 32, 16, 1024);
                        umma::MmaPair<INT8>(d_tmem, a_desc, b_desc, p.idesc, (kb > 0 || ks > 0) ? 1u : 0u);
                    }
                    umma::CommitPair(&empty[stage], 3);  // the stage is free in both CTAs once these MMAs have read it
                    if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                }
                if (!failed) umma::CommitPair(&tmem_full[acc], 3);
            }
        }
    } else {
        // ================================ epilogue (both CTAs, own 128 rows) ================================
        const int et = threadIdx.x - 64;            // 0 .. 255
        const int lane_group = warp & 3;
        const int col_group = (warp - 2) / 4;       // which 128-column half this warpgroup drains
        const int row = lane_group * 32 + lane;
        const double so_d = static_cast<double>(ie.out_scale);
        const double so_inv = INT8 ? 1.0 / so_d : 0.0;  // one divide per thread; see RequantFast for the error budget
        const float zp_f = static_cast<float>(ie.out_zp);
        const float so_f = fe.out_scale;
        const int64_t ldo = INT8 ? ie.ldo : fe.ldo;
        uint8_t* out8 = static_cast<uint8_t*>(INT8 ? ie.out : fe.out);
        const uint32_t leader_empty = MapToRank(SmemAddr(tmem_empty), 0);
        int64_t iter = 0;
        int64_t staged_nt = -1;
        for (int64_t u = pair_id; u < units; u += pairs, ++iter) {
            const int64_t mt = u % m_pairs, nt = u / m_pairs;
            const int acc = static_cast<int>(iter & 1);
            const uint32_t acc_phase = static_cast<uint32_t>((iter >> 1) & 1);
            const int64_t mg = mt * 256 + rank * 128 + row;
            const bool row_ok = mg < p.p_total;
            const int64_t n_begin = nt * C::kTileN;
            const int64_t n_left = p.q_total - n_begin;
            const int n_count = static_cast<int>(n_left < C::kTileN ? n_left : C::kTileN);
            if (p.fast && nt != staged_nt) {  // uniform across the epilogue warps
                EpilogueBarrier<C::kEpilogueThreads>();  // readers of the previous tile's constants are done
                for (int c = et; c < C::kTileN; c += C::kEpilogueThreads) {
                    const int64_t n = n_begin + c;
                    if (n < p.q_total) {
                        if constexpr (INT8) {
                            const double sd = static_cast<double>(ie.a_scale) * static_cast<double>(ie.w_scales[ie.per_channel ? n : 0]);
                            col_scale[c] = sd;
                            col_multd[c] = sd * so_inv;
                            col_mult[c] = static_cast<float>(sd * so_inv);
                        } else {
                            col_mult[c] = fe.w_channel_scales ? fe.ab_scale * fe.w_channel_scales[n] : fe.ab_scale;
                        }
                    }
                }
                EpilogueBarrier<C::kEpilogueThreads>();
                staged_nt = nt;
            }
            if (!failed && !MbarWait(&tmem_full[acc], acc_phase, p.status, 33, acc)) failed = true;
            umma::FenceAfterThreadSync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + static_cast<uint32_t>(acc * C::kTileN);
#pragma unroll 1
            for (int c0 = col_group * 128; c0 < (col_group + 1) * 128; c0 += 16) {
                if (c0 >= n_count) break;  // uniform across the warp
                uint32_t v[16];
                umma::TmemLoad16(taddr + c0, v);
                umma::TmemLoadWait();
                const int cnt = n_count - c0 < 16 ? n_count - c0 : 16;
                if (failed || !row_ok) continue;
                if (!p.fast) {
                    for (int j = 0; j < cnt; ++j) StoreOne<INT8>(fe, ie, p.e4m3, mg, n_begin + c0 + j, v[j]);
                    continue;
                }
                uint32_t b[16];
                if constexpr (INT8) {
                    uint32_t near = 0;
#pragma unroll
                    for (int j = 0; j < 16; ++j) b[j] = RequantEstimate(static_cast<int32_t>(v[j]), col_mult[c0 + j], zp_f, j, &near);
                    while (near != 0) {  // a few values in 10^4: decided in double
                        const int j = __ffs(near) - 1;
                        near &= near - 1;
                        int32_t vj = 0;
#pragma unroll
                        for (int i = 0; i < 16; ++i) vj = i == j ? static_cast<int32_t>(v[i]) : vj;  // keeps v[] in registers
                        const uint32_t exact = static_cast<uint8_t>(RequantInt32(vj, col_scale[c0 + j], col_multd[c0 + j], so_d, ie.out_zp));
#pragma unroll
                        for (int i = 0; i < 16; ++i) b[i] = i == j ? exact : b[i];
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        const float y0 = __fdiv_rn(__fmul_rn(__uint_as_float(v[j]), col_mult[c0 + j]), so_f);
                        const float y1 = __fdiv_rn(__fmul_rn(__uint_as_float(v[j + 1]), col_mult[c0 + j + 1]), so_f);
                        const uint32_t pair = EncodePair(p.e4m3, y0, y1);
                        b[j] = pair & 0xffu;
                        b[j + 1] = pair >> 8;
                    }
                }
                uint8_t* dst = out8 + mg * ldo + n_begin + c0;
                if (cnt == 16 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                    uint4 w;
                    w.x = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
                    w.y = b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24);
                    w.z = b[8] | (b[9] << 8) | (b[10] << 16) | (b[11] << 24);
                    w.w = b[12] | (b[13] << 8) | (b[14] << 16) | (b[15] << 24);
                    *reinterpret_cast<uint4*>(dst) = w;
                } else {
                    for (int j = 0; j < cnt; ++j) dst[j] = static_cast<uint8_t>(b[j]);
                }
            }
            // this CTA's half of the accumulator buffer is drained: tell the leader's MMA warp
            umma::FenceBeforeThreadSync();
            __syncwarp();
            if (lane == 0) MbarArriveRemote(leader_empty + acc * 8);
        }
    }

    // Neither CTA may leave (or free its tensor memory) while the leader's MMAs can still read the peer's shared
    // memory or write its tensor memory, or while remote arrivals are in flight.
    umma::FenceBeforeThreadSync();
    __syncthreads();
    ClusterArrive();
    ClusterWait();
    if (warp == 1) {
        umma::FenceAfterThreadSync();
        umma::TmemDeallocPair(tmem_base, C::kTmemCols);
    }
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

// Epilogue of four consecutive output channels p4 .. p4+3 of activation row q (swapped tiling), given their
// complete accumulators: the vectorised fast path or the generic per-element store.
// Returns the four output codes (channel p4 in the low byte) on the direct path, which the fused argmax reads.
template <bool INT8>
__device__ __forceinline__ uint32_t FinishFour(const TcParams& p, const Fp8Epilogue& fe, const Int8Epilogue& ie, int64_t q,
                                               int64_t p4, const uint32_t (&v)[4]) {
    if (!p.fast4) {
        for (int i = 0; i < 4; ++i)
            if (p4 + i < p.p_total) StoreOne<INT8>(fe, ie, p.e4m3, q, p4 + i, v[i]);
        return 0;
    }
    uint32_t b[4];
    if constexpr (INT8) {
        for (int i = 0; i < 4; ++i) {
            const int64_t n = p4 + i < p.p_total ? p4 + i : p.p_total - 1;
            const double sd = static_cast<double>(ie.a_scale) * static_cast<double>(ie.w_scales[ie.per_channel ? n : 0]);
            const double so_d = static_cast<double>(ie.out_scale);
            const double md = sd / so_d;
            b[i] = static_cast<uint8_t>(RequantFast(static_cast<int32_t>(v[i]), static_cast<float>(md), md, sd, so_d, ie.out_zp));
        }
    } else {
        float y[4];
        for (int i = 0; i < 4; ++i) {
            const int64_t n = p4 + i < p.p_total ? p4 + i : p.p_total - 1;
            const float mult = fe.w_channel_scales ? fe.ab_scale * fe.w_channel_scales[n] : fe.ab_scale;
            y[i] = __fdiv_rn(__fmul_rn(__uint_as_float(v[i]), mult), fe.out_scale);
        }
        const uint32_t lo = EncodePair(p.e4m3, y[0], y[1]), hi = EncodePair(p.e4m3, y[2], y[3]);
        b[0] = lo & 0xffu; b[1] = lo >> 8; b[2] = hi & 0xffu; b[3] = hi >> 8;
        if (fe.out_dtype != 0) {
            // fused Cast behind the MatMul: the decoded code times the output scale, as BF16 or FP32
            const float2 d01 = p.e4m3 ? DecodePair<FTH_B200_FP8E4M3>(static_cast<uint16_t>(lo)) : DecodePair<FTH_B200_FP8E5M2>(static_cast<uint16_t>(lo));
            const float2 d23 = p.e4m3 ? DecodePair<FTH_B200_FP8E4M3>(static_cast<uint16_t>(hi)) : DecodePair<FTH_B200_FP8E5M2>(static_cast<uint16_t>(hi));
            const float o[4] = {__fmul_rn(d01.x, fe.out_scale), __fmul_rn(d01.y, fe.out_scale), __fmul_rn(d23.x, fe.out_scale), __fmul_rn(d23.y, fe.out_scale)};
            const bool whole = p4 + 3 < p.p_total;
            if (fe.out_dtype == FTH_B200_BF16) {
                uint16_t* dst = static_cast<uint16_t*>(fe.out) + q * fe.ldo + p4;
                if (whole && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
                    uint2 t;
                    t.x = EncodeBf16Cast(o[0]) | (static_cast<uint32_t>(EncodeBf16Cast(o[1])) << 16);
                    t.y = EncodeBf16Cast(o[2]) | (static_cast<uint32_t>(EncodeBf16Cast(o[3])) << 16);
                    StoreWithPeers(p.args.peers, reinterpret_cast<uint2*>(dst), t);
                } else {
                    for (int i = 0; i < 4 && p4 + i < p.p_total; ++i) StoreWithPeers(p.args.peers, dst + i, EncodeBf16Cast(o[i]));
                }
            } else {
                float* dst = static_cast<float*>(fe.out) + q * fe.ldo + p4;
                if (whole && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) StoreWithPeers(p.args.peers, reinterpret_cast<float4*>(dst), make_float4(o[0], o[1], o[2], o[3]));
                else { for (int i = 0; i < 4 && p4 + i < p.p_total; ++i) StoreWithPeers(p.args.peers, dst + i, o[i]); }
            }
            return b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
        }
    }
    const int64_t ldo = INT8 ? ie.ldo : fe.ldo;
    uint8_t* dst = static_cast<uint8_t*>(INT8 ? ie.out : fe.out) + q * ldo + p4;
    if (p4 + 3 < p.p_total && (reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
        StoreWithPeers(p.args.peers, reinterpret_cast<uint32_t*>(dst), b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24));
    } else {
        for (int i = 0; i < 4 && p4 + i < p.p_total; ++i) StoreWithPeers(p.args.peers, dst + i, static_cast<uint8_t>(b[i]));
    }
    return b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
}


// Second pass of the split-K path (swapped tiling only: rows p are output channels n, columns q are
// activation rows m).  One thread owns four consecutive channels of one activation row: it adds the S partial
// accumulators in chunk order (the same order whatever the grid was), runs the epilogue and stores 4 bytes.
template <bool INT8>
__global__ void __launch_bounds__(256) SplitReduceKernel(TcParams p, Fp8Epilogue fe, Int8Epilogue ie) {
    // Launched with programmatic stream serialization: wait until the producing grid has completed and its
    // partial sums are visible.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t groups = p.p_pad / 4;
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    const int64_t q = idx / groups;
    const int64_t p4 = (idx % groups) * 4;
    const bool valid = idx < groups * p.q_total && p4 < p.p_total;
    if (!valid && p.args.argmax_keys == nullptr) return;
    const uint4* part = static_cast<const uint4*>(p.scratch);
    uint32_t v[4] = {0, 0, 0, 0};
    if (valid) {
    if constexpr (INT8) {
        int32_t sum[4] = {0, 0, 0, 0};
        uint4 t[8];
#pragma unroll
        for (int ss = 0; ss < 8; ++ss)  // all loads in flight before the first add
            t[ss] = ss < p.split ? __ldcg(&part[((static_cast<int64_t>(ss) * p.q_total + q) * p.p_pad + p4) / 4]) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int ss = 0; ss < 8; ++ss) {
            sum[0] += static_cast<int32_t>(t[ss].x); sum[1] += static_cast<int32_t>(t[ss].y);
            sum[2] += static_cast<int32_t>(t[ss].z); sum[3] += static_cast<int32_t>(t[ss].w);
        }
        for (int i = 0; i < 4; ++i) v[i] = static_cast<uint32_t>(sum[i]);
    } else {
        float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        uint4 t[8];
#pragma unroll
        for (int ss = 0; ss < 8; ++ss)  // all loads in flight before the first add
            t[ss] = ss < p.split ? __ldcg(&part[((static_cast<int64_t>(ss) * p.q_total + q) * p.p_pad + p4) / 4]) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int ss = 0; ss < 8; ++ss) {
            if (ss < p.split) {  // chunk order, and never add a zero that could flip the sign of -0
                sum[0] += __uint_as_float(t[ss].x); sum[1] += __uint_as_float(t[ss].y);
                sum[2] += __uint_as_float(t[ss].z); sum[3] += __uint_as_float(t[ss].w);
            }
        }
        for (int i = 0; i < 4; ++i) v[i] = __float_as_uint(sum[i]);
    }
    }
    const uint32_t codes = valid ? FinishFour<INT8>(p, fe, ie, q, p4, v) : 0u;
    if (p.args.argmax_keys != nullptr) {  // every lane of the warp is here
        unsigned long long key = 0ull;
        for (int i = 0; i < 4; ++i) {
            if (valid && p4 + i < p.p_total) {
                const unsigned long long k = ArgmaxKey<INT8>(p.e4m3, (codes >> (8 * i)) & 0xffu, p4 + i);
                key = k > key ? k : key;
            }
        }
        ArgmaxUpdate(p.args.argmax_keys, valid ? static_cast<int>(q) : -1, key);
    }
}

// ---------------------------------------------------------------------------------------------------------
// Decode-sized problems (M <= 32, one wave of CTAs): split-K inside a thread-block cluster.
//
// The S CTAs of a cluster work on the S K-chunks of one 128-channel weight tile, so S SMs pull the tile's bytes
// at the same time (one SM alone draws ~35 bytes per clock through TMA, which is what bounds a small
// projection).  Each CTA's accumulator leaves tensor memory once; its 128 rows are dealt out to the cluster's
// CTAs through distributed shared memory (CTA o receives rows o*L .. o*L+L-1 of every chunk, L = 128 / cluster
// size), and after one cluster barrier each CTA adds the chunks of its rows in chunk order — the order the
// two-kernel path uses, so both give the same bits — and runs the epilogue.  No scratch, no second launch.
//
// A fused Cast / QuantizeLinear in front of the MatMul is done here as well: the epilogue warps, idle while the
// weights stream, read the CTA's K-chunk of BF16 / FP16 / FP32 activations, convert, and write the 8-bit codes
// into the swizzled operand tile that the MMA reads (generic-proxy writes, made visible with fence.proxy.async).
// 8-bit activations arrive by TMA as before.  The activation chunk stays resident (kQBlocks blocks at most);
// only the weight tile goes through the ring.
// ---------------------------------------------------------------------------------------------------------
template <int BQ>
struct ClusterCfg {
    static constexpr int kQBlocks = 8;                       // K blocks of activations held per CTA
    static constexpr int kQBytes = kQBlocks * BQ * kBlockK;  // 16 KB / 32 KB
    static constexpr int kStages = BQ <= 16 ? 5 : 3;         // weight ring (16 KB per stage), upper limit
    static constexpr int kMaxStages = 8;                     // barrier slots
    static constexpr int kExchangeBytes = kBlockP * BQ * 4;  // partials of this CTA's rows, all chunks
    static constexpr uint32_t kTmemCols = 32;
    static constexpr int kThreads = 192;
    static constexpr size_t kSmemBytes = 1024 + static_cast<size_t>(kStages) * kPBytes + kQBytes + kExchangeBytes + 256;
    static int StagesFor(int64_t chunk_blocks) { return chunk_blocks < kStages ? static_cast<int>(chunk_blocks) : kStages; }
    static size_t SmemFor(int64_t chunk_blocks) {
        return 1024 + static_cast<size_t>(StagesFor(chunk_blocks)) * kPBytes + static_cast<size_t>(chunk_blocks) * BQ * kBlockK +
               kExchangeBytes + 256;
    }
};

// Four consecutive activation elements of a fused Cast (FP8) / QuantizeLinear (INT8) prologue.  The raw load and
// the conversion are separate so that a thread can have several loads in flight before it converts the first.
// `index` is a multiple of 4; `vec` says the base pointer is 16-byte aligned.
__device__ __forceinline__ uint4 LoadFourRaw(const LinearArgs& a, int64_t index, bool vec) {
    uint4 r = make_uint4(0, 0, 0, 0);
    if (a.a_dtype == FTH_B200_FP32) {
        const uint32_t* src = static_cast<const uint32_t*>(a.a) + index;
        if (vec) r = *reinterpret_cast<const uint4*>(src);
        else { r.x = src[0]; r.y = src[1]; r.z = src[2]; r.w = src[3]; }
    } else {
        const uint16_t* src = static_cast<const uint16_t*>(a.a) + index;
        if (vec) { const uint2 t = *reinterpret_cast<const uint2*>(src); r.x = t.x; r.y = t.y; }
        else { r.x = src[0] | (static_cast<uint32_t>(src[1]) << 16); r.y = src[2] | (static_cast<uint32_t>(src[3]) << 16); }
    }
    return r;
}
// Codes of the four elements, element 0 in the low byte.  `a_inv` is 1 / a_scale when that is exact (a power of
// two: x * a_inv and x / a_scale are then the same correctly rounded value), else 0.
template <bool INT8>
__device__ __forceinline__ uint32_t ConvertFourRaw(const LinearArgs& a, const Int8Epilogue& ie, int e4m3, float a_inv, uint4 raw) {
    float x[4];
    if (a.a_dtype == FTH_B200_FP32) {
        x[0] = __uint_as_float(raw.x); x[1] = __uint_as_float(raw.y); x[2] = __uint_as_float(raw.z); x[3] = __uint_as_float(raw.w);
    } else if (a.a_dtype == FTH_B200_BF16) {
        x[0] = __uint_as_float(raw.x << 16); x[1] = __uint_as_float(raw.x & 0xffff0000u);
        x[2] = __uint_as_float(raw.y << 16); x[3] = __uint_as_float(raw.y & 0xffff0000u);
    } else {
        const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
        const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
        x[0] = lo.x; x[1] = lo.y; x[2] = hi.x; x[3] = hi.y;
    }
    if constexpr (INT8) {
        uint32_t word = 0;
        for (int i = 0; i < 4; ++i) word |= static_cast<uint32_t>(static_cast<uint8_t>(QuantizeValue(x[i], ie.a_scale, ie.a_zp))) << (8 * i);
        return word;
    } else {
        float y[4];
        // a NaN skips the divide, as in the stand-alone Cast kernel
        if (a_inv != 0.0f) { for (int i = 0; i < 4; ++i) y[i] = (x[i] != x[i]) ? x[i] : __fmul_rn(x[i], a_inv); }
        else { for (int i = 0; i < 4; ++i) y[i] = (x[i] != x[i]) ? x[i] : __fdiv_rn(x[i], a.a_scale); }
        return EncodePair(e4m3, y[0], y[1]) | (EncodePair(e4m3, y[2], y[3]) << 16);
    }
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
        if (fe.out_dtype == FTH_B200_BF16) StoreWithPeers(p.args.peers, static_cast<uint16_t*>(fe.out) + o, EncodeBf16Cast(v));
        else StoreWithPeers(p.args.peers, static_cast<float*>(fe.out) + o, v);
        return code;
    }
}

template <bool INT8, bool P_MN, int BQ>
__global__ void __launch_bounds__(ClusterCfg<BQ>::kThreads, 2)
LinearClusterKernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, TcParams p,
                    Fp8Epilogue fe, Int8Epilogue ie) {
    using C = ClusterCfg<BQ>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // The ring and the activation tiles are sized per launch (p.ring_stages, p.chunk_blocks): a small projection
    // then takes ~30 KB instead of ~100 KB, and the CTAs of the next kernel in the stream can move in early.
    const int stages = p.ring_stages;
    uint8_t* q_tiles = ring + static_cast<size_t>(stages) * kPBytes;            // [chunk_blocks][BQ][128], 128-byte swizzle
    uint32_t* exchange = reinterpret_cast<uint32_t*>(q_tiles + p.chunk_blocks * (BQ * kBlockK));  // [chunk][L][BQ]
    uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(exchange) + C::kExchangeBytes);
    uint64_t* empty = full + C::kMaxStages;
    uint64_t* q_full = empty + C::kMaxStages;
    uint64_t* tmem_full = q_full + 1;
    uint64_t* x_full = tmem_full + 1;  // counts the bytes peers deliver into `exchange`
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(x_full + 1);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) FTH_TRACE(0);
    const bool convert = p.args.a_dtype != 0;

    if (threadIdx.x == 0) {
        TmaPrefetchDescriptor(&map_p);  // kernel parameters: safe to touch before the previous grid has finished
        if (!convert) TmaPrefetchDescriptor(&map_q);
        for (int s = 0; s < stages; ++s) { MbarInit(&full[s], 1); MbarInit(&empty[s], 1); }
        MbarInit(q_full, convert ? 128 : 1);
        MbarInit(tmem_full, 1);
        MbarInit(x_full, 1);
        FenceBarrierInit();
    }
    if (warp == 1) umma::TmemAlloc(tmem_base_slot, C::kTmemCols);
    umma::FenceBeforeThreadSync();
    __syncthreads();
    umma::FenceAfterThreadSync();
    const uint32_t tmem_base = *tmem_base_slot;
    if (threadIdx.x == 0) FTH_TRACE(1);
    ClusterArrive();  // "this CTA is running": peers wait for it before they write into our exchange buffer
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const uint32_t rank = ClusterRank();
    const uint32_t csize = ClusterSize();                  // a power of two
    const int cshift = 31 - __clz(static_cast<int>(csize));
    const int tile = static_cast<int>(blockIdx.x >> cshift);
    const int lshift = 7 - cshift;                         // log2 of L = rows of the tile this CTA finishes
    const int rows_per_cta = 1 << lshift;
    const int kb_begin = static_cast<int>(rank) * static_cast<int>(p.chunk_blocks);
    int nb = static_cast<int>(p.k_blocks) - kb_begin;
    if (nb > static_cast<int>(p.chunk_blocks)) nb = static_cast<int>(p.chunk_blocks);
    if (nb < 0) nb = 0;  // ranks beyond the split have no K range
    const int m = static_cast<int>(p.q_total);
    // Kernel parameters live in constant memory and every first touch of a line costs a few hundred cycles: read
    // what the roles need now, while the previous kernel in the stream may still be running.
    {
        const int64_t out_bits = reinterpret_cast<int64_t>(INT8 ? ie.out : fe.out);
        const int64_t ldo_bits = INT8 ? ie.ldo : fe.ldo;
        asm volatile("" ::"r"(p.split), "l"(p.p_total), "r"(p.fast4), "r"(p.e4m3), "r"(p.idesc), "l"(p.args.k), "l"(p.args.a),
                     "r"(p.args.a_dtype), "f"(p.args.a_scale), "f"(fe.out_scale), "f"(fe.ab_scale), "l"(fe.w_channel_scales),
                     "r"(fe.out_dtype), "l"(out_bits), "l"(ldo_bits), "f"(ie.a_scale), "f"(ie.out_scale), "l"(ie.w_scales),
                     "l"(p.status), "f"(p.a_inv), "f"(p.out_inv));
    }

    if (warp == 0) {
        // ================================ TMA producer ================================
        if (lane == 0 && nb > 0) {
            int stage = 0;
            uint32_t phase = 0;
            auto load_weights = [&](int kb) -> bool {
                // the first pass over the ring finds every stage free; later passes wait for the MMAs that read it
                if (kb >= stages && !MbarWait(&empty[stage], phase ^ 1u, p.status, 20, stage)) return false;
                const int32_t k0 = (kb_begin + kb) * kBlockK;
                const int32_t p0 = tile * kBlockP;
                uint8_t* ps = ring + static_cast<size_t>(stage) * kPBytes;
                MbarExpectTx(&full[stage], kPBytes);
                if constexpr (P_MN) TmaLoad2D(ps, &map_p, p0, k0, &full[stage]);
                else TmaLoad2D(ps, &map_p, k0, p0, &full[stage]);
                if (++stage == stages) { stage = 0; phase ^= 1u; }
                return true;
            };
            // Weights that no earlier work in the stream writes can be fetched before the previous kernel has
            // finished: their DRAM latency then overlaps its tail.
            int kb = 0;
            if (p.args.w_static) {
                for (; kb < nb && kb < stages; ++kb) load_weights(kb);
            }
            FTH_TRACE(3);
            asm volatile("griddepcontrol.wait;" ::: "memory");
            FTH_TRACE(2);
            if (!convert) {
                MbarExpectTx(q_full, static_cast<uint32_t>(nb) * BQ * kBlockK);
                for (int j = 0; j < nb; ++j) TmaLoad2D(q_tiles + j * (BQ * kBlockK), &map_q, (kb_begin + j) * kBlockK, 0, q_full);
            }
            for (; kb < nb; ++kb) {
                if (!load_weights(kb)) break;
            }
            FTH_TRACE(4);
        }
    } else if (warp == 1) {
        // ================================ MMA issuer ================================
        if (lane == 0 && nb > 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool failed = false;
            for (int kb = 0; kb < nb && !failed; ++kb) {
                if (!MbarWait(&full[stage], phase, p.status, 22, stage)) { failed = true; break; }
                if (kb == 0 && !MbarWait(q_full, 0, p.status, 21, 0)) { failed = true; break; }  // activations arrive last
                if (kb == 0) FTH_TRACE(5);
                umma::FenceAfterThreadSync();
                const uint32_t ps = SmemAddr(ring + static_cast<size_t>(stage) * kPBytes);
                const uint32_t qs = SmemAddr(q_tiles + kb * (BQ * kBlockK));
#pragma unroll
                for (int ks = 0; ks < kBlockK / 32; ++ks) {
                    const uint64_t a_desc = P_MN ? umma::SmemDesc(ps + ks * 4096, 16384, 1024) : umma::SmemDesc(ps + ks * 32, 16, 1024);
                    const uint64_t b_desc = umma::SmemDesc(qs + ks * 32, 16, 1024);
                    umma::Mma<INT8>(tmem_base, a_desc, b_desc, p.idesc, (kb > 0 || ks > 0) ? 1u : 0u);
                }
                umma::Commit(&empty[stage]);
                if (++stage == stages) { stage = 0; phase ^= 1u; }
            }
            FTH_TRACE(6);
            if (!failed) umma::Commit(tmem_full);
        }
    } else {
        // ====================== activation prologue, accumulator hand-out, reduce + epilogue ======================
        const int et = threadIdx.x - 64;  // 0 .. 127
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (convert && nb > 0) {
            // Four consecutive K elements of one activation row per item (one 32-bit word of the swizzled tile), four
            // items per thread and round so that their loads overlap.  Rows >= m stay unwritten: they only feed
            // accumulator columns nobody reads.  K beyond the end is zero.
            const int words_per_row = nb * 32;
            const int total = m * words_per_row;
            const bool vec = (reinterpret_cast<uintptr_t>(p.args.a) & 15) == 0;
            for (int base = et; base < total; base += 4 * 128) {
                uint4 raw[4];
                uint32_t dst[4];
                bool inside[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int item = base + j * 128;
                    const int row = item / words_per_row;
                    const int c = item - row * words_per_row;
                    const int kb = c >> 5, w4 = c & 31;
                    const int64_t k0 = static_cast<int64_t>(kb_begin + kb) * kBlockK + w4 * 4;
                    inside[j] = item < total && k0 < p.args.k;  // K is a multiple of 16: a group is in or out as a whole
                    dst[j] = SmemAddr(q_tiles) + kb * (BQ * kBlockK) + row * 128 + (((w4 >> 2) ^ (row & 7)) << 4) + ((w4 & 3) << 2);
                    raw[j] = inside[j] ? LoadFourRaw(p.args, static_cast<int64_t>(row) * p.args.k + k0, vec) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (base + j * 128 < total) {
                        const uint32_t word = inside[j] ? ConvertFourRaw<INT8>(p.args, ie, p.e4m3, p.a_inv, raw[j]) : 0u;
                        asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst[j]), "r"(word) : "memory");
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes → visible to the MMA's reads
            MbarArrive(q_full);
            if (et == 0) FTH_TRACE(7);
        }
        const int row = (warp & 3) * 32 + lane;  // TMEM lane = channel inside the tile
        // Bytes this CTA will receive: from each of the `split` chunks, its L rows of ceil(m / 4) 16-byte vectors.
        if (et == 0) MbarExpectTx(x_full, static_cast<uint32_t>(p.split) * rows_per_cta * ((m + 3) / 4) * 16);
        ClusterWait();  // every CTA of the cluster is running and has initialised its barriers
        if (et == 0) FTH_TRACE(8);
        if (nb > 0) {
            const bool ok = MbarWait(tmem_full, 0, p.status, 23, 0);
            if (et == 0) FTH_TRACE(9);
            umma::FenceAfterThreadSync();
            if (ok) {
                // Deal the accumulator rows out: row r goes to CTA r / L, slot [this chunk][r % L].  Each 16-byte
                // store reports its bytes to the receiver's barrier, so no cluster-wide barrier is needed.
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
                const uint32_t owner = static_cast<uint32_t>(row >> lshift);
                const uint32_t slot = SmemAddr(exchange) + (((rank << lshift) + (row & (rows_per_cta - 1))) * BQ) * 4;
                const uint32_t remote = MapToRank(slot, owner);
                const uint32_t remote_bar = MapToRank(SmemAddr(x_full), owner);
#pragma unroll
                for (int c0 = 0; c0 < BQ; c0 += 16) {
                    if (c0 >= m) break;  // uniform
                    uint32_t v[16];
                    umma::TmemLoad16(taddr + c0, v);
                    umma::TmemLoadWait();
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        if (c0 + j < m) StoreClusterAsync4(remote + (c0 + j) * 4, remote_bar, v[j], v[j + 1], v[j + 2], v[j + 3]);
                    }
                }
            }
        }
        if (et == 0) FTH_TRACE(10);
        // A CTA leaves only after everything addressed to it has landed, so no peer ever writes into a CTA that is gone.
        const bool delivered = MbarWait(x_full, 0, p.status, 24, 0);
        if (et == 0) FTH_TRACE(11);

        // One output per thread and round: channel r of this CTA's rows (fastest, so a warp stores consecutive
        // channels) of activation row q.  The chunks are added in chunk order, as the two-kernel path adds them.
        const int total = m << lshift;
        for (int base = 0; base < total; base += 128) {  // the same trip count in every lane: the argmax step below shuffles
            const int item = base + et;
            const bool valid = delivered && item < total;
            const int q = item >> lshift;
            const int r = item & (rows_per_cta - 1);
            const int64_t n = static_cast<int64_t>(tile) * kBlockP + (static_cast<int64_t>(rank) << lshift) + r;
            uint32_t code = 0;
            bool stored = false;
            if (valid) {
                uint32_t t[8];
#pragma unroll
                for (int ss = 0; ss < 8; ++ss) t[ss] = ss < p.split ? exchange[((ss << lshift) + r) * BQ + q] : 0u;  // all in flight
                uint32_t acc;
                if constexpr (INT8) {
                    int32_t sum = 0;
#pragma unroll
                    for (int ss = 0; ss < 8; ++ss) sum += static_cast<int32_t>(t[ss]);
                    acc = static_cast<uint32_t>(sum);
                } else {
                    float sum = 0.0f;
#pragma unroll
                    for (int ss = 0; ss < 8; ++ss) {
                        if (ss < p.split) sum += __uint_as_float(t[ss]);  // no zero is ever added: it could flip a -0
                    }
                    acc = __float_as_uint(sum);
                }
                if (et == 0) FTH_TRACE(14);
                if (n < p.p_total) { code = FinishOne<INT8>(p, fe, ie, q, n, acc); stored = true; }
            }
            if (p.args.argmax_keys != nullptr)
                ArgmaxUpdate(p.args.argmax_keys, stored ? q : -1, stored ? ArgmaxKey<INT8>(p.e4m3, code, n) : 0ull);
        }
    }
    if (warp < 2) {
        if (!(warp == 0 && lane == 0 && nb > 0)) asm volatile("griddepcontrol.wait;" ::: "memory");
        ClusterWait();
    }
    if (threadIdx.x == 64) FTH_TRACE(12);
    umma::FenceBeforeThreadSync();
    __syncthreads();
    if (warp == 1) {
        umma::FenceAfterThreadSync();
        umma::TmemDealloc(tmem_base, C::kTmemCols);
        if (lane == 0) FTH_TRACE(13);
    }
}

// ---------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------
int SmCountTc() {
    static int count = 0;
    if (count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) count = kNumSms;
    }
    return count;
}

// 1 / s when s is a normal power of two with a normal reciprocal (x * (1/s) then equals x / s bit for bit), else 0.
float ExactReciprocal(float s) {
    int e = 0;
    if (!(s > 0.0f) || !std::isnormal(s) || std::frexp(s, &e) != 0.5f) return 0.0f;
    const float inv = 1.0f / s;
    return std::isnormal(inv) ? inv : 0.0f;
}

int SwapBlockQ(int64_t m) { return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128; }

struct TcGeometry {
    bool swap;
    int bq;
    int split;
    int64_t chunk_blocks, k_blocks, p_total, q_total, p_tiles, q_tiles, units, p_pad;
    int cluster;  // > 0: single-launch cluster kernel with this many CTAs per weight tile
};

TcGeometry GeometryFor(const LinearArgs& a) {
    TcGeometry g;
    g.swap = a.m <= 128;
    g.bq = g.swap ? SwapBlockQ(a.m) : 256;
    g.p_total = g.swap ? a.n : a.m;
    g.q_total = g.swap ? a.m : a.n;
    g.p_tiles = (g.p_total + kBlockP - 1) / kBlockP;
    g.q_tiles = (g.q_total + g.bq - 1) / g.bq;
    g.k_blocks = (a.k + kBlockK - 1) / kBlockK;
    // K split: a function of K and M only, so column shards of a weight reproduce the full result bit for bit
    const int split_max = !g.swap ? 1 : (g.bq <= 16 ? 8 : g.bq <= 32 ? 4 : 2);
    const int64_t s0 = g.k_blocks < split_max ? g.k_blocks : split_max;
    g.chunk_blocks = (g.k_blocks + s0 - 1) / s0;
    g.split = static_cast<int>((g.k_blocks + g.chunk_blocks - 1) / g.chunk_blocks);
    g.units = g.p_tiles * g.q_tiles * g.split;
    g.p_pad = g.p_tiles * kBlockP;
    // Decode-sized problems that fit one wave of CTAs take the single-launch cluster kernel.  Which kernel runs
    // depends on N, but both add the same chunks in the same order, so the bits do not.
    g.cluster = 0;
    if (g.swap && g.bq <= 32 && g.q_tiles == 1 && g.chunk_blocks <= ClusterCfg<16>::kQBlocks) {
        int c = 1;
        while (c < g.split) c *= 2;
        // more than one wave of CTAs: the persistent kernel keeps its ring full across tiles and is faster (measured)
        if (g.p_tiles * c <= static_cast<int64_t>(SmCountTc()) * 2) g.cluster = c;
    }
    return g;
}


// Encoding a tensor map costs a few microseconds of host time; decode steps call the same (pointer, shape)
// pairs over and over, so the last few encodings are kept per host thread.
bool CachedMap(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint32_t box_cols, uint32_t box_rows) {
    struct Entry { const void* base; uint64_t cols, rows; uint32_t bc, br; CUtensorMap map; };
    thread_local Entry cache[16] = {};
    thread_local int next = 0;
    for (const Entry& e : cache) {
        if (e.base == base && e.cols == cols && e.rows == rows && e.bc == box_cols && e.br == box_rows) { *out = e.map; return true; }
    }
    CUtensorMap map;
    if (!MakeTensorMap2D(&map, base, cols, rows, cols, box_cols, box_rows, TmaSwizzle::k128B)) return false;
    cache[next] = Entry{base, cols, rows, box_cols, box_rows, map};
    next = (next + 1) % 16;
    *out = map;
    return true;
}

template <bool INT8, bool P_MN, int BQ>
int LaunchTyped(const CUtensorMap& map_p, const CUtensorMap& map_q, const TcParams& p, const Fp8Epilogue& fe,
                const Int8Epilogue& ie, cudaStream_t stream) {
    auto kernel = LinearTcgen05Kernel<INT8, P_MN, BQ>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg<BQ>::kSmemBytes)) != cudaSuccess) return FTH_B200_ERR_CUDA;
        configured = true;
    }
    const int64_t slots = static_cast<int64_t>(SmCountTc()) * Cfg<BQ>::kCtasPerSm;
    const int grid = static_cast<int>(p.units < slots ? p.units : slots);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(Cfg<BQ>::kThreads);
    cfg.dynamicSmemBytes = Cfg<BQ>::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, map_p, map_q, p, fe, ie) != cudaSuccess) return FTH_B200_ERR_CUDA;
    NoteLaunch("tcgen05");
    return CheckLaunch();
}

template <bool INT8>
int LaunchForLayout(const TcGeometry& g, bool weights_mn, const CUtensorMap& map_p, const CUtensorMap& map_q,
                    const TcParams& p, const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream) {
#define FTH_SWAP_CASE(BQV)                                                                            \
    case BQV:                                                                                         \
        return weights_mn ? LaunchTyped<INT8, true, BQV>(map_p, map_q, p, fe, ie, stream)             \
                          : LaunchTyped<INT8, false, BQV>(map_p, map_q, p, fe, ie, stream);
    switch (g.bq) {
        FTH_SWAP_CASE(16) FTH_SWAP_CASE(32) FTH_SWAP_CASE(64) FTH_SWAP_CASE(128)
        default: return FTH_B200_ERR_INVALID;
    }
#undef FTH_SWAP_CASE
}

template <bool INT8, bool Q_MN>
int LaunchPairTyped(const CUtensorMap& map_p, const CUtensorMap& map_q, const TcParams& p, const Fp8Epilogue& fe,
                    const Int8Epilogue& ie, cudaStream_t stream) {
    auto kernel = LinearPairKernel<INT8, Q_MN>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(PairCfg::kSmemBytes)) != cudaSuccess) return FTH_B200_ERR_CUDA;
        configured = true;
    }
    const int64_t units = ((p.p_total + 255) / 256) * p.q_tiles;
    const int64_t slots = SmCountTc() / 2;
    const int64_t pairs = units < slots ? units : slots;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(pairs * 2));
    cfg.blockDim = dim3(PairCfg::kThreads);
    cfg.dynamicSmemBytes = PairCfg::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    if (cudaLaunchKernelEx(&cfg, kernel, map_p, map_q, p, fe, ie) != cudaSuccess) return FTH_B200_ERR_CUDA;
    NoteLaunch("tcgen05");
    return CheckLaunch();
}

template <bool INT8, bool P_MN, int BQ>
int LaunchClusterTyped(const TcGeometry& g, const CUtensorMap& map_p, const CUtensorMap& map_q, const TcParams& p_in,
                       const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream) {
    TcParams p = p_in;
    p.ring_stages = ClusterCfg<BQ>::StagesFor(g.chunk_blocks);
    auto kernel = LinearClusterKernel<INT8, P_MN, BQ>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ClusterCfg<BQ>::kSmemBytes)) != cudaSuccess) return FTH_B200_ERR_CUDA;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(g.p_tiles * g.cluster));
    cfg.blockDim = dim3(ClusterCfg<BQ>::kThreads);
    cfg.dynamicSmemBytes = ClusterCfg<BQ>::SmemFor(g.chunk_blocks);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = static_cast<unsigned>(g.cluster);
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    if (cudaLaunchKernelEx(&cfg, kernel, map_p, map_q, p, fe, ie) != cudaSuccess) return FTH_B200_ERR_CUDA;
    NoteLaunch("tcgen05");
    return CheckLaunch();
}

template <bool INT8>
int LaunchCluster(const TcGeometry& g, bool weights_mn, const CUtensorMap& map_p, const CUtensorMap& map_q, const TcParams& p,
                  const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream) {
    if (g.bq == 16) {
        return weights_mn ? LaunchClusterTyped<INT8, true, 16>(g, map_p, map_q, p, fe, ie, stream)
                          : LaunchClusterTyped<INT8, false, 16>(g, map_p, map_q, p, fe, ie, stream);
    }
    return weights_mn ? LaunchClusterTyped<INT8, true, 32>(g, map_p, map_q, p, fe, ie, stream)
                      : LaunchClusterTyped<INT8, false, 32>(g, map_p, map_q, p, fe, ie, stream);
}

}  // namespace

// A fused Cast / QuantizeLinear in front of the MatMul runs as one elementwise pass that writes the quantised
// activations (1 byte each) to the front of the scratch buffer; TMA then reads them like any FP8 / INT8 input.
// The cluster kernel converts its activations itself and needs neither.
size_t PrologueBytes(const LinearArgs& a) {
    if (a.a_dtype == 0 || GeometryFor(a).cluster > 0) return 0;
    return static_cast<size_t>((a.m * a.k + 255) / 256 * 256);
}

bool Tcgen05Supported(int dtype, const LinearArgs& a) {
    if (a.zero_points) return false;                          // non-zero zero points: the CUDA-core kernels
    if (a.k % 16 != 0) return false;                          // TMA row pitch of the K-major activation tile
    if (!a.trans_b && a.n % 16 != 0) return false;            // TMA row pitch of [K,N] weights
    if (reinterpret_cast<uintptr_t>(a.w) % 16 != 0) return false;
    if (a.a_dtype == 0 && reinterpret_cast<uintptr_t>(a.a) % 16 != 0) return false;
    if (a.k < 32 || a.m < 1 || a.n < 1) return false;
    if (a.m > 0x7fffffff || a.n > 0x7fffffff || a.k > 0x7fffffff) return false;
    (void)dtype;
    return true;
}

// The four-/one-channel epilogues have a direct path when no bias, alpha or beta is in play (a fused output Cast is
// fine for FP8); that path also writes the peer replicas.
static bool DirectEpilogue(bool int8, const Fp8Epilogue& fe, const Int8Epilogue& ie) {
    if (int8) return ie.bias_mode == FTH_B200_BIAS_NONE && ie.out_dtype == 0 && !(ie.is_gemm && (ie.alpha != 1.0f || ie.beta != 1.0f));
    return fe.bias_mode == FTH_B200_BIAS_NONE && !(fe.is_gemm && fe.alpha != 1.0f);
}

bool Tcgen05StoresToPeers(int dtype, const LinearArgs& a, const Fp8Epilogue& fe, const Int8Epilogue& ie) {
    const TcGeometry g = GeometryFor(a);
    return g.swap && (g.cluster > 0 || g.split > 1) && DirectEpilogue(dtype == FTH_B200_INT8, fe, ie);
}

size_t Tcgen05ScratchBytes(int dtype, const LinearArgs& a) {
    (void)dtype;
    const TcGeometry g = GeometryFor(a);
    if (g.cluster > 0) return 0;
    return PrologueBytes(a) + (g.split == 1 ? 0 : static_cast<size_t>(g.split) * g.q_total * g.p_pad * 4);
}

int LaunchLinearTcgen05(int dtype, const LinearArgs& a_in, const Fp8Epilogue& fe, const Int8Epilogue& ie, void* scratch_in,
                        size_t scratch_bytes, cudaStream_t stream) {
    if (!Tcgen05Supported(dtype, a_in)) return FTH_B200_ERR_UNSUPPORTED;
    const TcGeometry g = GeometryFor(a_in);
    const size_t need = Tcgen05ScratchBytes(dtype, a_in);
    if (need > 0 && (scratch_in == nullptr || scratch_bytes < need || reinterpret_cast<uintptr_t>(scratch_in) % 256 != 0)) return FTH_B200_ERR_INVALID;
    const bool int8 = dtype == FTH_B200_INT8;
    LinearArgs a = a_in;
    void* scratch = scratch_in;
    if (a.a_dtype != 0 && g.cluster == 0) {
        int rc;
        if (int8) rc = LaunchQuantizePerTensor(a.a_dtype, a.a, ie.a_scale, ie.a_zp, static_cast<int8_t*>(scratch_in), a.m * a.k, stream);
        else rc = fth_b200_cast(a.a_dtype, a.a, 1.0f, dtype, scratch_in, a.a_scale, a.m * a.k, stream);
        if (rc != FTH_B200_OK) return rc;
        a.a = scratch_in;
        a.a_dtype = 0;
        scratch = static_cast<uint8_t*>(scratch_in) + PrologueBytes(a_in);
    }
    const bool weights_mn = !a.trans_b;

    CUtensorMap map_w, map_a, map_p, map_q;
    const uint32_t w_rows_box = g.swap ? kBlockP : 256;
    bool ok;
    if (weights_mn) ok = CachedMap(&map_w, a.w, static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.k), 128, 128);
    else ok = CachedMap(&map_w, a.w, static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.n), 128, w_rows_box);
    if (a.a_dtype != 0) map_a = map_w;  // cluster kernel with in-kernel conversion: the activation map is unused
    else ok = ok && CachedMap(&map_a, a.a, static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.m), 128,
                              g.swap ? static_cast<uint32_t>(g.bq) : kBlockP);
    if (!ok) return FTH_B200_ERR_CUDA;
    map_p = g.swap ? map_w : map_a;
    map_q = g.swap ? map_a : map_w;

    TcParams p;
    p.args = a;
    p.swap = g.swap;
    p.p_total = g.p_total; p.q_total = g.q_total; p.p_tiles = g.p_tiles; p.q_tiles = g.q_tiles;
    p.ring_stages = 0;
    p.split = g.split; p.chunk_blocks = g.chunk_blocks; p.k_blocks = g.k_blocks; p.units = g.units;
    p.p_pad = g.p_pad;
    p.e4m3 = dtype == FTH_B200_FP8E4M3;
    if (int8) p.fast = ie.bias_mode == FTH_B200_BIAS_NONE && ie.out_dtype == 0 && !(ie.is_gemm && (ie.alpha != 1.0f || ie.beta != 1.0f));
    else p.fast = fe.bias_mode == FTH_B200_BIAS_NONE && fe.out_dtype == 0 && !(fe.is_gemm && fe.alpha != 1.0f);
    p.fast4 = DirectEpilogue(int8, fe, ie);
    p.a_inv = int8 ? 0.0f : ExactReciprocal(a.a_scale);
    p.out_inv = int8 ? 0.0f : ExactReciprocal(fe.out_scale);
    p.scratch = scratch;
    p.status = DeviceStatusPtr();
    // operand formats: kind::f8f6f4 0 = E4M3, 1 = E5M2; kind::i8 1 = signed 8-bit.  D: 1 = F32, 2 = S32.
    const uint32_t fmt = int8 ? 1u : (dtype == FTH_B200_FP8E5M2 ? 1u : 0u);
    const bool p_mn = g.swap && weights_mn;
    const bool q_mn = !g.swap && weights_mn;
    p.idesc = umma::InstrDesc(int8 ? 2u : 1u, fmt, fmt, p_mn, q_mn, kBlockP, static_cast<uint32_t>(g.bq));
    if (g.cluster > 0) {
        return int8 ? LaunchCluster<true>(g, weights_mn, map_p, map_q, p, fe, ie, stream)
                    : LaunchCluster<false>(g, weights_mn, map_p, map_q, p, fe, ie, stream);
    }
    if (!g.swap) {
        // CTA pairs: each CTA stages 128 activation rows and 128 weight columns of a 256 x 256 tile
        CUtensorMap map_w_half = map_w;
        if (!weights_mn && !CachedMap(&map_w_half, a.w, static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.n), 128, 128)) return FTH_B200_ERR_CUDA;
        p.idesc = umma::InstrDesc(int8 ? 2u : 1u, fmt, fmt, false, q_mn, 256, 256);
        if (int8) return weights_mn ? LaunchPairTyped<true, true>(map_a, map_w_half, p, fe, ie, stream)
                                    : LaunchPairTyped<true, false>(map_a, map_w_half, p, fe, ie, stream);
        return weights_mn ? LaunchPairTyped<false, true>(map_a, map_w_half, p, fe, ie, stream)
                          : LaunchPairTyped<false, false>(map_a, map_w_half, p, fe, ie, stream);
    }
    const int rc = int8 ? LaunchForLayout<true>(g, weights_mn, map_p, map_q, p, fe, ie, stream)
                        : LaunchForLayout<false>(g, weights_mn, map_p, map_q, p, fe, ie, stream);
    if (rc != FTH_B200_OK || g.split == 1) return rc;
    const int64_t threads = (g.p_pad / 4) * g.q_total;
    const unsigned blocks = static_cast<unsigned>((threads + 255) / 256);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t err = int8 ? cudaLaunchKernelEx(&cfg, SplitReduceKernel<true>, p, fe, ie)
                                 : cudaLaunchKernelEx(&cfg, SplitReduceKernel<false>, p, fe, ie);
    if (err != cudaSuccess) return FTH_B200_ERR_CUDA;
    NoteLaunch("tcgen05");
    return CheckLaunch();
}

}  // namespace fth
