// Tensor-core linear kernel: tcgen05.mma (kind::f8f6f4 / kind::i8) with accumulators in tensor memory,
// operands staged by TMA into a 128-byte-swizzled shared-memory ring, fused scale / bias / requant / encode
// epilogue.  One persistent CTA per SM, warp-specialised:
//   warp 0     TMA producer (one thread)        — full[] / empty[] mbarriers per ring stage
//   warp 1     TMEM allocation + MMA issue (one thread)
//   warps 2-5  epilogue: tcgen05.ld from one of two accumulator buffers while the next tile's MMAs run
//
// The 128 TMEM lanes carry the "P" operand's rows, the accumulator columns the "Q" operand's rows:
//   normal (M > 128):  P = activations [M,K],  Q = weights       → D[m][n]
//   swapped (M <= 128): P = weights,           Q = activations  → D[n][m], so a decode-sized M pads only the
//                       narrow UMMA N dimension (16..128) and the weight stream fills all 128 lanes.
// Weights are consumed in the layout Feather stores them: [K,N] tiles are MN-major operands, [N,K] tiles
// K-major operands — no repacking pass, no second copy of the weights.
//
// Swapped mode splits K into S chunks (S depends on K only) so that a 28672-column weight gives ~1800 work
// units for 148 SMs; partial accumulators go to a global scratch buffer and the CTA delivering the last
// chunk of a tile adds them in chunk order and runs the epilogue (no CTA ever waits for another).
#include "common.cuh"
#include "linear_internal.h"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace fth {
namespace {

constexpr int kBlockP = 128;
constexpr int kBlockK = 128;  // bytes of K per ring stage = one 128-byte swizzle row
constexpr int kThreads = 192;
constexpr int kEpilogueThreads = 128;
constexpr int kPBytes = kBlockP * kBlockK;
constexpr size_t kSmemBudget = 200 * 1024;

struct TcParams {
    LinearArgs args;
    int swap;
    int64_t p_total, q_total;  // extents along TMEM lanes / accumulator columns
    int64_t p_tiles, q_tiles;
    int split;                 // K chunks per tile
    int64_t chunk_blocks;      // 128-byte K blocks per chunk
    int64_t k_blocks;          // ceil(K / 128)
    int64_t units;             // p_tiles * q_tiles * split
    uint32_t idesc;
    int fp8_dtype;
    void* scratch;             // [split][q_total][p_pad] partial accumulators
    int32_t* counters;         // [p_tiles * q_tiles], zero between launches
    int64_t p_pad;
    int* status;
};

template <int BQ>
struct Cfg {
    static constexpr int kQBytes = BQ * kBlockK;
    static constexpr int kStageBytes = kPBytes + kQBytes;
    static constexpr int kStagesRaw = static_cast<int>(kSmemBudget / kStageBytes);
    static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
    static constexpr uint32_t kTmemCols = 2 * BQ < 32 ? 32 : 2 * BQ;
    static constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void EpilogueBarrier() { asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory"); }

// Writes one finished accumulator value through the shared epilogue helpers.
template <bool INT8>
__device__ __forceinline__ void StoreOne(const Fp8Epilogue& fe, const Int8Epilogue& ie, int fp8_dtype, int64_t m, int64_t n,
                                         uint32_t raw) {
    if constexpr (INT8) {
        StoreInt8Result(ie, m, n, static_cast<int32_t>(raw), 0, 0);
    } else {
        if (fp8_dtype == FTH_B200_FP8E4M3) StoreFp8Result<FTH_B200_FP8E4M3>(fe, m, n, __uint_as_float(raw));
        else StoreFp8Result<FTH_B200_FP8E5M2>(fe, m, n, __uint_as_float(raw));
    }
}

template <bool INT8, bool P_MN, bool Q_MN, int BQ>
__global__ void __launch_bounds__(kThreads, 1)
LinearTcgen05Kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q, TcParams p,
                    Fp8Epilogue fe, Int8Epilogue ie) {
    using C = Cfg<BQ>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(C::kStages) * C::kStageBytes);
    uint64_t* empty = full + C::kStages;
    uint64_t* tmem_full = empty + C::kStages;   // [2]
    uint64_t* tmem_empty = tmem_full + 2;       // [2]
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    int32_t* last_flag = reinterpret_cast<int32_t*>(tmem_base_slot + 1);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) { MbarInit(&full[s], 1); MbarInit(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { MbarInit(&tmem_full[b], 1); MbarInit(&tmem_empty[b], 4); }
        FenceBarrierInit();
    }
    if (warp == 1) umma::TmemAlloc(tmem_base_slot, C::kTmemCols);
    umma::FenceBeforeThreadSync();
    __syncthreads();
    umma::FenceAfterThreadSync();
    const uint32_t tmem_base = *tmem_base_slot;

    // unit → (p tile, q tile, K chunk); q tile varies fastest after the chunk so CTAs running together share
    // the same weight rows through L2 in normal mode.
    auto decode_unit = [&](int64_t u, int64_t* pt, int64_t* qt, int* s) {
        *s = static_cast<int>(u % p.split);
        const int64_t t = u / p.split;
        if (p.swap) { *qt = t % p.q_tiles; *pt = t / p.q_tiles; }
        else { *pt = t % p.p_tiles; *qt = t / p.p_tiles; }
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
                    if constexpr (Q_MN) {
#pragma unroll
                        for (int j = 0; j < (BQ + 127) / 128; ++j) TmaLoad2D(qs + j * 16384, &map_q, q0 + j * 128, k0, &full[stage]);
                    } else {
                        TmaLoad2D(qs, &map_q, k0, q0, &full[stage]);
                    }
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
                const int acc = static_cast<int>(iter & 1);
                const uint32_t acc_phase = static_cast<uint32_t>((iter >> 1) & 1);
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
                        const uint64_t b_desc = Q_MN ? umma::SmemDesc(qs + ks * 4096, 16384, 1024) : umma::SmemDesc(qs + ks * 32, 16, 1024);
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
        const int et = threadIdx.x - 64;            // 0..127
        const int lane_group = warp & 3;            // TMEM lanes 32*lane_group .. +31 belong to this warp
        const int row = lane_group * 32 + lane;     // row inside the P tile
        bool failed = false;
        int64_t iter = 0;
        for (int64_t u = blockIdx.x; u < p.units; u += gridDim.x, ++iter) {
            int64_t pt, qt; int s;
            decode_unit(u, &pt, &qt, &s);
            const int acc = static_cast<int>(iter & 1);
            const uint32_t acc_phase = static_cast<uint32_t>((iter >> 1) & 1);
            if (!failed && !MbarWait(&tmem_full[acc], acc_phase, p.status, 13, acc)) failed = true;
            umma::FenceAfterThreadSync();
            const int64_t pg = pt * kBlockP + row;
            const int64_t q_begin = qt * BQ;
            const int64_t q_left = p.q_total - q_begin;
            const int q_count = static_cast<int>(q_left < BQ ? q_left : BQ);
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + static_cast<uint32_t>(acc * BQ);
#pragma unroll 1
            for (int c0 = 0; c0 < BQ; c0 += 16) {
                if (c0 >= q_count) break;  // uniform across the CTA
                uint32_t v[16];
                umma::TmemLoad16(taddr + c0, v);
                umma::TmemLoadWait();
                if (pg < p.p_total) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (c0 + j >= q_count) break;
                        const int64_t qg = q_begin + c0 + j;
                        if (p.split == 1) {
                            if (p.swap) StoreOne<INT8>(fe, ie, p.fp8_dtype, qg, pg, v[j]);
                            else StoreOne<INT8>(fe, ie, p.fp8_dtype, pg, qg, v[j]);
                        } else {
                            static_cast<uint32_t*>(p.scratch)[(static_cast<int64_t>(s) * p.q_total + qg) * p.p_pad + pg] = v[j];
                        }
                    }
                }
            }
            // accumulator buffer drained: hand it back to the MMA warp
            umma::FenceBeforeThreadSync();
            __syncwarp();
            if (lane == 0) MbarArrive(&tmem_empty[acc]);

            if (p.split > 1) {
                __threadfence();
                EpilogueBarrier();
                const int64_t tile = pt * p.q_tiles + qt;
                if (et == 0) {
                    const int32_t ticket = atomicAdd(&p.counters[tile], 1);
                    *last_flag = (ticket == p.split - 1);
                    if (ticket == p.split - 1) p.counters[tile] = 0;
                }
                EpilogueBarrier();
                if (*last_flag && pg < p.p_total) {
                    __threadfence();
                    for (int c = 0; c < q_count; ++c) {
                        const int64_t qg = q_begin + c;
                        uint32_t raw;
                        if constexpr (INT8) {
                            int32_t sum = 0;
                            for (int ss = 0; ss < p.split; ++ss)
                                sum += __ldcg(&static_cast<const int32_t*>(p.scratch)[(static_cast<int64_t>(ss) * p.q_total + qg) * p.p_pad + pg]);
                            raw = static_cast<uint32_t>(sum);
                        } else {
                            float sum = 0.0f;
                            for (int ss = 0; ss < p.split; ++ss)
                                sum += __ldcg(&static_cast<const float*>(p.scratch)[(static_cast<int64_t>(ss) * p.q_total + qg) * p.p_pad + pg]);
                            raw = __float_as_uint(sum);
                        }
                        if (p.swap) StoreOne<INT8>(fe, ie, p.fp8_dtype, qg, pg, raw);
                        else StoreOne<INT8>(fe, ie, p.fp8_dtype, pg, qg, raw);
                    }
                }
                EpilogueBarrier();
            }
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
// host side
// ---------------------------------------------------------------------------------------------------------
int SwapBlockQ(int64_t m) { return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128; }

struct TcGeometry {
    bool swap;
    int bq;
    int split;
    int64_t chunk_blocks, k_blocks, p_total, q_total, p_tiles, q_tiles, units, p_pad;
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
    return g;
}

size_t CounterBytes(const TcGeometry& g) { return static_cast<size_t>((g.p_tiles * g.q_tiles * 4 + 255) / 256 * 256); }

int SmCountTc() {
    static int count = 0;
    if (count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) count = kNumSms;
    }
    return count;
}

template <bool INT8, bool P_MN, bool Q_MN, int BQ>
int LaunchTyped(const CUtensorMap& map_p, const CUtensorMap& map_q, const TcParams& p, const Fp8Epilogue& fe,
                const Int8Epilogue& ie, cudaStream_t stream) {
    auto kernel = LinearTcgen05Kernel<INT8, P_MN, Q_MN, BQ>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg<BQ>::kSmemBytes)) != cudaSuccess) return FTH_B200_ERR_CUDA;
        configured = true;
    }
    const int grid = static_cast<int>(p.units < SmCountTc() ? p.units : SmCountTc());
    kernel<<<grid, kThreads, Cfg<BQ>::kSmemBytes, stream>>>(map_p, map_q, p, fe, ie);
    NoteLaunch("tcgen05");
    return CheckLaunch();
}

template <bool INT8>
int LaunchForLayout(const TcGeometry& g, bool weights_mn, const CUtensorMap& map_p, const CUtensorMap& map_q,
                    const TcParams& p, const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream) {
    if (!g.swap) {
        return weights_mn ? LaunchTyped<INT8, false, true, 256>(map_p, map_q, p, fe, ie, stream)
                          : LaunchTyped<INT8, false, false, 256>(map_p, map_q, p, fe, ie, stream);
    }
#define FTH_SWAP_CASE(BQV)                                                                                   \
    case BQV:                                                                                                \
        return weights_mn ? LaunchTyped<INT8, true, false, BQV>(map_p, map_q, p, fe, ie, stream)             \
                          : LaunchTyped<INT8, false, false, BQV>(map_p, map_q, p, fe, ie, stream);
    switch (g.bq) {
        FTH_SWAP_CASE(16) FTH_SWAP_CASE(32) FTH_SWAP_CASE(64) FTH_SWAP_CASE(128)
        default: return FTH_B200_ERR_INVALID;
    }
#undef FTH_SWAP_CASE
}

}  // namespace

bool Tcgen05Supported(int dtype, const LinearArgs& a) {
    if (a.a_dtype != 0 || a.zero_points) return false;       // fused Cast / QuantizeLinear prologue, zero points: other kernels
    if (a.k % 16 != 0) return false;                          // TMA row pitch of the K-major activation tile
    if (!a.trans_b && a.n % 16 != 0) return false;            // TMA row pitch of [K,N] weights
    if (reinterpret_cast<uintptr_t>(a.w) % 16 != 0 || reinterpret_cast<uintptr_t>(a.a) % 16 != 0) return false;
    if (a.k < 32 || a.m < 1 || a.n < 1) return false;
    if (a.m > 0x7fffffff || a.n > 0x7fffffff || a.k > 0x7fffffff) return false;
    (void)dtype;
    return true;
}

size_t Tcgen05ScratchBytes(int dtype, const LinearArgs& a) {
    (void)dtype;
    const TcGeometry g = GeometryFor(a);
    if (g.split == 1) return 0;
    return CounterBytes(g) + static_cast<size_t>(g.split) * g.q_total * g.p_pad * 4;
}

int LaunchLinearTcgen05(int dtype, const LinearArgs& a, const Fp8Epilogue& fe, const Int8Epilogue& ie, void* scratch,
                        size_t scratch_bytes, cudaStream_t stream) {
    if (!Tcgen05Supported(dtype, a)) return FTH_B200_ERR_UNSUPPORTED;
    const TcGeometry g = GeometryFor(a);
    if (g.split > 1 && (scratch == nullptr || scratch_bytes < Tcgen05ScratchBytes(dtype, a))) return FTH_B200_ERR_INVALID;
    const bool int8 = dtype == FTH_B200_INT8;
    const bool weights_mn = !a.trans_b;

    CUtensorMap map_w, map_a, map_p, map_q;
    const uint32_t w_rows_box = g.swap ? kBlockP : 256;
    bool ok;
    if (weights_mn) ok = MakeTensorMap2D(&map_w, a.w, static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.n), 128, 128, TmaSwizzle::k128B);
    else ok = MakeTensorMap2D(&map_w, a.w, static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.k), 128, w_rows_box, TmaSwizzle::k128B);
    ok = ok && MakeTensorMap2D(&map_a, a.a, static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.m), static_cast<uint64_t>(a.k), 128,
                               g.swap ? static_cast<uint32_t>(g.bq) : kBlockP, TmaSwizzle::k128B);
    if (!ok) return FTH_B200_ERR_CUDA;
    map_p = g.swap ? map_w : map_a;
    map_q = g.swap ? map_a : map_w;

    TcParams p;
    p.args = a;
    p.swap = g.swap;
    p.p_total = g.p_total; p.q_total = g.q_total; p.p_tiles = g.p_tiles; p.q_tiles = g.q_tiles;
    p.split = g.split; p.chunk_blocks = g.chunk_blocks; p.k_blocks = g.k_blocks; p.units = g.units;
    p.p_pad = g.p_pad;
    p.fp8_dtype = dtype;
    p.counters = static_cast<int32_t*>(scratch);
    p.scratch = scratch ? static_cast<uint8_t*>(scratch) + CounterBytes(g) : nullptr;
    p.status = DeviceStatusPtr();
    // operand formats: kind::f8f6f4 0 = E4M3, 1 = E5M2; kind::i8 1 = signed 8-bit.  D: 1 = F32, 2 = S32.
    const uint32_t fmt = int8 ? 1u : (dtype == FTH_B200_FP8E5M2 ? 1u : 0u);
    const bool p_mn = g.swap && weights_mn;
    const bool q_mn = !g.swap && weights_mn;
    p.idesc = umma::InstrDesc(int8 ? 2u : 1u, fmt, fmt, p_mn, q_mn, kBlockP, static_cast<uint32_t>(g.bq));
    return int8 ? LaunchForLayout<true>(g, weights_mn, map_p, map_q, p, fe, ie, stream)
                : LaunchForLayout<false>(g, weights_mn, map_p, map_q, p, fe, ie, stream);
}

}  // namespace fth
