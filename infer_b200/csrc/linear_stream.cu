// Persistent weight-streaming GEMV for [K,N] weights (FC / MatMul layout), M <= 2 (FP8) or M <= 4 (INT8).
//
// One CTA per SM.  A producer thread streams 128-row x 128-column weight pieces (16 KB) from HBM into an
// 8-deep shared-memory ring with TMA (cp.async.bulk.tensor, full/empty mbarriers), so 128 KB per SM are in
// flight without costing registers; eight consumer warps read the ring with conflict-free 16-byte loads and
// do the arithmetic on the CUDA cores (FP8: hardware decode + FP32 FMA; INT8: byte transpose + dp4a).
//
// Work is cut into units of (128-column tile) x (one of S K-chunks) that are dealt round-robin to the CTAs,
// fine enough (128 KB at K = 8192) to balance 148 SMs.  A unit's result is a partial sum over its K chunk;
// with S > 1 the partials go to a small global scratch buffer ([S][M][N] accumulators) and the CTA that
// delivers the last chunk of a column tile adds the S partials in chunk order, runs the epilogue and
// resets the tile's arrival counter — no waiting on other CTAs anywhere.  S and the chunk size depend on K
// alone, so a column shard of a weight gives bit-identical results to the same columns of the full weight.
#include <cstring>

#include "common.cuh"
#include "linear_internal.h"
#include "tma.cuh"

namespace fth {
namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;  // + producer warp
constexpr int kTileN = 128;
constexpr int kPieceRows = 128;
constexpr int kStageBytes = kTileN * kPieceRows;  // 16 KB
constexpr int kStages = 8;
constexpr int kMaxSplit = 8;

template <int DTYPE>
struct Acc { using type = float; };
template <>
struct Acc<FTH_B200_INT8> { using type = int32_t; };

struct StreamGeometry {
    int split;        // K chunks per column tile
    int64_t chunk;    // rows per chunk, a multiple of kPieceRows
    int64_t k_pad;    // split * chunk
    int64_t n_tiles;
    int64_t n_pad;    // n_tiles * kTileN
    int64_t units;
};

StreamGeometry GeometryFor(int64_t k, int64_t n) {
    StreamGeometry g;
    int64_t s = k / 128;
    if (s < 1) s = 1;
    if (s > kMaxSplit) s = kMaxSplit;
    int p = 1;
    while (p * 2 <= s) p *= 2;
    g.split = p;
    g.chunk = ((k + p - 1) / p + kPieceRows - 1) / kPieceRows * kPieceRows;
    g.k_pad = g.chunk * p;
    g.n_tiles = (n + kTileN - 1) / kTileN;
    g.n_pad = g.n_tiles * kTileN;
    g.units = g.n_tiles * p;
    return g;
}

__device__ __forceinline__ void ConsumerBarrier() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }

__device__ __forceinline__ void Transpose4x4(uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3, uint32_t (&c)[4]) {
    const uint32_t t0 = __byte_perm(r0, r1, 0x5140);
    const uint32_t t1 = __byte_perm(r2, r3, 0x5140);
    const uint32_t t2 = __byte_perm(r0, r1, 0x7362);
    const uint32_t t3 = __byte_perm(r2, r3, 0x7362);
    c[0] = __byte_perm(t0, t1, 0x5410);
    c[1] = __byte_perm(t0, t1, 0x7632);
    c[2] = __byte_perm(t2, t3, 0x5410);
    c[3] = __byte_perm(t2, t3, 0x7632);
}

struct StreamParams {
    LinearArgs args;
    StreamGeometry geo;
    void* scratch;       // [split][MB][n_pad] accumulators, then (INT8 with zero points) [split][n_pad] column sums
                         // and [split][MB] row sums
    int32_t* counters;   // [n_tiles], zero between launches
    int* status;
    int64_t m0;          // first activation row of this launch
};

template <int DTYPE, int MB>
__global__ void __launch_bounds__(kThreads, 1)
StreamKnKernel(const __grid_constant__ CUtensorMap w_map, StreamParams p, Fp8Epilogue fe, Int8Epilogue ie) {
    using T = typename Acc<DTYPE>::type;
    constexpr bool kInt8 = DTYPE == FTH_B200_INT8;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;                                         // kStages * 16 KB
    uint8_t* act = ring + kStages * kStageBytes;                  // activations: FP32 [MB][k_pad] or int8 permuted
    const size_t act_bytes = static_cast<size_t>(MB) * p.geo.k_pad * (kInt8 ? 1 : 4);
    T* red = reinterpret_cast<T*>(act + ((act_bytes + 127) / 128) * 128);     // [warps][MB][kTileN]
    int32_t* red_csum = reinterpret_cast<int32_t*>(red + kConsumerWarps * MB * kTileN);  // [warps][kTileN]
    int32_t* red_rsum = red_csum + kConsumerWarps * kTileN;       // [warps][MB]
    uint64_t* full = reinterpret_cast<uint64_t*>(red_rsum + kConsumerWarps * MB + 2);
    full = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(full) + 7) & ~uintptr_t(7));
    uint64_t* empty = full + kStages;
    int32_t* last_flag = reinterpret_cast<int32_t*>(empty + kStages);

    const int tid = threadIdx.x;
    const int warp = tid / 32, lane = tid % 32;
    const LinearArgs& args = p.args;
    const StreamGeometry& geo = p.geo;
    const bool need_sums = kInt8 && (ie.a_zp != 0 || ie.w_zps != nullptr);

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            MbarInit(&full[s], 1);
            MbarInit(&empty[s], kConsumerWarps);
        }
        FenceBarrierInit();
    }
    // ---- stage all activation rows of this launch (zero beyond K and beyond M) ----
    if constexpr (kInt8) {
        // byte for row k of piece q goes to word (q*32 + k%32), byte (k%128)/32: a consumer thread's four
        // rows rl, rl+32, rl+64, rl+96 of a piece then sit in one 32-bit word.
        int8_t* a_s = reinterpret_cast<int8_t*>(act);
        for (int64_t idx = tid; idx < MB * geo.k_pad; idx += kThreads) {
            const int64_t m = idx / geo.k_pad, k = idx % geo.k_pad;
            int8_t v = 0;
            if (k < args.k && p.m0 + m < args.m) v = LoadInt8Activation(args.a, (p.m0 + m) * args.k + k, args.a_dtype, ie.a_scale, ie.a_zp);
            const int64_t q = k / kPieceRows, r = k % kPieceRows;
            a_s[m * geo.k_pad + q * kPieceRows + (r % 32) * 4 + r / 32] = v;
        }
    } else {
        float* a_s = reinterpret_cast<float*>(act);
        for (int64_t idx = tid; idx < MB * geo.k_pad; idx += kThreads) {
            const int64_t m = idx / geo.k_pad, k = idx % geo.k_pad;
            float v = 0.0f;
            if (k < args.k && p.m0 + m < args.m) v = LoadActivation<DTYPE>(args.a, (p.m0 + m) * args.k + k, args.a_dtype, args.a_scale);
            a_s[idx] = v;
        }
    }
    __syncthreads();

    const int pieces_per_chunk = static_cast<int>(geo.chunk / kPieceRows);

    if (warp == kConsumerWarps) {
        // =========================== producer ===========================
        if (lane == 0) {
            TmaPrefetchDescriptor(&w_map);
            int stage = 0;
            uint32_t phase = 0;
            bool failed = false;
            for (int64_t u = blockIdx.x; u < geo.units && !failed; u += gridDim.x) {
                const int64_t tile = u / geo.split;
                const int s = static_cast<int>(u % geo.split);
                for (int q = 0; q < pieces_per_chunk; ++q) {
                    const int64_t row0 = s * geo.chunk + static_cast<int64_t>(q) * kPieceRows;
                    if (row0 >= args.k) break;  // consumers skip the same pieces
                    if (!MbarWait(&empty[stage], phase ^ 1u, p.status, 1, stage)) { failed = true; break; }
                    MbarExpectTx(&full[stage], kStageBytes);
                    TmaLoad2D(ring + stage * kStageBytes, &w_map, static_cast<int32_t>(tile * kTileN),
                              static_cast<int32_t>(row0), &full[stage]);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
        return;
    }

    // =========================== consumers ===========================
    const int cgp = tid % 8;   // 16-byte column group inside the 128-column tile
    const int rl = tid / 8;    // row lane 0..31: rows rl, rl+32, rl+64, rl+96 of each piece
    int stage = 0;
    uint32_t phase = 0;
    bool failed = false;  // after a timed-out wait this warp stops waiting but keeps the barrier pattern

    for (int64_t u = blockIdx.x; u < geo.units; u += gridDim.x) {
        const int64_t tile = u / geo.split;
        const int s = static_cast<int>(u % geo.split);
        T acc[MB][16];
        int32_t csum[16];
        int32_t rsum[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            rsum[m] = 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[m][j] = 0;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) csum[j] = 0;

        for (int q = 0; q < pieces_per_chunk; ++q) {
            const int64_t row0 = s * geo.chunk + static_cast<int64_t>(q) * kPieceRows;
            if (row0 >= args.k) break;
            if (!failed && !MbarWait(&full[stage], phase, p.status, 2, stage)) failed = true;
            const uint8_t* st = ring + stage * kStageBytes + cgp * 16;
            uint4 v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = *reinterpret_cast<const uint4*>(st + (rl + 32 * i) * kTileN);
            if constexpr (kInt8) {
                const int32_t* a_w = reinterpret_cast<const int32_t*>(act);
                int32_t aw[MB];
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    aw[m] = a_w[(m * geo.k_pad + row0) / 4 + rl];
                    if (need_sums) rsum[m] = __dp4a(aw[m], 0x01010101, rsum[m]);
                }
                const uint32_t* r0 = reinterpret_cast<const uint32_t*>(&v[0]);
                const uint32_t* r1 = reinterpret_cast<const uint32_t*>(&v[1]);
                const uint32_t* r2 = reinterpret_cast<const uint32_t*>(&v[2]);
                const uint32_t* r3 = reinterpret_cast<const uint32_t*>(&v[3]);
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    uint32_t cw[4];
                    Transpose4x4(r0[c4], r1[c4], r2[c4], r3[c4], cw);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
#pragma unroll
                        for (int m = 0; m < MB; ++m) acc[m][c4 * 4 + j] = __dp4a(static_cast<int32_t>(cw[j]), aw[m], acc[m][c4 * 4 + j]);
                        if (need_sums) csum[c4 * 4 + j] = __dp4a(static_cast<int32_t>(cw[j]), 0x01010101, csum[c4 * 4 + j]);
                    }
                }
            } else {
                const float* a_s = reinterpret_cast<const float*>(act);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t words[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
                    float av[MB];
#pragma unroll
                    for (int m = 0; m < MB; ++m) av[m] = a_s[m * geo.k_pad + row0 + rl + 32 * i];
#pragma unroll
                    for (int wd = 0; wd < 4; ++wd) {
                        const float2 lo = DecodePair<DTYPE>(static_cast<uint16_t>(words[wd] & 0xffffu));
                        const float2 hi = DecodePair<DTYPE>(static_cast<uint16_t>(words[wd] >> 16));
#pragma unroll
                        for (int m = 0; m < MB; ++m) {
                            acc[m][wd * 4 + 0] = fmaf(av[m], lo.x, acc[m][wd * 4 + 0]);
                            acc[m][wd * 4 + 1] = fmaf(av[m], lo.y, acc[m][wd * 4 + 1]);
                            acc[m][wd * 4 + 2] = fmaf(av[m], hi.x, acc[m][wd * 4 + 2]);
                            acc[m][wd * 4 + 3] = fmaf(av[m], hi.y, acc[m][wd * 4 + 3]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) MbarArrive(&empty[stage]);
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }

        // ---- combine the 4 row lanes of a warp (lane bits 3,4), then the 8 warps, in a fixed order ----
#pragma unroll
        for (int off = 8; off <= 16; off <<= 1) {
#pragma unroll
            for (int m = 0; m < MB; ++m) {
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[m][j] += __shfl_xor_sync(0xffffffffu, acc[m][j], off);
                if (need_sums) rsum[m] += __shfl_xor_sync(0xffffffffu, rsum[m], off);
            }
            if (need_sums) {
#pragma unroll
                for (int j = 0; j < 16; ++j) csum[j] += __shfl_xor_sync(0xffffffffu, csum[j], off);
            }
        }
        if (lane < 8) {
#pragma unroll
            for (int m = 0; m < MB; ++m) {
#pragma unroll
                for (int j = 0; j < 16; ++j) red[(warp * MB + m) * kTileN + lane * 16 + j] = acc[m][j];
            }
            if (need_sums) {
#pragma unroll
                for (int j = 0; j < 16; ++j) red_csum[warp * kTileN + lane * 16 + j] = csum[j];
                if (lane == 0) {
#pragma unroll
                    for (int m = 0; m < MB; ++m) red_rsum[warp * MB + m] = rsum[m];
                }
            }
        }
        ConsumerBarrier();

        const bool owner = tid < MB * kTileN;  // MB * 128 <= 256 for MB <= 2; larger MB loops below
        for (int idx = tid; idx < MB * kTileN; idx += kConsumers) {
            const int m = idx / kTileN, c = idx % kTileN;
            T sum = red[(0 * MB + m) * kTileN + c];
#pragma unroll
            for (int w = 1; w < kConsumerWarps; ++w) sum += red[(w * MB + m) * kTileN + c];
            int32_t cs = 0, rs = 0;
            if (need_sums) {
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) { cs += red_csum[w * kTileN + c]; rs += red_rsum[w * MB + m]; }
            }
            const int64_t col = tile * kTileN + c;
            if (geo.split == 1) {
                if (p.m0 + m < args.m && col < args.n) {
                    if constexpr (kInt8) StoreInt8Result(ie, p.m0 + m, col, sum, rs, cs);
                    else StoreFp8Result<DTYPE>(fe, p.m0 + m, col, sum);
                }
            } else {
                T* part = static_cast<T*>(p.scratch);
                part[(static_cast<int64_t>(s) * MB + m) * geo.n_pad + col] = sum;
                if (need_sums) {
                    int32_t* cpart = reinterpret_cast<int32_t*>(part + static_cast<int64_t>(geo.split) * MB * geo.n_pad);
                    int32_t* rpart = cpart + static_cast<int64_t>(geo.split) * geo.n_pad;
                    if (m == 0) cpart[static_cast<int64_t>(s) * geo.n_pad + col] = cs;
                    if (c == 0) rpart[(tile * geo.split + s) * MB + m] = rs;
                }
            }
        }
        (void)owner;
        if (geo.split > 1) {
            __threadfence();
            ConsumerBarrier();
            if (tid == 0) {
                const int32_t ticket = atomicAdd(&p.counters[tile], 1);
                *last_flag = (ticket == geo.split - 1);
                if (ticket == geo.split - 1) p.counters[tile] = 0;  // ready for the next launch
            }
            ConsumerBarrier();
            if (*last_flag) {
                __threadfence();
                const T* part = static_cast<const T*>(p.scratch);
                const int32_t* cpart = reinterpret_cast<const int32_t*>(part + static_cast<int64_t>(geo.split) * MB * geo.n_pad);
                const int32_t* rpart = cpart + static_cast<int64_t>(geo.split) * geo.n_pad;
                for (int idx = tid; idx < MB * kTileN; idx += kConsumers) {
                    const int m = idx / kTileN, c = idx % kTileN;
                    const int64_t col = tile * kTileN + c;
                    if (p.m0 + m >= args.m || col >= args.n) continue;
                    T sum = 0;
                    int32_t cs = 0, rs = 0;
                    for (int ss = 0; ss < geo.split; ++ss) {
                        sum += __ldcg(&part[(static_cast<int64_t>(ss) * MB + m) * geo.n_pad + col]);
                        if (need_sums) {
                            cs += __ldcg(&cpart[static_cast<int64_t>(ss) * geo.n_pad + col]);
                            rs += __ldcg(&rpart[(tile * geo.split + ss) * MB + m]);
                        }
                    }
                    if constexpr (kInt8) StoreInt8Result(ie, p.m0 + m, col, sum, rs, cs);
                    else StoreFp8Result<DTYPE>(fe, p.m0 + m, col, sum);
                }
            }
            ConsumerBarrier();  // last_flag and red are reused by the next unit
        } else {
            ConsumerBarrier();
        }
    }
}

template <int MB, bool INT8>
size_t SmemBytes(const StreamGeometry& g) {
    const size_t act = (static_cast<size_t>(MB) * g.k_pad * (INT8 ? 1 : 4) + 127) / 128 * 128;
    return static_cast<size_t>(kStages) * kStageBytes + act + kConsumerWarps * MB * kTileN * 4 +
           kConsumerWarps * kTileN * 4 + (kConsumerWarps * MB + 2) * 4 + 8 + 2 * kStages * 8 + 16;
}

constexpr size_t kSmemLimit = 227 * 1024;

// Small host-side cache of encoded tensor maps keyed by (pointer, K, N).
struct MapEntry { const void* w; int64_t k, n; CUtensorMap map; };
bool GetWeightMap(const void* w, int64_t k, int64_t n, CUtensorMap* out) {
    thread_local MapEntry cache[8];
    thread_local int next = 0;
    for (const auto& e : cache) {
        if (e.w == w && e.k == k && e.n == n) { *out = e.map; return true; }
    }
    CUtensorMap map;
    if (!MakeTensorMap2D(&map, w, static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(n), kTileN,
                         kPieceRows, TmaSwizzle::kNone)) return false;
    cache[next] = MapEntry{w, k, n, map};
    next = (next + 1) % 8;
    *out = map;
    return true;
}


template <int DTYPE, int MB>
int LaunchStream(const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie, void* scratch,
                 size_t scratch_bytes, cudaStream_t stream) {
    constexpr bool kInt8 = DTYPE == FTH_B200_INT8;
    const StreamGeometry geo = GeometryFor(args.k, args.n);
    const size_t smem = SmemBytes<MB, kInt8>(geo);
    if (smem > kSmemLimit) return FTH_B200_ERR_UNSUPPORTED;
    if (geo.split > 1 && (scratch == nullptr || scratch_bytes < StreamScratchBytes(DTYPE, args))) return FTH_B200_ERR_INVALID;
    CUtensorMap map;
    if (!GetWeightMap(args.w, args.k, args.n, &map)) return FTH_B200_ERR_CUDA;
    auto kernel = StreamKnKernel<DTYPE, MB>;
    if (EnsureDynamicSmem(reinterpret_cast<const void*>(kernel), kSmemLimit) != FTH_B200_OK) return FTH_B200_ERR_CUDA;
    StreamParams p;
    p.args = args;
    p.geo = geo;
    // counters live at the front of the scratch buffer (zeroed once by the owner, kept zero by the kernel)
    p.counters = static_cast<int32_t*>(scratch);
    p.scratch = scratch ? static_cast<uint8_t*>(scratch) + StreamCounterBytes(args) : nullptr;
    p.status = DeviceStatusPtr();
    const int grid = static_cast<int>(geo.units < SmCount() ? geo.units : SmCount());
    for (int64_t m0 = 0; m0 < args.m; m0 += MB) {
        p.m0 = m0;
        kernel<<<grid, kThreads, smem, stream>>>(map, p, fe, ie);
        NoteLaunch("stream");
    }
    return CheckLaunch();
}

}  // namespace

size_t StreamCounterBytes(const LinearArgs& args) {
    const StreamGeometry g = GeometryFor(args.k, args.n);
    return static_cast<size_t>((g.n_tiles * 4 + 255) / 256 * 256);
}

size_t StreamScratchBytes(int dtype, const LinearArgs& args) {
    const StreamGeometry g = GeometryFor(args.k, args.n);
    if (g.split == 1) return 0;
    const int mb = dtype == FTH_B200_INT8 ? 4 : 2;
    size_t bytes = StreamCounterBytes(args) + static_cast<size_t>(g.split) * mb * g.n_pad * 4;
    if (dtype == FTH_B200_INT8) bytes += static_cast<size_t>(g.split) * g.n_pad * 4 + static_cast<size_t>(g.units) * mb * 4;
    return bytes;
}

bool StreamSupported(int dtype, const LinearArgs& args) {
    if (args.trans_b || args.m < 1) return false;
    if (args.m > (dtype == FTH_B200_INT8 ? 4 : 2)) return false;
    if (args.n % 16 != 0 || reinterpret_cast<uintptr_t>(args.w) % 16 != 0) return false;  // TMA: 16-byte base and pitch
    const StreamGeometry g = GeometryFor(args.k, args.n);
    const int mb = args.m;
    const size_t act = static_cast<size_t>(mb > 2 ? 4 : mb) * g.k_pad * (dtype == FTH_B200_INT8 ? 1 : 4);
    return static_cast<size_t>(kStages) * kStageBytes + act + 24 * 1024 <= kSmemLimit;
}

int LaunchLinearStream(int dtype, const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie, void* scratch,
                       size_t scratch_bytes, cudaStream_t stream) {
    if (!StreamSupported(dtype, args)) return FTH_B200_ERR_UNSUPPORTED;
    switch (dtype) {
        case FTH_B200_FP8E4M3:
            return args.m == 1 ? LaunchStream<FTH_B200_FP8E4M3, 1>(args, fe, ie, scratch, scratch_bytes, stream)
                               : LaunchStream<FTH_B200_FP8E4M3, 2>(args, fe, ie, scratch, scratch_bytes, stream);
        case FTH_B200_FP8E5M2:
            return args.m == 1 ? LaunchStream<FTH_B200_FP8E5M2, 1>(args, fe, ie, scratch, scratch_bytes, stream)
                               : LaunchStream<FTH_B200_FP8E5M2, 2>(args, fe, ie, scratch, scratch_bytes, stream);
        case FTH_B200_INT8:
            if (args.m == 1) return LaunchStream<FTH_B200_INT8, 1>(args, fe, ie, scratch, scratch_bytes, stream);
            if (args.m == 2) return LaunchStream<FTH_B200_INT8, 2>(args, fe, ie, scratch, scratch_bytes, stream);
            return LaunchStream<FTH_B200_INT8, 4>(args, fe, ie, scratch, scratch_bytes, stream);
        default: return FTH_B200_ERR_INVALID;
    }
}

}  // namespace fth
