#include "linear_tc.cuh"

namespace fth {
namespace tc {
namespace {

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
//
// Column shards with replicas on other GPUs: 16-byte stores from registers, one row per lane, cross NVLink as 16-byte
// writes (measured 105-135 GB/s per GPU, so the sharded M = 4096 step was slower than the unsharded one).  With replicas
// the epilogue therefore puts the CTA's 128 x 256 output tile into shared memory (the sixth ring stage is given up for
// it) and one thread sends it to this GPU's buffer and to every replica as tile stores (cp.async.bulk.tensor, no
// multicast): full rows of 256 bytes per request, and the copy of tile i overlaps the MMAs and the epilogue of tile i+1.
// SM-issued stores to seven replicas still top out near 280 GB/s per GPU (measured, eight GPUs).  Where the caller has
// an NVLink multicast mapping of all ranks' buffers, the tile goes there ONCE instead (multimem.st from the epilogue
// threads, 512 contiguous bytes per warp): the switch replicates it, and a rank's links carry its output one time, not
// seven.
// ---------------------------------------------------------------------------------------------------------
struct PairCfg {
    static constexpr int kTileN = 256;
    static constexpr int kHalfN = 128;                          // B columns staged by one CTA
    static constexpr int kStageBytes = kPBytes + kHalfN * kBlockK;  // 32 KB
    static constexpr int kStages = 6;
    static constexpr int kStagesWithTileStores = 5;             // the last stage's 32 KB hold the output tile
    static constexpr int kOutTileBytes = kBlockP * kTileN;      // 128 rows x 256 one-byte outputs
    static_assert(kOutTileBytes <= kStageBytes, "the output tile takes the place of one ring stage");
    static constexpr uint32_t kTmemCols = 512;                  // two 256-column accumulator buffers
    static constexpr int kEpilogueThreads = 256;
    static constexpr int kThreads = 64 + kEpilogueThreads;
    static constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageBytes + 1024 + 256 + kTileN * 24;
};

template <bool INT8, bool Q_MN>
__global__ void __launch_bounds__(PairCfg::kThreads, 1)
LinearPairKernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                 const __grid_constant__ OutMaps out_maps, TcParams p, Fp8Epilogue fe, Int8Epilogue ie) {
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
    const bool tile_stores = out_maps.count > 0 || out_maps.multicast != nullptr;
    const int stages = tile_stores ? C::kStagesWithTileStores : C::kStages;
    uint8_t* out_tile = ring + static_cast<size_t>(C::kStagesWithTileStores) * C::kStageBytes;  // [128][256], only with tile_stores

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
    TouchConstantLines(p);
    if constexpr (INT8) TouchConstantLines(ie);
    else TouchConstantLines(fe);
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
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
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
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
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
        // gather signalling folded in (column shards): the peers must have published the previous step before the first
        // store into their buffers; this CTA arrives when all its tiles are stored
        uint32_t gather_step = 0;
        if (p.args.signal.world > 0) {
            gather_step = GatherStep(p.args.signal);
            if (et < p.args.signal.world) GatherWaitPrevious(p.args.signal, et, gather_step, p.status);
            EpilogueBarrier<C::kEpilogueThreads>();
        }
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
            if (tile_stores) {  // the stores of the previous tile must have read the shared-memory tile before it is rewritten
                if (et == 0 && out_maps.count > 0) BulkWaitGroupRead0();
                EpilogueBarrier<C::kEpilogueThreads>();
            }
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
                if (tile_stores) {
                    // columns past the end of the row and rows past M are never written: the tile store clips them
                    uint4 w;
                    w.x = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
                    w.y = b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24);
                    w.z = b[8] | (b[9] << 8) | (b[10] << 16) | (b[11] << 24);
                    w.w = b[12] | (b[13] << 8) | (b[14] << 16) | (b[15] << 24);
                    *reinterpret_cast<uint4*>(out_tile + row * C::kTileN + c0) = w;
                } else if (cnt == 16 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                    uint4 w;
                    w.x = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
                    w.y = b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24);
                    w.z = b[8] | (b[9] << 8) | (b[10] << 16) | (b[11] << 24);
                    w.w = b[12] | (b[13] << 8) | (b[14] << 16) | (b[15] << 24);
                    StoreWithPeers(p.args.peers, reinterpret_cast<uint4*>(dst), w);  // peers: a column shard's replicas on other GPUs
                } else {
                    for (int j = 0; j < cnt; ++j) StoreWithPeers(p.args.peers, dst + j, static_cast<uint8_t>(b[j]));
                }
            }
            // this CTA's half of the accumulator buffer is drained: tell the leader's MMA warp
            umma::FenceBeforeThreadSync();
            __syncwarp();
            if (lane == 0) MbarArriveRemote(leader_empty + acc * 8);
            if (tile_stores) {
                FenceProxyAsync();  // this thread's writes to the tile, visible to the copy engine
                EpilogueBarrier<C::kEpilogueThreads>();
                if (out_maps.multicast != nullptr) {
                    // 16 lanes per 256-byte row of the tile, two rows per warp and instruction; n is a multiple of 16
                    if (!failed) {
                        for (int c = et; c < C::kOutTileBytes / 16; c += C::kEpilogueThreads) {
                            const int r = c >> 4, col = (c & 15) * 16;
                            const int64_t gr = mt * 256 + rank * 128 + r;
                            if (gr < p.p_total && col < n_count)
                                MulticastStore16(out_maps.multicast + gr * out_maps.ldo + n_begin + col,
                                                 *reinterpret_cast<const uint4*>(out_tile + r * C::kTileN + col));
                        }
                    }
                } else if (et == 0 && !failed) {
                    const int32_t x = static_cast<int32_t>(n_begin), y = static_cast<int32_t>(mt * 256 + rank * 128);
                    // The destinations are taken in an order that differs from pair to pair and from tile to tile: every GPU
                    // runs this loop at the same time, and all of them starting with the same replica would queue up
                    // on that GPU's links while the others idle.
                    const int first = static_cast<int>((pair_id + iter + p.args.signal.rank) % out_maps.count);
                    for (int i = 0; i < out_maps.count; ++i) {
                        const int d = first + i < out_maps.count ? first + i : first + i - out_maps.count;
                        TmaStore2D(&out_maps.map[d], out_tile, x, y);
                    }
                    BulkCommitGroup();
                }
            }
        }
        if (out_maps.count > 0 && et == 0) {
            BulkWaitGroup0();                                  // every tile is written, here and in the replicas
            asm volatile("fence.proxy.async;" ::: "memory");   // ... and ordered in front of what this thread does next (the step flag)
        }
        if (p.args.signal.world > 0) {
            EpilogueBarrier<C::kEpilogueThreads>();
            if (et == 0) GatherArriveAndPublish(p.args.signal, gather_step, gridDim.x);
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

template <bool INT8, bool Q_MN>
int LaunchPairTyped(const CUtensorMap& map_p, const CUtensorMap& map_q, const OutMaps& out_maps, const TcParams& p, const Fp8Epilogue& fe,
                    const Int8Epilogue& ie, cudaStream_t stream) {
    auto kernel = LinearPairKernel<INT8, Q_MN>;
    if (EnsureDynamicSmem(reinterpret_cast<const void*>(kernel), PairCfg::kSmemBytes) != FTH_B200_OK) return FTH_B200_ERR_CUDA;
    const int64_t units = ((p.p_total + 255) / 256) * p.q_tiles;
    const int64_t slots = SmCount() / 2;
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
    if (cudaLaunchKernelEx(&cfg, kernel, map_p, map_q, out_maps, p, fe, ie) != cudaSuccess) return FTH_B200_ERR_CUDA;
    NoteLaunch("tcgen05");
    return CheckLaunch();
}

}  // namespace

int LaunchPair(bool int8, bool weights_mn, const CUtensorMap& map_a, const CUtensorMap& map_w, const OutMaps& out_maps, const TcParams& p,
               const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream) {
    if (int8) return weights_mn ? LaunchPairTyped<true, true>(map_a, map_w, out_maps, p, fe, ie, stream)
                                : LaunchPairTyped<true, false>(map_a, map_w, out_maps, p, fe, ie, stream);
    return weights_mn ? LaunchPairTyped<false, true>(map_a, map_w, out_maps, p, fe, ie, stream)
                      : LaunchPairTyped<false, false>(map_a, map_w, out_maps, p, fe, ie, stream);
}

}  // namespace tc
}  // namespace fth
