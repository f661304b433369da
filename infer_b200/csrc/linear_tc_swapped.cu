// Persistent weight-streaming kernel for M <= 128 (operands swapped: weights on the 128 TMEM lanes, activations on a
// 16..128-wide UMMA N) and the second pass of its split-K.  See linear_tcgen05.cu for how the kernel families divide the shapes.
#include "linear_tc.cuh"

namespace fth {
namespace tc {
namespace {

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
    // BQ <= 32 also has the folded form (all K chunks of a tile in one CTA, one accumulator per chunk): 8 x 16 or 4 x 32 columns
    static constexpr uint32_t kTmemCols = BQ == 16 ? 128 : kTmemColsRaw;
    static constexpr int kEpilogueThreads = 128;
    static constexpr int kThreads = 64 + kEpilogueThreads;
    static constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
};

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
    TouchConstantLines(p);
    if constexpr (INT8) TouchConstantLines(ie);
    else TouchConstantLines(fe);
    // Everything above (barriers, tensor memory, parameters) overlapped the tail of the previous kernel in the stream.
    // The activations may be that kernel's output and the output buffer may be its input: the producer thread and the
    // epilogue warps wait for it (griddepcontrol.wait, below) before they read the one or write the other.  The MMA
    // thread touches shared and tensor memory only.

    // unit → (p tile, q tile, K chunk).  [K,N] weights walk the column tiles fastest (chunk-major): the CTAs running
    // together then read whole contiguous weight rows of one K range, which keeps DRAM pages open; with [N,K]
    // weights the chunks of one tile are the contiguous direction, so the chunk index varies fastest instead.
    // Folded form (p.fold): a unit is a whole tile; its CTA walks the chunks s = 0 .. split-1 in turn, each into an
    // accumulator of its own, and the epilogue adds them in chunk order — the sums the reduce pass would form.
    auto decode_unit = [&](int64_t u, int64_t* pt, int64_t* qt, int* s) {
        int64_t t;
        if (p.fold) {
            *s = 0;
            t = u;
        } else if (P_MN) {
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
    const int chunks_per_unit = p.fold ? p.split : 1;

    if (warp == 0) {
        // ================================ TMA producer ================================
        if (lane == 0) {
            TmaPrefetchDescriptor(&map_p);
            TmaPrefetchDescriptor(&map_q);
            // Weights that nothing earlier in the stream writes are fetched before the dependency wait — one ring-full per
            // CTA (the first pass over the ring finds every stage free): the weight half of each stage first, the activation
            // half behind the wait.  A step that follows a short kernel (the activation coming in from the host, a norm in
            // front of an lm-head) then starts with its pipeline full.
            // pass 0: the weight tiles of the first `early` K blocks; pass 1: everything else, in the same order
            bool failed = false;
            auto produce = [&](int pass, int early) {
                int stage = 0;
                uint32_t phase = 0;
                int count = 0;
                for (int64_t u = blockIdx.x; u < p.units && !failed; u += gridDim.x) {
                    int64_t pt, qt; int s0;
                    decode_unit(u, &pt, &qt, &s0);
                    for (int s = s0; s < s0 + chunks_per_unit && !failed; ++s) {
                        const int64_t nb = blocks_of(s);
                        for (int64_t kb = 0; kb < nb; ++kb, ++count) {
                            const bool fetched_early = count < early;
                            if (pass == 0 && !fetched_early) return;
                            if (!fetched_early && !MbarWait(&empty[stage], phase ^ 1u, p.status, 10, stage)) { failed = true; break; }
                            const int32_t k0 = static_cast<int32_t>((static_cast<int64_t>(s) * p.chunk_blocks + kb) * kBlockK);
                            const int32_t p0 = static_cast<int32_t>(pt * kBlockP);
                            const int32_t q0 = static_cast<int32_t>(qt * BQ);
                            uint8_t* ps = ring + static_cast<size_t>(stage) * C::kStageBytes;
                            uint8_t* qs = ps + kPBytes;
                            if (pass == 0 || !fetched_early) {
                                MbarExpectTx(&full[stage], C::kStageBytes);  // both halves; the stage completes with the second
                                if constexpr (P_MN) TmaLoad2D(ps, &map_p, p0, k0, &full[stage]);
                                else TmaLoad2D(ps, &map_p, k0, p0, &full[stage]);
                            }
                            if (pass == 1) TmaLoad2D(qs, &map_q, k0, q0, &full[stage]);
                            if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                        }
                    }
                }
            };
            const int early = p.args.w_static ? C::kStages : 0;
            if (early > 0) produce(0, early);
            asm volatile("griddepcontrol.wait;" ::: "memory");
            produce(1, early);
        }
    } else if (warp == 1) {
        // ================================ MMA issuer ================================
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool failed = false;
            int64_t iter = 0;
            for (int64_t u = blockIdx.x; u < p.units && !failed; u += gridDim.x, ++iter) {
                int64_t pt, qt; int s0;
                decode_unit(u, &pt, &qt, &s0);
                // folded: the chunks' accumulators together are the one buffer, handed over once per tile
                const int acc = p.fold ? 0 : static_cast<int>(iter % kAcc);
                const uint32_t acc_phase = static_cast<uint32_t>((p.fold ? iter : iter / kAcc) & 1);
                if (!MbarWait(&tmem_empty[acc], acc_phase ^ 1u, p.status, 11, acc)) { failed = true; break; }
                umma::FenceAfterThreadSync();
                for (int s = s0; s < s0 + chunks_per_unit && !failed; ++s) {
                const int64_t nb = blocks_of(s);
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>((p.fold ? s : acc) * BQ);
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
                }
                if (!failed) umma::Commit(&tmem_full[acc]);
            }
        }
    } else {
        // ================================ epilogue ================================
        asm volatile("griddepcontrol.wait;" ::: "memory");  // the output buffer (and the scratch) may still be read by the kernel in front
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
        // Column shard, folded form: this kernel stores into the other GPUs' buffers itself, so it also carries the step
        // signalling — every rank must have published the previous step before the first such store, and the last block
        // to finish publishes this one.  (The flags polled here are in this GPU's memory.)
        const bool signalling = p.fold && p.args.signal.world > 0;
        uint32_t gather_step = 0;
        if (signalling) {
            gather_step = GatherStep(p.args.signal);
            if (et < p.args.signal.world) GatherWaitPrevious(p.args.signal, et, gather_step, p.status);
            EpilogueBarrier<C::kEpilogueThreads>();
        }

        for (int64_t u = blockIdx.x; u < p.units; u += gridDim.x, ++iter) {
            int64_t pt, qt; int s;
            decode_unit(u, &pt, &qt, &s);
            const int acc = p.fold ? 0 : static_cast<int>(iter % kAcc);
            const uint32_t acc_phase = static_cast<uint32_t>((p.fold ? iter : iter / kAcc) & 1);
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
                    // (only the folded form has replicas on other GPUs to write: without it a copy follows the launch)
                    if (group_ok) {
                        if ((lane & 3) == 0) {
                            if (p.fold) StoreWithPeers(p.args.peers, reinterpret_cast<uint32_t*>(dst), word);
                            else *reinterpret_cast<uint32_t*>(dst) = word;
                        }
                    } else if (row_ok) {
                        if (p.fold) StoreWithPeers(p.args.peers, dst + (lane & 3), static_cast<uint8_t>(b[j]));
                        else dst[lane & 3] = static_cast<uint8_t>(b[j]);
                    }
                }
            };

            if (!failed && !MbarWait(&tmem_full[acc], acc_phase, p.status, 13, acc)) failed = true;
            umma::FenceAfterThreadSync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + static_cast<uint32_t>(acc * BQ);
            if constexpr (BQ <= 32) {
                if (p.fold && !failed) {
                    // four activation rows at a time: the chunks' partial accumulators, all loads in flight before the
                    // first add, then summed in chunk order starting from +0, exactly as the reduce pass does (chunks
                    // beyond the split are skipped, not added as zeros)
#pragma unroll 1
                    for (int c0 = 0; c0 < q_count; c0 += 4) {
                        uint32_t t[8][4];
#pragma unroll
                        for (int ss = 0; ss < 8; ++ss)
                            if (ss < p.split) umma::TmemLoad4(taddr + static_cast<uint32_t>(ss * BQ + c0), t[ss]);
                        umma::TmemLoadWait();
                        uint32_t v[16];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if constexpr (INT8) {
                                int32_t sum = 0;
#pragma unroll
                                for (int ss = 0; ss < 8; ++ss) sum += ss < p.split ? static_cast<int32_t>(t[ss][j]) : 0;
                                v[j] = static_cast<uint32_t>(sum);
                            } else {
                                float sum = 0.0f;  // as the reduce pass starts
#pragma unroll
                                for (int ss = 0; ss < 8; ++ss)
                                    if (ss < p.split) sum += __uint_as_float(t[ss][j]);
                                v[j] = __float_as_uint(sum);
                            }
                        }
#pragma unroll
                        for (int j = 4; j < 16; ++j) v[j] = 0u;
                        finish(v, c0, q_count - c0 < 4 ? q_count - c0 : 4);
                    }
                }
            }
#pragma unroll 1
            for (int c0 = 0; c0 < BQ; c0 += 16) {
                if (p.fold) break;
                // uniform across the warp; after a wait has given up the accumulator is not valid: nothing is read or
                // stored any more (the status word tells the host), the loop only keeps handing buffers back
                if (c0 >= q_count || failed) break;
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
        if (signalling) {
            EpilogueBarrier<C::kEpilogueThreads>();  // every epilogue thread's stores are issued
            if (et == 0) GatherArriveAndPublish(p.args.signal, gather_step, gridDim.x);
        }
    }

    umma::FenceBeforeThreadSync();
    __syncthreads();
    if (warp == 1) {
        umma::FenceAfterThreadSync();
        umma::TmemDealloc(tmem_base, C::kTmemCols);
    }
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
    // partial sums are visible.  The parameters are fetched while it runs.
    TouchConstantLines(p);
    if constexpr (INT8) TouchConstantLines(ie);
    else TouchConstantLines(fe);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Column-sharded projection with the gather's signalling folded in: every rank must have published the previous
    // step before this pass stores into the peers' buffers; the last block of the pass publishes this step.
    const bool signalling = p.args.signal.world > 0;
    uint32_t gather_step = 0;
    if (signalling) {
        gather_step = GatherStep(p.args.signal);
        if (threadIdx.x < p.args.signal.world) GatherWaitPrevious(p.args.signal, threadIdx.x, gather_step, p.status);
        __syncthreads();
    }
    const int64_t groups = p.p_pad / 4;
    const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    const int64_t q = idx / groups;
    const int64_t p4 = (idx % groups) * 4;
    const bool valid = idx < groups * p.q_total && p4 < p.p_total;
    if (!valid && p.args.argmax_keys == nullptr && !signalling) return;
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
    if (signalling) {
        // This pass ends with a system-scope fence and the flag stores: the next kernel in the stream is released here,
        // behind the output stores, so that its launch and set-up overlap that tail (it touches no data, scratch
        // included, before this grid has completed).  Releasing it at the start of the pass, or at all when there is no
        // such tail, costs more than it gains: thread blocks of the next weight-streaming kernel moving in slow this
        // pass down (K = 8192, N = 28672, M = 1 on one GPU: 43.9 us per step with an early release, 42.1 us without).
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        __syncthreads();
        if (threadIdx.x == 0) GatherArriveAndPublish(p.args.signal, gather_step, gridDim.x);
    }
}

template <bool INT8, bool P_MN, int BQ>
int LaunchTyped(const CUtensorMap& map_p, const CUtensorMap& map_q, const TcParams& p, const Fp8Epilogue& fe,
                const Int8Epilogue& ie, cudaStream_t stream) {
    auto kernel = LinearTcgen05Kernel<INT8, P_MN, BQ>;
    if (EnsureDynamicSmem(reinterpret_cast<const void*>(kernel), Cfg<BQ>::kSmemBytes) != FTH_B200_OK) return FTH_B200_ERR_CUDA;
    const int64_t slots = static_cast<int64_t>(SmCount()) * Cfg<BQ>::kCtasPerSm;
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

}  // namespace

int LaunchSwapped(bool int8, const TcGeometry& g, bool weights_mn, const CUtensorMap& map_p, const CUtensorMap& map_q, const TcParams& p,
                  const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream) {
    const int rc = int8 ? LaunchForLayout<true>(g, weights_mn, map_p, map_q, p, fe, ie, stream)
                        : LaunchForLayout<false>(g, weights_mn, map_p, map_q, p, fe, ie, stream);
    if (rc != FTH_B200_OK || g.split == 1 || p.fold) return rc;
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

}  // namespace tc
}  // namespace fth
