#include "linear_tc.cuh"
#include "rowops.cuh"

namespace fth {
namespace tc {
namespace {

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
    static constexpr int kQBlocks = kClusterQBlocks;                       // K blocks of activations held per CTA
    static constexpr int kQBytes = kQBlocks * BQ * kBlockK;  // 16 KB / 32 KB
    static constexpr int kStages = BQ <= 16 ? 5 : 3;         // weight ring (16 KB per stage), upper limit
    static constexpr int kMaxStages = 8;                     // barrier slots
    static constexpr int kExchangeBytes = kBlockP * BQ * 4;  // partials of this CTA's rows, all chunks (per weight tile)
    static constexpr int kMaxTiles = 2;                      // weight tiles per CTA: a second weight on the same activation
    __host__ __device__ static constexpr uint32_t TmemCols(int tiles) { return tiles * BQ <= 32 ? 32u : 64u; }
    static constexpr int kThreads = 192;
    static constexpr int kNormBytes = 768;                   // a fused QwenRmsNorm: 1 / rms per row + four partial sums per row
    static constexpr size_t kSmemBytes = 1024 + static_cast<size_t>(kStages) * kPBytes + kQBytes + kMaxTiles * kExchangeBytes + 256 + kNormBytes;
    // Ring depth of a launch: its loads (chunk blocks x tiles) at most, and no deeper than lets two CTAs share an SM.
    static int StagesFor(int64_t chunk_blocks, int tiles) {
        const int64_t fixed = 1024 + chunk_blocks * BQ * kBlockK + static_cast<int64_t>(tiles) * kExchangeBytes + 256 + kNormBytes;
        int64_t stages = (113 * 1024 - fixed) / kPBytes;
        if (stages > kStages) stages = kStages;
        if (stages > chunk_blocks * tiles) stages = chunk_blocks * tiles;
        return stages < 1 ? 1 : static_cast<int>(stages);
    }
    static size_t SmemFor(int64_t chunk_blocks, int tiles) {
        return 1024 + static_cast<size_t>(StagesFor(chunk_blocks, tiles)) * kPBytes + static_cast<size_t>(chunk_blocks) * BQ * kBlockK +
               static_cast<size_t>(tiles) * kExchangeBytes + 256 + kNormBytes;
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

// Four activation elements as FP32 from their raw load (BF16 / FP16 / FP32).
__device__ __forceinline__ void WidenFour(int dtype, uint4 raw, float (&x)[4]) {
    if (dtype == FTH_B200_FP32) {
        x[0] = __uint_as_float(raw.x); x[1] = __uint_as_float(raw.y); x[2] = __uint_as_float(raw.z); x[3] = __uint_as_float(raw.w);
    } else if (dtype == FTH_B200_BF16) {
        x[0] = __uint_as_float(raw.x << 16); x[1] = __uint_as_float(raw.x & 0xffff0000u);
        x[2] = __uint_as_float(raw.y << 16); x[3] = __uint_as_float(raw.y & 0xffff0000u);
    } else {
        const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
        const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
        x[0] = lo.x; x[1] = lo.y; x[2] = hi.x; x[3] = hi.y;
    }
}
// The FP8 codes of four BF16-valued activations h (the Cast node in front of the MatMul): encode(h / a_scale).
__device__ __forceinline__ uint32_t CastFour(int e4m3, float a_scale, float a_inv, const float (&h)[4]) {
    float y[4];
    if (a_inv != 0.0f) { for (int i = 0; i < 4; ++i) y[i] = (h[i] != h[i]) ? h[i] : __fmul_rn(h[i], a_inv); }
    else { for (int i = 0; i < 4; ++i) y[i] = (h[i] != h[i]) ? h[i] : __fdiv_rn(h[i], a_scale); }
    return EncodePair(e4m3, y[0], y[1]) | (EncodePair(e4m3, y[2], y[3]) << 16);
}

// decode(code) for the fused Cast behind the MatMul.  Finite codes widen exactly through FP16 in hardware; Inf / NaN
// codes take the software path, whose NaN pattern is the reference's.
static __device__ __noinline__ float DecodeSpecial(int e4m3, uint32_t code) {
    return e4m3 ? Decode<FTH_B200_FP8E4M3>(static_cast<uint8_t>(code)) : Decode<FTH_B200_FP8E5M2>(static_cast<uint8_t>(code));
}
__device__ __forceinline__ float DecodeFast(int e4m3, uint32_t code) {
    const uint32_t mag = code & 0x7fu;
    if (e4m3 ? mag == 0x7fu : mag >= 0x7cu) return DecodeSpecial(e4m3, code);
    const uint16_t in = static_cast<uint16_t>(code & 0xffu);
    uint32_t pair;
    if (e4m3) asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"(in));
    else asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(pair) : "h"(in));
    return __half2float(__ushort_as_half(static_cast<unsigned short>(pair & 0xffffu)));
}

// The decoder-block node in front of the Cast, for four elements, with its own BF16 rounding point(s): QwenRmsNorm
// (x * inv * (weight + offset)) or Mul(SiLU(x), y).  Out of line: it keeps the four-item conversion loop short.
static __device__ __noinline__ void DecoderNodeFour(int prologue, int weight_dtype, float offset, float inv, uint2 raw, uint4 raw2, float (&h)[4]) {
    const float x[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u), __uint_as_float(raw.y << 16),
                        __uint_as_float(raw.y & 0xffff0000u)};
    float y[4];
    WidenFour(prologue == 1 ? weight_dtype : FTH_B200_BF16, raw2, y);
    if (prologue == 1) {
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = DecodeBf16(EncodeBf16Cast(__fmul_rn(__fmul_rn(x[i], inv), __fadd_rn(y[i], offset))));
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float sv = DecodeBf16(rowops::SiluToBf16(x[i]));   // SiLU node
            h[i] = DecodeBf16(EncodeBf16Cast(__fmul_rn(sv, y[i])));   // Mul node
        }
    }
}

// DEC: the decoder-block form — FP8 product of BF16 activations, BF16 out, per-tensor scales, no bias, no peers, no
// selection — with the activation prologue and the finishing step written out for exactly that case (these launches
// are latency-bound: every instruction between the producer's last store and this kernel's own counts), and with the
// operators a decoder block puts around the projection fused in (DecoderFusion).
template <bool INT8, bool P_MN, int BQ, bool DEC>
__global__ void __launch_bounds__(ClusterCfg<BQ>::kThreads, 2)  // (3 per SM for the decoder form: 92 registers; decode step 510 vs 517 us at M = 1 but 892 vs 833 us at M = 16)
LinearClusterKernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_p2,
                    const __grid_constant__ CUtensorMap map_q, TcParams p, Fp8Epilogue fe, Int8Epilogue ie) {
    using C = ClusterCfg<BQ>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // The ring and the activation tiles are sized per launch (p.ring_stages, p.chunk_blocks): a small projection
    // then takes ~30 KB instead of ~100 KB, and the CTAs of the next kernel in the stream can move in early.
    const int stages = p.ring_stages;
    uint8_t* q_tiles = ring + static_cast<size_t>(stages) * kPBytes;            // [chunk_blocks][BQ][128], 128-byte swizzle
    // A CTA may carry a second weight tile, with its own accumulator columns and its own exchange area: the same
    // columns of a second weight on the same activation (gate and up), or — for a weight with up to twice as many tiles
    // as one wave of clusters holds — the tile half the weight further on, so that such a projection is still one launch.
    const int cshift = 31 - __clz(static_cast<int>(ClusterSize()));  // the cluster size is a power of two
    const int tile = static_cast<int>(blockIdx.x >> cshift);
    const int tiles_here = p.tiles_per_cta > 1 && tile + p.second_tile_offset < p.p_tiles ? 2 : 1;
    uint32_t* exchange = reinterpret_cast<uint32_t*>(q_tiles + p.chunk_blocks * (BQ * kBlockK));  // [tile][chunk][L][BQ]
    uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(exchange) + tiles_here * C::kExchangeBytes);
    uint64_t* empty = full + C::kMaxStages;
    uint64_t* q_full = empty + C::kMaxStages;
    uint64_t* tmem_full = q_full + 1;
    uint64_t* x_full = tmem_full + 1;  // counts the bytes peers deliver into `exchange`
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(x_full + 1);
    float* norm_inv = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(full) + 256);  // [<= 32] 1 / rms per activation row
    float* norm_partial = norm_inv + 32;                                                  // [<= 32][4] one partial sum per row and epilogue warp

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const bool convert = p.args.a_dtype != 0;

    if (threadIdx.x == 0) {
        TmaPrefetchDescriptor(&map_p);  // kernel parameters: safe to touch before the previous grid has finished
        if (tiles_here > 1) TmaPrefetchDescriptor(&map_p2);
        if (!convert) TmaPrefetchDescriptor(&map_q);
        for (int s = 0; s < stages; ++s) { MbarInit(&full[s], 1); MbarInit(&empty[s], 1); }
        MbarInit(q_full, convert ? 128 : 1);
        MbarInit(tmem_full, 1);
        MbarInit(x_full, 1);
        FenceBarrierInit();
    }
    const uint32_t tmem_cols = C::TmemCols(tiles_here);
    if (warp == 1) umma::TmemAlloc(tmem_base_slot, tmem_cols);
    umma::FenceBeforeThreadSync();
    __syncthreads();
    umma::FenceAfterThreadSync();
    const uint32_t tmem_base = *tmem_base_slot;
    ClusterArrive();  // "this CTA is running": peers wait for it before they write into our exchange buffer
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const uint32_t rank = ClusterRank();
    const int lshift = 7 - cshift;                         // log2 of L = rows of the tile this CTA finishes
    const int rows_per_cta = 1 << lshift;
    const int kb_begin = static_cast<int>(rank) * static_cast<int>(p.chunk_blocks);
    int nb = static_cast<int>(p.k_blocks) - kb_begin;
    if (nb > static_cast<int>(p.chunk_blocks)) nb = static_cast<int>(p.chunk_blocks);
    if (nb < 0) nb = 0;  // ranks beyond the split have no K range
    const int m = static_cast<int>(p.q_total);
    // Every parameter line is pulled into the constant cache now, while the previous kernel in the stream may still
    // be running.
    TouchConstantLines(p);
    if constexpr (INT8) TouchConstantLines(ie);
    else TouchConstantLines(fe);

    if (warp == 0) {
        // ================================ TMA producer ================================
        if (lane == 0 && nb > 0) {
            int stage = 0;
            uint32_t phase = 0;
            const int loads = nb * tiles_here;
            auto load_weights = [&](int i) -> bool {
                // the first pass over the ring finds every stage free; later passes wait for the MMAs that read it
                if (i >= stages && !MbarWait(&empty[stage], phase ^ 1u, p.status, 20, stage)) return false;
                const bool second = i >= nb;  // the first weight's K blocks, then the second weight's
                const int32_t k0 = (kb_begin + (second ? i - nb : i)) * kBlockK;
                const CUtensorMap* map = second ? &map_p2 : &map_p;
                const int32_t p0 = (second ? tile + p.second_tile_offset : tile) * kBlockP;
                uint8_t* ps = ring + static_cast<size_t>(stage) * kPBytes;
                MbarExpectTx(&full[stage], kPBytes);
                if constexpr (P_MN) TmaLoad2D(ps, map, p0, k0, &full[stage]);
                else TmaLoad2D(ps, map, k0, p0, &full[stage]);
                if (++stage == stages) { stage = 0; phase ^= 1u; }
                return true;
            };
            // Weights that no earlier work in the stream writes can be fetched before the previous kernel has
            // finished: their DRAM latency then overlaps its tail.
            int kb = 0;
            if (p.args.w_static) {
                for (; kb < loads && kb < stages; ++kb) load_weights(kb);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            if (!convert) {
                MbarExpectTx(q_full, static_cast<uint32_t>(nb) * BQ * kBlockK);
                for (int j = 0; j < nb; ++j) TmaLoad2D(q_tiles + j * (BQ * kBlockK), &map_q, (kb_begin + j) * kBlockK, 0, q_full);
            }
            for (; kb < loads; ++kb) {
                if (!load_weights(kb)) break;
            }
        }
    } else if (warp == 1) {
        // ================================ MMA issuer ================================
        if (lane == 0 && nb > 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool failed = false;
            for (int i = 0; i < nb * tiles_here && !failed; ++i) {
                if (!MbarWait(&full[stage], phase, p.status, 22, stage)) { failed = true; break; }
                if (i == 0 && !MbarWait(q_full, 0, p.status, 21, 0)) { failed = true; break; }  // activations arrive last
                umma::FenceAfterThreadSync();
                const int kb = i >= nb ? i - nb : i;
                const uint32_t acc = tmem_base + (i >= nb ? BQ : 0);  // the second weight's accumulator sits beside the first's
                const uint32_t ps = SmemAddr(ring + static_cast<size_t>(stage) * kPBytes);
                const uint32_t qs = SmemAddr(q_tiles + kb * (BQ * kBlockK));
#pragma unroll
                for (int ks = 0; ks < kBlockK / 32; ++ks) {
                    const uint64_t a_desc = P_MN ? umma::SmemDesc(ps + ks * 4096, 16384, 1024) : umma::SmemDesc(ps + ks * 32, 16, 1024);
                    const uint64_t b_desc = umma::SmemDesc(qs + ks * 32, 16, 1024);
                    umma::Mma<INT8>(acc, a_desc, b_desc, p.idesc, (kb > 0 || ks > 0) ? 1u : 0u);
                }
                umma::Commit(&empty[stage]);
                if (++stage == stages) { stage = 0; phase ^= 1u; }
            }
            if (!failed) umma::Commit(tmem_full);
        }
    } else {
        // ====================== activation prologue, accumulator hand-out, reduce + epilogue ======================
        const int et = threadIdx.x - 64;  // 0 .. 127
        [[maybe_unused]] const DecoderFusion& fu = p.args.fusion;
        // DEC: the residual values of this thread's first two outputs, fetched right behind the dependency wait
        [[maybe_unused]] uint16_t residual_early[2] = {0, 0};
        if constexpr (DEC) {
            // ------------------------------------------------------------------------------------------------
            // Everything that does not depend on the producer runs in front of the wait: the places of this thread's
            // first four items and, when nothing in the stream writes them, the norm weights those items need.
            // Behind the wait the activation loads go out first, four per thread and with no branch between them.
            // ------------------------------------------------------------------------------------------------
            const uint16_t* act = static_cast<const uint16_t*>(p.args.a);
            const int K = static_cast<int>(p.args.k);
            const int prologue = fu.prologue;
            const int words_per_row = nb * 32;
            const int total = m * words_per_row;
            const uint32_t q_base = SmemAddr(q_tiles);
            int rows[4], k0[4];
            uint32_t dst[4];
            bool inside[4];
            uint2 raw[4];
            uint4 raw2[4];
            auto locate = [&](int base) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int item = base + j * 128;
                    const int row = item / words_per_row;
                    const int c = item - row * words_per_row;
                    const int kb = c >> 5, w4 = c & 31;
                    k0[j] = (kb_begin + kb) * kBlockK + w4 * 4;
                    inside[j] = item < total && k0[j] < K;  // K is a multiple of 16: a group is in or out as a whole
                    rows[j] = row;
                    dst[j] = q_base + kb * (BQ * kBlockK) + row * 128 + (((w4 >> 2) ^ (row & 7)) << 4) + ((w4 & 3) << 2);
                }
            };
            auto load_norm_weights = [&]() {
                if (fu.norm_weight_dtype == FTH_B200_FP32) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        raw2[j] = inside[j] ? *reinterpret_cast<const uint4*>(static_cast<const float*>(fu.norm_weight) + k0[j]) : make_uint4(0, 0, 0, 0);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint2 t = inside[j] ? *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(fu.norm_weight) + k0[j]) : make_uint2(0, 0);
                        raw2[j] = make_uint4(t.x, t.y, 0, 0);
                    }
                }
            };
            auto load_activations = [&]() {
#pragma unroll
                for (int j = 0; j < 4; ++j) raw[j] = inside[j] ? *reinterpret_cast<const uint2*>(act + rows[j] * K + k0[j]) : make_uint2(0, 0);
                if (prologue == 2) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint2 t = inside[j] ? *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(fu.a2) + rows[j] * K + k0[j]) : make_uint2(0, 0);
                        raw2[j] = make_uint4(t.x, t.y, 0, 0);
                    }
                }
            };
            const bool weights_early = prologue == 1 && p.args.w_static != 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) raw2[j] = make_uint4(0, 0, 0, 0);
            // (8-bit activations — a producer's epilogue has already run the Cast — arrive by TMA: no prologue at all)
            const bool prologue_here = convert && nb > 0;
            if (prologue_here) {
                locate(et);
                if (weights_early) load_norm_weights();
            }
            // the first two outputs this thread will finish (see the finishing loop below)
            int64_t early_at[2] = {-1, -1};
            if (fu.residual != nullptr) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int item = i * 128 + et;
                    const int q = item >> lshift, r = item & (rows_per_cta - 1);
                    const int64_t n = static_cast<int64_t>(tile) * kBlockP + (static_cast<int64_t>(rank) << lshift) + r;
                    if (item < (m << lshift) && n < p.p_total) early_at[i] = q * fe.ldo + n;  // a residual goes with the first weight only
                }
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            if (prologue_here) load_activations();
#pragma unroll
            for (int i = 0; i < 2; ++i)
                if (early_at[i] >= 0) residual_early[i] = static_cast<const uint16_t*>(fu.residual)[early_at[i]];
            if (prologue_here && prologue == 1) {
                // Fused QwenRmsNorm in front of the Cast: 1 / rms of every activation row, with the sum of squares added in
                // the order of the stand-alone kernel (128 threads that each add their groups of eight elements in turn, a
                // lane tree per warp, the four warps in order), so that the fused node returns the stand-alone node's bits.
                // One warp takes a whole row here: lane l plays the threads l, l + 32, l + 64, l + 96 of that kernel, so
                // the rows need no barrier between them and a row's loads are all in flight together.  Every CTA computes
                // every row for itself: a row is a few KB in L2.
                const int ew = et >> 5;
                const int groups = K >> 3;
                for (int row = ew; row < m; row += 4) {
                    const uint16_t* xr = act + row * K;
                    float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int g = 0; g < rowops::kRowGroups; ++g) {
                        if (g * rowops::kRowThreads >= groups) break;  // uniform
                        uint4 v[4];
#pragma unroll
                        for (int vt = 0; vt < 4; ++vt) {
                            const int gi = lane + 32 * vt + rowops::kRowThreads * g;
                            v[vt] = gi < groups ? *reinterpret_cast<const uint4*>(xr + gi * 8) : make_uint4(0, 0, 0, 0);
                        }
#pragma unroll
                        for (int vt = 0; vt < 4; ++vt) {
                            const uint32_t w[4] = {v[vt].x, v[vt].y, v[vt].z, v[vt].w};
#pragma unroll
                            for (int i = 0; i < 4; ++i) {  // a group beyond the row adds +0 to a sum that is never -0
                                const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xffff0000u);
                                part[vt] = __fadd_rn(part[vt], __fmul_rn(lo, lo));
                                part[vt] = __fadd_rn(part[vt], __fmul_rn(hi, hi));
                            }
                        }
                    }
#pragma unroll
                    for (int vt = 0; vt < 4; ++vt) part[vt] = rowops::WarpTreeSum(part[vt]);
                    if (lane == 0)
                        norm_inv[row] = rowops::InverseRms(__fadd_rn(__fadd_rn(__fadd_rn(part[0], part[1]), part[2]), part[3]), K, fu.norm_epsilon);
                }
                EpilogueBarrier<128>();
            }
            if (prologue_here) {
                if (prologue == 1 && !weights_early) load_norm_weights();
                for (int base = et;;) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (base + j * 128 < total) {
                            uint32_t word = 0u;
                            if (inside[j]) {
                                float h[4] = {__uint_as_float(raw[j].x << 16), __uint_as_float(raw[j].x & 0xffff0000u),
                                              __uint_as_float(raw[j].y << 16), __uint_as_float(raw[j].y & 0xffff0000u)};
                                if (prologue != 0)
                                    DecoderNodeFour(prologue, fu.norm_weight_dtype, fu.norm_offset, prologue == 1 ? norm_inv[rows[j]] : 0.0f, raw[j],
                                                    raw2[j], h);
                                word = CastFour(p.e4m3, p.args.a_scale, p.a_inv, h);
                            }
                            asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst[j]), "r"(word) : "memory");
                        }
                    }
                    base += 4 * 128;
                    if (base >= total) break;
                    locate(base);
                    load_activations();
                    if (prologue == 1) load_norm_weights();
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes → visible to the MMA's reads
                MbarArrive(q_full);
            }
        } else {
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
        }
        }
        const int row = (warp & 3) * 32 + lane;  // TMEM lane = channel inside the tile
        // Bytes this CTA will receive: from each of the `split` chunks, its L rows of ceil(m / 4) 16-byte vectors.
        if (et == 0) MbarExpectTx(x_full, static_cast<uint32_t>(p.split) * rows_per_cta * ((m + 3) / 4) * 16 * tiles_here);
        ClusterWait();  // every CTA of the cluster is running and has initialised its barriers
        if (nb > 0) {
            const bool ok = MbarWait(tmem_full, 0, p.status, 23, 0);
            umma::FenceAfterThreadSync();
            if (ok) {
                // Deal the accumulator rows out: row r goes to CTA r / L, slot [this chunk][r % L].  Each 16-byte
                // store reports its bytes to the receiver's barrier, so no cluster-wide barrier is needed.
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
                const uint32_t owner = static_cast<uint32_t>(row >> lshift);
                const uint32_t slot = SmemAddr(exchange) + (((rank << lshift) + (row & (rows_per_cta - 1))) * BQ) * 4;
                const uint32_t remote = MapToRank(slot, owner);
                const uint32_t remote_bar = MapToRank(SmemAddr(x_full), owner);
                for (int w = 0; w < tiles_here; ++w) {
#pragma unroll
                    for (int c0 = 0; c0 < BQ; c0 += 16) {
                        if (c0 >= m) break;  // uniform
                        uint32_t v[16];
                        umma::TmemLoad16(taddr + w * BQ + c0, v);
                        umma::TmemLoadWait();
#pragma unroll
                        for (int j = 0; j < 16; j += 4) {
                            if (c0 + j < m)
                                StoreClusterAsync4(remote + w * C::kExchangeBytes + (c0 + j) * 4, remote_bar, v[j], v[j + 1], v[j + 2], v[j + 3]);
                        }
                    }
                }
            }
        }
        // A CTA leaves only after everything addressed to it has landed, so no peer ever writes into a CTA that is gone.
        // Second phase of the cluster barrier: "this CTA has sent everything it will ever send".  The matching wait is
        // at the very end of the kernel, so that no CTA leaves while a peer could still store into its shared memory —
        // also when a bounded wait gave up somewhere.  In a healthy run every peer has long arrived by then.
        ClusterArriveRelaxed();
        const bool delivered = MbarWait(x_full, 0, p.status, 24, 0);

        if constexpr (DEC) {
            // One output per thread and round, as below, written out for BF16 <- E4M3 / E5M2 <- FP32 with per-tensor scales:
            // product scale, output Cast (encode, decode, BF16 rounding), then the fused Add node's own rounding point.
            const bool dual = tiles_here > 1;
            const float mult[2] = {fe.ab_scale, fu.ab_scale2};
            uint16_t* out = static_cast<uint16_t*>(fe.out);
            const uint16_t* residual = static_cast<const uint16_t*>(fu.residual);
            const int64_t n_base = static_cast<int64_t>(tile) * kBlockP + (static_cast<int64_t>(rank) << lshift);
            const int total = m << lshift;
            // the BF16 bits of one projection output: chunks added in chunk order, product scale, output Cast
            auto project = [&](int w, int r, int q) -> uint16_t {
                const uint32_t* part = exchange + w * (C::kExchangeBytes / 4);
                uint32_t t[8];
#pragma unroll
                for (int ss = 0; ss < 8; ++ss) t[ss] = ss < p.split ? part[((ss << lshift) + r) * BQ + q] : 0u;  // all in flight
                float sum = 0.0f;
#pragma unroll
                for (int ss = 0; ss < 8; ++ss) {
                    if (ss < p.split) sum += __uint_as_float(t[ss]);  // no zero is ever added: it could flip a -0
                }
                const float scaled = __fmul_rn(sum, mult[w]);
                const float y = p.out_inv != 0.0f ? __fmul_rn(scaled, p.out_inv) : __fdiv_rn(scaled, fe.out_scale);
                const uint32_t code = EncodePair(p.e4m3, y, 0.0f) & 0xffu;
                return EncodeBf16Cast(__fmul_rn(DecodeFast(p.e4m3, code), fe.out_scale));
            };
            for (int base = 0; base < total; base += 128) {
                const int item = base + et;
                if (!delivered || item >= total) break;
                const int q = item >> lshift;
                const int r = item & (rows_per_cta - 1);
                const int64_t n = n_base + r;
                if (n >= p.p_total) continue;
                uint16_t bits = project(0, r, q);
                const int64_t o = q * fe.ldo + n;
                if (dual) {
                    const uint16_t bits2 = project(1, r, q);
                    if (fu.epilogue == 1) {
                        // the SiLU and Mul nodes behind gate and up, each with its BF16 rounding point
                        bits = EncodeBf16Cast(__fmul_rn(DecodeBf16(rowops::SiluToBf16(DecodeBf16(bits))), DecodeBf16(bits2)));
                    } else {
                        static_cast<uint16_t*>(fu.out2)[q * fu.ldo2 + n] = bits2;
                    }
                }
                // fused Add node behind the output Cast (the residual connection): one more BF16 rounding point
                if (residual != nullptr) {
                    const uint16_t other = base == 0 ? residual_early[0] : base == 128 ? residual_early[1] : residual[o];
                    bits = EncodeBf16Cast(__fadd_rn(DecodeBf16(other), DecodeBf16(bits)));
                }
                out[o] = bits;
                if (fu.out_codes != nullptr) {
                    // the Cast node in front of the NEXT projection, run here once per output instead of once per CTA there
                    const float v = DecodeBf16(bits);
                    const float y = v != v ? v : (fu.codes_inv != 0.0f ? __fmul_rn(v, fu.codes_inv) : __fdiv_rn(v, fu.codes_scale));
                    static_cast<uint8_t*>(fu.out_codes)[q * fu.ldo_codes + n] = static_cast<uint8_t>(EncodePair(p.e4m3, y, 0.0f) & 0xffu);
                }
            }
        } else {
        // Column-sharded projection with the gather's signalling folded in: before the first store into the peers'
        // buffers every rank must have published the previous step.  The wait sits here, behind the whole weight
        // stream of this launch, so the NVLink round trip of the peers' flags is normally long over.
        uint32_t gather_step = 0;
        if (p.args.signal.world > 0) {
            gather_step = GatherStep(p.args.signal);
            if (et < p.args.signal.world) GatherWaitPrevious(p.args.signal, et, gather_step, p.status);
            EpilogueBarrier<128>();
        }

        // One output per thread and round: channel r of this CTA's rows (fastest, so a warp stores consecutive
        // channels) of activation row q.  The chunks are added in chunk order, as the two-kernel path adds them.
        const int total = m << lshift;
        for (int w = 0; w < tiles_here; ++w)
        for (int base = 0; base < total; base += 128) {  // the same trip count in every lane: the argmax step below shuffles
            const int item = base + et;
            const bool valid = delivered && item < total;
            const int q = item >> lshift;
            const int r = item & (rows_per_cta - 1);
            const int64_t n = static_cast<int64_t>(tile + w * p.second_tile_offset) * kBlockP + (static_cast<int64_t>(rank) << lshift) + r;
            const uint32_t* part = exchange + w * (C::kExchangeBytes / 4);
            uint32_t code = 0;
            bool stored = false;
            if (valid) {
                uint32_t t[8];
#pragma unroll
                for (int ss = 0; ss < 8; ++ss) t[ss] = ss < p.split ? part[((ss << lshift) + r) * BQ + q] : 0u;  // all in flight
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
                if (n < p.p_total) { code = FinishOne<INT8>(p, fe, ie, q, n, acc); stored = true; }
            }
            if (p.args.argmax_keys != nullptr)
                ArgmaxUpdate(p.args.argmax_keys, stored ? q : -1, stored ? ArgmaxKey<INT8>(p.e4m3, code, n) : 0ull);
        }
        if (p.args.signal.world > 0) {
            EpilogueBarrier<128>();  // every epilogue thread's peer stores are issued
            if (et == 0) GatherArriveAndPublish(p.args.signal, gather_step, gridDim.x);
        }
        }
    }
    if (warp < 2) {
        if (!(warp == 0 && lane == 0 && nb > 0)) asm volatile("griddepcontrol.wait;" ::: "memory");
        ClusterWait();
        ClusterArriveRelaxed();  // these warps send nothing: second phase right away
    }
    ClusterWait();  // second phase: every CTA of the cluster has finished sending
    umma::FenceBeforeThreadSync();
    __syncthreads();
    if (warp == 1) {
        umma::FenceAfterThreadSync();
        umma::TmemDealloc(tmem_base, tmem_cols);
    }
}

template <bool INT8, bool P_MN, int BQ, bool DEC>
int LaunchClusterTyped(const TcGeometry& g, const CUtensorMap& map_p, const CUtensorMap& map_p2, const CUtensorMap& map_q, const TcParams& p_in,
                       const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream) {
    TcParams p = p_in;
    p.ring_stages = ClusterCfg<BQ>::StagesFor(g.chunk_blocks, p.tiles_per_cta);
    auto kernel = LinearClusterKernel<INT8, P_MN, BQ, DEC>;
    if (EnsureDynamicSmem(reinterpret_cast<const void*>(kernel), ClusterCfg<BQ>::kSmemBytes) != FTH_B200_OK) return FTH_B200_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    const int64_t clusters = g.second_tile_offset > 0 ? g.second_tile_offset : g.p_tiles;
    cfg.gridDim = dim3(static_cast<unsigned>(clusters * g.cluster));
    cfg.blockDim = dim3(ClusterCfg<BQ>::kThreads);
    cfg.dynamicSmemBytes = ClusterCfg<BQ>::SmemFor(g.chunk_blocks, p.tiles_per_cta);
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
    if (cudaLaunchKernelEx(&cfg, kernel, map_p, map_p2, map_q, p, fe, ie) != cudaSuccess) return FTH_B200_ERR_CUDA;
    NoteLaunch("tcgen05");
    return CheckLaunch();
}

template <bool INT8, bool DEC>
int LaunchClusterFor(const TcGeometry& g, bool weights_mn, const CUtensorMap& map_p, const CUtensorMap& map_p2, const CUtensorMap& map_q,
                  const TcParams& p, const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream) {
    if (g.bq == 16) {
        return weights_mn ? LaunchClusterTyped<INT8, true, 16, DEC>(g, map_p, map_p2, map_q, p, fe, ie, stream)
                          : LaunchClusterTyped<INT8, false, 16, DEC>(g, map_p, map_p2, map_q, p, fe, ie, stream);
    }
    return weights_mn ? LaunchClusterTyped<INT8, true, 32, DEC>(g, map_p, map_p2, map_q, p, fe, ie, stream)
                      : LaunchClusterTyped<INT8, false, 32, DEC>(g, map_p, map_p2, map_q, p, fe, ie, stream);
}

}  // namespace

int LaunchCluster(bool int8, const TcGeometry& g, bool weights_mn, const CUtensorMap& map_p, const CUtensorMap& map_p2, const CUtensorMap& map_q,
                  const TcParams& p, const Fp8Epilogue& fe, const Int8Epilogue& ie, cudaStream_t stream) {
    if (int8) return LaunchClusterFor<true, false>(g, weights_mn, map_p, map_p2, map_q, p, fe, ie, stream);
    return p.decoder ? LaunchClusterFor<false, true>(g, weights_mn, map_p, map_p2, map_q, p, fe, ie, stream)
                     : LaunchClusterFor<false, false>(g, weights_mn, map_p, map_p2, map_q, p, fe, ie, stream);
}

}  // namespace tc
}  // namespace fth
