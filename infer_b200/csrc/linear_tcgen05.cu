// Tensor-core linear kernels: tcgen05.mma (kind::f8f6f4 / kind::i8) with accumulators in tensor memory, operands
// staged by TMA into 128-byte-swizzled shared memory, fused scale / bias / requant / encode epilogues.
// This file: shape → kernel family, scratch sizing, tensor maps and launch parameters.  The kernels live in
// linear_tc_pair.cu, linear_tc_swapped.cu and linear_tc_cluster.cu; what they share is in linear_tc.cuh.
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

#include "linear_tc.cuh"

namespace fth {
namespace tc {

// 1 / s when s is a normal power of two with a normal reciprocal (x * (1/s) then equals x / s bit for bit), else 0.
float ExactReciprocal(float s) {
    int e = 0;
    if (!(s > 0.0f) || !std::isnormal(s) || std::frexp(s, &e) != 0.5f) return 0.0f;
    const float inv = 1.0f / s;
    return std::isnormal(inv) ? inv : 0.0f;
}

int SwapBlockQ(int64_t m) { return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128; }
// longest row a fused QwenRmsNorm keeps in registers (128 threads x 4 groups x 8 elements)
int64_t rowops_max_hidden() { return 4096; }


namespace {

TcGeometry GeometryFor(const LinearArgs& a) {
    TcGeometry g;
    g.swap = a.m <= 128;
    g.bq = g.swap ? SwapBlockQ(a.m) : 256;
    // (a second weight that shares the activation, a decoder-block fusion, rides in the CTAs of the first one's tiles)
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
    g.tiles_per_cta = a.fusion.w2 != nullptr ? 2 : 1;
    g.second_tile_offset = 0;
    if (g.swap && g.bq <= 32 && g.q_tiles == 1 && g.chunk_blocks <= kClusterQBlocks) {
        int c = 1;
        while (c < g.split) c *= 2;
        // more than one wave of CTAs: the persistent kernel keeps its ring full across tiles and is faster (measured).
        // Decoder-block fusions exist in this kernel only; its CTAs are small (several fit an SM), so a higher limit.
        const int64_t wave = static_cast<int64_t>(SmCount()) * 2;
        if (g.p_tiles * c <= (a.fusion.active() ? wave * 3 / 2 : wave)) {
            g.cluster = c;
        } else if (!a.fusion.active() && g.bq <= 16 && (g.p_tiles + 1) / 2 * c <= wave * 4 / 5) {
            // up to two waves' worth of tiles: every CTA takes two of them (tile t and tile t + half), still one launch.
            // Measured against the persistent kernel + reduce pass at M = 1: K = 8192, N = 7168 (224 CTAs) 13.4 vs 15.9 us,
            // N = 6016 12.1 vs 15.1 us; with every CTA slot taken (K = 4096, N = 9472: 296 CTAs) 14.2 vs 13.1 us, hence the
            // margin below a full wave.
            g.cluster = c;
            g.tiles_per_cta = 2;
            g.second_tile_offset = static_cast<int>((g.p_tiles + 1) / 2);
        }
    }
    return g;
}


// M <= 32 on the persistent kernel: whether every CTA runs whole tiles (all K chunks, one accumulator in tensor memory
// each) and adds the chunks itself, in the reduce pass's order — one launch, no partial sums in memory, the same bits.
// A CTA then streams 128 weight columns alone, at ~45 GB/s: that needs about a hundred CTAs at work to keep HBM busy, in
// the last wave of tiles too.  Measured, FP8, one GPU, M = 1 (M = 16), folded against GEMV + reduce pass, us:
//   K = 8192:  64 tiles 22.8 / 17.3;  96: 23.7 / 22.8;  112: 24.0 / 25.9;  224: 40.0 / 43.1 (41.8 / 47.4);
//              296: 51.2 / 55.9 (53.5 / 61.3);  300: 64.9 / 58.0;  330: 66.7 / 61.5;  400: 71.9 / 75.3;  600: 108.7 / 108.5
//   K = 4096:  1187 tiles, M = 16: 108.4 / 130.5
bool FoldsSplit(const TcGeometry& g, int64_t m) {
    if (!g.swap || g.cluster != 0 || g.split <= 1 || g.bq > 32) return false;
    const int64_t tiles = g.p_tiles * g.q_tiles, slots = static_cast<int64_t>(SmCount()) * 2, busy = slots / 3;
    if (tiles < busy) return false;
    const int64_t last_wave = tiles % slots;
    if (tiles <= slots || last_wave == 0 || last_wave >= busy) return true;
    return tiles >= 4 * slots && m > 4;  // many waves, and partial sums that would weigh as much as the weights' tail
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

}  // namespace
}  // namespace tc

using namespace tc;

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

bool Tcgen05SelectsInEpilogue(int dtype, const LinearArgs& a, const Fp8Epilogue& fe, const Int8Epilogue& ie) {
    const TcGeometry g = GeometryFor(a);
    return g.swap && (g.cluster > 0 || g.split > 1) && DirectEpilogue(dtype == FTH_B200_INT8, fe, ie);
}

bool Tcgen05StoresToPeers(int dtype, const LinearArgs& a, const Fp8Epilogue& fe, const Int8Epilogue& ie) {
    if (Tcgen05SelectsInEpilogue(dtype, a, fe, ie)) return true;
    // the dense kernel's vectorised epilogue (native output dtype, no bias / alpha / beta) writes the replicas too
    const bool int8 = dtype == FTH_B200_INT8;
    return !GeometryFor(a).swap && DirectEpilogue(int8, fe, ie) && (int8 ? ie.out_dtype : fe.out_dtype) == 0;
}

// The decoder-block form of the single-launch cluster kernel: BF16 activations (16-byte aligned), FP8 product, BF16 out,
// per-tensor scales, no bias, nothing stored to peers, no selection.
static bool DecoderForm(int dtype, const LinearArgs& a, const Fp8Epilogue& fe, const Int8Epilogue& ie) {
    if (dtype == FTH_B200_INT8 || GeometryFor(a).cluster == 0) return false;
    // activations: BF16 (the kernel runs the Cast) or already FP8 codes of the projection's format (a producer ran it)
    if ((a.a_dtype != FTH_B200_BF16 && a.a_dtype != 0) || fe.out_dtype != FTH_B200_BF16 || !DirectEpilogue(false, fe, ie)) return false;
    if (fe.w_channel_scales != nullptr || a.argmax_keys != nullptr || a.peers.count != 0 || a.signal.world != 0) return false;
    return reinterpret_cast<uintptr_t>(a.a) % 16 == 0;
}

// QwenRmsNorm / SiLU * Mul in front, residual Add behind, a second weight beside: that form only.  FTH_B200_OK when
// LaunchLinearTcgen05 will run args.fusion.
int Tcgen05FusionStatus(int dtype, const LinearArgs& a, const Fp8Epilogue& fe, const Int8Epilogue& ie) {
    if (!Tcgen05Supported(dtype, a)) return FTH_B200_ERR_UNSUPPORTED;
    const DecoderFusion& fu = a.fusion;
    const TcGeometry g = GeometryFor(a);
    if (!DecoderForm(dtype, a, fe, ie)) return FTH_B200_ERR_UNSUPPORTED;
    if ((fu.prologue == 1 && reinterpret_cast<uintptr_t>(fu.norm_weight) % 16 != 0) ||
        (fu.prologue == 2 && reinterpret_cast<uintptr_t>(fu.a2) % 16 != 0)) return FTH_B200_ERR_UNSUPPORTED;
    if (fu.prologue < 0 || fu.prologue > 2) return FTH_B200_ERR_INVALID;
    if (fu.prologue != 0 && a.a_dtype != FTH_B200_BF16) return FTH_B200_ERR_INVALID;  // the nodes in front work on BF16 values
    if (fu.out_codes != nullptr && (fu.ldo_codes < a.n || (fu.w2 != nullptr && fu.epilogue == 0))) return FTH_B200_ERR_INVALID;
    if (fu.prologue == 1 && fu.norm_weight == nullptr) return FTH_B200_ERR_INVALID;
    if (fu.prologue == 1 && (fu.norm_weight_dtype != FTH_B200_BF16 && fu.norm_weight_dtype != FTH_B200_FP32)) return FTH_B200_ERR_UNSUPPORTED;
    if (fu.prologue == 1 && a.k > rowops_max_hidden()) return FTH_B200_ERR_UNSUPPORTED;
    if (fu.prologue == 2 && fu.a2 == nullptr) return FTH_B200_ERR_INVALID;
    if (fu.epilogue < 0 || fu.epilogue > 1 || (fu.epilogue == 1 && (fu.w2 == nullptr || fu.residual != nullptr))) return FTH_B200_ERR_INVALID;
    if (fu.w2 != nullptr) {
        if (fu.n2 != a.n) return FTH_B200_ERR_INVALID;  // the two weights' columns pair up
        if (fu.epilogue == 0 && (fu.out2 == nullptr || fu.ldo2 < fu.n2)) return FTH_B200_ERR_INVALID;
        if (reinterpret_cast<uintptr_t>(fu.w2) % 16 != 0) return FTH_B200_ERR_UNSUPPORTED;
    }
    return FTH_B200_OK;
}

bool Tcgen05SignalsInKernel(int dtype, const LinearArgs& a, const Fp8Epilogue& fe, const Int8Epilogue& ie) {
    // exactly the launches whose own epilogue writes the peers' buffers: their last block knows when all stores are out
    return Tcgen05StoresToPeers(dtype, a, fe, ie);
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
    if (a.fusion.active()) {
        const int rc = Tcgen05FusionStatus(dtype, a, fe, ie);
        if (rc != FTH_B200_OK) return rc;
        a.fusion.codes_inv = a.fusion.out_codes != nullptr ? ExactReciprocal(a.fusion.codes_scale) : 0.0f;
    }
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
    CUtensorMap map_p2 = map_p;  // two tiles of one weight per CTA: the same map
    if (a.fusion.w2 != nullptr) {
        if (weights_mn) ok = CachedMap(&map_p2, a.fusion.w2, static_cast<uint64_t>(a.fusion.n2), static_cast<uint64_t>(a.k), 128, 128);
        else ok = CachedMap(&map_p2, a.fusion.w2, static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.fusion.n2), 128, kBlockP);
        if (!ok) return FTH_B200_ERR_CUDA;
    }

    TcParams p;
    p.args = a;
    p.swap = g.swap;
    p.p_total = g.p_total; p.q_total = g.q_total; p.p_tiles = g.p_tiles; p.q_tiles = g.q_tiles;
    p.ring_stages = 0;
    p.split = g.split; p.chunk_blocks = g.chunk_blocks; p.k_blocks = g.k_blocks; p.units = g.units;
    p.tiles_per_cta = g.tiles_per_cta;
    p.second_tile_offset = g.second_tile_offset;
    p.p_pad = g.p_pad;
    p.e4m3 = dtype == FTH_B200_FP8E4M3;
    if (int8) p.fast = ie.bias_mode == FTH_B200_BIAS_NONE && ie.out_dtype == 0 && !(ie.is_gemm && (ie.alpha != 1.0f || ie.beta != 1.0f));
    else p.fast = fe.bias_mode == FTH_B200_BIAS_NONE && fe.out_dtype == 0 && !(fe.is_gemm && fe.alpha != 1.0f);
    p.fast4 = DirectEpilogue(int8, fe, ie);
    p.decoder = DecoderForm(dtype, a, fe, ie) && g.second_tile_offset == 0;  // (two tiles of one weight: the general form)
    p.a_inv = int8 ? 0.0f : ExactReciprocal(a.a_scale);
    p.out_inv = int8 ? 0.0f : ExactReciprocal(fe.out_scale);
    p.scratch = scratch;
    p.status = DeviceStatusPtr();
    p.fold = p.fast && a.argmax_keys == nullptr && FoldsSplit(g, a.m);
    if (p.fold) p.units = g.p_tiles * g.q_tiles;
    // operand formats: kind::f8f6f4 0 = E4M3, 1 = E5M2; kind::i8 1 = signed 8-bit.  D: 1 = F32, 2 = S32.
    const uint32_t fmt = int8 ? 1u : (dtype == FTH_B200_FP8E5M2 ? 1u : 0u);
    const bool p_mn = g.swap && weights_mn;
    const bool q_mn = !g.swap && weights_mn;
    p.idesc = umma::InstrDesc(int8 ? 2u : 1u, fmt, fmt, p_mn, q_mn, kBlockP, static_cast<uint32_t>(g.bq));
    if (g.cluster > 0) return LaunchCluster(int8, g, weights_mn, map_p, map_p2, map_q, p, fe, ie, stream);
    if (!g.swap) {
        // CTA pairs: each CTA stages 128 activation rows and 128 weight columns of a 256 x 256 tile
        CUtensorMap map_w_half = map_w;
        if (!weights_mn && !CachedMap(&map_w_half, a.w, static_cast<uint64_t>(a.k), static_cast<uint64_t>(a.n), 128, 128)) return FTH_B200_ERR_CUDA;
        // (Narrower tiles, 224 .. 128 columns, would fill the last wave of tiles better at M = 256 .. 1024; measured, they
        // are slower per column by more than that gains: K = 8192, N = 28672, FP8, M = 256: 63.8 us at 256 columns, 68.1 at
        // 224, 80.7 at 192; M = 4096: 645 / 850 / 824 us.)
        p.idesc = umma::InstrDesc(int8 ? 2u : 1u, fmt, fmt, false, q_mn, 256, 256);
        // Replicas on other GPUs, native one-byte output: whole tiles leave through tile stores (see linear_tc_pair.cu).
        OutMaps out_maps = {};
        uint8_t* out = static_cast<uint8_t*>(int8 ? ie.out : fe.out);
        const int64_t ldo = int8 ? ie.ldo : fe.ldo;
        bool tile_stores = a.peers.count > 0 && p.fast && ldo % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
        for (int r = 0; r < a.peers.count; ++r) tile_stores = tile_stores && a.peers.delta[r] % 16 == 0;
        if (tile_stores && a.peers.multicast_delta != 0 && a.n % 16 == 0 && a.peers.multicast_delta % 16 == 0) {
            out_maps.multicast = out + a.peers.multicast_delta;
            out_maps.ldo = ldo;
        } else if (tile_stores) {
            for (int d = 0; d <= a.peers.count; ++d) {
                const uint8_t* base = d == 0 ? out : out + a.peers.delta[d - 1];
                if (!MakeTensorMap2D(&out_maps.map[d], base, static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.m), static_cast<uint64_t>(ldo),
                                     256, kBlockP, TmaSwizzle::kNone)) return FTH_B200_ERR_CUDA;
            }
            out_maps.count = a.peers.count + 1;
        }
        return LaunchPair(int8, weights_mn, map_a, map_w_half, out_maps, p, fe, ie, stream);
    }
    return LaunchSwapped(int8, g, weights_mn, map_p, map_q, p, fe, ie, stream);
}

}  // namespace fth

