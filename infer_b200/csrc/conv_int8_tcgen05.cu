// INT8 Conv2D as an implicit GEMM on the tensor cores (stride 1, dilation 1, one group, symmetric
// quantisation): D[pixel][oc] = sum over (tap, ic) of X[pixel + tap][ic] * W[oc][tap][ic].
//
//   pass 1  NCHW -> NHWC copy of the input into the workspace, so that the 64 input channels of a pixel are
//           one contiguous 64-byte K-major row (1 byte per element: 1.6 MB at 64 x 160 x 160);
//   pass 0  (once per weight) OIHW -> [OC][KH][KW][IC] weight repack into the workspace;
//   pass 2  persistent kernel: a tile is 32 x 4 output pixels = the 128 TMEM lanes.  For every filter tap
//           and 64-channel block, TMA fetches the shifted 32 x 4 x 64-byte input window as one 4-D box —
//           coordinates outside the image are zero-filled by TMA, which is exactly the reference's "padded taps
//           contribute nothing" when the input zero point is 0 — into a 64-byte-swizzled ring; the repacked
//           weights (OC x taps x IC, 36 KB at 64 x 9 x 64) stay resident in shared memory for the CTA's
//           lifetime.  tcgen05.mma kind::i8 accumulates int32 in TMEM; the epilogue adds the int32 bias,
//           requantises exactly as the reference does, applies the optional INT8 ReLU table and writes NCHW.
#include "common.cuh"
#include "conv_internal.h"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace fth {
namespace {

constexpr int kTileW = 32, kTileH = 4;          // 128 output pixels per tile
constexpr int kRowBytes = 64;                   // one K block: 64 input channels of one tap
constexpr int kABytes = kTileW * kTileH * kRowBytes;  // 8 KB per ring stage
constexpr int kStages = 8;
// 16 epilogue warps: the requantisation is scalar code with long dependent chains, and one warp per scheduler ran it
// at ~0.2 instructions per clock.  Four warps share each 32-lane slice of tensor memory and split its channels.
constexpr int kEpilogueWarps = 16;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kAcc = 2;

struct ConvTcParams {
    ConvArgs c;
    int taps, cblocks, kblocks;   // kh*kw, ic/64, taps*cblocks
    int64_t tiles_w, tiles_h, tiles;
    uint32_t idesc;
    int* status;
};

// ---- pass 1: NCHW -> NHWC ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) NchwToNhwcKernel(const int8_t* __restrict__ x, int8_t* __restrict__ y, int64_t n, int64_t c,
                                                        int64_t h, int64_t w) {
    __shared__ int8_t tile[64][33];
    const int64_t w0 = static_cast<int64_t>(blockIdx.x) * 32;
    const int64_t c0 = static_cast<int64_t>(blockIdx.y) * 64;
    const int64_t nh = blockIdx.z;  // n * h + row
    const int64_t img = nh / h, row = nh % h;
    for (int idx = threadIdx.x; idx < 64 * 32; idx += 256) {
        const int cc = idx / 32, ww = idx % 32;
        tile[cc][ww] = (c0 + cc < c && w0 + ww < w) ? x[((img * c + c0 + cc) * h + row) * w + w0 + ww] : int8_t(0);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 64 * 32; idx += 256) {
        const int ww = idx / 64, cc = idx % 64;
        if (c0 + cc < c && w0 + ww < w) y[((img * h + row) * w + w0 + ww) * c + c0 + cc] = tile[cc][ww];
    }
}

// Same pass for the common aligned case (w % 4 == 0, c % 16 == 0, 4-byte aligned x, 16-byte aligned y): one block
// per image row and 64-channel block; 32-bit loads along w, a byte tile in shared memory, and 16-byte stores of 16
// channels of one pixel — the row's pixels x 64 channels are one contiguous run of the NHWC copy.
constexpr int kRowTileW = 256;  // widest row handled by the fast pass
__global__ void __launch_bounds__(256) NchwToNhwcRowKernel(const int8_t* __restrict__ x, int8_t* __restrict__ y, int64_t c, int64_t h,
                                                           int64_t w) {
    // lets the conv kernel behind it set up and fetch its weights while this pass runs
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ __align__(16) uint8_t tile[64][kRowTileW + 4];
    const int64_t c0 = static_cast<int64_t>(blockIdx.y) * 64;
    const int64_t nh = blockIdx.x;  // n * h + row
    const int64_t img = nh / h, row = nh % h;
    const int words = static_cast<int>(w / 4);
    const int channels = static_cast<int>(c - c0 < 64 ? c - c0 : 64);
    for (int idx = threadIdx.x; idx < channels * words; idx += 256) {
        const int cc = idx / words, w4 = idx - cc * words;
        const uint32_t v = *reinterpret_cast<const uint32_t*>(x + ((img * c + c0 + cc) * h + row) * w + w4 * 4);
        *reinterpret_cast<uint32_t*>(&tile[cc][w4 * 4]) = v;
    }
    __syncthreads();
    const int groups = channels / 16;
    for (int idx = threadIdx.x; idx < static_cast<int>(w) * groups; idx += 256) {
        const int px = idx / groups, g = idx - px * groups;
        uint32_t out[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int cc = g * 16 + q * 4;
            out[q] = tile[cc][px] | (static_cast<uint32_t>(tile[cc + 1][px]) << 8) | (static_cast<uint32_t>(tile[cc + 2][px]) << 16) |
                     (static_cast<uint32_t>(tile[cc + 3][px]) << 24);
        }
        *reinterpret_cast<uint4*>(y + ((img * h + row) * w + px) * c + c0 + g * 16) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// ---- pass 0: OIHW -> O(HW)I ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) PackConvWeightKernel(const int8_t* __restrict__ w, int8_t* __restrict__ out, int64_t oc,
                                                            int64_t ic, int64_t taps) {
    const int64_t total = oc * ic * taps;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t c = i % ic, t = (i / ic) % taps, o = i / (ic * taps);
        out[i] = w[(o * ic + c) * taps + t];
    }
}

// ---- pass 2: implicit GEMM ------------------------------------------------------------------------------------
template <int BQ>
__global__ void __launch_bounds__(kThreads, 1)
ConvTcgen05Kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, ConvTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* w_smem = base;                                          // kblocks * BQ * 64 bytes, resident
    const int w_block = BQ * kRowBytes;
    uint8_t* ring = w_smem + ((p.kblocks * w_block + 1023) / 1024) * 1024;  // kStages * 8 KB
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + kStages * kABytes);
    uint64_t* empty = full + kStages;
    uint64_t* tmem_full = empty + kStages;
    uint64_t* tmem_empty = tmem_full + kAcc;
    uint64_t* w_ready = tmem_empty + kAcc;
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(w_ready + 1);
    double* col_scale = reinterpret_cast<double*>(reinterpret_cast<uint8_t*>(full) + 256);  // [BQ]
    double* col_multd = col_scale + BQ;                                                    // [BQ]
    float* col_mult = reinterpret_cast<float*>(col_multd + BQ);                            // [BQ]
    int32_t* col_bias = reinterpret_cast<int32_t*>(col_mult + BQ);                         // [BQ]
    int8_t* lut = reinterpret_cast<int8_t*>(col_bias + BQ);                                // [256]

    const ConvArgs& c = p.c;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    constexpr uint32_t kTmemCols = kAcc * BQ < 32 ? 32 : kAcc * BQ;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { MbarInit(&full[s], 1); MbarInit(&empty[s], 1); }
        for (int b = 0; b < kAcc; ++b) { MbarInit(&tmem_full[b], 1); MbarInit(&tmem_empty[b], kEpilogueWarps); }
        MbarInit(w_ready, 1);
        FenceBarrierInit();
        TmaPrefetchDescriptor(&map_x);
        TmaPrefetchDescriptor(&map_w);
        // Weights packed by an earlier call are not written by anything still running: fetch them (the whole
        // repacked weight, once) before waiting for the layout pass in front of this kernel.
        if (c.weights_packed) {
            MbarExpectTx(w_ready, static_cast<uint32_t>(p.kblocks * w_block));
            for (int kb = 0; kb < p.kblocks; ++kb) TmaLoad2D(w_smem + kb * w_block, &map_w, kb * kRowBytes, 0, w_ready);
        }
    }
    if (warp == 1) umma::TmemAlloc(tmem_base_slot, kTmemCols);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // per-output-channel constants and the optional ReLU table, once per CTA
    const double so_d = static_cast<double>(c.out_scale);
    for (int o = threadIdx.x; o < BQ; o += kThreads) {
        if (o < c.oc) {
            const double sd = static_cast<double>(c.x_scale) * static_cast<double>(c.w_scales[c.per_channel ? o : 0]);
            col_scale[o] = sd;
            col_multd[o] = sd / so_d;
            col_mult[o] = static_cast<float>(sd / so_d);
            col_bias[o] = c.bias ? c.bias[o] : 0;
        }
    }
    if (c.relu_lut != nullptr)
        for (int i = threadIdx.x; i < 256; i += kThreads) lut[i] = c.relu_lut[i];
    umma::FenceBeforeThreadSync();
    __syncthreads();
    umma::FenceAfterThreadSync();
    const uint32_t tmem_base = *tmem_base_slot;

    auto decode_tile = [&](int64_t t, int64_t* n, int64_t* oh0, int64_t* ow0) {
        *ow0 = (t % p.tiles_w) * kTileW;
        const int64_t r = t / p.tiles_w;
        *oh0 = (r % p.tiles_h) * kTileH;
        *n = r / p.tiles_h;
    };

    if (warp == 0) {
        // One thread takes ~350 clocks per TMA it issues (expect + copy), which for a CTA with one or two tiles is most
        // of the time to the first MMA.  So the first pass over the ring — every stage is free — is issued by as many
        // lanes as there are stages, one k-block each, at once; lane 0 carries on alone from there.
        const int first = p.kblocks < kStages ? p.kblocks : kStages;
        if (blockIdx.x < p.tiles && lane < first) {
            int64_t n, oh0, ow0;
            decode_tile(blockIdx.x, &n, &oh0, &ow0);
            const int tap = lane / p.cblocks, cb = lane - tap * p.cblocks;
            const int ky = tap / static_cast<int>(c.kw), kx = tap - ky * static_cast<int>(c.kw);
            MbarExpectTx(&full[lane], kABytes);
            TmaLoad4D(ring + lane * kABytes, &map_x, cb * kRowBytes, static_cast<int32_t>(ow0 - c.pad_w) + kx,
                      static_cast<int32_t>(oh0 - c.pad_h) + ky, static_cast<int32_t>(n), &full[lane]);
        }
        __syncwarp();
        if (lane == 0) {
            if (!c.weights_packed) {  // packed by the kernel in front of this one: only now safe to read
                MbarExpectTx(w_ready, static_cast<uint32_t>(p.kblocks * w_block));
                for (int kb = 0; kb < p.kblocks; ++kb) TmaLoad2D(w_smem + kb * w_block, &map_w, kb * kRowBytes, 0, w_ready);
            }
            int issued = 0;
            int stage = 0;
            uint32_t phase = 0;
            bool failed = false;
            for (int64_t t = blockIdx.x; t < p.tiles && !failed; t += gridDim.x) {
                int64_t n, oh0, ow0;
                decode_tile(t, &n, &oh0, &ow0);
                const int32_t x0 = static_cast<int32_t>(ow0 - c.pad_w), y0 = static_cast<int32_t>(oh0 - c.pad_h);
                int ky = 0, kx = 0, cb = 0;  // k-block order: tap-major (ky, kx), then the 64-channel block
                for (int kb = 0; kb < p.kblocks; ++kb) {
                    if (issued >= first) {
                        // (stages of the first pass beyond `first` are free as well)
                        if (issued >= kStages && !MbarWait(&empty[stage], phase ^ 1u, p.status, 20, stage)) { failed = true; break; }
                        MbarExpectTx(&full[stage], kABytes);
                        TmaLoad4D(ring + stage * kABytes, &map_x, cb * kRowBytes, x0 + kx, y0 + ky, static_cast<int32_t>(n), &full[stage]);
                    }
                    ++issued;
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                    if (++cb == p.cblocks) { cb = 0; if (++kx == static_cast<int>(c.kw)) { kx = 0; ++ky; } }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool failed = !MbarWait(w_ready, 0, p.status, 21, 0);
            int64_t iter = 0;
            for (int64_t t = blockIdx.x; t < p.tiles && !failed; t += gridDim.x, ++iter) {
                const int acc = static_cast<int>(iter % kAcc);
                const uint32_t acc_phase = static_cast<uint32_t>((iter / kAcc) & 1);
                if (!MbarWait(&tmem_empty[acc], acc_phase ^ 1u, p.status, 22, acc)) { failed = true; break; }
                umma::FenceAfterThreadSync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BQ);
                for (int kb = 0; kb < p.kblocks; ++kb) {
                    if (!MbarWait(&full[stage], phase, p.status, 23, stage)) { failed = true; break; }
                    umma::FenceAfterThreadSync();
                    const uint32_t as = SmemAddr(ring + stage * kABytes);
                    const uint32_t ws = SmemAddr(w_smem + kb * w_block);
#pragma unroll
                    for (int ks = 0; ks < kRowBytes / 32; ++ks) {
                        umma::Mma<true>(d_tmem, umma::SmemDescSw64(as + ks * 32, 16, 512), umma::SmemDescSw64(ws + ks * 32, 16, 512),
                                        p.idesc, (kb > 0 || ks > 0) ? 1u : 0u);
                    }
                    umma::Commit(&empty[stage]);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (!failed) umma::Commit(&tmem_full[acc]);
            }
        }
    } else {
        const int lane_group = warp & 3;      // = row of the 32 x 4 pixel tile
        const int slice = (warp - 2) / 4;     // which 16-channel groups this warp requantises: slice, slice + 4, ...
        bool failed = false;
        int64_t iter = 0;
        for (int64_t t = blockIdx.x; t < p.tiles; t += gridDim.x, ++iter) {
            int64_t n, oh0, ow0;
            decode_tile(t, &n, &oh0, &ow0);
            const int acc = static_cast<int>(iter % kAcc);
            const uint32_t acc_phase = static_cast<uint32_t>((iter / kAcc) & 1);
            const int64_t oh = oh0 + lane_group, ow = ow0 + lane;
            const bool pix_ok = oh < c.oh && ow < c.ow;
            const int64_t ow_base = ow - (lane & 3);
            if (!failed && !MbarWait(&tmem_full[acc], acc_phase, p.status, 24, acc)) failed = true;
            umma::FenceAfterThreadSync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + static_cast<uint32_t>(acc * BQ);
            // Output is NCHW: for one channel the tile's 32 pixels of a row are contiguous.  Each thread requantises 16
            // channels of its pixel (independent chains, no branches between them), then every quad of lanes
            // transposes 4 channels x 4 pixels in registers (two shuffles + two byte permutes per 4 channels) so that
            // each lane stores one 32-bit word: 4 pixels of channel o + (lane & 3).
            const int quad = lane & 3;
            int8_t* out_px = c.out + ((n * c.oc) * c.oh + oh) * c.ow + ow_base;  // channel 0, this quad's first pixel
            const int64_t plane = c.oh * c.ow;
            const bool row_in = oh < c.oh;
            const bool quad_whole = row_in && ow_base + 3 < c.ow && ((reinterpret_cast<uintptr_t>(out_px) | static_cast<uintptr_t>(plane)) & 3) == 0;
            const bool use_lut = c.relu_lut != nullptr;
            const float zp_f = static_cast<float>(c.out_zp);
#pragma unroll 1
            for (int c0 = slice * 16; c0 < BQ; c0 += 16 * (kEpilogueWarps / 4)) {
                if (c0 >= c.oc) break;
                uint32_t v[16];
                umma::TmemLoad16(taddr + c0, v);
                umma::TmemLoadWait();
                uint32_t q[16];
                uint32_t near = 0;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int o = c0 + j < c.oc ? c0 + j : static_cast<int>(c.oc) - 1;  // clamp: no branch in the chain
                    q[j] = RequantEstimate(static_cast<int32_t>(v[j]) + col_bias[o], col_mult[o], zp_f, j, &near);
                }
                while (near != 0) {  // a few values in 10^4: decided in double
                    const int j = __ffs(near) - 1;
                    near &= near - 1;
                    const int o = c0 + j < c.oc ? c0 + j : static_cast<int>(c.oc) - 1;
                    int32_t vj = 0;
#pragma unroll
                    for (int i = 0; i < 16; ++i) vj = i == j ? static_cast<int32_t>(v[i]) : vj;  // keeps v[] in registers
                    const uint32_t exact = static_cast<uint8_t>(RequantInt32(vj + col_bias[o], col_scale[o], col_multd[o], so_d, c.out_zp));
#pragma unroll
                    for (int i = 0; i < 16; ++i) q[i] = i == j ? exact : q[i];
                }
                if (use_lut) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) q[j] = static_cast<uint8_t>(lut[static_cast<uint8_t>(q[j] + 128)]);
                }
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int o = c0 + 4 * g + quad;  // the channel this lane stores
                    // (the shuffles run in every lane: quads at the ragged edge differ only in how they store)
                    const uint32_t w = q[4 * g] | (q[4 * g + 1] << 8) | (q[4 * g + 2] << 16) | (q[4 * g + 3] << 24);
                    const uint32_t x = __shfl_xor_sync(0xffffffffu, w, 2);
                    const uint32_t r = (lane & 2) ? __byte_perm(x, w, 0x7632) : __byte_perm(w, x, 0x5410);
                    const uint32_t y = __shfl_xor_sync(0xffffffffu, r, 1);
                    const uint32_t t = (lane & 1) ? __byte_perm(y, r, 0x7351) : __byte_perm(r, y, 0x6240);
                    if (quad_whole) {
                        if (o < c.oc) *reinterpret_cast<uint32_t*>(out_px + o * plane) = t;
                    } else if (pix_ok) {  // ragged edge or unaligned rows: this thread's own bytes
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (c0 + 4 * g + i < c.oc) out_px[(c0 + 4 * g + i) * plane + quad] = static_cast<int8_t>(q[4 * g + i]);
                    }
                }
            }
            umma::FenceBeforeThreadSync();
            __syncwarp();
            if (lane == 0) MbarArrive(&tmem_empty[acc]);
        }
    }

    umma::FenceBeforeThreadSync();
    __syncthreads();
    if (warp == 1) {
        umma::FenceAfterThreadSync();
        umma::TmemDealloc(tmem_base, kTmemCols);
    }
}

int BlockQFor(int64_t oc) { return oc <= 32 ? 32 : oc <= 64 ? 64 : oc <= 128 ? 128 : 256; }

size_t Align256(size_t v) { return (v + 255) / 256 * 256; }

size_t SmemBytesFor(int bq, int kblocks) {
    return static_cast<size_t>((kblocks * bq * kRowBytes + 1023) / 1024 * 1024) + kStages * kABytes + 256 + bq * 24 + 256 + 1024;
}

template <int BQ>
int LaunchTyped(const CUtensorMap& map_x, const CUtensorMap& map_w, const ConvTcParams& p, size_t smem, cudaStream_t stream) {
    auto kernel = ConvTcgen05Kernel<BQ>;
    if (EnsureDynamicSmem(reinterpret_cast<const void*>(kernel), smem) != FTH_B200_OK) return FTH_B200_ERR_CUDA;
    const int sms = SmCount();
    const int grid = static_cast<int>(p.tiles < sms ? p.tiles : sms);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // set-up overlaps the layout pass in front
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, map_x, map_w, p) != cudaSuccess) return FTH_B200_ERR_CUDA;
    NoteLaunch("conv_tcgen05");
    return CheckLaunch();
}

}  // namespace

bool ConvTcgen05Supported(const ConvArgs& c) {
    if (c.stride_h != 1 || c.stride_w != 1 || c.dilation_h != 1 || c.dilation_w != 1 || c.group != 1) return false;
    if (c.x_zp != 0 || c.w_zps != nullptr) return false;  // TMA zero fill equals "tap skipped" only for zero point 0
    if (c.ic % 64 != 0 || c.oc < 1 || c.oc > 256) return false;
    if (c.workspace == nullptr || c.workspace_bytes < ConvTcgen05WorkspaceBytes(c)) return false;
    if (reinterpret_cast<uintptr_t>(c.workspace) % 256 != 0) return false;
    if (c.packed_w != nullptr && reinterpret_cast<uintptr_t>(c.packed_w) % 256 != 0) return false;
    const int kblocks = static_cast<int>(c.kh * c.kw * (c.ic / 64));
    if (SmemBytesFor(BlockQFor(c.oc), kblocks) > 220 * 1024) return false;
    if (c.batch > 0x7fffffff || c.ih > 0x7fffffff || c.iw > 0x7fffffff) return false;
    return true;
}

size_t ConvTcgen05WorkspaceBytes(const ConvArgs& c) {
    if (c.stride_h != 1 || c.stride_w != 1 || c.dilation_h != 1 || c.dilation_w != 1 || c.group != 1) return 0;
    if (c.x_zp != 0 || c.w_zps != nullptr || c.ic % 64 != 0 || c.oc > 256) return 0;
    const size_t nhwc = Align256(static_cast<size_t>(c.batch * c.ih * c.iw * c.ic));
    return c.packed_w != nullptr ? nhwc : nhwc + Align256(static_cast<size_t>(c.oc * c.kh * c.kw * c.ic));
}

size_t ConvPackedWeightBytes(const ConvArgs& c) {
    if (c.stride_h != 1 || c.stride_w != 1 || c.dilation_h != 1 || c.dilation_w != 1 || c.group != 1) return 0;
    if (c.x_zp != 0 || c.w_zps != nullptr || c.ic % 64 != 0 || c.oc > 256) return 0;
    return Align256(static_cast<size_t>(c.oc * c.kh * c.kw * c.ic));
}

int LaunchConvPackWeights(const ConvArgs& c, void* packed, cudaStream_t stream) {
    if (ConvPackedWeightBytes(c) == 0) return FTH_B200_ERR_UNSUPPORTED;
    if (packed == nullptr || reinterpret_cast<uintptr_t>(packed) % 256 != 0) return FTH_B200_ERR_INVALID;
    const int64_t taps = c.kh * c.kw;
    const int64_t total = c.oc * c.ic * taps;
    PackConvWeightKernel<<<static_cast<unsigned>((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184), 256, 0, stream>>>(
        c.w, static_cast<int8_t*>(packed), c.oc, c.ic, taps);
    NoteLaunch("conv_pack");
    return CheckLaunch();
}

int LaunchConvTcgen05(const ConvArgs& c, cudaStream_t stream) {
    if (!ConvTcgen05Supported(c)) return FTH_B200_ERR_UNSUPPORTED;
    int8_t* nhwc = static_cast<int8_t*>(c.workspace);
    const int8_t* packed = c.packed_w != nullptr ? c.packed_w : nhwc + Align256(static_cast<size_t>(c.batch * c.ih * c.iw * c.ic));
    const int64_t taps = c.kh * c.kw;
    if (c.packed_w == nullptr && !c.weights_packed) {
        const int64_t total = c.oc * c.ic * taps;
        PackConvWeightKernel<<<static_cast<unsigned>((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184), 256, 0, stream>>>(c.w, const_cast<int8_t*>(packed), c.oc, c.ic, taps);
        NoteLaunch("conv_tcgen05");
    }
    {
        const bool aligned = c.iw % 4 == 0 && c.iw <= kRowTileW && c.ic % 16 == 0 && reinterpret_cast<uintptr_t>(c.x) % 4 == 0 &&
                             c.batch * c.ih <= 0x7fffffff;
        if (aligned) {
            const dim3 grid(static_cast<unsigned>(c.batch * c.ih), static_cast<unsigned>((c.ic + 63) / 64));
            NchwToNhwcRowKernel<<<grid, 256, 0, stream>>>(c.x, nhwc, c.ic, c.ih, c.iw);
        } else {
            const dim3 grid(static_cast<unsigned>((c.iw + 31) / 32), static_cast<unsigned>((c.ic + 63) / 64), static_cast<unsigned>(c.batch * c.ih));
            NchwToNhwcKernel<<<grid, 256, 0, stream>>>(c.x, nhwc, c.batch, c.ic, c.ih, c.iw);
        }
        NoteLaunch("conv_tcgen05");
    }
    ConvTcParams p;
    p.c = c;
    if (c.packed_w != nullptr) p.c.weights_packed = 1;  // packed by an earlier, completed pass: may be fetched early
    p.taps = static_cast<int>(taps);
    p.cblocks = static_cast<int>(c.ic / 64);
    p.kblocks = p.taps * p.cblocks;
    p.tiles_w = (c.ow + kTileW - 1) / kTileW;
    p.tiles_h = (c.oh + kTileH - 1) / kTileH;
    p.tiles = p.tiles_w * p.tiles_h * c.batch;
    p.status = DeviceStatusPtr();
    const int bq = BlockQFor(c.oc);
    p.idesc = umma::InstrDesc(2u, 1u, 1u, false, false, 128u, static_cast<uint32_t>(bq));
    CUtensorMap map_x, map_w;
    const uint64_t dims[4] = {static_cast<uint64_t>(c.ic), static_cast<uint64_t>(c.iw), static_cast<uint64_t>(c.ih), static_cast<uint64_t>(c.batch)};
    const uint64_t strides[3] = {static_cast<uint64_t>(c.ic), static_cast<uint64_t>(c.iw * c.ic), static_cast<uint64_t>(c.ih * c.iw * c.ic)};
    const uint32_t box[4] = {kRowBytes, kTileW, kTileH, 1};
    if (!MakeTensorMap4D(&map_x, nhwc, dims, strides, box, TmaSwizzle::k64B)) return FTH_B200_ERR_CUDA;
    if (!MakeTensorMap2D(&map_w, packed, static_cast<uint64_t>(taps * c.ic), static_cast<uint64_t>(c.oc), static_cast<uint64_t>(taps * c.ic),
                         kRowBytes, static_cast<uint32_t>(bq), TmaSwizzle::k64B)) return FTH_B200_ERR_CUDA;
    const size_t smem = SmemBytesFor(bq, p.kblocks);
    switch (bq) {
        case 32: return LaunchTyped<32>(map_x, map_w, p, smem, stream);
        case 64: return LaunchTyped<64>(map_x, map_w, p, smem, stream);
        case 128: return LaunchTyped<128>(map_x, map_w, p, smem, stream);
        default: return LaunchTyped<256>(map_x, map_w, p, smem, stream);
    }
}

}  // namespace fth
