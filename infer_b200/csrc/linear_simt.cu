// Ragged-shape linear kernel on CUDA cores: any M, K, N, either weight layout, no alignment demands.
// It exists for the shapes the TMA / tcgen05 kernels cannot take (row strides that are not multiples of
// 16 bytes, tiny matrices) so that the backend never needs a CPU fallback; big aligned shapes are routed
// to the streaming and tensor-core kernels instead.
//
// 64 x 64 output tile per CTA, 256 threads, 4 x 4 outputs per thread, K consumed 32 at a time through
// shared memory.  FP8 operands are decoded once while staging; INT8 operands are widened to int32.
#include "common.cuh"
#include "linear_internal.h"

namespace fth {
namespace {

constexpr int kTile = 64;
constexpr int kStepK = 32;
constexpr int kThreads = 256;

template <int DTYPE>
struct Acc { using type = float; };
template <>
struct Acc<FTH_B200_INT8> { using type = int32_t; };

template <int DTYPE>
__global__ void __launch_bounds__(kThreads) LinearSimtKernel(LinearArgs args, Fp8Epilogue fe, Int8Epilogue ie) {
    using T = typename Acc<DTYPE>::type;
    __shared__ T a_tile[kStepK][kTile + 1];
    __shared__ T w_tile[kStepK][kTile + 1];

    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kTile;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * kTile;
    const int tx = threadIdx.x % 16;  // column group
    const int ty = threadIdx.x / 16;  // row group

    T acc[4][4];
    T row_sum[4] = {0, 0, 0, 0};
    T col_sum[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0;

    for (int64_t k0 = 0; k0 < args.k; k0 += kStepK) {
        // stage A: kTile rows x kStepK
        for (int idx = threadIdx.x; idx < kTile * kStepK; idx += kThreads) {
            const int r = idx / kStepK, c = idx % kStepK;
            const int64_t gm = m0 + r, gk = k0 + c;
            T v = 0;
            if (gm < args.m && gk < args.k) {
                if constexpr (DTYPE == FTH_B200_INT8) v = LoadInt8Activation(args.a, gm * args.k + gk, args.a_dtype, ie.a_scale, ie.a_zp);
                else v = LoadActivation<DTYPE>(args.a, gm * args.k + gk, args.a_dtype, args.a_scale);
            }
            a_tile[c][r] = v;
        }
        // stage W: kStepK x kTile (read along the contiguous dimension of the weight)
        for (int idx = threadIdx.x; idx < kTile * kStepK; idx += kThreads) {
            int kk, nn;
            if (args.trans_b) { nn = idx / kStepK; kk = idx % kStepK; }
            else { kk = idx / kTile; nn = idx % kTile; }
            const int64_t gk = k0 + kk, gn = n0 + nn;
            T v = 0;
            if (gk < args.k && gn < args.n) {
                const int64_t off = args.trans_b ? gn * args.k + gk : gk * args.n + gn;
                if constexpr (DTYPE == FTH_B200_INT8) v = static_cast<const int8_t*>(args.w)[off];
                else v = Decode<DTYPE>(static_cast<const uint8_t*>(args.w)[off]);
            }
            w_tile[kk][nn] = v;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < kStepK; ++kk) {
            T av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = a_tile[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = w_tile[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if constexpr (DTYPE == FTH_B200_INT8) acc[i][j] += av[i] * wv[j];
                    else acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
                }
            if constexpr (DTYPE == FTH_B200_INT8) {
#pragma unroll
                for (int i = 0; i < 4; ++i) { row_sum[i] += av[i]; col_sum[i] += wv[i]; }
            }
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t gm = m0 + ty * 4 + i;
        if (gm >= args.m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t gn = n0 + tx * 4 + j;
            if (gn >= args.n) continue;
            if constexpr (DTYPE == FTH_B200_INT8) StoreInt8Result(ie, gm, gn, acc[i][j], row_sum[i], col_sum[j]);
            else StoreFp8Result<DTYPE>(fe, gm, gn, acc[i][j]);
        }
    }
}

}  // namespace

int LaunchLinearSimt(int dtype, const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie,
                     cudaStream_t stream) {
    const dim3 grid(static_cast<unsigned>((args.n + kTile - 1) / kTile), static_cast<unsigned>((args.m + kTile - 1) / kTile));
    if (grid.y > 65535u) return FTH_B200_ERR_UNSUPPORTED;
    switch (dtype) {
        case FTH_B200_FP8E4M3: LinearSimtKernel<FTH_B200_FP8E4M3><<<grid, kThreads, 0, stream>>>(args, fe, ie); break;
        case FTH_B200_FP8E5M2: LinearSimtKernel<FTH_B200_FP8E5M2><<<grid, kThreads, 0, stream>>>(args, fe, ie); break;
        case FTH_B200_INT8: LinearSimtKernel<FTH_B200_INT8><<<grid, kThreads, 0, stream>>>(args, fe, ie); break;
        default: return FTH_B200_ERR_INVALID;
    }
    NoteLaunch("simt");
    return CheckLaunch();
}

}  // namespace fth
