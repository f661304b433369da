// Row helpers shared by the decoder-block operators (decoder_ops.cu) and the linear kernels that fuse them in front of a
// projection (linear_tc_cluster.cu): typed reads / writes of eight consecutive elements and the one summation order
// every kernel uses for the squares of a row, so that a fused QwenRmsNorm gives the bits of the stand-alone kernel.
#pragma once

#include "common.cuh"

namespace fth {
namespace rowops {

constexpr int kRowThreads = 128;  // threads that share one row
constexpr int kRowGroups = 4;     // groups of eight elements per thread held in registers: rows of up to 4096 elements

template <int DTYPE>
__device__ __forceinline__ float ReadFloat(const void* x, int64_t i) {
    if constexpr (DTYPE == FTH_B200_FP32) return static_cast<const float*>(x)[i];
    else if constexpr (DTYPE == FTH_B200_BF16) return DecodeBf16(static_cast<const uint16_t*>(x)[i]);
    else return __half2float(static_cast<const __half*>(x)[i]);
}
template <int DTYPE>
__device__ __forceinline__ void WriteFloat(void* out, int64_t i, float v) {
    if constexpr (DTYPE == FTH_B200_FP32) static_cast<float*>(out)[i] = v;
    else if constexpr (DTYPE == FTH_B200_BF16) static_cast<uint16_t*>(out)[i] = EncodeBf16Cast(v);
    else static_cast<__half*>(out)[i] = __float2half_rn(v);
}

// Eight consecutive elements starting at a multiple of eight (one 16-byte load for BF16 / FP16, two for FP32).
template <int DTYPE>
__device__ __forceinline__ void ReadEight(const void* x, int64_t i, bool vec, float (&v)[8]) {
    if (!vec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = ReadFloat<DTYPE>(x, i + j);
        return;
    }
    if constexpr (DTYPE == FTH_B200_FP32) {
        const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(x) + i);
        const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(x) + i + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + i);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if constexpr (DTYPE == FTH_B200_BF16) {
                v[2 * j] = __uint_as_float(w[j] << 16);
                v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
            } else {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                v[2 * j] = f.x;
                v[2 * j + 1] = f.y;
            }
        }
    }
}
template <int DTYPE>
__device__ __forceinline__ void WriteEight(void* out, int64_t i, bool vec, const float (&v)[8]) {
    if (!vec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) WriteFloat<DTYPE>(out, i + j, v[j]);
        return;
    }
    if constexpr (DTYPE == FTH_B200_FP32) {
        *reinterpret_cast<float4*>(static_cast<float*>(out) + i) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(static_cast<float*>(out) + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if constexpr (DTYPE == FTH_B200_BF16) {
                w[j] = EncodeBf16Cast(v[2 * j]) | (static_cast<uint32_t>(EncodeBf16Cast(v[2 * j + 1])) << 16);
            } else {
                const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
                w[j] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
        *reinterpret_cast<uint4*>(static_cast<uint16_t*>(out) + i) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

__device__ __forceinline__ bool Aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Lanes of a warp combined with an xor tree.
__device__ __forceinline__ float WarpTreeSum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// This thread's part of the sum of squares of a row of `hidden` <= 4096 elements starting at element `base`: the
// elements of its groups t, t + 128, t + 256, t + 384 (eight consecutive elements each), multiplied and added one
// after another in FP32.  The values are kept in `xv` for the second pass.
template <int X>
__device__ __forceinline__ float ThreadSumSquares(const void* x, int64_t base, int64_t hidden, bool vec, int t, float (&xv)[kRowGroups][8]) {
    const int64_t groups = (hidden + 7) / 8;
    float sum = 0.0f;
#pragma unroll
    for (int g = 0; g < kRowGroups; ++g) {
        const int64_t gi = t + static_cast<int64_t>(g) * kRowThreads;
        if (gi >= groups) continue;
        if (gi * 8 + 8 <= hidden) {
            ReadEight<X>(x, base + gi * 8, vec, xv[g]);
#pragma unroll
            for (int j = 0; j < 8; ++j) sum = __fadd_rn(sum, __fmul_rn(xv[g][j], xv[g][j]));
        } else {  // ragged last group
            for (int64_t c = gi * 8; c < hidden; ++c) {
                const float v = ReadFloat<X>(x, base + c);
                sum = __fadd_rn(sum, __fmul_rn(v, v));
            }
        }
    }
    return sum;
}
__device__ __forceinline__ float InverseRms(float sum_squares, int64_t hidden, float epsilon) {
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum_squares, static_cast<float>(hidden)), epsilon)));
}
// SiLU as the reference computes it, x / (1 + exp(-x)) in FP32, with exp evaluated in double and rounded to FP32 once
// (overflow gives +Inf and x / Inf = 0, as on the host).
__device__ __forceinline__ float SiluValue(float x) {
    const float e = static_cast<float>(exp(static_cast<double>(-x)));
    return __fdiv_rn(x, __fadd_rn(1.0f, e));
}

// The BF16 bits of the SiLU node's output, EncodeBf16Cast(SiluValue(x)), without the double-precision exponential on
// nearly every input.  expf is within 2 ulp of the correctly rounded exponential; 1 + e and the division are rounded the
// same way on both paths, so the FP32 quotient is at most a few FP32 steps off, and the BF16 rounding of both is the
// same unless the quotient sits that close to the midpoint between two BF16 values.  Those inputs, and Inf / NaN, take
// the exact path.  (tests/test_gpu_decoder_ops.py runs all 65536 BF16 inputs.)
static __device__ __noinline__ float SiluValueOutOfLine(float x) { return SiluValue(x); }
__device__ __forceinline__ uint16_t SiluToBf16(float x) {
    const float e = expf(-x);
    float s = __fdiv_rn(x, __fadd_rn(1.0f, e));
    const uint32_t low = __float_as_uint(s) & 0xffffu;
    const bool finite = (__float_as_uint(x) & 0x7f800000u) != 0x7f800000u;
    if (!finite || (low >= 0x7fc0u && low <= 0x8040u)) s = SiluValueOutOfLine(x);
    return EncodeBf16Cast(s);
}

}  // namespace rowops
}  // namespace fth
