// Shared device helpers: FP8 codec, exact INT8 requantisation, vector load helpers, launch bookkeeping.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fth_b200.h"

namespace fth {

constexpr int kNumSms = 148;  // B200: 2 dies x 74 SMs

// ---- launch bookkeeping (host) ---------------------------------------------------------------------
void NoteLaunch(const char* variant, int64_t launches = 1);
int CheckLaunch();  // FTH_B200_OK or FTH_B200_ERR_CUDA (reads and clears the last error)
void ClearStaleError();  // discards an error left behind by other code before this library launches
// Per-device launch set-up.  One process may drive several GPUs (one session per device), and both the SM count and
// a kernel's dynamic shared-memory limit belong to the device that is current at the launch.
int SmCount();  // SMs of the current device (looked up once per device)
// Raises `kernel`'s dynamic shared-memory limit to `bytes` on the current device unless it is already that high there.
int EnsureDynamicSmem(const void* kernel, size_t bytes);  // FTH_B200_OK or FTH_B200_ERR_CUDA

// ---- FP8 codec -------------------------------------------------------------------------------------
// Decode through the hardware converters: exact for every code, including subnormals, the E4M3 NaN
// codes (0x7F / 0xFF) and the E5M2 Inf / NaN codes (include/util/fp8.h:174-204).
template <int DTYPE>
__device__ __forceinline__ float2 DecodePair(uint16_t two_codes) {
    uint32_t h2;
    if constexpr (DTYPE == FTH_B200_FP8E4M3) {
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(two_codes));
    } else {
        asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(h2) : "h"(two_codes));
    }
    return __half22float2(*reinterpret_cast<__half2*>(&h2));
}

template <int DTYPE>
__device__ __forceinline__ float Decode(uint8_t code) {
    return DecodePair<DTYPE>(static_cast<uint16_t>(code)).x;
}

// Saturating round-to-nearest-even encode with the reference's treatment of non-finite inputs
// (include/util/fp8.h:148-172): E4M3 NaN → sign|0x7F, ±Inf → sign|0x7E; E5M2 NaN → sign|0x7D, ±Inf → sign|0x7C.
template <int DTYPE>
__device__ __forceinline__ uint8_t Encode(float value) {
    const uint32_t bits = __float_as_uint(value);
    if ((bits & 0x7f800000u) == 0x7f800000u) {
        const uint8_t sign = static_cast<uint8_t>((bits >> 24) & 0x80u);
        const bool nan = (bits & 0x007fffffu) != 0;
        if constexpr (DTYPE == FTH_B200_FP8E4M3) return sign | (nan ? 0x7fu : 0x7eu);
        return sign | (nan ? 0x7du : 0x7cu);
    }
    uint16_t packed;
    if constexpr (DTYPE == FTH_B200_FP8E4M3) {
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(packed) : "f"(0.0f), "f"(value));
    } else {
        asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(packed) : "f"(0.0f), "f"(value));
    }
    return static_cast<uint8_t>(packed & 0xffu);
}

// BF16 encoders of the reference: Cast quiets NaNs (include/util/bf16.h:35-46), DequantizeLinear does
// not (src/kernel/common/quantize_linear_utils.h:109-116).
__device__ __forceinline__ uint16_t EncodeBf16Cast(float value) {
    const uint32_t b = __float_as_uint(value);
    if ((b & 0x7f800000u) == 0x7f800000u && (b & 0x007fffffu) != 0) return static_cast<uint16_t>((b >> 16) | 0x0040u);
    return static_cast<uint16_t>((b + 0x7fffu + ((b >> 16) & 1u)) >> 16);
}
__device__ __forceinline__ uint16_t EncodeBf16Dq(float value) {
    const uint32_t b = __float_as_uint(value);
    const uint32_t low = b & 0xffffu;
    uint32_t high = b >> 16;
    if (low > 0x8000u || (low == 0x8000u && (high & 1u))) ++high;
    return static_cast<uint16_t>(high);
}
__device__ __forceinline__ float DecodeBf16(uint16_t bits) { return __uint_as_float(static_cast<uint32_t>(bits) << 16); }

// Reads one activation element as the value the reference MatMul would see.
//   a_dtype == 0 / dtype: decode(code)
//   a_dtype == BF16 / FP32: the Cast node in front is replayed: decode(encode(x / a_scale)).
template <int DTYPE>
__device__ __forceinline__ float LoadActivation(const void* a, int64_t index, int a_dtype, float a_scale) {
    if (a_dtype == FTH_B200_BF16) {
        const float x = DecodeBf16(static_cast<const uint16_t*>(a)[index]);
        return Decode<DTYPE>(Encode<DTYPE>(__fdiv_rn(x, a_scale)));
    }
    if (a_dtype == FTH_B200_FP32) {
        const float x = static_cast<const float*>(a)[index];
        return Decode<DTYPE>(Encode<DTYPE>(__fdiv_rn(x, a_scale)));
    }
    return Decode<DTYPE>(static_cast<const uint8_t*>(a)[index]);
}

// ---- FP8 epilogue ------------------------------------------------------------------------------------
struct Fp8Epilogue {
    float ab_scale;  // a_scale * w_scale (per-tensor) or a_scale alone when channel scales are given
    const float* w_channel_scales;
    float alpha, beta;
    int is_gemm;
    const uint8_t* bias;
    int bias_mode;
    float bias_scale;
    float out_scale;
    void* out;
    int out_dtype;
    int64_t ldo;
    int64_t n;
};

// y = alpha·acc·scales + beta·bias; code = encode(y / out_scale); store FP8, or the decoded value as
// BF16 / FP32 when a Cast node behind the MatMul is fused.
template <int DTYPE>
__device__ __forceinline__ void StoreFp8Result(const Fp8Epilogue& e, int64_t row, int64_t col, float acc) {
    float scale = e.ab_scale;
    if (e.w_channel_scales != nullptr) scale *= e.w_channel_scales[col];
    float y = __fmul_rn(acc, scale);
    if (e.is_gemm) y = __fmul_rn(y, e.alpha);
    if (e.bias_mode != FTH_B200_BIAS_NONE) {
        const int64_t bi = e.bias_mode == FTH_B200_BIAS_VECTOR ? col : row * e.n + col;
        float b = __fmul_rn(Decode<DTYPE>(e.bias[bi]), e.bias_scale);
        if (e.is_gemm) b = __fmul_rn(e.beta, b);
        y = __fadd_rn(y, b);
    }
    const uint8_t code = Encode<DTYPE>(__fdiv_rn(y, e.out_scale));
    const int64_t o = row * e.ldo + col;
    if (e.out_dtype == FTH_B200_BF16) {
        static_cast<uint16_t*>(e.out)[o] = EncodeBf16Cast(__fmul_rn(Decode<DTYPE>(code), e.out_scale));
    } else if (e.out_dtype == FTH_B200_FP32) {
        static_cast<float*>(e.out)[o] = __fmul_rn(Decode<DTYPE>(code), e.out_scale);
    } else {
        static_cast<uint8_t*>(e.out)[o] = code;
    }
}

// ---- INT8 requantisation ---------------------------------------------------------------------------
// The reference rule (src/kernel/common/int8_kernel_utils.h:159-179), operation by operation:
//   real = double(acc) * scale;  t = real / double(out_scale) + out_zp;  q = clamp(round_half_away(t)).
__device__ __forceinline__ int8_t RequantExact(double acc_real, double out_scale, int32_t out_zp) {
    const double t = __dadd_rn(__ddiv_rn(acc_real, out_scale), static_cast<double>(out_zp));
    const double r = round(t);  // ties away from zero, as std::round
    return static_cast<int8_t>(static_cast<int32_t>(fmax(-128.0, fmin(127.0, r))));
}

// Same result as RequantExact(double(acc) * scale, …) with one FMA on the common path.
// `mult` = scale / out_scale rounded once.  The exact sequence rounds three times, the FMA once, so for
// |t| < 256 the two values differ by less than 256 · 5 · 2^-53 < 1e-12.  Whenever the estimate is farther
// than 1e-6 from a rounding boundary (x.5) both therefore round to the same integer; otherwise the exact
// sequence runs.  For |estimate| >= 256 both are far outside [-128.5, 127.5] and clamp identically.
__device__ __forceinline__ int8_t RequantInt32(int32_t acc, double scale, double mult, double out_scale,
                                               int32_t out_zp) {
    const double est = fma(static_cast<double>(acc), mult, static_cast<double>(out_zp));
    if (est >= 256.0) return 127;
    if (est <= -256.0) return -128;
    const double fl = floor(est);
    const double frac = est - fl;
    if (fabs(frac - 0.5) < 1e-6) {
        return RequantExact(__dmul_rn(static_cast<double>(acc), scale), out_scale, out_zp);
    }
    const double r = frac < 0.5 ? fl : fl + 1.0;
    return static_cast<int8_t>(static_cast<int32_t>(fmax(-128.0, fmin(127.0, r))));
}

// INT8 requantisation in three stages, each deciding only what its error bound allows.
//   1. est = fma(float(acc), float(scale / out_scale), zp) differs from the exact value T by at most
//      (|T| + |zp|) * 4 * 2^-24 < 1e-4 for |T| <= 300 (three FP32 roundings), and the reference's double sequence
//      differs from T by less than 1e-12.  Farther than 2e-4 from a rounding boundary x.5, both round alike.
//      |est| >= 300 saturates either way.
//   2. The ~4 values in 10^4 inside that band take one double FMA with mult_d = scale / out_scale to within a few
//      2^-53 (RequantInt32: within 1e-12 of the reference's value, decided unless within 1e-6 of a boundary).
//   3. What is left runs the reference's own sequence (double multiply, divide, add, round).
// A warp takes a stage whenever one of its lanes needs it, and the double divide of stage 3 costs a thousand
// cycles: with stage 2 in between it is practically never reached.
__device__ __forceinline__ int8_t RequantFast(int32_t acc, float mult_f, double mult_d, double scale_d, double so_d, int32_t zp) {
    const float est = fmaf(__int2float_rn(acc), mult_f, static_cast<float>(zp));
    if (est >= 300.0f) return 127;
    if (est <= -300.0f) return -128;
    const float fl = floorf(est);
    const float frac = est - fl;
    if (fabsf(frac - 0.5f) < 2e-4f) return RequantInt32(acc, scale_d, mult_d, so_d, zp);
    const float r = frac < 0.5f ? fl : fl + 1.0f;
    return static_cast<int8_t>(static_cast<int32_t>(fmaxf(-128.0f, fminf(127.0f, r))));
}

// Stage 1 of RequantFast without a branch, for epilogues that requantise many accumulators per thread: straight-line
// code lets the independent chains overlap.  Returns the stage-1 result as an unsigned byte and sets bit `bit` of
// `near` when the estimate lies inside the undecided band; those few values are redone with RequantInt32
// afterwards.  Saturation falls out of the clamp (an estimate beyond +-300 is never inside the band).
__device__ __forceinline__ uint32_t RequantEstimate(int32_t acc, float mult_f, float zp_f, uint32_t bit, uint32_t* near) {
    const float est = fmaf(__int2float_rn(acc), mult_f, zp_f);
    const float fl = floorf(est);
    const float frac = est - fl;
    *near |= (fabsf(frac - 0.5f) < 2e-4f && fabsf(est) < 300.0f) ? (1u << bit) : 0u;
    const float r = frac < 0.5f ? fl : fl + 1.0f;
    return static_cast<uint32_t>(static_cast<int32_t>(fmaxf(-128.0f, fminf(127.0f, r)))) & 0xffu;
}

// QuantizeLinear on one value (include/quant/quantization.h:94-99).
__device__ __forceinline__ int8_t QuantizeValue(float value, float scale, int32_t zp) {
    const double t = __dadd_rn(__ddiv_rn(static_cast<double>(value), static_cast<double>(scale)),
                               static_cast<double>(zp));
    const double r = round(t);
    // NaN compares false in fmin/fmax chains the way std::min/std::max do in the reference:
    // std::min(127.0, NaN) = 127.0, std::max(-128.0, 127.0) = 127.0.
    if (r != r) return 127;
    return static_cast<int8_t>(static_cast<int32_t>(fmax(-128.0, fmin(127.0, r))));
}

struct Int8Epilogue {
    const float* w_scales;
    const int32_t* w_zps;
    int per_channel;
    float a_scale;
    int32_t a_zp;
    float out_scale;
    int32_t out_zp;
    const int32_t* bias;
    int bias_mode;
    int is_gemm;
    float alpha, beta;
    void* out;
    int out_dtype;
    int64_t ldo;
    int64_t n;
    int64_t k;
};

// Reads one INT8 activation; a_dtype == FP32 replays the QuantizeLinear node in front.
__device__ __forceinline__ int8_t LoadInt8Activation(const void* a, int64_t index, int a_dtype, float a_scale,
                                                     int32_t a_zp) {
    if (a_dtype == FTH_B200_FP32) return QuantizeValue(static_cast<const float*>(a)[index], a_scale, a_zp);
    return static_cast<const int8_t*>(a)[index];
}

// acc = Σ a·w over raw int8 values; row_sum = Σ_k a, col_sum = Σ_k w — used only when a zero point is
// non-zero:  Σ (a - za)(w - zw) = Σ a·w - zw·Σa - za·Σw + K·za·zw.
__device__ __forceinline__ void StoreInt8Result(const Int8Epilogue& e, int64_t row, int64_t col, int32_t raw,
                                                int32_t row_sum, int32_t col_sum) {
    const int32_t zw = e.w_zps != nullptr ? e.w_zps[e.per_channel ? col : 0] : 0;
    int64_t acc64 = raw;
    if (zw != 0 || e.a_zp != 0) {
        acc64 = static_cast<int64_t>(raw) - static_cast<int64_t>(zw) * row_sum -
                static_cast<int64_t>(e.a_zp) * col_sum + e.k * static_cast<int64_t>(e.a_zp) * zw;
    }
    int32_t b = 0;
    if (e.bias_mode != FTH_B200_BIAS_NONE) b = e.bias[e.bias_mode == FTH_B200_BIAS_VECTOR ? col : row * e.n + col];
    const double scale = static_cast<double>(e.a_scale) * static_cast<double>(e.w_scales[e.per_channel ? col : 0]);
    const double so = static_cast<double>(e.out_scale);
    int8_t q;
    if (e.is_gemm && (e.alpha != 1.0f || e.beta != 1.0f)) {
        const double accd = __dadd_rn(__dmul_rn(static_cast<double>(e.alpha), static_cast<double>(acc64)),
                                      __dmul_rn(static_cast<double>(e.beta), static_cast<double>(b)));
        q = RequantExact(__dmul_rn(accd, scale), so, e.out_zp);
    } else {
        // alpha = beta = 1: alpha·dot + beta·bias is the exact integer sum in double, as in FC.
        const int32_t acc = static_cast<int32_t>(acc64 + b);
        q = RequantInt32(acc, scale, scale / so, so, e.out_zp);
    }
    const int64_t o = row * e.ldo + col;
    if (e.out_dtype == FTH_B200_FP32) {
        static_cast<float*>(e.out)[o] = __fmul_rn(static_cast<float>(static_cast<int32_t>(q) - e.out_zp), e.out_scale);
    } else {
        static_cast<int8_t*>(e.out)[o] = q;
    }
}

// ---- streaming loads ---------------------------------------------------------------------------------
__device__ __forceinline__ uint4 LoadStream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

}  // namespace fth
