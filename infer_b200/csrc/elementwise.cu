// Cast, QuantizeLinear, DequantizeLinear, INT8 table lookup.
// All are HBM-bound byte streams: 16 bytes per thread per access on the widest side, grid-stride loops
// over a grid sized in multiples of the SM count.
#include "common.cuh"

namespace fth {
namespace {

constexpr int kThreads = 256;

inline int GridFor(int64_t work_items) {
    const int64_t blocks = (work_items + kThreads - 1) / kThreads;
    const int64_t cap = static_cast<int64_t>(kNumSms) * 8;
    return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

// ---- Cast ------------------------------------------------------------------------------------------
template <int IN>
__device__ __forceinline__ float ReadAs(const void* x, int64_t i, float in_scale) {
    if constexpr (IN == FTH_B200_FP32) return static_cast<const float*>(x)[i];
    else if constexpr (IN == FTH_B200_BF16) return DecodeBf16(static_cast<const uint16_t*>(x)[i]);
    else if constexpr (IN == FTH_B200_FP16) return __half2float(static_cast<const __half*>(x)[i]);
    else return __fmul_rn(Decode<IN>(static_cast<const uint8_t*>(x)[i]), in_scale);
}

template <int OUT>
__device__ __forceinline__ void WriteAs(void* out, int64_t i, float v, float out_scale) {
    if constexpr (OUT == FTH_B200_FP32) static_cast<float*>(out)[i] = v;
    else if constexpr (OUT == FTH_B200_BF16) static_cast<uint16_t*>(out)[i] = EncodeBf16Cast(v);
    else if constexpr (OUT == FTH_B200_FP16) static_cast<__half*>(out)[i] = __float2half_rn(v);
    else {
        // a NaN keeps its sign through the reference's division on the host; GPU arithmetic would canonicalise
        // it, so NaNs skip the divide
        static_cast<uint8_t*>(out)[i] = (v != v) ? Encode<OUT>(v) : Encode<OUT>(__fdiv_rn(v, out_scale));
    }
}

template <int N> struct Bytes { static constexpr int value = (N == FTH_B200_FP32) ? 4 : (N == FTH_B200_BF16 || N == FTH_B200_FP16) ? 2 : 1; };

// Each thread converts groups of 16 elements: the narrow side moves as one 16-byte access, the wide
// side as 2 or 4 of them.
template <int IN, int OUT>
__global__ void __launch_bounds__(kThreads) CastKernel(const void* __restrict__ x, void* __restrict__ out,
                                                       int64_t count, float in_scale, float out_scale,
                                                       int aligned) {
    // lets a dependent kernel launched with programmatic serialization set itself up while this one runs
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int64_t groups = count / 16;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    if (aligned) {
        for (int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; g < groups; g += stride) {
            alignas(16) uint8_t in_buf[16 * Bytes<IN>::value];
            alignas(16) uint8_t out_buf[16 * Bytes<OUT>::value];
            const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(x) + g * 16 * Bytes<IN>::value);
#pragma unroll
            for (int v = 0; v < Bytes<IN>::value; ++v) reinterpret_cast<uint4*>(in_buf)[v] = LoadStream16(src + v);
#pragma unroll
            for (int i = 0; i < 16; ++i) WriteAs<OUT>(out_buf, i, ReadAs<IN>(in_buf, i, in_scale), out_scale);
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(out) + g * 16 * Bytes<OUT>::value);
#pragma unroll
            for (int v = 0; v < Bytes<OUT>::value; ++v) dst[v] = reinterpret_cast<uint4*>(out_buf)[v];
        }
    }
    const int64_t start = aligned ? groups * 16 : 0;
    for (int64_t i = start + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < count; i += stride) {
        WriteAs<OUT>(out, i, ReadAs<IN>(x, i, in_scale), out_scale);
    }
}

template <int IN>
int LaunchCastOut(int out_dtype, const void* x, void* out, int64_t count, float in_scale, float out_scale,
                  cudaStream_t stream) {
    const int aligned = (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(out) % 16 == 0);
    const int grid = GridFor(count / 16 + 1);
    switch (out_dtype) {
#define FTH_CASE(OUT) case OUT: CastKernel<IN, OUT><<<grid, kThreads, 0, stream>>>(x, out, count, in_scale, out_scale, aligned); break;
        FTH_CASE(FTH_B200_FP32) FTH_CASE(FTH_B200_BF16) FTH_CASE(FTH_B200_FP16) FTH_CASE(FTH_B200_FP8E4M3)
        FTH_CASE(FTH_B200_FP8E5M2)
#undef FTH_CASE
        default: return FTH_B200_ERR_UNSUPPORTED;
    }
    NoteLaunch("cast");
    return CheckLaunch();
}

// ---- QuantizeLinear / DequantizeLinear ----------------------------------------------------------------
template <int IN>
__global__ void __launch_bounds__(kThreads) QuantizeKernel(const void* __restrict__ x, const float* __restrict__ scales,
                                                           const int32_t* __restrict__ zps, int64_t params,
                                                           int8_t* __restrict__ out, int64_t count, int64_t channels, int64_t inner) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * 4;
    for (int64_t base = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) * 4; base < count; base += stride) {
        int8_t q[4];
        const int lim = count - base < 4 ? static_cast<int>(count - base) : 4;
        for (int j = 0; j < lim; ++j) {
            const int64_t i = base + j;
            const int64_t c = params == 1 ? 0 : (inner == 1 ? i : i / inner) % channels;  // the channel axis may be an inner one
            q[j] = QuantizeValue(ReadAs<IN>(x, i, 1.0f), scales[c], zps[c]);
        }
        if (lim == 4 && (reinterpret_cast<uintptr_t>(out + base) & 3) == 0) {
            *reinterpret_cast<char4*>(out + base) = make_char4(q[0], q[1], q[2], q[3]);
        } else {
            for (int j = 0; j < lim; ++j) out[base + j] = q[j];
        }
    }
}

template <int OUT>
__global__ void __launch_bounds__(kThreads) DequantizeKernel(const int8_t* __restrict__ x, const float* __restrict__ scales,
                                                             const int32_t* __restrict__ zps, int64_t params,
                                                             void* __restrict__ out, int64_t count, int64_t channels, int64_t inner) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < count; i += stride) {
        const int64_t c = params == 1 ? 0 : (inner == 1 ? i : i / inner) % channels;
        const float v = __fmul_rn(static_cast<float>(static_cast<int32_t>(x[i]) - zps[c]), scales[c]);
        if constexpr (OUT == FTH_B200_FP32) static_cast<float*>(out)[i] = v;
        else if constexpr (OUT == FTH_B200_FP16) static_cast<__half*>(out)[i] = __float2half_rn(v);
        else static_cast<uint16_t*>(out)[i] = EncodeBf16Dq(v);
    }
}

// QuantizeLinear with one (scale, zero point) passed by value: the fused prologue of the tensor-core linear.
template <int IN>
__global__ void __launch_bounds__(kThreads) QuantizeScalarKernel(const void* __restrict__ x, float scale, int32_t zp,
                                                                 int8_t* __restrict__ out, int64_t count) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < count; i += stride)
        out[i] = QuantizeValue(ReadAs<IN>(x, i, 1.0f), scale, zp);
}

__global__ void __launch_bounds__(kThreads) LookupKernel(const int8_t* __restrict__ x, int8_t* __restrict__ out,
                                                         int64_t count, const int8_t* __restrict__ lut) {
    __shared__ int8_t table[256];
    table[threadIdx.x] = lut[threadIdx.x];
    __syncthreads();
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t groups = count / 16;
    const bool aligned = (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(out) % 16 == 0);
    if (aligned) {
        for (int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; g < groups; g += stride) {
            uint4 v = LoadStream16(reinterpret_cast<const uint4*>(x) + g);
            uint8_t* b = reinterpret_cast<uint8_t*>(&v);
#pragma unroll
            for (int i = 0; i < 16; ++i) b[i] = static_cast<uint8_t>(table[static_cast<uint8_t>(b[i] + 128)]);
            reinterpret_cast<uint4*>(out)[g] = v;
        }
    }
    for (int64_t i = (aligned ? groups * 16 : 0) + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < count;
         i += stride) {
        out[i] = table[static_cast<uint8_t>(static_cast<uint8_t>(x[i]) + 128)];
    }
}

}  // namespace

int LaunchQuantizePerTensor(int x_dtype, const void* x, float scale, int32_t zp, int8_t* out, int64_t count, cudaStream_t stream) {
    const int grid = GridFor(count);
    switch (x_dtype) {
        case FTH_B200_FP32: QuantizeScalarKernel<FTH_B200_FP32><<<grid, kThreads, 0, stream>>>(x, scale, zp, out, count); break;
        case FTH_B200_BF16: QuantizeScalarKernel<FTH_B200_BF16><<<grid, kThreads, 0, stream>>>(x, scale, zp, out, count); break;
        case FTH_B200_FP16: QuantizeScalarKernel<FTH_B200_FP16><<<grid, kThreads, 0, stream>>>(x, scale, zp, out, count); break;
        default: return FTH_B200_ERR_UNSUPPORTED;
    }
    NoteLaunch("quantize_linear");
    return CheckLaunch();
}

}  // namespace fth

using namespace fth;

extern "C" int fth_b200_cast(int32_t in_dtype, const void* x, float in_scale, int32_t out_dtype, void* out,
                             float out_scale, int64_t count, fth_b200_stream_t stream_) {
    ClearStaleError();
    auto stream = static_cast<cudaStream_t>(stream_);
    if (x == nullptr || out == nullptr || count < 0) return FTH_B200_ERR_INVALID;
    const bool in_fp8 = in_dtype == FTH_B200_FP8E4M3 || in_dtype == FTH_B200_FP8E5M2;
    const bool out_fp8 = out_dtype == FTH_B200_FP8E4M3 || out_dtype == FTH_B200_FP8E5M2;
    // HasValidFp8Quantization (src/kernel/fp8_host.h:150-157): finite, positive per-tensor scale.
    if (in_fp8 && !(in_scale > 0.0f && in_scale < INFINITY)) return FTH_B200_ERR_INVALID;
    if (out_fp8 && !(out_scale > 0.0f && out_scale < INFINITY)) return FTH_B200_ERR_INVALID;
    if (count == 0) return FTH_B200_OK;
    switch (in_dtype) {
        case FTH_B200_FP32: return LaunchCastOut<FTH_B200_FP32>(out_dtype, x, out, count, in_scale, out_scale, stream);
        case FTH_B200_BF16: return LaunchCastOut<FTH_B200_BF16>(out_dtype, x, out, count, in_scale, out_scale, stream);
        case FTH_B200_FP16: return LaunchCastOut<FTH_B200_FP16>(out_dtype, x, out, count, in_scale, out_scale, stream);
        case FTH_B200_FP8E4M3: return LaunchCastOut<FTH_B200_FP8E4M3>(out_dtype, x, out, count, in_scale, out_scale, stream);
        case FTH_B200_FP8E5M2: return LaunchCastOut<FTH_B200_FP8E5M2>(out_dtype, x, out, count, in_scale, out_scale, stream);
        default: return FTH_B200_ERR_UNSUPPORTED;
    }
}

extern "C" int fth_b200_quantize_linear(int32_t x_dtype, const void* x, const float* scales, const int32_t* zps,
                                        int64_t params, int8_t* out, int64_t rows, int64_t channels,
                                        fth_b200_stream_t stream_) {
    return fth_b200_quantize_linear_axis(x_dtype, x, scales, zps, params, out, rows, channels, 1, stream_);
}

extern "C" int fth_b200_quantize_linear_axis(int32_t x_dtype, const void* x, const float* scales, const int32_t* zps,
                                             int64_t params, int8_t* out, int64_t outer, int64_t channels, int64_t inner,
                                             fth_b200_stream_t stream_) {
    ClearStaleError();
    auto stream = static_cast<cudaStream_t>(stream_);
    if (!x || !scales || !zps || !out || outer <= 0 || channels <= 0 || inner <= 0) return FTH_B200_ERR_INVALID;
    if (params != 1 && params != channels) return FTH_B200_ERR_INVALID;
    const int64_t count = outer * channels * inner;
    const int grid = GridFor(count / 4 + 1);
    switch (x_dtype) {
        case FTH_B200_FP32: QuantizeKernel<FTH_B200_FP32><<<grid, kThreads, 0, stream>>>(x, scales, zps, params, out, count, channels, inner); break;
        case FTH_B200_BF16: QuantizeKernel<FTH_B200_BF16><<<grid, kThreads, 0, stream>>>(x, scales, zps, params, out, count, channels, inner); break;
        case FTH_B200_FP16: QuantizeKernel<FTH_B200_FP16><<<grid, kThreads, 0, stream>>>(x, scales, zps, params, out, count, channels, inner); break;
        default: return FTH_B200_ERR_UNSUPPORTED;
    }
    NoteLaunch("quantize_linear");
    return CheckLaunch();
}

extern "C" int fth_b200_dequantize_linear(const int8_t* x, const float* scales, const int32_t* zps, int64_t params,
                                          void* out, int32_t to_dtype, int64_t rows, int64_t channels,
                                          fth_b200_stream_t stream_) {
    return fth_b200_dequantize_linear_axis(x, scales, zps, params, out, to_dtype, rows, channels, 1, stream_);
}

extern "C" int fth_b200_dequantize_linear_axis(const int8_t* x, const float* scales, const int32_t* zps, int64_t params,
                                               void* out, int32_t to_dtype, int64_t outer, int64_t channels, int64_t inner,
                                               fth_b200_stream_t stream_) {
    ClearStaleError();
    auto stream = static_cast<cudaStream_t>(stream_);
    if (!x || !scales || !zps || !out || outer <= 0 || channels <= 0 || inner <= 0) return FTH_B200_ERR_INVALID;
    if (params != 1 && params != channels) return FTH_B200_ERR_INVALID;
    const int64_t count = outer * channels * inner;
    const int grid = GridFor(count);
    switch (to_dtype) {
        case FTH_B200_FP32: DequantizeKernel<FTH_B200_FP32><<<grid, kThreads, 0, stream>>>(x, scales, zps, params, out, count, channels, inner); break;
        case FTH_B200_BF16: DequantizeKernel<FTH_B200_BF16><<<grid, kThreads, 0, stream>>>(x, scales, zps, params, out, count, channels, inner); break;
        case FTH_B200_FP16: DequantizeKernel<FTH_B200_FP16><<<grid, kThreads, 0, stream>>>(x, scales, zps, params, out, count, channels, inner); break;
        default: return FTH_B200_ERR_INVALID;  // the reference accepts FP32 / FP16 / BF16 only
    }
    NoteLaunch("dequantize_linear");
    return CheckLaunch();
}

extern "C" int fth_b200_int8_lookup(const int8_t* x, int8_t* out, int64_t count, const int8_t* device_lut256,
                                    fth_b200_stream_t stream_) {
    ClearStaleError();
    auto stream = static_cast<cudaStream_t>(stream_);
    if (!x || !out || !device_lut256 || count < 0) return FTH_B200_ERR_INVALID;
    if (count == 0) return FTH_B200_OK;
    LookupKernel<<<GridFor(count / 16 + 1), kThreads, 0, stream>>>(x, out, count, device_lut256);
    NoteLaunch("int8_lookup");
    return CheckLaunch();
}

// Host-side INT8 ReLU table: lut[q + 128] = QuantizeInt8Value(max(0, float(q - zp_in)·s_in), s_out, zp_out)
// (src/kernel/common/int8_standard.cc:114-128; QuantizeInt8Value: include/quant/quantization.h:94-99).
#include <cmath>
extern "C" int fth_b200_int8_relu_table(float in_scale, int32_t in_zp, float out_scale, int32_t out_zp, int8_t* lut) {
    if (!lut || !(in_scale > 0.0f) || !(out_scale > 0.0f) || !std::isfinite(in_scale) || !std::isfinite(out_scale) ||
        in_zp < -128 || in_zp > 127 || out_zp < -128 || out_zp > 127) return FTH_B200_ERR_INVALID;
    for (int q = -128; q <= 127; ++q) {
        const float real = static_cast<float>(q - in_zp) * in_scale;
        const float relu = real > 0.0f ? real : 0.0f;
        const double t = static_cast<double>(relu) / static_cast<double>(out_scale) + out_zp;
        const double r = std::round(t);
        lut[q + 128] = static_cast<int8_t>(std::fmax(-128.0, std::fmin(127.0, r)));
    }
    return FTH_B200_OK;
}
