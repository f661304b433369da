// The small operators that sit between the quantized projections of a decoder block on the same stream:
// QwenRmsNorm, element-wise Add / Mul, SiLU, and SiLU(gate) * up as one launch.
//
// At decode size (one to sixteen rows of 1024 .. 3584 elements) each of them moves a few kilobytes: what they cost
// is a launch and one round trip to memory, so every kernel reads with 16-byte loads, keeps a row in registers
// between the two passes of the normalisation, and marks itself as a programmatic dependent of the kernel in front
// (set-up overlaps that kernel's tail; nothing is read before it has completed).
//
// Numerical contracts (the reference's Common kernels):
//   QwenRmsNorm  src/kernel/common/qwen_rms_norm.cc:71-95   FP32 math throughout;
//                out = x * (1 / sqrt(sum(x^2) / hidden + eps)) * (weight + weight_offset), rounded after each
//                multiply; BF16 output rounds to nearest even and quiets NaNs (include/util/bf16.h:35-46).
//                The reference adds the squares one after another in FP32; here a row is summed by 128 threads and a
//                tree, so the sum (and with it every output of the row) differs by the rounding error of the sequential
//                sum, a few parts in 10^6 at 1024 terms: at most one BF16 code after rounding, up to a few tens of FP32
//                steps for FP32 output.  The reference's own x86 and CUDA kernels reduce in other orders too.
//   Add / Mul    src/kernel/common/add.cc:80-109, mul.cc: float(lhs) op float(rhs), one rounding to the output
//                type.  Bit-exact.  rhs may be one row that is broadcast over the rows of lhs.
//   SiLU         src/kernel/common/silu.cc:38-55: x / (1 + exp(-x)) in FP32 with the C library's expf.  Here
//                exp is evaluated in double and rounded to FP32 once, which gives the correctly rounded value the C
//                library returns in all but a vanishing fraction of cases; FP32 add and divide as in the reference.
#include <cmath>

#include "common.cuh"
#include "rowops.cuh"

namespace fth {
namespace {

using namespace rowops;

constexpr int kThreads = 128;

bool Aligned16Host(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// One block per row.  kRowGroups groups of eight elements per thread stay in registers between the two passes when the
// row fits (hidden <= 128 * 8 * kRowGroups); longer rows are read twice.
constexpr int kGroups = kRowGroups;
static_assert(kThreads == kRowThreads, "the row helpers assume 128 threads per row");

// Sum over the block; every thread receives the total.  Fixed order (lane tree, then the four warps in order), so the
// result does not depend on scheduling.
__device__ __forceinline__ float BlockSum(float v, float* shared) {
    v = WarpTreeSum(v);
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) shared[warp] = v;
    __syncthreads();
    float total = shared[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) total = __fadd_rn(total, shared[w]);
    return total;
}

template <int X, int W, int OUT>
__global__ void __launch_bounds__(kThreads) RmsNormKernel(const void* __restrict__ x, const void* __restrict__ weight,
                                                          void* __restrict__ out, int64_t hidden, float epsilon, float weight_offset) {
    __shared__ float partial[kThreads / 32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int64_t row = blockIdx.x;
    const int64_t base = row * hidden;
    const void* xr = x;
    const bool vec_x = Aligned16(x) && ((base * (X == FTH_B200_FP32 ? 4 : 2)) & 15) == 0 && hidden % 8 == 0;
    const bool vec_w = Aligned16(weight) && hidden % 8 == 0;
    const bool vec_o = Aligned16(out) && ((base * (OUT == FTH_B200_FP32 ? 4 : 2)) & 15) == 0 && hidden % 8 == 0;
    const int64_t groups = (hidden + 7) / 8;
    const bool resident = groups <= static_cast<int64_t>(kThreads) * kGroups;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // both vectors are requested before either is used, so their latencies overlap
    float wv[kGroups][8];
    if (resident) {
#pragma unroll
        for (int g = 0; g < kGroups; ++g) {
            const int64_t gi = threadIdx.x + static_cast<int64_t>(g) * kThreads;
            if (gi < groups && gi * 8 + 8 <= hidden) ReadEight<W>(weight, gi * 8, vec_w, wv[g]);
        }
    }
    float xv[kGroups][8];
    float sum = 0.0f;
    if (resident) {
        sum = ThreadSumSquares<X>(xr, base, hidden, vec_x, threadIdx.x, xv);
    } else {
        for (int64_t c = threadIdx.x; c < hidden; c += kThreads) {
            const float v = ReadFloat<X>(xr, base + c);
            sum = __fadd_rn(sum, __fmul_rn(v, v));
        }
    }
    const float total = BlockSum(sum, partial);
    const float inverse_rms = InverseRms(total, hidden, epsilon);
    if (resident) {
#pragma unroll
        for (int g = 0; g < kGroups; ++g) {
            const int64_t gi = threadIdx.x + static_cast<int64_t>(g) * kThreads;
            if (gi >= groups) continue;
            if (gi * 8 + 8 <= hidden) {
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = __fmul_rn(__fmul_rn(xv[g][j], inverse_rms), __fadd_rn(wv[g][j], weight_offset));
                WriteEight<OUT>(out, base + gi * 8, vec_o, o);
            } else {
                for (int64_t c = gi * 8; c < hidden; ++c) {
                    const float v = ReadFloat<X>(xr, base + c);
                    WriteFloat<OUT>(out, base + c, __fmul_rn(__fmul_rn(v, inverse_rms), __fadd_rn(ReadFloat<W>(weight, c), weight_offset)));
                }
            }
        }
    } else {
        for (int64_t c = threadIdx.x; c < hidden; c += kThreads) {
            const float v = ReadFloat<X>(xr, base + c);
            WriteFloat<OUT>(out, base + c, __fmul_rn(__fmul_rn(v, inverse_rms), __fadd_rn(ReadFloat<W>(weight, c), weight_offset)));
        }
    }
}


enum { kOpAdd = 0, kOpMul = 1, kOpSilu = 2, kOpSiluMul = 3 };

// SiLU of one element, as the FP32 value the node's output rounding starts from.  A BF16 node takes the short path of
// rowops::SiluToBf16 (its result is the rounded output already; rounding it again changes nothing).
template <int DTYPE>
__device__ __forceinline__ float SiluOf(float x) {
    if constexpr (DTYPE == FTH_B200_BF16) return DecodeBf16(SiluToBf16(x));
    else return SiluValue(x);
}

// out[i] = lhs[i] op rhs[i % rhs_count]   (Add, Mul; rhs_count is the total count or one row)
// out[i] = silu(lhs[i])                    (SiLU)
// out[i] = round(silu(lhs[i])) * rhs[i]    (SiLU node followed by Mul node: both rounding points kept)
template <int DTYPE, int OP>
__global__ void __launch_bounds__(256) PointwiseKernel(const void* __restrict__ lhs, const void* __restrict__ rhs, void* __restrict__ out,
                                                       int64_t count, int64_t rhs_count, int vec) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t groups = vec ? count / 8 : 0;
    for (int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; g < groups; g += stride) {
        float a[8], b[8], o[8];
        ReadEight<DTYPE>(lhs, g * 8, true, a);
        if constexpr (OP != kOpSilu) ReadEight<DTYPE>(rhs, (g * 8) % rhs_count, true, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if constexpr (OP == kOpAdd) o[j] = __fadd_rn(a[j], b[j]);
            else if constexpr (OP == kOpMul) o[j] = __fmul_rn(a[j], b[j]);
            else if constexpr (OP == kOpSilu) o[j] = SiluOf<DTYPE>(a[j]);
            else {
                float s = SiluOf<DTYPE>(a[j]);
                if constexpr (DTYPE == FTH_B200_BF16) s = DecodeBf16(EncodeBf16Cast(s));
                else if constexpr (DTYPE == FTH_B200_FP16) s = __half2float(__float2half_rn(s));
                o[j] = __fmul_rn(s, b[j]);
            }
        }
        WriteEight<DTYPE>(out, g * 8, true, o);
    }
    for (int64_t i = groups * 8 + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < count; i += stride) {
        const float a = ReadFloat<DTYPE>(lhs, i);
        float o;
        if constexpr (OP == kOpSilu) {
            o = SiluOf<DTYPE>(a);
        } else {
            const float b = ReadFloat<DTYPE>(rhs, i % rhs_count);
            if constexpr (OP == kOpAdd) o = __fadd_rn(a, b);
            else if constexpr (OP == kOpMul) o = __fmul_rn(a, b);
            else {
                float s = SiluOf<DTYPE>(a);
                if constexpr (DTYPE == FTH_B200_BF16) s = DecodeBf16(EncodeBf16Cast(s));
                else if constexpr (DTYPE == FTH_B200_FP16) s = __half2float(__float2half_rn(s));
                o = __fmul_rn(s, b);
            }
        }
        WriteFloat<DTYPE>(out, i, o);
    }
}

template <typename Kernel, typename... Args>
int LaunchDependent(Kernel kernel, unsigned grid, unsigned block, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, args...) != cudaSuccess) return FTH_B200_ERR_CUDA;
    return CheckLaunch();
}

template <int X, int W>
int LaunchRmsNormOut(int out_dtype, const void* x, const void* w, void* out, int64_t rows, int64_t hidden, float eps, float offset, cudaStream_t s) {
    if (out_dtype == FTH_B200_FP32) return LaunchDependent(RmsNormKernel<X, W, FTH_B200_FP32>, static_cast<unsigned>(rows), kThreads, s, x, w, out, hidden, eps, offset);
    return LaunchDependent(RmsNormKernel<X, W, FTH_B200_BF16>, static_cast<unsigned>(rows), kThreads, s, x, w, out, hidden, eps, offset);
}

bool FloatType(int dtype) { return dtype == FTH_B200_FP32 || dtype == FTH_B200_BF16; }

template <int OP>
int LaunchPointwise(int dtype, const void* lhs, const void* rhs, void* out, int64_t count, int64_t rhs_count, cudaStream_t s) {
    const bool vec = Aligned16Host(lhs) && Aligned16Host(out) && (rhs == nullptr || Aligned16Host(rhs)) && rhs_count % 8 == 0;
    const int64_t items = (count + 7) / 8;
    int64_t blocks = (items + 255) / 256;
    const int64_t cap = static_cast<int64_t>(SmCount()) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    const unsigned grid = static_cast<unsigned>(blocks);
    const int v = vec ? 1 : 0;
    switch (dtype) {
        case FTH_B200_FP32: return LaunchDependent(PointwiseKernel<FTH_B200_FP32, OP>, grid, 256u, s, lhs, rhs, out, count, rhs_count, v);
        case FTH_B200_BF16: return LaunchDependent(PointwiseKernel<FTH_B200_BF16, OP>, grid, 256u, s, lhs, rhs, out, count, rhs_count, v);
        case FTH_B200_FP16: return LaunchDependent(PointwiseKernel<FTH_B200_FP16, OP>, grid, 256u, s, lhs, rhs, out, count, rhs_count, v);
        default: return FTH_B200_ERR_UNSUPPORTED;
    }
}

}  // namespace
}  // namespace fth

using namespace fth;

extern "C" int fth_b200_qwen_rms_norm(int32_t x_dtype, const void* x, int32_t weight_dtype, const void* weight, float weight_offset,
                                      float epsilon, int32_t out_dtype, void* out, int64_t rows, int64_t hidden, fth_b200_stream_t stream_) {
    ClearStaleError();
    if (x == nullptr || weight == nullptr || out == nullptr || rows <= 0 || hidden <= 0) return FTH_B200_ERR_INVALID;
    if (!(epsilon >= 0.0f) || !(epsilon < INFINITY)) return FTH_B200_ERR_INVALID;  // qwen_rms_norm.cc:51-53
    if (!FloatType(x_dtype) || !FloatType(weight_dtype) || !FloatType(out_dtype)) return FTH_B200_ERR_UNSUPPORTED;
    if (rows > 0x7fffffff) return FTH_B200_ERR_UNSUPPORTED;
    auto s = static_cast<cudaStream_t>(stream_);
    int rc;
    if (x_dtype == FTH_B200_FP32) {
        rc = weight_dtype == FTH_B200_FP32 ? LaunchRmsNormOut<FTH_B200_FP32, FTH_B200_FP32>(out_dtype, x, weight, out, rows, hidden, epsilon, weight_offset, s)
                                           : LaunchRmsNormOut<FTH_B200_FP32, FTH_B200_BF16>(out_dtype, x, weight, out, rows, hidden, epsilon, weight_offset, s);
    } else {
        rc = weight_dtype == FTH_B200_FP32 ? LaunchRmsNormOut<FTH_B200_BF16, FTH_B200_FP32>(out_dtype, x, weight, out, rows, hidden, epsilon, weight_offset, s)
                                           : LaunchRmsNormOut<FTH_B200_BF16, FTH_B200_BF16>(out_dtype, x, weight, out, rows, hidden, epsilon, weight_offset, s);
    }
    if (rc == FTH_B200_OK) NoteLaunch("rms_norm");
    return rc;
}

extern "C" int fth_b200_binary(int32_t op, int32_t dtype, const void* lhs, const void* rhs, void* out, int64_t count, int64_t rhs_count,
                               fth_b200_stream_t stream_) {
    ClearStaleError();
    if (lhs == nullptr || rhs == nullptr || out == nullptr || count <= 0) return FTH_B200_ERR_INVALID;
    if (rhs_count == 0) rhs_count = count;
    if (rhs_count < 0 || rhs_count > count || count % rhs_count != 0) return FTH_B200_ERR_INVALID;
    auto s = static_cast<cudaStream_t>(stream_);
    int rc;
    if (op == FTH_B200_BINARY_ADD) rc = LaunchPointwise<kOpAdd>(dtype, lhs, rhs, out, count, rhs_count, s);
    else if (op == FTH_B200_BINARY_MUL) rc = LaunchPointwise<kOpMul>(dtype, lhs, rhs, out, count, rhs_count, s);
    else return FTH_B200_ERR_INVALID;
    if (rc == FTH_B200_OK) NoteLaunch(op == FTH_B200_BINARY_ADD ? "add" : "mul");
    return rc;
}

extern "C" int fth_b200_silu(int32_t dtype, const void* x, void* out, int64_t count, fth_b200_stream_t stream_) {
    ClearStaleError();
    if (x == nullptr || out == nullptr || count <= 0) return FTH_B200_ERR_INVALID;
    const int rc = LaunchPointwise<kOpSilu>(dtype, x, nullptr, out, count, count, static_cast<cudaStream_t>(stream_));
    if (rc == FTH_B200_OK) NoteLaunch("silu");
    return rc;
}

extern "C" int fth_b200_silu_mul(int32_t dtype, const void* gate, const void* up, void* out, int64_t count, fth_b200_stream_t stream_) {
    ClearStaleError();
    if (gate == nullptr || up == nullptr || out == nullptr || count <= 0) return FTH_B200_ERR_INVALID;
    const int rc = LaunchPointwise<kOpSiluMul>(dtype, gate, up, out, count, count, static_cast<cudaStream_t>(stream_));
    if (rc == FTH_B200_OK) NoteLaunch("silu_mul");
    return rc;
}
