// TEST INFRASTRUCTURE — not part of the shipped library.
//
// C-ABI shim over the UNMODIFIED reference ("Feather") CPU kernels.  It is
// compiled together with the reference's own sources (read where they lie in
// the reference checkout; nothing is copied) into oracle/_ref/libfeather_ref.so
// by oracle/Makefile.  Only tests, the smoke check and the CPU-baseline leg of
// the benchmark may load it.
//
// Every call builds feather::Tensor objects around the caller's buffers,
// obtains the reference kernel from feather::KernelDispatcher exactly as the
// reference's own unit tests do (test/common_int8_kernel_test.cc:65-122,
// test/fp8_test.cc:768-820) and runs Prepare()/compute().
//
// device: 0 = DeviceType::COMMON (canonical numerical oracle)
//         1 = DeviceType::X86    (timed CPU baseline)
// op:     0 = "FC", 1 = "MatMul", 2 = "Gemm"
// dtype:  values of feather::DataType (INT8 = 1, FP8E4M3 = 12, FP8E5M2 = 13 …)

#include <chrono>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "core/kernel.h"
#include "core/tensor.h"
#include "quant/quantization.h"
#include "src/operator/params.h"
#include "util/bf16.h"
#include "util/fp8.h"
#include "util/types.h"

using feather::DataType;
using feather::DeviceType;
using feather::KernelBase;
using feather::KernelDispatcher;
using feather::QuantizationGranularity;
using feather::QuantizationParams;
using feather::Tensor;

namespace {

DeviceType ToDevice(int device) { return device == 1 ? DeviceType::X86 : DeviceType::COMMON; }

const char* OpName(int op) {
    switch (op) {
        case 0: return "FC";
        case 1: return "MatMul";
        case 2: return "Gemm";
        default: return "";
    }
}

size_t ElementBytes(DataType dtype) {
    switch (dtype) {
        case DataType::FP32: case DataType::INT32: return 4;
        case DataType::FP16: case DataType::BF16: return 2;
        case DataType::INT64: return 8;
        default: return 1;
    }
}

// Tensor holding a private copy of `bytes` with the given dtype and dims.
std::shared_ptr<Tensor> MakeTensor(const void* bytes, DataType dtype, const std::vector<int64_t>& dims) {
    size_t count = 1;
    for (int64_t d : dims) count *= static_cast<size_t>(d);
    const size_t size = count * ElementBytes(dtype);
    auto tensor = std::make_shared<Tensor>(size);
    tensor->Resize(dims);
    void* dst = tensor->mutable_data(size);
    if (bytes != nullptr && size != 0) std::memcpy(dst, bytes, size);
    tensor->set_data_type(dtype);
    return tensor;
}

QuantizationParams PerTensor(float scale, int32_t zero_point) {
    QuantizationParams q;
    q.enabled = true;
    q.scale = scale;
    q.zero_point = zero_point;
    q.granularity = QuantizationGranularity::kPerTensor;
    return q;
}

QuantizationParams PerChannel(int64_t axis, const float* scales, const int32_t* zero_points, int64_t channels) {
    QuantizationParams q;
    q.enabled = true;
    q.granularity = QuantizationGranularity::kPerChannel;
    q.axis = axis;
    q.scales.assign(scales, scales + channels);
    if (zero_points != nullptr) q.zero_points.assign(zero_points, zero_points + channels);
    else q.zero_points.assign(static_cast<size_t>(channels), 0);
    q.scale = q.scales.front();
    q.zero_point = q.zero_points.front();
    return q;
}

struct Handle {
    std::unique_ptr<KernelBase> kernel;
    std::shared_ptr<void> param;
    std::shared_ptr<Tensor> out;
    size_t out_bytes{0};
};

template <typename Param>
Handle* Finish(std::unique_ptr<KernelBase> kernel, std::shared_ptr<Param> param, std::shared_ptr<Tensor> out,
               size_t out_bytes) {
    if (!kernel) return nullptr;
    kernel->SetParam(param.get());
    auto* handle = new Handle();
    handle->kernel = std::move(kernel);
    handle->param = std::move(param);
    handle->out = std::move(out);
    handle->out_bytes = out_bytes;
    return handle;
}

}  // namespace

extern "C" {

// ---- FP8 codec (include/util/fp8.h:81-204) -------------------------------------------------
uint8_t ref_fp8_encode(int dtype, float value) {
    return dtype == static_cast<int>(DataType::FP8E4M3) ? feather::FloatToFp8E4M3(value)
                                                        : feather::FloatToFp8E5M2(value);
}
float ref_fp8_decode(int dtype, uint8_t bits) {
    return dtype == static_cast<int>(DataType::FP8E4M3) ? feather::Fp8E4M3ToFloat(bits)
                                                        : feather::Fp8E5M2ToFloat(bits);
}
void ref_fp8_encode_array(int dtype, const float* values, uint8_t* out, int64_t count) {
    for (int64_t i = 0; i < count; ++i) out[i] = ref_fp8_encode(dtype, values[i]);
}
void ref_fp8_decode_array(int dtype, const uint8_t* bits, float* out, int64_t count) {
    for (int64_t i = 0; i < count; ++i) out[i] = ref_fp8_decode(dtype, bits[i]);
}
uint16_t ref_float_to_bf16(float value) { return feather::FloatToBFloat16(value); }

// ---- INT8 scalar math (include/quant/quantization.h:94-103) --------------------------------
int8_t ref_quantize_int8_value(float value, float scale, int32_t zero_point) {
    return feather::QuantizeInt8Value(value, scale, zero_point);
}

// ---- FP8 FC / MatMul / Gemm -----------------------------------------------------------------
// bias_mode: 0 none, 1 vector [N], 2 matrix [M,N]; bias is FP8 of the same dtype.
void* ref_fp8_linear_create(int device, int op, int dtype, const uint8_t* a, float a_scale, const uint8_t* w,
                            float w_scale, const uint8_t* bias, float bias_scale, int bias_mode, float out_scale,
                            int64_t m, int64_t k, int64_t n, int trans_b, float alpha, float beta,
                            int immutable_weight) {
    const DataType dt = static_cast<DataType>(dtype);
    auto ta = MakeTensor(a, dt, {m, k});
    ta->set_quantization({true, a_scale});
    auto tw = MakeTensor(w, dt, trans_b ? std::vector<int64_t>{n, k} : std::vector<int64_t>{k, n});
    tw->set_quantization({true, w_scale});
    tw->set_immutable(immutable_weight != 0);
    std::shared_ptr<Tensor> tb;
    if (bias_mode == 1) tb = MakeTensor(bias, dt, {n});
    if (bias_mode == 2) tb = MakeTensor(bias, dt, {m, n});
    if (tb) tb->set_quantization({true, bias_scale});
    auto out = MakeTensor(nullptr, dt, {m, n});
    out->set_quantization({true, out_scale});

    auto kernel = KernelDispatcher::instance().create(ToDevice(device), dt, OpName(op));
    if (op == 0) {
        auto p = std::make_shared<feather::operators::FcParam>();
        p->input = ta; p->w = tw; p->bias = tb; p->out = out;
        return Finish(std::move(kernel), p, out, static_cast<size_t>(m * n));
    }
    if (op == 1) {
        auto p = std::make_shared<feather::operators::MatMulParam>();
        p->a = ta; p->b = tw; p->out = out;
        return Finish(std::move(kernel), p, out, static_cast<size_t>(m * n));
    }
    auto p = std::make_shared<feather::operators::GemmParam>();
    p->a = ta; p->b = tw; p->bias = tb; p->out = out;
    p->alpha = alpha; p->beta = beta; p->trans_a = false; p->trans_b = trans_b != 0;
    return Finish(std::move(kernel), p, out, static_cast<size_t>(m * n));
}

// ---- INT8 FC / MatMul / Gemm ----------------------------------------------------------------
// Weight quantisation: w_channels == 0 → per-tensor (w_scales[0], w_zps[0]); else per-channel on the
// output-channel axis (FC/MatMul: 1; Gemm trans_b: 0).  bias: int32, bias_mode as above.
void* ref_int8_linear_create(int device, int op, const int8_t* a, float a_scale, int32_t a_zp, const int8_t* w,
                             const float* w_scales, const int32_t* w_zps, int64_t w_channels, const int32_t* bias,
                             int bias_mode, float out_scale, int32_t out_zp, int64_t m, int64_t k, int64_t n,
                             int trans_b, float alpha, float beta) {
    auto ta = MakeTensor(a, DataType::INT8, {m, k});
    ta->set_quantization(PerTensor(a_scale, a_zp));
    auto tw = MakeTensor(w, DataType::INT8, trans_b ? std::vector<int64_t>{n, k} : std::vector<int64_t>{k, n});
    if (w_channels == 0) tw->set_quantization(PerTensor(w_scales[0], w_zps ? w_zps[0] : 0));
    else tw->set_quantization(PerChannel(trans_b ? 0 : 1, w_scales, w_zps, w_channels));
    tw->set_immutable(true);
    std::shared_ptr<Tensor> tb;
    if (bias_mode == 1) tb = MakeTensor(bias, DataType::INT32, {n});
    if (bias_mode == 2) tb = MakeTensor(bias, DataType::INT32, {m, n});
    auto out = MakeTensor(nullptr, DataType::INT8, {m, n});
    out->set_quantization(PerTensor(out_scale, out_zp));

    auto kernel = KernelDispatcher::instance().create(ToDevice(device), DataType::INT8, OpName(op));
    if (op == 0) {
        auto p = std::make_shared<feather::operators::FcParam>();
        p->input = ta; p->w = tw; p->bias = tb; p->out = out;
        return Finish(std::move(kernel), p, out, static_cast<size_t>(m * n));
    }
    if (op == 1) {
        auto p = std::make_shared<feather::operators::MatMulParam>();
        p->a = ta; p->b = tw; p->out = out;
        return Finish(std::move(kernel), p, out, static_cast<size_t>(m * n));
    }
    auto p = std::make_shared<feather::operators::GemmParam>();
    p->a = ta; p->b = tw; p->bias = tb; p->out = out;
    p->alpha = alpha; p->beta = beta; p->trans_a = false; p->trans_b = trans_b != 0;
    return Finish(std::move(kernel), p, out, static_cast<size_t>(m * n));
}

// ---- INT8 Conv2D (NCHW, weight OIHW) --------------------------------------------------------
void* ref_int8_conv2d_create(int device, const int8_t* x, float x_scale, int32_t x_zp, const int8_t* w,
                             const float* w_scales, const int32_t* w_zps, int64_t w_channels, const int32_t* bias,
                             float out_scale, int32_t out_zp, int64_t batch, int64_t ic, int64_t ih, int64_t iw,
                             int64_t oc, int64_t kh, int64_t kw, int32_t stride_h, int32_t stride_w, int32_t pad_h,
                             int32_t pad_w, int32_t dilation_h, int32_t dilation_w, int32_t group) {
    auto tx = MakeTensor(x, DataType::INT8, {batch, ic, ih, iw});
    tx->set_quantization(PerTensor(x_scale, x_zp));
    auto tw = MakeTensor(w, DataType::INT8, {oc, ic / group, kh, kw});
    if (w_channels == 0) tw->set_quantization(PerTensor(w_scales[0], w_zps ? w_zps[0] : 0));
    else tw->set_quantization(PerChannel(0, w_scales, w_zps, w_channels));
    tw->set_immutable(true);
    std::shared_ptr<Tensor> tb;
    if (bias != nullptr) tb = MakeTensor(bias, DataType::INT32, {oc});
    const int64_t oh = (ih + 2 * pad_h - dilation_h * (kh - 1) - 1) / stride_h + 1;
    const int64_t ow = (iw + 2 * pad_w - dilation_w * (kw - 1) - 1) / stride_w + 1;
    auto out = MakeTensor(nullptr, DataType::INT8, {batch, oc, oh, ow});
    out->set_quantization(PerTensor(out_scale, out_zp));
    auto p = std::make_shared<feather::operators::Conv2dParam>();
    p->input = tx; p->w = tw; p->bias = tb; p->out = out;
    p->stride_h = stride_h; p->stride_w = stride_w; p->pad_h = pad_h; p->pad_w = pad_w;
    p->dilation_h = dilation_h; p->dilation_w = dilation_w; p->group = group;
    auto kernel = KernelDispatcher::instance().create(ToDevice(device), DataType::INT8, "Conv2D");
    return Finish(std::move(kernel), p, out, static_cast<size_t>(batch * oc * oh * ow));
}

// ---- INT8 ReLU node (src/kernel/common/int8_standard.cc:102-176) ------------------------------
void* ref_int8_relu_create(int device, const int8_t* x, float x_scale, int32_t x_zp, float out_scale,
                           int32_t out_zp, int64_t count) {
    auto tx = MakeTensor(x, DataType::INT8, {count});
    tx->set_quantization(PerTensor(x_scale, x_zp));
    auto out = MakeTensor(nullptr, DataType::INT8, {count});
    out->set_quantization(PerTensor(out_scale, out_zp));
    auto p = std::make_shared<feather::operators::UnaryParam>();
    p->input = tx; p->out = out;
    auto kernel = KernelDispatcher::instance().create(ToDevice(device), DataType::INT8, "ReLU");
    return Finish(std::move(kernel), p, out, static_cast<size_t>(count));
}

// ---- Cast (src/kernel/common/cast.cc:62-126) --------------------------------------------------
// FP8 tensors carry a per-tensor scale; others ignore it.
void* ref_cast_create(int device, int in_dtype, const void* x, float in_scale, int out_dtype, float out_scale,
                      int64_t count) {
    const DataType in_dt = static_cast<DataType>(in_dtype);
    const DataType out_dt = static_cast<DataType>(out_dtype);
    auto tx = MakeTensor(x, in_dt, {count});
    if (in_dt == DataType::FP8E4M3 || in_dt == DataType::FP8E5M2) tx->set_quantization({true, in_scale});
    auto out = MakeTensor(nullptr, out_dt, {count});
    if (out_dt == DataType::FP8E4M3 || out_dt == DataType::FP8E5M2) out->set_quantization({true, out_scale});
    auto p = std::make_shared<feather::operators::CastParam>();
    p->input = tx; p->out = out; p->to = out_dt;
    // The Cast operator requests the kernel by its *input* dtype (src/operator/cast_op.cc:85-100).
    auto kernel = KernelDispatcher::instance().create(ToDevice(device), in_dt, "Cast");
    return Finish(std::move(kernel), p, out, static_cast<size_t>(count) * ElementBytes(out_dt));
}

// ---- QuantizeLinear / DequantizeLinear (COMMON only in the reference) ---------------------------
// x: [rows, channels]; scales/zps: `params` entries (1 = per-tensor, channels = per-channel on axis 1).
void* ref_quantize_linear_create(int x_dtype, const void* x, const float* scales, const int32_t* zps,
                                 int64_t params, int64_t rows, int64_t channels) {
    const DataType x_dt = static_cast<DataType>(x_dtype);
    auto tx = MakeTensor(x, x_dt, {rows, channels});
    auto ts = MakeTensor(scales, DataType::FP32, {params});
    auto tz = MakeTensor(zps, DataType::INT32, {params});
    auto out = MakeTensor(nullptr, DataType::INT8, {rows, channels});
    auto p = std::make_shared<feather::operators::QuantizeLinearParam>();
    p->input = tx; p->scale = ts; p->zero_point = tz; p->out = out; p->axis = 1;
    auto kernel = KernelDispatcher::instance().create(DeviceType::COMMON, x_dt, "QuantizeLinear");
    return Finish(std::move(kernel), p, out, static_cast<size_t>(rows * channels));
}

void* ref_dequantize_linear_create(const int8_t* x, const float* scales, const int32_t* zps, int64_t params,
                                   int64_t rows, int64_t channels, int to_dtype) {
    const DataType to = static_cast<DataType>(to_dtype);
    auto tx = MakeTensor(x, DataType::INT8, {rows, channels});
    auto ts = MakeTensor(scales, DataType::FP32, {params});
    auto tz = MakeTensor(zps, DataType::INT32, {params});
    auto out = MakeTensor(nullptr, to, {rows, channels});
    auto p = std::make_shared<feather::operators::DequantizeLinearParam>();
    p->input = tx; p->scale = ts; p->zero_point = tz; p->out = out; p->to = to; p->axis = 1;
    auto kernel = KernelDispatcher::instance().create(DeviceType::COMMON, DataType::INT8, "DequantizeLinear");
    return Finish(std::move(kernel), p, out, static_cast<size_t>(rows * channels) * ElementBytes(to));
}

// ---- QwenRmsNorm, Add / Mul, SiLU: the operators between the projections of a decoder block --------------------
// (src/kernel/common/qwen_rms_norm.cc:71-95, add.cc:80-109, mul.cc, silu.cc:38-55; x86 versions on device 1)
void* ref_qwen_rms_norm_create(int device, int x_dtype, const void* x, int w_dtype, const void* weight, float weight_offset,
                               float epsilon, int out_dtype, int64_t rows, int64_t hidden) {
    const DataType x_dt = static_cast<DataType>(x_dtype), w_dt = static_cast<DataType>(w_dtype), o_dt = static_cast<DataType>(out_dtype);
    auto p = std::make_shared<feather::operators::QwenRmsNormParam>();
    p->input = MakeTensor(x, x_dt, {rows, hidden});
    p->weight = MakeTensor(weight, w_dt, {hidden});
    p->epsilon = MakeTensor(&epsilon, DataType::FP32, {1});
    auto out = MakeTensor(nullptr, o_dt, {rows, hidden});
    p->out = out;
    p->weight_offset = weight_offset;
    auto kernel = KernelDispatcher::instance().create(ToDevice(device), x_dt, "QwenRmsNorm");
    return Finish(std::move(kernel), p, out, static_cast<size_t>(rows * hidden) * ElementBytes(o_dt));
}

// op: 0 = "Add", 1 = "Mul".  rhs is [rows, cols] or, when rhs_rows == 1, one row [cols] broadcast over lhs.
void* ref_binary_create(int device, int op, int dtype, const void* lhs, const void* rhs, int64_t rows, int64_t cols, int64_t rhs_rows) {
    const DataType dt = static_cast<DataType>(dtype);
    auto p = std::make_shared<feather::operators::BinaryParam>();
    p->lhs = MakeTensor(lhs, dt, {rows, cols});
    p->rhs = rhs_rows == 1 ? MakeTensor(rhs, dt, {cols}) : MakeTensor(rhs, dt, {rows, cols});
    auto out = MakeTensor(nullptr, dt, {rows, cols});
    p->out = out;
    auto kernel = KernelDispatcher::instance().create(ToDevice(device), dt, op == 0 ? "Add" : "Mul");
    return Finish(std::move(kernel), p, out, static_cast<size_t>(rows * cols) * ElementBytes(dt));
}

void* ref_silu_create(int device, int dtype, const void* x, int64_t count) {
    const DataType dt = static_cast<DataType>(dtype);
    auto p = std::make_shared<feather::operators::UnaryParam>();
    p->input = MakeTensor(x, dt, {count});
    auto out = MakeTensor(nullptr, dt, {count});
    p->out = out;
    auto kernel = KernelDispatcher::instance().create(ToDevice(device), dt, "SiLU");
    return Finish(std::move(kernel), p, out, static_cast<size_t>(count) * ElementBytes(dt));
}

// ---- fused lm-head projection + greedy selection (FP8: src/kernel/x86/linear_fp8.cc:733-1004; there is no COMMON
// kernel for it).  a [1, K], b [N, K] (vocabulary rows), per-tensor scales; returns the kernel whose output is one int64.
void* ref_qwen_gemm_argmax_create(int device, int dtype, const uint8_t* a, float a_scale, const uint8_t* b, float b_scale,
                                  float output_scale, int64_t k, int64_t n) {
    const DataType dt = static_cast<DataType>(dtype);
    auto p = std::make_shared<feather::operators::QwenGemmArgmaxParam>();
    p->a = MakeTensor(a, dt, {1, k});
    p->a->set_quantization({true, a_scale});
    p->b = MakeTensor(b, dt, {n, k});
    p->b->set_quantization({true, b_scale});
    p->b->set_immutable(true);
    auto out = MakeTensor(nullptr, DataType::INT64, {1});
    p->out = out;
    p->output_scale = output_scale;
    auto kernel = KernelDispatcher::instance().create(ToDevice(device), dt, "QwenGemmArgmax");
    return Finish(std::move(kernel), p, out, sizeof(int64_t));
}

// ---- handle operations ---------------------------------------------------------------------
int ref_kernel_device(void* handle) {
    return handle ? static_cast<int>(static_cast<Handle*>(handle)->kernel->device()) : -1;
}
int ref_kernel_supports(void* handle) {
    return handle && static_cast<Handle*>(handle)->kernel->Supports().ok() ? 1 : 0;
}
int ref_kernel_prepare(void* handle) { return handle ? static_cast<Handle*>(handle)->kernel->Prepare() : -1; }
int ref_kernel_compute(void* handle) { return handle ? static_cast<Handle*>(handle)->kernel->compute() : -1; }
int64_t ref_kernel_output_bytes(void* handle) {
    return handle ? static_cast<int64_t>(static_cast<Handle*>(handle)->out_bytes) : -1;
}
int ref_kernel_read_output(void* handle, void* dst, int64_t bytes) {
    if (!handle) return -1;
    auto* h = static_cast<Handle*>(handle);
    if (bytes < 0 || static_cast<size_t>(bytes) > h->out_bytes) return -1;
    std::memcpy(dst, h->out->raw_data(), static_cast<size_t>(bytes));
    return 0;
}
// Best wall-clock seconds of `repeats` compute() calls (std::chrono::steady_clock).
double ref_kernel_time_compute(void* handle, int repeats, int* status) {
    if (!handle) { if (status) *status = -1; return 0.0; }
    auto* h = static_cast<Handle*>(handle);
    double best = 1e300;
    int rc = 0;
    for (int i = 0; i < repeats; ++i) {
        const auto t0 = std::chrono::steady_clock::now();
        rc |= h->kernel->compute();
        const auto t1 = std::chrono::steady_clock::now();
        const double s = std::chrono::duration<double>(t1 - t0).count();
        if (s < best) best = s;
    }
    if (status) *status = rc;
    return best;
}
void ref_kernel_destroy(void* handle) { delete static_cast<Handle*>(handle); }

}  // extern "C"
