// Fused operator types of the B200 backend and the graph pass that introduces them.
//
// A `.fth` plan wraps every quantized projection in nodes of its own:
//   Cast(BF16 -> FP8) -> MatMul / Gemm(FP8) -> Cast(FP8 -> BF16)                 (tools/export_qwen35_model.py:883-900)
//   QuantizeLinear -> FC / MatMul / Gemm (INT8) -> DequantizeLinear               (src/quant/static_quantizer.cc:779-797)
//   Conv2D(INT8) -> ReLU(INT8)                                                    (static_quantizer.cc:312-328)
// On the GPU the wrappers cost a launch and a round trip through memory each — at decode size more than the product
// itself.  libfth_b200.so runs each chain as one launch that keeps every rounding point of the chain (the activation
// is quantised exactly as the Cast / QuantizeLinear node would, the product is quantised to the 8-bit intermediate
// with the intermediate value's own scale, and only then decoded), so the fused node returns the bytes of the chain.
//
// Everything goes through the reference's public extension points: three operator types with builders
// (OperatorRegistry::Register, include/core/operator_registry.h:46-50), kernel candidates for them
// (KernelDispatcher::RegisterCandidate, include/core/kernel.h:228-237) and a GraphPass
// (include/pass/graph_pass.h:29-36) that matches the chains and rewrites them with StaticGraph::ReplaceNodeDesc /
// RemoveNode (include/core/static_graph.h:72-87), the way src/pass/qwen_gemm_argmax_fusion_pass.cc:89-180 rewrites
// the FP8 lm-head.  A chain is rewritten only when the C ABI says it will run the fused descriptor; anything else is
// left as it was.
#include <cstring>
#include <unordered_map>

#include "b200_common.cuh"
#include "core/operator.h"
#include "core/operator_registry.h"
#include "core/static_graph.h"
#include "pass/graph_pass.h"
#include "src/operator/params.h"
#include "src/operator/tensor_op_utils.h"
#include "util/timer.h"

namespace feather {
namespace kernel {
namespace b200 {

const char* const kFusedCastMatMulCast = "FusedCastMatMulCast";
const char* const kFusedQLinearDQ = "FusedQLinearDQ";
const char* const kConv2DRelu = "Conv2DRelu";

// ---------------------------------------------------------------------------------------------------------
// Parameter structs (shared Tensor handles + scalars, with a tensor visitor so that sessions can rebind them)
// ---------------------------------------------------------------------------------------------------------
struct FusedCastMatMulCastParam : operators::ParamBase {
    std::shared_ptr<Tensor> x;    // BF16 / FP32 activation
    std::shared_ptr<Tensor> w;    // FP8 weight with its per-tensor scale; [K,N], or [N,K] when trans_b
    std::shared_ptr<Tensor> out;  // BF16 / FP32
    float a_scale{1.0f};          // scale of the FP8 activation the first Cast produced
    float proj_scale{1.0f};       // scale of the FP8 product the second Cast consumed
    bool trans_b{false};
    // Decoder-block neighbours absorbed by the pass (fth_b200_fp8_linear_fused; BF16 in and out, decode-sized M):
    std::shared_ptr<Tensor> norm_weight;  // a QwenRmsNorm node in front of the first Cast: its weight; null: none
    float norm_offset{0.0f}, norm_epsilon{0.0f};
    std::shared_ptr<Tensor> residual;     // an Add node behind the last Cast: its other addend; null: none
    std::shared_ptr<Tensor> w2;           // a second projection of the same activation, with Mul(SiLU(first), second) behind both
    bool fused() const { return norm_weight != nullptr || residual != nullptr || w2 != nullptr; }
    template <typename Visitor> void VisitTensors(Visitor&& visit) {
        visit(x); visit(w); visit(out);
        if (norm_weight) visit(norm_weight);
        if (residual) visit(residual);
        if (w2) visit(w2);
    }
};

struct FusedQLinearDQParam : operators::ParamBase {
    std::shared_ptr<Tensor> x;     // FP32 activation
    std::shared_ptr<Tensor> w;     // INT8 weight with per-tensor / per-output-channel parameters
    std::shared_ptr<Tensor> bias;  // INT32 or null
    std::shared_ptr<Tensor> out;   // FP32
    float in_scale{1.0f}, out_scale{1.0f};
    int32_t in_zp{0}, out_zp{0};
    int32_t op{FTH_B200_OP_MATMUL};
    bool trans_b{false};
    float alpha{1.0f}, beta{1.0f};
    template <typename Visitor> void VisitTensors(Visitor&& visit) { visit(x); visit(w); visit(bias); visit(out); }
};

struct Conv2DReluParam : operators::ParamBase {
    operators::Conv2dParam conv;  // conv.out is the ReLU node's output tensor (its quantisation = the ReLU output's)
    float conv_scale{1.0f};       // quantisation of the value between the two nodes
    int32_t conv_zp{0};
    template <typename Visitor> void VisitTensors(Visitor&& visit) { conv.VisitTensors(visit); }
};

namespace {

void* const kProbe = ProbePointer();

// One operator class for the three types: it owns the parameter struct and forwards to its kernel.
template <typename Param>
class FusedOp final : public OpBase {
   public:
    FusedOp(std::string name, const char* type, Param param, std::vector<std::shared_ptr<Tensor>> inputs, std::shared_ptr<Tensor> out)
        : OpBase(std::move(name), type), param_(std::move(param)) {
        SetInputs(std::move(inputs));
        SetOutputs({std::move(out)});
    }
    void AttachKernel(std::unique_ptr<KernelBase> kernel) override {
        kernel_ = std::move(kernel);
        if (kernel_ != nullptr) kernel_->SetParamOwner(std::make_shared<Param>(param_));
    }
    std::unique_ptr<KernelBase> DetachKernel() override { return std::move(kernel_); }
    bool HasKernel() const override { return kernel_ != nullptr; }
    const KernelBase* kernel() const override { return kernel_.get(); }
    int32_t Run() override { return kernel_ != nullptr ? kernel_->compute() : -1; }

   private:
    Param param_;
    std::unique_ptr<KernelBase> kernel_;
};

using Attributes = std::unordered_map<std::string, model::AttributeValue>;
float FloatAttr(const Attributes& a, const char* key, float fallback) {
    const auto it = a.find(key);
    if (it == a.end()) return fallback;
    if (const auto* v = std::get_if<float>(&it->second)) return *v;
    return fallback;
}
int64_t IntAttr(const Attributes& a, const char* key, int64_t fallback) {
    const auto it = a.find(key);
    if (it == a.end()) return fallback;
    if (const auto* v = std::get_if<int64_t>(&it->second)) return *v;
    return fallback;
}

bool IsFp8(DataType t) { return t == DataType::FP8E4M3 || t == DataType::FP8E5M2; }
bool IsWide(DataType t) { return t == DataType::BF16 || t == DataType::FP32; }

// M, K, N of x [.., K] times a 2-D weight.
bool LinearDims(const Tensor* x, const Tensor* w, bool trans_b, int64_t* m, int64_t* k, int64_t* n) {
    if (!x || !w || x->dims().size() < 2 || w->dims().size() != 2) return false;
    const auto& xd = x->dims().data();
    const auto& wd = w->dims().data();
    *k = xd.back();
    if (*k <= 0 || x->numel() <= 0) return false;
    *m = x->numel() / *k;
    *n = trans_b ? wd[0] : wd[1];
    return (trans_b ? wd[1] : wd[0]) == *k && *n > 0;
}

// The output tensor of a rewritten node already exists (it was the last node's output); a fresh node gets one.
std::shared_ptr<Tensor> OutputFor(const std::shared_ptr<Tensor>& declared, const Tensor* x, int64_t n, DataType dtype) {
    std::vector<int64_t> shape = x->dims().data();
    shape.back() = n;
    auto out = operators::tensor_op_detail::AllocateOutput(declared, shape, dtype);
    if (out) out->set_data_type(dtype);
    return out;
}

// ---------------------------------------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------------------------------------
bool Describe(const FusedCastMatMulCastParam* p, fth_b200_fp8_linear_desc* d) {
    int64_t m = 0, k = 0, n = 0;
    if (!p || !p->x || !p->w || !p->out || !IsWide(p->x->data_type()) || !IsFp8(p->w->data_type()) || !IsWide(p->out->data_type())) return false;
    if (!LinearDims(p->x.get(), p->w.get(), p->trans_b, &m, &k, &n) || p->out->numel() != m * n) return false;
    if (!HasCompatiblePerTensorQuantization(p->w->quantization())) return false;
    *d = fth_b200_fp8_linear_desc{};
    d->dtype = static_cast<int32_t>(p->w->data_type());
    d->op = p->trans_b ? FTH_B200_OP_GEMM : FTH_B200_OP_MATMUL;
    d->m = m; d->k = k; d->n = n; d->trans_b = p->trans_b ? 1 : 0;
    d->a_dtype = static_cast<int32_t>(p->x->data_type());
    d->out_dtype = static_cast<int32_t>(p->out->data_type());
    d->a_scale = p->a_scale; d->w_scale = p->w->quantization_scale(); d->bias_scale = 1.0f; d->out_scale = p->proj_scale;
    d->alpha = 1.0f; d->beta = 1.0f;
    return true;
}

// What the node carries around the projection, as the C ABI names it (pointers left null: the caller fills them in).
bool DescribeFusion(const FusedCastMatMulCastParam* p, const fth_b200_fp8_linear_desc& d, fth_b200_fp8_linear_fusion* f) {
    *f = fth_b200_fp8_linear_fusion{};
    if (p->norm_weight) {
        if (p->norm_weight->numel() != d.k || (p->norm_weight->data_type() != DataType::BF16 && p->norm_weight->data_type() != DataType::FP32)) return false;
        f->prologue = FTH_B200_FUSE_RMS_NORM;
        f->norm_weight_dtype = static_cast<int32_t>(p->norm_weight->data_type());
        f->norm_weight_offset = p->norm_offset;
        f->norm_epsilon = p->norm_epsilon;
    }
    if (p->residual && (p->residual->numel() != d.m * d.n || p->residual->data_type() != DataType::BF16)) return false;
    if (p->w2) {
        if (p->w2->data_type() != p->w->data_type() || p->w2->numel() != p->w->numel() || !HasCompatiblePerTensorQuantization(p->w2->quantization())) return false;
        f->w2_scale = p->w2->quantization_scale();
        f->n2 = d.n;
        f->epilogue = FTH_B200_FUSE_OUT_SILU_MUL;
    }
    return true;
}

bool Describe(const FusedQLinearDQParam* p, fth_b200_int8_linear_desc* d, Int8WeightParams* wq) {
    int64_t m = 0, k = 0, n = 0;
    if (!p || !p->x || !p->w || !p->out || p->x->data_type() != DataType::FP32 || p->out->data_type() != DataType::FP32) return false;
    if (!LinearDims(p->x.get(), p->w.get(), p->trans_b, &m, &k, &n) || p->out->numel() != m * n) return false;
    if (!ReadInt8Quantization(p->w.get(), true, p->trans_b ? 0 : 1, n, wq)) return false;
    int bias_mode = FTH_B200_BIAS_NONE;
    if (p->bias) {
        if (p->bias->data_type() != DataType::INT32) return false;
        if (p->bias->numel() == n) bias_mode = FTH_B200_BIAS_VECTOR;
        else if (p->bias->numel() == m * n) bias_mode = FTH_B200_BIAS_MATRIX;
        else return false;
    }
    *d = fth_b200_int8_linear_desc{};
    d->op = p->op; d->m = m; d->k = k; d->n = n; d->trans_b = p->trans_b ? 1 : 0;
    d->a_dtype = FTH_B200_FP32; d->out_dtype = FTH_B200_FP32;
    d->bias_mode = bias_mode;
    d->a_scale = p->in_scale; d->a_zp = p->in_zp;
    d->w_params = static_cast<int64_t>(wq->scales.size());
    d->w_zp_max_abs = wq->zp_max_abs;
    d->out_scale = p->out_scale; d->out_zp = p->out_zp;
    d->alpha = p->alpha; d->beta = p->beta;
    d->bias_max_abs = BiasMaxAbs(p->bias.get());
    return true;
}

bool Describe(const Conv2DReluParam* p, fth_b200_int8_conv2d_desc* d, Int8WeightParams* wq, Int8WeightParams* relu_q) {
    if (!p || !p->conv.input || !p->conv.w || !p->conv.out) return false;
    const operators::Conv2dParam& c = p->conv;
    if (c.input->layout() == DataLayout::NHWC || c.out->layout() == DataLayout::NHWC) return false;
    const auto& xd = c.input->dims().data();
    const auto& wd = c.w->dims().data();
    if (xd.size() != 4 || wd.size() != 4 || c.out->dims().size() != 4) return false;
    Int8WeightParams xq;
    if (!ReadInt8Quantization(c.input.get(), false, -1, 1, &xq) || !ReadInt8Quantization(c.w.get(), true, 0, wd[0], wq) ||
        !ReadInt8Quantization(c.out.get(), false, -1, 1, relu_q)) return false;
    if (c.bias && (c.bias->data_type() != DataType::INT32 || c.bias->numel() != wd[0])) return false;
    *d = fth_b200_int8_conv2d_desc{};
    d->batch = xd[0]; d->ic = xd[1]; d->ih = xd[2]; d->iw = xd[3]; d->oc = wd[0]; d->kh = wd[2]; d->kw = wd[3];
    d->stride_h = c.stride_h; d->stride_w = c.stride_w; d->pad_h = c.pad_h; d->pad_w = c.pad_w;
    d->dilation_h = c.dilation_h; d->dilation_w = c.dilation_w; d->group = c.group;
    d->x_scale = xq.scales[0]; d->x_zp = xq.zero_points[0];
    d->w_params = static_cast<int64_t>(wq->scales.size()); d->w_zp_max_abs = wq->zp_max_abs;
    d->out_scale = p->conv_scale; d->out_zp = p->conv_zp;  // the conv's own rounding point; the table maps it to the ReLU output
    d->bias_max_abs = BiasMaxAbs(c.bias.get());
    return true;
}

// ---------------------------------------------------------------------------------------------------------
// kernels
// ---------------------------------------------------------------------------------------------------------
class FusedCastMatMulCastKernel final : public B200Kernel {
   public:
    Status Supports() const override {
        fth_b200_fp8_linear_desc d;
        if (!Describe(ParamAs<FusedCastMatMulCastParam>(), &d)) return Status::Error(StatusCode::kUnsupported, "b200: not a fused Cast -> MatMul -> Cast");
        d.a = d.w = d.out = kProbe;
        d.workspace = kProbe; d.workspace_bytes = static_cast<size_t>(-1);
        auto* p = ParamAs<FusedCastMatMulCastParam>();
        if (p->fused()) {
            fth_b200_fp8_linear_fusion f;
            if (!DescribeFusion(p, d, &f)) return Status::Error(StatusCode::kUnsupported, "b200: decoder-block operands do not fit the projection");
            if (p->norm_weight) f.norm_weight = kProbe;
            if (p->residual) f.residual = kProbe;
            if (p->w2) f.w2 = kProbe;
            return FromAbi(fth_b200_fp8_linear_fused_supported(&d, &f), kFusedCastMatMulCast);
        }
        return FromAbi(fth_b200_fp8_linear_supported(&d), kFusedCastMatMulCast);
    }
    int32_t Prepare() override {
        fth_b200_fp8_linear_desc d;
        if (!Describe(ParamAs<FusedCastMatMulCastParam>(), &d)) return -1;
        d.a = d.w = d.out = kProbe;
        weights_resident_ = false;
        if (ParamAs<FusedCastMatMulCastParam>()->fused()) return 0;  // the single-launch kernel needs no scratch
        return workspace_.Reserve(fth_b200_fp8_linear_workspace_bytes(&d), true);
    }
    int32_t compute() override {
        AutoTimer timer("B200::FusedCastMatMulCast");
        auto* p = ParamAs<FusedCastMatMulCastParam>();
        fth_b200_fp8_linear_desc d;
        if (!Describe(p, &d)) return -1;
        void* x = nullptr; void* w = nullptr; void* out = nullptr;
        const size_t out_bytes = static_cast<size_t>(p->out->numel()) * DataTypeBytes(p->out->data_type());
        if (AcquireIn(p->x.get(), &x) != 0 || AcquireIn(p->w.get(), &w) != 0 ||
            cuda_detail::AcquireOutputTensorDevice(p->out.get(), out_bytes, &out) != 0) return -1;
        d.a = x; d.w = w; d.out = out;
        d.workspace = workspace_.get(); d.workspace_bytes = workspace_.bytes();
        d.weights_static = weights_resident_ ? 1 : 0;
        if (p->fused()) {
            fth_b200_fp8_linear_fusion f;
            void* norm_weight = nullptr; void* residual = nullptr; void* w2 = nullptr;
            if (!DescribeFusion(p, d, &f) || (p->norm_weight && AcquireIn(p->norm_weight.get(), &norm_weight) != 0) ||
                (p->residual && AcquireIn(p->residual.get(), &residual) != 0) || (p->w2 && AcquireIn(p->w2.get(), &w2) != 0)) return -1;
            f.norm_weight = norm_weight; f.residual = residual; f.w2 = w2;
            if (fth_b200_fp8_linear_fused(&d, &f, cuda_detail::InferenceStream()) != FTH_B200_OK) return -1;
            weights_resident_ = p->w->is_immutable() && (!p->w2 || p->w2->is_immutable()) && (!p->norm_weight || p->norm_weight->is_immutable());
            return FinishOut(p->out.get(), out_bytes);
        }
        if (fth_b200_fp8_linear(&d, cuda_detail::InferenceStream()) != FTH_B200_OK) return -1;
        weights_resident_ = p->w->is_immutable();
        return FinishOut(p->out.get(), out_bytes);
    }

   private:
    DeviceScratch workspace_;
    bool weights_resident_{false};
};

class FusedQLinearDQKernel final : public B200Kernel {
   public:
    Status Supports() const override {
        fth_b200_int8_linear_desc d;
        Int8WeightParams wq;
        if (!Describe(ParamAs<FusedQLinearDQParam>(), &d, &wq)) return Status::Error(StatusCode::kUnsupported, "b200: not a fused Q -> linear -> DQ");
        Probe(&d, wq);
        return FromAbi(fth_b200_int8_linear_supported(&d), kFusedQLinearDQ);
    }
    int32_t Prepare() override {
        fth_b200_int8_linear_desc d;
        Int8WeightParams wq;
        if (!Describe(ParamAs<FusedQLinearDQParam>(), &d, &wq)) return -1;
        if (scales_.Upload(wq.scales.data(), wq.scales.size() * sizeof(float)) != 0) return -1;
        has_zps_ = wq.zp_max_abs != 0;
        if (has_zps_ && zps_.Upload(wq.zero_points.data(), wq.zero_points.size() * sizeof(int32_t)) != 0) return -1;
        Probe(&d, wq);
        d.workspace = nullptr; d.workspace_bytes = 0;
        weights_resident_ = false;
        return workspace_.Reserve(fth_b200_int8_linear_workspace_bytes(&d), true);
    }
    int32_t compute() override {
        AutoTimer timer("B200::FusedQLinearDQ");
        auto* p = ParamAs<FusedQLinearDQParam>();
        fth_b200_int8_linear_desc d;
        Int8WeightParams wq;
        if (!Describe(p, &d, &wq) || scales_.get() == nullptr) return -1;
        void* x = nullptr; void* w = nullptr; void* bias = nullptr; void* out = nullptr;
        const size_t out_bytes = static_cast<size_t>(p->out->numel()) * sizeof(float);
        if (AcquireIn(p->x.get(), &x) != 0 || AcquireIn(p->w.get(), &w) != 0 || (p->bias && AcquireIn(p->bias.get(), &bias) != 0) ||
            cuda_detail::AcquireOutputTensorDevice(p->out.get(), out_bytes, &out) != 0) return -1;
        d.a = x; d.w = static_cast<const int8_t*>(w); d.bias = static_cast<const int32_t*>(bias); d.out = out;
        d.w_scales = static_cast<const float*>(scales_.get());
        d.w_zps = has_zps_ ? static_cast<const int32_t*>(zps_.get()) : nullptr;
        d.workspace = workspace_.get(); d.workspace_bytes = workspace_.bytes();
        d.weights_static = weights_resident_ ? 1 : 0;
        if (fth_b200_int8_linear(&d, cuda_detail::InferenceStream()) != FTH_B200_OK) return -1;
        weights_resident_ = p->w->is_immutable();
        return FinishOut(p->out.get(), out_bytes);
    }

   private:
    static void Probe(fth_b200_int8_linear_desc* d, const Int8WeightParams& wq) {
        d->a = kProbe; d->w = static_cast<const int8_t*>(kProbe); d->out = kProbe;
        d->w_scales = static_cast<const float*>(kProbe);
        if (wq.zp_max_abs != 0) d->w_zps = static_cast<const int32_t*>(kProbe);
        if (d->bias_mode != FTH_B200_BIAS_NONE) d->bias = static_cast<const int32_t*>(kProbe);
        d->workspace = kProbe; d->workspace_bytes = static_cast<size_t>(-1);
    }
    DeviceScratch scales_, zps_, workspace_;
    bool has_zps_{false}, weights_resident_{false};
};

class Conv2DReluKernel final : public B200Kernel {
   public:
    Status Supports() const override {
        fth_b200_int8_conv2d_desc d;
        Int8WeightParams wq, rq;
        if (!Describe(ParamAs<Conv2DReluParam>(), &d, &wq, &rq)) return Status::Error(StatusCode::kUnsupported, "b200: not a fused INT8 Conv2D -> ReLU");
        d.x = static_cast<const int8_t*>(kProbe); d.w = d.x; d.out = static_cast<int8_t*>(kProbe);
        d.w_scales = static_cast<const float*>(kProbe); d.relu_lut = d.x;
        if (wq.zp_max_abs != 0) d.w_zps = static_cast<const int32_t*>(kProbe);
        d.workspace = kProbe; d.workspace_bytes = static_cast<size_t>(-1);
        return FromAbi(fth_b200_int8_conv2d_supported(&d), kConv2DRelu);
    }
    int32_t Prepare() override {
        auto* p = ParamAs<Conv2DReluParam>();
        fth_b200_int8_conv2d_desc d;
        Int8WeightParams wq, rq;
        if (!Describe(p, &d, &wq, &rq)) return -1;
        if (scales_.Upload(wq.scales.data(), wq.scales.size() * sizeof(float)) != 0) return -1;
        has_zps_ = wq.zp_max_abs != 0;
        if (has_zps_ && zps_.Upload(wq.zero_points.data(), wq.zero_points.size() * sizeof(int32_t)) != 0) return -1;
        // the INT8 ReLU node as a table: conv output (s, zp) -> ReLU output (s, zp), src/kernel/common/int8_standard.cc:114-128
        int8_t lut[256];
        if (fth_b200_int8_relu_table(p->conv_scale, p->conv_zp, rq.scales[0], rq.zero_points[0], lut) != FTH_B200_OK) return -1;
        if (lut_.Upload(lut, sizeof(lut)) != 0) return -1;
        d.x = static_cast<const int8_t*>(kProbe); d.w = d.x; d.out = static_cast<int8_t*>(kProbe);
        d.w_scales = static_cast<const float*>(kProbe);
        packed_ = false;
        shared_packed_.reset();
        void* w_device = nullptr;
        if (p->conv.w->is_immutable() && AcquireIn(p->conv.w.get(), &w_device) == 0) {
            fth_b200_int8_conv2d_desc pack = d;
            pack.w = static_cast<const int8_t*>(w_device);
            shared_packed_ = PackedConvWeightCache::Acquire(p->conv.w.get(), pack);
        }
        if (shared_packed_) d.packed_w = static_cast<const int8_t*>(shared_packed_->get());
        return workspace_.Reserve(fth_b200_int8_conv2d_workspace_bytes(&d), true);
    }
    int32_t compute() override {
        AutoTimer timer("B200::Conv2DRelu");
        auto* p = ParamAs<Conv2DReluParam>();
        fth_b200_int8_conv2d_desc d;
        Int8WeightParams wq, rq;
        if (!Describe(p, &d, &wq, &rq) || scales_.get() == nullptr || lut_.get() == nullptr) return -1;
        void* x = nullptr; void* w = nullptr; void* bias = nullptr; void* out = nullptr;
        const size_t out_bytes = static_cast<size_t>(p->conv.out->numel());
        if (AcquireIn(p->conv.input.get(), &x) != 0 || AcquireIn(p->conv.w.get(), &w) != 0 ||
            (p->conv.bias && AcquireIn(p->conv.bias.get(), &bias) != 0) ||
            cuda_detail::AcquireOutputTensorDevice(p->conv.out.get(), out_bytes, &out) != 0) return -1;
        d.x = static_cast<const int8_t*>(x); d.w = static_cast<const int8_t*>(w); d.bias = static_cast<const int32_t*>(bias);
        d.out = static_cast<int8_t*>(out);
        d.w_scales = static_cast<const float*>(scales_.get());
        d.w_zps = has_zps_ ? static_cast<const int32_t*>(zps_.get()) : nullptr;
        d.relu_lut = static_cast<const int8_t*>(lut_.get());
        d.workspace = workspace_.get(); d.workspace_bytes = workspace_.bytes();
        d.weights_packed = packed_ ? 1 : 0;
        d.packed_w = shared_packed_ ? static_cast<const int8_t*>(shared_packed_->get()) : nullptr;
        if (fth_b200_int8_conv2d(&d, cuda_detail::InferenceStream()) != FTH_B200_OK) return -1;
        packed_ = p->conv.w->is_immutable();
        return FinishOut(p->conv.out.get(), out_bytes);
    }

   private:
    DeviceScratch scales_, zps_, lut_, workspace_;
    std::shared_ptr<DeviceScratch> shared_packed_;
    bool has_zps_{false}, packed_{false};
};

// ---------------------------------------------------------------------------------------------------------
// operator builders
// ---------------------------------------------------------------------------------------------------------
std::shared_ptr<OpBase> BuildFusedCastMatMulCast(const model::NodeDesc& node, OperatorRegistry::TensorMap& tensors,
                                                 const OperatorRegistry::BuildContext& context) {
    if (node.inputs.size() < 2 || node.inputs.size() > 5 || node.outputs.size() != 1) return nullptr;
    FusedCastMatMulCastParam param;
    param.x = tensors[node.inputs[0]];
    param.w = tensors[node.inputs[1]];
    // optional operands, in this order, each announced by its attribute
    size_t next = 2;
    std::vector<std::shared_ptr<Tensor>> extra;
    if (IntAttr(node.attributes, "norm", 0) != 0) {
        if (next >= node.inputs.size()) return nullptr;
        param.norm_weight = tensors[node.inputs[next++]];
        param.norm_offset = FloatAttr(node.attributes, "norm_offset", 0.0f);
        param.norm_epsilon = FloatAttr(node.attributes, "norm_epsilon", 0.0f);
        if (!param.norm_weight) return nullptr;
        extra.push_back(param.norm_weight);
    }
    if (IntAttr(node.attributes, "residual", 0) != 0) {
        if (next >= node.inputs.size()) return nullptr;
        param.residual = tensors[node.inputs[next++]];
        if (!param.residual) return nullptr;
        extra.push_back(param.residual);
    }
    if (IntAttr(node.attributes, "silu_mul", 0) != 0) {
        if (next >= node.inputs.size()) return nullptr;
        param.w2 = tensors[node.inputs[next++]];
        if (!param.w2) return nullptr;
        extra.push_back(param.w2);
    }
    if (next != node.inputs.size()) return nullptr;
    param.a_scale = FloatAttr(node.attributes, "a_scale", 0.0f);
    param.proj_scale = FloatAttr(node.attributes, "proj_scale", 0.0f);
    param.trans_b = IntAttr(node.attributes, "transB", 0) != 0;
    const int64_t to = IntAttr(node.attributes, "to", 16);
    const DataType out_dtype = to == 1 ? DataType::FP32 : DataType::BF16;
    int64_t m = 0, k = 0, n = 0;
    if (!param.x || !param.w || !LinearDims(param.x.get(), param.w.get(), param.trans_b, &m, &k, &n)) return nullptr;
    param.out = OutputFor(tensors[node.outputs[0]], param.x.get(), n, out_dtype);
    if (!param.out) return nullptr;
    param.out->set_quantization(QuantizationParams{});
    tensors[node.outputs[0]] = param.out;
    std::vector<std::shared_ptr<Tensor>> inputs{param.x, param.w};
    inputs.insert(inputs.end(), extra.begin(), extra.end());
    auto op = std::make_shared<FusedOp<FusedCastMatMulCastParam>>(node.name, kFusedCastMatMulCast, param, inputs, param.out);
    auto kernel = CreateKernelForTensor(context.device, kFusedCastMatMulCast, {param.x, param.w, param.out}, param.x->data_type());
    if (!kernel) return nullptr;
    op->AttachKernel(std::move(kernel));
    return op;
}

std::shared_ptr<OpBase> BuildFusedQLinearDQ(const model::NodeDesc& node, OperatorRegistry::TensorMap& tensors,
                                            const OperatorRegistry::BuildContext& context) {
    if (node.inputs.size() < 2 || node.inputs.size() > 3 || node.outputs.size() != 1) return nullptr;
    FusedQLinearDQParam param;
    param.x = tensors[node.inputs[0]];
    param.w = tensors[node.inputs[1]];
    param.bias = node.inputs.size() == 3 ? tensors[node.inputs[2]] : nullptr;
    param.in_scale = FloatAttr(node.attributes, "in_scale", 0.0f);
    param.out_scale = FloatAttr(node.attributes, "out_scale", 0.0f);
    param.in_zp = static_cast<int32_t>(IntAttr(node.attributes, "in_zp", 0));
    param.out_zp = static_cast<int32_t>(IntAttr(node.attributes, "out_zp", 0));
    param.op = static_cast<int32_t>(IntAttr(node.attributes, "linear_op", FTH_B200_OP_MATMUL));
    param.trans_b = IntAttr(node.attributes, "transB", 0) != 0;
    param.alpha = FloatAttr(node.attributes, "alpha", 1.0f);
    param.beta = FloatAttr(node.attributes, "beta", 1.0f);
    int64_t m = 0, k = 0, n = 0;
    if (!param.x || !param.w || !LinearDims(param.x.get(), param.w.get(), param.trans_b, &m, &k, &n)) return nullptr;
    param.out = OutputFor(tensors[node.outputs[0]], param.x.get(), n, DataType::FP32);
    if (!param.out) return nullptr;
    param.out->set_quantization(QuantizationParams{});
    tensors[node.outputs[0]] = param.out;
    std::vector<std::shared_ptr<Tensor>> inputs{param.x, param.w};
    if (param.bias) inputs.push_back(param.bias);
    auto op = std::make_shared<FusedOp<FusedQLinearDQParam>>(node.name, kFusedQLinearDQ, param, inputs, param.out);
    auto kernel = CreateKernelForTensor(context.device, kFusedQLinearDQ, {param.x, param.w, param.out}, DataType::FP32);
    if (!kernel) return nullptr;
    op->AttachKernel(std::move(kernel));
    return op;
}

std::shared_ptr<OpBase> BuildConv2DRelu(const model::NodeDesc& node, OperatorRegistry::TensorMap& tensors,
                                        const OperatorRegistry::BuildContext& context) {
    if (node.inputs.size() < 2 || node.inputs.size() > 3 || node.outputs.size() != 1) return nullptr;
    Conv2DReluParam param;
    operators::Conv2dParam& c = param.conv;
    c.input = tensors[node.inputs[0]];
    c.w = tensors[node.inputs[1]];
    c.bias = node.inputs.size() == 3 ? tensors[node.inputs[2]] : nullptr;
    c.out = tensors[node.outputs[0]];  // the ReLU node's output: shape, type and quantisation are already in place
    c.stride_h = static_cast<int32_t>(IntAttr(node.attributes, "stride_h", 1));
    c.stride_w = static_cast<int32_t>(IntAttr(node.attributes, "stride_w", 1));
    c.pad_h = static_cast<int32_t>(IntAttr(node.attributes, "pad_h", 0));
    c.pad_w = static_cast<int32_t>(IntAttr(node.attributes, "pad_w", 0));
    c.dilation_h = static_cast<int32_t>(IntAttr(node.attributes, "dilation_h", 1));
    c.dilation_w = static_cast<int32_t>(IntAttr(node.attributes, "dilation_w", 1));
    c.group = static_cast<int32_t>(IntAttr(node.attributes, "group", 1));
    param.conv_scale = FloatAttr(node.attributes, "conv_scale", 0.0f);
    param.conv_zp = static_cast<int32_t>(IntAttr(node.attributes, "conv_zp", 0));
    if (!c.input || !c.w || !c.out || !c.out->IsInitialized() || c.out->data_type() != DataType::INT8) return nullptr;
    std::vector<std::shared_ptr<Tensor>> inputs{c.input, c.w};
    if (c.bias) inputs.push_back(c.bias);
    auto op = std::make_shared<FusedOp<Conv2DReluParam>>(node.name, kConv2DRelu, param, inputs, c.out);
    auto kernel = CreateKernelForTensor(context.device, kConv2DRelu, {c.input, c.w, c.out}, DataType::INT8);
    if (!kernel) return nullptr;
    op->AttachKernel(std::move(kernel));
    return op;
}

// ---------------------------------------------------------------------------------------------------------
// the pass
// ---------------------------------------------------------------------------------------------------------
const model::NodeDesc* ModelNode(const StaticGraph& graph, const std::string& name) {
    for (const auto& n : graph.model().graph.nodes)
        if (n.name == name) return &n;
    return nullptr;
}

// The node that produces `value`, if `value` is used by `user` alone and is not a graph output.
const StaticNode* SoleProducer(const StaticGraph& graph, const std::string& value, const std::string& user) {
    if (graph.IsGraphOutputValue(value)) return nullptr;
    const auto users = graph.GetUsers(value);
    if (users.size() != 1 || users[0] != user) return nullptr;
    const std::string producer = graph.GetProducer(value);
    const StaticNode* node = producer.empty() ? nullptr : graph.GetNode(producer);
    return node != nullptr && !node->removed ? node : nullptr;
}

// One finite float / integer out of a scalar constant tensor (the Q / DQ parameters the static quantiser emits).
bool ScalarConstant(const StaticGraph& graph, const std::string& name, double* value) {
    const auto t = graph.GetTensor(name);
    if (!t || !t->IsInitialized() || t->numel() != 1) return false;
    switch (t->data_type()) {
        case DataType::FP32: *value = t->data<float>()[0]; return true;
        case DataType::INT8: *value = t->data<int8_t>()[0]; return true;
        case DataType::UINT8: *value = t->data<uint8_t>()[0]; return true;
        case DataType::INT32: *value = t->data<int32_t>()[0]; return true;
        case DataType::INT64: *value = static_cast<double>(t->data<int64_t>()[0]); return true;
        default: return false;
    }
}

class B200FusionPass final : public GraphPass {
   public:
    const std::string& name() const override { static const std::string n = "B200FusionPass"; return n; }
    bool SupportsDevice(DeviceType device) const override { return device == DeviceType::CUDA; }

    int32_t Run(StaticGraph* graph) override {
        if (graph == nullptr) return -1;
        std::vector<std::string> names;
        for (const auto& node : graph->nodes())
            if (!node.removed) names.push_back(node.name);
        for (const auto& n : names) {
            const StaticNode* node = graph->GetNode(n);
            if (node == nullptr || node->removed) continue;
            int rc = 0;
            if (node->op_type == "Cast") rc = FuseCastChain(graph, *node);
            else if (node->op_type == "DequantizeLinear") rc = FuseQdqChain(graph, *node);
            else if (node->op_type == "ReLU") rc = FuseConvRelu(graph, *node);
            if (rc != 0) return rc;
        }
        // Second phase: the decoder-block nodes around the fused projections of the first phase.  Gate / up pairs
        // first (they change which node reads the norm's output), then norms in front, then residual Adds behind.
        for (int phase = 0; phase < 3; ++phase) {
            names.clear();
            for (const auto& node : graph->nodes())
                if (!node.removed && node.op_type == (phase == 0 ? "Mul" : phase == 1 ? "QwenRmsNorm" : "Add")) names.push_back(node.name);
            for (const auto& n : names) {
                const StaticNode* node = graph->GetNode(n);
                if (node == nullptr || node->removed) continue;
                const int rc = phase == 0 ? FuseGateUp(graph, *node) : phase == 1 ? FuseNorm(graph, *node) : FuseResidual(graph, *node);
                if (rc != 0) return rc;
            }
        }
        return 0;
    }

   private:
    // ---- decoder-block fusions (second phase) -------------------------------------------------------------------
    // The parameter struct a FusedCastMatMulCast node of the graph would be built with (tensors from the graph).
    static bool ParamOfNode(const StaticGraph& graph, const StaticNode& node, const model::NodeDesc& desc, FusedCastMatMulCastParam* p) {
        if (node.inputs.size() < 2 || node.outputs.size() != 1) return false;
        p->x = graph.GetTensor(node.inputs[0]);
        p->w = graph.GetTensor(node.inputs[1]);
        p->out = graph.GetTensor(node.outputs[0]);
        p->a_scale = FloatAttr(desc.attributes, "a_scale", 0.0f);
        p->proj_scale = FloatAttr(desc.attributes, "proj_scale", 0.0f);
        p->trans_b = IntAttr(desc.attributes, "transB", 0) != 0;
        size_t next = 2;
        if (IntAttr(desc.attributes, "norm", 0) != 0 && next < node.inputs.size()) {
            p->norm_weight = graph.GetTensor(node.inputs[next++]);
            p->norm_offset = FloatAttr(desc.attributes, "norm_offset", 0.0f);
            p->norm_epsilon = FloatAttr(desc.attributes, "norm_epsilon", 0.0f);
        }
        if (IntAttr(desc.attributes, "residual", 0) != 0 && next < node.inputs.size()) p->residual = graph.GetTensor(node.inputs[next++]);
        if (IntAttr(desc.attributes, "silu_mul", 0) != 0 && next < node.inputs.size()) p->w2 = graph.GetTensor(node.inputs[next++]);
        return p->x && p->w && p->out && next == node.inputs.size();
    }
    // Would the library run this projection with these neighbours in one launch?
    static bool FusedFormSupported(const FusedCastMatMulCastParam& p) {
        fth_b200_fp8_linear_desc d;
        fth_b200_fp8_linear_fusion f;
        if (!Describe(&p, &d) || !DescribeFusion(&p, d, &f)) return false;
        d.a = d.w = d.out = kProbe;
        if (p.norm_weight) f.norm_weight = kProbe;
        if (p.residual) f.residual = kProbe;
        if (p.w2) f.w2 = kProbe;
        return fth_b200_fp8_linear_fused_supported(&d, &f) == FTH_B200_OK;
    }
    // The node list of a FusedCastMatMulCast node from its parameter struct (inputs in the builder's order).
    static model::NodeDesc DescOf(const std::string& name, const model::NodeDesc& base, const std::vector<std::string>& inputs,
                                  const std::vector<std::string>& outputs, const FusedCastMatMulCastParam& p) {
        model::NodeDesc r;
        r.name = name;
        r.op_type = kFusedCastMatMulCast;
        r.inputs = inputs;
        r.outputs = outputs;
        r.attributes = base.attributes;
        r.attributes["norm"] = int64_t{p.norm_weight ? 1 : 0};
        r.attributes["norm_offset"] = p.norm_offset;
        r.attributes["norm_epsilon"] = p.norm_epsilon;
        r.attributes["residual"] = int64_t{p.residual ? 1 : 0};
        r.attributes["silu_mul"] = int64_t{p.w2 ? 1 : 0};
        return r;
    }
    static const StaticNode* LiveNode(const StaticGraph& graph, const std::string& name) {
        const StaticNode* node = name.empty() ? nullptr : graph.GetNode(name);
        return node != nullptr && !node->removed ? node : nullptr;
    }

    // Mul(SiLU(gate(h)), up(h)) with gate and up two fused projections of the same activation -> one node with two
    // weights (matched from the Mul; either operand order).
    static int FuseGateUp(StaticGraph* graph, const StaticNode& mul) {
        if (mul.inputs.size() != 2 || mul.outputs.size() != 1) return 0;
        for (int order = 0; order < 2; ++order) {
            const std::string& silu_out = mul.inputs[static_cast<size_t>(order)];
            const std::string& up_out = mul.inputs[static_cast<size_t>(1 - order)];
            const StaticNode* silu = SoleProducer(*graph, silu_out, mul.name);
            const StaticNode* up = SoleProducer(*graph, up_out, mul.name);
            if (silu == nullptr || up == nullptr || silu->op_type != "SiLU" || silu->inputs.size() != 1 || up->op_type != kFusedCastMatMulCast) continue;
            const StaticNode* gate = SoleProducer(*graph, silu->inputs[0], silu->name);
            if (gate == nullptr || gate->op_type != kFusedCastMatMulCast || gate->inputs.size() != 2 || up->inputs.size() != 2 ||
                gate->inputs[0] != up->inputs[0]) continue;
            const model::NodeDesc* gate_desc = ModelNode(*graph, gate->name);
            const model::NodeDesc* up_desc = ModelNode(*graph, up->name);
            if (gate_desc == nullptr || up_desc == nullptr) continue;
            FusedCastMatMulCastParam g, u;
            if (!ParamOfNode(*graph, *gate, *gate_desc, &g) || !ParamOfNode(*graph, *up, *up_desc, &u)) continue;
            // one activation Cast and one output Cast serve both products: their scales and layouts must agree
            if (g.a_scale != u.a_scale || g.proj_scale != u.proj_scale || g.trans_b != u.trans_b || g.fused() || u.fused()) continue;
            const auto out = graph->GetTensor(mul.outputs[0]);
            if (!out || out->data_type() != DataType::BF16 || out->numel() != g.out->numel()) continue;
            g.w2 = u.w;
            g.out = out;
            if (!FusedFormSupported(g)) continue;
            const model::NodeDesc r = DescOf(mul.name, *gate_desc, {gate->inputs[0], gate->inputs[1], up->inputs[1]}, mul.outputs, g);
            const std::string gate_name = gate->name, up_name = up->name, silu_name = silu->name;
            if (!graph->ReplaceNodeDesc(r) || !graph->RemoveNode(silu_name) || !graph->RemoveNode(gate_name) || !graph->RemoveNode(up_name)) return -1;
            return 0;
        }
        return 0;
    }

    // QwenRmsNorm(x, weight, epsilon) whose output is read by fused projections only (q, k, v of an attention block; the
    // gate | up pair of an MLP block) -> every one of them normalises its activation itself and the norm node goes.
    // The row's 1 / rms is then computed once per projection instead of once: a few KB of L2 reads against a launch.
    static int FuseNorm(StaticGraph* graph, const StaticNode& norm) {
        if (norm.inputs.size() != 3 || norm.outputs.size() != 1 || graph->IsGraphOutputValue(norm.outputs[0])) return 0;
        const model::NodeDesc* norm_desc = ModelNode(*graph, norm.name);
        const auto x = graph->GetTensor(norm.inputs[0]);
        const auto weight = graph->GetTensor(norm.inputs[1]);
        double epsilon = 0.0;
        if (norm_desc == nullptr || !x || !weight || !weight->is_immutable() || x->data_type() != DataType::BF16 ||
            !ScalarConstant(*graph, norm.inputs[2], &epsilon)) return 0;
        const float offset = FloatAttr(norm_desc->attributes, "weight_offset", 0.0f);
        const std::vector<std::string> users = graph->GetUsers(norm.outputs[0]);
        if (users.empty()) return 0;
        std::vector<model::NodeDesc> replacements;
        for (const auto& user : users) {
            const StaticNode* proj = LiveNode(*graph, user);
            const model::NodeDesc* desc = proj != nullptr ? ModelNode(*graph, proj->name) : nullptr;
            FusedCastMatMulCastParam p;
            if (proj == nullptr || desc == nullptr || proj->op_type != kFusedCastMatMulCast || proj->inputs[0] != norm.outputs[0] ||
                !ParamOfNode(*graph, *proj, *desc, &p) || p.norm_weight || p.x->data_type() != DataType::BF16) return 0;
            for (size_t i = 1; i < proj->inputs.size(); ++i)
                if (proj->inputs[i] == norm.outputs[0]) return 0;  // also read as a residual: the value has to exist
            p.x = x;
            p.norm_weight = weight;
            p.norm_offset = offset;
            p.norm_epsilon = static_cast<float>(epsilon);
            if (!FusedFormSupported(p)) return 0;
            std::vector<std::string> inputs{norm.inputs[0], proj->inputs[1], norm.inputs[1]};
            inputs.insert(inputs.end(), proj->inputs.begin() + 2, proj->inputs.end());  // residual / second weight keep their places
            replacements.push_back(DescOf(proj->name, *desc, inputs, proj->outputs, p));
        }
        const std::string norm_name = norm.name;
        for (const auto& r : replacements)
            if (!graph->ReplaceNodeDesc(r)) return -1;
        return graph->RemoveNode(norm_name) ? 0 : -1;
    }

    // Add(residual, projection) with the projection read by the Add alone -> the projection adds the residual itself
    // (matched from the Add; either operand order).
    static int FuseResidual(StaticGraph* graph, const StaticNode& add) {
        if (add.inputs.size() != 2 || add.outputs.size() != 1) return 0;
        for (int order = 0; order < 2; ++order) {
            const StaticNode* proj = SoleProducer(*graph, add.inputs[static_cast<size_t>(order)], add.name);
            const std::string& other = add.inputs[static_cast<size_t>(1 - order)];
            if (proj == nullptr || proj->op_type != kFusedCastMatMulCast) continue;
            const model::NodeDesc* desc = ModelNode(*graph, proj->name);
            FusedCastMatMulCastParam p;
            if (desc == nullptr || !ParamOfNode(*graph, *proj, *desc, &p) || p.residual || p.w2) continue;
            const auto residual = graph->GetTensor(other);
            const auto out = graph->GetTensor(add.outputs[0]);
            if (!residual || !out || residual->data_type() != DataType::BF16 || out->data_type() != DataType::BF16 ||
                residual->numel() != p.out->numel() || out->numel() != p.out->numel()) continue;
            p.residual = residual;
            p.out = out;
            if (!FusedFormSupported(p)) continue;
            std::vector<std::string> inputs{proj->inputs[0], proj->inputs[1]};
            if (p.norm_weight) inputs.push_back(proj->inputs[2]);
            inputs.push_back(other);
            const model::NodeDesc r = DescOf(add.name, *desc, inputs, add.outputs, p);
            const std::string proj_name = proj->name;
            if (!graph->ReplaceNodeDesc(r) || !graph->RemoveNode(proj_name)) return -1;
            return 0;
        }
        return 0;
    }

    // Cast(wide -> FP8) -> MatMul / Gemm(transB, no bias, alpha = beta = 1) -> Cast(FP8 -> wide), matched from the last
    // Cast.  The lm-head form (the last Cast writes the graph output "logits" of a Qwen plan, [1,K] x [N,K]) becomes
    // QwenGemmArgmax as in the reference's own pass; every other chain becomes FusedCastMatMulCast.
    static int FuseCastChain(StaticGraph* graph, const StaticNode& last) {
        if (last.inputs.size() != 1 || last.outputs.size() != 1) return 0;
        const auto out = graph->GetTensor(last.outputs[0]);
        const auto mid = graph->GetTensor(last.inputs[0]);
        if (!out || !mid || !IsWide(out->data_type()) || !IsFp8(mid->data_type())) return 0;
        const StaticNode* mm = SoleProducer(*graph, last.inputs[0], last.name);
        if (mm == nullptr || (mm->op_type != "MatMul" && mm->op_type != "Gemm") || mm->inputs.size() != 2 || mm->outputs.size() != 1) return 0;
        bool trans_b = false;
        if (mm->op_type == "Gemm") {
            const model::NodeDesc* desc = ModelNode(*graph, mm->name);
            if (desc == nullptr || IntAttr(desc->attributes, "transA", 0) != 0 || FloatAttr(desc->attributes, "alpha", 1.0f) != 1.0f ||
                FloatAttr(desc->attributes, "beta", 1.0f) != 1.0f) return 0;
            trans_b = IntAttr(desc->attributes, "transB", 0) != 0;
        }
        const auto act = graph->GetTensor(mm->inputs[0]);
        const auto w = graph->GetTensor(mm->inputs[1]);
        if (!act || !w || act->data_type() != mid->data_type() || w->data_type() != mid->data_type() || !w->is_immutable() ||
            !HasCompatiblePerTensorQuantization(act->quantization()) || !HasCompatiblePerTensorQuantization(w->quantization()) ||
            !HasCompatiblePerTensorQuantization(mid->quantization())) return 0;
        const std::string first_name = graph->GetProducer(mm->inputs[0]);
        const StaticNode* first = first_name.empty() ? nullptr : graph->GetNode(first_name);
        if (first == nullptr || first->removed || first->op_type != "Cast" || first->inputs.size() != 1 || graph->IsGraphOutputValue(mm->inputs[0])) return 0;
        const auto x = graph->GetTensor(first->inputs[0]);
        if (!x || !IsWide(x->data_type())) return 0;

        FusedCastMatMulCastParam probe;
        probe.x = x; probe.w = w; probe.out = out;
        probe.a_scale = act->quantization_scale(); probe.proj_scale = mid->quantization_scale(); probe.trans_b = trans_b;
        fth_b200_fp8_linear_desc d;
        if (!Describe(&probe, &d)) return 0;
        d.a = d.w = d.out = kProbe;
        d.workspace = kProbe; d.workspace_bytes = static_cast<size_t>(-1);
        if (fth_b200_fp8_linear_supported(&d) != FTH_B200_OK) return 0;  // left as three nodes

        model::NodeDesc replacement;
        replacement.name = last.name;
        replacement.op_type = kFusedCastMatMulCast;
        replacement.inputs = {first->inputs[0], mm->inputs[1]};
        replacement.outputs = last.outputs;
        replacement.attributes["a_scale"] = probe.a_scale;
        replacement.attributes["proj_scale"] = probe.proj_scale;
        replacement.attributes["transB"] = int64_t{trans_b ? 1 : 0};
        replacement.attributes["to"] = int64_t{out->data_type() == DataType::FP32 ? 1 : 16};
        const std::string mm_name = mm->name, first_value = mm->inputs[0];
        if (!graph->ReplaceNodeDesc(replacement) || !graph->RemoveNode(mm_name)) return -1;
        // the first Cast may feed other projections of the same activation: it goes only when nothing reads it any more
        if (graph->GetUsers(first_value).empty() && !graph->RemoveNode(first_name)) return -1;
        return 0;
    }

    // QuantizeLinear(FP32) -> FC / MatMul / Gemm (INT8) -> DequantizeLinear(to FP32), matched from the DequantizeLinear.
    static int FuseQdqChain(StaticGraph* graph, const StaticNode& last) {
        if (last.inputs.size() != 3 || last.outputs.size() != 1) return 0;
        const auto out = graph->GetTensor(last.outputs[0]);
        const auto mid = graph->GetTensor(last.inputs[0]);
        if (!out || !mid || out->data_type() != DataType::FP32 || mid->data_type() != DataType::INT8) return 0;
        const StaticNode* lin = SoleProducer(*graph, last.inputs[0], last.name);
        if (lin == nullptr || lin->outputs.size() != 1 || lin->inputs.size() < 2 || lin->inputs.size() > 3) return 0;
        int32_t op;
        if (lin->op_type == "FC") op = FTH_B200_OP_FC;
        else if (lin->op_type == "MatMul") op = FTH_B200_OP_MATMUL;
        else if (lin->op_type == "Gemm") op = FTH_B200_OP_GEMM;
        else return 0;
        const model::NodeDesc* desc = ModelNode(*graph, lin->name);
        if (desc == nullptr) return 0;
        bool trans_b = false;
        float alpha = 1.0f, beta = 1.0f;
        if (op == FTH_B200_OP_GEMM) {
            if (IntAttr(desc->attributes, "transA", 0) != 0) return 0;
            trans_b = IntAttr(desc->attributes, "transB", 0) != 0;
            alpha = FloatAttr(desc->attributes, "alpha", 1.0f);
            beta = FloatAttr(desc->attributes, "beta", 1.0f);
        }
        const bool has_bias = lin->inputs.size() == 3 && !lin->inputs[2].empty();
        if (op == FTH_B200_OP_MATMUL && has_bias) return 0;
        const std::string q_name = graph->GetProducer(lin->inputs[0]);
        const StaticNode* q = q_name.empty() ? nullptr : graph->GetNode(q_name);
        if (q == nullptr || q->removed || q->op_type != "QuantizeLinear" || q->inputs.size() != 3 || graph->IsGraphOutputValue(lin->inputs[0])) return 0;
        const auto x = graph->GetTensor(q->inputs[0]);
        const auto w = graph->GetTensor(lin->inputs[1]);
        const auto bias = has_bias ? graph->GetTensor(lin->inputs[2]) : nullptr;
        if (!x || !w || x->data_type() != DataType::FP32 || w->data_type() != DataType::INT8 || !w->is_immutable()) return 0;
        double in_scale = 0, in_zp = 0, out_scale = 0, out_zp = 0;
        if (!ScalarConstant(*graph, q->inputs[1], &in_scale) || !ScalarConstant(*graph, q->inputs[2], &in_zp) ||
            !ScalarConstant(*graph, last.inputs[1], &out_scale) || !ScalarConstant(*graph, last.inputs[2], &out_zp)) return 0;
        // the linear node requantises to its declared output parameters; the DequantizeLinear must read them back with the same pair
        const QuantizationParams& mq = mid->quantization();
        if (!mq.enabled || mq.granularity != QuantizationGranularity::kPerTensor || mq.scale_at(0) != static_cast<float>(out_scale) ||
            mq.zero_point_at(0) != static_cast<int32_t>(out_zp)) return 0;

        FusedQLinearDQParam probe;
        probe.x = x; probe.w = w; probe.bias = bias; probe.out = out;
        probe.in_scale = static_cast<float>(in_scale); probe.in_zp = static_cast<int32_t>(in_zp);
        probe.out_scale = static_cast<float>(out_scale); probe.out_zp = static_cast<int32_t>(out_zp);
        probe.op = op; probe.trans_b = trans_b; probe.alpha = alpha; probe.beta = beta;
        fth_b200_int8_linear_desc d;
        Int8WeightParams wq;
        if (!Describe(&probe, &d, &wq)) return 0;
        d.a = kProbe; d.w = static_cast<const int8_t*>(kProbe); d.out = kProbe; d.w_scales = static_cast<const float*>(kProbe);
        if (wq.zp_max_abs != 0) d.w_zps = static_cast<const int32_t*>(kProbe);
        if (d.bias_mode != FTH_B200_BIAS_NONE) d.bias = static_cast<const int32_t*>(kProbe);
        d.workspace = kProbe; d.workspace_bytes = static_cast<size_t>(-1);
        if (fth_b200_int8_linear_supported(&d) != FTH_B200_OK) return 0;

        model::NodeDesc replacement;
        replacement.name = last.name;
        replacement.op_type = kFusedQLinearDQ;
        replacement.inputs = {q->inputs[0], lin->inputs[1]};
        if (has_bias) replacement.inputs.push_back(lin->inputs[2]);
        replacement.outputs = last.outputs;
        replacement.attributes["in_scale"] = probe.in_scale;
        replacement.attributes["in_zp"] = int64_t{probe.in_zp};
        replacement.attributes["out_scale"] = probe.out_scale;
        replacement.attributes["out_zp"] = int64_t{probe.out_zp};
        replacement.attributes["linear_op"] = int64_t{op};
        replacement.attributes["transB"] = int64_t{trans_b ? 1 : 0};
        replacement.attributes["alpha"] = alpha;
        replacement.attributes["beta"] = beta;
        const std::string lin_name = lin->name, q_value = lin->inputs[0];
        if (!graph->ReplaceNodeDesc(replacement) || !graph->RemoveNode(lin_name)) return -1;
        if (graph->GetUsers(q_value).empty() && !graph->RemoveNode(q_name)) return -1;
        return 0;
    }

    // Conv2D(INT8) -> ReLU(INT8), matched from the ReLU.
    static int FuseConvRelu(StaticGraph* graph, const StaticNode& last) {
        if (last.inputs.size() != 1 || last.outputs.size() != 1) return 0;
        const auto out = graph->GetTensor(last.outputs[0]);
        const auto mid = graph->GetTensor(last.inputs[0]);
        if (!out || !mid || out->data_type() != DataType::INT8 || mid->data_type() != DataType::INT8) return 0;
        const StaticNode* conv = SoleProducer(*graph, last.inputs[0], last.name);
        if (conv == nullptr || (conv->op_type != "Conv2D" && conv->op_type != "Conv") || conv->inputs.size() < 2 || conv->outputs.size() != 1) return 0;
        const model::NodeDesc* desc = ModelNode(*graph, conv->name);
        if (desc == nullptr) return 0;
        Int8WeightParams mq;
        if (!ReadInt8Quantization(mid.get(), false, -1, 1, &mq)) return 0;
        const bool has_bias = conv->inputs.size() > 2 && !conv->inputs[2].empty();
        Conv2DReluParam probe;
        probe.conv.input = graph->GetTensor(conv->inputs[0]);
        probe.conv.w = graph->GetTensor(conv->inputs[1]);
        probe.conv.bias = has_bias ? graph->GetTensor(conv->inputs[2]) : nullptr;
        probe.conv.out = out;
        probe.conv.stride_h = static_cast<int32_t>(IntAttr(desc->attributes, "stride_h", 1));
        probe.conv.stride_w = static_cast<int32_t>(IntAttr(desc->attributes, "stride_w", 1));
        probe.conv.pad_h = static_cast<int32_t>(IntAttr(desc->attributes, "pad_h", 0));
        probe.conv.pad_w = static_cast<int32_t>(IntAttr(desc->attributes, "pad_w", 0));
        probe.conv.dilation_h = static_cast<int32_t>(IntAttr(desc->attributes, "dilation_h", 1));
        probe.conv.dilation_w = static_cast<int32_t>(IntAttr(desc->attributes, "dilation_w", 1));
        probe.conv.group = static_cast<int32_t>(IntAttr(desc->attributes, "group", 1));
        probe.conv_scale = mq.scales[0];
        probe.conv_zp = mq.zero_points[0];
        if (!probe.conv.w || !probe.conv.w->is_immutable()) return 0;
        fth_b200_int8_conv2d_desc d;
        Int8WeightParams wq, rq;
        if (!Describe(&probe, &d, &wq, &rq)) return 0;
        d.x = static_cast<const int8_t*>(kProbe); d.w = d.x; d.out = static_cast<int8_t*>(kProbe);
        d.w_scales = static_cast<const float*>(kProbe); d.relu_lut = d.x;
        if (wq.zp_max_abs != 0) d.w_zps = static_cast<const int32_t*>(kProbe);
        d.workspace = kProbe; d.workspace_bytes = static_cast<size_t>(-1);
        if (fth_b200_int8_conv2d_supported(&d) != FTH_B200_OK) return 0;

        model::NodeDesc replacement;
        replacement.name = last.name;
        replacement.op_type = kConv2DRelu;
        replacement.inputs = {conv->inputs[0], conv->inputs[1]};
        if (has_bias) replacement.inputs.push_back(conv->inputs[2]);
        replacement.outputs = last.outputs;
        replacement.attributes = desc->attributes;
        replacement.attributes["conv_scale"] = probe.conv_scale;
        replacement.attributes["conv_zp"] = int64_t{probe.conv_zp};
        const std::string conv_name = conv->name;
        if (!graph->ReplaceNodeDesc(replacement) || !graph->RemoveNode(conv_name)) return -1;
        return 0;
    }
};

}  // namespace

// Registers the three operator types and their CUDA candidates.  Idempotent.
bool RegisterB200FusedOperators() {
    const char* off = std::getenv("FEATHER_DISABLE_B200");
    if (off != nullptr && off[0] == '1') return false;
    OperatorRegistry::instance().Register(kFusedCastMatMulCast, BuildFusedCastMatMulCast);
    OperatorRegistry::instance().Register(kFusedQLinearDQ, BuildFusedQLinearDQ);
    OperatorRegistry::instance().Register(kConv2DRelu, BuildConv2DRelu);
    for (DataType t : {DataType::BF16, DataType::FP32}) AddCandidate<FusedCastMatMulCastKernel>(t, kFusedCastMatMulCast, "b200.fused.cast_matmul_cast");
    AddCandidate<FusedQLinearDQKernel>(DataType::FP32, kFusedQLinearDQ, "b200.fused.q_linear_dq");
    AddCandidate<Conv2DReluKernel>(DataType::INT8, kConv2DRelu, "b200.fused.conv2d_relu");
    return true;
}

// The pass, to be appended to whatever pipeline a plan uses (StaticGraph::SetPassManager, include/core/static_graph.h:66).
std::unique_ptr<GraphPass> CreateB200FusionPass() { return std::unique_ptr<GraphPass>(new B200FusionPass()); }

}  // namespace b200
}  // namespace kernel
}  // namespace feather
