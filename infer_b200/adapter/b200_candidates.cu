// Feather-side adapter: KernelBase subclasses that put the sm_100a kernels of libfth_b200.so behind Feather's
// own kernel interface, and their registration as CUDA candidates in front of the reference's kernels.
//
// This file is compiled INSIDE a Feather build (it includes Feather headers; add it to the CUDA sources of the
// `infer` target and link libfth_b200.so).  It owns everything Feather-specific — Tensor, QuantizationParams,
// operators::*Param, the session's replica cache and stream — and hands plain pointers and sizes to the C ABI.
//
//   Supports()  capability check with the bound parameters (include/core/kernel.h:158).  A contract violation the
//               reference kernels answer with -1 stays kInvalidArgument at compute(); a valid request the new
//               kernels decline returns StatusCode::kUnsupported so FinalizeSelection (kernel.h:288-324) moves on
//               to the next CUDA candidate — never to a CPU kernel under KernelFallbackPolicy::kRequireRequested.
//   Prepare()   once per session (src/core/graph.cc:375-387), outside capture: uploads per-channel scales / zero
//               points, builds the INT8 ReLU table, allocates and zero-fills the split-K workspace.
//   compute()   no allocation, no synchronisation, no host read-back: device pointers come from the session's
//               replica cache (cuda_detail::CopyTensorToDevice / AllocateTensorOnDevice,
//               src/kernel/cuda/kernel_io.cuh:285-340) and the launch goes to cuda_detail::InferenceStream(), so
//               deferred host sync and CUDA-graph capture (src/kernel/backend.cc:80-118) keep working.
#include "b200_common.cuh"
#include "b200_shard.h"
#include "src/operator/params.h"
#include "util/bf16.h"
#include "util/timer.h"

namespace feather {
namespace kernel {
namespace b200 {

bool IsB200Kernel(const KernelBase* kernel) { return dynamic_cast<const B200Kernel*>(kernel) != nullptr; }

namespace {
// A node that is the current thread's rank of a column-sharded projection (ShardBindingScope): the descriptor is pointed
// at the group's gathered buffers, and after the launch the rank's own block is copied into the node's output tensor.
template <typename Desc>
const ShardBindingScope* BindShard(Desc* d, int64_t elem_bytes, void** node_out) {
    const ShardBindingScope* shard = ShardBindingScope::Current();
    if (shard == nullptr || !shard->Matches(d->m, d->n, elem_bytes) || d->bias_mode == FTH_B200_BIAS_MATRIX) return nullptr;
    *node_out = d->out;
    shard->group().Point(d, shard->rank());
    return shard;
}
template <typename Desc>
int FinishShard(const ShardBindingScope* shard, const Desc& d, void* node_out, int64_t elem_bytes, cudaStream_t stream) {
    if (shard == nullptr) return 0;
    const size_t row = static_cast<size_t>(d.n * elem_bytes);
    return cudaMemcpy2DAsync(node_out, row, d.out, static_cast<size_t>(d.ldo * elem_bytes), row, static_cast<size_t>(d.m),
                             cudaMemcpyDeviceToDevice, stream) == cudaSuccess ? 0 : -1;
}
}  // namespace
size_t PackedConvWeightEntries() { return PackedConvWeightCache::LiveEntries(); }

namespace {

void* const kProbe = ProbePointer();

// The three linear operators differ only in their parameter struct (src/operator/params.h:27-55, 141-150).
struct LinearView {
    Tensor* a{nullptr}; Tensor* w{nullptr}; Tensor* bias{nullptr}; Tensor* out{nullptr};
    float alpha{1.0f}, beta{1.0f};
    bool trans_a{false}, trans_b{false};
    int op{FTH_B200_OP_MATMUL};
};
bool View(operators::FcParam* p, LinearView* v) {
    if (!p) return false;
    *v = {p->input.get(), p->w.get(), p->bias.get(), p->out.get(), 1.0f, 1.0f, false, false, FTH_B200_OP_FC};
    return true;
}
bool View(operators::MatMulParam* p, LinearView* v) {
    if (!p) return false;
    *v = {p->a.get(), p->b.get(), nullptr, p->out.get(), 1.0f, 1.0f, false, false, FTH_B200_OP_MATMUL};
    return true;
}
bool View(operators::GemmParam* p, LinearView* v) {
    if (!p) return false;
    Tensor* bias = (p->bias && p->bias->IsInitialized()) ? p->bias.get() : nullptr;
    *v = {p->a.get(), p->b.get(), bias, p->out.get(), p->alpha, p->beta, p->trans_a, p->trans_b, FTH_B200_OP_GEMM};
    return true;
}

// M, K, N of a 2-D weight linear (leading activation dims fold into M); false for batched / broadcast B, which
// stays on the reference candidate.
bool LinearShape(const LinearView& v, int64_t* m, int64_t* k, int64_t* n) {
    if (!v.a || !v.w || !v.out || v.trans_a) return false;
    const auto& ad = v.a->dims().data();
    const auto& wd = v.w->dims().data();
    if (ad.size() < 2 || wd.size() != 2) return false;
    *k = ad.back();
    *m = *k > 0 ? v.a->numel() / *k : 0;
    const int64_t wk = v.trans_b ? wd[1] : wd[0];
    *n = v.trans_b ? wd[0] : wd[1];
    return *m > 0 && *k > 0 && *n > 0 && wk == *k && v.out->numel() == *m * *n;
}

int BiasMode(const Tensor* bias, int64_t m, int64_t n) {
    if (!bias) return FTH_B200_BIAS_NONE;
    if (bias->numel() == n) return FTH_B200_BIAS_VECTOR;
    return bias->numel() == m * n ? FTH_B200_BIAS_MATRIX : -1;
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------
// FP8 (E4M3 / E5M2) FC, MatMul, Gemm — in front of RunFp8Fc / RunFp8MatMul / RunFp8Gemm
// (src/kernel/cuda/fc.cu:91-142, matmul.cu:230-272, gemm.cu:125-183)
// ---------------------------------------------------------------------------------------------------------
template <DataType dtype, typename Param>
class Fp8LinearKernel final : public B200Kernel {
   public:
    // The factory runs inside the node's KernelSelectionScope (include/core/kernel.h:52-72): the scratch budget of the
    // request is read here and honoured below.
    Fp8LinearKernel() : workspace_limit_(KernelSelectionScope::WorkspaceLimit()) {}

    Status Supports() const override {
        fth_b200_fp8_linear_desc d;
        if (!Describe(&d)) return Status::Error(StatusCode::kUnsupported, "b200: not a 2-D FP8 linear");
        d.a = d.w = d.out = kProbe;
        if (d.bias_mode != FTH_B200_BIAS_NONE) d.bias = kProbe;
        if (ScratchMode(d) == Scratch::kOwned) {
            d.workspace = kProbe;  // Prepare() provides what workspace_bytes() asks for
            d.workspace_bytes = static_cast<size_t>(-1);
        }
        return FromAbi(fth_b200_fp8_linear_supported(&d), "FP8 linear");
    }

    int32_t Prepare() override {
        fth_b200_fp8_linear_desc d;
        const std::vector<float>* channel_scales = nullptr;
        if (!Describe(&d, nullptr, &channel_scales)) return -1;
        // per-channel weight scales go to the device once, here
        if (channel_scales != nullptr && scales_.Upload(channel_scales->data(), channel_scales->size() * sizeof(float)) != 0) return -1;
        d.a = d.w = d.out = kProbe;
        if (d.bias_mode != FTH_B200_BIAS_NONE) d.bias = kProbe;
        weights_resident_ = false;
        scratch_ = ScratchMode(d);
        if (scratch_ != Scratch::kOwned) return 0;
        return workspace_.Reserve(fth_b200_fp8_linear_workspace_bytes(&d), true);
    }

    int32_t compute() override {
        AutoTimer timer(dtype == DataType::FP8E4M3 ? "B200::Linear::FP8E4M3" : "B200::Linear::FP8E5M2");
        using T = cuda_detail::StorageT<dtype>;
        fth_b200_fp8_linear_desc d;
        LinearView v;
        if (!Describe(&d, &v)) return -1;
        // (IsTensorReady insists on a per-tensor scale, src/kernel/cuda/kernel_io.cuh:245-252: a weight with per-channel
        // scales, which Describe() has validated, is checked for its bytes only)
        const bool w_ready = d.w_channel_scales != nullptr
                                 ? v.w->IsInitialized() && v.w->data_type() == dtype && v.w->memory_size() >= static_cast<size_t>(d.k * d.n)
                                 : cuda_detail::IsTensorReady<dtype>(v.w);
        if (!cuda_detail::IsTensorReady<dtype>(v.a) || !w_ready || !cuda_detail::IsOutputReady<dtype>(v.out)) return -1;
        cuda_detail::DeviceBuffer<T> a, w, bias, out;
        if (cuda_detail::CopyTensorToDevice(v.a, &a) != 0 || cuda_detail::CopyTensorToDevice(v.w, &w) != 0 ||
            (v.bias && cuda_detail::CopyTensorToDevice(v.bias, &bias) != 0) ||
            cuda_detail::AllocateTensorOnDevice(v.out, &out) != 0) return -1;
        d.a = a.get(); d.w = w.get(); d.bias = v.bias ? bias.get() : nullptr; d.out = out.get();
        if (d.w_channel_scales != nullptr) {
            if (scales_.get() == nullptr) return -1;
            d.w_channel_scales = static_cast<const float*>(scales_.get());
        }
        d.workspace = workspace_.get(); d.workspace_bytes = workspace_.bytes();
        // An immutable weight is uploaded by the first call; from the second call on nothing on the stream writes it.
        d.weights_static = weights_resident_ ? 1 : 0;
        void* node_out = nullptr;
        const ShardBindingScope* shard = scratch_ == Scratch::kBuiltIn ? nullptr : BindShard(&d, 1, &node_out);
        const int rc = scratch_ == Scratch::kBuiltIn ? fth_b200_fp8_linear_noalloc(&d, cuda_detail::InferenceStream())
                                                     : fth_b200_fp8_linear(&d, cuda_detail::InferenceStream());
        if (rc != FTH_B200_OK || FinishShard(shard, d, node_out, 1, cuda_detail::InferenceStream()) != 0) return -1;
        weights_resident_ = v.w->is_immutable();
        return cuda_detail::CopyDeviceToTensor(&out, v.out);  // a no-op under deferred host sync
    }

   private:
    // Where split-K partial sums go.  Within the node's budget: a buffer this kernel allocates in Prepare().  Beyond it
    // (a plan built with workspace limit 0): the array inside the library image when the shape fits it, else no scratch
    // at all — the library then picks kernels that need none.
    enum class Scratch { kOwned, kBuiltIn, kNone };
    Scratch ScratchMode(const fth_b200_fp8_linear_desc& probe) const {
        fth_b200_fp8_linear_desc d = probe;
        d.workspace = nullptr; d.workspace_bytes = 0;
        const size_t need = fth_b200_fp8_linear_workspace_bytes(&d);
        if (need <= workspace_limit_) return Scratch::kOwned;
        return need <= fth_b200_noalloc_scratch_bytes() ? Scratch::kBuiltIn : Scratch::kNone;
    }

    bool Describe(fth_b200_fp8_linear_desc* d, LinearView* view = nullptr, const std::vector<float>** channel_scales = nullptr) const {
        LinearView v;
        if (!View(ParamAs<Param>(), &v)) return false;
        int64_t m = 0, k = 0, n = 0;
        if (!LinearShape(v, &m, &k, &n)) return false;
        // FP8 activations, bias and outputs carry one scale per tensor (include/util/types.h:96-101).  The weight may carry
        // one scale per output channel instead.  The reference's FP8 linear kernels read the scalar field only
        // (include/core/tensor.h:105; a non-scalar scheme "needs a kernel that explicitly implements their indexing
        // semantics", types.h:96-98), while its tensor metadata and the .fth files hold the vector already
        // (src/model/model_io.cc:228-246).  Here output channel n takes w_scale = scales[n].
        if (!HasCompatiblePerTensorQuantization(v.a->quantization()) || !HasCompatiblePerTensorQuantization(v.out->quantization())) return false;
        const QuantizationParams& wq = v.w->quantization();
        const bool per_channel = wq.enabled && wq.granularity == QuantizationGranularity::kPerChannel;
        if (per_channel) {
            const int64_t rank = static_cast<int64_t>(v.w->dims().size());
            const int64_t axis = wq.axis < 0 ? wq.axis + rank : wq.axis;
            if (rank != 2 || axis != (v.trans_b ? 0 : 1) || wq.block_size != 0 || wq.scales.size() != static_cast<size_t>(n)) return false;
            for (int32_t z : wq.zero_points) if (z != 0) return false;
            for (float sc : wq.scales) if (!(sc > 0.0f) || !std::isfinite(sc)) return false;
        } else if (!HasCompatiblePerTensorQuantization(wq)) {
            return false;
        }
        if (channel_scales) *channel_scales = per_channel ? &wq.scales : nullptr;
        const int bias_mode = BiasMode(v.bias, m, n);
        if (bias_mode < 0 || (v.bias && v.bias->data_type() != dtype)) return false;
        *d = fth_b200_fp8_linear_desc{};
        d->dtype = static_cast<int32_t>(dtype);
        d->op = v.op; d->m = m; d->k = k; d->n = n; d->trans_b = v.trans_b ? 1 : 0;
        d->bias_mode = bias_mode;
        d->a_scale = v.a->quantization_scale(); d->w_scale = per_channel ? 1.0f : v.w->quantization_scale();
        if (per_channel) d->w_channel_scales = static_cast<const float*>(kProbe);  // compute() points it at the uploaded copy
        d->bias_scale = v.bias ? v.bias->quantization_scale() : 1.0f;
        d->out_scale = v.out->quantization_scale();
        d->alpha = v.alpha; d->beta = v.beta;
        if (view) *view = v;
        return true;
    }

    DeviceScratch workspace_, scales_;
    bool weights_resident_{false};
    size_t workspace_limit_;
    Scratch scratch_{Scratch::kOwned};
};

// ---------------------------------------------------------------------------------------------------------
// INT8 FC, MatMul, Gemm — in front of RunCudaInt8Linear / RunCudaInt8MatMul (src/kernel/cuda/int8.cu:313-368)
// ---------------------------------------------------------------------------------------------------------
template <typename Param>
class Int8LinearKernel final : public B200Kernel {
   public:
    Int8LinearKernel() : workspace_limit_(KernelSelectionScope::WorkspaceLimit()) {}

    Status Supports() const override {
        fth_b200_int8_linear_desc d;
        Int8WeightParams wq;
        LinearView v;
        if (!Describe(&d, &wq, &v)) return Status::Error(StatusCode::kUnsupported, "b200: not a 2-D INT8 linear");
        d.a = kProbe; d.w = static_cast<const int8_t*>(kProbe); d.out = kProbe;
        d.w_scales = static_cast<const float*>(kProbe);
        if (wq.zp_max_abs != 0) d.w_zps = static_cast<const int32_t*>(kProbe);
        if (d.bias_mode != FTH_B200_BIAS_NONE) d.bias = static_cast<const int32_t*>(kProbe);
        // selection and compute() must decide the int32 overflow pre-check on the same numbers
        d.bias_max_abs = BiasMaxAbs(v.bias);
        if (WithinBudget(d)) { d.workspace = kProbe; d.workspace_bytes = static_cast<size_t>(-1); }
        return FromAbi(fth_b200_int8_linear_supported(&d), "INT8 linear");
    }

    // Scales and zero points go to the device once here — the reference uploads them on every call from a
    // temporary host vector, which is why its INT8 kernels cannot be captured (int8.cu:338-367).
    int32_t Prepare() override {
        fth_b200_int8_linear_desc d;
        Int8WeightParams wq;
        LinearView v;
        if (!Describe(&d, &wq, &v)) return -1;
        if (scales_.Upload(wq.scales.data(), wq.scales.size() * sizeof(float)) != 0) return -1;
        has_zps_ = wq.zp_max_abs != 0;
        if (has_zps_ && zps_.Upload(wq.zero_points.data(), wq.zero_points.size() * sizeof(int32_t)) != 0) return -1;
        bias_max_abs_ = BiasMaxAbs(v.bias);  // bias is an immutable INT32 constant produced by the static quantiser
        // An immutable weight keeps its quantisation parameters: compute() need not validate and copy the per-channel
        // vectors again (28672 entries at the largest projections: more host time per call than the kernel takes).
        weight_params_cached_ = v.w->is_immutable();
        cached_w_params_ = static_cast<int64_t>(wq.scales.size());
        cached_zp_max_abs_ = wq.zp_max_abs;
        d.a = kProbe; d.w = static_cast<const int8_t*>(kProbe); d.out = kProbe; d.w_scales = static_cast<const float*>(kProbe);
        weights_resident_ = false;
        if (!WithinBudget(d)) return 0;  // no scratch: the library picks kernels that need none
        return workspace_.Reserve(fth_b200_int8_linear_workspace_bytes(&d), true);
    }

    int32_t compute() override {
        AutoTimer timer("B200::Linear::INT8");
        fth_b200_int8_linear_desc d;
        Int8WeightParams wq;
        LinearView v;
        if (!Describe(&d, &wq, &v, weight_params_cached_) || scales_.get() == nullptr) return -1;
        cuda_detail::DeviceBuffer<int8_t> a, w, out;
        cuda_detail::DeviceBuffer<int32_t> bias;
        if (cuda_detail::CopyTensorToDevice(v.a, &a) != 0 || cuda_detail::CopyTensorToDevice(v.w, &w) != 0 ||
            (v.bias && cuda_detail::CopyTensorToDevice(v.bias, &bias) != 0) ||
            cuda_detail::AllocateTensorOnDevice(v.out, &out) != 0) return -1;
        d.a = a.get(); d.w = w.get(); d.bias = v.bias ? bias.get() : nullptr; d.out = out.get();
        d.w_scales = static_cast<const float*>(scales_.get());
        d.w_zps = has_zps_ ? static_cast<const int32_t*>(zps_.get()) : nullptr;
        d.bias_max_abs = bias_max_abs_;
        d.workspace = workspace_.get(); d.workspace_bytes = workspace_.bytes();
        d.weights_static = weights_resident_ ? 1 : 0;
        void* node_out = nullptr;
        const ShardBindingScope* shard = BindShard(&d, 1, &node_out);
        if (fth_b200_int8_linear(&d, cuda_detail::InferenceStream()) != FTH_B200_OK ||
            FinishShard(shard, d, node_out, 1, cuda_detail::InferenceStream()) != 0) return -1;
        weights_resident_ = v.w->is_immutable();
        return cuda_detail::CopyDeviceToTensor(&out, v.out);
    }

   private:
    bool WithinBudget(const fth_b200_int8_linear_desc& probe) const {
        fth_b200_int8_linear_desc d = probe;
        d.workspace = nullptr; d.workspace_bytes = 0;
        return fth_b200_int8_linear_workspace_bytes(&d) <= workspace_limit_;
    }

    bool Describe(fth_b200_int8_linear_desc* d, Int8WeightParams* wq, LinearView* view = nullptr, bool weight_cached = false) const {
        LinearView v;
        if (!View(ParamAs<Param>(), &v)) return false;
        int64_t m = 0, k = 0, n = 0;
        if (!LinearShape(v, &m, &k, &n)) return false;
        Int8WeightParams aq, oq;
        if (!ReadInt8Quantization(v.a, false, -1, 1, &aq) || !ReadInt8Quantization(v.out, false, -1, 1, &oq)) return false;
        if (weight_cached && (cached_w_params_ == 1 || cached_w_params_ == n)) {
            wq->scales.assign(static_cast<size_t>(cached_w_params_ == 1 ? 1 : 0), 0.0f);  // only the count and the bound are used
            wq->zp_max_abs = cached_zp_max_abs_;
        } else if (!ReadInt8Quantization(v.w, true, v.trans_b ? 0 : 1, n, wq)) {
            return false;
        }
        const int bias_mode = BiasMode(v.bias, m, n);
        if (bias_mode < 0 || (v.bias && v.bias->data_type() != DataType::INT32)) return false;
        *d = fth_b200_int8_linear_desc{};
        d->op = v.op; d->m = m; d->k = k; d->n = n; d->trans_b = v.trans_b ? 1 : 0;
        d->bias_mode = bias_mode;
        d->a_scale = aq.scales[0]; d->a_zp = aq.zero_points[0];
        d->w_params = weight_cached ? cached_w_params_ : static_cast<int64_t>(wq->scales.size());
        d->w_zp_max_abs = wq->zp_max_abs;
        d->out_scale = oq.scales[0]; d->out_zp = oq.zero_points[0];
        d->alpha = v.alpha; d->beta = v.beta;
        d->bias_max_abs = bias_max_abs_;
        if (view) *view = v;
        return true;
    }

    DeviceScratch scales_, zps_, workspace_;
    bool weights_resident_{false};
    bool has_zps_{false};
    bool weight_params_cached_{false};
    int64_t cached_w_params_{0};
    int32_t cached_zp_max_abs_{0};
    int64_t bias_max_abs_{0};
    size_t workspace_limit_;
};

// ---------------------------------------------------------------------------------------------------------
// INT8 Conv2D — in front of RunCudaInt8Conv2D (src/kernel/cuda/int8.cu:370-506).  NCHW only; other layouts
// stay on the reference candidate.
// ---------------------------------------------------------------------------------------------------------
class Int8Conv2dKernel final : public B200Kernel {
   public:
    Status Supports() const override {
        fth_b200_int8_conv2d_desc d;
        Int8WeightParams wq;
        if (!Describe(&d, &wq)) return Status::Error(StatusCode::kUnsupported, "b200: not an NCHW INT8 Conv2D");
        d.x = static_cast<const int8_t*>(kProbe); d.w = d.x; d.out = static_cast<int8_t*>(kProbe);
        d.w_scales = static_cast<const float*>(kProbe);
        if (wq.zp_max_abs != 0) d.w_zps = static_cast<const int32_t*>(kProbe);
        d.workspace = kProbe; d.workspace_bytes = static_cast<size_t>(-1);
        return FromAbi(fth_b200_int8_conv2d_supported(&d), "INT8 Conv2D");
    }

    int32_t Prepare() override {
        fth_b200_int8_conv2d_desc d;
        Int8WeightParams wq;
        if (!Describe(&d, &wq)) return -1;
        if (scales_.Upload(wq.scales.data(), wq.scales.size() * sizeof(float)) != 0) return -1;
        has_zps_ = wq.zp_max_abs != 0;
        if (has_zps_ && zps_.Upload(wq.zero_points.data(), wq.zero_points.size() * sizeof(int32_t)) != 0) return -1;
        auto* p = ParamAs<operators::Conv2dParam>();
        bias_max_abs_ = 0;
        if (p->bias) {
            const int32_t* b = p->bias->data<int32_t>();
            for (int64_t i = 0; i < p->bias->numel(); ++i) bias_max_abs_ = std::max<int64_t>(bias_max_abs_, std::llabs(static_cast<long long>(b[i])));
        }
        d.x = static_cast<const int8_t*>(kProbe); d.w = d.x; d.out = static_cast<int8_t*>(kProbe);
        d.w_scales = static_cast<const float*>(kProbe);
        packed_ = false;
        // an immutable weight is packed once per process and device, not once per session
        shared_packed_.reset();
        void* w_device = nullptr;
        if (p->w->is_immutable() && AcquireIn(p->w.get(), &w_device) == 0) {
            fth_b200_int8_conv2d_desc pack = d;
            pack.w = static_cast<const int8_t*>(w_device);
            shared_packed_ = PackedConvWeightCache::Acquire(p->w.get(), pack);
        }
        if (shared_packed_) d.packed_w = static_cast<const int8_t*>(shared_packed_->get());
        return workspace_.Reserve(fth_b200_int8_conv2d_workspace_bytes(&d), true);
    }

    int32_t compute() override {
        AutoTimer timer("B200::Conv2D::INT8");
        fth_b200_int8_conv2d_desc d;
        Int8WeightParams wq;
        if (!Describe(&d, &wq) || scales_.get() == nullptr) return -1;
        auto* p = ParamAs<operators::Conv2dParam>();
        cuda_detail::DeviceBuffer<int8_t> x, w, out;
        cuda_detail::DeviceBuffer<int32_t> bias;
        if (cuda_detail::CopyTensorToDevice(p->input.get(), &x) != 0 || cuda_detail::CopyTensorToDevice(p->w.get(), &w) != 0 ||
            (p->bias && cuda_detail::CopyTensorToDevice(p->bias.get(), &bias) != 0) ||
            cuda_detail::AllocateTensorOnDevice(p->out.get(), &out) != 0) return -1;
        d.x = x.get(); d.w = w.get(); d.bias = p->bias ? bias.get() : nullptr; d.out = out.get();
        d.w_scales = static_cast<const float*>(scales_.get());
        d.w_zps = has_zps_ ? static_cast<const int32_t*>(zps_.get()) : nullptr;
        d.bias_max_abs = bias_max_abs_;
        d.workspace = workspace_.get(); d.workspace_bytes = workspace_.bytes();
        d.weights_packed = packed_ ? 1 : 0;
        d.packed_w = shared_packed_ ? static_cast<const int8_t*>(shared_packed_->get()) : nullptr;
        if (fth_b200_int8_conv2d(&d, cuda_detail::InferenceStream()) != FTH_B200_OK) return -1;
        packed_ = p->w->is_immutable();  // without a shared packed copy: repacked once per session
        return cuda_detail::CopyDeviceToTensor(&out, p->out.get());
    }

   private:
    bool Describe(fth_b200_int8_conv2d_desc* d, Int8WeightParams* wq) const {
        auto* p = ParamAs<operators::Conv2dParam>();
        if (!p || !p->input || !p->w || !p->out) return false;
        if (p->input->layout() == DataLayout::NHWC || p->out->layout() == DataLayout::NHWC) return false;
        const auto& xd = p->input->dims().data();
        const auto& wd = p->w->dims().data();
        if (xd.size() != 4 || wd.size() != 4 || p->out->dims().size() != 4) return false;
        Int8WeightParams xq, oq;
        if (!ReadInt8Quantization(p->input.get(), false, -1, 1, &xq) || !ReadInt8Quantization(p->w.get(), true, 0, wd[0], wq) ||
            !ReadInt8Quantization(p->out.get(), false, -1, 1, &oq)) return false;
        if (p->bias && (p->bias->data_type() != DataType::INT32 || p->bias->numel() != wd[0])) return false;
        *d = fth_b200_int8_conv2d_desc{};
        d->batch = xd[0]; d->ic = xd[1]; d->ih = xd[2]; d->iw = xd[3]; d->oc = wd[0]; d->kh = wd[2]; d->kw = wd[3];
        d->stride_h = p->stride_h; d->stride_w = p->stride_w; d->pad_h = p->pad_h; d->pad_w = p->pad_w;
        d->dilation_h = p->dilation_h; d->dilation_w = p->dilation_w; d->group = p->group;
        d->x_scale = xq.scales[0]; d->x_zp = xq.zero_points[0];
        d->w_params = static_cast<int64_t>(wq->scales.size()); d->w_zp_max_abs = wq->zp_max_abs;
        d->out_scale = oq.scales[0]; d->out_zp = oq.zero_points[0];
        d->bias_max_abs = bias_max_abs_;
        return true;
    }

    DeviceScratch scales_, zps_, workspace_;
    std::shared_ptr<DeviceScratch> shared_packed_;
    bool has_zps_{false}, packed_{false};
    int64_t bias_max_abs_{0};
};

// ---------------------------------------------------------------------------------------------------------
// Cast among FP32 / FP16 / BF16 / FP8 — in front of CastFloatingKernelCuda (src/kernel/cuda/cast.cu:54-93)
// ---------------------------------------------------------------------------------------------------------
class CastKernelB200 final : public B200Kernel {
   public:
    static bool Floating(DataType t) {
        return t == DataType::FP32 || t == DataType::FP16 || t == DataType::BF16 || t == DataType::FP8E4M3 || t == DataType::FP8E5M2;
    }
    Status Supports() const override {
        auto* p = ParamAs<operators::CastParam>();
        if (!p || !p->input || !p->out || !Floating(p->input->data_type()) || !Floating(p->to))
            return Status::Error(StatusCode::kUnsupported, "b200: Cast between non-floating types");
        return Status::Ok();
    }
    int32_t compute() override {
        AutoTimer timer("B200::Cast");
        auto* p = ParamAs<operators::CastParam>();
        if (!p || !p->input || !p->out || p->out->dims().data() != p->input->dims().data()) return -1;
        void* in = nullptr; void* out = nullptr;
        const size_t in_bytes = static_cast<size_t>(p->input->numel()) * DataTypeBytes(p->input->data_type());
        const size_t out_bytes = static_cast<size_t>(p->input->numel()) * DataTypeBytes(p->to);
        if (cuda_detail::AcquireTensorDevice(p->input.get(), in_bytes, p->input->raw_data(), &in) != 0) return -1;
        p->out->set_data_type(p->to);
        if (cuda_detail::AcquireOutputTensorDevice(p->out.get(), out_bytes, &out) != 0) return -1;
        if (fth_b200_cast(static_cast<int32_t>(p->input->data_type()), in, p->input->quantization_scale(), static_cast<int32_t>(p->to),
                          out, p->out->quantization_scale(), p->input->numel(), cuda_detail::InferenceStream()) != FTH_B200_OK) return -1;
        if (cuda_detail::DeferredHostSyncEnabled()) return 0;
        return cuda_detail::SyncTensorToHost(p->out.get(), out_bytes, p->out->raw_data());
    }
};

// ---------------------------------------------------------------------------------------------------------
// QuantizeLinear / DequantizeLinear — the reference registers COMMON kernels only
// (src/kernel/common/quantize_linear.cc:24-42, dequantize_linear.cc:25-36), so a CUDA plan under
// kRequireRequested cannot be built without these two candidates.
// ---------------------------------------------------------------------------------------------------------
}  // namespace b200
}  // namespace kernel
}  // namespace feather

#include "src/kernel/common/quantize_linear_utils.h"

namespace feather {
namespace kernel {
namespace b200 {

template <typename Param>
class QdqBase : public B200Kernel {
   protected:
    // Reads the (constant) scale / zero-point tensors once and uploads them as float / int32 arrays.
    int32_t PrepareParams(Param* p) {
        if (!p || !p->input || !p->scale || !p->zero_point || !p->out) return -1;
        if (!quantize_linear_detail::BuildQuantizationParams(*p->input, *p->scale, *p->zero_point, p->axis, &quantization_)) return -1;
        std::vector<int32_t> zps = quantization_.zero_points;
        if (zps.size() == 1 && quantization_.scales.size() > 1) zps.assign(quantization_.scales.size(), zps[0]);
        if (scales_.Upload(quantization_.scales.data(), quantization_.scales.size() * sizeof(float)) != 0) return -1;
        return zps_.Upload(zps.data(), zps.size() * sizeof(int32_t));
    }
    // [outer, channels, inner] view of a tensor whose parameters run along quantization.axis (per tensor: one channel).
    template <typename Dims>
    static void ChannelExtents(const Dims& dims, const QuantizationParams& q, int64_t* channels, int64_t* inner) {
        *channels = 1;
        *inner = 1;
        if (q.granularity != QuantizationGranularity::kPerChannel || dims.empty()) { *channels = dims.empty() ? 1 : dims.back(); return; }
        const size_t axis = static_cast<size_t>(q.axis < 0 ? q.axis + static_cast<int64_t>(dims.size()) : q.axis);
        *channels = dims[axis];
        for (size_t i = axis + 1; i < dims.size(); ++i) *inner *= dims[i];
    }
    QuantizationParams quantization_;
    DeviceScratch scales_, zps_;
};

class QuantizeLinearKernelB200 final : public QdqBase<operators::QuantizeLinearParam> {
   public:
    Status Supports() const override {
        auto* p = ParamAs<operators::QuantizeLinearParam>();
        QuantizationParams q;
        if (!p || !p->input || !p->scale || !p->zero_point ||
            !quantize_linear_detail::BuildQuantizationParams(*p->input, *p->scale, *p->zero_point, p->axis, &q))
            return Status::Error(StatusCode::kInvalidArgument, "b200: bad QuantizeLinear parameters");
        return Status::Ok();  // per tensor, or per channel on any axis
    }
    int32_t Prepare() override { return PrepareParams(ParamAs<operators::QuantizeLinearParam>()) == 0 ? 0 : -1; }
    int32_t compute() override {
        AutoTimer timer("B200::QuantizeLinear");
        auto* p = ParamAs<operators::QuantizeLinearParam>();
        if (!p || scales_.get() == nullptr) return -1;
        const int64_t count = p->input->numel();
        int64_t channels = 1, inner = 1;
        ChannelExtents(p->input->dims().data(), quantization_, &channels, &inner);
        void* in = nullptr; void* out = nullptr;
        if (cuda_detail::AcquireTensorDevice(p->input.get(), static_cast<size_t>(count) * DataTypeBytes(p->input->data_type()),
                                             p->input->raw_data(), &in) != 0) return -1;
        p->out->Resize(p->input->dims().data());
        p->out->set_data_type(DataType::INT8);
        p->out->set_quantization(quantization_);  // the output's parameters are set at run time (quantize_linear_utils.h:273-276)
        if (cuda_detail::AcquireOutputTensorDevice(p->out.get(), static_cast<size_t>(count), &out) != 0) return -1;
        if (fth_b200_quantize_linear_axis(static_cast<int32_t>(p->input->data_type()), in, static_cast<const float*>(scales_.get()),
                                          static_cast<const int32_t*>(zps_.get()), static_cast<int64_t>(quantization_.scales.size()),
                                          static_cast<int8_t*>(out), count / (channels * inner), channels, inner,
                                          cuda_detail::InferenceStream()) != FTH_B200_OK) return -1;
        if (cuda_detail::DeferredHostSyncEnabled()) return 0;
        return cuda_detail::SyncTensorToHost(p->out.get(), static_cast<size_t>(count), p->out->raw_data());
    }
};

class DequantizeLinearKernelB200 final : public QdqBase<operators::DequantizeLinearParam> {
   public:
    Status Supports() const override {
        auto* p = ParamAs<operators::DequantizeLinearParam>();
        QuantizationParams q;
        if (!p || !p->input || !p->scale || !p->zero_point || p->input->data_type() != DataType::INT8 ||
            (p->to != DataType::FP32 && p->to != DataType::FP16 && p->to != DataType::BF16) ||
            !quantize_linear_detail::BuildQuantizationParams(*p->input, *p->scale, *p->zero_point, p->axis, &q))
            return Status::Error(StatusCode::kInvalidArgument, "b200: bad DequantizeLinear parameters");
        return Status::Ok();  // per tensor, or per channel on any axis
    }
    int32_t Prepare() override { return PrepareParams(ParamAs<operators::DequantizeLinearParam>()) == 0 ? 0 : -1; }
    int32_t compute() override {
        AutoTimer timer("B200::DequantizeLinear");
        auto* p = ParamAs<operators::DequantizeLinearParam>();
        if (!p || scales_.get() == nullptr) return -1;
        const int64_t count = p->input->numel();
        int64_t channels = 1, inner = 1;
        ChannelExtents(p->input->dims().data(), quantization_, &channels, &inner);
        const size_t out_bytes = static_cast<size_t>(count) * DataTypeBytes(p->to);
        void* in = nullptr; void* out = nullptr;
        if (cuda_detail::AcquireTensorDevice(p->input.get(), static_cast<size_t>(count), p->input->raw_data(), &in) != 0) return -1;
        p->out->Resize(p->input->dims().data());
        p->out->set_data_type(p->to);
        p->out->set_quantization(QuantizationParams{});
        if (cuda_detail::AcquireOutputTensorDevice(p->out.get(), out_bytes, &out) != 0) return -1;
        if (fth_b200_dequantize_linear_axis(static_cast<const int8_t*>(in), static_cast<const float*>(scales_.get()),
                                            static_cast<const int32_t*>(zps_.get()), static_cast<int64_t>(quantization_.scales.size()), out,
                                            static_cast<int32_t>(p->to), count / (channels * inner), channels, inner,
                                            cuda_detail::InferenceStream()) != FTH_B200_OK) return -1;
        if (cuda_detail::DeferredHostSyncEnabled()) return 0;
        return cuda_detail::SyncTensorToHost(p->out.get(), out_bytes, p->out->raw_data());
    }
};

// ---------------------------------------------------------------------------------------------------------
// The operators between the projections of a decoder block — in front of the reference's CUDA kernels
// (src/kernel/cuda/qwen_rms_norm.cu, add.cu, mul.cu, silu.cu), so that a Qwen plan keeps the whole block on the
// stream with this backend's launch behaviour (programmatic dependents, no per-call allocation).
// ---------------------------------------------------------------------------------------------------------
namespace {
bool PlainFloat(DataType t) { return t == DataType::FP32 || t == DataType::BF16; }
bool AnyFloat(DataType t) { return t == DataType::FP32 || t == DataType::BF16 || t == DataType::FP16; }

}  // namespace

class QwenRmsNormKernelB200 final : public B200Kernel {
   public:
    Status Supports() const override {
        auto* p = ParamAs<operators::QwenRmsNormParam>();
        if (!p || !p->input || !p->weight || !p->epsilon || !p->out) return Status::Error(StatusCode::kInvalidArgument, "b200: bad QwenRmsNorm parameters");
        if (!PlainFloat(p->input->data_type()) || !PlainFloat(p->weight->data_type()) || !PlainFloat(p->out->data_type()))
            return Status::Error(StatusCode::kUnsupported, "b200: QwenRmsNorm takes FP32 / BF16 tensors");
        return Status::Ok();
    }
    int32_t compute() override {
        AutoTimer timer("B200::QwenRmsNorm");
        auto* p = ParamAs<operators::QwenRmsNormParam>();
        if (!p || !p->input || !p->weight || !p->epsilon || !p->out || p->input->dims().empty() || p->epsilon->numel() != 1) return -1;
        const int64_t hidden = p->input->dims().data().back();
        if (hidden <= 0 || p->input->numel() % hidden != 0 || p->weight->numel() != hidden || p->out->numel() != p->input->numel()) return -1;
        float epsilon = 0.0f;  // a plan constant, read on the host as the reference's CUDA kernel does (qwen_rms_norm.cu:30-45)
        if (p->epsilon->data_type() == DataType::FP32) epsilon = p->epsilon->data<float>()[0];
        else if (p->epsilon->data_type() == DataType::BF16) epsilon = BFloat16ToFloat(p->epsilon->data<BFloat16>()[0].bits);
        else return -1;
        void* x = nullptr; void* w = nullptr; void* out = nullptr;
        const size_t out_bytes = static_cast<size_t>(p->out->numel()) * DataTypeBytes(p->out->data_type());
        if (AcquireIn(p->input.get(), &x) != 0 || AcquireIn(p->weight.get(), &w) != 0 ||
            cuda_detail::AcquireOutputTensorDevice(p->out.get(), out_bytes, &out) != 0) return -1;
        if (fth_b200_qwen_rms_norm(static_cast<int32_t>(p->input->data_type()), x, static_cast<int32_t>(p->weight->data_type()), w, p->weight_offset,
                                   epsilon, static_cast<int32_t>(p->out->data_type()), out, p->input->numel() / hidden, hidden,
                                   cuda_detail::InferenceStream()) != FTH_B200_OK) return -1;
        return FinishOut(p->out.get(), out_bytes);
    }
};

// Add / Mul with equal shapes, or a trailing-row rhs broadcast over lhs; other broadcasts stay on the reference kernel.
template <int kOp>
class BinaryKernelB200 final : public B200Kernel {
   public:
    Status Supports() const override {
        int64_t rhs_count = 0;
        return Shape(&rhs_count) ? Status::Ok() : Status::Error(StatusCode::kUnsupported, "b200: element-wise op with a general broadcast");
    }
    int32_t compute() override {
        AutoTimer timer(kOp == FTH_B200_BINARY_ADD ? "B200::Add" : "B200::Mul");
        auto* p = ParamAs<operators::BinaryParam>();
        int64_t rhs_count = 0;
        if (!Shape(&rhs_count)) return -1;
        const DataType dt = p->lhs->data_type();
        void* lhs = nullptr; void* rhs = nullptr; void* out = nullptr;
        p->out->set_data_type(dt);
        const size_t out_bytes = static_cast<size_t>(p->lhs->numel()) * DataTypeBytes(dt);
        if (AcquireIn(p->lhs.get(), &lhs) != 0 || AcquireIn(p->rhs.get(), &rhs) != 0 ||
            cuda_detail::AcquireOutputTensorDevice(p->out.get(), out_bytes, &out) != 0) return -1;
        if (fth_b200_binary(kOp, static_cast<int32_t>(dt), lhs, rhs, out, p->lhs->numel(), rhs_count, cuda_detail::InferenceStream()) != FTH_B200_OK) return -1;
        return FinishOut(p->out.get(), out_bytes);
    }

   private:
    bool Shape(int64_t* rhs_count) const {
        auto* p = ParamAs<operators::BinaryParam>();
        if (!p || !p->lhs || !p->rhs || !p->out || !AnyFloat(p->lhs->data_type()) || p->rhs->data_type() != p->lhs->data_type()) return false;
        const auto& l = p->lhs->dims().data();
        const auto& r = p->rhs->dims().data();
        if (l.empty() || p->lhs->numel() <= 0 || p->out->numel() != p->lhs->numel()) return false;
        if (l == r) { *rhs_count = p->lhs->numel(); return true; }
        // rhs = the trailing dimensions of lhs (leading 1s allowed): one row repeated over the leading dimensions
        size_t skip = 0;
        while (skip < r.size() && r[skip] == 1) ++skip;
        const size_t tail = r.size() - skip;
        if (tail == 0 || tail > l.size()) return false;
        for (size_t i = 0; i < tail; ++i)
            if (r[skip + i] != l[l.size() - tail + i]) return false;
        *rhs_count = p->rhs->numel();
        return true;
    }
};

class SiluKernelB200 final : public B200Kernel {
   public:
    Status Supports() const override {
        auto* p = ParamAs<operators::UnaryParam>();
        if (!p || !p->input || !p->out || !AnyFloat(p->input->data_type())) return Status::Error(StatusCode::kUnsupported, "b200: SiLU takes FP32 / FP16 / BF16");
        return Status::Ok();
    }
    int32_t compute() override {
        AutoTimer timer("B200::SiLU");
        auto* p = ParamAs<operators::UnaryParam>();
        if (!p || !p->input || !p->out || p->input->numel() <= 0) return -1;
        const DataType dt = p->input->data_type();
        void* x = nullptr; void* out = nullptr;
        p->out->set_data_type(dt);
        const size_t out_bytes = static_cast<size_t>(p->input->numel()) * DataTypeBytes(dt);
        if (AcquireIn(p->input.get(), &x) != 0 || cuda_detail::AcquireOutputTensorDevice(p->out.get(), out_bytes, &out) != 0) return -1;
        if (fth_b200_silu(static_cast<int32_t>(dt), x, out, p->input->numel(), cuda_detail::InferenceStream()) != FTH_B200_OK) return -1;
        return FinishOut(p->out.get(), out_bytes);
    }
};

// ---------------------------------------------------------------------------------------------------------
// Fused FP8 lm-head projection + greedy selection.  The reference has this node for FP8 on x86 only
// (QwenGemmArgmaxKernel<X86, FP8*>, src/kernel/x86/linear_fp8.cc:733-1004); its CUDA candidates are BF16
// (src/kernel/cuda/register_all.cu:139), so an FP8 Qwen plan cannot keep the node on the GPU without this one.
// ---------------------------------------------------------------------------------------------------------
template <DataType dtype>
class QwenGemmArgmaxKernelB200 final : public B200Kernel {
   public:
    Status Supports() const override {
        fth_b200_fp8_linear_desc d;
        if (!Describe(&d)) return Status::Error(StatusCode::kUnsupported, "b200: not an FP8 [1,K] x [N,K] lm-head");
        d.a = d.w = d.out = kProbe;
        d.workspace = kProbe; d.workspace_bytes = static_cast<size_t>(-1);
        return FromAbi(fth_b200_fp8_linear_supported(&d), "FP8 lm-head selection");
    }
    int32_t Prepare() override {
        fth_b200_fp8_linear_desc d;
        if (!Describe(&d)) return -1;
        d.a = d.w = d.out = kProbe;
        if (logits_.Reserve(static_cast<size_t>(d.n), false) != 0) return -1;  // the code row the selection runs over
        return workspace_.Reserve(fth_b200_fp8_linear_workspace_bytes(&d), true);
    }
    int32_t compute() override {
        AutoTimer timer("B200::QwenGemmArgmax::FP8");
        using T = cuda_detail::StorageT<dtype>;
        auto* p = ParamAs<operators::QwenGemmArgmaxParam>();
        fth_b200_fp8_linear_desc d;
        if (!Describe(&d) || logits_.get() == nullptr) return -1;
        cuda_detail::DeviceBuffer<T> a, b;
        void* token = nullptr;
        p->out->set_data_type(DataType::INT64);
        if (cuda_detail::CopyTensorToDevice(p->a.get(), &a) != 0 || cuda_detail::CopyTensorToDevice(p->b.get(), &b) != 0 ||
            cuda_detail::AcquireOutputTensorDevice(p->out.get(), sizeof(int64_t), &token) != 0) return -1;
        d.a = a.get(); d.w = b.get(); d.out = logits_.get();
        d.workspace = workspace_.get(); d.workspace_bytes = workspace_.bytes();
        d.weights_static = weights_resident_ ? 1 : 0;
        if (fth_b200_fp8_lm_head_argmax(&d, static_cast<int64_t*>(token), cuda_detail::InferenceStream()) != FTH_B200_OK) return -1;
        weights_resident_ = p->b->is_immutable();
        return FinishOut(p->out.get(), sizeof(int64_t));
    }

   private:
    bool Describe(fth_b200_fp8_linear_desc* d) const {
        auto* p = ParamAs<operators::QwenGemmArgmaxParam>();
        if (!p || !p->a || !p->b || !p->out || p->a->data_type() != dtype || p->b->data_type() != dtype) return false;
        if (p->a->dims().size() < 2 || p->b->dims().size() != 2) return false;
        if (!HasCompatiblePerTensorQuantization(p->a->quantization()) || !HasCompatiblePerTensorQuantization(p->b->quantization())) return false;
        const int64_t k = p->a->dims().data().back();
        const int64_t n = p->b->dims().data()[0];
        if (k <= 0 || n <= 0 || p->a->numel() != k || p->b->dims().data()[1] != k || p->out->numel() != 1) return false;
        *d = fth_b200_fp8_linear_desc{};
        d->dtype = static_cast<int32_t>(dtype);
        d->op = FTH_B200_OP_GEMM; d->m = 1; d->k = k; d->n = n; d->trans_b = 1;
        d->a_scale = p->a->quantization_scale(); d->w_scale = p->b->quantization_scale();
        d->bias_scale = 1.0f; d->out_scale = p->output_scale;
        d->alpha = 1.0f; d->beta = 1.0f;
        return true;
    }
    DeviceScratch logits_, workspace_;
    bool weights_resident_{false};
};

// ---------------------------------------------------------------------------------------------------------
// Registration.  Call once after the dispatcher exists (KernelDispatcher::instance() registers the built-in
// kernels lazily, include/core/kernel.h:212-225); the environment variable FEATHER_DISABLE_B200=1 leaves the
// reference candidates alone, so A/B runs against the reference CUDA kernels need one switch.
// ---------------------------------------------------------------------------------------------------------
bool RegisterB200Kernels() {
    const char* off = std::getenv("FEATHER_DISABLE_B200");
    if (off != nullptr && off[0] == '1') return false;
    AddCandidate<Fp8LinearKernel<DataType::FP8E4M3, operators::FcParam>>(DataType::FP8E4M3, "FC", "b200.fp8.fc");
    AddCandidate<Fp8LinearKernel<DataType::FP8E4M3, operators::MatMulParam>>(DataType::FP8E4M3, "MatMul", "b200.fp8.matmul");
    AddCandidate<Fp8LinearKernel<DataType::FP8E4M3, operators::GemmParam>>(DataType::FP8E4M3, "Gemm", "b200.fp8.gemm");
    AddCandidate<Fp8LinearKernel<DataType::FP8E5M2, operators::FcParam>>(DataType::FP8E5M2, "FC", "b200.fp8.fc");
    AddCandidate<Fp8LinearKernel<DataType::FP8E5M2, operators::MatMulParam>>(DataType::FP8E5M2, "MatMul", "b200.fp8.matmul");
    AddCandidate<Fp8LinearKernel<DataType::FP8E5M2, operators::GemmParam>>(DataType::FP8E5M2, "Gemm", "b200.fp8.gemm");
    AddCandidate<Int8LinearKernel<operators::FcParam>>(DataType::INT8, "FC", "b200.int8.fc");
    AddCandidate<Int8LinearKernel<operators::MatMulParam>>(DataType::INT8, "MatMul", "b200.int8.matmul");
    AddCandidate<Int8LinearKernel<operators::GemmParam>>(DataType::INT8, "Gemm", "b200.int8.gemm");
    AddCandidate<Int8Conv2dKernel>(DataType::INT8, "Conv2D", "b200.int8.conv2d");
    for (DataType t : {DataType::FP32, DataType::FP16, DataType::BF16}) AddCandidate<QuantizeLinearKernelB200>(t, "QuantizeLinear", "b200.quantize_linear");
    AddCandidate<DequantizeLinearKernelB200>(DataType::INT8, "DequantizeLinear", "b200.dequantize_linear");
    for (DataType t : {DataType::FP32, DataType::FP16, DataType::BF16, DataType::FP8E4M3, DataType::FP8E5M2}) AddCandidate<CastKernelB200>(t, "Cast", "b200.cast");
    for (DataType t : {DataType::FP32, DataType::BF16}) AddCandidate<QwenRmsNormKernelB200>(t, "QwenRmsNorm", "b200.qwen_rms_norm");
    for (DataType t : {DataType::FP32, DataType::FP16, DataType::BF16}) {
        AddCandidate<BinaryKernelB200<FTH_B200_BINARY_ADD>>(t, "Add", "b200.add");
        AddCandidate<BinaryKernelB200<FTH_B200_BINARY_MUL>>(t, "Mul", "b200.mul");
        AddCandidate<SiluKernelB200>(t, "SiLU", "b200.silu");
    }
    AddCandidate<QwenGemmArgmaxKernelB200<DataType::FP8E4M3>>(DataType::FP8E4M3, "QwenGemmArgmax", "b200.fp8.qwen_gemm_argmax");
    AddCandidate<QwenGemmArgmaxKernelB200<DataType::FP8E5M2>>(DataType::FP8E5M2, "QwenGemmArgmax", "b200.fp8.qwen_gemm_argmax");
    return true;
}

}  // namespace b200
}  // namespace kernel
}  // namespace feather
