// Host-buffer plans: Prepare()/compute() for one node with an immutable weight.
//
// create  = what KernelBase::Prepare() does once per session: upload weight, scales, zero points, bias and
//           tables, size the workspace.  Allocates and synchronises.
// run     = what compute() does in the reference CUDA kernels (src/kernel/cuda/matmul.cu:230-272):
//           activation host→device, launch, result device→host, on the caller's stream, then waits.
//           Decode-sized linear plans with page-locked host buffers skip the two copy-engine transfers (4.5 us and
//           6.6 us of a 74 us step, measured): a small kernel reads the activation from the host buffer, overlapped
//           with the next kernel's set-up, and the linear kernels store each output to the host buffer as they do to a
//           replica on another GPU; the two launches are replayed from a graph (one driver call per step).
// launch  = the same launch on device-resident buffers, no copies and no wait.
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"

namespace {

enum class Kind { kFp8Linear, kInt8Linear, kInt8Conv };

struct DeviceBuffer {
    void* ptr{nullptr};
    ~DeviceBuffer() { if (ptr) cudaFree(ptr); }
    int Upload(const void* host, size_t bytes) {
        if (bytes == 0) return FTH_B200_OK;
        if (cudaMalloc(&ptr, bytes) != cudaSuccess) return FTH_B200_ERR_CUDA;
        if (host && cudaMemcpy(ptr, host, bytes, cudaMemcpyHostToDevice) != cudaSuccess) return FTH_B200_ERR_CUDA;
        return FTH_B200_OK;
    }
};

// The address under which the GPU reaches a page-locked host buffer, or null (pageable memory, or not host memory).
void* DeviceViewOfHost(const void* host) {
    cudaPointerAttributes attr = {};
    if (cudaPointerGetAttributes(&attr, host) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return attr.type == cudaMemoryTypeHost ? attr.devicePointer : nullptr;
}

// Host buffer -> device buffer by the SMs (a few KB: one load per thread in flight beats a copy-engine transfer).
__global__ void __launch_bounds__(256) StageInKernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t bytes) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
    const int64_t groups = vec ? bytes / 16 : 0;
    for (int64_t g = t; g < groups; g += stride) reinterpret_cast<uint4*>(dst)[g] = reinterpret_cast<const uint4*>(src)[g];
    for (int64_t i = groups * 16 + t; i < bytes; i += stride) dst[i] = src[i];
}

int LaunchStageIn(const void* src, void* dst, int64_t bytes, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    const int64_t blocks = (bytes / 16 + 255) / 256;
    cfg.gridDim = dim3(static_cast<unsigned>(blocks < 1 ? 1 : blocks > 64 ? 64 : blocks));
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, StageInKernel, static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), bytes) != cudaSuccess)
        return FTH_B200_ERR_CUDA;
    return FTH_B200_OK;
}

size_t ElemBytes(int dtype) {
    switch (dtype) {
        case FTH_B200_FP32: case FTH_B200_INT32: return 4;
        case FTH_B200_BF16: case FTH_B200_FP16: return 2;
        default: return 1;
    }
}

}  // namespace

struct fth_b200_plan {
    Kind kind;
    fth_b200_fp8_linear_desc fp8{};
    fth_b200_int8_linear_desc int8{};
    fth_b200_int8_conv2d_desc conv{};
    DeviceBuffer in, out, w, bias, scales, zps, lut, workspace;
    int64_t in_bytes{0}, out_bytes{0};
    // fth_b200_plan_run on page-locked host buffers replays its two launches (activation in, linear kernel) from a
    // graph: one driver call per step instead of two launches with their descriptor work (8.5 us of host time per
    // linear launch through this ABI, measured, all of it in front of the GPU's first instruction).  Captured on a
    // stream of the plan's own for the pair of host buffers of the last call; another pair is captured again.
    cudaGraphExec_t step_exec{nullptr};
    cudaStream_t capture_stream{nullptr};
    const void* step_in{nullptr};
    void* step_out{nullptr};
    bool step_graph_failed{false};
    int direct_steps{0};  // steps launched kernel by kernel so far (the first one always is)
    ~fth_b200_plan() {
        if (step_exec) cudaGraphExecDestroy(step_exec);
        if (capture_stream) cudaStreamDestroy(capture_stream);
    }
};

#define FTH_TRY(expr) do { const int rc_ = (expr); if (rc_ != FTH_B200_OK) { delete p; return rc_; } } while (0)

extern "C" int fth_b200_plan_create_fp8_linear(const fth_b200_fp8_linear_desc* h, fth_b200_plan** plan) {
    if (!h || !plan || !h->w || h->m <= 0 || h->k <= 0 || h->n <= 0) return FTH_B200_ERR_INVALID;
    auto* p = new (std::nothrow) fth_b200_plan();
    if (!p) return FTH_B200_ERR_INVALID;
    p->kind = Kind::kFp8Linear;
    p->fp8 = *h;
    p->fp8.weights_static = 1;  // uploaded once, synchronously, below; never written again
    const int a_dtype = h->a_dtype ? h->a_dtype : h->dtype;
    const int out_dtype = h->out_dtype ? h->out_dtype : h->dtype;
    const int64_t ldo = h->ldo ? h->ldo : h->n;
    p->in_bytes = h->m * h->k * static_cast<int64_t>(ElemBytes(a_dtype));
    p->out_bytes = h->m * ldo * static_cast<int64_t>(ElemBytes(out_dtype));
    FTH_TRY(p->w.Upload(h->w, static_cast<size_t>(h->k * h->n)));
    FTH_TRY(p->in.Upload(nullptr, static_cast<size_t>(p->in_bytes)));
    FTH_TRY(p->out.Upload(nullptr, static_cast<size_t>(p->out_bytes)));
    if (h->bias_mode != FTH_B200_BIAS_NONE) {
        if (!h->bias) { delete p; return FTH_B200_ERR_INVALID; }
        FTH_TRY(p->bias.Upload(h->bias, static_cast<size_t>(h->bias_mode == FTH_B200_BIAS_VECTOR ? h->n : h->m * h->n)));
    }
    if (h->w_channel_scales) FTH_TRY(p->scales.Upload(h->w_channel_scales, static_cast<size_t>(h->n) * 4));
    p->fp8.w = p->w.ptr; p->fp8.bias = p->bias.ptr; p->fp8.w_channel_scales = static_cast<const float*>(p->scales.ptr);
    p->fp8.a = p->in.ptr; p->fp8.out = p->out.ptr;
    p->fp8.workspace = nullptr; p->fp8.workspace_bytes = 0;
    if (const size_t ws = fth_b200_fp8_linear_workspace_bytes(&p->fp8)) {
        FTH_TRY(p->workspace.Upload(nullptr, ws));
        if (cudaMemset(p->workspace.ptr, 0, ws) != cudaSuccess) { delete p; return FTH_B200_ERR_CUDA; }
        p->fp8.workspace = p->workspace.ptr; p->fp8.workspace_bytes = ws;
    }
    FTH_TRY(fth_b200_fp8_linear_supported(&p->fp8));
    *plan = p;
    return FTH_B200_OK;
}

extern "C" int fth_b200_plan_create_int8_linear(const fth_b200_int8_linear_desc* h, fth_b200_plan** plan) {
    if (!h || !plan || !h->w || !h->w_scales || h->m <= 0 || h->k <= 0 || h->n <= 0) return FTH_B200_ERR_INVALID;
    if (h->w_params != 1 && h->w_params != h->n) return FTH_B200_ERR_INVALID;
    auto* p = new (std::nothrow) fth_b200_plan();
    if (!p) return FTH_B200_ERR_INVALID;
    p->kind = Kind::kInt8Linear;
    p->int8 = *h;
    p->int8.weights_static = 1;
    const int a_dtype = h->a_dtype ? h->a_dtype : FTH_B200_INT8;
    const int out_dtype = h->out_dtype ? h->out_dtype : FTH_B200_INT8;
    const int64_t ldo = h->ldo ? h->ldo : h->n;
    p->in_bytes = h->m * h->k * static_cast<int64_t>(ElemBytes(a_dtype));
    p->out_bytes = h->m * ldo * static_cast<int64_t>(ElemBytes(out_dtype));
    FTH_TRY(p->w.Upload(h->w, static_cast<size_t>(h->k * h->n)));
    FTH_TRY(p->in.Upload(nullptr, static_cast<size_t>(p->in_bytes)));
    FTH_TRY(p->out.Upload(nullptr, static_cast<size_t>(p->out_bytes)));
    FTH_TRY(p->scales.Upload(h->w_scales, static_cast<size_t>(h->w_params) * 4));
    int32_t zp_max = 0;
    if (h->w_zps) {
        for (int64_t i = 0; i < h->w_params; ++i) {
            if (h->w_zps[i] < -128 || h->w_zps[i] > 127) { delete p; return FTH_B200_ERR_INVALID; }
            zp_max = std::max(zp_max, std::abs(h->w_zps[i]));
        }
        if (zp_max != 0) FTH_TRY(p->zps.Upload(h->w_zps, static_cast<size_t>(h->w_params) * 4));
    }
    for (int64_t i = 0; i < h->w_params; ++i)
        if (!(h->w_scales[i] > 0.0f) || !(h->w_scales[i] < INFINITY)) { delete p; return FTH_B200_ERR_INVALID; }
    int64_t bias_max = 0;
    if (h->bias_mode != FTH_B200_BIAS_NONE) {
        if (!h->bias) { delete p; return FTH_B200_ERR_INVALID; }
        const int64_t count = h->bias_mode == FTH_B200_BIAS_VECTOR ? h->n : h->m * h->n;
        for (int64_t i = 0; i < count; ++i) bias_max = std::max<int64_t>(bias_max, std::llabs(static_cast<long long>(h->bias[i])));
        FTH_TRY(p->bias.Upload(h->bias, static_cast<size_t>(count) * 4));
    }
    p->int8.w = static_cast<const int8_t*>(p->w.ptr);
    p->int8.w_scales = static_cast<const float*>(p->scales.ptr);
    p->int8.w_zps = static_cast<const int32_t*>(p->zps.ptr);
    p->int8.bias = static_cast<const int32_t*>(p->bias.ptr);
    p->int8.w_zp_max_abs = zp_max;
    p->int8.bias_max_abs = bias_max;
    p->int8.a = p->in.ptr; p->int8.out = p->out.ptr;
    p->int8.workspace = nullptr; p->int8.workspace_bytes = 0;
    if (const size_t ws = fth_b200_int8_linear_workspace_bytes(&p->int8)) {
        FTH_TRY(p->workspace.Upload(nullptr, ws));
        if (cudaMemset(p->workspace.ptr, 0, ws) != cudaSuccess) { delete p; return FTH_B200_ERR_CUDA; }
        p->int8.workspace = p->workspace.ptr; p->int8.workspace_bytes = ws;
    }
    FTH_TRY(fth_b200_int8_linear_supported(&p->int8));
    *plan = p;
    return FTH_B200_OK;
}

extern "C" int fth_b200_plan_create_int8_conv2d(const fth_b200_int8_conv2d_desc* h, fth_b200_plan** plan) {
    if (!h || !plan || !h->w || !h->w_scales || h->group <= 0 || h->oc <= 0) return FTH_B200_ERR_INVALID;
    if (h->w_params != 1 && h->w_params != h->oc) return FTH_B200_ERR_INVALID;
    // geometry first: everything below divides by these or sizes allocations from them
    if (h->batch <= 0 || h->ic <= 0 || h->ih <= 0 || h->iw <= 0 || h->kh <= 0 || h->kw <= 0) return FTH_B200_ERR_INVALID;
    if (h->stride_h <= 0 || h->stride_w <= 0 || h->dilation_h <= 0 || h->dilation_w <= 0 || h->pad_h < 0 || h->pad_w < 0) return FTH_B200_ERR_INVALID;
    if (h->ic % h->group != 0 || h->oc % h->group != 0) return FTH_B200_ERR_INVALID;
    auto* p = new (std::nothrow) fth_b200_plan();
    if (!p) return FTH_B200_ERR_INVALID;
    p->kind = Kind::kInt8Conv;
    p->conv = *h;
    const int64_t oh = (h->ih + 2 * h->pad_h - h->dilation_h * (h->kh - 1) - 1) / h->stride_h + 1;
    const int64_t ow = (h->iw + 2 * h->pad_w - h->dilation_w * (h->kw - 1) - 1) / h->stride_w + 1;
    if (oh <= 0 || ow <= 0) { delete p; return FTH_B200_ERR_INVALID; }
    p->in_bytes = h->batch * h->ic * h->ih * h->iw;
    p->out_bytes = h->batch * h->oc * oh * ow;
    FTH_TRY(p->w.Upload(h->w, static_cast<size_t>(h->oc * (h->ic / h->group) * h->kh * h->kw)));
    FTH_TRY(p->in.Upload(nullptr, static_cast<size_t>(p->in_bytes)));
    FTH_TRY(p->out.Upload(nullptr, static_cast<size_t>(p->out_bytes)));
    FTH_TRY(p->scales.Upload(h->w_scales, static_cast<size_t>(h->w_params) * 4));
    int32_t zp_max = 0;
    if (h->w_zps) {
        for (int64_t i = 0; i < h->w_params; ++i) zp_max = std::max(zp_max, std::abs(h->w_zps[i]));
        if (zp_max > 128) { delete p; return FTH_B200_ERR_INVALID; }
        if (zp_max != 0) FTH_TRY(p->zps.Upload(h->w_zps, static_cast<size_t>(h->w_params) * 4));
    }
    int64_t bias_max = 0;
    if (h->bias) {
        for (int64_t i = 0; i < h->oc; ++i) bias_max = std::max<int64_t>(bias_max, std::llabs(static_cast<long long>(h->bias[i])));
        FTH_TRY(p->bias.Upload(h->bias, static_cast<size_t>(h->oc) * 4));
    }
    if (h->relu_lut) FTH_TRY(p->lut.Upload(h->relu_lut, 256));
    p->conv.w = static_cast<const int8_t*>(p->w.ptr);
    p->conv.w_scales = static_cast<const float*>(p->scales.ptr);
    p->conv.w_zps = static_cast<const int32_t*>(p->zps.ptr);
    p->conv.bias = static_cast<const int32_t*>(p->bias.ptr);
    p->conv.relu_lut = static_cast<const int8_t*>(p->lut.ptr);
    p->conv.w_zp_max_abs = zp_max;
    p->conv.bias_max_abs = bias_max;
    p->conv.x = static_cast<const int8_t*>(p->in.ptr);
    p->conv.out = static_cast<int8_t*>(p->out.ptr);
    p->conv.workspace = nullptr; p->conv.workspace_bytes = 0; p->conv.weights_packed = 0;
    const size_t ws = fth_b200_int8_conv2d_workspace_bytes(&p->conv);
    if (ws) {
        FTH_TRY(p->workspace.Upload(nullptr, ws));
        p->conv.workspace = p->workspace.ptr;
        p->conv.workspace_bytes = ws;
    }
    FTH_TRY(fth_b200_int8_conv2d_supported(&p->conv));
    *plan = p;
    return FTH_B200_OK;
}

// `host_view`: when not null, the GPU's address of a host buffer that receives every output as well.
// Public form of the staging copy: either side may be a page-locked host buffer (the GPU reaches it under the address
// cudaPointerGetAttributes reports) or device memory.
extern "C" int fth_b200_small_copy(void* dst, const void* src, int64_t bytes, fth_b200_stream_t stream) {
    if (dst == nullptr || src == nullptr || bytes < 0) return FTH_B200_ERR_INVALID;
    if (bytes == 0) return FTH_B200_OK;
    auto view = [](const void* p) -> void* {
        cudaPointerAttributes attr = {};
        if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        if (attr.type == cudaMemoryTypeHost || attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) return attr.devicePointer;
        return nullptr;  // pageable host memory
    };
    void* d = view(dst);
    void* s = view(src);
    if (d == nullptr || s == nullptr) return FTH_B200_ERR_UNSUPPORTED;
    return LaunchStageIn(s, d, bytes, static_cast<cudaStream_t>(stream));
}

static int LaunchPlan(fth_b200_plan* p, const void* device_in, void* device_out, fth_b200_stream_t stream, void* host_view = nullptr) {
    if (!p || !device_in || !device_out) return FTH_B200_ERR_INVALID;
    switch (p->kind) {
        case Kind::kFp8Linear: {
            fth_b200_fp8_linear_desc d = p->fp8;
            d.a = device_in; d.out = device_out;
            if (host_view != nullptr) { d.gather_peers = 1; d.gather_out[0] = host_view; }
            return fth_b200_fp8_linear(&d, stream);
        }
        case Kind::kInt8Linear: {
            fth_b200_int8_linear_desc d = p->int8;
            d.a = device_in; d.out = device_out;
            if (host_view != nullptr) { d.gather_peers = 1; d.gather_out[0] = host_view; }
            return fth_b200_int8_linear(&d, stream);
        }
        case Kind::kInt8Conv: {
            fth_b200_int8_conv2d_desc d = p->conv;
            d.x = static_cast<const int8_t*>(device_in); d.out = static_cast<int8_t*>(device_out);
            const int rc = fth_b200_int8_conv2d(&d, stream);
            if (rc == FTH_B200_OK) p->conv.weights_packed = 1;  // the packed weights stay in the workspace
            return rc;
        }
    }
    return FTH_B200_ERR_INVALID;
}

// Records [activation in, linear kernel with the host buffer as a replica of the output] for this pair of host buffers.
// On any failure the plan keeps launching the two kernels one by one (step_graph_failed).
static void CaptureStep(fth_b200_plan* p, void* in_view, void* out_view) {
    if (p->step_exec) { cudaGraphExecDestroy(p->step_exec); p->step_exec = nullptr; }
    p->step_graph_failed = true;
    if (p->capture_stream == nullptr && cudaStreamCreateWithFlags(&p->capture_stream, cudaStreamNonBlocking) != cudaSuccess) {
        cudaGetLastError();
        return;
    }
    if (cudaStreamBeginCapture(p->capture_stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { cudaGetLastError(); return; }
    const bool recorded = LaunchStageIn(in_view, p->in.ptr, p->in_bytes, p->capture_stream) == FTH_B200_OK &&
                          LaunchPlan(p, p->in.ptr, p->out.ptr, p->capture_stream, out_view) == FTH_B200_OK;
    cudaGraph_t graph = nullptr;
    const bool ended = cudaStreamEndCapture(p->capture_stream, &graph) == cudaSuccess && graph != nullptr;
    if (recorded && ended && cudaGraphInstantiate(&p->step_exec, graph, 0) == cudaSuccess) {
        p->step_in = in_view;
        p->step_out = out_view;
        p->step_graph_failed = false;
    } else {
        cudaGetLastError();
        p->step_exec = nullptr;
    }
    if (graph) cudaGraphDestroy(graph);
}

extern "C" int fth_b200_plan_launch(fth_b200_plan* p, const void* device_in, void* device_out, fth_b200_stream_t stream) {
    return LaunchPlan(p, device_in, device_out, stream);
}

extern "C" int fth_b200_plan_run(fth_b200_plan* p, const void* host_in, void* host_out, fth_b200_stream_t stream_) {
    if (!p || !host_in || !host_out) return FTH_B200_ERR_INVALID;
    auto stream = static_cast<cudaStream_t>(stream_);
    // decode-sized linear plans: the GPU reads and writes page-locked host buffers itself (see the file header)
    const int64_t rows = p->kind == Kind::kFp8Linear ? p->fp8.m : p->kind == Kind::kInt8Linear ? p->int8.m : 0;
    const bool direct = rows >= 1 && rows <= 32 && p->in_bytes <= (64 << 10) && p->out_bytes <= (256 << 10);
    // asked on every call: an address that was page-locked last time may belong to a pageable buffer now
    void* in_view = direct ? DeviceViewOfHost(host_in) : nullptr;
    void* out_view = direct ? DeviceViewOfHost(host_out) : nullptr;
    // (the plan's first step is launched directly: what the library looks up once per device — the status word's address,
    // the kernels' shared-memory opt-in — must not happen inside a capture)
    if (in_view != nullptr && out_view != nullptr && !p->step_graph_failed && p->direct_steps > 0) {
        if (p->step_exec == nullptr || p->step_in != in_view || p->step_out != out_view) CaptureStep(p, in_view, out_view);
        if (p->step_exec != nullptr) {
            if (cudaGraphLaunch(p->step_exec, stream) != cudaSuccess) return FTH_B200_ERR_CUDA;
            return cudaStreamSynchronize(stream) == cudaSuccess ? FTH_B200_OK : FTH_B200_ERR_CUDA;
        }
    }
    if (in_view != nullptr) {
        if (LaunchStageIn(in_view, p->in.ptr, p->in_bytes, stream) != FTH_B200_OK) return FTH_B200_ERR_CUDA;
    } else if (cudaMemcpyAsync(p->in.ptr, host_in, static_cast<size_t>(p->in_bytes), cudaMemcpyHostToDevice, stream) != cudaSuccess) {
        return FTH_B200_ERR_CUDA;
    }
    const int rc = LaunchPlan(p, p->in.ptr, p->out.ptr, stream_, out_view);
    if (rc != FTH_B200_OK) return rc;
    if (out_view == nullptr &&
        cudaMemcpyAsync(host_out, p->out.ptr, static_cast<size_t>(p->out_bytes), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return FTH_B200_ERR_CUDA;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return FTH_B200_ERR_CUDA;
    if (p->direct_steps < 1) p->direct_steps = 1;
    return FTH_B200_OK;
}

extern "C" int64_t fth_b200_plan_input_bytes(const fth_b200_plan* p) { return p ? p->in_bytes : -1; }
extern "C" int64_t fth_b200_plan_output_bytes(const fth_b200_plan* p) { return p ? p->out_bytes : -1; }
extern "C" void fth_b200_plan_destroy(fth_b200_plan* p) { delete p; }
