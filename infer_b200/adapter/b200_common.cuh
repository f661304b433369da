// Shared by the adapter's translation units (b200_candidates.cu: the reference's own operator types; b200_fusion.cu:
// fused operator types and the graph pass that introduces them): status mapping, probe pointers, per-kernel device
// scratch, and readers of the reference's quantisation metadata.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <memory>
#include <mutex>
#include <utility>
#include <string>
#include <vector>

#include "core/kernel.h"
#include "fth_b200.h"
#include "quant/quantization.h"
#include "src/kernel/cuda/kernel_io.cuh"
#include "src/kernel/cuda/runtime.h"

namespace feather {
namespace kernel {
namespace b200 {

constexpr int kPriority = 10;  // reference CUDA kernels register with priority 0 (legacy registerKernel)

// Common base of every kernel of this backend, so that callers (and tests) can tell which candidate the
// dispatcher finally selected.
class B200Kernel : public KernelBase {};
bool IsB200Kernel(const KernelBase* kernel);

inline Status FromAbi(int rc, const char* what) {
    switch (rc) {
        case FTH_B200_OK: return Status::Ok();
        case FTH_B200_ERR_UNSUPPORTED:
        case FTH_B200_ERR_OVERFLOW:  // the reference candidate reports int32 overflow itself (int8.cu:101-110)
            return Status::Error(StatusCode::kUnsupported, std::string("b200 declines ") + what);
        default: return Status::Error(StatusCode::kInvalidArgument, std::string("b200 rejects ") + what);
    }
}

// A fixed, suitably aligned stand-in for device pointers during capability checks (nothing is dereferenced).
inline void* ProbePointer() { return reinterpret_cast<void*>(uintptr_t{1} << 20); }

// Device scratch owned by one kernel instance (one per session node): allocated in Prepare(), never in compute().
class DeviceScratch {
   public:
    DeviceScratch() = default;
    DeviceScratch(const DeviceScratch&) = delete;
    DeviceScratch& operator=(const DeviceScratch&) = delete;
    ~DeviceScratch() { if (ptr_) cudaFree(ptr_); }
    int Reserve(size_t bytes, bool zero) {
        if (bytes <= bytes_) return 0;
        if (ptr_) cudaFree(ptr_);
        ptr_ = nullptr; bytes_ = 0;
        if (cudaMalloc(&ptr_, bytes) != cudaSuccess) return -1;
        bytes_ = bytes;
        return zero && cudaMemsetAsync(ptr_, 0, bytes, cuda_detail::InferenceStream()) != cudaSuccess ? -1 : 0;
    }
    int Upload(const void* host, size_t bytes) {
        if (Reserve(bytes, false) != 0) return -1;
        return cudaMemcpyAsync(ptr_, host, bytes, cudaMemcpyHostToDevice, cuda_detail::InferenceStream()) == cudaSuccess &&
                       cudaStreamSynchronize(cuda_detail::InferenceStream()) == cudaSuccess ? 0 : -1;  // host vector is temporary
    }
    void* get() const { return ptr_; }
    size_t bytes() const { return bytes_; }
   private:
    void* ptr_{nullptr};
    size_t bytes_{0};
};

struct Int8WeightParams {
    std::vector<float> scales;
    std::vector<int32_t> zero_points;
    int32_t zp_max_abs{0};
};

// Mirrors int8_detail::BuildQuantizationView (src/kernel/common/int8_kernel_utils.h:55-84).
inline bool ReadInt8Quantization(const Tensor* t, bool allow_per_channel, int64_t axis, int64_t channels, Int8WeightParams* out) {
    if (!t || t->data_type() != DataType::INT8 || !t->IsInitialized()) return false;
    const QuantizationParams& q = t->quantization();
    if (!q.enabled || !ValidateQuantizationParams(q, t->dims().data())) return false;
    if (q.granularity == QuantizationGranularity::kPerChannel) {
        if (!allow_per_channel || q.axis != axis || q.scales.size() != static_cast<size_t>(channels)) return false;
        out->scales = q.scales;
        out->zero_points.resize(static_cast<size_t>(channels));
        for (int64_t c = 0; c < channels; ++c) out->zero_points[static_cast<size_t>(c)] = q.zero_point_at(static_cast<size_t>(c));
    } else if (q.granularity == QuantizationGranularity::kPerTensor) {
        out->scales = {q.scale_at(0)};
        out->zero_points = {q.zero_point_at(0)};
    } else {
        return false;
    }
    out->zp_max_abs = 0;
    for (int32_t z : out->zero_points) out->zp_max_abs = std::max(out->zp_max_abs, std::abs(z));
    return true;
}

// Largest |bias| of an INT32 bias constant that is readable on the host (the static quantiser's output), else 0.
inline int64_t BiasMaxAbs(const Tensor* bias) {
    int64_t worst = 0;
    if (bias && bias->IsInitialized() && bias->data_type() == DataType::INT32) {
        const int32_t* b = bias->data<int32_t>();
        for (int64_t i = 0; i < bias->numel(); ++i) worst = std::max<int64_t>(worst, std::llabs(static_cast<long long>(b[i])));
    }
    return worst;
}

// Device views of an input and an output tensor through the session's replica cache.
inline int AcquireIn(const Tensor* t, void** ptr) {
    return cuda_detail::AcquireTensorDevice(t, static_cast<size_t>(t->numel()) * DataTypeBytes(t->data_type()), t->raw_data(), ptr);
}
inline int FinishOut(Tensor* t, size_t bytes) {
    if (cuda_detail::DeferredHostSyncEnabled()) return 0;
    return cuda_detail::SyncTensorToHost(t, bytes, t->raw_data());
}

// Packed implicit-GEMM conv weights, one copy per immutable weight and device, shared by every session and plan that
// uses the weight (the reference keeps packed x86 layouts per weight the same way, src/kernel/x86/prepared_weight_cache.h;
// before this cache every session packed its own copy into its per-node workspace).  Sessions hold private host copies
// of a plan's constants (src/core/execution_plan.cc:430-470), so a weight is identified by its bytes — two 64-bit hashes
// over the content plus its shape — not by an address; the packed layout is a pure function of the content.  Entries are
// dropped when the last kernel that holds one goes away.
class PackedConvWeightCache {
   public:
    // `desc` describes the conv with desc->w already pointing at the weight ON THE DEVICE; packs on the inference stream
    // and waits, so that sessions on other streams may read the result.  Returns null when the geometry has no packed form.
    static std::shared_ptr<DeviceScratch> Acquire(const Tensor* weight, const fth_b200_int8_conv2d_desc& desc) {
        const size_t bytes = fth_b200_int8_conv2d_packed_weight_bytes(&desc);
        if (bytes == 0 || weight == nullptr || !weight->is_immutable()) return nullptr;
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess) return nullptr;
        const size_t count = static_cast<size_t>(weight->numel());
        const uint8_t* bytes_host = static_cast<const uint8_t*>(weight->raw_data());
        uint64_t h1 = 1469598103934665603ull, h2 = 0x9e3779b97f4a7c15ull;  // FNV-1a, and a multiply-rotate mix
        for (size_t i = 0; i < count; ++i) {
            h1 = (h1 ^ bytes_host[i]) * 1099511628211ull;
            h2 = ((h2 << 7) | (h2 >> 57)) + bytes_host[i] * 0xff51afd7ed558ccdull;
        }
        const Key key{h1, h2, device, desc.oc, desc.ic, desc.kh, desc.kw};
        std::lock_guard<std::mutex> lock(Mutex());
        auto& table = Table();
        for (auto it = table.begin(); it != table.end();) {
            if (it->second.expired()) { it = table.erase(it); continue; }
            if (it->first == key) {
                if (auto hit = it->second.lock()) return hit;
            }
            ++it;
        }
        auto packed = std::make_shared<DeviceScratch>();
        if (packed->Reserve(bytes, false) != 0) return nullptr;
        if (fth_b200_int8_conv2d_pack_weights(&desc, packed->get(), cuda_detail::InferenceStream()) != FTH_B200_OK) return nullptr;
        if (cudaStreamSynchronize(cuda_detail::InferenceStream()) != cudaSuccess) return nullptr;
        table.emplace_back(key, packed);
        return packed;
    }
    static size_t LiveEntries() {
        std::lock_guard<std::mutex> lock(Mutex());
        size_t n = 0;
        for (const auto& e : Table()) n += !e.second.expired();
        return n;
    }

   private:
    struct Key {
        uint64_t h1, h2; int device; int64_t oc, ic, kh, kw;
        bool operator==(const Key& o) const {
            return h1 == o.h1 && h2 == o.h2 && device == o.device && oc == o.oc && ic == o.ic && kh == o.kh && kw == o.kw;
        }
    };
    static std::mutex& Mutex() { static std::mutex m; return m; }
    static std::vector<std::pair<Key, std::weak_ptr<DeviceScratch>>>& Table() {
        static std::vector<std::pair<Key, std::weak_ptr<DeviceScratch>>> t;
        return t;
    }
};

template <typename K>
void AddCandidate(DataType dtype, const char* op, const char* id) {
    KernelDispatcher::instance().RegisterCandidate(DeviceType::CUDA, dtype, DataLayout::ND, op, id,
                                                   [] { return std::unique_ptr<KernelBase>(new K()); }, {}, kPriority);
}

}  // namespace b200
}  // namespace kernel
}  // namespace feather
