// TEST INFRASTRUCTURE — end-to-end check of the Feather adapter inside the real reference runtime.
//
// Linked against the unmodified reference library built WITH its CUDA backend (oracle/_ref/libfeather_ref_cuda.so),
// this repo's adapter (infer_b200/adapter/b200_candidates.cu) and libfth_b200.so.  It drives kernels the way the
// reference's own CUDA unit tests do (test/standard_int8_kernel_test.cc:127-162: execution context scope, deferred
// host sync, SyncTensorToHostIfNeeded) and mirrors its selection-contract tests
// (test/kernel_selection_contract_test.cc:86-203).
//
//   adapter_e2e select   host only: registration, candidate order, kRequireRequested, decline → next CUDA candidate
//   adapter_e2e run      needs a GPU: the new candidates run through the reference's CUDA runtime (replica cache,
//                        inference stream) and are compared with the reference's COMMON kernels on the same tensors
//   adapter_e2e time     needs a GPU: microseconds per compute() of FP8 / INT8 MatMul nodes through the reference
//                        runtime; with FEATHER_DISABLE_B200=1 the same nodes run on the reference's own CUDA kernels
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include <cuda_runtime.h>
#include <unistd.h>

#include "core/execution_plan.h"
#include "core/kernel.h"
#include "core/static_graph.h"
#include "core/tensor.h"
#include "model/model_io.h"
#include "b200_shard.h"
#include "fth_b200.h"
#include "pass/graph_pass.h"
#include "quant/static_quantizer.h"
#include "src/kernel/cuda/runtime.h"
#include "src/operator/params.h"
#include "util/bf16.h"
#include "util/fp8.h"

namespace feather { namespace kernel { namespace b200 {
bool RegisterB200Kernels();
bool RegisterB200FusedOperators();
std::unique_ptr<GraphPass> CreateB200FusionPass();
bool IsB200Kernel(const KernelBase* kernel);
size_t PackedConvWeightEntries();
}}}

using namespace feather;
namespace cuda = feather::kernel::cuda_detail;
using feather::kernel::b200::IsB200Kernel;

static int g_failures = 0;
#define CHECK_THAT(cond, what)                                                        \
    do {                                                                              \
        const bool ok_ = (cond);                                                      \
        std::printf("%s  %s\n", ok_ ? "ok  " : "FAIL", what);                        \
        if (!ok_) ++g_failures;                                                       \
    } while (0)

static uint32_t g_lcg = 0x12345678u;
static uint32_t NextRandom() { g_lcg = g_lcg * 1664525u + 1013904223u; return g_lcg >> 8; }
static float Uniform(float lo, float hi) { return lo + (hi - lo) * (NextRandom() % 100000) / 100000.0f; }

static size_t Bytes(DataType t) {
    switch (t) {
        case DataType::FP32: case DataType::INT32: return 4;
        case DataType::FP16: case DataType::BF16: return 2;
        case DataType::INT64: return 8;
        default: return 1;
    }
}

static std::shared_ptr<Tensor> MakeTensor(DataType dtype, const std::vector<int64_t>& dims, const void* data = nullptr) {
    size_t count = 1;
    for (int64_t d : dims) count *= static_cast<size_t>(d);
    auto t = std::make_shared<Tensor>(count * Bytes(dtype));
    t->Resize(dims);
    void* dst = t->mutable_data(count * Bytes(dtype));
    if (data) std::memcpy(dst, data, count * Bytes(dtype));
    else std::memset(dst, 0, count * Bytes(dtype));
    t->set_data_type(dtype);
    return t;
}

static QuantizationParams PerTensor(float scale, int32_t zp = 0) {
    QuantizationParams q;
    q.enabled = true; q.scale = scale; q.zero_point = zp;
    return q;
}
static QuantizationParams PerChannel(int64_t axis, const std::vector<float>& scales) {
    QuantizationParams q;
    q.enabled = true; q.granularity = QuantizationGranularity::kPerChannel; q.axis = axis;
    q.scales = scales; q.zero_points.assign(scales.size(), 0);
    q.scale = scales.front(); q.zero_point = 0;
    return q;
}

// create → bind parameters → FinalizeSelection, under kRequireRequested, exactly what OperatorRegistry::Create does.
template <typename Param>
static std::unique_ptr<KernelBase> Select(DeviceType device, DataType dtype, const char* op, Param* param, Status* status = nullptr) {
    KernelSelectionScope scope(KernelFallbackPolicy::kRequireRequested, nullptr);
    auto kernel = KernelDispatcher::instance().create(device, dtype, op);
    if (!kernel) { if (status) *status = KernelDispatcher::LastSelectionStatus(); return nullptr; }
    kernel->SetParam(param);
    const Status s = KernelBase::FinalizeSelection(&kernel);
    if (status) *status = s;
    return s.ok() ? std::move(kernel) : nullptr;
}

struct Fp8Case {
    std::shared_ptr<Tensor> a, w, out;
    operators::MatMulParam param;
};
static Fp8Case MakeFp8(DataType dt, int64_t m, int64_t k, int64_t n) {
    std::vector<uint8_t> a(static_cast<size_t>(m * k)), w(static_cast<size_t>(k * n));
    for (auto& v : a) v = dt == DataType::FP8E4M3 ? FloatToFp8E4M3(Uniform(-2, 2)) : FloatToFp8E5M2(Uniform(-2, 2));
    for (auto& v : w) v = dt == DataType::FP8E4M3 ? FloatToFp8E4M3(Uniform(-1, 1)) : FloatToFp8E5M2(Uniform(-1, 1));
    Fp8Case c;
    c.a = MakeTensor(dt, {m, k}, a.data()); c.a->set_quantization({true, 0.5f});
    c.w = MakeTensor(dt, {k, n}, w.data()); c.w->set_quantization({true, 0.03125f}); c.w->set_immutable(true);
    c.out = MakeTensor(dt, {m, n}); c.out->set_quantization({true, 0.25f});
    c.param.a = c.a; c.param.b = c.w; c.param.out = c.out;
    return c;
}

struct Int8Case {
    std::shared_ptr<Tensor> a, w, out;
    operators::MatMulParam param;
};
static Int8Case MakeInt8(int64_t m, int64_t k, int64_t n) {
    std::vector<int8_t> a(static_cast<size_t>(m * k)), w(static_cast<size_t>(k * n));
    for (auto& v : a) v = static_cast<int8_t>(static_cast<int>(NextRandom() % 255) - 127);
    for (auto& v : w) v = static_cast<int8_t>(static_cast<int>(NextRandom() % 255) - 127);
    std::vector<float> scales(static_cast<size_t>(n));
    for (auto& s : scales) s = Uniform(1e-3f, 1e-2f);
    Int8Case c;
    c.a = MakeTensor(DataType::INT8, {m, k}, a.data()); c.a->set_quantization(PerTensor(0.02f));
    c.w = MakeTensor(DataType::INT8, {k, n}, w.data()); c.w->set_quantization(PerChannel(1, scales)); c.w->set_immutable(true);
    c.out = MakeTensor(DataType::INT8, {m, n});
    c.out->set_quantization(PerTensor(2.33f * 73.3f * 73.3f * std::sqrt(static_cast<float>(k)) * 0.02f * 0.0055f / 127.0f));
    c.param.a = c.a; c.param.b = c.w; c.param.out = c.out;
    return c;
}

// ---------------------------------------------------------------------------------------------------------
// select: host only
// ---------------------------------------------------------------------------------------------------------
template <typename Param>
static int RunCommon(DataType dtype, const char* op, Param* param);

static void RunSelect() {
    // Before registration the reference cannot build a statically quantised INT8 plan for CUDA under
    // kRequireRequested: DequantizeLinear has no CUDA candidate and INT8 requests never fall back to COMMON.
    {
        KernelSelectionScope scope(KernelFallbackPolicy::kRequireRequested, nullptr);
        CHECK_THAT(KernelDispatcher::instance().create(DeviceType::CUDA, DataType::INT8, "DequantizeLinear") == nullptr,
                   "reference alone: create(CUDA, INT8, DequantizeLinear) under kRequireRequested is null");
        CHECK_THAT(KernelDispatcher::instance().create(DeviceType::CUDA, DataType::FP32, "QuantizeLinear") == nullptr,
                   "reference alone: create(CUDA, FP32, QuantizeLinear) under kRequireRequested is null");
    }
    CHECK_THAT(feather::kernel::b200::RegisterB200Kernels(), "RegisterB200Kernels()");
    {
        KernelSelectionScope scope(KernelFallbackPolicy::kRequireRequested, nullptr);
        const DataType fp8[] = {DataType::FP8E4M3, DataType::FP8E5M2, DataType::INT8};
        bool all = true;
        for (DataType dt : fp8)
            for (const char* op : {"FC", "MatMul", "Gemm"}) all = all && KernelDispatcher::instance().create(DeviceType::CUDA, dt, op) != nullptr;
        all = all && KernelDispatcher::instance().create(DeviceType::CUDA, DataType::INT8, "Conv2D") != nullptr;
        all = all && KernelDispatcher::instance().create(DeviceType::CUDA, DataType::INT8, "DequantizeLinear") != nullptr;
        all = all && KernelDispatcher::instance().create(DeviceType::CUDA, DataType::FP32, "QuantizeLinear") != nullptr;
        all = all && KernelDispatcher::instance().create(DeviceType::CUDA, DataType::BF16, "Cast") != nullptr;
        CHECK_THAT(all, "after registration every hot-path (dtype, op) has a CUDA candidate under kRequireRequested");
    }
    // the new candidate is tried first and accepted
    for (DataType dt : {DataType::FP8E4M3, DataType::FP8E5M2}) {
        Fp8Case c = MakeFp8(dt, 1, 1024, 3072);
        Status st;
        auto k = Select(DeviceType::CUDA, dt, "MatMul", &c.param, &st);
        CHECK_THAT(k && IsB200Kernel(k.get()) && k->device() == DeviceType::CUDA, "FP8 MatMul [1,1024]x[1024,3072] selects the b200 candidate");
    }
    {
        Int8Case c = MakeInt8(128, 1024, 1024);
        auto k = Select(DeviceType::CUDA, DataType::INT8, "MatMul", &c.param);
        CHECK_THAT(k && IsB200Kernel(k.get()), "INT8 MatMul [128,1024]x[1024,1024] per-channel selects the b200 candidate");
    }
    // An FP8 weight with one scale per output channel: the reference's linear kernels read the tensor's scalar scale only
    // (include/core/tensor.h:105) — the vector is ignored, every column gets scales[0]; the new candidate applies the
    // vector, on the output-channel axis only.
    {
        Fp8Case c = MakeFp8(DataType::FP8E4M3, 2, 512, 384);
        std::vector<float> scales(384);
        for (size_t i = 0; i < scales.size(); ++i) scales[i] = (i & 1) ? 0.0625f : 0.03125f;
        c.w->set_quantization(PerChannel(1, scales));
        {
            const bool ran = RunCommon(DataType::FP8E4M3, "MatMul", &c.param) == 0;
            std::vector<uint8_t> with_vector(static_cast<const uint8_t*>(c.out->raw_data()), static_cast<const uint8_t*>(c.out->raw_data()) + 2 * 384);
            c.w->set_quantization({true, scales.front()});
            const bool ran_scalar = RunCommon(DataType::FP8E4M3, "MatMul", &c.param) == 0;
            const bool same = std::memcmp(with_vector.data(), c.out->raw_data(), with_vector.size()) == 0;
            CHECK_THAT(ran && ran_scalar && same, "FP8 MatMul with per-channel weight scales: the reference's COMMON kernel ignores the vector (same bytes as scale = scales[0])");
            c.w->set_quantization(PerChannel(1, scales));
        }
        auto k = Select(DeviceType::CUDA, DataType::FP8E4M3, "MatMul", &c.param);
        CHECK_THAT(k && IsB200Kernel(k.get()), "FP8 MatMul with per-channel weight scales selects the b200 candidate");
        c.w->set_quantization(PerChannel(0, std::vector<float>(512, 0.03125f)));
        auto wrong_axis = Select(DeviceType::CUDA, DataType::FP8E4M3, "MatMul", &c.param);
        CHECK_THAT(!(wrong_axis && IsB200Kernel(wrong_axis.get())), "FP8 MatMul with scales along K: the b200 candidate declines");

        // The model file needs no new field for it: the reference's own writer and loader carry the vector (as its test
        // test/model_io_quantization_test.cc:27-78 shows for INT8), and the weight read back selects the b200 candidate.
        c.w->set_quantization(PerChannel(1, scales));
        model::ModelDesc file;
        file.name = "fp8_per_channel"; file.version = 1; file.graph.name = "main";
        file.graph.inputs = {"x"}; file.graph.outputs = {"y"};
        model::ValueDesc x, w, y;
        x.tensor.name = "x"; x.tensor.dims = {2, 512}; x.tensor.data_type = DataType::FP8E4M3; x.tensor.quantization = c.a->quantization();
        w.tensor.name = "w"; w.tensor.dims = {512, 384}; w.tensor.data_type = DataType::FP8E4M3; w.tensor.quantization = PerChannel(1, scales);
        w.constant = true;
        y.tensor.name = "y"; y.tensor.dims = {2, 384}; y.tensor.data_type = DataType::FP8E4M3; y.tensor.quantization = c.out->quantization();
        model::NodeDesc node;
        node.name = "projection"; node.op_type = "MatMul"; node.inputs = {"x", "w"}; node.outputs = {"y"};
        file.graph.values = {x, w, y};
        file.graph.nodes = {node};
        const std::string path = "/tmp/fth_b200_fp8_per_channel_" + std::to_string(static_cast<long long>(getpid())) + ".fth";
        model::ModelLoader loader;
        const bool saved = model::ModelWriter().Save(path, file, {{"w", c.w}}) && loader.Load(path);
        bool carried = false, selected = false;
        if (saved) {
            const QuantizationParams& q = loader.model().graph.values[1].tensor.quantization;
            carried = q.enabled && q.granularity == QuantizationGranularity::kPerChannel && q.axis == 1 && q.scales == scales;
            auto loaded = loader.CreateWeightTensor("w");
            if (loaded) {
                // the weight view takes the value's metadata itself (src/model/weight_store.cc: CreateTensorView)
                carried = carried && loaded->quantization().granularity == QuantizationGranularity::kPerChannel && loaded->quantization().scales == scales;
                loaded->set_immutable(true);
                carried = carried && std::memcmp(loaded->raw_data(), c.w->raw_data(), 512 * 384) == 0;
                operators::MatMulParam from_file = c.param;
                from_file.b = loaded;
                auto kf = Select(DeviceType::CUDA, DataType::FP8E4M3, "MatMul", &from_file);
                selected = kf && IsB200Kernel(kf.get());
            }
        }
        std::remove(path.c_str());
        CHECK_THAT(saved && carried && selected, "a .fth file written and read by the reference carries the per-channel FP8 scales; the loaded weight selects the b200 candidate");
    }
    // a request the new backend declines moves on to the reference's CUDA candidate, never to a CPU kernel
    {
        Fp8Case c = MakeFp8(DataType::FP8E4M3, 2, 64, 32);
        std::vector<uint8_t> wb(static_cast<size_t>(3 * 64 * 32), 0x38);
        c.w = MakeTensor(DataType::FP8E4M3, {3, 64, 32}, wb.data()); c.w->set_quantization({true, 1.0f});
        c.a = MakeTensor(DataType::FP8E4M3, {3, 2, 64}); c.a->set_quantization({true, 1.0f});
        c.out = MakeTensor(DataType::FP8E4M3, {3, 2, 32}); c.out->set_quantization({true, 1.0f});
        c.param.a = c.a; c.param.b = c.w; c.param.out = c.out;
        auto k = Select(DeviceType::CUDA, DataType::FP8E4M3, "MatMul", &c.param);
        CHECK_THAT(k && !IsB200Kernel(k.get()) && k->device() == DeviceType::CUDA,
                   "batched FP8 MatMul (rank-3 B): b200 answers kUnsupported, the reference CUDA kernel is selected");
    }
    {
        // the int32 accumulator could overflow (K * 128 * 128 > 2^31 - 1): declined up front
        Int8Case c = MakeInt8(1, 140000, 16);
        auto k = Select(DeviceType::CUDA, DataType::INT8, "MatMul", &c.param);
        CHECK_THAT(k && !IsB200Kernel(k.get()) && k->device() == DeviceType::CUDA, "INT8 K = 140000: b200 declines (overflow bound), reference CUDA kernel selected");
    }
    {
        // the operators between the projections, and the fused FP8 lm-head selection (no CUDA candidate in the reference)
        KernelSelectionScope scope(KernelFallbackPolicy::kRequireRequested, nullptr);
        bool all = true;
        for (const char* op : {"QwenRmsNorm", "Add", "Mul", "SiLU"}) {
            auto k = KernelDispatcher::instance().create(DeviceType::CUDA, DataType::BF16, op);
            all = all && k && IsB200Kernel(k.get());
        }
        CHECK_THAT(all, "BF16 QwenRmsNorm / Add / Mul / SiLU: the b200 candidate is first");
        auto k = KernelDispatcher::instance().create(DeviceType::CUDA, DataType::FP8E4M3, "QwenGemmArgmax");
        CHECK_THAT(k && IsB200Kernel(k.get()), "create(CUDA, FP8E4M3, QwenGemmArgmax) has a candidate (the reference registers BF16 only)");
    }
    {
        // a node built with a scratch budget of zero still selects the b200 candidate (built-in scratch, or kernels without scratch)
        Fp8Case c = MakeFp8(DataType::FP8E4M3, 4, 4096, 8192);
        KernelSelectionScope scope(KernelFallbackPolicy::kRequireRequested, nullptr, false, 0);
        auto k = KernelDispatcher::instance().create(DeviceType::CUDA, DataType::FP8E4M3, "MatMul");
        k->SetParam(&c.param);
        CHECK_THAT(KernelBase::FinalizeSelection(&k).ok() && IsB200Kernel(k.get()), "workspace limit 0: FP8 MatMul [4,4096]x[4096,8192] still selects the b200 candidate");
    }
    {
        // FEATHER selection without the strict policy still prefers CUDA candidates (priority order)
        Int8Case c = MakeInt8(4, 256, 64);
        KernelSelectionScope scope(KernelFallbackPolicy::kAllowCommon, nullptr);
        auto k = KernelDispatcher::instance().create(DeviceType::CUDA, DataType::INT8, "MatMul");
        k->SetParam(&c.param);
        CHECK_THAT(KernelBase::FinalizeSelection(&k).ok() && IsB200Kernel(k.get()), "kAllowCommon: the b200 candidate is still first");
    }
}

// ---------------------------------------------------------------------------------------------------------
// run: on a GPU, inside the reference's CUDA runtime
// ---------------------------------------------------------------------------------------------------------
static int CodeIndex(uint8_t c) { return (c & 0x80) ? -(c & 0x7f) : (c & 0x7f); }

template <typename Param>
static int RunCommon(DataType dtype, const char* op, Param* param) {
    auto k = KernelDispatcher::instance().create(DeviceType::COMMON, dtype, op);
    if (!k) return -1;
    k->SetParam(param);
    return k->compute();
}

static void RunPlansOnGpu();

static void RunGpu() {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        std::printf("skip  no CUDA device\n");
        return;
    }
    feather::kernel::b200::RegisterB200Kernels();
    auto context = cuda::CreateExecutionContext();
    cuda::ExecutionContextScope scope(context);

    // ---- FP8 MatMul (config 1 shape), both formats, twice (the second run hits the replica cache) ----
    for (DataType dt : {DataType::FP8E4M3, DataType::FP8E5M2}) {
        Fp8Case c = MakeFp8(dt, 1, 1024, 3072);
        auto k = Select(DeviceType::CUDA, dt, "MatMul", &c.param);
        bool ok = k && IsB200Kernel(k.get()) && k->Prepare() == 0;
        int max_dist = -1;
        if (ok) {
            cuda::DeferredHostSyncScope deferred;
            for (int run = 0; run < 2 && ok; ++run) {
                ok = k->compute() == 0 && cuda::SyncTensorToHostIfNeeded(c.out.get(), c.out->memory_size(), c.out->raw_data()) == 0;
            }
            std::vector<uint8_t> got(static_cast<const uint8_t*>(c.out->raw_data()), static_cast<const uint8_t*>(c.out->raw_data()) + 3072);
            auto ref_out = MakeTensor(dt, {1, 3072}); ref_out->set_quantization({true, 0.25f});
            operators::MatMulParam rp; rp.a = c.a; rp.b = c.w; rp.out = ref_out;
            ok = ok && RunCommon(dt, "MatMul", &rp) == 0;
            const uint8_t* want = static_cast<const uint8_t*>(ref_out->raw_data());
            max_dist = 0;
            for (int i = 0; i < 3072; ++i) max_dist = std::max(max_dist, std::abs(CodeIndex(got[i]) - CodeIndex(want[i])));
        }
        std::printf("      [%s] max code distance vs COMMON: %d\n", fth_b200_last_variant(), max_dist);
        CHECK_THAT(ok && max_dist >= 0 && max_dist <= 1, dt == DataType::FP8E4M3 ? "CUDA FP8E4M3 MatMul through the reference runtime matches COMMON within one code"
                                                                               : "CUDA FP8E5M2 MatMul through the reference runtime matches COMMON within one code");
    }

    // ---- FP8 MatMul whose weight carries one scale per output channel: column n is what COMMON gives with w_scale = scales[n] ----
    for (DataType dt : {DataType::FP8E4M3, DataType::FP8E5M2}) {
        const int64_t m = 3, kk = 1024, n = 2048;
        Fp8Case c = MakeFp8(dt, m, kk, n);
        std::vector<float> scales(static_cast<size_t>(n));
        for (size_t i = 0; i < scales.size(); ++i) scales[i] = (i & 1) ? 0.0625f : 0.03125f;
        c.w->set_quantization(PerChannel(1, scales));
        auto k = Select(DeviceType::CUDA, dt, "MatMul", &c.param);
        bool ok = k && IsB200Kernel(k.get()) && k->Prepare() == 0;
        if (ok) {
            cuda::DeferredHostSyncScope deferred;
            ok = k->compute() == 0 && cuda::SyncTensorToHostIfNeeded(c.out.get(), c.out->memory_size(), c.out->raw_data()) == 0;
        }
        const uint8_t* got = static_cast<const uint8_t*>(c.out->raw_data());
        int max_dist = ok ? 0 : -1, differ = 0;
        std::vector<uint8_t> first;
        for (int pass = 0; pass < 2 && ok; ++pass) {  // COMMON with the even columns' scale, then with the odd columns'
            c.w->set_quantization({true, pass == 0 ? 0.03125f : 0.0625f});
            auto ref_out = MakeTensor(dt, {m, n}); ref_out->set_quantization({true, 0.25f});
            operators::MatMulParam rp; rp.a = c.a; rp.b = c.w; rp.out = ref_out;
            ok = RunCommon(dt, "MatMul", &rp) == 0;
            const uint8_t* want = static_cast<const uint8_t*>(ref_out->raw_data());
            if (pass == 0) first.assign(want, want + m * n);
            for (int64_t i = 0; i < m * n && ok; ++i) {
                if ((i % n) % 2 != pass) continue;
                max_dist = std::max(max_dist, std::abs(CodeIndex(got[i]) - CodeIndex(want[i])));
            }
            if (pass == 1) for (int64_t i = 0; i < m * n; ++i) differ += first[static_cast<size_t>(i)] != want[i];
        }
        std::printf("      [%s] per-channel weight scales: max code distance vs COMMON column by column: %d (the two scales' results differ in %d bytes)\n",
                    fth_b200_last_variant(), max_dist, differ);
        CHECK_THAT(ok && max_dist >= 0 && max_dist <= 1 && differ > 0, dt == DataType::FP8E4M3 ? "CUDA FP8E4M3 MatMul with per-channel weight scales matches COMMON column by column"
                                                                                             : "CUDA FP8E5M2 MatMul with per-channel weight scales matches COMMON column by column");
    }

    // ---- INT8 MatMul (config 2 shape), per-channel weight scales: bit-exact ----
    {
        Int8Case c = MakeInt8(128, 1024, 1024);
        auto k = Select(DeviceType::CUDA, DataType::INT8, "MatMul", &c.param);
        bool ok = k && IsB200Kernel(k.get()) && k->Prepare() == 0;
        if (ok) {
            cuda::DeferredHostSyncScope deferred;
            ok = k->compute() == 0 && cuda::SyncTensorToHostIfNeeded(c.out.get(), c.out->memory_size(), c.out->raw_data()) == 0;
        }
        std::vector<int8_t> got(static_cast<const int8_t*>(c.out->raw_data()), static_cast<const int8_t*>(c.out->raw_data()) + 128 * 1024);
        auto ref_out = MakeTensor(DataType::INT8, {128, 1024}); ref_out->set_quantization(c.out->quantization());
        operators::MatMulParam rp; rp.a = c.a; rp.b = c.w; rp.out = ref_out;
        ok = ok && RunCommon(DataType::INT8, "MatMul", &rp) == 0;
        int diff = 0;
        for (int i = 0; i < 128 * 1024; ++i) diff += got[i] != static_cast<const int8_t*>(ref_out->raw_data())[i];
        std::printf("      [%s] bytes differing from COMMON: %d of %d\n", fth_b200_last_variant(), diff, 128 * 1024);
        CHECK_THAT(ok && diff == 0, "CUDA INT8 MatMul (M=128, per-channel) through the reference runtime is bit-exact with COMMON");
    }

    // ---- QuantizeLinear → INT8 MatMul → DequantizeLinear, all on CUDA with deferred host sync ----
    {
        const int64_t m = 4, kk = 512, n = 256;
        Int8Case c = MakeInt8(m, kk, n);
        std::vector<float> x(static_cast<size_t>(m * kk));
        for (auto& v : x) v = Uniform(-2.5f, 2.5f);
        auto xin = MakeTensor(DataType::FP32, {m, kk}, x.data());
        const float qs = 0.02f; const int32_t qz = 0;
        auto scale_t = MakeTensor(DataType::FP32, {1}, &qs);
        auto zp_t = MakeTensor(DataType::INT32, {1}, &qz);
        const float dqs = c.out->quantization().scale;
        auto dscale_t = MakeTensor(DataType::FP32, {1}, &dqs);
        auto y_gpu = MakeTensor(DataType::FP32, {m, n});
        auto q_gpu = MakeTensor(DataType::INT8, {m, kk});
        operators::QuantizeLinearParam qp; qp.input = xin; qp.scale = scale_t; qp.zero_point = zp_t; qp.out = q_gpu; qp.axis = -1;
        operators::MatMulParam mp; mp.a = q_gpu; mp.b = c.w; mp.out = c.out;
        operators::DequantizeLinearParam dp; dp.input = c.out; dp.scale = dscale_t; dp.zero_point = zp_t; dp.out = y_gpu; dp.to = DataType::FP32; dp.axis = -1;
        // QuantizeLinear sets its output's quantisation at run time; the MatMul candidate is selected after it has run once on COMMON metadata
        q_gpu->set_quantization(PerTensor(qs, qz));
        auto kq = Select(DeviceType::CUDA, DataType::FP32, "QuantizeLinear", &qp);
        auto km = Select(DeviceType::CUDA, DataType::INT8, "MatMul", &mp);
        auto kd = Select(DeviceType::CUDA, DataType::INT8, "DequantizeLinear", &dp);
        bool ok = kq && km && kd && IsB200Kernel(kq.get()) && IsB200Kernel(km.get()) && IsB200Kernel(kd.get()) &&
                  kq->Prepare() == 0 && km->Prepare() == 0 && kd->Prepare() == 0;
        if (ok) {
            cuda::DeferredHostSyncScope deferred;
            ok = kq->compute() == 0 && km->compute() == 0 && kd->compute() == 0 &&
                 cuda::SyncTensorToHostIfNeeded(y_gpu.get(), y_gpu->memory_size(), y_gpu->raw_data()) == 0;
        }
        std::vector<float> got(static_cast<const float*>(y_gpu->raw_data()), static_cast<const float*>(y_gpu->raw_data()) + m * n);
        // the same three nodes on COMMON
        auto q_ref = MakeTensor(DataType::INT8, {m, kk});
        auto o_ref = MakeTensor(DataType::INT8, {m, n}); o_ref->set_quantization(c.out->quantization());
        auto y_ref = MakeTensor(DataType::FP32, {m, n});
        operators::QuantizeLinearParam qr = qp; qr.out = q_ref;
        operators::MatMulParam mr; mr.a = q_ref; mr.b = c.w; mr.out = o_ref;
        operators::DequantizeLinearParam dr = dp; dr.input = o_ref; dr.out = y_ref;
        ok = ok && RunCommon(DataType::FP32, "QuantizeLinear", &qr) == 0 && RunCommon(DataType::INT8, "MatMul", &mr) == 0 &&
             RunCommon(DataType::INT8, "DequantizeLinear", &dr) == 0;
        int diff = 0;
        for (int64_t i = 0; i < m * n; ++i) diff += std::memcmp(&got[static_cast<size_t>(i)], static_cast<const float*>(y_ref->raw_data()) + i, 4) != 0;
        std::printf("      Q -> MatMul -> DQ on CUDA: %d of %d floats differ from COMMON\n", diff, static_cast<int>(m * n));
        CHECK_THAT(ok && diff == 0, "QuantizeLinear -> INT8 MatMul -> DequantizeLinear runs entirely on CUDA candidates, identical to COMMON");
    }

    // ---- per-channel QuantizeLinear / DequantizeLinear on axis 1 of an NCHW activation ----
    {
        const int64_t n = 2, ch = 6, h = 5, w = 9, count = n * ch * h * w;
        std::vector<float> x(static_cast<size_t>(count));
        for (auto& v : x) v = Uniform(-3.0f, 3.0f);
        std::vector<float> sc(static_cast<size_t>(ch));
        std::vector<int32_t> zp(static_cast<size_t>(ch));
        for (int64_t i = 0; i < ch; ++i) { sc[static_cast<size_t>(i)] = 0.01f + 0.005f * static_cast<float>(i); zp[static_cast<size_t>(i)] = static_cast<int32_t>(i) - 3; }
        auto xin = MakeTensor(DataType::FP32, {n, ch, h, w}, x.data());
        auto scale_t = MakeTensor(DataType::FP32, {ch}, sc.data());
        auto zp_t = MakeTensor(DataType::INT32, {ch}, zp.data());
        auto q_gpu = MakeTensor(DataType::INT8, {n, ch, h, w});
        auto q_ref = MakeTensor(DataType::INT8, {n, ch, h, w});
        auto y_gpu = MakeTensor(DataType::FP32, {n, ch, h, w});
        auto y_ref = MakeTensor(DataType::FP32, {n, ch, h, w});
        operators::QuantizeLinearParam qp; qp.input = xin; qp.scale = scale_t; qp.zero_point = zp_t; qp.out = q_gpu; qp.axis = 1;
        operators::QuantizeLinearParam qr = qp; qr.out = q_ref;
        bool ok = RunCommon(DataType::FP32, "QuantizeLinear", &qr) == 0;
        auto kq = Select(DeviceType::CUDA, DataType::FP32, "QuantizeLinear", &qp);
        ok = ok && kq && IsB200Kernel(kq.get()) && kq->Prepare() == 0 && kq->compute() == 0;
        operators::DequantizeLinearParam dp; dp.input = q_ref; dp.scale = scale_t; dp.zero_point = zp_t; dp.out = y_gpu; dp.to = DataType::FP32; dp.axis = 1;
        operators::DequantizeLinearParam dr = dp; dr.out = y_ref;
        ok = ok && RunCommon(DataType::INT8, "DequantizeLinear", &dr) == 0;
        auto kd = Select(DeviceType::CUDA, DataType::INT8, "DequantizeLinear", &dp);
        ok = ok && kd && IsB200Kernel(kd.get()) && kd->Prepare() == 0 && kd->compute() == 0;
        const bool same_q = ok && std::memcmp(q_gpu->raw_data(), q_ref->raw_data(), static_cast<size_t>(count)) == 0;
        const bool same_y = ok && std::memcmp(y_gpu->raw_data(), y_ref->raw_data(), static_cast<size_t>(count) * 4) == 0;
        CHECK_THAT(same_q && same_y, "per-channel QuantizeLinear / DequantizeLinear on axis 1 of [N,C,H,W] run on the CUDA candidates, identical to COMMON");
    }

    // ---- INT8 Conv2D 3x3 pad 1 with int32 bias ----
    {
        const int64_t ic = 64, oc = 64, h = 24, w = 40;
        std::vector<int8_t> x(static_cast<size_t>(ic * h * w)), wt(static_cast<size_t>(oc * ic * 9));
        for (auto& v : x) v = static_cast<int8_t>(static_cast<int>(NextRandom() % 256) - 128);
        for (auto& v : wt) v = static_cast<int8_t>(static_cast<int>(NextRandom() % 256) - 128);
        std::vector<float> scales(static_cast<size_t>(oc));
        for (auto& s : scales) s = Uniform(1e-3f, 1e-2f);
        std::vector<int32_t> bias(static_cast<size_t>(oc));
        for (auto& b : bias) b = static_cast<int32_t>(NextRandom() % 65536) - 32768;
        auto tx = MakeTensor(DataType::INT8, {1, ic, h, w}, x.data()); tx->set_quantization(PerTensor(0.05f));
        auto tw = MakeTensor(DataType::INT8, {oc, ic, 3, 3}, wt.data()); tw->set_quantization(PerChannel(0, scales)); tw->set_immutable(true);
        auto tb = MakeTensor(DataType::INT32, {oc}, bias.data());
        const QuantizationParams oq = PerTensor(2.33f * 74.0f * 74.0f * 24.0f * 0.05f * 0.0055f / 127.0f);
        auto out = MakeTensor(DataType::INT8, {1, oc, h, w}); out->set_quantization(oq);
        auto ref = MakeTensor(DataType::INT8, {1, oc, h, w}); ref->set_quantization(oq);
        operators::Conv2dParam cp; cp.input = tx; cp.w = tw; cp.bias = tb; cp.out = out;
        cp.stride_h = cp.stride_w = 1; cp.pad_h = cp.pad_w = 1; cp.dilation_h = cp.dilation_w = 1; cp.group = 1;
        operators::Conv2dParam cr = cp; cr.out = ref;
        auto k = Select(DeviceType::CUDA, DataType::INT8, "Conv2D", &cp);
        bool ok = k && IsB200Kernel(k.get()) && k->Prepare() == 0;
        if (ok) {
            cuda::DeferredHostSyncScope deferred;
            ok = k->compute() == 0 && k->compute() == 0 &&
                 cuda::SyncTensorToHostIfNeeded(out.get(), out->memory_size(), out->raw_data()) == 0;
        }
        ok = ok && RunCommon(DataType::INT8, "Conv2D", &cr) == 0;
        const int diff = ok ? std::memcmp(out->raw_data(), ref->raw_data(), static_cast<size_t>(oc * h * w)) : 1;
        std::printf("      [%s]\n", fth_b200_last_variant());
        CHECK_THAT(ok && diff == 0, "CUDA INT8 Conv2D 3x3 (64->64, int32 bias) through the reference runtime is bit-exact with COMMON");
    }
    // ---- the operators between the projections: QwenRmsNorm, Add, SiLU on BF16 [4,1024] ----
    {
        const int64_t rows = 4, hidden = 1024;
        std::vector<uint16_t> x(static_cast<size_t>(rows * hidden)), g(static_cast<size_t>(hidden)), y(static_cast<size_t>(rows * hidden));
        for (auto& v : x) v = FloatToBFloat16(Uniform(-3, 3));
        for (auto& v : g) v = FloatToBFloat16(Uniform(-0.2f, 0.2f));
        for (auto& v : y) v = FloatToBFloat16(Uniform(-1, 1));
        const float eps = 1e-6f;
        auto tx = MakeTensor(DataType::BF16, {rows, hidden}, x.data());
        auto tg = MakeTensor(DataType::BF16, {hidden}, g.data());
        auto ty = MakeTensor(DataType::BF16, {rows, hidden}, y.data());
        auto te = MakeTensor(DataType::FP32, {1}, &eps);
        auto Steps = [](const Tensor* a, const Tensor* b, int64_t n) {
            int worst = 0;
            const uint16_t* pa = static_cast<const uint16_t*>(a->raw_data());
            const uint16_t* pb = static_cast<const uint16_t*>(b->raw_data());
            for (int64_t i = 0; i < n; ++i) {
                const int va = (pa[i] & 0x8000) ? -(pa[i] & 0x7fff) : (pa[i] & 0x7fff);
                const int vb = (pb[i] & 0x8000) ? -(pb[i] & 0x7fff) : (pb[i] & 0x7fff);
                worst = std::max(worst, std::abs(va - vb));
            }
            return worst;
        };
        // QwenRmsNorm (weight offset 1)
        auto o1 = MakeTensor(DataType::BF16, {rows, hidden}); auto r1 = MakeTensor(DataType::BF16, {rows, hidden});
        operators::QwenRmsNormParam np; np.input = tx; np.weight = tg; np.epsilon = te; np.out = o1; np.weight_offset = 1.0f;
        operators::QwenRmsNormParam nr = np; nr.out = r1;
        auto kn = Select(DeviceType::CUDA, DataType::BF16, "QwenRmsNorm", &np);
        // Add (residual) and SiLU
        auto o2 = MakeTensor(DataType::BF16, {rows, hidden}); auto r2 = MakeTensor(DataType::BF16, {rows, hidden});
        operators::BinaryParam ap; ap.lhs = tx; ap.rhs = ty; ap.out = o2;
        operators::BinaryParam ar = ap; ar.out = r2;
        auto ka = Select(DeviceType::CUDA, DataType::BF16, "Add", &ap);
        auto o3 = MakeTensor(DataType::BF16, {rows, hidden}); auto r3 = MakeTensor(DataType::BF16, {rows, hidden});
        operators::UnaryParam sp; sp.input = tx; sp.out = o3;
        operators::UnaryParam sr = sp; sr.out = r3;
        auto ks = Select(DeviceType::CUDA, DataType::BF16, "SiLU", &sp);
        bool ok = kn && ka && ks && IsB200Kernel(kn.get()) && IsB200Kernel(ka.get()) && IsB200Kernel(ks.get());
        if (ok) {
            cuda::DeferredHostSyncScope deferred;
            ok = kn->compute() == 0 && ka->compute() == 0 && ks->compute() == 0 &&
                 cuda::SyncTensorToHostIfNeeded(o1.get(), o1->memory_size(), o1->raw_data()) == 0 &&
                 cuda::SyncTensorToHostIfNeeded(o2.get(), o2->memory_size(), o2->raw_data()) == 0 &&
                 cuda::SyncTensorToHostIfNeeded(o3.get(), o3->memory_size(), o3->raw_data()) == 0;
        }
        ok = ok && RunCommon(DataType::BF16, "QwenRmsNorm", &nr) == 0 && RunCommon(DataType::BF16, "Add", &ar) == 0 && RunCommon(DataType::BF16, "SiLU", &sr) == 0;
        const int d1 = ok ? Steps(o1.get(), r1.get(), rows * hidden) : 99, d2 = ok ? Steps(o2.get(), r2.get(), rows * hidden) : 99,
                  d3 = ok ? Steps(o3.get(), r3.get(), rows * hidden) : 99;
        std::printf("      BF16 codes from COMMON: QwenRmsNorm %d, Add %d, SiLU %d\n", d1, d2, d3);
        CHECK_THAT(ok && d1 <= 1 && d2 == 0 && d3 <= 1, "CUDA QwenRmsNorm / Add / SiLU (BF16) through the reference runtime: within one code / exact / within one code of COMMON");
    }

    // ---- fused FP8 lm-head selection against the reference's own x86 kernel (exact integer data, ties and a NaN row) ----
    {
        const int64_t k = 64, n = 640;
        std::vector<uint8_t> a(static_cast<size_t>(k)), b(static_cast<size_t>(n * k));
        for (auto& v : a) v = FloatToFp8E4M3(static_cast<float>(static_cast<int>(NextRandom() % 5) - 2));
        for (auto& v : b) v = FloatToFp8E4M3(static_cast<float>(static_cast<int>(NextRandom() % 5) - 2));
        for (int64_t row : {int64_t{77}, int64_t{300}, int64_t{639}, int64_t{10}})
            for (int64_t c = 0; c < k; ++c) {
                const float av = Fp8E4M3ToFloat(a[static_cast<size_t>(c)]);
                b[static_cast<size_t>(row * k + c)] = FloatToFp8E4M3(av > 0 ? 2.0f : (av < 0 ? -2.0f : 0.0f));
            }
        b[static_cast<size_t>(10 * k + 3)] = 0x7f;  // row 10 would win but holds a NaN
        auto ta = MakeTensor(DataType::FP8E4M3, {1, k}, a.data()); ta->set_quantization({true, 1.0f});
        auto tb = MakeTensor(DataType::FP8E4M3, {n, k}, b.data()); tb->set_quantization({true, 1.0f}); tb->set_immutable(true);
        auto tok = MakeTensor(DataType::INT64, {1}); auto tok_ref = MakeTensor(DataType::INT64, {1});
        operators::QwenGemmArgmaxParam gp; gp.a = ta; gp.b = tb; gp.out = tok; gp.output_scale = 2.0f;
        operators::QwenGemmArgmaxParam gr = gp; gr.out = tok_ref;
        auto kg = Select(DeviceType::CUDA, DataType::FP8E4M3, "QwenGemmArgmax", &gp);
        bool ok = kg && IsB200Kernel(kg.get()) && kg->Prepare() == 0;
        if (ok) {
            cuda::DeferredHostSyncScope deferred;
            ok = kg->compute() == 0 && cuda::SyncTensorToHostIfNeeded(tok.get(), tok->memory_size(), tok->raw_data()) == 0;
        }
        auto kx = KernelDispatcher::instance().create(DeviceType::X86, DataType::FP8E4M3, "QwenGemmArgmax");
        ok = ok && kx != nullptr;
        if (ok) { kx->SetParam(&gr); ok = kx->Prepare() == 0 && kx->compute() == 0; }
        const long long got = ok ? static_cast<const int64_t*>(tok->raw_data())[0] : -99, want = ok ? static_cast<const int64_t*>(tok_ref->raw_data())[0] : -98;
        std::printf("      token: b200 %lld, reference x86 kernel %lld\n", got, want);
        CHECK_THAT(ok && got == want && got == 77, "CUDA FP8 QwenGemmArgmax selects the token the reference's x86 kernel selects (lowest index among ties, NaN row skipped)");
    }

    // ---- a node built with a scratch budget of zero: same bytes as the node with its own scratch buffer ----
    {
        Fp8Case c1 = MakeFp8(DataType::FP8E4M3, 4, 4096, 8192);
        Fp8Case c0 = c1;
        c0.out = MakeTensor(DataType::FP8E4M3, {4, 8192}); c0.out->set_quantization({true, 0.25f});
        c0.param.out = c0.out;
        auto k1 = Select(DeviceType::CUDA, DataType::FP8E4M3, "MatMul", &c1.param);
        std::unique_ptr<KernelBase> k0;
        {
            KernelSelectionScope budget(KernelFallbackPolicy::kRequireRequested, nullptr, false, 0);
            k0 = KernelDispatcher::instance().create(DeviceType::CUDA, DataType::FP8E4M3, "MatMul");
            if (k0) { k0->SetParam(&c0.param); if (!KernelBase::FinalizeSelection(&k0).ok()) k0.reset(); }
        }
        bool ok = k1 && k0 && IsB200Kernel(k0.get()) && k1->Prepare() == 0 && k0->Prepare() == 0;
        if (ok) {
            cuda::DeferredHostSyncScope deferred;
            ok = k1->compute() == 0 && k0->compute() == 0 &&
                 cuda::SyncTensorToHostIfNeeded(c1.out.get(), c1.out->memory_size(), c1.out->raw_data()) == 0 &&
                 cuda::SyncTensorToHostIfNeeded(c0.out.get(), c0.out->memory_size(), c0.out->raw_data()) == 0;
        }
        CHECK_THAT(ok && std::memcmp(c1.out->raw_data(), c0.out->raw_data(), 4 * 8192) == 0,
                   "workspace limit 0: FP8 MatMul [4,4096]x[4096,8192] runs without allocating scratch and gives the same bytes");
    }
    RunPlansOnGpu();
    CHECK_THAT(fth_b200_device_status() == 0, "no bounded device-side wait gave up");
}

// ---------------------------------------------------------------------------------------------------------
// plans: whole graphs through StaticGraph -> passes -> CompiledGraph -> ExecutionSession, as the runners do
// ---------------------------------------------------------------------------------------------------------
using model::ModelDesc;
using model::NodeDesc;
using model::ValueDesc;
using TensorTable = std::unordered_map<std::string, std::shared_ptr<Tensor>>;

static ValueDesc Value(const std::string& name, std::vector<int64_t> dims, DataType dtype, bool constant = false, float fp8_scale = 0.0f) {
    ValueDesc v;
    v.tensor.name = name;
    v.tensor.dims = std::move(dims);
    v.tensor.data_type = dtype;
    v.constant = constant;
    if (fp8_scale > 0.0f) { v.tensor.quantization.enabled = true; v.tensor.quantization.scale = fp8_scale; }
    return v;
}

// The exporter's projection pattern (tools/export_qwen35_model.py:883-900) twice over one activation:
//   h -> Cast(E5M2) -> MatMul(gate) -> Cast(BF16) -> gate_out ;  h -> Cast(E5M2) -> MatMul(up) -> Cast(BF16) -> up_out
struct Fp8Plan {
    ModelDesc model;
    TensorTable weights;
    std::shared_ptr<Tensor> input;
};
static Fp8Plan MakeFp8Plan() {
    const int64_t hidden = 1024, inter = 3584;
    const float act_scale = 1.0f / 512, w_scale = 1.0f / 1048576, out_scale = 1.0f / 512;
    Fp8Plan p;
    p.model.name = "b200_fp8_projections"; p.model.version = 1; p.model.graph.name = "main";
    p.model.graph.inputs = {"h"};
    p.model.graph.outputs = {"gate_out", "up_out"};
    p.model.graph.values = {Value("h", {1, hidden}, DataType::BF16)};
    std::vector<uint16_t> h(static_cast<size_t>(hidden));
    for (auto& v : h) v = FloatToBFloat16(Uniform(-3, 3));
    p.input = MakeTensor(DataType::BF16, {1, hidden}, h.data());
    for (const char* name : {"gate", "up"}) {
        const std::string n = name;
        std::vector<uint8_t> w(static_cast<size_t>(hidden * inter));
        for (auto& v : w) v = FloatToFp8E5M2(Uniform(-40000, 40000));
        auto wt = MakeTensor(DataType::FP8E5M2, {hidden, inter}, w.data());
        wt->set_quantization({true, w_scale});
        wt->set_immutable(true);
        p.weights[n + "_w"] = wt;
        p.model.graph.values.push_back(Value(n + "_in8", {1, hidden}, DataType::FP8E5M2, false, act_scale));
        p.model.graph.values.push_back(Value(n + "_w", {hidden, inter}, DataType::FP8E5M2, true, w_scale));
        p.model.graph.values.push_back(Value(n + "_out8", {1, inter}, DataType::FP8E5M2, false, out_scale));
        p.model.graph.values.push_back(Value(n + "_out", {1, inter}, DataType::BF16));
        NodeDesc c0; c0.name = n + "_to_fp8"; c0.op_type = "Cast"; c0.inputs = {"h"}; c0.outputs = {n + "_in8"}; c0.attributes["to"] = int64_t{19};
        NodeDesc mm; mm.name = n + "_matmul"; mm.op_type = "MatMul"; mm.inputs = {n + "_in8", n + "_w"}; mm.outputs = {n + "_out8"};
        NodeDesc c1; c1.name = n + "_to_bf16"; c1.op_type = "Cast"; c1.inputs = {n + "_out8"}; c1.outputs = {n + "_out"}; c1.attributes["to"] = int64_t{16};
        p.model.graph.nodes.push_back(c0); p.model.graph.nodes.push_back(mm); p.model.graph.nodes.push_back(c1);
    }
    return p;
}

// The MLP half of a Qwen decoder block as the exporter writes it, every projection wrapped in its two Casts:
//   h = QwenRmsNorm(x, g, eps);  a = Mul(SiLU(gate(h)), up(h));  y = Add(x, down(a))
static Fp8Plan MakeDecoderMlpPlan() {
    const int64_t hidden = 1024, inter = 3584;
    const float act_scale = 1.0f / 512, w_scale = 1.0f / 1048576, out_scale = 1.0f / 512;
    Fp8Plan p;
    p.model.name = "b200_decoder_mlp"; p.model.version = 1; p.model.graph.name = "main";
    p.model.graph.inputs = {"x"};
    p.model.graph.outputs = {"y"};
    p.model.graph.values = {Value("x", {1, hidden}, DataType::BF16), Value("g", {hidden}, DataType::BF16, true), Value("eps", {1}, DataType::FP32, true),
                            Value("h", {1, hidden}, DataType::BF16), Value("s", {1, inter}, DataType::BF16), Value("a", {1, inter}, DataType::BF16),
                            Value("y", {1, hidden}, DataType::BF16)};
    std::vector<uint16_t> x(static_cast<size_t>(hidden)), g(static_cast<size_t>(hidden));
    for (auto& v : x) v = FloatToBFloat16(Uniform(-3, 3));
    for (auto& v : g) v = FloatToBFloat16(Uniform(-0.2f, 0.2f));
    p.input = MakeTensor(DataType::BF16, {1, hidden}, x.data());
    p.weights["g"] = MakeTensor(DataType::BF16, {hidden}, g.data());
    p.weights["g"]->set_immutable(true);
    const float eps = 1e-6f;
    p.weights["eps"] = MakeTensor(DataType::FP32, {1}, &eps);
    p.weights["eps"]->set_immutable(true);
    NodeDesc norm; norm.name = "norm"; norm.op_type = "QwenRmsNorm"; norm.inputs = {"x", "g", "eps"}; norm.outputs = {"h"}; norm.attributes["weight_offset"] = 1.0f;
    p.model.graph.nodes.push_back(norm);
    auto projection = [&](const std::string& n, const std::string& in, int64_t k, int64_t cols, float magnitude) {
        std::vector<uint8_t> w(static_cast<size_t>(k * cols));
        for (auto& v : w) v = FloatToFp8E5M2(Uniform(-magnitude, magnitude));
        auto wt = MakeTensor(DataType::FP8E5M2, {k, cols}, w.data());
        wt->set_quantization({true, w_scale});
        wt->set_immutable(true);
        p.weights[n + "_w"] = wt;
        p.model.graph.values.push_back(Value(n + "_in8", {1, k}, DataType::FP8E5M2, false, act_scale));
        p.model.graph.values.push_back(Value(n + "_w", {k, cols}, DataType::FP8E5M2, true, w_scale));
        p.model.graph.values.push_back(Value(n + "_out8", {1, cols}, DataType::FP8E5M2, false, out_scale));
        p.model.graph.values.push_back(Value(n + "_out", {1, cols}, DataType::BF16));
        NodeDesc c0; c0.name = n + "_to_fp8"; c0.op_type = "Cast"; c0.inputs = {in}; c0.outputs = {n + "_in8"}; c0.attributes["to"] = int64_t{19};
        NodeDesc mm; mm.name = n + "_matmul"; mm.op_type = "MatMul"; mm.inputs = {n + "_in8", n + "_w"}; mm.outputs = {n + "_out8"};
        NodeDesc c1; c1.name = n + "_to_bf16"; c1.op_type = "Cast"; c1.inputs = {n + "_out8"}; c1.outputs = {n + "_out"}; c1.attributes["to"] = int64_t{16};
        p.model.graph.nodes.push_back(c0); p.model.graph.nodes.push_back(mm); p.model.graph.nodes.push_back(c1);
    };
    projection("gate", "h", hidden, inter, 40000.0f);
    projection("up", "h", hidden, inter, 40000.0f);
    NodeDesc silu; silu.name = "silu"; silu.op_type = "SiLU"; silu.inputs = {"gate_out"}; silu.outputs = {"s"};
    NodeDesc mul; mul.name = "mul"; mul.op_type = "Mul"; mul.inputs = {"s", "up_out"}; mul.outputs = {"a"};
    p.model.graph.nodes.push_back(silu); p.model.graph.nodes.push_back(mul);
    projection("down", "a", inter, hidden, 20000.0f);
    NodeDesc add; add.name = "add"; add.op_type = "Add"; add.inputs = {"x", "down_out"}; add.outputs = {"y"};
    p.model.graph.nodes.push_back(add);
    return p;
}

// The front of an attention block: one QwenRmsNorm read by three projections.
static Fp8Plan MakeNormQkvPlan() {
    const int64_t hidden = 1024;
    const float act_scale = 1.0f / 512, w_scale = 1.0f / 1048576, out_scale = 1.0f / 512;
    Fp8Plan p;
    p.model.name = "b200_norm_qkv"; p.model.version = 1; p.model.graph.name = "main";
    p.model.graph.inputs = {"x"};
    p.model.graph.outputs = {"q_out", "k_out", "v_out"};
    p.model.graph.values = {Value("x", {1, hidden}, DataType::BF16), Value("g", {hidden}, DataType::BF16, true), Value("eps", {1}, DataType::FP32, true),
                            Value("h", {1, hidden}, DataType::BF16)};
    std::vector<uint16_t> x(static_cast<size_t>(hidden)), g(static_cast<size_t>(hidden));
    for (auto& v : x) v = FloatToBFloat16(Uniform(-3, 3));
    for (auto& v : g) v = FloatToBFloat16(Uniform(-0.2f, 0.2f));
    p.input = MakeTensor(DataType::BF16, {1, hidden}, x.data());
    p.weights["g"] = MakeTensor(DataType::BF16, {hidden}, g.data());
    p.weights["g"]->set_immutable(true);
    const float eps = 1e-6f;
    p.weights["eps"] = MakeTensor(DataType::FP32, {1}, &eps);
    p.weights["eps"]->set_immutable(true);
    NodeDesc norm; norm.name = "norm"; norm.op_type = "QwenRmsNorm"; norm.inputs = {"x", "g", "eps"}; norm.outputs = {"h"}; norm.attributes["weight_offset"] = 1.0f;
    p.model.graph.nodes.push_back(norm);
    for (const char* name : {"q", "k", "v"}) {
        const std::string n = name;
        std::vector<uint8_t> w(static_cast<size_t>(hidden * hidden));
        for (auto& v : w) v = FloatToFp8E5M2(Uniform(-40000, 40000));
        auto wt = MakeTensor(DataType::FP8E5M2, {hidden, hidden}, w.data());
        wt->set_quantization({true, w_scale});
        wt->set_immutable(true);
        p.weights[n + "_w"] = wt;
        p.model.graph.values.push_back(Value(n + "_in8", {1, hidden}, DataType::FP8E5M2, false, act_scale));
        p.model.graph.values.push_back(Value(n + "_w", {hidden, hidden}, DataType::FP8E5M2, true, w_scale));
        p.model.graph.values.push_back(Value(n + "_out8", {1, hidden}, DataType::FP8E5M2, false, out_scale));
        p.model.graph.values.push_back(Value(n + "_out", {1, hidden}, DataType::BF16));
        NodeDesc c0; c0.name = n + "_to_fp8"; c0.op_type = "Cast"; c0.inputs = {"h"}; c0.outputs = {n + "_in8"}; c0.attributes["to"] = int64_t{19};
        NodeDesc mm; mm.name = n + "_matmul"; mm.op_type = "MatMul"; mm.inputs = {n + "_in8", n + "_w"}; mm.outputs = {n + "_out8"};
        NodeDesc c1; c1.name = n + "_to_bf16"; c1.op_type = "Cast"; c1.inputs = {n + "_out8"}; c1.outputs = {n + "_out"}; c1.attributes["to"] = int64_t{16};
        p.model.graph.nodes.push_back(c0); p.model.graph.nodes.push_back(mm); p.model.graph.nodes.push_back(c1);
    }
    return p;
}

// A float model quantised by the reference's own static quantiser (src/quant/static_quantizer.cc:602-806):
//   x -> Conv2D 3x3 (64 -> 64, bias) -> ReLU -> Flatten -> Gemm (bias) -> y
struct Int8Plan {
    ModelDesc model;
    TensorTable weights;
    std::shared_ptr<Tensor> input;
    StaticQuantizationReport report;
    bool ok{false};
};
static Int8Plan MakeInt8Plan() {
    const int64_t c = 64, h = 8, w = 32, features = c * h * w, classes = 256;
    ModelDesc m;
    m.name = "b200_static_int8"; m.version = 1; m.graph.name = "main";
    m.graph.inputs = {"x"}; m.graph.outputs = {"y"};
    m.graph.values = {Value("x", {1, c, h, w}, DataType::FP32), Value("conv_w", {c, c, 3, 3}, DataType::FP32, true),
                      Value("conv_b", {c}, DataType::FP32, true), Value("conv_out", {1, c, h, w}, DataType::FP32),
                      Value("relu_out", {1, c, h, w}, DataType::FP32), Value("flat", {1, features}, DataType::FP32),
                      Value("fc_w", {features, classes}, DataType::FP32, true), Value("fc_b", {classes}, DataType::FP32, true),
                      Value("y", {1, classes}, DataType::FP32)};
    NodeDesc conv; conv.name = "conv"; conv.op_type = "Conv2D"; conv.inputs = {"x", "conv_w", "conv_b"}; conv.outputs = {"conv_out"};
    conv.attributes["stride_h"] = int64_t{1}; conv.attributes["stride_w"] = int64_t{1}; conv.attributes["pad_h"] = int64_t{1};
    conv.attributes["pad_w"] = int64_t{1}; conv.attributes["dilation_h"] = int64_t{1}; conv.attributes["dilation_w"] = int64_t{1};
    conv.attributes["group"] = int64_t{1};
    NodeDesc relu; relu.name = "relu"; relu.op_type = "ReLU"; relu.inputs = {"conv_out"}; relu.outputs = {"relu_out"};
    NodeDesc flat; flat.name = "flatten"; flat.op_type = "Flatten"; flat.inputs = {"relu_out"}; flat.outputs = {"flat"}; flat.attributes["axis"] = int64_t{1};
    NodeDesc gemm; gemm.name = "classifier"; gemm.op_type = "Gemm"; gemm.inputs = {"flat", "fc_w", "fc_b"}; gemm.outputs = {"y"};
    m.graph.nodes = {conv, relu, flat, gemm};
    TensorTable weights;
    auto Fill = [](std::vector<int64_t> dims, float lo, float hi) {
        size_t count = 1;
        for (int64_t d : dims) count *= static_cast<size_t>(d);
        std::vector<float> v(count);
        for (auto& x : v) x = Uniform(lo, hi);
        return MakeTensor(DataType::FP32, dims, v.data());
    };
    weights["conv_w"] = Fill({c, c, 3, 3}, -0.08f, 0.08f);
    weights["conv_b"] = Fill({c}, -0.5f, 0.5f);
    weights["fc_w"] = Fill({features, classes}, -0.02f, 0.02f);
    weights["fc_b"] = Fill({classes}, -0.5f, 0.5f);
    Int8Plan p;
    p.input = Fill({1, c, h, w}, -2.0f, 2.0f);
    StaticQuantizationConfig config;
    config.strict = true; config.symmetric = true; config.per_channel_weights = true;
    const ActivationQuantization x_q{2.0f / 127, 0}, conv_q{3.0f / 127, 0}, relu_q{2.5f / 127, 0}, y_q{6.0f / 127, 0};
    for (const char* n : {"x"}) config.activations[n] = x_q;
    for (const char* n : {"conv_out", "conv"}) config.activations[n] = conv_q;
    for (const char* n : {"relu_out", "relu", "flat", "flatten"}) config.activations[n] = relu_q;
    for (const char* n : {"y", "classifier"}) config.activations[n] = y_q;
    p.ok = StaticQuantizeModel(m, weights, config, &p.model, &p.weights, &p.report) == 0;
    for (auto& item : p.weights)
        if (item.second) item.second->set_immutable(true);
    return p;
}

// One classifier layer through the same quantiser: x [4,512] -> Gemm (bias) -> y, i.e. QuantizeLinear -> Gemm -> DequantizeLinear.
static Int8Plan MakeInt8GemmPlan() {
    const int64_t m_rows = 4, k = 512, n = 256;
    ModelDesc m;
    m.name = "b200_static_int8_gemm"; m.version = 1; m.graph.name = "main";
    m.graph.inputs = {"x"}; m.graph.outputs = {"y"};
    m.graph.values = {Value("x", {m_rows, k}, DataType::FP32), Value("fc_w", {k, n}, DataType::FP32, true), Value("fc_b", {n}, DataType::FP32, true),
                      Value("y", {m_rows, n}, DataType::FP32)};
    NodeDesc gemm; gemm.name = "classifier"; gemm.op_type = "Gemm"; gemm.inputs = {"x", "fc_w", "fc_b"}; gemm.outputs = {"y"};
    m.graph.nodes = {gemm};
    auto Fill = [](std::vector<int64_t> dims, float lo, float hi) {
        size_t count = 1;
        for (int64_t d : dims) count *= static_cast<size_t>(d);
        std::vector<float> v(count);
        for (auto& x : v) x = Uniform(lo, hi);
        return MakeTensor(DataType::FP32, dims, v.data());
    };
    TensorTable weights;
    weights["fc_w"] = Fill({k, n}, -0.05f, 0.05f);
    weights["fc_b"] = Fill({n}, -0.5f, 0.5f);
    Int8Plan p;
    p.input = Fill({m_rows, k}, -2.0f, 2.0f);
    StaticQuantizationConfig config;
    config.strict = true; config.symmetric = true; config.per_channel_weights = true;
    config.activations["x"] = ActivationQuantization{2.0f / 127, 0};
    for (const char* name : {"y", "classifier"}) config.activations[name] = ActivationQuantization{2.5f / 127, 0};
    p.ok = StaticQuantizeModel(m, weights, config, &p.model, &p.weights, &p.report) == 0;
    for (auto& item : p.weights)
        if (item.second) item.second->set_immutable(true);
    return p;
}

struct PlanRun {
    bool ok{false};
    std::string error;
    std::vector<std::string> op_types;                  // live nodes after the passes, in order
    std::unordered_map<std::string, std::vector<uint8_t>> outputs;
    int b200_kernels{0}, kernels{0};
};

// device COMMON: the reference's canonical kernels.  device CUDA: kRequireRequested, the default pass pipeline plus
// (with_fusion) this backend's pass; `execute` false stops after the passes (host only).
static PlanRun RunPlan(const ModelDesc& model, const TensorTable& weights, const std::string& input_name, const std::shared_ptr<Tensor>& input,
                       DeviceType device, bool with_fusion, bool execute) {
    PlanRun r;
    StaticGraph graph;
    graph.SetKernelDevice(device);
    if (device == DeviceType::CUDA) graph.SetFallbackPolicy(KernelFallbackPolicy::kRequireRequested);
    auto passes = CreateDefaultPassManager();
    if (with_fusion) passes->AddPass(feather::kernel::b200::CreateB200FusionPass());
    graph.SetPassManager(passes);
    if (graph.SetModel(model) != 0 || graph.SetTensor(input_name, input) != 0) { r.error = "SetModel / SetTensor"; return r; }
    for (const auto& item : weights)
        if (graph.SetTensor(item.first, item.second) != 0) { r.error = "SetTensor " + item.first; return r; }
    Status st = graph.BuildStatus();
    if (!st.ok()) { r.error = "build: " + st.message(); return r; }
    st = graph.ApplyPassesStatus();
    if (!st.ok()) { r.error = "passes: " + st.message(); return r; }
    for (const auto& node : graph.nodes())
        if (!node.removed) r.op_types.push_back(node.op_type);
    if (!execute) { r.ok = true; return r; }
    std::shared_ptr<const CompiledGraph> compiled;
    st = CompiledGraph::Compile(graph, &compiled);
    if (!st.ok()) { r.error = "compile: " + st.message(); return r; }
    std::unique_ptr<ExecutionSession> session;
    st = compiled->CreateSession(&session);
    if (!st.ok()) { r.error = "session: " + st.message(); return r; }
    for (int run = 0; run < 2; ++run) {  // the second run reuses resident weights and prepared kernels
        st = session->BindInput(input_name, input);
        if (st.ok()) st = session->Run();
        if (!st.ok()) { r.error = "run: " + st.message(); return r; }
    }
    for (const auto& name : model.graph.outputs) {
        std::shared_ptr<Tensor> out;
        st = session->ReadOutput(name, &out);
        if (!st.ok() || !out) { r.error = "read " + name + ": " + st.message(); return r; }
        const size_t bytes = static_cast<size_t>(out->numel()) * Bytes(out->data_type());
        const uint8_t* p = static_cast<const uint8_t*>(out->raw_data());
        r.outputs[name] = std::vector<uint8_t>(p, p + bytes);
    }
    r.ok = true;
    return r;
}

static int Count(const std::vector<std::string>& ops, const char* type) {
    int n = 0;
    for (const auto& o : ops) n += o == type;
    return n;
}
static std::string Join(const std::vector<std::string>& ops) {
    std::string s;
    for (const auto& o : ops) s += (s.empty() ? "" : " ") + o;
    return s;
}

// host only: the pass rewrites the chains (and leaves alone what the backend would decline)
static void RunPlanRewrite() {
    feather::kernel::b200::RegisterB200Kernels();
    CHECK_THAT(feather::kernel::b200::RegisterB200FusedOperators(), "RegisterB200FusedOperators()");
    {
        Fp8Plan p = MakeFp8Plan();
        PlanRun plain = RunPlan(p.model, p.weights, "h", p.input, DeviceType::CUDA, false, false);
        PlanRun fused = RunPlan(p.model, p.weights, "h", p.input, DeviceType::CUDA, true, false);
        std::printf("      FP8 plan: %s  ->  %s  %s\n", Join(plain.op_types).c_str(), Join(fused.op_types).c_str(), fused.error.c_str());
        CHECK_THAT(plain.ok && plain.op_types.size() == 6 && fused.ok && fused.op_types.size() == 2 && Count(fused.op_types, "FusedCastMatMulCast") == 2,
                   "pass: two Cast -> MatMul -> Cast projections of one activation become two FusedCastMatMulCast nodes (6 nodes -> 2)");
    }
    {
        Fp8Plan p = MakeDecoderMlpPlan();
        PlanRun plain = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, false, false);
        PlanRun fused = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, true, false);
        std::printf("      decoder MLP plan: %s  ->  %s  %s%s\n", Join(plain.op_types).c_str(), Join(fused.op_types).c_str(), plain.error.c_str(), fused.error.c_str());
        CHECK_THAT(plain.ok && plain.op_types.size() == 13 && fused.ok && fused.op_types.size() == 2 && Count(fused.op_types, "FusedCastMatMulCast") == 2,
                   "pass: QwenRmsNorm + gate | up + SiLU * Mul become one node, down + the residual Add another (13 nodes -> 2)");
    }
    {
        Fp8Plan p = MakeNormQkvPlan();
        PlanRun plain = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, false, false);
        PlanRun fused = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, true, false);
        std::printf("      norm + q / k / v plan: %s  ->  %s  %s%s\n", Join(plain.op_types).c_str(), Join(fused.op_types).c_str(), plain.error.c_str(), fused.error.c_str());
        CHECK_THAT(plain.ok && plain.op_types.size() == 10 && fused.ok && fused.op_types.size() == 3 && Count(fused.op_types, "FusedCastMatMulCast") == 3,
                   "pass: a QwenRmsNorm read by three projections moves into each of them (10 nodes -> 3)");
    }
    {
        Int8Plan p = MakeInt8Plan();
        CHECK_THAT(p.ok && p.report.quantized_nodes.size() == 4, "the reference's StaticQuantizeModel quantises Conv2D / ReLU / Flatten / Gemm");
        PlanRun plain = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, false, false);
        PlanRun fused = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, true, false);
        std::printf("      INT8 plan: %s  ->  %s  %s%s\n", Join(plain.op_types).c_str(), Join(fused.op_types).c_str(), plain.error.c_str(), fused.error.c_str());
        CHECK_THAT(plain.ok && fused.ok && Count(fused.op_types, "Conv2DRelu") == 1 && Count(fused.op_types, "ReLU") == 0 &&
                       fused.op_types.size() < plain.op_types.size(),
                   "pass: the quantiser's Conv2D -> ReLU pair becomes one Conv2DRelu node; the plan builds for CUDA under kRequireRequested");
    }
    {
        Int8Plan p = MakeInt8GemmPlan();
        PlanRun plain = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, false, false);
        PlanRun fused = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, true, false);
        std::printf("      INT8 Gemm plan: %s  ->  %s  %s%s\n", Join(plain.op_types).c_str(), Join(fused.op_types).c_str(), plain.error.c_str(), fused.error.c_str());
        CHECK_THAT(p.ok && plain.ok && plain.op_types.size() == 3 && fused.ok && fused.op_types.size() == 1 && Count(fused.op_types, "FusedQLinearDQ") == 1,
                   "pass: the quantiser's QuantizeLinear -> Gemm -> DequantizeLinear becomes one FusedQLinearDQ node");
    }
}

// GPU: the same plans executed; outputs against the COMMON run of the unfused plan
static void RunPlansOnGpu() {
    feather::kernel::b200::RegisterB200FusedOperators();
    {
        Fp8Plan p = MakeFp8Plan();
        PlanRun ref = RunPlan(p.model, p.weights, "h", p.input, DeviceType::COMMON, false, true);
        PlanRun plain = RunPlan(p.model, p.weights, "h", p.input, DeviceType::CUDA, false, true);
        PlanRun fused = RunPlan(p.model, p.weights, "h", p.input, DeviceType::CUDA, true, true);
        bool ok = ref.ok && plain.ok && fused.ok;
        int worst = -1;
        if (ok) {
            worst = 0;
            for (const char* name : {"gate_out", "up_out"}) {
                ok = ok && fused.outputs[name] == plain.outputs[name];  // the fused node returns the bytes of the three-node chain
                const uint16_t* a = reinterpret_cast<const uint16_t*>(fused.outputs[name].data());
                const uint16_t* b = reinterpret_cast<const uint16_t*>(ref.outputs[name].data());
                for (size_t i = 0; i < fused.outputs[name].size() / 2; ++i) {
                    // both are decoded E5M2 codes times a power of two: compare as codes
                    const int ca = CodeIndex(FloatToFp8E5M2(BFloat16ToFloat(a[i]) * 512.0f)), cb = CodeIndex(FloatToFp8E5M2(BFloat16ToFloat(b[i]) * 512.0f));
                    worst = std::max(worst, std::abs(ca - cb));
                }
            }
        }
        std::printf("      FP8 plan on CUDA: %s%s%s; max code distance from the COMMON plan %d\n", ref.error.c_str(), plain.error.c_str(), fused.error.c_str(), worst);
        CHECK_THAT(ok && worst >= 0 && worst <= 1, "FP8 projection plan: fused plan == unfused CUDA plan byte for byte, both within one code of the COMMON plan");
    }
    {
        Fp8Plan p = MakeNormQkvPlan();
        PlanRun plain = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, false, true);
        PlanRun fused = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, true, true);
        bool ok = plain.ok && fused.ok && fused.op_types.size() == 3;
        for (const char* name : {"q_out", "k_out", "v_out"}) ok = ok && fused.outputs[name] == plain.outputs[name] && !fused.outputs[name].empty();
        CHECK_THAT(ok, "norm + q / k / v plan: three launches with the norm inside return the bytes of the ten nodes");
    }
    {
        Fp8Plan p = MakeDecoderMlpPlan();
        PlanRun ref = RunPlan(p.model, p.weights, "x", p.input, DeviceType::COMMON, false, true);
        PlanRun plain = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, false, true);
        PlanRun fused = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, true, true);
        bool ok = ref.ok && plain.ok && fused.ok && fused.op_types.size() == 2;
        int differ_plain = -1, differ_ref = -1;
        double cosine = 0.0;
        if (ok) {
            differ_plain = differ_ref = 0;
            const uint16_t* f = reinterpret_cast<const uint16_t*>(fused.outputs["y"].data());
            const uint16_t* c = reinterpret_cast<const uint16_t*>(plain.outputs["y"].data());
            const uint16_t* r = reinterpret_cast<const uint16_t*>(ref.outputs["y"].data());
            double dot = 0, nf = 0, nr = 0;
            for (size_t i = 0; i < fused.outputs["y"].size() / 2; ++i) {
                differ_plain += f[i] != c[i];
                differ_ref += f[i] != r[i];
                const double a = BFloat16ToFloat(f[i]), b = BFloat16ToFloat(r[i]);
                dot += a * b; nf += a * a; nr += b * b;
            }
            cosine = dot / std::sqrt(nf * nr);
        }
        std::printf("      decoder MLP plan on CUDA (%zu nodes fused to %zu): %d outputs differ from the node-by-node CUDA plan, %d from the COMMON plan (cosine %.6f) %s%s%s\n",
                    plain.op_types.size(), fused.op_types.size(), differ_plain, differ_ref, cosine, ref.error.c_str(), plain.error.c_str(), fused.error.c_str());
        CHECK_THAT(ok && differ_plain == 0 && cosine >= 0.9999,
                   "decoder MLP plan: the two fused launches return the bytes of the thirteen nodes, and the COMMON plan's result up to single codes");
    }
    {
        Int8Plan p = MakeInt8Plan();
        PlanRun ref = RunPlan(p.model, p.weights, "x", p.input, DeviceType::COMMON, false, true);
        PlanRun plain = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, false, true);
        PlanRun fused = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, true, true);
        const bool ok = p.ok && ref.ok && plain.ok && fused.ok;
        std::printf("      INT8 plan on CUDA: %s%s%s\n", ref.error.c_str(), plain.error.c_str(), fused.error.c_str());
        CHECK_THAT(ok && plain.outputs["y"] == ref.outputs["y"], "statically quantised plan (the reference's own quantiser) on CUDA under kRequireRequested: identical to COMMON");
        CHECK_THAT(ok && fused.outputs["y"] == ref.outputs["y"], "the same plan with Conv2D -> ReLU fused by the pass: identical to COMMON");
    }
    {
        // two sessions of one compiled plan share one packed copy of the conv weight; it goes away with the last session
        Int8Plan p = MakeInt8Plan();
        StaticGraph graph;
        graph.SetKernelDevice(DeviceType::CUDA);
        graph.SetFallbackPolicy(KernelFallbackPolicy::kRequireRequested);
        auto passes = CreateDefaultPassManager();
        passes->AddPass(feather::kernel::b200::CreateB200FusionPass());
        graph.SetPassManager(passes);
        bool ok = p.ok && graph.SetModel(p.model) == 0 && graph.SetTensor("x", p.input) == 0;
        for (const auto& item : p.weights) ok = ok && graph.SetTensor(item.first, item.second) == 0;
        ok = ok && graph.BuildStatus().ok() && graph.ApplyPassesStatus().ok();
        std::shared_ptr<const CompiledGraph> compiled;
        ok = ok && CompiledGraph::Compile(graph, &compiled).ok();
        size_t during = 0;
        std::vector<uint8_t> first_out, second_out;
        if (ok) {
            std::unique_ptr<ExecutionSession> first, second;
            ok = compiled->CreateSession(&first).ok() && compiled->CreateSession(&second).ok();
            for (auto* session : {first.get(), second.get()}) {
                if (!ok) break;
                ok = session->BindInput("x", p.input).ok() && session->Run().ok();
                std::shared_ptr<Tensor> out;
                ok = ok && session->ReadOutput("y", &out).ok() && out != nullptr;
                if (ok) {
                    const uint8_t* b = static_cast<const uint8_t*>(out->raw_data());
                    (session == first.get() ? first_out : second_out).assign(b, b + out->numel() * 4);
                }
            }
            during = feather::kernel::b200::PackedConvWeightEntries();
        }
        const size_t after = feather::kernel::b200::PackedConvWeightEntries();
        std::printf("      packed conv weights alive: %zu with two sessions, %zu after both are gone\n", during, after);
        CHECK_THAT(ok && during == 1 && after == 0 && first_out == second_out && !first_out.empty(),
                   "two sessions of one plan share ONE packed copy of the conv weight (packed once per weight, not per session)");
    }
    {
        Int8Plan p = MakeInt8GemmPlan();
        PlanRun ref = RunPlan(p.model, p.weights, "x", p.input, DeviceType::COMMON, false, true);
        PlanRun plain = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, false, true);
        PlanRun fused = RunPlan(p.model, p.weights, "x", p.input, DeviceType::CUDA, true, true);
        std::printf("      INT8 Gemm plan on CUDA: %s%s%s\n", ref.error.c_str(), plain.error.c_str(), fused.error.c_str());
        if (ref.ok && plain.ok && fused.ok) {
            const float* r = reinterpret_cast<const float*>(ref.outputs["y"].data());
            const float* u = reinterpret_cast<const float*>(plain.outputs["y"].data());
            const float* f = reinterpret_cast<const float*>(fused.outputs["y"].data());
            const size_t count = ref.outputs["y"].size() / 4;
            int du = 0, df = 0, shown = 0;
            for (size_t i = 0; i < count; ++i) {
                du += u[i] != r[i];
                if (f[i] != r[i]) {
                    ++df;
                    if (shown++ < 6) std::printf("        y[%zu]: COMMON %.6f, unfused CUDA %.6f, fused %.6f\n", i, r[i], u[i], f[i]);
                }
            }
            std::printf("      of %zu outputs: unfused CUDA plan differs in %d, fused plan in %d\n", count, du, df);
        }
        CHECK_THAT(p.ok && ref.ok && fused.ok && fused.outputs["y"] == ref.outputs["y"],
                   "QuantizeLinear -> Gemm -> DequantizeLinear as one FusedQLinearDQ node on CUDA: identical to the three COMMON nodes");
    }
}

// ---------------------------------------------------------------------------------------------------------
// time: the same MatMul nodes through the reference runtime, on whichever CUDA candidate is selected
// ---------------------------------------------------------------------------------------------------------
template <typename Case>
static void TimeNode(const char* what, DataType dtype, Case* c, int repeats) {
    auto k = Select(DeviceType::CUDA, dtype, "MatMul", &c->param);
    if (!k || k->Prepare() != 0) { std::printf("time  %s: no kernel\n", what); ++g_failures; return; }
    cuda::DeferredHostSyncScope deferred;
    for (int i = 0; i < 3; ++i) k->compute();
    cuda::SynchronizeInferenceStream();
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaEventRecord(e0, cuda::InferenceStream());
    int rc = 0;
    for (int i = 0; i < repeats; ++i) rc |= k->compute();
    cudaEventRecord(e1, cuda::InferenceStream());
    cudaEventSynchronize(e1);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    std::printf("time  %s: %.2f us per compute() on %s (%s), rc %d\n", what, ms * 1000.0f / repeats,
                IsB200Kernel(k.get()) ? "the b200 candidate" : "the reference CUDA kernel", IsB200Kernel(k.get()) ? fth_b200_last_variant() : "reference", rc);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
}

static void RunTime() {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) { std::printf("skip  no CUDA device\n"); return; }
    const bool registered = feather::kernel::b200::RegisterB200Kernels();
    std::printf("time  b200 candidates %s\n", registered ? "registered" : "disabled (FEATHER_DISABLE_B200=1): reference CUDA kernels");
    auto context = cuda::CreateExecutionContext();
    cuda::ExecutionContextScope scope(context);
    { Fp8Case c = MakeFp8(DataType::FP8E4M3, 1, 1024, 3072); TimeNode("FP8E4M3 MatMul M=1 K=1024 N=3072 (config 1)", DataType::FP8E4M3, &c, 200); }
    { Fp8Case c = MakeFp8(DataType::FP8E4M3, 1, 8192, 28672); TimeNode("FP8E4M3 MatMul M=1 K=8192 N=28672 (config 5)", DataType::FP8E4M3, &c, 50); }
    { Fp8Case c = MakeFp8(DataType::FP8E4M3, 256, 8192, 8192); TimeNode("FP8E4M3 MatMul M=256 K=8192 N=8192", DataType::FP8E4M3, &c, 20); }
    { Int8Case c = MakeInt8(128, 1024, 1024); TimeNode("INT8 MatMul M=128 K=1024 N=1024 per-channel (config 2)", DataType::INT8, &c, 50); }
    { Int8Case c = MakeInt8(1, 8192, 28672); TimeNode("INT8 MatMul M=1 K=8192 N=28672 per-channel (config 5)", DataType::INT8, &c, 20); }
}

// ---------------------------------------------------------------------------------------------------------
// shard: one process, one CudaExecutionContext per GPU, a column-sharded MatMul node per rank on the B200 candidates,
// gathered through a ShardGroup (infer_b200/adapter/b200_shard.h).  Needs two GPUs.
// ---------------------------------------------------------------------------------------------------------
template <typename Case>
static void RunShardCase(const char* what, DataType dt, Case& full, int64_t m, int64_t k, int64_t n, int world) {
    using feather::kernel::b200::ShardBindingScope;
    using feather::kernel::b200::ShardGroup;
    // the unsharded node on GPU 0 is the reference for the bytes
    std::vector<uint8_t> want(static_cast<size_t>(m * n));
    bool ok = true;
    {
        (void)cudaSetDevice(0);
        auto context = cuda::CreateExecutionContext();
        cuda::ExecutionContextScope scope(context);
        auto kernel = Select(DeviceType::CUDA, dt, "MatMul", &full.param);
        ok = kernel && IsB200Kernel(kernel.get()) && kernel->Prepare() == 0 && kernel->compute() == 0;
        if (ok) std::memcpy(want.data(), full.out->raw_data(), want.size());
    }
    std::vector<int> devices;
    for (int r = 0; r < world; ++r) devices.push_back(r);
    auto group = ShardGroup::Create(devices, m, n);
    ok = ok && group != nullptr;
    struct Rank {
        std::shared_ptr<cuda::CudaExecutionContext> context;
        std::shared_ptr<Tensor> a, w, out;
        operators::MatMulParam param;
        std::unique_ptr<KernelBase> kernel;
    };
    std::vector<Rank> ranks(static_cast<size_t>(world));
    for (int r = 0; r < world && ok; ++r) {
        Rank& R = ranks[static_cast<size_t>(r)];
        const auto cols = group->Columns(r);
        const int64_t width = cols.second - cols.first;
        std::vector<uint8_t> slice(static_cast<size_t>(k * width));
        const uint8_t* w = static_cast<const uint8_t*>(full.w->raw_data());
        for (int64_t row = 0; row < k; ++row) std::memcpy(&slice[static_cast<size_t>(row * width)], w + row * n + cols.first, static_cast<size_t>(width));
        R.w = MakeTensor(dt, {k, width}, slice.data());
        QuantizationParams wq = full.w->quantization();
        if (wq.granularity == QuantizationGranularity::kPerChannel) {
            wq.scales.assign(wq.scales.begin() + cols.first, wq.scales.begin() + cols.second);
            wq.zero_points.assign(wq.zero_points.begin() + cols.first, wq.zero_points.begin() + cols.second);
            wq.scale = wq.scales.front();
        }
        R.w->set_quantization(wq);
        R.w->set_immutable(true);
        R.out = MakeTensor(dt, {m, width});
        R.out->set_quantization(full.out->quantization());
        R.a = MakeTensor(dt, {m, k}, full.a->raw_data());  // the activation is replicated: every rank has its own copy
        R.a->set_quantization(full.a->quantization());
        R.param.a = R.a; R.param.b = R.w; R.param.out = R.out;
        ok = cudaSetDevice(group->device(r)) == cudaSuccess;
        R.context = cuda::CreateExecutionContext();  // records the GPU that is current when its stream is first created
        cuda::ExecutionContextScope scope(R.context);
        R.kernel = Select(DeviceType::CUDA, dt, "MatMul", &R.param);
        ok = ok && R.kernel && IsB200Kernel(R.kernel.get()) && R.kernel->Prepare() == 0;
    }
    int wrong_gathered = 0, wrong_block = 0, status = 0;
    for (int step = 1; step <= 3 && ok; ++step) {
        group->NextStep();
        for (int r = 0; r < world && ok; ++r) {
            Rank& R = ranks[static_cast<size_t>(r)];
            cuda::ExecutionContextScope scope(R.context);
            ShardBindingScope bind(group, r);
            ok = R.kernel->compute() == 0;
        }
        for (int r = 0; r < world && ok; ++r) {
            Rank& R = ranks[static_cast<size_t>(r)];
            cuda::ExecutionContextScope scope(R.context);
            std::vector<uint8_t> gathered(want.size());
            ok = group->Wait(r, cuda::InferenceStream()) == FTH_B200_OK && cuda::SynchronizeInferenceStream() == 0 &&
                 cudaMemcpy(gathered.data(), group->Buffer(r, group->Parity()), gathered.size(), cudaMemcpyDeviceToHost) == cudaSuccess;
            status |= fth_b200_device_status();
            for (size_t i = 0; i < want.size(); ++i) wrong_gathered += gathered[i] != want[i];
            const auto cols = group->Columns(r);
            const int64_t width = cols.second - cols.first;
            const uint8_t* block = static_cast<const uint8_t*>(R.out->raw_data());
            for (int64_t row = 0; row < m; ++row)
                for (int64_t c = 0; c < width; ++c) wrong_block += block[row * width + c] != want[static_cast<size_t>(row * n + cols.first + c)];
            if (ok) (void)cudaMemset(group->Buffer(r, group->Parity()), 0x5A, want.size());  // the next use of this parity must rewrite it
        }
    }
    for (auto& R : ranks) {
        if (!R.context) continue;
        cuda::ExecutionContextScope scope(R.context);
        R.kernel.reset();
    }
    (void)cudaSetDevice(0);
    std::printf("      %s on %d GPUs: %d gathered bytes and %d bytes of the nodes' own outputs differ from the unsharded node; device status %d\n",
                what, world, wrong_gathered, wrong_block, status);
    CHECK_THAT(ok && wrong_gathered == 0 && wrong_block == 0 && status == 0, what);
}

static void RunShard() {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count < 2) {
        std::printf("skip  fewer than two CUDA devices\n");
        return;
    }
    feather::kernel::b200::RegisterB200Kernels();
    const int world = count >= 4 ? 4 : 2;
    {
        Fp8Case c = MakeFp8(DataType::FP8E4M3, 1, 4096, 8192);
        RunShardCase("column-sharded FP8 MatMul [1,4096]x[4096,8192] (single-launch kernel): every rank's gathered row == the unsharded node", DataType::FP8E4M3, c, 1, 4096, 8192, world);
    }
    {
        Fp8Case c = MakeFp8(DataType::FP8E5M2, 16, 8192, 16384);
        RunShardCase("column-sharded FP8 MatMul [16,8192]x[8192,16384] (weight stream + reduce pass)", DataType::FP8E5M2, c, 16, 8192, 16384, world);
    }
    {
        Fp8Case c = MakeFp8(DataType::FP8E4M3, 300, 512, 2048);
        RunShardCase("column-sharded FP8 MatMul [300,512]x[512,2048] (dense kernel, tile stores into the other GPUs)", DataType::FP8E4M3, c, 300, 512, 2048, world);
    }
    {
        Int8Case c = MakeInt8(8, 1024, 4096);
        RunShardCase("column-sharded INT8 MatMul [8,1024]x[1024,4096], per-channel scales sliced with the columns", DataType::INT8, c, 8, 1024, 4096, world);
    }
}

int main(int argc, char** argv) {
    const std::string mode = argc > 1 ? argv[1] : "select";
    if (mode == "select") { RunSelect(); RunPlanRewrite(); }
    else if (mode == "run") RunGpu();
    else if (mode == "time") RunTime();
    else if (mode == "shard") RunShard();
    else { std::fprintf(stderr, "usage: adapter_e2e select|run|time\n"); return 2; }
    std::printf("%s: %d failure(s)\n", mode.c_str(), g_failures);
    return g_failures == 0 ? 0 : 1;
}
