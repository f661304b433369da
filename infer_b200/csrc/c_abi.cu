// C ABI entry points for the linear ops: validation (the contract checks of the reference kernels),
// shape split between kernel families, launch bookkeeping.
#include <cmath>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "linear_internal.h"

namespace fth {

namespace {
thread_local const char* g_last_variant = "none";
thread_local int64_t g_launches = 0;
}  // namespace

void NoteLaunch(const char* variant, int64_t launches) {
    g_last_variant = variant;
    g_launches += launches;
}

int CheckLaunch() { return cudaGetLastError() == cudaSuccess ? FTH_B200_OK : FTH_B200_ERR_CUDA; }
// A non-sticky error some other library left behind in this thread (NCCL's peer-access probes do) must not be blamed on
// the next launch here: every entry point that launches starts by discarding it.
void ClearStaleError() { (void)cudaGetLastError(); }

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
int g_sm_count[kMaxDevices] = {};
struct SmemOptIn { const void* kernel; int device; size_t bytes; };
std::vector<SmemOptIn> g_smem_opt_in;
}  // namespace

int SmCount() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return kNumSms;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_sm_count[device] == 0) {
        int count = 0;
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) count = kNumSms;
        g_sm_count[device] = count;
    }
    return g_sm_count[device];
}

int EnsureDynamicSmem(const void* kernel, size_t bytes) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return FTH_B200_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    for (SmemOptIn& e : g_smem_opt_in) {
        if (e.kernel == kernel && e.device == device) {
            if (e.bytes >= bytes) return FTH_B200_OK;
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) != cudaSuccess) return FTH_B200_ERR_CUDA;
            e.bytes = bytes;
            return FTH_B200_OK;
        }
    }
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) != cudaSuccess) return FTH_B200_ERR_CUDA;
    g_smem_opt_in.push_back(SmemOptIn{kernel, device, bytes});
    return FTH_B200_OK;
}

namespace {

bool ValidScale(float s) { return std::isfinite(s) && s > 0.0f; }  // fp8_host.h:150-157, quantization.h:64-66
bool IsFp8(int dtype) { return dtype == FTH_B200_FP8E4M3 || dtype == FTH_B200_FP8E5M2; }

int ValidateFp8(const fth_b200_fp8_linear_desc* d) {
    if (d == nullptr || !IsFp8(d->dtype)) return FTH_B200_ERR_INVALID;
    if (d->m <= 0 || d->k <= 0 || d->n <= 0 || !d->a || !d->w || !d->out) return FTH_B200_ERR_INVALID;
    if (d->op < FTH_B200_OP_FC || d->op > FTH_B200_OP_GEMM) return FTH_B200_ERR_INVALID;
    if (!ValidScale(d->a_scale) || !ValidScale(d->out_scale)) return FTH_B200_ERR_INVALID;
    if (d->w_channel_scales == nullptr && !ValidScale(d->w_scale)) return FTH_B200_ERR_INVALID;
    if (d->bias_mode < FTH_B200_BIAS_NONE || d->bias_mode > FTH_B200_BIAS_MATRIX) return FTH_B200_ERR_INVALID;
    if (d->bias_mode != FTH_B200_BIAS_NONE && (!d->bias || !ValidScale(d->bias_scale))) return FTH_B200_ERR_INVALID;
    if (d->op == FTH_B200_OP_MATMUL && d->bias_mode != FTH_B200_BIAS_NONE) return FTH_B200_ERR_INVALID;
    if (d->op == FTH_B200_OP_GEMM && (!std::isfinite(d->alpha) || !std::isfinite(d->beta))) return FTH_B200_ERR_INVALID;
    if (d->trans_b && d->op != FTH_B200_OP_GEMM) return FTH_B200_ERR_INVALID;  // only GemmParam has trans_b
    if (d->a_dtype != 0 && d->a_dtype != d->dtype && d->a_dtype != FTH_B200_BF16 && d->a_dtype != FTH_B200_FP32) return FTH_B200_ERR_UNSUPPORTED;
    if (d->out_dtype != 0 && d->out_dtype != d->dtype && d->out_dtype != FTH_B200_BF16 && d->out_dtype != FTH_B200_FP32) return FTH_B200_ERR_UNSUPPORTED;
    if (d->ldo != 0 && d->ldo < d->n) return FTH_B200_ERR_INVALID;
    if (d->m > (int64_t{1} << 31) || d->n > (int64_t{1} << 31) || d->k > (int64_t{1} << 31)) return FTH_B200_ERR_UNSUPPORTED;
    return FTH_B200_OK;
}

int ValidateInt8(const fth_b200_int8_linear_desc* d) {
    if (d == nullptr) return FTH_B200_ERR_INVALID;
    if (d->m <= 0 || d->k <= 0 || d->n <= 0 || !d->a || !d->w || !d->out || !d->w_scales) return FTH_B200_ERR_INVALID;
    if (d->op < FTH_B200_OP_FC || d->op > FTH_B200_OP_GEMM) return FTH_B200_ERR_INVALID;
    if (!ValidScale(d->a_scale) || !ValidScale(d->out_scale)) return FTH_B200_ERR_INVALID;
    if (d->a_zp < -128 || d->a_zp > 127 || d->out_zp < -128 || d->out_zp > 127) return FTH_B200_ERR_INVALID;
    if (d->w_params != 1 && d->w_params != d->n) return FTH_B200_ERR_INVALID;
    if (d->bias_mode < FTH_B200_BIAS_NONE || d->bias_mode > FTH_B200_BIAS_MATRIX) return FTH_B200_ERR_INVALID;
    if (d->bias_mode != FTH_B200_BIAS_NONE && !d->bias) return FTH_B200_ERR_INVALID;
    if (d->op == FTH_B200_OP_MATMUL && d->bias_mode != FTH_B200_BIAS_NONE) return FTH_B200_ERR_INVALID;
    if (d->op == FTH_B200_OP_GEMM && (!std::isfinite(d->alpha) || !std::isfinite(d->beta))) return FTH_B200_ERR_INVALID;
    if (d->trans_b && d->op != FTH_B200_OP_GEMM) return FTH_B200_ERR_INVALID;
    if (d->a_dtype != 0 && d->a_dtype != FTH_B200_INT8 && d->a_dtype != FTH_B200_FP32) return FTH_B200_ERR_UNSUPPORTED;
    if (d->out_dtype != 0 && d->out_dtype != FTH_B200_INT8 && d->out_dtype != FTH_B200_FP32) return FTH_B200_ERR_UNSUPPORTED;
    if (d->ldo != 0 && d->ldo < d->n) return FTH_B200_ERR_INVALID;
    if (d->w_zp_max_abs < 0 || d->w_zp_max_abs > 128 || d->bias_max_abs < 0) return FTH_B200_ERR_INVALID;
    // Every running sum must stay inside int32 (FitsInt32 after each term, int8_kernel_utils.h:99-114).
    // Decide it on the host from the worst case, as the reference's x86 path does (x86/int8.cc:1963-1980),
    // so that no device-side error flag or synchronisation is needed.
    if (d->k > (int64_t{1} << 31)) return FTH_B200_ERR_OVERFLOW;  // also keeps the product below from wrapping
    const int64_t a_span = 128 + (d->a_zp < 0 ? -d->a_zp : d->a_zp);
    const int64_t w_span = 128 + d->w_zp_max_abs;
    const int64_t worst = d->k * a_span * w_span + d->bias_max_abs;
    if (worst > 2147483647LL) return FTH_B200_ERR_OVERFLOW;
    if (d->m > (int64_t{1} << 31) || d->n > (int64_t{1} << 31)) return FTH_B200_ERR_UNSUPPORTED;
    return FTH_B200_OK;
}

bool Tcgen05Usable(int dtype, const LinearArgs& args, const void* workspace, size_t workspace_bytes) {
    if (!Tcgen05Supported(dtype, args)) return false;
    const size_t need = Tcgen05ScratchBytes(dtype, args);
    return need == 0 || (workspace != nullptr && workspace_bytes >= need);
}

bool StreamUsable(int dtype, const LinearArgs& args, const void* workspace, size_t workspace_bytes) {
    if (!StreamSupported(dtype, args)) return false;
    const size_t need = StreamScratchBytes(dtype, args);
    return need == 0 || (workspace != nullptr && workspace_bytes >= need);
}

int PickVariant(int requested, int dtype, const LinearArgs& args, const void* workspace, size_t workspace_bytes) {
    if (requested == FTH_B200_VARIANT_SIMT) return FTH_B200_VARIANT_SIMT;
    if (requested == FTH_B200_VARIANT_SKINNY) return SkinnySupported(dtype, args) ? requested : FTH_B200_ERR_UNSUPPORTED;
    if (requested == FTH_B200_VARIANT_TCGEN05) {
        if (!Tcgen05Supported(dtype, args)) return FTH_B200_ERR_UNSUPPORTED;
        return Tcgen05Usable(dtype, args, workspace, workspace_bytes) ? requested : FTH_B200_ERR_INVALID;
    }
    if (requested == FTH_B200_VARIANT_STREAM) {
        if (!StreamSupported(dtype, args)) return FTH_B200_ERR_UNSUPPORTED;
        return StreamUsable(dtype, args, workspace, workspace_bytes) ? requested : FTH_B200_ERR_INVALID;
    }
    if (requested != FTH_B200_VARIANT_AUTO) return FTH_B200_ERR_INVALID;
    // Shape split.  Every shape TMA can address runs on the tensor cores: decode shapes (M <= 128) with the
    // weights on the 128 TMEM lanes, where the kernel is a pure HBM weight stream; dense shapes with 128 x 256
    // tiles.  Shapes the tensor-core kernel declines (fused Cast / QuantizeLinear prologue, zero points,
    // strides TMA cannot express, no scratch) stream on the CUDA cores; ragged leftovers take the tile kernel.
    if (Tcgen05Usable(dtype, args, workspace, workspace_bytes)) return FTH_B200_VARIANT_TCGEN05;
    if (StreamUsable(dtype, args, workspace, workspace_bytes)) return FTH_B200_VARIANT_STREAM;
    if (SkinnySupported(dtype, args)) return FTH_B200_VARIANT_SKINNY;
    return FTH_B200_VARIANT_SIMT;
}

int Dispatch(int variant, int dtype, const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie,
             void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    switch (variant) {
        case FTH_B200_VARIANT_SIMT: return LaunchLinearSimt(dtype, args, fe, ie, stream);
        case FTH_B200_VARIANT_SKINNY: return LaunchLinearSkinny(dtype, args, fe, ie, stream);
        case FTH_B200_VARIANT_TCGEN05: return LaunchLinearTcgen05(dtype, args, fe, ie, workspace, workspace_bytes, stream);
        case FTH_B200_VARIANT_STREAM: return LaunchLinearStream(dtype, args, fe, ie, workspace, workspace_bytes, stream);
        default: return variant;  // negative status from PickVariant
    }
}

// Scratch the kernel family that will run needs: AUTO takes the tensor-core kernels whenever they support the shape
// (they never fall back to the TMA-ring GEMV then), so only their need counts.
size_t WorkspaceFor(int variant, int dtype, const LinearArgs& args) {
    const bool tc = Tcgen05Supported(dtype, args);
    const size_t tc_bytes = tc ? Tcgen05ScratchBytes(dtype, args) : 0;
    const size_t stream_bytes = StreamSupported(dtype, args) ? StreamScratchBytes(dtype, args) : 0;
    if (variant == FTH_B200_VARIANT_TCGEN05) return tc_bytes;
    if (variant == FTH_B200_VARIANT_STREAM) return stream_bytes;
    if (variant == FTH_B200_VARIANT_AUTO) return tc ? tc_bytes : stream_bytes;
    return 0;
}

// Peer replicas of the output: byte distance from the local output to each peer's copy.
template <typename Desc>
int BuildPeers(const Desc* d, PeerOut* peers) {
    peers->count = 0;
    peers->multicast_delta = 0;
    if (d->gather_peers < 0 || d->gather_peers > kMaxPeers) return FTH_B200_ERR_INVALID;
    for (int r = 0; r < d->gather_peers; ++r) {
        if (d->gather_out[r] == nullptr) return FTH_B200_ERR_INVALID;
        peers->delta[r] = static_cast<int64_t>(reinterpret_cast<intptr_t>(d->gather_out[r]) - reinterpret_cast<intptr_t>(d->out));
    }
    peers->count = d->gather_peers;
    if (d->gather_peers > 0 && d->gather_multicast_out != nullptr)
        peers->multicast_delta = static_cast<int64_t>(reinterpret_cast<intptr_t>(d->gather_multicast_out) - reinterpret_cast<intptr_t>(d->out));
    return FTH_B200_OK;
}

template <typename Desc>
int BuildSignal(const Desc* d, GatherSignal* signal) {
    *signal = GatherSignal{};
    if (d->gather_world == 0) return FTH_B200_OK;
    if (d->gather_world < 1 || d->gather_world > kMaxPeers + 1 || d->gather_rank < 0 || d->gather_rank >= d->gather_world) return FTH_B200_ERR_INVALID;
    for (int r = 0; r < d->gather_world; ++r) {
        if (d->gather_flags[r] == nullptr) return FTH_B200_ERR_INVALID;
        signal->flags[r] = static_cast<uint32_t*>(d->gather_flags[r]);
    }
    signal->world = d->gather_world;
    signal->rank = d->gather_rank;
    return FTH_B200_OK;
}

// Runs the chosen kernel family; when the output has peer replicas and that kernel does not write them itself, a
// block copy follows on the same stream.  Gather signalling the kernel does not fold in becomes two small kernels
// around it: wait for the peers' previous step in front, publish this step behind the last store.
int Run(int variant, int dtype, const LinearArgs& args_in, const Fp8Epilogue& fe, const Int8Epilogue& ie, void* workspace,
        size_t workspace_bytes, cudaStream_t stream) {
    if (variant < 0) return variant;
    LinearArgs args = args_in;
    const bool signalling = args.signal.world > 0;
    const bool stores_peers = variant == FTH_B200_VARIANT_TCGEN05 && Tcgen05StoresToPeers(dtype, args, fe, ie);
    const bool folded = signalling && variant == FTH_B200_VARIANT_TCGEN05 && Tcgen05SignalsInKernel(dtype, args, fe, ie);
    if (signalling && !folded) {
        args.signal.world = 0;
        const int rc = LaunchGatherWaitPrevious(args_in.signal, stream);
        if (rc != FTH_B200_OK) return rc;
    }
    int rc = Dispatch(variant, dtype, args, fe, ie, workspace, workspace_bytes, stream);
    if (rc != FTH_B200_OK) return rc;
    if (args.peers.count > 0 && !stores_peers) {
        const bool int8 = dtype == FTH_B200_INT8;
        const int out_dtype = int8 ? ie.out_dtype : fe.out_dtype;
        const int elem = out_dtype == FTH_B200_FP32 ? 4 : (out_dtype == FTH_B200_BF16 || out_dtype == FTH_B200_FP16) ? 2 : 1;
        rc = LaunchPeerCopy(int8 ? ie.out : fe.out, args.m, args.n, int8 ? ie.ldo : fe.ldo, elem, args.peers, stream);
        if (rc != FTH_B200_OK) return rc;
    }
    if (signalling && !folded) return LaunchGatherPublish(args_in.signal, stream);
    return FTH_B200_OK;
}

void BuildFp8(const fth_b200_fp8_linear_desc* d, LinearArgs* args, Fp8Epilogue* fe) {
    args->a = d->a; args->w = d->w; args->m = d->m; args->k = d->k; args->n = d->n; args->trans_b = d->trans_b;
    args->a_dtype = (d->a_dtype == d->dtype) ? 0 : d->a_dtype;
    args->a_scale = d->a_scale;
    args->zero_points = 0;
    args->w_static = d->weights_static != 0;
    args->peers.count = 0;
    args->argmax_keys = nullptr;
    args->signal = GatherSignal{};
    args->fusion = DecoderFusion{};
    fe->ab_scale = d->w_channel_scales ? d->a_scale : d->a_scale * d->w_scale;
    fe->w_channel_scales = d->w_channel_scales;
    fe->is_gemm = d->op == FTH_B200_OP_GEMM;
    fe->alpha = fe->is_gemm ? d->alpha : 1.0f;
    fe->beta = fe->is_gemm ? d->beta : 1.0f;
    fe->bias = static_cast<const uint8_t*>(d->bias);
    fe->bias_mode = d->bias_mode;
    fe->bias_scale = d->bias_scale;
    fe->out_scale = d->out_scale;
    fe->out = d->out;
    fe->out_dtype = (d->out_dtype == d->dtype) ? 0 : d->out_dtype;
    fe->ldo = d->ldo ? d->ldo : d->n;
    fe->n = d->n;
}

void BuildInt8(const fth_b200_int8_linear_desc* d, LinearArgs* args, Int8Epilogue* ie) {
    args->a = d->a; args->w = d->w; args->m = d->m; args->k = d->k; args->n = d->n; args->trans_b = d->trans_b;
    args->a_dtype = (d->a_dtype == FTH_B200_INT8) ? 0 : d->a_dtype;
    args->a_scale = d->a_scale;
    args->zero_points = (d->a_zp != 0 || d->w_zps != nullptr) ? 1 : 0;
    args->w_static = d->weights_static != 0;
    args->peers.count = 0;
    args->argmax_keys = nullptr;
    args->signal = GatherSignal{};
    args->fusion = DecoderFusion{};
    ie->w_scales = d->w_scales; ie->w_zps = d->w_zps; ie->per_channel = d->w_params != 1;
    ie->a_scale = d->a_scale; ie->a_zp = d->a_zp; ie->out_scale = d->out_scale; ie->out_zp = d->out_zp;
    ie->bias = d->bias; ie->bias_mode = d->bias_mode;
    ie->is_gemm = d->op == FTH_B200_OP_GEMM;
    ie->alpha = ie->is_gemm ? d->alpha : 1.0f;
    ie->beta = ie->is_gemm ? d->beta : 1.0f;
    ie->out = d->out;
    ie->out_dtype = (d->out_dtype == FTH_B200_INT8) ? 0 : d->out_dtype;
    ie->ldo = d->ldo ? d->ldo : d->n;
    ie->n = d->n; ie->k = d->k;
}

}  // namespace
}  // namespace fth

using namespace fth;

extern "C" int fth_b200_abi_version(void) { return 5; }
extern "C" const char* fth_b200_last_variant(void) { return g_last_variant; }
extern "C" int64_t fth_b200_launch_count(void) { return g_launches; }
extern "C" void fth_b200_reset_launch_count(void) { g_launches = 0; }

extern "C" int fth_b200_fp8_linear_supported(const fth_b200_fp8_linear_desc* d) {
    const int rc = ValidateFp8(d);
    if (rc != FTH_B200_OK) return rc;
    LinearArgs args; Fp8Epilogue fe;
    BuildFp8(d, &args, &fe);
    const int v = PickVariant(d->variant, d->dtype, args, d->workspace, d->workspace_bytes);
    return v < 0 ? v : FTH_B200_OK;
}

extern "C" size_t fth_b200_fp8_linear_workspace_bytes(const fth_b200_fp8_linear_desc* d) {
    if (ValidateFp8(d) != FTH_B200_OK) return 0;
    LinearArgs args; Fp8Epilogue fe;
    BuildFp8(d, &args, &fe);
    return WorkspaceFor(d->variant, d->dtype, args);
}

extern "C" int fth_b200_fp8_linear(const fth_b200_fp8_linear_desc* d, fth_b200_stream_t stream) {
    ClearStaleError();
    const int rc = ValidateFp8(d);
    if (rc != FTH_B200_OK) return rc;
    LinearArgs args; Fp8Epilogue fe; Int8Epilogue ie = {};
    BuildFp8(d, &args, &fe);
    if (BuildPeers(d, &args.peers) != FTH_B200_OK || BuildSignal(d, &args.signal) != FTH_B200_OK) return FTH_B200_ERR_INVALID;
    return Run(PickVariant(d->variant, d->dtype, args, d->workspace, d->workspace_bytes), d->dtype, args, fe, ie,
               d->workspace, d->workspace_bytes, static_cast<cudaStream_t>(stream));
}

static int Fp8LinearArgmax(const fth_b200_fp8_linear_desc* d, int64_t* indices, int64_t none_value, fth_b200_stream_t stream_) {
    ClearStaleError();
    const int rc = ValidateFp8(d);
    if (rc != FTH_B200_OK) return rc;
    if (indices == nullptr || reinterpret_cast<uintptr_t>(indices) % 8 != 0) return FTH_B200_ERR_INVALID;
    auto stream = static_cast<cudaStream_t>(stream_);
    LinearArgs args; Fp8Epilogue fe; Int8Epilogue ie = {};
    BuildFp8(d, &args, &fe);
    if (BuildPeers(d, &args.peers) != FTH_B200_OK) return FTH_B200_ERR_INVALID;
    const int variant = PickVariant(d->variant, d->dtype, args, d->workspace, d->workspace_bytes);
    if (variant < 0) return variant;
    // only the decode-sized tensor-core kernels carry the fused selection (their epilogue sees every output once)
    if (variant != FTH_B200_VARIANT_TCGEN05 || !Tcgen05SelectsInEpilogue(d->dtype, args, fe, ie)) return FTH_B200_ERR_UNSUPPORTED;
    if (cudaMemsetAsync(indices, 0, static_cast<size_t>(d->m) * 8, stream) != cudaSuccess) return FTH_B200_ERR_CUDA;
    args.argmax_keys = reinterpret_cast<unsigned long long*>(indices);
    const int run = Run(variant, d->dtype, args, fe, ie, d->workspace, d->workspace_bytes, stream);
    if (run != FTH_B200_OK) return run;
    return LaunchArgmaxFinalize(args.argmax_keys, d->m, none_value, stream);
}

extern "C" int fth_b200_fp8_linear_argmax(const fth_b200_fp8_linear_desc* d, int64_t* indices, fth_b200_stream_t stream) {
    return Fp8LinearArgmax(d, indices, -1, stream);
}

extern "C" int fth_b200_fp8_lm_head_argmax(const fth_b200_fp8_linear_desc* d, int64_t* token, fth_b200_stream_t stream) {
    if (d == nullptr || d->m != 1 || !d->trans_b || d->bias_mode != FTH_B200_BIAS_NONE) return FTH_B200_ERR_INVALID;
    return Fp8LinearArgmax(d, token, 0, stream);
}

static int BuildFused(const fth_b200_fp8_linear_desc* d, const fth_b200_fp8_linear_fusion* f, LinearArgs* args, Fp8Epilogue* fe) {
    const int rc = ValidateFp8(d);
    if (rc != FTH_B200_OK) return rc;
    if (f == nullptr) return FTH_B200_ERR_INVALID;
    BuildFp8(d, args, fe);
    DecoderFusion& fu = args->fusion;
    fu.prologue = f->prologue;
    fu.norm_weight = f->norm_weight; fu.norm_weight_dtype = f->norm_weight_dtype;
    fu.norm_offset = f->norm_weight_offset; fu.norm_epsilon = f->norm_epsilon;
    fu.a2 = f->a2;
    fu.residual = f->residual;
    fu.w2 = f->w2; fu.out2 = f->out2; fu.n2 = f->n2; fu.ldo2 = f->ldo2 ? f->ldo2 : f->n2;
    fu.ab_scale2 = d->a_scale * f->w2_scale;
    fu.epilogue = f->epilogue;
    fu.out_codes = f->out_codes;
    fu.codes_scale = f->out_codes_scale;
    fu.codes_inv = 0.0f;  // set by the launcher
    fu.ldo_codes = f->ldo_codes ? f->ldo_codes : d->n;
    if (fu.out_codes != nullptr && !ValidScale(f->out_codes_scale)) return FTH_B200_ERR_INVALID;
    if (fu.prologue == 1 && (!std::isfinite(fu.norm_epsilon) || fu.norm_epsilon < 0.0f)) return FTH_B200_ERR_INVALID;
    if (fu.w2 != nullptr && !ValidScale(f->w2_scale)) return FTH_B200_ERR_INVALID;
    Int8Epilogue ie = {};
    return Tcgen05FusionStatus(d->dtype, *args, *fe, ie);
}

extern "C" int fth_b200_fp8_linear_fused_supported(const fth_b200_fp8_linear_desc* d, const fth_b200_fp8_linear_fusion* f) {
    LinearArgs args; Fp8Epilogue fe;
    return BuildFused(d, f, &args, &fe);
}

extern "C" int fth_b200_fp8_linear_fused(const fth_b200_fp8_linear_desc* d, const fth_b200_fp8_linear_fusion* f, fth_b200_stream_t stream) {
    ClearStaleError();
    LinearArgs args; Fp8Epilogue fe; Int8Epilogue ie = {};
    const int rc = BuildFused(d, f, &args, &fe);
    if (rc != FTH_B200_OK) return rc;
    return LaunchLinearTcgen05(d->dtype, args, fe, ie, nullptr, 0, static_cast<cudaStream_t>(stream));
}

extern "C" int fth_b200_int8_linear_supported(const fth_b200_int8_linear_desc* d) {
    const int rc = ValidateInt8(d);
    if (rc != FTH_B200_OK) return rc;
    LinearArgs args; Int8Epilogue ie;
    BuildInt8(d, &args, &ie);
    const int v = PickVariant(d->variant, FTH_B200_INT8, args, d->workspace, d->workspace_bytes);
    return v < 0 ? v : FTH_B200_OK;
}

extern "C" size_t fth_b200_int8_linear_workspace_bytes(const fth_b200_int8_linear_desc* d) {
    if (ValidateInt8(d) != FTH_B200_OK) return 0;
    LinearArgs args; Int8Epilogue ie;
    BuildInt8(d, &args, &ie);
    return WorkspaceFor(d->variant, FTH_B200_INT8, args);
}

extern "C" int fth_b200_int8_linear(const fth_b200_int8_linear_desc* d, fth_b200_stream_t stream) {
    ClearStaleError();
    const int rc = ValidateInt8(d);
    if (rc != FTH_B200_OK) return rc;
    LinearArgs args; Int8Epilogue ie; Fp8Epilogue fe = {};
    BuildInt8(d, &args, &ie);
    if (BuildPeers(d, &args.peers) != FTH_B200_OK || BuildSignal(d, &args.signal) != FTH_B200_OK) return FTH_B200_ERR_INVALID;
    return Run(PickVariant(d->variant, FTH_B200_INT8, args, d->workspace, d->workspace_bytes), FTH_B200_INT8, args,
               fe, ie, d->workspace, d->workspace_bytes, static_cast<cudaStream_t>(stream));
}
