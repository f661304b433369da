// Internal launcher interface shared by the linear kernel families and the C ABI dispatch.
#pragma once

#include "common.cuh"

namespace fth {

// Other GPUs' copies of the output buffer (column-sharded projections): every byte a kernel stores at address X of
// the local output is also stored at X + delta[r].  The buffers are peer-mapped device memory of the same shape.
constexpr int kMaxPeers = 7;
struct PeerOut {
    int count;
    int64_t delta[kMaxPeers];
    int64_t multicast_delta;  // X + multicast_delta is X in a multicast mapping of all ranks' buffers; 0: none
};

// Step signalling of a gather, folded into the kernels: flags[r] is rank r's flag array (uint32; slot [q] = last step rank
// q has published there), this rank's own array also holds the step counter (slot [world]) and the arrival counter of the
// running launch (slot [world + 1]).
struct GatherSignal {
    uint32_t* flags[kMaxPeers + 1];
    int world;  // 0: off
    int rank;
};

// Decoder-block operators fused around an FP8 projection with BF16 activations and BF16 outputs (single-launch cluster
// kernel only): what runs in front of the Cast that quantises the activation, what runs behind the Cast that widens
// the product, and a second weight that shares the activation.
struct DecoderFusion {
    int prologue;             // 0: none; 1: QwenRmsNorm(a) ; 2: Mul(SiLU(a), a2)
    const void* norm_weight;  // prologue 1: [K] weight (BF16 or FP32), offset and epsilon of the node
    int norm_weight_dtype;
    float norm_offset, norm_epsilon;
    const void* a2;           // prologue 2: the second BF16 input [M,K]
    const void* residual;     // epilogue: out = Add(residual, out); BF16, laid out like out; null: none
    const void* w2;           // second weight [K,n2] / [n2,K] on the same activation (n2 == n); null: none
    float ab_scale2;          // a_scale * scale of w2
    void* out2;               // its BF16 output [M,n2], row stride ldo2
    int64_t n2, ldo2;
    int epilogue;             // with w2: 1 = out receives Mul(SiLU(first product), second product); out2 is not written
    void* out_codes;          // also store Cast(out -> FP8 of the projection's format, codes_scale) [M, N], row stride ldo_codes; null: none
    float codes_scale, codes_inv;  // (codes_inv: the exact reciprocal of a power-of-two scale, else 0)
    int64_t ldo_codes;
    bool active() const { return prologue != 0 || residual != nullptr || w2 != nullptr || out_codes != nullptr; }
};

// Operand description common to FP8 and INT8 linear kernels.
struct LinearArgs {
    const void* a;   // [M,K] activations (FP8 / INT8, or BF16 / FP32 when a Cast / QuantizeLinear is fused)
    const void* w;   // [K,N] or [N,K] weights, one byte per element
    int64_t m, k, n;
    int trans_b;
    int a_dtype;     // 0 = same as the weight dtype
    float a_scale;   // used only by the fused-cast activation load
    int zero_points; // INT8: activation or weight zero point is non-zero
    int w_static;    // no earlier work in the stream writes the weights: they may be read before it has finished
    PeerOut peers;   // replicas of the output on other GPUs (count 0: none)
    unsigned long long* argmax_keys;  // [m] running (value, index) maxima of each output row, or null
    GatherSignal signal;              // world 0: none
    DecoderFusion fusion;             // inactive unless set by fth_b200_fp8_linear_fused
};

int LaunchLinearSimt(int dtype, const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie,
                     cudaStream_t stream);

// Weight-streaming GEMV / skinny GEMM for M <= kSkinnyMaxM.
constexpr int kSkinnyMaxM = 16;
bool SkinnySupported(int dtype, const LinearArgs& args);
int LaunchLinearSkinny(int dtype, const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie,
                       cudaStream_t stream);

// Persistent TMA-ring GEMV for [K,N] weights.
bool StreamSupported(int dtype, const LinearArgs& args);
size_t StreamCounterBytes(const LinearArgs& args);
size_t StreamScratchBytes(int dtype, const LinearArgs& args);
int LaunchLinearStream(int dtype, const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie, void* scratch,
                       size_t scratch_bytes, cudaStream_t stream);

// QuantizeLinear with scalar parameters (elementwise.cu), used as the fused prologue of the tensor-core linear.
int LaunchQuantizePerTensor(int x_dtype, const void* x, float scale, int32_t zp, int8_t* out, int64_t count, cudaStream_t stream);

// tcgen05 / TMEM / TMA dense GEMM.
bool Tcgen05Supported(int dtype, const LinearArgs& args);
size_t Tcgen05ScratchBytes(int dtype, const LinearArgs& args);
int LaunchLinearTcgen05(int dtype, const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie, void* scratch,
                        size_t scratch_bytes, cudaStream_t stream);
// True when that launch writes the peer replicas from its own epilogue (otherwise the caller copies the block over).
bool Tcgen05StoresToPeers(int dtype, const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie);
// True when that launch can also run the fused greedy selection (the decode-sized kernels, direct epilogue).
bool Tcgen05SelectsInEpilogue(int dtype, const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie);

// Turns the packed (value, index) keys a fused argmax left in `keys` into int64 indices in place; a row without a
// candidate receives `none_value`.
int LaunchArgmaxFinalize(unsigned long long* keys, int64_t m, int64_t none_value, cudaStream_t stream);

// FTH_B200_OK when the tensor-core family runs args.fusion (decoder-block operators fused around the projection).
int Tcgen05FusionStatus(int dtype, const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie);
// True when that launch also does the gather's step signalling itself (args.signal).
bool Tcgen05SignalsInKernel(int dtype, const LinearArgs& args, const Fp8Epilogue& fe, const Int8Epilogue& ie);
// The two halves of a gather step as kernels of their own, for kernel families that do not fold them in: wait until every
// rank has published the previous step / count this step and publish it everywhere.
int LaunchGatherWaitPrevious(const GatherSignal& signal, cudaStream_t stream);
int LaunchGatherPublish(const GatherSignal& signal, cudaStream_t stream);

// Copies the [m, n] output block (elements of `elem_bytes`, row stride ldo elements) to every peer replica.
int LaunchPeerCopy(const void* out, int64_t m, int64_t n, int64_t ldo, int elem_bytes, const PeerOut& peers, cudaStream_t stream);

}  // namespace fth
