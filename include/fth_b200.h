/*
 * fth_b200.h — C ABI of the B200 (sm_100a) quantized-linear backend for Feather.
 *
 * Every entry point takes plain pointers and sizes, launches hand-written CUDA kernels on the caller's
 * stream and returns an int status (0 = ok, negative = FTH_B200_ERR_*).  Unless a comment says otherwise
 * an entry point never allocates, never synchronises and never reads device memory back, so it is legal
 * inside CUDA-graph capture (the reference's CUDA INT8 kernels are not: src/kernel/cuda/int8.cu:287-367).
 * There is no CPU fallback anywhere below this header: a shape or contract the kernels do not implement
 * returns FTH_B200_ERR_UNSUPPORTED so that the caller (Feather's KernelBase::Supports(),
 * include/core/kernel.h:158) can answer StatusCode::kUnsupported and let the next CUDA candidate try.
 *
 * Each declaration names the reference interface it replaces (paths are relative to the Feather tree).
 */
#ifndef FTH_B200_H
#define FTH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque CUDA stream handle (cudaStream_t). */
typedef void* fth_b200_stream_t;

/* Element types; the values are feather::DataType's (include/util/types.h:32-47). */
enum {
    FTH_B200_INT8 = 1,
    FTH_B200_FP16 = 3,
    FTH_B200_FP32 = 4,
    FTH_B200_INT32 = 5,
    FTH_B200_BF16 = 11,
    FTH_B200_FP8E4M3 = 12,
    FTH_B200_FP8E5M2 = 13
};

/* Status codes. */
enum {
    FTH_B200_OK = 0,
    FTH_B200_ERR_INVALID = -1,     /* null pointer, bad size, non-finite scale: the reference kernels return -1 */
    FTH_B200_ERR_UNSUPPORTED = -2, /* valid request this backend declines (→ StatusCode::kUnsupported) */
    FTH_B200_ERR_CUDA = -3,        /* a CUDA runtime / driver call failed */
    FTH_B200_ERR_OVERFLOW = -4,    /* K·255·255 + max|bias| may leave int32 (int8_kernel_utils.h:99-114) */
    FTH_B200_ERR_TIMEOUT = -5,     /* a bounded device-side wait gave up (read from a status word) */
    FTH_B200_ERR_SCRATCH_LIMIT = -6 /* fth_b200_fp8_linear_noalloc: the shape needs more than the built-in scratch */
};

/* Operator flavour: decides how bias / alpha / beta enter (FC and MatMul: alpha = beta = 1). */
enum { FTH_B200_OP_FC = 0, FTH_B200_OP_MATMUL = 1, FTH_B200_OP_GEMM = 2 };

/* Bias layout, the encoding of src/kernel/cuda/linear_kernels.cuh:40-42. */
enum { FTH_B200_BIAS_NONE = 0, FTH_B200_BIAS_VECTOR = 1, FTH_B200_BIAS_MATRIX = 2 };

/* Kernel family selector for `variant` (0 lets the library split by shape). */
enum {
    FTH_B200_VARIANT_AUTO = 0,
    FTH_B200_VARIANT_SIMT = 1,   /* ragged-shape CUDA-core tile kernel (any M, K, N, any alignment) */
    FTH_B200_VARIANT_SKINNY = 2, /* weight-streaming GEMV / skinny GEMM with direct 16-byte loads, M <= 16 */
    FTH_B200_VARIANT_TCGEN05 = 3,/* tcgen05 MMA, TMEM accumulators, TMA-fed shared-memory tiles */
    FTH_B200_VARIANT_STREAM = 4  /* persistent GEMV, weights staged through a TMA shared-memory ring ([K,N] weights) */
};

int fth_b200_abi_version(void);
/* Name of the kernel family the last call on this host thread launched ("skinny", "tcgen05", "simt", …);
 * the counterpart of LastCudaFp8MatmulBackend() (src/kernel/cuda/runtime.h:141-143). */
const char* fth_b200_last_variant(void);
/* Reads and clears the per-device status word (synchronises the device): 0 when no bounded device-side wait
 * ever gave up, else (site << 16) | detail of the first that did. */
int fth_b200_device_status(void);
/* Kernels launched by this library on this host thread since the last reset. */
int64_t fth_b200_launch_count(void);
void fth_b200_reset_launch_count(void);

/* -------------------------------------------------------------------------------------------------
 * FP8 (E4M3 / E5M2) FC, MatMul, Gemm.
 * Replaces RunFp8Fc / RunFp8MatMul / RunFp8Gemm → LaunchFp8MatMulKernelCuda
 * (src/kernel/cuda/fc.cu:91-142, matmul.cu:230-272, gemm.cu:125-183, linear_kernels.cuh:815-837) and
 * follows the numerical contract of the Common kernels (src/kernel/common/fc.cc:48-76, gemm.cc:62-99):
 *
 *   acc = Σ_k decode(a[m,k]) · decode(w[k,n])              FP32 accumulation
 *   y   = alpha · acc · a_scale · w_scale(n) + beta · decode(bias) · bias_scale
 *   out = encode_saturating_rne(y / out_scale)             (include/util/fp8.h:81-172)
 *
 * a [M,K] row-major; w [K,N] row-major, or [N,K] when trans_b; out [M,N] with row stride ldo elements.
 * a_dtype may be BF16 or FP32 instead of `dtype`: the activation is then first quantised exactly as the
 * reference's Cast node would (encode(x / a_scale), src/kernel/common/cast.cc:103-110).  out_dtype may be
 * BF16 or FP32: the FP8 result is then decoded again (decode(out)·out_scale) as the Cast node after the
 * MatMul would; both rounding points are kept, so the fused call equals Cast → MatMul → Cast.
 * w_channel_scales (device, N floats) is an extension the reference cannot express (its FP8 tensors are
 * per-tensor only, src/kernel/fp8_host.h:150-157); when non-null it replaces w_scale.
 * ------------------------------------------------------------------------------------------------- */
typedef struct {
    int32_t dtype;     /* FTH_B200_FP8E4M3 or FTH_B200_FP8E5M2: weight, bias and FP8 output format */
    int32_t op;        /* FTH_B200_OP_* */
    int64_t m, k, n;
    int32_t trans_b;   /* 0: w is [K,N]; 1: w is [N,K] (GemmParam::trans_b) */
    int32_t a_dtype;   /* 0 or dtype: FP8 activations; FTH_B200_BF16 / FTH_B200_FP32: fused Cast prologue */
    int32_t out_dtype; /* 0 or dtype: FP8 output; FTH_B200_BF16 / FTH_B200_FP32: fused Cast epilogue */
    int32_t bias_mode; /* FTH_B200_BIAS_*; bias is FP8 of `dtype` */
    const void* a;
    const void* w;
    const void* bias;
    void* out;
    int64_t ldo;       /* output row stride in elements; 0 means n */
    float a_scale, w_scale, bias_scale, out_scale;
    const float* w_channel_scales;
    float alpha, beta;
    /* Device scratch (256-byte aligned) of the kernel family `variant` selects: split-K partial sums and, for a fused
     * Cast / QuantizeLinear that runs as a separate pass, the 8-bit activations.  fth_b200_fp8_linear_workspace_bytes
     * says how much that family needs for this descriptor — 0 for shapes the single-launch cluster kernel and the dense
     * kernel take.  The figure is an upper bound over the entry points that take the descriptor: a decode-sized call with
     * a wide weight adds its K chunks in tensor memory and leaves the scratch untouched, the lm-head call with the same
     * descriptor still uses it.  It must be zero-filled once after allocation (VARIANT_STREAM keeps arrival counters in it and leaves
     * them zero again).  Calls that share a workspace must not overlap on the GPU.  May be null: the library then picks
     * kernels that need no scratch. */
    void* workspace;
    size_t workspace_bytes;
    int32_t variant;      /* FTH_B200_VARIANT_* */
    /* 1: nothing queued earlier on the stream writes `w` (an initializer, as FC / MatMul weights are in a compiled
     * plan), so the kernel may fetch weights while the previous kernel is still finishing.  0: no assumption. */
    int32_t weights_static;
    /* Column-sharded projections on several GPUs of one box: `gather_peers` other ranks hold a buffer shaped like this
     * rank's output buffer; gather_out[r] is the peer-mapped address in rank r's buffer that corresponds to `out`.
     * Every output element is stored there as well (by the tensor-core kernels' own epilogue when no bias, alpha or
     * beta is involved; by a block copy behind the kernel otherwise).  Follow the call with fth_b200_gather_sync.  No counterpart in the reference
     * (one CudaExecutionContext = one device, src/kernel/cuda/runtime.cu:318-321). */
    int32_t gather_peers;   /* 0 .. 7 */
    void* gather_out[7];
    /* Gather signalling folded into the kernel (gather_world >= 2; 0: off, end the step with fth_b200_gather_sync
     * instead).  gather_flags[r] is rank r's flag array as in fth_b200_gather_sync (peer-mapped; [gather_rank] is this
     * rank's own; room for gather_world + 2 words each, zero-filled at creation).  The kernel takes the step number s
     * from the counter in its own array, holds its first store into the peers' buffers until every rank has signalled
     * step s - 1 (so nobody is still reading the buffer pair being overwritten; bounded wait, reported through
     * fth_b200_device_status), and when its last thread block has stored its outputs it publishes s in every rank's
     * array.  A consumer of the gathered buffer waits for the other ranks' data with fth_b200_gather_wait; the next
     * step's kernel does so by itself.  Kernel families without this path get the same steps as small kernels around
     * them.  All ranks must use one protocol (this one or fth_b200_gather_sync) for the life of a flag array. */
    int32_t gather_world;
    int32_t gather_rank;
    void* gather_flags[8];
    /* Optional, with gather_peers > 0: the address that corresponds to `out` in an NVLink multicast mapping (NVLS) that
     * covers the output buffers of ALL ranks, this rank's included — one store there is delivered to every GPU by the
     * switch, so a rank's output crosses its links once instead of gather_peers times.  Used by the dense (M > 128)
     * kernel for one-byte outputs when n is a multiple of 16; every other kernel keeps storing to gather_out[], which
     * must still be filled in.  Null: not available.  (The mapping itself is the host's business: cuMulticastCreate /
     * cuMulticastBindMem, or torch.distributed._symmetric_memory as infer_b200/sharded.py does.) */
    void* gather_multicast_out;
} fth_b200_fp8_linear_desc;

int fth_b200_fp8_linear(const fth_b200_fp8_linear_desc* desc, fth_b200_stream_t stream);
/* The same linear plus greedy selection over each output row, fused into the epilogue: indices[row] receives the column
 * of the largest decoded output value (NaN codes skipped, ties to the lowest column, -1 when a row has no candidate) —
 * what an ArgMax node behind the MatMul would return, with the rule of the reference's fused BF16 lm-head kernel
 * (src/kernel/cuda/qwen_gemm_argmax.cu:55-64), which has no FP8 counterpart.  The output is written as usual.  Decode-sized
 * shapes on the tensor-core kernels only (FTH_B200_ERR_UNSUPPORTED otherwise; run the linear and an ArgMax node then). */
int fth_b200_fp8_linear_argmax(const fth_b200_fp8_linear_desc* desc, int64_t* indices, fth_b200_stream_t stream);
/* The fused lm-head node: a [1,K] times the [N,K] vocabulary weight (trans_b = 1, Gemm), greedy selection, one int64
 * token.  Replaces QwenGemmArgmaxKernel (param src/operator/params.h:152-168), whose FP8 form exists in the reference
 * for x86 only (src/kernel/x86/linear_fp8.cc:733-1004: the accumulator is quantised to an FP8 code with
 * desc->out_scale = QwenGemmArgmaxParam::output_scale, the decoded code times that scale is rounded to BF16, NaN is
 * skipped, the first index wins among equal values, and token 0 is returned when there is no candidate); its CUDA
 * candidates are BF16 only (src/kernel/cuda/qwen_gemm_argmax.cu:85-172).  Distinct FP8 codes stay distinct and ordered
 * after the BF16 rounding, so selecting on the decoded code is the same rule.  desc->out still receives the [1,N] codes. */
int fth_b200_fp8_lm_head_argmax(const fth_b200_fp8_linear_desc* desc, int64_t* token, fth_b200_stream_t stream);
/* Capability check only (what Supports() calls): 0 if fth_b200_fp8_linear would run this descriptor. */
int fth_b200_fp8_linear_supported(const fth_b200_fp8_linear_desc* desc);
size_t fth_b200_fp8_linear_workspace_bytes(const fth_b200_fp8_linear_desc* desc);

/* -------------------------------------------------------------------------------------------------
 * A decode-sized FP8 projection with the decoder-block operators around it in the same launch.  The descriptor is the
 * projection itself as the Qwen exporter wraps it — Cast(BF16 -> FP8) -> MatMul -> Cast(FP8 -> BF16), i.e. a_dtype =
 * out_dtype = FTH_B200_BF16 — and `fusion` names what else the plan holds around it:
 *   prologue  FTH_B200_FUSE_RMS_NORM: the activation is first normalised as the QwenRmsNorm node in front would
 *             (src/kernel/common/qwen_rms_norm.cc:71-95, BF16 output); FTH_B200_FUSE_SILU_MUL: the activation is
 *             Mul(SiLU(a), a2) of two BF16 tensors (the SiLU and Mul nodes between gate / up and the down projection).
 *   residual  BF16, laid out like `out`: out = Add(residual, out) (the residual connection behind o / down).
 *   w2        a second weight of the same format and layout on the same activation (gate and up): [K,n2] / [n2,K],
 *             n2 = desc->n, with scale w2_scale, output out2 [M,n2] (row stride ldo2, 0 = n2).
 *   epilogue  FTH_B200_FUSE_OUT_SILU_MUL (needs w2, no residual): desc->out receives Mul(SiLU(first product), second
 *             product), the activation of the down projection; out2 is not written and may be null.
 *   out_codes (with out_codes_scale, row stride ldo_codes, 0 = n): every output is also stored as the FP8 code the Cast
 *             node in front of the NEXT projection would make of it (format = desc->dtype) — that projection then takes
 *             the codes as its activation (a_dtype = 0) and runs no Cast of its own.  Not with a second weight unless the
 *             SiLU * Mul epilogue joins the two products.
 * desc->a_dtype may be 0 here (activations that are such codes already) when no prologue is asked for.
 * A norm weight is read ahead of the work queued in front of the call when desc->weights_static says the same of the
 * projection weights: it is a constant of the model like them.
 * Every rounding point of the unfused nodes is kept (BF16 after the norm / SiLU / Mul, FP8 after the Cast, FP8 after
 * the product, BF16 after the second Cast and after the Add), and the squares of a row are summed in the order
 * fth_b200_qwen_rms_norm uses, so the call returns the bytes of the separate calls.  Shapes of the single-launch
 * kernel only (M <= 32, K <= 4096 with a norm); FTH_B200_ERR_UNSUPPORTED otherwise: run the nodes one by one then.
 * No counterpart in the reference, which runs each node as its own kernel (src/kernel/cuda/{qwen_rms_norm,silu,mul,add}.cu).
 * ------------------------------------------------------------------------------------------------- */
enum { FTH_B200_FUSE_NONE = 0, FTH_B200_FUSE_RMS_NORM = 1, FTH_B200_FUSE_SILU_MUL = 2 };
enum { FTH_B200_FUSE_OUT_NONE = 0, FTH_B200_FUSE_OUT_SILU_MUL = 1 };
typedef struct {
    int32_t prologue;            /* FTH_B200_FUSE_* */
    int32_t norm_weight_dtype;   /* FTH_B200_BF16 or FTH_B200_FP32 */
    const void* norm_weight;     /* [K] */
    float norm_weight_offset;    /* QwenRmsNormParam::weight_offset */
    float norm_epsilon;
    const void* a2;              /* prologue SILU_MUL: BF16 [M,K] */
    const void* residual;        /* BF16 or null */
    const void* w2;              /* or null */
    float w2_scale;
    void* out2;
    int64_t n2;
    int64_t ldo2;
    int32_t epilogue;            /* FTH_B200_FUSE_OUT_* */
    float out_codes_scale;
    void* out_codes;             /* or null */
    int64_t ldo_codes;
} fth_b200_fp8_linear_fusion;
int fth_b200_fp8_linear_fused(const fth_b200_fp8_linear_desc* desc, const fth_b200_fp8_linear_fusion* fusion, fth_b200_stream_t stream);
int fth_b200_fp8_linear_fused_supported(const fth_b200_fp8_linear_desc* desc, const fth_b200_fp8_linear_fusion* fusion);

/* FP8 linear for callers that cannot hand over a scratch buffer because they may not allocate one: a Feather
 * node built with a workspace limit of zero, or a session whose device memory was fixed when its plan was
 * compiled.  No counterpart in the reference.  Same contract and results as fth_b200_fp8_linear on the
 * tensor-core kernel family (desc->variant, workspace and workspace_bytes are ignored), but the split-K
 * partial sums go to an array built into the library image — fth_b200_noalloc_scratch_bytes() = 4 MiB of device
 * global memory that every GPU which loads the library holds until the process exits.  The call allocates
 * nothing and frees nothing.
 *   - A shape whose partial sums do not fit (fth_b200_fp8_linear_workspace_bytes > 4 MiB; for K >= 1024, M = 1 fits up to
 *     N = 131072 and M = 16 up to N = 8192) returns FTH_B200_ERR_SCRATCH_LIMIT; shapes the tensor-core
 *     family declines return FTH_B200_ERR_UNSUPPORTED.
 *   - The first call on each device looks the array's device address up (cudaGetSymbolAddress) with that device
 *     current; make that first call before starting any stream capture.
 *   - All calls on a device share the one array.  Nothing in it has to start at zero and a call reads only
 *     what it wrote itself, but two calls that overlap on the GPU (different streams, no ordering) race. */
int fth_b200_fp8_linear_noalloc(const fth_b200_fp8_linear_desc* desc, fth_b200_stream_t stream);
size_t fth_b200_noalloc_scratch_bytes(void);

/* -------------------------------------------------------------------------------------------------
 * INT8 FC, MatMul, Gemm (bit-exact with the Common kernels).
 * Replaces RunCudaInt8Linear / RunCudaInt8MatMul → Int8LinearKernel / Int8MatMulKernel
 * (src/kernel/cuda/int8.cu:112-208, 313-368); contract of src/kernel/common/fc.cc:105-159,
 * gemm.cc:136-198, matmul.cc:156-261 and int8_kernel_utils.h:159-179:
 *
 *   acc  = Σ_k (a - a_zp)(w - w_zp[n])                      int32 (the host rejects shapes that could overflow)
 *   FC / MatMul: real = double(acc + bias) · (double(a_scale) · w_scale[n])
 *   Gemm:        real = (double(alpha)·acc + double(beta)·bias) · (double(a_scale) · w_scale[n])
 *   out  = clamp(round_half_away(real / double(out_scale) + out_zp), -128, 127)
 *
 * w_scales / w_zps are DEVICE arrays with w_params entries: 1 (per tensor) or n (per output channel);
 * w_zps may be null (all zero).  bias is int32 [N] or [M,N].
 * a_dtype FP32 fuses QuantizeLinear (quantization.h:94-99) in front, out_dtype FP32 fuses
 * DequantizeLinear ((q - out_zp)·out_scale) behind; both keep the int8 rounding point.
 * ------------------------------------------------------------------------------------------------- */
typedef struct {
    int32_t op;
    int64_t m, k, n;
    int32_t trans_b;
    int32_t a_dtype;   /* 0 / FTH_B200_INT8, or FTH_B200_FP32 (fused QuantizeLinear) */
    int32_t out_dtype; /* 0 / FTH_B200_INT8, or FTH_B200_FP32 (fused DequantizeLinear) */
    int32_t bias_mode;
    const void* a;
    const int8_t* w;
    const int32_t* bias;
    void* out;
    int64_t ldo;
    float a_scale;
    int32_t a_zp;
    const float* w_scales;
    const int32_t* w_zps;
    int64_t w_params;
    int32_t w_zp_max_abs; /* host-known bound on |w_zp| (0 when symmetric); used by the overflow pre-check */
    float out_scale;
    int32_t out_zp;
    float alpha, beta;
    int64_t bias_max_abs; /* host-known bound on |bias| for the overflow pre-check */
    void* workspace;      /* as in fth_b200_fp8_linear_desc */
    size_t workspace_bytes;
    int32_t variant;
    int32_t weights_static; /* as in fth_b200_fp8_linear_desc */
    int32_t gather_peers;   /* as in fth_b200_fp8_linear_desc */
    void* gather_out[7];
    int32_t gather_world;   /* as in fth_b200_fp8_linear_desc */
    int32_t gather_rank;
    void* gather_flags[8];
    void* gather_multicast_out;   /* as in fth_b200_fp8_linear_desc */
} fth_b200_int8_linear_desc;

int fth_b200_int8_linear(const fth_b200_int8_linear_desc* desc, fth_b200_stream_t stream);
int fth_b200_int8_linear_supported(const fth_b200_int8_linear_desc* desc);
size_t fth_b200_int8_linear_workspace_bytes(const fth_b200_int8_linear_desc* desc);

/* -------------------------------------------------------------------------------------------------
 * INT8 Conv2D, NCHW activations, OIHW weights, int32 bias, optional fused INT8 ReLU table.
 * Replaces RunCudaInt8Conv2D → Int8Conv2DKernel (src/kernel/cuda/int8.cu:217-285, 370-506); contract of
 * src/kernel/common/conv2d.cc:481-581 (padded taps contribute nothing).  When relu_lut is non-null the
 * 256-entry table of the INT8 ReLU node (src/kernel/common/int8_standard.cc:114-128) is applied to the
 * requantised int8 value, i.e. Conv2D → ReLU in one launch with both rounding points kept.
 * `workspace` (device, fth_b200_int8_conv2d_workspace_bytes) is used by the implicit-GEMM path for the
 * channels-last copy of the input and the repacked weights; it may be null for VARIANT_SIMT.
 * ------------------------------------------------------------------------------------------------- */
typedef struct {
    int64_t batch, ic, ih, iw, oc, kh, kw;
    int32_t stride_h, stride_w, pad_h, pad_w, dilation_h, dilation_w, group;
    const int8_t* x;
    const int8_t* w;
    const int32_t* bias; /* [OC] or null */
    int8_t* out;
    float x_scale;
    int32_t x_zp;
    const float* w_scales; /* device, w_params entries (1 or OC) */
    const int32_t* w_zps;  /* device or null */
    int64_t w_params;
    int32_t w_zp_max_abs;
    float out_scale;
    int32_t out_zp;
    const int8_t* relu_lut; /* device, 256 entries indexed by q + 128, or null */
    int64_t bias_max_abs;
    void* workspace;
    size_t workspace_bytes;
    int32_t weights_packed; /* 1: workspace already holds the packed weights of a previous call (same w) */
    int32_t variant;
    /* Optional: the weight in the implicit-GEMM layout, made once per weight by fth_b200_int8_conv2d_pack_weights
     * (device memory the caller owns and may share between sessions and plans that use the same weight — the
     * counterpart of the reference's per-weight cache of packed x86 layouts, src/kernel/x86/prepared_weight_cache.h).
     * When non-null the call never repacks, `weights_packed` is ignored and `workspace` only holds the channels-last
     * copy of the input. */
    const int8_t* packed_w;
} fth_b200_int8_conv2d_desc;

int fth_b200_int8_conv2d(const fth_b200_int8_conv2d_desc* desc, fth_b200_stream_t stream);
int fth_b200_int8_conv2d_supported(const fth_b200_int8_conv2d_desc* desc);
size_t fth_b200_int8_conv2d_workspace_bytes(const fth_b200_int8_conv2d_desc* desc);
/* Size of, and the pass that fills, the packed copy of desc->w for desc->packed_w ([OC][KH][KW][IC], 256-byte aligned
 * destination).  0 / FTH_B200_ERR_UNSUPPORTED when the implicit-GEMM kernel does not take the geometry (nothing to pack). */
size_t fth_b200_int8_conv2d_packed_weight_bytes(const fth_b200_int8_conv2d_desc* desc);
int fth_b200_int8_conv2d_pack_weights(const fth_b200_int8_conv2d_desc* desc, void* packed, fth_b200_stream_t stream);

/* Builds the 256-entry INT8 ReLU table on the host (src/kernel/common/int8_standard.cc:114-128). */
int fth_b200_int8_relu_table(float in_scale, int32_t in_zp, float out_scale, int32_t out_zp, int8_t* lut256);
/* Standalone INT8 ReLU node through a device table (RunUnaryInt8Lookup, int8_standard.cc:148-176). */
int fth_b200_int8_lookup(const int8_t* x, int8_t* out, int64_t count, const int8_t* device_lut256,
                         fth_b200_stream_t stream);

/* -------------------------------------------------------------------------------------------------
 * QuantizeLinear / DequantizeLinear.  The reference has COMMON kernels only
 * (src/kernel/common/quantize_linear.cc:24-42, dequantize_linear.cc:25-36), so a CUDA plan with
 * KernelFallbackPolicy::kRequireRequested cannot be built without these.  Contract:
 * src/kernel/common/quantize_linear_utils.h:236-341.  x is [rows, channels]; scales / zps are DEVICE
 * arrays with `params` entries: 1 (per tensor) or `channels` (per channel on the last axis).
 * ------------------------------------------------------------------------------------------------- */
int fth_b200_quantize_linear(int32_t x_dtype, const void* x, const float* scales, const int32_t* zps,
                             int64_t params, int8_t* out, int64_t rows, int64_t channels,
                             fth_b200_stream_t stream);
int fth_b200_dequantize_linear(const int8_t* x, const float* scales, const int32_t* zps, int64_t params, void* out,
                               int32_t to_dtype, int64_t rows, int64_t channels, fth_b200_stream_t stream);
/* The same two nodes with the channel axis anywhere: x is [outer, channels, inner] (QuantizeLinearParam::axis names the
 * middle extent; inner = 1 is the last-axis form above). */
int fth_b200_quantize_linear_axis(int32_t x_dtype, const void* x, const float* scales, const int32_t* zps,
                                  int64_t params, int8_t* out, int64_t outer, int64_t channels, int64_t inner,
                                  fth_b200_stream_t stream);
int fth_b200_dequantize_linear_axis(const int8_t* x, const float* scales, const int32_t* zps, int64_t params, void* out,
                                    int32_t to_dtype, int64_t outer, int64_t channels, int64_t inner,
                                    fth_b200_stream_t stream);

/* Cast among FP32 / FP16 / BF16 / FP8 with per-tensor FP8 scales.
 * Replaces CastFloatingKernelCuda (src/kernel/cuda/cast.cu:54-93); contract src/kernel/common/cast.cc:62-126. */
int fth_b200_cast(int32_t in_dtype, const void* x, float in_scale, int32_t out_dtype, void* out, float out_scale,
                  int64_t count, fth_b200_stream_t stream);

/* -------------------------------------------------------------------------------------------------
 * The operators between the quantized projections of a decoder block, for plans that keep the whole block on
 * the stream: QwenRmsNorm, Add, Mul, SiLU.  All are launched as programmatic dependents of the kernel in front.
 *
 * QwenRmsNorm replaces QwenRmsNormKernelCuda (src/kernel/cuda/qwen_rms_norm.cu:78-104); contract of the Common
 * kernel (src/kernel/common/qwen_rms_norm.cc:71-95): FP32 math,
 *   out[r,c] = x[r,c] * (1 / sqrt(sum_c x[r,c]^2 / hidden + epsilon)) * (weight[c] + weight_offset),
 * x / weight / out each FP32 or BF16.  The sum of squares is reduced in parallel, so an output may differ from the
 * Common kernel's (which adds the squares one after another) by one BF16 code, or by a few parts in 10^6 for FP32
 * output (its x86 and CUDA kernels reduce in other orders as well and sit as far from it).
 * Add / Mul replace the BF16 / FP16 / FP32 kernels of src/kernel/cuda/add.cu and mul.cu (contract
 * src/kernel/common/add.cc:80-109): out[i] = lhs[i] op rhs[i % rhs_count], one rounding; rhs_count = 0 means
 * same shape, else it is the length of the rhs row broadcast over lhs (count % rhs_count == 0).  Bit-exact.
 * SiLU replaces SiluDirectKernelCuda (src/kernel/cuda/silu.cu:39-47); contract src/kernel/common/silu.cc:38-55:
 * x / (1 + exp(-x)) in FP32.  fth_b200_silu_mul is the SiLU node followed by the Mul node in one launch
 * (out = round(silu(gate)) * up, both rounding points kept).
 * ------------------------------------------------------------------------------------------------- */
enum { FTH_B200_BINARY_ADD = 0, FTH_B200_BINARY_MUL = 1 };
int fth_b200_qwen_rms_norm(int32_t x_dtype, const void* x, int32_t weight_dtype, const void* weight, float weight_offset,
                           float epsilon, int32_t out_dtype, void* out, int64_t rows, int64_t hidden,
                           fth_b200_stream_t stream);
int fth_b200_binary(int32_t op, int32_t dtype, const void* lhs, const void* rhs, void* out, int64_t count,
                    int64_t rhs_count, fth_b200_stream_t stream);
int fth_b200_silu(int32_t dtype, const void* x, void* out, int64_t count, fth_b200_stream_t stream);
int fth_b200_silu_mul(int32_t dtype, const void* gate, const void* up, void* out, int64_t count,
                      fth_b200_stream_t stream);

/* -------------------------------------------------------------------------------------------------
 * Host-buffer plans: the shape of KernelBase::Prepare() / compute() (include/core/kernel.h:162-163) for a
 * linear node whose weight is immutable.  create() uploads weight, scales and bias once (it allocates and
 * synchronises — never call it during capture); run() copies the activation from host memory, launches,
 * and copies the result back, all on `stream`, then waits for the stream.  A decode-sized linear plan (M <= 32) whose
 * two host buffers are page-locked needs no copy-engine transfer: a small kernel reads the activation from the host
 * buffer and the linear kernel stores its output there as well; after the plan's first run() the two launches are
 * recorded for the pair of host buffers in use and replayed with one graph launch (another pair of buffers records again).  A plan is
 * used by one thread at a time, and `stream` must not be capturing.
 * ------------------------------------------------------------------------------------------------- */
typedef struct fth_b200_plan fth_b200_plan;

/* Pointers in `host_desc` are HOST pointers (a and out may be null here; they are given to run()). */
int fth_b200_plan_create_fp8_linear(const fth_b200_fp8_linear_desc* host_desc, fth_b200_plan** plan);
int fth_b200_plan_create_int8_linear(const fth_b200_int8_linear_desc* host_desc, fth_b200_plan** plan);
int fth_b200_plan_create_int8_conv2d(const fth_b200_int8_conv2d_desc* host_desc, fth_b200_plan** plan);
int fth_b200_plan_run(fth_b200_plan* plan, const void* host_in, void* host_out, fth_b200_stream_t stream);
/* Device-resident variant of run(): no copies, no wait. */
int fth_b200_plan_launch(fth_b200_plan* plan, const void* device_in, void* device_out, fth_b200_stream_t stream);
/* A few KB between a page-locked host buffer and device memory (either direction, or device to device), copied by the SMs
 * on `stream`: for the activation row and the result row of a decode step this is quicker than a copy-engine transfer
 * (4.5 / 6.6 us each in a 74 us step).  FTH_B200_ERR_UNSUPPORTED when a pointer is pageable host memory: use
 * cudaMemcpyAsync then.  No counterpart in the reference. */
int fth_b200_small_copy(void* dst, const void* src, int64_t bytes, fth_b200_stream_t stream);
int64_t fth_b200_plan_input_bytes(const fth_b200_plan* plan);
int64_t fth_b200_plan_output_bytes(const fth_b200_plan* plan);
void fth_b200_plan_destroy(fth_b200_plan* plan);

/* ---- multi-GPU gather without a collective library (no counterpart in the reference) -------------------------
 * fth_b200_peer_buffer_create allocates zeroed device memory and returns a 64-byte handle another process of the same
 * box turns into a peer-mapped pointer with fth_b200_peer_buffer_open (CUDA IPC).  fth_b200_gather_sync ends a
 * gather step: on `stream`, after this rank's earlier work, it writes `epoch` into slot [rank] of every rank's flag
 * array (rank_flags[r]: uint32[world], peer-mapped; rank_flags[rank] is this rank's own) and waits, for at most one
 * second, until every slot of its own array has reached `epoch`; a time-out is reported through
 * fth_b200_device_status.  Epochs grow by one per step; flags are never reset.  epoch = 0 takes the step number from a
 * counter on the device (slot [world] of this rank's own array, incremented by the call), so that a captured CUDA graph
 * can be replayed; all ranks must then use epoch = 0 for every step.  Each array has room for world + 2 words.
 * fth_b200_gather_wait only waits (bounded, same reporting) until every rank has signalled the step this rank signalled
 * last — the consumer side of the signalling that the linear kernels do themselves (gather_world in their descriptors).
 * A wait that runs out does NOT fail the stream: the kernel records the site and the missing rank in the status word and
 * returns, and what follows on the stream reads a buffer some ranks have not written.  A caller must therefore read
 * fth_b200_device_status() — at the latest where it hands a result that depends on a gathered buffer to its own caller —
 * and treat a non-zero word as a failed step. */
#define FTH_B200_PEER_HANDLE_BYTES 64
int fth_b200_peer_buffer_create(size_t bytes, void** ptr, unsigned char* handle);
int fth_b200_peer_buffer_open(const unsigned char* handle, void** ptr);
int fth_b200_peer_buffer_close(void* ptr);
int fth_b200_peer_buffer_destroy(void* ptr);
int fth_b200_gather_sync(void* const* rank_flags, int32_t world, int32_t rank, uint32_t epoch, fth_b200_stream_t stream);
int fth_b200_gather_wait(void* const* rank_flags, int32_t world, int32_t rank, fth_b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FTH_B200_H */
