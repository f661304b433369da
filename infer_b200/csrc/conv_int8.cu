// INT8 Conv2D (NCHW activations, OIHW weights): C ABI entry, validation, and the general direct kernel.
// The implicit-GEMM tensor-core kernel for the common case lives in conv_int8_tcgen05.cu.
#include <cmath>

#include "common.cuh"
#include "conv_internal.h"

namespace fth {
namespace {

constexpr int kThreads = 256;
constexpr int kOcPerThread = 4;

// General direct convolution: any stride, padding, dilation, groups and zero points.  One thread owns
// one output pixel and kOcPerThread consecutive output channels of one group, so every input byte it
// loads is used kOcPerThread times; adjacent threads own adjacent pixels (coalesced along W).
__global__ void __launch_bounds__(kThreads) ConvDirectKernel(ConvArgs c) {
    const int64_t ocg = c.oc / c.group, icg = c.ic / c.group;
    const int64_t oc_blocks = (ocg + kOcPerThread - 1) / kOcPerThread;
    const int64_t pixels = c.oh * c.ow;
    const int64_t total = c.batch * c.group * oc_blocks * pixels;
    for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t pix = idx % pixels;
        int64_t rest = idx / pixels;
        const int64_t ob = rest % oc_blocks; rest /= oc_blocks;
        const int64_t g = rest % c.group;
        const int64_t b = rest / c.group;
        const int64_t oy = pix / c.ow, ox = pix % c.ow;
        const int64_t oc0 = g * ocg + ob * kOcPerThread;
        const int noc = static_cast<int>((ocg - ob * kOcPerThread) < kOcPerThread ? (ocg - ob * kOcPerThread) : kOcPerThread);

        int32_t acc[kOcPerThread] = {0, 0, 0, 0};
        int32_t wzp[kOcPerThread] = {0, 0, 0, 0};
        if (c.w_zps != nullptr)
            for (int j = 0; j < noc; ++j) wzp[j] = c.w_zps[c.per_channel ? oc0 + j : 0];
        for (int64_t ci = 0; ci < icg; ++ci) {
            const int8_t* xin = c.x + ((b * c.ic + g * icg + ci) * c.ih) * c.iw;
            for (int64_t ky = 0; ky < c.kh; ++ky) {
                const int64_t iy = oy * c.stride_h + ky * c.dilation_h - c.pad_h;
                if (iy < 0 || iy >= c.ih) continue;  // padded taps contribute nothing (common/conv2d.cc:552-556)
                for (int64_t kx = 0; kx < c.kw; ++kx) {
                    const int64_t ix = ox * c.stride_w + kx * c.dilation_w - c.pad_w;
                    if (ix < 0 || ix >= c.iw) continue;
                    const int32_t xv = static_cast<int32_t>(xin[iy * c.iw + ix]) - c.x_zp;
#pragma unroll
                    for (int j = 0; j < kOcPerThread; ++j) {
                        if (j < noc) {
                            const int32_t wv = c.w[(((oc0 + j) * icg + ci) * c.kh + ky) * c.kw + kx];
                            acc[j] += xv * (wv - wzp[j]);
                        }
                    }
                }
            }
        }
        for (int j = 0; j < noc; ++j) {
            const int64_t o = oc0 + j;
            const int32_t total_acc = acc[j] + (c.bias ? c.bias[o] : 0);
            const double scale = static_cast<double>(c.x_scale) * static_cast<double>(c.w_scales[c.per_channel ? o : 0]);
            const double so = static_cast<double>(c.out_scale);
            int8_t q = RequantInt32(total_acc, scale, scale / so, so, c.out_zp);
            if (c.relu_lut != nullptr) q = c.relu_lut[static_cast<uint8_t>(static_cast<uint8_t>(q) + 128)];
            c.out[((b * c.oc + o) * c.oh + oy) * c.ow + ox] = q;
        }
    }
}

bool ValidScale(float s) { return std::isfinite(s) && s > 0.0f; }

int Validate(const fth_b200_int8_conv2d_desc* d, ConvArgs* c) {
    if (d == nullptr || !d->x || !d->w || !d->out || !d->w_scales) return FTH_B200_ERR_INVALID;
    if (d->batch <= 0 || d->ic <= 0 || d->ih <= 0 || d->iw <= 0 || d->oc <= 0 || d->kh <= 0 || d->kw <= 0) return FTH_B200_ERR_INVALID;
    if (d->stride_h <= 0 || d->stride_w <= 0 || d->dilation_h <= 0 || d->dilation_w <= 0 || d->group <= 0) return FTH_B200_ERR_INVALID;
    if (d->pad_h < 0 || d->pad_w < 0) return FTH_B200_ERR_INVALID;
    if (d->ic % d->group != 0 || d->oc % d->group != 0) return FTH_B200_ERR_INVALID;
    if (!ValidScale(d->x_scale) || !ValidScale(d->out_scale)) return FTH_B200_ERR_INVALID;
    if (d->x_zp < -128 || d->x_zp > 127 || d->out_zp < -128 || d->out_zp > 127) return FTH_B200_ERR_INVALID;
    if (d->w_params != 1 && d->w_params != d->oc) return FTH_B200_ERR_INVALID;
    if (d->w_zp_max_abs < 0 || d->w_zp_max_abs > 128 || d->bias_max_abs < 0) return FTH_B200_ERR_INVALID;
    const int64_t oh = (d->ih + 2 * d->pad_h - d->dilation_h * (d->kh - 1) - 1) / d->stride_h + 1;
    const int64_t ow = (d->iw + 2 * d->pad_w - d->dilation_w * (d->kw - 1) - 1) / d->stride_w + 1;
    if (oh <= 0 || ow <= 0) return FTH_B200_ERR_INVALID;
    const int64_t taps = (d->ic / d->group) * d->kh * d->kw;
    const int64_t a_span = 128 + (d->x_zp < 0 ? -d->x_zp : d->x_zp);
    if (taps * a_span * (128 + d->w_zp_max_abs) + d->bias_max_abs > 2147483647LL) return FTH_B200_ERR_OVERFLOW;
    c->x = d->x; c->w = d->w; c->bias = d->bias; c->out = d->out;
    c->batch = d->batch; c->ic = d->ic; c->ih = d->ih; c->iw = d->iw; c->oc = d->oc; c->kh = d->kh; c->kw = d->kw;
    c->oh = oh; c->ow = ow;
    c->stride_h = d->stride_h; c->stride_w = d->stride_w; c->pad_h = d->pad_h; c->pad_w = d->pad_w;
    c->dilation_h = d->dilation_h; c->dilation_w = d->dilation_w; c->group = d->group;
    c->x_scale = d->x_scale; c->x_zp = d->x_zp; c->w_scales = d->w_scales; c->w_zps = d->w_zps;
    c->per_channel = d->w_params != 1; c->out_scale = d->out_scale; c->out_zp = d->out_zp;
    c->relu_lut = d->relu_lut;
    c->workspace = d->workspace; c->workspace_bytes = d->workspace_bytes; c->weights_packed = d->weights_packed;
    c->packed_w = d->packed_w;
    return FTH_B200_OK;
}

int PickVariant(int requested, const ConvArgs& c) {
    if (requested == FTH_B200_VARIANT_SIMT) return FTH_B200_VARIANT_SIMT;
    if (requested == FTH_B200_VARIANT_TCGEN05) return ConvTcgen05Supported(c) ? requested : FTH_B200_ERR_UNSUPPORTED;
    if (requested != FTH_B200_VARIANT_AUTO) return FTH_B200_ERR_INVALID;
    return ConvTcgen05Supported(c) ? FTH_B200_VARIANT_TCGEN05 : FTH_B200_VARIANT_SIMT;
}

}  // namespace
}  // namespace fth

using namespace fth;

extern "C" int fth_b200_int8_conv2d_supported(const fth_b200_int8_conv2d_desc* d) {
    ConvArgs c;
    const int rc = Validate(d, &c);
    if (rc != FTH_B200_OK) return rc;
    const int v = PickVariant(d->variant, c);
    return v < 0 ? v : FTH_B200_OK;
}

extern "C" size_t fth_b200_int8_conv2d_workspace_bytes(const fth_b200_int8_conv2d_desc* d) {
    ConvArgs c;
    if (Validate(d, &c) != FTH_B200_OK) return 0;
    return ConvTcgen05WorkspaceBytes(c);
}

extern "C" size_t fth_b200_int8_conv2d_packed_weight_bytes(const fth_b200_int8_conv2d_desc* d) {
    ConvArgs c;
    if (Validate(d, &c) != FTH_B200_OK) return 0;
    return ConvPackedWeightBytes(c);
}

extern "C" int fth_b200_int8_conv2d_pack_weights(const fth_b200_int8_conv2d_desc* d, void* packed, fth_b200_stream_t stream) {
    ClearStaleError();
    ConvArgs c;
    const int rc = Validate(d, &c);
    if (rc != FTH_B200_OK) return rc;
    return LaunchConvPackWeights(c, packed, static_cast<cudaStream_t>(stream));
}

extern "C" int fth_b200_int8_conv2d(const fth_b200_int8_conv2d_desc* d, fth_b200_stream_t stream_) {
    ClearStaleError();
    auto stream = static_cast<cudaStream_t>(stream_);
    ConvArgs c;
    const int rc = Validate(d, &c);
    if (rc != FTH_B200_OK) return rc;
    const int v = PickVariant(d->variant, c);
    if (v < 0) return v;
    if (v == FTH_B200_VARIANT_TCGEN05) return LaunchConvTcgen05(c, stream);
    const int64_t ocg = c.oc / c.group;
    const int64_t total = c.batch * c.group * ((ocg + kOcPerThread - 1) / kOcPerThread) * c.oh * c.ow;
    int64_t blocks = (total + kThreads - 1) / kThreads;
    const int64_t cap = static_cast<int64_t>(kNumSms) * 16;
    if (blocks > cap) blocks = cap;
    ConvDirectKernel<<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(c);
    NoteLaunch("conv_direct");
    return CheckLaunch();
}
