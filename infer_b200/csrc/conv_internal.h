// Internal interface between the INT8 Conv2D entry point and its kernel families.
#pragma once

#include "common.cuh"

namespace fth {

struct ConvArgs {
    const int8_t* x;
    const int8_t* w;
    const int32_t* bias;
    int8_t* out;
    int64_t batch, ic, ih, iw, oc, kh, kw, oh, ow;
    int32_t stride_h, stride_w, pad_h, pad_w, dilation_h, dilation_w, group;
    float x_scale;
    int32_t x_zp;
    const float* w_scales;
    const int32_t* w_zps;
    int per_channel;
    float out_scale;
    int32_t out_zp;
    const int8_t* relu_lut;
    void* workspace;
    size_t workspace_bytes;
    int weights_packed;
    const int8_t* packed_w;  // caller-owned packed weight, or null (then it lives behind the NHWC copy in the workspace)
};

bool ConvTcgen05Supported(const ConvArgs& c);
size_t ConvTcgen05WorkspaceBytes(const ConvArgs& c);
int LaunchConvTcgen05(const ConvArgs& c, cudaStream_t stream);
size_t ConvPackedWeightBytes(const ConvArgs& c);
int LaunchConvPackWeights(const ConvArgs& c, void* packed, cudaStream_t stream);

}  // namespace fth
