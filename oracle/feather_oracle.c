/* TEST INFRASTRUCTURE — not part of the shipped library.
 *
 * Plain-C restatement of the reference's ("Feather") portable Common kernels for the quantized-linear
 * path.  Only tests, the smoke check and the CPU-baseline leg of the benchmark may load it; the CUDA
 * library never links or calls it.
 *
 * Parity pin: every function below is checked against (1) the known-answer values of the reference's own
 * unit tests and (2) outputs of the unmodified reference library (oracle/_ref/libfeather_ref.so) on seeded
 * inputs, stored as fixtures under tests/golden/ — see tests/test_oracle_*.py.
 *
 * Compile with -ffp-contract=off: the reference builds its Common kernels for baseline x86-64, so their
 * `sum += a * b` is a separate multiply and add (no FMA).
 *
 * OpenMP is used only across independent outputs, so threading never changes a result.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define FO_E4M3 12 /* feather::DataType::FP8E4M3, include/util/types.h:45 */
#define FO_E5M2 13 /* feather::DataType::FP8E5M2, include/util/types.h:46 */
#define FO_FP16 3
#define FO_FP32 4
#define FO_BF16 11

static uint32_t f2u(float v) { uint32_t b; memcpy(&b, &v, 4); return b; }
static float u2f(uint32_t b) { float v; memcpy(&v, &b, 4); return v; }

/* ---- FP8 codec: include/util/fp8.h:66-204 ---------------------------------------------------------- */

/* fp8.h:66-73 — round half to even on a non-negative value. */
static int32_t round_nearest_even(float value) {
    const int32_t lower = (int32_t)value;
    const float fraction = value - (float)lower;
    if (fraction > 0.5f || (fraction == 0.5f && (lower & 1) != 0)) return lower + 1;
    return lower;
}

/* fp8.h:81-146 — saturating RNE encode of a finite magnitude. */
static uint8_t encode_finite(float mag, uint8_t sign, int mbits, int bias, int max_exp, int max_man, int has_inf) {
    const float min_normal = has_inf ? 0.00006103515625f : 0.015625f;
    const float quantum = has_inf ? 0.0000152587890625f : 0.001953125f;
    const float max_finite = has_inf ? 57344.0f : 448.0f;
    const uint8_t max_code = has_inf ? 0x7bU : 0x7eU;
    const int exp_mask = has_inf ? 0x1f : 0x0f;
    if (mag < min_normal) {
        const int32_t sub = round_nearest_even(mag / quantum);
        if (sub <= 0) return sign;
        if (sub >= (1 << mbits)) return (uint8_t)(sign | (1 << mbits));
        return (uint8_t)(sign | sub);
    }
    if (mag > max_finite) return (uint8_t)(sign | max_code);
    int exponent = 0;
    float fraction = mag;
    while (fraction >= 2.0f) { fraction *= 0.5f; ++exponent; }
    while (fraction < 1.0f) { fraction *= 2.0f; --exponent; }
    int32_t man = round_nearest_even((fraction - 1.0f) * (float)(1 << mbits));
    if (man >= (1 << mbits)) { man = 0; ++exponent; }
    if (exponent > max_exp) return (uint8_t)(sign | max_code);
    int field = exponent + bias;
    if (field <= 0) {
        const int32_t sub = round_nearest_even(mag / quantum);
        if (sub <= 0) return sign;
        if (sub >= (1 << mbits)) return (uint8_t)(sign | (1 << mbits));
        return (uint8_t)(sign | sub);
    }
    if (field >= exp_mask) {
        field = exp_mask;
        if (man > max_man) man = max_man;
    }
    return (uint8_t)(sign | (field << mbits) | man);
}

/* fp8.h:148-172 — NaN → 0x7F (E4M3) / 0x7D (E5M2); Inf → 0x7E (saturate) / 0x7C. */
uint8_t fo_fp8_encode(int dtype, float value) {
    const uint32_t bits = f2u(value);
    const uint8_t sign = (uint8_t)((bits >> 24) & 0x80u);
    const uint32_t exponent = (bits >> 23) & 0xffu;
    const uint32_t mantissa = bits & 0x7fffffu;
    const float mag = value < 0.0f ? -value : value;
    if (dtype == FO_E4M3) {
        if (exponent == 0xffu) return (uint8_t)(sign | (mantissa != 0 ? 0x7fU : 0x7eU));
        return encode_finite(mag, sign, 3, 7, 8, 6, 0);
    }
    if (exponent == 0xffu) return (uint8_t)(sign | (mantissa == 0 ? 0x7cU : 0x7dU));
    return encode_finite(mag, sign, 2, 15, 15, 3, 1);
}

/* fp8.h:174-204 */
float fo_fp8_decode(int dtype, uint8_t bits) {
    const uint8_t sign = bits & 0x80u;
    float value;
    if (dtype == FO_E4M3) {
        const int e = (bits >> 3) & 0x0f, m = bits & 0x07;
        if (e == 0 && m == 0) return sign ? -0.0f : 0.0f;
        if (e == 15 && m == 7) return u2f(0x7fc00000u);
        value = e == 0 ? (float)m * 0.001953125f : (1.0f + (float)m * 0.125f) * ldexpf(1.0f, e - 7);
    } else {
        const int e = (bits >> 2) & 0x1f, m = bits & 0x03;
        if (e == 0 && m == 0) return sign ? -0.0f : 0.0f;
        if (e == 31) return m == 0 ? (sign ? u2f(0xff800000u) : u2f(0x7f800000u)) : u2f(0x7fc00000u);
        value = e == 0 ? (float)m * 0.0000152587890625f : (1.0f + (float)m * 0.25f) * ldexpf(1.0f, e - 15);
    }
    return sign ? -value : value;
}

void fo_fp8_encode_array(int dtype, const float* v, uint8_t* out, int64_t n) {
#pragma omp parallel for schedule(static) if (n > 65536)
    for (int64_t i = 0; i < n; ++i) out[i] = fo_fp8_encode(dtype, v[i]);
}
void fo_fp8_decode_array(int dtype, const uint8_t* b, float* out, int64_t n) {
#pragma omp parallel for schedule(static) if (n > 65536)
    for (int64_t i = 0; i < n; ++i) out[i] = fo_fp8_decode(dtype, b[i]);
}

/* ---- 16-bit floats ---------------------------------------------------------------------------------- */

/* include/util/bf16.h:35-46 — RNE, NaN quieted (used by Cast). */
uint16_t fo_bf16_encode(float value) {
    const uint32_t b = f2u(value);
    if ((b & 0x7f800000u) == 0x7f800000u && (b & 0x007fffffu) != 0) return (uint16_t)((b >> 16) | 0x0040u);
    return (uint16_t)((b + 0x7fffu + ((b >> 16) & 1u)) >> 16);
}
/* src/kernel/common/quantize_linear_utils.h:109-116 — RNE without NaN quieting (used by DequantizeLinear). */
uint16_t fo_bf16_encode_dq(float value) {
    const uint32_t b = f2u(value);
    const uint32_t low = b & 0xffffu;
    uint32_t high = b >> 16;
    if (low > 0x8000u || (low == 0x8000u && (high & 1u))) ++high;
    return (uint16_t)high;
}
float fo_bf16_decode(uint16_t bits) { return u2f((uint32_t)bits << 16); }
/* IEEE binary16, RNE both ways (hardware conversion semantics). */
uint16_t fo_f16_encode(float value) { _Float16 h = (_Float16)value; uint16_t b; memcpy(&b, &h, 2); return b; }
float fo_f16_decode(uint16_t bits) { _Float16 h; memcpy(&h, &bits, 2); return (float)h; }

/* ---- INT8 scalar math --------------------------------------------------------------------------------- */

/* include/quant/quantization.h:94-99 — FP64 divide, add zero point, round ties AWAY from zero, clamp. */
int8_t fo_quantize_int8_value(float value, float scale, int32_t zero_point) {
    const double t = (double)value / (double)scale + zero_point;
    const double r = round(t);
    const double c = fmax(-128.0, fmin(127.0, r));
    return (int8_t)c;
}

/* src/kernel/common/int8_kernel_utils.h:159-173 — returns 0 on success, -1 on a non-finite value. */
static int quantize_real(double real, float out_scale, int32_t out_zp, int8_t* result) {
    if (!isfinite(real) || !isfinite(out_scale) || out_scale <= 0.0f) return -1;
    const double t = real / (double)out_scale + out_zp;
    if (!isfinite(t)) return -1;
    const double r = round(t);
    *result = (int8_t)fmax(-128.0, fmin(127.0, r));
    return 0;
}

static int fits_int32(int64_t v) { return v >= INT32_MIN && v <= INT32_MAX; }

/* ---- FP8 FC / MatMul / Gemm: src/kernel/common/fc.cc:48-76, matmul.cc:56-154, gemm.cc:62-99 -------------
 * a [M,K]; w [K,N] (trans_b: [N,K]); bias FP8 [N] (mode 1) or [M,N] (mode 2), mode 0 none.
 * op 0 FC / 1 MatMul: sum (+ bias);  op 2 Gemm: sum *= alpha; sum += beta * bias.
 * Each term is (decode(a)·s_a)·(decode(w)·s_w) in FP32, added in ascending k; the result is
 * encode(sum / s_out) with an FP32 divide (src/kernel/common/kernel_io.h:58-78).
 * fo_fp8_linear_plain is the loop nest as the reference writes it (one output at a time); fo_fp8_linear below
 * computes the same values in the same per-output order, blocked over columns so that large slices finish in
 * seconds.  tests/test_oracle_blocked.py checks that the two agree byte for byte. */
int fo_fp8_linear_plain(int op, int dtype, const uint8_t* a, float a_scale, const uint8_t* w, float w_scale,
                  const uint8_t* bias, float bias_scale, int bias_mode, uint8_t* out, float out_scale, int64_t m,
                  int64_t k, int64_t n, int trans_b, float alpha, float beta) {
    if (m <= 0 || k <= 0 || n <= 0 || !a || !w || !out) return -1;
    float dec_a[256], dec_w[256], dec_b[256];
    for (int i = 0; i < 256; ++i) {
        dec_a[i] = fo_fp8_decode(dtype, (uint8_t)i) * a_scale;
        dec_w[i] = fo_fp8_decode(dtype, (uint8_t)i) * w_scale;
        dec_b[i] = fo_fp8_decode(dtype, (uint8_t)i) * bias_scale;
    }
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t i = 0; i < m; ++i) {
        for (int64_t j = 0; j < n; ++j) {
            float sum = 0.0f;
            if (trans_b) {
                const uint8_t* wr = w + j * k;
                for (int64_t t = 0; t < k; ++t) sum += dec_a[a[i * k + t]] * dec_w[wr[t]];
            } else {
                for (int64_t t = 0; t < k; ++t) sum += dec_a[a[i * k + t]] * dec_w[w[t * n + j]];
            }
            if (op == 2) {
                sum *= alpha;
                if (bias_mode == 1) sum += beta * dec_b[bias[j]];
                else if (bias_mode == 2) sum += beta * dec_b[bias[i * n + j]];
            } else {
                if (bias_mode == 1) sum += dec_b[bias[j]];
                else if (bias_mode == 2) sum += dec_b[bias[i * n + j]];
            }
            out[i * n + j] = fo_fp8_encode(dtype, sum / out_scale);
        }
    }
    return 0;
}

/* Column-blocked evaluation of the same contract.  A block of FO_BLOCK output columns is decoded once
 * (value·s_w, the factor the plain loop multiplies with) and every activation row then walks k in ascending order
 * with one partial sum per column: each output still sees sum = ((0 + a_0·w_0) + a_1·w_1) + …, an FP32 multiply
 * followed by an FP32 add (no contraction: the file is compiled with -ffp-contract=off), so the bits are the
 * plain loop's.  Threads split column blocks only. */
#define FO_BLOCK 64
int fo_fp8_linear(int op, int dtype, const uint8_t* a, float a_scale, const uint8_t* w, float w_scale,
                  const uint8_t* bias, float bias_scale, int bias_mode, uint8_t* out, float out_scale, int64_t m,
                  int64_t k, int64_t n, int trans_b, float alpha, float beta) {
    if (m <= 0 || k <= 0 || n <= 0 || !a || !w || !out) return -1;
    float dec_a[256], dec_w[256], dec_b[256];
    for (int i = 0; i < 256; ++i) {
        dec_a[i] = fo_fp8_decode(dtype, (uint8_t)i) * a_scale;
        dec_w[i] = fo_fp8_decode(dtype, (uint8_t)i) * w_scale;
        dec_b[i] = fo_fp8_decode(dtype, (uint8_t)i) * bias_scale;
    }
    const int64_t blocks = (n + FO_BLOCK - 1) / FO_BLOCK;
    int failed = 0;
#pragma omp parallel
    {
        float* wdec = (float*)malloc((size_t)k * FO_BLOCK * sizeof(float));
        float* arow = (float*)malloc((size_t)k * sizeof(float));
        if (!wdec || !arow) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp for schedule(dynamic, 1)
        for (int64_t jb = 0; jb < blocks; ++jb) {
            if (!wdec || !arow) continue;
            const int64_t j0 = jb * FO_BLOCK;
            const int cnt = (int)(n - j0 < FO_BLOCK ? n - j0 : FO_BLOCK);
            if (trans_b) {
                for (int c = 0; c < FO_BLOCK; ++c) {
                    if (c < cnt) { const uint8_t* wr = w + (j0 + c) * k; for (int64_t t = 0; t < k; ++t) wdec[t * FO_BLOCK + c] = dec_w[wr[t]]; }
                    else { for (int64_t t = 0; t < k; ++t) wdec[t * FO_BLOCK + c] = 0.0f; }
                }
            } else {
                for (int64_t t = 0; t < k; ++t) {
                    const uint8_t* wr = w + t * n + j0;
                    for (int c = 0; c < FO_BLOCK; ++c) wdec[t * FO_BLOCK + c] = c < cnt ? dec_w[wr[c]] : 0.0f;
                }
            }
            for (int64_t i = 0; i < m; ++i) {
                for (int64_t t = 0; t < k; ++t) arow[t] = dec_a[a[i * k + t]];
                float sum[FO_BLOCK];
                for (int c = 0; c < FO_BLOCK; ++c) sum[c] = 0.0f;
                for (int64_t t = 0; t < k; ++t) {
                    const float av = arow[t];
                    const float* wr = wdec + t * FO_BLOCK;
                    for (int c = 0; c < FO_BLOCK; ++c) sum[c] += av * wr[c];
                }
                for (int c = 0; c < cnt; ++c) {
                    const int64_t j = j0 + c;
                    float s = sum[c];
                    if (op == 2) {
                        s *= alpha;
                        if (bias_mode == 1) s += beta * dec_b[bias[j]];
                        else if (bias_mode == 2) s += beta * dec_b[bias[i * n + j]];
                    } else {
                        if (bias_mode == 1) s += dec_b[bias[j]];
                        else if (bias_mode == 2) s += dec_b[bias[i * n + j]];
                    }
                    out[i * n + j] = fo_fp8_encode(dtype, s / out_scale);
                }
            }
        }
        free(wdec);
        free(arow);
    }
    return failed ? -1 : 0;
}

/* ---- INT8 FC / MatMul / Gemm: src/kernel/common/fc.cc:105-159, gemm.cc:136-198, matmul.cc:156-261 --------
 * w_scales/w_zps hold `w_channels` entries (per output channel) or one entry when w_channels == 0.
 * bias int32 [N] (mode 1) / [M,N] (mode 2).  Returns -1 if any running sum leaves int32. */
int fo_int8_linear_plain(int op, const int8_t* a, float a_scale, int32_t a_zp, const int8_t* w, const float* w_scales,
                   const int32_t* w_zps, int64_t w_channels, const int32_t* bias, int bias_mode, int8_t* out,
                   float out_scale, int32_t out_zp, int64_t m, int64_t k, int64_t n, int trans_b, float alpha,
                   float beta) {
    if (m <= 0 || k <= 0 || n <= 0 || !a || !w || !out) return -1;
    int failed = 0;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t i = 0; i < m; ++i) {
        for (int64_t j = 0; j < n; ++j) {
            const int32_t wzp = w_zps ? (w_channels ? w_zps[j] : w_zps[0]) : 0;
            const float ws = w_channels ? w_scales[j] : w_scales[0];
            int64_t acc = 0;
            int bad = 0;
            for (int64_t t = 0; t < k; ++t) {
                const int32_t wv = trans_b ? w[j * k + t] : w[t * n + j];
                acc += (int64_t)((int32_t)a[i * k + t] - a_zp) * (wv - wzp);
                if (!fits_int32(acc)) bad = 1;
            }
            const int32_t b = bias_mode == 1 ? bias[j] : bias_mode == 2 ? bias[i * n + j] : 0;
            const double scale = (double)a_scale * ws; /* double·float → double, fc.cc:150-151 */
            double real;
            if (op == 2) {
                real = ((double)alpha * (double)acc + (double)beta * (double)b) * scale; /* gemm.cc:185-190 */
            } else {
                acc += b;
                if (!fits_int32(acc)) bad = 1;
                real = (double)acc * scale;
            }
            int8_t q = 0;
            if (bad || quantize_real(real, out_scale, out_zp, &q) != 0) {
#pragma omp atomic write
                failed = 1;
            }
            out[i * n + j] = q;
        }
    }
    return failed ? -1 : 0;
}

/* Column-blocked evaluation of fo_int8_linear_plain.  Integer sums do not depend on the order of their terms, and
 * when K·(128+|zp_a|)·(128+max|zp_w|) + max|bias| fits int32 no prefix of any sum can leave int32, so the plain
 * loop's overflow checks cannot fire and 32-bit accumulation gives the same accumulator.  Shapes outside that
 * bound take the plain loop. */
int fo_int8_linear(int op, const int8_t* a, float a_scale, int32_t a_zp, const int8_t* w, const float* w_scales,
                   const int32_t* w_zps, int64_t w_channels, const int32_t* bias, int bias_mode, int8_t* out,
                   float out_scale, int32_t out_zp, int64_t m, int64_t k, int64_t n, int trans_b, float alpha,
                   float beta) {
    if (m <= 0 || k <= 0 || n <= 0 || !a || !w || !out) return -1;
    int64_t wzp_max = 0, bias_max = 0;
    if (w_zps) {
        const int64_t cnt = w_channels ? n : 1;
        for (int64_t j = 0; j < cnt; ++j) { const int64_t v = llabs((long long)w_zps[j]); if (v > wzp_max) wzp_max = v; }
    }
    if (bias_mode) {
        const int64_t cnt = bias_mode == 1 ? n : m * n;
        for (int64_t j = 0; j < cnt; ++j) { const int64_t v = llabs((long long)bias[j]); if (v > bias_max) bias_max = v; }
    }
    const int64_t worst = k * (128 + llabs((long long)a_zp)) * (128 + wzp_max) + bias_max;
    if (worst > INT32_MAX || k > (1 << 24))
        return fo_int8_linear_plain(op, a, a_scale, a_zp, w, w_scales, w_zps, w_channels, bias, bias_mode, out, out_scale,
                                    out_zp, m, k, n, trans_b, alpha, beta);
    const int64_t blocks = (n + FO_BLOCK - 1) / FO_BLOCK;
    int failed = 0;
#pragma omp parallel
    {
        int32_t* wq = (int32_t*)malloc((size_t)k * FO_BLOCK * sizeof(int32_t));
        int32_t* arow = (int32_t*)malloc((size_t)k * sizeof(int32_t));
        if (!wq || !arow) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp for schedule(dynamic, 1)
        for (int64_t jb = 0; jb < blocks; ++jb) {
            if (!wq || !arow) continue;
            const int64_t j0 = jb * FO_BLOCK;
            const int cnt = (int)(n - j0 < FO_BLOCK ? n - j0 : FO_BLOCK);
            for (int c = 0; c < FO_BLOCK; ++c) {
                const int64_t j = j0 + c;
                const int32_t wzp = (c < cnt && w_zps) ? (w_channels ? w_zps[j] : w_zps[0]) : 0;
                for (int64_t t = 0; t < k; ++t) {
                    int32_t v = 0;
                    if (c < cnt) v = (int32_t)(trans_b ? w[j * k + t] : w[t * n + j]) - wzp;
                    wq[t * FO_BLOCK + c] = v;
                }
            }
            for (int64_t i = 0; i < m; ++i) {
                for (int64_t t = 0; t < k; ++t) arow[t] = (int32_t)a[i * k + t] - a_zp;
                int32_t sum[FO_BLOCK];
                for (int c = 0; c < FO_BLOCK; ++c) sum[c] = 0;
                for (int64_t t = 0; t < k; ++t) {
                    const int32_t av = arow[t];
                    const int32_t* wr = wq + t * FO_BLOCK;
                    for (int c = 0; c < FO_BLOCK; ++c) sum[c] += av * wr[c];
                }
                for (int c = 0; c < cnt; ++c) {
                    const int64_t j = j0 + c;
                    const float ws = w_channels ? w_scales[j] : w_scales[0];
                    int64_t acc = sum[c];
                    const int32_t b = bias_mode == 1 ? bias[j] : bias_mode == 2 ? bias[i * n + j] : 0;
                    const double scale = (double)a_scale * ws;
                    double real;
                    if (op == 2) real = ((double)alpha * (double)acc + (double)beta * (double)b) * scale;
                    else { acc += b; real = (double)acc * scale; }
                    int8_t q = 0;
                    if (quantize_real(real, out_scale, out_zp, &q) != 0) {
#pragma omp atomic write
                        failed = 1;
                    }
                    out[i * n + j] = q;
                }
            }
        }
        free(wq);
        free(arow);
    }
    return failed ? -1 : 0;
}

/* ---- INT8 Conv2D, NCHW / OIHW: src/kernel/common/conv2d.cc:481-581 ---------------------------------------
 * Padded taps are skipped (they contribute 0); accumulator starts from the int32 bias. */
int fo_int8_conv2d(const int8_t* x, float x_scale, int32_t x_zp, const int8_t* w, const float* w_scales,
                   const int32_t* w_zps, int64_t w_channels, const int32_t* bias, int8_t* out, float out_scale,
                   int32_t out_zp, int64_t batch, int64_t ic, int64_t ih, int64_t iw, int64_t oc, int64_t kh,
                   int64_t kw, int32_t stride_h, int32_t stride_w, int32_t pad_h, int32_t pad_w, int32_t dil_h,
                   int32_t dil_w, int32_t group) {
    if (group <= 0 || ic % group || oc % group) return -1;
    const int64_t icg = ic / group, ocg = oc / group;
    const int64_t oh = (ih + 2 * pad_h - dil_h * (kh - 1) - 1) / stride_h + 1;
    const int64_t ow = (iw + 2 * pad_w - dil_w * (kw - 1) - 1) / stride_w + 1;
    if (oh <= 0 || ow <= 0) return -1;
    int failed = 0;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < batch; ++b) {
        for (int64_t o = 0; o < oc; ++o) {
            const int64_t g = o / ocg;
            const int32_t wzp = w_zps ? (w_channels ? w_zps[o] : w_zps[0]) : 0;
            const double scale = (double)x_scale * (w_channels ? w_scales[o] : w_scales[0]);
            for (int64_t y = 0; y < oh; ++y) {
                for (int64_t xw = 0; xw < ow; ++xw) {
                    int64_t acc = bias ? bias[o] : 0;
                    int bad = 0;
                    for (int64_t c = 0; c < icg; ++c) {
                        const int64_t gc = g * icg + c;
                        for (int64_t ky = 0; ky < kh; ++ky) {
                            const int64_t iy = y * stride_h + ky * dil_h - pad_h;
                            if (iy < 0 || iy >= ih) continue;
                            for (int64_t kx = 0; kx < kw; ++kx) {
                                const int64_t ix = xw * stride_w + kx * dil_w - pad_w;
                                if (ix < 0 || ix >= iw) continue;
                                acc += (int64_t)((int32_t)x[((b * ic + gc) * ih + iy) * iw + ix] - x_zp) *
                                       ((int32_t)w[((o * icg + c) * kh + ky) * kw + kx] - wzp);
                                if (!fits_int32(acc)) bad = 1;
                            }
                        }
                    }
                    int8_t q = 0;
                    if (bad || quantize_real((double)acc * scale, out_scale, out_zp, &q) != 0) {
#pragma omp atomic write
                        failed = 1;
                    }
                    out[((b * oc + o) * oh + y) * ow + xw] = q;
                }
            }
        }
    }
    return failed ? -1 : 0;
}

/* ---- INT8 ReLU node: src/kernel/common/int8_standard.cc:114-128,148-176 --------------------------------
 * lut[q+128] = QuantizeInt8Value(max(0, float(q - zp_in)·s_in), s_out, zp_out). */
void fo_int8_relu_lut(float in_scale, int32_t in_zp, float out_scale, int32_t out_zp, int8_t* lut256) {
    for (int32_t q = -128; q <= 127; ++q) {
        const float real = (float)(q - in_zp) * in_scale;
        const float r = real > 0.0f ? real : 0.0f;
        lut256[q + 128] = fo_quantize_int8_value(r, out_scale, out_zp);
    }
}
void fo_int8_relu(const int8_t* x, int8_t* out, int64_t count, float in_scale, int32_t in_zp, float out_scale,
                  int32_t out_zp) {
    int8_t lut[256];
    fo_int8_relu_lut(in_scale, in_zp, out_scale, out_zp, lut);
    for (int64_t i = 0; i < count; ++i) out[i] = lut[(int32_t)x[i] + 128];
}

/* ---- QuantizeLinear / DequantizeLinear: src/kernel/common/quantize_linear_utils.h:236-341 ---------------
 * x [rows, channels]; `params` == 1 → per-tensor, == channels → per-channel on the last axis. */
static float read_float(int dtype, const void* p, int64_t i) {
    if (dtype == FO_FP32) return ((const float*)p)[i];
    if (dtype == FO_FP16) return fo_f16_decode(((const uint16_t*)p)[i]);
    return fo_bf16_decode(((const uint16_t*)p)[i]);
}
int fo_quantize_linear(int x_dtype, const void* x, const float* scales, const int32_t* zps, int64_t params,
                       int8_t* out, int64_t rows, int64_t channels) {
    if (params != 1 && params != channels) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < rows * channels; ++i) {
        const int64_t c = params == 1 ? 0 : i % channels;
        out[i] = fo_quantize_int8_value(read_float(x_dtype, x, i), scales[c], zps[c]);
    }
    return 0;
}
int fo_dequantize_linear(const int8_t* x, const float* scales, const int32_t* zps, int64_t params, void* out,
                         int to_dtype, int64_t rows, int64_t channels) {
    if (params != 1 && params != channels) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < rows * channels; ++i) {
        const int64_t c = params == 1 ? 0 : i % channels;
        const float v = (float)((int32_t)x[i] - zps[c]) * scales[c];
        if (to_dtype == FO_FP32) ((float*)out)[i] = v;
        else if (to_dtype == FO_FP16) ((uint16_t*)out)[i] = fo_f16_encode(v);
        else ((uint16_t*)out)[i] = fo_bf16_encode_dq(v);
    }
    return 0;
}

/* ---- Cast among FP32 / FP16 / BF16 / FP8: src/kernel/common/cast.cc:62-126 --------------------------------
 * Read: FP8 → decode·s_in; Write: FP8 ← encode(v / s_out), BF16 via util/bf16.h (NaN quieted). */
int fo_cast(int in_dtype, const void* x, float in_scale, int out_dtype, void* out, float out_scale, int64_t count) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        float v;
        if (in_dtype == FO_E4M3 || in_dtype == FO_E5M2) v = fo_fp8_decode(in_dtype, ((const uint8_t*)x)[i]) * in_scale;
        else v = read_float(in_dtype, x, i);
        if (out_dtype == FO_FP32) ((float*)out)[i] = v;
        else if (out_dtype == FO_BF16) ((uint16_t*)out)[i] = fo_bf16_encode(v);
        else if (out_dtype == FO_FP16) ((uint16_t*)out)[i] = fo_f16_encode(v);
        else ((uint8_t*)out)[i] = fo_fp8_encode(out_dtype, v / out_scale);
    }
    return 0;
}

/* ---- QwenRmsNorm: src/kernel/common/qwen_rms_norm.cc:71-95 ----------------------------------------------------
 * x / weight / out FP32 or BF16.  Squares are added one after another in FP32; inverse_rms = 1 / sqrt(sum / hidden + eps);
 * out = x * inverse_rms * (weight + weight_offset), each multiply rounded; BF16 output through util/bf16.h. */
int fo_qwen_rms_norm(int x_dtype, const void* x, int w_dtype, const void* w, float weight_offset, float epsilon,
                     int out_dtype, void* out, int64_t rows, int64_t hidden) {
    if (rows <= 0 || hidden <= 0 || !x || !w || !out) return -1;
    if ((x_dtype != FO_FP32 && x_dtype != FO_BF16) || (w_dtype != FO_FP32 && w_dtype != FO_BF16) ||
        (out_dtype != FO_FP32 && out_dtype != FO_BF16) || !isfinite(epsilon) || epsilon < 0.0f) return -1;
#pragma omp parallel for schedule(static) if (rows > 8)
    for (int64_t r = 0; r < rows; ++r) {
        float sum_square = 0.0f;
        for (int64_t c = 0; c < hidden; ++c) {
            const float v = read_float(x_dtype, x, r * hidden + c);
            sum_square += v * v;
        }
        const float inverse_rms = 1.0f / sqrtf(sum_square / (float)hidden + epsilon);
        for (int64_t c = 0; c < hidden; ++c) {
            const float v = read_float(x_dtype, x, r * hidden + c);
            const float scale = read_float(w_dtype, w, c) + weight_offset;
            const float y = v * inverse_rms * scale;
            if (out_dtype == FO_BF16) ((uint16_t*)out)[r * hidden + c] = fo_bf16_encode(y);
            else ((float*)out)[r * hidden + c] = y;
        }
    }
    return 0;
}

/* ---- Add / Mul (src/kernel/common/add.cc:80-109, mul.cc) and SiLU (src/kernel/common/silu.cc:38-55) -------------
 * FP32 / FP16 / BF16: read as float, one operation, one rounding to the output type (TensorIO<dtype>::Write).
 * rhs is the same shape (rhs_count == count) or one trailing row broadcast over lhs.  op: 0 Add, 1 Mul. */
static void write_float(int dtype, void* out, int64_t i, float v) {
    if (dtype == FO_FP32) ((float*)out)[i] = v;
    else if (dtype == FO_FP16) ((uint16_t*)out)[i] = fo_f16_encode(v);
    else ((uint16_t*)out)[i] = fo_bf16_encode(v);
}
int fo_binary(int op, int dtype, const void* lhs, const void* rhs, void* out, int64_t count, int64_t rhs_count) {
    if (count <= 0 || rhs_count <= 0 || count % rhs_count != 0 || (op != 0 && op != 1)) return -1;
    for (int64_t i = 0; i < count; ++i) {
        const float a = read_float(dtype, lhs, i), b = read_float(dtype, rhs, i % rhs_count);
        write_float(dtype, out, i, op == 0 ? a + b : a * b);
    }
    return 0;
}
int fo_silu(int dtype, const void* x, void* out, int64_t count) {
    for (int64_t i = 0; i < count; ++i) {
        const float v = read_float(dtype, x, i);
        write_float(dtype, out, i, v / (1.0f + expf(-v)));
    }
    return 0;
}
