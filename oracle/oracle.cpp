// CPU oracle for the quantized operator path of the ENN GPU userdriver.
//
// TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or calls this file; it is the
// checker the parity tests, the smoke test and the CPU-baseline leg of the benchmark compare against.
//
// The reference has no CPU implementation of quantized Conv2D / DepthwiseConv2D / Deconvolution /
// FullyConnected: the arithmetic exists only as OpenCL C kernel text plus host C++ that derives the
// requantisation parameters.  This file restates both in plain C++ (NHWC activations; the reference runs
// NCHW and transposes around it, results are the same set of numbers).  Each function cites the reference
// lines it follows (paths relative to the reference's src/userdriver/gpu unless stated).
//
// Parity pins:
//   * host quantisation math is cross-checked against the reference's own QuantizationUtil.cpp /
//     KernelUtil.cpp compiled from the reference tree (oracle/_ref, see oracle/Makefile) and against
//     fixtures generated from that build (tests/golden/quant_host.json);
//   * per-channel conv arithmetic is pinned by the reference known-answer test
//     gpu_userdriver_test.cc:474-575 (tests/golden/kat_perchannel_conv.json);
//   * the kernel restatements are pinned against the reference's OWN OpenCL C kernel text: oracle/ref_dump_kernels.cpp
//     extracts the registered source strings at build time and oracle/ref_kernels_shim.cpp compiles them as C++ and
//     replays the operators' host launch sequence.  Covered: conv_per_channel_quantized, depthwise_conv,
//     depthwise_conv_per_channel, matrixTrans / weightAlign / convBackGemmRXR / PERCHANNELconvBackGemmRXR /
//     convertBottomDiff2[_per_channel], avepooling_tflite, eltwiseAddQuantized_opt, and the per-tensor u8 convolution of
//     CLGEMMConvolutionQuantized: pad_opt, convert_optimized / convertBlocked2, alignQuantizedWeight_gemm,
//     quantizedGemmBlocked (live comparison where the reference tree is mounted, tests/golden/ref_kernels.npz elsewhere).
//   * Not executed: the other per-tensor conv variants (direct3x3_8x4, gemm_block4x4: ARM dot-product built-ins and
//     texture-style layouts).  They compute the value of quantizedGemmBlocked with the zero-point terms folded into the
//     bias (DirectConvolutionKernel.cpp:4871-4884, ConvolutionGEMM1xXkernels.cpp:2003-2013).  FullyConnected: see orc_fc /
//     orc_fc_float below.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../include/enn_b200.h"

extern "C" {

// ---------------------------------------------------------------------------------------------
// Host quantisation helpers
// ---------------------------------------------------------------------------------------------

// operators/cl_quantized_utils/QuantizationUtil.cpp:8-21 (QuantizeMultiplier) and :29-35
// (QuantizeMultiplierSmallerThanOneExp just forwards the signed shift).
void orc_quantize_multiplier(double m, int32_t *qm, int32_t *shift) {
    if (m == 0.) {
        *qm = 0;
        *shift = 0;
        return;
    }
    int e = 0;
    const double q = std::frexp(m, &e);
    int64_t q_fixed = static_cast<int64_t>(std::round(q * (1ll << 31)));
    if (q_fixed == (1ll << 31)) {
        q_fixed /= 2;
        ++e;
    }
    *qm = static_cast<int32_t>(q_fixed);
    *shift = e;
}

// operators/cl_quantized_utils/KernelUtil.cpp:7-25.  Returns 0 on success, 1 on failure; on failure the
// multiplier is left untouched (callers pass 0.0 and ignore the status, so the op then yields out_zp).
int32_t orc_conv_multiplier(double in_scale, double w_scale, double bias_scale, double out_scale, double *mult) {
    const double prod = in_scale * w_scale;
    if (!(std::abs(prod - bias_scale) <= 1e-6 * std::min(prod, bias_scale))) return 1;
    if (!(prod >= 0)) return 1;
    *mult = prod / out_scale;
    return 0;
}

// operators/cl_quantized_utils/KernelUtil.cpp:27-71.
void orc_activation_range(int32_t act, int32_t act_dtype, float scale, int32_t zp, int32_t *amin, int32_t *amax) {
    const int32_t qmin = act_dtype == ENN_B200_S8 ? -128 : 0;
    const int32_t qmax = act_dtype == ENN_B200_S8 ? 127 : 255;
    auto quantize = [scale, zp](float f) { return zp + static_cast<int32_t>(std::round(f / scale)); };
    if (act == ENN_B200_ACT_RELU) {
        *amin = std::max(qmin, quantize(0.0f));
        *amax = qmax;
    } else if (act == ENN_B200_ACT_RELU6) {
        *amin = std::max(qmin, quantize(0.0f));
        *amax = std::min(qmax, quantize(6.0f));
    } else if (act == ENN_B200_ACT_RELU1) {
        *amin = std::max(qmin, quantize(-1.0f));
        *amax = std::min(qmax, quantize(1.0f));
    } else {
        *amin = qmin;
        *amax = qmax;
    }
}

// gemmlowp SaturatingRoundingDoublingHighMul as the reference states it:
// QuantizationUtil.cpp:100-108 (host) and common/CLKernels.hpp:121-127 (kernel macro): sign-dependent nudge,
// C truncating division by 2^31.
int32_t orc_srdhm(int32_t a, int32_t b) {
    const bool overflow = a == b && a == std::numeric_limits<int32_t>::min();
    const int64_t ab = static_cast<int64_t>(a) * static_cast<int64_t>(b);
    const int32_t nudge = ab >= 0 ? (1 << 30) : (1 - (1 << 30));
    const int32_t hi = static_cast<int32_t>((ab + nudge) / (1ll << 31));
    return overflow ? std::numeric_limits<int32_t>::max() : hi;
}

// QuantizationUtil.cpp:110-117, CLKernels.hpp:145-151: rounds half away from zero.
int32_t orc_rdivpot(int32_t x, int32_t exponent) {
    const int32_t mask = static_cast<int32_t>((1ll << exponent) - 1);
    const int32_t remainder = x & mask;
    const int32_t threshold = (mask >> 1) + ((x < 0) ? 1 : 0);
    return (x >> exponent) + ((remainder > threshold) ? 1 : 0);
}

// The kernels' requantisation tail (CLKernels.hpp:153-168 reQuantized, preceded in every kernel by
// `acc = acc * (1 << left_shift)`, e.g. cl_kernels/ConvolutionKernels.cpp:1357-1371).  The multiply wraps
// in int32 exactly as the OpenCL int does.
static inline int32_t requant(int32_t acc, int32_t mult, int32_t shift, int32_t out_zp, int32_t amin, int32_t amax) {
    const int32_t ls = shift > 0 ? shift : 0;
    const int32_t rs = shift > 0 ? 0 : -shift;
    acc = static_cast<int32_t>(static_cast<uint32_t>(acc) * (1u << ls));
    int32_t x = orc_rdivpot(orc_srdhm(acc, mult), rs);
    x += out_zp;
    x = std::max(x, amin);
    x = std::min(x, amax);
    return x;
}

int32_t orc_requant(int32_t acc, int32_t mult, int32_t shift, int32_t out_zp, int32_t amin, int32_t amax) {
    return requant(acc, mult, shift, out_zp, amin, amax);
}

// Per-output-channel (multiplier, shift) as the operators derive them on every execute():
//   per-tensor : CLGEMMConvolutionQuantized.cpp:162-166 (scales are floats widened to double;
//                multiplier stays 0.0 when the bias-scale check fails)
//   per-channel: CLConvolutionPerChannelQuantized.cpp:87-99, CLDepthwiseConvolutionPerChannelQuantized.cpp:140-150,
//                CLDeconvolutionPerChannelQuantized.cpp:147-160 (bias scale is the *float* product in*scale[c])
void orc_derive_requant(int32_t cout, int32_t per_channel, float in_scale, float w_scale, float bias_scale,
                        float out_scale, const float *pc_scales, int32_t *mult, int32_t *shift) {
    for (int32_t c = 0; c < cout; ++c) {
        double real = 0.0;
        if (per_channel) {
            const float ws = pc_scales[c];
            const float bs = in_scale * ws;
            orc_conv_multiplier(in_scale, ws, bs, out_scale, &real);
        } else {
            orc_conv_multiplier(in_scale, w_scale, bias_scale, out_scale, &real);
        }
        orc_quantize_multiplier(real, &mult[c], &shift[c]);
    }
}

static inline int32_t load_act(const void *p, int64_t i, int32_t dtype) {
    return dtype == ENN_B200_S8 ? static_cast<int32_t>(static_cast<const int8_t *>(p)[i])
                                : static_cast<int32_t>(static_cast<const uint8_t *>(p)[i]);
}
static inline void store_act(void *p, int64_t i, int32_t dtype, int32_t v) {
    if (dtype == ENN_B200_S8)
        static_cast<int8_t *>(p)[i] = static_cast<int8_t>(v);
    else
        static_cast<uint8_t *>(p)[i] = static_cast<uint8_t>(v);
}

// Output size: CLConvolution.cpp:99-104  (in + pads - ((k-1)d+1) + s) / s.
static inline int32_t conv_out_dim(int32_t in, int32_t p0, int32_t p1, int32_t k, int32_t d, int32_t s) {
    return (in + p0 + p1 - ((k - 1) * d + 1) + s) / s;
}

void orc_conv_out_dims(const enn_b200_conv_desc *d, int32_t *oh, int32_t *ow) {
    *oh = d->out_h > 0 ? d->out_h : conv_out_dim(d->h, d->pad_t, d->pad_b, d->kh, d->dil_h, d->stride_h);
    *ow = d->out_w > 0 ? d->out_w : conv_out_dim(d->w, d->pad_l, d->pad_r, d->kw, d->dil_w, d->stride_w);
}

// Deconvolution output size (ANDROID_NN form): CLDeconvolution.cpp:82-87  in*s + k - s - pad_t - pad_b.
void orc_deconv_out_dims(const enn_b200_conv_desc *d, int32_t *oh, int32_t *ow) {
    *oh = d->out_h > 0 ? d->out_h : d->h * d->stride_h + d->kh - d->stride_h - d->pad_t - d->pad_b;
    *ow = d->out_w > 0 ? d->out_w : d->w * d->stride_w + d->kw - d->stride_w - d->pad_l - d->pad_r;
}

// ---------------------------------------------------------------------------------------------
// Conv2D.  Arithmetic: cl_kernels/ConvolutionKernels.cpp:1317-1375 (conv_per_channel_quantized: the naive
// direct form; with one (multiplier, shift) pair for all channels it is the value quantizedGemmBlocked
// :956-1274 and direct3x3_8x4 produce).  Out-of-image taps are skipped, which equals the reference's
// pre-padding with the input zero point ((za + input_offset) == 0).  Dilation follows the GEMM1xX path
// (in_h = out_h*stride + k_h*dilation - pad_top).
// Weight index: OIHW  g*(Cin/g)*(Cout/g)*Kh*Kw + oc*(Cin/g)*Kh*Kw + ic*Kh*Kw + kh*Kw + kw  (:1336-1343)
//               OHWI  ((o*Kh + kh)*Kw + kw)*(Cin/g) + ic  (ANDROID_NN, converted by convertToNCHW first).
// ---------------------------------------------------------------------------------------------
int32_t orc_conv2d(const enn_b200_conv_desc *d, const void *in, const void *w, const int32_t *bias,
                   const float *pc_scales, void *out) {
    int32_t oh, ow;
    orc_conv_out_dims(d, &oh, &ow);
    const int32_t g = d->groups > 0 ? d->groups : 1;
    const int32_t cin_g = d->cin / g, cout_g = d->cout / g;
    std::vector<int32_t> mult(d->cout), shift(d->cout);
    orc_derive_requant(d->cout, d->per_channel, d->in_scale, d->w_scale, d->bias_scale, d->out_scale, pc_scales,
                       mult.data(), shift.data());
    int32_t amin, amax;
    orc_activation_range(d->activation, d->act_dtype, d->out_scale, d->out_zp, &amin, &amax);
    const int32_t in_off = -d->in_zp;
    const int32_t w_off = d->per_channel ? 0 : -d->w_zp;  // CLConvolutionPerChannelQuantized.cpp:150 passes 0
#pragma omp parallel for collapse(2) schedule(static)
    for (int32_t b = 0; b < d->n; ++b) {
        for (int32_t oy = 0; oy < oh; ++oy) {
            for (int32_t ox = 0; ox < ow; ++ox) {
                for (int32_t oc = 0; oc < d->cout; ++oc) {
                    const int32_t grp = oc / cout_g, ocg = oc % cout_g;
                    int32_t acc = 0;
                    for (int32_t ky = 0; ky < d->kh; ++ky) {
                        const int32_t iy = oy * d->stride_h + ky * d->dil_h - d->pad_t;
                        if (iy < 0 || iy >= d->h) continue;
                        for (int32_t kx = 0; kx < d->kw; ++kx) {
                            const int32_t ix = ox * d->stride_w + kx * d->dil_w - d->pad_l;
                            if (ix < 0 || ix >= d->w) continue;
                            const int64_t ibase = ((static_cast<int64_t>(b) * d->h + iy) * d->w + ix) * d->cin + grp * cin_g;
                            for (int32_t ic = 0; ic < cin_g; ++ic) {
                                int64_t widx;
                                if (d->weight_layout == ENN_B200_W_OHWI)
                                    widx = ((static_cast<int64_t>(oc) * d->kh + ky) * d->kw + kx) * cin_g + ic;
                                else
                                    widx = static_cast<int64_t>(grp) * cin_g * cout_g * d->kh * d->kw +
                                           static_cast<int64_t>(ocg) * cin_g * d->kh * d->kw +
                                           static_cast<int64_t>(ic) * d->kh * d->kw + ky * d->kw + kx;
                                const int32_t a = load_act(in, ibase + ic, d->act_dtype);
                                const int32_t wv = load_act(w, widx, d->weight_dtype);
                                acc += (a + in_off) * (wv + w_off);
                            }
                        }
                    }
                    acc += bias[oc];
                    const int32_t v = requant(acc, mult[oc], shift[oc], d->out_zp, amin, amax);
                    store_act(out, ((static_cast<int64_t>(b) * oh + oy) * ow + ox) * d->cout + oc, d->act_dtype, v);
                }
            }
        }
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------
// DepthwiseConv2D.  cl_kernels/DepthwiseconvolutionKernels.cpp:1273-1371 (Q_DEPTHWISE_CONV and
// Q_DEPTHWISE_CONV_PER_CHANNEL) after the `pad` pre-pass that fills the border with the input zero point
// (CLDepthwiseConvolutionPerChannelQuantized.cpp:207-239), i.e. border taps contribute 0.
// out channel oc = c*depth_multiplier + dep reads input channel c; acc starts from bias[oc];
// weight index OIHW: oc*Kh*Kw + i*Kw + j (:1302,1352); OHWI ([1][Kh][Kw][Cout]): (i*Kw + j)*Cout + oc.
// The signed variant adds 128 to data and zero points on both sides (host :130-138, kernel :2402-2403),
// which cancels, so it is the same formula on int8 data.
// ---------------------------------------------------------------------------------------------
int32_t orc_depthwise(const enn_b200_conv_desc *d, const void *in, const void *w, const int32_t *bias,
                      const float *pc_scales, void *out) {
    int32_t oh, ow;
    orc_conv_out_dims(d, &oh, &ow);
    const int32_t dm = d->groups > 0 ? d->groups : 1;
    const int32_t real = d->cin * dm;      // channels that have a filter
    std::vector<int32_t> mult(d->cout), shift(d->cout);
    orc_derive_requant(d->cout, d->per_channel, d->in_scale, d->w_scale, d->bias_scale, d->out_scale, pc_scales,
                       mult.data(), shift.data());
    int32_t amin, amax;
    orc_activation_range(d->activation, d->act_dtype, d->out_scale, d->out_zp, &amin, &amax);
    const int32_t in_off = -d->in_zp;
    const int32_t w_off = -d->w_zp;  // per-channel filters carry zero point 0
#pragma omp parallel for collapse(2) schedule(static)
    for (int32_t b = 0; b < d->n; ++b) {
        for (int32_t oy = 0; oy < oh; ++oy) {
            for (int32_t ox = 0; ox < ow; ++ox) {
                for (int32_t oc = 0; oc < d->cout; ++oc) {
                    const int32_t c = oc / dm;
                    int32_t acc = bias[oc];
                    // Output channels past cin * depth_multiplier have no filter: bias only
                    // (depthwise_conv_unequal, DepthwiseconvolutionKernels.cpp:1242-1271; the filter tensor holds
                    // cin * depth_multiplier channels).
                    for (int32_t i = 0; i < d->kh && oc < real; ++i) {
                        const int32_t iy = oy * d->stride_h + i * d->dil_h - d->pad_t;
                        if (iy < 0 || iy >= d->h) continue;
                        for (int32_t j = 0; j < d->kw; ++j) {
                            const int32_t ix = ox * d->stride_w + j * d->dil_w - d->pad_l;
                            if (ix < 0 || ix >= d->w) continue;
                            const int64_t widx = d->weight_layout == ENN_B200_W_OHWI
                                                     ? (static_cast<int64_t>(i) * d->kw + j) * real + oc
                                                     : static_cast<int64_t>(oc) * d->kh * d->kw + i * d->kw + j;
                            const int32_t a =
                                load_act(in, ((static_cast<int64_t>(b) * d->h + iy) * d->w + ix) * d->cin + c, d->act_dtype);
                            const int32_t wv = load_act(w, widx, d->weight_dtype);
                            acc += (a + in_off) * (wv + w_off);
                        }
                    }
                    const int32_t v = requant(acc, mult[oc], shift[oc], d->out_zp, amin, amax);
                    store_act(out, ((static_cast<int64_t>(b) * oh + oy) * ow + ox) * d->cout + oc, d->act_dtype, v);
                }
            }
        }
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Deconvolution.  cl_kernels/DeconvolutionKernels.cpp:24-145 (convBackGemmRXR: col[co,kh,kw][ih,iw] =
// sum_ci (a+in_off)(w+w_off)) followed by :147-260 (convertBottomDiff2[_per_channel]: col2im gather over
// h_col/w_col with h_im = oh + pad_t, kernel row = h_im - h_col*stride; then + bias, requant).  Only pad_t
// and pad_l enter (CLDeconvolutionQuantized.cpp:254-256).
// Weight index: IOHW  ci*(Cout*Kh*Kw) + co*Kh*Kw + kh*Kw + kw (matrixTrans source, :13-22)
//               OHWI  ((co*Kh + kh)*Kw + kw)*Cin + ci           (weightAlign source, :8-11)
// group_size is 1 on the quantized path (CLDeconvolutionQuantized.cpp:77 "group_==1").
// ---------------------------------------------------------------------------------------------
int32_t orc_deconv(const enn_b200_conv_desc *d, const void *in, const void *w, const int32_t *bias,
                   const float *pc_scales, void *out) {
    int32_t oh, ow;
    orc_deconv_out_dims(d, &oh, &ow);
    std::vector<int32_t> mult(d->cout), shift(d->cout);
    orc_derive_requant(d->cout, d->per_channel, d->in_scale, d->w_scale, d->bias_scale, d->out_scale, pc_scales,
                       mult.data(), shift.data());
    int32_t amin, amax;
    orc_activation_range(d->activation, d->act_dtype, d->out_scale, d->out_zp, &amin, &amax);
    const int32_t in_off = -d->in_zp;
    const int32_t w_off = d->per_channel ? 0 : -d->w_zp;
    const int32_t kh = d->kh, kw = d->kw, sh = d->stride_h, sw = d->stride_w;
#pragma omp parallel for collapse(2) schedule(static)
    for (int32_t b = 0; b < d->n; ++b) {
        for (int32_t oy = 0; oy < oh; ++oy) {
            for (int32_t ox = 0; ox < ow; ++ox) {
                const int32_t h_im = oy + d->pad_t, w_im = ox + d->pad_l;
                const int32_t w_col_start = (w_im < kw) ? 0 : (w_im - kw) / sw + 1;
                const int32_t w_col_end = std::min(w_im / sw + 1, d->w);
                const int32_t h_col_start = (h_im < kh) ? 0 : (h_im - kh) / sh + 1;
                const int32_t h_col_end = std::min(h_im / sh + 1, d->h);
                for (int32_t co = 0; co < d->cout; ++co) {
                    int32_t val = 0;
                    for (int32_t hc = h_col_start; hc < h_col_end; ++hc) {
                        for (int32_t wc = w_col_start; wc < w_col_end; ++wc) {
                            const int32_t ky = h_im - hc * sh, kx = w_im - wc * sw;
                            const int64_t ibase = ((static_cast<int64_t>(b) * d->h + hc) * d->w + wc) * d->cin;
                            for (int32_t ci = 0; ci < d->cin; ++ci) {
                                const int64_t widx =
                                    d->weight_layout == ENN_B200_W_OHWI
                                        ? ((static_cast<int64_t>(co) * kh + ky) * kw + kx) * d->cin + ci
                                        : static_cast<int64_t>(ci) * d->cout * kh * kw +
                                              static_cast<int64_t>(co) * kh * kw + ky * kw + kx;
                                const int32_t a = load_act(in, ibase + ci, d->act_dtype);
                                const int32_t wv = load_act(w, widx, d->weight_dtype);
                                val += (a + in_off) * (wv + w_off);
                            }
                        }
                    }
                    val += bias[co];
                    const int32_t v = requant(val, mult[co], shift[co], d->out_zp, amin, amax);
                    store_act(out, ((static_cast<int64_t>(b) * oh + oy) * ow + ox) * d->cout + co, d->act_dtype, v);
                }
            }
        }
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------
// FullyConnected, integer definition: the 1x1 CONV_2D contraction (ConvolutionKernels.cpp:1317-1375) on
// [M][K] x [N][K]^T.  (The reference's CLBaseFullyConnected emulates FC in FP32; see orc_fc_float.)
// ---------------------------------------------------------------------------------------------
int32_t orc_fc(const enn_b200_fc_desc *d, const void *in, const void *w, const int32_t *bias,
               const float *pc_scales, void *out) {
    std::vector<int32_t> mult(d->n), shift(d->n);
    orc_derive_requant(d->n, d->per_channel, d->in_scale, d->w_scale, d->bias_scale, d->out_scale, pc_scales,
                       mult.data(), shift.data());
    int32_t amin, amax;
    orc_activation_range(d->activation, d->act_dtype, d->out_scale, d->out_zp, &amin, &amax);
    const int32_t in_off = -d->in_zp;
    const int32_t w_off = d->per_channel ? 0 : -d->w_zp;
    const int64_t K = d->k;
    const bool fast = d->act_dtype == ENN_B200_U8 && d->weight_dtype == ENN_B200_S8;
#pragma omp parallel for collapse(2) schedule(static)
    for (int32_t m = 0; m < d->m; ++m) {
        for (int32_t n = 0; n < d->n; ++n) {
            int32_t acc = 0;
            if (fast) {
                const uint8_t *a = static_cast<const uint8_t *>(in) + m * K;
                const int8_t *b = static_cast<const int8_t *>(w) + n * K;
                for (int64_t k = 0; k < K; ++k) acc += (static_cast<int32_t>(a[k]) + in_off) * (static_cast<int32_t>(b[k]) + w_off);
            } else {
                for (int64_t k = 0; k < K; ++k)
                    acc += (load_act(in, m * K + k, d->act_dtype) + in_off) * (load_act(w, n * K + k, d->weight_dtype) + w_off);
            }
            acc += bias[n];
            store_act(out, static_cast<int64_t>(m) * d->n + n, d->act_dtype,
                      requant(acc, mult[n], shift[n], d->out_zp, amin, amax));
        }
    }
    return 0;
}

// Informational restatement of the reference's float emulation of quantized FC
// (cl_optimized_impls/CLBaseFullyConnected.cpp:88-122,260-277: dequantize input/weight/bias to FP32,
// accumulate in FP32, then cl_kernels/QuantizationKernels.cpp:7-35: round(x * (1/scale) + zp), saturate;
// activation clamp applied afterwards in the quantized domain, CLRelu6.cpp:67-81).  The accumulation
// order of the split/merge kernels depends on computeSplitNum; plain left-to-right order is used here, so
// this is only used to count how often the float path and the integer definition disagree.
int32_t orc_fc_float(const enn_b200_fc_desc *d, const void *in, const void *w, const int32_t *bias, void *out) {
    int32_t amin, amax;
    orc_activation_range(d->activation, d->act_dtype, d->out_scale, d->out_zp, &amin, &amax);
    const int32_t qmin = d->act_dtype == ENN_B200_S8 ? -128 : 0, qmax = d->act_dtype == ENN_B200_S8 ? 127 : 255;
    const float inv = 1.0f / d->out_scale;
#pragma omp parallel for collapse(2) schedule(static)
    for (int32_t m = 0; m < d->m; ++m) {
        for (int32_t n = 0; n < d->n; ++n) {
            float acc = 0.f;
            for (int64_t k = 0; k < d->k; ++k) {
                const float x = d->in_scale * static_cast<float>(load_act(in, static_cast<int64_t>(m) * d->k + k, d->act_dtype) - d->in_zp);
                const float y = d->w_scale * static_cast<float>(load_act(w, static_cast<int64_t>(n) * d->k + k, d->weight_dtype) - d->w_zp);
                acc += x * y;
            }
            acc += d->bias_scale * static_cast<float>(bias[n]);
            int32_t q = static_cast<int32_t>(std::round(acc * inv + static_cast<float>(d->out_zp)));
            q = std::min(std::max(q, qmin), qmax);
            q = std::min(std::max(q, amin), amax);
            store_act(out, static_cast<int64_t>(m) * d->n + n, d->act_dtype, q);
        }
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Quantized add, u8 integer kernel: host parameters CLAddQuantized.cpp:72-88 (left_shift 20, the three
// TFLite multipliers; `2 * std::max(float, float)` is evaluated in float and then widened), kernel
// cl_kernels/AddKernelsQauntized.cpp:135-219.  A stage whose negated shift is outside [0, 31] leaves its
// value undefined in the kernel; such parameter sets are rejected here (return 3).
// ---------------------------------------------------------------------------------------------
int32_t orc_add_params(const enn_b200_add_desc *d, int32_t *p /* [in0_mult,in0_shift,in1_mult,in1_shift,out_mult,out_shift,amin,amax] */) {
    const int left_shift = 20;
    const float twice_f = 2 * std::max(d->in0_scale, d->in1_scale);
    const double twice_max = twice_f;
    const double m0 = d->in0_scale / twice_max;
    const double m1 = d->in1_scale / twice_max;
    const double mo = twice_max / ((1 << left_shift) * d->out_scale);
    orc_quantize_multiplier(m0, &p[0], &p[1]);
    orc_quantize_multiplier(m1, &p[2], &p[3]);
    orc_quantize_multiplier(mo, &p[4], &p[5]);
    if (d->activation != ENN_B200_ACT_NONE) {
        orc_activation_range(d->activation, d->act_dtype, d->out_scale, d->out_zp, &p[6], &p[7]);
    } else {
        p[6] = d->act_dtype == ENN_B200_S8 ? -128 : 0;
        p[7] = d->act_dtype == ENN_B200_S8 ? 127 : 255;
    }
    for (int i = 1; i <= 5; i += 2)
        if (-p[i] < 0 || -p[i] > 31) return 3;
    return 0;
}

int32_t orc_add(const enn_b200_add_desc *d, const void *a, const void *b, void *out) {
    int32_t p[8];
    const int32_t st = orc_add_params(d, p);
    if (st) return st;
    const int left_shift = 20;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < d->count; ++i) {
        const int32_t v0 = -d->in0_zp + load_act(a, i, d->act_dtype);
        const int32_t v1 = -d->in1_zp + load_act(b, i, d->act_dtype);
        const int32_t s0 = v0 * (1 << left_shift);
        const int32_t s1 = v1 * (1 << left_shift);
        const int32_t x0 = orc_rdivpot(orc_srdhm(s0, p[0]), -p[1]);
        const int32_t x1 = orc_rdivpot(orc_srdhm(s1, p[2]), -p[3]);
        const int32_t raw = x0 + x1;
        int32_t o = orc_rdivpot(orc_srdhm(raw, p[4]), -p[5]) + d->out_zp;
        o = std::max(p[6], o);
        o = std::min(p[7], o);
        store_act(out, i, d->act_dtype, o);
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Average pool: cl_kernels/AveragepoolKernels.cpp:8-54 (avepooling_tflite): window clipped to the image,
// (sum + n/2)/n over the valid count, clamp to the activation range, no rescale.
// ---------------------------------------------------------------------------------------------
int32_t orc_avgpool(const enn_b200_pool_desc *d, const void *in, void *out) {
    int32_t amin, amax;
    orc_activation_range(d->activation, d->act_dtype, d->out_scale, d->out_zp, &amin, &amax);
#pragma omp parallel for collapse(2) schedule(static)
    for (int32_t b = 0; b < d->n; ++b) {
        for (int32_t oy = 0; oy < d->out_h; ++oy) {
            for (int32_t ox = 0; ox < d->out_w; ++ox) {
                int32_t si = oy * d->stride_h - d->pad_t, sj = ox * d->stride_w - d->pad_l;
                int32_t ei = std::min(si + d->kh, d->h), ej = std::min(sj + d->kw, d->w);
                si = std::max(si, 0);
                sj = std::max(sj, 0);
                const int32_t pool = (ei - si) * (ej - sj);
                for (int32_t c = 0; c < d->c; ++c) {
                    int32_t s = 0;
                    for (int32_t i = si; i < ei; ++i)
                        for (int32_t j = sj; j < ej; ++j)
                            s += load_act(in, ((static_cast<int64_t>(b) * d->h + i) * d->w + j) * d->c + c, d->act_dtype);
                    int32_t q = (s + pool / 2) / pool;
                    q = std::max(q, amin);
                    q = std::min(q, amax);
                    store_act(out, ((static_cast<int64_t>(b) * d->out_h + oy) * d->out_w + ox) * d->c + c, d->act_dtype, q);
                }
            }
        }
    }
    return 0;
}

// ---- MaxPool: MaxpoolKernels.cpp:33-58 (window clipped to the image, start at the type's minimum, clamp) ----
int32_t orc_maxpool(const enn_b200_pool_desc *d, const void *in, void *out) {
    int32_t amin, amax;
    orc_activation_range(d->activation, d->act_dtype, d->out_scale, d->out_zp, &amin, &amax);
#pragma omp parallel for collapse(2)
    for (int32_t b = 0; b < d->n; ++b)
        for (int32_t oy = 0; oy < d->out_h; ++oy)
            for (int32_t ox = 0; ox < d->out_w; ++ox)
                for (int32_t c = 0; c < d->c; ++c) {
                    int32_t start_i = oy * d->stride_h - d->pad_t, start_j = ox * d->stride_w - d->pad_l;
                    const int32_t end_i = std::min(start_i + d->kh, d->h), end_j = std::min(start_j + d->kw, d->w);
                    start_i = std::max(start_i, 0);
                    start_j = std::max(start_j, 0);
                    int32_t m = d->act_dtype == ENN_B200_S8 ? -128 : 0;
                    for (int32_t i = start_i; i < end_i; ++i)
                        for (int32_t j = start_j; j < end_j; ++j)
                            m = std::max(m, load_act(in, ((static_cast<int64_t>(b) * d->h + i) * d->w + j) * d->c + c, d->act_dtype));
                    m = std::max(m, amin);
                    m = std::min(m, amax);
                    store_act(out, ((static_cast<int64_t>(b) * d->out_h + oy) * d->out_w + ox) * d->c + c, d->act_dtype, m);
                }
    return 0;
}

// ---- Mean: MeanKernels.cpp (sum_axis + mean, or mean_feature_opt): integer sum over the reduced axes divided by their
//      element count with C truncation; no rescaling.  dims are in memory order. ----
int32_t orc_mean(const enn_b200_mean_desc *d, const void *in, void *out) {
    const int32_t *D = d->dims;
    int64_t count = 1;
    int32_t keep[4];
    for (int a = 0; a < 4; ++a) {
        keep[a] = (d->axis_mask & (1 << a)) ? 0 : 1;
        if (!keep[a]) count *= D[a];
    }
    const int32_t O[4] = {keep[0] ? D[0] : 1, keep[1] ? D[1] : 1, keep[2] ? D[2] : 1, keep[3] ? D[3] : 1};
    for (int32_t o0 = 0; o0 < O[0]; ++o0)
        for (int32_t o1 = 0; o1 < O[1]; ++o1)
            for (int32_t o2 = 0; o2 < O[2]; ++o2)
                for (int32_t o3 = 0; o3 < O[3]; ++o3) {
                    int32_t sum = 0;
                    for (int32_t i0 = 0; i0 < (keep[0] ? 1 : D[0]); ++i0)
                        for (int32_t i1 = 0; i1 < (keep[1] ? 1 : D[1]); ++i1)
                            for (int32_t i2 = 0; i2 < (keep[2] ? 1 : D[2]); ++i2)
                                for (int32_t i3 = 0; i3 < (keep[3] ? 1 : D[3]); ++i3)
                                    sum += load_act(in, ((static_cast<int64_t>(o0 + i0) * D[1] + o1 + i1) * D[2] + o2 + i2) * D[3] + o3 + i3, d->act_dtype);
                    store_act(out, ((static_cast<int64_t>(o0) * O[1] + o1) * O[2] + o2) * O[3] + o3, d->act_dtype, sum / static_cast<int32_t>(count));
                }
    return 0;
}

// ---- Concat: ConcatKernels.cpp:399-470 (Q_CONCAT_AXIS*): copy when the scales are equal, else float requantisation
//      value = (int)round(x * scale + bias) + zp_out with scale = s_in * (1 / s_out), bias = -zp_in * scale. ----
int32_t orc_concat(const enn_b200_concat_desc *d, const void *const *ins, void *out) {
    int64_t out_inner = 0;
    for (int i = 0; i < d->n_inputs; ++i) out_inner += d->inner[i];
    const int32_t qmin = d->act_dtype == ENN_B200_S8 ? -128 : 0, qmax = d->act_dtype == ENN_B200_S8 ? 127 : 255;
    int64_t off = 0;
    for (int i = 0; i < d->n_inputs; ++i) {
        const float inverse_output_scale = 1.f / d->out_scale;
        const float scale = d->in_scale[i] * inverse_output_scale;
        const float bias = static_cast<float>(-d->in_zp[i]) * scale;
        for (int64_t r = 0; r < d->outer; ++r)
            for (int64_t c = 0; c < d->inner[i]; ++c) {
                const int32_t x = load_act(ins[i], r * d->inner[i] + c, d->act_dtype);
                int32_t v = x;
                if (d->in_scale[i] != d->out_scale) {
                    const float prod = static_cast<float>(x) * scale;
                    v = static_cast<int32_t>(std::round(prod + bias)) + d->out_zp;
                    v = v > qmin ? v : qmin;
                    v = v < qmax ? v : qmax;
                }
                store_act(out, r * out_inner + off + c, d->act_dtype, v);
            }
        off += d->inner[i];
    }
    return 0;
}

// ---- Softmax: CLSoftmax.cpp:81-150 = dequantise (DequantizationKernels.cpp:7-40: scale * ((float)x - zp)), float
//      softmax_axis2 (SoftmaxKernels.cpp:8-32: maximum, exp((x - max) * beta) summed in channel order, division), quantise
//      (QuantizationKernels.cpp:7-35: round(x * (1 / scale) + zp), saturated).  Multiply and add are separate roundings. ----
int32_t orc_softmax(const enn_b200_softmax_desc *d, const void *in, void *out) {
    const float inverse_scale = 1 / d->out_scale;
    const float lo = d->act_dtype == ENN_B200_S8 ? -128.f : 0.f, hi = d->act_dtype == ENN_B200_S8 ? 127.f : 255.f;
    std::vector<float> e(d->channels);
    for (int64_t o = 0; o < d->outer; ++o)
        for (int64_t i = 0; i < d->inner; ++i) {
            const int64_t base = o * d->channels * d->inner + i;
            auto deq = [&](int32_t c) {
                const float centred = static_cast<float>(load_act(in, base + c * d->inner, d->act_dtype)) - static_cast<float>(d->in_zp);
                return d->in_scale * centred;
            };
            float mx = deq(0);
            for (int32_t c = 1; c < d->channels; ++c)
                if (deq(c) > mx) mx = deq(c);
            float sum = 0.0f;
            for (int32_t c = 0; c < d->channels; ++c) {
                const float diff = deq(c) - mx;
                e[c] = std::exp(diff * d->beta);
                sum += e[c];
            }
            for (int32_t c = 0; c < d->channels; ++c) {
                const float p = e[c] / sum;
                const float scaled = p * inverse_scale;
                float q = std::round(scaled + static_cast<float>(d->out_zp));
                q = std::min(std::max(q, lo), hi);
                store_act(out, base + c * d->inner, d->act_dtype, static_cast<int32_t>(q));
            }
        }
    return 0;
}

// ---- bilinear Resize: ResizeBilinearKernels.cpp:41-83 on NHWC bytes; scales as CLResizeBilinear.cpp computes them.
//      Float interpolation of the raw bytes (no rescaling), products summed left to right, truncated. ----
int32_t orc_resize_bilinear(const enn_b200_resize_desc *d, const void *in, void *out) {
    float hs = static_cast<float>(d->h) / d->out_h, ws = static_cast<float>(d->w) / d->out_w;
    if (d->align_corners && d->out_h > 1) hs = static_cast<float>(d->h - 1) / (d->out_h - 1);
    if (d->align_corners && d->out_w > 1) ws = static_cast<float>(d->w - 1) / (d->out_w - 1);
    for (int32_t b = 0; b < d->n; ++b)
        for (int32_t oy = 0; oy < d->out_h; ++oy)
            for (int32_t ox = 0; ox < d->out_w; ++ox) {
                float input_y, input_x;
                if (d->half_pixel_centers) {
                    const float ty = (static_cast<float>(oy) + 0.5f) * hs, tx = (static_cast<float>(ox) + 0.5f) * ws;
                    input_y = ty - 0.5f;
                    input_x = tx - 0.5f;
                } else {
                    input_y = oy * hs;
                    input_x = ox * ws;
                }
                const uint32_t y0 = static_cast<uint32_t>(std::fmax(std::floor(input_y), 0.f)), x0 = static_cast<uint32_t>(std::fmax(std::floor(input_x), 0.f));
                const int32_t y1 = static_cast<int32_t>(std::fmin(std::ceil(input_y), static_cast<float>(d->h - 1)));
                const int32_t x1 = static_cast<int32_t>(std::fmin(std::ceil(input_x), static_cast<float>(d->w - 1)));
                const float dy = input_y - y0, dx = input_x - x0;
                const float omy = 1 - dy, omx = 1 - dx;
                const float w00 = omy * omx, w01 = dy * omx, w10 = omy * dx, w11 = dy * dx;
                for (int32_t c = 0; c < d->c; ++c) {
                    auto at = [&](int32_t y, int32_t x) {
                        return static_cast<float>(load_act(in, ((static_cast<int64_t>(b) * d->h + y) * d->w + x) * d->c + c, d->act_dtype));
                    };
                    const float p00 = at(y0, x0) * w00, p01 = at(y1, x0) * w01, p10 = at(y0, x1) * w10, p11 = at(y1, x1) * w11;
                    float v = p00 + p01;
                    v = v + p10;
                    v = v + p11;
                    store_act(out, ((static_cast<int64_t>(b) * d->out_h + oy) * d->out_w + ox) * d->c + c, d->act_dtype, static_cast<int32_t>(v));
                }
            }
    return 0;
}

// Worker threads of the following calls (a launcher may have exported OMP_NUM_THREADS=1 for its ranks).
void orc_set_num_threads(int32_t n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int32_t orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
