#include "quant_host.h"

#include <algorithm>
#include <cmath>

#include "../../include/enn_b200.h"

namespace enn_b200 {

void quantize_multiplier(double real_multiplier, int32_t *quantized_multiplier, int32_t *shift) {
    if (real_multiplier == 0.) {
        *quantized_multiplier = 0;
        *shift = 0;
        return;
    }
    int exponent = 0;
    const double significand = std::frexp(real_multiplier, &exponent);
    int64_t fixed = static_cast<int64_t>(std::round(significand * 2147483648.0));
    if (fixed == 2147483648ll) {  // significand rounded up to 1.0
        fixed >>= 1;
        ++exponent;
    }
    *quantized_multiplier = static_cast<int32_t>(fixed);
    *shift = exponent;
}

bool conv_multiplier(double in_scale, double w_scale, double bias_scale, double out_scale, double *multiplier) {
    const double product = in_scale * w_scale;
    if (!(std::abs(product - bias_scale) <= 1e-6 * std::min(product, bias_scale))) return false;
    if (!(product >= 0)) return false;
    *multiplier = product / out_scale;
    return true;
}

void activation_range(int32_t activation, int32_t act_dtype, float scale, int32_t zero_point, int32_t *act_min,
                      int32_t *act_max) {
    const int32_t qmin = act_dtype == ENN_B200_S8 ? -128 : 0;
    const int32_t qmax = act_dtype == ENN_B200_S8 ? 127 : 255;
    auto q = [&](float real) { return zero_point + static_cast<int32_t>(std::round(real / scale)); };
    switch (activation) {
        case ENN_B200_ACT_RELU:
            *act_min = std::max(qmin, q(0.f));
            *act_max = qmax;
            break;
        case ENN_B200_ACT_RELU6:
            *act_min = std::max(qmin, q(0.f));
            *act_max = std::min(qmax, q(6.f));
            break;
        case ENN_B200_ACT_RELU1:
            *act_min = std::max(qmin, q(-1.f));
            *act_max = std::min(qmax, q(1.f));
            break;
        default:
            *act_min = qmin;
            *act_max = qmax;
    }
}

bool derive_requant(int32_t cout, bool per_channel, float in_scale, float w_scale, float bias_scale,
                    float out_scale, const float *pc_scales, std::vector<int32_t> *mult,
                    std::vector<int32_t> *shift) {
    mult->resize(cout);
    shift->resize(cout);
    bool ok = true;
    for (int32_t c = 0; c < cout; ++c) {
        double real = 0.0;  // stays 0 when the scale check fails: the op then emits out_zp everywhere
        if (per_channel) {
            // The per-channel operators pass the float product in_scale * scales[c] as the bias scale
            // (CLConvolutionPerChannelQuantized.cpp:89-93).
            const float ws = pc_scales[c];
            const float bs = in_scale * ws;
            conv_multiplier(in_scale, ws, bs, out_scale, &real);
        } else {
            conv_multiplier(in_scale, w_scale, bias_scale, out_scale, &real);
        }
        quantize_multiplier(real, &(*mult)[c], &(*shift)[c]);
        if ((*shift)[c] < -31 || (*shift)[c] > 30) ok = false;
    }
    return ok;
}

uint8_t concat_requant_byte(uint8_t byte, bool is_signed, float in_scale, int32_t in_zp, float out_scale, int32_t out_zp) {
    const int32_t x = is_signed ? static_cast<int32_t>(static_cast<int8_t>(byte)) : static_cast<int32_t>(byte);
    const volatile float inverse_output_scale = 1.f / out_scale;
    const volatile float scale = in_scale * inverse_output_scale;
    const volatile float bias = static_cast<float>(-in_zp) * scale;
    const volatile float prod = static_cast<float>(x) * scale;
    const volatile float sum = prod + bias;
    int32_t value = static_cast<int32_t>(std::round(sum)) + out_zp;
    const int32_t qmin = is_signed ? -128 : 0, qmax = is_signed ? 127 : 255;
    value = value > qmin ? value : qmin;
    value = value < qmax ? value : qmax;
    return static_cast<uint8_t>(value);
}

void softmax_exp_table(bool is_signed, float in_scale, int32_t in_zp, float beta, float *table) {
    float deq[256];
    for (int b = 0; b < 256; ++b) {
        const int32_t x = is_signed ? static_cast<int32_t>(static_cast<int8_t>(b)) : b;
        const volatile float centred = static_cast<float>(x) - static_cast<float>(in_zp);
        deq[b] = in_scale * centred;
    }
    for (int m = 0; m < 256; ++m)
        for (int b = 0; b < 256; ++b) {
            const volatile float diff = deq[b] - deq[m];
            const volatile float arg = diff * beta;
            table[m * 256 + b] = std::exp(static_cast<float>(arg));
        }
}

void resize_scales(int32_t in_h, int32_t in_w, int32_t out_h, int32_t out_w, bool align_corners, float *height_scale, float *width_scale) {
    *height_scale = static_cast<float>(in_h) / out_h;
    *width_scale = static_cast<float>(in_w) / out_w;
    if (align_corners && out_h > 1) *height_scale = static_cast<float>(in_h - 1) / (out_h - 1);
    if (align_corners && out_w > 1) *width_scale = static_cast<float>(in_w - 1) / (out_w - 1);
}

}  // namespace enn_b200
