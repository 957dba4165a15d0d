// Thin extern "C" wrappers around the REFERENCE's own host quantisation code, compiled from the reference
// source tree where it lies (never copied): operators/cl_quantized_utils/QuantizationUtil.cpp and
// KernelUtil.cpp.  Test infrastructure only: used to validate oracle.cpp and to generate the fixtures in
// tests/golden/.  Built by oracle/Makefile into oracle/_ref/ when the reference tree is present.
#include <cstdint>

#include "userdriver/gpu/operators/cl_quantized_utils/KernelUtil.hpp"
#include "userdriver/gpu/operators/cl_quantized_utils/QuantizationUtil.hpp"

using namespace enn::ud::gpu;

extern "C" {

void ref_quantize_multiplier(double m, int32_t *qm, int32_t *shift) {
    int s = 0;
    QuantizeMultiplierSmallerThanOneExp(m, qm, &s);
    *shift = s;
}

int32_t ref_conv_multiplier(double in_scale, double w_scale, double bias_scale, double out_scale, double *mult) {
    return static_cast<int32_t>(GetQuantizedConvolutionMultipler(in_scale, w_scale, bias_scale, out_scale, mult));
}

void ref_activation_range(int32_t act, int32_t act_dtype, float scale, int32_t zp, int32_t *amin, int32_t *amax) {
    ActivationInfo::ActivationType t = ActivationInfo::ActivationType::NONE;
    if (act == 1) t = ActivationInfo::ActivationType::RELU;
    if (act == 2) t = ActivationInfo::ActivationType::RELU1;
    if (act == 3) t = ActivationInfo::ActivationType::RELU6;
    if (act_dtype == 1)
        CalculateActivationRangeInt8(t, scale, zp, amin, amax);
    else
        CalculateActivationRangeUint8(t, scale, zp, amin, amax);
}

// QuantizationUtil.hpp:102-110 (gemmlowp SRDHM + RoundingDivideByPOT).
int32_t ref_multiply_by_quantized_multiplier(int32_t x, int32_t qm, int32_t shift) {
    return MultiplyByQuantizedMultiplier(x, qm, shift);
}

int32_t ref_srdhm(int32_t a, int32_t b) { return gemmlowp::SaturatingRoundingDoublingHighMul(a, b); }
int32_t ref_rdivpot(int32_t x, int32_t e) { return gemmlowp::RoundingDivideByPOT(x, e); }

}  // extern "C"
