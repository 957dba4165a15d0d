// Host-side derivation of requantisation parameters, done once at prepare time.
#pragma once
#include <stdint.h>
#include <vector>

namespace enn_b200 {

// QuantizationUtil.cpp:8-21 / :29-35: frexp split, Q0.31 significand, signed exponent.
void quantize_multiplier(double real_multiplier, int32_t *quantized_multiplier, int32_t *shift);

// KernelUtil.cpp:7-25.  Returns false (and leaves *multiplier alone) when the bias scale does not match
// in_scale * w_scale within 1e-6 relative, or the product is negative.
bool conv_multiplier(double in_scale, double w_scale, double bias_scale, double out_scale, double *multiplier);

// KernelUtil.cpp:27-71.
void activation_range(int32_t activation, int32_t act_dtype, float scale, int32_t zero_point, int32_t *act_min,
                      int32_t *act_max);

// Per-output-channel multiplier/shift vectors; per-tensor ops replicate one pair.
// Returns false when a derived right shift falls outside [0, 31] (undefined in the reference kernels).
bool derive_requant(int32_t cout, bool per_channel, float in_scale, float w_scale, float bias_scale,
                    float out_scale, const float *pc_scales, std::vector<int32_t> *mult,
                    std::vector<int32_t> *shift);

// Float helpers of the graph operators the reference computes in floating point.  Every operation is a separate
// IEEE single-precision multiply / add / subtract / divide (no fused multiply-add), in the order of the kernel text.
// ConcatKernels.cpp:417-433: scale = s_in * (1 / s_out), bias = -zp_in * scale, round(x * scale + bias) + zp_out, clamp.
uint8_t concat_requant_byte(uint8_t byte, bool is_signed, float in_scale, int32_t in_zp, float out_scale, int32_t out_zp);
// exp((dequant(x) - dequant(m)) * beta) for every pair of bytes (row m = byte of the maximum, column x), with
// dequant(b) = scale * ((float)b - zp) (DequantizationKernels.cpp:7-40, SoftmaxKernels.cpp:19-26).  table: 256 x 256.
void softmax_exp_table(bool is_signed, float in_scale, int32_t in_zp, float beta, float *table);
// CLResizeBilinear.cpp: in / out, or (in - 1) / (out - 1) with align_corners and more than one output row / column.
void resize_scales(int32_t in_h, int32_t in_w, int32_t out_h, int32_t out_w, bool align_corners, float *height_scale, float *width_scale);

}  // namespace enn_b200
