// Fixed-point requantisation shared by host code and every kernel epilogue.
// Reproduces the reference's two-stage rounding exactly:
//   stage 1  SaturatingRoundingDoublingHighMul  (common/CLKernels.hpp:121-127, QuantizationUtil.cpp:100-108)
//   stage 2  RoundingDivideByPOT, ties away from zero (CLKernels.hpp:145-151, QuantizationUtil.cpp:110-117)
//   then + output zero point and clamp (CLKernels.hpp:153-168 reQuantized).
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define ENN_HD __host__ __device__ __forceinline__
#else
#define ENN_HD inline
#endif

// The reference forms (ab + nudge) / 2^31 with nudge = 2^30 for ab >= 0 and 1 - 2^30 otherwise and C
// truncating division.  For ab < 0 truncation of (ab + 1 - 2^30) equals flooring of (ab + 2^30), so both
// signs reduce to one arithmetic shift: round half toward +infinity.
ENN_HD int32_t enn_srdhm(int32_t a, int32_t b) {
    if (a == b && a == INT32_MIN) return INT32_MAX;
    const int64_t ab = static_cast<int64_t>(a) * static_cast<int64_t>(b);
    return static_cast<int32_t>((ab + (1ll << 30)) >> 31);
}

// exponent in [0, 31].
ENN_HD int32_t enn_rdivpot(int32_t x, int32_t exponent) {
    const int32_t mask = static_cast<int32_t>((1ll << exponent) - 1);
    const int32_t remainder = x & mask;
    const int32_t threshold = (mask >> 1) + (x < 0 ? 1 : 0);
    return (x >> exponent) + (remainder > threshold ? 1 : 0);
}

// shift > 0: left shift applied to the accumulator before stage 1 (wrapping int32 multiply, as the
// kernels' `acc * (1 << left_shift)`); shift <= 0: right shift of stage 2.
ENN_HD int32_t enn_requant(int32_t acc, int32_t mult, int32_t shift, int32_t out_zp, int32_t act_min,
                           int32_t act_max) {
    const int32_t ls = shift > 0 ? shift : 0;
    const int32_t rs = shift > 0 ? 0 : -shift;
    acc = static_cast<int32_t>(static_cast<uint32_t>(acc) << ls);
    int32_t x = enn_rdivpot(enn_srdhm(acc, mult), rs) + out_zp;
    x = x < act_min ? act_min : x;
    x = x > act_max ? act_max : x;
    return x;
}
