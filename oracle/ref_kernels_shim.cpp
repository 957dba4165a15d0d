// Runs the REFERENCE's own OpenCL C kernel text on the CPU (test infrastructure only).
//
// oracle/ref_dump_kernels.cpp extracts, at build time, the source strings the reference registers for the
// quantized kernels (operators/cl_kernels/*.cpp via common/CLKernels.hpp) into oracle/_ref/ref_kernels_gen.inc.
// That text is plain C apart from a handful of OpenCL built-ins, which the prelude below supplies; the wrappers
// replay the host launch sequence of the reference operators (argument order, global sizes, NCHW layout, the
// zero-point padding pre-pass) and expose NHWC in / NHWC out entry points with the descriptor the oracle uses.
// Requantisation parameters come from the reference's own host code (QuantizationUtil.cpp / KernelUtil.cpp).
#include <algorithm>
#include <climits>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include "../include/enn_b200.h"
#include "userdriver/gpu/operators/cl_quantized_utils/KernelUtil.hpp"
#include "userdriver/gpu/operators/cl_quantized_utils/QuantizationUtil.hpp"

namespace ocl {

// ---- OpenCL C compatibility prelude -------------------------------------------------------------------
typedef unsigned char uchar;
typedef unsigned int uint;
static thread_local size_t g_id[3], g_size[3];
static inline size_t get_global_id(int i) { return g_id[i]; }
static inline size_t get_global_size(int i) { return g_size[i]; }
#define __kernel static
#define __global
#undef max
#undef min
#define max(a, b) ((a) > (b) ? (a) : (b))
#define min(a, b) ((a) < (b) ? (a) : (b))

// OpenCL vector types: named components (.s0 ... .sf, .lo / .hi on 16-vectors) over the same storage as an array.
template <typename T, int N>
struct vecn;
template <typename T>
struct vecn<T, 2> {
    union { T v[2]; struct { T s0, s1; }; };
    vecn() = default;
    explicit vecn(T a) { v[0] = v[1] = a; }
};
template <typename T>
struct vecn<T, 3> {
    union { T v[3]; struct { T s0, s1, s2; }; };
    vecn() = default;
    explicit vecn(T a) { v[0] = v[1] = v[2] = a; }
};
template <typename T>
struct vecn<T, 4> {
    union { T v[4]; struct { T s0, s1, s2, s3; }; };
    vecn() = default;
    vecn(T a) { v[0] = v[1] = v[2] = v[3] = a; }
    vecn(T a, T b, T c, T d) { v[0] = a; v[1] = b; v[2] = c; v[3] = d; }
};
template <typename T>
struct vecn<T, 8> {
    union { T v[8]; struct { T s0, s1, s2, s3, s4, s5, s6, s7; }; };
    vecn() = default;
    template <typename U> vecn(U a) { for (int i = 0; i < 8; ++i) v[i] = static_cast<T>(a); }       // int8 x = 0.0f
    template <int M> vecn<T, M> sub(int first) const { vecn<T, M> r; for (int i = 0; i < M; ++i) r.v[i] = v[first + i]; return r; }
};
template <typename T>
struct vecn<T, 16> {
    union {
        T v[16];
        struct { T s0, s1, s2, s3, s4, s5, s6, s7, s8, s9, sa, sb, sc, sd, se, sf; };
        struct { vecn<T, 8> lo, hi; };
    };
    vecn() = default;
    explicit vecn(T a) { for (int i = 0; i < 16; ++i) v[i] = a; }
    template <typename U> explicit vecn(U a) { for (int i = 0; i < 16; ++i) v[i] = static_cast<T>(a); }   // (uchar16)int_value
    template <int M> vecn<T, M> sub(int first) const { vecn<T, M> r; for (int i = 0; i < M; ++i) r.v[i] = v[first + i]; return r; }
};
template <typename T> using vec4 = vecn<T, 4>;
typedef vecn<int, 2> int2;
typedef vecn<int, 3> int3;
typedef vecn<int, 4> int4;
typedef vecn<int, 8> int8;
typedef vecn<int, 16> int16;
typedef vecn<uchar, 3> uchar3;
typedef vecn<uchar, 4> uchar4;
typedef vecn<uchar, 8> uchar8;
typedef vecn<uchar, 16> uchar16;
typedef vecn<char, 4> char4;
typedef vecn<short, 2> short2;
typedef vecn<short, 3> short3;
typedef vecn<short, 4> short4;
typedef vecn<short, 8> short8;
typedef vecn<short, 16> short16;
template <typename T, int N>
static inline vecn<T, N> operator+(const vecn<T, N> &a, const vecn<T, N> &b) { vecn<T, N> r; for (int i = 0; i < N; ++i) r.v[i] = static_cast<T>(a.v[i] + b.v[i]); return r; }
template <typename T, int N>
static inline vecn<T, N> operator*(const vecn<T, N> &a, const vecn<T, N> &b) { vecn<T, N> r; for (int i = 0; i < N; ++i) r.v[i] = static_cast<T>(a.v[i] * b.v[i]); return r; }
template <typename T, int N, typename S>
static inline vecn<T, N> operator+(const vecn<T, N> &a, S b) { vecn<T, N> r; for (int i = 0; i < N; ++i) r.v[i] = static_cast<T>(a.v[i] + b); return r; }
template <typename T, int N>
static inline vecn<T, N> &operator+=(vecn<T, N> &a, const vecn<T, N> &b) { a = a + b; return a; }
template <int N, typename T>
static inline vecn<T, N> vloadn(size_t off, const T *p) { vecn<T, N> r; for (int i = 0; i < N; ++i) r.v[i] = p[N * off + i]; return r; }
template <typename T> static inline vecn<T, 2> vload2(size_t off, const T *p) { return vloadn<2>(off, p); }
template <typename T> static inline vecn<T, 3> vload3(size_t off, const T *p) { return vloadn<3>(off, p); }
template <typename T> static inline vecn<T, 4> vload4(size_t off, const T *p) { return vloadn<4>(off, p); }
template <typename T> static inline vecn<T, 8> vload8(size_t off, const T *p) { return vloadn<8>(off, p); }
template <typename T> static inline vecn<T, 16> vload16(size_t off, const T *p) { return vloadn<16>(off, p); }
template <typename T, int N>
static inline void vstoren(const vecn<T, N> &v, size_t off, T *p) { for (int i = 0; i < N; ++i) p[N * off + i] = v.v[i]; }
template <typename T> static inline void vstore2(const vecn<T, 2> &v, size_t off, T *p) { vstoren(v, off, p); }
template <typename T> static inline void vstore3(const vecn<T, 3> &v, size_t off, T *p) { vstoren(v, off, p); }
template <typename T> static inline void vstore4(const vecn<T, 4> &v, size_t off, T *p) { vstoren(v, off, p); }
template <typename T> static inline void vstore8(const vecn<T, 8> &v, size_t off, T *p) { vstoren(v, off, p); }
template <typename T> static inline void vstore16(const vecn<T, 16> &v, size_t off, T *p) { vstoren(v, off, p); }
template <typename D, typename T, int N>
static inline vecn<D, N> convert_vec(const vecn<T, N> &v) { vecn<D, N> r; for (int i = 0; i < N; ++i) r.v[i] = static_cast<D>(v.v[i]); return r; }
template <typename T> static inline int4 convert_int4(const vecn<T, 4> &v) { return convert_vec<int>(v); }
template <typename T> static inline int8 convert_int8(const vecn<T, 8> &v) { return convert_vec<int>(v); }
template <typename T> static inline int16 convert_int16(const vecn<T, 16> &v) { return convert_vec<int>(v); }
template <typename T> static inline short2 convert_short2(const vecn<T, 2> &v) { return convert_vec<short>(v); }
template <typename T> static inline short3 convert_short3(const vecn<T, 3> &v) { return convert_vec<short>(v); }
template <typename T> static inline short4 convert_short4(const vecn<T, 4> &v) { return convert_vec<short>(v); }
template <typename T> static inline short8 convert_short8(const vecn<T, 8> &v) { return convert_vec<short>(v); }

#include "_ref/ref_kernels_gen.inc"

#undef max
#undef min

template <typename F>
static void run3(size_t g0, size_t g1, size_t g2, F f) {
    g_size[0] = g0; g_size[1] = g1; g_size[2] = g2;
    for (size_t a = 0; a < g0; ++a)
        for (size_t b = 0; b < g1; ++b)
            for (size_t c = 0; c < g2; ++c) {
                g_id[0] = a; g_id[1] = b; g_id[2] = c;
                f();
            }
}

}  // namespace ocl

namespace {

using enn::ud::gpu::CalculateActivationRangeUint8;
using enn::ud::gpu::GetQuantizedConvolutionMultipler;
using enn::ud::gpu::QuantizeMultiplierSmallerThanOneExp;

ActivationInfo::ActivationType act_type(int a) {
    switch (a) {
        case ENN_B200_ACT_RELU: return ActivationInfo::ActivationType::RELU;
        case ENN_B200_ACT_RELU1: return ActivationInfo::ActivationType::RELU1;
        case ENN_B200_ACT_RELU6: return ActivationInfo::ActivationType::RELU6;
        default: return ActivationInfo::ActivationType::NONE;
    }
}

void act_range(const enn_b200_conv_desc *d, bool honour_disabled, int32_t *lo, int32_t *hi) {
    if (honour_disabled && d->activation == ENN_B200_ACT_NONE) {   // `activation_info_.isEnabled() == false` branches
        *lo = 0;
        *hi = 255;
        return;
    }
    CalculateActivationRangeUint8(act_type(d->activation), d->out_scale, d->out_zp, lo, hi);
}

// Per-channel multipliers as CLConvolutionPerChannelQuantized.cpp:87-99 (and the depthwise / deconv twins).
void per_channel_params(const enn_b200_conv_desc *d, const float *scales, std::vector<int32_t> *m, std::vector<int32_t> *s) {
    m->resize(d->cout);
    s->resize(d->cout);
    for (int i = 0; i < d->cout; ++i) {
        double real = 0.0;
        GetQuantizedConvolutionMultipler(d->in_scale, scales[i], d->in_scale * scales[i], d->out_scale, &real);
        int sh = 0;
        QuantizeMultiplierSmallerThanOneExp(real, &(*m)[i], &sh);
        (*s)[i] = sh;
    }
}

void per_tensor_params(const enn_b200_conv_desc *d, int32_t *m, int *s) {
    double real = 0.0;
    GetQuantizedConvolutionMultipler(d->in_scale, d->w_scale, d->bias_scale, d->out_scale, &real);
    QuantizeMultiplierSmallerThanOneExp(real, m, s);
}

std::vector<uint8_t> nhwc_to_nchw(const uint8_t *x, int n, int h, int w, int c) {
    std::vector<uint8_t> o(static_cast<size_t>(n) * c * h * w);
    for (int b = 0; b < n; ++b)
        for (int y = 0; y < h; ++y)
            for (int xx = 0; xx < w; ++xx)
                for (int k = 0; k < c; ++k) o[((static_cast<size_t>(b) * c + k) * h + y) * w + xx] = x[((static_cast<size_t>(b) * h + y) * w + xx) * c + k];
    return o;
}
void nchw_to_nhwc(const std::vector<uint8_t> &x, uint8_t *o, int n, int h, int w, int c) {
    for (int b = 0; b < n; ++b)
        for (int k = 0; k < c; ++k)
            for (int y = 0; y < h; ++y)
                for (int xx = 0; xx < w; ++xx) o[((static_cast<size_t>(b) * h + y) * w + xx) * c + k] = x[((static_cast<size_t>(b) * c + k) * h + y) * w + xx];
}
int out_dim(int in, int p0, int p1, int k, int dil, int s) { return (in + p0 + p1 - ((k - 1) * dil + 1) + s) / s; }
size_t align_to(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

extern "C" {

// CLConvolutionPerChannelQuantized::execute (file lines 74-160) -> conv_per_channel_quantized.
// Weights: OHWI (ANDROID_NN, converted to OIHW first as the operator does) or OIHW.  u8 activations, int8 weights.
int32_t ref_conv_per_channel(const enn_b200_conv_desc *d, const uint8_t *in, const int8_t *w, const int32_t *bias, const float *scales,
                             uint8_t *out) {
    if (!d->per_channel || d->act_dtype != ENN_B200_U8 || d->dil_h > 1 || d->dil_w > 1) return 3;
    const int g = d->groups > 0 ? d->groups : 1, cig = d->cin / g;
    const int oh = out_dim(d->h, d->pad_t, d->pad_b, d->kh, 1, d->stride_h), ow = out_dim(d->w, d->pad_l, d->pad_r, d->kw, 1, d->stride_w);
    std::vector<uint8_t> x = nhwc_to_nchw(in, d->n, d->h, d->w, d->cin);
    std::vector<int8_t> wo(static_cast<size_t>(d->cout) * cig * d->kh * d->kw);
    for (int o = 0; o < d->cout; ++o)
        for (int i = 0; i < cig; ++i)
            for (int ky = 0; ky < d->kh; ++ky)
                for (int kx = 0; kx < d->kw; ++kx) {
                    const size_t dst = ((static_cast<size_t>(o) * cig + i) * d->kh + ky) * d->kw + kx;
                    wo[dst] = d->weight_layout == ENN_B200_W_OHWI ? w[((static_cast<size_t>(o) * d->kh + ky) * d->kw + kx) * cig + i] : w[dst];
                }
    std::vector<int32_t> m, s;
    per_channel_params(d, scales, &m, &s);
    int32_t lo, hi;
    act_range(d, true, &lo, &hi);
    std::vector<uint8_t> y(static_cast<size_t>(d->n) * d->cout * oh * ow);
    for (int grp = 0; grp < g; ++grp)
        ocl::run3(d->n, d->cout / g, static_cast<size_t>(oh) * ow, [&] {
            ocl::conv_per_channel_quantized_INT8(x.data(), reinterpret_cast<const char *>(wo.data()), bias, m.data(), s.data(), y.data(), g, grp,
                                                 d->kh, d->kw, d->stride_h, d->stride_w, d->pad_l, d->pad_t, d->cout, oh, ow, d->cin, d->h,
                                                 d->w, -d->in_zp, 0, d->out_zp, lo, hi);
        });
    nchw_to_nhwc(y, out, d->n, oh, ow, d->cout);
    return 0;
}

// CLDepthwiseConvolutionPerChannelQuantized::execute (file lines 99-264) and the general branch of
// CLDepthwiseConvolutionQuantized: `pad` pre-pass with the input zero point, then depthwise_conv[_per_channel].
// Weights [Cout][1][Kh][Kw] (OIHW) or [1][Kh][Kw][Cout] (ANDROID_NN, converted first).
int32_t ref_depthwise(const enn_b200_conv_desc *d, const uint8_t *in, const void *w, const int32_t *bias, const float *scales,
                      uint8_t *out) {
    if (d->act_dtype != ENN_B200_U8 || d->dil_h > 1 || d->dil_w > 1) return 3;
    const int dm = d->groups > 0 ? d->groups : 1;
    const int oh = out_dim(d->h, d->pad_t, d->pad_b, d->kh, 1, d->stride_h), ow = out_dim(d->w, d->pad_l, d->pad_r, d->kw, 1, d->stride_w);
    const int ph = d->h + d->pad_t + d->pad_b, pw = d->w + d->pad_l + d->pad_r;
    std::vector<uint8_t> x = nhwc_to_nchw(in, d->n, d->h, d->w, d->cin);
    std::vector<uint8_t> xp(static_cast<size_t>(d->n) * d->cin * ph * pw, static_cast<uint8_t>(d->in_zp));   // pad kernel: zero = input zero point
    for (int b = 0; b < d->n * d->cin; ++b)
        for (int yy = 0; yy < d->h; ++yy)
            std::memcpy(&xp[(static_cast<size_t>(b) * ph + yy + d->pad_t) * pw + d->pad_l], &x[(static_cast<size_t>(b) * d->h + yy) * d->w], d->w);
    // The filter holds cin * depth_multiplier channels; output channels past those are written by depthwise_conv_unequal
    // (per-tensor class only, and its indexing is that of one image: CLDepthwiseConvolutionQuantized.cpp:651-671).
    const int real = d->cin * dm;
    if (real > d->cout || (real < d->cout && (d->per_channel || d->n != 1))) return 3;
    std::vector<uint8_t> wo(static_cast<size_t>(real) * d->kh * d->kw);
    const uint8_t *wsrc = static_cast<const uint8_t *>(w);
    for (int o = 0; o < real; ++o)
        for (int k = 0; k < d->kh * d->kw; ++k)
            wo[static_cast<size_t>(o) * d->kh * d->kw + k] = d->weight_layout == ENN_B200_W_OHWI ? wsrc[static_cast<size_t>(k) * real + o] : wsrc[static_cast<size_t>(o) * d->kh * d->kw + k];
    std::vector<uint8_t> y(static_cast<size_t>(d->n) * d->cout * oh * ow);
    int32_t lo, hi;
    if (d->per_channel) {
        std::vector<int32_t> m, s;
        per_channel_params(d, scales, &m, &s);
        act_range(d, true, &lo, &hi);
        ocl::run3(d->n, d->cin, align_to(static_cast<size_t>(oh) * ow, 32), [&] {
            ocl::depthwise_conv_per_channel_INT8(xp.data(), reinterpret_cast<const char *>(wo.data()), bias, y.data(), ph, pw, d->kh, d->kw,
                                                 d->stride_h, d->stride_w, oh, ow, dm, -d->in_zp, -d->w_zp, d->out_zp, m.data(), s.data(), lo, hi);
        });
    } else {
        int32_t m;
        int s;
        per_tensor_params(d, &m, &s);
        s *= -1;   // CLDepthwiseConvolutionQuantized.cpp:223, undone inside the kernel
        act_range(d, false, &lo, &hi);
        ocl::run3(d->n, d->cin, align_to(static_cast<size_t>(oh) * ow, 32), [&] {
            ocl::depthwise_conv_INT8(xp.data(), wo.data(), bias, y.data(), ph, pw, d->kh, d->kw, d->stride_h, d->stride_w, oh, ow, dm, -d->in_zp,
                                     -d->w_zp, d->out_zp, m, s, lo, hi);
        });
        if (real < d->cout)
            ocl::run3(d->n, d->cout - real, static_cast<size_t>(oh) * ow, [&] { ocl::depthwise_conv_unequal_INT8(bias, y.data(), real, d->out_zp, m, s, lo, hi); });
    }
    nchw_to_nhwc(y, out, d->n, oh, ow, d->cout);
    return 0;
}

// CLDeconvolutionQuantized::execute (file lines 108-288) / CLDeconvolutionPerChannelQuantized::execute:
// zero-point pre-filled aligned buffers, matrixTrans (or weightAlign for ANDROID_NN) of the filter, matrixTrans of
// the input per batch, convBackGemmRXR per batch into the int32 column buffer, convertBottomDiff2.
int32_t ref_deconv(const enn_b200_conv_desc *d, const uint8_t *in, const void *w, const int32_t *bias, const float *scales, uint8_t *out) {
    if (d->act_dtype != ENN_B200_U8) return 3;
    const int oh = d->out_h > 0 ? d->out_h : d->h * d->stride_h + d->kh - d->stride_h - d->pad_t - d->pad_b;
    const int ow = d->out_w > 0 ? d->out_w : d->w * d->stride_w + d->kw - d->stride_w - d->pad_l - d->pad_r;
    const uint32_t cin = d->cin, cout = d->cout, kk = d->kh * d->kw;
    const uint32_t col = align_to(cin, 8), row_filter = kk * cout, row_input = d->h * d->w;
    const uint32_t filter_align_height = align_to(row_filter, 8);
    std::vector<uint8_t> x = nhwc_to_nchw(in, d->n, d->h, d->w, d->cin);
    const uint8_t wfill = d->per_channel ? 0 : static_cast<uint8_t>(d->w_zp);
    std::vector<uint8_t> fbuf(static_cast<size_t>(col) * filter_align_height, wfill);
    std::vector<uint8_t> ibuf(static_cast<size_t>(d->n) * row_input * col, static_cast<uint8_t>(d->in_zp));
    const uint8_t *wsrc = static_cast<const uint8_t *>(w);
    if (d->weight_layout == ENN_B200_W_OHWI) {
        ocl::run3(row_filter, cin, 1, [&] { ocl::weightAlign_INT8(wsrc, fbuf.data(), col, cin); });
    } else {
        ocl::run3(1, row_filter, cin, [&] { ocl::matrixTrans_INT8(wsrc, fbuf.data(), col, 0, 1); });
    }
    for (int b = 0; b < d->n; ++b) ocl::run3(1, row_input, cin, [&] { ocl::matrixTrans_INT8(x.data(), ibuf.data(), col, b, 1); });
    std::vector<int32_t> cbuf(static_cast<size_t>(d->n) * row_input * row_filter, 0);
    const size_t g1 = align_to((row_filter + 7) / 8, 4), g2 = align_to(row_input, 32);
    for (int b = 0; b < d->n; ++b) {
        if (d->per_channel)
            ocl::run3(1, g1, g2, [&] {
                ocl::PERCHANNELconvBackGemmRXR_INT8(reinterpret_cast<const char *>(fbuf.data()), ibuf.data(), cbuf.data(), row_filter, col, row_input, b, 1,
                                                    -d->in_zp, 0);
            });
        else
            ocl::run3(1, g1, g2, [&] {
                ocl::convBackGemmRXR_INT8(fbuf.data(), ibuf.data(), cbuf.data(), row_filter, col, row_input, b, 1, -d->in_zp, -d->w_zp);
            });
    }
    std::vector<uint8_t> y(static_cast<size_t>(d->n) * cout * oh * ow);
    int32_t lo, hi;
    CalculateActivationRangeUint8(act_type(d->activation), d->out_scale, d->out_zp, &lo, &hi);
    if (d->per_channel) {
        std::vector<int32_t> m, s;
        per_channel_params(d, scales, &m, &s);
        ocl::run3(static_cast<size_t>(d->n) * cout, align_to(oh, 4), align_to(ow, 32), [&] {
            ocl::convertBottomDiff2_per_channel_INT8(cbuf.data(), bias, y.data(), oh, ow, cout, d->kh, d->kw, d->pad_t, d->pad_l, d->stride_h,
                                                     d->stride_w, d->h, d->w, d->out_zp, m.data(), s.data(), lo, hi);
        });
    } else {
        int32_t m;
        int s;
        per_tensor_params(d, &m, &s);
        s *= -1;   // CLDeconvolutionQuantized.cpp:130
        ocl::run3(static_cast<size_t>(d->n) * cout, align_to(oh, 4), align_to(ow, 32), [&] {
            ocl::convertBottomDiff2_INT8(cbuf.data(), bias, y.data(), oh, ow, cout, d->kh, d->kw, d->pad_t, d->pad_l, d->stride_h, d->stride_w, d->h,
                                         d->w, d->out_zp, m, s, lo, hi);
        });
    }
    nchw_to_nhwc(y, out, d->n, oh, ow, cout);
    return 0;
}

// CLAveragepool::averagepool_quant (CLAveragepool.cpp:175-224) -> avepooling_tflite.
int32_t ref_avgpool(const enn_b200_pool_desc *d, const uint8_t *in, uint8_t *out) {
    std::vector<uint8_t> x = nhwc_to_nchw(in, d->n, d->h, d->w, d->c);
    std::vector<uint8_t> y(static_cast<size_t>(d->n) * d->c * d->out_h * d->out_w);
    int32_t lo, hi;
    CalculateActivationRangeUint8(act_type(d->activation), d->out_scale, d->out_zp, &lo, &hi);
    ocl::run3(d->n, d->c, align_to(static_cast<size_t>(d->out_h) * d->out_w, 32), [&] {
        ocl::avepooling_tflite_INT8(x.data(), y.data(), d->h, d->w, d->out_h, d->out_w, d->kh, d->kw, d->stride_h, d->stride_w, d->pad_t, d->pad_l,
                                    hi, lo);
    });
    nchw_to_nhwc(y, out, d->n, d->out_h, d->out_w, d->c);
    return 0;
}

// CLAddQuantized::execute (CLAddQuantized.cpp:70-165), u8 branch -> eltwiseAddQuantized_opt.
int32_t ref_add(const enn_b200_add_desc *d, const uint8_t *a, const uint8_t *b, uint8_t *out) {
    const int left_shift = 20;
    const double twice_max_input_scale = 2 * std::max(d->in0_scale, d->in1_scale);
    const double m0 = d->in0_scale / twice_max_input_scale, m1 = d->in1_scale / twice_max_input_scale;
    const double mo = twice_max_input_scale / ((1 << left_shift) * d->out_scale);
    int32_t q0, q1, qo;
    int s0, s1, so;
    QuantizeMultiplierSmallerThanOneExp(m0, &q0, &s0);
    QuantizeMultiplierSmallerThanOneExp(m1, &q1, &s1);
    QuantizeMultiplierSmallerThanOneExp(mo, &qo, &so);
    int32_t lo = 0, hi = 255;
    if (d->activation != ENN_B200_ACT_NONE) CalculateActivationRangeUint8(act_type(d->activation), d->out_scale, d->out_zp, &lo, &hi);
    std::vector<uint8_t> ta(a, a + d->count), tb(b, b + d->count);
    ocl::run3(1, static_cast<size_t>(d->count), 1, [&] {
        ocl::eltwiseAddQuantized_opt_INT8(ta.data(), tb.data(), out, left_shift, -d->in0_zp, -d->in1_zp, d->out_zp, s0, s1, so, q0, q1, qo, lo, hi);
    });
    return 0;
}

// CLGEMMConvolutionQuantized (per-tensor u8 convolution; cl_optimized_impls/CLGEMMConvolutionQuantized.cpp): weights to
// int16 with the zero point removed and interleaved four rows at a time (alignQuantizedWeight_gemm, once at
// initialize), then per execute: CLPadConvert (pad_opt with the input zero point, then convert_optimized for one group
// or convertBlocked2 per group) and quantizedGemmBlocked per group.  Buffer sizes, argument order and global sizes
// follow the host code.  Padding entries beyond the real reduction length are never written by the reference and meet
// padding weights; here both buffers start zeroed, so those products are zero.
int32_t ref_conv_per_tensor(const enn_b200_conv_desc *d, const uint8_t *in, const uint8_t *w, const int32_t *bias, uint8_t *out) {
    if (d->per_channel || d->act_dtype != ENN_B200_U8 || d->weight_dtype != ENN_B200_U8 || d->dil_h > 1 || d->dil_w > 1) return 3;
    const uint32_t g = d->groups > 0 ? d->groups : 1, cig = d->cin / g, cog = d->cout / g;
    const int oh = out_dim(d->h, d->pad_t, d->pad_b, d->kh, 1, d->stride_h), ow = out_dim(d->w, d->pad_l, d->pad_r, d->kw, 1, d->stride_w);
    // weights as OIHW (ANDROID_NN models are converted first, CLGEMMConvolutionQuantized.cpp initialize)
    std::vector<uint8_t> wo(static_cast<size_t>(d->cout) * cig * d->kh * d->kw);
    for (int o = 0; o < d->cout; ++o)
        for (uint32_t i = 0; i < cig; ++i)
            for (int ky = 0; ky < d->kh; ++ky)
                for (int kx = 0; kx < d->kw; ++kx) {
                    const size_t dst = ((static_cast<size_t>(o) * cig + i) * d->kh + ky) * d->kw + kx;
                    wo[dst] = d->weight_layout == ENN_B200_W_OHWI ? w[((static_cast<size_t>(o) * d->kh + ky) * d->kw + kx) * cig + i] : w[dst];
                }
    // alignQuantizedWeightGEMM
    const uint32_t src_unit_count = cig * d->kh * d->kw, dst_align_count = align_to(src_unit_count, 16);
    const uint32_t group_top_channel = cog, aligned_group_top_channel = align_to(cog, 16);
    const uint32_t align_weight_height = dst_align_count, align_weight_width = aligned_group_top_channel * g;
    std::vector<short> wq(static_cast<size_t>(align_weight_height) * align_weight_width + 64, 0);
    wo.resize(wo.size() + 16, 0);     // the 8-wide loads of the last row may read a few bytes past the tensor
    ocl::run3(d->cout, align_to((src_unit_count + 7) / 8, 12), 1, [&] {
        ocl::alignQuantizedWeight_gemm_INT8(wo.data(), wq.data(), src_unit_count, dst_align_count, group_top_channel, aligned_group_top_channel,
                                            -d->w_zp);
    });
    // CLPadConvert::execute
    const int ph = d->h + d->pad_t + d->pad_b, pw = d->w + d->pad_l + d->pad_r;
    std::vector<uint8_t> x = nhwc_to_nchw(in, d->n, d->h, d->w, d->cin);
    const size_t slack = 64;          // pad_opt loads 16 bytes around every row start, also left of the tensor
    std::vector<uint8_t> xs(x.size() + 2 * slack, 0);
    std::memcpy(xs.data() + slack, x.data(), x.size());
    const uint8_t *x0 = xs.data() + slack;
    std::vector<uint8_t> xp;
    const uint8_t *padded = x0;
    if (d->pad_t || d->pad_b || d->pad_l || d->pad_r) {
        xp.assign(static_cast<size_t>(d->n) * d->cin * ph * pw + slack, 0);
        ocl::run3(static_cast<size_t>(d->n) * d->cin, align_to(ph, 4), align_to((pw + 15) / 16, 64), [&] {
            ocl::pad_opt_INT8(x0, xp.data(), d->in_zp, d->pad_t, d->pad_l, d->h, d->w, ph, pw);
        });
        padded = xp.data();
    }
    const uint32_t align_input_height = align_to(static_cast<size_t>(oh) * ow, 12) * g, align_input_width = dst_align_count;
    std::vector<uint8_t> col(static_cast<size_t>(d->n) * align_input_height * align_input_width + slack, 0);
    const uint32_t add_pad_height = d->pad_t || d->pad_b || d->pad_l || d->pad_r ? ph : d->h;
    const uint32_t add_pad_width = d->pad_t || d->pad_b || d->pad_l || d->pad_r ? pw : d->w;
    const uint32_t group_height = align_input_height / g;
    if (g == 1) {
        ocl::run3(d->n, static_cast<size_t>(oh) * ow, align_to(static_cast<size_t>(d->cin) * d->kh, 16), [&] {
            ocl::convert_optimized_INT8(padded, col.data(), d->kw, d->kh, d->stride_w, d->stride_h, add_pad_height, add_pad_width, cig, group_height,
                                        align_input_width, ow, oh);
        });
    } else {
        for (uint32_t i = 0; i < g; ++i)
            ocl::run3(d->n, align_to(static_cast<size_t>(oh) * ow, 16), align_to(static_cast<size_t>(d->cin) * d->kh * d->kw / g, 16), [&] {
                ocl::convertBlocked2_INT8(padded, col.data(), d->kw, d->kh, d->stride_w, d->stride_h, add_pad_height, add_pad_width, cig, group_height,
                                          align_input_width, i, ow, g, oh);
            });
    }
    // execute(): multiplier, then quantizedGEMMRun per group
    int32_t m;
    int s;
    per_tensor_params(d, &m, &s);
    s *= -1;                          // CLGEMMConvolutionQuantized::execute; undone inside the kernel
    int32_t lo, hi;
    act_range(d, true, &lo, &hi);
    std::vector<uint8_t> y(static_cast<size_t>(d->n) * d->cout * oh * ow + slack, 0);
    for (uint32_t i = 0; i < g; ++i)
        ocl::run3(d->n, align_weight_width / g / 4, align_input_height / g, [&] {
            ocl::quantizedGemmBlocked_INT8(col.data(), wq.data(), bias, y.data(), align_input_width, d->cout, oh * ow, g, i, -d->in_zp, d->out_zp, m,
                                           s, lo, hi);
        });
    y.resize(static_cast<size_t>(d->n) * d->cout * oh * ow);
    nchw_to_nhwc(y, out, d->n, oh, ow, d->cout);
    return 0;
}

// CLMaxpool::maxpool_quant (CLMaxpool.cpp:144-186) -> maxpooling.
int32_t ref_maxpool(const enn_b200_pool_desc *d, const uint8_t *in, uint8_t *out) {
    if (d->act_dtype != ENN_B200_U8) return 3;
    std::vector<uint8_t> x = nhwc_to_nchw(in, d->n, d->h, d->w, d->c);
    std::vector<uint8_t> y(static_cast<size_t>(d->n) * d->c * d->out_h * d->out_w);
    int32_t lo, hi;
    CalculateActivationRangeUint8(act_type(d->activation), d->out_scale, d->out_zp, &lo, &hi);
    ocl::run3(d->n, d->c, align_to(static_cast<size_t>(d->out_h) * d->out_w, 16), [&] {
        ocl::maxpooling_INT8(x.data(), y.data(), d->h, d->w, d->kh, d->kw, d->stride_h, d->stride_w, d->pad_t, d->pad_l, d->out_w, d->out_h, hi, lo);
    });
    nchw_to_nhwc(y, out, d->n, d->out_h, d->out_w, d->c);
    return 0;
}

// CLMean::execute (CLMean.cpp:107-240) on a tensor given in the reference's own NCHW dims: the global-average-pool form
// (mean_feature_opt) when the reduced axes are the trailing ones, else quant8_to_int32 (a widening copy), the halving
// sum_axis passes and mean.  `axis_mask` bit i = dims[i]; output keeps the order of the surviving dims.
int32_t ref_mean(const int32_t *dims, int32_t axis_mask, const uint8_t *in, uint8_t *out) {
    const uint32_t D[4] = {static_cast<uint32_t>(dims[0]), static_cast<uint32_t>(dims[1]), static_cast<uint32_t>(dims[2]), static_cast<uint32_t>(dims[3])};
    size_t total = static_cast<size_t>(D[0]) * D[1] * D[2] * D[3], out_size = 1;
    int min_ax = 4, max_ax = -1;
    for (int a = 0; a < 4; ++a) {
        if (axis_mask & (1 << a)) {
            min_ax = std::min(min_ax, a);
            max_ax = std::max(max_ax, a);
        } else {
            out_size *= D[a];
        }
    }
    if (max_ax < 0) return 3;
    const int num_elements_in_axis = static_cast<int>(total / out_size);
    size_t between = 1, after = 1;
    for (int a = min_ax; a <= max_ax; ++a) between *= D[a];
    for (int a = max_ax + 1; a < 4; ++a) after *= D[a];
    if (between == static_cast<size_t>(num_elements_in_axis) && after == 1) {      // isFitFeatureMeanOpt
        std::vector<uint8_t> x(in, in + total);
        x.resize(total + 16, 0);
        ocl::run3(out_size, 1, 1, [&] { ocl::mean_feature_opt_INT8(x.data(), out, num_elements_in_axis, num_elements_in_axis); });
        return 0;
    }
    std::vector<int> acc(in, in + total);          // quant8_to_int32
    acc.resize(total + 1, 0);
    uint32_t dm[4] = {D[0], D[1], D[2], D[3]};
    for (int ax = 3; ax >= 0; --ax) {
        if (!(axis_mask & (1 << ax))) continue;
        uint32_t k = 1;
        for (int i = ax + 1; i < 4; ++i) k *= D[i];
        while (dm[ax] > 1) {
            const uint32_t offset = dm[ax] - (dm[ax] >> 1);
            if (offset * 2 > dm[ax]) dm[ax] = offset - 1;
            else dm[ax] = offset;
            const uint32_t offset_k = offset * k;
            ocl::run3(total, 1, 1, [&] { ocl::sum_axis_INT8(acc.data(), offset_k, D[0], D[1], D[2], D[3], dm[0], dm[1], dm[2], dm[3]); });
            dm[ax] = offset;
        }
    }
    ocl::run3(total, 1, 1, [&] { ocl::mean_INT8(acc.data(), out, num_elements_in_axis, D[0], D[1], D[2], D[3], dm[0], dm[1], dm[2], dm[3]); });
    return 0;
}

// CLConcat::concatAxis1 with is_quant (CLConcat.cpp:381-452): inputs [N][C_i][H*W] concatenated along C.
int32_t ref_concat_axis1(int32_t n_inputs, int32_t n, const int32_t *channels, int32_t hw, const float *in_scale, const int32_t *in_zp,
                         float out_scale, int32_t out_zp, const uint8_t *const *ins, uint8_t *out) {
    uint32_t cout = 0;
    for (int i = 0; i < n_inputs; ++i) cout += channels[i];
    const uint32_t batch_offset = cout * hw;
    uint32_t offset = 0;
    for (int i = 0; i < n_inputs; ++i) {
        std::vector<uint8_t> x(ins[i], ins[i] + static_cast<size_t>(n) * channels[i] * hw);
        ocl::run3(n, channels[i], hw, [&] {
            ocl::concat_axis1_INT8(x.data(), out, batch_offset, hw, offset, in_scale[i], in_zp[i], out_scale, out_zp, 0, 255);
        });
        offset += channels[i] * hw;
    }
    return 0;
}

// CLResizeBilinear::execute, general kernel (CLResizeBilinear.cpp:279-300) -> resize_bilinear.
int32_t ref_resize_bilinear(const enn_b200_resize_desc *d, const uint8_t *in, uint8_t *out) {
    if (d->act_dtype != ENN_B200_U8) return 3;
    std::vector<uint8_t> x = nhwc_to_nchw(in, d->n, d->h, d->w, d->c);
    std::vector<uint8_t> y(static_cast<size_t>(d->n) * d->c * d->out_h * d->out_w);
    float hs = static_cast<float>(d->h) / d->out_h, ws = static_cast<float>(d->w) / d->out_w;
    if (d->align_corners && d->out_h > 1) hs = static_cast<float>(d->h - 1) / (d->out_h - 1);
    if (d->align_corners && d->out_w > 1) ws = static_cast<float>(d->w - 1) / (d->out_w - 1);
    ocl::run3(align_to(y.size(), 16), 1, 1, [&] {
        ocl::resize_bilinear_INT8(x.data(), y.data(), d->h, d->w, d->n, d->c, d->out_h, d->out_w, hs, ws, d->half_pixel_centers ? 1 : 0);
    });
    nchw_to_nhwc(y, out, d->n, d->out_h, d->out_w, d->c);
    return 0;
}

int32_t ref_has_kernels(void) { return 1; }

}  // extern "C"
