// The remaining quantized graph operators of the reference's u8 models: MaxPool, Mean, Concat, Softmax and bilinear
// Resize (CLMaxpool.cpp, CLMean.cpp, CLConcat.cpp, CLSoftmax.cpp, CLResizeBilinear.cpp and their kernels).  They are
// small, memory-bound passes between the convolutions; each is one launch over NHWC (or any memory-order) bytes with
// coalesced accesses along the innermost dimension.  Integer operators are exact; the two that the reference computes
// in float (Softmax, Resize; also Concat's requantisation) take every float operation either from a host-built table
// or as an explicitly unfused multiply / add, so that the bytes are reproducible across compilers.
#include <cmath>
#include <cstring>
#include <new>

#include "internal.h"
#include "quant_host.h"

namespace enn_b200 {

namespace {

__device__ __forceinline__ int32_t ld_act(const void *p, int64_t i, int is_signed) {
    return is_signed ? static_cast<int32_t>(static_cast<const int8_t *>(p)[i]) : static_cast<int32_t>(static_cast<const uint8_t *>(p)[i]);
}

// ---- MaxPool (MaxpoolKernels.cpp:33-58): window clipped to the image, starts from the type's minimum, clamp ----
__global__ void maxpool_kernel(PoolGeom p, const void *__restrict__ in, uint8_t *__restrict__ out, int64_t total) {
    pdl_wait();
    pdl_trigger();
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int32_t c = static_cast<int32_t>(idx % p.c);
    int64_t q = idx / p.c;
    const int32_t ox = static_cast<int32_t>(q % p.ow);
    q /= p.ow;
    const int32_t oy = static_cast<int32_t>(q % p.oh);
    const int32_t b = static_cast<int32_t>(q / p.oh);
    int32_t si = oy * p.sh - p.pt, sj = ox * p.sw - p.pl;
    const int32_t ei = min(si + p.kh, p.h), ej = min(sj + p.kw, p.w);
    si = max(si, 0);
    sj = max(sj, 0);
    int32_t m = p.is_signed ? -128 : 0;
    for (int32_t i = si; i < ei; ++i)
        for (int32_t j = sj; j < ej; ++j) m = max(m, ld_act(in, ((static_cast<int64_t>(b) * p.h + i) * p.w + j) * p.c + c, p.is_signed));
    m = max(m, p.act_min);
    m = min(m, p.act_max);
    out[idx] = static_cast<uint8_t>(m);
}

// ---- Mean (MeanKernels.cpp): integer sum over the reduced axes, C division by the element count ----
struct MeanGeom {
    int32_t d[4];        // input dims, memory order
    int32_t keep[4];     // 1: the axis survives
    int32_t count;       // reduced elements per output
    int32_t is_signed;
};

__global__ void mean_kernel(MeanGeom g, const void *__restrict__ in, uint8_t *__restrict__ out, int64_t total) {
    pdl_wait();
    pdl_trigger();
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    // output position -> coordinates of the kept axes (innermost fastest, so neighbouring threads read neighbouring bytes)
    int32_t o[4];
    int64_t r = idx;
    for (int a = 3; a >= 0; --a) {
        const int32_t extent = g.keep[a] ? g.d[a] : 1;
        o[a] = static_cast<int32_t>(r % extent);
        r /= extent;
    }
    int32_t sum = 0;
    const int32_t e0 = g.keep[0] ? 1 : g.d[0], e1 = g.keep[1] ? 1 : g.d[1], e2 = g.keep[2] ? 1 : g.d[2], e3 = g.keep[3] ? 1 : g.d[3];
    for (int32_t i0 = 0; i0 < e0; ++i0)
        for (int32_t i1 = 0; i1 < e1; ++i1)
            for (int32_t i2 = 0; i2 < e2; ++i2)
                for (int32_t i3 = 0; i3 < e3; ++i3) {
                    const int64_t ii = ((static_cast<int64_t>(o[0] + i0) * g.d[1] + o[1] + i1) * g.d[2] + o[2] + i2) * g.d[3] + o[3] + i3;
                    sum += ld_act(in, ii, g.is_signed);
                }
    out[idx] = static_cast<uint8_t>(sum / g.count);
}

// ---- Concat (ConcatKernels.cpp:399-470): copy or table look-up (the float requantisation of each input byte, built on
//      the host with the reference's formula) into the input's column range of the output ----
struct ConcatPart {
    const uint8_t *in;
    int64_t inner, offset;
    int32_t use_lut;
};
struct ConcatArgs {
    ConcatPart part[ENN_B200_CONCAT_MAX_INPUTS];
    const uint8_t *lut;      // [n_inputs][256]
    int64_t out_inner;
    int32_t n_inputs;
};

__global__ void concat_kernel(ConcatArgs a, uint8_t *__restrict__ out, int64_t outer) {
    pdl_wait();
    pdl_trigger();
    const int which = blockIdx.y;
    const ConcatPart pt = a.part[which];
    const int64_t total = outer * pt.inner;
    const uint8_t *lut = a.lut + which * 256;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t row = idx / pt.inner, col = idx - row * pt.inner;
        const uint8_t v = pt.in[idx];
        out[row * a.out_inner + pt.offset + col] = pt.use_lut ? __ldg(lut + v) : v;
    }
}

// ---- Softmax (SoftmaxKernels.cpp:8-32 after DequantizationKernels.cpp / before QuantizationKernels.cpp) ----
// One thread per (outer, inner) position walks the channels in order, as the reference's work-item does, so that the
// float sum has the same order.  exp((x - max) * beta) on dequantised bytes takes 256 x 256 values; they come from a
// host-built table indexed by (max byte, byte).
struct SoftmaxGeom {
    int64_t outer, inner;
    int32_t channels, is_signed;
    float inv_out_scale;
    int32_t out_zp;
    const float *exp_lut;    // [256][256]: row = byte of the row maximum, column = byte
};

__global__ void softmax_kernel(SoftmaxGeom g, const uint8_t *__restrict__ in, uint8_t *__restrict__ out, int64_t total) {
    pdl_wait();
    pdl_trigger();
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int64_t o = idx / g.inner, i = idx - o * g.inner;
    const uint8_t *src = in + o * g.channels * g.inner + i;
    uint8_t *dst = out + o * g.channels * g.inner + i;
    // the dequantisation is monotonic in the byte (as an unsigned or signed integer), so the maximum can be taken on bytes
    int32_t mx = g.is_signed ? -128 : 0;
    for (int32_t c = 0; c < g.channels; ++c) mx = max(mx, g.is_signed ? static_cast<int32_t>(static_cast<int8_t>(src[c * g.inner])) : static_cast<int32_t>(src[c * g.inner]));
    const float *row = g.exp_lut + (static_cast<uint32_t>(mx) & 0xff) * 256;
    float sum = 0.0f;
    for (int32_t c = 0; c < g.channels; ++c) sum = __fadd_rn(sum, __ldg(row + src[c * g.inner]));
    for (int32_t c = 0; c < g.channels; ++c) {
        const float p = __fdiv_rn(__ldg(row + src[c * g.inner]), sum);
        float q = roundf(__fadd_rn(__fmul_rn(p, g.inv_out_scale), static_cast<float>(g.out_zp)));
        const float lo = g.is_signed ? -128.0f : 0.0f, hi = g.is_signed ? 127.0f : 255.0f;
        q = fminf(fmaxf(q, lo), hi);
        dst[c * g.inner] = static_cast<uint8_t>(static_cast<int32_t>(q));
    }
}

// ---- bilinear Resize (ResizeBilinearKernels.cpp:41-83): float interpolation of the raw bytes, truncated ----
struct ResizeGeom {
    int32_t n, h, w, c, oh, ow;
    float hs, ws;
    int32_t half_pixel, is_signed;
};

__global__ void resize_bilinear_kernel(ResizeGeom g, const void *__restrict__ in, uint8_t *__restrict__ out, int64_t total) {
    pdl_wait();
    pdl_trigger();
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int32_t c = static_cast<int32_t>(idx % g.c);
    int64_t q = idx / g.c;
    const int32_t ox = static_cast<int32_t>(q % g.ow);
    q /= g.ow;
    const int32_t oy = static_cast<int32_t>(q % g.oh);
    const int32_t b = static_cast<int32_t>(q / g.oh);
    const float fy = g.half_pixel ? __fsub_rn(__fmul_rn(__fadd_rn(static_cast<float>(oy), 0.5f), g.hs), 0.5f) : __fmul_rn(static_cast<float>(oy), g.hs);
    const float fx = g.half_pixel ? __fsub_rn(__fmul_rn(__fadd_rn(static_cast<float>(ox), 0.5f), g.ws), 0.5f) : __fmul_rn(static_cast<float>(ox), g.ws);
    const uint32_t y0 = static_cast<uint32_t>(fmaxf(floorf(fy), 0.0f)), x0 = static_cast<uint32_t>(fmaxf(floorf(fx), 0.0f));
    const int32_t y1 = static_cast<int32_t>(fminf(ceilf(fy), static_cast<float>(g.h - 1))), x1 = static_cast<int32_t>(fminf(ceilf(fx), static_cast<float>(g.w - 1)));
    const float dy = __fsub_rn(fy, static_cast<float>(y0)), dx = __fsub_rn(fx, static_cast<float>(x0));
    const float w00 = __fmul_rn(__fsub_rn(1.0f, dy), __fsub_rn(1.0f, dx)), w01 = __fmul_rn(dy, __fsub_rn(1.0f, dx));
    const float w10 = __fmul_rn(__fsub_rn(1.0f, dy), dx), w11 = __fmul_rn(dy, dx);
    auto at = [&](int32_t y, int32_t x) {
        return static_cast<float>(ld_act(in, ((static_cast<int64_t>(b) * g.h + y) * g.w + x) * g.c + c, g.is_signed));
    };
    // x0y0 * w + x0y1 * w + x1y0 * w + x1y1 * w, summed left to right
    float v = __fmul_rn(at(static_cast<int32_t>(y0), static_cast<int32_t>(x0)), w00);
    v = __fadd_rn(v, __fmul_rn(at(y1, static_cast<int32_t>(x0)), w01));
    v = __fadd_rn(v, __fmul_rn(at(static_cast<int32_t>(y0), x1), w10));
    v = __fadd_rn(v, __fmul_rn(at(y1, x1), w11));
    out[idx] = static_cast<uint8_t>(static_cast<int32_t>(v));
}

unsigned blocks_for(int64_t total, int threads = 256) { return static_cast<unsigned>((total + threads - 1) / threads); }

}  // namespace

// Device state of the operators above, owned by the op handle.
struct GraphOpState {
    MeanGeom mean{};
    ConcatArgs concat{};
    int64_t concat_outer = 0;
    SoftmaxGeom softmax{};
    ResizeGeom resize{};
};

cudaError_t launch_maxpool(const PoolGeom &p, const void *in, void *out, cudaStream_t s) {
    const int64_t total = static_cast<int64_t>(p.n) * p.oh * p.ow * p.c;
    if (total == 0) return cudaSuccess;
    launch_pdl(maxpool_kernel, dim3(blocks_for(total)), dim3(256), 0, s, p, in, static_cast<uint8_t *>(out), total);
    return cudaGetLastError();
}

cudaError_t launch_graph_op(enn_b200_op *op, const void *const *ins, int n_in, void *out) {
    GraphOpState *st = static_cast<GraphOpState *>(op->graph_state);
    cudaStream_t s = op->ctx->stream;
    uint8_t *o = static_cast<uint8_t *>(out);
    switch (op->kind) {
        case OP_MEAN: {
            const int64_t total = op->info.out_bytes;
            if (total == 0) return cudaSuccess;
            launch_pdl(mean_kernel, dim3(blocks_for(total, 128)), dim3(128), 0, s, st->mean, ins[0], o, total);
            break;
        }
        case OP_CONCAT: {
            ConcatArgs a = st->concat;
            if (n_in != a.n_inputs) return cudaErrorInvalidValue;
            int64_t largest = 0;
            for (int i = 0; i < n_in; ++i) {
                a.part[i].in = static_cast<const uint8_t *>(ins[i]);
                largest = a.part[i].inner > largest ? a.part[i].inner : largest;
            }
            const int64_t per = st->concat_outer * largest;
            if (per == 0) return cudaSuccess;
            const unsigned bx = static_cast<unsigned>(per / 256 + 1 < 4096 ? per / 256 + 1 : 4096);
            launch_pdl(concat_kernel, dim3(bx, static_cast<unsigned>(n_in)), dim3(256), 0, s, a, o, st->concat_outer);
            break;
        }
        case OP_SOFTMAX: {
            const int64_t total = st->softmax.outer * st->softmax.inner;
            if (total == 0) return cudaSuccess;
            launch_pdl(softmax_kernel, dim3(blocks_for(total, 64)), dim3(64), 0, s, st->softmax, static_cast<const uint8_t *>(ins[0]), o, total);
            break;
        }
        case OP_RESIZE: {
            const int64_t total = op->info.out_bytes;
            if (total == 0) return cudaSuccess;
            launch_pdl(resize_bilinear_kernel, dim3(blocks_for(total)), dim3(256), 0, s, st->resize, ins[0], o, total);
            break;
        }
        default:
            return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

void graph_op_release(enn_b200_op *op) {
    delete static_cast<GraphOpState *>(op->graph_state);
    op->graph_state = nullptr;
}

}  // namespace enn_b200

using namespace enn_b200;

namespace {
int32_t gfail(enn_b200_context *ctx, int32_t st, const char *msg) {
    if (ctx) ctx->last_error = msg;
    return st;
}

enn_b200_op *new_graph_op(enn_b200_context *ctx, int kind) {
    enn_b200_op *op = new (std::nothrow) enn_b200_op();
    if (!op) return nullptr;
    op->ctx = ctx;
    op->kind = kind;
    op->impl = ENN_B200_IMPL_ELTWISE;
    op->info.impl = op->impl;
    op->info.kernel_launches = 1;
    op->graph_state = new (std::nothrow) GraphOpState();
    if (!op->graph_state) {
        delete op;
        return nullptr;
    }
    return op;
}

template <typename T>
bool upload(enn_b200_op *op, const std::vector<T> &v, const T **dev) {
    void *p = nullptr;
    if (cudaMalloc(&p, v.size() * sizeof(T)) != cudaSuccess) return false;
    op->owned.push_back(p);
    if (cudaMemcpy(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) return false;
    *dev = static_cast<const T *>(p);
    return true;
}
}  // namespace

extern "C" {

int32_t enn_b200_maxpool_prepare(enn_b200_context *ctx, const enn_b200_pool_desc *d, enn_b200_op **out) {
    if (!ctx || !d || !out) return gfail(ctx, ENN_B200_INVALID_PARAMS, "null argument");
    *out = nullptr;
    if (d->n < 0 || d->h <= 0 || d->w <= 0 || d->c <= 0 || d->kh <= 0 || d->kw <= 0 || d->stride_h <= 0 || d->stride_w <= 0 ||
        d->out_h <= 0 || d->out_w <= 0 || d->pad_t < 0 || d->pad_l < 0 || !(d->out_scale > 0.f))
        return gfail(ctx, ENN_B200_INVALID_PARAMS, "bad pool descriptor");
    enn_b200_op *op = new (std::nothrow) enn_b200_op();
    if (!op) return gfail(ctx, ENN_B200_FAILURE, "out of host memory");
    op->ctx = ctx;
    op->kind = OP_MAXPOOL;
    op->impl = ENN_B200_IMPL_ELTWISE;
    PoolGeom &p = op->pool;
    p.n = d->n; p.h = d->h; p.w = d->w; p.c = d->c; p.kh = d->kh; p.kw = d->kw; p.sh = d->stride_h; p.sw = d->stride_w;
    p.pt = d->pad_t; p.pl = d->pad_l; p.oh = d->out_h; p.ow = d->out_w;
    p.is_signed = d->act_dtype == ENN_B200_S8;
    activation_range(d->activation, d->act_dtype, d->out_scale, d->out_zp, &p.act_min, &p.act_max);
    op->info.impl = op->impl;
    op->info.in_bytes = static_cast<int64_t>(d->n) * d->h * d->w * d->c;
    op->info.out_bytes = static_cast<int64_t>(d->n) * d->out_h * d->out_w * d->c;
    op->info.algorithmic_bytes = op->info.in_bytes + op->info.out_bytes;
    op->info.act_min = p.act_min; op->info.act_max = p.act_max;
    op->info.kernel_launches = 1;
    op->info.out_n = d->n; op->info.out_h = d->out_h; op->info.out_w = d->out_w; op->info.out_c = d->c;
    *out = op;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_mean_prepare(enn_b200_context *ctx, const enn_b200_mean_desc *d, enn_b200_op **out) {
    if (!ctx || !d || !out) return gfail(ctx, ENN_B200_INVALID_PARAMS, "null argument");
    *out = nullptr;
    int64_t in_elems = 1, out_elems = 1, count = 1;
    for (int a = 0; a < 4; ++a) {
        if (d->dims[a] <= 0) return gfail(ctx, ENN_B200_INVALID_PARAMS, "mean: dims must be positive");
        in_elems *= d->dims[a];
        if (d->axis_mask & (1 << a)) count *= d->dims[a];
        else out_elems *= d->dims[a];
    }
    if ((d->axis_mask & ~15) || count > (1 << 23)) return gfail(ctx, ENN_B200_INVALID_PARAMS, "mean: bad axis mask or too many elements per output");
    enn_b200_op *op = new_graph_op(ctx, OP_MEAN);
    if (!op) return gfail(ctx, ENN_B200_FAILURE, "out of host memory");
    MeanGeom &g = static_cast<GraphOpState *>(op->graph_state)->mean;
    for (int a = 0; a < 4; ++a) {
        g.d[a] = d->dims[a];
        g.keep[a] = (d->axis_mask & (1 << a)) ? 0 : 1;
    }
    g.count = static_cast<int32_t>(count);
    g.is_signed = d->act_dtype == ENN_B200_S8;
    op->info.in_bytes = in_elems; op->info.out_bytes = out_elems;
    op->info.algorithmic_bytes = in_elems + out_elems;
    op->info.out_n = g.keep[0] ? g.d[0] : 1; op->info.out_h = g.keep[1] ? g.d[1] : 1; op->info.out_w = g.keep[2] ? g.d[2] : 1;
    op->info.out_c = g.keep[3] ? g.d[3] : 1;
    op->info.act_min = g.is_signed ? -128 : 0; op->info.act_max = g.is_signed ? 127 : 255;
    *out = op;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_concat_prepare(enn_b200_context *ctx, const enn_b200_concat_desc *d, enn_b200_op **out) {
    if (!ctx || !d || !out) return gfail(ctx, ENN_B200_INVALID_PARAMS, "null argument");
    *out = nullptr;
    if (d->n_inputs < 1 || d->n_inputs > ENN_B200_CONCAT_MAX_INPUTS || d->outer < 0 || !(d->out_scale > 0.f))
        return gfail(ctx, ENN_B200_INVALID_PARAMS, "bad concat descriptor");
    enn_b200_op *op = new_graph_op(ctx, OP_CONCAT);
    if (!op) return gfail(ctx, ENN_B200_FAILURE, "out of host memory");
    GraphOpState *st = static_cast<GraphOpState *>(op->graph_state);
    const bool is_signed = d->act_dtype == ENN_B200_S8;
    std::vector<uint8_t> lut(static_cast<size_t>(d->n_inputs) * 256);
    int64_t off = 0;
    for (int i = 0; i < d->n_inputs; ++i) {
        if (d->inner[i] < 0 || !(d->in_scale[i] > 0.f)) {
            enn_b200_op_release(op);
            return gfail(ctx, ENN_B200_INVALID_PARAMS, "bad concat input");
        }
        ConcatPart &p = st->concat.part[i];
        p.in = nullptr; p.inner = d->inner[i]; p.offset = off;
        p.use_lut = d->in_scale[i] != d->out_scale;      // equal scales: plain copy, whatever the zero points (ConcatKernels.cpp:423)
        off += d->inner[i];
        for (int b = 0; b < 256; ++b) lut[i * 256 + b] = concat_requant_byte(static_cast<uint8_t>(b), is_signed, d->in_scale[i], d->in_zp[i], d->out_scale, d->out_zp);
    }
    st->concat.out_inner = off;
    st->concat.n_inputs = d->n_inputs;
    st->concat_outer = d->outer;
    if (!upload(op, lut, &st->concat.lut)) {
        enn_b200_op_release(op);
        return gfail(ctx, ENN_B200_CUDA_FAILURE, "concat: table upload failed");
    }
    op->info.in_bytes = d->outer * off; op->info.out_bytes = d->outer * off;
    op->info.algorithmic_bytes = 2 * d->outer * off;
    op->info.out_n = 1; op->info.out_h = 1; op->info.out_w = static_cast<int32_t>(d->outer); op->info.out_c = static_cast<int32_t>(off);
    op->info.act_min = is_signed ? -128 : 0; op->info.act_max = is_signed ? 127 : 255;
    *out = op;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_softmax_prepare(enn_b200_context *ctx, const enn_b200_softmax_desc *d, enn_b200_op **out) {
    if (!ctx || !d || !out) return gfail(ctx, ENN_B200_INVALID_PARAMS, "null argument");
    *out = nullptr;
    if (d->outer < 0 || d->channels <= 0 || d->inner <= 0 || !(d->in_scale > 0.f) || !(d->out_scale > 0.f))
        return gfail(ctx, ENN_B200_INVALID_PARAMS, "bad softmax descriptor");
    enn_b200_op *op = new_graph_op(ctx, OP_SOFTMAX);
    if (!op) return gfail(ctx, ENN_B200_FAILURE, "out of host memory");
    SoftmaxGeom &g = static_cast<GraphOpState *>(op->graph_state)->softmax;
    g.outer = d->outer; g.inner = d->inner; g.channels = d->channels;
    g.is_signed = d->act_dtype == ENN_B200_S8;
    g.inv_out_scale = 1 / d->out_scale;          // CLQuantization::execute passes 1 / scale as a float
    g.out_zp = d->out_zp;
    std::vector<float> lut(256 * 256);
    softmax_exp_table(g.is_signed != 0, d->in_scale, d->in_zp, d->beta, lut.data());
    if (!upload(op, lut, &g.exp_lut)) {
        enn_b200_op_release(op);
        return gfail(ctx, ENN_B200_CUDA_FAILURE, "softmax: table upload failed");
    }
    const int64_t elems = d->outer * d->channels * d->inner;
    op->info.in_bytes = elems; op->info.out_bytes = elems;
    op->info.algorithmic_bytes = 2 * elems;
    op->info.out_n = 1; op->info.out_h = static_cast<int32_t>(d->outer); op->info.out_w = d->channels; op->info.out_c = static_cast<int32_t>(d->inner);
    op->info.act_min = g.is_signed ? -128 : 0; op->info.act_max = g.is_signed ? 127 : 255;
    *out = op;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_resize_bilinear_prepare(enn_b200_context *ctx, const enn_b200_resize_desc *d, enn_b200_op **out) {
    if (!ctx || !d || !out) return gfail(ctx, ENN_B200_INVALID_PARAMS, "null argument");
    *out = nullptr;
    if (d->n < 0 || d->h <= 0 || d->w <= 0 || d->c <= 0 || d->out_h <= 0 || d->out_w <= 0) return gfail(ctx, ENN_B200_INVALID_PARAMS, "bad resize descriptor");
    enn_b200_op *op = new_graph_op(ctx, OP_RESIZE);
    if (!op) return gfail(ctx, ENN_B200_FAILURE, "out of host memory");
    ResizeGeom &g = static_cast<GraphOpState *>(op->graph_state)->resize;
    g.n = d->n; g.h = d->h; g.w = d->w; g.c = d->c; g.oh = d->out_h; g.ow = d->out_w;
    resize_scales(d->h, d->w, d->out_h, d->out_w, d->align_corners != 0, &g.hs, &g.ws);
    g.half_pixel = d->half_pixel_centers != 0;
    g.is_signed = d->act_dtype == ENN_B200_S8;
    op->info.in_bytes = static_cast<int64_t>(d->n) * d->h * d->w * d->c;
    op->info.out_bytes = static_cast<int64_t>(d->n) * d->out_h * d->out_w * d->c;
    op->info.algorithmic_bytes = op->info.in_bytes + op->info.out_bytes;
    op->info.out_n = d->n; op->info.out_h = d->out_h; op->info.out_w = d->out_w; op->info.out_c = d->c;
    op->info.act_min = g.is_signed ? -128 : 0; op->info.act_max = g.is_signed ? 127 : 255;
    *out = op;
    return ENN_B200_SUCCESS;
}

}  // extern "C"
