// extern "C" surface of the library: context / memory shim and operator prepare / execute / release.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "internal.h"
#include "quant_host.h"
#include "requant.h"

using namespace enn_b200;

namespace {

int32_t fail(enn_b200_context *ctx, int32_t status, const std::string &msg) {
    if (ctx) ctx->last_error = msg;
    return status;
}

int32_t cuda_fail(enn_b200_context *ctx, cudaError_t e, const char *what) {
    return fail(ctx, ENN_B200_CUDA_FAILURE, std::string(what) + ": " + cudaGetErrorString(e));
}

#define ENN_CUDA(ctx, call)                                        \
    do {                                                           \
        cudaError_t e__ = (call);                                  \
        if (e__ != cudaSuccess) return cuda_fail(ctx, e__, #call); \
    } while (0)

template <typename T>
int32_t upload_vec(enn_b200_op *op, const std::vector<T> &v, T **dev) {
    void *p = nullptr;
    const size_t bytes = (v.size() ? v.size() : 1) * sizeof(T);
    ENN_CUDA(op->ctx, cudaMalloc(&p, bytes));
    op->owned.push_back(p);
    if (!v.empty()) ENN_CUDA(op->ctx, cudaMemcpyAsync(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice, op->ctx->stream));
    // The source vector is a host temporary: finish the copy before it dies.
    ENN_CUDA(op->ctx, cudaStreamSynchronize(op->ctx->stream));
    *dev = static_cast<T *>(p);
    return ENN_B200_SUCCESS;
}


int32_t conv_out_dim(int32_t in, int32_t p0, int32_t p1, int32_t k, int32_t d, int32_t s) {
    return (in + p0 + p1 - ((k - 1) * d + 1) + s) / s;  // CLConvolution.cpp:99-104
}

bool valid_common(const enn_b200_conv_desc *d) {
    if (d->n < 0 || d->h <= 0 || d->w <= 0 || d->cin <= 0 || d->cout <= 0) return false;
    if (d->kh <= 0 || d->kw <= 0 || d->stride_h <= 0 || d->stride_w <= 0) return false;
    if (d->pad_t < 0 || d->pad_b < 0 || d->pad_l < 0 || d->pad_r < 0) return false;
    if (d->act_dtype != ENN_B200_U8 && d->act_dtype != ENN_B200_S8) return false;
    if (d->weight_dtype != ENN_B200_U8 && d->weight_dtype != ENN_B200_S8) return false;
    if (d->activation < ENN_B200_ACT_NONE || d->activation > ENN_B200_ACT_RELU6) return false;
    if (!(d->in_scale > 0.f) || !(d->out_scale > 0.f)) return false;
    return true;
}

// Fills geometry, clamp range and the per-channel requant vectors shared by conv / depthwise / deconv / fc.
int32_t setup_quant(enn_b200_op *op, const enn_b200_conv_desc *d, const int32_t *bias_host, const float *pc_scales) {
    ConvGeom &g = op->g;
    g.in_zp = d->in_zp;
    g.w_zp = d->per_channel ? 0 : d->w_zp;  // per-channel kernels are handed weight_offset 0
    g.out_zp = d->out_zp;
    g.a_signed = d->act_dtype == ENN_B200_S8;
    g.w_signed = d->weight_dtype == ENN_B200_S8;
    activation_range(d->activation, d->act_dtype, d->out_scale, d->out_zp, &g.act_min, &g.act_max);
    if (d->per_channel && !pc_scales) return fail(op->ctx, ENN_B200_INVALID_PARAMS, "per_channel set but per_channel_scales is null");
    std::vector<int32_t> mult, shift;
    if (!derive_requant(d->cout, d->per_channel != 0, d->in_scale, d->w_scale, d->bias_scale, d->out_scale, pc_scales, &mult, &shift))
        return fail(op->ctx, ENN_B200_INVALID_PARAMS, "requantisation shift outside [-31, 30]");
    std::vector<int32_t> bias(bias_host, bias_host + d->cout);
    int32_t *dm = nullptr, *ds = nullptr, *db = nullptr;
    int32_t st;
    if ((st = upload_vec(op, mult, &dm)) || (st = upload_vec(op, shift, &ds)) || (st = upload_vec(op, bias, &db))) return st;
    op->rq = Requant{dm, ds, db};
    op->info.act_min = g.act_min;
    op->info.act_max = g.act_max;
    return ENN_B200_SUCCESS;
}

void fill_info(enn_b200_op *op, int64_t in_elems, int64_t out_elems, int64_t macs, int64_t weight_bytes, int32_t cout,
               bool per_channel) {
    op->info.in_bytes = in_elems;
    op->info.out_bytes = out_elems;
    op->info.macs = macs;
    op->info.algorithmic_bytes = in_elems + out_elems + weight_bytes + static_cast<int64_t>(cout) * 4 * (per_channel ? 3 : 1);
    op->info.kernel_launches = 1;
}

}  // namespace

namespace enn_b200 {

static bool g_pdl_on = true;     // process-wide; option "no_pdl" of any context turns it off
bool pdl_enabled() { return g_pdl_on; }

// mma_peak.cu
double measure_mma_peak(enn_b200_context *ctx, int kind, int n, int iters);
// gemm_tc.cu
int32_t tc_plan_conv(enn_b200_op *op, const void *weights_hwio_host);
int32_t tc_execute(enn_b200_op *op, const void *in, void *out);
void tc_release(enn_b200_op *op);
bool tc_available(const enn_b200_context *ctx);
int32_t tc_test_starve_next(enn_b200_op *op);
int32_t tc_fuse_add(enn_b200_op *op, const AddParams &add, bool conv_is_second);
void tc_set_residual(enn_b200_op *op, const void *res);
void tc_clear_error(enn_b200_op *op);
}  // namespace enn_b200

extern "C" {

const char *enn_b200_version(void) { return "enn_b200 0.1 (sm_100a)"; }

int32_t enn_b200_context_create(int32_t device, enn_b200_context **out) {
    if (!out) return ENN_B200_INVALID_PARAMS;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) return ENN_B200_CUDA_FAILURE;
    if (device < 0 || device >= count) return ENN_B200_INVALID_PARAMS;
    enn_b200_context *ctx = new (std::nothrow) enn_b200_context();
    if (!ctx) return ENN_B200_FAILURE;
    ctx->device = device;
    if (cudaSetDevice(device) != cudaSuccess || cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete ctx;
        return ENN_B200_CUDA_FAILURE;
    }
    cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, device);
    cudaDeviceGetAttribute(&ctx->cc_major, cudaDevAttrComputeCapabilityMajor, device);
    cudaDeviceGetAttribute(&ctx->cc_minor, cudaDevAttrComputeCapabilityMinor, device);
    cudaDriverEntryPointQueryResult qres;
    void *fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
        ctx->encode_tiled = fn;
    *out = ctx;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_context_destroy(enn_b200_context *ctx) {
    if (!ctx) return ENN_B200_INVALID_PARAMS;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->aux_ready) {
        for (int i = 0; i < enn_b200_context::kAuxStreams; ++i) {
            cudaStreamSynchronize(ctx->aux_streams[i]);
            cudaStreamDestroy(ctx->aux_streams[i]);
            cudaEventDestroy(ctx->ev_join[i]);
        }
        cudaEventDestroy(ctx->ev_fork);
    }
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_malloc(enn_b200_context *ctx, size_t bytes, void **dev_ptr) {
    if (!ctx || !dev_ptr) return ENN_B200_INVALID_PARAMS;
    *dev_ptr = nullptr;
    ENN_CUDA(ctx, cudaSetDevice(ctx->device));
    ENN_CUDA(ctx, cudaMalloc(dev_ptr, bytes ? bytes : 1));
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_free(enn_b200_context *ctx, void *dev_ptr) {
    if (!ctx) return ENN_B200_INVALID_PARAMS;
    if (!dev_ptr) return ENN_B200_SUCCESS;
    ENN_CUDA(ctx, cudaSetDevice(ctx->device));
    ENN_CUDA(ctx, cudaFree(dev_ptr));
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_upload(enn_b200_context *ctx, void *dev_dst, const void *host_src, size_t bytes) {
    if (!ctx || (bytes && (!dev_dst || !host_src))) return ENN_B200_INVALID_PARAMS;
    if (!bytes) return ENN_B200_SUCCESS;
    ENN_CUDA(ctx, cudaMemcpyAsync(dev_dst, host_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_download(enn_b200_context *ctx, void *host_dst, const void *dev_src, size_t bytes) {
    if (!ctx || (bytes && (!host_dst || !dev_src))) return ENN_B200_INVALID_PARAMS;
    if (bytes) ENN_CUDA(ctx, cudaMemcpyAsync(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    ENN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_copy_device(enn_b200_context *ctx, void *dev_dst, const void *dev_src, size_t bytes) {
    if (!ctx || (bytes && (!dev_dst || !dev_src))) return fail(ctx, ENN_B200_INVALID_PARAMS, "bad copy arguments");
    if (bytes) ENN_CUDA(ctx, cudaMemcpyAsync(dev_dst, dev_src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_stream_sync(enn_b200_context *ctx) {
    if (!ctx) return ENN_B200_INVALID_PARAMS;
    ENN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return ENN_B200_SUCCESS;
}

// Device timer on the context's stream (two events): what an operator-level profiler brackets an execute() with.
struct enn_b200_timer {
    enn_b200_context *ctx = nullptr;
    cudaEvent_t a = nullptr, b = nullptr;
    bool started = false, stopped = false;
};

int32_t enn_b200_timer_create(enn_b200_context *ctx, enn_b200_timer **out) {
    if (!ctx || !out) return ENN_B200_INVALID_PARAMS;
    *out = nullptr;
    ENN_CUDA(ctx, cudaSetDevice(ctx->device));
    enn_b200_timer *t = new (std::nothrow) enn_b200_timer();
    if (!t) return fail(ctx, ENN_B200_FAILURE, "out of host memory");
    t->ctx = ctx;
    if (cudaEventCreate(&t->a) != cudaSuccess || cudaEventCreate(&t->b) != cudaSuccess) {
        if (t->a) cudaEventDestroy(t->a);
        delete t;
        return fail(ctx, ENN_B200_CUDA_FAILURE, "event creation failed");
    }
    *out = t;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_timer_start(enn_b200_timer *t) {
    if (!t) return ENN_B200_INVALID_PARAMS;
    ENN_CUDA(t->ctx, cudaEventRecord(t->a, t->ctx->stream));
    t->started = true;
    t->stopped = false;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_timer_stop(enn_b200_timer *t) {
    if (!t || !t->started) return ENN_B200_INVALID_PARAMS;
    ENN_CUDA(t->ctx, cudaEventRecord(t->b, t->ctx->stream));
    t->stopped = true;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_timer_elapsed_us(enn_b200_timer *t, float *us) {
    if (!t || !us || !t->stopped) return ENN_B200_INVALID_PARAMS;
    ENN_CUDA(t->ctx, cudaEventSynchronize(t->b));
    float ms = 0.f;
    ENN_CUDA(t->ctx, cudaEventElapsedTime(&ms, t->a, t->b));
    *us = ms * 1000.f;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_timer_destroy(enn_b200_timer *t) {
    if (!t) return ENN_B200_INVALID_PARAMS;
    cudaEventDestroy(t->a);
    cudaEventDestroy(t->b);
    delete t;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_host_alloc(size_t bytes, void **host_ptr) {
    if (!host_ptr) return ENN_B200_INVALID_PARAMS;
    return cudaHostAlloc(host_ptr, bytes ? bytes : 1, cudaHostAllocDefault) == cudaSuccess ? ENN_B200_SUCCESS : ENN_B200_CUDA_FAILURE;
}

int32_t enn_b200_host_free(void *host_ptr) {
    if (!host_ptr) return ENN_B200_SUCCESS;
    return cudaFreeHost(host_ptr) == cudaSuccess ? ENN_B200_SUCCESS : ENN_B200_CUDA_FAILURE;
}

int32_t enn_b200_last_error(enn_b200_context *ctx, char *buf, size_t buf_len) {
    if (!buf || !buf_len) return ENN_B200_SUCCESS;
    const std::string s = ctx ? ctx->last_error : std::string("null context");
    std::snprintf(buf, buf_len, "%s", s.c_str());
    return ENN_B200_SUCCESS;
}

void *enn_b200_stream(enn_b200_context *ctx) { return ctx ? static_cast<void *>(ctx->stream) : nullptr; }

int32_t enn_b200_context_set_option(enn_b200_context *ctx, const char *name, int32_t value) {
    if (!ctx || !name) return ENN_B200_INVALID_PARAMS;
    static const char *const known[] = {"no_pdl", "no_relu_mode", "no_relu_hi", "no_relu_sat", "no_wide_store", "no_grouped_tc", "no_first_layer", "no_implicit", "no_gemv",
                                        "no_narrow_span", "no_pack", "pack_wide", "no_bres", "no_bres_k1", "no_fan_out", "tc_bn",
                                        "tc_pair", "tc_raster", "epi_g", "dw_legacy", "no_fuse", "fuse_all", "dw_rows", "grid_cap", "no_out_stream", "no_narrow_n"};
    bool ok = false;
    for (const char *k : known) ok = ok || std::strcmp(k, name) == 0;
    if (!ok) return fail(ctx, ENN_B200_INVALID_PARAMS, std::string("unknown option: ") + name);
    if (std::strcmp(name, "tc_bn") == 0 && value != 0 && value < 96) return fail(ctx, ENN_B200_INVALID_PARAMS, "tc_bn must be 0 or at least 96");
    ctx->options[name] = value;
    if (std::strcmp(name, "no_pdl") == 0) g_pdl_on = value == 0;
    return ENN_B200_SUCCESS;
}

void enn_b200_quantize_multiplier(double real_multiplier, int32_t *quantized_multiplier, int32_t *shift) {
    quantize_multiplier(real_multiplier, quantized_multiplier, shift);
}

int32_t enn_b200_conv_multiplier(double in_scale, double w_scale, double bias_scale, double out_scale, double *multiplier) {
    return conv_multiplier(in_scale, w_scale, bias_scale, out_scale, multiplier) ? ENN_B200_SUCCESS : ENN_B200_FAILURE;
}

void enn_b200_activation_range(int32_t activation, int32_t act_dtype, float scale, int32_t zero_point, int32_t *act_min,
                               int32_t *act_max) {
    activation_range(activation, act_dtype, scale, zero_point, act_min, act_max);
}

int32_t enn_b200_measure_mma_peak(enn_b200_context *ctx, int32_t kind, int32_t n, int32_t iters, double *tera_ops) {
    if (!ctx || !tera_ops) return ENN_B200_INVALID_PARAMS;
    // 2^16 groups keep every SM busy for a few milliseconds; more would hold a shared GPU for no better figure.
    if (iters < 1 || iters > (1 << 16)) return fail(ctx, ENN_B200_INVALID_PARAMS, "iters must be within 1 .. 65536");
    const double v = measure_mma_peak(ctx, kind, n, iters);
    if (v < 0) return fail(ctx, ENN_B200_FAILURE, "tensor-pipe peak measurement failed");
    *tera_ops = v;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_requant_host(int32_t acc, int32_t mult, int32_t shift, int32_t out_zp, int32_t act_min, int32_t act_max) {
    return enn_requant(acc, mult, shift, out_zp, act_min, act_max);
}

// ------------------------------------------------------------------------------------------------------
// Conv2D
// ------------------------------------------------------------------------------------------------------
static int32_t conv_like_prepare_const(enn_b200_context *ctx, const enn_b200_conv_desc *d, const void *w_host,
                                       const int32_t *bias_host, const float *pc_scales, int kind, enn_b200_op **out) {
    if (!ctx || !d || !w_host || !bias_host || !out) return fail(ctx, ENN_B200_INVALID_PARAMS, "null argument");
    *out = nullptr;
    if (!valid_common(d)) return fail(ctx, ENN_B200_INVALID_PARAMS, "bad descriptor");
    const int32_t groups = d->groups > 0 ? d->groups : 1;
    const int32_t dil_h = d->dil_h > 0 ? d->dil_h : 1, dil_w = d->dil_w > 0 ? d->dil_w : 1;
    if (kind == OP_CONV && (d->cin % groups || d->cout % groups)) return fail(ctx, ENN_B200_INVALID_PARAMS, "channels not divisible by groups");
    // cout > cin * depth_multiplier: the channels past the filter's are bias only (depthwise_conv_unequal, CLDepthwiseConvolutionQuantized.cpp:183-186)
    if (kind == OP_DEPTHWISE && d->cout < d->cin * groups) return fail(ctx, ENN_B200_INVALID_PARAMS, "depthwise cout < cin * depth_multiplier");
    if (kind == OP_DECONV && groups != 1) return fail(ctx, ENN_B200_INVALID_PARAMS, "quantized deconvolution supports group_size 1 only");
    if (kind == OP_DECONV && d->weight_layout == ENN_B200_W_OIHW) return fail(ctx, ENN_B200_INVALID_PARAMS, "deconvolution weights are IOHW or OHWI");
    if (kind != OP_DECONV && d->weight_layout == ENN_B200_W_IOHW) return fail(ctx, ENN_B200_INVALID_PARAMS, "IOHW is a deconvolution layout");
    ENN_CUDA(ctx, cudaSetDevice(ctx->device));

    enn_b200_op *op = new (std::nothrow) enn_b200_op();
    if (!op) return fail(ctx, ENN_B200_FAILURE, "out of host memory");
    op->ctx = ctx;
    op->kind = kind;
    ConvGeom &g = op->g;
    g.n = d->n; g.h = d->h; g.w = d->w; g.cin = d->cin;
    g.cout = d->cout; g.kh = d->kh; g.kw = d->kw;
    g.sh = d->stride_h; g.sw = d->stride_w; g.dh = dil_h; g.dw = dil_w;
    g.pt = d->pad_t; g.pl = d->pad_l;
    g.groups = groups;
    g.cin_g = kind == OP_CONV ? d->cin / groups : d->cin;
    g.cout_g = kind == OP_CONV ? d->cout / groups : d->cout;
    if (kind == OP_DECONV) {
        // CLDeconvolution.cpp:82-87 (explicit output size wins, as TRANSPOSE_CONV carries one)
        g.oh = d->out_h > 0 ? d->out_h : d->h * d->stride_h + d->kh - d->stride_h - d->pad_t - d->pad_b;
        g.ow = d->out_w > 0 ? d->out_w : d->w * d->stride_w + d->kw - d->stride_w - d->pad_l - d->pad_r;
    } else {
        g.oh = d->out_h > 0 ? d->out_h : conv_out_dim(d->h, d->pad_t, d->pad_b, d->kh, dil_h, d->stride_h);
        g.ow = d->out_w > 0 ? d->out_w : conv_out_dim(d->w, d->pad_l, d->pad_r, d->kw, dil_w, d->stride_w);
    }
    if (g.oh <= 0 || g.ow <= 0) {
        delete op;
        return fail(ctx, ENN_B200_INVALID_PARAMS, "empty output");
    }
    int32_t st = setup_quant(op, d, bias_host, pc_scales);
    if (st) {
        enn_b200_op_release(op);
        return st;
    }

    // Re-pack weights once, on the host, into [Kh][Kw][Cin/g][Cout] (conv, deconv) or [Kh][Kw][Cout]
    // (depthwise), raw bytes.  This replaces the reference's alignQuantizedWeight_gemm / matrixTrans /
    // convertToNCHW passes run in initialize().
    const int32_t kh = d->kh, kw = d->kw, cout = d->cout;
    const int32_t cig = kind == OP_DEPTHWISE ? 1 : g.cin_g;
    const int32_t dw_real = d->cin * groups;      // depthwise: output channels that have a filter
    std::vector<uint8_t> packed(static_cast<size_t>(kh) * kw * cig * cout);
    const uint8_t *src = static_cast<const uint8_t *>(w_host);
    for (int32_t oc = 0; oc < cout; ++oc) {
        const int32_t grp = kind == OP_CONV ? oc / g.cout_g : 0, ocg = kind == OP_CONV ? oc % g.cout_g : oc;
        for (int32_t ky = 0; ky < kh; ++ky)
            for (int32_t kx = 0; kx < kw; ++kx)
                for (int32_t ic = 0; ic < cig; ++ic) {
                    int64_t si;
                    if (kind == OP_DEPTHWISE) {
                        if (oc >= dw_real) {      // no filter for this channel: the zero-point byte makes every product zero
                            packed[((static_cast<size_t>(ky) * kw + kx) * cig + ic) * cout + oc] = static_cast<uint8_t>(d->per_channel ? 0 : d->w_zp);
                            continue;
                        }
                        si = d->weight_layout == ENN_B200_W_OHWI ? (static_cast<int64_t>(ky) * kw + kx) * dw_real + oc
                                                                  : static_cast<int64_t>(oc) * kh * kw + ky * kw + kx;
                    } else if (d->weight_layout == ENN_B200_W_OHWI) {
                        si = ((static_cast<int64_t>(oc) * kh + ky) * kw + kx) * cig + ic;
                    } else if (d->weight_layout == ENN_B200_W_IOHW) {
                        si = static_cast<int64_t>(ic) * cout * kh * kw + static_cast<int64_t>(oc) * kh * kw + ky * kw + kx;
                    } else {
                        si = static_cast<int64_t>(grp) * cig * g.cout_g * kh * kw + static_cast<int64_t>(ocg) * cig * kh * kw +
                             static_cast<int64_t>(ic) * kh * kw + ky * kw + kx;
                    }
                    packed[((static_cast<size_t>(ky) * kw + kx) * cig + ic) * cout + oc] = src[si];
                }
    }
    uint8_t *wd = nullptr;
    if ((st = upload_vec(op, packed, &wd))) {
        enn_b200_op_release(op);
        return st;
    }
    op->w_direct = wd;

    const int64_t out_px = static_cast<int64_t>(g.n) * g.oh * g.ow;
    int64_t macs;
    if (kind == OP_DEPTHWISE)
        macs = out_px * cout * kh * kw;
    else if (kind == OP_DECONV)
        macs = static_cast<int64_t>(g.n) * g.h * g.w * g.cin * cout * kh * kw;
    else
        macs = out_px * cout * kh * kw * g.cin_g;
    fill_info(op, static_cast<int64_t>(g.n) * g.h * g.w * g.cin, out_px * cout, macs, static_cast<int64_t>(packed.size()), cout,
              d->per_channel != 0);
    op->info.out_n = g.n; op->info.out_h = g.oh; op->info.out_w = g.ow; op->info.out_c = cout;
    op->impl = kind == OP_DEPTHWISE ? ENN_B200_IMPL_DEPTHWISE : ENN_B200_IMPL_DIRECT;
    if (kind == OP_DEPTHWISE && dw3x3_eligible(g)) {
        // Constants of the 3x3 fast path (depthwise.cu): folded bias, stage-2 addend, packed tap words.
        std::vector<int32_t> mult, shift;
        derive_requant(cout, d->per_channel != 0, d->in_scale, d->w_scale, d->bias_scale, d->out_scale, pc_scales, &mult, &shift);
        std::vector<int32_t> chan(static_cast<size_t>(cout) * 4);
        std::vector<uint32_t> wp(static_cast<size_t>(cout) * 3);
        bool ok = true;
        for (int32_t c = 0; c < cout && ok; ++c) {
            int64_t wsum = 0, wabs = 0;
            for (int32_t ky = 0; ky < 3; ++ky) {
                uint32_t word = 0;
                for (int32_t kx = 0; kx < 3; ++kx) {
                    const uint8_t raw = packed[(static_cast<size_t>(ky) * 3 + kx) * cout + c];
                    const int32_t wv = g.w_signed ? static_cast<int32_t>(static_cast<int8_t>(raw)) : static_cast<int32_t>(raw);
                    wsum += wv;
                    wabs += wv < 0 ? -wv : wv;
                    word |= static_cast<uint32_t>(raw) << (8 * kx);
                }
                wp[static_cast<size_t>(c) * 3 + ky] = word;
            }
            const int64_t folded = static_cast<int64_t>(bias_host[c]) - static_cast<int64_t>(g.in_zp) * wsum +
                                   9ll * g.in_zp * g.w_zp;
            const int32_t e = shift[c] > 0 ? -1 : -shift[c];
            // |accumulator| bound: 9 taps of a in [0,255] against w, the w_zp * sum(a) term and the folded bias.
            const int64_t acc_bound = 255 * wabs + 9ll * 255 * (g.w_zp < 0 ? -g.w_zp : g.w_zp) + (folded < 0 ? -folded : folded);
            // stage-2 addend with the output zero point and the (negated) lower clamp folded in
            const int64_t zo_eff = static_cast<int64_t>(g.out_zp) - g.act_min;
            const int64_t addend = e > 0 ? (1ll << (e - 1)) + zo_eff * (1ll << e) : zo_eff;
            if (e < 0 || folded > INT32_MAX || folded < INT32_MIN || acc_bound + 2 + (addend < 0 ? -addend : addend) >= (1ll << 31)) {
                ok = false;   // left shift or possible overflow of the fused stage-2 form: keep the general kernel
                break;
            }
            chan[c * 4 + 0] = mult[c];
            chan[c * 4 + 1] = static_cast<int32_t>(addend);
            chan[c * 4 + 2] = e | ((e > 0 ? 31 : 32) << 8);
            chan[c * 4 + 3] = static_cast<int32_t>(folded);
        }
        // ReLU-type output (lower clamp == output zero point) with right shifts only: merged one-shift form.
        bool relu = ok && g.out_zp == g.act_min && !ctx->opt("no_relu_mode");
        for (int32_t c = 0; c < cout && relu; ++c)
            if ((chan[c * 4 + 2] & 0xff) < 1 || chan[c * 4 + 0] < 0) relu = false;
        if (relu) {
            for (int32_t c = 0; c < cout; ++c) {
                const int32_t m0 = chan[c * 4 + 0], e = chan[c * 4 + 2] & 0xff;
                const int64_t cc = static_cast<int64_t>(chan[c * 4 + 3]) * m0 + (1ll << 30) + (1ll << (30 + e));
                chan[c * 4 + 0] = static_cast<int32_t>(static_cast<uint32_t>(static_cast<uint64_t>(cc) & 0xffffffffu));
                chan[c * 4 + 1] = static_cast<int32_t>(static_cast<uint32_t>(static_cast<uint64_t>(cc) >> 32));
                chan[c * 4 + 2] = m0;
                chan[c * 4 + 3] = e - 1;
            }
            op->dw_relu = true;
        }
        if (ok) {
            int32_t *dc = nullptr;
            uint32_t *dwp = nullptr;
            if ((st = upload_vec(op, chan, &dc)) || (st = upload_vec(op, wp, &dwp))) {
                enn_b200_op_release(op);
                return st;
            }
            op->dw_chan = dc;
            op->dw_w = dwp;
            // Row-ring variant (C % 16 == 0): input rows staged in shared memory by bulk copies; the default where it applies.
            dw_ring_plan(op);
        }
    }
    if (kind != OP_DEPTHWISE && tc_available(ctx)) {
        st = tc_plan_conv(op, packed.data());
        if (st == ENN_B200_SUCCESS && op->tc) op->impl = ENN_B200_IMPL_TCGEN05;
        else if (st != ENN_B200_SUCCESS && st != ENN_B200_INVALID_PARAMS) {
            enn_b200_op_release(op);
            return st;
        }
    }
    // The tensor-core plan may have chosen its weight-streaming GEMV for very small M; report that.
    if (!(op->impl == ENN_B200_IMPL_TCGEN05 && op->info.impl == ENN_B200_IMPL_GEMV)) op->info.impl = op->impl;
    *out = op;
    return ENN_B200_SUCCESS;
}

// Filter and / or bias as runtime tensors: plan with whatever is constant (zeros stand in for the rest), remember
// what a rebind needs.
static int32_t conv_like_prepare(enn_b200_context *ctx, const enn_b200_conv_desc *d, const void *w_host,
                                 const int32_t *bias_host, const float *pc_scales, int kind, enn_b200_op **out) {
    if (!d || (!d->weights_as_input && !d->bias_as_input)) return conv_like_prepare_const(ctx, d, w_host, bias_host, pc_scales, kind, out);
    if (!ctx || !out) return fail(ctx, ENN_B200_INVALID_PARAMS, "null argument");
    *out = nullptr;
    if (!valid_common(d)) return fail(ctx, ENN_B200_INVALID_PARAMS, "bad descriptor");
    if ((!d->weights_as_input && !w_host) || (!d->bias_as_input && !bias_host)) return fail(ctx, ENN_B200_INVALID_PARAMS, "constant tensor missing");
    if (d->per_channel && !pc_scales) return fail(ctx, ENN_B200_INVALID_PARAMS, "per-channel scales missing");
    const int64_t groups = d->groups > 0 ? d->groups : 1;
    int64_t w_elems = static_cast<int64_t>(d->cout) * d->kh * d->kw;
    if (kind == OP_CONV) w_elems *= d->cin / groups;
    else if (kind == OP_DECONV) w_elems *= d->cin;
    else w_elems = static_cast<int64_t>(d->cin) * groups * d->kh * d->kw;      // depthwise: the filter's own channels
    std::unique_ptr<RuntimeConstants> dyn(new (std::nothrow) RuntimeConstants());
    if (!dyn) return fail(ctx, ENN_B200_FAILURE, "out of host memory");
    dyn->weights = d->weights_as_input != 0;
    dyn->bias = d->bias_as_input != 0;
    dyn->desc = *d;
    dyn->desc.weights_as_input = dyn->desc.bias_as_input = 0;
    dyn->prepare_kind = kind;
    if (d->per_channel) dyn->scales.assign(pc_scales, pc_scales + d->cout);
    dyn->w_host.assign(static_cast<size_t>(w_elems), 0);
    if (w_host) std::memcpy(dyn->w_host.data(), w_host, dyn->w_host.size());
    dyn->b_host.assign(static_cast<size_t>(d->cout), 0);
    if (bias_host) std::memcpy(dyn->b_host.data(), bias_host, dyn->b_host.size() * sizeof(int32_t));
    const int32_t st = conv_like_prepare_const(ctx, &dyn->desc, dyn->w_host.data(), dyn->b_host.data(),
                                               d->per_channel ? dyn->scales.data() : nullptr, kind, out);
    if (st == ENN_B200_SUCCESS) (*out)->dyn = std::move(dyn);
    return st;
}

int32_t enn_b200_conv2d_prepare(enn_b200_context *ctx, const enn_b200_conv_desc *desc, const void *weights_host,
                                const int32_t *bias_host, const float *per_channel_scales, enn_b200_op **op) {
    return conv_like_prepare(ctx, desc, weights_host, bias_host, per_channel_scales, OP_CONV, op);
}

int32_t enn_b200_depthwise_prepare(enn_b200_context *ctx, const enn_b200_conv_desc *desc, const void *weights_host,
                                   const int32_t *bias_host, const float *per_channel_scales, enn_b200_op **op) {
    return conv_like_prepare(ctx, desc, weights_host, bias_host, per_channel_scales, OP_DEPTHWISE, op);
}

int32_t enn_b200_deconv_prepare(enn_b200_context *ctx, const enn_b200_conv_desc *desc, const void *weights_host,
                                const int32_t *bias_host, const float *per_channel_scales, enn_b200_op **op) {
    return conv_like_prepare(ctx, desc, weights_host, bias_host, per_channel_scales, OP_DECONV, op);
}

int32_t enn_b200_fc_prepare(enn_b200_context *ctx, const enn_b200_fc_desc *d, const void *weights_host,
                            const int32_t *bias_host, const float *per_channel_scales, enn_b200_op **op) {
    if (!d) return fail(ctx, ENN_B200_INVALID_PARAMS, "null descriptor");
    if (d->m < 0 || d->k <= 0 || d->n <= 0) return fail(ctx, ENN_B200_INVALID_PARAMS, "bad FC shape");
    // [M][K] x [N][K]^T is the 1x1 convolution over M "pixels" with OHWI weights.
    enn_b200_conv_desc c;
    std::memset(&c, 0, sizeof(c));
    c.n = d->m; c.h = 1; c.w = 1; c.cin = d->k;
    c.cout = d->n; c.kh = 1; c.kw = 1;
    c.stride_h = c.stride_w = 1; c.dil_h = c.dil_w = 1;
    c.groups = 1;
    c.activation = d->activation; c.act_dtype = d->act_dtype; c.weight_dtype = d->weight_dtype;
    c.weight_layout = ENN_B200_W_OHWI;
    c.per_channel = d->per_channel;
    c.in_scale = d->in_scale; c.in_zp = d->in_zp; c.w_scale = d->w_scale; c.w_zp = d->w_zp;
    c.bias_scale = d->bias_scale; c.out_scale = d->out_scale; c.out_zp = d->out_zp;
    c.weights_as_input = d->weights_as_input; c.bias_as_input = d->bias_as_input;
    int32_t st = conv_like_prepare(ctx, &c, weights_host, bias_host, per_channel_scales, OP_CONV, op);
    if (st == ENN_B200_SUCCESS) (*op)->kind = OP_FC;
    return st;
}

int32_t enn_b200_add_prepare(enn_b200_context *ctx, const enn_b200_add_desc *d, enn_b200_op **out) {
    if (!ctx || !d || !out) return fail(ctx, ENN_B200_INVALID_PARAMS, "null argument");
    *out = nullptr;
    if (d->count < 0 || !(d->in0_scale > 0.f) || !(d->in1_scale > 0.f) || !(d->out_scale > 0.f))
        return fail(ctx, ENN_B200_INVALID_PARAMS, "bad add descriptor");
    enn_b200_op *op = new (std::nothrow) enn_b200_op();
    if (!op) return fail(ctx, ENN_B200_FAILURE, "out of host memory");
    op->ctx = ctx;
    op->kind = OP_ADD;
    op->impl = ENN_B200_IMPL_ELTWISE;
    op->count = d->count;
    AddParams &p = op->add;
    // CLAddQuantized.cpp:72-88: `2 * std::max(float, float)` is a float product, widened afterwards.
    const float twice_f = 2 * (d->in0_scale > d->in1_scale ? d->in0_scale : d->in1_scale);
    const double twice = twice_f;
    quantize_multiplier(d->in0_scale / twice, &p.m0, &p.s0);
    quantize_multiplier(d->in1_scale / twice, &p.m1, &p.s1);
    quantize_multiplier(twice / ((1 << 20) * d->out_scale), &p.mo, &p.so);
    if (p.s0 > 0 || p.s0 < -31 || p.s1 > 0 || p.s1 < -31 || p.so > 0 || p.so < -31) {
        delete op;
        return fail(ctx, ENN_B200_INVALID_PARAMS, "add: a stage shift is outside [-31, 0] (undefined in the reference kernel)");
    }
    p.in0_off = -d->in0_zp; p.in1_off = -d->in1_zp; p.out_off = d->out_zp;
    p.is_signed = d->act_dtype == ENN_B200_S8;
    if (d->activation != ENN_B200_ACT_NONE) {
        activation_range(d->activation, d->act_dtype, d->out_scale, d->out_zp, &p.act_min, &p.act_max);
    } else {
        p.act_min = p.is_signed ? -128 : 0;
        p.act_max = p.is_signed ? 127 : 255;
    }
    {
        std::vector<int32_t> lut(512);
        for (int32_t b = 0; b < 256; ++b) {
            const int32_t v = p.is_signed ? static_cast<int32_t>(static_cast<int8_t>(b)) : b;
            lut[b] = enn_rdivpot(enn_srdhm((p.in0_off + v) * (1 << 20), p.m0), -p.s0);
            lut[256 + b] = enn_rdivpot(enn_srdhm((p.in1_off + v) * (1 << 20), p.m1), -p.s1);
        }
        int32_t *dl = nullptr;
        const int32_t st = upload_vec(op, lut, &dl);
        if (st != ENN_B200_SUCCESS) {
            enn_b200_op_release(op);
            return st;
        }
        p.lut = dl;
        std::vector<uint8_t> lut2(65536);
        for (uint32_t a = 0; a < 256; ++a)
            for (uint32_t b = 0; b < 256; ++b) {
                int32_t o = enn_rdivpot(enn_srdhm(lut[a] + lut[256 + b], p.mo), -p.so) + p.out_off;
                o = o < p.act_min ? p.act_min : o;
                o = o > p.act_max ? p.act_max : o;
                lut2[add_lut2_index(a, b)] = static_cast<uint8_t>(o);
            }
        uint8_t *dl2 = nullptr;
        const int32_t st2 = upload_vec(op, lut2, &dl2);
        if (st2 != ENN_B200_SUCCESS) {
            enn_b200_op_release(op);
            return st2;
        }
        p.lut2 = dl2;
        const cudaError_t ae = add_kernel_init();
        if (ae != cudaSuccess) {
            enn_b200_op_release(op);
            return cuda_fail(ctx, ae, "add_kernel_init");
        }
    }
    op->info.impl = op->impl;
    op->info.in_bytes = 2 * d->count; op->info.out_bytes = d->count;
    op->info.algorithmic_bytes = 3 * d->count;
    op->info.act_min = p.act_min; op->info.act_max = p.act_max;
    op->info.kernel_launches = 1;
    op->info.out_n = 1; op->info.out_h = 1; op->info.out_w = 1; op->info.out_c = static_cast<int32_t>(d->count);
    *out = op;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_avgpool_prepare(enn_b200_context *ctx, const enn_b200_pool_desc *d, enn_b200_op **out) {
    if (!ctx || !d || !out) return fail(ctx, ENN_B200_INVALID_PARAMS, "null argument");
    *out = nullptr;
    if (d->n < 0 || d->h <= 0 || d->w <= 0 || d->c <= 0 || d->kh <= 0 || d->kw <= 0 || d->stride_h <= 0 || d->stride_w <= 0 ||
        d->out_h <= 0 || d->out_w <= 0 || d->pad_t < 0 || d->pad_l < 0 || !(d->out_scale > 0.f))
        return fail(ctx, ENN_B200_INVALID_PARAMS, "bad pool descriptor");
    enn_b200_op *op = new (std::nothrow) enn_b200_op();
    if (!op) return fail(ctx, ENN_B200_FAILURE, "out of host memory");
    op->ctx = ctx;
    op->kind = OP_AVGPOOL;
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

int32_t enn_b200_op_set_impl(enn_b200_op *op, int32_t impl) {
    if (!op) return ENN_B200_INVALID_PARAMS;
    if (op->kind == OP_CONV || op->kind == OP_FC || op->kind == OP_DECONV) {
        if (impl == ENN_B200_IMPL_DIRECT) {
            op->impl = impl;
        } else if ((impl == ENN_B200_IMPL_TCGEN05 || impl == ENN_B200_IMPL_GEMV) && op->tc) {
            // GEMV is the tensor-core plan's own choice for M <= 8; both names select that plan.
            op->impl = ENN_B200_IMPL_TCGEN05;
        } else {
            return fail(op->ctx, ENN_B200_INVALID_PARAMS, "kernel family not available for this op");
        }
        op->info.impl = op->impl;
        return ENN_B200_SUCCESS;
    }
    if (op->kind == OP_DEPTHWISE && (impl == ENN_B200_IMPL_DIRECT || impl == ENN_B200_IMPL_DEPTHWISE)) {
        // DIRECT selects the general kernel, DEPTHWISE the 3x3 fast path when the geometry has one.
        op->impl = impl;
        op->info.impl = impl;
        return ENN_B200_SUCCESS;
    }
    return impl == op->impl ? ENN_B200_SUCCESS : fail(op->ctx, ENN_B200_INVALID_PARAMS, "op has a single kernel family");
}

int32_t enn_b200_op_execute(enn_b200_op *op, const void *in, void *out) {
    if (!op) return ENN_B200_INVALID_PARAMS;
    enn_b200_context *ctx = op->ctx;
    if (!in || !out) return fail(ctx, ENN_B200_INVALID_PARAMS, "null device pointer");
    if (op->dyn && !op->dyn->bound) return fail(ctx, ENN_B200_FAILURE, "filter / bias are runtime tensors: call enn_b200_op_rebind_constants first");
    if (op->fused_add && op->impl != ENN_B200_IMPL_TCGEN05) return fail(ctx, ENN_B200_INVALID_PARAMS, "an operator with a fused add runs on the tensor-core path only");
    cudaError_t e = cudaSuccess;
    switch (op->kind) {
        case OP_CONV:
        case OP_FC:
            if (op->impl == ENN_B200_IMPL_TCGEN05) return tc_execute(op, in, out);
            e = launch_conv_direct(op->g, op->rq, in, op->w_direct, out, ctx->stream);
            break;
        case OP_DECONV:
            if (op->impl == ENN_B200_IMPL_TCGEN05) return tc_execute(op, in, out);
            e = launch_deconv_direct(op->g, op->rq, in, op->w_direct, out, ctx->stream);
            break;
        case OP_DEPTHWISE:
            if (op->dw_ring && op->impl == ENN_B200_IMPL_DEPTHWISE) {
                e = dw_ring_launch(op, in, out);
                if (e == cudaErrorLaunchFailure) return fail(ctx, ENN_B200_CUDA_FAILURE, "depthwise kernel gave up on a barrier wait earlier");
                if (e != cudaErrorNotSupported) break;
            }
            // The register-streamed kernel reads and writes 32-bit words: other alignments take the general kernel.
            if (op->dw_chan && op->impl == ENN_B200_IMPL_DEPTHWISE &&
                ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 3) == 0) {
                e = launch_dw3x3(op->g, op->dw_chan, op->dw_relu, op->dw_w, in, out, ctx->sm_count, ctx->stream);
                break;
            }
            e = launch_depthwise(op->g, op->rq, in, op->w_direct, out, ctx->sm_count, ctx->stream);
            break;
        case OP_AVGPOOL:
            e = launch_avgpool(op->pool, in, out, ctx->stream);
            break;
        case OP_MAXPOOL:
            e = launch_maxpool(op->pool, in, out, ctx->stream);
            break;
        case OP_MEAN:
        case OP_SOFTMAX:
        case OP_RESIZE:
            e = launch_graph_op(op, &in, 1, out);
            break;
        case OP_CONCAT:
            if (op->info.in_bytes != op->info.out_bytes || !op->graph_state) return fail(ctx, ENN_B200_FAILURE, "bad concat state");
            e = launch_graph_op(op, &in, 1, out);       // a one-input concatenation
            if (e == cudaErrorInvalidValue) return fail(ctx, ENN_B200_INVALID_PARAMS, "this concatenation needs enn_b200_op_execute_n");
            break;
        default:
            return fail(ctx, ENN_B200_INVALID_PARAMS, "op needs enn_b200_op_execute2");
    }
    if (e != cudaSuccess) return cuda_fail(ctx, e, "kernel launch");
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_op_execute2(enn_b200_op *op, const void *in0, const void *in1, void *out) {
    if (!op) return ENN_B200_INVALID_PARAMS;
    if (!in0 || !in1 || !out) return fail(op->ctx, ENN_B200_INVALID_PARAMS, "null device pointer");
    if (op->fused_add) {      // convolution + add: in0 feeds the convolution, in1 is the add's other input
        tc_set_residual(op, in1);
        return enn_b200_op_execute(op, in0, out);
    }
    if (op->kind != OP_ADD) return fail(op->ctx, ENN_B200_INVALID_PARAMS, "not a two-input op");
    cudaError_t e = launch_add(op->add, op->count, in0, in1, out, op->ctx->sm_count, op->ctx->stream);
    if (e != cudaSuccess) return cuda_fail(op->ctx, e, "add launch");
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_op_execute_n(enn_b200_op *op, const void *const *ins, int32_t n_in, void *out) {
    if (!op) return ENN_B200_INVALID_PARAMS;
    if (!ins || !out || n_in < 1) return fail(op->ctx, ENN_B200_INVALID_PARAMS, "null device pointer");
    for (int i = 0; i < n_in; ++i)
        if (!ins[i]) return fail(op->ctx, ENN_B200_INVALID_PARAMS, "null device pointer");
    if (op->kind == OP_CONCAT) {
        cudaError_t e = launch_graph_op(op, ins, n_in, out);
        if (e == cudaErrorInvalidValue) return fail(op->ctx, ENN_B200_INVALID_PARAMS, "wrong number of inputs for this concatenation");
        if (e != cudaSuccess) return cuda_fail(op->ctx, e, "concat launch");
        return ENN_B200_SUCCESS;
    }
    if (op->kind == OP_ADD || op->fused_add)
        return n_in == 2 ? enn_b200_op_execute2(op, ins[0], ins[1], out) : fail(op->ctx, ENN_B200_INVALID_PARAMS, "this operator takes two inputs");
    return n_in == 1 ? enn_b200_op_execute(op, ins[0], out) : fail(op->ctx, ENN_B200_INVALID_PARAMS, "this operator takes one input");
}

int32_t enn_b200_op_info(const enn_b200_op *op, enn_b200_op_info_t *info) {
    if (!op || !info) return ENN_B200_INVALID_PARAMS;
    *info = op->info;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_op_test_starve_next(enn_b200_op *op) {
    if (!op) return ENN_B200_INVALID_PARAMS;
    if (op->impl != ENN_B200_IMPL_TCGEN05 || !op->tc) return fail(op->ctx, ENN_B200_INVALID_PARAMS, "the self-test needs an operator on the tensor-core kernel");
    return tc_test_starve_next(op) == ENN_B200_SUCCESS ? ENN_B200_SUCCESS
                                                       : fail(op->ctx, ENN_B200_INVALID_PARAMS, "this plan has no starved form (GEMV, first layer or CTA pairs)");
}

int32_t enn_b200_op_clear_error(enn_b200_op *op) {
    if (!op) return ENN_B200_INVALID_PARAMS;
    if (op->tc) tc_clear_error(op);
    if (op->dw_ring) dw_ring_clear_error(op);
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_op_fuse_add(enn_b200_op *conv, enn_b200_op *add, int32_t conv_is_second_input) {
    if (!conv || !add || !conv->ctx) return ENN_B200_INVALID_PARAMS;
    enn_b200_context *ctx = conv->ctx;
    if (conv->kind != OP_CONV || add->kind != OP_ADD || add->ctx != ctx || conv->fused_add || conv->dyn || conv->impl != ENN_B200_IMPL_TCGEN05 ||
        !conv->tc || !add->add.lut || add->count != conv->info.out_bytes)
        return fail(ctx, ENN_B200_INVALID_PARAMS, "fuse_add: not a tensor-core convolution and an add over its output");
    const int32_t st = tc_fuse_add(conv, add->add, conv_is_second_input != 0);
    if (st != ENN_B200_SUCCESS) return fail(ctx, st, "fuse_add: this convolution's plan cannot take the add (mode, tiling or shared memory)");
    conv->fused_add = add;                // owned from here on: the table lives in its allocations
    conv->info.act_min = add->info.act_min;
    conv->info.act_max = add->info.act_max;
    conv->info.in_bytes += conv->info.out_bytes;
    conv->info.algorithmic_bytes += conv->info.out_bytes;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_op_rebind_constants(enn_b200_op *op, const void *weights_dev, const int32_t *bias_dev) {
    if (!op || !op->ctx) return ENN_B200_INVALID_PARAMS;
    enn_b200_context *ctx = op->ctx;
    if (!op->dyn) return fail(ctx, ENN_B200_INVALID_PARAMS, "operator was prepared with constant filter and bias");
    RuntimeConstants &dyn = *op->dyn;
    if ((dyn.weights && !weights_dev) || (dyn.bias && !bias_dev)) return fail(ctx, ENN_B200_INVALID_PARAMS, "null runtime tensor");
    ENN_CUDA(ctx, cudaSetDevice(ctx->device));
    if (dyn.weights) ENN_CUDA(ctx, cudaMemcpyAsync(dyn.w_host.data(), weights_dev, dyn.w_host.size(), cudaMemcpyDeviceToHost, ctx->stream));
    if (dyn.bias)
        ENN_CUDA(ctx, cudaMemcpyAsync(dyn.b_host.data(), bias_dev, dyn.b_host.size() * sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
    // Also orders the swap below after every launch of this operator that is still in flight on the stream.
    ENN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    enn_b200_op *fresh = nullptr;
    const int32_t st = conv_like_prepare_const(ctx, &dyn.desc, dyn.w_host.data(), dyn.b_host.data(),
                                               dyn.desc.per_channel ? dyn.scales.data() : nullptr, dyn.prepare_kind, &fresh);
    if (st != ENN_B200_SUCCESS) return st;
    fresh->kind = op->kind;                // FullyConnected keeps its kind
    fresh->dyn = std::move(op->dyn);
    fresh->dyn->bound = true;
    std::swap(*op, *fresh);
    enn_b200_op_release(fresh);            // the previous plan and its device constants
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_op_release(enn_b200_op *op) {
    if (!op) return ENN_B200_INVALID_PARAMS;
    if (op->ctx) cudaSetDevice(op->ctx->device);
    if (op->tc) tc_release(op);
    if (op->dw_ring) dw_ring_release(op);
    if (op->graph_state) graph_op_release(op);
    if (op->fused_add) enn_b200_op_release(op->fused_add);
    for (void *p : op->owned) cudaFree(p);
    delete op;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_nchw_to_nhwc(enn_b200_context *ctx, const void *src, void *dst, int32_t n, int32_t c, int32_t h, int32_t w) {
    if (!ctx || !src || !dst || n < 0 || c <= 0 || h <= 0 || w <= 0) return fail(ctx, ENN_B200_INVALID_PARAMS, "bad transpose arguments");
    cudaError_t e = launch_transpose_nchw_nhwc(src, dst, n, c, h, w, true, ctx->stream);
    return e == cudaSuccess ? ENN_B200_SUCCESS : cuda_fail(ctx, e, "transpose launch");
}

int32_t enn_b200_nhwc_to_nchw(enn_b200_context *ctx, const void *src, void *dst, int32_t n, int32_t c, int32_t h, int32_t w) {
    if (!ctx || !src || !dst || n < 0 || c <= 0 || h <= 0 || w <= 0) return fail(ctx, ENN_B200_INVALID_PARAMS, "bad transpose arguments");
    cudaError_t e = launch_transpose_nchw_nhwc(src, dst, n, c, h, w, false, ctx->stream);
    return e == cudaSuccess ? ENN_B200_SUCCESS : cuda_fail(ctx, e, "transpose launch");
}

}  // extern "C"
