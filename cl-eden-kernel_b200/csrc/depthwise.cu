// DepthwiseConv2D, NHWC.  Value: DepthwiseconvolutionKernels.cpp:1273-1371 after the zero-point `pad`
// pre-pass (border taps contribute nothing).  HBM-bound: no tensor cores.
#include "internal.h"
#include "requant.h"

namespace enn_b200 {

// General form: any kernel size, stride, dilation, depth multiplier, signedness.  One thread per
// (pixel, output channel), channel fastest.  Weights packed [Kh][Kw][Cout].
__global__ void depthwise_generic_kernel(ConvGeom g, Requant rq, const void *__restrict__ in,
                                         const void *__restrict__ w, uint8_t *__restrict__ out, int64_t total) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int32_t oc = static_cast<int32_t>(idx % g.cout);
    int64_t p = idx / g.cout;
    const int32_t ox = static_cast<int32_t>(p % g.ow);
    p /= g.ow;
    const int32_t oy = static_cast<int32_t>(p % g.oh);
    const int32_t b = static_cast<int32_t>(p / g.oh);
    const int32_t c = oc / g.groups;
    int32_t acc = rq.bias[oc];
    for (int32_t ky = 0; ky < g.kh; ++ky) {
        const int32_t iy = oy * g.sh + ky * g.dh - g.pt;
        if (iy < 0 || iy >= g.h) continue;
        for (int32_t kx = 0; kx < g.kw; ++kx) {
            const int32_t ix = ox * g.sw + kx * g.dw - g.pl;
            if (ix < 0 || ix >= g.w) continue;
            const int64_t ii = ((static_cast<int64_t>(b) * g.h + iy) * g.w + ix) * g.cin + c;
            const int64_t wi = (static_cast<int64_t>(ky) * g.kw + kx) * g.cout + oc;
            const int32_t a = g.a_signed ? static_cast<int32_t>(static_cast<const int8_t *>(in)[ii])
                                         : static_cast<int32_t>(static_cast<const uint8_t *>(in)[ii]);
            const int32_t wv = g.w_signed ? static_cast<int32_t>(static_cast<const int8_t *>(w)[wi])
                                          : static_cast<int32_t>(static_cast<const uint8_t *>(w)[wi]);
            acc += (a - g.in_zp) * (wv - g.w_zp);
        }
    }
    out[idx] = static_cast<uint8_t>(enn_requant(acc, rq.mult[oc], rq.shift[oc], g.out_zp, g.act_min, g.act_max));
}

cudaError_t launch_depthwise(const ConvGeom &g, const Requant &rq, const void *in, const void *w, void *out,
                             int sm_count, cudaStream_t s) {
    (void)sm_count;
    const int64_t total = static_cast<int64_t>(g.n) * g.oh * g.ow * g.cout;
    if (total == 0) return cudaSuccess;
    const int threads = 256;
    depthwise_generic_kernel<<<static_cast<unsigned>((total + threads - 1) / threads), threads, 0, s>>>(
        g, rq, in, w, static_cast<uint8_t *>(out), total);
    return cudaGetLastError();
}

}  // namespace enn_b200
