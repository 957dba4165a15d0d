// CUDA-core kernels that accept every geometry the reference operators accept (groups, dilation, stride,
// ragged sizes, signed or unsigned bytes).  They are the general path; the tensor-core implicit GEMM in
// gemm_tc.cu takes over the dense contractions it can tile.
#include "internal.h"
#include "requant.h"

namespace enn_b200 {

__device__ __forceinline__ int32_t load_byte(const void *p, int64_t i, int is_signed) {
    return is_signed ? static_cast<int32_t>(static_cast<const int8_t *>(p)[i])
                     : static_cast<int32_t>(static_cast<const uint8_t *>(p)[i]);
}

// One thread per (output pixel, output channel), channel fastest so that weight reads coalesce and the
// activation read is a warp broadcast.  Weights are packed [Kh][Kw][Cin/g][Cout].
// Value: ConvolutionKernels.cpp:1317-1375 (out-of-image taps contribute nothing).
__global__ void conv_direct_kernel(ConvGeom g, Requant rq, const void *__restrict__ in, const void *__restrict__ w,
                                   uint8_t *__restrict__ out, int64_t total) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int32_t oc = static_cast<int32_t>(idx % g.cout);
    int64_t p = idx / g.cout;
    const int32_t ox = static_cast<int32_t>(p % g.ow);
    p /= g.ow;
    const int32_t oy = static_cast<int32_t>(p % g.oh);
    const int32_t b = static_cast<int32_t>(p / g.oh);
    const int32_t grp = oc / g.cout_g;
    int32_t acc = 0;
    for (int32_t ky = 0; ky < g.kh; ++ky) {
        const int32_t iy = oy * g.sh + ky * g.dh - g.pt;
        if (iy < 0 || iy >= g.h) continue;
        for (int32_t kx = 0; kx < g.kw; ++kx) {
            const int32_t ix = ox * g.sw + kx * g.dw - g.pl;
            if (ix < 0 || ix >= g.w) continue;
            const int64_t ibase = ((static_cast<int64_t>(b) * g.h + iy) * g.w + ix) * g.cin + grp * g.cin_g;
            const int64_t wbase = (static_cast<int64_t>(ky) * g.kw + kx) * g.cin_g * g.cout + oc;
            for (int32_t ic = 0; ic < g.cin_g; ++ic) {
                const int32_t a = load_byte(in, ibase + ic, g.a_signed) - g.in_zp;
                const int32_t wv = load_byte(w, wbase + static_cast<int64_t>(ic) * g.cout, g.w_signed) - g.w_zp;
                acc += a * wv;
            }
        }
    }
    acc += rq.bias[oc];
    out[idx] = static_cast<uint8_t>(enn_requant(acc, rq.mult[oc], rq.shift[oc], g.out_zp, g.act_min, g.act_max));
}

cudaError_t launch_conv_direct(const ConvGeom &g, const Requant &rq, const void *in, const void *w, void *out,
                               cudaStream_t s) {
    const int64_t total = static_cast<int64_t>(g.n) * g.oh * g.ow * g.cout;
    if (total == 0) return cudaSuccess;
    const int threads = 256;
    const int64_t blocks = (total + threads - 1) / threads;
    conv_direct_kernel<<<static_cast<unsigned>(blocks), threads, 0, s>>>(g, rq, in, w, static_cast<uint8_t *>(out), total);
    return cudaGetLastError();
}

// Transposed convolution in gather form: DeconvolutionKernels.cpp:147-198 (the col2im index walk) with the
// GEMM of :24-145 folded in, so no int32 column buffer exists.  Weights packed [Kh][Kw][Cin][Cout].
__global__ void deconv_direct_kernel(ConvGeom g, Requant rq, const void *__restrict__ in, const void *__restrict__ w,
                                     uint8_t *__restrict__ out, int64_t total) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int32_t oc = static_cast<int32_t>(idx % g.cout);
    int64_t p = idx / g.cout;
    const int32_t ox = static_cast<int32_t>(p % g.ow);
    p /= g.ow;
    const int32_t oy = static_cast<int32_t>(p % g.oh);
    const int32_t b = static_cast<int32_t>(p / g.oh);
    const int32_t h_im = oy + g.pt, w_im = ox + g.pl;
    const int32_t wc0 = (w_im < g.kw) ? 0 : (w_im - g.kw) / g.sw + 1;
    const int32_t wc1 = min(w_im / g.sw + 1, g.w);
    const int32_t hc0 = (h_im < g.kh) ? 0 : (h_im - g.kh) / g.sh + 1;
    const int32_t hc1 = min(h_im / g.sh + 1, g.h);
    int32_t acc = 0;
    for (int32_t hc = hc0; hc < hc1; ++hc) {
        for (int32_t wc = wc0; wc < wc1; ++wc) {
            const int32_t ky = h_im - hc * g.sh, kx = w_im - wc * g.sw;
            const int64_t ibase = ((static_cast<int64_t>(b) * g.h + hc) * g.w + wc) * g.cin;
            const int64_t wbase = (static_cast<int64_t>(ky) * g.kw + kx) * g.cin * g.cout + oc;
            for (int32_t ic = 0; ic < g.cin; ++ic) {
                const int32_t a = load_byte(in, ibase + ic, g.a_signed) - g.in_zp;
                const int32_t wv = load_byte(w, wbase + static_cast<int64_t>(ic) * g.cout, g.w_signed) - g.w_zp;
                acc += a * wv;
            }
        }
    }
    acc += rq.bias[oc];
    out[idx] = static_cast<uint8_t>(enn_requant(acc, rq.mult[oc], rq.shift[oc], g.out_zp, g.act_min, g.act_max));
}

cudaError_t launch_deconv_direct(const ConvGeom &g, const Requant &rq, const void *in, const void *w, void *out,
                                 cudaStream_t s) {
    const int64_t total = static_cast<int64_t>(g.n) * g.oh * g.ow * g.cout;
    if (total == 0) return cudaSuccess;
    const int threads = 256;
    const int64_t blocks = (total + threads - 1) / threads;
    deconv_direct_kernel<<<static_cast<unsigned>(blocks), threads, 0, s>>>(g, rq, in, w, static_cast<uint8_t *>(out), total);
    return cudaGetLastError();
}

// Quantized add: AddKernelsQauntized.cpp:135-219 (left shift 20, three SRDHM + rounding-shift stages).
__global__ void add_kernel(AddParams p, int64_t count, const uint8_t *__restrict__ a, const uint8_t *__restrict__ b,
                           uint8_t *__restrict__ out) {
    pdl_wait();
    pdl_trigger();
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        const int32_t v0 = p.in0_off + load_byte(a, i, p.is_signed);
        const int32_t v1 = p.in1_off + load_byte(b, i, p.is_signed);
        const int32_t x0 = enn_rdivpot(enn_srdhm(v0 * (1 << 20), p.m0), -p.s0);
        const int32_t x1 = enn_rdivpot(enn_srdhm(v1 * (1 << 20), p.m1), -p.s1);
        int32_t o = enn_rdivpot(enn_srdhm(x0 + x1, p.mo), -p.so) + p.out_off;
        o = max(p.act_min, o);
        o = min(p.act_max, o);
        out[i] = static_cast<uint8_t>(o);
    }
}

// 16 bytes per thread per step; used when count and pointers allow.  The first two stages depend on one input byte
// each and come from the operator's tables (staged in shared memory); the last stage is computed.
__global__ void add_kernel_vec(AddParams p, int64_t count16, const uint4 *__restrict__ a, const uint4 *__restrict__ b,
                               uint4 *__restrict__ out) {
    __shared__ int32_t s_lut[512];
    for (int i = threadIdx.x; i < 512; i += blockDim.x) s_lut[i] = p.lut[i];      // operator constants, not a tensor
    __syncthreads();
    pdl_wait();
    pdl_trigger();
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count16; i += stride) {
        const uint4 va = a[i], vb = b[i];
        const uint32_t wa[4] = {va.x, va.y, va.z, va.w};
        const uint32_t wb[4] = {vb.x, vb.y, vb.z, vb.w};
        uint32_t wo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t r = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t ba = (wa[j] >> (8 * k)) & 0xff, bb = (wb[j] >> (8 * k)) & 0xff;
                const int32_t x0 = s_lut[ba], x1 = s_lut[256 + bb];
                int32_t o = enn_rdivpot(enn_srdhm(x0 + x1, p.mo), -p.so) + p.out_off;
                o = max(p.act_min, o);
                o = min(p.act_max, o);
                r |= (static_cast<uint32_t>(o) & 0xff) << (8 * k);
            }
            wo[j] = r;
        }
        out[i] = make_uint4(wo[0], wo[1], wo[2], wo[3]);
    }
}

// Large tensors: the operator's 64 KB pair table in shared memory, 16 bytes per thread per step, one byte lookup per
// output.  The table belongs to the operator, so it is staged before the wait on the kernel that produces the inputs.
constexpr int kAddLut2Threads = 256;
constexpr int64_t kAddLut2MinCount = 1 << 20;      // below this the table staging costs more than the arithmetic it saves

__global__ void __launch_bounds__(kAddLut2Threads) add_kernel_lut2(AddParams p, int64_t count16, const uint4 *__restrict__ a,
                                                                  const uint4 *__restrict__ b, uint4 *__restrict__ out) {
    extern __shared__ uint4 s_lut2_q[];
    const uint4 *src = reinterpret_cast<const uint4 *>(p.lut2);
    for (int i = threadIdx.x; i < 4096; i += blockDim.x) s_lut2_q[i] = __ldg(src + i);
    __syncthreads();
    pdl_wait();
    pdl_trigger();
    const uint8_t *lut = reinterpret_cast<const uint8_t *>(s_lut2_q);
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    auto combine = [&](const uint4 &va, const uint4 &vb) {
        const uint32_t wa[4] = {va.x, va.y, va.z, va.w};
        const uint32_t wb[4] = {vb.x, vb.y, vb.z, vb.w};
        uint32_t wo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                // (a byte k) << 8 | (b byte k): bytes {b.k, a.k, zero, zero}
                const uint32_t idx = __byte_perm(wb[j], wa[j], 0x7700u | (static_cast<uint32_t>(4 + k) << 4) | static_cast<uint32_t>(k)) & 0xffffu;
                o[k] = lut[idx ^ ((idx >> 6) & 0x7cu)];
            }
            wo[j] = o[0] | (o[1] << 8) | (o[2] << 16) | (o[3] << 24);
        }
        return make_uint4(wo[0], wo[1], wo[2], wo[3]);
    };
    // Two steps per iteration with all four loads issued first: the kernel waits on its global loads more than on anything else.
    int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + stride < count16; i += 2 * stride) {
        const uint4 va0 = a[i], vb0 = b[i], va1 = a[i + stride], vb1 = b[i + stride];
        out[i] = combine(va0, vb0);
        out[i + stride] = combine(va1, vb1);
    }
    if (i < count16) out[i] = combine(a[i], b[i]);
}

// Called once per prepared add operator (with its device current): the pair-table kernel needs 64 KB of dynamic shared memory.
cudaError_t add_kernel_init() {
    return cudaFuncSetAttribute(add_kernel_lut2, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
}

cudaError_t launch_add(const AddParams &p, int64_t count, const void *a, const void *b, void *out, int sm_count,
                       cudaStream_t s) {
    if (count == 0) return cudaSuccess;
    if (count >= kAddLut2MinCount && p.lut2 &&
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
        const int64_t n16 = count / 16;
        const int64_t want = (n16 + kAddLut2Threads * 4 - 1) / (kAddLut2Threads * 4);      // at least four steps per thread
        const int blocks = static_cast<int>(want < static_cast<int64_t>(sm_count) * 3 ? want : static_cast<int64_t>(sm_count) * 3);
        launch_pdl(add_kernel_lut2, dim3(blocks), dim3(kAddLut2Threads), 65536, s, p, n16, static_cast<const uint4 *>(a),
                   static_cast<const uint4 *>(b), static_cast<uint4 *>(out));
        const int64_t tail = count - n16 * 16;
        if (tail > 0)
            launch_pdl(add_kernel, dim3(1), dim3(32), 0, s, p, tail, static_cast<const uint8_t *>(a) + n16 * 16,
                       static_cast<const uint8_t *>(b) + n16 * 16, static_cast<uint8_t *>(out) + n16 * 16);
        return cudaGetLastError();
    }
    const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const int threads = 256;
    if (aligned && count >= 16) {
        const int64_t n16 = count / 16;
        const int64_t want = (n16 + threads - 1) / threads;
        const int blocks = static_cast<int>(want < static_cast<int64_t>(sm_count) * 8 ? want : static_cast<int64_t>(sm_count) * 8);
        launch_pdl(add_kernel_vec, dim3(blocks), dim3(threads), 0, s, p, n16, static_cast<const uint4 *>(a), static_cast<const uint4 *>(b),
                   static_cast<uint4 *>(out));
        const int64_t tail = count - n16 * 16;
        if (tail > 0) {
            launch_pdl(add_kernel, dim3(1), dim3(32), 0, s, p, tail, static_cast<const uint8_t *>(a) + n16 * 16,
                       static_cast<const uint8_t *>(b) + n16 * 16, static_cast<uint8_t *>(out) + n16 * 16);
        }
    } else {
        const int64_t want = (count + threads - 1) / threads;
        const int blocks = static_cast<int>(want < static_cast<int64_t>(sm_count) * 8 ? want : static_cast<int64_t>(sm_count) * 8);
        launch_pdl(add_kernel, dim3(blocks), dim3(threads), 0, s, p, count, static_cast<const uint8_t *>(a), static_cast<const uint8_t *>(b),
                   static_cast<uint8_t *>(out));
    }
    return cudaGetLastError();
}

// Average pool: AveragepoolKernels.cpp:8-54.  One thread per (pixel, channel), channel fastest (NHWC).
__global__ void avgpool_kernel(PoolGeom p, const void *__restrict__ in, uint8_t *__restrict__ out, int64_t total) {
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
    const int32_t pool = (ei - si) * (ej - sj);
    int32_t sum = 0;
    for (int32_t i = si; i < ei; ++i)
        for (int32_t j = sj; j < ej; ++j)
            sum += load_byte(in, ((static_cast<int64_t>(b) * p.h + i) * p.w + j) * p.c + c, p.is_signed);
    int32_t v = (sum + pool / 2) / pool;
    v = max(v, p.act_min);
    v = min(v, p.act_max);
    out[idx] = static_cast<uint8_t>(v);
}

// Four channels per thread (C % 4 == 0, windows of at most 256 taps): one 32-bit load per tap, the four byte sums kept
// as two words of two 16-bit lanes.  Signed bytes are flipped to unsigned on load and the bias taken out of the sum.
__global__ void avgpool_vec4_kernel(PoolGeom p, const uint32_t *__restrict__ in, uint32_t *__restrict__ out, int64_t total4) {
    pdl_wait();
    pdl_trigger();
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total4) return;
    const int32_t c4n = p.c >> 2;
    const int32_t c4 = static_cast<int32_t>(idx % c4n);
    int64_t q = idx / c4n;
    const int32_t ox = static_cast<int32_t>(q % p.ow);
    q /= p.ow;
    const int32_t oy = static_cast<int32_t>(q % p.oh);
    const int32_t b = static_cast<int32_t>(q / p.oh);
    int32_t si = oy * p.sh - p.pt, sj = ox * p.sw - p.pl;
    const int32_t ei = min(si + p.kh, p.h), ej = min(sj + p.kw, p.w);
    si = max(si, 0);
    sj = max(sj, 0);
    const int32_t pool = (ei - si) * (ej - sj);
    const uint32_t flip = p.is_signed ? 0x80808080u : 0u;
    uint32_t even = 0, odd = 0;          // bytes 0, 2 and bytes 1, 3 as 16-bit lanes
    for (int32_t i = si; i < ei; ++i) {
        const uint32_t *row = in + (static_cast<int64_t>(b) * p.h + i) * p.w * c4n + c4;
#pragma unroll 7
        for (int32_t j = sj; j < ej; ++j) {
            const uint32_t v = __ldg(row + static_cast<int64_t>(j) * c4n) ^ flip;
            even += v & 0x00ff00ffu;
            odd += (v >> 8) & 0x00ff00ffu;
        }
    }
    const int32_t bias = p.is_signed ? 128 * pool : 0;
    const int32_t sums[4] = {static_cast<int32_t>(even & 0xffff) - bias, static_cast<int32_t>(odd & 0xffff) - bias,
                             static_cast<int32_t>(even >> 16) - bias, static_cast<int32_t>(odd >> 16) - bias};
    uint32_t r = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        int32_t v = (sums[k] + pool / 2) / pool;
        v = max(v, p.act_min);
        v = min(v, p.act_max);
        r |= (static_cast<uint32_t>(v) & 0xff) << (8 * k);
    }
    out[idx] = r;
}

cudaError_t launch_avgpool(const PoolGeom &p, const void *in, void *out, cudaStream_t s) {
    const int64_t total = static_cast<int64_t>(p.n) * p.oh * p.ow * p.c;
    if (total == 0) return cudaSuccess;
    const int threads = 256;
    if ((p.c & 3) == 0 && p.kh * p.kw <= 256 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 3) == 0) {
        const int64_t total4 = total / 4;
        const int th = 128;
        launch_pdl(avgpool_vec4_kernel, dim3(static_cast<unsigned>((total4 + th - 1) / th)), dim3(th), 0, s, p,
                   static_cast<const uint32_t *>(in), static_cast<uint32_t *>(out), total4);
        return cudaGetLastError();
    }
    launch_pdl(avgpool_kernel, dim3(static_cast<unsigned>((total + threads - 1) / threads)), dim3(threads), 0, s, p, in,
               static_cast<uint8_t *>(out), total);
    return cudaGetLastError();
}

// NCHW <-> NHWC for one-byte elements: CLRuntime.cpp:1477-1620.  Tiled through shared memory so both
// sides are coalesced.  Grid: (ceil(HW/32), ceil(C/32), N).
__global__ void transpose_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int rows, int cols) {
    // src viewed as [batch][rows][cols] -> dst [batch][cols][rows]
    __shared__ uint8_t tile[32][33];
    const int64_t base = static_cast<int64_t>(blockIdx.z) * rows * cols;
    int r = blockIdx.y * 32 + threadIdx.y, c = blockIdx.x * 32 + threadIdx.x;
    if (r < rows && c < cols) tile[threadIdx.y][threadIdx.x] = src[base + static_cast<int64_t>(r) * cols + c];
    __syncthreads();
    c = blockIdx.x * 32 + threadIdx.y;
    r = blockIdx.y * 32 + threadIdx.x;
    if (r < rows && c < cols) dst[base + static_cast<int64_t>(c) * rows + r] = tile[threadIdx.x][threadIdx.y];
}

cudaError_t launch_transpose_nchw_nhwc(const void *src, void *dst, int n, int c, int h, int w, bool to_nhwc,
                                       cudaStream_t s) {
    if (n == 0 || c == 0 || h * w == 0) return cudaSuccess;
    const int rows = to_nhwc ? c : h * w;   // NCHW -> NHWC: [C][HW] -> [HW][C]
    const int cols = to_nhwc ? h * w : c;
    dim3 block(32, 32), grid((cols + 31) / 32, (rows + 31) / 32, n);
    transpose_kernel<<<grid, block, 0, s>>>(static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst), rows, cols);
    return cudaGetLastError();
}

}  // namespace enn_b200
