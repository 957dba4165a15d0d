// DepthwiseConv2D, NHWC.  Value: DepthwiseconvolutionKernels.cpp:1273-1371 after the zero-point `pad`
// pre-pass (border taps contribute nothing).  HBM-bound: no tensor cores.
//
// Two kernels:
//   depthwise_generic_kernel  any kernel size / stride / dilation / depth multiplier / signedness;
//   dw3x3_kernel              3x3, stride 1 or 2, dilation 1, multiplier 1, C % 4 == 0, u8 activations: the
//                             case every reference 3x3 variant (depthwise_conv_3x3s1_pad_merge, ..3x3s2..,
//                             depthwise_conv_per_channel) covers and the one the benchmark configuration uses.
#include <cuda.h>

#include <cstdlib>
#include <new>

#include "internal.h"
#include "requant.h"

namespace enn_b200 {

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
    // channels past cin * multiplier carry zero-point weights (prepare): any valid input channel will do
    const int32_t c = min(oc / g.groups, g.cin - 1);
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

// ------------------------------------------------------------------------------------------------------
// 3x3 fast path.
//
// A thread owns 4 channels (one 32-bit word of an NHWC pixel) x a strip of 4 output pixels along W and walks
// down TH output rows.  Each input row of the strip (6 pixels for stride 1, 9 for stride 2) is read once,
// byte-transposed with PRMT so that one register holds 4 consecutive pixels of ONE channel, and kept in a
// ring of three rows.  A 3-tap row product is then one dp4a against a packed weight word (w0,w1,w2,0) or
// (0,w0,w1,w2): 12 dp4a + 4 PRMT replace 36 multiply-adds per channel and output row.
//
// Zero points: the border is filled with the input zero point (what the reference's `pad` kernel writes), so
//   sum (a - za)(w - zw) = sum a*w - zw * sum a - za * sum w + 9 za zw
// with the last two terms folded into the bias at prepare time.  Per-channel int8 filters have zw == 0; the
// u8 per-tensor case carries `sum a` in a second dp4a chain (NEED_ASUM).
//
// Requantisation per output: one 32x32->64 multiply-add (stage 1), one funnel shift, and stage 2 written as
//   (x + 2^(e-1) + (zo << e) - [x < 0 and e > 0]) >> e
// which equals RoundingDivideByPOT(x, e) + zo (ties away from zero); prepare checks that it cannot overflow.
// ------------------------------------------------------------------------------------------------------
struct DwChan {   // per-channel constants, 16 bytes
    int32_t mult;
    int32_t addend;   // 2^(e-1) + (out_zp << e), e = right shift
    int32_t e;        // right shift | (sign shift << 8): sign shift is 31 when e > 0 else 32
    int32_t bias;     // bias - za * sum(w) + 9 * za * zw
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
template <bool W_SIGNED>
__device__ __forceinline__ int32_t dp4a_us(uint32_t a, uint32_t b, int32_t c) {
    int32_t d;
    if (W_SIGNED)
        asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    else
        asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t shr_clamp(uint32_t a, uint32_t s) {   // PTX shr clamps s >= 32 to 0 result
    uint32_t d;
    asm("shr.u32 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(s));
    return d;
}
__device__ __forceinline__ uint32_t pack_sat_u8(int32_t hi, int32_t lo, uint32_t upper) {
    uint32_t d;   // d = { upper[15:0], sat_u8(hi), sat_u8(lo) }
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(hi), "r"(lo), "r"(upper));
    return d;
}

// Transposed input row for 4 channels: lo[c] holds the first four pixels of channel c's window, hi[c] the
// four pixels starting two (stride 1) or four (stride 2) positions later, x8[c] (stride 2) positions 6,7,8.
template <int STRIDE>
struct DwRow {
    uint32_t lo[4], hi[4], x8[STRIDE == 2 ? 4 : 1];
};

template <int STRIDE>
struct DwRaw {
    uint32_t p[STRIDE == 1 ? 6 : 9];
};

// Issues the global loads of one input row of the strip (border positions read as the input zero point).
// `colp` points at (batch b, row 0, pixel ix0, channel quad) and `colmask` has bit i set when pixel ix0+i lies
// inside the image, so the per-row work is one row offset and predicated loads.
template <int STRIDE>
__device__ __forceinline__ void dw_issue_row(DwRaw<STRIDE> &raw, const uint8_t *__restrict__ colp, uint32_t row_pitch,
                                             uint32_t cin, int h, int iy, uint32_t colmask, uint32_t zaw) {
    constexpr int NP = STRIDE == 1 ? 6 : 9;
    const bool row_ok = iy >= 0 && iy < h;
    const uint8_t *rowp = colp + static_cast<uint32_t>(row_ok ? iy : 0) * row_pitch;
    const uint32_t m = row_ok ? colmask : 0u;
#pragma unroll
    for (int i = 0; i < NP; ++i) {
        raw.p[i] = zaw;
        if (m & (1u << i)) raw.p[i] = __ldg(reinterpret_cast<const uint32_t *>(rowp + static_cast<uint32_t>(i) * cin));
    }
}

// 4x4 byte transposes: pixel-major words -> channel-major words.
template <int STRIDE>
__device__ __forceinline__ void dw_transpose_row(DwRow<STRIDE> &r, const DwRaw<STRIDE> &raw) {
    constexpr int NP = STRIDE == 1 ? 6 : 9;
    const uint32_t *p = raw.p;
    {
        const uint32_t t0 = prmt(p[0], p[1], 0x5140), t1 = prmt(p[0], p[1], 0x7362);
        const uint32_t t2 = prmt(p[2], p[3], 0x5140), t3 = prmt(p[2], p[3], 0x7362);
        r.lo[0] = prmt(t0, t2, 0x5410); r.lo[1] = prmt(t0, t2, 0x7632);
        r.lo[2] = prmt(t1, t3, 0x5410); r.lo[3] = prmt(t1, t3, 0x7632);
    }
    if (STRIDE == 1) {
        // hi = pixels 2..5 (its first two intermediate words are the second two of lo; the compiler merges them)
        const uint32_t t0 = prmt(p[2], p[3], 0x5140), t1 = prmt(p[2], p[3], 0x7362);
        const uint32_t t2 = prmt(p[4], p[5], 0x5140), t3 = prmt(p[4], p[5], 0x7362);
        r.hi[0] = prmt(t0, t2, 0x5410); r.hi[1] = prmt(t0, t2, 0x7632);
        r.hi[2] = prmt(t1, t3, 0x5410); r.hi[3] = prmt(t1, t3, 0x7632);
    } else {
        // hi = pixels 4..7, x8 = pixels 6,7,8 (bytes 2,3 of hi and the channel byte of pixel 8)
        const uint32_t t0 = prmt(p[4], p[5], 0x5140), t1 = prmt(p[4], p[5], 0x7362);
        const uint32_t t2 = prmt(p[6], p[7], 0x5140), t3 = prmt(p[6], p[7], 0x7362);
        r.hi[0] = prmt(t0, t2, 0x5410); r.hi[1] = prmt(t0, t2, 0x7632);
        r.hi[2] = prmt(t1, t3, 0x5410); r.hi[3] = prmt(t1, t3, 0x7632);
        const uint32_t q = p[NP - 1];
        r.x8[0] = prmt(r.hi[0], q, 0x0432); r.x8[1] = prmt(r.hi[1], q, 0x0532);
        r.x8[2] = prmt(r.hi[2], q, 0x0632); r.x8[3] = prmt(r.hi[3], q, 0x0732);
    }
}

// 128-thread blocks, four per SM (16 warps at the 128-register budget the kernel needs to stay spill-free). Five
// blocks at 96 registers spill and lose more in a chain of layers than the extra warps gain; 256-thread blocks at
// the same occupancy drain more slowly before the next layer's GEMM CTA, which needs the whole SM, can start.
constexpr int kDwThreads = 128;

template <int STRIDE, bool W_SIGNED, bool NEED_ASUM, bool FIRST>
__device__ __forceinline__ void dw_accumulate(int32_t (&acc)[4][4], int32_t (&asum)[NEED_ASUM ? 4 : 1][4],
                                              const DwRow<STRIDE> &r, const uint32_t (&wlo)[4], const uint32_t (&whi)[4],
                                              const int32_t (&bias)[4]) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        if (FIRST) {   // the first tap row starts every chain from the folded bias: no separate initialisation
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc[c][j] = bias[c];
                if (NEED_ASUM) asum[c][j] = 0;
            }
        }
        if (STRIDE == 1) {
            acc[c][0] = dp4a_us<W_SIGNED>(r.lo[c], wlo[c], acc[c][0]);
            acc[c][1] = dp4a_us<W_SIGNED>(r.lo[c], whi[c], acc[c][1]);
            acc[c][2] = dp4a_us<W_SIGNED>(r.hi[c], wlo[c], acc[c][2]);
            acc[c][3] = dp4a_us<W_SIGNED>(r.hi[c], whi[c], acc[c][3]);
            if (NEED_ASUM) {
                asum[c][0] = dp4a_us<false>(r.lo[c], 0x00010101u, asum[c][0]);
                asum[c][1] = dp4a_us<false>(r.lo[c], 0x01010100u, asum[c][1]);
                asum[c][2] = dp4a_us<false>(r.hi[c], 0x00010101u, asum[c][2]);
                asum[c][3] = dp4a_us<false>(r.hi[c], 0x01010100u, asum[c][3]);
            }
        } else {
            // outputs use window positions {0,1,2}, {2,3,4}, {4,5,6}, {6,7,8}
            const uint32_t mid = prmt(r.lo[c], r.hi[c], 0x0432);   // positions 2,3,4
            acc[c][0] = dp4a_us<W_SIGNED>(r.lo[c], wlo[c], acc[c][0]);
            acc[c][1] = dp4a_us<W_SIGNED>(mid, wlo[c], acc[c][1]);
            acc[c][2] = dp4a_us<W_SIGNED>(r.hi[c], wlo[c], acc[c][2]);
            acc[c][3] = dp4a_us<W_SIGNED>(r.x8[c], wlo[c], acc[c][3]);
            if (NEED_ASUM) {
                asum[c][0] = dp4a_us<false>(r.lo[c], 0x00010101u, asum[c][0]);
                asum[c][1] = dp4a_us<false>(mid, 0x00010101u, asum[c][1]);
                asum[c][2] = dp4a_us<false>(r.hi[c], 0x00010101u, asum[c][2]);
                asum[c][3] = dp4a_us<false>(r.x8[c], 0x00010101u, asum[c][3]);
            }
        }
    }
}

// w_packed: [C][3] words, bytes (w[ky][0], w[ky][1], w[ky][2], 0) of channel c.
// The lower clamp is folded into the stage-2 addend (addend -= act_min << e), so the epilogue clamps
// (v - act_min) to [0, act_max - act_min] with one min-with-relu and adds act_min back per packed word.
// RELU: the operator's lower clamp equals its output zero point and every channel shifts right by e >= 1: the tie
// correction cannot change a clamped result, so bias and both rounding terms fold into one 64-bit addend per channel,
// q = acc * M0 + C with C = bias * M0 + 2^30 + 2^(30+e), result = hi32(q) >> (e - 1); DwChan then holds
// {C low, C high, M0, e - 1}.
template <int STRIDE, bool W_SIGNED, bool NEED_ASUM, bool RELU>
__global__ void __launch_bounds__(kDwThreads, 4)
dw3x3_kernel(ConvGeom g, const DwChan *__restrict__ chan, const uint32_t *__restrict__ w_packed,
             const uint8_t *__restrict__ in, uint8_t *__restrict__ out, int th, int nyt, int nstrip, int64_t total) {
    pdl_trigger();
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (tid >= total) return;
    const int cqn = g.cin >> 2;
    const int cq = static_cast<int>(tid % cqn);
    int64_t t = tid / cqn;
    const int strip = static_cast<int>(t % nstrip);
    t /= nstrip;
    const int yt = static_cast<int>(t % nyt);
    const int b = static_cast<int>(t / nyt);

    uint32_t wlo[3][4], whi[3][4];
    int32_t mult[4], addend[4], esh[4], bias[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const DwChan ch = chan[cq * 4 + c];
        if (RELU) {
            mult[c] = ch.e; addend[c] = ch.mult; esh[c] = ch.bias; bias[c] = ch.addend;    // M0, C low, e - 1, C high
        } else {
            mult[c] = ch.mult; addend[c] = ch.addend; esh[c] = ch.e; bias[c] = ch.bias;
        }
#pragma unroll
        for (int ky = 0; ky < 3; ++ky) {
            wlo[ky][c] = w_packed[(cq * 4 + c) * 3 + ky];
            whi[ky][c] = wlo[ky][c] << 8;
        }
    }
    const uint32_t zaw = (static_cast<uint32_t>(g.in_zp) & 0xff) * 0x01010101u;
    const int ox0 = strip * 4;
    const int ix0 = ox0 * STRIDE - g.pl;
    const int oy0 = yt * th;
    const int oy1 = min(oy0 + th, g.oh);
    const int h = g.h;
    const uint32_t cin = static_cast<uint32_t>(g.cin);
    const uint32_t row_pitch = static_cast<uint32_t>(g.w) * cin;
    constexpr int NP = STRIDE == 1 ? 6 : 9;
    uint32_t colmask = 0;
#pragma unroll
    for (int i = 0; i < NP; ++i)
        if (ix0 + i >= 0 && ix0 + i < g.w) colmask |= 1u << i;
    // Pointer to (b, row 0, pixel ix0, quad cq); ix0 may be negative, masked loads never touch those bytes.
    const uint8_t *colp = in + (static_cast<int64_t>(b) * h * g.w + ix0) * static_cast<int64_t>(cin) + cq * 4;
    const int32_t hi_clamp = g.act_max - g.act_min;
    const uint32_t lo_word = (static_cast<uint32_t>(g.act_min) & 0xff) * 0x01010101u;
    const uint32_t cout = static_cast<uint32_t>(g.cout);
    uint8_t *orow = out + ((static_cast<int64_t>(b) * g.oh + oy0) * g.ow + ox0) * static_cast<int64_t>(cout) + cq * 4;
    const uint32_t out_pitch = static_cast<uint32_t>(g.ow) * cout;
    uint32_t omask = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (ox0 + j < g.ow) omask |= 1u << j;

    const int32_t zero4[4] = {0, 0, 0, 0};
    // One output row: accumulate three input rows, requantise, store 4 pixels x 4 channels.
    auto emit = [&](const DwRow<STRIDE> &r0, const DwRow<STRIDE> &r1, const DwRow<STRIDE> &r2) {
        int32_t acc[4][4];
        int32_t asum[NEED_ASUM ? 4 : 1][4];
        if constexpr (RELU) dw_accumulate<STRIDE, W_SIGNED, NEED_ASUM, true>(acc, asum, r0, wlo[0], whi[0], zero4);
        else dw_accumulate<STRIDE, W_SIGNED, NEED_ASUM, true>(acc, asum, r0, wlo[0], whi[0], bias);
        dw_accumulate<STRIDE, W_SIGNED, NEED_ASUM, false>(acc, asum, r1, wlo[1], whi[1], bias);
        dw_accumulate<STRIDE, W_SIGNED, NEED_ASUM, false>(acc, asum, r2, wlo[2], whi[2], bias);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int32_t y[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                int32_t a = acc[c][j];
                if (NEED_ASUM) a -= g.w_zp * asum[c][j];
                int32_t v;
                if (RELU) {
                    int64_t cc;
                    asm("mov.b64 %0, {%1, %2};" : "=l"(cc) : "r"(addend[c]), "r"(bias[c]));
                    const int64_t q = static_cast<int64_t>(a) * mult[c] + cc;
                    v = static_cast<int32_t>(q >> 32) >> esh[c];
                } else {
                    const int64_t p = static_cast<int64_t>(a) * mult[c] + (1ll << 30);
                    const int32_t x = static_cast<int32_t>(p >> 31);
                    v = (x + addend[c] - static_cast<int32_t>(shr_clamp(static_cast<uint32_t>(x), esh[c] >> 8))) >> (esh[c] & 0xff);
                }
                y[c] = __vimin_s32_relu(v, hi_clamp);
            }
            if (omask & (1u << j)) {
                const uint32_t hi = pack_sat_u8(y[3], y[2], 0);
                *reinterpret_cast<uint32_t *>(orow + static_cast<uint32_t>(j) * cout) = pack_sat_u8(y[1], y[0], hi) + lo_word;
            }
        }
        orow += out_pitch;
    };

    // Everything above read only the operator's own constants (weights, per-channel words) and overlaps the tail of the
    // kernel before this one; its tensors are complete from here on.
    pdl_wait();
    // Ring of three transposed rows; the loop is unrolled over the ring so no register copies are needed.
    // The raw loads of the next input row(s) are issued before the current output row is computed, so
    // their latency overlaps the dp4a / requantisation work.
    DwRow<STRIDE> ra, rb, rc;
    const int iy0 = oy0 * STRIDE - g.pt;
    {
        DwRaw<STRIDE> r0;
        dw_issue_row<STRIDE>(r0, colp, row_pitch, cin, h, iy0, colmask, zaw);
        dw_transpose_row<STRIDE>(ra, r0);
    }
    if constexpr (STRIDE == 1) {
        DwRaw<STRIDE> nx;
        dw_issue_row<STRIDE>(nx, colp, row_pitch, cin, h, iy0 + 1, colmask, zaw);
        dw_transpose_row<STRIDE>(rb, nx);
        dw_issue_row<STRIDE>(nx, colp, row_pitch, cin, h, iy0 + 2, colmask, zaw);
        for (int oy = oy0; oy < oy1; oy += 3) {
            const int iy = oy - g.pt;
            dw_transpose_row<STRIDE>(rc, nx);
            dw_issue_row<STRIDE>(nx, colp, row_pitch, cin, h, iy + 3, colmask, zaw);
            emit(ra, rb, rc);
            if (oy + 1 < oy1) {
                dw_transpose_row<STRIDE>(ra, nx);
                dw_issue_row<STRIDE>(nx, colp, row_pitch, cin, h, iy + 4, colmask, zaw);
                emit(rb, rc, ra);
            }
            if (oy + 2 < oy1) {
                dw_transpose_row<STRIDE>(rb, nx);
                dw_issue_row<STRIDE>(nx, colp, row_pitch, cin, h, iy + 5, colmask, zaw);
                emit(rc, ra, rb);
            }
        }
    } else {
        DwRaw<STRIDE> n1, n2;
        dw_issue_row<STRIDE>(n1, colp, row_pitch, cin, h, iy0 + 1, colmask, zaw);
        dw_issue_row<STRIDE>(n2, colp, row_pitch, cin, h, iy0 + 2, colmask, zaw);
        for (int oy = oy0; oy < oy1; oy += 2) {
            const int iy = oy * 2 - g.pt;
            dw_transpose_row<STRIDE>(rb, n1);
            dw_transpose_row<STRIDE>(rc, n2);
            dw_issue_row<STRIDE>(n1, colp, row_pitch, cin, h, iy + 3, colmask, zaw);
            dw_issue_row<STRIDE>(n2, colp, row_pitch, cin, h, iy + 4, colmask, zaw);
            emit(ra, rb, rc);
            if (oy + 1 < oy1) {
                dw_transpose_row<STRIDE>(rb, n1);
                dw_transpose_row<STRIDE>(ra, n2);
                dw_issue_row<STRIDE>(n1, colp, row_pitch, cin, h, iy + 5, colmask, zaw);
                dw_issue_row<STRIDE>(n2, colp, row_pitch, cin, h, iy + 6, colmask, zaw);
                emit(rc, rb, ra);
            }
        }
    }
}

__device__ __forceinline__ uint32_t dw_smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ uint32_t dw_lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// ------------------------------------------------------------------------------------------------------
// 3x3 fast path, row-ring form (C % 16 == 0, at most 256 channel quads; above 224 as one CTA of eight consumer warps per
// SM instead of two of seven): the default for the MobileNetV2-style layers.
//
// The register-streamed kernel above keeps about 12 KB of loads in flight per SM, a third of what the HBM latency
// needs, and spends instructions on per-load predicates and addresses.  Here the input reaches shared memory through
// the bulk-copy engine instead: a CTA owns one x tile (4 * ns output columns, all C channels) and a contiguous range
// of output rows; a producer thread streams the input rows of that tile into a ring of row slots with one
// `cp.async.bulk` per row (the (4 ns - 1) s + 3 pixels of a row are contiguous in NHWC because the tile spans all
// channels), up to the whole ring ahead of the consumers, so tens of KB per SM are in flight whatever the register
// budget.  Consumer threads (4 channels x 4 output pixels each, as above) wait on the slot's mbarrier, read their six
// (stride 1) or nine (stride 2) words with shared-memory loads at fixed offsets, release the slot as soon as the row
// sits transposed in registers, and run the same dp4a / fused requantisation code.  No border predicate is left in
// the loop: pixels left and right of the image are slot positions that no copy ever writes and that hold the input
// zero point from the start (a CTA keeps its x tile for its whole life), rows above and below the image are read
// from a constant row of zero points.
// Every wait is bounded; a thread that gives up records a code, raises the CTA's abort flag and all roles leave.
// ------------------------------------------------------------------------------------------------------
struct DwRingParams {
    int32_t n, h, w, c, oh, ow, pt, pl;
    int32_t q;              // channel quads per pixel (C / 4)
    int32_t ns;             // strips of 4 output columns per x tile
    int32_t tx_n;           // x tiles per row
    int32_t ctas_per_tx;    // CTAs that share the rows of one x tile (grid = tx_n * ctas_per_tx)
    int32_t slot_px;        // pixels per ring slot: (4 ns - 1) s + 3
    int32_t nr;             // ring slots
    uint32_t pitch;         // bytes per slot (multiple of 128)
    int32_t in_zp, w_zp, act_min, act_max;
    const uint8_t *zrow;    // one slot's worth of input zero points in global memory (source of the rows outside the image)
    int32_t *err;           // host-mapped error word
};

constexpr int kDwRingConsumers = 224;                   // consumer threads per CTA (7 warps): two CTAs per SM
constexpr int kDwRingThreads = kDwRingConsumers + 32;   // + the producer warp
constexpr int kDwRingConsumersBig = 256;                // layers with 225-256 channel quads (960 channels): 8 consumer warps, one CTA per SM
constexpr int kDwRingThreadsBig = kDwRingConsumersBig + 32;
constexpr uint32_t kDwSpinLimit = 1u << 22;

__device__ __forceinline__ bool dw_mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait; false after the limit or once another thread has raised the abort flag.
__device__ __forceinline__ bool dw_mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int32_t *err, int code) {
    for (uint32_t i = 0; i < kDwSpinLimit; ++i) {
        if (dw_mbar_try(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    if (err) *reinterpret_cast<volatile int32_t *>(err) = code;
    return false;
}

// RQ: 0 two-stage requantisation, 1 merged ReLU form, 2 merged ReLU form whose clamp is the saturation of the byte pack
// itself (lower clamp 0, upper clamp 255: no min / max and no offset to add back).
template <int STRIDE, bool W_SIGNED, bool NEED_ASUM, int RQ, bool BIG = false>
__global__ void __launch_bounds__(BIG ? kDwRingThreadsBig : kDwRingThreads, BIG ? 1 : 2)
dw3x3_ring_kernel(const DwRingParams p, const DwChan *__restrict__ chan, const uint32_t *__restrict__ w_packed,
                  const uint8_t *__restrict__ in, uint8_t *__restrict__ out) {
    extern __shared__ uint8_t dw_ring_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(dw_ring_raw) + 127) & ~static_cast<uintptr_t>(127));
    constexpr int NP = STRIDE == 1 ? 6 : 9;
    constexpr bool RELU = RQ != 0;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ncw = (static_cast<int>(blockDim.x) >> 5) - 1;        // consumer warps; the last warp produces
    const uint32_t ring = dw_smem_u32(smem);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + static_cast<size_t>(p.nr) * p.pitch);
    const uint32_t full0 = dw_smem_u32(bars), empty0 = full0 + 8u * p.nr;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 2 * p.nr);
    pdl_trigger();
    if (tid == 0) {
        for (int i = 0; i < p.nr; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full0 + 8 * i) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty0 + 8 * i), "r"(ncw) : "memory");
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    {   // every slot starts as zero points; the copies overwrite the in-image pixel range only
        const uint32_t zaw = (static_cast<uint32_t>(p.in_zp) & 0xff) * 0x01010101u;
        const uint32_t n16 = static_cast<uint32_t>(p.nr) * (p.pitch >> 4);
        for (uint32_t i = tid; i < n16; i += blockDim.x)
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(ring + i * 16), "r"(zaw) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // ordered before the bulk copies into the same bytes
    }
    __syncthreads();

    // This CTA: x tile `tx`, output rows [u0, u1) of the N * OH rows of that tile column (row u = image * OH + oy).
    const int tx = static_cast<int>(blockIdx.x) / p.ctas_per_tx, part = static_cast<int>(blockIdx.x) - tx * p.ctas_per_tx;
    const int64_t units = static_cast<int64_t>(p.n) * p.oh;
    const int u0 = static_cast<int>(units * part / p.ctas_per_tx), u1 = static_cast<int>(units * (part + 1) / p.ctas_per_tx);
    const int ox0 = tx * p.ns * 4;
    const int ix_start = ox0 * STRIDE - p.pl;
    const int ix_lo = ix_start < 0 ? 0 : ix_start;
    const int ix_hi = ix_start + p.slot_px < p.w ? ix_start + p.slot_px : p.w;

    if (warp == ncw) {
        // ---------------- producer: one bulk copy per input row, in the order the consumers take them ----------------
        // Rows above and below the image are copied from a row of zero points in global memory, so that the consumers
        // treat every row alike.
        if (lane == 0 && ix_hi > ix_lo) {
            pdl_wait();         // the input tensor is complete from here on
            const uint32_t bytes = static_cast<uint32_t>(ix_hi - ix_lo) * p.c;
            const uint32_t dst_off = static_cast<uint32_t>(ix_lo - ix_start) * p.c;
            const int64_t row_bytes = static_cast<int64_t>(p.w) * p.c;
            uint32_t slot = 0, phase = 0;
            bool ok = true;
            for (int u = u0; u < u1 && ok;) {
                const int img = u / p.oh, oy0 = u - img * p.oh;
                const int cnt = min(p.oh - oy0, u1 - u);
                const int iy_a = oy0 * STRIDE - p.pt, iy_b = (oy0 + cnt - 1) * STRIDE - p.pt + 2;
                const uint8_t *img_base = in + static_cast<int64_t>(img) * p.h * row_bytes + static_cast<int64_t>(ix_lo) * p.c;
                for (int iy = iy_a; iy <= iy_b; ++iy) {
                    const uint8_t *src = static_cast<unsigned>(iy) < static_cast<unsigned>(p.h) ? img_base + iy * row_bytes : p.zrow;
                    if (!dw_mbar_try(empty0 + 8 * slot, phase ^ 1) && !dw_mbar_wait(empty0 + 8 * slot, phase ^ 1, abort_flag, p.err, 11)) { ok = false; break; }
                    const uint32_t bar = full0 + 8 * slot;
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(ring + slot * p.pitch + dst_off), "l"(src), "r"(bytes), "r"(bar) : "memory");
                    if (++slot == static_cast<uint32_t>(p.nr)) { slot = 0; phase ^= 1; }
                }
                u += cnt;
            }
            if (!ok) {      // copies still in flight get a bounded chance to land before the shared memory is given back
                for (int s2 = 0; s2 < p.nr; ++s2)
                    for (uint32_t i = 0; i < (1u << 16); ++i)
                        if (dw_mbar_try(full0 + 8 * s2, 0) || dw_mbar_try(full0 + 8 * s2, 1)) break;
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int nthr = p.ns * p.q;                      // real tasks; the last warp's surplus lanes shadow the last task
    const int task = tid < nthr ? tid : nthr - 1;
    const int strip = task / p.q, cq = task - strip * p.q;
    uint32_t wlo[3][4], whi[STRIDE == 1 ? 3 : 1][4];
    int32_t mult[4], esh[4];
    int32_t addend[RELU ? 1 : 4], bias[RELU ? 1 : 4];
    int64_t cc[RELU ? 4 : 1];       // merged form: the 64-bit addend, held as a register pair from the start
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const int4 ch = __ldg(reinterpret_cast<const int4 *>(chan) + cq * 4 + c);
        if constexpr (RELU) {       // {C low, C high, M0, e - 1}
            mult[c] = ch.z; esh[c] = ch.w;
            cc[c] = static_cast<int64_t>((static_cast<uint64_t>(static_cast<uint32_t>(ch.y)) << 32) | static_cast<uint32_t>(ch.x));
        } else {
            mult[c] = ch.x; addend[c] = ch.y; esh[c] = ch.z; bias[c] = ch.w;
        }
#pragma unroll
        for (int ky = 0; ky < 3; ++ky) {
            wlo[ky][c] = __ldg(w_packed + (cq * 4 + c) * 3 + ky);
            if (STRIDE == 1) whi[ky][c] = wlo[ky][c] << 8;
        }
    }
    const uint32_t cpix = static_cast<uint32_t>(p.c);
    const int32_t hi_clamp = p.act_max - p.act_min;
    const uint32_t lo_word = (static_cast<uint32_t>(p.act_min) & 0xff) * 0x01010101u;
    const bool live = tid < nthr;
    const bool st0 = live && ox0 + strip * 4 + 0 < p.ow, st1 = live && ox0 + strip * 4 + 1 < p.ow;
    const bool st2 = live && ox0 + strip * 4 + 2 < p.ow, st3 = live && ox0 + strip * 4 + 3 < p.ow;
    const uint32_t out_pitch = static_cast<uint32_t>(p.ow) * cpix;
    const int32_t zero4[4] = {0, 0, 0, 0};

    // Ring position of the next row to take: its slot's read address for this thread, its barrier and the phase.
    const uint32_t rd0 = ring + static_cast<uint32_t>(strip * 4 * STRIDE) * cpix + static_cast<uint32_t>(cq) * 4;
    const uint32_t rd_end = rd0 + static_cast<uint32_t>(p.nr) * p.pitch;
    uint32_t rd = rd0, bar_a = full0, phase_a = 0;
    const uint32_t rel_off = 8u * p.nr;         // empty barrier of a slot = its full barrier + rel_off
    bool ok = true;
    uint8_t *orow = out;

    // Reads this thread's words of the next input row; returns the barrier to signal once they have been used.
    auto issue = [&](DwRaw<STRIDE> &raw) -> uint32_t {
        // Every lane looks once (the usual case: the row landed long ago); otherwise the lanes wait, bounded, and agree
        // on the outcome, so that a warp always leaves the row loop as a whole.
        if (!__all_sync(0xffffffffu, dw_mbar_try(bar_a, phase_a)))
            ok = __all_sync(0xffffffffu, dw_mbar_wait(bar_a, phase_a, abort_flag, p.err, 12));
#pragma unroll
        for (int i = 0; i < NP; ++i) raw.p[i] = dw_lds32(rd + static_cast<uint32_t>(i) * cpix);
        const uint32_t rel = bar_a + rel_off;
        rd += p.pitch;
        bar_a += 8;
        if (rd == rd_end) { rd = rd0; bar_a = full0; phase_a ^= 1; }
        return rel;
    };
    // Hands a slot back to the producer; the row's words are in registers by now.
    auto release = [&](uint32_t rel) {
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(rel) : "memory");
    };
    auto emit = [&](const DwRow<STRIDE> &r0, const DwRow<STRIDE> &r1, const DwRow<STRIDE> &r2) {
        int32_t acc[4][4];
        int32_t asum[NEED_ASUM ? 4 : 1][4];
        if constexpr (RELU) {
            dw_accumulate<STRIDE, W_SIGNED, NEED_ASUM, true>(acc, asum, r0, wlo[0], whi[0], zero4);
            dw_accumulate<STRIDE, W_SIGNED, NEED_ASUM, false>(acc, asum, r1, wlo[1], whi[STRIDE == 1 ? 1 : 0], zero4);
            dw_accumulate<STRIDE, W_SIGNED, NEED_ASUM, false>(acc, asum, r2, wlo[2], whi[STRIDE == 1 ? 2 : 0], zero4);
        } else {
            dw_accumulate<STRIDE, W_SIGNED, NEED_ASUM, true>(acc, asum, r0, wlo[0], whi[0], bias);
            dw_accumulate<STRIDE, W_SIGNED, NEED_ASUM, false>(acc, asum, r1, wlo[1], whi[STRIDE == 1 ? 1 : 0], bias);
            dw_accumulate<STRIDE, W_SIGNED, NEED_ASUM, false>(acc, asum, r2, wlo[2], whi[STRIDE == 1 ? 2 : 0], bias);
        }
        uint32_t word[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int32_t y[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                int32_t a = acc[c][j];
                if (NEED_ASUM) a -= p.w_zp * asum[c][j];
                int32_t v;
                if constexpr (RELU) {
                    const int64_t qv = static_cast<int64_t>(a) * mult[c] + cc[c];
                    v = static_cast<int32_t>(qv >> 32) >> esh[c];
                } else {
                    const int64_t pr = static_cast<int64_t>(a) * mult[c] + (1ll << 30);
                    const int32_t x = static_cast<int32_t>(pr >> 31);
                    v = (x + addend[c] - static_cast<int32_t>(shr_clamp(static_cast<uint32_t>(x), esh[c] >> 8))) >> (esh[c] & 0xff);
                }
                y[c] = RQ == 2 ? v : __vimin_s32_relu(v, hi_clamp);
            }
            const uint32_t hi = pack_sat_u8(y[3], y[2], 0);
            word[j] = pack_sat_u8(y[1], y[0], hi);
            if (RQ != 2) word[j] += lo_word;      // u8 outputs: byte + act_min <= act_max, no carry between bytes
        }
        if (st0) *reinterpret_cast<uint32_t *>(orow) = word[0];
        if (st1) *reinterpret_cast<uint32_t *>(orow + cpix) = word[1];
        if (st2) *reinterpret_cast<uint32_t *>(orow + 2 * cpix) = word[2];
        if (st3) *reinterpret_cast<uint32_t *>(orow + 3 * cpix) = word[3];
        orow += out_pitch;
    };

    pdl_wait();     // the tensor this kernel writes is no longer read by the kernel before it
    for (int u = u0; u < u1 && ok;) {
        const int img = u / p.oh, oy0 = u - img * p.oh;
        const int cnt = min(p.oh - oy0, u1 - u);
        u += cnt;
        orow = out + ((static_cast<int64_t>(img) * p.oh + oy0) * p.ow + ox0 + strip * 4) * static_cast<int64_t>(cpix) + cq * 4;
        DwRow<STRIDE> ra, rb, rc;
        if constexpr (STRIDE == 1) {
            // input rows oy0 - pt ... oy0 - pt + cnt + 1, one per output row after the first three
            DwRaw<STRIDE> nx;
            uint32_t rel = issue(nx);
            dw_transpose_row<STRIDE>(ra, nx);
            release(rel);
            rel = issue(nx);
            dw_transpose_row<STRIDE>(rb, nx);
            release(rel);
            rel = issue(nx);
            for (int r = 0; r < cnt && ok; r += 3) {
                dw_transpose_row<STRIDE>(rc, nx);
                release(rel);
                if (r + 1 < cnt) rel = issue(nx);
                emit(ra, rb, rc);
                if (r + 1 < cnt) {
                    dw_transpose_row<STRIDE>(ra, nx);
                    release(rel);
                    if (r + 2 < cnt) rel = issue(nx);
                    emit(rb, rc, ra);
                }
                if (r + 2 < cnt) {
                    dw_transpose_row<STRIDE>(rb, nx);
                    release(rel);
                    if (r + 3 < cnt) rel = issue(nx);
                    emit(rc, ra, rb);
                }
            }
        } else {
            // input rows 2 oy0 - pt ... 2 oy0 - pt + 2 cnt, two per output row after the first
            DwRaw<STRIDE> n1, n2;
            uint32_t rel1 = issue(n1), rel2;
            dw_transpose_row<STRIDE>(ra, n1);
            release(rel1);
            rel1 = issue(n1);
            rel2 = issue(n2);
            for (int r = 0; r < cnt && ok; r += 2) {
                dw_transpose_row<STRIDE>(rb, n1);
                release(rel1);
                dw_transpose_row<STRIDE>(rc, n2);
                release(rel2);
                if (r + 1 < cnt) {
                    rel1 = issue(n1);
                    rel2 = issue(n2);
                }
                emit(ra, rb, rc);
                if (r + 1 < cnt) {
                    dw_transpose_row<STRIDE>(rb, n1);
                    release(rel1);
                    dw_transpose_row<STRIDE>(ra, n2);
                    release(rel2);
                    if (r + 2 < cnt) {
                        rel1 = issue(n1);
                        rel2 = issue(n2);
                    }
                    emit(rc, rb, ra);
                }
            }
        }
    }
}

bool dw3x3_eligible(const ConvGeom &g) {
    return g.kh == 3 && g.kw == 3 && g.dh == 1 && g.dw == 1 && g.groups == 1 && g.sh == g.sw && (g.sh == 1 || g.sh == 2) &&
           (g.cin % 4) == 0 && g.cout == g.cin && !g.a_signed;
}

// Launch shape of the row-ring kernel for one geometry.
struct DwRingPlan {
    DwRingParams prm{};
    int grid = 0, threads = 0;
    size_t smem = 0;
    int32_t *err_host = nullptr;       // pinned + mapped
    int32_t *err_dev = nullptr;
    void *zrow_dev = nullptr;          // row of input zero points
};

// Chooses tile width, ring depth and grid; returns false when the geometry is outside the kernel's domain.
bool dw_ring_plan(enn_b200_op *op) {
    const ConvGeom &g = op->g;
    enn_b200_context *ctx = op->ctx;
    if (!dw3x3_eligible(g) || (g.cin & 15) != 0 || !op->dw_chan || ctx->cc_major < 9 || ctx->opt("dw_legacy")) return false;
    const int q = g.cin / 4, s = g.sh;
    if (q > kDwRingConsumersBig || g.n <= 0) return false;
    const int strips = (g.ow + 3) / 4;
    int ns_max = (q > kDwRingConsumers ? kDwRingConsumersBig : kDwRingConsumers) / q;
    if (ns_max > strips) ns_max = strips;
    const int tx_n = (strips + ns_max - 1) / ns_max;
    const int ns = (strips + tx_n - 1) / tx_n;
    DwRingPlan *pl = new (std::nothrow) DwRingPlan();
    if (!pl) return false;
    DwRingParams &p = pl->prm;
    p.n = g.n; p.h = g.h; p.w = g.w; p.c = g.cin; p.oh = g.oh; p.ow = g.ow; p.pt = g.pt; p.pl = g.pl;
    p.q = q; p.ns = ns; p.tx_n = tx_n;
    p.slot_px = (4 * ns - 1) * s + 3;
    p.pitch = (static_cast<uint32_t>(p.slot_px) * g.cin + 127u) & ~127u;
    // CTAs per SM: what the 128-register budget allows for this block size (at most four); they share the shared memory,
    // and a ring of up to 16 rows each keeps 50-100 KB per SM in flight.
    const int threads = 32 * ((ns * q + 31) / 32 + 1);
    int per_sm = 65536 / (threads * 128);
    per_sm = per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm);
    const size_t budget = static_cast<size_t>(216 * 1024) / per_sm;
    int nr = static_cast<int>((budget - 512) / p.pitch);
    if (ctx->opt("dw_rows") > 0 && ctx->opt("dw_rows") < nr) nr = ctx->opt("dw_rows");   // tuning override
    if (nr > 16) nr = 16;
    // the kernels' dynamic shared memory limit is set to 110 KB (a ring of long rows: stride 2 with over 900 channels)
    const size_t smem_cap = 108 * 1024;
    if (static_cast<size_t>(nr) * (p.pitch + 16) + 192 > smem_cap) nr = static_cast<int>((smem_cap - 192) / (p.pitch + 16));
    if (nr < 4) {
        delete pl;
        return false;
    }
    p.nr = nr;
    p.in_zp = g.in_zp; p.w_zp = g.w_zp; p.act_min = g.act_min; p.act_max = g.act_max;
    // One wave of CTAs, each with at least a few output rows so that the two halo rows stay cheap.
    const int64_t units = static_cast<int64_t>(g.n) * g.oh;
    int per_tx = (per_sm * ctx->launch_sms()) / tx_n;
    if (per_tx < 1) per_tx = 1;
    const int64_t min_rows = 6;
    if (per_tx > (units + min_rows - 1) / min_rows) per_tx = static_cast<int>((units + min_rows - 1) / min_rows);
    p.ctas_per_tx = per_tx;
    pl->grid = per_tx * tx_n;
    pl->threads = threads;
    pl->smem = static_cast<size_t>(nr) * p.pitch + static_cast<size_t>(nr) * 16 + 64 + 128;
    if (cudaMalloc(&pl->zrow_dev, p.pitch) != cudaSuccess || cudaMemset(pl->zrow_dev, g.in_zp & 0xff, p.pitch) != cudaSuccess) {
        if (pl->zrow_dev) cudaFree(pl->zrow_dev);
        delete pl;
        return false;
    }
    p.zrow = static_cast<const uint8_t *>(pl->zrow_dev);
    if (cudaHostAlloc(reinterpret_cast<void **>(&pl->err_host), sizeof(int32_t), cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer(reinterpret_cast<void **>(&pl->err_dev), pl->err_host, 0) != cudaSuccess) {
        if (pl->err_host) cudaFreeHost(pl->err_host);
        cudaFree(pl->zrow_dev);
        delete pl;
        return false;
    }
    *pl->err_host = 0;
    p.err = pl->err_dev;
    op->dw_ring = pl;
    return true;
}

void dw_ring_release(enn_b200_op *op) {
    DwRingPlan *pl = static_cast<DwRingPlan *>(op->dw_ring);
    if (!pl) return;
    if (pl->err_host) cudaFreeHost(pl->err_host);
    if (pl->zrow_dev) cudaFree(pl->zrow_dev);
    delete pl;
    op->dw_ring = nullptr;
}

void dw_ring_clear_error(enn_b200_op *op) {
    DwRingPlan *pl = static_cast<DwRingPlan *>(op->dw_ring);
    if (pl && pl->err_host) *pl->err_host = 0;
}

// Returns cudaErrorNotSupported when the plan cannot serve this call (pointers not aligned for the bulk copies and the
// 32-bit stores), cudaErrorLaunchFailure when an earlier launch gave up on a barrier wait.
cudaError_t dw_ring_launch(enn_b200_op *op, const void *in, void *out) {
    DwRingPlan *pl = static_cast<DwRingPlan *>(op->dw_ring);
    if (!pl || (reinterpret_cast<uintptr_t>(in) & 15) != 0 || (reinterpret_cast<uintptr_t>(out) & 3) != 0) return cudaErrorNotSupported;
    if (*pl->err_host != 0) return cudaErrorLaunchFailure;
    const ConvGeom &g = op->g;
    const DwChan *c = static_cast<const DwChan *>(op->dw_chan);
    const uint32_t *w = static_cast<const uint32_t *>(op->dw_w);
    const uint8_t *i = static_cast<const uint8_t *>(in);
    uint8_t *o = static_cast<uint8_t *>(out);
    cudaStream_t s = op->ctx->stream;
    const bool asum = g.w_zp != 0;
    const int rq = !op->dw_relu ? 0 : ((g.act_min == 0 && g.act_max >= 255) ? 2 : 1);
    static bool attr_set = false;
#define ENN_DWR_ATTR(ST, WS, AS) \
    cudaFuncSetAttribute(dw3x3_ring_kernel<ST, WS, AS, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024); \
    cudaFuncSetAttribute(dw3x3_ring_kernel<ST, WS, AS, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024); \
    cudaFuncSetAttribute(dw3x3_ring_kernel<ST, WS, AS, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024); \
    cudaFuncSetAttribute(dw3x3_ring_kernel<ST, WS, AS, 0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024); \
    cudaFuncSetAttribute(dw3x3_ring_kernel<ST, WS, AS, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024); \
    cudaFuncSetAttribute(dw3x3_ring_kernel<ST, WS, AS, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024)
    if (!attr_set) {
        ENN_DWR_ATTR(1, true, true); ENN_DWR_ATTR(1, true, false); ENN_DWR_ATTR(1, false, true); ENN_DWR_ATTR(1, false, false);
        ENN_DWR_ATTR(2, true, true); ENN_DWR_ATTR(2, true, false); ENN_DWR_ATTR(2, false, true); ENN_DWR_ATTR(2, false, false);
        attr_set = true;
    }
#undef ENN_DWR_ATTR
    const bool big = pl->threads > kDwRingThreads;
#define ENN_DWR(ST, WS, AS, RQ)                                                                                                            \
    (big ? launch_pdl(dw3x3_ring_kernel<ST, WS, AS, RQ, true>, dim3(pl->grid), dim3(pl->threads), pl->smem, s, pl->prm, c, w, i, o) \
         : launch_pdl(dw3x3_ring_kernel<ST, WS, AS, RQ>, dim3(pl->grid), dim3(pl->threads), pl->smem, s, pl->prm, c, w, i, o))
#define ENN_DWR_R(ST, WS, AS) (rq == 0 ? ENN_DWR(ST, WS, AS, 0) : (rq == 1 ? ENN_DWR(ST, WS, AS, 1) : ENN_DWR(ST, WS, AS, 2)))
    if (g.sh == 1) {
        if (g.w_signed) { if (asum) ENN_DWR_R(1, true, true); else ENN_DWR_R(1, true, false); }
        else            { if (asum) ENN_DWR_R(1, false, true); else ENN_DWR_R(1, false, false); }
    } else {
        if (g.w_signed) { if (asum) ENN_DWR_R(2, true, true); else ENN_DWR_R(2, true, false); }
        else            { if (asum) ENN_DWR_R(2, false, true); else ENN_DWR_R(2, false, false); }
    }
#undef ENN_DWR_R
#undef ENN_DWR
    return cudaGetLastError();
}

cudaError_t launch_dw3x3(const ConvGeom &g, const void *chan, bool relu_form, const void *w_packed, const void *in, void *out,
                         int sm_count, cudaStream_t s) {
    const int nstrip = (g.ow + 3) / 4;
    const int cqn = g.cin / 4;
    // Rows per thread: as tall as possible while the grid still fills the machine several times over.
    const int64_t want_threads = static_cast<int64_t>(sm_count) * 512 * 2;
    int th = g.oh;
    while (th > 8 && static_cast<int64_t>(g.n) * ((g.oh + th - 1) / th) * nstrip * cqn < want_threads) th = (th + 1) / 2;
    const int nyt = (g.oh + th - 1) / th;
    const int64_t total = static_cast<int64_t>(g.n) * nyt * nstrip * cqn;
    if (total == 0) return cudaSuccess;
    const int threads = kDwThreads;
    const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
    const DwChan *c = static_cast<const DwChan *>(chan);
    const uint32_t *w = static_cast<const uint32_t *>(w_packed);
    const uint8_t *i = static_cast<const uint8_t *>(in);
    uint8_t *o = static_cast<uint8_t *>(out);
    const bool need_asum = g.w_zp != 0;
#define ENN_DW_LAUNCH(ST, WS, AS)                                                                                                          \
    (relu_form ? launch_pdl(dw3x3_kernel<ST, WS, AS, true>, dim3(blocks), dim3(threads), 0, s, g, c, w, i, o, th, nyt, nstrip, total)     \
               : launch_pdl(dw3x3_kernel<ST, WS, AS, false>, dim3(blocks), dim3(threads), 0, s, g, c, w, i, o, th, nyt, nstrip, total))
    if (g.sh == 1) {
        if (g.w_signed) { if (need_asum) ENN_DW_LAUNCH(1, true, true); else ENN_DW_LAUNCH(1, true, false); }
        else            { if (need_asum) ENN_DW_LAUNCH(1, false, true); else ENN_DW_LAUNCH(1, false, false); }
    } else {
        if (g.w_signed) { if (need_asum) ENN_DW_LAUNCH(2, true, true); else ENN_DW_LAUNCH(2, true, false); }
        else            { if (need_asum) ENN_DW_LAUNCH(2, false, true); else ENN_DW_LAUNCH(2, false, false); }
    }
#undef ENN_DW_LAUNCH
    return cudaGetLastError();
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
