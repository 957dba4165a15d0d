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
        // hi = pixels 2..5
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

// ------------------------------------------------------------------------------------------------------
// 3x3 fast path with TMA-staged input tiles (C % 16 == 0).
//
// A persistent CTA walks tiles of TH x (4 * NS) output pixels x CT channels.  The input window of a tile
// (with its one-pixel halo) is fetched by ONE 4-D tensor-map copy into shared memory, double buffered, so the
// copy of tile i+1 runs while tile i is computed; out-of-image positions arrive as zeros and are overwritten
// with the input zero point before use.  Threads then run the same transposed-row / dp4a / fused requantisation
// code as dw3x3_kernel, but every load is a shared-memory load at a compile-time offset: no per-load address
// arithmetic, no border predicates, no global-load latency in the math loop.
// Thread = (channel quad, strip of 4 output columns, row group); a row group owns R consecutive output rows.
// ------------------------------------------------------------------------------------------------------
struct DwTmaParams {
    int32_t n, h, w, c, oh, ow, pt, pl;
    int32_t ns, rg, r;            // strips per tile, row groups per tile, output rows per row group
    int32_t th, wt;               // output rows / columns per tile (rg * r, 4 * ns)
    int32_t win, hin;             // input window per tile (box extents in W and H)
    int32_t tiles_x, tiles_y, cblks, total_tiles;
    int32_t in_zp, w_zp, act_min, act_max;
    uint32_t tile_bytes;          // bytes one tensor-map copy delivers (win * hin * CT)
    uint32_t buf_pitch;           // distance between the two shared-memory buffers (tile_bytes rounded up to 128)
    int32_t *err;                 // host-mapped error word
};

__device__ __forceinline__ uint32_t dw_smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ uint32_t dw_lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

template <int STRIDE, int CT, bool W_SIGNED, bool NEED_ASUM>
__global__ void __launch_bounds__(256, 2)
dw3x3_tma_kernel(const __grid_constant__ CUtensorMap map_in, DwTmaParams p, const DwChan *__restrict__ chan,
                 const uint32_t *__restrict__ w_packed, uint8_t *__restrict__ out) {
    extern __shared__ uint8_t dw_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(dw_smem_raw) + 127) & ~static_cast<uintptr_t>(127));
    __shared__ uint64_t full_bar[2];
    __shared__ int s_ok;
    constexpr int QN = CT / 4;
    constexpr int NP = STRIDE == 1 ? 6 : 9;
    const int tid = threadIdx.x;
    const int cq = tid % QN;
    const int strip = (tid / QN) % p.ns;
    const int rgi = tid / (QN * p.ns);
    const uint32_t buf0 = dw_smem_u32(smem);
    const uint32_t bar0 = dw_smem_u32(&full_bar[0]);
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0 + 8) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    auto tile_coords = [&](int tile, int &cb, int &img, int &ty, int &tx) {
        tx = tile % p.tiles_x;
        int t = tile / p.tiles_x;
        ty = t % p.tiles_y;
        t /= p.tiles_y;
        img = t % p.n;
        cb = t / p.n;              // channel block is the slowest index: a CTA keeps its weights for many tiles
    };
    auto issue = [&](int tile, int buf) {
        int cb, img, ty, tx;
        tile_coords(tile, cb, img, ty, tx);
        const uint32_t bar = bar0 + 8 * buf;
        const uint32_t dst = buf0 + buf * p.buf_pitch;
        const int x = tx * p.wt * STRIDE - p.pl, y = ty * p.th * STRIDE - p.pt;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(p.tile_bytes) : "memory");
        asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                     ::"r"(dst), "l"(&map_in), "r"(bar), "r"(cb * CT), "r"(x), "r"(y), "r"(img)
                     : "memory");
    };

    uint32_t wlo[3][4], whi[3][4];
    int32_t mult[4], addend[4], esh[4], bias[4];
    int loaded_cb = -1;
    const uint32_t zaw = (static_cast<uint32_t>(p.in_zp) & 0xff) * 0x01010101u;
    const int32_t hi_clamp = p.act_max - p.act_min;
    const uint32_t lo_word = (static_cast<uint32_t>(p.act_min) & 0xff) * 0x01010101u;
    const uint32_t row_pitch = static_cast<uint32_t>(p.win) * CT;

    int it = 0;
    if (tid == 0 && static_cast<int>(blockIdx.x) < p.total_tiles) issue(blockIdx.x, 0);
    for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        int cb, img, ty, tx;
        tile_coords(tile, cb, img, ty, tx);
        // Prefetch the next tile into the other buffer (its last readers finished before the barrier that ended
        // the previous iteration), then wait, bounded, for this tile.
        if (tid == 0) {
            const int next = tile + gridDim.x;
            if (next < p.total_tiles) issue(next, buf ^ 1);
            const uint32_t bar = bar0 + 8 * buf, parity = (it >> 1) & 1;
            int ok = 0;
            for (uint32_t i = 0; i < (1u << 24) && !ok; ++i) {
                uint32_t done;
                asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                             : "=r"(done) : "r"(bar), "r"(parity) : "memory");
                ok = done != 0;
            }
            if (!ok && p.err) *reinterpret_cast<volatile int32_t *>(p.err) = 7;
            s_ok = ok;
        }
        __syncthreads();
        if (!s_ok) break;            // uniform: every thread reads the same flag
        {   // every thread observes the completed phase itself before touching the tile
            uint32_t done;
            asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                         : "=r"(done) : "r"(bar0 + 8 * buf), "r"((it >> 1) & 1) : "memory");
            (void)done;
        }
        const uint32_t tbase = buf0 + buf * p.buf_pitch;
        const int ix0 = tx * p.wt * STRIDE - p.pl, iy0 = ty * p.th * STRIDE - p.pt;
        // Zero-filled positions outside the image become the input zero point (what the reference's pad kernel writes).
        if (zaw != 0 && (ix0 < 0 || iy0 < 0 || ix0 + p.win > p.w || iy0 + p.hin > p.h)) {
            for (int px = tid; px < p.win * p.hin; px += 256) {
                const int ry = px / p.win, rx = px - ry * p.win;
                if (iy0 + ry < 0 || iy0 + ry >= p.h || ix0 + rx < 0 || ix0 + rx >= p.w) {
                    const uint32_t a = tbase + static_cast<uint32_t>(px) * CT;
#pragma unroll
                    for (int k = 0; k < CT; k += 16)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(a + k), "r"(zaw) : "memory");
                }
            }
            __syncthreads();
        }
        if (cb != loaded_cb) {
            loaded_cb = cb;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int ch = cb * CT + cq * 4 + c;
                const DwChan v = chan[ch];
                mult[c] = v.mult; addend[c] = v.addend; esh[c] = v.e; bias[c] = v.bias;
#pragma unroll
                for (int ky = 0; ky < 3; ++ky) {
                    wlo[ky][c] = w_packed[ch * 3 + ky];
                    whi[ky][c] = wlo[ky][c] << 8;
                }
            }
        }
        // This thread: output rows oy0 .. oy0 + r - 1 of the tile, columns ox0 .. ox0 + 3, channels cb*CT + cq*4 ..
        const int oy0 = ty * p.th + rgi * p.r;
        const int ox0 = tx * p.wt + strip * 4;
        const int rows = min(p.r, p.oh - oy0);
        if (rows > 0 && ox0 < p.ow) {
            uint32_t omask = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (ox0 + j < p.ow) omask |= 1u << j;
            // shared address of (local input row rgi*r*STRIDE, local pixel strip*4*STRIDE, channel quad)
            uint32_t srow = tbase + (static_cast<uint32_t>(rgi * p.r * STRIDE) * p.win + static_cast<uint32_t>(strip * 4 * STRIDE)) * CT + cq * 4;
            uint8_t *orow = out + ((static_cast<int64_t>(img) * p.oh + oy0) * p.ow + ox0) * static_cast<int64_t>(p.c) + cb * CT + cq * 4;
            const uint32_t out_pitch = static_cast<uint32_t>(p.ow) * p.c;
            const uint32_t cpix = static_cast<uint32_t>(p.c);

            auto load_row = [&](DwRow<STRIDE> &r) {
                DwRaw<STRIDE> raw;
#pragma unroll
                for (int i = 0; i < NP; ++i) raw.p[i] = dw_lds32(srow + i * CT);
                srow += row_pitch;
                dw_transpose_row<STRIDE>(r, raw);
            };
            auto emit = [&](const DwRow<STRIDE> &r0, const DwRow<STRIDE> &r1, const DwRow<STRIDE> &r2) {
                int32_t acc[4][4];
                int32_t asum[NEED_ASUM ? 4 : 1][4];
                dw_accumulate<STRIDE, W_SIGNED, NEED_ASUM, true>(acc, asum, r0, wlo[0], whi[0], bias);
                dw_accumulate<STRIDE, W_SIGNED, NEED_ASUM, false>(acc, asum, r1, wlo[1], whi[1], bias);
                dw_accumulate<STRIDE, W_SIGNED, NEED_ASUM, false>(acc, asum, r2, wlo[2], whi[2], bias);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int32_t y[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        int32_t a = acc[c][j];
                        if (NEED_ASUM) a -= p.w_zp * asum[c][j];
                        const int64_t pr = static_cast<int64_t>(a) * mult[c] + (1ll << 30);
                        const int32_t x = static_cast<int32_t>(pr >> 31);
                        const int32_t v = (x + addend[c] - static_cast<int32_t>(shr_clamp(static_cast<uint32_t>(x), esh[c] >> 8))) >> (esh[c] & 0xff);
                        y[c] = __vimin_s32_relu(v, hi_clamp);
                    }
                    if (omask & (1u << j)) {
                        const uint32_t hi = pack_sat_u8(y[3], y[2], 0);
                        *reinterpret_cast<uint32_t *>(orow + static_cast<uint32_t>(j) * cpix) = pack_sat_u8(y[1], y[0], hi) + lo_word;
                    }
                }
                orow += out_pitch;
            };
            DwRow<STRIDE> ra, rb, rc;
            load_row(ra);
            if constexpr (STRIDE == 1) {
                load_row(rb);
                for (int oy = 0; oy < rows; oy += 3) {
                    load_row(rc);
                    emit(ra, rb, rc);
                    if (oy + 1 < rows) { load_row(ra); emit(rb, rc, ra); }
                    if (oy + 2 < rows) { load_row(rb); emit(rc, ra, rb); }
                }
            } else {
                for (int oy = 0; oy < rows; oy += 2) {
                    load_row(rb);
                    load_row(rc);
                    emit(ra, rb, rc);
                    if (oy + 1 < rows) { load_row(rb); load_row(ra); emit(rc, rb, ra); }
                }
            }
        }
        __syncthreads();             // all reads of this buffer are done before it is refilled two tiles later
    }
}

bool dw3x3_eligible(const ConvGeom &g) {
    return g.kh == 3 && g.kw == 3 && g.dh == 1 && g.dw == 1 && g.groups == 1 && g.sh == g.sw && (g.sh == 1 || g.sh == 2) &&
           (g.cin % 4) == 0 && !g.a_signed;
}

typedef CUresult (*DwEncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                    const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DwTmaPlan {
    DwTmaParams prm{};
    int ct = 0;
    int grid = 0;
    size_t smem = 0;
    CUtensorMap map{};
    const void *map_ptr = nullptr;
    int32_t *err_host = nullptr;
    int32_t *err_dev = nullptr;
};

// Chooses the tile shape; returns false when the geometry is outside this kernel's domain.
bool dw_tma_plan(enn_b200_op *op) {
    const ConvGeom &g = op->g;
    enn_b200_context *ctx = op->ctx;
    if (!dw3x3_eligible(g) || (g.cin & 15) != 0 || !ctx->encode_tiled || ctx->cc_major != 10 || !op->dw_chan) return false;
    if (g.n <= 0) return false;
    DwTmaPlan *pl = new (std::nothrow) DwTmaPlan();
    if (!pl) return false;
    DwTmaParams &p = pl->prm;
    const int s = g.sh;
    pl->ct = (g.cin % 64 == 0) ? 64 : ((g.cin % 32 == 0) ? 32 : 16);
    const int qn = pl->ct / 4;
    int ns = 1;
    while (ns < 8 && ns * 4 < g.ow) ns *= 2;
    while (qn * ns > 256) ns /= 2;
    const int rg = 256 / (qn * ns);
    int r = (g.oh + rg - 1) / rg;
    if (r > 8) r = 8;
    if (r < 1) r = 1;
    auto bytes_for = [&](int rr) {
        const int th = rg * rr, wt = 4 * ns;
        return static_cast<size_t>(wt * s + 3 - s) * (th * s + 3 - s) * pl->ct;
    };
    while (r > 1 && bytes_for(r) > 48 * 1024) --r;
    if (bytes_for(r) > 100 * 1024) {
        delete pl;
        return false;
    }
    p.n = g.n; p.h = g.h; p.w = g.w; p.c = g.cin; p.oh = g.oh; p.ow = g.ow; p.pt = g.pt; p.pl = g.pl;
    p.ns = ns; p.rg = rg; p.r = r; p.th = rg * r; p.wt = 4 * ns;
    p.win = p.wt * s + 3 - s; p.hin = p.th * s + 3 - s;
    p.tiles_x = (g.ow + p.wt - 1) / p.wt; p.tiles_y = (g.oh + p.th - 1) / p.th; p.cblks = g.cin / pl->ct;
    const int64_t total = static_cast<int64_t>(p.tiles_x) * p.tiles_y * p.cblks * g.n;
    if (total > INT32_MAX) {
        delete pl;
        return false;
    }
    p.total_tiles = static_cast<int32_t>(total);
    p.in_zp = g.in_zp; p.w_zp = g.w_zp; p.act_min = g.act_min; p.act_max = g.act_max;
    p.tile_bytes = static_cast<uint32_t>(bytes_for(r));
    p.buf_pitch = (p.tile_bytes + 127u) & ~127u;
    pl->smem = 2 * static_cast<size_t>(p.buf_pitch) + 128;
    pl->grid = p.total_tiles < 2 * ctx->sm_count ? p.total_tiles : 2 * ctx->sm_count;
    if (cudaHostAlloc(reinterpret_cast<void **>(&pl->err_host), sizeof(int32_t), cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer(reinterpret_cast<void **>(&pl->err_dev), pl->err_host, 0) != cudaSuccess) {
        if (pl->err_host) cudaFreeHost(pl->err_host);
        delete pl;
        return false;
    }
    *pl->err_host = 0;
    p.err = pl->err_dev;
    op->dw_tma = pl;
    return true;
}

void dw_tma_release(enn_b200_op *op) {
    DwTmaPlan *pl = static_cast<DwTmaPlan *>(op->dw_tma);
    if (!pl) return;
    if (pl->err_host) cudaFreeHost(pl->err_host);
    delete pl;
    op->dw_tma = nullptr;
}

template <int STRIDE, int CT>
static cudaError_t dw_tma_launch_t(const DwTmaPlan *pl, const ConvGeom &g, const void *chan, const void *wp, void *out, cudaStream_t s) {
    const DwChan *c = static_cast<const DwChan *>(chan);
    const uint32_t *w = static_cast<const uint32_t *>(wp);
    uint8_t *o = static_cast<uint8_t *>(out);
    const bool asum = g.w_zp != 0;
#define ENN_DWT(WS, AS)                                                                                                      \
    do {                                                                                                                     \
        cudaFuncSetAttribute(dw3x3_tma_kernel<STRIDE, CT, WS, AS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024); \
        dw3x3_tma_kernel<STRIDE, CT, WS, AS><<<pl->grid, 256, pl->smem, s>>>(pl->map, pl->prm, c, w, o);                     \
    } while (0)
    if (g.w_signed) { if (asum) ENN_DWT(true, true); else ENN_DWT(true, false); }
    else            { if (asum) ENN_DWT(false, true); else ENN_DWT(false, false); }
#undef ENN_DWT
    return cudaGetLastError();
}

// Returns cudaErrorNotSupported when the plan cannot be used for this call (misaligned input pointer).
cudaError_t dw_tma_launch(enn_b200_op *op, const void *in, void *out) {
    DwTmaPlan *pl = static_cast<DwTmaPlan *>(op->dw_tma);
    enn_b200_context *ctx = op->ctx;
    if (!pl || (reinterpret_cast<uintptr_t>(in) & 15) != 0) return cudaErrorNotSupported;
    if (*pl->err_host != 0) return cudaErrorLaunchFailure;
    const ConvGeom &g = op->g;
    if (pl->map_ptr != in) {
        DwEncodeTiledFn fn = reinterpret_cast<DwEncodeTiledFn>(ctx->encode_tiled);
        cuuint64_t dims[4] = {static_cast<cuuint64_t>(g.cin), static_cast<cuuint64_t>(g.w), static_cast<cuuint64_t>(g.h), static_cast<cuuint64_t>(g.n)};
        cuuint64_t strides[3] = {static_cast<cuuint64_t>(g.cin), static_cast<cuuint64_t>(g.w) * g.cin, static_cast<cuuint64_t>(g.h) * g.w * g.cin};
        cuuint32_t box[4] = {static_cast<cuuint32_t>(pl->ct), static_cast<cuuint32_t>(pl->prm.win), static_cast<cuuint32_t>(pl->prm.hin), 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        if (fn(&pl->map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(in), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorNotSupported;
        pl->map_ptr = in;
    }
    cudaStream_t s = ctx->stream;
    if (g.sh == 1) {
        if (pl->ct == 64) return dw_tma_launch_t<1, 64>(pl, g, op->dw_chan, op->dw_w, out, s);
        if (pl->ct == 32) return dw_tma_launch_t<1, 32>(pl, g, op->dw_chan, op->dw_w, out, s);
        return dw_tma_launch_t<1, 16>(pl, g, op->dw_chan, op->dw_w, out, s);
    }
    if (pl->ct == 64) return dw_tma_launch_t<2, 64>(pl, g, op->dw_chan, op->dw_w, out, s);
    if (pl->ct == 32) return dw_tma_launch_t<2, 32>(pl, g, op->dw_chan, op->dw_w, out, s);
    return dw_tma_launch_t<2, 16>(pl, g, op->dw_chan, op->dw_w, out, s);
}


cudaError_t launch_dw3x3(const ConvGeom &g, const void *chan, bool relu_form, const void *w_packed, const void *in, void *out,
                         int sm_count, cudaStream_t s) {
    const int nstrip = (g.ow + 3) / 4;
    const int cqn = g.cin / 4;
    // Rows per thread: as tall as possible while the grid still fills the machine several times over.
    const int64_t want_threads = static_cast<int64_t>(sm_count) * 512 * 2;
    int th = g.oh;
    while (th > 8 && static_cast<int64_t>(g.n) * ((g.oh + th - 1) / th) * nstrip * cqn < want_threads) th = (th + 1) / 2;
    if (const char *ev = getenv("ENN_B200_DW_TH")) th = atoi(ev) > 0 ? atoi(ev) : th;   // tuning override
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
