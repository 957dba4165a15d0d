// Tensor-core path for the dense contractions (Conv2D, FullyConnected, Deconvolution):
// TMA -> 128B-swizzled shared memory -> tcgen05.mma kind::i8 (int32 accumulators in TMEM) -> tcgen05.ld ->
// fused bias / zero-point / fixed-point requantisation / clamp epilogue -> NHWC bytes.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer of the A tiles (one lane)
//   warp 1      TMEM allocation, MMA issue (one lane)
//   warps 2..13 epilogue: each thread owns one accumulator row (= one output pixel) and a share of its columns
//   warp 14     TMA producer of the B tiles (one lane)
// Two accumulator buffers in TMEM let the epilogue of tile i overlap the MMAs of tile i+1.
//
// Value computed (ConvolutionKernels.cpp:956-1274 / :1317-1375): for output row m, column n
//   acc = sum_k (a[m][k] - za) (w[n][k] - zw) + bias[n]
// evaluated as  sum_k a*w'  -  zw' * sum_k a  +  bias'[n]   with w' = w - 128 for u8 weights (always fits int8),
// zw' = zw - 128 (0 for per-channel int8 filters) and bias'[n] = bias[n] - za * sum_k w'[n][k] + K za zw'.
// sum_k a comes out of the same MMA as one extra all-ones weight row per N tile (only when zw' != 0).
//
// Every wait on an mbarrier is bounded: after kSpinLimit failed polls the thread records an error code in
// host-visible memory, raises a CTA-wide abort flag and every role falls through to the common exit, where
// TMEM is released.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <type_traits>

#include "internal.h"
#include "requant.h"

namespace enn_b200 {

bool tc_available(const enn_b200_context *ctx);
int32_t tc_plan_conv(enn_b200_op *op, const void *weights_hwio_host);
int32_t tc_execute(enn_b200_op *op, const void *in, void *out);
void tc_release(enn_b200_op *op);
int32_t tc_test_starve_next(enn_b200_op *op);
int32_t tc_fuse_add(enn_b200_op *op, const AddParams &add, bool conv_is_second);
void tc_set_residual(enn_b200_op *op, const void *res);
void tc_clear_error(enn_b200_op *op);

namespace {

// Measurement aids (operands loaded once, epilogue or stores skipped, per-role wait counters) change results or add
// host synchronisation; they exist only in development builds (-DENN_B200_DEV) and compile to nothing otherwise.
#ifdef ENN_B200_DEV
#define ENN_DBG_MODE(p) ((p).dbg_mode)
#define ENN_DBG_PTR(p) ((p).dbg)
#else
#define ENN_DBG_MODE(p) 0
#define ENN_DBG_PTR(p) static_cast<long long *>(nullptr)
#endif

constexpr int kBM = 128;            // rows per tile = UMMA M
constexpr int kBK = 128;            // bytes of K per stage = one 128B swizzle atom = 4 UMMA K steps
constexpr int kMaxBN = 256;         // UMMA N limit
// Epilogue warps: 3 per TMEM lane quarter, splitting the 16-column chunks.  The epilogue is bound by dependent integer
// latencies, not by warp count: 12 warps with 128 registers (room for the compiler to interleave the 8 outputs of a half
// chunk) run the MobileNetV2 graph 6 % faster than 24 warps capped at 72 registers; 8 and 16 warps are 1 % behind.
constexpr int kEpiWarps = 8;
constexpr int kColGroups = kEpiWarps / 4;
constexpr int kChunksPerWarp = (kMaxBN / 16 + kColGroups - 1) / kColGroups;   // chunks one warp can own
// Warp 0 loads the A tiles, warp 1 issues the MMAs, warps 2 .. kEpiWarps + 1 are the epilogue (warp & 3 is the TMEM lane
// quarter a warp may read); long-K GEMMs are launched with one more warp that loads the B tiles.
// 128 registers per thread is the ceiling for this shape: a scheduler with four resident warps has 16384 registers.
// (Handing registers from the producer / MMA warps to the epilogue warps with setmaxnreg was measured: that code needs
// over 100 registers itself, and with 80 / 144 the 1x1 layers ran 40 % slower.)
constexpr int kThreadsOneProducer = 64 + 32 * kEpiWarps;
constexpr int kThreads = kThreadsOneProducer + 32;
constexpr uint32_t kSpinLimit = 1u << 24;

struct ColParam {   // per output column, 16 bytes
    int32_t mult;
    int32_t addend;   // stage-2 addend: 2^(e-1) + ((out_zp - act_min) << e)
    int32_t esh;      // right shift e >= 1 of the fused form; negative: general requantisation, `addend` = raw shift
    int32_t bias;     // folded bias'
};

struct TcParams {
    int32_t M, N, K;
    int32_t tiles_m, tiles_n, k_blocks;
    int32_t group;          // M tiles computed side by side in one accumulator buffer (group * bn_rows <= 256 columns)
    int32_t tiles_mg;       // ceil(tiles_m / group)
    int32_t raster;         // M groups per rasterisation band (see tile_coords)
    int32_t bn_rows;        // B rows per N tile in shared memory (= UMMA N), multiple of 16
    int32_t bn_data;        // real output columns per N tile
    int32_t stages;
    int32_t kpack;          // k-blocks that share one pipeline stage (one barrier round trip per kpack k-blocks)
    int32_t b_res;          // implicit convolutions: the whole B operand (one N tile, every tap) is loaded once and stays in shared memory
    int32_t need_asum;      // 1: column bn_data of each accumulator tile holds sum_k a
    int32_t zw_eff;         // zw'
    int32_t a_signed;
    int32_t act_min, act_max, out_zp;
    int32_t two;            // 1: CTA-pair mode (tiles_mg counts pairs of M tiles, group == 1, kpack == 1)
    int32_t mode;           // epilogue mode (kModeNudge ...), see tc_requant
    uint32_t idesc;
    const ColParam *cols;   // [tiles_n][bn_rows]
    uint8_t *out;           // output tensor base
    // Row m of the GEMM is output position (img, qy, qx) of a qh x qw grid; its first byte lives at
    // out + out_base + img * out_sn + qy * out_sy + qx * out_sx.  A plain [M][N] result uses qh = 1, qw = M.
    int32_t qh, qw;
    int64_t out_base, out_sn, out_sy, out_sx;
    // Implicit-convolution mode (taps > 0): an M tile is a patch of conv_ht x conv_wt output positions of one image;
    // k-block kb = (tap, channel chunk) and its A tile is the 4-D box {span channels, conv_wt, conv_ht, 1} of the
    // (zero-point padded) NHWC input at (chunk * span, tx * conv_wt + tap_dx, ty * conv_ht + tap_dy, image).
    int32_t taps, cchunks;
    int32_t conv_ht, conv_wt, conv_ty, conv_tx;
    int32_t span;           // bytes of K per k-block = swizzle span of both operand tiles: 128, 64 or 32
    int32_t k_pad;          // row pitch of the packed B matrix (K rounded up to 128)
    int16_t tap_dx[64], tap_dy[64];
    int32_t *err;           // host-mapped error word
    long long *dbg;         // optional per-CTA cycle counters [grid][8] (null in normal use)
    int32_t dbg_mode;       // development switches (0 in normal use)
    int32_t sat_plain;      // kModeReluHi whose clamp is [0, 255] on unsigned bytes: run the kModeReluSat kernel
    int32_t no_wide_store;  // tuning: keep 16-byte stores
    // Fused quantized add (kernels with FADD): the add operator's parameters and stage-1 tables (2 x 256 words, staged in
    // shared memory at add_off), the other addend (same layout as the output), and which addend the convolution's result is.
    AddParams add;
    int32_t add_on;
    const uint8_t *add_res;
    int32_t add_off;
    int32_t add_swap;       // 1: the convolution result is the add's second input
    int32_t epi_g;          // M tiles of a work unit the epilogue requantises together per column (1, 2 or 4)
    int32_t test_starve;    // self-test of the bounded waits: no operand copy is issued and the waits give up early
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait of the single-thread roles (producers, MMA issuer).  Callers look at the barrier with the non-blocking
// test_wait first (the common case: already complete); what is left waits with try_wait, which parks the thread in
// hardware between looks instead of spinning through issue slots that the epilogue warps of the same scheduler need.
__device__ __forceinline__ bool mbar_wait_fast(uint32_t bar, uint32_t parity, volatile int *abort_flag, int32_t *err, int code,
                                               uint32_t looks = kSpinLimit >> 7) {
    for (uint32_t i = 0; i < looks; ++i) {       // by default 2^17 looks of up to 10 us: gives up after about a second
        // suspend-time hint (ns): stay parked until the phase completes instead of coming back every few hundred cycles
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity), "r"(10000u)
            : "memory");
        if (ok) return true;
        if ((i & 63u) == 63u && *abort_flag) return false;
    }
    *abort_flag = 1;
    if (err) *reinterpret_cast<volatile int32_t *>(err) = code;
    return false;
}
// Bounded wait.  Returns false after the limit (or when another thread already aborted the CTA).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int32_t *err, int code) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    if (err) *reinterpret_cast<volatile int32_t *>(err) = code;
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t c0, int32_t c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
                 : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t c0, int32_t c1, int32_t c2, int32_t c3) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- CTA-pair (cta_group::2) forms: two CTAs of a cluster compute one 256-row tile, each holding its own 128 rows of
// A, half of the B rows and its 128 accumulator lanes.  The MMA is issued by the rank-0 CTA only.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// The tile lands in this CTA's shared memory; the bytes are counted on the rank-0 CTA's barrier (cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar_cluster, int32_t c0, int32_t c1) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// Arrives on the barrier at this offset in both CTAs of the pair once the MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask) : "memory");
}

// One k-block: KS (1, 2 or 4) MMAs over consecutive 32-byte K slices of the A tile at descriptor address `lo_a` and the
// B tile at `lo_b` (16-byte units; `desc_hi` = the constant upper descriptor word).  All descriptors are formed first, then
// the MMAs follow each other as one uninterrupted instruction run.  The first MMA overwrites the accumulator when
// `accumulate_first` is 0.
template <bool TWO, int KS>
__device__ __forceinline__ void umma_i8_run(uint32_t d_tmem, uint32_t desc_hi, uint32_t lo_a, uint32_t lo_b, uint32_t idesc,
                                            uint32_t accumulate_first) {
#define ENN_MMA_PAIR "tcgen05.mma.cta_group::2.kind::i8"
#define ENN_MMA_ONE "tcgen05.mma.cta_group::1.kind::i8"
#define ENN_DESC(I, OFF)                                                       \
    "add.u32 t, %2, " #OFF ";\n\tmov.b64 a" #I ", {t, %1};\n\t"                 \
    "add.u32 t, %3, " #OFF ";\n\tmov.b64 b" #I ", {t, %1};\n\t"
#define ENN_RUN_HEAD                                                                                  \
    "{\n\t.reg .pred p, q;\n\t.reg .b64 a0, a1, a2, a3, b0, b1, b2, b3;\n\t.reg .b32 t;\n\t"           \
    "setp.ne.b32 p, %5, 0;\n\t"                                                                       \
    "setp.eq.b32 q, %5, %5;\n\t"
#define ENN_RUN_ARGS ::"r"(d_tmem), "r"(desc_hi), "r"(lo_a), "r"(lo_b), "r"(idesc), "r"(accumulate_first) : "memory"
#define ENN_RUN(MMA)                                                                                                   \
    if (KS == 4)                                                                                                       \
        asm volatile(ENN_RUN_HEAD ENN_DESC(0, 0) ENN_DESC(1, 2) ENN_DESC(2, 4) ENN_DESC(3, 6)                         \
                     MMA " [%0], a0, b0, %4, p;\n\t" MMA " [%0], a1, b1, %4, q;\n\t" MMA " [%0], a2, b2, %4, q;\n\t" \
                     MMA " [%0], a3, b3, %4, q;\n\t}" ENN_RUN_ARGS);                                                   \
    else if (KS == 2)                                                                                                  \
        asm volatile(ENN_RUN_HEAD ENN_DESC(0, 0) ENN_DESC(1, 2)                                                       \
                     MMA " [%0], a0, b0, %4, p;\n\t" MMA " [%0], a1, b1, %4, q;\n\t}" ENN_RUN_ARGS);                   \
    else                                                                                                               \
        asm volatile(ENN_RUN_HEAD ENN_DESC(0, 0) MMA " [%0], a0, b0, %4, p;\n\t}" ENN_RUN_ARGS);
    if (TWO) { ENN_RUN(ENN_MMA_PAIR) } else { ENN_RUN(ENN_MMA_ONE) }
#undef ENN_RUN
#undef ENN_RUN_ARGS
#undef ENN_RUN_HEAD
#undef ENN_DESC
#undef ENN_MMA_ONE
#undef ENN_MMA_PAIR
}

__device__ __forceinline__ void tmem_ld_x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_x1(uint32_t taddr, uint32_t &r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile in shared memory, 128-byte rows, 128B swizzle: rows are 128 bytes apart, groups of 8
// rows 1024 bytes apart (stride byte offset), descriptor version 1, layout type 2 (SWIZZLE_128B).
// `span` = bytes per row = swizzle span (128 / 64 / 32): groups of 8 rows are 8 * span bytes apart and the layout
// type is SWIZZLE_128B (2), SWIZZLE_64B (4) or SWIZZLE_32B (6).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t span = 128) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);        // start address, 16-byte units
    d |= static_cast<uint64_t>(1) << 16;                            // leading byte offset (unused for swizzled K-major)
    d |= static_cast<uint64_t>((8 * span) >> 4) << 32;              // stride byte offset
    d |= static_cast<uint64_t>(1) << 46;                            // descriptor version
    d |= static_cast<uint64_t>(span == 128 ? 2 : (span == 64 ? 4 : 6)) << 61;
    return d;
}

__device__ __forceinline__ uint32_t pack_sat_u8_tc(int32_t hi, int32_t lo, uint32_t upper) {
    uint32_t d;
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(hi), "r"(lo), "r"(upper));
    return d;
}

// Work unit `tile` -> (M tile group tg, N tile tn).  Units are numbered band by band: a band is `raster` consecutive M
// groups, and inside a band the M index runs fastest.  The units in flight at one time (one per SM) then share few A and
// few B tiles, so that both operands stay L2 resident for large problems.
__device__ __forceinline__ void tile_coords(const TcParams &p, int tile, int &tg, int &tn) {
    if (p.tiles_n == 1) {       // the usual convolution case: no division (every epilogue thread runs this per tile)
        tg = tile;
        tn = 0;
        return;
    }
    if (p.raster == p.tiles_mg && p.tiles_n <= 4) {     // one band, few N tiles: subtract instead of dividing
        tg = tile;
        tn = 0;
        while (tg >= p.tiles_mg) {
            tg -= p.tiles_mg;
            ++tn;
        }
        return;
    }
    const int band = p.raster * p.tiles_n;
    const int b = tile / band, r = tile - b * band;
    const int g0 = b * p.raster;
    const int gw = min(p.raster, p.tiles_mg - g0);      // the last band may be narrower
    tn = r / gw;
    tg = g0 + (r - tn * gw);
}

// Epilogue modes (one kernel variant each; the planner picks the cheapest one every column of the operator allows):
//   kModeNudge   fused two-stage form below, every column a right shift e >= 1;
//   kModeGeneral as kModeNudge, but columns flagged esh < 0 take the general code (left shifts, e == 0, wide ranges);
//   kModeReluTwo lower clamp == output zero point (ReLU-type outputs): a negative stage-1 value ends at the clamp with or
//                without the tie correction, so the correction is dropped and the bias, both rounding terms and a left
//                shift ls fold into one 64-bit addend: q = acc * M0 + C, C = bias * M0 + 2^(30-ls) (+ 2^(e-1+31-ls) when
//                e >= 1); result = (q >> (31 - ls)) >> e.  Covers e == 0 and left shifts, which otherwise need the
//                general code.
//   kModeReluHi  the same with one shift, hi32(q) >> (e - 1), for operators whose columns all have e >= 1 and ls == 0
//                (two ALU instructions per output fewer; option no_relu_hi keeps the two-shift form).
// ColParam words: {mult, addend, esh, bias} for the first two modes, {C low, C high, mult, shifts} for the ReLU modes
// (shifts = e - 1 for kModeReluHi, (31 - ls) | e << 8 for kModeReluTwo).
constexpr size_t kWidePackWeightBytes = 100 * 1024;    // resident block-diagonal weights of a wide-row pixel packing
constexpr int kModeNudge = 0, kModeGeneral = 1, kModeReluHi = 2, kModeReluTwo = 3;
// kModeReluHi for outputs whose clamp is the whole unsigned byte (lower clamp 0, upper clamp 255, unsigned bytes): the
// saturating byte pack is the clamp, so the min / max and the add of the lower clamp to the packed word are left out.
// A kernel template value only: the plan and the ColParam contents are those of kModeReluHi.
constexpr int kModeReluSat = 4;

// The constants of one column in registers.  The ReLU modes read {C, (M0, shifts)} as two 64-bit words, so that the
// 64-bit addend arrives as a register pair and need not be assembled from two 32-bit registers.
struct ColRegs {
    int4 v;
    int64_t cc;
};
// `p` points into shared memory (derived from the kernel's shared array, so the compiler emits shared loads with
// the constant part of the address as the instruction's immediate offset).
template <int MODE>
__device__ __forceinline__ void ld_col_shared(const uint8_t *p, ColRegs &c) {
    __builtin_assume(__isShared(p));
    if (MODE >= kModeReluHi) {
        const longlong2 v = *reinterpret_cast<const longlong2 *>(p);
        c.cc = v.x;
        asm("mov.b64 {%0, %1}, %2;" : "=r"(c.v.z), "=r"(c.v.w) : "l"(v.y));
    } else {
        c.v = *reinterpret_cast<const int4 *>(p);
    }
}

// Requantise one accumulator (bias not yet added) to (value - act_min) in [0, act_max - act_min]; kModeReluSat leaves
// the clamp to the caller's saturating pack.
// Fast form (esh = right shift e >= 1): stage 1 is one 32x32->64 multiply-add and a funnel shift, stage 2 is
// (x + addend - [x < 0]) >> e with addend = 2^(e-1) + ((out_zp - act_min) << e), i.e. RoundingDivideByPOT
// (ties away from zero) with the zero point and the lower clamp folded in.
template <int MODE>
__device__ __forceinline__ int32_t tc_requant(int32_t acc, const ColRegs &cr, int32_t hi_clamp, int32_t out_zp, int32_t act_min,
                                              int32_t act_max) {
    const int4 &c = cr.v;
    if (MODE >= kModeReluHi) {
        const int64_t q = static_cast<int64_t>(acc) * c.z + cr.cc;
        int32_t lo, hi;
        asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(q));
        int32_t v;
        if (MODE == kModeReluTwo) {
            const int32_t xa = static_cast<int32_t>(__funnelshift_r(static_cast<uint32_t>(lo), static_cast<uint32_t>(hi), static_cast<uint32_t>(c.w)));
            v = xa >> (c.w >> 8);
        } else {
            v = hi >> c.w;
        }
        if (MODE == kModeReluSat) return v;
        return __vimin_s32_relu(v, hi_clamp);
    }
    acc += c.w;
    if (MODE == kModeGeneral && c.z < 0) return enn_requant(acc, c.x, c.y, out_zp, act_min, act_max) - act_min;   // c.y = raw shift
    const int64_t p = static_cast<int64_t>(acc) * c.x + (1ll << 30);
    const int32_t x = static_cast<int32_t>(p >> 31);
    const int32_t v = (x + c.y - static_cast<int32_t>(static_cast<uint32_t>(x) >> 31)) >> c.z;
    return __vimin_s32_relu(v, hi_clamp);
}
// The same from the four 32-bit words of a ColParam.
template <int MODE>
__device__ __forceinline__ int32_t tc_requant(int32_t acc, const int4 &c, int32_t hi_clamp, int32_t out_zp, int32_t act_min,
                                              int32_t act_max) {
    ColRegs cr;
    cr.v = c;
    cr.cc = 0;
    if (MODE >= kModeReluHi) asm("mov.b64 %0, {%1, %2};" : "=l"(cr.cc) : "r"(c.x), "r"(c.y));
    return tc_requant<MODE>(acc, cr, hi_clamp, out_zp, act_min, act_max);
}

// The k loop of one accumulator tile for the common big-GEMM shape (four K slices per k-block, one k-block per stage),
// unrolled over the D stages of the ring: stage addresses, barrier addresses and descriptors are then loop invariants
// held in registers, and a k-block costs the MMA thread a barrier look-up, the four MMAs, a commit and a counter.
// The ring position carries over from tile to tile, so the unrolled sequence is entered at the current stage.
#define ENN_KB(S)                                                                                                        \
    {                                                                                                                    \
        const uint32_t bar = full0 + 8 * (S);                                                                            \
        if (!mbar_test_wait(bar, phase) && !mbar_wait_fast(bar, phase, abort_flag, err, 3)) return false;                \
        umma_i8_run<TWO, 4>(d_tmem, desc_hi, lo0 + (S) * stage16, lo0 + (S) * stage16 + a16, idesc, acc);                \
        acc = 1;                                                                                                         \
        if (TWO) umma_commit_pair(empty0 + 8 * (S));                                                                     \
        else umma_commit(empty0 + 8 * (S));                                                                              \
        if (--n == 0) {                                                                                                  \
            stage = (S) + 1;                                                                                             \
            break;                                                                                                       \
        }                                                                                                                \
    }
#define ENN_TILE_FN(NAME, D, CASES)                                                                                      \
    template <bool TWO>                                                                                                  \
    __device__ __forceinline__ bool NAME(uint32_t d_tmem, int n, uint32_t &stage, uint32_t &phase, uint32_t full0,       \
                                         uint32_t empty0, uint32_t desc_hi, uint32_t lo0, uint32_t stage16, uint32_t a16, \
                                         uint32_t idesc, volatile int *abort_flag, int32_t *err) {                      \
        uint32_t acc = 0;                                                                                                \
        for (;;) {                                                                                                       \
            switch (stage) { CASES }                                                                                     \
            if (n == 0) break;                                                                                           \
            stage = 0;                                                                                                   \
            phase ^= 1;                                                                                                  \
        }                                                                                                                \
        if (stage == (D)) {                                                                                              \
            stage = 0;                                                                                                   \
            phase ^= 1;                                                                                                  \
        }                                                                                                                \
        return true;                                                                                                     \
    }
ENN_TILE_FN(mma_tile_d4, 4, case 0: ENN_KB(0) case 1: ENN_KB(1) case 2: ENN_KB(2) case 3: ENN_KB(3))
ENN_TILE_FN(mma_tile_d6, 6, case 0: ENN_KB(0) case 1: ENN_KB(1) case 2: ENN_KB(2) case 3: ENN_KB(3) case 4: ENN_KB(4) case 5: ENN_KB(5))
#undef ENN_TILE_FN
#undef ENN_KB

// Fused add: the 16 requantised bytes of a chunk (four words) and the 16 bytes of the other addend at the same place go
// through the quantized add exactly as add_kernel_vec computes it (kernels_direct.cu): stage 1 of either input from the
// operator's tables in shared memory, stage 2 computed.
struct FaddCtx {
    uint32_t lut_u32;       // 2 x 256 words in shared memory: input-0 table, input-1 table
    int32_t mo, so, out_off, act_min, act_max;
    bool swap;
};
__device__ __forceinline__ uint32_t fadd_word(uint32_t y, uint32_t r, const FaddCtx &f) {
    const uint32_t a = f.swap ? r : y, b = f.swap ? y : r;
    uint32_t word = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t ba = (a >> (8 * k)) & 0xff, bb = (b >> (8 * k)) & 0xff;
        int32_t x0, x1;
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(x0) : "r"(f.lut_u32 + ba * 4));
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(x1) : "r"(f.lut_u32 + 1024 + bb * 4));
        int32_t o = enn_rdivpot(enn_srdhm(x0 + x1, f.mo), -f.so) + f.out_off;
        o = max(f.act_min, o);
        o = min(f.act_max, o);
        word |= (static_cast<uint32_t>(o) & 0xff) << (8 * k);
    }
    return word;
}
__device__ __forceinline__ void fadd_chunk(uint32_t (&w)[4], const uint8_t *res, const FaddCtx &f) {
    const uint4 r = *reinterpret_cast<const uint4 *>(res);      // plain load: the output may be written over this addend
    w[0] = fadd_word(w[0], r.x, f);
    w[1] = fadd_word(w[1], r.y, f);
    w[2] = fadd_word(w[2], r.z, f);
    w[3] = fadd_word(w[3], r.w, f);
}

// TWO: CTA-pair mode (launched as clusters of 2; plain GEMM operands only, group == 1, kpack == 1): the pair owns M
// tiles 2t and 2t + 1 of one N tile, every B byte is read from L2 once per pair, and a stage per CTA is A plus half of B.
template <bool ASUM, int MODE, bool TWO, bool FADD = false>
__global__ void __launch_bounds__(kThreads, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled tiles.
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t span = static_cast<uint32_t>(p.span);
    const uint32_t a_bytes = kBM * span;
    const uint32_t b_bytes = static_cast<uint32_t>(TWO ? p.bn_rows >> 1 : p.bn_rows) * span;
    const bool bres = !TWO && p.b_res != 0;
    const uint32_t b_stride = (b_bytes + 1023u) & ~1023u;             // resident B: distance between its k-blocks
    const uint32_t kb_bytes = a_bytes + (bres ? 0u : b_bytes);        // one k-block of a stage: A tile, then B tile unless B is resident
    const uint32_t rank = TWO ? cluster_ctarank() : 0;
    const int tile_first = TWO ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int tile_step = TWO ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
    const uint32_t stage_bytes = kb_bytes * static_cast<uint32_t>(p.kpack);
    uint8_t *tiles = smem;
    // Per-epilogue-warp copies of the N tile's column constants (kEpiWarps x 256 x 16 bytes): private to a warp, so
    // refreshing them needs only a warp-level sync.
    uint8_t *b_resident = smem + static_cast<size_t>(p.stages) * stage_bytes;
    int4 *s_cols = reinterpret_cast<int4 *>(b_resident + (bres ? static_cast<size_t>(p.k_blocks) * b_stride : 0));
    const uint32_t s_cols_u32 = smem_u32(s_cols);
    // The same place as a pointer that is visibly derived from the shared array (for loads written in C++).
    const uint8_t *s_cols_sp = smem_raw + (s_cols_u32 - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_cols + kEpiWarps * kChunksPerWarp * 16);
    // bars: full[stages], empty[stages], tmem_full[2], tmem_empty[2]
    const int nst = p.stages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * nst + 5);      // bars[2 * nst + 4]: resident B loaded
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool dbg = ENN_DBG_PTR(p) != nullptr;
    const bool split = blockDim.x == kThreads;      // launched with the separate B producer warp
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + nst);
    const uint32_t tfull0 = smem_u32(bars + 2 * nst), tempty0 = smem_u32(bars + 2 * nst + 2);

    if (threadIdx.x == 0) {
        for (int s = 0; s < nst; ++s) {
            mbar_init(full0 + 8 * s, split ? 2 : 1);        // one expect-tx arrival per producer
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(tempty0 + 16, 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull0 + 8 * b, 1);
            mbar_init(tempty0 + 8 * b, TWO ? 2 * kEpiWarps : kEpiWarps);      // one arrival per epilogue warp (of both CTAs)
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (TWO) tmem_alloc_pair(smem_u32(tmem_slot), 512);
        else tmem_alloc(smem_u32(tmem_slot), 512);
    }
    // Column constants: when those of all N tiles fit the staging area they are loaded here once, shared by every
    // epilogue warp (any warp can then take any chunk); otherwise each epilogue warp keeps private copies of the
    // columns it owns and refreshes them when the N tile changes.
    const bool cols_shared = p.tiles_n * p.bn_rows <= kEpiWarps * kChunksPerWarp * 16;
    if (cols_shared)
        for (int i = threadIdx.x; i < p.tiles_n * p.bn_rows; i += blockDim.x) s_cols[i] = __ldg(reinterpret_cast<const int4 *>(p.cols) + i);
    FaddCtx fadd{};
    if (FADD) {     // the add operator's stage-1 tables: constants of the plan, staged ahead of the launch dependency
        fadd.lut_u32 = smem_u32(smem) + static_cast<uint32_t>(p.add_off);
        fadd.mo = p.add.mo; fadd.so = p.add.so; fadd.out_off = p.add.out_off; fadd.act_min = p.add.act_min; fadd.act_max = p.add.act_max;
        fadd.swap = p.add_swap != 0;
        for (int i = threadIdx.x; i < 512; i += blockDim.x)
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(fadd.lut_u32 + i * 4), "r"(__ldg(p.add.lut + i)) : "memory");
    }
    tc_fence_before();
    __syncthreads();
    if (TWO) cluster_sync_all();        // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Resident weights (the operator's only N tile: every k-block of B, once) are constants of the plan: their copy
    // starts here, ahead of the wait below, and the MMA issuer picks it up on its barrier.
    const bool starve = p.test_starve != 0;      // self-test: nothing is copied, so the first wait of the MMA issuer runs out
    if (bres && threadIdx.x == 0 && !starve) {
        const uint32_t bb = tempty0 + 16;
        mbar_expect_tx(bb, b_bytes * static_cast<uint32_t>(p.k_blocks));
        for (int kb = 0; kb < p.k_blocks; ++kb) tma_load_2d(smem_u32(b_resident) + kb * b_stride, &map_b, bb, kb * static_cast<int>(span), 0);
    }
    // Everything above touched only this launch's own resources and constants; the activations of the kernel before
    // this one are complete (and the tensor this one writes is no longer read) from here on.
    pdl_wait();
    pdl_trigger();

    // Work unit = (N tile, group of `group` consecutive M tiles).  For narrow N several M tiles share one accumulator
    // buffer, so that every epilogue warp has columns to work on.
    const int total_tiles = p.tiles_mg * p.tiles_n;

    if (warp == 0 || warp == kEpiWarps + 2) {
        // ---------------- TMA producers: warp 0 loads the A tiles, the last warp the B tiles ----------------
        // (one thread issuing both operands of every k-block cannot keep up with the tensor pipe)
        // Big-GEMM shape (plain operands, one k-block per stage, an even number of stages, separate A and B warps): a
        // thread issues about one tensor copy per 420 cycles, which is also about what the tensor pipe needs per
        // k-block, so two lanes of each producer warp take the k-blocks in turn (two lanes issuing in step reach
        // 1.7 x the rate of one).  A stage always belongs to the same lane, so each lane meets its stages' phases in order.
        const bool pair_lanes = !starve && split && p.taps == 0 && p.group == 1 && p.kpack == 1 && (nst & 1) == 0 && p.k_blocks >= 8 &&
                                !(ENN_DBG_MODE(p) & 9);
        if (pair_lanes) {
            const int nl = 2;      // lanes that share the issue (four measured slightly worse than two)
            if (lane < nl) {
                const bool is_a = warp == 0;
                const CUtensorMap *map = is_a ? &map_a : &map_b;
                const uint32_t tx = is_a ? a_bytes : b_bytes;
                const uint32_t sa0 = smem_u32(tiles) + (is_a ? 0u : a_bytes);
                const int my_tiles = tile_first < total_tiles ? (total_tiles - tile_first + tile_step - 1) / tile_step : 0;
                int t = 0, kb = lane, t_cur = -1, row = 0;
                uint32_t stage = static_cast<uint32_t>(lane), phase = 0;
                bool ok = true;
                while (t < my_tiles) {
                    if (t != t_cur) {
                        t_cur = t;
                        int tg, tn;
                        tile_coords(p, tile_first + t * tile_step, tg, tn);
                        if (TWO) row = is_a ? (tg * 2 + static_cast<int>(rank)) * kBM : tn * p.bn_rows + static_cast<int>(rank) * (p.bn_rows >> 1);
                        else row = is_a ? tg * kBM : tn * p.bn_rows;
                    }
                    const uint32_t ebar = empty0 + 8 * stage;
                    if (!mbar_test_wait(ebar, phase ^ 1) && !mbar_wait_fast(ebar, phase ^ 1, abort_flag, p.err, 1)) { ok = false; break; }
                    const uint32_t bar = full0 + 8 * stage;
                    if (TWO) {      // rank 0 expects the bytes of both CTAs; every load reports to rank 0's barrier
                        if (rank == 0) mbar_expect_tx(bar, 2 * tx);
                        tma_load_2d_pair(sa0 + stage * stage_bytes, map, mapa_rank(bar, 0), kb * static_cast<int>(span), row);
                    } else {
                        mbar_expect_tx(bar, tx);
                        tma_load_2d(sa0 + stage * stage_bytes, map, bar, kb * static_cast<int>(span), row);
                    }
                    stage += nl;
                    if (stage >= static_cast<uint32_t>(nst)) { stage -= nst; phase ^= 1; }
                    kb += nl;
                    while (kb >= p.k_blocks) { kb -= p.k_blocks; ++t; }
                }
                if (!ok) {
                    for (int s2 = 0; s2 < nst; ++s2)
                        for (uint32_t i = 0; i < (1u << 16); ++i)
                            if (mbar_try_wait(full0 + 8 * s2, 0) || mbar_try_wait(full0 + 8 * s2, 1)) break;
                }
            }
        } else if (!starve && !TWO && !split && bres && (nst & 1) == 0 && !(ENN_DBG_MODE(p) & 9)) {
            // Resident weights (implicit convolutions, narrow pointwise layers): only A tiles are left to load, and the copy
            // issue rate of one thread still bounds the kernel, so lanes 0 and 1 fill alternate stages (a stage keeps its lane).
            if (lane < 2) {
                const uint32_t a_tx = p.taps > 0 ? static_cast<uint32_t>(p.conv_ht * p.conv_wt) * span : a_bytes;
                const uint32_t sa0 = smem_u32(tiles);
                const int gpt = (p.k_blocks + p.kpack - 1) / p.kpack;      // stages per M tile
                const int per_img = p.taps > 0 ? p.conv_ty * p.conv_tx : 1;
                int tile = tile_first, j = 0, g = 0, tg = 0, tn = 0, nsub = 0;
                bool done = tile >= total_tiles, ok = true;
                if (!done) {
                    tile_coords(p, tile, tg, tn);
                    nsub = min(p.group, p.tiles_m - tg * p.group);
                }
                auto advance = [&](int n) {
                    for (int s2 = 0; s2 < n && !done; ++s2) {
                        if (++g < gpt) continue;
                        g = 0;
                        if (++j < nsub) continue;
                        j = 0;
                        tile += tile_step;
                        if (tile >= total_tiles) {
                            done = true;
                        } else {
                            tile_coords(p, tile, tg, tn);
                            nsub = min(p.group, p.tiles_m - tg * p.group);
                        }
                    }
                };
                advance(lane);
                uint32_t stage = static_cast<uint32_t>(lane), phase = 0;
                int tm_cur = -1, img = 0, ty = 0, tx = 0;
                while (!done) {
                    const int tm = tg * p.group + j;
                    if (tm != tm_cur && p.taps > 0) {          // patch (img, ty, tx) of the output grid
                        img = tm / per_img;
                        const int rem = tm - img * per_img;
                        ty = rem / p.conv_tx;
                        tx = rem - ty * p.conv_tx;
                    }
                    tm_cur = tm;
                    const int kb0 = g * p.kpack, nkb = min(p.kpack, p.k_blocks - kb0);
                    const uint32_t ebar = empty0 + 8 * stage;
                    if (!mbar_test_wait(ebar, phase ^ 1) && !mbar_wait_fast(ebar, phase ^ 1, abort_flag, p.err, 1)) { ok = false; break; }
                    const uint32_t bar = full0 + 8 * stage;
                    mbar_expect_tx(bar, a_tx * nkb);
                    uint32_t sa = sa0 + stage * stage_bytes;
                    if (p.taps > 0) {
                        int tap = kb0 / p.cchunks, cc = kb0 - tap * p.cchunks;
                        for (int q = 0; q < nkb; ++q, sa += kb_bytes) {
                            tma_load_4d(sa, &map_a, bar, cc * static_cast<int>(span), tx * p.conv_wt + p.tap_dx[tap], ty * p.conv_ht + p.tap_dy[tap], img);
                            if (++cc == p.cchunks) { cc = 0; ++tap; }
                        }
                    } else {
                        for (int q = 0; q < nkb; ++q, sa += kb_bytes) tma_load_2d(sa, &map_a, bar, (kb0 + q) * static_cast<int>(span), tm * kBM);
                    }
                    stage += 2;
                    if (stage >= static_cast<uint32_t>(nst)) { stage -= nst; phase ^= 1; }
                    advance(2);
                }
                if (!ok) {
                    for (int s2 = 0; s2 < nst; ++s2)
                        for (uint32_t i = 0; i < (1u << 16); ++i)
                            if (mbar_try_wait(full0 + 8 * s2, 0) || mbar_try_wait(full0 + 8 * s2, 1)) break;
                }
            }
        } else if (lane == 0 && !starve) {
            // WHICH: 0 = the A tiles, 1 = the B tiles, 2 = both (launches without the separate B producer warp)
            auto produce = [&](auto which) {
                constexpr int WHICH = decltype(which)::value;
                constexpr bool DO_A = WHICH != 1, DO_B = WHICH != 0;
                uint32_t stage = 0, phase = 0, filled = 0;
                const uint32_t sa_stage0 = smem_u32(tiles);
                uint32_t sa_stage = sa_stage0;
                // bytes this producer's loads add to a k-block (pairs: of both CTAs, counted on rank 0's barrier)
                const uint32_t a_tx = p.taps > 0 ? static_cast<uint32_t>(p.conv_ht * p.conv_wt) * span : a_bytes;
                const uint32_t kb_tx = ((DO_A ? a_tx : 0u) + (DO_B && !bres ? b_bytes : 0u)) * (TWO ? 2u : 1u);
                bool ok = true;
                long long t_wait = 0;
                for (int tile = tile_first; tile < total_tiles && ok; tile += tile_step) {
                    int tg, tn;
                    tile_coords(p, tile, tg, tn);
                    const int nsub = min(p.group, p.tiles_m - tg * p.group);
                    for (int j = 0; j < nsub && ok; ++j) {
                        const int tm = TWO ? tg * 2 + static_cast<int>(rank) : tg * p.group + j;
                        int img = 0, ty = 0, tx = 0;
                        if (DO_A && p.taps > 0) {       // patch (img, ty, tx) of the output grid
                            const int per_img = p.conv_ty * p.conv_tx;
                            img = tm / per_img;
                            const int rem = tm - img * per_img;
                            ty = rem / p.conv_tx;
                            tx = rem - ty * p.conv_tx;
                        }
                        int tap = 0, cc = 0;
                        const int row_a = tm * kBM;
                        const int row_b = tn * p.bn_rows + (TWO ? static_cast<int>(rank) * (p.bn_rows >> 1) : 0);
                        const int kstep_b = static_cast<int>(span);
                        for (int kb0 = 0; kb0 < p.k_blocks; kb0 += p.kpack) {
                            const int nkb = min(p.kpack, p.k_blocks - kb0);
                            const uint32_t ebar = empty0 + 8 * stage;
                            const long long t0 = dbg ? clock64() : 0;
                            if (!mbar_test_wait(ebar, phase ^ 1) && !mbar_wait_fast(ebar, phase ^ 1, abort_flag, p.err, 1)) { ok = false; break; }
                            if (dbg) t_wait += clock64() - t0;
                            const uint32_t bar = full0 + 8 * stage;
                            uint32_t sa = sa_stage;
                            if ((ENN_DBG_MODE(p) & 1) && filled >= static_cast<uint32_t>(p.stages)) {
                                // development switch: operands stay as first loaded (measures the MMA side alone; results are wrong)
                                if (rank == 0) mbar_arrive(bar);
                            } else if (TWO) {
                                // rank 0 expects the bytes of both CTAs; every load reports to rank 0's barrier
                                if (rank == 0) mbar_expect_tx(bar, kb_tx * nkb);
                                const uint32_t bar0 = mapa_rank(bar, 0);
                                for (int q = 0; q < nkb; ++q, sa += kb_bytes) {
                                    if (DO_A) tma_load_2d_pair(sa, &map_a, bar0, (kb0 + q) * kstep_b, row_a);
                                    if (DO_B) tma_load_2d_pair(sa + a_bytes, &map_b, bar0, (kb0 + q) * kstep_b, row_b);
                                }
                            } else {
                                mbar_expect_tx(bar, kb_tx * nkb);
                                for (int q = 0; q < nkb; ++q, sa += kb_bytes) {
                                    if (DO_A) {
                                        if (p.taps > 0) {
                                            tma_load_4d(sa, &map_a, bar, cc * static_cast<int>(span), tx * p.conv_wt + p.tap_dx[tap], ty * p.conv_ht + p.tap_dy[tap], img);
                                            if (++cc == p.cchunks) { cc = 0; ++tap; }
                                        } else {
                                            tma_load_2d(sa, &map_a, bar, (kb0 + q) * kstep_b, row_a);
                                        }
                                    }
                                    if (DO_B && !bres) tma_load_2d(sa + a_bytes, &map_b, bar, (kb0 + q) * kstep_b, row_b);
                                }
                            }
                            ++filled;
                            sa_stage += stage_bytes;
                            if (++stage == static_cast<uint32_t>(nst)) { stage = 0; phase ^= 1; sa_stage = sa_stage0; }
                        }
                    }
                }
                if (dbg && DO_A) ENN_DBG_PTR(p)[blockIdx.x * 8 + 0] = t_wait;
                if (!ok) {
                    // Give copies already in flight a bounded chance to land before shared memory is released.
                    for (int s = 0; s < nst; ++s)
                        for (uint32_t i = 0; i < (1u << 16); ++i)
                            if (mbar_try_wait(full0 + 8 * s, 0) || mbar_try_wait(full0 + 8 * s, 1)) break;
                }
            };
            if (!split) produce(std::integral_constant<int, 2>{});
            else if (warp == 0) produce(std::integral_constant<int, 0>{});
            else produce(std::integral_constant<int, 1>{});
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // The tensor pipe has next to no queue in front of it: whatever this thread executes between two MMAs is
        // time the pipe idles.  So the MMAs of a k-block go out as one uninterrupted run with every operand already in
        // a register, and the bookkeeping between k-blocks (commit, ring advance, barrier look-up, descriptor
        // addresses) is kept to a few instructions.
        if (lane == 0 && rank == 0) {
            uint32_t stage = 0, phase = 0;
            uint32_t it = 0;
            bool ok = true;
            const uint32_t idesc = p.idesc;
            const uint32_t desc_hi = static_cast<uint32_t>(make_smem_desc(0, span) >> 32);
            const uint32_t lo0 = smem_u32(tiles) >> 4;                 // descriptor address field of stage 0 (16-byte units)
            const uint32_t stage16 = stage_bytes >> 4, kb16 = kb_bytes >> 4, a16 = a_bytes >> 4;
            // K slices per k-block: the whole span, except that the last k-block of a plain GEMM stops after the slices
            // that hold real K (rounded up to 1, 2 or 4: the operands are zero beyond K, so a surplus slice adds nothing).
            const int ks = static_cast<int>(span >> 5);
            int ks_last = ks;
            if (p.taps == 0) {
                const int real = (p.K - (p.k_blocks - 1) * static_cast<int>(span) + 31) >> 5;
                ks_last = real <= 1 ? 1 : (real == 2 ? 2 : 4);
            }
            uint32_t lo_stage = lo0;
            const uint32_t bres_lo = smem_u32(b_resident) >> 4, bstride16 = b_stride >> 4;
            const uint32_t looks = starve ? 64u : (kSpinLimit >> 7);
            if (bres && !mbar_wait_fast(tempty0 + 16, 0, abort_flag, p.err, 5, looks)) ok = false;
            long long t_tempty = 0, t_begin = dbg ? clock64() : 0;
            unsigned long long ns_begin = 0;
            if (dbg) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns_begin));
            for (int tile = tile_first; tile < total_tiles && ok; tile += tile_step, ++it) {
                const uint32_t ab = it & 1, use = it >> 1;
                // wait until the epilogue has drained this accumulator buffer
                const long long t0 = dbg ? clock64() : 0;
                if (!mbar_wait_fast(tempty0 + 8 * ab, (use & 1) ^ 1, abort_flag, p.err, 2, looks)) { ok = false; break; }
                if (dbg) t_tempty += clock64() - t0;
                if (TWO) asm volatile("fence.acq_rel.cluster;" ::: "memory");   // half of the arrivals came from the peer CTA
                tc_fence_after();
                int tg, tn_unused;
                tile_coords(p, tile, tg, tn_unused);
                const int nsub = min(p.group, p.tiles_m - tg * p.group);
                for (int j = 0; j < nsub && ok; ++j) {
                    const uint32_t d_tmem = tmem_base + ab * kMaxBN + j * p.bn_rows;
                    if (ks == 4 && ks_last == 4 && p.kpack == 1 && !bres && p.stages == (TWO ? 6 : 4) && !starve) {
                        // big-GEMM shape: 256-wide tiles give four stages per CTA, six per CTA of a pair
                        if constexpr (TWO) ok = mma_tile_d6<true>(d_tmem, p.k_blocks, stage, phase, full0, empty0, desc_hi, lo0, stage16, a16, idesc, abort_flag, p.err);
                        else ok = mma_tile_d4<false>(d_tmem, p.k_blocks, stage, phase, full0, empty0, desc_hi, lo0, stage16, a16, idesc, abort_flag, p.err);
                        lo_stage = lo0 + stage * stage16;
                        continue;
                    }
                    auto k_loop = [&](auto ks_tag) {
                        constexpr int KS = decltype(ks_tag)::value;
                        int kb = 0;
                        while (kb < p.k_blocks) {
                            const uint32_t bar = full0 + 8 * stage;
                            if (!mbar_test_wait(bar, phase) && !mbar_wait_fast(bar, phase, abort_flag, p.err, 3, looks)) { ok = false; break; }
                            uint32_t lo = lo_stage;
                            const int kb_end = min(kb + p.kpack, p.k_blocks);
                            for (; kb < kb_end; ++kb, lo += kb16) {
                                const uint32_t lo_b = bres ? bres_lo + kb * bstride16 : lo + a16;
                                if (KS == 4 && kb == p.k_blocks - 1 && ks_last != 4) {
                                    if (ks_last == 1) umma_i8_run<TWO, 1>(d_tmem, desc_hi, lo, lo_b, idesc, kb != 0);
                                    else umma_i8_run<TWO, 2>(d_tmem, desc_hi, lo, lo_b, idesc, kb != 0);
                                } else {
                                    umma_i8_run<TWO, KS>(d_tmem, desc_hi, lo, lo_b, idesc, kb != 0);
                                }
                            }
                            // frees the stage (in both CTAs of a pair) when these MMAs have read it
                            if (TWO) umma_commit_pair(empty0 + 8 * stage);
                            else umma_commit(empty0 + 8 * stage);
                            lo_stage += stage16;
                            if (++stage == static_cast<uint32_t>(p.stages)) { stage = 0; phase ^= 1; lo_stage = lo0; }
                        }
                    };
                    if (ks == 4) k_loop(std::integral_constant<int, 4>{});
                    else if (ks == 2) k_loop(std::integral_constant<int, 2>{});
                    else k_loop(std::integral_constant<int, 1>{});
                }
                if (ok) {                                  // accumulator complete
                    if (TWO) umma_commit_pair(tfull0 + 8 * ab);
                    else umma_commit(tfull0 + 8 * ab);
                }
            }
            if (dbg) {
                unsigned long long ns_end;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns_end));
                ENN_DBG_PTR(p)[blockIdx.x * 8 + 3] = t_tempty; ENN_DBG_PTR(p)[blockIdx.x * 8 + 4] = clock64() - t_begin;
                ENN_DBG_PTR(p)[blockIdx.x * 8 + 7] = static_cast<long long>(ns_end - ns_begin);
            }
        }
    } else {
        // ---------------- epilogue: thread = accumulator row, warp = (lane quarter, column share) ----------------
        const int q = warp & 3;                            // TMEM lane group this warp may access
        const int cgrp = (warp - 2) >> 2;                  // which share of the 16-column chunks this warp takes
        const int row_in_tile = q * 32 + lane;
        const int32_t hi_clamp = p.act_max - p.act_min;
        // The lower clamp is added back to the packed bytes.  Unsigned outputs: byte + act_min <= act_max <= 255, so a
        // plain 32-bit add never carries between bytes.  Signed outputs (act_min may be negative): the bytes get
        // act_min + 128 (0..127, sums again <= 255) and the sign bit of every byte is flipped afterwards.
        const uint32_t sign_word = p.a_signed ? 0x80808080u : 0u;
        const uint32_t lo_word = (static_cast<uint32_t>(p.act_min + (p.a_signed ? 128 : 0)) & 0xff) * 0x01010101u;
        const int64_t st_bits = p.out_base | p.out_sn | p.out_sy | p.out_sx | p.bn_data | static_cast<int64_t>(reinterpret_cast<uintptr_t>(p.out));
        const int st_align = (st_bits & 15) == 0 ? 16 : ((st_bits & 7) == 0 ? 8 : 1);   // widest store every row start allows
        const bool st_fast = st_align == 16 && (p.N & 15) == 0;      // every chunk is one aligned 16-byte store
        const bool whole_rows = st_fast && p.taps == 0 && !(ENN_DBG_MODE(p) & 4);   // rows of a full M tile are all real: see the chunk loop
        const int patch_y = p.taps > 0 ? row_in_tile / p.conv_wt : 0;   // this thread's position in the output patch
        const int patch_x = p.taps > 0 ? row_in_tile - patch_y * p.conv_wt : 0;
        const int cps_mod = (p.bn_data >> 4) % kColGroups;
        // Several M tiles of a unit requantised together (shared column constants): flat row-major outputs with aligned rows only.
        const ptrdiff_t res_delta = FADD ? p.add_res - p.out : 0;      // other addend of a fused add: same offsets as the output
        const bool flat = !TWO && st_fast && p.taps == 0 && p.qh == 1 && ENN_DBG_MODE(p) == 0;
        // 32-byte stores: rows and pairs of chunks start on 32-byte boundaries, the constants of all columns are shared
        const bool wide_ok = flat && (st_bits & 31) == 0 && (p.bn_data & 31) == 0 && cols_shared && !p.no_wide_store;
        uint32_t wrot = 0;
        const int epi_g = flat && p.epi_g > 1 ? p.epi_g : 0;      // 0: the one-tile loop below
        const uint32_t rot_step = static_cast<uint32_t>((((p.group + max(epi_g, 1) - 1) / max(epi_g, 1)) * (p.bn_data >> 4)) % kColGroups);
        uint32_t it = 0;
        bool ok = true;
        int loaded_tn = -1;
        long long t_tfull = 0, t_begin = dbg ? clock64() : 0;
        for (int tile = tile_first; tile < total_tiles && ok; tile += tile_step, ++it) {
            int tg, tn;
            tile_coords(p, tile, tg, tn);
            const int nsub = min(p.group, p.tiles_m - tg * p.group);
            const uint32_t ab = it & 1, use = it >> 1;
            const long long t0 = dbg ? clock64() : 0;
            // Chunk c of the buffer = 16 columns cc of M tile j: c = j * cps + cc.  This warp owns chunks
            // cgrp, cgrp + kColGroups, ...; it keeps private copies of the constants of the columns it meets.
            const int cps = p.bn_data >> 4;
            const uint32_t my_cols = s_cols_u32 + (warp - 2) * (kChunksPerWarp * 16 * 16);
            if (!cols_shared && tn != loaded_tn) {
                const int4 *src = reinterpret_cast<const int4 *>(p.cols + static_cast<size_t>(tn) * p.bn_rows);
                __syncwarp();
                for (int i = lane; i < kChunksPerWarp * 16; i += 32) {
                    const int c = (i >> 4) * kColGroups + cgrp;
                    if (c < p.group * cps) {
                        const int4 v = __ldg(src + (c % cps) * 16 + (i & 15));
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_cols + i * 16), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                    }
                }
                __syncwarp();
                loaded_tn = tn;
            }
            if (!mbar_wait(tfull0 + 8 * ab, use & 1, abort_flag, p.err, 4)) { ok = false; break; }
            if (dbg) t_tfull += clock64() - t0;
            tc_fence_after();
            const uint32_t t_row = tmem_base + ab * kMaxBN + (static_cast<uint32_t>(q * 32) << 16);
            const int n_base = tn * p.bn_data;
            const int n_cols = min(p.bn_data, p.N - n_base);

            // Walk this warp's chunks M tile by M tile: chunk c = j * cps + cc belongs to this warp when c = cgrp (mod
            // kColGroups); `first` is the first such cc of M tile j and moves by -cps (mod kColGroups) from one M tile to
            // the next.  Everything that depends only on the M tile (row pointer, row sum) is computed once per j.
            // With shared constants the column groups that get one chunk more than the others change from tile to tile
            // (the chunks of a buffer rarely divide evenly over the groups).
            int first = cgrp;
            if (cols_shared) {
                first += static_cast<int>((it * rot_step) % kColGroups);
                if (first >= kColGroups) first -= kColGroups;
            }
            uint32_t lc_private = my_cols;
            const uint32_t lc_shared = s_cols_u32 + static_cast<uint32_t>(tn * p.bn_rows) * 16;
            const uint8_t *out_tile = p.out + p.out_base + n_base;
            // G M tiles at a time: the 16 bytes of constants a column needs are loaded from shared memory once and serve G
            // outputs (those loads are what saturates first in the one-tile form: two LSU wavefronts per output and warp).
            constexpr bool kPlainPack = MODE == kModeReluSat;      // packed bytes are final: no lower clamp to add, no sign flip
            auto multi_tiles = [&](auto gtag) {
                constexpr int G = decltype(gtag)::value;
                for (int j0 = 0; j0 < nsub; j0 += G, ++wrot) {
                    const int gn = min(G, nsub - j0);
                    const int m0 = (tg * p.group + j0) * kBM;
                    // Decided alike by every epilogue warp: all G tiles lie inside the matrix and every chunk is 16 real columns
                    // (no conditions in the loop); then, where rows and chunk pairs start on 32-byte boundaries, a thread's two
                    // chunks leave as one 32-byte store (a whole sector, half as many requests to the L2 as 16-byte stores).
                    const bool full = gn == G && m0 + G * kBM <= p.M && n_cols == (cps << 4);
                    const bool wide = full && wide_ok;
                    int wfirst = cgrp + static_cast<int>(wrot % kColGroups);      // 32-column chunk wc belongs to group (wc - wrot) mod kColGroups
                    if (wfirst >= kColGroups) wfirst -= kColGroups;
                    if (wide ? wfirst < (cps >> 1) : first < cps) {
                        uint8_t *orow[G];
                        bool live[G];
                        int32_t asum_term[G];
                        uint32_t t_tile[G];
#pragma unroll
                        for (int i = 0; i < G; ++i) {
                            const int m = m0 + i * kBM + row_in_tile;
                            live[i] = i < gn && m < p.M;
                            orow[i] = const_cast<uint8_t *>(out_tile) + static_cast<int64_t>(live[i] ? m : 0) * p.out_sx;
                            // a slot the unit does not have re-reads the first one (unused)
                            t_tile[i] = t_row + (j0 + i < p.group ? j0 + i : j0) * p.bn_rows;
                            asum_term[i] = 0;
                            if (ASUM) {
                                uint32_t rs;
                                tmem_ld_x1(t_tile[i] + p.bn_data, rs);       // warp-collective
                                tmem_ld_wait();
                                asum_term[i] = p.zw_eff * static_cast<int32_t>(rs);
                            }
                        }
                        // One chunk loop.  STORE 0: 16-byte global stores under the per-row and per-chunk conditions; 1: stores
                        // without conditions.  CW: 16-column chunks per step (2 with STORE 1 only).
                        auto chunks = [&](auto storetag, auto widthtag) {
                            constexpr int STORE = decltype(storetag)::value;
                            constexpr int CW = decltype(widthtag)::value;
                            for (int c0 = CW == 2 ? wfirst << 5 : first << 4; c0 < (cps << 4); c0 += kColGroups * 16 * CW) {
                                const uint32_t lc = (CW == 2 || cols_shared) ? lc_shared + c0 * 16 : lc_private;
                                const uint8_t *lcp = s_cols_sp + (lc - s_cols_u32);
                                if (CW == 1) lc_private += 256;
                                uint32_t w[G][4 * CW];
                                // Accumulators: one 16-column load per tile while the registers allow it (G <= 2), else 8 columns.
                                constexpr int LW = G <= 2 ? 16 : 8;
#pragma unroll
                                for (int part = 0; part < 16 * CW / LW; ++part) {
                                    uint32_t r[G][LW];
#pragma unroll
                                    for (int i = 0; i < G; ++i) {      // warp-collective
                                        if constexpr (LW == 16) tmem_ld_x16(t_tile[i] + c0 + 16 * part, r[i]);
                                        else tmem_ld_x8(t_tile[i] + c0 + 8 * part, r[i]);
                                    }
                                    tmem_ld_wait();
#pragma unroll
                                    for (int jj = 0; jj < LW / 4; ++jj) {
                                        int32_t y[G][4];
#pragma unroll
                                        for (int b = 0; b < 4; ++b) {
                                            ColRegs cv;
                                            ld_col_shared<MODE>(lcp + (part * LW + jj * 4 + b) * 16, cv);
#pragma unroll
                                            for (int i = 0; i < G; ++i) {
                                                int32_t acc = static_cast<int32_t>(r[i][jj * 4 + b]);
                                                if (ASUM) acc -= asum_term[i];
                                                y[i][b] = tc_requant<MODE>(acc, cv, hi_clamp, p.out_zp, p.act_min, p.act_max);
                                            }
                                        }
#pragma unroll
                                        for (int i = 0; i < G; ++i) {
                                            const uint32_t hi = pack_sat_u8_tc(y[i][3], y[i][2], 0);
                                            const uint32_t pk = pack_sat_u8_tc(y[i][1], y[i][0], hi);
                                            w[i][part * (LW / 4) + jj] = kPlainPack ? pk : ((pk + lo_word) ^ sign_word);
                                        }
                                    }
                                }
                                if constexpr (FADD) {
#pragma unroll
                                    for (int i = 0; i < G; ++i)
                                        if (STORE == 1 || (live[i] && c0 < n_cols)) {
#pragma unroll
                                            for (int h = 0; h < CW; ++h) {
                                                uint32_t (&wq)[4] = *reinterpret_cast<uint32_t (*)[4]>(&w[i][4 * h]);
                                                fadd_chunk(wq, orow[i] + c0 + 16 * h + res_delta, fadd);
                                            }
                                        }
                                }
                                if constexpr (CW == 2) {
#pragma unroll
                                    for (int i = 0; i < G; ++i)
                                        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(orow[i] + c0), "r"(w[i][0]), "r"(w[i][1]),
                                                     "r"(w[i][2]), "r"(w[i][3]), "r"(w[i][4]), "r"(w[i][5]), "r"(w[i][6]), "r"(w[i][7])
                                                     : "memory");
                                } else if (STORE == 1 || c0 < n_cols) {
#pragma unroll
                                    for (int i = 0; i < G; ++i)
                                        if (STORE == 1 || live[i]) *reinterpret_cast<uint4 *>(orow[i] + c0) = make_uint4(w[i][0], w[i][1], w[i][2], w[i][3]);
                                }
                            }
                        };
                        constexpr std::integral_constant<int, 1> one{};
                        if (wide) chunks(one, std::integral_constant<int, 2>{});
                        else if (full) chunks(one, one);
                        else chunks(std::integral_constant<int, 0>{}, one);
                    }
                    first -= cps_mod;
                    if (first < 0) first += kColGroups;
                }
            };
            if (epi_g == 4) multi_tiles(std::integral_constant<int, 4>{});
            else if (epi_g == 2) multi_tiles(std::integral_constant<int, 2>{});
            for (int j = 0; j < nsub && epi_g == 0 && !(ENN_DBG_MODE(p) & 2); ++j) {
                if (first < cps) {
                    const int tm = TWO ? tg * 2 + static_cast<int>(rank) : tg * p.group + j;
                    const int m = tm * kBM + row_in_tile;
                    bool row_ok = m < p.M;
                    uint8_t *orow;
                    if (p.taps > 0) {
                        const int per_img = p.conv_ty * p.conv_tx;
                        const int img = tm / per_img, rem = tm - img * per_img;
                        const int ty = rem / p.conv_tx, tx = rem - ty * p.conv_tx;
                        const int qy = ty * p.conv_ht + patch_y, qx = tx * p.conv_wt + patch_x;
                        row_ok = patch_y < p.conv_ht && qy < p.qh && qx < p.qw;
                        orow = const_cast<uint8_t *>(out_tile) + img * p.out_sn + (row_ok ? qy : 0) * p.out_sy + (row_ok ? qx : 0) * p.out_sx;
                    } else if (p.qh == 1) {
                        orow = const_cast<uint8_t *>(out_tile) + static_cast<int64_t>(row_ok ? m : 0) * p.out_sx;
                    } else {
                        const int mq = row_ok ? m : 0;
                        const int img = mq / (p.qh * p.qw), rem = mq - img * (p.qh * p.qw);
                        const int qy = rem / p.qw, qx = rem - qy * p.qw;
                        orow = const_cast<uint8_t *>(out_tile) + img * p.out_sn + qy * p.out_sy + qx * p.out_sx;
                    }
                    const uint32_t t_tile = t_row + j * p.bn_rows;
                    int32_t asum_term = 0;
                    if (ASUM) {
                        uint32_t rs;
                        tmem_ld_x1(t_tile + p.bn_data, rs);       // warp-collective
                        tmem_ld_wait();
                        asum_term = p.zw_eff * static_cast<int32_t>(rs);
                    }
                    // Requantises the 8 accumulators of one half chunk into two packed words.
                    auto half_chunk = [&](const uint32_t (&r)[8], uint32_t lc_half, uint32_t &w0, uint32_t &w1) {
#pragma unroll
                        for (int jj = 0; jj < 2; ++jj) {
                            int32_t y[4];
#pragma unroll
                            for (int b = 0; b < 4; ++b) {
                                ColRegs cv;
                                ld_col_shared<MODE>(s_cols_sp + (lc_half - s_cols_u32) + (jj * 4 + b) * 16, cv);
                                int32_t acc = static_cast<int32_t>(r[jj * 4 + b]);
                                if (ASUM) acc -= asum_term;
                                y[b] = tc_requant<MODE>(acc, cv, hi_clamp, p.out_zp, p.act_min, p.act_max);
                            }
                            const uint32_t hi = pack_sat_u8_tc(y[3], y[2], 0);
                            const uint32_t pk = pack_sat_u8_tc(y[1], y[0], hi);
                            (jj == 0 ? w0 : w1) = kPlainPack ? pk : ((pk + lo_word) ^ sign_word);
                        }
                    };
                    if (whole_rows && n_cols == (cps << 4) && m + (kBM - 1 - row_in_tile) < p.M) {
                        // The usual case, decided per warp: the M tile lies inside the matrix, every chunk is 16 real columns and
                        // one aligned 16-byte store.  No per-thread conditions, so nothing here diverges.
                        for (int c0 = first << 4; c0 < (cps << 4); c0 += kColGroups * 16, lc_private += 256) {
                            const uint32_t lc = cols_shared ? lc_shared + c0 * 16 : lc_private;
                            uint32_t w[4];
#pragma unroll
                            for (int half = 0; half < 2; ++half) {
                                uint32_t r[8];
                                tmem_ld_x8(t_tile + c0 + 8 * half, r);      // warp-collective
                                tmem_ld_wait();
                                half_chunk(r, lc + half * 128, w[half * 2], w[half * 2 + 1]);
                            }
                            if constexpr (FADD) fadd_chunk(w, orow + c0 + res_delta, fadd);
                            *reinterpret_cast<uint4 *>(orow + c0) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    } else {
                    for (int c0 = first << 4; c0 < (cps << 4); c0 += kColGroups * 16, lc_private += 256) {
                        const uint32_t lc = cols_shared ? lc_shared + c0 * 16 : lc_private;
                        // two 8-column loads per chunk: half the accumulator registers live at a time
                        uint32_t w[4];
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            uint32_t r[8];
                            tmem_ld_x8(t_tile + c0 + 8 * half, r);      // warp-collective
                            tmem_ld_wait();
                            if (row_ok && c0 < n_cols) half_chunk(r, lc + half * 128, w[half * 2], w[half * 2 + 1]);
                        }
                        if (row_ok && c0 < n_cols) {
                            if constexpr (FADD) fadd_chunk(w, orow + c0 + res_delta, fadd);      // fused operators have 16-byte rows (plan)
                            if (ENN_DBG_MODE(p) & 4) {
                                // development switch: no stores (isolates the store path; only one lane keeps the values alive)
                                if ((w[0] ^ w[1] ^ w[2] ^ w[3]) == 0x12345678u && lane == 33) orow[0] = 1;
                            } else if (st_fast) {
                                *reinterpret_cast<uint4 *>(orow + c0) = make_uint4(w[0], w[1], w[2], w[3]);
                            } else {
                                const int left = n_cols - c0;
                                if (st_align == 16 && left >= 16) {
                                    *reinterpret_cast<uint4 *>(orow + c0) = make_uint4(w[0], w[1], w[2], w[3]);
                                } else if (st_align >= 8 && left >= 8) {
                                    *reinterpret_cast<uint2 *>(orow + c0) = make_uint2(w[0], w[1]);
                                    if (left >= 16) {
                                        *reinterpret_cast<uint2 *>(orow + c0 + 8) = make_uint2(w[2], w[3]);
                                    } else {
#pragma unroll
                                        for (int b = 8; b < 16; ++b)
                                            if (b < left) orow[c0 + b] = static_cast<uint8_t>(w[b >> 2] >> (8 * (b & 3)));
                                    }
                                } else {
#pragma unroll
                                    for (int b = 0; b < 16; ++b)
                                        if (b < left) orow[c0 + b] = static_cast<uint8_t>(w[b >> 2] >> (8 * (b & 3)));
                                }
                            }
                        }
                    }
                }
                }
                // first chunk of this warp in the next M tile
                first -= cps_mod;
                if (first < 0) first += kColGroups;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (TWO) mbar_arrive_cluster(mapa_rank(tempty0 + 8 * ab, 0));
                else mbar_arrive(tempty0 + 8 * ab);
            }
        }
        if (dbg && threadIdx.x == 64) { ENN_DBG_PTR(p)[blockIdx.x * 8 + 5] = t_tfull; ENN_DBG_PTR(p)[blockIdx.x * 8 + 6] = clock64() - t_begin; }
    }

    tc_fence_before();
    __syncthreads();
    if (TWO) cluster_sync_all();        // no signal may reach a CTA that has left
    tc_fence_after();
    if (warp == 1) {
        if (TWO) tmem_dealloc_pair(tmem_base, 512);
        else tmem_dealloc(tmem_base, 512);
    }
}

// ------------------------------------------------------------------------------------------------------
// GEMV for FullyConnected / 1x1 convolutions with very few rows (M <= 8): the contraction is bound by reading the
// N x K weight matrix once from HBM, so tensor cores are not used.  A warp owns one output column: its lanes
// stream that column's K bytes with 16-byte loads (the weights are the same K-major int8 tiles the tensor-core
// kernel uses), multiply with dp4a against the activations held in shared memory, and reduce with shuffles.
// The epilogue constants and the zero-point folding are the tensor-core kernel's (ColParam).
// ------------------------------------------------------------------------------------------------------
constexpr int kGemvMaxM = 8;
constexpr int kGemvWarps = 8;
constexpr int kGemvAhead = 8;       // 16-byte weight loads per lane issued before anything else

template <bool A_SIGNED>
__device__ __forceinline__ int32_t dp4a_as(uint32_t a, uint32_t w, int32_t c) {
    int32_t d;
    if (A_SIGNED)
        asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(w), "r"(c));
    else
        asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(w), "r"(c));
    return d;
}

template <bool A_SIGNED, int M>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_kernel(const uint8_t *__restrict__ a, const int8_t *__restrict__ w, const ColParam *__restrict__ cols, uint8_t *__restrict__ out,
            int N, int K, int k_pad, int bn_rows, int bn_data, int zw_eff, int out_zp, int act_min, int act_max) {
    extern __shared__ uint4 gemv_smem[];            // M rows of K bytes
    const int k16 = K >> 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * kGemvWarps + warp;
    const bool active = n < N;
    const int tn = active ? n / bn_data : 0, r = active ? n - tn * bn_data : 0;
    const uint4 *wrow = reinterpret_cast<const uint4 *>(w + (static_cast<size_t>(tn) * bn_rows + r) * k_pad);
    // The weights are the operator's constants: the first kGemvAhead 512-byte pieces of this warp's column (all of it up
    // to K = 4096) are requested before the wait on the kernel that produces the activations and before the
    // activations are staged, so that the whole weight stream is in flight from the first instruction on.
    pdl_trigger();
    uint4 wpre[kGemvAhead];
#pragma unroll
    for (int u = 0; u < kGemvAhead; ++u) {
        const int i = lane + 32 * u;
        wpre[u] = active && i < k16 ? __ldg(wrow + i) : make_uint4(0u, 0u, 0u, 0u);
    }
    pdl_wait();
    for (int i = threadIdx.x; i < M * k16; i += blockDim.x) gemv_smem[i] = __ldg(reinterpret_cast<const uint4 *>(a) + i);
    __syncthreads();
    if (!active) return;
    int32_t acc[M], asum[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = asum[m] = 0;
    auto mac = [&](int i, const uint4 &wv) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const uint4 av = gemv_smem[m * k16 + i];
            acc[m] = dp4a_as<A_SIGNED>(av.x, wv.x, acc[m]);
            acc[m] = dp4a_as<A_SIGNED>(av.y, wv.y, acc[m]);
            acc[m] = dp4a_as<A_SIGNED>(av.z, wv.z, acc[m]);
            acc[m] = dp4a_as<A_SIGNED>(av.w, wv.w, acc[m]);
            if (zw_eff != 0) {
                asum[m] = dp4a_as<A_SIGNED>(av.x, 0x01010101u, asum[m]);
                asum[m] = dp4a_as<A_SIGNED>(av.y, 0x01010101u, asum[m]);
                asum[m] = dp4a_as<A_SIGNED>(av.z, 0x01010101u, asum[m]);
                asum[m] = dp4a_as<A_SIGNED>(av.w, 0x01010101u, asum[m]);
            }
        }
    };
#pragma unroll
    for (int u = 0; u < kGemvAhead; ++u) {
        const int i = lane + 32 * u;
        if (i < k16) mac(i, wpre[u]);
    }
#pragma unroll 4
    for (int i = lane + 32 * kGemvAhead; i < k16; i += 32) mac(i, __ldg(wrow + i));
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], off);
            asum[m] += __shfl_xor_sync(0xffffffffu, asum[m], off);
        }
    if (lane == 0) {
        const ColParam c = cols[static_cast<size_t>(tn) * bn_rows + r];
        const int4 cv = make_int4(c.mult, c.addend, c.esh, c.bias);
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const int32_t v = acc[m] - zw_eff * asum[m];
            out[static_cast<size_t>(m) * N + n] = static_cast<uint8_t>(tc_requant<kModeGeneral>(v, cv, act_max - act_min, out_zp, act_min, act_max) + act_min);
        }
    }
}

template <bool A_SIGNED>
void launch_gemv(int M, const void *a, const void *w, const ColParam *cols, void *out, const TcParams &p, int k_pad, cudaStream_t s) {
    const int blocks = (p.N + kGemvWarps - 1) / kGemvWarps;
    const size_t smem = static_cast<size_t>(M) * p.K;
#define ENN_GEMV(MM)                                                                                                          \
    launch_pdl(gemv_kernel<A_SIGNED, MM>, dim3(blocks), dim3(kGemvWarps * 32), smem, s, static_cast<const uint8_t *>(a),      \
               static_cast<const int8_t *>(w), cols, static_cast<uint8_t *>(out), p.N, p.K, k_pad, p.bn_rows, p.bn_data, p.zw_eff,  \
               p.out_zp, p.act_min, p.act_max)
    switch (M) {
        case 1: ENN_GEMV(1); break;
        case 2: ENN_GEMV(2); break;
        case 3: ENN_GEMV(3); break;
        case 4: ENN_GEMV(4); break;
        case 5: ENN_GEMV(5); break;
        case 6: ENN_GEMV(6); break;
        case 7: ENN_GEMV(7); break;
        default: ENN_GEMV(8); break;
    }
#undef ENN_GEMV
}

// ------------------------------------------------------------------------------------------------------
// im2col: gathers the A operand of a convolution that the kernel above cannot read in place (taps, strides,
// dilation, channel counts that are not a multiple of 16) into a [M][Kp] byte matrix in scratch memory.
// Positions outside the image are written as the input zero point (the reference's pad kernels do the same,
// PadConvertKernels.cpp:241-373), so they contribute (za - za) * w = 0 and the bias fold is the same for every
// output position; bytes k >= K pad the row to a multiple of 16 and meet zero weights.
// Row m = (img, oy, ox) of an oh x ow grid; column k = (ky * kw + kx) * cin + c;
// input pixel iy = oy * sy + ky * dy + y0, ix = ox * sx + kx * dx + x0.
// ------------------------------------------------------------------------------------------------------
struct Im2colGeom {
    int32_t n, h, w, cin;
    int32_t oh, ow, kh, kw;
    int32_t sy, sx, dy, dx, y0, x0;
    int32_t K, Kp;
    uint32_t fill;      // input zero point replicated in 4 bytes
    const int2 *ktab;   // per reduction index k < Kp: {byte offset from the tap-(0,0) pixel, dy << 16 | (dx & 0xffff)}; offset < 0: padding
};

// One thread writes 16 output bytes.  GRAN = 16 / 8: cin is a multiple of GRAN, so the 16 bytes are 1 / 2 aligned
// loads; GRAN = 1: any channel count, one byte at a time through the per-k offset table.
template <int GRAN>
__global__ void im2col_kernel(Im2colGeom g, const uint8_t *__restrict__ in, uint8_t *__restrict__ out, int64_t total16) {
    const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= total16) return;
    const int kp16 = g.Kp >> 4;
    const int k0 = static_cast<int>(t % kp16) << 4;
    int64_t m = t / kp16;
    const int ox = static_cast<int>(m % g.ow);
    m /= g.ow;
    const int oy = static_cast<int>(m % g.oh);
    const int img = static_cast<int>(m / g.oh);
    const int by = oy * g.sy + g.y0, bx = ox * g.sx + g.x0;      // input pixel of tap (0, 0)
    uint4 v = make_uint4(0, 0, 0, 0);
    if (GRAN == 16) {
        if (k0 < g.K) {
            const int tap = k0 / g.cin, c = k0 - tap * g.cin;
            const int ky = tap / g.kw, kx = tap - ky * g.kw;
            const int iy = by + ky * g.dy, ix = bx + kx * g.dx;
            if (iy >= 0 && iy < g.h && ix >= 0 && ix < g.w)
                v = __ldg(reinterpret_cast<const uint4 *>(in + ((static_cast<int64_t>(img) * g.h + iy) * g.w + ix) * g.cin + c));
            else
                v = make_uint4(g.fill, g.fill, g.fill, g.fill);
        }
    } else if (GRAN == 8) {
        uint2 h[2] = {make_uint2(0, 0), make_uint2(0, 0)};
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const int k = k0 + 8 * s;
            if (k < g.K) {
                const int tap = k / g.cin, c = k - tap * g.cin;
                const int ky = tap / g.kw, kx = tap - ky * g.kw;
                const int iy = by + ky * g.dy, ix = bx + kx * g.dx;
                if (iy >= 0 && iy < g.h && ix >= 0 && ix < g.w)
                    h[s] = __ldg(reinterpret_cast<const uint2 *>(in + ((static_cast<int64_t>(img) * g.h + iy) * g.w + ix) * g.cin + c));
                else
                    h[s] = make_uint2(g.fill, g.fill);
            }
        }
        v = make_uint4(h[0].x, h[0].y, h[1].x, h[1].y);
    } else {
        const uint8_t *base = in + ((static_cast<int64_t>(img) * g.h + by) * g.w + bx) * g.cin;
        uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int2 e = __ldg(g.ktab + k0 + i);
            uint32_t b = 0;
            const int dy = e.y >> 16, dx = static_cast<int16_t>(e.y & 0xffff);
            if (k0 + i < g.K) {
                const int iy = by + dy, ix = bx + dx;
                b = g.fill & 0xff;
                if (iy >= 0 && iy < g.h && ix >= 0 && ix < g.w) b = __ldg(base + e.x);
            }
            w[i >> 2] |= b << (8 * (i & 3));
        }
        v = make_uint4(w[0], w[1], w[2], w[3]);
    }
    reinterpret_cast<uint4 *>(out)[t] = v;
}

// ------------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------------
// Copies an NHWC tensor into a larger one with `lo_y` / `lo_x` extra rows / columns before and extra ones after, filled
// with the input zero point: what the reference's pad kernels produce (PadConvertKernels.cpp:241-373), so that the
// tap boxes of the implicit convolution never meet a border.  One thread writes 16 bytes (C % 16 == 0).
__global__ void pad_nhwc_kernel(const uint8_t *__restrict__ in, uint8_t *__restrict__ out, int n, int h, int w, int c, int hp, int wp, int lo_y,
                                int lo_x, uint32_t fill, int64_t total16) {
    const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= total16) return;
    const int c16 = c >> 4;
    const int cc = static_cast<int>(t % c16);
    int64_t r = t / c16;
    const int x = static_cast<int>(r % wp);
    r /= wp;
    const int y = static_cast<int>(r % hp);
    const int img = static_cast<int>(r / hp);
    const int iy = y - lo_y, ix = x - lo_x;
    uint4 v = make_uint4(fill, fill, fill, fill);
    if (iy >= 0 && iy < h && ix >= 0 && ix < w) v = __ldg(reinterpret_cast<const uint4 *>(in + ((static_cast<int64_t>(img) * h + iy) * w + ix) * c) + cc);
    reinterpret_cast<uint4 *>(out)[t] = v;
}

void launch_im2col(const Im2colGeom &ig, const void *in, uint8_t *dst, int64_t total16, unsigned blocks, cudaStream_t s) {
    const uint8_t *src = static_cast<const uint8_t *>(in);
    const uintptr_t a = reinterpret_cast<uintptr_t>(in);
    if ((ig.cin & 15) == 0 && (a & 15) == 0) im2col_kernel<16><<<blocks, 256, 0, s>>>(ig, src, dst, total16);
    else if ((ig.cin & 7) == 0 && (a & 7) == 0) im2col_kernel<8><<<blocks, 256, 0, s>>>(ig, src, dst, total16);
    else if (ig.ktab) im2col_kernel<1><<<blocks, 256, 0, s>>>(ig, src, dst, total16);
}

// ------------------------------------------------------------------------------------------------------
// First-layer convolution: 3x3 taps over 3 input channels (K = 27), any stride, Cout a multiple of 16.  Gathering
// 27-byte rows into a matrix and running the GEMM costs two extra passes over a matrix three times the size of the
// image, for almost no MMA work; here a thread owns a few output pixels, builds their 27 window bytes in registers
// (three 9-byte row segments, read with aligned words and funnel shifts), and walks the output channels with the
// packed int8 weights and epilogue constants of the tensor-core plan broadcast from shared memory: 7 dp4a and the
// same exact requantisation per output byte.  Border pixels take a bytewise path with the input zero point as fill.
// ------------------------------------------------------------------------------------------------------
template <bool A_SIGNED>
__device__ __forceinline__ int32_t dp4a_aw(uint32_t a, uint32_t w, int32_t c) {
    int32_t d;
    if (A_SIGNED) asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(w), "r"(c));
    else asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(w), "r"(c));
    return d;
}

// Byte k of the 27-byte window stream = byte (k % 9) of row segment k / 9; a row segment sits in three words.
template <int D>
__device__ __forceinline__ uint32_t window_word(const uint32_t (&src)[9]) {
    uint32_t v = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int k = 4 * D + i;
        if (k < 27) {
            const int sb = (k / 9) * 12 + (k % 9);      // byte index in src viewed as 36 bytes
            // place byte sb % 4 of src[sb / 4] at position i of v, keep v's other bytes
            const uint32_t sel = (i == 0 ? 0x3214u : i == 1 ? 0x3240u : i == 2 ? 0x3410u : 0x4210u) + (static_cast<uint32_t>(sb % 4) << (4 * i));
            v = __byte_perm(v, src[sb / 4], sel);
        }
    }
    return v;
}

constexpr int kFirstLayerPixels = 2;       // output pixels per thread of conv3x3c3_kernel (1: 103 us, 2: 95 us, 4: 102 us on the MobileNetV2 stem)

struct Conv3x3c3Params {
    int32_t n, h, w, oh, ow, sy, sx, y0, x0;
    int32_t M, N, k_pad;
    int32_t zw_eff, act_min, act_max, out_zp;
    uint32_t fill;
    int64_t in_bytes;
};

template <bool A_SIGNED, bool ASUM, int MODE>
__global__ void __launch_bounds__(256) conv3x3c3_kernel(Conv3x3c3Params g, const uint8_t *__restrict__ in, const int8_t *__restrict__ wq,
                                                        const ColParam *__restrict__ cols, uint8_t *__restrict__ out) {
    extern __shared__ uint4 smem_q[];
    uint4 *s_w = smem_q;                 // [N][2] : 32 weight bytes per output channel (27 real, 5 zero)
    uint4 *s_c = smem_q + 2 * g.N;       // [N]    : epilogue constants
    for (int i = threadIdx.x; i < 2 * g.N; i += blockDim.x)
        s_w[i] = *reinterpret_cast<const uint4 *>(wq + static_cast<size_t>(i >> 1) * g.k_pad + (i & 1) * 16);
    for (int i = threadIdx.x; i < g.N; i += blockDim.x) s_c[i] = *reinterpret_cast<const uint4 *>(cols + i);
    __syncthreads();
    pdl_wait();         // weights and constants above belong to the plan; the image may come from the kernel before
    pdl_trigger();
    const uint8_t *sw_p = reinterpret_cast<const uint8_t *>(s_w), *sc_p = reinterpret_cast<const uint8_t *>(s_c);
    constexpr bool kPlainPack = MODE == kModeReluSat;      // packed bytes are final: no lower clamp to add, no sign flip
    const int32_t hi_clamp = g.act_max - g.act_min;
    // lower clamp added back per byte; signed outputs go through act_min + 128 and a sign-bit flip (no carries between bytes)
    const uint32_t sign_word = A_SIGNED ? 0x80808080u : 0u;
    const uint32_t lo_word = (static_cast<uint32_t>(g.act_min + (A_SIGNED ? 128 : 0)) & 0xff) * 0x01010101u;

    // Window of output pixel m as 7 words (27 bytes + 1 zero) and its row-sum term.
    auto load_window = [&](int m, uint32_t (&a)[7], int32_t &asum_term) {
        const int ox = m % g.ow, t = m / g.ow;
        const int oy = t % g.oh, img = t / g.oh;
        const int iy0 = oy * g.sy + g.y0, ix0 = ox * g.sx + g.x0;
        uint32_t src[9];
        const int64_t row0 = ((static_cast<int64_t>(img) * g.h + iy0) * g.w + ix0) * 3;
        const bool interior = iy0 >= 0 && iy0 + 3 <= g.h && ix0 >= 0 && ix0 + 3 <= g.w &&
                              row0 + 2ll * g.w * 3 + 12 <= g.in_bytes;      // the aligned words of the last row stay inside the tensor
        if (interior) {
#pragma unroll
            for (int r = 0; r < 3; ++r) {
                const uint8_t *pr = in + row0 + static_cast<int64_t>(r) * g.w * 3;
                const uintptr_t pa = reinterpret_cast<uintptr_t>(pr);
                const uint32_t *q = reinterpret_cast<const uint32_t *>(pa & ~static_cast<uintptr_t>(3));
                const uint32_t sh = static_cast<uint32_t>(pa & 3) * 8;
                const uint32_t q0 = __ldg(q), q1 = __ldg(q + 1), q2 = __ldg(q + 2);
                src[3 * r] = __funnelshift_r(q0, q1, sh);
                src[3 * r + 1] = __funnelshift_r(q1, q2, sh);
                src[3 * r + 2] = q2 >> sh;
            }
        } else {
#pragma unroll
            for (int r = 0; r < 3; ++r) {
                const int iy = iy0 + r;
                uint32_t wd[3] = {0, 0, 0};
#pragma unroll
                for (int b = 0; b < 9; ++b) {
                    const int ix = ix0 + b / 3;
                    uint32_t v = g.fill & 0xff;
                    if (iy >= 0 && iy < g.h && ix >= 0 && ix < g.w) v = in[((static_cast<int64_t>(img) * g.h + iy) * g.w + ix) * 3 + b % 3];
                    wd[b / 4] |= v << (8 * (b % 4));
                }
                src[3 * r] = wd[0]; src[3 * r + 1] = wd[1]; src[3 * r + 2] = wd[2];
            }
        }
        a[0] = window_word<0>(src); a[1] = window_word<1>(src); a[2] = window_word<2>(src); a[3] = window_word<3>(src);
        a[4] = window_word<4>(src); a[5] = window_word<5>(src); a[6] = window_word<6>(src);
        asum_term = 0;
        if (ASUM) {
            int32_t sa = 0;
#pragma unroll
            for (int d = 0; d < 7; ++d) sa = dp4a_aw<A_SIGNED>(a[d], d == 6 ? 0x00010101u : 0x01010101u, sa);
            asum_term = g.zw_eff * sa;
        }
    };

    // A thread owns kFirstLayerPixels neighbouring output pixels: every weight and constant word fetched from shared
    // memory (three 16-byte loads per output channel, the busiest unit of this kernel) then serves that many outputs.
    constexpr int P = kFirstLayerPixels;
    for (int m = P * (blockIdx.x * blockDim.x + threadIdx.x); m < g.M; m += P * gridDim.x * blockDim.x) {
        uint32_t a[P][7];
        int32_t asum[P];
#pragma unroll
        for (int i = 0; i < P; ++i) load_window(m + i < g.M ? m + i : m, a[i], asum[i]);
        uint8_t *orow = out + static_cast<int64_t>(m) * g.N;
        for (int n0 = 0; n0 < g.N; n0 += 16) {
            uint32_t wout[P][4];
            // Plain shared loads from pointers into the shared array: the per-channel part of every address is an immediate.
            const uint8_t *wp = sw_p + n0 * 32, *cp = sc_p + n0 * 16;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                int32_t y[P][4];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const int nl = jj * 4 + b;
                    const uint4 w0 = *reinterpret_cast<const uint4 *>(wp + nl * 32);
                    const uint4 w1 = *reinterpret_cast<const uint4 *>(wp + nl * 32 + 16);
                    ColRegs cv;
                    ld_col_shared<MODE>(cp + nl * 16, cv);
#pragma unroll
                    for (int i = 0; i < P; ++i) {
                        int32_t acc = 0;
                        acc = dp4a_aw<A_SIGNED>(a[i][0], w0.x, acc);
                        acc = dp4a_aw<A_SIGNED>(a[i][1], w0.y, acc);
                        acc = dp4a_aw<A_SIGNED>(a[i][2], w0.z, acc);
                        acc = dp4a_aw<A_SIGNED>(a[i][3], w0.w, acc);
                        acc = dp4a_aw<A_SIGNED>(a[i][4], w1.x, acc);
                        acc = dp4a_aw<A_SIGNED>(a[i][5], w1.y, acc);
                        acc = dp4a_aw<A_SIGNED>(a[i][6], w1.z, acc);
                        if (ASUM) acc -= asum[i];
                        y[i][b] = tc_requant<MODE>(acc, cv, hi_clamp, g.out_zp, g.act_min, g.act_max);
                    }
                }
#pragma unroll
                for (int i = 0; i < P; ++i) {
                    const uint32_t hi = pack_sat_u8_tc(y[i][3], y[i][2], 0);
                    const uint32_t pk = pack_sat_u8_tc(y[i][1], y[i][0], hi);
                    wout[i][jj] = kPlainPack ? pk : ((pk + lo_word) ^ sign_word);
                }
            }
#pragma unroll
            for (int i = 0; i < P; ++i)
                if (m + i < g.M) *reinterpret_cast<uint4 *>(orow + static_cast<int64_t>(i) * g.N + n0) = make_uint4(wout[i][0], wout[i][1], wout[i][2], wout[i][3]);
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// One GEMM launch: an operator is one of these (convolution, FullyConnected) or one per output parity class
// (transposed convolution).
struct TcGemm {
    TcParams prm{};
    CUtensorMap map_b{};
    CUtensorMap map_a{};
    const void *map_a_ptr = nullptr;   // A pointer map_a was encoded for
    // Small cache of activation maps for callers that alternate between a few input buffers.
    static constexpr int kMapCache = 8;
    CUtensorMap map_cache[kMapCache];
    const void *map_cache_ptr[kMapCache] = {nullptr};
    int map_cache_next = 0;
    void *w_dev = nullptr;
    void *cols_dev = nullptr;
    void *ktab_dev = nullptr;          // im2col offset table (byte-granular gather only)
    size_t smem_bytes = 0;
    int grid = 0;
    int threads = 0;                   // kThreads (separate B producer warp) for long-K GEMMs, else kThreadsOneProducer
    bool gather = false;               // A is gathered into scratch by im2col first
    bool first_layer = false;          // 3x3 taps over 3 channels: conv3x3c3_kernel instead of gather + GEMM
    bool use_gemv = false;             // M <= 8 read in place: weight-streaming GEMV instead of the tensor-core kernel
    // Implicit convolution (stride-1 taps read as TMA boxes, no gathered matrix): the source is either the caller's
    // tensor (input zero point 0: the zero OOB fill is already right) or a zero-point padded copy in scratch.
    bool implicit = false;
    bool padded = false;
    bool runs_pad = false;             // this GEMM launches the pad pass (the first padded GEMM of the operator)
    int32_t pad_lo_y = 0, pad_lo_x = 0, hp = 0, wp = 0;
    Im2colGeom ig{};
    CUtensorMap map_a_static{};        // A map over the library's static scratch array (no-allocation entry point)
    const void *map_a_static_ptr = nullptr;
};

struct TcPlan {
    std::vector<TcGemm> gemms;
    void *scratch = nullptr;           // im2col matrix, shared by the GEMMs of the op (they run in stream order)
    size_t scratch_bytes = 0;
    bool fan_out = false;              // the GEMMs are independent (deconvolution classes): run them side by side
    int32_t *err_host = nullptr;       // pinned + mapped
    int32_t *err_dev = nullptr;
    bool starve_next = false;          // the next execute runs the bounded-wait self-test (tc_test_starve_next)
    bool fused_add = false;            // convolution + quantized add (tc_fuse_add)
    const uint8_t *residual = nullptr; // the add's other input for the next execute
};

CUtensorMapSwizzle swizzle_of(uint32_t span) {
    return span == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (span == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

bool encode_2d(enn_b200_context *ctx, CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer, uint64_t pitch,
               uint32_t box_inner, uint32_t box_outer) {
    EncodeTiledFn fn = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled);
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {pitch};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_of(box_inner), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// NHWC activation tensor {C, W, H, N} with a box of {span channels, box_w, box_h, 1}.
bool encode_nhwc(enn_b200_context *ctx, CUtensorMap *map, const void *base, uint64_t c, uint64_t w, uint64_t h, uint64_t n, uint32_t span,
                 uint32_t box_w, uint32_t box_h) {
    EncodeTiledFn fn = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled);
    if (!fn) return false;
    cuuint64_t dims[4] = {c, w, h, n};
    cuuint64_t strides[3] = {c, w * c, h * w * c};
    cuuint32_t box[4] = {span, box_w, box_h, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle_of(span), CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

struct QuantHost {   // host copies of what setup_quant uploaded
    std::vector<int32_t> mult, shift, bias;
};

// Builds one GEMM: packs B, folds zero points into the bias, derives the epilogue constants, sizes the launch.
// weight(n, k) returns the raw weight byte of output column n at reduction index k (k < K).
template <typename WeightFn>
int32_t build_gemm(enn_b200_context *ctx, const ConvGeom &g, const QuantHost &qh, int32_t M, int32_t N, int32_t K, WeightFn weight,
                   TcGemm *gm, uint32_t implicit_span = 0, bool want_resident = false) {
    TcParams &p = gm->prm;
    p.M = M; p.N = N; p.K = K;
    // K bytes per k-block.  Implicit convolutions bring theirs (the channel chunk); plain GEMMs with a short K use 32-
    // or 64-byte rows, so that the TMA does not spend its time zero-filling 128-byte rows that are mostly padding.
    uint32_t span = implicit_span ? implicit_span : (K <= 32 ? 32u : (K <= 64 ? 64u : static_cast<uint32_t>(kBK)));
    if (ctx->opt("no_narrow_span") && !implicit_span) span = kBK;
    p.span = static_cast<int32_t>(span);
    const int32_t zw_eff = g.w_signed ? g.w_zp : g.w_zp - 128;   // weights as signed bytes: int8 stays, u8 becomes w - 128
    p.zw_eff = zw_eff;
    p.need_asum = zw_eff != 0;
    p.a_signed = g.a_signed;
    p.act_min = g.act_min; p.act_max = g.act_max; p.out_zp = g.out_zp;
    const int32_t extra = p.need_asum ? 16 : 0;
    int32_t max_data = kMaxBN - extra;
    if (ctx->has_opt("tc_bn")) max_data = ctx->opt("tc_bn") >= 96 && ctx->opt("tc_bn") <= max_data ? (ctx->opt("tc_bn") & ~15) : max_data;   // tuning override, 96 columns at least
    p.tiles_m = (M + kBM - 1) / kBM;
    // One k-block and many output channels (the MobileNetV2 expand layers): the layer's time is its epilogue's.  Tiles of
    // at most 128 columns let two M tiles share an accumulator buffer and be requantised together, so that every load of
    // a column's constants serves two outputs (28 x 28 x 32 -> 192 at 256 images: 24.2 -> 21.1 us; 14 x 14 x 96 -> 576:
    // 21.7 -> 19.9 us; 56 x 56 x 24 -> 144 in its four-pixel packing, 576 columns: 73.8 -> 65.4 us; 384 and 960 columns:
    // no change).  Not with the extra column of the activation sums, which would leave room for one M tile only.
    if (!implicit_span && !ctx->has_opt("tc_bn") && !ctx->opt("no_narrow_n") && K <= static_cast<int32_t>(span) && N > 128 && extra == 0 &&
        M > kGemvMaxM && max_data > 128)
        max_data = 128;
    // N tiling: as few tiles as possible, but split further while the grid would leave SMs idle.
    int32_t tiles_n = (N + max_data - 1) / max_data;
    while (static_cast<int64_t>(p.tiles_m) * tiles_n < ctx->launch_sms() && (N + tiles_n) / (tiles_n + 1) >= 32) ++tiles_n;
    int32_t bn_data = (((N + tiles_n - 1) / tiles_n) + 15) & ~15;
    tiles_n = (N + bn_data - 1) / bn_data;
    if (static_cast<int64_t>(p.tiles_m) * tiles_n > ctx->sm_count && bn_data >= 128) {
        // Several waves of tiles: a slightly narrower tile can save a whole wave (time ~ waves x tile width).
        int64_t best = ((static_cast<int64_t>(p.tiles_m) * tiles_n + ctx->sm_count - 1) / ctx->sm_count) * bn_data;
        for (int32_t cand = bn_data - 16; cand >= bn_data - 64 && cand >= 128; cand -= 16) {
            const int32_t tn = (N + cand - 1) / cand;
            const int64_t cost = ((static_cast<int64_t>(p.tiles_m) * tn + ctx->sm_count - 1) / ctx->sm_count) * cand;
            if (cost < best) {
                best = cost;
                bn_data = cand;
                tiles_n = tn;
            }
        }
    }
    // CTA pairs (cta_group::2): two SMs share one 256-row tile and every B byte is fetched once per pair.  Used for plain
    // GEMMs with several waves of 256-wide tiles, long K and large operands ((M+N) K >= 32 MB): 8192^3 runs 7 % faster
    // than on the one-CTA kernel, 4096^3 6 % (51.6 against 54.7 us).  Option tc_pair = 0 / 1 overrides the size rule.
    const bool pair_ok = span == kBK && !implicit_span && p.tiles_m >= 2 && (K + kBK - 1) / kBK >= 8 && bn_data >= 128 &&
                         static_cast<int64_t>(p.tiles_m) * tiles_n >= 2ll * ctx->sm_count;
    bool two = pair_ok && (static_cast<int64_t>(M) + N) * K >= (32ll << 20);
    int32_t forced_rows = 0;
    if (ctx->has_opt("tc_pair")) {
        const int ev = ctx->opt("tc_pair");
        two = pair_ok && ev != 0;
        if (ev >= 128) forced_rows = ev & ~31;      // tuning: that UMMA N instead of 256
    }
    if (two) {
        const int32_t rows = forced_rows >= 128 && forced_rows <= kMaxBN ? forced_rows : kMaxBN;   // the pair's UMMA N
        if (rows - extra <= max_data) {
            bn_data = rows - extra;
            tiles_n = (N + bn_data - 1) / bn_data;
        } else {
            two = false;
        }
    }
    p.two = two ? 1 : 0;
    p.tiles_n = tiles_n;
    p.bn_data = bn_data;
    p.bn_rows = bn_data + extra;
    p.k_blocks = (K + static_cast<int32_t>(span) - 1) / static_cast<int32_t>(span);
    p.group = two ? 1 : kMaxBN / p.bn_rows;
    if (p.group > p.tiles_m) p.group = p.tiles_m;
    // keep at least ~2 work units per SM before widening the groups
    while (p.group > 1 && static_cast<int64_t>((p.tiles_m + p.group - 1) / p.group) * tiles_n < 2ll * ctx->sm_count) --p.group;
    p.tiles_mg = two ? (p.tiles_m + 1) / 2 : (p.tiles_m + p.group - 1) / p.group;
    // Bands only pay when the operands do not stay L2 resident by themselves (their coordinates cost two divisions per
    // tile in every epilogue thread).
    const bool big_operands = (static_cast<int64_t>(M) + N) * K > (48ll << 20);
    p.raster = !big_operands ? p.tiles_mg : (two ? 8 : 16);
    if (ctx->opt("tc_raster") > 0) p.raster = ctx->opt("tc_raster");   // tuning override
    if (p.raster > p.tiles_mg) p.raster = p.tiles_mg;
    const int32_t k_pad = ((K + kBK - 1) / kBK) * kBK;
    p.k_pad = k_pad;
    p.idesc = (2u << 4) | (static_cast<uint32_t>(g.a_signed ? 1 : 0) << 7) | (1u << 10) |
              (static_cast<uint32_t>(p.bn_rows >> 3) << 17) | (static_cast<uint32_t>((p.two ? 2 * kBM : kBM) >> 4) << 24);

    // Packed B: [tiles_n][bn_rows][k_pad] int8, zero padded; row bn_data of each tile is all ones (sum_k a).
    std::vector<int8_t> wb(static_cast<size_t>(tiles_n) * p.bn_rows * k_pad, 0);
    std::vector<ColParam> cols(static_cast<size_t>(tiles_n) * p.bn_rows);
    std::memset(cols.data(), 0, cols.size() * sizeof(ColParam));
    const int64_t amax = g.a_signed ? 128 : 255;
    const int64_t zo_eff = static_cast<int64_t>(g.out_zp) - g.act_min;
    std::vector<int64_t> folded_v(N), bound_v(N);
    for (int32_t n = 0; n < N; ++n) {
        const int32_t tn = n / bn_data, r = n % bn_data;
        int8_t *dst = wb.data() + (static_cast<size_t>(tn) * p.bn_rows + r) * k_pad;
        int64_t wsum = 0, wabs = 0;
        for (int32_t k = 0; k < K; ++k) {
            const uint8_t raw = weight(n, k);
            const int32_t wv = g.w_signed ? static_cast<int32_t>(static_cast<int8_t>(raw)) : static_cast<int32_t>(raw) - 128;
            dst[k] = static_cast<int8_t>(wv);
            wsum += wv;
            wabs += wv < 0 ? -wv : wv;
        }
        const int64_t folded = static_cast<int64_t>(qh.bias[n]) - static_cast<int64_t>(g.in_zp) * wsum +
                               static_cast<int64_t>(K) * g.in_zp * zw_eff;
        folded_v[n] = folded;
        // bound on |accumulator + folded bias|
        bound_v[n] = amax * wabs + static_cast<int64_t>(K) * amax * (zw_eff < 0 ? -zw_eff : zw_eff) + (folded < 0 ? -folded : folded);
    }
    // ReLU-type outputs (lower clamp == output zero point): can every column use the merged form?
    bool relu_hi = zo_eff == 0 && M > kGemvMaxM && !ctx->opt("no_relu_mode"), relu_two = relu_hi;
    for (int32_t n = 0; n < N && relu_two; ++n) {
        const int32_t sh = qh.shift[n];
        const int32_t ls = sh > 0 ? sh : 0, e = sh > 0 ? 0 : -sh;
        const bool in_range = folded_v[n] <= INT32_MAX && folded_v[n] >= INT32_MIN && bound_v[n] < (1ll << 31) && qh.mult[n] >= 0;
        if (!in_range || ls > 30 || e > 31) relu_hi = relu_two = false;
        if (ls > 0 || e < 1) relu_hi = false;
        // two-shift form: the left-shifted accumulator must not wrap (the reference multiplies in int32) and the
        // stage-1 value plus the rounding term must fit 32 bits
        if ((bound_v[n] << ls) + (e >= 1 ? (1ll << (e - 1)) : 0) + 1 >= (1ll << 31)) relu_two = false;
    }
    p.mode = relu_hi && !ctx->opt("no_relu_hi") ? kModeReluHi : (relu_two ? kModeReluTwo : kModeNudge);
    // The clamp is the whole unsigned byte: the saturating pack of the epilogue does it (kModeReluSat).
    p.sat_plain = p.mode == kModeReluHi && !p.a_signed && p.act_min == 0 && p.act_max >= 255 && !ctx->opt("no_relu_sat");
    for (int32_t n = 0; n < N; ++n) {
        const int32_t tn = n / bn_data, r = n % bn_data;
        const int64_t folded = folded_v[n];
        ColParam &c = cols[static_cast<size_t>(tn) * p.bn_rows + r];
        if (p.mode == kModeReluHi || p.mode == kModeReluTwo) {
            const int32_t sh = qh.shift[n];
            const int32_t ls = sh > 0 ? sh : 0, e = sh > 0 ? 0 : -sh;
            int64_t cc = folded * qh.mult[n];
            int32_t word;
            if (p.mode == kModeReluHi) {
                cc += (1ll << 30) + (1ll << (30 + e));
                word = e - 1;
            } else {
                const int32_t s1 = 31 - ls;
                cc += (1ll << (30 - ls)) + (e >= 1 ? (1ll << (e - 1 + s1)) : 0);
                word = s1 | (e << 8);
            }
            c.mult = static_cast<int32_t>(static_cast<uint32_t>(static_cast<uint64_t>(cc) & 0xffffffffu));   // word 0: C low
            c.addend = static_cast<int32_t>(static_cast<uint32_t>(static_cast<uint64_t>(cc) >> 32));            // word 1: C high
            c.esh = qh.mult[n];                                                                                // word 2: M0
            c.bias = word;                                                                                     // word 3: shifts
            continue;
        }
        c.mult = qh.mult[n];
        c.bias = static_cast<int32_t>(folded);     // wraps like the reference's int32 accumulation
        const int32_t e = qh.shift[n] > 0 ? -1 : -qh.shift[n];
        const int64_t addend = e > 0 ? (1ll << (e - 1)) + zo_eff * (1ll << e) : zo_eff;
        if (e < 1 || folded > INT32_MAX || folded < INT32_MIN || bound_v[n] + 2 + (addend < 0 ? -addend : addend) >= (1ll << 31)) {
            c.addend = qh.shift[n];                // general path keeps the raw signed shift
            c.esh = INT32_MIN;
            p.mode = kModeGeneral;
        } else {
            c.addend = static_cast<int32_t>(addend);
            c.esh = e;
        }
    }
    if (p.need_asum)
        for (int32_t tn = 0; tn < tiles_n; ++tn) {
            int8_t *dst = wb.data() + (static_cast<size_t>(tn) * p.bn_rows + bn_data) * k_pad;
            for (int32_t k = 0; k < K; ++k) dst[k] = 1;
        }
    cudaError_t e;
    if ((e = cudaMalloc(&gm->w_dev, wb.size())) != cudaSuccess || (e = cudaMalloc(&gm->cols_dev, cols.size() * sizeof(ColParam))) != cudaSuccess ||
        (e = cudaMemcpy(gm->w_dev, wb.data(), wb.size(), cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemcpy(gm->cols_dev, cols.data(), cols.size() * sizeof(ColParam), cudaMemcpyHostToDevice)) != cudaSuccess) {
        ctx->last_error = std::string("tensor-core plan: ") + cudaGetErrorString(e);
        return ENN_B200_CUDA_FAILURE;
    }
    p.cols = static_cast<const ColParam *>(gm->cols_dev);
    if (!encode_2d(ctx, &gm->map_b, gm->w_dev, k_pad, static_cast<uint64_t>(tiles_n) * p.bn_rows, k_pad, span, p.two ? p.bn_rows / 2 : p.bn_rows)) {
        ctx->last_error = "cuTensorMapEncodeTiled failed for the weight tensor";
        return ENN_B200_CUDA_FAILURE;
    }
    // Several small k-blocks share a pipeline stage so that a barrier round trip covers ~32 KB of operands.
    // Implicit convolutions and narrow pointwise layers are bound by the producer's copy issue (a thread issues one tensor
    // copy per ~420 cycles and a tile needs one A and one B copy per k-block): when the weights of the only N tile fit,
    // they are loaded once per CTA and stay resident, the stages hold A only, and the producer issues half as many copies.
    const size_t b_tile = (static_cast<size_t>(p.bn_rows) * span + 1023) & ~static_cast<size_t>(1023);
    p.b_res = ((implicit_span != 0 || p.bn_rows <= 64 || want_resident || (p.k_blocks == 1 && !ctx->opt("no_bres_k1"))) && !p.two && tiles_n == 1 && M > kGemvMaxM && b_tile * p.k_blocks <= (want_resident ? kWidePackWeightBytes : 72 * 1024) &&
               !ctx->opt("no_bres")) ? 1 : 0;
    const size_t kb_bytes = p.b_res ? static_cast<size_t>(kBM) * span : (static_cast<size_t>(kBM) + (p.two ? p.bn_rows / 2 : p.bn_rows)) * span;
    p.kpack = static_cast<int32_t>((32 * 1024) / kb_bytes);
    if (p.kpack < 1 || p.two) p.kpack = 1;
    if (p.kpack > p.k_blocks) p.kpack = p.k_blocks;
    if (p.kpack > 8) p.kpack = 8;
    const size_t fixed = static_cast<size_t>(kEpiWarps) * kChunksPerWarp * 16 * sizeof(ColParam) + 1024 + 1024;   // column constants, barriers, slack
    const size_t resident = p.b_res ? b_tile * p.k_blocks : 0;
    const size_t stage_bytes = kb_bytes * p.kpack;
    int stages = static_cast<int>((227 * 1024 - fixed - resident) / stage_bytes);
    if (stages > 8) stages = 8;
    if (p.b_res && stages >= 3 && (stages & 1)) --stages;      // two producer lanes on alternate stages need an even ring
    if (stages < 2) return ENN_B200_INVALID_PARAMS;
    p.stages = stages;
    gm->smem_bytes = stages * stage_bytes + fixed + resident;
    const int total_tiles = p.tiles_mg * p.tiles_n;
    gm->grid = total_tiles < ctx->launch_sms() ? total_tiles : ctx->launch_sms();
    if (p.two) gm->grid = 2 * (total_tiles < ctx->launch_sms() / 2 ? total_tiles : ctx->launch_sms() / 2);
    // One thread cannot issue both operands of every k-block fast enough for a long MMA-bound k loop; short, epilogue-
    // bound problems are better off without the extra warp.
    gm->threads = (p.kpack == 1 && p.k_blocks >= 8) ? kThreads : kThreadsOneProducer;
    p.epi_g = p.two ? 1 : (p.group >= 4 ? 4 : (p.group >= 2 ? 2 : 1));
    p.no_wide_store = ctx->opt("no_wide_store") ? 1 : 0;
    if (ctx->has_opt("epi_g")) { const int ev = ctx->opt("epi_g"); p.epi_g = ev == 4 || ev == 2 ? (ev <= p.group ? ev : p.epi_g) : 1; }   // tuning override
    return ENN_B200_SUCCESS;
}

void free_plan(TcPlan *plan) {
    if (!plan) return;
    for (auto &gm : plan->gemms) {
        if (gm.w_dev) cudaFree(gm.w_dev);
        if (gm.cols_dev) cudaFree(gm.cols_dev);
        if (gm.ktab_dev) cudaFree(gm.ktab_dev);
    }
    if (plan->scratch) cudaFree(plan->scratch);
    if (plan->err_host) cudaFreeHost(plan->err_host);
    delete plan;
}

template <bool ASUM, int MODE>
void launch_tc_gemm_variant(const TcGemm &gm, const CUtensorMap &map_a, const TcParams &p, cudaStream_t stream) {
    if (!p.two) {
        launch_pdl(tc_gemm_kernel<ASUM, MODE, false>, dim3(static_cast<unsigned>(gm.grid)), dim3(static_cast<unsigned>(gm.threads)), gm.smem_bytes, stream, map_a, gm.map_b, p);
        return;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(gm.grid));
    cfg.blockDim = dim3(static_cast<unsigned>(gm.threads));
    cfg.dynamicSmemBytes = gm.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, tc_gemm_kernel<ASUM, MODE, true>, map_a, gm.map_b, p);
}

void launch_first_layer(enn_b200_context *ctx, const TcGemm &gm, const void *in, void *out) {
    const TcParams &p = gm.prm;
    const Im2colGeom &ig = gm.ig;
    Conv3x3c3Params g{};
    g.n = ig.n; g.h = ig.h; g.w = ig.w; g.oh = ig.oh; g.ow = ig.ow; g.sy = ig.sy; g.sx = ig.sx; g.y0 = ig.y0; g.x0 = ig.x0;
    g.M = p.M; g.N = p.N; g.k_pad = p.k_pad;
    g.zw_eff = p.zw_eff; g.act_min = p.act_min; g.act_max = p.act_max; g.out_zp = p.out_zp;
    g.fill = ig.fill;
    g.in_bytes = static_cast<int64_t>(ig.n) * ig.h * ig.w * 3;
    const size_t smem = static_cast<size_t>(p.N) * 48;
    const int64_t want = ((static_cast<int64_t>(p.M) + kFirstLayerPixels - 1) / kFirstLayerPixels + 255) / 256;
    const unsigned blocks = static_cast<unsigned>(want < 8ll * ctx->sm_count ? want : 8ll * ctx->sm_count);
    const uint8_t *src = static_cast<const uint8_t *>(in);
    const int8_t *wq = static_cast<const int8_t *>(gm.w_dev);
    uint8_t *dst = static_cast<uint8_t *>(out);
#define ENN_FL(S, A, G) launch_pdl(conv3x3c3_kernel<S, A, G>, dim3(blocks), dim3(256), smem, ctx->stream, g, src, wq, p.cols, dst)
#define ENN_FL_MODE(S, A)                                           \
    switch (p.mode) {                                               \
        case kModeNudge: ENN_FL(S, A, kModeNudge); break;           \
        case kModeGeneral: ENN_FL(S, A, kModeGeneral); break;       \
        case kModeReluHi:                                           \
            if (p.sat_plain && !S) ENN_FL(S, A, kModeReluSat);      \
            else ENN_FL(S, A, kModeReluHi);                         \
            break;                                                  \
        default: ENN_FL(S, A, kModeReluTwo); break;                 \
    }
    if (p.a_signed) {
        if (p.need_asum) { ENN_FL_MODE(true, true) } else { ENN_FL_MODE(true, false) }
    } else {
        if (p.need_asum) { ENN_FL_MODE(false, true) } else { ENN_FL_MODE(false, false) }
    }
#undef ENN_FL_MODE
#undef ENN_FL
}

template <bool ASUM>
void launch_tc_gemm_mode(const TcGemm &gm, const CUtensorMap &map_a, const TcParams &p, cudaStream_t stream) {
    if (p.add_on) {      // fused add: one-CTA kernels of the two-stage modes only (the plan checks)
        if (p.mode == kModeNudge)
            launch_pdl(tc_gemm_kernel<ASUM, kModeNudge, false, true>, dim3(static_cast<unsigned>(gm.grid)), dim3(static_cast<unsigned>(gm.threads)), gm.smem_bytes,
                       stream, map_a, gm.map_b, p);
        else
            launch_pdl(tc_gemm_kernel<ASUM, kModeGeneral, false, true>, dim3(static_cast<unsigned>(gm.grid)), dim3(static_cast<unsigned>(gm.threads)), gm.smem_bytes,
                       stream, map_a, gm.map_b, p);
        return;
    }
    switch (p.mode) {
        case kModeNudge: launch_tc_gemm_variant<ASUM, kModeNudge>(gm, map_a, p, stream); break;
        case kModeGeneral: launch_tc_gemm_variant<ASUM, kModeGeneral>(gm, map_a, p, stream); break;
        case kModeReluHi:
            if (p.sat_plain) launch_tc_gemm_variant<ASUM, kModeReluSat>(gm, map_a, p, stream);
            else launch_tc_gemm_variant<ASUM, kModeReluHi>(gm, map_a, p, stream);
            break;
        default: launch_tc_gemm_variant<ASUM, kModeReluTwo>(gm, map_a, p, stream); break;
    }
}

void launch_tc_gemm(const TcGemm &gm, const CUtensorMap &map_a, const TcParams &p, cudaStream_t stream) {
    if (p.need_asum) launch_tc_gemm_mode<true>(gm, map_a, p, stream);
    else launch_tc_gemm_mode<false>(gm, map_a, p, stream);
}

template <bool ASUM, int MODE>
void set_tc_gemm_smem_attr() {
    cudaFuncSetAttribute(tc_gemm_kernel<ASUM, MODE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(tc_gemm_kernel<ASUM, MODE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
}

}  // namespace

bool tc_available(const enn_b200_context *ctx) { return ctx && ctx->cc_major == 10 && ctx->encode_tiled != nullptr; }

// Plans the tensor-core path of a convolution, FullyConnected or transposed convolution.  `w_hwio` is the host
// copy of the weights in [Kh][Kw][Cin][Cout] order (raw bytes).  Returns INVALID_PARAMS when the geometry is
// not one this path covers (grouped convolutions); the caller then keeps the direct kernel.
int32_t tc_plan_conv(enn_b200_op *op, const void *w_hwio) {
    const ConvGeom &g = op->g;
    enn_b200_context *ctx = op->ctx;
    const uint8_t *w = static_cast<const uint8_t *>(w_hwio);
    const int32_t N = g.cout, cin = g.cin;
    // Grouped convolution (the reference runs one GEMM per group, CLGEMMConvolutionQuantized.cpp:202-265) is the dense
    // convolution with block-diagonal weights: outside a channel's own group the weight is the weight zero point, whose
    // terms vanish in the zero-point algebra.  The tensor pipe has the room (it idles in every convolution of this size);
    // the dense weights must stay small, or the direct kernel takes the operator.
    if (g.groups != 1 && (op->kind != OP_CONV || g.groups > 32 || static_cast<int64_t>(g.kh) * g.kw * cin * N > (8ll << 20) ||
                          ctx->opt("no_grouped_tc")))
        return ENN_B200_INVALID_PARAMS;

    QuantHost qh;
    qh.mult.resize(N); qh.shift.resize(N); qh.bias.resize(N);
    if (cudaMemcpy(qh.mult.data(), op->rq.mult, sizeof(int32_t) * N, cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(qh.shift.data(), op->rq.shift, sizeof(int32_t) * N, cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(qh.bias.data(), op->rq.bias, sizeof(int32_t) * N, cudaMemcpyDeviceToHost) != cudaSuccess)
        return ENN_B200_CUDA_FAILURE;

    TcPlan *plan = new (std::nothrow) TcPlan();
    if (!plan) return ENN_B200_FAILURE;
    auto bail = [&](int32_t st) {
        free_plan(plan);
        return st;
    };
    const uint32_t fill = (static_cast<uint32_t>(g.in_zp) & 0xff) * 0x01010101u;
    int32_t st = ENN_B200_SUCCESS;

    // Decides how a GEMM whose A operand is described by `ig` (grid oh x ow per image, taps kh x kw) gets that operand and
    // builds it: implicit convolution (stride-1 taps, Cin % 32 == 0) or gathered matrix.  `weight(n, k)` uses k = tap * cin + c.
    auto make_conv_gemm = [&](TcGemm &gm, const Im2colGeom &ig, auto weight) -> int32_t {
        const int32_t K = ig.kh * ig.kw * cin;
        const int32_t taps = ig.kh * ig.kw;
        uint32_t span = 0;
        if (ig.sy == 1 && ig.sx == 1 && (cin & 31) == 0 && taps <= 64 && !ctx->opt("no_implicit"))
            span = (cin % 128 == 0) ? 128 : ((cin % 64 == 0) ? 64 : 32);
        const int64_t M64 = static_cast<int64_t>(ig.n) * ig.oh * ig.ow;
        if (M64 <= 0 || M64 > INT32_MAX) return ENN_B200_INVALID_PARAMS;
        gm.ig = ig;
        if (!span) {
            int32_t st2 = build_gemm(ctx, g, qh, static_cast<int32_t>(M64), N, K, weight, &gm);
            if (st2 != ENN_B200_SUCCESS) return st2;
            gm.gather = true;
            gm.ig.K = K; gm.ig.Kp = (K + 15) & ~15;
            gm.first_layer = ig.kh == 3 && ig.kw == 3 && cin == 3 && ig.dy == 1 && ig.dx == 1 && (N & 15) == 0 && gm.prm.tiles_n == 1 &&
                             M64 >= 4096 && !ctx->opt("no_first_layer");
            const size_t need = static_cast<size_t>(M64) * gm.ig.Kp;
            if (need > plan->scratch_bytes) plan->scratch_bytes = need;
            return ENN_B200_SUCCESS;
        }
        // patch of the output grid per M tile: as wide as the grid allows, rows to fill 128 accumulator rows
        const int32_t wt = ig.ow < kBM ? ig.ow : kBM;
        int32_t ht = kBM / wt;
        if (ht > ig.oh) ht = ig.oh;
        const int32_t tx = (ig.ow + wt - 1) / wt, ty = (ig.oh + ht - 1) / ht;
        const int64_t tiles = static_cast<int64_t>(ig.n) * tx * ty;
        if (tiles * kBM > INT32_MAX) return ENN_B200_INVALID_PARAMS;
        int32_t st2 = build_gemm(ctx, g, qh, static_cast<int32_t>(tiles * kBM), N, K, weight, &gm, span);
        if (st2 != ENN_B200_SUCCESS) return st2;
        TcParams &p = gm.prm;
        p.taps = taps; p.cchunks = cin / static_cast<int32_t>(span); p.span = static_cast<int32_t>(span);
        p.conv_ht = ht; p.conv_wt = wt; p.conv_ty = ty; p.conv_tx = tx;
        int32_t min_dy = 0, max_dy = 0, min_dx = 0, max_dx = 0;
        for (int32_t ky = 0; ky < ig.kh; ++ky)
            for (int32_t kx = 0; kx < ig.kw; ++kx) {
                const int32_t dy = ky * ig.dy + ig.y0, dx = kx * ig.dx + ig.x0;
                min_dy = dy < min_dy ? dy : min_dy; max_dy = dy > max_dy ? dy : max_dy;
                min_dx = dx < min_dx ? dx : min_dx; max_dx = dx > max_dx ? dx : max_dx;
            }
        gm.implicit = true;
        gm.padded = g.in_zp != 0;            // zero OOB fill already equals the zero point otherwise
        gm.pad_lo_y = gm.padded ? -min_dy : 0;
        gm.pad_lo_x = gm.padded ? -min_dx : 0;
        const int32_t hi_y = ig.oh - 1 + max_dy - (ig.h - 1), hi_x = ig.ow - 1 + max_dx - (ig.w - 1);
        gm.hp = gm.padded ? gm.pad_lo_y + ig.h + (hi_y > 0 ? hi_y : 0) : ig.h;
        gm.wp = gm.padded ? gm.pad_lo_x + ig.w + (hi_x > 0 ? hi_x : 0) : ig.w;
        for (int32_t ky = 0; ky < ig.kh; ++ky)
            for (int32_t kx = 0; kx < ig.kw; ++kx) {
                p.tap_dy[ky * ig.kw + kx] = static_cast<int16_t>(ky * ig.dy + ig.y0 + gm.pad_lo_y);
                p.tap_dx[ky * ig.kw + kx] = static_cast<int16_t>(kx * ig.dx + ig.x0 + gm.pad_lo_x);
            }
        if (gm.padded) {
            const size_t need = static_cast<size_t>(ig.n) * gm.hp * gm.wp * cin;
            if (need > plan->scratch_bytes) plan->scratch_bytes = need;
        }
        return ENN_B200_SUCCESS;
    };

    if (op->kind != OP_DECONV) {
        const int64_t M64 = static_cast<int64_t>(g.n) * g.oh * g.ow;
        if (M64 <= 0 || M64 > INT32_MAX) return bail(ENN_B200_INVALID_PARAMS);
        const int32_t K = g.kh * g.kw * cin;
        const bool pointwise = g.kh == 1 && g.kw == 1 && g.sh == 1 && g.sw == 1 && g.pt == 0 && g.pl == 0 && g.oh == g.h && g.ow == g.w;
        bool in_place = pointwise && (cin & 15) == 0;
        plan->gemms.resize(1);
        TcGemm &gm = plan->gemms[0];
        // `w` is [Kh][Kw][Cin / groups][Cout]; k = tap * cin + c over all input channels
        const int32_t cin_g = cin / g.groups, cout_g = N / g.groups;
        const uint8_t zero_w = static_cast<uint8_t>(g.w_zp);
        auto weight = [&](int32_t n, int32_t k) -> uint8_t {
            if (g.groups == 1) return w[static_cast<size_t>(k) * N + n];
            const int32_t tap = k / cin, c = k - tap * cin;
            return c / cin_g == n / cout_g ? w[(static_cast<size_t>(tap) * cin_g + c % cin_g) * N + n] : zero_w;
        };
        // Pixel packing: with K of 16, 32 or 64 bytes and few output channels, f = 128 / K consecutive pixels are one
        // 128-byte row of the activation tensor.  The GEMM [M/f][fK] x blockdiag(W, ..., W) -> [M/f][fN] is the same
        // memory as [M][K] x W -> [M][N] when the off-diagonal weights equal the weight zero point (their terms vanish
        // in the zero-point algebra), and the TMA then fetches one full line per row instead of f short ones, which is
        // what bounds these layers.  The extra MMA work (f times) is free: the tensor pipe idles in them.
        // A channel count that is not a multiple of 16 (24) cannot be read in place at all (TMA row pitch); packed rows of
        // f * K bytes can, which removes the gather pass; several N tiles are accepted in that case.
        int32_t pack = 1;
        // Not for layers with 96 or more output channels whose rows can be read in place: their time is the epilogue's, not
        // the row fetches', and unpacked they keep two M tiles per work unit, which halves the epilogue's loads of the
        // column constants (112 x 112 x 16 -> 96: 161 us packed, 152 us in place).
        const bool epilogue_heavy = N >= 96 && (K & 15) == 0;
        if (pointwise && M64 >= 4096 && K <= 64 && !epilogue_heavy && !ctx->opt("no_pack")) {
            const int32_t zw_eff = g.w_signed ? g.w_zp : g.w_zp - 128;
            for (int32_t f = 8; f >= 2 && pack == 1; f >>= 1) {
                if (f * K > 128 || (f * K) % 16 != 0 || M64 % f != 0) continue;
                if (f * N <= kMaxBN - (zw_eff != 0 ? 16 : 0)) pack = f;
            }
            // Rows that cannot be read in place (K = 24) and whose packed form needs several N tiles anyway: the smallest
            // packing, so that an M tile's rows are copied for as few N tiles as possible (56 x 56 x 24 -> 144 at 256
            // images: 61.5 us as pixel pairs, 65.0 us as groups of four).
            for (int32_t f = 2; f <= 8 && pack == 1 && (K & 15) != 0; f <<= 1)
                if (f * K <= 128 && (f * K) % 16 == 0 && M64 % f == 0) pack = f;
            if (pack > 1) in_place = true;
        }
        // Wider rows that are not whole 128-byte lines (K = 96, 144, 192 ...: the MobileNetV2 project layers).  In place,
        // every 128-byte box row of such a tensor straddles two lines and the last k-block is mostly padding; with f pixels
        // per row of f * K bytes the k-blocks are (mostly) aligned full lines and the f * N output bytes of a row are whole
        // 16-byte stores.  The block-diagonal weights (f^2 times the layer's) must stay resident in shared memory, and the
        // layer must keep two waves of M tiles, or the packing costs more than it saves.
        bool wide_pack = false;
        if (pointwise && pack == 1 && M64 >= 4096 && K > 64 && (K & 127) != 0 && (K & 15) == 0 && !ctx->opt("no_pack")) {
            const int32_t zw_eff = g.w_signed ? g.w_zp : g.w_zp - 128;
            const int32_t extra = zw_eff != 0 ? 16 : 0;
            const int32_t forced = ctx->opt("pack_wide");   // tuning override (1 = off)
            for (int32_t f = 8; f >= 2 && pack == 1 && forced != 1; f >>= 1) {
                if ((forced > 1 && f != forced) || M64 % f != 0 || f * N > kMaxBN - extra) continue;
                const size_t kp = (static_cast<size_t>(f) * K + 127) & ~static_cast<size_t>(127);
                const size_t rows = ((static_cast<size_t>(f) * N + 15) & ~static_cast<size_t>(15)) + extra;
                if (rows * kp <= kWidePackWeightBytes && M64 / f >= 2ll * kBM * ctx->sm_count) { pack = f; wide_pack = true; in_place = true; }
            }
        }
        if (in_place && pack > 1) {
            QuantHost qp;
            for (int32_t r = 0; r < pack; ++r) {
                qp.mult.insert(qp.mult.end(), qh.mult.begin(), qh.mult.end());
                qp.shift.insert(qp.shift.end(), qh.shift.begin(), qh.shift.end());
                qp.bias.insert(qp.bias.end(), qh.bias.begin(), qh.bias.end());
            }
            const uint8_t zero_raw = static_cast<uint8_t>(g.w_zp);
            auto packed_weight = [&](int32_t n, int32_t k) -> uint8_t {
                return n / N == k / K ? weight(n % N, k % K) : zero_raw;
            };
            st = build_gemm(ctx, g, qp, static_cast<int32_t>(M64 / pack), pack * N, pack * K, packed_weight, &gm, 0, wide_pack);
            if (st != ENN_B200_SUCCESS) return bail(st);
            gm.prm.qh = 1; gm.prm.qw = static_cast<int32_t>(M64 / pack);
            gm.prm.out_base = 0; gm.prm.out_sn = 0; gm.prm.out_sy = 0; gm.prm.out_sx = pack * N;
        } else if (in_place) {
            st = build_gemm(ctx, g, qh, static_cast<int32_t>(M64), N, K, weight, &gm);
            if (st != ENN_B200_SUCCESS) return bail(st);
            gm.use_gemv = M64 <= kGemvMaxM && (K & 15) == 0 && static_cast<size_t>(M64) * K <= 48 * 1024 && !ctx->opt("no_gemv");
            if (gm.use_gemv) op->info.impl = ENN_B200_IMPL_GEMV;
            gm.prm.qh = 1; gm.prm.qw = static_cast<int32_t>(M64);
            gm.prm.out_base = 0; gm.prm.out_sn = 0; gm.prm.out_sy = 0; gm.prm.out_sx = N;
        } else {
            Im2colGeom ig{};
            ig.n = g.n; ig.h = g.h; ig.w = g.w; ig.cin = cin;
            ig.oh = g.oh; ig.ow = g.ow; ig.kh = g.kh; ig.kw = g.kw;
            ig.sy = g.sh; ig.sx = g.sw; ig.dy = g.dh; ig.dx = g.dw; ig.y0 = -g.pt; ig.x0 = -g.pl;
            ig.fill = fill;
            st = make_conv_gemm(gm, ig, weight);
            if (st != ENN_B200_SUCCESS) return bail(st);
            if (gm.implicit) {
                gm.prm.qh = g.oh; gm.prm.qw = g.ow;
                gm.prm.out_base = 0;
                gm.prm.out_sn = static_cast<int64_t>(g.oh) * g.ow * N;
                gm.prm.out_sy = static_cast<int64_t>(g.ow) * N;
                gm.prm.out_sx = N;
            } else {
                gm.prm.qh = 1; gm.prm.qw = static_cast<int32_t>(M64);
                gm.prm.out_base = 0; gm.prm.out_sn = 0; gm.prm.out_sy = 0; gm.prm.out_sx = N;
                }
        }
    } else {
        // Transposed convolution (DeconvolutionKernels.cpp:24-198) split by output parity: outputs with
        // (oy + pad_t) % sh == py only ever meet kernel rows ky = py + sh * jy, so each class (py, px) is a
        // stride-1 correlation over the input with its own small filter:
        //   out[n, sh*q - pad_t + py, ...] = sum_{jy,jx,c} in[n, q - jy, r - jx, c] * w[c][co][py + sh*jy][px + sw*jx].
        plan->gemms.reserve(static_cast<size_t>(g.sh) * g.sw);
        for (int32_t py = 0; py < g.sh; ++py) {
            for (int32_t px = 0; px < g.sw; ++px) {
                const int32_t jy_n = py < g.kh ? (g.kh - py + g.sh - 1) / g.sh : 0;
                const int32_t jx_n = px < g.kw ? (g.kw - px + g.sw - 1) / g.sw : 0;
                // q range: 0 <= sh*q - pad_t + py < oh
                const int32_t q_lo = (g.pt - py + g.sh - 1 >= 0) ? (g.pt - py + g.sh - 1) / g.sh : 0;
                const int32_t q_hi = (g.oh - 1 + g.pt - py) >= 0 ? (g.oh - 1 + g.pt - py) / g.sh : -1;
                const int32_t r_lo = (g.pl - px + g.sw - 1 >= 0) ? (g.pl - px + g.sw - 1) / g.sw : 0;
                const int32_t r_hi = (g.ow - 1 + g.pl - px) >= 0 ? (g.ow - 1 + g.pl - px) / g.sw : -1;
                const int32_t qh_n = q_hi - q_lo + 1, qw_n = r_hi - r_lo + 1;
                if (qh_n <= 0 || qw_n <= 0) continue;
                // A class without taps (stride larger than the kernel) still has outputs: requant(bias).  One
                // zero-weight dummy tap keeps it on the same code path.
                const int32_t jy_e = jy_n > 0 ? jy_n : 1, jx_e = jx_n > 0 ? jx_n : 1;
                const bool empty = jy_n == 0 || jx_n == 0;
                plan->gemms.emplace_back();
                TcGemm &gm = plan->gemms.back();
                Im2colGeom ig{};
                ig.n = g.n; ig.h = g.h; ig.w = g.w; ig.cin = cin;
                ig.oh = qh_n; ig.ow = qw_n; ig.kh = jy_e; ig.kw = jx_e;
                ig.sy = 1; ig.sx = 1; ig.dy = -1; ig.dx = -1; ig.y0 = q_lo; ig.x0 = r_lo;
                ig.fill = fill;
                st = make_conv_gemm(gm, ig, [&](int32_t n, int32_t k) -> uint8_t {
                    const int32_t tap = k / cin, c = k - tap * cin;
                    const int32_t jy = tap / jx_e, jx = tap - jy * jx_e;
                    if (empty) return static_cast<uint8_t>(g.w_zp);
                    const int32_t ky = py + g.sh * jy, kx = px + g.sw * jx;
                    return w[((static_cast<size_t>(ky) * g.kw + kx) * cin + c) * N + n];
                });
                if (st != ENN_B200_SUCCESS) return bail(st);
                gm.prm.qh = qh_n; gm.prm.qw = qw_n;
                const int32_t oy0 = g.sh * q_lo - g.pt + py, ox0 = g.sw * r_lo - g.pl + px;
                gm.prm.out_base = (static_cast<int64_t>(oy0) * g.ow + ox0) * N;
                gm.prm.out_sn = static_cast<int64_t>(g.oh) * g.ow * N;
                gm.prm.out_sy = static_cast<int64_t>(g.sh) * g.ow * N;
                gm.prm.out_sx = static_cast<int64_t>(g.sw) * N;
            }
        }
        if (plan->gemms.empty()) return bail(ENN_B200_INVALID_PARAMS);
        // The classes write disjoint outputs and only read the (padded) input: give each a share of the SMs and launch
        // them on side streams, so that their launch and pipeline latencies overlap instead of adding up.
        const int ncls = static_cast<int>(plan->gemms.size());
        bool all_implicit = true;
        for (auto &gm : plan->gemms) all_implicit = all_implicit && gm.implicit;
        if (ncls > 1 && ncls <= enn_b200_context::kAuxStreams + 1 && all_implicit && !ctx->opt("no_fan_out")) {
            plan->fan_out = true;
            const int share = ctx->launch_sms() / ncls > 0 ? ctx->launch_sms() / ncls : 1;
            for (auto &gm : plan->gemms)
                if (gm.grid > share) gm.grid = share;
        }
    }

    {   // All implicit GEMMs of an operator read the same input: one padded copy with the union of their margins.
        int32_t lo_y = 0, lo_x = 0, hi_y = 0, hi_x = 0;
        bool any = false;
        for (auto &gm : plan->gemms)
            if (gm.implicit && gm.padded) {
                any = true;
                lo_y = gm.pad_lo_y > lo_y ? gm.pad_lo_y : lo_y;
                lo_x = gm.pad_lo_x > lo_x ? gm.pad_lo_x : lo_x;
                const int32_t hy = gm.hp - gm.pad_lo_y - g.h, hx = gm.wp - gm.pad_lo_x - g.w;
                hi_y = hy > hi_y ? hy : hi_y;
                hi_x = hx > hi_x ? hx : hi_x;
            }
        if (any) {
            bool first = true;
            for (auto &gm : plan->gemms)
                if (gm.implicit && gm.padded) {
                    for (int32_t t = 0; t < gm.prm.taps; ++t) {
                        gm.prm.tap_dy[t] = static_cast<int16_t>(gm.prm.tap_dy[t] + lo_y - gm.pad_lo_y);
                        gm.prm.tap_dx[t] = static_cast<int16_t>(gm.prm.tap_dx[t] + lo_x - gm.pad_lo_x);
                    }
                    gm.pad_lo_y = lo_y; gm.pad_lo_x = lo_x;
                    gm.hp = lo_y + g.h + hi_y; gm.wp = lo_x + g.w + hi_x;
                    gm.runs_pad = first;
                    first = false;
                    const size_t need = static_cast<size_t>(g.n) * gm.hp * gm.wp * cin;
                    if (need > plan->scratch_bytes) plan->scratch_bytes = need;
                }
        }
    }
    if (plan->scratch_bytes > (static_cast<size_t>(8) << 30)) return bail(ENN_B200_INVALID_PARAMS);   // keep the direct kernel
    cudaError_t e;
    if ((plan->scratch_bytes && (e = cudaMalloc(&plan->scratch, plan->scratch_bytes)) != cudaSuccess) ||
        (e = cudaHostAlloc(reinterpret_cast<void **>(&plan->err_host), sizeof(int32_t), cudaHostAllocMapped)) != cudaSuccess ||
        (e = cudaHostGetDevicePointer(reinterpret_cast<void **>(&plan->err_dev), plan->err_host, 0)) != cudaSuccess) {
        ctx->last_error = std::string("tensor-core plan: ") + cudaGetErrorString(e);
        return bail(ENN_B200_CUDA_FAILURE);
    }
    *plan->err_host = 0;
    int launches = 0;
    for (auto &gm : plan->gemms) {
        gm.prm.err = plan->err_dev;
        launches += ((gm.gather && !gm.first_layer) || (gm.implicit && gm.runs_pad)) ? 2 : 1;
        if (gm.implicit && gm.padded) {
            if (!encode_nhwc(ctx, &gm.map_a, plan->scratch, cin, gm.wp, gm.hp, g.n, gm.prm.span, gm.prm.conv_wt, gm.prm.conv_ht)) {
                ctx->last_error = "cuTensorMapEncodeTiled failed for the padded activation tensor";
                return bail(ENN_B200_CUDA_FAILURE);
            }
            gm.map_a_ptr = plan->scratch;
        }
        if (gm.gather) {   // the offset table also serves as the fallback for misaligned input pointers
            // Byte-granular gather: per reduction index, the byte offset of (ky, kx, c) from the tap-(0,0) pixel
            // and the tap's pixel displacement.
            const Im2colGeom &ig = gm.ig;
            std::vector<int2> tab(ig.Kp, make_int2(0, 0));
            for (int32_t k = 0; k < ig.K; ++k) {
                const int32_t tap = k / ig.cin, c = k - tap * ig.cin;
                const int32_t ky = tap / ig.kw, kx = tap - ky * ig.kw;
                const int32_t dy = ky * ig.dy, dx = kx * ig.dx;
                tab[k].x = (dy * ig.w + dx) * ig.cin + c;
                tab[k].y = (dy << 16) | (dx & 0xffff);
            }
            if (cudaMalloc(&gm.ktab_dev, tab.size() * sizeof(int2)) != cudaSuccess ||
                cudaMemcpy(gm.ktab_dev, tab.data(), tab.size() * sizeof(int2), cudaMemcpyHostToDevice) != cudaSuccess) {
                ctx->last_error = "tensor-core plan: offset table upload failed";
                return bail(ENN_B200_CUDA_FAILURE);
            }
            gm.ig.ktab = static_cast<const int2 *>(gm.ktab_dev);
        }
        if (gm.gather) {
            if (!encode_2d(ctx, &gm.map_a, plan->scratch, gm.ig.Kp, gm.prm.M, gm.ig.Kp, static_cast<uint32_t>(gm.prm.span), kBM)) {
                ctx->last_error = "cuTensorMapEncodeTiled failed for the gathered activation matrix";
                return bail(ENN_B200_CUDA_FAILURE);
            }
            gm.map_a_ptr = plan->scratch;
        }
    }
    op->info.kernel_launches = launches;
    static bool attr_set = false;
    if (!attr_set) {
        set_tc_gemm_smem_attr<false, kModeNudge>();
        set_tc_gemm_smem_attr<false, kModeGeneral>();
        set_tc_gemm_smem_attr<false, kModeReluHi>();
        set_tc_gemm_smem_attr<false, kModeReluTwo>();
        set_tc_gemm_smem_attr<false, kModeReluSat>();
        set_tc_gemm_smem_attr<true, kModeNudge>();
        set_tc_gemm_smem_attr<true, kModeGeneral>();
        set_tc_gemm_smem_attr<true, kModeReluHi>();
        set_tc_gemm_smem_attr<true, kModeReluTwo>();
        set_tc_gemm_smem_attr<true, kModeReluSat>();
        cudaFuncSetAttribute(tc_gemm_kernel<false, kModeNudge, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        cudaFuncSetAttribute(tc_gemm_kernel<false, kModeGeneral, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        cudaFuncSetAttribute(tc_gemm_kernel<true, kModeNudge, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        cudaFuncSetAttribute(tc_gemm_kernel<true, kModeGeneral, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        attr_set = true;
    }
    op->tc = plan;
    return ENN_B200_SUCCESS;
}

// Turns a planned convolution into convolution + quantized add (`add`: the prepared add operator's parameters and tables).
// INVALID_PARAMS when this plan cannot take it; the caller then keeps the two operators.
int32_t tc_fuse_add(enn_b200_op *op, const AddParams &add, bool conv_is_second) {
    TcPlan *plan = static_cast<TcPlan *>(op->tc);
    if (!plan || plan->gemms.size() != 1 || plan->fused_add) return ENN_B200_INVALID_PARAMS;
    TcGemm &gm = plan->gemms[0];
    TcParams &p = gm.prm;
    if (gm.first_layer || gm.use_gemv || p.two || (p.mode != kModeNudge && p.mode != kModeGeneral) || (p.N & 15) != 0 || (p.out_base & 15) != 0 ||
        (p.out_sx & 15) != 0 || (p.out_sy & 15) != 0 || (p.out_sn & 15) != 0 || p.M == 0 || !add.lut || add.is_signed != p.a_signed)
        return ENN_B200_INVALID_PARAMS;
    if (gm.smem_bytes + 2048 > 227 * 1024) return ENN_B200_INVALID_PARAMS;
    p.add_off = static_cast<int32_t>(gm.smem_bytes - 1024);      // behind the barriers; the last 1024 bytes are the alignment slack
    gm.smem_bytes += 2048;
    p.add = add;
    p.add_on = 1;
    p.add_swap = conv_is_second ? 1 : 0;
    plan->fused_add = true;
    return ENN_B200_SUCCESS;
}

// The other addend of a fused operator for the next tc_execute.
void tc_set_residual(enn_b200_op *op, const void *res) {
    if (TcPlan *plan = static_cast<TcPlan *>(op->tc)) plan->residual = static_cast<const uint8_t *>(res);
}

int32_t tc_execute(enn_b200_op *op, const void *in, void *out) {
    TcPlan *plan = static_cast<TcPlan *>(op->tc);
    enn_b200_context *ctx = op->ctx;
    if (!plan) return ENN_B200_FAILURE;
    if (*plan->err_host != 0) {
        char buf[96];
        std::snprintf(buf, sizeof(buf), "tensor-core kernel gave up on a barrier wait (code %d)", *plan->err_host);
        ctx->last_error = buf;
        return ENN_B200_CUDA_FAILURE;
    }
    #ifdef ENN_B200_DEV
    const bool fan_out = plan->fan_out && !getenv("ENN_B200_TC_DEBUG");
#else
    const bool fan_out = plan->fan_out;
#endif
    if (fan_out && !ctx->aux_ready) {
        bool ok = cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming) == cudaSuccess;
        for (int i = 0; i < enn_b200_context::kAuxStreams && ok; ++i)
            ok = cudaStreamCreateWithFlags(&ctx->aux_streams[i], cudaStreamNonBlocking) == cudaSuccess &&
                 cudaEventCreateWithFlags(&ctx->ev_join[i], cudaEventDisableTiming) == cudaSuccess;
        if (!ok) {
            ctx->last_error = "could not create the side streams";
            return ENN_B200_CUDA_FAILURE;
        }
        ctx->aux_ready = true;
    }
    const bool starve = plan->starve_next;
    plan->starve_next = false;
    int cls = 0;             // index of the GEMM among those launched (fan-out: 0 runs on the main stream)
    bool forked = false;
    for (auto &gm : plan->gemms) {
        TcParams &p = gm.prm;
        if (p.M == 0) continue;
        if (gm.first_layer && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
            launch_first_layer(ctx, gm, in, out);
            cudaError_t fe = cudaGetLastError();
            if (fe != cudaSuccess) {
                ctx->last_error = std::string("conv3x3c3_kernel launch: ") + cudaGetErrorString(fe);
                return ENN_B200_CUDA_FAILURE;
            }
            continue;
        }
        if (gm.gather) {
            const int64_t total16 = static_cast<int64_t>(p.M) * (gm.ig.Kp >> 4);
            const unsigned blocks = static_cast<unsigned>((total16 + 255) / 256);
            launch_im2col(gm.ig, in, static_cast<uint8_t *>(plan->scratch), total16, blocks, ctx->stream);
        } else if (gm.implicit) {
            if ((reinterpret_cast<uintptr_t>(in) & 15) != 0) {
                ctx->last_error = "tensor-core path needs a 16-byte aligned input pointer";
                return ENN_B200_INVALID_PARAMS;
            }
            const Im2colGeom &ig = gm.ig;
            if (gm.padded && !gm.runs_pad) {
                // the padded copy was written by an earlier GEMM of this operator in the same execute
            } else if (gm.padded) {
                const int64_t total16 = static_cast<int64_t>(ig.n) * gm.hp * gm.wp * (ig.cin >> 4);
                pad_nhwc_kernel<<<static_cast<unsigned>((total16 + 255) / 256), 256, 0, ctx->stream>>>(
                    static_cast<const uint8_t *>(in), static_cast<uint8_t *>(plan->scratch), ig.n, ig.h, ig.w, ig.cin, gm.hp, gm.wp, gm.pad_lo_y,
                    gm.pad_lo_x, ig.fill, total16);
            } else if (gm.map_a_ptr != in) {
                if (!encode_nhwc(ctx, &gm.map_a, in, ig.cin, ig.w, ig.h, ig.n, p.span, p.conv_wt, p.conv_ht)) {
                    ctx->last_error = "cuTensorMapEncodeTiled failed for the activation tensor";
                    return ENN_B200_CUDA_FAILURE;
                }
                gm.map_a_ptr = in;
            }
        } else {
            if ((reinterpret_cast<uintptr_t>(in) & 15) != 0) {
                ctx->last_error = "tensor-core path needs a 16-byte aligned input pointer";
                return ENN_B200_INVALID_PARAMS;
            }
            if (gm.use_gemv) {
                // few rows: HBM-bound on the weights, CUDA-core GEMV over the same packed weights and constants
                const int k_pad = p.k_pad;
                if (p.a_signed) launch_gemv<true>(p.M, in, gm.w_dev, p.cols, out, p, k_pad, ctx->stream);
                else launch_gemv<false>(p.M, in, gm.w_dev, p.cols, out, p, k_pad, ctx->stream);
                cudaError_t ge = cudaGetLastError();
                if (ge != cudaSuccess) {
                    ctx->last_error = std::string("gemv_kernel launch: ") + cudaGetErrorString(ge);
                    return ENN_B200_CUDA_FAILURE;
                }
                continue;
            }
            if (gm.map_a_ptr != in) {
                int hit = -1;
                for (int i = 0; i < TcGemm::kMapCache; ++i)
                    if (gm.map_cache_ptr[i] == in) hit = i;
                if (hit < 0) {
                    hit = gm.map_cache_next;
                    gm.map_cache_next = (gm.map_cache_next + 1) % TcGemm::kMapCache;
                    if (!encode_2d(ctx, &gm.map_cache[hit], in, p.K, p.M, p.K, static_cast<uint32_t>(p.span), kBM)) {
                        ctx->last_error = "cuTensorMapEncodeTiled failed for the activation tensor";
                        return ENN_B200_CUDA_FAILURE;
                    }
                    gm.map_cache_ptr[hit] = in;
                }
                gm.map_a = gm.map_cache[hit];
                gm.map_a_ptr = in;
            }
        }
        p.out = static_cast<uint8_t *>(out);
        if (plan->fused_add) {
            if (!plan->residual || ((reinterpret_cast<uintptr_t>(plan->residual) | reinterpret_cast<uintptr_t>(out)) & 15) != 0) {
                ctx->last_error = "fused convolution + add needs the second addend and 16-byte aligned pointers";
                return ENN_B200_INVALID_PARAMS;
            }
            p.add_res = plan->residual;
        }
        p.test_starve = starve ? 1 : 0;
#ifdef ENN_B200_DEV
        p.dbg_mode = getenv("ENN_B200_TC_MODE") ? atoi(getenv("ENN_B200_TC_MODE")) : 0;
        static long long *dbg_buf = nullptr;
        const bool dbg = getenv("ENN_B200_TC_DEBUG") != nullptr;     // development aid: role wait-cycle counters of CTA 0
        if (dbg) {
            if (!dbg_buf) cudaMallocManaged(&dbg_buf, sizeof(long long) * 8 * 1024);
            p.dbg = dbg_buf;
        }
#endif
        cudaStream_t gs = ctx->stream;
        if (fan_out) {
            if (!forked) {       // everything the classes read (input, padded copy) is ordered before this point
                cudaEventRecord(ctx->ev_fork, ctx->stream);
                forked = true;
            }
            if (cls > 0) {
                gs = ctx->aux_streams[cls - 1];
                cudaStreamWaitEvent(gs, ctx->ev_fork, 0);
            }
        }
        launch_tc_gemm(gm, gm.map_a, p, gs);
        if (fan_out && cls > 0) {
            cudaEventRecord(ctx->ev_join[cls - 1], gs);
            cudaStreamWaitEvent(ctx->stream, ctx->ev_join[cls - 1], 0);
        }
        ++cls;
#ifdef ENN_B200_DEV
        if (dbg) {
            cudaStreamSynchronize(ctx->stream);
            const long long *d = p.dbg;
            std::fprintf(stderr, "tc dbg cta0: tiles %d x %d (group %d) k_blocks %d stages %d | producer wait %lld | mma tempty-wait %lld / %lld | epi tfull-wait %lld / %lld | mma thread %lld ns\n",
                         p.tiles_m, p.tiles_n, p.group, p.k_blocks, p.stages, d[0], d[3], d[4], d[5], d[6], d[7]);
            p.dbg = nullptr;
        }
#endif
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
            ctx->last_error = std::string("tc_gemm_kernel launch: ") + cudaGetErrorString(e);
            return ENN_B200_CUDA_FAILURE;
        }
    }
    return ENN_B200_SUCCESS;
}

// Self-test hook for the bounded waits: the next tc_execute of this operator issues no operand copies, so the MMA
// issuer's first wait (shortened to a fraction of a millisecond) runs out, the CTA-wide abort flag ends every other role,
// TMEM is released and the error code reaches the host.  Nothing is in flight when the kernel gives up.
int32_t tc_test_starve_next(enn_b200_op *op) {
    TcPlan *plan = static_cast<TcPlan *>(op->tc);
    if (!plan) return ENN_B200_INVALID_PARAMS;
    for (auto &gm : plan->gemms)
        if (gm.use_gemv || gm.first_layer || gm.prm.two) return ENN_B200_INVALID_PARAMS;   // pairs: the peer CTA would only see its own, long limit
    plan->starve_next = true;
    return ENN_B200_SUCCESS;
}

// Forgets a recorded barrier time-out so that the operator can be executed again.
void tc_clear_error(enn_b200_op *op) {
    TcPlan *plan = static_cast<TcPlan *>(op->tc);
    if (plan && plan->err_host) *plan->err_host = 0;
}

void tc_release(enn_b200_op *op) {
    free_plan(static_cast<TcPlan *>(op->tc));
    op->tc = nullptr;
}

// ------------------------------------------------------------------------------------------------------
// Execution without any allocation: the gathered A matrix lives in a fixed device array that is part of the
// loaded module instead of the plan's own scratch buffer.
// ------------------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = static_cast<size_t>(32) << 20;
static __device__ __align__(256) uint8_t g_static_scratch[kStaticScratchBytes];
// The array's name is only a host-side handle; the device address differs per device and is looked up once per
// device with that device current.
static uint8_t *g_static_scratch_addr[64] = {nullptr};
static std::mutex g_static_scratch_mutex;      // guards the table above (first calls from several host threads)

int32_t tc_execute_static(enn_b200_op *op, const void *in, void *out) {
    enn_b200_context *ctx = op->ctx;
    TcPlan *plan = static_cast<TcPlan *>(op->tc);
    if (!plan || op->impl != ENN_B200_IMPL_TCGEN05 || plan->fused_add) {
        ctx->last_error = "enn_b200_op_execute_noalloc: the operator is not bound to the tensor-core path (or has a fused add)";
        return ENN_B200_INVALID_PARAMS;
    }
    size_t need = 0;
    for (auto &gm : plan->gemms) {
        if (!gm.gather) {
            ctx->last_error = "enn_b200_op_execute_noalloc: this operator has no gathered input matrix; call enn_b200_op_execute";
            return ENN_B200_INVALID_PARAMS;
        }
        const size_t bytes = static_cast<size_t>(gm.prm.M) * gm.ig.Kp;
        if (bytes > need) need = bytes;
    }
    if (need > kStaticScratchBytes) {
        char buf[160];
        std::snprintf(buf, sizeof(buf), "enn_b200_op_execute_noalloc: gathered matrix needs %zu bytes, the static scratch holds %zu",
                      need, kStaticScratchBytes);
        ctx->last_error = buf;
        return ENN_B200_INVALID_PARAMS;
    }
    if (ctx->device < 0 || ctx->device >= 64) return ENN_B200_INVALID_PARAMS;
    uint8_t *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        scratch = g_static_scratch_addr[ctx->device];
        if (!scratch) {
            // The symbol's address belongs to the device that is current during the lookup; the caller's own current
            // device is put back afterwards.
            int prev = -1;
            cudaGetDevice(&prev);
            if (cudaSetDevice(ctx->device) != cudaSuccess) return ENN_B200_CUDA_FAILURE;
            void *addr = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&addr, g_static_scratch);
            if (prev >= 0 && prev != ctx->device) cudaSetDevice(prev);
            if (e != cudaSuccess || !addr) {
                ctx->last_error = std::string("enn_b200_op_execute_noalloc: cudaGetSymbolAddress failed: ") + cudaGetErrorString(e);
                return ENN_B200_CUDA_FAILURE;
            }
            scratch = g_static_scratch_addr[ctx->device] = static_cast<uint8_t *>(addr);
        }
    }
    if (*plan->err_host != 0) {
        ctx->last_error = "tensor-core kernel gave up on a barrier wait earlier";
        return ENN_B200_CUDA_FAILURE;
    }
    for (auto &gm : plan->gemms) {
        TcParams p = gm.prm;     // private copy: the handle's own launch state is left untouched
        if (p.M == 0) continue;
        if (gm.map_a_static_ptr != scratch) {
            if (!encode_2d(ctx, &gm.map_a_static, scratch, gm.ig.Kp, p.M, gm.ig.Kp, static_cast<uint32_t>(p.span), kBM)) {
                ctx->last_error = "cuTensorMapEncodeTiled failed for the static scratch";
                return ENN_B200_CUDA_FAILURE;
            }
            gm.map_a_static_ptr = scratch;
        }
        const int64_t total16 = static_cast<int64_t>(p.M) * (gm.ig.Kp >> 4);
        const unsigned blocks = static_cast<unsigned>((total16 + 255) / 256);
        launch_im2col(gm.ig, in, scratch, total16, blocks, ctx->stream);
        p.out = static_cast<uint8_t *>(out);
        p.dbg = nullptr;
        p.dbg_mode = 0;
        p.test_starve = 0;
        launch_tc_gemm(gm, gm.map_a_static, p, ctx->stream);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
            ctx->last_error = std::string("enn_b200_op_execute_noalloc launch: ") + cudaGetErrorString(e);
            return ENN_B200_CUDA_FAILURE;
        }
    }
    return ENN_B200_SUCCESS;
}

}  // namespace enn_b200

// For callers that must not allocate device memory at run time: a convolution or transposed convolution whose
// input is gathered into a scratch matrix normally keeps that matrix in a buffer obtained with cudaMalloc when
// the operator is prepared.  A component that runs where allocation is off limits (a real-time inference loop that
// cannot afford the device-wide synchronisation an allocation may imply, or a host that pre-reserved all device
// memory for something else) can run the same operator through this entry point instead: the gathered matrix is
// placed in a 32 MiB array that belongs to the library image, so the call performs no cudaMalloc / cudaFree and no
// allocating library routine.  The first call on a device looks the array's device address up
// (cudaGetSymbolAddress) and encodes one tensor map; make that first call before any stream capture starts.
// Every call on a device uses the same array and leaves its last gathered matrix there; the gather overwrites all
// the bytes the GEMM will read, so nothing needs clearing, but two calls whose kernels overlap on the GPU (different
// streams or contexts) race on it.  Operators that need more than 32 MiB of scratch, or none, are rejected with
// ENN_B200_INVALID_PARAMS and a message.
extern "C" int32_t enn_b200_op_execute_noalloc(enn_b200_op *op, const void *in_dev, void *out_dev) {
    if (!op) return ENN_B200_INVALID_PARAMS;
    if (!in_dev || !out_dev) {
        op->ctx->last_error = "null device pointer";
        return ENN_B200_INVALID_PARAMS;
    }
    if (op->dyn && !op->dyn->bound) {
        op->ctx->last_error = "filter / bias are runtime tensors: call enn_b200_op_rebind_constants first";
        return ENN_B200_FAILURE;
    }
    return enn_b200::tc_execute_static(op, in_dev, out_dev);
}
