// Measures the sustained rate of tcgen05.mma on this device: every SM runs one CTA that issues a long chain
// of 128 x N x K-step MMAs on resident shared-memory tiles (no global traffic), so the result is the
// tensor-pipe ceiling the implicit-GEMM kernel is compared against.  kind 0: kind::i8 (u8 x s8 -> s32, K
// step 32), kind 1: kind::f16 with bf16 operands (-> f32, K step 16); kinds 2 and 3: the same on pseudo-random
// operand bytes instead of zeros.
#include <cuda_runtime.h>

#include "internal.h"

namespace enn_b200 {
namespace {

__device__ __forceinline__ uint32_t pk_smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

template <int KIND>
__global__ void __launch_bounds__(128, 1) mma_peak_kernel(int n, int iters, int random_fill, int *err) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    // A: 128 rows x 128 bytes, B: 256 rows x 128 bytes; zero filled, or pseudo-random bytes (the operand bit toggling of
    // real data, which is what the power management sees in a real GEMM).
    for (int i = threadIdx.x; i < (128 + 256) * 128 / 16; i += blockDim.x) {
        uint32_t h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t x = (static_cast<uint32_t>(i) * 4u + j) * 2654435761u + blockIdx.x * 40503u;
            x ^= x >> 15; x *= 2246822519u; x ^= x >> 13;
            if (KIND == 1) x &= 0x3FFF3FFFu;      // bf16: keep the exponents small (finite values)
            h[j] = random_fill ? x : 0u;
        }
        reinterpret_cast<uint4 *>(smem)[i] = make_uint4(h[0], h[1], h[2], h[3]);
    }
    const uint32_t bar_a = pk_smem_u32(&bar);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_a) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy zero fill -> async-proxy MMA reads
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(pk_smem_u32(&tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    if (threadIdx.x == 0) {
        const uint32_t sa = pk_smem_u32(smem);
        uint64_t d = 0;
        d |= static_cast<uint64_t>(1) << 16;
        d |= static_cast<uint64_t>(1024 >> 4) << 32;
        d |= static_cast<uint64_t>(1) << 46;
        d |= static_cast<uint64_t>(2) << 61;
        const uint64_t da = d | ((sa & 0x3FFFF) >> 4), db = d | (((sa + 128 * 128) & 0x3FFFF) >> 4);
        const uint32_t idesc = KIND == 0 ? (2u << 4) | (0u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (8u << 24)
                                         : (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (8u << 24);
        // The tensor pipe only reaches its full rate when the MMAs follow each other without other instructions in
        // between (there is next to no queue in front of it), so the four K slices go out as one instruction run with
        // loop-invariant operands.
        const uint64_t a0 = da, a1 = da + 2, a2 = da + 4, a3 = da + 6, b0 = db, b1 = db + 2, b2 = db + 4, b3 = db + 6;
        for (int it = 0; it < iters; ++it) {
            if (KIND == 0)
                asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %10, 0;\n\tsetp.eq.b32 q, %10, %10;\n\t"
                             "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %5, %9, p;\n\t"
                             "tcgen05.mma.cta_group::1.kind::i8 [%0], %2, %6, %9, q;\n\t"
                             "tcgen05.mma.cta_group::1.kind::i8 [%0], %3, %7, %9, q;\n\t"
                             "tcgen05.mma.cta_group::1.kind::i8 [%0], %4, %8, %9, q;\n\t}"
                             ::"r"(tmem_base), "l"(a0), "l"(a1), "l"(a2), "l"(a3), "l"(b0), "l"(b1), "l"(b2), "l"(b3), "r"(idesc), "r"(it) : "memory");
            else
                asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %10, 0;\n\tsetp.eq.b32 q, %10, %10;\n\t"
                             "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %5, %9, p;\n\t"
                             "tcgen05.mma.cta_group::1.kind::f16 [%0], %2, %6, %9, q;\n\t"
                             "tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %7, %9, q;\n\t"
                             "tcgen05.mma.cta_group::1.kind::f16 [%0], %4, %8, %9, q;\n\t}"
                             ::"r"(tmem_base), "l"(a0), "l"(a1), "l"(a2), "l"(a3), "l"(b0), "l"(b1), "l"(b2), "l"(b3), "r"(idesc), "r"(it) : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_a) : "memory");
        bool done = false;
        for (uint32_t i = 0; i < (1u << 26) && !done; ++i) {
            uint32_t ok;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(bar_a) : "memory");
            done = ok != 0;
        }
        if (!done) *reinterpret_cast<volatile int *>(err) = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (threadIdx.x < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
}

}  // namespace

// Returns achieved tera-operations per second (2 * MACs) over the whole device, or a negative value on error.
double measure_mma_peak(enn_b200_context *ctx, int kind, int n, int iters) {
    if (!ctx || ctx->cc_major != 10 || kind < 0 || kind > 3 || n < 16 || n > 256 || (n & 15) || iters < 1) return -1.0;
    int *err = nullptr;
    if (cudaMalloc(&err, sizeof(int)) != cudaSuccess) return -1.0;
    cudaMemsetAsync(err, 0, sizeof(int), ctx->stream);
    const size_t smem = (128 + 256) * 128 + 1024;
    cudaFuncSetAttribute(mma_peak_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    cudaFuncSetAttribute(mma_peak_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    const int random_fill = kind >> 1;
    auto launch = [&](int its) {
        if ((kind & 1) == 0) mma_peak_kernel<0><<<ctx->sm_count, 128, smem, ctx->stream>>>(n, its, random_fill, err);
        else mma_peak_kernel<1><<<ctx->sm_count, 128, smem, ctx->stream>>>(n, its, random_fill, err);
    };
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    launch(iters / 4 + 1);   // warm-up
    cudaEventRecord(e0, ctx->stream);
    launch(iters);
    cudaEventRecord(e1, ctx->stream);
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    int herr = 0;
    cudaMemcpy(&herr, err, sizeof(int), cudaMemcpyDeviceToHost);
    cudaFree(err);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess || herr != 0 || ms <= 0.f) return -1.0;
    const double kstep = (kind & 1) == 0 ? 32.0 : 16.0;
    const double ops = 2.0 * 128.0 * n * kstep * 4.0 * iters * ctx->sm_count;
    return ops / (ms * 1e-3) / 1e12;
}

}  // namespace enn_b200
