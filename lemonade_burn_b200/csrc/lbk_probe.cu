// lbk_int8_peak_probe: how fast this GPU's tensor cores execute tcgen05.mma kind::i8 when nothing
// feeds them: the denominator of the prefill GEMM's "fraction of int8 peak".
//
// One CTA per SM. The A operand (128 weight rows x 128 columns of u8 codes) sits in tensor memory,
// the B operand (n token rows x 128 columns of s8) in shared memory, both written once; one thread
// then issues `iters` groups of four MMAs (K = 32 each) into one accumulator without waiting for
// anything, and a single commit at the end tells when the pipe has drained. No loads, no epilogue:
// what is measured is the issue and execution rate of the instruction the GEMM kernel is built on,
// in the same operand arrangement (A from TMEM, B from shared memory through a SWIZZLE_128B
// descriptor). The numbers in the operands do not matter and the accumulator is never read.
// The reference has no counterpart (its kernels are CPU SIMD).
#include "lbk_internal.cuh"
#include "lbk_ptx.cuh"

namespace lbk {
namespace {

// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

template <int N>
__global__ void __launch_bounds__(128, 1) int8_peak_kernel(int iters, int *err_word) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_u32(smem_raw), base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    __shared__ uint32_t s_tmem;
    __shared__ uint64_t s_bar;
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < N * 128 / 4; i += 128) reinterpret_cast<uint32_t *>(sm)[i] = 0x01010101u * (i & 3);
    ptx::fence_proxy_async();
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(&s_bar), 1);
        ptx::fence_barrier_init();
    }
    constexpr uint32_t kCols = N + 128 <= 256 ? 256 : 512;  // accumulator + one A tile, a power of two
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(&s_tmem)), "r"(kCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tm = s_tmem;
    {   // the A tile: every warp fills its 32 lanes, 128 columns of 32-bit words (4 codes each)
        const uint32_t v = 0x01000201u;
        for (int c = 0; c < 128; c += 8)
            asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(tm + (static_cast<uint32_t>(warp * 32) << 16) + N + c), "r"(v) : "memory");
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // instruction descriptor: s32 accumulator, A u8 (unsigned), B s8, M = 128, N
    constexpr uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((N >> 3) << 17) | ((128 >> 4) << 24);
    if (threadIdx.x == 0) {
        for (int i = 0; i < iters; ++i) {
            const uint32_t at = tm + N + (i & 3) * 32;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
                asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p; }" ::"r"(tm), "r"(at + ks * 8),
                             "l"(smem_desc(base + ks * 32)), "r"(idesc), "r"(1u)
                             : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ptx::smem_u32(&s_bar)) : "memory");
        if (!ptx::mbar_wait(ptx::smem_u32(&s_bar), 0, 1u << 26)) atomicExch(err_word, 8);  // bounded: the pipe drains in milliseconds
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tm), "r"(kCols) : "memory");
    }
}

template <int N>
int run_probe(Ctx *ctx, int iters, double *tops) {
    const size_t smem = static_cast<size_t>(N) * 128 + 1024;
    LBK_CUDA(cudaFuncSetAttribute(int8_peak_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    cudaStream_t st = ctx->own_stream;
    cudaEvent_t a, b;
    LBK_CUDA(cudaEventCreate(&a));
    LBK_CUDA(cudaEventCreate(&b));
    int8_peak_kernel<N><<<ctx->sm_count, 128, smem, st>>>(64, ctx->err_word);  // warm-up
    LBK_CUDA(cudaEventRecord(a, st));
    int8_peak_kernel<N><<<ctx->sm_count, 128, smem, st>>>(iters, ctx->err_word);
    LBK_CUDA(cudaEventRecord(b, st));
    LBK_CUDA(cudaGetLastError());
    ctx->launches += 2;
    LBK_CUDA(cudaEventSynchronize(b));
    float ms = 0.0f;
    LBK_CUDA(cudaEventElapsedTime(&ms, a, b));
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    *tops = 2.0 * 128.0 * N * 128.0 * static_cast<double>(iters) * ctx->sm_count / (static_cast<double>(ms) * 1e-3) / 1e12;
    return LBK_OK;
}

}  // namespace
}  // namespace lbk

using namespace lbk;

extern "C" int lbk_int8_peak_probe(lbk_ctx *c, size_t token_rows, size_t iterations, double *tops_out) {
    if (!c || !tops_out) return fail(LBK_ERR_INVALID, "lbk_int8_peak_probe: null argument");
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (iterations < 1 || iterations > (1u << 22)) return fail(LBK_ERR_INVALID, "1 .. 2^22 iterations (got %zu)", iterations);
    LBK_CUDA(cudaSetDevice(ctx->device));
    const int it = static_cast<int>(iterations);
    switch (token_rows) {
        case 64: return run_probe<64>(ctx, it, tops_out);
        case 128: return run_probe<128>(ctx, it, tops_out);
        case 192: return run_probe<192>(ctx, it, tops_out);
        case 256: return run_probe<256>(ctx, it, tops_out);
        default: return fail(LBK_ERR_UNSUPPORTED, "the probe is built for 64, 128, 192 or 256 token rows (got %zu)", token_rows);
    }
}
