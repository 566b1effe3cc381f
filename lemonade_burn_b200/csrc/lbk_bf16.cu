// f32 activations x bf16 weights (the tied, unquantised LM head).
//
// Replaces bf16_gemv / dot_scalar / dot_avx2 / dot_avx512 (crates/lb-ternary/src/bf16.rs:14-105)
// and the bf16_linear op above them (crates/lb-model/src/ops.rs:199-218):
// out[t, r] = sum_k x[t, k] * bf16(W[r, k]), f32 products and f32 accumulation.
// HBM-bound: W (rows*cols*2 bytes) is read once per group of up to kTok token rows.
// Summation order differs from the reference's 8-lane order, so results agree to rounding,
// not bit for bit (the reference allows 1e-4 absolute, bf16.rs:113-136).
#include "lbk_internal.cuh"
#include "lbk_ptx.cuh"

namespace lbk {

namespace {

constexpr int kThreads = 256;
constexpr int kTok = 4;  // token rows per pass over W

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// One warp per weight row at a time; x rows staged in shared memory.
template <int T>
__global__ void __launch_bounds__(kThreads) bf16_linear_kernel(const float *__restrict__ x,
                                                              const uint16_t *__restrict__ w,
                                                              int rows, int cols, int m_total,
                                                              int t0, float *__restrict__ out) {
    ptx::pdl_trigger();
    ptx::pdl_wait();

    extern __shared__ float s_x[];  // [T][cols]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < T * cols; i += kThreads) {
        const int t = i / cols, c = i - t * cols;
        s_x[i] = (t0 + t < m_total) ? x[static_cast<size_t>(t0 + t) * cols + c] : 0.0f;
    }
    __syncthreads();
    const int warps_total = gridDim.x * (kThreads / 32);
    const bool vec = (cols & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
    for (int r = blockIdx.x * (kThreads / 32) + warp; r < rows; r += warps_total) {
        const uint16_t *wr = w + static_cast<size_t>(r) * cols;
        float acc[T];
#pragma unroll
        for (int t = 0; t < T; ++t) acc[t] = 0.0f;
        if (vec) {
            const uint4 *w4 = reinterpret_cast<const uint4 *>(wr);
#pragma unroll 4
            for (int i = lane; i < (cols >> 3); i += 32) {
                const uint4 v = __ldcs(w4 + i);  // streamed once: evict-first
                const float f[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y),
                                    bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    const float4 xa = *reinterpret_cast<const float4 *>(s_x + t * cols + i * 8);
                    const float4 xb = *reinterpret_cast<const float4 *>(s_x + t * cols + i * 8 + 4);
                    acc[t] = fmaf(f[0], xa.x, acc[t]); acc[t] = fmaf(f[1], xa.y, acc[t]);
                    acc[t] = fmaf(f[2], xa.z, acc[t]); acc[t] = fmaf(f[3], xa.w, acc[t]);
                    acc[t] = fmaf(f[4], xb.x, acc[t]); acc[t] = fmaf(f[5], xb.y, acc[t]);
                    acc[t] = fmaf(f[6], xb.z, acc[t]); acc[t] = fmaf(f[7], xb.w, acc[t]);
                }
            }
        } else {
            for (int i = lane; i < cols; i += 32) {
                const float f = __uint_as_float(static_cast<uint32_t>(wr[i]) << 16);
#pragma unroll
                for (int t = 0; t < T; ++t) acc[t] = fmaf(f, s_x[t * cols + i], acc[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            float v = acc[t];
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && t0 + t < m_total) out[static_cast<size_t>(t0 + t) * rows + r] = v;
        }
    }
}

}  // namespace

int launch_bf16_linear(Ctx *ctx, const float *x, size_t m, const uint16_t *w, size_t rows,
                       size_t cols, float *out, cudaStream_t stream) {
    if (m == 0 || rows == 0) return LBK_OK;
    const size_t smem1 = cols * sizeof(float);
    if (smem1 * kTok > ctx->smem_optin)
        return fail(LBK_ERR_UNSUPPORTED, "bf16_linear: %zu columns do not fit in shared memory", cols);
    const int grid = ctx->sm_count * 4;
    for (size_t t0 = 0; t0 < m; t0 += kTok) {
        const size_t left = m - t0;
        if (left >= kTok) {
            const size_t smem = smem1 * kTok;
            LBK_CUDA(cudaFuncSetAttribute(bf16_linear_kernel<kTok>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            LBK_CUDA(launch_chained(bf16_linear_kernel<kTok>, dim3(grid), dim3(kThreads), smem, stream, x, w, static_cast<int>(rows), static_cast<int>(cols), static_cast<int>(m), static_cast<int>(t0), out));
        } else if (left >= 2) {
            const size_t smem = smem1 * 2;
            LBK_CUDA(cudaFuncSetAttribute(bf16_linear_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            LBK_CUDA(launch_chained(bf16_linear_kernel<2>, dim3(grid), dim3(kThreads), smem, stream, x, w, static_cast<int>(rows), static_cast<int>(cols), static_cast<int>(m), static_cast<int>(t0), out));
            if (left == 3) {  // the odd last row
                LBK_CUDA(cudaFuncSetAttribute(bf16_linear_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem1)));
                LBK_CUDA(launch_chained(bf16_linear_kernel<1>, dim3(grid), dim3(kThreads), smem1, stream, x, w, static_cast<int>(rows), static_cast<int>(cols), static_cast<int>(m), static_cast<int>(t0 + 2), out));
                ctx->launches++;
            }
        } else {
            LBK_CUDA(cudaFuncSetAttribute(bf16_linear_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem1)));
            LBK_CUDA(launch_chained(bf16_linear_kernel<1>, dim3(grid), dim3(kThreads), smem1, stream, x, w, static_cast<int>(rows), static_cast<int>(cols), static_cast<int>(m), static_cast<int>(t0), out));
        }
        LBK_CUDA(cudaGetLastError());
        ctx->launches++;
    }
    return LBK_OK;
}

}  // namespace lbk
