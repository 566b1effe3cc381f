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

// Two to sixteen token rows per pass over W on the tensor cores (mma.sync m16n8k16, bf16 x bf16 ->
// f32). The f32 activations are split into two bf16 terms, x = hi + lo with lo = bf16(x - hi), so
// that the products are those of the reference's f32 math to within 2^-17 relative; W's bf16 values
// are exact. Token rows are the MMA's M side, 16 weight rows per warp step its N side.
//
// K is consumed 32 columns at a time and the MMA's k slots are permuted so that every lane's
// operands are contiguous: lane (g, t) loads the 16 bytes W[row g][32c + 8t .. 8t+7] (eight rows x
// 64 contiguous bytes per load instruction, whole sectors) and one 16-byte word of x per token row
// at the same columns; slots (2t, 2t+1) and (2t+8, 2t+9) of the first MMA take columns 8t+0..3,
// those of the second 8t+4..7. The permutation is the same for both operands, so the sum is the
// plain dot product.
constexpr int kMmaTok = 16;

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t f32_to_bf16_rn(float v) {  // round to nearest even; NaN kept a NaN
    const uint32_t u = __float_as_uint(v);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (u >> 16) | 0x40u;
    return (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
}

//
// Long rows go through in column chunks (`c0`, `ccols`: whole 32-column slices) so that sixteen token
// rows of a chunk fit in shared memory; the launches of one token group run one after the other on
// the stream and every chunk after the first adds to what the earlier ones stored (`accumulate`), in
// chunk order, so the sum has one fixed order.
constexpr int kMmaThreads = 512;  // sixteen warps: twice the loads in flight per SM of the eight the FMA kernel uses
// TT = token tiles of 16 rows per pass over W: 1 (2..16 rows) or 2 (17 rows and more: half the passes)
template <int TT>
__global__ void __launch_bounds__(kMmaThreads) bf16_linear_mma_kernel(const float *__restrict__ x, const uint16_t *__restrict__ w, int rows,
                                                                     int cols, int m_total, int t0, int xs_stride /* bytes */, int c0, int ccols,
                                                                     int accumulate, float *__restrict__ out) {
    ptx::pdl_trigger();
    ptx::pdl_wait();
    extern __shared__ __align__(16) uint8_t s_raw[];
    constexpr int kTokRows = TT * kMmaTok;
    uint8_t *s_hi = s_raw, *s_lo = s_raw + kTokRows * xs_stride;  // [16 TT tokens][xs_stride] bf16
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    for (int i = tid; i < kTokRows * (ccols >> 1); i += kMmaThreads) {  // two columns per step
        const int tk = i / (ccols >> 1), c = (i - tk * (ccols >> 1)) * 2;
        float2 v = make_float2(0.f, 0.f);
        if (t0 + tk < m_total) v = *reinterpret_cast<const float2 *>(x + static_cast<size_t>(t0 + tk) * cols + c0 + c);
        const uint32_t h0 = f32_to_bf16_rn(v.x), h1 = f32_to_bf16_rn(v.y);
        const uint32_t l0 = f32_to_bf16_rn(v.x - __uint_as_float(h0 << 16)), l1 = f32_to_bf16_rn(v.y - __uint_as_float(h1 << 16));
        *reinterpret_cast<uint32_t *>(s_hi + tk * xs_stride + c * 2) = h0 | (h1 << 16);
        *reinterpret_cast<uint32_t *>(s_lo + tk * xs_stride + c * 2) = l0 | (l1 << 16);
    }
    __syncthreads();
    const int slices = ccols >> 5;
    const int groups = (rows + 15) >> 4;  // 16 weight rows per warp step
    const int warps_total = gridDim.x * (kMmaThreads / 32);
    const uint8_t *xa = s_hi + g * xs_stride + t * 16, *xb = s_hi + (g + 8) * xs_stride + t * 16;
    const size_t lo_off = static_cast<size_t>(kTokRows) * xs_stride;
    const size_t tile_off = static_cast<size_t>(kMmaTok) * xs_stride;
    for (int grp = blockIdx.x * (kMmaThreads / 32) + warp; grp < groups; grp += warps_total) {
        const int r0 = grp * 16;
        const int ra = min(r0 + g, rows - 1), rb = min(r0 + 8 + g, rows - 1);  // clamped rows are computed and dropped
        const uint4 *wa = reinterpret_cast<const uint4 *>(w + static_cast<size_t>(ra) * cols + c0) + t;
        const uint4 *wb = reinterpret_cast<const uint4 *>(w + static_cast<size_t>(rb) * cols + c0) + t;
        float d0[TT][4], d1[TT][4];
#pragma unroll
        for (int tt = 0; tt < TT; ++tt)
#pragma unroll
            for (int e = 0; e < 4; ++e) d0[tt][e] = d1[tt][e] = 0.f;
        // Software pipeline over groups of kPf slices: the next group's 2 * kPf loads are issued before
        // the current group's MMAs, so that a warp always has loads in flight (without it a warp
        // alternated between waiting for its loads and computing, and the table streamed at 1.9 TB/s).
        constexpr int kPf = 4;
        uint4 ca[kPf], cb[kPf];
#pragma unroll
        for (int u = 0; u < kPf; ++u) {
            ca[u] = u < slices ? __ldcs(wa + u * 4) : make_uint4(0u, 0u, 0u, 0u);  // streamed once
            cb[u] = u < slices ? __ldcs(wb + u * 4) : make_uint4(0u, 0u, 0u, 0u);
        }
        for (int c0s = 0; c0s < slices; c0s += kPf) {
            uint4 na[kPf], nb[kPf];
#pragma unroll
            for (int u = 0; u < kPf; ++u) {
                const int c = c0s + kPf + u;
                na[u] = c < slices ? __ldcs(wa + c * 4) : make_uint4(0u, 0u, 0u, 0u);
                nb[u] = c < slices ? __ldcs(wb + c * 4) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < kPf; ++u) {
                const int c = c0s + u;
                if (c < slices) {
                    const uint4 va = ca[u], vb = cb[u];
#pragma unroll
                    for (int tt = 0; tt < TT; ++tt) {
                        const uint8_t *pa = xa + tt * tile_off + c * 64, *pb = xb + tt * tile_off + c * 64;
                        const uint4 h0 = *reinterpret_cast<const uint4 *>(pa), h1 = *reinterpret_cast<const uint4 *>(pb);
                        const uint4 l0 = *reinterpret_cast<const uint4 *>(pa + lo_off), l1 = *reinterpret_cast<const uint4 *>(pb + lo_off);
                        mma_bf16(d0[tt], h0.x, h1.x, h0.y, h1.y, va.x, va.y);
                        mma_bf16(d0[tt], h0.z, h1.z, h0.w, h1.w, va.z, va.w);
                        mma_bf16(d0[tt], l0.x, l1.x, l0.y, l1.y, va.x, va.y);
                        mma_bf16(d0[tt], l0.z, l1.z, l0.w, l1.w, va.z, va.w);
                        mma_bf16(d1[tt], h0.x, h1.x, h0.y, h1.y, vb.x, vb.y);
                        mma_bf16(d1[tt], h0.z, h1.z, h0.w, h1.w, vb.z, vb.w);
                        mma_bf16(d1[tt], l0.x, l1.x, l0.y, l1.y, vb.x, vb.y);
                        mma_bf16(d1[tt], l0.z, l1.z, l0.w, l1.w, vb.z, vb.w);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kPf; ++u) {
                ca[u] = na[u];
                cb[u] = nb[u];
            }
        }
        // D[token][row]: lane (g, t) holds tokens g, g+8 and rows 2t, 2t+1 of each 8-row half
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const float *d = half ? d1[tt] : d0[tt];
                const int row = r0 + half * 8 + 2 * t;
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int tk = t0 + tt * kMmaTok + g + hh * 8;
                    if (tk < m_total) {
                        float *o = out + static_cast<size_t>(tk) * rows + row;
                        if (row < rows) o[0] = accumulate ? o[0] + d[hh * 2] : d[hh * 2];
                        if (row + 1 < rows) o[1] = accumulate ? o[1] + d[hh * 2 + 1] : d[hh * 2 + 1];
                    }
                }
            }
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
    // two or more token rows: tensor cores, sixteen rows per pass over W (needs whole 32-column slices
    // and 16-byte aligned rows; anything else takes the FMA kernel below)
    // Rows go through in column chunks (whole 32-column slices) sized so that the staged token rows fit
    // in shared memory: 16 token rows per pass over W with chunks of at most 3072 columns; from 17 rows
    // on, 32 token rows per pass with chunks of at most 1536 (half the passes over W).
    const int tt = m > static_cast<size_t>(kMmaTok) ? 2 : 1;
    const size_t max_chunk = tt == 2 ? 1536 : 3072;
    const size_t n_chunks = (cols + max_chunk - 1) / max_chunk;
    const size_t chunk = ((cols + n_chunks - 1) / n_chunks + 31) / 32 * 32;
    const int xs_stride = static_cast<int>(chunk * 2 + 64);  // +64: the 16-byte loads of two token rows land on distinct banks
    const size_t smem = static_cast<size_t>(2 * tt * kMmaTok) * xs_stride;
    if (m >= 2 && (cols & 31) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 7) == 0 && smem <= ctx->smem_optin) {
        if (tt == 2) LBK_CUDA(cudaFuncSetAttribute(bf16_linear_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        else LBK_CUDA(cudaFuncSetAttribute(bf16_linear_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        for (size_t t0 = 0; t0 < m; t0 += static_cast<size_t>(tt) * kMmaTok) {
            for (size_t c0 = 0; c0 < cols; c0 += chunk) {
                const size_t cc = cols - c0 < chunk ? cols - c0 : chunk;
                if (tt == 2)
                    LBK_CUDA(launch_chained(bf16_linear_mma_kernel<2>, dim3(ctx->sm_count), dim3(kMmaThreads), smem, stream, x, w, static_cast<int>(rows),
                                            static_cast<int>(cols), static_cast<int>(m), static_cast<int>(t0), xs_stride, static_cast<int>(c0),
                                            static_cast<int>(cc), c0 ? 1 : 0, out));
                else
                    LBK_CUDA(launch_chained(bf16_linear_mma_kernel<1>, dim3(ctx->sm_count), dim3(kMmaThreads), smem, stream, x, w, static_cast<int>(rows),
                                            static_cast<int>(cols), static_cast<int>(m), static_cast<int>(t0), xs_stride, static_cast<int>(c0),
                                            static_cast<int>(cc), c0 ? 1 : 0, out));
                ctx->launches++;
            }
        }
        return LBK_OK;
    }
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
