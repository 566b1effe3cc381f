// Per-token absmax int8 activation quantiser, standalone form.
//
// Replaces quantize_acts / quantize_acts_into / quantize_row_scalar / quantize_row_avx2
// (crates/lb-ternary/src/quant.rs:37-193): one CTA per token row computes
// scale = 127/max(amax,1e-5), q = clamp(round_half_even(x*scale)), sum(q), and writes q
// zero padded to padded_cols(k). The decode GEMV has its own fused copy of this; this
// kernel feeds the prefill GEMM and the quantize_acts entry point.
#include "lbk_internal.cuh"

namespace lbk {

namespace {

constexpr int kQThreads = 256;

__device__ __forceinline__ int quant_one(float v, float scale) {
    int r = __float2int_rn(__fmul_rn(v, scale));  // NaN -> 0 like `NaN as i8` (quant.rs:115-118)
    return max(-128, min(127, r));
}

// amax_in: per-row max|x| supplied by the caller (tensor-parallel: the maximum over all ranks'
// column slices), or null to compute it here. amax_out: when non-null only the row maximum is
// written and nothing is quantised.
__global__ void __launch_bounds__(kQThreads) quantize_kernel(const float *__restrict__ x, int k,
                                                            int kp, int8_t *__restrict__ q,
                                                            float *__restrict__ scale,
                                                            int32_t *__restrict__ sum,
                                                            const float *__restrict__ amax_in,
                                                            float *__restrict__ amax_out) {
    __shared__ float s_f[kQThreads / 32];
    __shared__ int s_i[kQThreads / 32];
    __shared__ float s_scale;
    // A kernel launched behind this one with programmatic stream serialisation (the prefill GEMM)
    // may start its prologue now; it waits for this grid's results with griddepcontrol.wait.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *xr = x + static_cast<size_t>(row) * k;
    int8_t *qr = q + static_cast<size_t>(row) * kp;
    const bool vec = (k & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;

    // Rows of up to kRowCache float4 per thread are read once and kept in registers between the
    // maximum and the rounding (prefill feeds this kernel 2048 rows of 2560..6912 floats).
    constexpr int kRowCache = 8;
    float4 cache[kRowCache];
    const int n4 = k >> 2;
    const bool cached = vec && n4 <= kRowCache * kQThreads;
    float am = 0.0f;  // fmaxf drops a NaN operand, as f32::max does (quant.rs:101-104)
    if (cached) {
        const float4 *x4 = reinterpret_cast<const float4 *>(xr);
#pragma unroll
        for (int j = 0; j < kRowCache; ++j) {
            const int i = tid + j * kQThreads;
            cache[j] = i < n4 ? __ldg(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (amax_in == nullptr) {
#pragma unroll
            for (int j = 0; j < kRowCache; ++j)
                am = fmaxf(am, fmaxf(fmaxf(fabsf(cache[j].x), fabsf(cache[j].y)), fmaxf(fabsf(cache[j].z), fabsf(cache[j].w))));
        }
    }
    if (amax_in != nullptr) {
        am = amax_in[row];
    } else if (cached) {
        // done above
    } else if (vec) {
        const float4 *x4 = reinterpret_cast<const float4 *>(xr);
        for (int i = tid; i < (k >> 2); i += kQThreads) {
            float4 v = __ldg(x4 + i);
            am = fmaxf(am, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
    } else {
        for (int i = tid; i < k; i += kQThreads) am = fmaxf(am, fabsf(__ldg(xr + i)));
    }
    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    if (lane == 0) s_f[warp] = am;
    __syncthreads();
    if (tid == 0) {
        float a = 0.0f;
        for (int w = 0; w < kQThreads / 32; ++w) a = fmaxf(a, s_f[w]);
        if (amax_out != nullptr) amax_out[row] = a;
        s_scale = __fdiv_rn(127.0f, fmaxf(a, 1e-5f));
    }
    __syncthreads();
    if (amax_out != nullptr) return;
    const float sc = s_scale;
    int acc = 0;
    if (cached) {
#pragma unroll
        for (int j = 0; j < kRowCache; ++j) {
            const int i = (tid + j * kQThreads) * 4;
            if (i < kp) {  // columns past k hold zeros, which quantise to zero
                const int q0 = quant_one(cache[j].x, sc), q1 = quant_one(cache[j].y, sc);
                const int q2 = quant_one(cache[j].z, sc), q3 = quant_one(cache[j].w, sc);
                acc += q0 + q1 + q2 + q3;
                *reinterpret_cast<uint32_t *>(qr + i) = (q0 & 255) | ((q1 & 255) << 8) | ((q2 & 255) << 16) |
                                                        (static_cast<uint32_t>(q3 & 255) << 24);
            }
        }
        for (int i = (tid + kRowCache * kQThreads) * 4; i < kp; i += kQThreads * 4) *reinterpret_cast<uint32_t *>(qr + i) = 0u;
    } else
    for (int i = tid * 4; i < kp; i += kQThreads * 4) {
        int q0 = 0, q1 = 0, q2 = 0, q3 = 0;
        if (vec && i + 3 < k) {
            float4 v = __ldg(reinterpret_cast<const float4 *>(xr + i));
            q0 = quant_one(v.x, sc); q1 = quant_one(v.y, sc);
            q2 = quant_one(v.z, sc); q3 = quant_one(v.w, sc);
        } else {
            if (i < k) q0 = quant_one(__ldg(xr + i), sc);
            if (i + 1 < k) q1 = quant_one(__ldg(xr + i + 1), sc);
            if (i + 2 < k) q2 = quant_one(__ldg(xr + i + 2), sc);
            if (i + 3 < k) q3 = quant_one(__ldg(xr + i + 3), sc);
        }
        acc += q0 + q1 + q2 + q3;
        *reinterpret_cast<uint32_t *>(qr + i) = (q0 & 255) | ((q1 & 255) << 8) | ((q2 & 255) << 16) |
                                                (static_cast<uint32_t>(q3 & 255) << 24);
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) s_i[warp] = acc;
    __syncthreads();
    if (tid == 0) {
        int s = 0;
        for (int w = 0; w < kQThreads / 32; ++w) s += s_i[w];
        scale[row] = sc;
        sum[row] = s;
    }
}

// y[t, r] = (float)dot[t, r] * (1 / (s_a[t] * s_w)): the epilogue of gemm.rs:141,158 as a kernel
// of its own, for dots that were summed across ranks first.
__global__ void __launch_bounds__(256) scale_epilogue_kernel(const int32_t *__restrict__ dots,
                                                            const float *__restrict__ ascale, float wscale,
                                                            int rows, size_t total, float *__restrict__ out) {
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float inv = __fdiv_rn(1.0f, __fmul_rn(ascale[i / rows], wscale));
        out[i] = __fmul_rn(__int2float_rn(dots[i]), inv);
    }
}

// The same for up to LBK_MAX_GROUP matrices that share the token rows, in one launch (blockIdx.y is
// the matrix). `clean`: the sums live in the context's own accumulation buffer, which is kept zero
// between launches: every word is zeroed again once it has been read.
struct EpilogueGroup {
    int32_t *dots[LBK_MAX_GROUP];
    float *out[LBK_MAX_GROUP];
    float wscale[LBK_MAX_GROUP];
    int rows[LBK_MAX_GROUP];
    int clean[LBK_MAX_GROUP];
};
__global__ void __launch_bounds__(256) scale_epilogue_group_kernel(const EpilogueGroup g, const float *__restrict__ ascale, int m) {
    const int mat = blockIdx.y, rows = g.rows[mat];
    int32_t *dots = g.dots[mat];
    float *out = g.out[mat];
    if (!out) return;
    const float ws = g.wscale[mat];
    const size_t total = static_cast<size_t>(m) * rows;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float inv = __fdiv_rn(1.0f, __fmul_rn(ascale[i / rows], ws));
        out[i] = __fmul_rn(__int2float_rn(dots[i]), inv);
        if (g.clean[mat]) dots[i] = 0;
    }
}

}  // namespace

int launch_scale_epilogue_group(Ctx *ctx, int n, int32_t *const *dots, float *const *outs, const float *wscale, const int *rows, const bool *clean,
                                const float *ascale, size_t m, cudaStream_t stream) {
    EpilogueGroup g{};
    size_t most = 0;
    for (int i = 0; i < n; ++i) {
        g.dots[i] = dots[i];
        g.out[i] = outs[i];
        g.wscale[i] = wscale[i];
        g.rows[i] = rows[i];
        g.clean[i] = clean[i] ? 1 : 0;
        if (outs[i] && m * static_cast<size_t>(rows[i]) > most) most = m * static_cast<size_t>(rows[i]);
    }
    if (most == 0) return LBK_OK;
    size_t blocks = (most + 255) / 256;
    if (blocks > static_cast<size_t>(ctx->sm_count) * 8) blocks = static_cast<size_t>(ctx->sm_count) * 8;
    scale_epilogue_group_kernel<<<dim3(static_cast<unsigned>(blocks), static_cast<unsigned>(n)), 256, 0, stream>>>(g, ascale, static_cast<int>(m));
    LBK_CUDA(cudaGetLastError());
    ctx->launches++;
    return LBK_OK;
}

int launch_scale_epilogue(Ctx *ctx, const int32_t *dots, const float *ascale, float wscale, size_t m, size_t rows,
                          float *out, cudaStream_t stream) {
    const size_t total = m * rows;
    if (total == 0) return LBK_OK;
    size_t blocks = (total + 255) / 256;
    if (blocks > static_cast<size_t>(ctx->sm_count) * 8) blocks = static_cast<size_t>(ctx->sm_count) * 8;
    scale_epilogue_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(dots, ascale, wscale, static_cast<int>(rows), total, out);
    LBK_CUDA(cudaGetLastError());
    ctx->launches++;
    return LBK_OK;
}

int launch_quantize_ex(Ctx *ctx, const float *x, size_t m, size_t k, int8_t *q, float *scale, int32_t *sum,
                       const float *amax_in, float *amax_out, cudaStream_t stream) {
    if (m == 0) return LBK_OK;
    const size_t kp = lbk_padded_cols(k);
    quantize_kernel<<<static_cast<unsigned>(m), kQThreads, 0, stream>>>(x, static_cast<int>(k), static_cast<int>(kp), q,
                                                                        scale, sum, amax_in, amax_out);
    LBK_CUDA(cudaGetLastError());
    ctx->launches++;
    return LBK_OK;
}

int launch_quantize(Ctx *ctx, const float *x, size_t m, size_t k, int8_t *q, float *scale,
                    int32_t *sum, cudaStream_t stream) {
    if (m == 0) return LBK_OK;
    const size_t kp = lbk_padded_cols(k);
    quantize_kernel<<<static_cast<unsigned>(m), kQThreads, 0, stream>>>(
        x, static_cast<int>(k), static_cast<int>(kp), q, scale, sum, nullptr, nullptr);
    LBK_CUDA(cudaGetLastError());
    ctx->launches++;
    return LBK_OK;
}

}  // namespace lbk
