// Decoder-step glue around the ternary projections: the pieces of BitNet::forward
// (crates/lb-model/src/model.rs:305-374) that are not matmuls, as small CUDA kernels.
//
//   embed            model.rs:274-282   bf16 table row -> f32
//   rms_norm         model.rs:267-272   x * (1 / sqrt(mean(x^2) + eps)) * w
//   rope + KV append model.rs:295-303, 334-347   rotate-half RoPE on q and k, k/v stored as bf16
//   GQA attention    model.rs:350-357   softmax(q K^T / sqrt(hd)) V over the cached positions,
//                                       split over the sequence ("flash decoding"), f32 math
//   relu^2 * up      model.rs:363
//   residual add     model.rs:359,365
//   argmax           crates/lb-model/src/sample.rs:17-25   first index of the maximum
//
// Every kernel that depends on the decode position reads it from device memory (`pos_dev`), so a
// whole decode step can be captured once in a CUDA graph and replayed for every token. The batch
// dimension is `b` independent sequences, each with its own cache slab. All bandwidth-bound;
// float results agree with the reference to rounding (its tensor library's summation order is
// not visible), not bit for bit.
#include "lbk_internal.cuh"

namespace lbk {

namespace {

__device__ __forceinline__ float bf16_to_f32(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }
// round-to-nearest-even, as a tensor library's f32 -> bf16 cast does
__device__ __forceinline__ uint16_t f32_to_bf16(float f) {
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // NaN
    u += 0x7fffu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}

__device__ __forceinline__ float block_sum(float v, float *s_red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < nw; ++w) t += s_red[w];
    return t;
}

__global__ void embed_kernel(const uint16_t *__restrict__ table, const int *__restrict__ tokens, int hidden,
                             float *__restrict__ out) {
    const int b = blockIdx.x;
    const uint16_t *row = table + static_cast<size_t>(tokens[b]) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[static_cast<size_t>(b) * hidden + i] = bf16_to_f32(row[i]);
}

__global__ void __launch_bounds__(256) rms_norm_kernel(const float *x, const float *__restrict__ w, int n,
                                                      float eps, float *out) {  // out may alias x
    __shared__ float s_red[8];
    const float *xr = x + static_cast<size_t>(blockIdx.x) * n;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += 256) ss += xr[i] * xr[i];
    const float mean = block_sum(ss, s_red) / static_cast<float>(n);
    const float r = 1.0f / sqrtf(mean + eps);
    for (int i = threadIdx.x; i < n; i += 256) out[static_cast<size_t>(blockIdx.x) * n + i] = xr[i] * r * w[i];
}

// One block per (sequence, head). q heads first, then k heads (which are also written to the
// cache together with v). cos/sin: [max_pos][hd] with both halves duplicated (model.rs:213-230).
__global__ void rope_append_kernel(float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                   const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                   const int *__restrict__ pos_dev, int nh, int kvh, int hd, int cap,
                                   uint16_t *__restrict__ kcache, uint16_t *__restrict__ vcache) {
    const int b = blockIdx.y, h = blockIdx.x, pos = *pos_dev;
    const float *c = cos_t + static_cast<size_t>(pos) * hd, *s = sin_t + static_cast<size_t>(pos) * hd;
    const int half = hd >> 1;
    if (h < nh) {
        float *qh = q + (static_cast<size_t>(b) * nh + h) * hd;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float x1 = qh[i], x2 = qh[i + half];
            // x * cos + rotate_half(x) * sin, rotate_half = cat(-x2, x1)   (model.rs:298-302)
            qh[i] = x1 * c[i] + (-x2) * s[i];
            qh[i + half] = x2 * c[i + half] + x1 * s[i + half];
        }
    } else {
        const int kh = h - nh;
        const float *kk = k + (static_cast<size_t>(b) * kvh + kh) * hd;
        const float *vv = v + (static_cast<size_t>(b) * kvh + kh) * hd;
        const size_t slot = ((static_cast<size_t>(b) * kvh + kh) * cap + pos) * hd;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float x1 = kk[i], x2 = kk[i + half];
            kcache[slot + i] = f32_to_bf16(x1 * c[i] + (-x2) * s[i]);
            kcache[slot + i + half] = f32_to_bf16(x2 * c[i + half] + x1 * s[i + half]);
            vcache[slot + i] = f32_to_bf16(vv[i]);
            vcache[slot + i + half] = f32_to_bf16(vv[i + half]);
        }
    }
}

// Split-KV decode attention, head dim 128. Grid (splits, kvh, b); one warp per query head of the
// group (group <= 8), lane owns 4 of the 128 dims. Each block covers a contiguous slice of the
// positions and writes (max, sum, unnormalised acc) per query head; combine_kernel merges them.
constexpr int kHd = 128;
constexpr int kPartStride = kHd + 4;  // acc[128], max, sum, 2 pad floats: keeps rows 16-byte aligned
__global__ void __launch_bounds__(256) attn_partial_kernel(const float *__restrict__ q, const uint16_t *__restrict__ kc,
                                                          const uint16_t *__restrict__ vc, const int *__restrict__ pos_dev,
                                                          int nh, int kvh, int cap, float scaling, int splits,
                                                          float *__restrict__ part /* [b][nh][splits][kPartStride] */) {
    const int sp = blockIdx.x, kh = blockIdx.y, b = blockIdx.z;
    const int group = nh / kvh, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp >= group) return;
    const int total = *pos_dev + 1;  // keys 0..pos
    const int per = (total + splits - 1) / splits;
    const int p0 = sp * per, p1 = min(total, p0 + per);
    const int head = kh * group + warp;
    const float4 qv = *reinterpret_cast<const float4 *>(q + (static_cast<size_t>(b) * nh + head) * kHd + lane * 4);
    const uint16_t *kb = kc + (static_cast<size_t>(b) * kvh + kh) * cap * kHd;
    const uint16_t *vb = vc + (static_cast<size_t>(b) * kvh + kh) * cap * kHd;
    float mx = -INFINITY, sum = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = p0; p < p1; ++p) {
        const uint2 kr = *reinterpret_cast<const uint2 *>(kb + static_cast<size_t>(p) * kHd + lane * 4);
        float d = qv.x * bf16_to_f32(kr.x & 0xffff) + qv.y * bf16_to_f32(kr.x >> 16) + qv.z * bf16_to_f32(kr.y & 0xffff) +
                  qv.w * bf16_to_f32(kr.y >> 16);
        for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        const float sc = d * scaling;
        const float nm = fmaxf(mx, sc);
        const float corr = __expf(mx - nm), w = __expf(sc - nm);
        const uint2 vr = *reinterpret_cast<const uint2 *>(vb + static_cast<size_t>(p) * kHd + lane * 4);
        acc.x = acc.x * corr + w * bf16_to_f32(vr.x & 0xffff);
        acc.y = acc.y * corr + w * bf16_to_f32(vr.x >> 16);
        acc.z = acc.z * corr + w * bf16_to_f32(vr.y & 0xffff);
        acc.w = acc.w * corr + w * bf16_to_f32(vr.y >> 16);
        sum = sum * corr + w;
        mx = nm;
    }
    float *o = part + ((static_cast<size_t>(b) * nh + head) * splits + sp) * kPartStride;
    *reinterpret_cast<float4 *>(o + lane * 4) = acc;
    if (lane == 0) {
        o[kHd] = mx;
        o[kHd + 1] = sum;
    }
}

__global__ void __launch_bounds__(128) attn_combine_kernel(const float *__restrict__ part, int splits,
                                                          float *__restrict__ out /* [b][nh*hd] */) {
    const size_t bh = blockIdx.x;  // b * nh + head
    const float *p = part + bh * splits * kPartStride;
    float mx = -INFINITY;
    for (int s = 0; s < splits; ++s) mx = fmaxf(mx, p[s * kPartStride + kHd]);
    float sum = 0.0f, acc = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float m = p[s * kPartStride + kHd];
        if (m == -INFINITY) continue;  // empty slice
        const float w = __expf(m - mx);
        sum += w * p[s * kPartStride + kHd + 1];
        acc += w * p[s * kPartStride + threadIdx.x];
    }
    out[bh * kHd + threadIdx.x] = acc / sum;
}

__global__ void relu2_mul_kernel(const float *__restrict__ g, const float *__restrict__ u, size_t n, float *__restrict__ out) {
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float r = fmaxf(g[i], 0.0f);
        out[i] = r * r * u[i];
    }
}

__global__ void add_inplace_kernel(float *__restrict__ x, const float *__restrict__ y, size_t n) {
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x)
        x[i] += y[i];
}

// First index of the maximum (strict >, sample.rs:17-25): compare (value desc, index asc).
__global__ void __launch_bounds__(1024) argmax_kernel(const float *__restrict__ logits, int n, int *__restrict__ out) {
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    const float *row = logits + static_cast<size_t>(blockIdx.x) * n;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {  // ascending i: strict > keeps the first maximum
        const float v = row[i];
        if (v > bv) {
            bv = v;
            bi = i;
        }
    }
    auto better = [](float v, int i, float bv2, int bi2) { return v > bv2 || (v == bv2 && i < bi2); };
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_v[warp] = bv; s_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < (blockDim.x >> 5) ? s_v[lane] : -INFINITY;
        bi = lane < (blockDim.x >> 5) ? s_i[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        // the reference starts from index 0 and only moves on a strict >: a NaN in front, or a row
        // with nothing above -inf, stays at 0
        if (lane == 0) out[blockIdx.x] = (bi == 0x7fffffff || row[0] != row[0]) ? 0 : bi;
    }
}

__global__ void advance_pos_kernel(int *pos) { *pos += 1; }

}  // namespace
}  // namespace lbk

using namespace lbk;

#define LBK_DEC_PRE(name)                                              \
    if (!c) return fail(LBK_ERR_INVALID, name ": context is null");     \
    Ctx *ctx = reinterpret_cast<Ctx *>(c);                              \
    LBK_CUDA(cudaSetDevice(ctx->device));                               \
    cudaStream_t st = static_cast<cudaStream_t>(stream)

#define LBK_DEC_POST()          \
    LBK_CUDA(cudaGetLastError()); \
    ctx->launches++;            \
    return LBK_OK

extern "C" {

int lbk_embed_bf16(lbk_ctx *c, const uint16_t *table_dev, const int32_t *tokens_dev, size_t b, size_t hidden, float *out_dev, void *stream) {
    LBK_DEC_PRE("lbk_embed_bf16");
    if (b == 0) return LBK_OK;
    if (!table_dev || !tokens_dev || !out_dev) return fail(LBK_ERR_INVALID, "lbk_embed_bf16: null buffer");
    embed_kernel<<<static_cast<unsigned>(b), 256, 0, st>>>(table_dev, tokens_dev, static_cast<int>(hidden), out_dev);
    LBK_DEC_POST();
}

int lbk_rms_norm(lbk_ctx *c, const float *x_dev, const float *w_dev, size_t rows, size_t n, float eps, float *out_dev, void *stream) {
    LBK_DEC_PRE("lbk_rms_norm");
    if (rows == 0) return LBK_OK;
    if (!x_dev || !w_dev || !out_dev || n == 0) return fail(LBK_ERR_INVALID, "lbk_rms_norm: null buffer or empty row");
    rms_norm_kernel<<<static_cast<unsigned>(rows), 256, 0, st>>>(x_dev, w_dev, static_cast<int>(n), eps, out_dev);
    LBK_DEC_POST();
}

int lbk_rope_kv_append(lbk_ctx *c, float *q_dev, const float *k_dev, const float *v_dev, const float *cos_dev, const float *sin_dev,
                       const int32_t *pos_dev, size_t b, size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap,
                       uint16_t *kcache_dev, uint16_t *vcache_dev, void *stream) {
    LBK_DEC_PRE("lbk_rope_kv_append");
    if (b == 0) return LBK_OK;
    if (!q_dev || !k_dev || !v_dev || !cos_dev || !sin_dev || !pos_dev || !kcache_dev || !vcache_dev)
        return fail(LBK_ERR_INVALID, "lbk_rope_kv_append: null buffer");
    if (head_dim & 1) return fail(LBK_ERR_SHAPE, "head_dim must be even");
    dim3 grid(static_cast<unsigned>(n_heads + kv_heads), static_cast<unsigned>(b));
    rope_append_kernel<<<grid, 64, 0, st>>>(q_dev, k_dev, v_dev, cos_dev, sin_dev, pos_dev, static_cast<int>(n_heads),
                                            static_cast<int>(kv_heads), static_cast<int>(head_dim), static_cast<int>(cap),
                                            kcache_dev, vcache_dev);
    LBK_DEC_POST();
}

int lbk_attn_decode(lbk_ctx *c, const float *q_dev, const uint16_t *kcache_dev, const uint16_t *vcache_dev, const int32_t *pos_dev,
                    size_t b, size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap, size_t splits, float *scratch_dev,
                    float *out_dev, void *stream) {
    LBK_DEC_PRE("lbk_attn_decode");
    if (b == 0) return LBK_OK;
    if (!q_dev || !kcache_dev || !vcache_dev || !pos_dev || !scratch_dev || !out_dev) return fail(LBK_ERR_INVALID, "lbk_attn_decode: null buffer");
    if (head_dim != kHd) return fail(LBK_ERR_UNSUPPORTED, "attention kernel is built for head_dim 128, got %zu", head_dim);
    if (kv_heads == 0 || n_heads % kv_heads || n_heads / kv_heads > 8) return fail(LBK_ERR_UNSUPPORTED, "query group size must be 1..8");
    if (splits == 0) return fail(LBK_ERR_INVALID, "splits must be positive");
    dim3 grid(static_cast<unsigned>(splits), static_cast<unsigned>(kv_heads), static_cast<unsigned>(b));
    attn_partial_kernel<<<grid, 256, 0, st>>>(q_dev, kcache_dev, vcache_dev, pos_dev, static_cast<int>(n_heads), static_cast<int>(kv_heads),
                                              static_cast<int>(cap), 1.0f / sqrtf(static_cast<float>(head_dim)), static_cast<int>(splits),
                                              scratch_dev);
    LBK_CUDA(cudaGetLastError());
    attn_combine_kernel<<<static_cast<unsigned>(b * n_heads), kHd, 0, st>>>(scratch_dev, static_cast<int>(splits), out_dev);
    ctx->launches++;
    LBK_DEC_POST();
}

int lbk_relu2_mul(lbk_ctx *c, const float *g_dev, const float *u_dev, size_t n, float *out_dev, void *stream) {
    LBK_DEC_PRE("lbk_relu2_mul");
    if (n == 0) return LBK_OK;
    if (!g_dev || !u_dev || !out_dev) return fail(LBK_ERR_INVALID, "lbk_relu2_mul: null buffer");
    relu2_mul_kernel<<<static_cast<unsigned>((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184), 256, 0, st>>>(g_dev, u_dev, n, out_dev);
    LBK_DEC_POST();
}

int lbk_add_inplace(lbk_ctx *c, float *x_dev, const float *y_dev, size_t n, void *stream) {
    LBK_DEC_PRE("lbk_add_inplace");
    if (n == 0) return LBK_OK;
    if (!x_dev || !y_dev) return fail(LBK_ERR_INVALID, "lbk_add_inplace: null buffer");
    add_inplace_kernel<<<static_cast<unsigned>((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184), 256, 0, st>>>(x_dev, y_dev, n);
    LBK_DEC_POST();
}

int lbk_argmax(lbk_ctx *c, const float *logits_dev, size_t rows, size_t n, int32_t *out_dev, void *stream) {
    LBK_DEC_PRE("lbk_argmax");
    if (rows == 0) return LBK_OK;
    if (!logits_dev || !out_dev || n == 0) return fail(LBK_ERR_INVALID, "lbk_argmax: null buffer or empty row");
    argmax_kernel<<<static_cast<unsigned>(rows), 1024, 0, st>>>(logits_dev, static_cast<int>(n), out_dev);
    LBK_DEC_POST();
}

int lbk_advance_pos(lbk_ctx *c, int32_t *pos_dev, void *stream) {
    LBK_DEC_PRE("lbk_advance_pos");
    if (!pos_dev) return fail(LBK_ERR_INVALID, "lbk_advance_pos: null buffer");
    advance_pos_kernel<<<1, 1, 0, st>>>(pos_dev);
    LBK_DEC_POST();
}

}  // extern "C"
