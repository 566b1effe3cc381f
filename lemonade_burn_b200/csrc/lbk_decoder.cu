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
#include "lbk_ptx.cuh"

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
    ptx::pdl_trigger();  // the next kernel of the step may be scheduled now
    ptx::pdl_wait();     // everything this kernel reads or overwrites is settled from here on

    const int b = blockIdx.x;
    const uint16_t *row = table + static_cast<size_t>(tokens[b]) * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[static_cast<size_t>(b) * hidden + i] = bf16_to_f32(row[i]);
}

__global__ void __launch_bounds__(256) rms_norm_kernel(const float *x, const float *__restrict__ w, int n,
                                                      float eps, float *out) {
    ptx::pdl_trigger();  // the next kernel of the step may be scheduled now
    ptx::pdl_wait();     // everything this kernel reads or overwrites is settled from here on (out may alias x)

    __shared__ float s_red[8];
    const float *xr = x + static_cast<size_t>(blockIdx.x) * n;
    float *orow = out + static_cast<size_t>(blockIdx.x) * n;
    const bool vec = (n & 3) == 0 && n <= 8192 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) |
                                                     reinterpret_cast<uintptr_t>(w)) & 15) == 0;
    if (vec) {
        // the row is read once and stays in registers between the reduction and the scaling
        const int n4 = n >> 2;
        float4 v[8];
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = threadIdx.x + j * 256;
            v[j] = i < n4 ? reinterpret_cast<const float4 *>(xr)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
        const float r = 1.0f / sqrtf(block_sum(ss, s_red) / static_cast<float>(n) + eps);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = threadIdx.x + j * 256;
            if (i < n4) {
                const float4 g = __ldg(reinterpret_cast<const float4 *>(w) + i);
                reinterpret_cast<float4 *>(orow)[i] = make_float4(v[j].x * r * g.x, v[j].y * r * g.y, v[j].z * r * g.z, v[j].w * r * g.w);
            }
        }
        return;
    }
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += 256) ss += xr[i] * xr[i];
    const float mean = block_sum(ss, s_red) / static_cast<float>(n);
    const float r = 1.0f / sqrtf(mean + eps);
    for (int i = threadIdx.x; i < n; i += 256) orow[i] = xr[i] * r * w[i];
}

// A position read from device memory is trusted by nobody: a step replayed once too often (a
// recorded graph launched after the cache filled up) would otherwise write K/V rows past the
// sequence's slab and read the RoPE tables out of range. Every kernel that takes its position
// from `pos_dev` checks it first; a block whose position is outside [0, cap) records error code 7
// in the context's error word and returns before touching memory. `last` is the highest
// position the kernel uses (pos itself for one token, pos + n - 1 for a prompt pass). The reference
// asserts the same on the host (model.rs:309).
__device__ __forceinline__ bool pos_in_cache(int first, int last, int cap, int *err_word) {
    if (first >= 0 && last < cap && first <= last) return true;
    if (threadIdx.x == 0) atomicExch(err_word, 7);
    return false;
}

// One block per (sequence, head). q heads first, then k heads (which are also written to the
// cache together with v). cos/sin: [max_pos][hd] with both halves duplicated (model.rs:213-230).
__global__ void rope_append_kernel(float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                   const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                   const int *__restrict__ pos_dev, int pos_stride, int nh, int kvh, int hd, int cap,
                                   uint16_t *__restrict__ kcache, uint16_t *__restrict__ vcache, int *err_word) {
    ptx::pdl_trigger();  // the next kernel of the step may be scheduled now
    ptx::pdl_wait();     // everything this kernel reads or overwrites is settled from here on

    const int b = blockIdx.y, h = blockIdx.x, pos = pos_dev[b * pos_stride];  // stride 0: one position for all sequences
    if (!pos_in_cache(pos, pos, cap, err_word)) return;
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
                                                          int pos_stride, int nh, int kvh, int cap, float scaling, int splits,
                                                          float *__restrict__ part /* [b][nh][splits][kPartStride] */, int *err_word) {
    ptx::pdl_trigger();  // the next kernel of the step may be scheduled now
    ptx::pdl_wait();     // everything this kernel reads or overwrites is settled from here on

    const int sp = blockIdx.x, kh = blockIdx.y, b = blockIdx.z;
    const int group = nh / kvh, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total = pos_dev[b * pos_stride] + 1;  // keys 0..pos
    if (!pos_in_cache(total - 1, total - 1, cap, err_word)) return;
    if (warp >= group) return;
    const int per = (total + splits - 1) / splits;
    const int p0 = sp * per, p1 = min(total, p0 + per);
    const int head = kh * group + warp;
    const float4 qv = *reinterpret_cast<const float4 *>(q + (static_cast<size_t>(b) * nh + head) * kHd + lane * 4);
    const uint16_t *kb = kc + (static_cast<size_t>(b) * kvh + kh) * cap * kHd;
    const uint16_t *vb = vc + (static_cast<size_t>(b) * kvh + kh) * cap * kHd;
    float mx = -INFINITY, sum = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    constexpr int U = 8;  // positions in flight per iteration: their loads and shuffle trees overlap
    for (int pc = p0; pc < p1; pc += U) {
        float sc[U];
        uint2 vr[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int p = pc + j < p1 ? pc + j : p1 - 1;
            const uint2 kr = *reinterpret_cast<const uint2 *>(kb + static_cast<size_t>(p) * kHd + lane * 4);
            vr[j] = *reinterpret_cast<const uint2 *>(vb + static_cast<size_t>(p) * kHd + lane * 4);
            sc[j] = qv.x * bf16_to_f32(kr.x & 0xffff) + qv.y * bf16_to_f32(kr.x >> 16) + qv.z * bf16_to_f32(kr.y & 0xffff) +
                    qv.w * bf16_to_f32(kr.y >> 16);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int j = 0; j < U; ++j) sc[j] += __shfl_xor_sync(0xffffffffu, sc[j], o);
        float nm = mx;
#pragma unroll
        for (int j = 0; j < U; ++j) {
            sc[j] = pc + j < p1 ? sc[j] * scaling : -INFINITY;
            nm = fmaxf(nm, sc[j]);
        }
        const float corr = __expf(mx - nm);
        acc.x *= corr; acc.y *= corr; acc.z *= corr; acc.w *= corr;
        sum *= corr;
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const float w = __expf(sc[j] - nm);  // 0 for the padded tail
            acc.x += w * bf16_to_f32(vr[j].x & 0xffff);
            acc.y += w * bf16_to_f32(vr[j].x >> 16);
            acc.z += w * bf16_to_f32(vr[j].y & 0xffff);
            acc.w += w * bf16_to_f32(vr[j].y >> 16);
            sum += w;
        }
        mx = nm;
    }
    float *o = part + ((static_cast<size_t>(b) * nh + head) * splits + sp) * kPartStride;
    *reinterpret_cast<float4 *>(o + lane * 4) = acc;
    if (lane == 0) {
        o[kHd] = mx;
        o[kHd + 1] = sum;
    }
}

// The same slice-of-positions kernel for grouped-query attention with the K/V rows staged in
// shared memory: the warps of a block are the query heads of ONE KV head, so the rows are fetched
// from HBM once per block (128-bit loads, all in flight at once: one DRAM round trip per 32
// positions) instead of once per warp, and the per-position warp reductions of the kernel above
// disappear: for q.K lane p owns position p and walks its row (K rows are padded to 272 bytes, which
// makes the 16-byte reads of 8 neighbouring lanes hit distinct banks; q is read as a broadcast);
// for P.V lane l owns dims 4l..4l+3 and the weights travel by shuffle.
constexpr int kAttnChunk = 32;           // positions staged at a time (one per lane)
constexpr int kKRow = kHd * 2 + 16;      // bytes per staged K row
constexpr int kVRow = kHd * 2;           // bytes per staged V row
__global__ void __launch_bounds__(256) attn_partial_staged_kernel(const float *__restrict__ q, const uint16_t *__restrict__ kc,
                                                                 const uint16_t *__restrict__ vc, const int *__restrict__ pos_dev,
                                                                 int pos_stride, int nh, int kvh, int cap, float scaling, int splits,
                                                                 float *__restrict__ part /* [b][nh][splits][kPartStride] */, int *err_word) {
    ptx::pdl_trigger();
    ptx::pdl_wait();
    __shared__ __align__(16) uint8_t s_k[kAttnChunk * kKRow];
    __shared__ __align__(16) uint8_t s_v[kAttnChunk * kVRow];
    __shared__ __align__(16) float s_q[8 * kHd];
    const int sp = blockIdx.x, kh = blockIdx.y, b = blockIdx.z;
    const int group = nh / kvh, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nthr = blockDim.x;
    const int total = pos_dev[b * pos_stride] + 1;  // keys 0..pos
    if (!pos_in_cache(total - 1, total - 1, cap, err_word)) return;
    const int per = (total + splits - 1) / splits;
    const int p0 = sp * per, p1 = min(total, p0 + per);
    const int head = kh * group + warp;
    for (int i = tid; i < group * kHd; i += nthr) s_q[i] = q[(static_cast<size_t>(b) * nh + kh * group) * kHd + i] * scaling;
    const uint16_t *kb = kc + (static_cast<size_t>(b) * kvh + kh) * cap * kHd;
    const uint16_t *vb = vc + (static_cast<size_t>(b) * kvh + kh) * cap * kHd;
    float mx = -INFINITY, sum = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int pc = p0; pc < p1; pc += kAttnChunk) {
        const int n = min(kAttnChunk, p1 - pc);
        __syncthreads();  // the previous chunk has been consumed (and s_q is written, first time round)
        // stage n rows of K and of V, 16 segments of 16 bytes per row: every load is issued before
        // the first store, so the chunk costs one trip to HBM
        constexpr int kSegIters = kAttnChunk * 16 / 128;  // blocks of 128 threads and more (4 query heads per KV head)
        uint4 kreg[kSegIters], vreg[kSegIters];
#pragma unroll
        for (int j = 0; j < kSegIters; ++j) {
            const int i = tid + j * nthr;
            if (i < n * 16) {
                const int r = i >> 4, seg = i & 15;
                kreg[j] = *reinterpret_cast<const uint4 *>(kb + static_cast<size_t>(pc + r) * kHd + seg * 8);
                vreg[j] = *reinterpret_cast<const uint4 *>(vb + static_cast<size_t>(pc + r) * kHd + seg * 8);
            }
        }
#pragma unroll
        for (int j = 0; j < kSegIters; ++j) {
            const int i = tid + j * nthr;
            if (i < n * 16) {
                const int r = i >> 4, seg = i & 15;
                *reinterpret_cast<uint4 *>(s_k + r * kKRow + seg * 16) = kreg[j];
                *reinterpret_cast<uint4 *>(s_v + r * kVRow + seg * 16) = vreg[j];
            }
        }
        __syncthreads();
        // q.K: lane p walks row p
        float sc = -INFINITY;
        if (lane < n) {
            const uint8_t *kr = s_k + lane * kKRow;
            const float *qh = s_q + warp * kHd;
            float d0 = 0.f, d1 = 0.f;
#pragma unroll
            for (int it = 0; it < kHd / 8; ++it) {
                const uint4 kk = *reinterpret_cast<const uint4 *>(kr + it * 16);
                const float4 qa = *reinterpret_cast<const float4 *>(qh + it * 8), qb = *reinterpret_cast<const float4 *>(qh + it * 8 + 4);
                d0 += qa.x * bf16_to_f32(kk.x & 0xffff) + qa.y * bf16_to_f32(kk.x >> 16) + qa.z * bf16_to_f32(kk.y & 0xffff) +
                      qa.w * bf16_to_f32(kk.y >> 16);
                d1 += qb.x * bf16_to_f32(kk.z & 0xffff) + qb.y * bf16_to_f32(kk.z >> 16) + qb.z * bf16_to_f32(kk.w & 0xffff) +
                      qb.w * bf16_to_f32(kk.w >> 16);
            }
            sc = d0 + d1;
        }
        float nm = sc;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) nm = fmaxf(nm, __shfl_xor_sync(0xffffffffu, nm, o));
        nm = fmaxf(nm, mx);
        const float corr = __expf(mx - nm);
        const float w = lane < n ? __expf(sc - nm) : 0.0f;
        float ws = w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ws += __shfl_xor_sync(0xffffffffu, ws, o);
        sum = sum * corr + ws;
        acc.x *= corr; acc.y *= corr; acc.z *= corr; acc.w *= corr;
        // P.V: lane l owns dims 4l..4l+3
        const uint8_t *vr = s_v + lane * 8;
#pragma unroll 8
        for (int p = 0; p < n; ++p) {
            const float wp = __shfl_sync(0xffffffffu, w, p);
            const uint2 vv = *reinterpret_cast<const uint2 *>(vr + p * kVRow);
            acc.x += wp * bf16_to_f32(vv.x & 0xffff);
            acc.y += wp * bf16_to_f32(vv.x >> 16);
            acc.z += wp * bf16_to_f32(vv.y & 0xffff);
            acc.w += wp * bf16_to_f32(vv.y >> 16);
        }
        mx = nm;
    }
    float *o = part + ((static_cast<size_t>(b) * nh + head) * splits + sp) * kPartStride;
    *reinterpret_cast<float4 *>(o + lane * 4) = acc;
    if (lane == 0) {
        o[kHd] = mx;
        o[kHd + 1] = sum;
    }
}

// The whole attention of a decode step in one launch, for grouped queries (4..8 query heads per KV
// head, head dim 128): RoPE on q and on the new k (model.rs:298-302), the new position's K/V row
// appended to the bf16 cache, the staged slice kernel above, and the merge of the slices done by
// whichever block of a KV head finishes last (each block counts itself after publishing its
// partial results; the counter resets itself). Grid (splits, kvh, b), block 32 * group threads.
// `counters`: b * kvh ints, zero before the first launch.
template <bool MERGE>
__global__ void __launch_bounds__(256, 3) attn_fused_kernel(const float *__restrict__ q_raw, const float *__restrict__ k_new,
                                                        const float *__restrict__ v_new, const float *__restrict__ cos_t,
                                                        const float *__restrict__ sin_t, const int *__restrict__ pos_dev, int pos_stride, int nh,
                                                        int kvh, int cap, float scaling, int splits, uint16_t *__restrict__ kc,
                                                        uint16_t *__restrict__ vc, float *__restrict__ part, int *__restrict__ counters,
                                                        float *__restrict__ out /* [b][nh*hd] */, int *err_word) {
    ptx::pdl_trigger();
    ptx::pdl_wait();
    __shared__ __align__(16) uint8_t s_k[kAttnChunk * kKRow];  // later: the merge's weights, [group][splits]
    __shared__ __align__(16) uint8_t s_v[kAttnChunk * kVRow];
    __shared__ __align__(16) float s_q[8 * kHd];
    __shared__ int s_last;
    const int sp = blockIdx.x, kh = blockIdx.y, b = blockIdx.z;
    const int group = nh / kvh, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nthr = blockDim.x;
    const int pos = pos_dev[b * pos_stride], total = pos + 1;  // keys 0..pos
    if (!pos_in_cache(pos, pos, cap, err_word)) return;  // every block of the sequence leaves: the counters stay zero
    const int per = (total + splits - 1) / splits;
    const int p0 = sp * per, p1 = min(total, p0 + per);
    const int head = kh * group + warp;
    const float *cs = cos_t + static_cast<size_t>(pos) * kHd, *sn = sin_t + static_cast<size_t>(pos) * kHd;
    // x * cos + rotate_half(x) * sin, rotate_half = cat(-x2, x1), then the 1/sqrt(d) of the scores
    for (int i = tid; i < group * kHd; i += nthr) {
        const int d = i & (kHd - 1);
        const float *qh = q_raw + (static_cast<size_t>(b) * nh + kh * group) * kHd + (i - d);
        const float v = d < kHd / 2 ? qh[d] * cs[d] + (-qh[d + kHd / 2]) * sn[d] : qh[d] * cs[d] + qh[d - kHd / 2] * sn[d];
        s_q[i] = v * scaling;
    }
    uint16_t *kb = kc + (static_cast<size_t>(b) * kvh + kh) * cap * kHd;
    uint16_t *vb = vc + (static_cast<size_t>(b) * kvh + kh) * cap * kHd;
    float mx = -INFINITY, sum = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int pc = p0; pc < p1; pc += kAttnChunk) {
        const int n = min(kAttnChunk, p1 - pc);
        __syncthreads();  // the previous chunk has been consumed (and s_q is written, first time round)
        constexpr int kSegIters = kAttnChunk * 16 / 128;
        uint4 kreg[kSegIters], vreg[kSegIters];
#pragma unroll
        for (int j = 0; j < kSegIters; ++j) {
            const int i = tid + j * nthr;
            if (i < n * 16 && pc + (i >> 4) != pos) {  // the row of the new position is not in the cache yet
                const int r = i >> 4, seg = i & 15;
                kreg[j] = *reinterpret_cast<const uint4 *>(kb + static_cast<size_t>(pc + r) * kHd + seg * 8);
                vreg[j] = *reinterpret_cast<const uint4 *>(vb + static_cast<size_t>(pc + r) * kHd + seg * 8);
            }
        }
#pragma unroll
        for (int j = 0; j < kSegIters; ++j) {
            const int i = tid + j * nthr;
            if (i < n * 16 && pc + (i >> 4) != pos) {
                const int r = i >> 4, seg = i & 15;
                *reinterpret_cast<uint4 *>(s_k + r * kKRow + seg * 16) = kreg[j];
                *reinterpret_cast<uint4 *>(s_v + r * kVRow + seg * 16) = vreg[j];
            }
        }
        if (pos >= pc && pos < pc + n && tid < kHd) {
            // the new position: RoPE on k, both rows rounded to bf16 as the cache holds them, stored
            // in the cache by this block (the only one whose slice contains the position)
            const float *kn = k_new + (static_cast<size_t>(b) * kvh + kh) * kHd, *vn = v_new + (static_cast<size_t>(b) * kvh + kh) * kHd;
            const int d = tid;
            const float kr = d < kHd / 2 ? kn[d] * cs[d] + (-kn[d + kHd / 2]) * sn[d] : kn[d] * cs[d] + kn[d - kHd / 2] * sn[d];
            const uint16_t kbits = f32_to_bf16(kr), vbits = f32_to_bf16(vn[d]);
            reinterpret_cast<uint16_t *>(s_k + (pos - pc) * kKRow)[d] = kbits;
            reinterpret_cast<uint16_t *>(s_v + (pos - pc) * kVRow)[d] = vbits;
            kb[static_cast<size_t>(pos) * kHd + d] = kbits;
            vb[static_cast<size_t>(pos) * kHd + d] = vbits;
        }
        __syncthreads();
        float sc = -INFINITY;
        if (lane < n) {
            const uint8_t *kr = s_k + lane * kKRow;
            const float *qh = s_q + warp * kHd;
            float d0 = 0.f, d1 = 0.f;
#pragma unroll
            for (int it = 0; it < kHd / 8; ++it) {
                const uint4 kk = *reinterpret_cast<const uint4 *>(kr + it * 16);
                const float4 qa = *reinterpret_cast<const float4 *>(qh + it * 8), qb = *reinterpret_cast<const float4 *>(qh + it * 8 + 4);
                d0 += qa.x * bf16_to_f32(kk.x & 0xffff) + qa.y * bf16_to_f32(kk.x >> 16) + qa.z * bf16_to_f32(kk.y & 0xffff) +
                      qa.w * bf16_to_f32(kk.y >> 16);
                d1 += qb.x * bf16_to_f32(kk.z & 0xffff) + qb.y * bf16_to_f32(kk.z >> 16) + qb.z * bf16_to_f32(kk.w & 0xffff) +
                      qb.w * bf16_to_f32(kk.w >> 16);
            }
            sc = d0 + d1;
        }
        float nm = sc;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) nm = fmaxf(nm, __shfl_xor_sync(0xffffffffu, nm, o));
        nm = fmaxf(nm, mx);
        const float corr = __expf(mx - nm);
        const float w = lane < n ? __expf(sc - nm) : 0.0f;
        float ws = w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ws += __shfl_xor_sync(0xffffffffu, ws, o);
        sum = sum * corr + ws;
        acc.x *= corr; acc.y *= corr; acc.z *= corr; acc.w *= corr;
        const uint8_t *vr = s_v + lane * 8;
#pragma unroll 8
        for (int p = 0; p < n; ++p) {
            const float wp = __shfl_sync(0xffffffffu, w, p);
            const uint2 vv = *reinterpret_cast<const uint2 *>(vr + p * kVRow);
            acc.x += wp * bf16_to_f32(vv.x & 0xffff);
            acc.y += wp * bf16_to_f32(vv.x >> 16);
            acc.z += wp * bf16_to_f32(vv.y & 0xffff);
            acc.w += wp * bf16_to_f32(vv.y >> 16);
        }
        mx = nm;
    }
    float *prt = part + (static_cast<size_t>(b) * nh + head) * splits * kPartStride;
    float *o = prt + static_cast<size_t>(sp) * kPartStride;
    *reinterpret_cast<float4 *>(o + lane * 4) = acc;
    if (lane == 0) {
        o[kHd] = mx;
        o[kHd + 1] = sum;
    }
    if (!MERGE) return;  // the caller merges the slices with attn_combine_kernel
    // ---- merge by the last block of this KV head --------------------------------------------
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int *cnt = counters + b * kvh + kh;
        const int old = atomicAdd(cnt, 1);
        s_last = old == splits - 1;
        if (s_last) *cnt = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float *s_w = reinterpret_cast<float *>(s_k) + warp * splits;  // this head's weights exp(m_s - m); splits <= 256
    float gm = -INFINITY;
    for (int s2 = lane; s2 < splits; s2 += 32) gm = fmaxf(gm, __ldcg(prt + s2 * kPartStride + kHd));
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, o2));
    float gs = 0.0f;
    for (int s2 = lane; s2 < splits; s2 += 32) {
        const float m = __ldcg(prt + s2 * kPartStride + kHd);
        const float w = m == -INFINITY ? 0.0f : __expf(m - gm);  // empty slices weigh nothing
        s_w[s2] = w;
        gs += w * __ldcg(prt + s2 * kPartStride + kHd + 1);
    }
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) gs += __shfl_xor_sync(0xffffffffu, gs, o2);
    __syncwarp();
    float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int s2 = 0; s2 < splits; ++s2) {
        const float w = s_w[s2];
        const float4 a = __ldcg(reinterpret_cast<const float4 *>(prt + s2 * kPartStride) + lane);
        tot.x += w * a.x; tot.y += w * a.y; tot.z += w * a.z; tot.w += w * a.w;
    }
    const float inv = 1.0f / gs;
    *reinterpret_cast<float4 *>(out + (static_cast<size_t>(b) * nh + head) * kHd + lane * 4) = make_float4(tot.x * inv, tot.y * inv, tot.z * inv, tot.w * inv);
}

// ---- prompt ingestion: n consecutive positions of ONE sequence at once -----------------------------
// RoPE on the n query rows (in place) and the n new key rows, which are appended with the value
// rows at positions pos0 .. pos0 + n - 1 of sequence `seq` (model.rs:298-302, 339-341).
__global__ void __launch_bounds__(256) rope_append_rows_kernel(float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                                              const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                                              const int *__restrict__ pos_dev, int nh, int kvh, int hd, int cap, int seq,
                                                              uint16_t *__restrict__ kcache, uint16_t *__restrict__ vcache, int *err_word) {
    ptx::pdl_trigger();
    ptx::pdl_wait();
    const int row = blockIdx.x, pos = *pos_dev + row, half = hd >> 1;  // one block per prompt row, all its heads
    if (!pos_in_cache(*pos_dev, *pos_dev + static_cast<int>(gridDim.x) - 1, cap, err_word)) return;
    const float *c = cos_t + static_cast<size_t>(pos) * hd, *s = sin_t + static_cast<size_t>(pos) * hd;
    for (int it = threadIdx.x; it < (nh + kvh) * half; it += blockDim.x) {
        const int h = it / half, i = it - h * half;
        if (h < nh) {
            float *qh = q + (static_cast<size_t>(row) * nh + h) * hd;
            const float x1 = qh[i], x2 = qh[i + half];
            qh[i] = x1 * c[i] + (-x2) * s[i];
            qh[i + half] = x2 * c[i + half] + x1 * s[i + half];
        } else {
            const int kh = h - nh;
            const float *kk = k + (static_cast<size_t>(row) * kvh + kh) * hd;
            const float *vv = v + (static_cast<size_t>(row) * kvh + kh) * hd;
            const size_t slot = ((static_cast<size_t>(seq) * kvh + kh) * cap + pos) * hd;
            const float x1 = kk[i], x2 = kk[i + half];
            kcache[slot + i] = f32_to_bf16(x1 * c[i] + (-x2) * s[i]);
            kcache[slot + i + half] = f32_to_bf16(x2 * c[i + half] + x1 * s[i + half]);
            vcache[slot + i] = f32_to_bf16(vv[i]);
            vcache[slot + i + half] = f32_to_bf16(vv[i + half]);
        }
    }
}

// Causal attention of n query rows of one sequence over its cache, on the tensor cores: a block
// takes one KV head and 16-row tiles of the query heads that share it (one warp per (head, tile): 16 query rows x 128 dimensions),
// walks the keys in chunks of 64 staged in shared memory as bf16 (two stages: the next chunk's
// asynchronous copies run under this chunk's arithmetic) and keeps the running softmax in
// the accumulator layout of mma.sync m16n8k16 (scores S = Q K^T: 8 tiles of 16x8; output O += P V:
// 16 tiles of 16x8). The f32 queries and the probabilities are each split into two bf16 terms
// (x = hi + lo, |error| <= 2^-17 |x|), so that the only rounding beyond f32 summation is the bf16
// of the cache itself, as in the decode kernels. Row i of the prompt sees keys 0 .. pos0 + i.
constexpr int kPfKeys = 64;          // keys per staged chunk (32, with three blocks per SM instead of two, measured the same or slower)
constexpr int kPfNJ = kPfKeys / 8;   // score tiles (16 rows x 8 keys) per chunk
constexpr int kPfRow = kHd * 2 + 16; // bytes per staged row: eight consecutive rows start in eight different 16-byte bank groups
constexpr int kPfQWarp = 2 * 16 * kPfRow;  // one warp's queries: hi and lo, 16 rows each
constexpr int kPfStage = 2 * kPfKeys * kPfRow;  // one staged chunk: keys, then values

__device__ __forceinline__ uint32_t pack_bf16(float lo_elem, float hi_elem) {
    return static_cast<uint32_t>(f32_to_bf16(lo_elem)) | (static_cast<uint32_t>(f32_to_bf16(hi_elem)) << 16);
}
__device__ __forceinline__ float bf16_round(float x) { return bf16_to_f32(f32_to_bf16(x)); }

__global__ void __launch_bounds__(256) attn_prompt_mma_kernel(const float *__restrict__ q, const uint16_t *__restrict__ kc,
                                                             const uint16_t *__restrict__ vc, const int *__restrict__ pos_dev, int n, int nh,
                                                             int kvh, int cap, int seq, float scaling, float *__restrict__ out /* [n][nh*hd] */, int *err_word) {
    ptx::pdl_trigger();
    ptx::pdl_wait();
    if (!pos_in_cache(*pos_dev, *pos_dev + n - 1, cap, err_word)) return;
    extern __shared__ __align__(16) uint8_t pf_smem[];
    uint8_t *s_kv = pf_smem, *s_q = pf_smem + 2 * kPfStage;  // two stages of [K chunk][V chunk], then the queries
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3, nthr = blockDim.x;
    const int group = nh / kvh, tiles_per_block = (nthr >> 5) / group;
    const int kh = blockIdx.x, btile = gridDim.y - 1 - blockIdx.y;  // the late rows see the most keys: they start first
    const int head = kh * group + warp % group;
    const int row0 = (btile * tiles_per_block + warp / group) * 16;
    const int pos0 = *pos_dev;
    // this warp's queries, scaled, as hi + lo
    uint8_t *qw = s_q + warp * kPfQWarp;
    for (int r = 0; r < 16; ++r) {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < n) x = *reinterpret_cast<const float4 *>(q + (static_cast<size_t>(row0 + r) * nh + head) * kHd + lane * 4);
        x.x *= scaling; x.y *= scaling; x.z *= scaling; x.w *= scaling;
        const float hx = bf16_round(x.x), hy = bf16_round(x.y), hz = bf16_round(x.z), hw = bf16_round(x.w);
        *reinterpret_cast<uint2 *>(qw + r * kPfRow + lane * 8) = make_uint2(pack_bf16(hx, hy), pack_bf16(hz, hw));
        *reinterpret_cast<uint2 *>(qw + (16 + r) * kPfRow + lane * 8) = make_uint2(pack_bf16(x.x - hx, x.y - hy), pack_bf16(x.z - hz, x.w - hw));
    }
    __syncwarp();
    const int block_rows_end = min(n, (btile + 1) * tiles_per_block * 16);
    const int total = pos0 + block_rows_end;             // keys 0 .. total-1 are seen by some row of the block
    const int lim0 = pos0 + row0 + g, lim1 = lim0 + 8;   // the last key this thread's two rows see
    const uint16_t *kb = kc + (static_cast<size_t>(seq) * kvh + kh) * cap * kHd;
    const uint16_t *vb = vc + (static_cast<size_t>(seq) * kvh + kh) * cap * kHd;
    // ldmatrix lane addresses (see the fragment layouts of mma.m16n8k16)
    const uint32_t q_hi = ptx::smem_u32(qw) + ((lane & 7) + 8 * ((lane >> 3) & 1)) * kPfRow + (lane >> 4) * 16;
    const uint32_t q_lo = q_hi + 16 * kPfRow;
    const uint32_t k_lane0 = ptx::smem_u32(s_kv) + (lane & 7) * kPfRow + (lane >> 3) * 16;
    const uint32_t v_lane0 = ptx::smem_u32(s_kv) + kPfKeys * kPfRow + ((lane & 7) + 8 * ((lane >> 3) & 1)) * kPfRow + (lane >> 4) * 16;
    // chunk `pc` into stage `buf`: asynchronous copies, one group per chunk; rows past the end are zeros
    // (their weights are zero, but their bits must be numbers)
    auto stage = [&](int buf, int pc) {
        const int cnt = min(kPfKeys, total - pc);
        uint8_t *dk = s_kv + buf * kPfStage, *dv = dk + kPfKeys * kPfRow;
        for (int i = tid; i < kPfKeys * 16; i += nthr) {
            const int r = i >> 4, sg = i & 15;
            if (r < cnt) {
                ptx::cp_async_16(ptx::smem_u32(dk + r * kPfRow + sg * 16), kb + static_cast<size_t>(pc + r) * kHd + sg * 8);
                ptx::cp_async_16(ptx::smem_u32(dv + r * kPfRow + sg * 16), vb + static_cast<size_t>(pc + r) * kHd + sg * 8);
            } else {
                *reinterpret_cast<uint4 *>(dk + r * kPfRow + sg * 16) = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4 *>(dv + r * kPfRow + sg * 16) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        ptx::cp_async_commit();
    };
    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    stage(0, 0);
    for (int pc = 0, it = 0; pc < total; pc += kPfKeys, ++it) {
        if (it) __syncthreads();  // everyone is done with the stage that the next chunk overwrites
        if (pc + kPfKeys < total) {
            stage((it & 1) ^ 1, pc + kPfKeys);
            ptx::cp_async_wait<1>();
        } else {
            ptx::cp_async_wait<0>();
        }
        __syncthreads();  // this chunk has landed, for every thread's copies
        if (pc > pos0 + row0 + 15) continue;  // none of this warp's rows sees this chunk (the barriers are at the loop's top)
        const uint32_t k_lane = k_lane0 + (it & 1) * kPfStage, v_lane = v_lane0 + (it & 1) * kPfStage;
        float s[kPfNJ][4];
#pragma unroll
        for (int j = 0; j < kPfNJ; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
        for (int kp = 0; kp < 4; ++kp) {  // 32 dimensions at a time
            uint32_t ah0[4], al0[4], ah1[4], al1[4];
            ptx::ldmatrix_x4(ah0, q_hi + kp * 64);
            ptx::ldmatrix_x4(al0, q_lo + kp * 64);
            ptx::ldmatrix_x4(ah1, q_hi + kp * 64 + 32);
            ptx::ldmatrix_x4(al1, q_lo + kp * 64 + 32);
#pragma unroll
            for (int j = 0; j < kPfNJ; ++j) {
                uint32_t b[4];
                ptx::ldmatrix_x4(b, k_lane + j * 8 * kPfRow + kp * 64);
                ptx::mma_bf16(s[j], ah0, b[0], b[1]);
                ptx::mma_bf16(s[j], al0, b[0], b[1]);
                ptx::mma_bf16(s[j], ah1, b[2], b[3]);
                ptx::mma_bf16(s[j], al1, b[2], b[3]);
            }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < kPfNJ; ++j) {
            const int key = pc + 8 * j + 2 * t;
            if (key > lim0) s[j][0] = -INFINITY;
            if (key + 1 > lim0) s[j][1] = -INFINITY;
            if (key > lim1) s[j][2] = -INFINITY;
            if (key + 1 > lim1) s[j][3] = -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
            mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        // key 0 is visible to every row and lies in the first chunk, so the maxima are finite from there on
        const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
        const float corr0 = __expf(m0 - nm0), corr1 = __expf(m1 - nm1);
        m0 = nm0;
        m1 = nm1;
        float ps0 = 0.0f, ps1 = 0.0f;
#pragma unroll
        for (int j = 0; j < kPfNJ; ++j) {
            s[j][0] = __expf(s[j][0] - nm0);
            s[j][1] = __expf(s[j][1] - nm0);
            s[j][2] = __expf(s[j][2] - nm1);
            s[j][3] = __expf(s[j][3] - nm1);
            ps0 += s[j][0] + s[j][1];
            ps1 += s[j][2] + s[j][3];
        }
        l0 = l0 * corr0 + ps0;  // this thread's share of the row sums; the four lanes of a row meet at the end
        l1 = l1 * corr1 + ps1;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            o[j][0] *= corr0; o[j][1] *= corr0;
            o[j][2] *= corr1; o[j][3] *= corr1;
        }
#pragma unroll
        for (int kk = 0; kk < kPfKeys / 16; ++kk) {  // 16 keys at a time
            if (pc + 16 * kk > pos0 + row0 + 15) break;  // the rest of the chunk is masked for the whole tile
            uint32_t ph[4], pl[4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {  // score tiles 2kk and 2kk+1 are the two key halves of this step
                const float *sv = s[2 * kk + h];
                const float h0 = bf16_round(sv[0]), h1 = bf16_round(sv[1]), h2 = bf16_round(sv[2]), h3 = bf16_round(sv[3]);
                ph[2 * h] = pack_bf16(h0, h1);
                ph[2 * h + 1] = pack_bf16(h2, h3);
                pl[2 * h] = pack_bf16(sv[0] - h0, sv[1] - h1);
                pl[2 * h + 1] = pack_bf16(sv[2] - h2, sv[3] - h3);
            }
#pragma unroll
            for (int jp = 0; jp < 8; ++jp) {  // 16 dimensions at a time
                uint32_t b[4];
                ptx::ldmatrix_x4_trans(b, v_lane + kk * 16 * kPfRow + jp * 32);
                ptx::mma_bf16(o[2 * jp], ph, b[0], b[1]);
                ptx::mma_bf16(o[2 * jp], pl, b[0], b[1]);
                ptx::mma_bf16(o[2 * jp + 1], ph, b[2], b[3]);
                ptx::mma_bf16(o[2 * jp + 1], pl, b[2], b[3]);
            }
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
    const int r0 = row0 + g, r1 = r0 + 8;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        if (r0 < n) *reinterpret_cast<float2 *>(out + (static_cast<size_t>(r0) * nh + head) * kHd + 8 * j + 2 * t) = make_float2(o[j][0] * inv0, o[j][1] * inv0);
        if (r1 < n) *reinterpret_cast<float2 *>(out + (static_cast<size_t>(r1) * nh + head) * kHd + 8 * j + 2 * t) = make_float2(o[j][2] * inv1, o[j][3] * inv1);
    }
}

// Decode attention for batches, on the tensor cores. The staged kernel above reads every staged K/V
// row from shared memory once per query head of the group (8 x amplification at eight query heads per
// KV head) and is bound by shared-memory bandwidth near 60 % of the HBM rate; here the query heads
// that share a KV head are the rows of ONE mma.sync tile (16 rows, the group's heads first, the rest
// zero), so a staged row is read once whatever the group size. A block takes one slice of the key
// range of one (sequence, KV head); keys go through shared memory in chunks of 64 with two stages of
// asynchronous copies, as in the prompt kernel, whose arithmetic this is (scores and output in the
// accumulator layout of m16n8k16, queries and probabilities as two bf16 terms each); the four warps
// of a block take 16 keys of a chunk each, keep their own running softmax, and meet once at the end.
// RoPE on q and on the new k, and the append of the new K/V row, are done here as in
// attn_fused_kernel. Output: the slice's unnormalised sum, maximum and weight per head in `part`
// (attn_combine_kernel merges the slices), or the finished rows in `out` when there is one slice.
constexpr int kDmWarps = 4;
constexpr int kDmStage = 2 * kPfKeys * kPfRow;              // one staged chunk: 64 keys, then 64 values
constexpr int kDmQ = 2 * 8 * kPfRow;                        // the group's queries: hi and lo, 8 rows each (a group has at most 8 heads)
constexpr int kDmSmem = 2 * kDmStage + kDmQ;
constexpr int kDmMergeRow = kHd + 4;                        // floats per (warp, head) in the merge area (aliases stage 0)
static_assert(kDmWarps * 8 * kDmMergeRow * 4 <= kDmStage, "the merge area must fit in a stage");

__global__ void __launch_bounds__(kDmWarps * 32) attn_decode_mma_kernel(const float *__restrict__ q_raw, const float *__restrict__ k_new,
                                                                       const float *__restrict__ v_new, const float *__restrict__ cos_t,
                                                                       const float *__restrict__ sin_t, const int *__restrict__ pos_dev, int pos_stride,
                                                                       int nh, int kvh, int cap, float scaling, int splits, uint16_t *__restrict__ kc,
                                                                       uint16_t *__restrict__ vc, float *__restrict__ part,
                                                                       float *__restrict__ out /* [b][nh*hd] */, int *err_word) {
    ptx::pdl_trigger();
    ptx::pdl_wait();
    extern __shared__ __align__(16) uint8_t dm_smem[];
    uint8_t *s_kv = dm_smem, *s_q = dm_smem + 2 * kDmStage;
    const int sp = blockIdx.x, kh = blockIdx.y, b = blockIdx.z;
    const int group = nh / kvh, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int pos = pos_dev[b * pos_stride], total = pos + 1;  // keys 0..pos
    if (!pos_in_cache(pos, pos, cap, err_word)) return;
    // slices are whole chunks, so that only the last one is ragged
    const int per = ((total + splits - 1) / splits + kPfKeys - 1) / kPfKeys * kPfKeys;
    const int p0 = min(total, sp * per), p1 = min(total, p0 + per);
    const float *cs = cos_t + static_cast<size_t>(pos) * kHd, *sn = sin_t + static_cast<size_t>(pos) * kHd;
    uint16_t *kb = kc + (static_cast<size_t>(b) * kvh + kh) * cap * kHd;
    uint16_t *vb = vc + (static_cast<size_t>(b) * kvh + kh) * cap * kHd;
    // the new position's row: RoPE on k (model.rs:298-302), both rows rounded to bf16 and stored in the
    // cache by the one block whose slice holds the position, before that slice is staged
    if (pos >= p0 && pos < p1 && tid < kHd) {
        const float *kn = k_new + (static_cast<size_t>(b) * kvh + kh) * kHd, *vn = v_new + (static_cast<size_t>(b) * kvh + kh) * kHd;
        const int d = tid;
        // x * cos + rotate_half(x) * sin as two rounded products and a rounded sum: the reference's tensor
        // ops do not fuse a multiply with an add (model.rs:298-302)
        const float rot = d < kHd / 2 ? -kn[d + kHd / 2] : kn[d - kHd / 2];
        const float kr = __fadd_rn(__fmul_rn(kn[d], cs[d]), __fmul_rn(rot, sn[d]));
        kb[static_cast<size_t>(pos) * kHd + d] = f32_to_bf16(kr);
        vb[static_cast<size_t>(pos) * kHd + d] = f32_to_bf16(vn[d]);
        __threadfence();  // the asynchronous copies below read the row back through L2
    }
    // the group's queries: RoPE, the 1/sqrt(d) of the scores, split into two bf16 terms; rows past the group are zero
    for (int r = warp; r < 8; r += kDmWarps) {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < group) {
            const float *qh = q_raw + (static_cast<size_t>(b) * nh + kh * group + r) * kHd;
            const int d = lane * 4, dp = (d + kHd / 2) & (kHd - 1);
            const float4 a = *reinterpret_cast<const float4 *>(qh + d), o2 = *reinterpret_cast<const float4 *>(qh + dp);
            const float4 c4 = *reinterpret_cast<const float4 *>(cs + d), s4 = *reinterpret_cast<const float4 *>(sn + d);
            const float sg = d < kHd / 2 ? -1.0f : 1.0f;  // rotate_half = cat(-x2, x1)
            x = make_float4(__fadd_rn(__fmul_rn(a.x, c4.x), __fmul_rn(sg * o2.x, s4.x)) * scaling, __fadd_rn(__fmul_rn(a.y, c4.y), __fmul_rn(sg * o2.y, s4.y)) * scaling,
                            __fadd_rn(__fmul_rn(a.z, c4.z), __fmul_rn(sg * o2.z, s4.z)) * scaling, __fadd_rn(__fmul_rn(a.w, c4.w), __fmul_rn(sg * o2.w, s4.w)) * scaling);
        }
        const float hx = bf16_round(x.x), hy = bf16_round(x.y), hz = bf16_round(x.z), hw = bf16_round(x.w);
        *reinterpret_cast<uint2 *>(s_q + r * kPfRow + lane * 8) = make_uint2(pack_bf16(hx, hy), pack_bf16(hz, hw));
        *reinterpret_cast<uint2 *>(s_q + (8 + r) * kPfRow + lane * 8) = make_uint2(pack_bf16(x.x - hx, x.y - hy), pack_bf16(x.z - hz, x.w - hw));
    }
    __syncthreads();  // the new row is in the cache and the queries are in shared memory
    // Only rows 0..7 of the 16-row tile exist: the lanes that would address rows 8..15 read rows 0..7
    // again and the fragments of rows g + 8 (registers 1 and 3) are cleared after the load.
    const uint32_t q_hi = ptx::smem_u32(s_q) + (lane & 7) * kPfRow + (lane >> 4) * 16;
    const uint32_t q_lo = q_hi + 8 * kPfRow;
    const uint32_t k_lane0 = ptx::smem_u32(s_kv) + (warp * 16 + (lane & 7)) * kPfRow + (lane >> 3) * 16;
    const uint32_t v_lane0 = ptx::smem_u32(s_kv) + kPfKeys * kPfRow + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * kPfRow + (lane >> 4) * 16;
    auto stage = [&](int buf, int pc) {
        const int cnt = min(kPfKeys, p1 - pc);
        uint8_t *dk = s_kv + buf * kDmStage, *dv = dk + kPfKeys * kPfRow;
        for (int i = tid; i < kPfKeys * 16; i += kDmWarps * 32) {
            const int r = i >> 4, sg = i & 15;
            if (r < cnt) {
                ptx::cp_async_16(ptx::smem_u32(dk + r * kPfRow + sg * 16), kb + static_cast<size_t>(pc + r) * kHd + sg * 8);
                ptx::cp_async_16(ptx::smem_u32(dv + r * kPfRow + sg * 16), vb + static_cast<size_t>(pc + r) * kHd + sg * 8);
            } else {  // rows past the slice: their weights are zero, but their bits must be numbers
                *reinterpret_cast<uint4 *>(dk + r * kPfRow + sg * 16) = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4 *>(dv + r * kPfRow + sg * 16) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        ptx::cp_async_commit();
    };
    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    float m0 = -INFINITY, l0 = 0.0f;  // rows g + 8 of the tile are never real heads (group <= 8)
    if (p0 < p1) stage(0, p0);
    for (int pc = p0, it = 0; pc < p1; pc += kPfKeys, ++it) {
        if (it) __syncthreads();  // everyone is done with the stage that the next chunk overwrites
        if (pc + kPfKeys < p1) {
            stage((it & 1) ^ 1, pc + kPfKeys);
            ptx::cp_async_wait<1>();
        } else {
            ptx::cp_async_wait<0>();
        }
        __syncthreads();  // this chunk has landed, for every thread's copies
        const int key0 = pc + warp * 16;  // this warp's 16 keys of the chunk
        if (key0 >= p1) continue;
        const uint32_t k_lane = k_lane0 + (it & 1) * kDmStage, v_lane = v_lane0 + (it & 1) * kDmStage;
        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
        for (int kp = 0; kp < 4; ++kp) {  // 32 dimensions at a time
            uint32_t ah0[4], al0[4], ah1[4], al1[4];
            ptx::ldmatrix_x4(ah0, q_hi + kp * 64);
            ptx::ldmatrix_x4(al0, q_lo + kp * 64);
            ptx::ldmatrix_x4(ah1, q_hi + kp * 64 + 32);
            ptx::ldmatrix_x4(al1, q_lo + kp * 64 + 32);
            ah0[1] = ah0[3] = al0[1] = al0[3] = ah1[1] = ah1[3] = al1[1] = al1[3] = 0u;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t bb[4];
                ptx::ldmatrix_x4(bb, k_lane + j * 8 * kPfRow + kp * 64);
                ptx::mma_bf16(s[j], ah0, bb[0], bb[1]);
                ptx::mma_bf16(s[j], al0, bb[0], bb[1]);
                ptx::mma_bf16(s[j], ah1, bb[2], bb[3]);
                ptx::mma_bf16(s[j], al1, bb[2], bb[3]);
            }
        }
        float mx0 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int key = key0 + 8 * j + 2 * t;
            if (key >= p1) s[j][0] = -INFINITY;
            if (key + 1 >= p1) s[j][1] = -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        const float nm0 = fmaxf(m0, mx0);           // key0 < p1: at least one key of the tile is real, so nm0 is finite
        const float corr0 = __expf(m0 - nm0);
        m0 = nm0;
        float ps0 = 0.0f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            s[j][0] = __expf(s[j][0] - nm0);
            s[j][1] = __expf(s[j][1] - nm0);
            s[j][2] = 0.0f;                         // rows g + 8: no head there
            s[j][3] = 0.0f;
            ps0 += s[j][0] + s[j][1];
        }
        l0 = l0 * corr0 + ps0;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            o[j][0] *= corr0;
            o[j][1] *= corr0;
        }
        uint32_t ph[4], pl[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {  // the two score tiles are the two key halves of this 16-key step
            const float h0 = bf16_round(s[h][0]), h1 = bf16_round(s[h][1]);
            ph[2 * h] = pack_bf16(h0, h1);
            ph[2 * h + 1] = 0u;
            pl[2 * h] = pack_bf16(s[h][0] - h0, s[h][1] - h1);
            pl[2 * h + 1] = 0u;
        }
#pragma unroll
        for (int jp = 0; jp < 8; ++jp) {  // 16 dimensions at a time
            uint32_t bb[4];
            ptx::ldmatrix_x4_trans(bb, v_lane + jp * 32);
            ptx::mma_bf16(o[2 * jp], ph, bb[0], bb[1]);
            ptx::mma_bf16(o[2 * jp], pl, bb[0], bb[1]);
            ptx::mma_bf16(o[2 * jp + 1], ph, bb[2], bb[3]);
            ptx::mma_bf16(o[2 * jp + 1], pl, bb[2], bb[3]);
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    // the four warps' shares of the slice meet in shared memory (the stages are free now)
    __syncthreads();
    float *s_m = reinterpret_cast<float *>(s_kv);
    {
        float *row = s_m + (warp * 8 + g) * kDmMergeRow;
#pragma unroll
        for (int j = 0; j < 16; ++j) *reinterpret_cast<float2 *>(row + 8 * j + 2 * t) = make_float2(o[j][0], o[j][1]);
        if (t == 0) {
            row[kHd] = m0;
            row[kHd + 1] = l0;
        }
    }
    __syncthreads();
    const int head_r = tid >> 4, d0 = (tid & 15) * 8;  // 16 threads per head, 8 dimensions each
    if (head_r < group) {
        float gm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kDmWarps; ++w) gm = fmaxf(gm, s_m[(w * 8 + head_r) * kDmMergeRow + kHd]);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, sum = 0.0f;
#pragma unroll
        for (int w = 0; w < kDmWarps; ++w) {
            const float *row = s_m + (w * 8 + head_r) * kDmMergeRow;
            const float wm = row[kHd];
            const float wt = wm == -INFINITY ? 0.0f : __expf(wm - gm);  // a warp without keys weighs nothing
            sum += wt * row[kHd + 1];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += wt * row[d0 + e];
        }
        const int head = kh * group + head_r;
        if (splits == 1) {
            const float inv = 1.0f / sum;
            float *dst = out + (static_cast<size_t>(b) * nh + head) * kHd + d0;
            *reinterpret_cast<float4 *>(dst) = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
            *reinterpret_cast<float4 *>(dst + 4) = make_float4(acc[4] * inv, acc[5] * inv, acc[6] * inv, acc[7] * inv);
        } else {
            float *dst = part + ((static_cast<size_t>(b) * nh + head) * splits + sp) * kPartStride;
            *reinterpret_cast<float4 *>(dst + d0) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            *reinterpret_cast<float4 *>(dst + d0 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            if ((tid & 15) == 0) {
                dst[kHd] = gm;      // -inf for an empty slice: the merge gives it no weight
                dst[kHd + 1] = sum;
            }
        }
    }
}

__global__ void __launch_bounds__(256) attn_combine_kernel(const float *__restrict__ part, int splits,
                                                          float *__restrict__ out /* [b][nh*hd] */) {
    ptx::pdl_trigger();  // the next kernel of the step may be scheduled now
    ptx::pdl_wait();     // everything this kernel reads or overwrites is settled from here on

    extern __shared__ float s_w[];  // [splits] weights exp(m_s - m)
    __shared__ float s_red[8];
    __shared__ float s_half[kHd];
    const size_t bh = blockIdx.x;  // b * nh + head
    const float *p = part + bh * splits * kPartStride;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float mx = -INFINITY;
    for (int s = tid; s < splits; s += 256) mx = fmaxf(mx, p[s * kPartStride + kHd]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
    mx = s_red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, s_red[w]);
    float sum = 0.0f;
    for (int s = tid; s < splits; s += 256) {
        const float m = p[s * kPartStride + kHd];
        const float w = m == -INFINITY ? 0.0f : __expf(m - mx);  // empty slices weigh nothing
        s_w[s] = w;
        sum += w * p[s * kPartStride + kHd + 1];
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncthreads();
    if (lane == 0) s_red[warp] = sum;
    __syncthreads();
    sum = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) sum += s_red[w];
    // two halves of the slices side by side, 128 dimensions each, many loads in flight
    const int d = tid & (kHd - 1), half = tid >> 7;
    const int s0 = half ? (splits + 1) / 2 : 0, s1 = half ? splits : (splits + 1) / 2;
    float acc = 0.0f;
#pragma unroll 16
    for (int s = s0; s < s1; ++s) acc += s_w[s] * p[s * kPartStride + d];
    if (half) s_half[d] = acc;
    __syncthreads();
    if (!half) out[bh * kHd + d] = (acc + s_half[d]) / sum;
}

// x += y, then out = rms_norm(x): the residual add of model.rs:359,365 fused with the norm that
// follows it (model.rs:361 and the next layer's :332 / the final :369).
__global__ void __launch_bounds__(256) add_rms_norm_kernel(float *x, const float *__restrict__ y, const float *__restrict__ w, int n,
                                                          float eps, float *__restrict__ out) {
    ptx::pdl_trigger();  // the next kernel of the step may be scheduled now
    ptx::pdl_wait();     // everything this kernel reads or overwrites is settled from here on

    __shared__ float s_red[8];
    float *xr = x + static_cast<size_t>(blockIdx.x) * n;
    const float *yr = y + static_cast<size_t>(blockIdx.x) * n;
    float *orow = out + static_cast<size_t>(blockIdx.x) * n;
    const int n4 = n >> 2;  // callers guarantee n % 4 == 0, n <= 8192, 16-byte aligned rows
    float4 v[8];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) {
            const float4 a = reinterpret_cast<const float4 *>(xr)[i], c = reinterpret_cast<const float4 *>(yr)[i];
            v[j] = make_float4(a.x + c.x, a.y + c.y, a.z + c.z, a.w + c.w);
            reinterpret_cast<float4 *>(xr)[i] = v[j];
        } else {
            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
    }
    const float r = 1.0f / sqrtf(block_sum(ss, s_red) / static_cast<float>(n) + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) {
            const float4 g = __ldg(reinterpret_cast<const float4 *>(w) + i);
            reinterpret_cast<float4 *>(orow)[i] = make_float4(v[j].x * r * g.x, v[j].y * r * g.y, v[j].z * r * g.z, v[j].w * r * g.w);
        }
    }
}

// out = rms_norm(relu(g)^2 * u) (model.rs:363-364 in one pass).
__global__ void __launch_bounds__(256) relu2_mul_rms_norm_kernel(const float *__restrict__ g, const float *__restrict__ u,
                                                                const float *__restrict__ w, int n, float eps, float *__restrict__ out) {
    ptx::pdl_trigger();  // the next kernel of the step may be scheduled now
    ptx::pdl_wait();     // everything this kernel reads or overwrites is settled from here on

    __shared__ float s_red[8];
    const float *gr = g + static_cast<size_t>(blockIdx.x) * n, *ur = u + static_cast<size_t>(blockIdx.x) * n;
    float *orow = out + static_cast<size_t>(blockIdx.x) * n;
    const int n4 = n >> 2;
    float4 v[8];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) {
            const float4 a = reinterpret_cast<const float4 *>(gr)[i], c = reinterpret_cast<const float4 *>(ur)[i];
            const float r0 = fmaxf(a.x, 0.f), r1 = fmaxf(a.y, 0.f), r2 = fmaxf(a.z, 0.f), r3 = fmaxf(a.w, 0.f);
            v[j] = make_float4(r0 * r0 * c.x, r1 * r1 * c.y, r2 * r2 * c.z, r3 * r3 * c.w);
        } else {
            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
    }
    const float r = 1.0f / sqrtf(block_sum(ss, s_red) / static_cast<float>(n) + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) {
            const float4 gw = __ldg(reinterpret_cast<const float4 *>(w) + i);
            reinterpret_cast<float4 *>(orow)[i] = make_float4(v[j].x * r * gw.x, v[j].y * r * gw.y, v[j].z * r * gw.z, v[j].w * r * gw.w);
        }
    }
}

// A norm whose result feeds a projection directly: the normalised row is quantised where it stands
// (quant.rs:100-118: scale = 127 / max(amax, 1e-5), round half to even, clamp, sum) instead of going
// to memory as f32 and through the quantise kernel. PRE selects what is normalised: x (LBK_PRE_RMS),
// x + y with the sum written back to x (LBK_PRE_ADD_RMS), relu(x)^2 * y (LBK_PRE_RELU2_MUL_RMS). The
// f32 values that get quantised are computed exactly as the norm kernels above compute them, so
// the int8 rows equal those of norm kernel + quantise kernel bit for bit.
template <int PRE>
__global__ void __launch_bounds__(256) norm_quant_kernel(float *x, const float *__restrict__ y, const float *__restrict__ w, int n, int kp,
                                                        float eps, int8_t *__restrict__ q, float *__restrict__ scale, int32_t *__restrict__ sum) {
    ptx::pdl_trigger();
    ptx::pdl_wait();
    __shared__ float s_red[8];
    __shared__ int s_isum[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float *xr = x + static_cast<size_t>(blockIdx.x) * n;
    const float *yr = y ? y + static_cast<size_t>(blockIdx.x) * n : nullptr;
    const int n4 = n >> 2;  // callers guarantee n % 4 == 0, n <= 8192, 16-byte aligned rows
    float4 v[8];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = tid + j * 256;
        if (i < n4) {
            const float4 a = reinterpret_cast<const float4 *>(xr)[i];
            if (PRE == LBK_PRE_RMS) {
                v[j] = a;
            } else if (PRE == LBK_PRE_ADD_RMS) {
                const float4 c = reinterpret_cast<const float4 *>(yr)[i];
                v[j] = make_float4(a.x + c.x, a.y + c.y, a.z + c.z, a.w + c.w);
                reinterpret_cast<float4 *>(xr)[i] = v[j];
            } else {
                const float4 c = reinterpret_cast<const float4 *>(yr)[i];
                const float r0 = fmaxf(a.x, 0.f), r1 = fmaxf(a.y, 0.f), r2 = fmaxf(a.z, 0.f), r3 = fmaxf(a.w, 0.f);
                v[j] = make_float4(r0 * r0 * c.x, r1 * r1 * c.y, r2 * r2 * c.z, r3 * r3 * c.w);
            }
        } else {
            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
    }
    const float r = 1.0f / sqrtf(block_sum(ss, s_red) / static_cast<float>(n) + eps);
    float am = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = tid + j * 256;
        if (i < n4) {
            const float4 gw = __ldg(reinterpret_cast<const float4 *>(w) + i);
            v[j] = make_float4(v[j].x * r * gw.x, v[j].y * r * gw.y, v[j].z * r * gw.z, v[j].w * r * gw.w);
            am = fmaxf(am, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));  // fmaxf drops a NaN, as f32::max does
        }
    }
    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    __syncthreads();  // block_sum's readers are done with s_red
    if (lane == 0) s_red[warp] = am;
    __syncthreads();
    am = s_red[0];
#pragma unroll
    for (int wv = 1; wv < 8; ++wv) am = fmaxf(am, s_red[wv]);
    const float sc = __fdiv_rn(127.0f, fmaxf(am, 1e-5f));
    int8_t *qr = q + static_cast<size_t>(blockIdx.x) * kp;
    int acc = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = (tid + j * 256) * 4;
        if (i < kp) {  // columns from n to kp hold zeros
            int qv[4];
            const float f[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int t = __float2int_rn(__fmul_rn(f[e], sc));  // NaN -> 0 like `NaN as i8`
                qv[e] = max(-128, min(127, t));
                acc += qv[e];
            }
            *reinterpret_cast<uint32_t *>(qr + i) = (qv[0] & 255) | ((qv[1] & 255) << 8) | ((qv[2] & 255) << 16) | (static_cast<uint32_t>(qv[3] & 255) << 24);
        }
    }
    for (int i = (tid + 8 * 256) * 4; i < kp; i += 256 * 4) *reinterpret_cast<uint32_t *>(qr + i) = 0u;
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) s_isum[warp] = acc;
    __syncthreads();
    if (tid == 0) {
        int t = 0;
#pragma unroll
        for (int wv = 0; wv < 8; ++wv) t += s_isum[wv];
        scale[blockIdx.x] = sc;
        sum[blockIdx.x] = t;
    }
}

__global__ void relu2_mul_kernel(const float *__restrict__ g, const float *__restrict__ u, size_t n, float *__restrict__ out) {
    ptx::pdl_trigger();  // the next kernel of the step may be scheduled now
    ptx::pdl_wait();     // everything this kernel reads or overwrites is settled from here on

    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float r = fmaxf(g[i], 0.0f);
        out[i] = r * r * u[i];
    }
}

__global__ void add_inplace_kernel(float *__restrict__ x, const float *__restrict__ y, size_t n) {
    ptx::pdl_trigger();  // the next kernel of the step may be scheduled now
    ptx::pdl_wait();     // everything this kernel reads or overwrites is settled from here on

    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x)
        x[i] += y[i];
}

// First index of the maximum (strict >, sample.rs:17-25), two stages: kArgParts blocks per row
// reduce their slice to (value, index), then one warp merges them. Order: value desc, index asc.
constexpr int kArgParts = 32;
constexpr size_t kSmallScratchRows = 256;
static_assert(kSmallScratchRows * kArgParts * 8 <= kSmallScratchBytes, "context small scratch too small");
__device__ __forceinline__ bool arg_better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

__global__ void __launch_bounds__(256) argmax_part_kernel(const float *__restrict__ logits, int n, float *__restrict__ pv,
                                                         int *__restrict__ pi) {
    ptx::pdl_trigger();  // the next kernel of the step may be scheduled now
    ptx::pdl_wait();     // everything this kernel reads or overwrites is settled from here on

    __shared__ float s_v[8];
    __shared__ int s_i[8];
    const float *row = logits + static_cast<size_t>(blockIdx.y) * n;
    const int per = (n + kArgParts - 1) / kArgParts;
    const int i0 = blockIdx.x * per, i1 = min(n, i0 + per);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = i0 + threadIdx.x; i < i1; i += 256) {  // ascending i: strict > keeps the first maximum
        const float v = row[i];
        if (v > bv) {
            bv = v;
            bi = i;
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (arg_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_v[warp] = bv; s_i[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w2 = 1; w2 < 8; ++w2)
            if (arg_better(s_v[w2], s_i[w2], bv, bi)) { bv = s_v[w2]; bi = s_i[w2]; }
        pv[blockIdx.y * kArgParts + blockIdx.x] = bv;
        pi[blockIdx.y * kArgParts + blockIdx.x] = bi;
    }
}

__global__ void __launch_bounds__(32) argmax_merge_kernel(const float *__restrict__ logits, int n, const float *__restrict__ pv,
                                                         const int *__restrict__ pi, int *__restrict__ out) {
    ptx::pdl_trigger();  // the next kernel of the step may be scheduled now
    ptx::pdl_wait();     // everything this kernel reads or overwrites is settled from here on

    const int lane = threadIdx.x;
    float bv = lane < kArgParts ? pv[blockIdx.x * kArgParts + lane] : -INFINITY;
    int bi = lane < kArgParts ? pi[blockIdx.x * kArgParts + lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (arg_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    // the reference starts from index 0 and only moves on a strict >: a NaN in front, or a row
    // with nothing above -inf, stays at 0
    const float first = logits[static_cast<size_t>(blockIdx.x) * n];
    if (lane == 0) out[blockIdx.x] = (bi == 0x7fffffff || first != first) ? 0 : bi;
}

// pos[i] += 1 for the sequences that took part in the step (all of them without a mask)
// Saturates far below overflow: a position that was already refused by the kernels above (code 7)
// must stay refused however often the step is replayed, never wrap round to a valid one.
__global__ void advance_pos_kernel(int *pos, const int *__restrict__ active, int n) {
    ptx::pdl_trigger();  // the next kernel of the step may be scheduled now
    ptx::pdl_wait();     // everything this kernel reads or overwrites is settled from here on
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && (!active || active[i]) && pos[i] < (1 << 30)) pos[i] += 1;
}

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
    LBK_CUDA(launch_chained(embed_kernel, dim3(static_cast<unsigned>(b)), dim3(256), 0, st, table_dev, tokens_dev, static_cast<int>(hidden), out_dev));
    LBK_DEC_POST();
}

int lbk_rms_norm(lbk_ctx *c, const float *x_dev, const float *w_dev, size_t rows, size_t n, float eps, float *out_dev, void *stream) {
    LBK_DEC_PRE("lbk_rms_norm");
    if (rows == 0) return LBK_OK;
    if (!x_dev || !w_dev || !out_dev || n == 0) return fail(LBK_ERR_INVALID, "lbk_rms_norm: null buffer or empty row");
    LBK_CUDA(launch_chained(rms_norm_kernel, dim3(static_cast<unsigned>(rows)), dim3(256), 0, st, x_dev, w_dev, static_cast<int>(n), eps, out_dev));
    LBK_DEC_POST();
}

static int rope_kv_append_impl(lbk_ctx *c, float *q_dev, const float *k_dev, const float *v_dev, const float *cos_dev, const float *sin_dev,
                               const int32_t *pos_dev, int pos_stride, size_t b, size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap,
                               uint16_t *kcache_dev, uint16_t *vcache_dev, void *stream) {
    LBK_DEC_PRE("lbk_rope_kv_append");
    if (b == 0) return LBK_OK;
    if (!q_dev || !k_dev || !v_dev || !cos_dev || !sin_dev || !pos_dev || !kcache_dev || !vcache_dev)
        return fail(LBK_ERR_INVALID, "lbk_rope_kv_append: null buffer");
    if (head_dim & 1) return fail(LBK_ERR_SHAPE, "head_dim must be even");
    dim3 grid(static_cast<unsigned>(n_heads + kv_heads), static_cast<unsigned>(b));
    LBK_CUDA(launch_chained(rope_append_kernel, dim3(grid), dim3(64), 0, st, q_dev, k_dev, v_dev, cos_dev, sin_dev, pos_dev, pos_stride, static_cast<int>(n_heads),
                                            static_cast<int>(kv_heads), static_cast<int>(head_dim), static_cast<int>(cap),
                                            kcache_dev, vcache_dev, ctx->err_word));
    LBK_DEC_POST();
}

int lbk_rope_kv_append(lbk_ctx *c, float *q_dev, const float *k_dev, const float *v_dev, const float *cos_dev, const float *sin_dev,
                       const int32_t *pos_dev, size_t b, size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap,
                       uint16_t *kcache_dev, uint16_t *vcache_dev, void *stream) {
    return rope_kv_append_impl(c, q_dev, k_dev, v_dev, cos_dev, sin_dev, pos_dev, 0, b, n_heads, kv_heads, head_dim, cap, kcache_dev, vcache_dev, stream);
}

int lbk_rope_kv_append_seq(lbk_ctx *c, float *q_dev, const float *k_dev, const float *v_dev, const float *cos_dev, const float *sin_dev,
                           const int32_t *pos_dev, size_t b, size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap,
                           uint16_t *kcache_dev, uint16_t *vcache_dev, void *stream) {
    return rope_kv_append_impl(c, q_dev, k_dev, v_dev, cos_dev, sin_dev, pos_dev, 1, b, n_heads, kv_heads, head_dim, cap, kcache_dev, vcache_dev, stream);
}

static int attn_decode_impl(lbk_ctx *c, const float *q_dev, const uint16_t *kcache_dev, const uint16_t *vcache_dev, const int32_t *pos_dev,
                            int pos_stride, size_t b, size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap, size_t splits,
                            float *scratch_dev, float *out_dev, void *stream) {
    LBK_DEC_PRE("lbk_attn_decode");
    if (b == 0) return LBK_OK;
    if (!q_dev || !kcache_dev || !vcache_dev || !pos_dev || !scratch_dev || !out_dev) return fail(LBK_ERR_INVALID, "lbk_attn_decode: null buffer");
    if (head_dim != kHd) return fail(LBK_ERR_UNSUPPORTED, "attention kernel is built for head_dim 128, got %zu", head_dim);
    if (kv_heads == 0 || n_heads % kv_heads || n_heads / kv_heads > 8) return fail(LBK_ERR_UNSUPPORTED, "query group size must be 1..8");
    if (splits == 0) return fail(LBK_ERR_INVALID, "splits must be positive");
    if (splits > 4096) return fail(LBK_ERR_UNSUPPORTED, "at most 4096 splits");
    dim3 grid(static_cast<unsigned>(splits), static_cast<unsigned>(kv_heads), static_cast<unsigned>(b));
    const bool staged = n_heads / kv_heads >= 4;  // several query heads share the rows: fetch them once per block
    LBK_CUDA(launch_chained(staged ? attn_partial_staged_kernel : attn_partial_kernel, dim3(grid), dim3(static_cast<unsigned>(32 * (n_heads / kv_heads))), 0, st, q_dev, kcache_dev, vcache_dev, pos_dev, pos_stride, static_cast<int>(n_heads), static_cast<int>(kv_heads),
                                              static_cast<int>(cap), 1.0f / sqrtf(static_cast<float>(head_dim)), static_cast<int>(splits),
                                              scratch_dev, ctx->err_word));
    LBK_CUDA(cudaGetLastError());
    LBK_CUDA(launch_chained(attn_combine_kernel, dim3(static_cast<unsigned>(b * n_heads)), dim3(256), (splits + 1) * sizeof(float), st, scratch_dev, static_cast<int>(splits), out_dev));
    ctx->launches++;
    LBK_DEC_POST();
}

int lbk_attn_decode(lbk_ctx *c, const float *q_dev, const uint16_t *kcache_dev, const uint16_t *vcache_dev, const int32_t *pos_dev,
                    size_t b, size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap, size_t splits, float *scratch_dev,
                    float *out_dev, void *stream) {
    return attn_decode_impl(c, q_dev, kcache_dev, vcache_dev, pos_dev, 0, b, n_heads, kv_heads, head_dim, cap, splits, scratch_dev, out_dev, stream);
}

int lbk_attn_decode_seq(lbk_ctx *c, const float *q_dev, const uint16_t *kcache_dev, const uint16_t *vcache_dev, const int32_t *pos_dev,
                        size_t b, size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap, size_t splits, float *scratch_dev,
                        float *out_dev, void *stream) {
    return attn_decode_impl(c, q_dev, kcache_dev, vcache_dev, pos_dev, 1, b, n_heads, kv_heads, head_dim, cap, splits, scratch_dev, out_dev, stream);
}

int lbk_rope_kv_append_rows(lbk_ctx *c, float *q_dev, const float *k_dev, const float *v_dev, const float *cos_dev, const float *sin_dev,
                            const int32_t *pos_dev, size_t n, size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap, size_t seq,
                            uint16_t *kcache_dev, uint16_t *vcache_dev, void *stream) {
    LBK_DEC_PRE("lbk_rope_kv_append_rows");
    if (n == 0) return LBK_OK;
    if (!q_dev || !k_dev || !v_dev || !cos_dev || !sin_dev || !pos_dev || !kcache_dev || !vcache_dev)
        return fail(LBK_ERR_INVALID, "lbk_rope_kv_append_rows: null buffer");
    if (head_dim == 0 || (head_dim & 1)) return fail(LBK_ERR_INVALID, "head_dim must be even");
    LBK_CUDA(launch_chained(rope_append_rows_kernel, dim3(static_cast<unsigned>(n)), dim3(256), 0, st, q_dev, k_dev, v_dev, cos_dev, sin_dev, pos_dev, static_cast<int>(n_heads),
                            static_cast<int>(kv_heads), static_cast<int>(head_dim), static_cast<int>(cap), static_cast<int>(seq), kcache_dev,
                            vcache_dev, ctx->err_word));
    LBK_DEC_POST();
}

int lbk_attn_prefill(lbk_ctx *c, const float *q_dev, const uint16_t *kcache_dev, const uint16_t *vcache_dev, const int32_t *pos_dev, size_t n,
                     size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap, size_t seq, float *out_dev, void *stream) {
    LBK_DEC_PRE("lbk_attn_prefill");
    if (n == 0) return LBK_OK;
    if (!q_dev || !kcache_dev || !vcache_dev || !pos_dev || !out_dev) return fail(LBK_ERR_INVALID, "lbk_attn_prefill: null buffer");
    if (head_dim != kHd) return fail(LBK_ERR_UNSUPPORTED, "attention kernel is built for head_dim 128, got %zu", head_dim);
    if (kv_heads == 0 || n_heads % kv_heads || n_heads / kv_heads > 8) return fail(LBK_ERR_UNSUPPORTED, "query group size must be 1..8");
    if (n > 65535) return fail(LBK_ERR_UNSUPPORTED, "at most 65535 rows per call");
    // 64 rows and more: 128-row tiles on tcgen05; fewer: 16-row tiles on mma.sync (a 128-row tile would be mostly padding)
    if (n >= 64) return launch_attn_prompt_tc(ctx, q_dev, kcache_dev, vcache_dev, pos_dev, n, n_heads, kv_heads, cap, seq, out_dev, st);
    const size_t group = n_heads / kv_heads;
    const size_t warps = (group == 1 || group == 2) ? 4 : group;  // one warp per (query head, 16-row tile)
    const size_t rows_per_block = warps / group * 16;
    const size_t smem = 2 * kPfStage + warps * kPfQWarp;
    static bool attr_set = false;  // the same value for every call; setting it twice is harmless
    if (!attr_set) {
        LBK_CUDA(cudaFuncSetAttribute(attn_prompt_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * kPfStage + 8 * kPfQWarp));
        attr_set = true;
    }
    dim3 grid(static_cast<unsigned>(kv_heads), static_cast<unsigned>((n + rows_per_block - 1) / rows_per_block));
    LBK_CUDA(launch_chained(attn_prompt_mma_kernel, grid, dim3(static_cast<unsigned>(32 * warps)), smem, st, q_dev, kcache_dev, vcache_dev, pos_dev,
                            static_cast<int>(n), static_cast<int>(n_heads), static_cast<int>(kv_heads), static_cast<int>(cap), static_cast<int>(seq),
                            1.0f / sqrtf(static_cast<float>(head_dim)), out_dev, ctx->err_word));
    LBK_DEC_POST();
}

int lbk_attn_decode_fused_supported(size_t n_heads, size_t kv_heads, size_t head_dim, size_t splits) {
    return head_dim == kHd && kv_heads != 0 && n_heads % kv_heads == 0 && n_heads / kv_heads >= 4 && n_heads / kv_heads <= 8 && splits >= 1 &&
                   splits <= 256
               ? 1
               : 0;
}

static int attn_decode_fused_impl(lbk_ctx *c, const float *q_dev, const float *k_dev, const float *v_dev, const float *cos_dev,
                                  const float *sin_dev, const int32_t *pos_dev, int pos_stride, size_t b, size_t n_heads, size_t kv_heads,
                                  size_t head_dim, size_t cap, size_t splits, uint16_t *kcache_dev, uint16_t *vcache_dev, float *scratch_dev,
                                  int32_t *counters_dev, float *out_dev, void *stream) {
    LBK_DEC_PRE("lbk_attn_decode_fused");
    if (b == 0) return LBK_OK;
    if (!q_dev || !k_dev || !v_dev || !cos_dev || !sin_dev || !pos_dev || !kcache_dev || !vcache_dev || !scratch_dev || !counters_dev || !out_dev)
        return fail(LBK_ERR_INVALID, "lbk_attn_decode_fused: null buffer");
    if (!lbk_attn_decode_fused_supported(n_heads, kv_heads, head_dim, splits))
        return fail(LBK_ERR_UNSUPPORTED, "lbk_attn_decode_fused: head_dim 128, 4..8 query heads per KV head and at most 256 splits");
    dim3 grid(static_cast<unsigned>(splits), static_cast<unsigned>(kv_heads), static_cast<unsigned>(b));
    // Eight sequences and more: the tensor-core kernel (one pass over the staged rows for all query
    // heads of a group); below that the step is a latency chain and the staged kernel's shape is kept.
    if (b >= 8) {
        // Fewer, longer slices than the caller's count when the batch alone fills the GPU: a block's fixed
        // work (queries, merge, partial results) is then spread over several 64-key chunks and the two
        // stages overlap. About four waves of three blocks per SM; the scratch layout follows the count used.
        const size_t want = (12 * static_cast<size_t>(ctx->sm_count) + b * kv_heads - 1) / (b * kv_heads);
        if (want < splits) splits = want < 1 ? 1 : want;
        grid = dim3(static_cast<unsigned>(splits), static_cast<unsigned>(kv_heads), static_cast<unsigned>(b));
        static bool attr_set = false;  // the same value for every call; setting it twice is harmless
        if (!attr_set) {
            LBK_CUDA(cudaFuncSetAttribute(attn_decode_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDmSmem));
            attr_set = true;
        }
        LBK_CUDA(launch_chained(attn_decode_mma_kernel, grid, dim3(kDmWarps * 32), static_cast<size_t>(kDmSmem), st, q_dev, k_dev, v_dev, cos_dev, sin_dev,
                                pos_dev, pos_stride, static_cast<int>(n_heads), static_cast<int>(kv_heads), static_cast<int>(cap),
                                1.0f / sqrtf(static_cast<float>(head_dim)), static_cast<int>(splits), kcache_dev, vcache_dev, scratch_dev, out_dev,
                                ctx->err_word));
        if (splits > 1) {
            LBK_CUDA(cudaGetLastError());
            LBK_CUDA(launch_chained(attn_combine_kernel, dim3(static_cast<unsigned>(b * n_heads)), dim3(256), (splits + 1) * sizeof(float), st,
                                    scratch_dev, static_cast<int>(splits), out_dev));
            ctx->launches++;
        }
        LBK_DEC_POST();
    }
    // Merging inside the kernel (by the last block of a KV head) saves a launch but serialises the
    // merge of a whole KV head in one block; measured slower than the separate combine kernel
    // (1.60 ms against 1.49 ms per batch-1 step), so it is used only when there is a single slice.
    if (splits == 1) {
        LBK_CUDA(launch_chained(attn_fused_kernel<true>, grid, dim3(static_cast<unsigned>(32 * (n_heads / kv_heads))), 0, st, q_dev, k_dev, v_dev,
                                cos_dev, sin_dev, pos_dev, pos_stride, static_cast<int>(n_heads), static_cast<int>(kv_heads), static_cast<int>(cap),
                                1.0f / sqrtf(static_cast<float>(head_dim)), static_cast<int>(splits), kcache_dev, vcache_dev, scratch_dev,
                                counters_dev, out_dev, ctx->err_word));
    } else {
        LBK_CUDA(launch_chained(attn_fused_kernel<false>, grid, dim3(static_cast<unsigned>(32 * (n_heads / kv_heads))), 0, st, q_dev, k_dev, v_dev,
                                cos_dev, sin_dev, pos_dev, pos_stride, static_cast<int>(n_heads), static_cast<int>(kv_heads), static_cast<int>(cap),
                                1.0f / sqrtf(static_cast<float>(head_dim)), static_cast<int>(splits), kcache_dev, vcache_dev, scratch_dev,
                                counters_dev, out_dev, ctx->err_word));
        LBK_CUDA(launch_chained(attn_combine_kernel, dim3(static_cast<unsigned>(b * n_heads)), dim3(256), (splits + 1) * sizeof(float), st,
                                scratch_dev, static_cast<int>(splits), out_dev));
        ctx->launches++;
    }
    LBK_DEC_POST();
}

int lbk_relu2_mul(lbk_ctx *c, const float *g_dev, const float *u_dev, size_t n, float *out_dev, void *stream) {
    LBK_DEC_PRE("lbk_relu2_mul");
    if (n == 0) return LBK_OK;
    if (!g_dev || !u_dev || !out_dev) return fail(LBK_ERR_INVALID, "lbk_relu2_mul: null buffer");
    LBK_CUDA(launch_chained(relu2_mul_kernel, dim3(static_cast<unsigned>((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184)), dim3(256), 0, st, g_dev, u_dev, n, out_dev));
    LBK_DEC_POST();
}

int lbk_add_inplace(lbk_ctx *c, float *x_dev, const float *y_dev, size_t n, void *stream) {
    LBK_DEC_PRE("lbk_add_inplace");
    if (n == 0) return LBK_OK;
    if (!x_dev || !y_dev) return fail(LBK_ERR_INVALID, "lbk_add_inplace: null buffer");
    LBK_CUDA(launch_chained(add_inplace_kernel, dim3(static_cast<unsigned>((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184)), dim3(256), 0, st, x_dev, y_dev, n));
    LBK_DEC_POST();
}

static bool fused_norm_ok(const void *a, const void *b2, const void *w, const void *o, size_t n) {
    return (n & 3) == 0 && n <= 8192 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b2) | reinterpret_cast<uintptr_t>(w) |
                                           reinterpret_cast<uintptr_t>(o)) & 15) == 0;
}

int lbk_add_rms_norm(lbk_ctx *c, float *x_dev, const float *y_dev, const float *w_dev, size_t rows, size_t n, float eps, float *out_dev,
                     void *stream) {
    LBK_DEC_PRE("lbk_add_rms_norm");
    if (rows == 0) return LBK_OK;
    if (!x_dev || !y_dev || !w_dev || !out_dev || n == 0) return fail(LBK_ERR_INVALID, "lbk_add_rms_norm: null buffer or empty row");
    if (!fused_norm_ok(x_dev, y_dev, w_dev, out_dev, n))
        return fail(LBK_ERR_UNSUPPORTED, "lbk_add_rms_norm needs 16-byte aligned rows of a multiple of 4, at most 8192, columns");
    LBK_CUDA(launch_chained(add_rms_norm_kernel, dim3(static_cast<unsigned>(rows)), dim3(256), 0, st, x_dev, y_dev, w_dev, static_cast<int>(n), eps, out_dev));
    LBK_DEC_POST();
}

int lbk_relu2_mul_rms_norm(lbk_ctx *c, const float *g_dev, const float *u_dev, const float *w_dev, size_t rows, size_t n, float eps,
                           float *out_dev, void *stream) {
    LBK_DEC_PRE("lbk_relu2_mul_rms_norm");
    if (rows == 0) return LBK_OK;
    if (!g_dev || !u_dev || !w_dev || !out_dev || n == 0) return fail(LBK_ERR_INVALID, "lbk_relu2_mul_rms_norm: null buffer or empty row");
    if (!fused_norm_ok(g_dev, u_dev, w_dev, out_dev, n))
        return fail(LBK_ERR_UNSUPPORTED, "lbk_relu2_mul_rms_norm needs 16-byte aligned rows of a multiple of 4, at most 8192, columns");
    LBK_CUDA(launch_chained(relu2_mul_rms_norm_kernel, dim3(static_cast<unsigned>(rows)), dim3(256), 0, st, g_dev, u_dev, w_dev, static_cast<int>(n), eps, out_dev));
    LBK_DEC_POST();
}

int lbk_norm_quant_supported(size_t n) { return n != 0 && n % 4 == 0 && n <= 8192 ? 1 : 0; }

int lbk_norm_quant(lbk_ctx *c, int pre, float *x_dev, const float *y_dev, const float *w_dev, size_t rows, size_t n, float eps, int8_t *q_dev,
                   float *scale_dev, int32_t *sum_dev, void *stream) {
    LBK_DEC_PRE("lbk_norm_quant");
    if (rows == 0) return LBK_OK;
    if (!x_dev || !w_dev || !q_dev || !scale_dev || !sum_dev || (pre != LBK_PRE_RMS && !y_dev)) return fail(LBK_ERR_INVALID, "lbk_norm_quant: null buffer");
    if (!lbk_norm_quant_supported(n)) return fail(LBK_ERR_UNSUPPORTED, "lbk_norm_quant: rows of a multiple of 4 and at most 8192 values");
    if ((reinterpret_cast<uintptr_t>(x_dev) | reinterpret_cast<uintptr_t>(y_dev) | reinterpret_cast<uintptr_t>(w_dev) | reinterpret_cast<uintptr_t>(q_dev)) & 15)
        return fail(LBK_ERR_INVALID, "lbk_norm_quant: buffers must be 16-byte aligned");
    const int kp = static_cast<int>((n + 127) / 128 * 128);
    const dim3 grid(static_cast<unsigned>(rows)), block(256);
    if (pre == LBK_PRE_RMS) {
        LBK_CUDA(launch_chained(norm_quant_kernel<LBK_PRE_RMS>, grid, block, 0, st, x_dev, y_dev, w_dev, static_cast<int>(n), kp, eps, q_dev, scale_dev, sum_dev));
    } else if (pre == LBK_PRE_ADD_RMS) {
        LBK_CUDA(launch_chained(norm_quant_kernel<LBK_PRE_ADD_RMS>, grid, block, 0, st, x_dev, y_dev, w_dev, static_cast<int>(n), kp, eps, q_dev, scale_dev, sum_dev));
    } else if (pre == LBK_PRE_RELU2_MUL_RMS) {
        LBK_CUDA(launch_chained(norm_quant_kernel<LBK_PRE_RELU2_MUL_RMS>, grid, block, 0, st, x_dev, y_dev, w_dev, static_cast<int>(n), kp, eps, q_dev, scale_dev, sum_dev));
    } else {
        return fail(LBK_ERR_INVALID, "lbk_norm_quant: unknown transform %d", pre);
    }
    LBK_DEC_POST();
}

int lbk_argmax(lbk_ctx *c, const float *logits_dev, size_t rows, size_t n, int32_t *out_dev, void *stream) {
    LBK_DEC_PRE("lbk_argmax");
    if (rows == 0) return LBK_OK;
    if (!logits_dev || !out_dev || n == 0) return fail(LBK_ERR_INVALID, "lbk_argmax: null buffer or empty row");
    // per-row partial (value, index) pairs live in a small buffer the context owns from start-up
    // (never reallocated, so captured graphs stay valid); larger batches go through in slices
    float *pv = static_cast<float *>(ctx->small_scratch);
    int *pi = reinterpret_cast<int *>(pv + kSmallScratchRows * kArgParts);
    for (size_t r0 = 0; r0 < rows; r0 += kSmallScratchRows) {
        const size_t nr = rows - r0 < kSmallScratchRows ? rows - r0 : kSmallScratchRows;
        LBK_CUDA(launch_chained(argmax_part_kernel, dim3(dim3(kArgParts, static_cast<unsigned>(nr))), dim3(256), 0, st, logits_dev + r0 * n, static_cast<int>(n), pv, pi));
        LBK_CUDA(cudaGetLastError());
        LBK_CUDA(launch_chained(argmax_merge_kernel, dim3(static_cast<unsigned>(nr)), dim3(32), 0, st, logits_dev + r0 * n, static_cast<int>(n), pv, pi, out_dev + r0));
        LBK_CUDA(cudaGetLastError());
        ctx->launches += 2;
    }
    return LBK_OK;
}

int lbk_attn_decode_fused(lbk_ctx *c, const float *q_dev, const float *k_dev, const float *v_dev, const float *cos_dev, const float *sin_dev,
                          const int32_t *pos_dev, size_t b, size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap, size_t splits,
                          uint16_t *kcache_dev, uint16_t *vcache_dev, float *scratch_dev, int32_t *counters_dev, float *out_dev, void *stream) {
    return attn_decode_fused_impl(c, q_dev, k_dev, v_dev, cos_dev, sin_dev, pos_dev, 0, b, n_heads, kv_heads, head_dim, cap, splits, kcache_dev,
                                  vcache_dev, scratch_dev, counters_dev, out_dev, stream);
}

int lbk_attn_decode_fused_seq(lbk_ctx *c, const float *q_dev, const float *k_dev, const float *v_dev, const float *cos_dev, const float *sin_dev,
                              const int32_t *pos_dev, size_t b, size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap, size_t splits,
                              uint16_t *kcache_dev, uint16_t *vcache_dev, float *scratch_dev, int32_t *counters_dev, float *out_dev,
                              void *stream) {
    return attn_decode_fused_impl(c, q_dev, k_dev, v_dev, cos_dev, sin_dev, pos_dev, 1, b, n_heads, kv_heads, head_dim, cap, splits, kcache_dev,
                                  vcache_dev, scratch_dev, counters_dev, out_dev, stream);
}

int lbk_advance_pos(lbk_ctx *c, int32_t *pos_dev, void *stream) {
    LBK_DEC_PRE("lbk_advance_pos");
    if (!pos_dev) return fail(LBK_ERR_INVALID, "lbk_advance_pos: null buffer");
    LBK_CUDA(launch_chained(advance_pos_kernel, dim3(1), dim3(32), 0, st, pos_dev, static_cast<const int *>(nullptr), 1));
    LBK_DEC_POST();
}

int lbk_advance_pos_seq(lbk_ctx *c, int32_t *pos_dev, const int32_t *active_dev, size_t b, void *stream) {
    LBK_DEC_PRE("lbk_advance_pos_seq");
    if (b == 0) return LBK_OK;
    if (!pos_dev) return fail(LBK_ERR_INVALID, "lbk_advance_pos_seq: null buffer");
    LBK_CUDA(launch_chained(advance_pos_kernel, dim3(static_cast<unsigned>((b + 127) / 128)), dim3(128), 0, st, pos_dev, active_dev, static_cast<int>(b)));
    LBK_DEC_POST();
}

}  // extern "C"
