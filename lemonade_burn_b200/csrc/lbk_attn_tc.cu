// Causal attention of the rows of a prompt pass on the 5th-generation tensor cores.
//
// The step it is part of: BitNet::forward with m > 1 rows (crates/lb-model/src/model.rs:331-357:
// q k^T / sqrt(d), causal mask, softmax in f32, times v, per head with grouped KV heads). Row i of
// the pass sits at position pos0 + i and sees keys 0 .. pos0 + i of the sequence's bf16 cache.
//
// One CTA takes 128 query rows of one head and walks the keys in blocks of 128:
//
//   TMA thread      K and V blocks [128 keys][128 dims] bf16 from the cache into a two-stage ring
//                   (SWIZZLE_128B, two 64-dimension halves each)
//   MMA thread      S = Q K^T: tcgen05.mma kind::f16, A = the queries (shared memory, written once by
//                   the CTA as two bf16 terms hi + lo, log2(e)/sqrt(d) folded in), B = the K block as it
//                   lies in the cache (K-major), f32 scores in tensor memory; then O_j = P V: A = the
//                   probabilities from TENSOR MEMORY (two bf16 terms again), B = the V block as it
//                   lies in the cache: its contraction index (the key) is the strided one, which is
//                   the MN-major operand form of the instruction, so V is never transposed
//   4 softmax warps thread r owns query row r = TMEM lane r: a row's maximum and sum are plain loops
//                   over the thread's own 128 scores (no shuffles); exp, the two bf16 terms of every
//                   probability written back to tensor memory as the next MMA's A operand; the
//                   block's P V product is read from tensor memory and added to the running output,
//                   which lives in the thread's registers with the usual max/sum rescaling
//
// f32 queries and probabilities as hi + lo (|error| <= 2^-17 |x|) keep the only rounding beyond f32
// summation the bf16 of the cache itself, as in the decode kernels. What this replaces: the same
// arithmetic on mma.sync with 16-row tiles per warp (attn_prompt_mma_kernel), which stays for
// passes of fewer than 64 rows.
//
// Rows of V past the keys written so far may hold anything (they are multiplied by exact zeros,
// and 0 * NaN is NaN): the block that reaches past them has them zeroed in shared memory first.
#include "lbk_internal.cuh"
#include "lbk_ptx.cuh"
#include "lbk_tcgen05.cuh"

namespace lbk {

namespace {

using namespace tc;

constexpr int kHd = 128;
constexpr int kTile = 128;                  // query rows per CTA = keys per block
constexpr int kHalf = kTile * 128;          // bytes of a [128 rows][64 dims] bf16 half tile
constexpr int kQBytes = 4 * kHalf;          // hi half 0, hi half 1, lo half 0, lo half 1
constexpr int kStageBytes = 4 * kHalf;      // K half 0, K half 1, V half 0, V half 1
constexpr int kStages = 2;
constexpr int kBars = kQBytes + kStages * kStageBytes;
constexpr int kMisc = kBars + 16 * 8;
constexpr int kSmem = kMisc + 64 + 1024;
constexpr int kThreads = 6 * 32;            // warps 0-3 softmax (TMEM lane quadrants), 4 TMA, 5 MMA
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 128, kColPhi = 256, kColPlo = 320;

struct AttnParams {
    CUtensorMap k, v;     // bytes [cache rows][256], box [128][128], SWIZZLE_128B
    const float *q;       // [n][nh][128], RoPE applied
    const int *pos_dev;   // position of row 0
    float *out;           // [n][nh * 128]
    int n, nh, kvh, cap, seq;
    float scaling;        // log2(e) / sqrt(d)
    int *err_word;
};

// two f32 -> one word of two bf16 (round to nearest even), `first` in the low half
__device__ __forceinline__ uint32_t bf16_pair(float first, float second) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(second), "f"(first));
    return d;
}
// x = hi + lo with hi = bf16(x), lo = bf16(x - hi), for two values at once
__device__ __forceinline__ void split_pair(float x0, float x1, uint32_t &hi, uint32_t &lo) {
    hi = bf16_pair(x0, x1);
    lo = bf16_pair(x0 - __uint_as_float(hi << 16), x1 - __uint_as_float(hi & 0xffff0000u));
}
__device__ __forceinline__ float ex2(float x) {  // 2^x, the hardware's approximation (what __expf is built on)
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
                 "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}

// MN-major SWIZZLE_128B operand (the V block: 64 dimensions contiguous, 8 keys to a 1024-byte
// group): groups of 8 keys 1024 bytes apart (stride byte offset), the two 64-dimension halves
// 16 KB apart (leading byte offset)
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(kHalf >> 4) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d_tmem), "l"(adesc), "l"(bdesc),
                 "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }" ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc),
                 "r"(idesc), "r"(accumulate)
                 : "memory");
}

__global__ void __launch_bounds__(kThreads, 1) attn_prompt_tc_kernel(const __grid_constant__ AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t bar0 = base + kBars;
    volatile uint32_t *s_tmem = reinterpret_cast<volatile uint32_t *>(sm + kMisc);
    volatile int *s_abort = reinterpret_cast<volatile int *>(sm + kMisc + 4);
    auto bar = [&](int idx) { return bar0 + idx * 8; };
    constexpr int kKFull = 0, kVFull = 2, kKvEmpty = 4, kSFull = 6, kPReady = 7, kOFull = 8;
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(bar(kKFull + s), 1);
            ptx::mbar_init(bar(kVFull + s), 1);
            ptx::mbar_init(bar(kKvEmpty + s), 1);
        }
        ptx::mbar_init(bar(kSFull), 1);
        ptx::mbar_init(bar(kPReady), 4);
        ptx::mbar_init(bar(kOFull), 1);
        *s_abort = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 5) {
        tmem_alloc(base + kMisc, kTmemCols);
        tmem_relinquish();
    }
    ptx::pdl_trigger();
    ptx::pdl_wait();  // q, the cache rows of this pass and the position are the kernels' in front
    const int head = blockIdx.x, tile = static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y);  // the late rows see the most keys: they start first
    const int kh = head / (p.nh / p.kvh);
    const int pos0 = *p.pos_dev;
    const int row0 = tile * kTile;
    const int rows_here = p.n - row0 < kTile ? p.n - row0 : kTile;
    const int written = pos0 + p.n;                          // keys 0 .. written-1 hold numbers
    const int n_blocks = (pos0 + row0 + rows_here - 1) / kTile + 1;  // key blocks some row of the tile sees
    const bool pos_ok = pos0 >= 0 && written <= p.cap;
    if (!pos_ok && tid == 0) atomicExch(p.err_word, 7);
    // the queries of the tile: scaled, as hi + lo, in the K-major SWIZZLE_128B layout (row r of a half
    // tile at r * 128, its 16-byte units XOR-ed with r & 7)
    if (warp < 4) {
        const int r = warp * 32 + lane;
        const bool live = r < rows_here && pos_ok;
        const float *qr = p.q + (static_cast<size_t>(row0 + (live ? r : 0)) * p.nh + head) * kHd;
#pragma unroll 4
        for (int u = 0; u < 16; ++u) {  // 16-byte unit u of the row: dimensions 8u .. 8u+7
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
            if (live) {
                a = *reinterpret_cast<const float4 *>(qr + 8 * u);
                b = *reinterpret_cast<const float4 *>(qr + 8 * u + 4);
            }
            const float x[8] = {a.x * p.scaling, a.y * p.scaling, a.z * p.scaling, a.w * p.scaling, b.x * p.scaling, b.y * p.scaling, b.z * p.scaling, b.w * p.scaling};
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) split_pair(x[2 * e], x[2 * e + 1], hi[e], lo[e]);
            const int half = u >> 3, unit = u & 7;
            uint8_t *dst = sm + half * kHalf + r * 128 + ((unit ^ (r & 7)) << 4);
            *reinterpret_cast<uint4 *>(dst) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4 *>(dst + 2 * kHalf) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
        ptx::fence_proxy_async();  // the tensor core reads these through the asynchronous proxy
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    bool ok = pos_ok;
    const int nb = ok ? n_blocks : 0;
    const int cache_row0 = (p.seq * p.kvh + kh) * p.cap;

    if (warp == 4) {
        // ================= TMA producer =================
        if (lane == 0) {
            for (int j = 0; j < nb; ++j) {
                const int s = j & 1;
                if (j >= kStages && !wait_bar(bar(kKvEmpty + s), ((j >> 1) - 1) & 1, s_abort)) {
                    ok = false;
                    break;
                }
                const uint32_t st = base + kQBytes + s * kStageBytes;
                const int y = cache_row0 + j * kTile;
                ptx::mbar_arrive_expect_tx(bar(kKFull + s), 2 * kHalf);
                ptx::tma_load_2d(st, &p.k, bar(kKFull + s), 0, y);
                ptx::tma_load_2d(st + kHalf, &p.k, bar(kKFull + s), 128, y);
                ptx::mbar_arrive_expect_tx(bar(kVFull + s), 2 * kHalf);
                ptx::tma_load_2d(st + 2 * kHalf, &p.v, bar(kVFull + s), 0, y);
                ptx::tma_load_2d(st + 3 * kHalf, &p.v, bar(kVFull + s), 128, y);
            }
        }
    } else if (warp == 5) {
        // ================= MMA issuer (one thread) =================
        if (lane == 0 && nb > 0) {
            // D f32, A and B bf16, M = 128, N = 128; for P V the B operand is MN-major (bit 16)
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
            constexpr uint32_t idesc_o = idesc_s | (1u << 16);
            const uint64_t q_desc = smem_desc_sw128(base);
            auto issue_s = [&](int j) {  // S = Qhi K^T + Qlo K^T over the 8 steps of 16 dimensions
                const uint64_t k_desc = smem_desc_sw128(base + kQBytes + (j & 1) * kStageBytes);
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const uint64_t off = static_cast<uint64_t>((ks >> 2) * (kHalf >> 4) + (ks & 3) * 2);
                        umma_f16_ss(tmem_base + kColS, q_desc + static_cast<uint64_t>(t * 2 * (kHalf >> 4)) + off, k_desc + off, idesc_s, (t | ks) ? 1u : 0u);
                    }
                umma_commit(bar(kSFull));
            };
            if (!wait_bar(bar(kKFull), 0, s_abort)) ok = false;
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int j = 0; j < nb && ok; ++j) {
                const int s = j & 1;
                if (!wait_bar(bar(kPReady), j & 1, s_abort) || !wait_bar(bar(kVFull + s), (j >> 1) & 1, s_abort)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint64_t v_desc = smem_desc_mn_sw128(base + kQBytes + s * kStageBytes + 2 * kHalf);
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)  // 16 keys a step: 8 columns of P, two 1024-byte key groups of V
                        umma_f16_ts(tmem_base + kColO, tmem_base + (t ? kColPlo : kColPhi) + ks * 8, v_desc + static_cast<uint64_t>(ks * (2048 >> 4)), idesc_o,
                                    (t | ks) ? 1u : 0u);
                umma_commit(bar(kOFull));
                umma_commit(bar(kKvEmpty + s));  // every MMA that read this stage is before this point
                if (j + 1 < nb) {
                    if (!wait_bar(bar(kKFull + (s ^ 1)), ((j + 1) >> 1) & 1, s_abort)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    issue_s(j + 1);
                }
            }
        }
    } else {
        // ================= softmax and output (warps 0..3 = TMEM lane quadrants) =================
        const int r = warp * 32 + lane;
        const int qpos = pos0 + row0 + r;  // the last key this row sees
        const uint32_t lane_field = static_cast<uint32_t>(warp * 32) << 16;
        float o[kHd];
#pragma unroll
        for (int i = 0; i < kHd; ++i) o[i] = 0.0f;
        float m = -INFINITY, l = 0.0f;
        for (int j = 0; j < nb; ++j) {
            if (!wait_bar(bar(kSFull), j & 1, s_abort)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const int key0 = j * kTile;
            const bool diag = key0 + kTile - 1 > qpos;  // some keys of this block are in this row's future
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_base + lane_field + kColS + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (!diag || key0 + c * 32 + i <= qpos) mx = fmaxf(mx, __uint_as_float(v[i]));
            }
            // key 0 <= qpos always: from the first block on the maximum is finite for rows that exist
            const float nm = fmaxf(m, mx);
            const float corr = ex2(m - nm);
            m = nm;
            float ps = 0.0f;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_base + lane_field + kColS + c * 32, v);
                tmem_ld_wait();
                uint32_t ph[16], pl[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float e0 = ex2(__uint_as_float(v[2 * i]) - nm), e1 = ex2(__uint_as_float(v[2 * i + 1]) - nm);
                    if (diag) {
                        if (key0 + c * 32 + 2 * i > qpos) e0 = 0.0f;
                        if (key0 + c * 32 + 2 * i + 1 > qpos) e1 = 0.0f;
                    }
                    ps += e0 + e1;
                    split_pair(e0, e1, ph[i], pl[i]);
                }
                tmem_st16(tmem_base + lane_field + kColPhi + c * 16, ph);
                tmem_st16(tmem_base + lane_field + kColPlo + c * 16, pl);
            }
            l = l * corr + ps;
            // rows of V that no kernel has written: zero them before the tensor core multiplies them by zeros
            if (key0 + kTile > written) {
                if (!wait_bar(bar(kVFull + (j & 1)), (j >> 1) & 1, s_abort)) {
                    ok = false;
                    break;
                }
                if (key0 + r >= written) {
                    uint8_t *vrow = sm + kQBytes + (j & 1) * kStageBytes + 2 * kHalf + r * 128;
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        *reinterpret_cast<uint4 *>(vrow + u * 16) = make_uint4(0u, 0u, 0u, 0u);
                        *reinterpret_cast<uint4 *>(vrow + kHalf + u * 16) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                ptx::fence_proxy_async();
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar(kPReady));
            if (corr != 1.0f) {
#pragma unroll
                for (int i = 0; i < kHd; ++i) o[i] *= corr;
            }
            if (!wait_bar(bar(kOFull), j & 1, s_abort)) {
                ok = false;
                break;
            }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_base + lane_field + kColO + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[c * 32 + i] += __uint_as_float(v[i]);
            }
            tc_fence_before();
        }
        if (ok && r < rows_here) {
            const float inv = 1.0f / l;
            float *dst = p.out + (static_cast<size_t>(row0 + r) * p.nh + head) * kHd;
#pragma unroll
            for (int i = 0; i < kHd; i += 4) *reinterpret_cast<float4 *>(dst + i) = make_float4(o[i] * inv, o[i + 1] * inv, o[i + 2] * inv, o[i + 3] * inv);
        }
    }
    if (!ok && pos_ok && lane == 0) atomicExch(p.err_word, 5);
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace

int attn_tc_init(Ctx *ctx) {
    if (static_cast<size_t>(kSmem) > ctx->smem_optin) return fail(LBK_ERR_UNSUPPORTED, "prompt attention kernel needs %d B of shared memory", kSmem);
    LBK_CUDA(cudaFuncSetAttribute(attn_prompt_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    return LBK_OK;
}

int launch_attn_prompt_tc(Ctx *ctx, const float *q, const uint16_t *kc, const uint16_t *vc, const int32_t *pos_dev, size_t n, size_t nh, size_t kvh,
                          size_t cap, size_t seq, float *out, cudaStream_t stream) {
    AttnParams p{};
    const size_t cache_rows = (seq + 1) * kvh * cap;  // the rows of the cache up to and including this sequence's
    LBK_TRY(encode_bytes_map(&p.k, kc, 256, cache_rows, 256, 128, kTile));
    LBK_TRY(encode_bytes_map(&p.v, vc, 256, cache_rows, 256, 128, kTile));
    p.q = q;
    p.pos_dev = pos_dev;
    p.out = out;
    p.n = static_cast<int>(n);
    p.nh = static_cast<int>(nh);
    p.kvh = static_cast<int>(kvh);
    p.cap = static_cast<int>(cap);
    p.seq = static_cast<int>(seq);
    p.scaling = 1.4426950408889634f / sqrtf(static_cast<float>(kHd));  // scores in units of log 2: the softmax is 2^(s - max)
    p.err_word = ctx->err_word;
    const dim3 grid(static_cast<unsigned>(nh), static_cast<unsigned>((n + kTile - 1) / kTile));
    LBK_CUDA(launch_chained(attn_prompt_tc_kernel, grid, dim3(kThreads), static_cast<size_t>(kSmem), stream, p));
    LBK_CUDA(cudaGetLastError());
    ctx->launches++;
    return LBK_OK;
}

}  // namespace lbk
