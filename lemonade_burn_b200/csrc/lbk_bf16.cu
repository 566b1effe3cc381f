// f32 activations x bf16 weights (the tied, unquantised LM head).
//
// Replaces bf16_gemv / dot_scalar / dot_avx2 / dot_avx512 (crates/lb-ternary/src/bf16.rs:14-105)
// and the bf16_linear op above them (crates/lb-model/src/ops.rs:199-218):
// out[t, r] = sum_k x[t, k] * bf16(W[r, k]), f32 products and f32 accumulation.
// HBM-bound: W (rows*cols*2 bytes) is read once per pass: one token row on the FMA kernel, up to
// 64 rows per pass on tcgen05 (bf16_head_kernel below), up to kTok = 4 rows per pass on the FMA
// kernel for rows that are not whole 16-byte units.
// Summation order differs from the reference's 8-lane order, so results agree to rounding,
// not bit for bit (the reference allows 1e-4 absolute, bf16.rs:113-136).
#include "lbk_internal.cuh"
#include "lbk_ptx.cuh"
#include "lbk_tcgen05.cuh"

namespace lbk {

namespace {

using namespace tc;

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

__device__ __forceinline__ uint32_t f32_to_bf16_rn(float v) {  // round to nearest even; NaN kept a NaN
    const uint32_t u = __float_as_uint(v);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (u >> 16) | 0x40u;
    return (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
}

// ---- two token rows and more: the 5th-generation tensor cores ----------------------------------
//
// out[t, r] = sum_k x[t, k] * W[r, k] as a tcgen05 GEMM (kind::f16, bf16 operands, f32 accumulators in
// tensor memory). The 128 table rows of a tile are the MMA's M side, the token rows its N side. An
// f32 activation is two bf16 terms, x = hi + lo with lo = bf16(x - hi) (a product is then the
// reference's f32 product to within 2^-17 relative; W's bf16 values are exact): the hi rows and the
// lo rows of up to 64 tokens are ONE B operand of up to 128 rows, so that one instruction does both
// terms, and the epilogue adds the two halves of the accumulator. Accuracy: the difference from the
// reference's sums is the tensor core's own f32 accumulation (its order and rounding), growing with
// the column count: 3e-6 / 7e-6 / 1e-5 of max |out| at 2560 / 6912 / 8192 columns, measured; a third
// bf16 term (x exactly) changed none of these digits and is not used. The reference allows 1e-4
// absolute (bf16.rs:113-136). Both operands come straight from shared memory, where TMA puts them
// (SWIZZLE_128B, 64 columns = 128 bytes a K block); no thread touches the table. One persistent CTA
// per SM walks the table's 128-row tiles, each over the whole of K: the table is read once per 64
// token rows, the activations (2 x 64 x cols bf16, L2 resident) once per tile. Bound: HBM,
// rows * cols * 2 bytes.
//
// What it replaced: an mma.sync kernel that took 16 or 32 token rows per pass over the table and ran
// at 2 TB/s (its activation fragments came from shared memory once per 16 table rows: four bytes of
// shared-memory reads per table byte). Rows that are not whole 16-byte units, or longer than the
// context's activation buffer, take the FMA kernel above, four token rows per pass.
constexpr int kTcTokMax = 64;                  // token rows per pass over the table
constexpr int kTcRows = 128;                   // table rows per tile (MMA M, TMEM lanes)
constexpr int kTcKB = 64;                      // columns per stage: 128 bytes of bf16
constexpr int kTcTerms = 2;                    // bf16 terms per f32 activation
constexpr int kTcStages = 6;
constexpr int kTcWBytes = kTcRows * 128;       // 16 KB
constexpr int kTcXBytes = kTcTerms * kTcTokMax * 128; // 16 KB
constexpr int kTcStageBytes = kTcWBytes + kTcXBytes;
constexpr int kTcBars = kTcStages * kTcStageBytes;
constexpr int kTcMisc = kTcBars + 32 * 8;
constexpr int kTcSmem = kTcMisc + 64 + 1024;
constexpr int kTcThreads = 6 * 32;             // warps 0-3 epilogue, 4 TMA, 5 MMA
constexpr uint32_t kTcTmemCols = 256;          // two accumulators of up to 128 columns
constexpr size_t kTcMaxCols = 32768;           // the activation buffer of the context is sized for this (8 MB)

struct HeadParams {
    CUtensorMap w;      // bytes [rows][cols * 2], box [128][128], SWIZZLE_128B
    CUtensorMap x;      // bytes [2 * ntp][cols * 2] (hi rows, then lo rows), box [2 * ntp][128], SWIZZLE_128B
    float *out;         // [m][rows]; this pass writes token rows t0 .. t0 + ntok - 1
    int rows, k_blocks, tiles, ntp, ntok, t0;
    int *err_word;
};

// x f32 [ntok][cols] -> bf16 [2 * ntp][cols]: rows 0 .. ntp-1 the hi terms, ntp .. 2 ntp-1 the lo terms
// (hi = bf16(x), lo = bf16(x - hi)); token rows past ntok zero
__global__ void __launch_bounds__(256) split_x_kernel(const float *__restrict__ x, int cols, int ntok, int ntp, uint16_t *__restrict__ xs) {
    ptx::pdl_trigger();
    ptx::pdl_wait();
    const int pairs = cols >> 1;
    for (int i = blockIdx.x * 256 + threadIdx.x; i < ntp * pairs; i += gridDim.x * 256) {
        const int tk = i / pairs, c = (i - tk * pairs) * 2;
        float2 v = make_float2(0.f, 0.f);
        if (tk < ntok) v = *reinterpret_cast<const float2 *>(x + static_cast<size_t>(tk) * cols + c);
        const uint32_t h0 = f32_to_bf16_rn(v.x), h1 = f32_to_bf16_rn(v.y);
        const uint32_t l0 = f32_to_bf16_rn(v.x - __uint_as_float(h0 << 16)), l1 = f32_to_bf16_rn(v.y - __uint_as_float(h1 << 16));
        *reinterpret_cast<uint32_t *>(xs + static_cast<size_t>(tk) * cols + c) = h0 | (h1 << 16);
        *reinterpret_cast<uint32_t *>(xs + static_cast<size_t>(ntp + tk) * cols + c) = l0 | (l1 << 16);
    }
}

// the four K = 16 steps of one 64-column block: both descriptors advance 32 bytes (2 units) a step
__device__ __forceinline__ void umma_bf16_ss_block(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate_first) {
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        ".reg .b64 a1, a2, a3, b1, b2, b3;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "setp.eq.b32 q, 0, 0;\n"
        "add.u64 a1, %1, 2;\n"
        "add.u64 a2, %1, 4;\n"
        "add.u64 a3, %1, 6;\n"
        "add.u64 b1, %2, 2;\n"
        "add.u64 b2, %2, 4;\n"
        "add.u64 b3, %2, 6;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, q;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, q;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, q;\n"
        "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate_first)
        : "memory");
}

__global__ void __launch_bounds__(kTcThreads, 1) bf16_head_kernel(const __grid_constant__ HeadParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t bar0 = base + kTcBars;
    volatile uint32_t *s_tmem = reinterpret_cast<volatile uint32_t *>(sm + kTcMisc);
    volatile int *s_abort = reinterpret_cast<volatile int *>(sm + kTcMisc + 4);
    // barriers: full[stage], empty[stage], acc_full[2], acc_empty[2]
    auto bar = [&](int idx) { return bar0 + idx * 8; };
    constexpr int kFull = 0, kEmpty = kTcStages, kAccFull = 2 * kTcStages, kAccEmpty = 2 * kTcStages + 2;
    if (tid == 0) {
        for (int i = 0; i < kTcStages; ++i) {
            ptx::mbar_init(bar(kFull + i), 1);
            ptx::mbar_init(bar(kEmpty + i), 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(bar(kAccFull + a), 1);
            ptx::mbar_init(bar(kAccEmpty + a), 4);
        }
        *s_abort = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 5) {
        tmem_alloc(base + kTcMisc, kTcTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    ptx::pdl_trigger();
    const int n = kTcTerms * p.ntp;  // MMA N: the hi rows and the lo rows of this pass's tokens
    bool ok = true;

    if (warp == 4) {
        // ================= TMA producer =================
        if (lane == 0) {
            const int my_tiles = p.tiles > static_cast<int>(blockIdx.x) ? (p.tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x) : 0;
            const int total = my_tiles * p.k_blocks;
            const int pre = total < kTcStages ? total : kTcStages;
            const uint32_t stage_tx = static_cast<uint32_t>(kTcWBytes + n * 128);
            // The table is a constant: the first ring of its blocks is on its way before the kernel in
            // front (the one that writes the activations' two terms) is known to be complete.
            for (int it = 0; it < pre; ++it) {
                const int tile = static_cast<int>(blockIdx.x) + (it / p.k_blocks) * static_cast<int>(gridDim.x), kb = it % p.k_blocks;
                ptx::mbar_arrive_expect_tx(bar(kFull + it), stage_tx);
                ptx::tma_load_2d(base + it * kTcStageBytes, &p.w, bar(kFull + it), kb * 128, tile * kTcRows);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int it = 0; it < pre; ++it)
                ptx::tma_load_2d(base + it * kTcStageBytes + kTcWBytes, &p.x, bar(kFull + it), (it % p.k_blocks) * 128, 0);
            int s = 0, round = 1, tile = static_cast<int>(blockIdx.x) + (pre / p.k_blocks) * static_cast<int>(gridDim.x), kb = pre % p.k_blocks;
            for (int it = pre; it < total; ++it) {
                if (!wait_bar(bar(kEmpty + s), (round - 1) & 1, s_abort)) {
                    ok = false;
                    break;
                }
                ptx::mbar_arrive_expect_tx(bar(kFull + s), stage_tx);
                ptx::tma_load_2d(base + s * kTcStageBytes, &p.w, bar(kFull + s), kb * 128, tile * kTcRows);
                ptx::tma_load_2d(base + s * kTcStageBytes + kTcWBytes, &p.x, bar(kFull + s), kb * 128, 0);
                if (++s == kTcStages) {
                    s = 0;
                    ++round;
                }
                if (++kb == p.k_blocks) {
                    kb = 0;
                    tile += static_cast<int>(gridDim.x);
                }
            }
        }
    } else if (warp == 5) {
        // ================= MMA issuer (one thread) =================
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | ((kTcRows >> 4) << 24);
            const uint64_t adesc0 = smem_desc_sw128(base), bdesc0 = smem_desc_sw128(base + kTcWBytes);
            int it = 0, tcount = 0;
            for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++tcount) {
                const int a = tcount & 1, around = tcount >> 1;
                if (around > 0 && !wait_bar(bar(kAccEmpty + a), (around - 1) & 1, s_abort)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + a * 128;
                for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
                    const int s = it % kTcStages, round = it / kTcStages;
                    if (!wait_bar(bar(kFull + s), round & 1, s_abort)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t off = static_cast<uint64_t>(s) * (kTcStageBytes >> 4);
                    umma_bf16_ss_block(d_tmem, adesc0 + off, bdesc0 + off, idesc, kb ? 1u : 0u);
                    umma_commit(bar(kEmpty + s));  // the stage is free once these MMAs retire
                }
                if (!ok) break;
                umma_commit(bar(kAccFull + a));
            }
        }
    } else {
        // ================= epilogue (warps 0..3 = TMEM lane quadrants 0..3) =================
        asm volatile("griddepcontrol.wait;" ::: "memory");  // out may still be read by the kernel in front
        int tcount = 0;
        for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++tcount) {
            const int a = tcount & 1, around = tcount >> 1;
            if (!wait_bar(bar(kAccFull + a), around & 1, s_abort)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const int row = tile * kTcRows + warp * 32 + lane;
            const uint32_t acc = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + a * 128;
#pragma unroll 1
            for (int c = 0; c * 32 < p.ntok; ++c) {
                uint32_t hi[32], lo[32];
                tmem_ld32(acc + c * 32, hi);
                tmem_ld32(acc + p.ntp + c * 32, lo);
                tmem_ld_wait();
                if (row < p.rows) {
                    float *o = p.out + static_cast<size_t>(p.t0 + c * 32) * p.rows + row;
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i < p.ntok) o[static_cast<size_t>(i) * p.rows] = __fadd_rn(__uint_as_float(hi[i]), __uint_as_float(lo[i]));
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar(kAccEmpty + a));
        }
    }
    if (!ok && lane == 0) atomicExch(p.err_word, 5);
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTcTmemCols);
    }
}

}  // namespace

int bf16_init(Ctx *ctx) {
    if (static_cast<size_t>(kTcSmem) > ctx->smem_optin) return fail(LBK_ERR_UNSUPPORTED, "bf16 head kernel needs %d B of shared memory", kTcSmem);
    LBK_CUDA(cudaFuncSetAttribute(bf16_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem));
    // the activations' bf16 terms of one pass: [2 * 64 token rows][up to kTcMaxCols]
    LBK_CUDA(cudaMalloc(&ctx->bf16_x, kTcTerms * kTcTokMax * kTcMaxCols * sizeof(uint16_t)));
    return LBK_OK;
}

// two token rows and more, rows of whole 16-byte units: the tcgen05 kernel, 64 token rows per pass
static int launch_bf16_head_tc(Ctx *ctx, const float *x, size_t m, const uint16_t *w, size_t rows, size_t cols, float *out, cudaStream_t stream) {
    HeadParams p{};
    LBK_TRY(encode_bytes_map(&p.w, w, cols * 2, rows, cols * 2, 128, kTcRows));
    p.rows = static_cast<int>(rows);
    p.k_blocks = static_cast<int>((cols + kTcKB - 1) / kTcKB);
    p.tiles = static_cast<int>((rows + kTcRows - 1) / kTcRows);
    p.out = out;
    p.err_word = ctx->err_word;
    uint16_t *xs = static_cast<uint16_t *>(ctx->bf16_x);
    const int grid = p.tiles < ctx->sm_count ? p.tiles : ctx->sm_count;
    for (size_t t0 = 0; t0 < m; t0 += kTcTokMax) {
        const int ntok = static_cast<int>(m - t0 < static_cast<size_t>(kTcTokMax) ? m - t0 : kTcTokMax);
        const int ntp = (ntok + 15) & ~15;
        const size_t pairs = static_cast<size_t>(ntp) * (cols >> 1);
        const unsigned sgrid = static_cast<unsigned>((pairs + 255) / 256 < static_cast<size_t>(ctx->sm_count) * 4 ? (pairs + 255) / 256 : static_cast<size_t>(ctx->sm_count) * 4);
        LBK_CUDA(launch_chained(split_x_kernel, dim3(sgrid), dim3(256), 0, stream, x + t0 * cols, static_cast<int>(cols), ntok, ntp, xs));
        LBK_TRY(encode_bytes_map(&p.x, xs, cols * 2, static_cast<size_t>(kTcTerms * ntp), cols * 2, 128, kTcTerms * ntp));
        p.ntp = ntp;
        p.ntok = ntok;
        p.t0 = static_cast<int>(t0);
        LBK_CUDA(launch_chained(bf16_head_kernel, dim3(static_cast<unsigned>(grid)), dim3(kTcThreads), static_cast<size_t>(kTcSmem), stream, p));
        LBK_CUDA(cudaGetLastError());
        ctx->launches += 2;
    }
    return LBK_OK;
}

int launch_bf16_linear(Ctx *ctx, const float *x, size_t m, const uint16_t *w, size_t rows,
                       size_t cols, float *out, cudaStream_t stream) {
    if (m == 0 || rows == 0) return LBK_OK;
    if (m >= 2 && (cols & 7) == 0 && cols <= kTcMaxCols && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 7) == 0)
        return launch_bf16_head_tc(ctx, x, m, w, rows, cols, out, stream);
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
