// Prefill GEMM (more than 16 token rows): int8 activations x packed ternary weights on the
// 5th-generation tensor cores (tcgen05.mma kind::i8, accumulators in TMEM).
//
// Replaces ternary_gemm_multi's prefill branch and the AVX-512 register tile under it
// (crates/lb-ternary/src/gemm.rs:155-194, 245-268, 483-550). Per output tile of 128 token rows x
// 256 weight rows, per 128-column block of K (one packed 32-byte block per weight row):
//
//   TMA warp       int8 activations [128 tok][128 B] (SWIZZLE_128B) and packed weights
//                  [256 rows][32 B] into a 3-stage ring
//   4 expander     2 bits -> u8 codes, written as the K-major SWIZZLE_128B tile the MMA wants:
//   warps          (word >> 2k) & 0x03030303 is four consecutive columns k*32 + j..j+3, so every
//                  16 packed bytes become four 16-byte stores, no shuffles (pack.rs:10-13)
//   MMA thread     4 x tcgen05.mma (M=128 tokens, N=256 rows, K=32), s8 x u8 -> s32 in TMEM;
//                  tcgen05.commit frees the stage / publishes the accumulator
//   4 epilogue     tcgen05.ld, dot = acc - sum(q) (codes are w+1: gemm.rs:6-9,306-308),
//   warps          y = (float)dot * (1/(s_a*s_w)) (gemm.rs:158,178), stores [token][row]
//
// Two 256-column accumulators in TMEM let the epilogue of one tile overlap the MMAs of the next.
// Bound: int8 tensor pipe. Work per call: 2*m*rows*cols integer operations.
#include "lbk_internal.cuh"
#include "lbk_ptx.cuh"

namespace lbk {

namespace {

constexpr int kBM = 128;           // token rows per tile (MMA M)
constexpr int kBN = 256;           // weight rows per tile (MMA N)
constexpr int kBK = 128;           // columns per stage = one packed block
constexpr int kStages = 3;
constexpr int kActBytes = kBM * kBK;          // 16 KB int8, swizzled
constexpr int kExpBytes = kBN * kBK;          // 32 KB u8 codes, swizzled
constexpr int kPackBytes = kBN * kBlockBytes; //  8 KB packed
constexpr int kStageBytes = kActBytes + kExpBytes + kPackBytes;
constexpr int kEpiWarps = 4, kExpWarps = 4;
constexpr int kTmaWarp = 4, kMmaWarp = 5, kExpWarp0 = 6;
constexpr int kThreads = (kEpiWarps + 2 + kExpWarps) * 32;  // 320
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kWaitLimit = 1u << 22;

// instruction descriptor: D s32, A s8 (activations), B u8 (codes), both K-major, N=256, M=128
constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (0u << 10) | ((kBN >> 3) << 17) | ((kBM >> 4) << 24);

struct GemmParams {
    CUtensorMap act;                    // int8 [m][kp], box [128][128], SWIZZLE_128B
    CUtensorMap wpk[LBK_MAX_GROUP];     // u8 [rows][rb], box [256][32]
    float *out[LBK_MAX_GROUP];
    int32_t *iout[LBK_MAX_GROUP];
    float wscale[LBK_MAX_GROUP];
    int rows[LBK_MAX_GROUP];
    int tile_end[LBK_MAX_GROUP];        // running tile count up to and including matrix i
    int n_mat, m, m_tiles, k_blocks, total_tiles;
    const float *qscale;
    const int32_t *qsum;
    int *err_word;
};

// ---- tcgen05 wrappers ----------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// mbarrier arrive once every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major SWIZZLE_128B shared-memory matrix descriptor: rows of 128 bytes, 8-row groups 1024 B
// apart (SBO), version 1, layout type 2; `addr` may be advanced by 32 B per K=32 step.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);   // start address
    d |= static_cast<uint64_t>(1) << 16;                  // leading byte offset (unused for SW128 K-major)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;          // stride byte offset
    d |= static_cast<uint64_t>(1) << 46;                  // descriptor version (Blackwell)
    d |= static_cast<uint64_t>(2) << 61;                  // SWIZZLE_128B
    return d;
}

// Bounded wait that also gives up as soon as another role has flagged an abort.
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

struct Smem {
    uint32_t stage[kStages];      // byte offsets from the aligned base
    uint32_t bars;                // mbarriers
    uint32_t misc;                // tmem base, abort flag
    uint32_t total;
};
__host__ __device__ inline Smem smem_map() {
    Smem s;
    uint32_t o = 0;
    for (int i = 0; i < kStages; ++i) {
        s.stage[i] = o;
        o += kStageBytes;
    }
    s.bars = o;
    o += 32 * 8;
    s.misc = o;
    o += 64;
    s.total = o;
    return s;
}
// barrier indices
constexpr int kBarFullAct = 0;               // [kStages] TMA activations landed
constexpr int kBarFullPack = kStages;        // [kStages] TMA packed weights landed
constexpr int kBarFullExp = 2 * kStages;     // [kStages] expanders finished the u8 tile
constexpr int kBarEmpty = 3 * kStages;       // [kStages] MMAs that read the stage completed
constexpr int kBarAccFull = 4 * kStages;     // [2] accumulator complete
constexpr int kBarAccEmpty = 4 * kStages + 2;// [2] accumulator drained by the epilogue

__global__ void __launch_bounds__(kThreads, 1) gemm_kernel(const __grid_constant__ GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const Smem S = smem_map();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t bar0 = base + S.bars;
    volatile uint32_t *s_tmem = reinterpret_cast<volatile uint32_t *>(sm + S.misc);
    volatile int *s_abort = reinterpret_cast<volatile int *>(sm + S.misc + 4);

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            ptx::mbar_init(bar0 + (kBarFullAct + i) * 8, 1);
            ptx::mbar_init(bar0 + (kBarFullPack + i) * 8, 1);
            ptx::mbar_init(bar0 + (kBarFullExp + i) * 8, kExpWarps);
            ptx::mbar_init(bar0 + (kBarEmpty + i) * 8, 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(bar0 + (kBarAccFull + a) * 8, 1);
            ptx::mbar_init(bar0 + (kBarAccEmpty + a) * 8, kEpiWarps);
        }
        *s_abort = 0;
        ptx::fence_barrier_init();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(base + S.misc, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;

    const int k_blocks = p.k_blocks;
    bool ok = true;

    if (warp == kTmaWarp) {
        // ================= TMA producer =================
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
                int mat = 0;
                while (mat < p.n_mat - 1 && tile >= p.tile_end[mat]) ++mat;
                const int local = tile - (mat ? p.tile_end[mat - 1] : 0);
                const int m_tile = local % p.m_tiles, n_tile = local / p.m_tiles;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % kStages, round = it / kStages;
                    if (round > 0 && !wait_bar(bar0 + (kBarEmpty + s) * 8, (round - 1) & 1, s_abort)) {
                        ok = false;
                        break;
                    }
                    const uint32_t st = base + S.stage[s];
                    ptx::mbar_arrive_expect_tx(bar0 + (kBarFullAct + s) * 8, kActBytes);
                    ptx::tma_load_2d(st, &p.act, bar0 + (kBarFullAct + s) * 8, kb * kBK, m_tile * kBM);
                    ptx::mbar_arrive_expect_tx(bar0 + (kBarFullPack + s) * 8, kPackBytes);
                    ptx::tma_load_2d(st + kActBytes + kExpBytes, &p.wpk[mat], bar0 + (kBarFullPack + s) * 8,
                                     kb * kBlockBytes, n_tile * kBN);
                }
            }
        }
    } else if (warp >= kExpWarp0) {
        // ================= expanders: packed 2-bit -> swizzled K-major u8 =================
        const int et = tid - kExpWarp0 * 32;  // 0..127; rows et and et + 128 of the tile
        int it = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
            for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                const int s = it % kStages, round = it / kStages;
                if (!wait_bar(bar0 + (kBarFullPack + s) * 8, round & 1, s_abort)) {
                    ok = false;
                    break;
                }
                const uint8_t *pk = sm + S.stage[s] + kActBytes + kExpBytes;
                uint8_t *ex = sm + S.stage[s] + kActBytes;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int r = et + h * 128;
                    const uint4 w0 = *reinterpret_cast<const uint4 *>(pk + r * kBlockBytes);       // bytes j = 0..15
                    const uint4 w1 = *reinterpret_cast<const uint4 *>(pk + r * kBlockBytes + 16);  // bytes j = 16..31
                    uint8_t *row = ex + r * 128;
                    const int x = r & 7;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        uint4 c0, c1;
                        c0.x = (w0.x >> (2 * k)) & 0x03030303u; c0.y = (w0.y >> (2 * k)) & 0x03030303u;
                        c0.z = (w0.z >> (2 * k)) & 0x03030303u; c0.w = (w0.w >> (2 * k)) & 0x03030303u;
                        c1.x = (w1.x >> (2 * k)) & 0x03030303u; c1.y = (w1.y >> (2 * k)) & 0x03030303u;
                        c1.z = (w1.z >> (2 * k)) & 0x03030303u; c1.w = (w1.w >> (2 * k)) & 0x03030303u;
                        // columns k*32 + 0..15 are 16-byte unit 2k, columns k*32 + 16..31 unit 2k+1
                        *reinterpret_cast<uint4 *>(row + (((2 * k) ^ x) << 4)) = c0;
                        *reinterpret_cast<uint4 *>(row + (((2 * k + 1) ^ x) << 4)) = c1;
                    }
                }
                ptx::fence_proxy_async();  // generic-proxy stores -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar0 + (kBarFullExp + s) * 8);
            }
        }
    } else if (warp == kMmaWarp) {
        // ================= MMA issuer (one thread) =================
        if (lane == 0) {
            int it = 0, tcount = 0;
            for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, ++tcount) {
                const int a = tcount & 1, around = tcount >> 1;
                if (around > 0 && !wait_bar(bar0 + (kBarAccEmpty + a) * 8, (around - 1) & 1, s_abort)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + a * kBN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % kStages, round = it / kStages;
                    if (!wait_bar(bar0 + (kBarFullAct + s) * 8, round & 1, s_abort) ||
                        !wait_bar(bar0 + (kBarFullExp + s) * 8, round & 1, s_abort)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = base + S.stage[s], b_addr = a_addr + kActBytes;
#pragma unroll
                    for (int ks = 0; ks < kBK / 32; ++ks)
                        umma_i8(d_tmem, smem_desc_sw128(a_addr + ks * 32), smem_desc_sw128(b_addr + ks * 32), kIdesc,
                                (kb | ks) ? 1u : 0u);
                    umma_commit(bar0 + (kBarEmpty + s) * 8);  // stage reusable once these MMAs retire
                }
                if (!ok) break;
                umma_commit(bar0 + (kBarAccFull + a) * 8);    // accumulator complete
            }
        }
    } else {
        // ================= epilogue (warps 0..3 = TMEM lane quadrants 0..3) =================
        int tcount = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, ++tcount) {
            const int a = tcount & 1, around = tcount >> 1;
            int mat = 0;
            while (mat < p.n_mat - 1 && tile >= p.tile_end[mat]) ++mat;
            const int local = tile - (mat ? p.tile_end[mat - 1] : 0);
            const int m_tile = local % p.m_tiles, n_tile = local / p.m_tiles;
            const int token = m_tile * kBM + warp * 32 + lane;
            const int rows = p.rows[mat];
            float *out = p.out[mat];
            int32_t *iout = p.iout[mat];
            int qs = 0;
            float inv = 0.0f;
            if (token < p.m) {
                qs = p.qsum[token];
                if (out) inv = __fdiv_rn(1.0f, __fmul_rn(p.qscale[token], p.wscale[mat]));  // gemm.rs:158
            }
            if (!wait_bar(bar0 + (kBarAccFull + a) * 8, around & 1, s_abort)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const bool vec = (rows & 3) == 0;
#pragma unroll 1
            for (int c = 0; c < kBN / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + a * kBN + c * 32, v);
                tmem_ld_wait();
                const int row0 = n_tile * kBN + c * 32;
                if (token < p.m && row0 < rows) {
                    const size_t o = static_cast<size_t>(token) * rows + row0;
                    if (vec && row0 + 32 <= rows) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            const int d0 = static_cast<int>(v[i]) - qs, d1 = static_cast<int>(v[i + 1]) - qs;
                            const int d2 = static_cast<int>(v[i + 2]) - qs, d3 = static_cast<int>(v[i + 3]) - qs;
                            if (iout) *reinterpret_cast<int4 *>(iout + o + i) = make_int4(d0, d1, d2, d3);
                            if (out)
                                *reinterpret_cast<float4 *>(out + o + i) =
                                    make_float4(__fmul_rn(__int2float_rn(d0), inv), __fmul_rn(__int2float_rn(d1), inv),
                                                __fmul_rn(__int2float_rn(d2), inv), __fmul_rn(__int2float_rn(d3), inv));
                        }
                    } else {
                        for (int i = 0; i < 32 && row0 + i < rows; ++i) {
                            const int d = static_cast<int>(v[i]) - qs;
                            if (iout) iout[o + i] = d;
                            if (out) out[o + i] = __fmul_rn(__int2float_rn(d), inv);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar0 + (kBarAccEmpty + a) * 8);
        }
    }

    if (!ok && lane == 0) atomicExch(p.err_word, 5);
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace

int gemm_init(Ctx *ctx) {
    const Smem S = smem_map();
    if (S.total + 1024 > ctx->smem_optin) return fail(LBK_ERR_UNSUPPORTED, "gemm kernel needs %u B of shared memory", S.total + 1024);
    LBK_CUDA(cudaFuncSetAttribute(gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(S.total + 1024)));
    return LBK_OK;
}

int launch_gemm(Ctx *ctx, const GroupArgs &g, cudaStream_t stream) {
    if (!g.q || !g.qsum) return fail(LBK_ERR_INVALID, "gemm: quantised activations are required");
    if (g.n < 1 || g.n > LBK_MAX_GROUP) return fail(LBK_ERR_INVALID, "group size %d not in 1..%d", g.n, LBK_MAX_GROUP);
    if (g.m == 0) return LBK_OK;
    GemmParams p{};
    const size_t kp = g.w[0]->kp;
    LBK_TRY(encode_act_map(&p.act, g.q, g.m, kp));
    p.m = static_cast<int>(g.m);
    p.m_tiles = static_cast<int>((g.m + kBM - 1) / kBM);
    p.k_blocks = static_cast<int>(kp / kBK);
    int tiles = 0;
    for (int i = 0; i < g.n; ++i) {
        const Weight *w = g.w[i];
        if (w->kp != kp) return fail(LBK_ERR_SHAPE, "inner dimension mismatch");
        if (g.out[i] && !g.qscale) return fail(LBK_ERR_INVALID, "gemm: f32 outputs need the activation scales");
        p.wpk[i] = w->tmap_gemm;
        p.out[i] = g.out[i];
        p.iout[i] = g.iout[i];
        p.wscale[i] = w->scale;
        p.rows[i] = static_cast<int>(w->rows);
        tiles += p.m_tiles * static_cast<int>((w->rows + kBN - 1) / kBN);
        p.tile_end[i] = tiles;
    }
    p.n_mat = g.n;
    p.total_tiles = tiles;
    p.qscale = g.qscale;
    p.qsum = g.qsum;
    p.err_word = ctx->err_word;
    if (tiles == 0 || p.k_blocks == 0) return LBK_OK;
    const Smem S = smem_map();
    const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    gemm_kernel<<<grid, kThreads, S.total + 1024, stream>>>(p);
    LBK_CUDA(cudaGetLastError());
    ctx->launches++;
    return LBK_OK;
}

}  // namespace lbk
