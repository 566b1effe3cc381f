// Decode GEMV (1..16 token rows): packed 2-bit ternary weights x int8 activations.
//
// Replaces ternary_gemm_multi's decode branch and its SIMD inner loops
// (crates/lb-ternary/src/gemm.rs:128-154, 329-588) together with the activation quantiser
// in front of it (crates/lb-ternary/src/quant.rs:45-118), as one bandwidth-bound kernel:
//
//   prologue  every CTA quantises the (tiny, L2-resident) activation rows itself: absmax,
//             scale = 127/max(amax,1e-5), round-half-even, clamp, sum(q)   -> shared memory
//   stream    every warp owns a contiguous run of 16-row weight tiles and its own ring of
//             TMA stages ([16 rows][128 packed bytes], SWIZZLE_128B); nothing in the main
//             loop synchronises across warps
//   decode    a packed word w holds 4 bytes j..j+3; (w & (0x03030303 << 2k)) is the code of
//             columns k*32 + j..j+3 scaled by 4^k, still a valid u8, so one LOP3 per four
//             weights feeds mma.sync.m16n8k32 (u8 x s8 -> s32) with the 16 weight rows as
//             the M side and the token rows as the N side; four accumulator sets (one per
//             k) are recombined with exact shifts at the end of the tile
//   epilogue  dot = sum(code*q) - sum(q) (gemm.rs:306-308), y = (float)dot * (1/(s_a*s_w))
//             (gemm.rs:141,150), bit-identical to the reference
//
// Algorithmic bytes per call: the packed weights once, plus m*k*4 activation bytes and
// m*rows*4 output bytes.
#include "lbk_internal.cuh"
#include "lbk_ptx.cuh"

namespace lbk {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 6;                             // TMA ring depth per warp
constexpr int kTileRows = 16;                          // weight rows per MMA tile
constexpr int kChunkBytes = 128;                       // packed bytes per row per stage
constexpr int kChunkCols = kChunkBytes * 4;            // 512 columns
constexpr int kStageBytes = kTileRows * kChunkBytes;   // 2048
constexpr uint32_t kWaitLimit = 1u << 22;              // polls before a wait gives up
constexpr int kMaxM = LBK_GEMV_MAX_M;

struct GemvParams {
    CUtensorMap tmap[LBK_MAX_GROUP];
    float *out[LBK_MAX_GROUP];
    int32_t *iout[LBK_MAX_GROUP];
    float wscale[LBK_MAX_GROUP];
    int rows[LBK_MAX_GROUP];
    int tile_end[LBK_MAX_GROUP];  // running count of 16-row tiles up to and including matrix i
    int n_mat;
    int m;
    int k;         // logical columns
    int chunks;    // ceil(row_bytes / 128)
    int xq_stride; // bytes between token rows of the quantised activations in shared memory
    int total_tiles;
    const float *x;        // f32 [m, k], or null when q is given
    const int8_t *q;       // int8 [m, kp]
    const float *qscale;   // f32 [m]
    const int32_t *qsum;   // i32 [m]
    int *err_word;
};

// Shared-memory carve-up (offsets from a 1024-byte aligned base).
struct SmemLayout {
    uint32_t stages;   // kWarps * kStages * kStageBytes
    uint32_t bars;     // kWarps * kStages * 8
    uint32_t part;     // f32/i32 [kMaxM][kWarps] reduction scratch
    uint32_t scale;    // f32 [kMaxM]
    uint32_t sum;      // i32 [kMaxM]
    uint32_t inv;      // f32 [LBK_MAX_GROUP][kMaxM]
    uint32_t xq;       // m * xq_stride
    uint32_t total;
};

__host__ __device__ inline SmemLayout smem_layout(int m, int xq_stride) {
    SmemLayout L;
    uint32_t o = 0;
    L.stages = o; o += kWarps * kStages * kStageBytes;
    L.bars = o;   o += kWarps * kStages * 8;
    L.part = o;   o += kMaxM * kWarps * 4;
    L.scale = o;  o += kMaxM * 4;
    L.sum = o;    o += kMaxM * 4;
    L.inv = o;    o += LBK_MAX_GROUP * kMaxM * 4;
    o = (o + 127u) & ~127u;
    L.xq = o;     o += static_cast<uint32_t>(m) * static_cast<uint32_t>(xq_stride);
    L.total = o;
    return L;
}

// Position of natural column n inside a token row of the shared activation buffer. The
// order puts, for every MMA, the eight bytes a lane needs next to those of its three
// neighbours: [chunk][k-group][c][t][8] with n = (chunk*4 + t)*128 + kgroup*32 + c*8 + e.
__device__ __forceinline__ uint32_t xq_pos(uint32_t n) {
    uint32_t chunk = n >> 9, t = (n >> 7) & 3, kk = (n >> 5) & 3, c = (n >> 3) & 3, e = n & 7;
    return ((((chunk * 4 + kk) * 4 + c) * 4 + t) << 3) + e;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// quant.rs:115-118: (v*scale).round_ties_even().clamp(-128,127) as i8, NaN -> 0.
__device__ __forceinline__ int quant_one(float v, float scale) {
    int r = __float2int_rn(__fmul_rn(v, scale));  // NaN -> 0, saturates
    return max(-128, min(127, r));
}

template <int MT>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const SmemLayout L = smem_layout(p.m, p.xq_stride);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    // ---- this warp's run of tiles --------------------------------------------------------
    const long long gw = static_cast<long long>(blockIdx.x) * kWarps + warp;
    const long long nw = static_cast<long long>(gridDim.x) * kWarps;
    const int tile_begin = static_cast<int>(gw * p.total_tiles / nw);
    const int tile_end = static_cast<int>((gw + 1) * p.total_tiles / nw);
    const int chunks = p.chunks;
    const int n_items = (tile_end - tile_begin) * chunks;

    const uint32_t stage0 = base + L.stages + warp * (kStages * kStageBytes);
    const uint32_t bar0 = base + L.bars + warp * (kStages * 8);

    // producer state (lane 0 only): next item to issue
    int issue_tile = tile_begin, issue_chunk = 0, issue_mat = 0;
    auto issue = [&](int s) {  // s: the ring stage the next item goes into
        while (issue_mat < p.n_mat - 1 && issue_tile >= p.tile_end[issue_mat]) ++issue_mat;
        const int tile_in_mat = issue_tile - (issue_mat ? p.tile_end[issue_mat - 1] : 0);
        ptx::mbar_arrive_expect_tx(bar0 + s * 8, kStageBytes);
        ptx::tma_load_2d(stage0 + s * kStageBytes, &p.tmap[issue_mat], bar0 + s * 8,
                         issue_chunk * kChunkBytes, tile_in_mat * kTileRows);
        if (++issue_chunk == chunks) {
            issue_chunk = 0;
            ++issue_tile;
        }
    };

    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) ptx::mbar_init(bar0 + s * 8, 1);
        ptx::fence_barrier_init();
        const int first = n_items < kStages ? n_items : kStages;
        for (int i = 0; i < first; ++i) issue(i);
    }

    // ---- prologue: quantised activations into shared memory ------------------------------
    float *s_part = reinterpret_cast<float *>(sm + L.part);
    float *s_scale = reinterpret_cast<float *>(sm + L.scale);
    int *s_sum = reinterpret_cast<int *>(sm + L.sum);
    float *s_inv = reinterpret_cast<float *>(sm + L.inv);
    uint8_t *s_xq = sm + L.xq;
    const int m = p.m, k = p.k;
    const int kfill = chunks * kChunkCols;  // columns held per token row (zero padded)

    if (p.x != nullptr) {
        const bool vec = (k & 3) == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15) == 0;
        // pass 1: per-token absmax (quant.rs:101-104)
        for (int tk = 0; tk < m; ++tk) {
            const float *xr = p.x + static_cast<size_t>(tk) * k;
            float am = 0.0f;
            if (vec) {
                const float4 *x4 = reinterpret_cast<const float4 *>(xr);
                for (int i = tid; i < (k >> 2); i += kThreads) {
                    float4 v = __ldg(x4 + i);
                    am = fmaxf(am, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                }
            } else {
                for (int i = tid; i < k; i += kThreads) am = fmaxf(am, fabsf(__ldg(xr + i)));
            }
            am = warp_max(am);
            if (lane == 0) s_part[tk * kWarps + warp] = am;
        }
        __syncthreads();
        if (tid < m) {
            float am = 0.0f;
            for (int w = 0; w < kWarps; ++w) am = fmaxf(am, s_part[tid * kWarps + w]);
            s_scale[tid] = __fdiv_rn(127.0f, fmaxf(am, 1e-5f));  // quant.rs:105
        }
        __syncthreads();
        // pass 2: quantise four columns per thread step, accumulate sum(q)
        int *s_parti = reinterpret_cast<int *>(s_part);
        for (int tk = 0; tk < m; ++tk) {
            const float *xr = p.x + static_cast<size_t>(tk) * k;
            const float sc = s_scale[tk];
            uint8_t *dst = s_xq + static_cast<size_t>(tk) * p.xq_stride;
            int acc = 0;
            for (int i = tid * 4; i < kfill; i += kThreads * 4) {
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
                uint32_t word = (q0 & 255) | ((q1 & 255) << 8) | ((q2 & 255) << 16) |
                                (static_cast<uint32_t>(q3 & 255) << 24);
                *reinterpret_cast<uint32_t *>(dst + xq_pos(i)) = word;
            }
            acc = warp_sum(acc);
            if (lane == 0) s_parti[tk * kWarps + warp] = acc;
        }
        __syncthreads();
        if (tid < m) {
            int s = 0;
            for (int w = 0; w < kWarps; ++w) s += s_parti[tid * kWarps + w];
            s_sum[tid] = s;
        }
    } else {
        // already quantised (ternary_gemm_i32 / ternary_gemm_multi entry points): re-order
        const int kp = (k + kBlock - 1) / kBlock * kBlock;
        for (int tk = 0; tk < m; ++tk) {
            const uint32_t *src = reinterpret_cast<const uint32_t *>(p.q + static_cast<size_t>(tk) * kp);
            uint8_t *dst = s_xq + static_cast<size_t>(tk) * p.xq_stride;
            for (int i = tid * 4; i < kfill; i += kThreads * 4)
                *reinterpret_cast<uint32_t *>(dst + xq_pos(i)) = i < kp ? __ldg(src + (i >> 2)) : 0u;
        }
        if (tid < m) {
            s_scale[tid] = p.qscale ? p.qscale[tid] : 1.0f;
            s_sum[tid] = p.qsum[tid];
        }
    }
    __syncthreads();
    if (tid < m * p.n_mat) {
        const int mi = tid / m, tk = tid % m;
        // gemm.rs:141: inv = 1.0 / (x.scale * w.scale)
        s_inv[mi * kMaxM + tk] = __fdiv_rn(1.0f, __fmul_rn(s_scale[tk], p.wscale[mi]));
    }
    __syncthreads();

    if (n_items == 0) return;

    // ---- main loop -----------------------------------------------------------------------
    // Lane (g, t) reads 16-byte units 2t and 2t+1 of rows g and g+8 of the stage: block t of
    // the chunk's four blocks, bytes 0..15 and 16..31. The 128B swizzle (unit ^= row & 7)
    // spreads the eight lanes of a quarter warp over all banks.
    const uint32_t offA = g * 128 + (((2 * t) ^ g) << 4);
    const uint32_t offB = g * 128 + (((2 * t + 1) ^ g) << 4);
    const uint8_t *xrow[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        int tok = mt * 8 + g;
        tok = tok < m ? tok : m - 1;  // lanes beyond the last token re-read it; never stored
        xrow[mt] = s_xq + static_cast<size_t>(tok) * p.xq_stride + t * 8;
    }
    const uint8_t *stage_ptr = sm + L.stages + warp * (kStages * kStageBytes);

    int acc[MT][4][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[mt][kk][j] = 0;

    int tile = tile_begin, chunk = 0, mat = 0;
    int s = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int item = 0; item < n_items; ++item) {
        if (!ptx::mbar_wait(bar0 + s * 8, phase, kWaitLimit)) {
            ok = false;
            break;
        }
        const uint8_t *st = stage_ptr + s * kStageBytes;
        const uint4 W0 = *reinterpret_cast<const uint4 *>(st + offA);
        const uint4 W1 = *reinterpret_cast<const uint4 *>(st + offB);
        const uint4 V0 = *reinterpret_cast<const uint4 *>(st + 1024 + offA);
        const uint4 V1 = *reinterpret_cast<const uint4 *>(st + 1024 + offB);
        const uint32_t wlo[4] = {W0.x, W0.z, W1.x, W1.z};  // row g,   first word of pair c
        const uint32_t whi[4] = {W0.y, W0.w, W1.y, W1.w};  // row g,   second word
        const uint32_t vlo[4] = {V0.x, V0.z, V1.x, V1.z};  // row g+8
        const uint32_t vhi[4] = {V0.y, V0.w, V1.y, V1.w};
        const uint32_t xoff = static_cast<uint32_t>(chunk) * kChunkCols;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const uint32_t mask = 0x03030303u << (2 * kk);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t a0 = wlo[c] & mask, a1 = vlo[c] & mask;
                const uint32_t a2 = whi[c] & mask, a3 = vhi[c] & mask;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint2 b = *reinterpret_cast<const uint2 *>(xrow[mt] + xoff + ((kk * 4 + c) << 5));
                    ptx::mma_u8s8(acc[mt][kk], a0, a1, a2, a3, b.x, b.y);
                }
            }
        }
        __syncwarp();  // every lane has read the stage before it is refilled
        if (lane == 0 && item + kStages < n_items) issue(s);
        if (++s == kStages) {
            s = 0;
            phase ^= 1;
        }

        if (++chunk == chunks) {
            // ---- tile epilogue -----------------------------------------------------------
            while (mat < p.n_mat - 1 && tile >= p.tile_end[mat]) ++mat;
            const int row0 = (tile - (mat ? p.tile_end[mat - 1] : 0)) * kTileRows;
            const int rows = p.rows[mat];
            float *out = p.out[mat];
            int32_t *iout = p.iout[mat];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int v = acc[mt][0][j] + (acc[mt][1][j] >> 2) + (acc[mt][2][j] >> 4) +
                                  (acc[mt][3][j] >> 6);
                    const int row = row0 + g + ((j & 2) ? 8 : 0);
                    const int tok = mt * 8 + 2 * t + (j & 1);
                    if (row < rows && tok < m) {
                        const int d = v - s_sum[tok];  // gemm.rs:306-308
                        const size_t o = static_cast<size_t>(tok) * rows + row;
                        if (iout) iout[o] = d;
                        if (out) out[o] = __fmul_rn(__int2float_rn(d), s_inv[mat * kMaxM + tok]);
                    }
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) acc[mt][kk][j] = 0;
                }
            chunk = 0;
            ++tile;
        }
    }
    if (!ok && lane == 0) atomicExch(p.err_word, 1);
}

}  // namespace

static int xq_stride_for(size_t kp) {
    const size_t chunks = (kp / 4 + kChunkBytes - 1) / kChunkBytes;
    return static_cast<int>(chunks * kChunkCols + 32);  // +32: token rows land on distinct banks
}

bool gemv_fits(const Ctx *ctx, size_t kp, size_t m) {
    if (m == 0 || m > kMaxM) return false;
    const SmemLayout L = smem_layout(static_cast<int>(m), xq_stride_for(kp));
    return static_cast<size_t>(L.total) + 1024 <= ctx->smem_optin;
}

int gemv_init(Ctx *ctx) {
    const int smem = static_cast<int>(ctx->smem_optin);
    LBK_CUDA(cudaFuncSetAttribute(gemv_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    LBK_CUDA(cudaFuncSetAttribute(gemv_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    return LBK_OK;
}

int launch_gemv(Ctx *ctx, const GroupArgs &g, cudaStream_t stream) {
    if (g.n < 1 || g.n > LBK_MAX_GROUP) return fail(LBK_ERR_INVALID, "group size %d not in 1..%d", g.n, LBK_MAX_GROUP);
    if (g.m < 1 || g.m > kMaxM) return fail(LBK_ERR_UNSUPPORTED, "gemv kernel serves 1..%d token rows, got %zu", kMaxM, g.m);
    GemvParams p{};
    const size_t cols = g.w[0]->cols, kp = g.w[0]->kp;
    int tiles = 0;
    for (int i = 0; i < g.n; ++i) {
        const Weight *w = g.w[i];
        if (w->cols != cols) return fail(LBK_ERR_SHAPE, "inner dimension mismatch: %zu vs %zu", w->cols, cols);
        p.tmap[i] = w->tmap_gemv;
        p.out[i] = g.out[i];
        p.iout[i] = g.iout[i];
        p.wscale[i] = w->scale;
        p.rows[i] = static_cast<int>(w->rows);
        tiles += static_cast<int>((w->rows + kTileRows - 1) / kTileRows);
        p.tile_end[i] = tiles;
    }
    p.n_mat = g.n;
    p.m = static_cast<int>(g.m);
    p.k = static_cast<int>(cols);
    p.chunks = static_cast<int>((kp / 4 + kChunkBytes - 1) / kChunkBytes);
    p.xq_stride = xq_stride_for(kp);
    p.total_tiles = tiles;
    p.x = g.x;
    p.q = g.q;
    p.qscale = g.qscale;
    p.qsum = g.qsum;
    p.err_word = ctx->err_word;
    if (tiles == 0) return LBK_OK;

    const SmemLayout L = smem_layout(p.m, p.xq_stride);
    const size_t smem = static_cast<size_t>(L.total) + 1024;
    if (smem > ctx->smem_optin)
        return fail(LBK_ERR_UNSUPPORTED, "gemv: %zu token rows of %zu columns need %zu B of shared memory (limit %zu)",
                    g.m, cols, smem, ctx->smem_optin);
    const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    if (p.m <= 8)
        gemv_kernel<1><<<grid, kThreads, smem, stream>>>(p);
    else
        gemv_kernel<2><<<grid, kThreads, smem, stream>>>(p);
    LBK_CUDA(cudaGetLastError());
    ctx->launches++;
    return LBK_OK;
}

}  // namespace lbk
