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
#include "lbk_gemv_core.cuh"

namespace lbk {

using namespace gemv;

namespace {

// Field order matters: kernel parameters sit in constant memory and every 64-byte line of them is a
// cold miss at kernel start (about 300 ns each, serialised where one value decides the next load).
// Everything the set-up needs comes first, in two lines; the tensor maps, which only the TMA unit
// reads, come last.
struct GemvParams {
    int n_mat;
    int m;
    int k;         // logical columns
    int chunks;    // ceil(row_bytes / 128)
    int xq_stride; // bytes between token rows of the quantised activations in shared memory
    int total_tiles;
    int split;             // 1: a CTA's warps share its tiles chunk by chunk and add up in shared memory
    int acc_tiles;         // tiles per CTA at most (size of that shared-memory area)
    const float *x;        // f32 [m, k], or null when q is given
    const int8_t *q;       // int8 [m, kp]
    const float *qscale;   // f32 [m]
    const int32_t *qsum;   // i32 [m]
    int pre;               // LBK_PRE_*: transform of x before the quantiser (register-cached rows only)
    float pre_eps;
    const float *pre_y;
    const float *pre_w;
    float *pre_xout;
    int *err_word;
    int tile_end[LBK_MAX_GROUP];  // running count of 16-row tiles up to and including matrix i
    int rows[LBK_MAX_GROUP];
    float wscale[LBK_MAX_GROUP];
    float *out[LBK_MAX_GROUP];
    int32_t *iout[LBK_MAX_GROUP];
    alignas(64) CUtensorMap tmap[LBK_MAX_GROUP];
};

// Shared-memory carve-up (offsets from a 1024-byte aligned base).
struct SmemLayout {
    uint32_t stages;   // kWarps * kStages * kStageBytes
    uint32_t full;     // kWarps * kStages mbarriers: stage filled (TMA complete_tx)
    uint32_t part;     // f32 [kMaxM][kWarps] partial maxima
    uint32_t parti;    // i32 [kMaxM][kWarps] partial sums
    uint32_t scale;    // f32 [kMaxM]
    uint32_t sum;      // i32 [kMaxM]
    uint32_t inv;      // f32 [LBK_MAX_GROUP][kMaxM]
    uint32_t xq;       // m * xq_stride
    uint32_t acc;      // i32 [acc_tiles][MT][128]: sums of tiles whose chunks are spread over several warps
    uint32_t total;
};

__host__ __device__ inline SmemLayout smem_layout(int m, int xq_stride, int acc_tiles = 0) {
    SmemLayout L;
    uint32_t o = 0;
    L.stages = o; o += kWarps * kStages * kStageBytes;
    L.full = o;   o += kWarps * kStages * 8;
    L.part = o;   o += kMaxM * kWarps * 4;
    L.parti = o;  o += kMaxM * kWarps * 4;
    L.scale = o;  o += kMaxM * 4;
    L.sum = o;    o += kMaxM * 4;
    L.inv = o;    o += LBK_MAX_GROUP * kMaxM * 4;
    o = (o + 127u) & ~127u;
    L.xq = o;     o += static_cast<uint32_t>(m) * static_cast<uint32_t>(xq_stride);
    o = (o + 15u) & ~15u;
    L.acc = o;    o += static_cast<uint32_t>(acc_tiles) * (m > 8 ? 2u : 1u) * 128u * 4u;
    L.total = o;
    return L;
}

// Every warp owns a contiguous run of 16-row tiles and a ring of kStages TMA stages that its
// lane 0 keeps full; the main loop never synchronises across warps.
template <int MT>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const SmemLayout L = smem_layout(p.m, p.xq_stride, p.split ? p.acc_tiles : 0);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int chunks = p.chunks;
    ptx::pdl_trigger();  // the kernel after this one may be scheduled; it orders itself with pdl_wait

    // ---- this warp's run --------------------------------------------------------------------
    // Whole tiles per warp when every warp has several; otherwise (the decode shapes: 160..864
    // tiles for 2368 warps) a CTA takes a contiguous range of tiles and its 16 warps share the
    // range's stages (tile x chunk) equally, so that a tile of 14 chunks is streamed by up to 14
    // warps at once instead of by one warp in 14 turns. Partial sums meet in shared memory.
    const long long gw = static_cast<long long>(blockIdx.x) * kWarps + warp;
    const long long nw = static_cast<long long>(gridDim.x) * kWarps;
    int tile_begin, chunk_begin, n_items, cta_tile0 = 0, cta_stages = 0;
    if (p.split) {
        cta_tile0 = static_cast<int>(static_cast<long long>(blockIdx.x) * p.total_tiles / gridDim.x);
        const int cta_tile1 = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * p.total_tiles / gridDim.x);
        cta_stages = (cta_tile1 - cta_tile0) * chunks;
        const int s0 = cta_stages * warp / kWarps, s1 = cta_stages * (warp + 1) / kWarps;
        tile_begin = cta_tile0 + s0 / chunks;
        chunk_begin = s0 % chunks;
        n_items = s1 - s0;
    } else {
        tile_begin = static_cast<int>(gw * p.total_tiles / nw);
        const int tile_end = static_cast<int>((gw + 1) * p.total_tiles / nw);
        chunk_begin = 0;
        n_items = (tile_end - tile_begin) * chunks;
    }
    const uint32_t stage0 = base + L.stages + warp * (kStages * kStageBytes);
    const uint32_t full0 = base + L.full + warp * (kStages * 8);

    // issue cursor (lane 0 only): next item to fetch
    int issue_tile = tile_begin, issue_chunk = chunk_begin, issue_mat = 0;
    const uint64_t stream_once = ptx::policy_evict_first();  // weights are read once per launch
    auto issue = [&](int s) {  // s: the ring stage the next item goes into
        while (issue_mat < p.n_mat - 1 && issue_tile >= p.tile_end[issue_mat]) ++issue_mat;
        const int tile_in_mat = issue_tile - (issue_mat ? p.tile_end[issue_mat - 1] : 0);
        ptx::mbar_arrive_expect_tx(full0 + s * 8, kStageBytes);
        ptx::tma_load_2d_hint(stage0 + s * kStageBytes, &p.tmap[issue_mat], full0 + s * 8,
                         issue_chunk * kChunkBytes, tile_in_mat * kTileRows, stream_once);
        if (++issue_chunk == chunks) {
            issue_chunk = 0;
            ++issue_tile;
        }
    };
    // The activation row loads are issued before lane 0 sets up the ring, so that both latency
    // chains (row from L2, first TMA issues) run side by side. P warps share a token row;
    // kWarps/P rows are in flight at once.
    const int m = p.m, k = p.k;
    const int P = m > 8 ? 1 : (m > 4 ? 2 : (m > 2 ? 4 : (m > 1 ? 8 : 16)));
    const int rows_at_once = kWarps / P;
    const int sub = warp % P, slot = warp / P;
    const int idx = sub * 32 + lane, nthr = P * 32;
    const bool vec = (k & 3) == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15) == 0;
    const bool cached = p.x != nullptr && vec && ((k >> 2) + nthr - 1) / nthr <= kCacheV && m <= rows_at_once;
    // Weights do not depend on the kernel before this one, activations do: set up the ring and
    // start the first weight loads, THEN wait for the predecessor (a chained launch overlaps all of
    // this with its tail), then read the activation rows.
    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) ptx::mbar_init(full0 + s * 8, 1);
        ptx::fence_barrier_init();
        const int first = n_items < kStages ? n_items : kStages;
        for (int i = 0; i < first; ++i) issue(i);
    }
    ptx::pdl_wait();
    RowCache rc;
    if (cached && slot < m) load_cached(p.x + static_cast<size_t>(slot) * k, k, idx, nthr, rc);
    // input transform (decoder step): second operand and norm weights, loaded alongside the row
    RowCache rc_y, rc_w;
    if (p.pre != 0 && cached && slot < m) {
        load_cached(p.pre_w, k, idx, nthr, rc_w);
        if (p.pre != LBK_PRE_RMS) load_cached(p.pre_y + static_cast<size_t>(slot) * k, k, idx, nthr, rc_y);
    }

    // ---- prologue: quantised activations into shared memory (overlaps the first loads) -----
    float *s_part = reinterpret_cast<float *>(sm + L.part);
    int *s_parti = reinterpret_cast<int *>(sm + L.parti);
    float *s_scale = reinterpret_cast<float *>(sm + L.scale);
    int *s_sum = reinterpret_cast<int *>(sm + L.sum);
    float *s_inv = reinterpret_cast<float *>(sm + L.inv);
    uint8_t *s_xq = sm + L.xq;
    const int kfill = chunks * kChunkCols;  // columns held per token row (zero padded)
    int *s_acc = reinterpret_cast<int *>(sm + L.acc);
    if (p.split)
        for (int i = tid; i < p.acc_tiles * MT * 128; i += kThreads) s_acc[i] = 0;  // published by the barriers below

    if (p.x != nullptr) {
        if (cached) {
            // one row per warp group, read once and kept in registers across the reduction
            const bool have = slot < m;
            if (p.pre != 0) {
                // residual add / gate, then RMS norm with weights (model.rs:85-98,331-366), all on the
                // registers that hold the row; the sum of squares is reduced like the maximum below
                if (have) {
                    float ss = 0.0f;
#pragma unroll
                    for (int j = 0; j < kCacheV; ++j) {
                        float4 v = rc.v[j];
                        const float4 y = rc_y.v[j];
                        if (p.pre == LBK_PRE_ADD_RMS) {
                            v.x += y.x; v.y += y.y; v.z += y.z; v.w += y.w;
                            const int i = idx + j * nthr;
                            if (blockIdx.x == 0 && i < (k >> 2))
                                reinterpret_cast<float4 *>(p.pre_xout + static_cast<size_t>(slot) * k)[i] = v;
                        } else if (p.pre == LBK_PRE_RELU2_MUL_RMS) {
                            const float a = fmaxf(v.x, 0.f), b = fmaxf(v.y, 0.f), c = fmaxf(v.z, 0.f), d = fmaxf(v.w, 0.f);
                            v = make_float4(a * a * y.x, b * b * y.y, c * c * y.z, d * d * y.w);
                        }
                        rc.v[j] = v;
                        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    if (lane == 0) s_part[slot * kWarps + sub] = ss;
                }
                __syncthreads();
                if (have) {
                    float ss = 0.0f;
                    for (int w = 0; w < P; ++w) ss += s_part[slot * kWarps + w];
                    const float r = 1.0f / sqrtf(ss / static_cast<float>(k) + p.pre_eps);
#pragma unroll
                    for (int j = 0; j < kCacheV; ++j) {
                        const float4 w4 = rc_w.v[j];
                        rc.v[j] = make_float4(rc.v[j].x * r * w4.x, rc.v[j].y * r * w4.y, rc.v[j].z * r * w4.z, rc.v[j].w * r * w4.w);
                    }
                }
                __syncthreads();  // s_part is reused for the maxima
            }
            if (have) {
                const float am = warp_max(max_cached(rc));
                if (lane == 0) s_part[slot * kWarps + sub] = am;
            }
            __syncthreads();
            if (have) {
                float am = 0.0f;
                for (int w = 0; w < P; ++w) am = fmaxf(am, s_part[slot * kWarps + w]);
                const float sc = __fdiv_rn(127.0f, fmaxf(am, 1e-5f));  // quant.rs:105
                uint8_t *dst = s_xq + static_cast<size_t>(slot) * p.xq_stride;
                int acc = quantize_cached(rc, kfill, sc, dst, idx, nthr);
                zero_tail(dst, nthr * kCacheV * 4, kfill, idx, nthr);
                acc = warp_sum(acc);
                if (lane == 0) {
                    s_parti[slot * kWarps + sub] = acc;
                    if (sub == 0) s_scale[slot] = sc;
                }
            }
        } else {
            // a warp serves at most two rows: tk = slot and slot + rows_at_once
#pragma unroll
            for (int r = 0; r < 2; ++r) {  // quant.rs:101-104
                const int tk = slot + r * rows_at_once;
                if (tk < m) {
                    float am = warp_max(absmax_span(p.x + static_cast<size_t>(tk) * k, k, vec, idx, nthr));
                    if (lane == 0) s_part[tk * kWarps + sub] = am;
                }
            }
            __syncthreads();
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int tk = slot + r * rows_at_once;
                if (tk < m) {
                    float am = 0.0f;
                    for (int w = 0; w < P; ++w) am = fmaxf(am, s_part[tk * kWarps + w]);
                    const float sc = __fdiv_rn(127.0f, fmaxf(am, 1e-5f));  // quant.rs:105
                    int acc = quantize_span(p.x + static_cast<size_t>(tk) * k, k, kfill, vec, sc,
                                            s_xq + static_cast<size_t>(tk) * p.xq_stride, idx, nthr);
                    acc = warp_sum(acc);
                    if (lane == 0) {
                        s_parti[tk * kWarps + sub] = acc;
                        if (sub == 0) s_scale[tk] = sc;
                    }
                }
            }
        }
        __syncthreads();
        if (tid >= 32 && tid < 32 + m) {  // a different warp from the one that writes s_inv below: both run at once
            const int tk = tid - 32;
            int s = 0;
            for (int w = 0; w < P; ++w) s += s_parti[tk * kWarps + w];
            s_sum[tk] = s;
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
        __syncthreads();  // s_scale of this branch is written right above
    }
    if (tid < m * p.n_mat) {
        const int mi = tid / m, tk = tid % m;
        // gemm.rs:141: inv = 1.0 / (x.scale * w.scale)
        s_inv[mi * kMaxM + tk] = __fdiv_rn(1.0f, __fmul_rn(s_scale[tk], p.wscale[mi]));
    }
    __syncthreads();

    if (n_items == 0 && !p.split) return;

    // ---- main loop -----------------------------------------------------------------------
    const LaneOffsets off = lane_offsets(lane);
    const uint8_t *xrow[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        int tok = mt * 8 + g;
        tok = tok < m ? tok : m - 1;  // lanes beyond the last token re-read it; never stored
        xrow[mt] = s_xq + static_cast<size_t>(tok) * p.xq_stride + t * 16;
    }
    const uint8_t *stage_ptr = sm + L.stages + warp * (kStages * kStageBytes);

    int acc[MT][2][4][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[mt][h][kk][j] = 0;

    int tile = tile_begin, chunk = chunk_begin, mat = 0;
    int s = 0;
    uint32_t phase = 0;
    bool ok = true;
    // dot = acc - sum(q) (gemm.rs:306-308), y = (float)dot * inv (gemm.rs:141) for one 16-row tile;
    // v(mt, j) gives the complete sum of element j of token group mt
    auto write_tile = [&](int tile_id, auto &&v) {
        while (mat < p.n_mat - 1 && tile_id >= p.tile_end[mat]) ++mat;
        const int row0 = (tile_id - (mat ? p.tile_end[mat - 1] : 0)) * kTileRows;
        const int rows = p.rows[mat];
        float *out = p.out[mat];
        int32_t *iout = p.iout[mat];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int val = v(mt, j);
                const int row = row0 + g + ((j & 2) ? 8 : 0);
                const int tok = mt * 8 + 2 * t + (j & 1);
                if (row < rows && tok < m) {
                    const int d = val - s_sum[tok];
                    const size_t o = static_cast<size_t>(tok) * rows + row;
                    if (iout) iout[o] = d;
                    if (out) out[o] = __fmul_rn(__int2float_rn(d), s_inv[mat * kMaxM + tok]);
                }
            }
    };
    int first_chunk = chunk_begin;  // chunk at which this warp entered the current tile
    for (int item = 0; item < n_items; ++item) {
        if (!ptx::mbar_wait(full0 + s * 8, phase, kWaitLimit)) {
            ok = false;
            break;
        }
        consume_stage<MT>(stage_ptr + s * kStageBytes, off, xrow, static_cast<uint32_t>(chunk) * kChunkCols, acc);
        __syncwarp();  // every lane has read the stage before it is refilled
        if (lane == 0 && item + kStages < n_items) issue(s);
        if (++s == kStages) {
            s = 0;
            phase ^= 1;
        }
        const bool tile_done = ++chunk == chunks;
        if (tile_done || item + 1 == n_items) {
            if (tile_done && first_chunk == 0) {
                // this warp streamed the whole tile: write it out directly
                write_tile(tile, [&](int mt, int j) { return take_acc<MT>(acc, mt, j); });
            } else {
                // part of a tile: add this warp's sums to the tile's record in shared memory
                int *rec = s_acc + (static_cast<size_t>(tile - cta_tile0) * MT) * 128 + lane * 4;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int j = 0; j < 4; ++j) atomicAdd(rec + mt * 128 + j, take_acc<MT>(acc, mt, j));
            }
            if (tile_done) {
                chunk = 0;
                first_chunk = 0;
                ++tile;
            }
        }
    }
    if (p.split) {
        __syncthreads();  // every warp's partial sums are in shared memory
        if (ok && cta_stages > 0) {
            // tiles that no single warp streamed alone: warp w finishes local tiles w, w + 16, ...
            const int n_local = cta_stages / chunks;
            auto owner = [&](int stage) {  // the warp whose run [S*w/16, S*(w+1)/16) holds `stage`
                int w = static_cast<int>(static_cast<long long>(stage) * kWarps / cta_stages);
                while (w + 1 < kWarps && cta_stages * (w + 1) / kWarps <= stage) ++w;
                while (w > 0 && cta_stages * w / kWarps > stage) --w;
                return w;
            };
            mat = 0;
            for (int tl = warp; tl < n_local; tl += kWarps) {
                if (owner(tl * chunks) == owner(tl * chunks + chunks - 1)) continue;  // written directly above
                const int *rec = s_acc + (static_cast<size_t>(tl) * MT) * 128 + lane * 4;
                write_tile(cta_tile0 + tl, [&](int mt, int j) { return rec[mt * 128 + j]; });
            }
        }
    }
    if (!ok && lane == 0) atomicExch(p.err_word, 1);
}

}  // namespace


int gemv_xq_stride(size_t kp) {
    const size_t chunks = (kp / 4 + kChunkBytes - 1) / kChunkBytes;
    return static_cast<int>(chunks * kChunkCols + 64);  // +64: the 128-bit loads of two token rows land on distinct banks
}

// The transform runs where a token row is read once into registers: same conditions as `cached`
// in the kernel (16-byte aligned rows are the caller's business and checked there).
bool gemv_pre_supported(size_t m, size_t cols) {
    if (m == 0 || m > kMaxM || (cols & 3)) return false;
    const size_t P = m > 8 ? 1 : (m > 4 ? 2 : (m > 2 ? 4 : (m > 1 ? 8 : 16)));
    const size_t nthr = P * 32;
    return (cols / 4 + nthr - 1) / nthr <= static_cast<size_t>(kCacheV) && m <= kWarps / P;
}

bool gemv_fits(const Ctx *ctx, size_t kp, size_t m) {
    if (m == 0 || m > kMaxM) return false;
    const SmemLayout L = smem_layout(static_cast<int>(m), gemv_xq_stride(kp));
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
    p.xq_stride = gemv_xq_stride(kp);
    p.total_tiles = tiles;
    p.x = g.x;
    p.q = g.q;
    p.qscale = g.qscale;
    p.qsum = g.qsum;
    p.err_word = ctx->err_word;
    p.pre = g.pre;
    p.pre_y = g.pre_y;
    p.pre_w = g.pre_w;
    p.pre_xout = g.pre_xout;
    p.pre_eps = g.pre_eps;
    if (g.pre != 0 && !(g.x && gemv_pre_supported(g.m, cols)))
        return fail(LBK_ERR_UNSUPPORTED, "input transform: %zu token rows of %zu columns are not held in registers by the decode kernel", g.m, cols);
    if (tiles == 0) return LBK_OK;

    // few tiles per warp: let the 16 warps of a CTA share its tiles chunk by chunk
    const int grid_for = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    const int tiles_per_cta = (tiles + grid_for - 1) / grid_for;
    p.split = tiles_per_cta <= 32 && tiles < 4 * ctx->sm_count * kWarps ? 1 : 0;
    p.acc_tiles = p.split ? tiles_per_cta : 0;
    SmemLayout L = smem_layout(p.m, p.xq_stride, p.acc_tiles);
    if (p.split && static_cast<size_t>(L.total) + 1024 > ctx->smem_optin) {
        p.split = 0;
        p.acc_tiles = 0;
        L = smem_layout(p.m, p.xq_stride, 0);
    }
    const size_t smem = static_cast<size_t>(L.total) + 1024;
    if (smem > ctx->smem_optin)
        return fail(LBK_ERR_UNSUPPORTED, "gemv: %zu token rows of %zu columns need %zu B of shared memory (limit %zu)",
                    g.m, cols, smem, ctx->smem_optin);
    const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    if (p.m <= 8)
        LBK_CUDA(launch_chained(gemv_kernel<1>, dim3(grid), dim3(kThreads), smem, stream, p));
    else
        LBK_CUDA(launch_chained(gemv_kernel<2>, dim3(grid), dim3(kThreads), smem, stream, p));
    LBK_CUDA(cudaGetLastError());
    ctx->launches++;
    return LBK_OK;
}

}  // namespace lbk
