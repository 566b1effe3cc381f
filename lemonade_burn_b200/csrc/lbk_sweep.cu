// Persistent decode sweep: a whole recorded sequence of fused ternary-linear groups (one token
// row each) in ONE launch.
//
// Stands in for the reference's per-token loop of 120 parallel regions
// (crates/lb-ternary/benches/kbench.rs:148-194; crates/lb-model/src/model.rs:331-366 issues the
// same four fused ops per layer). The concatenated weight stream of all groups, counted in
// 2 KB stages ([16 rows][128 B] boxes), is cut into runs of EQUAL stage count, one run per warp
// (148 CTAs x 16 warps), each walked with the warp's own TMA ring. A cut may fall inside a
// 16-row tile: the two warps that share such a tile each leave their int32 partial sums in a
// small workspace and bump a counter; whichever arrives second adds the two and writes the
// outputs. Nobody waits for anybody. The activation rows of the groups a CTA touches are
// quantised once per CTA into shared memory. Groups must not depend on each other's outputs.
// Arithmetic per output element is exactly that of the single-group kernel (integer partial
// sums add exactly).
#include <vector>

#include "lbk_gemv_core.cuh"

namespace lbk {

using namespace gemv;

#ifndef LBK_SWEEP_STAGES
#define LBK_SWEEP_STAGES 3
#endif
constexpr int kSweepStages = LBK_SWEEP_STAGES;  // TMA ring depth per warp in this kernel
constexpr int kHandoffInts = 64;  // [0,16) first half's partials, [16,32) second half's, [32] arrivals
constexpr int kMaxSlots = 4;  // groups one CTA's warps may touch (activation slots in shared memory)

struct alignas(64) SweepMat {
    CUtensorMap tmap;
    float *out;
    int32_t *iout;
    float wscale;
    int rows;
    int pad_[10];
};

struct alignas(16) SweepGroup {
    const float *x;
    int k;
    int chunks;
    int n_mat;
    int mat0;                      // index of the group's first SweepMat
    int tile0;                     // global index of the group's first tile
    int tiles;
    int tile_end[LBK_MAX_GROUP];   // running count of 16-row tiles up to and including matrix i
};

// What a CTA needs to quantise one activation row, in one 16-byte load.
struct alignas(16) SlotRec {
    const float *x;
    int k;
    int chunks;
};

struct alignas(16) CtaRec {
    int group0;   // first group the CTA's warps touch
    int n_slots;  // how many groups they touch (<= kMaxSlots)
    int pad_[2];
    SlotRec slot[kMaxSlots];
};

struct SweepParams {
    const SweepMat *mats;
    const SweepGroup *groups;
    const int4 *warp_run;    // [n_warps] {first tile, stages in the run, group of the first tile, first chunk}
    int *handoff;            // [n_warps + 1][kHandoffInts]: partial sums of tiles shared by two warps
    const CtaRec *cta;       // [grid]
    int xq_bytes;            // bytes per activation slot
    int *err_word;
};

namespace {

// tile_end[i] without dynamic indexing (keeps the group record in registers)
__device__ __forceinline__ int tile_end_of(const SweepGroup &g, int i) {
    return i == 0 ? g.tile_end[0] : (i == 1 ? g.tile_end[1] : (i == 2 ? g.tile_end[2] : g.tile_end[3]));
}

static_assert(sizeof(SweepGroup) == 48, "SweepGroup is read as three 16-byte words");
__device__ __forceinline__ SweepGroup load_group(const SweepGroup *g, uint64_t policy) {
    union {
        SweepGroup grp;
        uint4 w[3];
    } u;
#pragma unroll
    for (int i = 0; i < 3; ++i) u.w[i] = ptx::ldg_hint(reinterpret_cast<const uint4 *>(g) + i, policy);
    return u.grp;
}

// Every warp walks its own run of tiles; its lane 0 keeps the warp's TMA ring full. The
// activation rows of the (at most kMaxSlots) groups the CTA touches are quantised once, by the
// whole CTA, while the first loads are in flight.
__global__ void __launch_bounds__(kThreads, 1) sweep_kernel(const SweepParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int gw = blockIdx.x * kWarps + warp;
    // The tables and activation rows are read again by the next launch while half a gigabyte of
    // weights streams through L2 in between: ask L2 to keep the former and drop the latter first.
    const uint64_t keep = ptx::policy_evict_last(), stream_once = ptx::policy_evict_first();
    const uint4 run_u = ptx::ldg_hint(p.warp_run + gw, keep);
    const int4 run = make_int4(run_u.x, run_u.y, run_u.z, run_u.w);
    const int t_begin = run.x, n_stages = run.y, c_begin = run.w;
    const uint4 chead_u = ptx::ldg_hint(p.cta + blockIdx.x, keep);
    const int4 chead = make_int4(chead_u.x, chead_u.y, chead_u.z, chead_u.w);
    const int slot_g0 = chead.x, n_slots = chead.y;

    // Two chains of dependent loads start here and are interleaved on purpose: (a) this warp
    // group's activation row (slot record -> row), (b) lane 0's first TMA loads (group record ->
    // tensor map). The row loads are issued first and consumed after the TMA issue.
    const int q_slot = warp >> 2, q_sub = warp & 3;
    const int q_idx = q_sub * 32 + lane;
    constexpr int q_nthr = 128;
    const bool q_have = q_slot < n_slots;
    const float *q_x = nullptr;
    int q_k = 0, q_kfill = 0;
    bool q_vec = false, q_cached = false;
    RowCache rc;
    if (q_have) {
        const uint4 rec_u = ptx::ldg_hint(&p.cta[blockIdx.x].slot[q_slot], keep);
        const int4 rec = make_int4(rec_u.x, rec_u.y, rec_u.z, rec_u.w);
        q_x = reinterpret_cast<const float *>((static_cast<unsigned long long>(static_cast<unsigned>(rec.y)) << 32) |
                                              static_cast<unsigned>(rec.x));
        q_k = rec.z;
        q_kfill = rec.w * kChunkCols;
        q_vec = (q_k & 3) == 0 && (reinterpret_cast<uintptr_t>(q_x) & 15) == 0;
        q_cached = q_vec && ((q_k >> 2) + q_nthr - 1) / q_nthr <= kCacheV;
        if (q_cached) load_cached_hint(q_x, q_k, q_idx, q_nthr, rc, keep);
    }

    constexpr uint32_t kRing = kSweepStages * kStageBytes;
    const uint32_t stage0 = base + warp * kRing;
    const uint8_t *stage_ptr = sm + warp * kRing;
    const uint32_t full0 = base + kWarps * kRing + warp * (kSweepStages * 8);
    uint8_t *s_misc = sm + kWarps * kRing + kWarps * kSweepStages * 8;       // reductions, scales, sums
    float *s_part = reinterpret_cast<float *>(s_misc);                  // [kMaxSlots][4]
    int *s_parti = reinterpret_cast<int *>(s_misc + 64);                // [kMaxSlots][4]
    float *s_scale = reinterpret_cast<float *>(s_misc + 128);           // [kMaxSlots]
    int *s_sum = reinterpret_cast<int *>(s_misc + 144);                 // [kMaxSlots]
    uint8_t *s_xq = s_misc + 256;                                       // [kMaxSlots][xq_bytes]

    // ---- issue cursor (meaningful on lane 0 only): kept incremental so that the common case is
    // the two PTX instructions plus a counter; matrices and groups change on a slow path.
    int ig = run.z;
    SweepGroup igrp = load_group(p.groups + (n_stages > 0 ? ig : 0), keep);
    int ichunk = c_begin, ichunks = igrp.chunks, imat = 0, irow = 0, imat_left = 0, issued = 0;
    const CUtensorMap *itmap = nullptr;
    {
        const int local = t_begin - igrp.tile0;
        while (imat < igrp.n_mat - 1 && local >= tile_end_of(igrp, imat)) ++imat;
        const int mat_base = imat ? tile_end_of(igrp, imat - 1) : 0;
        irow = (local - mat_base) * kTileRows;
        imat_left = tile_end_of(igrp, imat) - local;
        itmap = &p.mats[igrp.mat0 + imat].tmap;
    }
    auto issue = [&](int s) {
        while (imat_left == 0) {  // the previous tile was the last one of its matrix
            if (++imat == igrp.n_mat) {
                igrp = load_group(p.groups + ++ig, keep);
                imat = 0;
                ichunks = igrp.chunks;
            }
            imat_left = tile_end_of(igrp, imat) - (imat ? tile_end_of(igrp, imat - 1) : 0);
            irow = 0;
            itmap = &p.mats[igrp.mat0 + imat].tmap;
        }
        ptx::mbar_arrive_expect_tx(full0 + s * 8, kStageBytes);
        ptx::tma_load_2d_hint(stage0 + s * kStageBytes, itmap, full0 + s * 8, ichunk * kChunkBytes, irow, stream_once);
        ++issued;
        if (++ichunk == ichunks) {
            ichunk = 0;
            irow += kTileRows;
            --imat_left;
        }
    };
    if (lane == 0) {
        for (int s = 0; s < kSweepStages; ++s) ptx::mbar_init(full0 + s * 8, 1);
        ptx::fence_barrier_init();
        for (int s = 0; s < kSweepStages && issued < n_stages; ++s) issue(s);
    }

    // ---- CTA prologue: quantise the activation row of every group this CTA touches ----------
    // (quant.rs:100-118). Four warps per slot; rows of up to 4096 columns are read once.
    {
        if (q_have) {
            const float am = warp_max(q_cached ? max_cached(rc) : absmax_span(q_x, q_k, q_vec, q_idx, q_nthr));
            if (lane == 0) s_part[q_slot * 4 + q_sub] = am;
        }
        __syncthreads();
        if (q_have) {
            const float am = fmaxf(fmaxf(s_part[q_slot * 4], s_part[q_slot * 4 + 1]),
                                   fmaxf(s_part[q_slot * 4 + 2], s_part[q_slot * 4 + 3]));
            const float sc = __fdiv_rn(127.0f, fmaxf(am, 1e-5f));
            uint8_t *dst = s_xq + static_cast<size_t>(q_slot) * p.xq_bytes;
            int acc;
            if (q_cached) {
                acc = quantize_cached(rc, q_kfill, sc, dst, q_idx, q_nthr);
                zero_tail(dst, q_nthr * kCacheV * 4, q_kfill, q_idx, q_nthr);
            } else {
                acc = quantize_span(q_x, q_k, q_kfill, q_vec, sc, dst, q_idx, q_nthr);
            }
            acc = warp_sum(acc);
            if (lane == 0) {
                s_parti[q_slot * 4 + q_sub] = acc;
                if (q_sub == 0) s_scale[q_slot] = sc;
            }
        }
        __syncthreads();
        if (tid < n_slots) s_sum[tid] = s_parti[tid * 4] + s_parti[tid * 4 + 1] + s_parti[tid * 4 + 2] + s_parti[tid * 4 + 3];
        __syncthreads();
    }
    if (n_stages <= 0) return;

    // ---- consume cursor ----------------------------------------------------------------
    const LaneOffsets off = lane_offsets(lane);
    const uint8_t *xrow[1] = {s_xq + t * 16};
    int acc[1][2][4][4];  // written by the first stage of every tile

    int cg = run.z - 1;  // forces the first group set-up
    SweepGroup cgrp{};
    int cmat = -1, mat_tile_base = 0, mat_tile_end = 0, rows = 0;
    float *out = nullptr;
    int32_t *iout = nullptr;
    float a_scale = 0.0f, inv = 0.0f;
    int a_sum = 0;
    int s = 0, tile = t_begin;
    uint32_t phase = 0;
    bool ok = true;

    // dot = acc - sum(q), y = (float)dot * (1/(s_a*s_w)) for the 16 rows of `tile`; v_lo / v_hi are
    // the complete sums of rows g and g + 8 (meaningful on lanes with t == 0).
    auto write_tile = [&](int v_lo, int v_hi) {
        const int local = tile - cgrp.tile0;
        if (cmat < 0 || local >= mat_tile_end) {
            if (cmat < 0) cmat = 0;
            while (cmat < cgrp.n_mat - 1 && local >= tile_end_of(cgrp, cmat)) ++cmat;
            mat_tile_end = tile_end_of(cgrp, cmat);
            mat_tile_base = cmat ? tile_end_of(cgrp, cmat - 1) : 0;
            const SweepMat *mt = p.mats + cgrp.mat0 + cmat;
            rows = __ldg(&mt->rows);
            out = mt->out;
            iout = mt->iout;
            inv = __fdiv_rn(1.0f, __fmul_rn(a_scale, __ldg(&mt->wscale)));  // gemm.rs:141
        }
        const int row0 = (local - mat_tile_base) * kTileRows;
        if (t == 0) {  // token 0 lives in column 0 of the tile
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = row0 + g + h * 8;
                if (row < rows) {
                    const int d = (h ? v_hi : v_lo) - a_sum;
                    if (iout) iout[row] = d;
                    if (out) out[row] = __fmul_rn(__int2float_rn(d), inv);
                }
            }
        }
    };
    // This warp holds only part of the tile's columns: leave the partial sums for the warp that
    // holds the rest, or, when that warp has been here already, add its sums and finish the tile.
    // `second` tells which half of the record is ours. Both warps write before they count, so the
    // later one always finds the other's numbers; the record is left zeroed for the next launch.
    auto share_tile = [&](int boundary, bool second, int v_lo, int v_hi) {
        int *rec = p.handoff + static_cast<size_t>(boundary) * kHandoffInts;
        const int mine = second ? 16 : 0, theirs = second ? 0 : 16;
        if (t == 0) {
            __stcg(rec + mine + g, v_lo);
            __stcg(rec + mine + 8 + g, v_hi);
            __threadfence();
        }
        __syncwarp();
        int arrived = 0;
        if (lane == 0) arrived = atomicAdd(rec + 32, 1);
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (arrived == 0) return;
        __threadfence();
        int o_lo = 0, o_hi = 0;
        if (t == 0) {
            o_lo = __ldcg(rec + theirs + g);
            o_hi = __ldcg(rec + theirs + 8 + g);
        }
        __syncwarp();
        if (lane == 0) __stcg(rec + 32, 0);
        write_tile(v_lo + o_lo, v_hi + o_hi);
    };

    // One pass of the outer loop per tile (or per part of a tile at either end of the run).
    for (int remaining = n_stages, c0 = c_begin; remaining > 0 && ok; c0 = 0, ++tile) {
        if (tile >= cgrp.tile0 + cgrp.tiles) {
            // ---- the run enters another group: switch to its activation slot
            do {
                cgrp = load_group(p.groups + ++cg, keep);
            } while (tile >= cgrp.tile0 + cgrp.tiles);
            const int slot = cg - slot_g0;
            xrow[0] = s_xq + static_cast<size_t>(slot) * p.xq_bytes + t * 16;
            a_scale = s_scale[slot];
            a_sum = s_sum[slot];
            cmat = -1;
        }
        const int c1 = min(cgrp.chunks, c0 + remaining);
        remaining -= c1 - c0;
        for (int chunk = c0; chunk < c1; ++chunk) {
            if (!ptx::mbar_wait(full0 + s * 8, phase, kWaitLimit)) {
                ok = false;
                break;
            }
            if (chunk == c0) consume_stage<1, true>(stage_ptr + s * kStageBytes, off, xrow, static_cast<uint32_t>(chunk) * kChunkCols, acc);
            else consume_stage<1, false>(stage_ptr + s * kStageBytes, off, xrow, static_cast<uint32_t>(chunk) * kChunkCols, acc);
            __syncwarp();  // every lane has read the stage before it is refilled
            if (lane == 0 && issued < n_stages) issue(s);
            if (++s == kSweepStages) {
                s = 0;
                phase ^= 1;
            }
        }
        if (!ok) break;
        // columns 1..7 of the MMA tile repeat token 0 and are never read
        const int v_lo = read_acc<1>(acc, 0, 0), v_hi = read_acc<1>(acc, 0, 2);
        if (c0 > 0) share_tile(gw, true, v_lo, v_hi);             // the previous warp holds the first columns
        else if (c1 < cgrp.chunks) share_tile(gw + 1, false, v_lo, v_hi);  // the next warp holds the rest
        else write_tile(v_lo, v_hi);
    }
    if (!ok && lane == 0) atomicExch(p.err_word, 2);
}

}  // namespace

// ---- host side: tables and launch ---------------------------------------------------------

struct SweepTables {
    SweepMat *mats = nullptr;
    SweepGroup *groups = nullptr;
    int4 *warp_run = nullptr;
    CtaRec *cta = nullptr;
    int *handoff = nullptr;
    int xq_bytes = 0;
    int grid = 0;
    size_t smem = 0;
};

void sweep_free(SweepTables *t) {
    if (!t) return;
    cudaFree(t->mats);
    cudaFree(t->groups);
    cudaFree(t->warp_run);
    cudaFree(t->cta);
    cudaFree(t->handoff);
    delete t;
}

int sweep_init(Ctx *ctx) {
    LBK_CUDA(cudaFuncSetAttribute(sweep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(ctx->smem_optin)));
    return LBK_OK;
}

// Builds the device tables for `groups` (each with m == 1 and f32 input). Returns
// LBK_ERR_UNSUPPORTED when a group's activation row does not fit the per-warp slice.
int sweep_build(Ctx *ctx, const std::vector<GroupArgs> &groups, SweepTables **out) {
    *out = nullptr;
    std::vector<SweepMat> mats;
    std::vector<SweepGroup> grps;
    std::vector<int> tile_chunks;  // per global tile: stages it costs
    int max_chunks = 0, tiles_total = 0;
    for (const GroupArgs &g : groups) {
        SweepGroup sg{};
        sg.x = g.x;
        sg.k = static_cast<int>(g.w[0]->cols);
        sg.chunks = static_cast<int>((g.w[0]->rb + kChunkBytes - 1) / kChunkBytes);
        sg.n_mat = g.n;
        sg.mat0 = static_cast<int>(mats.size());
        sg.tile0 = tiles_total;
        int t = 0;
        for (int i = 0; i < g.n; ++i) {
            SweepMat sm{};
            sm.tmap = g.w[i]->tmap_gemv;
            sm.out = g.out[i];
            sm.iout = g.iout[i];
            sm.wscale = g.w[i]->scale;
            sm.rows = static_cast<int>(g.w[i]->rows);
            t += static_cast<int>((g.w[i]->rows + kTileRows - 1) / kTileRows);
            sg.tile_end[i] = t;
            mats.push_back(sm);
        }
        sg.tiles = t;
        tiles_total += t;
        for (int i = 0; i < t; ++i) tile_chunks.push_back(sg.chunks);
        if (sg.chunks > max_chunks) max_chunks = sg.chunks;
        if (t > 0 && sg.chunks > 0) grps.push_back(sg);
        else mats.resize(sg.mat0);
    }
    SweepTables *tb = new SweepTables();
    tb->xq_bytes = max_chunks * kChunkCols;
    tb->smem = static_cast<size_t>(kWarps) * (kSweepStages * kStageBytes + kSweepStages * 8) + 256 +
               static_cast<size_t>(kMaxSlots) * tb->xq_bytes + 1024;
    if (tb->smem > ctx->smem_optin) {
        delete tb;
        return fail(LBK_ERR_UNSUPPORTED, "sweep: %d columns per activation row need %zu B of shared memory (limit %zu)",
                    max_chunks * kChunkCols, tb->smem, ctx->smem_optin);
    }
    if (grps.empty()) {
        *out = tb;
        return LBK_OK;
    }
    // Runs of equal stage count: warp w owns stages [total*w/nw, total*(w+1)/nw) of the stream. When
    // the share is short against a tile (tiny plans) cuts are moved to tile boundaries instead, so
    // that no tile is ever shared by more than two warps.
    const int grid = ctx->sm_count;
    const int nw = grid * kWarps;
    std::vector<long long> tile_start(tiles_total + 1);
    tile_start[0] = 0;
    for (int i = 0; i < tiles_total; ++i) tile_start[i + 1] = tile_start[i] + tile_chunks[i];
    const long long total = tile_start[tiles_total];
    const bool split = total / nw >= 2LL * max_chunks;
    std::vector<long long> cut(nw + 1);
    std::vector<int> cut_tile(nw + 1);
    {
        int tile = 0;
        for (int w = 0; w <= nw; ++w) {
            long long c = total * w / nw;
            while (tile < tiles_total && tile_start[tile + 1] <= c) ++tile;
            if (!split && tile < tiles_total && c > tile_start[tile]) c = tile_start[++tile];  // round up to a tile boundary
            if (c < tile_start[tile]) c = tile_start[tile];  // an earlier cut was rounded past this one
            cut[w] = c;
            cut_tile[w] = tile;  // the tile that holds stage c (tiles_total at the very end)
        }
    }
    auto group_of_tile = [&](int tile) {
        size_t lo = 0, hi = grps.size() - 1;
        while (lo < hi) {
            const size_t mid = (lo + hi) / 2;
            if (tile >= grps[mid].tile0 + grps[mid].tiles) lo = mid + 1;
            else hi = mid;
        }
        return static_cast<int>(lo);
    };
    std::vector<int4> runs(nw);
    std::vector<CtaRec> ctas(grid);
    for (int w = 0; w < nw; ++w) {
        const int n = static_cast<int>(cut[w + 1] - cut[w]);
        const int t0 = cut_tile[w] < tiles_total ? cut_tile[w] : tiles_total - 1;
        runs[w] = make_int4(t0, n, group_of_tile(t0), n > 0 ? static_cast<int>(cut[w] - tile_start[t0]) : 0);
    }
    for (int c = 0; c < grid; ++c) {
        // groups between the CTA's first stage and its last one
        const long long s0 = cut[c * kWarps], s1 = cut[(c + 1) * kWarps];
        int n = 0, g0 = 0;
        if (s1 > s0) {
            g0 = group_of_tile(cut_tile[c * kWarps]);
            int last_tile = cut_tile[(c + 1) * kWarps];
            if (last_tile >= tiles_total || tile_start[last_tile] == s1) --last_tile;  // s1 - 1 lies in the tile before
            n = group_of_tile(last_tile) - g0 + 1;
        }
        if (n > kMaxSlots) {
            delete tb;
            return fail(LBK_ERR_UNSUPPORTED, "sweep: a CTA's run spans %d groups (limit %d); groups are too small", n, kMaxSlots);
        }
        CtaRec rec{};
        rec.group0 = g0;
        rec.n_slots = n;
        for (int i = 0; i < n; ++i) {
            rec.slot[i].x = grps[g0 + i].x;
            rec.slot[i].k = grps[g0 + i].k;
            rec.slot[i].chunks = grps[g0 + i].chunks;
        }
        ctas[c] = rec;
    }
    tb->grid = grid;
    cudaError_t e = cudaMalloc(&tb->mats, mats.size() * sizeof(SweepMat));
    if (e == cudaSuccess) e = cudaMalloc(&tb->groups, grps.size() * sizeof(SweepGroup));
    if (e == cudaSuccess) e = cudaMalloc(&tb->warp_run, runs.size() * sizeof(int4));
    if (e == cudaSuccess) e = cudaMalloc(&tb->cta, ctas.size() * sizeof(CtaRec));
    const size_t handoff_bytes = static_cast<size_t>(nw + 1) * kHandoffInts * sizeof(int);
    if (e == cudaSuccess) e = cudaMalloc(&tb->handoff, handoff_bytes);
    if (e == cudaSuccess) e = cudaMemset(tb->handoff, 0, handoff_bytes);
    if (e == cudaSuccess) e = cudaMemcpy(tb->mats, mats.data(), mats.size() * sizeof(SweepMat), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(tb->groups, grps.data(), grps.size() * sizeof(SweepGroup), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(tb->warp_run, runs.data(), runs.size() * sizeof(int4), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(tb->cta, ctas.data(), ctas.size() * sizeof(CtaRec), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        sweep_free(tb);
        return fail(LBK_ERR_CUDA, "sweep tables: %s", cudaGetErrorString(e));
    }
    *out = tb;
    return LBK_OK;
}


int sweep_launch(Ctx *ctx, const SweepTables *tb, cudaStream_t stream) {
    if (!tb || tb->grid == 0) return LBK_OK;
    SweepParams p{};
    p.mats = tb->mats;
    p.groups = tb->groups;
    p.warp_run = tb->warp_run;
    p.cta = tb->cta;
    p.handoff = tb->handoff;
    p.xq_bytes = tb->xq_bytes;
    p.err_word = ctx->err_word;
    sweep_kernel<<<tb->grid, kThreads, tb->smem, stream>>>(p);
    LBK_CUDA(cudaGetLastError());
    ctx->launches++;
    return LBK_OK;
}

}  // namespace lbk
