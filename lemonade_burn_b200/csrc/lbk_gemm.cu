// Prefill GEMM (more than 16 token rows): int8 activations x packed ternary weights on the
// 5th-generation tensor cores (tcgen05.mma kind::i8, accumulators AND the weight operand in TMEM).
//
// Replaces ternary_gemm_multi's prefill branch and the AVX-512 register tile under it
// (crates/lb-ternary/src/gemm.rs:155-194, 245-268, 483-550).
//
// Orientation: the 128 weight rows of a tile are the MMA's M side, NT token rows its N side
// (D[row][token] in TMEM). Per 128-column block of K (one packed 32-byte block per weight row):
//
//   2 TMA threads  int8 activations [NT tok][128 B] (SWIZZLE_128B, the K-major B operand) and
//                  packed weights [128 rows][128 B] (four K blocks a box) into shared-memory rings
//                  of their own
//   2 x 4 expander thread r owns weight row r = TMEM lane r: 32 packed bytes -> 32 words of u8
//   warps          codes, word c = columns 4c..4c+3 = (packed word >> 2k) & 0x03030303; the two
//                  sets of four warps take alternate K blocks (one set alone was the bottleneck)
//                  (pack.rs:10-13: no shuffles), written straight to TMEM with tcgen05.st.
//                  The expanded tile never touches shared memory: expanding into shared memory
//                  cost 112 KB of shared-memory traffic per 512 cycles of MMA and starved the
//                  tensor pipe (measured 27 % of peak).
//   MMA thread     4 x tcgen05.mma (A from TMEM, u8; B from shared memory, s8; K = 32 each);
//                  tcgen05.commit frees the rings / publishes the accumulator
//   4 epilogue     tcgen05.ld, dot = acc - sum(q) (codes are w+1: gemm.rs:6-9,306-308),
//   warps          y = (float)dot * (1/(s_a*s_w)) (gemm.rs:158,178); a warp's 32 lanes are 32
//                  consecutive weight rows, so every store instruction writes 128 contiguous bytes
//
// TMEM columns: two accumulators of NT columns (the epilogue of one tile overlaps the MMAs of the
// next) + a ring of 32-column weight tiles, two hand-off groups deep (4 tiles at NT = 192, 8 at
// NT = 64). Bound: int8 tensor pipe; 2*m*rows*cols ops.
#include "lbk_internal.cuh"
#include "lbk_ptx.cuh"
#include "lbk_tcgen05.cuh"

namespace lbk {

namespace {

constexpr int kBMW = 128;          // weight rows per tile (MMA M, TMEM lanes)
constexpr int kBK = 128;           // columns per stage = one packed block
constexpr int kPackBlocks = 4;      // K-blocks per packed-weight stage: [128 rows][128 B] boxes
constexpr int kPackBytes = kBMW * kBlockBytes * kPackBlocks;  // 16 KB, SWIZZLE_128B
constexpr int kEpiWarps = 4, kExpWarps = 4, kExpSets = 2;
// warps 0-3 epilogue, 4-7 and 8-11 expanders (warp % 4 = the TMEM lane quadrant a warp may touch)
// warp 12 feeds the activation ring, warp 14 the packed-weight ring: two threads, so that the weight
// stream from HBM runs ahead by its own ring's depth whatever the activation ring is waiting for
constexpr int kExpWarp0 = 4, kTmaWarp = 12, kMmaWarp = 13, kPackWarp = 14;
constexpr int kThreads = 15 * 32;
constexpr uint32_t kTmemCols = 512;

template <int NT>  // capacity in token rows per tile (MMA N): 192 or 64; a launch uses nt <= NT
struct Cfg {
    static constexpr int kActBytes = NT * kBK;                  // multiple of 1024 for NT = 192, 64
    static constexpr int kLoadStages = NT == 192 ? 6 : 12;      // activation ring, in K blocks
    static constexpr int kGroup = NT == 192 ? 2 : 4;            // K blocks per hand-off (see kBarFull below)
    static constexpr int kGroupStages = kLoadStages / kGroup;   // activation ring in hand-off units
    static constexpr int kAStages = 2 * kGroup;                 // expanded weight tiles in TMEM (32 columns each): two groups
    // Packed-weight ring, 16 KB a stage. With 64 token rows the weights come straight from HBM (no
    // other token tile shares them through L2) and the ring has to cover the memory latency.
    static constexpr int kPackStages = NT == 192 ? 3 : 8;
    static constexpr uint32_t kPack0 = kLoadStages * kActBytes;
    static constexpr uint32_t kAcc0 = 0, kAcc1 = NT, kA0 = 2 * NT;  // TMEM column map: two accumulators, then the weight tiles
    static_assert(2 * NT + kAStages * 32 <= 512, "TMEM budget");
    static_assert(kGroup == 2 || kGroup == kPackBlocks, "a group is half a packed-weight stage or a whole one");
    // instruction descriptor without N: D s32, A u8 (codes, TMEM), B s8 (activations), K-major, M=128
    static constexpr uint32_t kIdesc = (2u << 4) | (0u << 7) | (1u << 10) | ((kBMW >> 4) << 24);
    static constexpr uint32_t kBars = kPack0 + kPackStages * kPackBytes;
    static constexpr uint32_t kMisc = kBars + 48 * 8;
    static constexpr uint32_t kTok = kMisc + 64;              // per-token sum(q) and 1/(s_a*s_w): 2 x [2][NT]
    static constexpr uint32_t kTotal = kTok + 2 * 2 * NT * 4;
    // Hand-off is by GROUPS of kGroup K blocks. Every barrier wait in the MMA thread drains the
    // tensor pipe for a few hundred cycles whatever the MMA shape (measured: 4 MMAs + one wait per
    // loop turn run at 590 cycles a turn, 8 MMAs + one wait at 900), so a wait has to buy as many
    // MMAs as shared memory and TMEM allow: 2 blocks of 192 token rows, 4 blocks of 64. One "full"
    // barrier per group collects both operands: the activation bytes of its blocks (TMA
    // transaction count) and one arrival from each of the eight expander warps (set 0 expands the
    // group's even blocks, set 1 its odd ones; a warp with no block at the ragged end of K arrives
    // all the same). One "consumed" barrier per group (a single tcgen05.commit) releases the
    // activation stages and, two groups later, the TMEM weight slots.
    static constexpr int kBarFull = 0;                        // [group stages]
    static constexpr int kBarConsumed = kLoadStages;          // [group stages]
    static constexpr int kBarFullPack = 2 * kLoadStages;      // [PS] packed weights landed
    static constexpr int kBarEmptyPack = kBarFullPack + kPackStages;  // [PS] expanders are done with them
    static constexpr int kBarAccFull = kBarEmptyPack + kPackStages;   // [2]
    static constexpr int kBarAccEmpty = kBarAccFull + 2;      // [2]
    static_assert(kBarAccEmpty + 2 <= 48, "barrier area too small");
    static_assert(kTotal + 1024 <= 232448, "shared memory budget");
    static_assert(2 < kGroupStages, "a consumed-barrier phase must still be observable two groups later");
};

struct GemmParams {
    CUtensorMap act;                    // int8 [m][kp], box [NT][128], SWIZZLE_128B
    CUtensorMap wpk[LBK_MAX_GROUP];     // u8 [rows][rb], box [128][128], SWIZZLE_128B
    float *out[LBK_MAX_GROUP];
    int32_t *iout[LBK_MAX_GROUP];
    float wscale[LBK_MAX_GROUP];
    int rows[LBK_MAX_GROUP];
    int tile_end[LBK_MAX_GROUP];        // running tile count up to and including matrix i
    int n_mat, m, m_tiles, k_blocks, total_tiles;
    int nt;                             // token rows per tile in this launch (multiple of 16, <= capacity)
    int ksplit, kb_part;                // every tile's K blocks are cut into ksplit parts of kb_part blocks (a multiple of 4)
    int32_t *acc[LBK_MAX_GROUP];        // ksplit > 1: zeroed int32 [m][rows] that the parts add their sums into
    const float *qscale;
    const int32_t *qsum;
    int *err_word;
    // matrix 0's int32 dots by token owner (see GroupArgs): rows of scatter_mt tokens per owner
    int32_t *scatter[8];
    int scatter_world, scatter_mt;
};

using namespace tc;

// A operand from TMEM (u8 codes), B from shared memory (s8 activations).
// The four K = 32 steps of one 128-column block in one go: A advances 8 TMEM columns and B 32
// bytes (2 descriptor units) per step; only the first step may start a fresh accumulator.
__device__ __forceinline__ void umma_i8_ts_block(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate_first) {
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        ".reg .b64 b1, b2, b3;\n"
        ".reg .b32 a1, a2, a3;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "setp.eq.b32 q, 0, 0;\n"
        "add.u64 b1, %2, 2;\n"
        "add.u64 b2, %2, 4;\n"
        "add.u64 b3, %2, 6;\n"
        "add.u32 a1, %1, 8;\n"
        "add.u32 a2, %1, 16;\n"
        "add.u32 a3, %1, 24;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [a1], b1, %3, q;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [a2], b2, %3, q;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [a3], b3, %3, q;\n"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate_first)
        : "memory");
}
// SC: matrix 0's int32 dots go to the token owners' buffers (GemmParams::scatter) instead of iout: an instantiation of its
// own, so that the ordinary kernel's epilogue keeps its registers
template <int NT, bool SC>
__global__ void __launch_bounds__(kThreads, 1) gemm_kernel(const __grid_constant__ GemmParams p) {
    using C = Cfg<NT>;
    constexpr int G = C::kGroup, PG = C::kGroupStages, PS = C::kPackStages;
    static_assert(kExpSets == 2 && kPackBlocks == 4, "the group hand-off assumes these");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t bar0 = base + C::kBars;
    volatile uint32_t *s_tmem = reinterpret_cast<volatile uint32_t *>(sm + C::kMisc);
    volatile int *s_abort = reinterpret_cast<volatile int *>(sm + C::kMisc + 4);
    auto bar = [&](int idx) { return bar0 + idx * 8; };

    if (tid == 0) {
        for (int i = 0; i < PG; ++i) {
            ptx::mbar_init(bar(C::kBarFull + i), 1 + kExpWarps * kExpSets);
            ptx::mbar_init(bar(C::kBarConsumed + i), 1);
        }
        for (int i = 0; i < PS; ++i) {
            ptx::mbar_init(bar(C::kBarFullPack + i), 1);
            ptx::mbar_init(bar(C::kBarEmptyPack + i), kExpWarps * kExpSets);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(bar(C::kBarAccFull + a), 1);
            ptx::mbar_init(bar(C::kBarAccEmpty + a), kEpiWarps);
        }
        *s_abort = 0;
        ptx::fence_barrier_init();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(base + C::kMisc, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;
    // When the launch was programmatic, everything above overlapped the tail of the kernel before
    // this one (the quantiser that produces this kernel's activations). The roles that read its
    // results or write what it may still read (activation loads, epilogue) wait for it below; the
    // packed weights are constants, and their loads start at once. The kernel behind this one may be
    // scheduled as blocks of this one retire (it orders itself with its own wait).
    ptx::pdl_trigger();

    const int k_blocks = p.k_blocks;
    bool ok = true;
    // tile -> (matrix, weight-row tile, token tile); token tiles vary fastest so that CTAs
    // running side by side share the same packed weights in L2
    auto decode_tile = [&](int tile, int &mat, int &m_tile, int &n_tile) {
        mat = 0;
        while (mat < p.n_mat - 1 && tile >= p.tile_end[mat]) ++mat;
        const int local = tile - (mat ? p.tile_end[mat - 1] : 0);
        m_tile = local % p.m_tiles;
        n_tile = local / p.m_tiles;
    };

    // A work item is one tile, or one of the ksplit equal parts of a tile's K blocks. All roles walk
    // items blockIdx.x, blockIdx.x + gridDim.x, ...
    const int total_items = p.total_tiles * p.ksplit;
    auto item_range = [&](int item, int &tile, int &kb0, int &kb1) {
        tile = item / p.ksplit;
        const int part = item - tile * p.ksplit;
        kb0 = part * p.kb_part;
        kb1 = kb0 + p.kb_part < k_blocks ? kb0 + p.kb_part : k_blocks;
    };

    if (warp == kPackWarp) {
        // ================= TMA producer: packed weights =================
        if (lane == 0) {
            int pit = 0;
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
                int tile, kb0, kb1, mat, m_tile, n_tile;
                item_range(item, tile, kb0, kb1);
                decode_tile(tile, mat, m_tile, n_tile);
                for (int kb = kb0; kb < kb1; kb += kPackBlocks, ++pit) {  // kb0 is a multiple of kPackBlocks
                    const int ps = pit % PS, pround = pit / PS;
                    if (pround > 0 && !wait_bar(bar(C::kBarEmptyPack + ps), (pround - 1) & 1, s_abort)) {
                        ok = false;
                        break;
                    }
                    ptx::mbar_arrive_expect_tx(bar(C::kBarFullPack + ps), kPackBytes);
                    ptx::tma_load_2d(base + C::kPack0 + ps * kPackBytes, &p.wpk[mat], bar(C::kBarFullPack + ps), kb * kBlockBytes, n_tile * kBMW);
                }
            }
        }
    } else if (warp == kTmaWarp) {
        // ================= TMA producer: activations =================
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            int gr = 0;  // groups of activation blocks
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
                int tile, kb0, kb1, mat, m_tile, n_tile;
                item_range(item, tile, kb0, kb1);
                decode_tile(tile, mat, m_tile, n_tile);
                for (int kb = kb0; kb < kb1; kb += G, ++gr) {
                    const int s = gr % PG, round = gr / PG;
                    if (round > 0 && !wait_bar(bar(C::kBarConsumed + s), (round - 1) & 1, s_abort)) {
                        ok = false;
                        break;
                    }
                    const int nblk = kb1 - kb < G ? kb1 - kb : G;
                    ptx::mbar_arrive_expect_tx(bar(C::kBarFull + s), static_cast<uint32_t>(nblk * p.nt) * kBK);
                    for (int b = 0; b < nblk; ++b)
                        ptx::tma_load_2d(base + (s * G + b) * C::kActBytes, &p.act, bar(C::kBarFull + s), (kb + b) * kBK, m_tile * p.nt);
                }
            }
        }
    } else if (warp >= kExpWarp0 && warp < kExpWarp0 + kExpWarps * kExpSets) {
        // ================= expanders: packed 2-bit -> u8 codes in TMEM =================
        const int quad = (warp - kExpWarp0) % kExpWarps, set = (warp - kExpWarp0) / kExpWarps;
        const int r = quad * 32 + lane;  // weight row of the tile = TMEM lane
        const uint32_t lane_field = static_cast<uint32_t>(quad * 32) << 16;
        // Ring positions are counters (no divisions in the loop): group `gr` uses barrier slot `sp`
        // and the TMEM slots of parity gr & 1; (lg, lg_phase) follow group gr - 2, whose MMAs were
        // the last readers of those TMEM slots; (ps, pphase) follow the packed-weight stage.
        int gr = 0, sp = 0, lg = PG - 2, ps = -1;
        uint32_t lg_phase = 1, pphase = 1;
        for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
            int tile, kb0, kb1;
            item_range(item, tile, kb0, kb1);
            for (int kb = kb0; kb < kb1; kb += G, ++gr) {
                if ((kb % kPackBlocks) == 0) {
                    if (++ps == PS) ps = 0;
                    if (ps == 0) pphase ^= 1u;
                    if (!wait_bar(bar(C::kBarFullPack + ps), pphase, s_abort)) {
                        ok = false;
                        break;
                    }
                }
                bool wrote = false;
#pragma unroll
                for (int b = set; b < G; b += kExpSets) {  // this warp's blocks of the group
                    if (kb + b >= kb1) break;
                    if (!wrote) {
                        // the TMEM slots of this parity were last read by group gr - 2
                        if (gr >= 2 && !wait_bar(bar(C::kBarConsumed + lg), lg_phase, s_abort)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        wrote = true;
                    }
                    // row r of the [128][128 B] swizzled stage; this block's 32 bytes are units 2*sub, 2*sub+1
                    const int sub = ((kb + b) % kPackBlocks);
                    const uint8_t *pk = sm + C::kPack0 + ps * kPackBytes + r * 128;
                    const int x = r & 7;
                    const uint4 w0 = *reinterpret_cast<const uint4 *>(pk + (((2 * sub) ^ x) << 4));      // packed bytes j = 0..15
                    const uint4 w1 = *reinterpret_cast<const uint4 *>(pk + (((2 * sub + 1) ^ x) << 4));  // packed bytes j = 16..31
                    const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                    uint32_t v[32];  // word 8k + i = columns k*32 + 4i .. 4i+3
#pragma unroll
                    for (int k = 0; k < 4; ++k)
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[8 * k + i] = (w[i] >> (2 * k)) & 0x03030303u;
                    tmem_st32(tmem_base + lane_field + C::kA0 + ((gr & 1) * G + b) * 32, v);
                }
                if (!ok) break;
                // this warp's last read of the packed stage is behind it when the stage's last block is
                if (((kb + G) % kPackBlocks) == 0 || kb + G >= kb1) {
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(bar(C::kBarEmptyPack + ps));
                }
                if (wrote) {
                    tmem_st_wait();
                    tc_fence_before();
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar(C::kBarFull + sp));
                if (++sp == PG) sp = 0;
                if (++lg == PG) {
                    lg = 0;
                    lg_phase ^= 1u;
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ================= MMA issuer (one thread) =================
        if (lane == 0) {
            // Ring positions are kept as counters: this thread's instruction stream is the critical
            // path of the whole CTA (one thread issues every MMA), so no divisions by the ring size here.
            int tcount = 0, sp = 0;
            uint32_t full_phase = 0, pa = 0;
            const uint64_t bdesc0 = smem_desc_sw128(base);  // activation block stage 0; stage s adds s * kActBytes / 16
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++tcount) {
                const int a = tcount & 1, around = tcount >> 1;
                if (around > 0 && !wait_bar(bar(C::kBarAccEmpty + a), (around - 1) & 1, s_abort)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (a ? C::kAcc1 : C::kAcc0);
                // N of this tile: the launch's token tile, less for the last tile of a ragged batch
                int tile, kb0, kb1, mat, m_tile, n_tile;
                item_range(item, tile, kb0, kb1);
                decode_tile(tile, mat, m_tile, n_tile);
                const int left = p.m - m_tile * p.nt;
                const int n_mma = left < p.nt ? (left + 15) & ~15 : p.nt;
                const uint32_t idesc = C::kIdesc | (static_cast<uint32_t>(n_mma >> 3) << 17);
                for (int kb = kb0; kb < kb1; kb += G) {
                    if (!wait_bar(bar(C::kBarFull + sp), full_phase, s_abort)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_tmem = tmem_base + C::kA0 + pa * (G * 32);
                    const uint64_t bdesc = bdesc0 + static_cast<uint64_t>(sp * G * (C::kActBytes >> 4));
                    umma_i8_ts_block(d_tmem, a_tmem, bdesc, idesc, kb != kb0 ? 1u : 0u);
#pragma unroll
                    for (int b = 1; b < G; ++b)
                        if (kb + b < kb1) umma_i8_ts_block(d_tmem, a_tmem + b * 32, bdesc + static_cast<uint64_t>(b * (C::kActBytes >> 4)), idesc, 1u);
                    umma_commit(bar(C::kBarConsumed + sp));  // both operands' slots are reusable once these MMAs retire
                    if (++sp == PG) {
                        sp = 0;
                        full_phase ^= 1u;
                    }
                    pa ^= 1u;
                }
                if (!ok) break;
                umma_commit(bar(C::kBarAccFull + a));  // accumulator complete
            }
        }
    } else if (warp < kEpiWarps) {
        // ================= epilogue (warps 0..3 = TMEM lane quadrants 0..3) =================
        int *s_qs = reinterpret_cast<int *>(sm + C::kTok);
        float *s_inv = reinterpret_cast<float *>(sm + C::kTok + 2 * NT * 4);
        asm volatile("griddepcontrol.wait;" ::: "memory");
        int tcount = 0;
        for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++tcount) {
            const int a = tcount & 1, around = tcount >> 1;
            int tile, kb0, kb1, mat, m_tile, n_tile;
            item_range(item, tile, kb0, kb1);
            decode_tile(tile, mat, m_tile, n_tile);
            const int rows = p.rows[mat];
            const int row = n_tile * kBMW + warp * 32 + lane;
            const int nt = p.nt;
            const int tok0 = m_tile * nt;
            float *out = p.out[mat];
            int32_t *iout = p.iout[mat];
            // per-token terms of this tile (each warp fills its own copy: no cross-warp barrier)
            int *qs = s_qs + a * NT;  // reuse by accumulator parity is safe: see acc_empty below
            float *inv = s_inv + a * NT;
            if (warp == 0) {
                for (int i = lane; i < ((nt + 31) & ~31); i += 32) {
                    const int tk = tok0 + i;
                    qs[i] = tk < p.m ? p.qsum[tk] : 0;
                    inv[i] = (tk < p.m && p.qscale) ? __fdiv_rn(1.0f, __fmul_rn(p.qscale[tk], p.wscale[mat])) : 0.0f;  // gemm.rs:158
                }
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");  // the four epilogue warps
            if (!wait_bar(bar(C::kBarAccFull + a), around & 1, s_abort)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const int ntok = p.m - tok0 < nt ? p.m - tok0 : nt;
#pragma unroll 1
            for (int c = 0; c * 32 < ntok; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + (a ? C::kAcc1 : C::kAcc0) + c * 32, v);
                // per-token terms into registers first: the stores below may alias the shared
                // arrays as far as the compiler knows, which would serialise load -> store pairs
                int q[32];
                float sc[32];
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const int4 q4 = *reinterpret_cast<const int4 *>(qs + c * 32 + i);
                    const float4 s4 = *reinterpret_cast<const float4 *>(inv + c * 32 + i);
                    q[i] = q4.x; q[i + 1] = q4.y; q[i + 2] = q4.z; q[i + 3] = q4.w;
                    sc[i] = s4.x; sc[i + 1] = s4.y; sc[i + 2] = s4.z; sc[i + 3] = s4.w;
                }
                tmem_ld_wait();
                if constexpr (SC) {
                    // The reduce-scatter of a row-parallel layer starts here: the int32 dots of a token go straight
                    // into the buffer of the rank that owns the token (plain stores into peer memory, 128 consecutive
                    // bytes per warp instruction), while the MMAs of the next tile run.
                    if (row < rows) {
                        const int tk = tok0 + c * 32;
                        int o = tk / p.scatter_mt, lt = tk - o * p.scatter_mt;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (c * 32 + i < ntok) p.scatter[o][static_cast<size_t>(lt) * rows + row] = static_cast<int>(v[i]) - q[i];
                            if (++lt == p.scatter_mt) {
                                lt = 0;
                                ++o;
                            }
                        }
                    }
                    continue;
                }
                if (p.ksplit > 1) {
                    // one of several parts of this tile: add the sums into the zeroed int32 buffer
                    // (the part that starts at block 0 also takes off sum(q)); a small kernel scales later
                    if (row < rows) {
                        int32_t *dst = p.acc[mat] + static_cast<size_t>(tok0 + c * 32) * rows + row;
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (c * 32 + i < ntok) atomicAdd(dst + static_cast<size_t>(i) * rows, static_cast<int>(v[i]) - (kb0 == 0 ? q[i] : 0));
                    }
                    continue;
                }
                if (row < rows) {
                    const size_t o0 = static_cast<size_t>(tok0 + c * 32) * rows + row;
                    if (c * 32 + 32 <= ntok) {
                        if (out) {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                out[o0 + static_cast<size_t>(i) * rows] = __fmul_rn(__int2float_rn(static_cast<int>(v[i]) - q[i]), sc[i]);
                        }
                        if (iout) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) iout[o0 + static_cast<size_t>(i) * rows] = static_cast<int>(v[i]) - q[i];
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (c * 32 + i < ntok) {
                                const int d = static_cast<int>(v[i]) - q[i];
                                if (iout) iout[o0 + static_cast<size_t>(i) * rows] = d;
                                if (out) out[o0 + static_cast<size_t>(i) * rows] = __fmul_rn(__int2float_rn(d), sc[i]);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            asm volatile("bar.sync 2, 128;" ::: "memory");  // all four warps are done with qs/inv of this parity
            if (lane == 0) ptx::mbar_arrive(bar(C::kBarAccEmpty + a));
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

template <int NT>
static int init_one(Ctx *ctx) {
    const size_t smem = Cfg<NT>::kTotal + 1024;
    if (smem > ctx->smem_optin) return fail(LBK_ERR_UNSUPPORTED, "gemm kernel needs %zu B of shared memory", smem);
    LBK_CUDA(cudaFuncSetAttribute(gemm_kernel<NT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    LBK_CUDA(cudaFuncSetAttribute(gemm_kernel<NT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    return LBK_OK;
}

int gemm_init(Ctx *ctx) {
    LBK_TRY(init_one<192>(ctx));
    LBK_TRY(init_one<64>(ctx));
    LBK_CUDA(cudaMalloc(&ctx->gemm_acc, kGemmAccBytes));
    LBK_CUDA(cudaMemset(ctx->gemm_acc, 0, kGemmAccBytes));  // kept zero between launches: the scaling kernel zeroes what it reads
    return LBK_OK;
}

// Parts to cut every tile's K blocks into. A launch with few tiles against the SM count (small
// token batches, tensor-parallel shards) or with a ragged last round leaves SMs idle; parts add
// their int32 sums into a zeroed buffer and a small kernel scales them afterwards. Cost model in
// K-block times of one CTA (about 500 cycles); the parts' atomic adds, the scaling launch and its
// traffic are charged as 30 (14 was tried once the zeroing launches were gone: the 70B-shaped gate/up
// projection at 64 token rows then split in two and took twice as long, 14.7 MB of sums added twice).
static int choose_ksplit(int tiles, int k_blocks, int sms, int *kb_part) {
    int best = 1;
    long long best_cost = static_cast<long long>((tiles + sms - 1) / sms) * k_blocks;
    *kb_part = k_blocks;
    for (int s = 2; s <= 8; ++s) {
        const int per = ((k_blocks + s - 1) / s + kPackBlocks - 1) / kPackBlocks * kPackBlocks;
        if (per < 2 * kPackBlocks) break;
        const int parts = (k_blocks + per - 1) / per;
        if (parts != s) continue;  // rounding made fewer parts: that count is or was tried as itself
        const long long cost = static_cast<long long>((static_cast<long long>(tiles) * s + sms - 1) / sms) * per + 30;
        if (cost * 100 < best_cost * 85) {
            best_cost = cost;
            best = s;
            *kb_part = per;
        }
    }
    return best;
}


// Token rows per tile for a launch: the multiple of 16 (at most 192) whose tile count fills whole
// rounds of the grid best. Per K block a tile costs the larger of the tensor-pipe time
// (proportional to nt, about 400 cycles at nt = 192) and the issue thread's turn-around (about
// 470 cycles whatever nt is: measured), plus the epilogue's share that the next tile cannot hide.
static int choose_nt(size_t m, int row_tiles, int k_blocks, int sms) {
    if (m <= 64) return static_cast<int>((m + 15) & ~static_cast<size_t>(15));
    int best_nt = 192;
    double best = 1e30;
    for (int tiles_m = static_cast<int>((m + 191) / 192); tiles_m <= static_cast<int>((m + 63) / 64); ++tiles_m) {
        const int nt = static_cast<int>(((m + tiles_m - 1) / tiles_m + 15) & ~static_cast<size_t>(15));
        if (nt > 192 || nt < 64) continue;
        const long long tiles = static_cast<long long>(row_tiles) * ((m + nt - 1) / nt);
        const long long rounds = (tiles + sms - 1) / sms;
        const double block = nt * (400.0 / 192.0) > 470.0 ? nt * (400.0 / 192.0) : 470.0;
        const double cost = static_cast<double>(rounds) * (k_blocks * block + 12.0 * nt);
        if (cost < best) {
            best = cost;
            best_nt = nt;
        }
    }
    return best_nt;
}

int launch_gemm(Ctx *ctx, const GroupArgs &g, cudaStream_t stream) {
    if (!g.q || !g.qsum) return fail(LBK_ERR_INVALID, "gemm: quantised activations are required");
    if (g.n < 1 || g.n > LBK_MAX_GROUP) return fail(LBK_ERR_INVALID, "group size %d not in 1..%d", g.n, LBK_MAX_GROUP);
    if (g.m == 0) return LBK_OK;
    GemmParams p{};
    const size_t kp = g.w[0]->kp;
    int row_tiles = 0;
    for (int i = 0; i < g.n; ++i) row_tiles += static_cast<int>((g.w[i]->rows + kBMW - 1) / kBMW);
    const int nt = choose_nt(g.m, row_tiles, static_cast<int>(kp / kBK), ctx->sm_count);
    LBK_TRY(encode_act_map(&p.act, g.q, g.m, kp, nt));
    p.nt = nt;
    p.m = static_cast<int>(g.m);
    p.m_tiles = static_cast<int>((g.m + nt - 1) / nt);
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
        tiles += p.m_tiles * static_cast<int>((w->rows + kBMW - 1) / kBMW);
        p.tile_end[i] = tiles;
    }
    p.n_mat = g.n;
    p.total_tiles = tiles;
    p.qscale = g.qscale;
    p.qsum = g.qsum;
    p.err_word = ctx->err_word;
    if (tiles == 0 || p.k_blocks == 0) return LBK_OK;
    p.ksplit = choose_ksplit(tiles, p.k_blocks, ctx->sm_count, &p.kb_part);
    p.scatter_world = g.scatter_world;
    p.scatter_mt = g.scatter_mt;
    for (int i = 0; i < 8; ++i) p.scatter[i] = g.scatter_base[i];
    if (g.scatter_world) {
        if (g.n != 1 || g.scatter_mt < 1) return fail(LBK_ERR_INVALID, "gemm: scattered outputs take one matrix");
        p.ksplit = 1;  // parts of a tile would have to add into peer memory
        p.kb_part = p.k_blocks;
    }
    if (p.ksplit > 1) {
        // int32 targets: the caller's integer outputs where given, else slices of the context's buffer
        size_t need = 0;
        for (int i = 0; i < g.n; ++i)
            if (!g.iout[i]) need += (g.m * g.w[i]->rows * sizeof(int32_t) + 255) / 256 * 256;
        if (need > kGemmAccBytes) {
            p.ksplit = 1;
            p.kb_part = p.k_blocks;
        } else {
            size_t off = 0;
            for (int i = 0; i < g.n; ++i) {
                const size_t bytes = g.m * g.w[i]->rows * sizeof(int32_t);
                if (g.iout[i]) {
                    p.acc[i] = g.iout[i];
                    LBK_CUDA(cudaMemsetAsync(p.acc[i], 0, bytes, stream));  // the caller's buffer holds whatever it held
                } else {
                    // the context's buffer is zero at rest (launch_scale_epilogue_group zeroes what it reads)
                    p.acc[i] = reinterpret_cast<int32_t *>(reinterpret_cast<char *>(ctx->gemm_acc) + off);
                    off += (bytes + 255) / 256 * 256;
                }
            }
        }
    }
    const int items = tiles * p.ksplit;
    const int grid = items < ctx->sm_count ? items : ctx->sm_count;
    // programmatic stream serialisation: this grid may start while the previous kernel of the
    // stream is still draining (see griddepcontrol.wait in the kernel)
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(kThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (nt > 64) {
        cfg.dynamicSmemBytes = Cfg<192>::kTotal + 1024;
        if (p.scatter_world) LBK_CUDA(cudaLaunchKernelEx(&cfg, gemm_kernel<192, true>, p));
        else LBK_CUDA(cudaLaunchKernelEx(&cfg, gemm_kernel<192, false>, p));
    } else {
        cfg.dynamicSmemBytes = Cfg<64>::kTotal + 1024;
        if (p.scatter_world) LBK_CUDA(cudaLaunchKernelEx(&cfg, gemm_kernel<64, true>, p));
        else LBK_CUDA(cudaLaunchKernelEx(&cfg, gemm_kernel<64, false>, p));
    }
    LBK_CUDA(cudaGetLastError());
    ctx->launches++;
    if (p.ksplit > 1) {  // one launch scales every matrix of the group (and zeroes the context's sums again)
        int32_t *dots[LBK_MAX_GROUP];
        float *outs[LBK_MAX_GROUP];
        float ws[LBK_MAX_GROUP];
        int rows[LBK_MAX_GROUP];
        bool clean[LBK_MAX_GROUP];
        bool any = false;
        for (int i = 0; i < g.n; ++i) {
            dots[i] = p.acc[i];
            outs[i] = g.out[i];
            ws[i] = g.w[i]->scale;
            rows[i] = static_cast<int>(g.w[i]->rows);
            clean[i] = g.iout[i] == nullptr;
            any = any || g.out[i] != nullptr || clean[i];
        }
        if (any) LBK_TRY(launch_scale_epilogue_group(ctx, g.n, dots, outs, ws, rows, clean, g.qscale, g.m, stream));
    }
    return LBK_OK;
}

}  // namespace lbk
