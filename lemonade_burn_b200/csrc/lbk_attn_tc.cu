// Causal attention of the rows of a prompt pass on the 5th-generation tensor cores.
//
// The step it is part of: BitNet::forward with m > 1 rows (crates/lb-model/src/model.rs:331-357:
// q k^T / sqrt(d), causal mask, softmax in f32, times v, per head with grouped KV heads). Row i of
// the pass sits at position pos0 + i and sees keys 0 .. pos0 + i of the sequence's bf16 cache.
//
// One CTA takes 128 query rows of one head and walks the keys in blocks of 128:
//
//   TMA thread      K blocks (a ring of three) and V blocks (a ring of two), [128 keys][128 dims] bf16
//                   from the cache (SWIZZLE_128B, two 64-dimension halves each)
//   MMA thread      S = Q K^T: tcgen05.mma kind::f16, A = the queries (shared memory, written once by
//                   the CTA as two bf16 terms hi + lo, log2(e)/sqrt(d) folded in), B = the K block as it
//                   lies in the cache (K-major), f32 scores in tensor memory; O += P V: A = the
//                   probabilities from TENSOR MEMORY (two bf16 terms again), B = the V block as it
//                   lies in the cache: its contraction index (the key) is the strided one, which is
//                   the MN-major operand form of the instruction, so V is never transposed. The
//                   output accumulates in tensor memory over all key blocks.
//   4 softmax warps thread r owns query row r = TMEM lane r: it takes its 128 scores into registers
//                   (the score buffer is free for the next block's Q K^T from then on), finds the
//                   row's maximum with a plain loop, and writes 2^(s - m) as two bf16 terms into one
//                   of two probability buffers in tensor memory. m is the maximum the row's earlier
//                   probabilities were scaled with; it is only moved (and the output in tensor
//                   memory and the running sum rescaled, by a whole warp at a time) when a block's
//                   maximum exceeds it by more than 8, i.e. probabilities stay below 2^8: the
//                   quotient O / sum at the end does not depend on m.
//
// While the threads work on block j the tensor core runs Q K^T of block j + 1 and P V of block j - 1.
// f32 queries and probabilities as hi + lo (|error| <= 2^-17 |x|) keep the only rounding beyond f32
// summation the bf16 of the cache itself, as in the decode kernels; the sums over keys are the
// tensor core's f32 accumulation (about 2e-8 of the largest output per 16 keys, measured on the bf16
// head: 5e-6 at 2048 keys). What this replaces: the same arithmetic on mma.sync with 16-row tiles
// per warp (attn_prompt_mma_kernel), which stays for passes of fewer than 64 rows.
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
constexpr int kBlockBytes = 2 * kHalf;      // a K or V block: two halves
constexpr int kKStages = 3, kVStages = 2;
constexpr int kK0 = kQBytes, kV0 = kK0 + kKStages * kBlockBytes;
constexpr int kBars = kV0 + kVStages * kBlockBytes;
constexpr int kMisc = kBars + 24 * 8;
constexpr int kPairMax = kMisc + 64;         // [2 halves][128 rows] f32: a row's two threads tell each other their maxima
constexpr int kSmem = kPairMax + 2 * kTile * 4 + 1024;
static_assert(kSmem <= 232448, "shared memory budget");
constexpr int kSoftWarps = 8;                // two per TMEM lane quadrant: warp w and w + 4 share rows, each takes 64 of a block's 128 keys
constexpr int kTmaWarp = 8, kMmaWarp = 9;
constexpr int kThreads = 10 * 32;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 128, kColP = 256;  // P buffer b: hi at kColP + 128 b, lo 64 columns further
constexpr float kRescaleStep = 8.0f;        // in units of log 2

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
    // kPReady and kOFull are pairs, one barrier per block parity: a wait for block j's completion can then never be
    // answered by block j - 2's (a barrier's parity says which of two CONSECUTIVE phases completed, no more)
    constexpr int kKFull = 0, kKEmpty = 3, kVFull = 6, kVEmpty = 8, kSFull = 10, kSFree = 11, kPReady = 12, kOFull = 14;
    if (tid == 0) {
        for (int s = 0; s < kKStages; ++s) {
            ptx::mbar_init(bar(kKFull + s), 1);
            ptx::mbar_init(bar(kKEmpty + s), 1);
        }
        for (int s = 0; s < kVStages; ++s) {
            ptx::mbar_init(bar(kVFull + s), 1);
            ptx::mbar_init(bar(kVEmpty + s), 1);
        }
        ptx::mbar_init(bar(kSFull), 1);
        ptx::mbar_init(bar(kSFree), kSoftWarps);
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(bar(kPReady + i), kSoftWarps);
            ptx::mbar_init(bar(kOFull + i), 1);
        }
        *s_abort = 0;
        ptx::fence_barrier_init();
    }
    if (warp == kMmaWarp) {
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
    if (warp < kSoftWarps) {
        const int r = (warp & 3) * 32 + lane;
        const bool live = r < rows_here && pos_ok;
        const float *qr = p.q + (static_cast<size_t>(row0 + (live ? r : 0)) * p.nh + head) * kHd;
#pragma unroll 4
        for (int u = (warp >> 2) * 8; u < (warp >> 2) * 8 + 8; ++u) {  // 16-byte unit u of the row: dimensions 8u .. 8u+7; a row's two threads take a half each
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

    if (warp == kTmaWarp) {
        // ================= TMA producer =================
        if (lane == 0) {
            int ks = 0, kround = 0;
            for (int j = 0; j < nb; ++j) {
                const int y = cache_row0 + j * kTile;
                if (kround > 0 && !wait_bar(bar(kKEmpty + ks), (kround - 1) & 1, s_abort)) {
                    ok = false;
                    break;
                }
                const uint32_t kst = base + kK0 + ks * kBlockBytes;
                ptx::mbar_arrive_expect_tx(bar(kKFull + ks), kBlockBytes);
                ptx::tma_load_2d(kst, &p.k, bar(kKFull + ks), 0, y);
                ptx::tma_load_2d(kst + kHalf, &p.k, bar(kKFull + ks), 128, y);
                if (++ks == kKStages) {
                    ks = 0;
                    ++kround;
                }
                const int vs = j & 1;
                if (j >= kVStages && !wait_bar(bar(kVEmpty + vs), ((j >> 1) - 1) & 1, s_abort)) {
                    ok = false;
                    break;
                }
                const uint32_t vst = base + kV0 + vs * kBlockBytes;
                ptx::mbar_arrive_expect_tx(bar(kVFull + vs), kBlockBytes);
                ptx::tma_load_2d(vst, &p.v, bar(kVFull + vs), 0, y);
                ptx::tma_load_2d(vst + kHalf, &p.v, bar(kVFull + vs), 128, y);
            }
        }
    } else if (warp == kMmaWarp) {
        // ================= MMA issuer (one thread) =================
        if (lane == 0 && nb > 0) {
            // D f32, A and B bf16, M = 128, N = 128; for P V the B operand is MN-major (bit 16)
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
            constexpr uint32_t idesc_o = idesc_s | (1u << 16);
            const uint64_t q_desc = smem_desc_sw128(base);
            int ks = 0, kphase = 0;  // ring position of the K block the next Q K^T reads
            auto issue_s = [&]() {   // S = Qhi K^T + Qlo K^T over the 8 steps of 16 dimensions
                const uint64_t k_desc = smem_desc_sw128(base + kK0 + ks * kBlockBytes);
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                    for (int st = 0; st < 8; ++st) {
                        const uint64_t off = static_cast<uint64_t>((st >> 2) * (kHalf >> 4) + (st & 3) * 2);
                        umma_f16_ss(tmem_base + kColS, q_desc + static_cast<uint64_t>(t * 2 * (kHalf >> 4)) + off, k_desc + off, idesc_s, (t | st) ? 1u : 0u);
                    }
                umma_commit(bar(kSFull));
                umma_commit(bar(kKEmpty + ks));
                if (++ks == kKStages) {
                    ks = 0;
                    kphase ^= 1;
                }
            };
            auto issue_pv = [&](int j) {  // O += Phi V + Plo V over the 8 steps of 16 keys: 8 columns of P, two 1024-byte key groups of V
                const int vs = j & 1;
                const uint64_t v_desc = smem_desc_mn_sw128(base + kV0 + vs * kBlockBytes);
                const uint32_t p_hi = tmem_base + kColP + (j & 1) * 128;
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                    for (int st = 0; st < 8; ++st)
                        umma_f16_ts(tmem_base + kColO, p_hi + t * 64 + st * 8, v_desc + static_cast<uint64_t>(st * (2048 >> 4)), idesc_o, (j | t | st) ? 1u : 0u);
                umma_commit(bar(kOFull + (j & 1)));
                umma_commit(bar(kVEmpty + vs));
            };
            // Every wait of this thread lets the tensor pipe run dry (its issue runs barely ahead of
            // execution), so a turn of the loop waits once, for everything the next 32 MMAs need, and then
            // issues P V of block j - 1 and Q K^T of block j + 1 back to back. P V goes first: Q K^T of
            // block j is then always issued after P V of block j - 2, so scores of block j in the score
            // buffer mean that the probability buffer of that parity has been read (the threads write
            // block j's probabilities on that ground).
            if (!wait_bar(bar(kKFull + 0), 0, s_abort)) ok = false;
            if (ok) {
                tc_fence_after();
                issue_s();
            }
            for (int j = 0; j <= nb && ok; ++j) {
                const bool has_pv = j > 0, has_s = j + 1 < nb;
                if (!has_pv && !has_s) continue;
                if (has_pv && (!wait_bar(bar(kPReady + ((j - 1) & 1)), ((j - 1) >> 1) & 1, s_abort) || !wait_bar(bar(kVFull + ((j - 1) & 1)), ((j - 1) >> 1) & 1, s_abort))) {
                    ok = false;
                    break;
                }
                // the threads hold block j's scores in registers: the score buffer is free
                if (has_s && (!wait_bar(bar(kSFree), j & 1, s_abort) || !wait_bar(bar(kKFull + ks), kphase, s_abort))) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (has_pv) issue_pv(j - 1);
                if (has_s) issue_s();
            }
        }
    } else {
        // ================= softmax and output (warps 0..7: quadrant warp & 3, key half warp >> 2) =================
        const int quad = warp & 3, kh2 = warp >> 2;
        const int r = quad * 32 + lane;
        const int qpos = pos0 + row0 + r;  // the last key this row sees
        const uint32_t lane_field = static_cast<uint32_t>(quad * 32) << 16;
        float *s_pair = reinterpret_cast<float *>(sm + kPairMax);
        float m = -INFINITY, l = 0.0f;     // m: the maximum the probabilities so far were scaled with; l: this thread's half of the row's sum
        // a wait whose outcome the whole warp shares: the tensor-memory loads and stores below are warp-wide instructions
        auto wait_all = [&](uint32_t b, uint32_t parity) { return __all_sync(0xffffffffu, wait_bar(b, parity, s_abort)) != 0; };
        auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory"); };  // the two warps of a quadrant
        // Every warp meets its partner exactly twice per block and once after the loop, whatever a wait
        // returned: a warp whose wait gave up (ok = false) skips the work, never the meetings.
        for (int j = 0; j < nb; ++j) {
            uint32_t sv[kTile / 2];  // keys kh2 * 64 .. + 63 of the block
            float *pair = s_pair;
            if (ok && !wait_all(bar(kSFull), j & 1)) ok = false;
            if (ok) {
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < 2; ++c) tmem_ld32(tmem_base + lane_field + kColS + kh2 * 64 + c * 32, reinterpret_cast<uint32_t(&)[32]>(sv[c * 32]));
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar(kSFree));
                const int key0 = j * kTile + kh2 * 64;
                if (key0 + 63 > qpos) {  // some of these keys are in this row's future
#pragma unroll
                    for (int i = 0; i < kTile / 2; ++i)
                        if (key0 + i > qpos) sv[i] = 0xff800000u;  // -inf: 2^(-inf - m) = 0
                }
                float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                for (int i = 0; i < kTile / 2; i += 4) {
                    mx0 = fmaxf(mx0, __uint_as_float(sv[i]));
                    mx1 = fmaxf(mx1, __uint_as_float(sv[i + 1]));
                    mx2 = fmaxf(mx2, __uint_as_float(sv[i + 2]));
                    mx3 = fmaxf(mx3, __uint_as_float(sv[i + 3]));
                }
                pair[kh2 * kTile + r] = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            }
            pair_sync();
            const float mx = fmaxf(pair[r], pair[kTile + r]);  // the row's maximum over the block; both threads of the row hold the same m and mx
            pair_sync();  // both have read before the next block's maxima are written
            if (!ok) continue;
            // key 0 <= qpos always: in the first block the maximum is finite for rows that exist
            if (__any_sync(0xffffffffu, j == 0 || mx > m + kRescaleStep)) {
                const float nm = fmaxf(m, mx);
                if (j > 0) {
                    // the output so far (P V of every earlier block) is complete and nothing adds to it before
                    // both warps of the quadrant say their probabilities are ready
                    if (!wait_all(bar(kOFull + ((j - 1) & 1)), ((j - 1) >> 1) & 1)) {
                        ok = false;
                        continue;
                    }
                    tc_fence_after();
                    const float corr = ex2(m - nm);
                    l *= corr;
#pragma unroll 1
                    for (int c = 0; c < 2; ++c) {  // this warp's 64 columns of the output
                        uint32_t v[32];
                        tmem_ld32(tmem_base + lane_field + kColO + kh2 * 64 + c * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
                        tmem_st32(tmem_base + lane_field + kColO + kh2 * 64 + c * 32, v);
                    }
                }
                m = nm;
            }
            float ps0 = 0.0f, ps1 = 0.0f;
            const uint32_t p_hi = tmem_base + lane_field + kColP + (j & 1) * 128 + kh2 * 32;  // two keys a column
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t ph[16], pl[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float e0 = ex2(__uint_as_float(sv[c * 32 + 2 * i]) - m), e1 = ex2(__uint_as_float(sv[c * 32 + 2 * i + 1]) - m);
                    ps0 += e0;
                    ps1 += e1;
                    split_pair(e0, e1, ph[i], pl[i]);
                }
                tmem_st16(p_hi + c * 16, ph);
                tmem_st16(p_hi + 64 + c * 16, pl);
            }
            l += ps0 + ps1;
            // rows of V that no kernel has written: zero them before the tensor core multiplies them by zeros
            if (j * kTile + kTile > written) {
                if (!wait_all(bar(kVFull + (j & 1)), (j >> 1) & 1)) {
                    ok = false;
                    continue;
                }
                if (j * kTile + r >= written) {  // thread (row r, half kh2) zeroes one 64-dimension half of V row r
                    uint8_t *vrow = sm + kV0 + (j & 1) * kBlockBytes + kh2 * kHalf + r * 128;
#pragma unroll
                    for (int u = 0; u < 8; ++u) *reinterpret_cast<uint4 *>(vrow + u * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
                ptx::fence_proxy_async();
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar(kPReady + (j & 1)));
        }
        if (ok && nb > 0) {
            if (!wait_all(bar(kOFull + ((nb - 1) & 1)), ((nb - 1) >> 1) & 1)) ok = false;
            tc_fence_after();
        }
        // the row's sum: the two halves meet
        float *pair_l = s_pair;
        pair_l[kh2 * kTile + r] = l;
        pair_sync();
        const float lsum = pair_l[r] + pair_l[kTile + r];
        if (ok && nb > 0) {
            const float inv = 1.0f / lsum;
            float *dst = p.out + (static_cast<size_t>(row0 + (r < rows_here ? r : 0)) * p.nh + head) * kHd + kh2 * 64;
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {  // this warp's 64 dimensions of the row
                uint32_t v[32];
                tmem_ld32(tmem_base + lane_field + kColO + kh2 * 64 + c * 32, v);
                tmem_ld_wait();
                if (r < rows_here) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4 *>(dst + c * 32 + i) = make_float4(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv,
                                                                                    __uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
                }
            }
            tc_fence_before();
        }
    }
    if (!ok && pos_ok && lane == 0) atomicExch(p.err_word, 5);
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
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
