// Shared device code of the decode GEMV kernels (single fused group and persistent sweep).
//
// Data path, common to both:
//   * a warp owns a ring of kStages TMA stages, each one box of [16 weight rows][128 packed
//     bytes] (= 512 columns) laid down with the 128-byte swizzle;
//   * lane (g, t) of the warp reads 16-byte units 2t and 2t+1 of rows g and g+8: packed
//     block t of the chunk's four blocks; one AND with 0x03030303 << 2k turns a packed word
//     into the four codes of columns k*32 + j..j+3 scaled by 4^k (a valid u8);
//   * mma.sync.m16n8k32 (u8 x s8 -> s32): the 16 weight rows are the M side, token rows the N
//     side; per k-group and per parity of the word pair there is a separate accumulator set
//     (8 independent chains per 8 tokens) because a dependent IMMA issues only ~96 cycles
//     after its predecessor on this part;
//   * quantised activations sit in shared memory in the order the B fragments want them.
#pragma once

#include "lbk_internal.cuh"
#include "lbk_ptx.cuh"

namespace lbk {
namespace gemv {

// One stage takes a warp ~700 cycles end to end (barrier wait, shared loads, 64 LOP3, 16 IMMA of
// ~96 cycles latency, re-issue), mostly latency, so throughput comes from warps in flight: 16
// warps x 3 stages measured faster than 8 x 6 at the same 96 KB of loads in flight per SM.
constexpr int kWarps = 16;                            // warps per CTA; each streams its own ring
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 3;                            // TMA ring depth per warp
constexpr int kTileRows = 16;                         // weight rows per MMA tile
constexpr int kChunkBytes = 128;                      // packed bytes per row per stage
constexpr int kChunkCols = kChunkBytes * 4;           // 512 columns
constexpr int kStageBytes = kTileRows * kChunkBytes;  // 2048
constexpr uint32_t kWaitLimit = 1u << 22;             // polls before a wait gives up
constexpr int kMaxM = LBK_GEMV_MAX_M;

// Position of natural column n inside a token row of the shared activation buffer:
// [chunk][k-group][c/2][t][c%2][8] with n = (chunk*4 + t)*128 + kgroup*32 + c*8 + e. The sixteen
// bytes a lane needs for two consecutive MMAs are one 128-bit load, next to those of its three
// neighbours.
__device__ __forceinline__ uint32_t xq_pos(uint32_t n) {
    uint32_t chunk = n >> 9, t = (n >> 7) & 3, kk = (n >> 5) & 3, c = (n >> 3) & 3, e = n & 7;
    return ((((chunk * 4 + kk) * 2 + (c >> 1)) * 4 + t) << 4) + ((c & 1) << 3) + e;
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

__device__ __forceinline__ uint32_t pack4(int q0, int q1, int q2, int q3) {
    return (q0 & 255) | ((q1 & 255) << 8) | ((q2 & 255) << 16) | (static_cast<uint32_t>(q3 & 255) << 24);
}

// max|x| over x[lo + 4*step*j ...] handled by `nthr` cooperating threads (thread index `idx`).
__device__ __forceinline__ float absmax_span(const float *xr, int k, bool vec, int idx, int nthr) {
    float am = 0.0f;  // fmaxf drops a NaN operand, as f32::max does (quant.rs:101-104)
    if (vec) {
        const float4 *x4 = reinterpret_cast<const float4 *>(xr);
#pragma unroll 8
        for (int i = idx; i < (k >> 2); i += nthr) {
            const float4 v = __ldg(x4 + i);
            am = fmaxf(am, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
    } else {
        for (int i = idx; i < k; i += nthr) am = fmaxf(am, fabsf(__ldg(xr + i)));
    }
    return am;
}

// Quantises columns [0, kfill) of one row (zeros beyond k) into `dst` in xq_pos order, four
// columns per thread step; returns this thread's part of sum(q).
__device__ __forceinline__ int quantize_span(const float *xr, int k, int kfill, bool vec, float sc,
                                             uint8_t *dst, int idx, int nthr) {
    int acc = 0;
#pragma unroll 4
    for (int i = idx * 4; i < kfill; i += nthr * 4) {
        int q0 = 0, q1 = 0, q2 = 0, q3 = 0;
        if (vec && i + 3 < k) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(xr + i));
            q0 = quant_one(v.x, sc); q1 = quant_one(v.y, sc);
            q2 = quant_one(v.z, sc); q3 = quant_one(v.w, sc);
        } else {
            if (i < k) q0 = quant_one(__ldg(xr + i), sc);
            if (i + 1 < k) q1 = quant_one(__ldg(xr + i + 1), sc);
            if (i + 2 < k) q2 = quant_one(__ldg(xr + i + 2), sc);
            if (i + 3 < k) q3 = quant_one(__ldg(xr + i + 3), sc);
        }
        acc += q0 + q1 + q2 + q3;
        *reinterpret_cast<uint32_t *>(dst + xq_pos(i)) = pack4(q0, q1, q2, q3);
    }
    return acc;
}

// One-pass variant for rows short enough to hold in registers: a thread keeps up to kCacheV
// float4 of the row between the max and the rounding, so the row is read once.
constexpr int kCacheV = 8;
struct RowCache {
    float4 v[kCacheV];
};
__device__ __forceinline__ void load_cached(const float *xr, int k, int idx, int nthr, RowCache &rc) {
    const float4 *x4 = reinterpret_cast<const float4 *>(xr);
    const int n4 = k >> 2;
#pragma unroll
    for (int j = 0; j < kCacheV; ++j) {
        const int i = idx + j * nthr;
        rc.v[j] = i < n4 ? __ldg(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}
// load_cached with an L2 policy: rows that are read again by every launch ask to stay resident
__device__ __forceinline__ void load_cached_hint(const float *xr, int k, int idx, int nthr, RowCache &rc, uint64_t policy) {
    const float4 *x4 = reinterpret_cast<const float4 *>(xr);
    const int n4 = k >> 2;
#pragma unroll
    for (int j = 0; j < kCacheV; ++j) {
        const int i = idx + j * nthr;
        if (i < n4) {
            const uint4 u = ptx::ldg_hint(x4 + i, policy);
            rc.v[j] = make_float4(__uint_as_float(u.x), __uint_as_float(u.y), __uint_as_float(u.z), __uint_as_float(u.w));
        } else {
            rc.v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
}
__device__ __forceinline__ float max_cached(const RowCache &rc) {
    float am = 0.0f;
#pragma unroll
    for (int j = 0; j < kCacheV; ++j)
        am = fmaxf(am, fmaxf(fmaxf(fabsf(rc.v[j].x), fabsf(rc.v[j].y)), fmaxf(fabsf(rc.v[j].z), fabsf(rc.v[j].w))));
    return am;
}
__device__ __forceinline__ float absmax_cached(const float *xr, int k, int idx, int nthr, RowCache &rc) {
    load_cached(xr, k, idx, nthr, rc);
    float am = 0.0f;
#pragma unroll
    for (int j = 0; j < kCacheV; ++j)
        am = fmaxf(am, fmaxf(fmaxf(fabsf(rc.v[j].x), fabsf(rc.v[j].y)), fmaxf(fabsf(rc.v[j].z), fabsf(rc.v[j].w))));
    return am;
}
__device__ __forceinline__ int quantize_cached(const RowCache &rc, int kfill, float sc, uint8_t *dst, int idx, int nthr) {
    int acc = 0;
#pragma unroll
    for (int j = 0; j < kCacheV; ++j) {
        const int i = (idx + j * nthr) * 4;
        if (i < kfill) {  // lanes past k hold zeros, which quantise to zero
            const int q0 = quant_one(rc.v[j].x, sc), q1 = quant_one(rc.v[j].y, sc);
            const int q2 = quant_one(rc.v[j].z, sc), q3 = quant_one(rc.v[j].w, sc);
            acc += q0 + q1 + q2 + q3;
            *reinterpret_cast<uint32_t *>(dst + xq_pos(i)) = pack4(q0, q1, q2, q3);
        }
    }
    return acc;
}
// quantize_cached for a single warp whose cache starts at column `col0`
__device__ __forceinline__ int quantize_cached_at(const RowCache &rc, int col0, int kfill, float sc, uint8_t *dst, int lane) {
    int acc = 0;
#pragma unroll
    for (int j = 0; j < kCacheV; ++j) {
        const int i = col0 + (lane + j * 32) * 4;
        if (i < kfill) {
            const int q0 = quant_one(rc.v[j].x, sc), q1 = quant_one(rc.v[j].y, sc);
            const int q2 = quant_one(rc.v[j].z, sc), q3 = quant_one(rc.v[j].w, sc);
            acc += q0 + q1 + q2 + q3;
            *reinterpret_cast<uint32_t *>(dst + xq_pos(i)) = pack4(q0, q1, q2, q3);
        }
    }
    return acc;
}
// zero [from, kfill) of a row when the cached path covered fewer columns than kfill
__device__ __forceinline__ void zero_tail(uint8_t *dst, int from, int kfill, int idx, int nthr) {
    for (int i = from + idx * 4; i < kfill; i += nthr * 4) *reinterpret_cast<uint32_t *>(dst + xq_pos(i)) = 0u;
}

// Per-lane byte offsets into a stage for the two 16-byte units of rows g and g+8.
struct LaneOffsets {
    uint32_t a, b;
};
__device__ __forceinline__ LaneOffsets lane_offsets(int lane) {
    const int g = lane >> 2, t = lane & 3;
    LaneOffsets o;
    o.a = g * 128 + (((2 * t) ^ g) << 4);      // the 128B swizzle: unit ^= row & 7
    o.b = g * 128 + (((2 * t + 1) ^ g) << 4);
    return o;
}

// One stage: 16 rows x 512 columns against MT groups of 8 token rows. xrow[mt] points at
// this lane's 16-byte slot (t*16) of the token row it feeds; xoff = chunk * 512.
// FIRST: the accumulators are overwritten by this stage (first stage of a tile) instead of added to.
template <int MT, bool FIRST = false>
__device__ __forceinline__ void consume_stage(const uint8_t *st, LaneOffsets off,
                                              const uint8_t *const (&xrow)[MT], uint32_t xoff,
                                              int (&acc)[MT][2][4][4]) {
    const uint4 W0 = *reinterpret_cast<const uint4 *>(st + off.a);
    const uint4 W1 = *reinterpret_cast<const uint4 *>(st + off.b);
    const uint4 V0 = *reinterpret_cast<const uint4 *>(st + 1024 + off.a);
    const uint4 V1 = *reinterpret_cast<const uint4 *>(st + 1024 + off.b);
    const uint32_t wlo[4] = {W0.x, W0.z, W1.x, W1.z};  // row g,   first word of pair c
    const uint32_t whi[4] = {W0.y, W0.w, W1.y, W1.w};  // row g,   second word
    const uint32_t vlo[4] = {V0.x, V0.z, V1.x, V1.z};  // row g+8
    const uint32_t vhi[4] = {V0.y, V0.w, V1.y, V1.w};
#pragma unroll
    for (int cp = 0; cp < 2; ++cp) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const uint32_t mask = 0x03030303u << (2 * kk);
            uint4 b[MT];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) b[mt] = *reinterpret_cast<const uint4 *>(xrow[mt] + xoff + ((kk * 2 + cp) << 6));
#pragma unroll
            for (int ci = 0; ci < 2; ++ci) {
                const int c = cp * 2 + ci;
                const uint32_t a0 = wlo[c] & mask, a1 = vlo[c] & mask;
                const uint32_t a2 = whi[c] & mask, a3 = vhi[c] & mask;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    if (FIRST && cp == 0) ptx::mma_u8s8_init(acc[mt][ci][kk], a0, a1, a2, a3, ci ? b[mt].z : b[mt].x, ci ? b[mt].w : b[mt].y);
                    else ptx::mma_u8s8(acc[mt][ci][kk], a0, a1, a2, a3, ci ? b[mt].z : b[mt].x, ci ? b[mt].w : b[mt].y);
                }
            }
        }
    }
}

// sum over the accumulator sets of element j, undoing the 4^k scaling (exact: each set is a
// multiple of its factor), then zero them for the next tile.
template <int MT>
__device__ __forceinline__ int take_acc(int (&acc)[MT][2][4][4], int mt, int j) {
    int v = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        v += acc[mt][h][0][j] + (acc[mt][h][1][j] >> 2) + (acc[mt][h][2][j] >> 4) + (acc[mt][h][3][j] >> 6);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) acc[mt][h][kk][j] = 0;
    }
    return v;
}

// take_acc without the zeroing, for accumulators that the next tile's first stage overwrites
template <int MT>
__device__ __forceinline__ int read_acc(const int (&acc)[MT][2][4][4], int mt, int j) {
    int v = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) v += acc[mt][h][0][j] + (acc[mt][h][1][j] >> 2) + (acc[mt][h][2][j] >> 4) + (acc[mt][h][3][j] >> 6);
    return v;
}

}  // namespace gemv
}  // namespace lbk
