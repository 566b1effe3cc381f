// Tensor-parallel row-parallel layer (o, down) as two kernels that talk to the other ranks'
// GPUs directly over NVLink peer memory, instead of six operations with two NCCL calls:
//
//   tp_quantize_kernel      per-token max|x| of this rank's column slice, exchanged with every rank
//                           (one 8-byte peer store per rank and token), then the quantiser of
//                           quant.rs:100-118 with the maximum over the WHOLE row
//   (the caller's GEMM writes this rank's int32 partial dots into its own region)
//   tp_reduce_scale_kernel  tells the peers that the partial dots are there, waits for theirs,
//                           adds all ranks' int32 dots (exact, order-free) and applies the scale
//                           epilogue of gemm.rs:141
//
// The reference has no multi-device path (nearest relative: the two-socket row split of
// crates/lb-model/src/ops.rs:255-297). Every rank owns one "region" of device memory with the same
// layout; the regions are opened in every process through CUDA IPC handles. Only plain loads and
// stores cross NVLink: no multimem, no TMA, no multicast. Every wait on another rank is bounded;
// when one runs out the kernel sets the context's error word and goes on, so a missing peer costs
// wrong numbers and an LBK_ERR_TIMEOUT, never a hang.
//
// Why no buffer is overwritten while a slow peer still reads it: a rank starts the next layer's
// GEMM (which rewrites its partial dots) only after the next tp_quantize_kernel, which needs every
// peer's maxima for that layer, and a peer publishes those only after its own
// tp_reduce_scale_kernel of this layer has finished reading. The exchange slots alternate by the
// parity of a device-side sequence number for the same reason.
#include <cstring>

#include "lbk_internal.cuh"
#include "lbk_ptx.cuh"

namespace lbk {

constexpr int kTpMaxWorld = 8;
constexpr int kTpMaxTokens = 256;                   // token rows per call on the fused path
constexpr int kTpMaxRows = 2048;                    // token rows per call on the token-sharded path
constexpr int kTpMaxWidth = 8192;                   // widest row that is reduced and gathered (the hidden size)
constexpr int kTpGatherFRows = kTpMaxRows;          // token rows whose normalised f32 rows can be gathered (the head's input)
constexpr size_t kTpPartialBytes = static_cast<size_t>(kTpMaxRows) * kTpMaxWidth * 4;  // int32 partial dots of one call
constexpr uint32_t kTpWaitLimit = 1u << 24;         // default: polls of a peer's word before giving up (lbk_tp_comm_set_wait_limit)

// The same layout in every rank's region.
struct TpRegion {
    unsigned long long amax[2][kTpMaxWorld][kTpMaxTokens];  // (sequence << 32) | float bits, written by rank r
    unsigned int ready[kTpMaxWorld][32];                    // [r][0]: sequence of rank r's partial dots (padded)
    unsigned int q_seq, q_done, r_seq, r_done;              // this rank's own counters (never written by peers)
    unsigned int pad_[28];
    int32_t partial[kTpPartialBytes / 4];
    // ---- token-sharded path: statistics exchange, reduce-scatter flags, gathered rows ----
    unsigned long long stat[2][2][kTpMaxWorld][kTpMaxRows];  // [parity][round][writer][token]: (sequence << 32) | float bits
    unsigned long long best[2][kTpMaxWorld][kTpMaxRows];     // [parity][writer][token]: (ordered logit << 32) | ~index
    unsigned int rs_ready[kTpMaxWorld][32];                  // [r][0]: sequence of rank r's partial dots
    unsigned int ag_ready[kTpMaxWorld][32];                  // [r][0]: sequence of the rows rank r has written into THIS region
    unsigned int am_ready[kTpMaxWorld][32];                  // [r][0]: sequence of rank r's entries of `best` in THIS region
    unsigned int nq_seq, nq_done, rg_seq, rg_spare, rg_written, am_seq, pad2_[26];
    float gather_scale[kTpMaxRows];                          // per-token activation scale of the gathered rows
    int32_t gather_sum[kTpMaxRows];                          // per-token sum of the gathered int8 codes
    int8_t gather_q[static_cast<size_t>(kTpMaxRows) * kTpMaxWidth];     // all tokens' quantised rows, written by their owners
    float gather_f[static_cast<size_t>(kTpGatherFRows) * kTpMaxWidth];  // all tokens' normalised f32 rows (head input)
};

struct TpComm {
    Ctx *ctx;
    int world, rank;
    TpRegion *region[kTpMaxWorld];  // region[r] as mapped in this process; region[rank] is local
    uint32_t wait_limit = kTpWaitLimit;
};

namespace {

struct TpPtrs {
    TpRegion *r[kTpMaxWorld];
};

__device__ __forceinline__ int quant_one(float v, float scale) {
    int r = __float2int_rn(__fmul_rn(v, scale));  // NaN -> 0 like `NaN as i8` (quant.rs:115-118)
    return max(-128, min(127, r));
}

// One CTA per token row. Same arithmetic as quantize_kernel; only the maximum is the one over
// all ranks' slices.
__global__ void __launch_bounds__(256) tp_quantize_kernel(const TpPtrs peers, int world, int rank, const float *__restrict__ x, int k,
                                                          int kp, int8_t *__restrict__ q, float *__restrict__ scale,
                                                          int32_t *__restrict__ sum, int *err_word, uint32_t wait_limit) {
    __shared__ float s_f[8];
    __shared__ int s_i[8];
    __shared__ float s_scale;
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    TpRegion *me = peers.r[rank];
    const unsigned int seq = *reinterpret_cast<volatile unsigned int *>(&me->q_seq);
    const int par = seq & 1;
    const float *xr = x + static_cast<size_t>(row) * k;
    int8_t *qr = q + static_cast<size_t>(row) * kp;
    const bool vec = (k & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;

    float am = 0.0f;  // fmaxf drops a NaN operand, as f32::max does (quant.rs:101-104)
    if (vec) {
        const float4 *x4 = reinterpret_cast<const float4 *>(xr);
        for (int i = tid; i < (k >> 2); i += 256) {
            const float4 v = __ldg(x4 + i);
            am = fmaxf(am, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
    } else {
        for (int i = tid; i < k; i += 256) am = fmaxf(am, fabsf(__ldg(xr + i)));
    }
    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    if (lane == 0) s_f[warp] = am;
    __syncthreads();
    if (warp == 0) {
        float a = lane < 8 ? s_f[lane] : 0.0f;
        for (int o = 4; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        a = __shfl_sync(0xffffffffu, a, 0);
        // lane r publishes this rank's maximum in rank r's region, then waits for rank r's in its own
        const unsigned long long word = (static_cast<unsigned long long>(seq) << 32) | __float_as_uint(a);
        float other = 0.0f;
        bool ok = true;
        if (lane < world) {
            *reinterpret_cast<volatile unsigned long long *>(&peers.r[lane]->amax[par][rank][row]) = word;
            volatile unsigned long long *slot = &me->amax[par][lane][row];
            unsigned long long got = 0;
            uint32_t polls = 0;
            while (((got = *slot) >> 32) != seq) {
                if (++polls > wait_limit) {
                    ok = false;
                    break;
                }
            }
            other = __uint_as_float(static_cast<unsigned int>(got));
        }
        if (!ok) atomicExch(err_word, 6);
        for (int o = 16; o > 0; o >>= 1) other = fmaxf(other, __shfl_xor_sync(0xffffffffu, other, o));
        if (lane == 0) s_scale = __fdiv_rn(127.0f, fmaxf(other, 1e-5f));
    }
    __syncthreads();
    const float sc = s_scale;
    int acc = 0;
    for (int i = tid * 4; i < kp; i += 256 * 4) {
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
        *reinterpret_cast<uint32_t *>(qr + i) = (q0 & 255) | ((q1 & 255) << 8) | ((q2 & 255) << 16) |
                                                (static_cast<uint32_t>(q3 & 255) << 24);
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) s_i[warp] = acc;
    __syncthreads();
    if (tid == 0) {
        int s = 0;
        for (int w = 0; w < 8; ++w) s += s_i[w];
        scale[row] = sc;
        sum[row] = s;
        // the last CTA to finish moves the sequence on: every CTA has read it by then
        __threadfence();
        if (atomicAdd(&me->q_done, 1u) == gridDim.x - 1) {
            me->q_done = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned int *>(&me->q_seq) = seq + 1;
        }
    }
}

// out[t, r] = (float)(sum over ranks of dots[t, r]) * (1 / (scale[t] * wscale)) (gemm.rs:141).
// `total4` = m * rows / 4 (rows is a multiple of 4 on this path).
__global__ void __launch_bounds__(256) tp_reduce_scale_kernel(const TpPtrs peers, int world, int rank, const float *__restrict__ ascale,
                                                              float wscale, int rows, int total4, float *__restrict__ out,
                                                              int32_t *__restrict__ dots_out, int *err_word, uint32_t wait_limit) {
    TpRegion *me = peers.r[rank];
    const unsigned int seq = *reinterpret_cast<volatile unsigned int *>(&me->r_seq);
    const int tid = threadIdx.x;
    // this rank's partial dots were written by the kernel before this one (complete at the kernel
    // boundary); the fence orders them, system wide, before the flag that tells every peer so
    if (blockIdx.x == 0 && tid < world) {
        __threadfence_system();
        *reinterpret_cast<volatile unsigned int *>(&peers.r[tid]->ready[rank][0]) = seq;
    }
    if (tid < world) {
        volatile unsigned int *flag = &me->ready[tid][0];
        uint32_t polls = 0;
        while (static_cast<int>(*flag - seq) < 0) {  // a peer can only be at this call or, once we are through, past it
            if (++polls > wait_limit) {
                atomicExch(err_word, 6);
                break;
            }
        }
    }
    __syncthreads();
    for (int i = blockIdx.x * 256 + tid; i < total4; i += gridDim.x * 256) {
        // One 16-byte volatile load per rank, all in flight before the first add. Volatile: the same
        // addresses hold new numbers every call, and a peer's memory must not be served from a stale line.
        int4 v[kTpMaxWorld];
#pragma unroll
        for (int r = 0; r < kTpMaxWorld; ++r) {
            v[r] = make_int4(0, 0, 0, 0);
            if (r < world) {
                const int4 *src = reinterpret_cast<const int4 *>(peers.r[r]->partial) + i;
                asm volatile("ld.volatile.global.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v[r].x), "=r"(v[r].y), "=r"(v[r].z), "=r"(v[r].w) : "l"(src));
            }
        }
        int4 acc = make_int4(0, 0, 0, 0);
#pragma unroll
        for (int r = 0; r < kTpMaxWorld; ++r) {
            acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w;
        }
        const int e = i * 4;
        const float inv = __fdiv_rn(1.0f, __fmul_rn(ascale[e / rows], wscale));
        reinterpret_cast<float4 *>(out)[i] = make_float4(__fmul_rn(__int2float_rn(acc.x), inv), __fmul_rn(__int2float_rn(acc.y), inv),
                                                        __fmul_rn(__int2float_rn(acc.z), inv), __fmul_rn(__int2float_rn(acc.w), inv));
        if (dots_out) reinterpret_cast<int4 *>(dots_out)[i] = acc;
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&me->r_done, 1u) == gridDim.x - 1) {
            me->r_done = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned int *>(&me->r_seq) = seq + 1;
        }
    }
}


// =================================================================================================
// Token-sharded path. A row-parallel layer (o, down) of the decoder step as
//
//   tp_norm_quant_kernel       sub-norm + per-token quantisation of this rank's COLUMN slice of the
//                              layer input, for all tokens: two 8-byte exchanges per token (the
//                              slice's sum of squares, then its max |normalised value|), so that the
//                              norm and the scale are those of the whole row (model.rs:358,364;
//                              quant.rs:100-118)
//   (GEMM: int32 partial dots of the slice into this rank's region)
//   tp_reduce_norm_gather_kernel  each rank owns ceil(m/world) TOKENS. For its tokens it adds the
//                              int32 partial dots of all ranks (reads 1/world of every peer's
//                              buffer: exact, order-free), applies the scale epilogue (gemm.rs:141),
//                              adds the residual row it keeps for those tokens, applies the NEXT
//                              norm (full rows are local now: no exchange), quantises, and stores
//                              the int8 row with its scale and sum into EVERY rank's region, from
//                              where the next column-parallel GEMM of every rank reads all tokens.
//
// Per layer and rank this moves (world-1)/world * m * hidden * 4 bytes in (reduce-scatter) and
// (world-1)/world * m * hidden bytes out (all-gather), against world * m * hidden * 4 in for a
// one-shot all-reduce; the element-wise work is done once per token, not once per rank.
//
// Why nothing is overwritten too early. gather_q of call N is written by a rank only after it has
// seen every rank's rs_ready flag of call N, which a rank raises after its own row-parallel GEMM
// of call N, i.e. after its earlier GEMM that read gather_q of call N-1 (stream order). A rank's
// partial dots of call N are read by the peers before they raise ag_ready of call N, and the rank
// leaves its kernel (and reaches the GEMM that overwrites them) only after it has seen all of those.
// The statistics slots alternate by the parity of the sequence number; a rank can be at most one
// call ahead of a peer because every call needs every peer's value of that call.

constexpr int kNqThreads = 1024;
constexpr int kNqCache = 8;  // float4 per thread: column slices of up to 32768 columns (8192 with 256 threads)
constexpr size_t kTpManyRows = 256;  // from this many token rows on (a prompt pass) the exchange kernels run 256 threads a block

__device__ __forceinline__ float block_sum_f(float v, float *s_red, int nwarps) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.0f;
    for (int w = 0; w < nwarps; ++w) total += s_red[w];  // fixed order
    return total;
}

__device__ __forceinline__ float block_max_f(float v, float *s_red, int nwarps) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.0f;
    for (int w = 0; w < nwarps; ++w) total = fmaxf(total, s_red[w]);
    return total;
}

__device__ __forceinline__ int block_sum_i(int v, int *s_red, int nwarps) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    int total = 0;
    for (int w = 0; w < nwarps; ++w) total += s_red[w];
    return total;
}

// Warp 0 of a block: publishes `mine` for (round, row) in every rank's region and collects all
// ranks' values. Sum: added in rank order, so that every rank derives the same bits. Max: order-free.
__device__ __forceinline__ float exchange_stat(const TpPtrs &peers, int world, int rank, int par, int round, int row, unsigned int seq,
                                               float mine, bool is_sum, int *err_word, uint32_t wait_limit) {
    if (world == 1) return mine;  // total = 0 + mine and max(0, mine): the same bits as the loop below gives
    const int lane = threadIdx.x & 31;
    float other = 0.0f;
    bool ok = true;
    if (lane < world) {
        const unsigned long long word = (static_cast<unsigned long long>(seq) << 32) | __float_as_uint(mine);
        *reinterpret_cast<volatile unsigned long long *>(&peers.r[lane]->stat[par][round][rank][row]) = word;
        volatile unsigned long long *slot = &peers.r[rank]->stat[par][round][lane][row];
        unsigned long long got = 0;
        uint32_t polls = 0;
        while (((got = *slot) >> 32) != seq) {
            if (++polls > wait_limit) {
                ok = false;
                break;
            }
        }
        other = __uint_as_float(static_cast<unsigned int>(got));
    }
    if (!ok) atomicExch(err_word, 6);
    float total = 0.0f;
    for (int r = 0; r < world; ++r) {
        const float v = __shfl_sync(0xffffffffu, other, r);
        total = is_sum ? total + v : fmaxf(total, v);
    }
    return total;
}

// One CTA per token row. PRE = LBK_PRE_RMS: s = x; LBK_PRE_RELU2_MUL_RMS: s = relu(x)^2 * y.
// Then n_i = (s_i * r) * w_i with r = 1/sqrt(sum over ALL ranks of s^2 / k_full + eps), and the
// quantiser of quant.rs:100-118 with the maximum over all ranks.
// T threads a block: 1024 for a decode batch (few rows: the latency of one row counts, and rows of up to
// 32768 columns fit), 256 for the many rows of a prompt pass when a row fits (four rows in flight per SM
// instead of one: a row's chain of load, three block reductions and two exchanges no longer idles the SM).
template <int PRE, int T>
__global__ void __launch_bounds__(T) tp_norm_quant_kernel(const TpPtrs peers, int world, int rank, const float *__restrict__ x,
                                                                  const float *__restrict__ y, const float *__restrict__ w, int kl, int k_full,
                                                                  float eps, int8_t *__restrict__ q, float *__restrict__ scale,
                                                                  int32_t *__restrict__ sum, int *err_word, uint32_t wait_limit) {
    __shared__ float s_red[T / 32];
    __shared__ int s_redi[T / 32];
    __shared__ float s_bcast;
    // Launched with programmatic stream serialisation: the kernel behind this one (the row-parallel
    // GEMM) may be scheduled now and stream its first weight tiles while this one runs; it waits for
    // this grid's results itself. Everything this kernel reads was written by kernels that are
    // complete once the wait below returns.
    ptx::pdl_trigger();
    ptx::pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    TpRegion *me = peers.r[rank];
    const unsigned int seq = *reinterpret_cast<volatile unsigned int *>(&me->nq_seq);
    const int par = seq & 1;
    const int n4 = kl >> 2;
    const float4 *xr = reinterpret_cast<const float4 *>(x + static_cast<size_t>(row) * kl);
    const float4 *yr = y ? reinterpret_cast<const float4 *>(y + static_cast<size_t>(row) * kl) : nullptr;
    float4 v[kNqCache];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kNqCache; ++j) {
        const int i = tid + j * T;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) {
            const float4 a = xr[i];
            if (PRE == LBK_PRE_RMS) {
                v[j] = a;
            } else {
                const float4 c = yr[i];
                const float r0 = fmaxf(a.x, 0.f), r1 = fmaxf(a.y, 0.f), r2 = fmaxf(a.z, 0.f), r3 = fmaxf(a.w, 0.f);
                v[j] = make_float4(r0 * r0 * c.x, r1 * r1 * c.y, r2 * r2 * c.z, r3 * r3 * c.w);
            }
        }
        ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
    }
    ss = block_sum_f(ss, s_red, T / 32);
    if (tid < 32) {
        const float total = exchange_stat(peers, world, rank, par, 0, row, seq, ss, true, err_word, wait_limit);
        if (tid == 0) s_bcast = 1.0f / sqrtf(total / static_cast<float>(k_full) + eps);
    }
    __syncthreads();
    const float r = s_bcast;
    float am = 0.0f;
#pragma unroll
    for (int j = 0; j < kNqCache; ++j) {
        const int i = tid + j * T;
        if (i < n4) {
            const float4 gw = __ldg(reinterpret_cast<const float4 *>(w) + i);
            v[j] = make_float4(v[j].x * r * gw.x, v[j].y * r * gw.y, v[j].z * r * gw.z, v[j].w * r * gw.w);
            am = fmaxf(am, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));  // fmaxf drops a NaN, as f32::max does
        }
    }
    am = block_max_f(am, s_red, T / 32);
    __syncthreads();  // s_bcast has been read by everybody
    if (tid < 32) {
        const float total = exchange_stat(peers, world, rank, par, 1, row, seq, am, false, err_word, wait_limit);
        if (tid == 0) s_bcast = __fdiv_rn(127.0f, fmaxf(total, 1e-5f));
    }
    __syncthreads();
    const float sc = s_bcast;
    int8_t *qr = q + static_cast<size_t>(row) * kl;  // kl is a whole number of 128-column blocks: no padding
    int acc = 0;
#pragma unroll
    for (int j = 0; j < kNqCache; ++j) {
        const int i = tid + j * T;
        if (i < n4) {
            const int q0 = quant_one(v[j].x, sc), q1 = quant_one(v[j].y, sc), q2 = quant_one(v[j].z, sc), q3 = quant_one(v[j].w, sc);
            acc += q0 + q1 + q2 + q3;
            reinterpret_cast<uint32_t *>(qr)[i] = (q0 & 255) | ((q1 & 255) << 8) | ((q2 & 255) << 16) | (static_cast<uint32_t>(q3 & 255) << 24);
        }
    }
    acc = block_sum_i(acc, s_redi, T / 32);
    if (tid == 0) {
        scale[row] = sc;
        sum[row] = acc;
        if (world == 1) return;  // no exchange happened: the sequence number was not used
        __threadfence();
        if (atomicAdd(&me->nq_done, 1u) == gridDim.x - 1) {  // the last CTA moves the sequence on: every CTA has read it
            me->nq_done = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned int *>(&me->nq_seq) = seq + 1;
        }
    }
}

// The same for the many rows of a prompt pass when a row is too long for 256 threads' registers: the row's
// values live in shared memory (4 bytes a column: 112 KB at 28672 columns, two blocks per SM; 56 KB at
// half of that, three or four), the threads keep only their running sums, and 512 threads a block leave
// room for several blocks per SM, so that one row's exchanges overlap another row's loads. Element by
// element the arithmetic is tp_norm_quant_kernel's.
constexpr int kNqSmemThreads = 512;
template <int PRE>
__global__ void __launch_bounds__(kNqSmemThreads) tp_norm_quant_smem_kernel(const TpPtrs peers, int world, int rank, const float *__restrict__ x,
                                                                           const float *__restrict__ y, const float *__restrict__ w, int kl, int k_full,
                                                                           float eps, int8_t *__restrict__ q, float *__restrict__ scale,
                                                                           int32_t *__restrict__ sum, int *err_word, uint32_t wait_limit) {
    constexpr int T = kNqSmemThreads;
    extern __shared__ __align__(16) float4 s_row[];
    __shared__ float s_red[T / 32];
    __shared__ int s_redi[T / 32];
    __shared__ float s_bcast;
    ptx::pdl_trigger();
    ptx::pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    TpRegion *me = peers.r[rank];
    const unsigned int seq = *reinterpret_cast<volatile unsigned int *>(&me->nq_seq);
    const int par = seq & 1;
    const int n4 = kl >> 2;
    const float4 *xr = reinterpret_cast<const float4 *>(x + static_cast<size_t>(row) * kl);
    const float4 *yr = y ? reinterpret_cast<const float4 *>(y + static_cast<size_t>(row) * kl) : nullptr;
    float ss = 0.0f;
#pragma unroll 4
    for (int i = tid; i < n4; i += T) {
        const float4 a = xr[i];
        float4 v;
        if (PRE == LBK_PRE_RMS) {
            v = a;
        } else {
            const float4 c = yr[i];
            const float r0 = fmaxf(a.x, 0.f), r1 = fmaxf(a.y, 0.f), r2 = fmaxf(a.z, 0.f), r3 = fmaxf(a.w, 0.f);
            v = make_float4(r0 * r0 * c.x, r1 * r1 * c.y, r2 * r2 * c.z, r3 * r3 * c.w);
        }
        s_row[i] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = block_sum_f(ss, s_red, T / 32);
    if (tid < 32) {
        const float total = exchange_stat(peers, world, rank, par, 0, row, seq, ss, true, err_word, wait_limit);
        if (tid == 0) s_bcast = 1.0f / sqrtf(total / static_cast<float>(k_full) + eps);
    }
    __syncthreads();
    const float r = s_bcast;
    float am = 0.0f;
#pragma unroll 4
    for (int i = tid; i < n4; i += T) {
        const float4 gw = __ldg(reinterpret_cast<const float4 *>(w) + i);
        float4 v = s_row[i];
        v = make_float4(v.x * r * gw.x, v.y * r * gw.y, v.z * r * gw.z, v.w * r * gw.w);
        s_row[i] = v;
        am = fmaxf(am, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    am = block_max_f(am, s_red, T / 32);
    __syncthreads();  // s_bcast has been read by everybody
    if (tid < 32) {
        const float total = exchange_stat(peers, world, rank, par, 1, row, seq, am, false, err_word, wait_limit);
        if (tid == 0) s_bcast = __fdiv_rn(127.0f, fmaxf(total, 1e-5f));
    }
    __syncthreads();
    const float sc = s_bcast;
    int8_t *qr = q + static_cast<size_t>(row) * kl;
    int acc = 0;
#pragma unroll 4
    for (int i = tid; i < n4; i += T) {
        const float4 v = s_row[i];
        const int q0 = quant_one(v.x, sc), q1 = quant_one(v.y, sc), q2 = quant_one(v.z, sc), q3 = quant_one(v.w, sc);
        acc += q0 + q1 + q2 + q3;
        reinterpret_cast<uint32_t *>(qr)[i] = (q0 & 255) | ((q1 & 255) << 8) | ((q2 & 255) << 16) | (static_cast<uint32_t>(q3 & 255) << 24);
    }
    acc = block_sum_i(acc, s_redi, T / 32);
    if (tid == 0) {
        scale[row] = sc;
        sum[row] = acc;
        if (world == 1) return;
        __threadfence();
        if (atomicAdd(&me->nq_done, 1u) == gridDim.x - 1) {
            me->nq_done = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned int *>(&me->nq_seq) = seq + 1;
        }
    }
}

struct RgArgs {
    int world, rank, m, hidden, mt;   // mt = ceil(m / world) tokens per rank
    int reduce;                       // 1: add all ranks' partial dots (read from their regions), scale, add to the residual; 2: the same, but the
                                      // ranks' GEMMs have already stored their dots of this rank's tokens into THIS region ([source rank][mt][hidden]); 0: the residual rows are the input
    int gather_f32;                   // 1: gather the normalised f32 rows (head input) instead of int8 rows
    const float *ascale;              // [m] activation scales of the row-parallel GEMM's input (reduce = 1)
    float wscale;
    float *xres;                      // [mt][hidden] residual rows of this rank's tokens
    const float *w;                   // [hidden] gain of the norm that follows
    float eps;
    float *y_out;                     // optional [mt][hidden]: the projection's scaled output rows
    int *err_word;
    uint32_t wait_limit;
};

// One CTA per token this rank owns (a single CTA if it owns none: it still raises and awaits the flags).
// T threads a block as in tp_norm_quant_kernel: 1024 for decode batches, 256 for the rows of a prompt pass.
template <int T>
__global__ void __launch_bounds__(T) tp_reduce_norm_gather_kernel(const TpPtrs peers, const RgArgs a) {
    __shared__ float s_red[T / 32];
    __shared__ int s_redi[T / 32];
    ptx::pdl_trigger();  // the column-parallel GEMM behind this kernel may start fetching its weights
    ptx::pdl_wait();     // the partial dots (the GEMM before this kernel) are complete from here on
    const int tid = threadIdx.x, world = a.world, rank = a.rank, H = a.hidden;
    TpRegion *me = peers.r[rank];
    const unsigned int seq = *reinterpret_cast<volatile unsigned int *>(&me->rg_seq);
    const int t0 = rank * a.mt;
    const int own = max(0, min(a.m - t0, a.mt));
    const int lt = blockIdx.x;  // local token
    if (a.reduce && world > 1) {
        // this rank's partial dots were written by the kernel before this one, which is complete (the
        // wait above): they sit in this GPU's memory, where the peers' loads find them. The flag tells
        // every peer so.
        if (blockIdx.x == 0 && tid < world) {
            __threadfence_system();
            *reinterpret_cast<volatile unsigned int *>(&peers.r[tid]->rs_ready[rank][0]) = seq;
        }
        if (tid < world) {
            volatile unsigned int *flag = &me->rs_ready[tid][0];
            uint32_t polls = 0;
            while (static_cast<int>(*flag - seq) < 0) {
                if (++polls > a.wait_limit) {
                    atomicExch(a.err_word, 6);
                    break;
                }
            }
        }
        __syncthreads();
    }
    if (lt < own) {
        const int t = t0 + lt, n4 = H >> 2;
        constexpr int kIt = kTpMaxWidth / 4 / T;  // 16-byte units of a row per thread
        float4 v[kIt];
        float ss = 0.0f;
#pragma unroll
        for (int it = 0; it < kIt; ++it) {
            const int g = tid + it * T;
            v[it] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (g < n4) {
                float4 x = reinterpret_cast<const float4 *>(a.xres + static_cast<size_t>(lt) * H)[g];
                if (a.reduce) {
                    // one 16-byte load per rank, all in flight before the first add; volatile: the same
                    // addresses hold new numbers every call
                    int4 d[kTpMaxWorld];
#pragma unroll
                    for (int r = 0; r < kTpMaxWorld; ++r) {
                        d[r] = make_int4(0, 0, 0, 0);
                        if (r < world) {
                            const int4 *src = a.reduce == 2 ? reinterpret_cast<const int4 *>(me->partial + (static_cast<size_t>(r) * a.mt + lt) * H) + g
                                                            : reinterpret_cast<const int4 *>(peers.r[r]->partial + static_cast<size_t>(t) * H) + g;
                            asm volatile("ld.volatile.global.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(d[r].x), "=r"(d[r].y), "=r"(d[r].z), "=r"(d[r].w) : "l"(src));
                        }
                    }
                    int4 acc = make_int4(0, 0, 0, 0);
#pragma unroll
                    for (int r = 0; r < kTpMaxWorld; ++r) {
                        acc.x += d[r].x; acc.y += d[r].y; acc.z += d[r].z; acc.w += d[r].w;
                    }
                    const float inv = __fdiv_rn(1.0f, __fmul_rn(a.ascale[t], a.wscale));  // gemm.rs:141
                    const float4 yv = make_float4(__fmul_rn(__int2float_rn(acc.x), inv), __fmul_rn(__int2float_rn(acc.y), inv),
                                                  __fmul_rn(__int2float_rn(acc.z), inv), __fmul_rn(__int2float_rn(acc.w), inv));
                    if (a.y_out) reinterpret_cast<float4 *>(a.y_out + static_cast<size_t>(lt) * H)[g] = yv;
                    x = make_float4(x.x + yv.x, x.y + yv.y, x.z + yv.z, x.w + yv.w);  // the residual add (model.rs:359,365)
                    reinterpret_cast<float4 *>(a.xres + static_cast<size_t>(lt) * H)[g] = x;
                }
                v[it] = x;
            }
            ss += v[it].x * v[it].x + v[it].y * v[it].y + v[it].z * v[it].z + v[it].w * v[it].w;
        }
        const float r = 1.0f / sqrtf(block_sum_f(ss, s_red, T / 32) / static_cast<float>(H) + a.eps);
        float am = 0.0f;
#pragma unroll
        for (int it = 0; it < kIt; ++it) {
            const int g = tid + it * T;
            if (g < n4) {
                const float4 gw = __ldg(reinterpret_cast<const float4 *>(a.w) + g);
                v[it] = make_float4(v[it].x * r * gw.x, v[it].y * r * gw.y, v[it].z * r * gw.z, v[it].w * r * gw.w);
                am = fmaxf(am, fmaxf(fmaxf(fabsf(v[it].x), fabsf(v[it].y)), fmaxf(fabsf(v[it].z), fabsf(v[it].w))));
            }
        }
        if (a.gather_f32) {
#pragma unroll
            for (int it = 0; it < kIt; ++it) {
                const int g = tid + it * T;
                if (g < n4)
                    for (int p = 0; p < world; ++p) reinterpret_cast<float4 *>(peers.r[p]->gather_f + static_cast<size_t>(t) * H)[g] = v[it];
            }
        } else {
            const float sc = __fdiv_rn(127.0f, fmaxf(block_max_f(am, s_red, T / 32), 1e-5f));
            int acc = 0;
#pragma unroll
            for (int it = 0; it < kIt; ++it) {
                const int g = tid + it * T;
                if (g < n4) {
                    const int q0 = quant_one(v[it].x, sc), q1 = quant_one(v[it].y, sc), q2 = quant_one(v[it].z, sc), q3 = quant_one(v[it].w, sc);
                    acc += q0 + q1 + q2 + q3;
                    const uint32_t word = (q0 & 255) | ((q1 & 255) << 8) | ((q2 & 255) << 16) | (static_cast<uint32_t>(q3 & 255) << 24);
                    for (int p = 0; p < world; ++p) reinterpret_cast<uint32_t *>(peers.r[p]->gather_q + static_cast<size_t>(t) * H)[g] = word;
                }
            }
            acc = block_sum_i(acc, s_redi, T / 32);
            if (tid < world) {
                peers.r[tid]->gather_scale[t] = sc;
                peers.r[tid]->gather_sum[t] = acc;
            }
        }
    }
    // Every row this rank owns is in every region once ALL its CTAs are here. The CTA that arrives
    // last says so to every rank and then waits until every peer has said the same; the others leave
    // at once. The kernel ends when that CTA ends, so whatever follows in the stream finds all tokens'
    // rows in this rank's region, and no CTA waits for a peer while CTAs of its own grid still have
    // to be scheduled. One fence per CTA: the block barrier orders every thread's stores before
    // thread 0's fence, and the fence is cumulative. The last CTA also moves the sequence number on:
    // every CTA of the grid has read it by then. With one rank there is nobody to tell.
    if (world == 1) return;
    __syncthreads();
    __shared__ int s_last;
    if (tid == 0) {
        __threadfence_system();
        s_last = atomicAdd(&me->rg_written, 1u) == gridDim.x - 1;
        if (s_last) me->rg_written = 0;
    }
    __syncthreads();
    if (s_last) {
        if (tid < world) {
            __threadfence_system();  // the other CTAs' rows, seen through the count, before the flag
            *reinterpret_cast<volatile unsigned int *>(&peers.r[tid]->ag_ready[rank][0]) = seq;
            volatile unsigned int *flag = &me->ag_ready[tid][0];
            uint32_t polls = 0;
            while (static_cast<int>(*flag - seq) < 0) {
                if (++polls > a.wait_limit) {
                    atomicExch(a.err_word, 6);
                    break;
                }
            }
        }
        __syncthreads();
        if (tid == 0) *reinterpret_cast<volatile unsigned int *>(&me->rg_seq) = seq + 1;
    }
}

// Greedy token over a vocabulary split by rows across ranks (sample.rs:17-25: the FIRST maximum).
// One CTA; thread t owns token t. idx_local[t] is this rank's first maximum of its slice.
__device__ __forceinline__ unsigned int ordered_bits(float f) {
    const unsigned int u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__global__ void __launch_bounds__(1024) tp_argmax_kernel(const TpPtrs peers, int world, int rank, const float *__restrict__ logits, const int32_t *__restrict__ idx_local,
                                                        int m, int vl, int32_t *__restrict__ next, int *err_word, uint32_t wait_limit) {
    ptx::pdl_trigger();
    ptx::pdl_wait();
    TpRegion *me = peers.r[rank];
    const unsigned int seq = *reinterpret_cast<volatile unsigned int *>(&me->am_seq);
    const int par = seq & 1, tid = threadIdx.x;
    for (int t = tid; t < m; t += blockDim.x) {
        const int li = idx_local[t];
        const unsigned int gi = static_cast<unsigned int>(rank * vl + li);
        const unsigned long long key = (static_cast<unsigned long long>(ordered_bits(logits[static_cast<size_t>(t) * vl + li])) << 32) | (~gi);
        for (int p = 0; p < world; ++p) peers.r[p]->best[par][rank][t] = key;
    }
    __syncthreads();
    if (tid < world) {
        __threadfence_system();  // cumulative over the barrier: every thread's keys are out before the flag
        *reinterpret_cast<volatile unsigned int *>(&peers.r[tid]->am_ready[rank][0]) = seq;
        volatile unsigned int *flag = &me->am_ready[tid][0];
        uint32_t polls = 0;
        while (static_cast<int>(*flag - seq) < 0) {
            if (++polls > wait_limit) {
                atomicExch(err_word, 6);
                break;
            }
        }
    }
    __syncthreads();
    for (int t = tid; t < m; t += blockDim.x) {
        unsigned long long bestk = 0;
        for (int r = 0; r < world; ++r) {
            const unsigned long long k = *reinterpret_cast<volatile unsigned long long *>(&me->best[par][r][t]);
            bestk = k > bestk ? k : bestk;  // larger logit first, then the smaller index (its complement is larger)
        }
        next[t] = static_cast<int32_t>(~static_cast<unsigned int>(bestk));
    }
    __syncthreads();
    if (tid == 0) *reinterpret_cast<volatile unsigned int *>(&me->am_seq) = seq + 1;
}

}  // namespace

}  // namespace lbk

using namespace lbk;

extern "C" {

size_t lbk_tp_region_bytes(void) { return sizeof(TpRegion); }
size_t lbk_tp_max_tokens(void) { return kTpMaxTokens; }
size_t lbk_tp_partial_bytes(void) { return kTpPartialBytes; }

int lbk_tp_region_alloc(lbk_ctx *c, void **region_out, unsigned char handle_out[64]) {
    if (!c || !region_out || !handle_out) return fail(LBK_ERR_INVALID, "lbk_tp_region_alloc: null argument");
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    LBK_CUDA(cudaSetDevice(ctx->device));
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, sizeof(TpRegion));
    if (e != cudaSuccess) return fail(LBK_ERR_NOMEM, "tensor-parallel region: %s", cudaGetErrorString(e));
    LBK_CUDA(cudaMemset(p, 0, sizeof(TpRegion)));  // sequences start at 1 so that a zeroed slot never matches
    const unsigned int one = 1;
    LBK_CUDA(cudaMemcpy(&static_cast<TpRegion *>(p)->q_seq, &one, sizeof(one), cudaMemcpyHostToDevice));
    LBK_CUDA(cudaMemcpy(&static_cast<TpRegion *>(p)->r_seq, &one, sizeof(one), cudaMemcpyHostToDevice));
    LBK_CUDA(cudaMemcpy(&static_cast<TpRegion *>(p)->nq_seq, &one, sizeof(one), cudaMemcpyHostToDevice));
    LBK_CUDA(cudaMemcpy(&static_cast<TpRegion *>(p)->rg_seq, &one, sizeof(one), cudaMemcpyHostToDevice));
    LBK_CUDA(cudaMemcpy(&static_cast<TpRegion *>(p)->am_seq, &one, sizeof(one), cudaMemcpyHostToDevice));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI passes IPC handles as 64 bytes");
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(LBK_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    }
    std::memcpy(handle_out, &h, 64);
    *region_out = p;
    return LBK_OK;
}

int lbk_tp_region_open(lbk_ctx *c, const unsigned char handle[64], void **region_out) {
    if (!c || !handle || !region_out) return fail(LBK_ERR_INVALID, "lbk_tp_region_open: null argument");
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    LBK_CUDA(cudaSetDevice(ctx->device));
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(LBK_ERR_CUDA, "cudaIpcOpenMemHandle: %s (are the GPUs peers?)", cudaGetErrorString(e));
    *region_out = p;
    return LBK_OK;
}

int lbk_tp_region_close(lbk_ctx *c, void *region) {
    if (!c || !region) return LBK_OK;
    LBK_CUDA(cudaSetDevice(reinterpret_cast<Ctx *>(c)->device));
    LBK_CUDA(cudaIpcCloseMemHandle(region));
    return LBK_OK;
}

int lbk_tp_region_free(lbk_ctx *c, void *region) {
    if (!c || !region) return LBK_OK;
    LBK_CUDA(cudaSetDevice(reinterpret_cast<Ctx *>(c)->device));
    LBK_CUDA(cudaDeviceSynchronize());
    LBK_CUDA(cudaFree(region));
    return LBK_OK;
}

int lbk_tp_comm_create(lbk_ctx *c, int world, int rank, void *const *regions, lbk_tp_comm **out) {
    if (!c || !regions || !out) return fail(LBK_ERR_INVALID, "lbk_tp_comm_create: null argument");
    if (world < 1 || world > kTpMaxWorld || rank < 0 || rank >= world)
        return fail(LBK_ERR_INVALID, "rank %d of %d (at most %d ranks)", rank, world, kTpMaxWorld);
    for (int r = 0; r < world; ++r)
        if (!regions[r]) return fail(LBK_ERR_INVALID, "region of rank %d is null", r);
    TpComm *t = new (std::nothrow) TpComm();
    if (!t) return fail(LBK_ERR_NOMEM, "out of host memory");
    t->ctx = reinterpret_cast<Ctx *>(c);
    t->world = world;
    t->rank = rank;
    for (int r = 0; r < kTpMaxWorld; ++r) t->region[r] = r < world ? static_cast<TpRegion *>(regions[r]) : nullptr;
    *out = reinterpret_cast<lbk_tp_comm *>(t);
    return LBK_OK;
}

int lbk_tp_comm_destroy(lbk_tp_comm *t) {
    delete reinterpret_cast<TpComm *>(t);
    return LBK_OK;
}

int lbk_tp_comm_set_wait_limit(lbk_tp_comm *t, uint32_t polls) {
    if (!t) return fail(LBK_ERR_INVALID, "tensor-parallel communicator is null");
    if (polls == 0) return fail(LBK_ERR_INVALID, "a wait limit of 0 polls would give up before looking");
    reinterpret_cast<TpComm *>(t)->wait_limit = polls;
    return LBK_OK;
}

void *lbk_tp_partial_buffer(lbk_tp_comm *t) {
    if (!t) return nullptr;
    TpComm *tc = reinterpret_cast<TpComm *>(t);
    return tc->region[tc->rank]->partial;
}

static TpPtrs ptrs_of(const TpComm *tc) {
    TpPtrs p{};
    for (int r = 0; r < kTpMaxWorld; ++r) p.r[r] = tc->region[r];
    return p;
}

int lbk_tp_quantize(lbk_tp_comm *t, const float *x_dev, size_t m, size_t k, int8_t *q_dev, float *scale_dev, int32_t *sum_dev,
                    void *stream) {
    if (!t) return fail(LBK_ERR_INVALID, "tensor-parallel communicator is null");
    TpComm *tc = reinterpret_cast<TpComm *>(t);
    if (m == 0) return fail(LBK_ERR_INVALID, "lbk_tp_quantize: every rank must take part, m = 0 is not a call");
    if (m > kTpMaxTokens) return fail(LBK_ERR_UNSUPPORTED, "lbk_tp_quantize takes at most %d token rows (got %zu)", kTpMaxTokens, m);
    if (!x_dev || !q_dev || !scale_dev || !sum_dev || k == 0) return fail(LBK_ERR_INVALID, "lbk_tp_quantize: null buffer or empty row");
    LBK_CUDA(cudaSetDevice(tc->ctx->device));
    tp_quantize_kernel<<<static_cast<unsigned>(m), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        ptrs_of(tc), tc->world, tc->rank, x_dev, static_cast<int>(k), static_cast<int>(lbk_padded_cols(k)), q_dev, scale_dev, sum_dev,
        tc->ctx->err_word, tc->wait_limit);
    LBK_CUDA(cudaGetLastError());
    tc->ctx->launches++;
    return LBK_OK;
}

int lbk_tp_reduce_scale(lbk_tp_comm *t, const float *scale_dev, float wscale, size_t m, size_t rows, float *out_dev,
                        int32_t *dots_out_dev, void *stream) {
    if (!t) return fail(LBK_ERR_INVALID, "tensor-parallel communicator is null");
    TpComm *tc = reinterpret_cast<TpComm *>(t);
    if (m == 0 || rows == 0) return fail(LBK_ERR_INVALID, "lbk_tp_reduce_scale: every rank must take part, an empty call is not a call");
    if (!scale_dev || !out_dev) return fail(LBK_ERR_INVALID, "lbk_tp_reduce_scale: null buffer");
    if ((rows & 3) || m * rows * sizeof(int32_t) > kTpPartialBytes || (reinterpret_cast<uintptr_t>(out_dev) & 15) ||
        (reinterpret_cast<uintptr_t>(dots_out_dev) & 15))
        return fail(LBK_ERR_UNSUPPORTED, "lbk_tp_reduce_scale needs rows %% 4 == 0, 16-byte aligned outputs and m * rows * 4 <= %zu", kTpPartialBytes);
    LBK_CUDA(cudaSetDevice(tc->ctx->device));
    const int total4 = static_cast<int>(m * rows / 4);
    int grid = (total4 + 255) / 256;
    if (grid > 2 * tc->ctx->sm_count) grid = 2 * tc->ctx->sm_count;
    tp_reduce_scale_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(ptrs_of(tc), tc->world, tc->rank, scale_dev, wscale,
                                                                               static_cast<int>(rows), total4, out_dev, dots_out_dev,
                                                                               tc->ctx->err_word, tc->wait_limit);
    LBK_CUDA(cudaGetLastError());
    tc->ctx->launches++;
    return LBK_OK;
}

size_t lbk_tp_max_rows(void) { return kTpMaxRows; }
size_t lbk_tp_max_width(void) { return kTpMaxWidth; }
size_t lbk_tp_max_f32_rows(void) { return kTpGatherFRows; }

int lbk_tp_token_range(const lbk_tp_comm *t, size_t m, size_t *first_out, size_t *count_out) {
    if (!t || !first_out || !count_out) return fail(LBK_ERR_INVALID, "lbk_tp_token_range: null argument");
    const TpComm *tc = reinterpret_cast<const TpComm *>(t);
    const size_t mt = (m + tc->world - 1) / tc->world, t0 = static_cast<size_t>(tc->rank) * mt;
    *first_out = t0 < m ? t0 : m;
    *count_out = t0 < m ? (m - t0 < mt ? m - t0 : mt) : 0;
    return LBK_OK;
}

int lbk_tp_norm_quant(lbk_tp_comm *t, int pre, const float *x_dev, const float *y_dev, const float *w_dev, size_t m, size_t k_local,
                      size_t k_full, float eps, int8_t *q_dev, float *scale_dev, int32_t *sum_dev, void *stream) {
    if (!t) return fail(LBK_ERR_INVALID, "tensor-parallel communicator is null");
    TpComm *tc = reinterpret_cast<TpComm *>(t);
    if (pre != LBK_PRE_RMS && pre != LBK_PRE_RELU2_MUL_RMS) return fail(LBK_ERR_INVALID, "lbk_tp_norm_quant: transform %d (LBK_PRE_RMS or LBK_PRE_RELU2_MUL_RMS)", pre);
    if (m == 0 || m > kTpMaxRows) return fail(LBK_ERR_UNSUPPORTED, "lbk_tp_norm_quant takes 1..%d token rows (got %zu); every rank must take part", kTpMaxRows, m);
    if (!x_dev || !w_dev || !q_dev || !scale_dev || !sum_dev || (pre == LBK_PRE_RELU2_MUL_RMS && !y_dev)) return fail(LBK_ERR_INVALID, "lbk_tp_norm_quant: null buffer");
    if (k_local == 0 || k_local % 128 || k_local > static_cast<size_t>(kNqCache) * kNqThreads * 4 || k_full < k_local)
        return fail(LBK_ERR_UNSUPPORTED, "lbk_tp_norm_quant: the column slice must be a multiple of 128 columns, at most %d (got %zu of %zu)", kNqCache * kNqThreads * 4, k_local, k_full);
    if ((reinterpret_cast<uintptr_t>(x_dev) | reinterpret_cast<uintptr_t>(y_dev) | reinterpret_cast<uintptr_t>(w_dev) | reinterpret_cast<uintptr_t>(q_dev)) & 15)
        return fail(LBK_ERR_UNSUPPORTED, "lbk_tp_norm_quant needs 16-byte aligned buffers");
    LBK_CUDA(cudaSetDevice(tc->ctx->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const dim3 grid(static_cast<unsigned>(m));
    const bool small_blocks = m >= kTpManyRows && k_local <= static_cast<size_t>(kNqCache) * 256 * 4;
#define LBK_NQ_LAUNCH(PRE, T)                                                                                                                            \
    LBK_CUDA(launch_chained(tp_norm_quant_kernel<PRE, T>, grid, dim3(T), 0, st, ptrs_of(tc), tc->world, tc->rank, x_dev, y_dev, w_dev, static_cast<int>(k_local), \
                            static_cast<int>(k_full), eps, q_dev, scale_dev, sum_dev, tc->ctx->err_word, tc->wait_limit))
    if (m >= kTpManyRows && !small_blocks) {
        // long rows of a prompt pass: the row in shared memory
        const size_t smem = k_local * sizeof(float);
        static bool attr_set = false;  // the same values for every call; setting them twice is harmless
        if (!attr_set) {
            LBK_CUDA(cudaFuncSetAttribute(tp_norm_quant_smem_kernel<LBK_PRE_RMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, kNqCache * kNqThreads * 16));
            LBK_CUDA(cudaFuncSetAttribute(tp_norm_quant_smem_kernel<LBK_PRE_RELU2_MUL_RMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, kNqCache * kNqThreads * 16));
            attr_set = true;
        }
        if (pre == LBK_PRE_RMS)
            LBK_CUDA(launch_chained(tp_norm_quant_smem_kernel<LBK_PRE_RMS>, grid, dim3(kNqSmemThreads), smem, st, ptrs_of(tc), tc->world, tc->rank, x_dev, y_dev, w_dev,
                                    static_cast<int>(k_local), static_cast<int>(k_full), eps, q_dev, scale_dev, sum_dev, tc->ctx->err_word, tc->wait_limit));
        else
            LBK_CUDA(launch_chained(tp_norm_quant_smem_kernel<LBK_PRE_RELU2_MUL_RMS>, grid, dim3(kNqSmemThreads), smem, st, ptrs_of(tc), tc->world, tc->rank, x_dev, y_dev,
                                    w_dev, static_cast<int>(k_local), static_cast<int>(k_full), eps, q_dev, scale_dev, sum_dev, tc->ctx->err_word, tc->wait_limit));
    } else if (pre == LBK_PRE_RMS) {
        if (small_blocks) LBK_NQ_LAUNCH(LBK_PRE_RMS, 256);
        else LBK_NQ_LAUNCH(LBK_PRE_RMS, 1024);
    } else {
        if (small_blocks) LBK_NQ_LAUNCH(LBK_PRE_RELU2_MUL_RMS, 256);
        else LBK_NQ_LAUNCH(LBK_PRE_RELU2_MUL_RMS, 1024);
    }
#undef LBK_NQ_LAUNCH
    LBK_CUDA(cudaGetLastError());
    tc->ctx->launches++;
    return LBK_OK;
}

int lbk_tp_reduce_norm_gather(lbk_tp_comm *t, int flags, const float *ascale_dev, float wscale, float *xres_dev, const float *w_dev, float eps,
                              size_t m, size_t hidden, float *y_out_dev, void *stream) {
    if (!t) return fail(LBK_ERR_INVALID, "tensor-parallel communicator is null");
    TpComm *tc = reinterpret_cast<TpComm *>(t);
    const bool reduce = !(flags & LBK_TP_NO_REDUCE), f32 = (flags & LBK_TP_GATHER_F32) != 0, scattered = (flags & LBK_TP_SCATTERED) != 0;
    if (scattered && !reduce) return fail(LBK_ERR_INVALID, "lbk_tp_reduce_norm_gather: LBK_TP_SCATTERED goes with a reduction");
    if (m == 0 || m > kTpMaxRows || (f32 && m > kTpGatherFRows))
        return fail(LBK_ERR_UNSUPPORTED, "lbk_tp_reduce_norm_gather takes 1..%d token rows (%d when f32 rows are gathered), got %zu; every rank must take part", kTpMaxRows, kTpGatherFRows, m);
    if (hidden == 0 || hidden % 128 || hidden > kTpMaxWidth) return fail(LBK_ERR_UNSUPPORTED, "lbk_tp_reduce_norm_gather: rows of a multiple of 128 and at most %d columns (got %zu)", kTpMaxWidth, hidden);
    if (!xres_dev || !w_dev || (reduce && !ascale_dev)) return fail(LBK_ERR_INVALID, "lbk_tp_reduce_norm_gather: null buffer");
    if ((reinterpret_cast<uintptr_t>(xres_dev) | reinterpret_cast<uintptr_t>(w_dev) | reinterpret_cast<uintptr_t>(y_out_dev)) & 15)
        return fail(LBK_ERR_UNSUPPORTED, "lbk_tp_reduce_norm_gather needs 16-byte aligned buffers");
    LBK_CUDA(cudaSetDevice(tc->ctx->device));
    RgArgs a{};
    a.world = tc->world;
    a.rank = tc->rank;
    a.m = static_cast<int>(m);
    a.hidden = static_cast<int>(hidden);
    a.mt = static_cast<int>((m + tc->world - 1) / tc->world);
    a.reduce = reduce ? (scattered ? 2 : 1) : 0;
    a.gather_f32 = f32 ? 1 : 0;
    a.ascale = ascale_dev;
    a.wscale = wscale;
    a.xres = xres_dev;
    a.w = w_dev;
    a.eps = eps;
    a.y_out = y_out_dev;
    a.err_word = tc->ctx->err_word;
    a.wait_limit = tc->wait_limit;
    const int t0 = a.rank * a.mt, own = a.m - t0 < 0 ? 0 : (a.m - t0 < a.mt ? a.m - t0 : a.mt);
    const dim3 rgrid(static_cast<unsigned>(own > 0 ? own : 1));
    if (m >= kTpManyRows) LBK_CUDA(launch_chained(tp_reduce_norm_gather_kernel<256>, rgrid, dim3(256), 0, static_cast<cudaStream_t>(stream), ptrs_of(tc), a));
    else LBK_CUDA(launch_chained(tp_reduce_norm_gather_kernel<1024>, rgrid, dim3(1024), 0, static_cast<cudaStream_t>(stream), ptrs_of(tc), a));
    LBK_CUDA(cudaGetLastError());
    tc->ctx->launches++;
    return LBK_OK;
}

// The row-parallel projection with the first half of its exchange inside: the tcgen05 GEMM on this rank's
// column slice, whose epilogue stores the int32 dots of every token into the region of the rank that owns the
// token (peer stores; [source rank][token of the owner][row]). lbk_tp_reduce_norm_gather with LBK_TP_SCATTERED
// then adds up what arrived in its own region.
int lbk_tp_gemm_scatter(lbk_tp_comm *t, const lbk_weight *w, const int8_t *q_dev, const int32_t *sum_dev, size_t m, void *stream) {
    if (!t || !w) return fail(LBK_ERR_INVALID, "lbk_tp_gemm_scatter: null communicator or weight");
    TpComm *tc = reinterpret_cast<TpComm *>(t);
    const Weight *wt = reinterpret_cast<const Weight *>(w);
    if (m < 17 || m > kTpMaxRows) return fail(LBK_ERR_UNSUPPORTED, "lbk_tp_gemm_scatter takes 17..%d token rows (got %zu)", kTpMaxRows, m);
    if (!q_dev || !sum_dev) return fail(LBK_ERR_INVALID, "lbk_tp_gemm_scatter: null q/sum");
    const size_t mt = (m + tc->world - 1) / tc->world;
    if (wt->rows > kTpMaxWidth || static_cast<size_t>(tc->world) * mt * wt->rows * sizeof(int32_t) > kTpPartialBytes)
        return fail(LBK_ERR_UNSUPPORTED, "lbk_tp_gemm_scatter: %zu rows x %zu tokens do not fit the exchange buffer", static_cast<size_t>(wt->rows), m);
    LBK_CUDA(cudaSetDevice(tc->ctx->device));
    GroupArgs g;
    g.w[0] = wt;
    g.out[0] = nullptr;
    g.iout[0] = nullptr;
    g.n = 1;
    g.m = m;
    g.q = q_dev;
    g.qsum = sum_dev;
    g.scatter_world = tc->world;
    g.scatter_mt = static_cast<int>(mt);
    for (int o = 0; o < tc->world; ++o) g.scatter_base[o] = tc->region[o]->partial + static_cast<size_t>(tc->rank) * mt * wt->rows;
    return launch_gemm(tc->ctx, g, static_cast<cudaStream_t>(stream));
}

const int8_t *lbk_tp_gather_q(lbk_tp_comm *t) { return t ? reinterpret_cast<TpComm *>(t)->region[reinterpret_cast<TpComm *>(t)->rank]->gather_q : nullptr; }
const float *lbk_tp_gather_scale(lbk_tp_comm *t) { return t ? reinterpret_cast<TpComm *>(t)->region[reinterpret_cast<TpComm *>(t)->rank]->gather_scale : nullptr; }
const int32_t *lbk_tp_gather_sum(lbk_tp_comm *t) { return t ? reinterpret_cast<TpComm *>(t)->region[reinterpret_cast<TpComm *>(t)->rank]->gather_sum : nullptr; }
const float *lbk_tp_gather_f32(lbk_tp_comm *t) { return t ? reinterpret_cast<TpComm *>(t)->region[reinterpret_cast<TpComm *>(t)->rank]->gather_f : nullptr; }

int lbk_tp_argmax(lbk_tp_comm *t, const float *logits_local_dev, const int32_t *idx_local_dev, size_t m, size_t vocab_local, int32_t *next_dev, void *stream) {
    if (!t) return fail(LBK_ERR_INVALID, "tensor-parallel communicator is null");
    TpComm *tc = reinterpret_cast<TpComm *>(t);
    if (m == 0 || m > kTpMaxRows) return fail(LBK_ERR_UNSUPPORTED, "lbk_tp_argmax takes 1..%d token rows (got %zu)", kTpMaxRows, m);
    if (!logits_local_dev || !idx_local_dev || !next_dev || vocab_local == 0) return fail(LBK_ERR_INVALID, "lbk_tp_argmax: null buffer or empty slice");
    LBK_CUDA(cudaSetDevice(tc->ctx->device));
    LBK_CUDA(launch_chained(tp_argmax_kernel, dim3(1), dim3(1024), 0, static_cast<cudaStream_t>(stream), ptrs_of(tc), tc->world, tc->rank, logits_local_dev, idx_local_dev,
                            static_cast<int>(m), static_cast<int>(vocab_local), next_dev, tc->ctx->err_word, tc->wait_limit));
    LBK_CUDA(cudaGetLastError());
    tc->ctx->launches++;
    return LBK_OK;
}

}  // extern "C"
