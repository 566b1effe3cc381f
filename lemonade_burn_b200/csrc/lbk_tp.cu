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

namespace lbk {

constexpr int kTpMaxWorld = 8;
constexpr int kTpMaxTokens = 256;                   // token rows per call on the fused path
constexpr size_t kTpPartialBytes = 8u << 20;        // int32 partial dots of one call
constexpr uint32_t kTpWaitLimit = 1u << 24;         // default: polls of a peer's word before giving up (lbk_tp_comm_set_wait_limit)

// The same layout in every rank's region.
struct TpRegion {
    unsigned long long amax[2][kTpMaxWorld][kTpMaxTokens];  // (sequence << 32) | float bits, written by rank r
    unsigned int ready[kTpMaxWorld][32];                    // [r][0]: sequence of rank r's partial dots (padded)
    unsigned int q_seq, q_done, r_seq, r_done;              // this rank's own counters (never written by peers)
    unsigned int pad_[28];
    int32_t partial[kTpPartialBytes / 4];
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

}  // extern "C"
