// lbk_ternary_linear_prefill_static: the prefill form of the fused ternary op for callers that
// must not allocate device memory.
//
// Who needs this: code that runs where cudaMalloc is off limits -- inside a real-time or
// latency-critical serving loop that forbids allocator calls after start-up, under a memory
// budget owned by another component (an inference server that hands out every byte itself), or
// in a process whose CUDA context was set up by a host application that does not let plug-ins
// grow the heap. The regular entry point (lbk_ternary_linear_n) keeps the quantised activations
// of the prefill path in context scratch that grows on demand with cudaMalloc; this one keeps
// them in the fixed array below instead and calls nothing that allocates.
//
// The array is part of the library image: every GPU that loads liblbk.so holds its
// LBK_STATIC_SCRATCH_BYTES (8 MiB + 64 KiB) until the process exits, whether or not this entry
// point is ever called.
#include "lbk_internal.cuh"

namespace {

constexpr size_t kQBytes = 8u << 20;        // int8 activations: m * padded_cols(cols) <= 8 MiB
constexpr size_t kMaxTokens = 4096;         // per-token scale and sum live behind the activations
constexpr size_t kScaleOff = kQBytes;
constexpr size_t kSumOff = kQBytes + kMaxTokens * sizeof(float);
constexpr size_t kTotalBytes = kQBytes + 2 * kMaxTokens * sizeof(float);
static_assert(kTotalBytes == LBK_STATIC_SCRATCH_BYTES, "header and implementation disagree on the scratch size");

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device pointer.
static __device__ __align__(256) unsigned char g_static_scratch[kTotalBytes];

constexpr int kMaxDevices = 64;
void *g_scratch_addr[kMaxDevices] = {};  // device address of g_static_scratch, per device

// First use on a device: resolve the array's device address (with that device current).
int scratch_for_device(int device, unsigned char **out) {
    if (device < 0 || device >= kMaxDevices) return lbk::fail(LBK_ERR_UNSUPPORTED, "device index %d is beyond %d", device, kMaxDevices - 1);
    if (!g_scratch_addr[device]) {
        void *ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr)
            return lbk::fail(LBK_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed on device %d: %s", device, cudaGetErrorString(e));
        g_scratch_addr[device] = ptr;
    }
    *out = static_cast<unsigned char *>(g_scratch_addr[device]);
    return LBK_OK;
}

}  // namespace

extern "C" int lbk_ternary_linear_prefill_static(lbk_ctx *c, const float *x_dev, size_t m, const lbk_weight *const *ws, size_t n,
                                                 float *const *outs_dev, int32_t *const *iouts_dev, void *stream) {
    using namespace lbk;
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ws || n < 1 || n > LBK_MAX_GROUP) return fail(LBK_ERR_INVALID, "group of %zu matrices (1..%d allowed)", n, LBK_MAX_GROUP);
    GroupArgs g;
    g.n = static_cast<int>(n);
    g.m = m;
    for (size_t i = 0; i < n; ++i) {
        const Weight *w = reinterpret_cast<const Weight *>(ws[i]);
        if (!w) return fail(LBK_ERR_INVALID, "matrix %zu is null", i);
        if (w->ctx != ctx) return fail(LBK_ERR_INVALID, "matrix %zu belongs to another context", i);
        if (w->cols != reinterpret_cast<const Weight *>(ws[0])->cols)
            return fail(LBK_ERR_SHAPE, "inner dimension mismatch: matrix %zu has %zu columns, matrix 0 has %zu", i, w->cols,
                        reinterpret_cast<const Weight *>(ws[0])->cols);
        g.w[i] = w;
        g.out[i] = outs_dev ? outs_dev[i] : nullptr;
        g.iout[i] = iouts_dev ? iouts_dev[i] : nullptr;
        if (m && w->rows && !g.out[i] && !g.iout[i]) return fail(LBK_ERR_INVALID, "matrix %zu has no output buffer", i);
    }
    if (m == 0) return LBK_OK;
    const size_t cols = g.w[0]->cols, kp = g.w[0]->kp;
    if (cols == 0) return fail(LBK_ERR_UNSUPPORTED, "matrices without columns are not served by the static-scratch entry point");
    if (!x_dev) return fail(LBK_ERR_INVALID, "x_dev is null");
    if (m > kMaxTokens || m * kp > kQBytes)
        return fail(LBK_ERR_UNSUPPORTED,
                    "static scratch too small: %zu token rows x %zu padded columns = %zu bytes of int8 activations; "
                    "the limits are %zu bytes and %zu token rows (use lbk_ternary_linear_n, which allocates)",
                    m, kp, m * kp, kQBytes, kMaxTokens);
    LBK_CUDA(cudaSetDevice(ctx->device));
    unsigned char *scratch = nullptr;
    LBK_TRY(scratch_for_device(ctx->device, &scratch));
    int8_t *q = reinterpret_cast<int8_t *>(scratch);
    float *scale = reinterpret_cast<float *>(scratch + kScaleOff);
    int32_t *sum = reinterpret_cast<int32_t *>(scratch + kSumOff);
    // Nothing in the array has to start at zero: the quantiser overwrites every byte the GEMM
    // reads (all m rows, padding columns included, and m scales and sums); rows past m are never
    // read (the tensor map ends at row m).
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LBK_TRY(launch_quantize(ctx, x_dev, m, cols, q, scale, sum, st));
    g.q = q;
    g.qscale = scale;
    g.qsum = sum;
    return launch_gemm(ctx, g, st);
}
