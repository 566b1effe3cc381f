// C ABI of the lbk library: context, weights, the host-pointer entry points that mirror
// lb-ternary's public functions one to one, and the device-pointer fast path.
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "lbk_internal.cuh"

namespace lbk {

// ---- errors --------------------------------------------------------------------------
static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int fail(int status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}

// ---- tensor maps ---------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

static int encode_2d_u8(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer,
                        uint64_t pitch, uint32_t box_inner, uint32_t box_outer,
                        CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(LBK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {pitch};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LBK_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return LBK_OK;
}

int encode_weight_maps(Weight *w) {
    // GEMV: [16 rows][128 bytes] boxes with the 128-byte swizzle; rows/bytes past the matrix
    // edge are filled with zero bytes (code 0), which the kernels pair with zero activations.
    LBK_TRY(encode_2d_u8(&w->tmap_gemv, w->data, w->rb, w->rows, w->rb, 128, 16, CU_TENSOR_MAP_SWIZZLE_128B));
    // GEMM: [128 rows][128 bytes] boxes (four packed blocks per row) with the 128-byte swizzle.
    LBK_TRY(encode_2d_u8(&w->tmap_gemm, w->data, w->rb, w->rows, w->rb, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B));
    return LBK_OK;
}

// Quantised activations int8 [m][kp] as [box_rows][128 bytes] boxes with the 128-byte swizzle
// (the K-major operand layout of the tensor core); rows past m read as zeros.
int encode_act_map(CUtensorMap *map, const int8_t *q, size_t m, size_t kp, int box_rows) {
    return encode_2d_u8(map, q, kp, m, kp, 128, static_cast<uint32_t>(box_rows), CU_TENSOR_MAP_SWIZZLE_128B);
}

int encode_bytes_map(CUtensorMap *map, const void *base, size_t inner, size_t outer, size_t pitch, int box_inner, int box_outer) {
    return encode_2d_u8(map, base, inner, outer, pitch, static_cast<uint32_t>(box_inner), static_cast<uint32_t>(box_outer), CU_TENSOR_MAP_SWIZZLE_128B);
}

// Grow-only scratch. A block that has been handed out is never freed before the context is
// destroyed: a CUDA graph recorded by a caller (a decode step captured at 5..8 sequences, whose
// projections take the quantise + GEMM path) has this address baked in, and a later, larger request
// must not turn it into a dangling pointer. A larger request gets a new block; the old ones stay
// (each at least 1.25x its predecessor, so together they hold less than five times the largest).
int ctx_scratch(Ctx *ctx, size_t bytes, void **out) {
    if (bytes > ctx->scratch_bytes) {
        const size_t want = bytes + (bytes >> 2) + 4096;
        void *fresh = nullptr;
        cudaError_t e = cudaMalloc(&fresh, want);
        if (e != cudaSuccess) return fail(LBK_ERR_NOMEM, "cudaMalloc(%zu) failed: %s", want, cudaGetErrorString(e));
        if (ctx->scratch) ctx->retired_scratch.push_back(ctx->scratch);
        ctx->scratch = fresh;
        ctx->scratch_bytes = want;
    }
    *out = ctx->scratch;
    return LBK_OK;
}

// What a non-zero error word means. Code 7 is written by the decoder-step kernels when a position
// read from device memory lies outside the cache; every other code marks a bounded wait that ran out.
int device_error_status(int word) {
    if (word == 7)
        return fail(LBK_ERR_INVALID, "a decode position was outside its cache (position < 0 or >= capacity); the kernels of that step "
                                     "refused to run and its results are invalid");
    return fail(LBK_ERR_TIMEOUT, "a bounded device-side wait gave up (code %d); results of that launch are invalid", word);
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Carves `n` sub-buffers out of the context scratch (256-byte aligned each).
static int carve(Ctx *ctx, const size_t *sizes, int n, void **ptrs) {
    size_t total = 0;
    for (int i = 0; i < n; ++i) total += align_up(sizes[i], 256);
    void *base = nullptr;
    LBK_TRY(ctx_scratch(ctx, total, &base));
    size_t off = 0;
    for (int i = 0; i < n; ++i) {
        ptrs[i] = static_cast<char *>(base) + off;
        off += align_up(sizes[i], 256);
    }
    return LBK_OK;
}

static int check_group(const lbk_weight *const *ws, size_t n, const Ctx *ctx) {
    if (!ws || n < 1 || n > LBK_MAX_GROUP) return fail(LBK_ERR_INVALID, "group of %zu matrices (1..%d allowed)", n, LBK_MAX_GROUP);
    for (size_t i = 0; i < n; ++i) {
        const Weight *w = reinterpret_cast<const Weight *>(ws[i]);
        if (!w) return fail(LBK_ERR_INVALID, "matrix %zu is null", i);
        if (w->ctx != ctx) return fail(LBK_ERR_INVALID, "matrix %zu belongs to another context", i);
        if (w->cols != reinterpret_cast<const Weight *>(ws[0])->cols)
            return fail(LBK_ERR_SHAPE, "inner dimension mismatch: matrix %zu has %zu columns, matrix 0 has %zu",
                        i, w->cols, reinterpret_cast<const Weight *>(ws[0])->cols);
    }
    return LBK_OK;
}

// GEMV kernel or quantise + tcgen05 GEMM? The GEMV kernel streams the weights once per eight token
// rows and its arithmetic grows with the rows; the GEMM path costs two launches but is flat in m.
// Measured per call at 2B4T shapes (K 2560: q/k/v, o, gate/up; K 6912: down), GEMV against GEMM:
// 4 rows 5.7 / 9.2 us and 9.3 / 13.3 us; 8 rows 7.6 / 9.4 and 15.0 / 13.3; 9 rows 9.7 / 9.4 and
// 23.3 / 13.4; 16 rows 12.9 / 9.9 and 25.4 / 13.4. lbk_set_gemv_rows(ctx, n) replaces the rule by
// "GEMV up to n rows" on that context.
bool use_gemv(const Ctx *ctx, size_t kp, size_t m) {
    if (m > LBK_GEMV_MAX_M || !gemv_fits(ctx, kp, m)) return false;
    if (ctx->gemv_rows > 0) return m <= static_cast<size_t>(ctx->gemv_rows);
    return m <= 4 || (m <= 8 && kp < 4096);
}

// Dispatch of one fused group on device buffers: GEMV kernel for small m, else quantise (if
// needed) + the tcgen05 GEMM.
static int run_group(Ctx *ctx, GroupArgs g, cudaStream_t stream, int8_t *q_scratch, float *s_scratch,
                     int32_t *sum_scratch) {
    if (g.m == 0) return LBK_OK;
    const size_t kp = g.w[0]->kp;
    if (kp == 0) {  // no columns: every dot product is 0, and so is 0 * inv
        for (int i = 0; i < g.n; ++i) {
            const size_t cnt = g.m * g.w[i]->rows;
            if (g.out[i] && cnt) LBK_CUDA(cudaMemsetAsync(g.out[i], 0, cnt * sizeof(float), stream));
            if (g.iout[i] && cnt) LBK_CUDA(cudaMemsetAsync(g.iout[i], 0, cnt * sizeof(int32_t), stream));
        }
        return LBK_OK;
    }
    if (use_gemv(ctx, kp, g.m)) return launch_gemv(ctx, g, stream);
    if (g.x) {
        if (!q_scratch) return fail(LBK_ERR_INVALID, "internal: GEMM path needs quantiser scratch");
        LBK_TRY(launch_quantize(ctx, g.x, g.m, g.w[0]->cols, q_scratch, s_scratch, sum_scratch, stream));
        g.x = nullptr;
        g.q = q_scratch;
        g.qscale = s_scratch;
        g.qsum = sum_scratch;
    }
    return launch_gemm(ctx, g, stream);
}

}  // namespace lbk

using namespace lbk;

static Ctx *C_(lbk_ctx *c) { return reinterpret_cast<Ctx *>(c); }
static const Weight *W_(const lbk_weight *w) { return reinterpret_cast<const Weight *>(w); }

extern "C" {

const char *lbk_last_error(void) { return g_err; }
int lbk_abi_version(void) { return 1; }

size_t lbk_padded_cols(size_t cols) { return (cols + kBlock - 1) / kBlock * kBlock; }
size_t lbk_row_bytes(size_t cols) { return lbk_padded_cols(cols) / 4; }

int lbk_init(int device, lbk_ctx **out) {
    if (!out) return fail(LBK_ERR_INVALID, "lbk_init: out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(LBK_ERR_CUDA, "no CUDA device: %s", e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    if (device < 0 || device >= count) return fail(LBK_ERR_INVALID, "device %d out of range (0..%d)", device, count - 1);
    cudaDeviceProp prop;
    LBK_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(LBK_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
    LBK_CUDA(cudaSetDevice(device));
    Ctx *ctx = new (std::nothrow) Ctx();
    if (!ctx) return fail(LBK_ERR_NOMEM, "out of host memory");
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    if (cudaMalloc(&ctx->small_scratch, kSmallScratchBytes) != cudaSuccess || cudaMalloc(&ctx->err_word, sizeof(int)) != cudaSuccess || cudaMemset(ctx->err_word, 0, sizeof(int)) != cudaSuccess ||
        cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete ctx;
        return fail(LBK_ERR_CUDA, "context setup failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    int s = kernels_init(ctx);
    if (s != LBK_OK) {
        lbk_destroy(reinterpret_cast<lbk_ctx *>(ctx));
        return s;
    }
    *out = reinterpret_cast<lbk_ctx *>(ctx);
    return LBK_OK;
}

int lbk_destroy(lbk_ctx *c) {
    if (!c) return LBK_OK;
    Ctx *ctx = C_(c);
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    if (ctx->scratch) cudaFree(ctx->scratch);
    for (void *p : ctx->retired_scratch) cudaFree(p);
    if (ctx->err_word) cudaFree(ctx->err_word);
    if (ctx->small_scratch) cudaFree(ctx->small_scratch);
    if (ctx->gemm_acc) cudaFree(ctx->gemm_acc);
    if (ctx->bf16_x) cudaFree(ctx->bf16_x);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
    return LBK_OK;
}

int lbk_check_device_error(lbk_ctx *c) {
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    Ctx *ctx = C_(c);
    LBK_CUDA(cudaSetDevice(ctx->device));
    LBK_CUDA(cudaDeviceSynchronize());
    int word = 0;
    LBK_CUDA(cudaMemcpy(&word, ctx->err_word, sizeof(int), cudaMemcpyDeviceToHost));
    if (word != 0) {
        LBK_CUDA(cudaMemset(ctx->err_word, 0, sizeof(int)));
        // a launch that gave up may have left partial sums in the split-K buffer, which is zero at rest
        if (ctx->gemm_acc) LBK_CUDA(cudaMemset(ctx->gemm_acc, 0, kGemmAccBytes));
        return device_error_status(word);
    }
    return LBK_OK;
}

int lbk_set_gemv_rows(lbk_ctx *c, int rows) {
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    if (rows < 0 || rows > LBK_GEMV_MAX_M) return fail(LBK_ERR_INVALID, "lbk_set_gemv_rows: %d is outside 0..%d", rows, LBK_GEMV_MAX_M);
    C_(c)->gemv_rows = rows;
    return LBK_OK;
}

uint64_t lbk_launch_count(const lbk_ctx *c) { return c ? reinterpret_cast<const Ctx *>(c)->launches : 0; }

// ---- weights -------------------------------------------------------------------------

static int make_weight(Ctx *ctx, size_t rows, size_t cols, const void *dev, bool owned, float scale, lbk_weight **out) {
    Weight *w = new (std::nothrow) Weight();
    if (!w) return fail(LBK_ERR_NOMEM, "out of host memory");
    w->ctx = ctx;
    w->rows = rows;
    w->cols = cols;
    w->kp = lbk_padded_cols(cols);
    w->rb = w->kp / 4;
    w->data = static_cast<const uint8_t *>(dev);
    w->owned = owned;
    w->scale = scale;
    if (rows > 0 && cols > 0) {
        int s = encode_weight_maps(w);
        if (s != LBK_OK) {
            delete w;
            return s;
        }
    }
    *out = reinterpret_cast<lbk_weight *>(w);
    return LBK_OK;
}

static int check_dims(size_t rows, size_t cols) {
    if (rows > (1u << 30) || cols > (1u << 18))
        return fail(LBK_ERR_UNSUPPORTED, "matrix %zu x %zu exceeds the supported size (rows <= 2^30, cols <= 2^18)", rows, cols);
    return LBK_OK;
}

int lbk_weight_upload(lbk_ctx *c, size_t rows, size_t cols, const uint8_t *packed, size_t packed_len, float scale,
                      lbk_weight **out) {
    if (!c || !out) return fail(LBK_ERR_INVALID, "lbk_weight_upload: null argument");
    *out = nullptr;
    Ctx *ctx = C_(c);
    LBK_TRY(check_dims(rows, cols));
    const size_t need = rows * lbk_row_bytes(cols);
    if (packed_len != need)  // pack.rs:40
        return fail(LBK_ERR_SHAPE, "packed data length mismatch: got %zu bytes, %zu x %zu needs %zu", packed_len, rows, cols, need);
    if (need && !packed) return fail(LBK_ERR_INVALID, "packed is null");
    LBK_CUDA(cudaSetDevice(ctx->device));
    void *dev = nullptr;
    if (need) {
        cudaError_t e = cudaMalloc(&dev, need);
        if (e != cudaSuccess) return fail(LBK_ERR_NOMEM, "cudaMalloc(%zu) failed: %s", need, cudaGetErrorString(e));
        e = cudaMemcpy(dev, packed, need, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) {
            cudaFree(dev);
            return fail(LBK_ERR_CUDA, "upload failed: %s", cudaGetErrorString(e));
        }
    }
    int s = make_weight(ctx, rows, cols, dev, true, scale, out);
    if (s != LBK_OK && dev) cudaFree(dev);
    return s;
}

int lbk_weight_wrap(lbk_ctx *c, size_t rows, size_t cols, const void *packed_dev, float scale, lbk_weight **out) {
    if (!c || !out) return fail(LBK_ERR_INVALID, "lbk_weight_wrap: null argument");
    *out = nullptr;
    LBK_TRY(check_dims(rows, cols));
    if (rows * cols && !packed_dev) return fail(LBK_ERR_INVALID, "packed_dev is null");
    if (reinterpret_cast<uintptr_t>(packed_dev) & 15) return fail(LBK_ERR_INVALID, "packed_dev must be 16-byte aligned");
    LBK_CUDA(cudaSetDevice(C_(c)->device));
    return make_weight(C_(c), rows, cols, packed_dev, false, scale, out);
}

int lbk_weight_free(lbk_weight *w_) {
    if (!w_) return LBK_OK;
    Weight *w = reinterpret_cast<Weight *>(w_);
    if (w->owned && w->data) {
        cudaSetDevice(w->ctx->device);
        cudaFree(const_cast<uint8_t *>(w->data));
    }
    delete w;
    return LBK_OK;
}

int lbk_weight_download(const lbk_weight *w_, uint8_t *packed_out, size_t len) {
    if (!w_ || (len && !packed_out)) return fail(LBK_ERR_INVALID, "lbk_weight_download: null argument");
    const Weight *w = W_(w_);
    if (len != w->rows * w->rb) return fail(LBK_ERR_SHAPE, "packed data length mismatch: got %zu bytes, %zu x %zu needs %zu", len, w->rows, w->cols, w->rows * w->rb);
    if (len == 0) return LBK_OK;
    LBK_CUDA(cudaSetDevice(w->ctx->device));
    LBK_CUDA(cudaMemcpy(packed_out, w->data, len, cudaMemcpyDeviceToHost));
    return LBK_OK;
}

size_t lbk_weight_rows(const lbk_weight *w) { return w ? W_(w)->rows : 0; }
size_t lbk_weight_cols(const lbk_weight *w) { return w ? W_(w)->cols : 0; }
float lbk_weight_scale(const lbk_weight *w) { return w ? W_(w)->scale : 0.0f; }
const void *lbk_weight_data(const lbk_weight *w) { return w ? W_(w)->data : nullptr; }

// ---- device-pointer entry points -----------------------------------------------------

int lbk_quantize_acts_dev(lbk_ctx *c, const float *x_dev, size_t m, size_t k, int8_t *q_dev, float *scale_dev,
                          int32_t *sum_dev, void *stream) {
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    if (m && (!q_dev || !scale_dev || !sum_dev || (k && !x_dev))) return fail(LBK_ERR_INVALID, "lbk_quantize_acts_dev: null buffer");
    LBK_CUDA(cudaSetDevice(C_(c)->device));
    return launch_quantize(C_(c), x_dev, m, k, q_dev, scale_dev, sum_dev, static_cast<cudaStream_t>(stream));
}

int lbk_absmax_dev(lbk_ctx *c, const float *x_dev, size_t m, size_t k, float *amax_dev, void *stream) {
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    if (m && (!amax_dev || (k && !x_dev))) return fail(LBK_ERR_INVALID, "lbk_absmax_dev: null buffer");
    LBK_CUDA(cudaSetDevice(C_(c)->device));
    return launch_quantize_ex(C_(c), x_dev, m, k, nullptr, nullptr, nullptr, nullptr, amax_dev, static_cast<cudaStream_t>(stream));
}

int lbk_quantize_acts_amax_dev(lbk_ctx *c, const float *x_dev, size_t m, size_t k, const float *amax_dev, int8_t *q_dev,
                               float *scale_dev, int32_t *sum_dev, void *stream) {
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    if (m && (!q_dev || !scale_dev || !sum_dev || !amax_dev || (k && !x_dev))) return fail(LBK_ERR_INVALID, "lbk_quantize_acts_amax_dev: null buffer");
    LBK_CUDA(cudaSetDevice(C_(c)->device));
    return launch_quantize_ex(C_(c), x_dev, m, k, q_dev, scale_dev, sum_dev, amax_dev, nullptr, static_cast<cudaStream_t>(stream));
}

int lbk_scale_epilogue_dev(lbk_ctx *c, const int32_t *dots_dev, const float *scale_dev, float wscale, size_t m, size_t rows,
                           float *out_dev, void *stream) {
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    if (m * rows && (!dots_dev || !scale_dev || !out_dev)) return fail(LBK_ERR_INVALID, "lbk_scale_epilogue_dev: null buffer");
    LBK_CUDA(cudaSetDevice(C_(c)->device));
    return launch_scale_epilogue(C_(c), dots_dev, scale_dev, wscale, m, rows, out_dev, static_cast<cudaStream_t>(stream));
}

static int fill_group(GroupArgs &g, const lbk_weight *const *ws, size_t n, float *const *outs, int32_t *const *iouts, size_t m) {
    g.n = static_cast<int>(n);
    g.m = m;
    for (size_t i = 0; i < n; ++i) {
        g.w[i] = W_(ws[i]);
        g.out[i] = outs ? outs[i] : nullptr;
        g.iout[i] = iouts ? iouts[i] : nullptr;
        if (m && g.w[i]->rows && !g.out[i] && !g.iout[i]) return fail(LBK_ERR_INVALID, "matrix %zu has no output buffer", i);
    }
    return LBK_OK;
}

int lbk_ternary_linear_n(lbk_ctx *c, const float *x_dev, size_t m, const lbk_weight *const *ws, size_t n,
                         float *const *outs_dev, int32_t *const *iouts_dev, void *stream) {
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    Ctx *ctx = C_(c);
    LBK_TRY(check_group(ws, n, ctx));
    if (m && W_(ws[0])->cols && !x_dev) return fail(LBK_ERR_INVALID, "x_dev is null");
    LBK_CUDA(cudaSetDevice(ctx->device));
    GroupArgs g;
    LBK_TRY(fill_group(g, ws, n, outs_dev, iouts_dev, m));
    g.x = x_dev;
    int8_t *q = nullptr;
    float *s = nullptr;
    int32_t *sum = nullptr;
    const size_t kp = g.w[0]->kp;
    if (!use_gemv(ctx, kp, m)) {
        // GEMM path: quantised activations go through context scratch. The scratch is shared
        // by every call on this context, so such calls must be issued on one stream.
        size_t sizes[3] = {m * kp, m * sizeof(float), m * sizeof(int32_t)};
        void *ptrs[3];
        LBK_TRY(carve(ctx, sizes, 3, ptrs));
        q = static_cast<int8_t *>(ptrs[0]);
        s = static_cast<float *>(ptrs[1]);
        sum = static_cast<int32_t *>(ptrs[2]);
    }
    return run_group(ctx, g, static_cast<cudaStream_t>(stream), q, s, sum);
}

int lbk_ternary_linear_pre_supported(size_t m, size_t cols) { return gemv_pre_supported(m, cols) ? 1 : 0; }

int lbk_ternary_linear_pre(lbk_ctx *c, int pre, const float *x_dev, const float *y_dev, const float *w_dev, float eps, float *xout_dev,
                           size_t m, const lbk_weight *const *ws, size_t n, float *const *outs_dev, int32_t *const *iouts_dev,
                           void *stream) {
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    Ctx *ctx = C_(c);
    LBK_TRY(check_group(ws, n, ctx));
    if (pre != LBK_PRE_RMS && pre != LBK_PRE_ADD_RMS && pre != LBK_PRE_RELU2_MUL_RMS) return fail(LBK_ERR_INVALID, "unknown input transform %d", pre);
    if (m == 0) return LBK_OK;
    if (!x_dev || !w_dev || (pre != LBK_PRE_RMS && !y_dev) || (pre == LBK_PRE_ADD_RMS && !xout_dev))
        return fail(LBK_ERR_INVALID, "lbk_ternary_linear_pre: null buffer");
    if ((reinterpret_cast<uintptr_t>(x_dev) | reinterpret_cast<uintptr_t>(y_dev) | reinterpret_cast<uintptr_t>(w_dev) |
         reinterpret_cast<uintptr_t>(xout_dev)) & 15)
        return fail(LBK_ERR_UNSUPPORTED, "lbk_ternary_linear_pre needs 16-byte aligned buffers");
    const size_t cols = W_(ws[0])->cols;
    if (!gemv_pre_supported(m, cols) || !gemv_fits(ctx, W_(ws[0])->kp, m))
        return fail(LBK_ERR_UNSUPPORTED, "lbk_ternary_linear_pre: %zu token rows of %zu columns are not supported", m, cols);
    LBK_CUDA(cudaSetDevice(ctx->device));
    GroupArgs g;
    LBK_TRY(fill_group(g, ws, n, outs_dev, iouts_dev, m));
    g.x = x_dev;
    g.pre = pre;
    g.pre_y = y_dev;
    g.pre_w = w_dev;
    g.pre_xout = xout_dev;
    g.pre_eps = eps;
    return launch_gemv(ctx, g, static_cast<cudaStream_t>(stream));
}

int lbk_ternary_gemm_dev(lbk_ctx *c, const lbk_weight *const *ws, size_t n, const int8_t *q_dev, const float *scale_dev,
                         const int32_t *sum_dev, size_t m, float *const *outs_dev, int32_t *const *iouts_dev, void *stream) {
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    Ctx *ctx = C_(c);
    LBK_TRY(check_group(ws, n, ctx));
    if (m && (!q_dev || !sum_dev)) return fail(LBK_ERR_INVALID, "lbk_ternary_gemm_dev: null q/sum");
    if (m && outs_dev && !scale_dev) return fail(LBK_ERR_INVALID, "f32 outputs need the activation scales");
    LBK_CUDA(cudaSetDevice(ctx->device));
    GroupArgs g;
    LBK_TRY(fill_group(g, ws, n, outs_dev, iouts_dev, m));
    g.q = q_dev;
    g.qscale = scale_dev;
    g.qsum = sum_dev;
    return run_group(ctx, g, static_cast<cudaStream_t>(stream), nullptr, nullptr, nullptr);
}

int lbk_bf16_linear(lbk_ctx *c, const float *x_dev, size_t m, const uint16_t *w_dev, size_t rows, size_t cols,
                    float *out_dev, void *stream) {
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    if (m * rows && (!out_dev || (cols && (!x_dev || !w_dev)))) return fail(LBK_ERR_INVALID, "lbk_bf16_linear: null buffer");
    LBK_CUDA(cudaSetDevice(C_(c)->device));
    return launch_bf16_linear(C_(c), x_dev, m, w_dev, rows, cols, out_dev, static_cast<cudaStream_t>(stream));
}

// ---- host-pointer entry points -------------------------------------------------------

int lbk_quantize_acts(lbk_ctx *c, const float *x, size_t m, size_t k, int8_t *q, float *scale, int32_t *sum) {
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    if (m == 0) return LBK_OK;
    if (!q || !scale || !sum || (k && !x)) return fail(LBK_ERR_INVALID, "lbk_quantize_acts: null buffer");
    Ctx *ctx = C_(c);
    LBK_CUDA(cudaSetDevice(ctx->device));
    const size_t kp = lbk_padded_cols(k);
    size_t sizes[4] = {m * k * sizeof(float), m * kp, m * sizeof(float), m * sizeof(int32_t)};
    void *d[4];
    LBK_TRY(carve(ctx, sizes, 4, d));
    cudaStream_t st = ctx->own_stream;
    if (m * k) LBK_CUDA(cudaMemcpyAsync(d[0], x, sizes[0], cudaMemcpyHostToDevice, st));
    LBK_TRY(launch_quantize(ctx, static_cast<float *>(d[0]), m, k, static_cast<int8_t *>(d[1]), static_cast<float *>(d[2]),
                            static_cast<int32_t *>(d[3]), st));
    if (m * kp) LBK_CUDA(cudaMemcpyAsync(q, d[1], sizes[1], cudaMemcpyDeviceToHost, st));
    LBK_CUDA(cudaMemcpyAsync(scale, d[2], sizes[2], cudaMemcpyDeviceToHost, st));
    LBK_CUDA(cudaMemcpyAsync(sum, d[3], sizes[3], cudaMemcpyDeviceToHost, st));
    LBK_CUDA(cudaStreamSynchronize(st));
    return LBK_OK;
}

// Shared body of the host-pointer GEMM entry points. Exactly one of x / (q, sum) is given.
static int host_group(Ctx *ctx, const lbk_weight *const *ws, size_t n, size_t m, bool from_x, const float *x,
                      const int8_t *q, const float *scale, const int32_t *sum, float *const *outs,
                      int32_t *const *iouts) {
    LBK_TRY(check_group(ws, n, ctx));
    if (m == 0) return LBK_OK;
    LBK_CUDA(cudaSetDevice(ctx->device));
    const size_t cols = W_(ws[0])->cols, kp = W_(ws[0])->kp;
    // scratch: [x f32 | q | scale | sum | per matrix f32 out, i32 out]
    std::vector<size_t> sizes;
    sizes.push_back(m * cols * sizeof(float));
    sizes.push_back(m * kp);
    sizes.push_back(m * sizeof(float));
    sizes.push_back(m * sizeof(int32_t));
    for (size_t i = 0; i < n; ++i) {
        sizes.push_back(m * W_(ws[i])->rows * sizeof(float));
        sizes.push_back(m * W_(ws[i])->rows * sizeof(int32_t));
    }
    std::vector<void *> d(sizes.size());
    LBK_TRY(carve(ctx, sizes.data(), static_cast<int>(sizes.size()), d.data()));
    cudaStream_t st = ctx->own_stream;
    GroupArgs g;
    g.n = static_cast<int>(n);
    g.m = m;
    for (size_t i = 0; i < n; ++i) {
        g.w[i] = W_(ws[i]);
        g.out[i] = (outs && outs[i]) ? static_cast<float *>(d[4 + 2 * i]) : nullptr;
        g.iout[i] = (iouts && iouts[i]) ? static_cast<int32_t *>(d[5 + 2 * i]) : nullptr;
        if (g.w[i]->rows && !g.out[i] && !g.iout[i]) return fail(LBK_ERR_INVALID, "matrix %zu has no output buffer", i);
    }
    if (from_x) {
        if (m * cols) LBK_CUDA(cudaMemcpyAsync(d[0], x, sizes[0], cudaMemcpyHostToDevice, st));
        g.x = static_cast<float *>(d[0]);
    } else {
        if (m * kp) LBK_CUDA(cudaMemcpyAsync(d[1], q, sizes[1], cudaMemcpyHostToDevice, st));
        LBK_CUDA(cudaMemcpyAsync(d[3], sum, sizes[3], cudaMemcpyHostToDevice, st));
        if (scale) LBK_CUDA(cudaMemcpyAsync(d[2], scale, sizes[2], cudaMemcpyHostToDevice, st));
        g.q = static_cast<int8_t *>(d[1]);
        g.qsum = static_cast<int32_t *>(d[3]);
        g.qscale = scale ? static_cast<float *>(d[2]) : nullptr;
    }
    LBK_TRY(run_group(ctx, g, st, static_cast<int8_t *>(d[1]), static_cast<float *>(d[2]), static_cast<int32_t *>(d[3])));
    for (size_t i = 0; i < n; ++i) {
        const size_t cnt = m * g.w[i]->rows;
        if (!cnt) continue;
        if (g.out[i]) LBK_CUDA(cudaMemcpyAsync(outs[i], g.out[i], cnt * sizeof(float), cudaMemcpyDeviceToHost, st));
        if (g.iout[i]) LBK_CUDA(cudaMemcpyAsync(iouts[i], g.iout[i], cnt * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    }
    LBK_CUDA(cudaStreamSynchronize(st));
    int word = 0;
    LBK_CUDA(cudaMemcpy(&word, ctx->err_word, sizeof(int), cudaMemcpyDeviceToHost));
    if (word) {
        LBK_CUDA(cudaMemset(ctx->err_word, 0, sizeof(int)));
        if (ctx->gemm_acc) LBK_CUDA(cudaMemset(ctx->gemm_acc, 0, kGemmAccBytes));
        return device_error_status(word);
    }
    return LBK_OK;
}

int lbk_ternary_gemm_i32(lbk_ctx *c, const lbk_weight *w, const int8_t *q, const int32_t *sum, size_t m, int32_t *out) {
    if (!c || !w) return fail(LBK_ERR_INVALID, "lbk_ternary_gemm_i32: null handle");
    if (m && (!q || !sum || !out)) return fail(LBK_ERR_INVALID, "lbk_ternary_gemm_i32: null buffer");
    const lbk_weight *ws[1] = {w};
    int32_t *iouts[1] = {out};
    return host_group(C_(c), ws, 1, m, false, nullptr, q, nullptr, sum, nullptr, iouts);
}

int lbk_ternary_gemm_multi(lbk_ctx *c, const lbk_weight *const *ws, size_t n, const int8_t *q, const float *scale,
                           const int32_t *sum, size_t m, float *const *outs) {
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    if (m && (!q || !scale || !sum || !outs)) return fail(LBK_ERR_INVALID, "lbk_ternary_gemm_multi: null buffer");
    return host_group(C_(c), ws, n, m, false, nullptr, q, scale, sum, outs, nullptr);
}

int lbk_ternary_linear_host(lbk_ctx *c, const float *x, size_t m, const lbk_weight *const *ws, size_t n, float *const *outs,
                            int32_t *const *iouts) {
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    if (m && !x && ws && n && ws[0] && W_(ws[0])->cols) return fail(LBK_ERR_INVALID, "x is null");
    if (m && !outs && !iouts) return fail(LBK_ERR_INVALID, "no output buffers");
    return host_group(C_(c), ws, n, m, true, x, nullptr, nullptr, nullptr, outs, iouts);
}

int lbk_bf16_gemv_host(lbk_ctx *c, const uint16_t *w, size_t rows, size_t cols, const float *x, float *out) {
    if (!c) return fail(LBK_ERR_INVALID, "context is null");
    if (rows == 0) return LBK_OK;
    if (!out || (cols && (!w || !x))) return fail(LBK_ERR_INVALID, "lbk_bf16_gemv_host: null buffer");
    Ctx *ctx = C_(c);
    LBK_CUDA(cudaSetDevice(ctx->device));
    size_t sizes[3] = {rows * cols * sizeof(uint16_t), cols * sizeof(float), rows * sizeof(float)};
    void *d[3];
    LBK_TRY(carve(ctx, sizes, 3, d));
    cudaStream_t st = ctx->own_stream;
    if (rows * cols) {
        LBK_CUDA(cudaMemcpyAsync(d[0], w, sizes[0], cudaMemcpyHostToDevice, st));
        LBK_CUDA(cudaMemcpyAsync(d[1], x, sizes[1], cudaMemcpyHostToDevice, st));
    }
    LBK_TRY(launch_bf16_linear(ctx, static_cast<float *>(d[1]), 1, static_cast<uint16_t *>(d[0]), rows, cols,
                               static_cast<float *>(d[2]), st));
    LBK_CUDA(cudaMemcpyAsync(out, d[2], sizes[2], cudaMemcpyDeviceToHost, st));
    LBK_CUDA(cudaStreamSynchronize(st));
    return LBK_OK;
}

}  // extern "C"
