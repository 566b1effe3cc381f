// Internal declarations shared by the lbk translation units (not part of the C ABI).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <utility>
#include <vector>

#include "lbk.h"

namespace lbk {

constexpr int kBlock = 128;      // weights per packed block (pack.rs:18)
constexpr int kBlockBytes = 32;  // bytes per packed block   (pack.rs:19)

// ---- error plumbing ------------------------------------------------------------------
void set_error(const char *fmt, ...);
int fail(int status, const char *fmt, ...);

#define LBK_CUDA(expr)                                                                       \
    do {                                                                                     \
        cudaError_t e__ = (expr);                                                            \
        if (e__ != cudaSuccess)                                                              \
            return ::lbk::fail(LBK_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                 \
                               cudaGetErrorString(e__), __FILE__, __LINE__);                 \
    } while (0)

#define LBK_TRY(expr)                \
    do {                             \
        int s__ = (expr);            \
        if (s__ != LBK_OK) return s__; \
    } while (0)

constexpr size_t kSmallScratchBytes = 64 * 1024;
constexpr size_t kGemmAccBytes = 32u << 20;

// ---- handles -------------------------------------------------------------------------
struct Ctx {
    int device = 0;
    int sm_count = 0;
    size_t smem_optin = 0;
    int *err_word = nullptr;     // device: non-zero once a bounded wait gave up
    uint64_t launches = 0;
    // grow-only device scratch for the host-pointer entry points and the GEMM pre-pass
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    std::vector<void *> retired_scratch;  // earlier, smaller scratch blocks: kept until lbk_destroy (recorded graphs may point into them)
    cudaStream_t own_stream = nullptr;  // used by the host-pointer entry points
    void *bf16_x = nullptr;             // allocated once at init: the bf16 head's activations as two bf16 terms (one pass of 64 token rows)
    void *small_scratch = nullptr;      // kSmallScratchBytes, allocated once at init (reductions)
    int32_t *gemm_acc = nullptr;        // kGemmAccBytes, allocated once at init: int32 sums of a prefill GEMM split along K
    int gemv_rows = 0;                  // lbk_set_gemv_rows: 0 = measured rule, n = fused kernel up to n token rows
};

struct Weight {
    Ctx *ctx = nullptr;
    size_t rows = 0, cols = 0, kp = 0, rb = 0;
    const uint8_t *data = nullptr;  // device
    bool owned = false;
    float scale = 1.0f;
    alignas(64) CUtensorMap tmap_gemv;  // box [16 rows][128 B], SWIZZLE_128B
    alignas(64) CUtensorMap tmap_gemm;  // box [128 rows][128 B], SWIZZLE_128B (prefill expander)
};

int ctx_scratch(Ctx *ctx, size_t bytes, void **out);
int device_error_status(int word);  // status and message for a non-zero error word
// One-time per-context kernel attribute set-up (opt-in shared memory sizes).
int kernels_init(Ctx *ctx);
int gemv_init(Ctx *ctx);
int gemm_init(Ctx *ctx);
int sweep_init(Ctx *ctx);
int encode_weight_maps(Weight *w);
int encode_act_map(CUtensorMap *map, const int8_t *q, size_t m, size_t kp, int box_rows);
// bytes [outer][inner] with row pitch `pitch`, boxes [box_outer][box_inner bytes], 128-byte swizzle, zeros past the edges
int encode_bytes_map(CUtensorMap *map, const void *base, size_t inner, size_t outer, size_t pitch, int box_inner, int box_outer);

// ---- launchers -----------------------------------------------------------------------
struct GroupArgs {
    const Weight *w[LBK_MAX_GROUP];
    float *out[LBK_MAX_GROUP];
    int32_t *iout[LBK_MAX_GROUP];
    int n = 0;
    size_t m = 0;
    // tcgen05 GEMM only, one matrix: the int32 dots of token row t go to scatter_base[t / scatter_mt] at row
    // t % scatter_mt instead of iout (the tensor-parallel layers: the bases are the token owners' buffers, peer memory)
    int scatter_world = 0, scatter_mt = 0;
    int32_t *scatter_base[8] = {};
    // exactly one of x (f32, quantised inside the kernel) or q/scale/sum is set
    const float *x = nullptr;
    const int8_t *q = nullptr;
    const float *qscale = nullptr;
    const int32_t *qsum = nullptr;
    // Optional transform of the f32 input inside the decode kernel (decoder step, model.rs:331-366):
    // LBK_PRE_RMS            x' = rms_norm(x) * pre_w
    // LBK_PRE_ADD_RMS        s = x + pre_y (written to pre_xout by one CTA), x' = rms_norm(s) * pre_w
    // LBK_PRE_RELU2_MUL_RMS  s = relu(x)^2 * pre_y, x' = rms_norm(s) * pre_w
    int pre = 0;
    const float *pre_y = nullptr;
    const float *pre_w = nullptr;
    float *pre_xout = nullptr;
    float pre_eps = 0.0f;
};
bool gemv_pre_supported(size_t m, size_t cols);

// Launch with programmatic stream serialisation: the grid may be scheduled while the previous
// kernel of the stream drains; the kernel orders itself with ptx::pdl_wait().
template <typename... KArgs, typename... Args>
cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Fused GEMV kernel (m <= LBK_GEMV_MAX_M). Returns LBK_ERR_UNSUPPORTED when the quantised
// activations do not fit in shared memory next to the weight ring.
int launch_gemv(Ctx *ctx, const GroupArgs &g, cudaStream_t stream);
bool gemv_fits(const Ctx *ctx, size_t kp, size_t m);

int gemv_xq_stride(size_t kp);

// Persistent sweep over recorded groups (lbk_sweep.cu).
struct SweepTables;
int sweep_build(Ctx *ctx, const std::vector<GroupArgs> &groups, SweepTables **out);
int sweep_launch(Ctx *ctx, const SweepTables *tb, cudaStream_t stream);
void sweep_free(SweepTables *tb);

int launch_quantize(Ctx *ctx, const float *x, size_t m, size_t k, int8_t *q, float *scale,
                    int32_t *sum, cudaStream_t stream);

int launch_quantize_ex(Ctx *ctx, const float *x, size_t m, size_t k, int8_t *q, float *scale, int32_t *sum,
                       const float *amax_in, float *amax_out, cudaStream_t stream);
int launch_scale_epilogue(Ctx *ctx, const int32_t *dots, const float *ascale, float wscale, size_t m, size_t rows,
                          float *out, cudaStream_t stream);

int launch_scale_epilogue_group(Ctx *ctx, int n, int32_t *const *dots, float *const *outs, const float *wscale, const int *rows, const bool *clean,
                                const float *ascale, size_t m, cudaStream_t stream);

// tcgen05 int8 GEMM on quantised inputs (any m).
int launch_gemm(Ctx *ctx, const GroupArgs &g, cudaStream_t stream);

int bf16_init(Ctx *ctx);

// causal attention of a prompt pass on tcgen05 (head_dim 128)
int attn_tc_init(Ctx *ctx);
int launch_attn_prompt_tc(Ctx *ctx, const float *q, const uint16_t *kc, const uint16_t *vc, const int32_t *pos_dev, size_t n, size_t nh, size_t kvh,
                          size_t cap, size_t seq, float *out, cudaStream_t stream);
int launch_bf16_linear(Ctx *ctx, const float *x, size_t m, const uint16_t *w, size_t rows,
                       size_t cols, float *out, cudaStream_t stream);

}  // namespace lbk
