/*
 * lbk — B200 (sm_100a) kernels for lemonade-burn's packed 2-bit ternary x int8 matmul path.
 *
 * Plain C ABI: pointers and sizes only. Every entry point returns an lbk_status; nothing
 * throws or aborts across the boundary. `lbk_last_error()` gives the message of the last
 * failure on the calling thread. The reference (Rust) panics via assert! on shape/dtype
 * mismatch (crates/lb-ternary/src/pack.rs:40, gemm.rs:129-134,197-200;
 * crates/lb-model/src/ops.rs:232,303-308): a binding turns a non-zero status into the same
 * panic / Err.
 *
 * Layout contract (crates/lb-ternary/src/pack.rs:1-24): a weight matrix W[rows, cols] is
 * row-major packed, cols padded to a multiple of 128; each 128-weight block is 32 bytes;
 * byte j of a block holds in bits 2k..2k+1 the code (w + 1) of column block*128 + k*32 + j.
 * One f32 scale per matrix = 1 / mean|W|. Activations are f32 [m, cols] row-major.
 * Outputs are [m, rows] row-major (x @ W^T), as in gemm.rs:117.
 *
 * Threading: one caller thread at a time per context (the reference drives its kernels from
 * one model thread, crates/lb-server/src/main.rs:385-387). Device-pointer entry points are
 * asynchronous on the given stream; host-pointer entry points synchronise before returning.
 */
#ifndef LBK_H
#define LBK_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum lbk_status {
    LBK_OK = 0,
    LBK_ERR_INVALID = 1,     /* null pointer, bad handle, bad count */
    LBK_ERR_SHAPE = 2,       /* a shape/length the reference would assert on */
    LBK_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed */
    LBK_ERR_UNSUPPORTED = 4, /* valid request outside what the kernels cover (size limits) */
    LBK_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up; results are invalid */
    LBK_ERR_NOMEM = 6
} lbk_status;

typedef struct lbk_ctx lbk_ctx;       /* one per device; owns scratch and the error word   */
typedef struct lbk_weight lbk_weight; /* a packed ternary matrix resident in device memory */
typedef struct lbk_plan lbk_plan;     /* a recorded sequence of fused ternary-linear groups */

#define LBK_MAX_GROUP 4   /* matrices sharing one input in a fused call (q/k/v, gate/up)  */
#define LBK_GEMV_MAX_M 16 /* token rows served by the bandwidth-bound GEMV kernel         */

/* Message of the last failure on this thread ("" if none). Never NULL. */
const char *lbk_last_error(void);
/* ABI version, bumped on any signature change. */
int lbk_abi_version(void);

/* ---- context --------------------------------------------------------------------------- */

/* Creates a context on CUDA device `device`. Fails with LBK_ERR_UNSUPPORTED unless the
 * device is compute capability 10.x. No counterpart in the reference (CPU only). */
int lbk_init(int device, lbk_ctx **out);
int lbk_destroy(lbk_ctx *ctx);
/* Reads and clears the device-side error word. Synchronises the device. Returns LBK_OK;
 * LBK_ERR_TIMEOUT when a bounded wait inside a kernel gave up; LBK_ERR_INVALID when a decoder-step
 * kernel found its position (read from pos_dev) outside [0, cap): such a kernel touches no memory
 * and the step's results are invalid (the reference asserts pos0 + m <= rope_len on the host,
 * crates/lb-model/src/model.rs:309). */
int lbk_check_device_error(lbk_ctx *ctx);
/* Number of kernel launches this context has issued since creation (benchmark bookkeeping). */
uint64_t lbk_launch_count(const lbk_ctx *ctx);
/* Which kernel serves few token rows. rows = 0 (the default) keeps the measured rule of
 * lbk_ternary_linear_n; rows = n (1..LBK_GEMV_MAX_M) sends every call of at most n token rows to the
 * fused bandwidth-bound kernel and the rest to quantise + GEMM. The results are the same bits either
 * way; the setting exists for measurements and for hosts whose shapes differ from the ones the rule
 * was measured on. The reference's counterpart is the kernel selector (gemm.rs:25-92, LB_KERNEL). */
int lbk_set_gemv_rows(lbk_ctx *ctx, int rows);

/* Measures the rate at which this GPU executes the int8 tensor-core instruction the prefill GEMM is
 * built on (tcgen05.mma kind::i8, 128 weight rows x token_rows x K 32; operands resident, nothing
 * loaded or stored): one kernel of `iterations` groups of four MMAs per SM, timed with CUDA events on
 * the context's stream. tops_out: 1e12 multiply-add operations x 2 per second. token_rows: 64, 128,
 * 192 or 256. This is the measured denominator of "fraction of int8 peak"; it has no counterpart in
 * the reference. Synchronous; about 20000 iterations take a few milliseconds. */
int lbk_int8_peak_probe(lbk_ctx *ctx, size_t token_rows, size_t iterations, double *tops_out);

/* ---- layout helpers: crates/lb-ternary/src/pack.rs:22-24,83-85 -------------------------- */

size_t lbk_padded_cols(size_t cols);
size_t lbk_row_bytes(size_t cols);

/* ---- weights: TernaryView::new / PackedTernary (pack.rs:28-81) -------------------------- */

/* Copies `packed` (rows * lbk_row_bytes(cols) bytes, host) to the device. packed_len must
 * equal that product (pack.rs:40 asserts the same) else LBK_ERR_SHAPE. */
int lbk_weight_upload(lbk_ctx *ctx, size_t rows, size_t cols, const uint8_t *packed,
                      size_t packed_len, float scale, lbk_weight **out);
/* Borrows device memory that already holds the packed rows (pitch = lbk_row_bytes(cols),
 * 16-byte aligned base), e.g. a slice of a safetensors buffer copied to the GPU, or a
 * contiguous row range of another matrix (how the reference splits rows across memory
 * domains, crates/lb-model/src/ops.rs:255-297). The caller keeps ownership. */
int lbk_weight_wrap(lbk_ctx *ctx, size_t rows, size_t cols, const void *packed_dev, float scale,
                    lbk_weight **out);
int lbk_weight_free(lbk_weight *w);
size_t lbk_weight_rows(const lbk_weight *w);
size_t lbk_weight_cols(const lbk_weight *w);
float lbk_weight_scale(const lbk_weight *w);
const void *lbk_weight_data(const lbk_weight *w); /* device pointer */
/* Copies the packed rows back to host memory (len must be rows * lbk_row_bytes(cols)): the bytes a
 * PackedTernary holds in `data` (pack.rs:60-65). Synchronous. */
int lbk_weight_download(const lbk_weight *w, uint8_t *packed_out, size_t len);

/* ---- host-pointer entry points: one per public function of lb-ternary -------------------
 * All buffers are HOST memory; the call copies in, runs the CUDA kernels, copies out and
 * synchronises. These are what a drop-in binding of the Rust functions calls. */

/* quantize_acts (crates/lb-ternary/src/quant.rs:37-75). x: f32 [m, k]. q: int8
 * [m, lbk_padded_cols(k)] zero padded; scale[m] = 127/max|x|; sum[m] = sum of q. */
int lbk_quantize_acts(lbk_ctx *ctx, const float *x, size_t m, size_t k, int8_t *q, float *scale,
                      int32_t *sum);

/* ternary_gemm_i32 (crates/lb-ternary/src/gemm.rs:95-114). q: int8 [m, padded_cols],
 * sum: i32 [m]. out: i32 [m, rows], exact. */
int lbk_ternary_gemm_i32(lbk_ctx *ctx, const lbk_weight *w, const int8_t *q, const int32_t *sum,
                         size_t m, int32_t *out);

/* ternary_gemm_multi (gemm.rs:128-195; ternary_gemm :117 is n == 1). n <= LBK_MAX_GROUP
 * matrices of equal cols share q. outs[i]: f32 [m, rows_i] =
 * (float)dot * (1.0f / (scale[t] * wscale_i)), bit-identical to separate calls. */
int lbk_ternary_gemm_multi(lbk_ctx *ctx, const lbk_weight *const *ws, size_t n, const int8_t *q,
                           const float *scale, const int32_t *sum, size_t m, float *const *outs);

/* The fused op of crates/lb-model/src/ops.rs:301-329 (ternary_linear / ternary_linear2 /
 * ternary_linear3 for n = 1, 2, 3) on HOST buffers: x f32 [m, cols]; outs[i] f32
 * [m, rows_i]; iouts (may be NULL, entries may be NULL) receives the exact int32 dots. */
int lbk_ternary_linear_host(lbk_ctx *ctx, const float *x, size_t m, const lbk_weight *const *ws,
                            size_t n, float *const *outs, int32_t *const *iouts);

/* bf16_gemv (crates/lb-ternary/src/bf16.rs:14-27) on HOST buffers. w: bf16 bits
 * [rows, cols]; x f32 [cols]; out f32 [rows]. Float: summation order differs from the
 * reference's 8-lane order, agreement is to rounding (bf16.rs:113-136 allows 1e-4 abs). */
int lbk_bf16_gemv_host(lbk_ctx *ctx, const uint16_t *w, size_t rows, size_t cols, const float *x,
                       float *out);

/* ---- device-pointer entry points (the fast path; asynchronous on `stream`) --------------
 * `stream` is a cudaStream_t passed as void* (NULL = legacy default stream). */

/* ops.rs:301-329 with everything resident: per-token absmax int8 quantisation, the packed
 * ternary x int8 dot in int32, and the 1/(s_a*s_w) epilogue. Few token rows (up to 4, or up to 8
 * when the rows are shorter than 4096 columns) run one fused bandwidth-bound kernel; more rows run
 * quantise + the tcgen05 int8 GEMM, which is flat in m where the fused kernel's arithmetic grows
 * with it. The results are the same bits either way.
 * x_dev: f32 [m, cols] (16-byte aligned); outs_dev[i]: f32 [m, rows_i]; iouts_dev may be NULL.
 * The quantise + GEMM path keeps the quantised rows in scratch memory of the context, which grows
 * (cudaMalloc) the first time a larger m * cols is seen: make the first call of each shape outside
 * any stream capture, and issue all calls of one context on one stream (they share that scratch).
 * A block once handed out stays valid until lbk_destroy, so a recorded graph keeps working after
 * later, larger calls. */
int lbk_ternary_linear_n(lbk_ctx *ctx, const float *x_dev, size_t m, const lbk_weight *const *ws,
                         size_t n, float *const *outs_dev, int32_t *const *iouts_dev,
                         void *stream);

/* No counterpart in the reference (its CPU path owns its own Vec buffers). Same operation and
 * results as lbk_ternary_linear_n on the prefill path (quantise, then the tensor-core GEMM), for
 * callers that may not allocate device memory: a serving loop that bans allocator calls after
 * start-up, a process whose memory budget belongs to another component, a plug-in inside a host
 * application that owns the CUDA heap. The quantised activations live in a fixed array inside the
 * library image (LBK_STATIC_SCRATCH_BYTES on every GPU that loads the library, until exit), so the
 * call makes no cudaMalloc/cudaFree and uses no allocating library routine.
 *   Limits: m <= 4096 token rows and m * lbk_padded_cols(cols) <= 8 MiB; beyond that the call
 *   returns LBK_ERR_UNSUPPORTED and says so in lbk_last_error().
 *   The first call on a device looks up the array's device address (cudaGetSymbolAddress); make
 *   that first call before any stream capture.
 *   All calls share the one array, and it keeps the previous call's contents (nothing in it needs
 *   clearing: each call overwrites all it reads). Two calls that overlap on the GPU -- different
 *   streams, or different contexts on the same device -- race on it; serialise them. */
#define LBK_STATIC_SCRATCH_BYTES ((8u << 20) + 2u * 4096u * 4u)
int lbk_ternary_linear_prefill_static(lbk_ctx *ctx, const float *x_dev, size_t m,
                                      const lbk_weight *const *ws, size_t n, float *const *outs_dev,
                                      int32_t *const *iouts_dev, void *stream);

/* quantize_acts (quant.rs:37-75) device to device. q_dev: int8 [m, padded_cols(k)]. */
int lbk_quantize_acts_dev(lbk_ctx *ctx, const float *x_dev, size_t m, size_t k, int8_t *q_dev,
                          float *scale_dev, int32_t *sum_dev, void *stream);

/* Tensor-parallel pieces. The reference has no multi-device path; its nearest relative is the
 * two-socket row split of crates/lb-model/src/ops.rs:255-297. When the columns (K) of a matrix are
 * split across ranks, per-token quantisation still has to use the maximum over the whole row
 * (quant.rs:101-105), and the int32 dots of the slices add up exactly:
 *   lbk_absmax_dev              amax[t] = max|x[t, :]| of this rank's column slice
 *   (all-reduce MAX over ranks, done by the caller)
 *   lbk_quantize_acts_amax_dev  quantize_acts with scale = 127 / max(amax[t], 1e-5) given
 *   lbk_ternary_gemm_dev        int32 dots of the slice (iouts only)
 *   (all-reduce SUM of the int32 dots, done by the caller: exact, order independent)
 *   lbk_scale_epilogue_dev      out[t, r] = (float)dot * (1 / (scale[t] * wscale))  (gemm.rs:141) */
int lbk_absmax_dev(lbk_ctx *ctx, const float *x_dev, size_t m, size_t k, float *amax_dev, void *stream);
int lbk_quantize_acts_amax_dev(lbk_ctx *ctx, const float *x_dev, size_t m, size_t k, const float *amax_dev,
                               int8_t *q_dev, float *scale_dev, int32_t *sum_dev, void *stream);
int lbk_scale_epilogue_dev(lbk_ctx *ctx, const int32_t *dots_dev, const float *scale_dev, float wscale,
                           size_t m, size_t rows, float *out_dev, void *stream);

/* The row-parallel layer fused with its two exchanges, over NVLink peer memory (plain loads and
 * stores; no reference counterpart). Every rank allocates one region, passes its 64-byte CUDA IPC
 * handle to the other ranks (the caller's transport: torch.distributed, MPI, a file), opens theirs
 * and builds a communicator from the `world` region pointers (its own at index `rank`).
 *   lbk_tp_quantize       = lbk_absmax_dev + all-reduce MAX + lbk_quantize_acts_amax_dev, one kernel;
 *                           at most lbk_tp_max_tokens() token rows
 *   lbk_tp_partial_buffer   where lbk_ternary_gemm_dev must write this rank's int32 dots
 *   lbk_tp_reduce_scale   = all-reduce SUM of the int32 dots + lbk_scale_epilogue_dev, one kernel;
 *                           m * rows * 4 <= lbk_tp_partial_bytes(), rows % 4 == 0; dots_out_dev
 *                           (optional) receives the summed int32 dots
 * All ranks must make the same calls in the same order, alternating quantize / reduce_scale.
 * Waits on a peer are bounded: a rank that never arrives yields LBK_ERR_TIMEOUT from
 * lbk_check_device_error, not a hang. Results are bit-identical to the unsharded operator. */
typedef struct lbk_tp_comm lbk_tp_comm;
#define LBK_PRE_RMS 1            /* input transforms, see lbk_ternary_linear_pre */
#define LBK_PRE_ADD_RMS 2
#define LBK_PRE_RELU2_MUL_RMS 3
size_t lbk_tp_region_bytes(void);
size_t lbk_tp_max_tokens(void);
size_t lbk_tp_partial_bytes(void);
int lbk_tp_region_alloc(lbk_ctx *ctx, void **region_out, unsigned char handle_out[64]);
int lbk_tp_region_open(lbk_ctx *ctx, const unsigned char handle[64], void **region_out);
int lbk_tp_region_close(lbk_ctx *ctx, void *region);
int lbk_tp_region_free(lbk_ctx *ctx, void *region);
int lbk_tp_comm_create(lbk_ctx *ctx, int world, int rank, void *const *regions, lbk_tp_comm **out);
int lbk_tp_comm_destroy(lbk_tp_comm *comm);
/* How many times a kernel of this communicator looks at a peer's word before it gives up (default
 * 2^24, several seconds). A peer that never arrives then costs LBK_ERR_TIMEOUT from
 * lbk_check_device_error and invalid results of that call; the context stays usable. The
 * reference turns a failed request into an error reply instead of a dead worker
 * (crates/lb-server/src/main.rs:92-100); this is the device-side half of the same rule. */
int lbk_tp_comm_set_wait_limit(lbk_tp_comm *comm, uint32_t polls);
void *lbk_tp_partial_buffer(lbk_tp_comm *comm);
int lbk_tp_quantize(lbk_tp_comm *comm, const float *x_dev, size_t m, size_t k, int8_t *q_dev, float *scale_dev,
                    int32_t *sum_dev, void *stream);
int lbk_tp_reduce_scale(lbk_tp_comm *comm, const float *scale_dev, float wscale, size_t m, size_t rows,
                        float *out_dev, int32_t *dots_out_dev, void *stream);

/* The token-sharded form of the same layer, for the decoder step (no reference counterpart; the step
 * it serves is crates/lb-model/src/model.rs:331-366). Every rank owns ceil(m / world) consecutive
 * token rows (lbk_tp_token_range) and keeps the residual stream for those tokens only.
 *   lbk_tp_norm_quant            the sub-norm in front of a row-parallel projection (attn_sub_norm,
 *                                ffn_sub_norm; pre = LBK_PRE_RMS on x, or LBK_PRE_RELU2_MUL_RMS on
 *                                relu(x)^2 * y) and the activation quantiser, on this rank's COLUMN
 *                                slice [m, k_local] of the input, for all m tokens. The mean of squares
 *                                is over all k_full columns and the quantiser's maximum over the whole
 *                                row: two 8-byte exchanges per token inside the kernel. w_dev is the
 *                                slice of the gain. k_local: a multiple of 128, at most 32768.
 *   (lbk_ternary_gemm_dev writes the slice's int32 dots into lbk_tp_partial_buffer)
 *   lbk_tp_reduce_norm_gather    for this rank's tokens: sum of all ranks' int32 dots (exact), scale
 *                                epilogue with ascale_dev[t] * wscale (gemm.rs:141), xres += that row
 *                                (the residual, [own tokens][hidden]), the next norm with gain w_dev
 *                                over the full row, the quantiser, and the int8 row + scale + sum
 *                                stored into every rank's region. When the call returns to the stream
 *                                all m tokens' rows are in THIS rank's region: lbk_tp_gather_q
 *                                ([m][hidden] int8), lbk_tp_gather_scale, lbk_tp_gather_sum, ready for
 *                                lbk_ternary_gemm_dev of the next column-parallel group.
 *                                flags: LBK_TP_NO_REDUCE (xres already holds the rows: the embedding,
 *                                before the first layer), LBK_TP_GATHER_F32 (gather the normalised rows
 *                                as f32, lbk_tp_gather_f32: the head's input; m <= lbk_tp_max_f32_rows).
 *                                y_out_dev (optional, [own tokens][hidden]) receives the projection's rows.
 *   lbk_tp_argmax                greedy token over a head whose vocabulary rows are split across ranks:
 *                                idx_local_dev[t] = lbk_argmax of this rank's logits_local_dev
 *                                [m][vocab_local]; next_dev[t] = first maximum over all ranks
 *                                (sample.rs:17-25).
 * m <= lbk_tp_max_rows(), hidden <= lbk_tp_max_width() and a multiple of 128. All ranks make the same
 * calls in the same order; waits are bounded as above. Integer sums are exact, so the projection rows
 * equal the unsharded operator's bits whenever the quantised inputs do; the sub-norm's sum of squares
 * is added in rank order, which can differ from the single-GPU kernel's order in the last bit. */
#define LBK_TP_NO_REDUCE 1
#define LBK_TP_GATHER_F32 2
#define LBK_TP_SCATTERED 4   /* the partial dots were stored by lbk_tp_gemm_scatter, not by lbk_ternary_gemm_dev */
size_t lbk_tp_max_rows(void);
size_t lbk_tp_max_width(void);
size_t lbk_tp_max_f32_rows(void);
int lbk_tp_token_range(const lbk_tp_comm *comm, size_t m, size_t *first_out, size_t *count_out);
int lbk_tp_norm_quant(lbk_tp_comm *comm, int pre, const float *x_dev, const float *y_dev, const float *w_dev, size_t m, size_t k_local,
                      size_t k_full, float eps, int8_t *q_dev, float *scale_dev, int32_t *sum_dev, void *stream);
int lbk_tp_reduce_norm_gather(lbk_tp_comm *comm, int flags, const float *ascale_dev, float wscale, float *xres_dev, const float *w_dev,
                              float eps, size_t m, size_t hidden, float *y_out_dev, void *stream);
/* The row-parallel projection fused with the first half of its exchange (17 .. lbk_tp_max_rows() token rows): the
 * tcgen05 GEMM on this rank's column slice stores the int32 dots of every token row straight into the region of the
 * rank that owns the row, tile by tile, from its epilogue (plain stores into peer memory; what
 * lbk_ternary_gemm_dev + the peer loads of lbk_tp_reduce_norm_gather do in two steps). Follow it with
 * lbk_tp_reduce_norm_gather(flags | LBK_TP_SCATTERED). The sums are the same integers either way. */
int lbk_tp_gemm_scatter(lbk_tp_comm *comm, const lbk_weight *w, const int8_t *q_dev, const int32_t *sum_dev, size_t m, void *stream);
const int8_t *lbk_tp_gather_q(lbk_tp_comm *comm);
const float *lbk_tp_gather_scale(lbk_tp_comm *comm);
const int32_t *lbk_tp_gather_sum(lbk_tp_comm *comm);
const float *lbk_tp_gather_f32(lbk_tp_comm *comm);
int lbk_tp_argmax(lbk_tp_comm *comm, const float *logits_local_dev, const int32_t *idx_local_dev, size_t m, size_t vocab_local,
                  int32_t *next_dev, void *stream);

/* ternary_gemm_multi (gemm.rs:128-195) on already quantised device inputs. */
int lbk_ternary_gemm_dev(lbk_ctx *ctx, const lbk_weight *const *ws, size_t n, const int8_t *q_dev,
                         const float *scale_dev, const int32_t *sum_dev, size_t m,
                         float *const *outs_dev, int32_t *const *iouts_dev, void *stream);

/* bf16_linear (crates/lb-model/src/ops.rs:199-218): x f32 [m, cols] @ W^T, W bf16
 * [rows, cols] -> out f32 [m, rows], all device memory. */
int lbk_bf16_linear(lbk_ctx *ctx, const float *x_dev, size_t m, const uint16_t *w_dev, size_t rows,
                    size_t cols, float *out_dev, void *stream);

/* ---- decoder-step glue: the non-matmul parts of BitNet::forward (crates/lb-model/src/model.rs:305-374)
 * All device pointers; `b` independent sequences; kernels that depend on the decode position read
 * it from pos_dev (device int32), so a captured CUDA graph of one step can be replayed per token. */

/* embed (model.rs:274-282): out[b, hidden] = f32(table[tokens[b], :]), table is bf16 bits. */
int lbk_embed_bf16(lbk_ctx *ctx, const uint16_t *table_dev, const int32_t *tokens_dev, size_t b, size_t hidden,
                   float *out_dev, void *stream);
/* rms_norm (model.rs:267-272): out = x * (1/sqrt(mean(x^2) + eps)) * w over rows of n. */
int lbk_rms_norm(lbk_ctx *ctx, const float *x_dev, const float *w_dev, size_t rows, size_t n, float eps,
                 float *out_dev, void *stream);
/* apply_rope on q (in place) and k, then k and v stored as bf16 at position *pos_dev of the caches
 * [b][kv_heads][cap][head_dim] (model.rs:295-303,334-347; the reference keeps f32 caches). cos/sin:
 * f32 [max_pos][head_dim], both halves duplicated (model.rs:213-230). */
int lbk_rope_kv_append(lbk_ctx *ctx, float *q_dev, const float *k_dev, const float *v_dev, const float *cos_dev,
                       const float *sin_dev, const int32_t *pos_dev, size_t b, size_t n_heads, size_t kv_heads,
                       size_t head_dim, size_t cap, uint16_t *kcache_dev, uint16_t *vcache_dev, void *stream);
/* Grouped-query attention of one new token per sequence over keys 0..*pos_dev (model.rs:350-357),
 * head_dim 128, split over the sequence. scratch_dev: b*n_heads*splits*(head_dim+4) floats, 16-byte aligned. */
int lbk_attn_decode(lbk_ctx *ctx, const float *q_dev, const uint16_t *kcache_dev, const uint16_t *vcache_dev,
                    const int32_t *pos_dev, size_t b, size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap,
                    size_t splits, float *scratch_dev, float *out_dev, void *stream);
/* relu(g)^2 * u (model.rs:363). */
int lbk_relu2_mul(lbk_ctx *ctx, const float *g_dev, const float *u_dev, size_t n, float *out_dev, void *stream);
/* x += y (the residual adds of model.rs:359,365). */
int lbk_add_inplace(lbk_ctx *ctx, float *x_dev, const float *y_dev, size_t n, void *stream);
/* A norm whose result goes straight into a projection: the normalised rows leave as the quantised
 * activations of quant.rs:37-75 (q_dev int8 [rows][padded(n)], scale_dev[rows], sum_dev[rows]) ready
 * for lbk_ternary_gemm_dev, with the same bits as lbk_rms_norm / lbk_add_rms_norm /
 * lbk_relu2_mul_rms_norm followed by lbk_quantize_acts_dev. `pre` as for lbk_ternary_linear_pre:
 * LBK_PRE_RMS (x), LBK_PRE_ADD_RMS (x += y first; x_dev is updated), LBK_PRE_RELU2_MUL_RMS
 * (relu(x)^2 * y). n % 4 == 0 and n <= 8192 (lbk_norm_quant_supported); 16-byte aligned buffers. */
int lbk_norm_quant_supported(size_t n);
int lbk_norm_quant(lbk_ctx *ctx, int pre, float *x_dev, const float *y_dev, const float *w_dev, size_t rows, size_t n,
                   float eps, int8_t *q_dev, float *scale_dev, int32_t *sum_dev, void *stream);
/* Prompt ingestion: n consecutive positions of ONE sequence (`seq` of the cache's batch) at once.
 * lbk_rope_kv_append_rows: RoPE on q_dev [n][n_heads*hd] in place and on k_dev [n][kv_heads*hd];
 * k and v_dev are appended at positions *pos_dev .. *pos_dev + n - 1.
 * lbk_attn_prefill: causal attention of those n rows (row i sees keys 0 .. *pos_dev + i), head_dim
 * 128, out_dev [n][n_heads*hd]. Neither advances *pos_dev. */
int lbk_rope_kv_append_rows(lbk_ctx *ctx, float *q_dev, const float *k_dev, const float *v_dev, const float *cos_dev,
                            const float *sin_dev, const int32_t *pos_dev, size_t n, size_t n_heads, size_t kv_heads,
                            size_t head_dim, size_t cap, size_t seq, uint16_t *kcache_dev, uint16_t *vcache_dev,
                            void *stream);
int lbk_attn_prefill(lbk_ctx *ctx, const float *q_dev, const uint16_t *kcache_dev, const uint16_t *vcache_dev,
                     const int32_t *pos_dev, size_t n, size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap,
                     size_t seq, float *out_dev, void *stream);
/* lbk_rope_kv_append + lbk_attn_decode in one launch, for 4..8 query heads per KV head, head_dim
 * 128 and at most 256 splits (lbk_attn_decode_fused_supported): q_dev, k_dev, v_dev are the raw
 * projections ([b][n_heads*128], [b][kv_heads*128] x 2); the new position's K/V row is appended to
 * the caches by the kernel. scratch as for lbk_attn_decode; counters_dev: b * kv_heads ints, zero
 * before the first call (the kernel leaves them zero). */
int lbk_attn_decode_fused_supported(size_t n_heads, size_t kv_heads, size_t head_dim, size_t splits);
/* The `_seq` forms read ONE POSITION PER SEQUENCE (pos_dev: b ints), for batches whose sequences
 * have different lengths (continuous batching; the reference has no batch dimension). Everything
 * else as in the forms above, which use pos_dev[0] for all sequences. lbk_advance_pos_seq adds one
 * to the positions whose active_dev entry is non-zero (to all when active_dev is NULL). */
int lbk_rope_kv_append_seq(lbk_ctx *ctx, float *q_dev, const float *k_dev, const float *v_dev, const float *cos_dev,
                           const float *sin_dev, const int32_t *pos_dev, size_t b, size_t n_heads, size_t kv_heads,
                           size_t head_dim, size_t cap, uint16_t *kcache_dev, uint16_t *vcache_dev, void *stream);
int lbk_attn_decode_seq(lbk_ctx *ctx, const float *q_dev, const uint16_t *kcache_dev, const uint16_t *vcache_dev,
                        const int32_t *pos_dev, size_t b, size_t n_heads, size_t kv_heads, size_t head_dim, size_t cap,
                        size_t splits, float *scratch_dev, float *out_dev, void *stream);
int lbk_attn_decode_fused_seq(lbk_ctx *ctx, const float *q_dev, const float *k_dev, const float *v_dev, const float *cos_dev,
                              const float *sin_dev, const int32_t *pos_dev, size_t b, size_t n_heads, size_t kv_heads,
                              size_t head_dim, size_t cap, size_t splits, uint16_t *kcache_dev, uint16_t *vcache_dev,
                              float *scratch_dev, int32_t *counters_dev, float *out_dev, void *stream);
int lbk_advance_pos_seq(lbk_ctx *ctx, int32_t *pos_dev, const int32_t *active_dev, size_t b, void *stream);
int lbk_attn_decode_fused(lbk_ctx *ctx, const float *q_dev, const float *k_dev, const float *v_dev, const float *cos_dev,
                          const float *sin_dev, const int32_t *pos_dev, size_t b, size_t n_heads, size_t kv_heads,
                          size_t head_dim, size_t cap, size_t splits, uint16_t *kcache_dev, uint16_t *vcache_dev,
                          float *scratch_dev, int32_t *counters_dev, float *out_dev, void *stream);
/* Fusions of the above for the decode step (rows of a multiple of 4, at most 8192, columns;
 * 16-byte aligned): x += y then out = rms_norm(x) (model.rs:359-361, 365 + the next norm); and
 * out = rms_norm(relu(g)^2 * u) (model.rs:363-364). */
int lbk_add_rms_norm(lbk_ctx *ctx, float *x_dev, const float *y_dev, const float *w_dev, size_t rows, size_t n,
                     float eps, float *out_dev, void *stream);
int lbk_relu2_mul_rms_norm(lbk_ctx *ctx, const float *g_dev, const float *u_dev, const float *w_dev, size_t rows,
                           size_t n, float eps, float *out_dev, void *stream);
/* ternary_linear_n for 1..16 token rows with the element-wise work that precedes the projection in
 * the decoder step (model.rs:331-366) done inside the same kernel, on the registers that hold the
 * input row: `pre` = LBK_PRE_RMS (x' = rms_norm(x) * w), LBK_PRE_ADD_RMS (s = x + y, written to
 * xout_dev; x' = rms_norm(s) * w) or LBK_PRE_RELU2_MUL_RMS (s = relu(x)^2 * y; x' = rms_norm(s) * w).
 * x, y, w, xout: 16-byte aligned, xout must not alias x or y. LBK_ERR_UNSUPPORTED when
 * lbk_ternary_linear_pre_supported(m, cols) is 0 (rows too long to hold in registers at that m):
 * use the separate kernels above then. */
int lbk_ternary_linear_pre_supported(size_t m, size_t cols);
int lbk_ternary_linear_pre(lbk_ctx *ctx, int pre, const float *x_dev, const float *y_dev, const float *w_dev, float eps,
                           float *xout_dev, size_t m, const lbk_weight *const *ws, size_t n, float *const *outs_dev,
                           int32_t *const *iouts_dev, void *stream);
/* argmax (crates/lb-model/src/sample.rs:17-25): first index of the maximum of each row. */
int lbk_argmax(lbk_ctx *ctx, const float *logits_dev, size_t rows, size_t n, int32_t *out_dev, void *stream);
/* *pos_dev += 1 (cache.len = total, model.rs:367). The caller keeps the position below `cap`: a
 * step launched at position >= cap is refused by its kernels (see lbk_check_device_error). */
int lbk_advance_pos(lbk_ctx *ctx, int32_t *pos_dev, void *stream);

/* ---- the decoder as a native runtime (crates/lb-model/src/model.rs) ----------------------------
 * lbk_model_load      BitNet::load (model.rs:149-232): `dir/config.json` + `dir/model.lbt.safetensors`
 *                     as lb-convert writes them; the format check and the supported family
 *                     (relu2, tied embeddings) are the reference's; head_dim must be 128.
 * lbk_model_new_cache BitNet::new_cache (model.rs:234-236): here bf16, of fixed capacity
 *                     (0 = max_position_embeddings), for `batch` (1..16) independent sequences.
 * lbk_model_forward   BitNet::forward (model.rs:305-374) for one sequence (cache of batch 1):
 *                     appends `n` tokens at cache.len and writes the logits of every token
 *                     ([n][vocab], all_logits != 0) or of the last one ([vocab]) to host memory.
 *                     Several tokens go through the projections together, up to 4096 rows a pass.
 * lbk_model_decode    one new token for each of the cache's sequences: tokens_dev int32 [batch];
 *                     logits_dev f32 [batch][vocab] and/or next_dev int32 [batch] (greedy argmax,
 *                     sample.rs:17-25) may be null. Asynchronous on `stream`.
 * A step is recorded into a CUDA graph at a cache's first use and replayed afterwards. */
typedef struct lbk_model lbk_model;
typedef struct lbk_kv_cache lbk_kv_cache;
typedef struct lbk_model_config {
    size_t hidden_size, intermediate_size, num_attention_heads, num_key_value_heads, num_hidden_layers, vocab_size,
        max_position_embeddings;
    float rms_norm_eps, rope_theta;
    int bos_token_id;
} lbk_model_config;
int lbk_model_load(lbk_ctx *ctx, const char *directory, lbk_model **out);
/* The same loader for one rank of a tensor-parallel group (the reference has one process and no
 * sharding; its loader is model.rs:149-232). q/k/v/gate/up keep rows [rank*rows/world, ...) of the
 * packed matrix, a contiguous range of the file; o/down keep columns [rank*cols/world, ...), a whole
 * number of 128-column blocks, cut out of every packed row while loading. Norm gains, the embedding /
 * head table and the RoPE tables are whole on every rank. The parts are read with the accessors
 * below (lbk_model_new_cache refuses a sharded model: its step needs the other ranks).
 * Loading never holds more host memory than two pinned staging buffers (lbk_load_stats.staging_bytes):
 * file -> pinned buffer -> device, one buffer being refilled while the other one's copy is in flight;
 * all packed matrices of the rank live in one device allocation. */
int lbk_model_load_shard(lbk_ctx *ctx, const char *directory, int rank, int world, lbk_model **out);
typedef struct lbk_load_stats {
    double seconds;          /* wall clock of the load, device copies finished */
    size_t bytes_read;       /* from the file */
    size_t bytes_to_device;  /* copied host -> device (less than bytes_read for column shards) */
    size_t staging_bytes;    /* pinned host memory the loader held */
} lbk_load_stats;
int lbk_model_load_stats(const lbk_model *model, lbk_load_stats *out);
/* Parts of a loaded model (owned by it; device pointers). */
#define LBK_LIN_Q 0
#define LBK_LIN_K 1
#define LBK_LIN_V 2
#define LBK_LIN_O 3
#define LBK_LIN_GATE 4
#define LBK_LIN_UP 5
#define LBK_LIN_DOWN 6
#define LBK_NORM_INPUT 0
#define LBK_NORM_POST_ATTN 1
#define LBK_NORM_ATTN_SUB 2
#define LBK_NORM_FFN_SUB 3
#define LBK_NORM_FINAL 4
const lbk_weight *lbk_model_linear(const lbk_model *model, size_t layer, int which);
const float *lbk_model_norm(const lbk_model *model, size_t layer, int which); /* `layer` is ignored for LBK_NORM_FINAL */
const uint16_t *lbk_model_embedding(const lbk_model *model);
const float *lbk_model_rope_cos(const lbk_model *model);
const float *lbk_model_rope_sin(const lbk_model *model);
int lbk_model_get_config(const lbk_model *model, lbk_model_config *out);
int lbk_model_free(lbk_model *model);
int lbk_model_new_cache(lbk_model *model, size_t batch, size_t capacity, lbk_kv_cache **out);
size_t lbk_kv_cache_len(const lbk_kv_cache *cache);
int lbk_kv_cache_reset(lbk_kv_cache *cache);
int lbk_kv_cache_free(lbk_kv_cache *cache);
int lbk_model_forward(lbk_model *model, lbk_kv_cache *cache, const uint32_t *tokens, size_t n, int all_logits,
                      float *logits_out);
int lbk_model_decode(lbk_model *model, lbk_kv_cache *cache, const int32_t *tokens_dev, float *logits_dev,
                     int32_t *next_dev, void *stream);
/* Rows a prompt pass takes at once (1..8192; default 4096). More rows fill the GEMM's tile rounds
 * better, fewer bound the work buffers (about 150 KB per row at 2B4T shapes). */
int lbk_model_set_prefill_rows(lbk_model *model, size_t rows);
/* Length of sequence `seq` of a cache (lbk_kv_cache_len is sequence 0). */
size_t lbk_kv_cache_len_seq(const lbk_kv_cache *cache, size_t seq);

/* ---- continuous batching ------------------------------------------------------------------------
 * The reference's server hands requests to ONE worker that runs them one after the other
 * (crates/lb-server/src/main.rs:92-166); a batched decode step only pays off with a scheduler in
 * front of it. lbk_batcher owns a cache of `slots` sequences (1..16) of `capacity` positions each
 * (0: the model's max_position_embeddings).
 * lbk_batcher_submit    queues a request (prompt of n >= 1 tokens, at most max_new_tokens generated,
 *                       generation also ends after eos_token unless it is negative, or when the
 *                       slot's positions are used up) and returns its id.
 * lbk_batcher_step      moves queued requests into free slots (the prompt pass of lbk_model_forward,
 *                       into that slot; the first token comes from its last row), then advances every
 *                       occupied slot by one greedy token (argmax, sample.rs:17-25) with the recorded
 *                       decode step; sequences have their own positions, finished ones free their slot
 *                       at once. pending_out (may be NULL): requests still queued or running.
 * lbk_batcher_poll      tokens generated so far for a request (at most `capacity` are copied, n_out is
 *                       the full count) and whether it has finished.
 * lbk_batcher_forget    drops a finished request's record.
 * Calls on one batcher must not overlap. */
typedef struct lbk_batcher lbk_batcher;
int lbk_batcher_create(lbk_model *model, size_t slots, size_t capacity, lbk_batcher **out);
int lbk_batcher_submit(lbk_batcher *batcher, const uint32_t *prompt, size_t n, size_t max_new_tokens, int32_t eos_token,
                       uint64_t *id_out);
int lbk_batcher_step(lbk_batcher *batcher, size_t *pending_out);
int lbk_batcher_poll(lbk_batcher *batcher, uint64_t id, uint32_t *tokens_out, size_t capacity, size_t *n_out, int *done_out);
int lbk_batcher_forget(lbk_batcher *batcher, uint64_t id);
int lbk_batcher_destroy(lbk_batcher *batcher);

/* ---- plans: a whole decode-like sequence in one launch -----------------------------------
 * The reference runs 4 fused ternary ops per layer x 30 layers = 120 parallel regions per
 * token (crates/lb-ternary/benches/kbench.rs:148-194, crates/lb-model/src/model.rs:331-366).
 * A plan records such a sequence once and replays it with a single persistent-kernel
 * launch. Groups in a plan must be independent: none may read another's outputs, because the
 * launch walks all of them at once (the reference's sweep has no decoder math between them either). */
int lbk_plan_create(lbk_ctx *ctx, lbk_plan **out);
/* Appends one fused group (same meaning as lbk_ternary_linear_n with m == 1). With x_dev
 * and outs_dev both NULL the group reads its input from, and writes its f32 outputs to, the
 * plan's own device arenas (allocated by lbk_plan_finalize; slots in order of addition:
 * inputs are `cols` floats each, outputs rows_0 + rows_1 + ... floats each). */
int lbk_plan_add(lbk_plan *plan, const float *x_dev, const lbk_weight *const *ws, size_t n,
                 float *const *outs_dev, int32_t *const *iouts_dev);
int lbk_plan_finalize(lbk_plan *plan);
int lbk_plan_run(lbk_plan *plan, void *stream);
/* One decode-like step on HOST buffers, for plans whose groups all use the arenas: copies
 * x_host (every group's input row, concatenated) to the device, runs the plan, copies every
 * group's outputs back to y_host and synchronises `stream`. This is the host-buffer form of
 * the reference's per-token loop (crates/lb-ternary/benches/kbench.rs:173-190). */
int lbk_plan_run_host(lbk_plan *plan, const float *x_host, size_t x_len, float *y_host,
                      size_t y_len, void *stream);
size_t lbk_plan_input_elems(const lbk_plan *plan);
size_t lbk_plan_output_elems(const lbk_plan *plan);
const float *lbk_plan_input_arena(const lbk_plan *plan);  /* device pointers, after finalize */
const float *lbk_plan_output_arena(const lbk_plan *plan);
/* Packed weight bytes one run streams (the figure kbench reports bandwidth on, kbench.rs:61). */
size_t lbk_plan_weight_bytes(const lbk_plan *plan);
int lbk_plan_destroy(lbk_plan *plan);

/* ---- converter: master weights -> packed ternary, on the device --------------------------------
 * lb-convert's per-tensor work (crates/lb-convert/src/main.rs:62-87) for n BitLinear weights at
 * once: absmean scale with an f64 sum (lb-ternary/src/pack.rs:129-138), ternary values
 * clamp(round_ties_even(w * scale), -1, 1) (pack.rs:140-142), packed rows in the layout of
 * pack.rs:88-103 (padding columns hold zero weights). src_dev: [rows][cols] row-major, f32 or bf16
 * bits; packed_dev: rows * padded(cols)/4 bytes, 4-byte aligned. On the host afterwards:
 * scales_out[n] (the stored `wscale` = 1/mean|W|), counts_out[n][3] (how many -1, 0, +1; may be
 * NULL) and sha256_out[n][32] (digest of the int8 ternary array [rows*cols], the value the
 * converter's --check compares with torch, main.rs:141-170; may be NULL: one GPU thread per
 * tensor walks the digest chain, about 0.03 s per million weights of the largest tensor, all tensors
 * side by side: 0.5 s for a 2B4T-shaped model).
 * Synchronises `stream`. */
#define LBK_DTYPE_F32 0
#define LBK_DTYPE_BF16 1
typedef struct lbk_convert_item {
    const void *src_dev;
    size_t rows, cols;
    uint8_t *packed_dev;
} lbk_convert_item;
int lbk_convert_bitlinear(lbk_ctx *ctx, const lbk_convert_item *items, size_t n, int src_dtype, float *scales_out,
                          uint64_t *counts_out, uint8_t *sha256_out, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* LBK_H */
