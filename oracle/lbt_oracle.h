/*
 * CPU oracle for the packed 2-bit ternary x int8 matmul path of lemonade-burn.
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain-C restatement of the reference's scalar
 * algorithm. It exists to check the CUDA library; nothing in the product path may call,
 * link or load it. Only the tests, the smoke check and the CPU-baseline leg of the
 * benchmark use it.
 *
 * Parity status: PINNED for the integer/byte path (packing, activation quantisation,
 * int32 dot products, f32 scale epilogue) against the known-answer vectors held by the
 * reference's own unit tests (crates/lb-ternary/src/quant.rs:201-216,
 * crates/lb-ternary/src/pack.rs:149-170, crates/ternary-kernels/src/quant.rs:34-42,
 * crates/ternary-kernels/src/pack.rs:86-107, crates/lb-ternary/tests/golden.rs:108-122,
 * 181-194) and against the installed `transformers.integrations.bitnet` ActQuant /
 * WeightQuant, which the reference states it mirrors. The reference itself is Rust and
 * cannot be compiled where this was written, so no output of the reference binary pins it.
 *
 * Every function names the reference file:line it follows.
 */
#ifndef LBT_ORACLE_H
#define LBT_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LBT_BLOCK 128       /* weights per packed block   (pack.rs:18) */
#define LBT_BLOCK_BYTES 32  /* bytes per packed block     (pack.rs:19) */

/* pack.rs:22-24 */
size_t lbt_padded_cols(size_t cols);
/* pack.rs:83-85 */
size_t lbt_row_bytes(size_t cols);

/* pack.rs:88-103: one row of {-1,0,1} -> row_bytes(cols) packed bytes, pad = code 1. */
void lbt_pack_row(const int8_t *values, size_t cols, uint8_t *out);
/* pack.rs:69-78 (PackedTernary::from_ternary): row-major [rows, cols] -> packed. */
void lbt_pack_matrix(const int8_t *values, size_t rows, size_t cols, uint8_t *out);
/* pack.rs:106-116: packed row (padded length) -> ternary values. */
void lbt_unpack_row(const uint8_t *row, size_t padded, int8_t *out);

/* ternary-kernels/src/pack.rs:46-69: the second statement of the same layout
 * (pre-fill 0x55, then overwrite 2-bit fields column by column). */
void lbt_tk_pack_ternary(const int8_t *t, size_t n, size_t k, uint8_t *out);
/* ternary-kernels/src/pack.rs:72-81 */
void lbt_tk_unpack_row(const uint8_t *packed_row, size_t kp, int8_t *out);

/* pack.rs:135-138: f64 sum of |w|, one rounding to f32. */
float lbt_absmean_f32(const float *w, size_t n);
/* pack.rs:140-142 */
void lbt_ternarize_with_scale(const float *w, size_t n, float scale, int8_t *out);
/* pack.rs:129-133: returns the scale 1/max(mean|w|,1e-5). */
float lbt_ternarize_absmean(const float *w, size_t n, int8_t *out);

/* quant.rs:100-118 (quantize_row_scalar + quant_one). q gets n codes. */
void lbt_quantize_row_scalar(const float *x, size_t n, int8_t *q, float *scale, int32_t *sum);
/* quant.rs:45-75 (quantize_acts_into): q is m * padded_cols(k) bytes, zero padded. */
void lbt_quantize_acts(const float *x, size_t m, size_t k, int8_t *q, float *scale, int32_t *sum);

/* gemm.rs:329-343 (codes_dot_scalar): acc[t] += sum_k code[k] * x[t*stride + k]. */
void lbt_codes_dot_scalar(const uint8_t *row, size_t row_len, const int8_t *x, size_t stride,
                          size_t ntok, int32_t *acc);

/* gemm.rs:95-114 + 292-310 (ternary_gemm_i32 through dot_row):
 * out[t*rows + r] = codes_dot - sum[t]. q is [m, padded_cols(cols)]. */
void lbt_ternary_gemm_i32(const uint8_t *packed, size_t rows, size_t cols, const int8_t *q,
                          const int32_t *sum, size_t m, int32_t *out);

/* ternary-kernels/src/reference.rs:7-16 (gemv_i32_reference): unpack every weight,
 * sum a*b in i32, one token. */
void lbt_gemv_i32_reference(const uint8_t *packed, size_t n, size_t kp, const int8_t *q,
                            int32_t *out);
/* ternary-kernels/src/reference.rs:18-28 (linear_f64_reference). */
void lbt_linear_f64_reference(const int8_t *t, size_t n, size_t k, float dequant, const int8_t *q,
                              float a_scale, double *out);

/* gemm.rs:117-195 (ternary_gemm / ternary_gemm_multi, one matrix):
 * out[t*rows + r] = (float)dot * (1.0f / (scale[t] * wscale)). */
void lbt_ternary_gemm(const uint8_t *packed, size_t rows, size_t cols, float wscale,
                      const int8_t *q, const float *scale, const int32_t *sum, size_t m,
                      float *out);

/* bf16.rs:9-27,38-51 (bf16_gemv with dot_scalar: 8 f32 lanes, lane sum, scalar tail). */
void lbt_bf16_gemv(const uint16_t *w, size_t rows, size_t cols, const float *x, float *out);

/* sample.rs:17-25 (argmax: first index of the maximum, strict >). */
uint32_t lbt_argmax(const float *logits, size_t n);

#ifdef __cplusplus
}
#endif
#endif
