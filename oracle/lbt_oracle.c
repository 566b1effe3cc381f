/*
 * CPU oracle (test infrastructure only; see lbt_oracle.h for the rules and parity status).
 * Build: gcc -O2 -fno-fast-math -ffp-contract=off -fPIC -shared (see oracle/Makefile).
 * -ffp-contract=off matters: the reference never fuses a multiply with an add.
 */
#include "lbt_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

size_t lbt_padded_cols(size_t cols) { return (cols + LBT_BLOCK - 1) / LBT_BLOCK * LBT_BLOCK; }

size_t lbt_row_bytes(size_t cols) { return lbt_padded_cols(cols) / 4; }

/* pack.rs:88-103. Byte j of block b, bits 2k..2k+1 <- code (w+1)&3 of column b*128+k*32+j. */
void lbt_pack_row(const int8_t *values, size_t cols, uint8_t *out) {
    size_t nb = lbt_padded_cols(cols) / LBT_BLOCK;
    for (size_t b = 0; b < nb; b++) {
        for (size_t j = 0; j < LBT_BLOCK_BYTES; j++) {
            uint8_t v = 0;
            for (size_t k = 0; k < 4; k++) {
                size_t idx = b * LBT_BLOCK + k * 32 + j;
                int w = idx < cols ? values[idx] : 0;
                v |= (uint8_t)(((uint8_t)(w + 1) & 3u) << (2 * k));
            }
            out[b * LBT_BLOCK_BYTES + j] = v;
        }
    }
}

void lbt_pack_matrix(const int8_t *values, size_t rows, size_t cols, uint8_t *out) {
    size_t rb = lbt_row_bytes(cols);
    for (size_t r = 0; r < rows; r++) lbt_pack_row(values + r * cols, cols, out + r * rb);
}

/* pack.rs:106-116 */
void lbt_unpack_row(const uint8_t *row, size_t padded, int8_t *out) {
    size_t nb = padded / LBT_BLOCK;
    for (size_t b = 0; b < nb; b++)
        for (size_t j = 0; j < LBT_BLOCK_BYTES; j++) {
            uint8_t byte = row[b * LBT_BLOCK_BYTES + j];
            for (size_t k = 0; k < 4; k++)
                out[b * LBT_BLOCK + k * 32 + j] = (int8_t)(((byte >> (2 * k)) & 3) - 1);
        }
}

/* ternary-kernels/src/pack.rs:46-69 */
void lbt_tk_pack_ternary(const int8_t *t, size_t n, size_t k, uint8_t *out) {
    size_t kp = lbt_padded_cols(k), rb = kp / 4;
    memset(out, 0x55, n * rb);
    for (size_t r = 0; r < n; r++) {
        uint8_t *dst = out + r * rb;
        for (size_t c = 0; c < k; c++) {
            uint8_t code = (uint8_t)(t[r * k + c] + 1);
            size_t b = c / LBT_BLOCK, within = c % LBT_BLOCK, i = within / 32, j = within % 32;
            uint8_t *byte = &dst[b * LBT_BLOCK_BYTES + j];
            *byte = (uint8_t)((*byte & ~(3u << (2 * i))) | (code << (2 * i)));
        }
    }
}

/* ternary-kernels/src/pack.rs:72-81 */
void lbt_tk_unpack_row(const uint8_t *packed_row, size_t kp, int8_t *out) {
    for (size_t c = 0; c < kp; c++) {
        size_t b = c / LBT_BLOCK, within = c % LBT_BLOCK;
        uint8_t byte = packed_row[b * LBT_BLOCK_BYTES + within % 32];
        out[c] = (int8_t)(((byte >> (2 * (within / 32))) & 3) - 1);
    }
}

/* pack.rs:135-138 */
float lbt_absmean_f32(const float *w, size_t n) {
    double s = 0.0;
    for (size_t i = 0; i < n; i++) s += fabs((double)w[i]);
    return (float)(s / (double)n);
}

/* Rust `f32 as i8`: NaN -> 0, otherwise saturating truncation. */
static int8_t f32_as_i8(float v) {
    if (v != v) return 0;
    if (v <= -128.0f) return -128;
    if (v >= 127.0f) return 127;
    return (int8_t)v;
}

/* Rust f32::clamp(lo, hi): NaN stays NaN. */
static float clampf(float v, float lo, float hi) {
    if (v < lo) return lo;
    if (v > hi) return hi;
    return v;
}

/* pack.rs:140-142: (v*scale).round_ties_even().clamp(-1,1) as i8 */
void lbt_ternarize_with_scale(const float *w, size_t n, float scale, int8_t *out) {
    for (size_t i = 0; i < n; i++) out[i] = f32_as_i8(clampf(rintf(w[i] * scale), -1.0f, 1.0f));
}

/* pack.rs:129-133 */
float lbt_ternarize_absmean(const float *w, size_t n, int8_t *out) {
    float mean = lbt_absmean_f32(w, n);
    float scale = 1.0f / fmaxf(mean, 1e-5f);
    lbt_ternarize_with_scale(w, n, scale, out);
    return scale;
}

/* quant.rs:100-118. f32::max ignores a NaN operand, as fmaxf does. */
void lbt_quantize_row_scalar(const float *x, size_t n, int8_t *q, float *scale, int32_t *sum) {
    float amax = 0.0f;
    for (size_t i = 0; i < n; i++) amax = fmaxf(amax, fabsf(x[i]));
    float s = 127.0f / fmaxf(amax, 1e-5f);
    int32_t acc = 0;
    for (size_t i = 0; i < n; i++) {
        int8_t r = f32_as_i8(clampf(rintf(x[i] * s), -128.0f, 127.0f));
        q[i] = r;
        acc += r;
    }
    *scale = s;
    *sum = acc;
}

/* quant.rs:45-75 */
void lbt_quantize_acts(const float *x, size_t m, size_t k, int8_t *q, float *scale, int32_t *sum) {
    size_t kp = lbt_padded_cols(k);
    memset(q, 0, m * kp);
    for (size_t i = 0; i < m; i++)
        lbt_quantize_row_scalar(x + i * k, k, q + i * kp, &scale[i], &sum[i]);
}

/* gemm.rs:329-343 */
void lbt_codes_dot_scalar(const uint8_t *row, size_t row_len, const int8_t *x, size_t stride,
                          size_t ntok, int32_t *acc) {
    size_t nb = row_len / LBT_BLOCK_BYTES;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = row + b * LBT_BLOCK_BYTES;
        for (size_t k = 0; k < 4; k++)
            for (size_t j = 0; j < LBT_BLOCK_BYTES; j++) {
                int32_t c = (blk[j] >> (2 * k)) & 3;
                size_t idx = b * LBT_BLOCK + k * 32 + j;
                for (size_t t = 0; t < ntok; t++) acc[t] += c * (int32_t)x[t * stride + idx];
            }
    }
}

/* gemm.rs:95-114 with dot_row (gemm.rs:292-310): token tiles of <= 4, then subtract sum. */
void lbt_ternary_gemm_i32(const uint8_t *packed, size_t rows, size_t cols, const int8_t *q,
                          const int32_t *sum, size_t m, int32_t *out) {
    size_t kp = lbt_padded_cols(cols), rb = kp / 4;
    for (size_t r = 0; r < rows; r++) {
        const uint8_t *row = packed + r * rb;
        size_t t = 0;
        while (t < m) {
            size_t tt = m - t < 4 ? m - t : 4;
            int32_t acc[4] = {0, 0, 0, 0};
            lbt_codes_dot_scalar(row, rb, q + t * kp, kp, tt, acc);
            for (size_t i = 0; i < tt; i++) out[(t + i) * rows + r] = acc[i] - sum[t + i];
            t += tt;
        }
    }
}

/* ternary-kernels/src/reference.rs:7-16 */
void lbt_gemv_i32_reference(const uint8_t *packed, size_t n, size_t kp, const int8_t *q,
                            int32_t *out) {
    size_t rb = kp / 4;
    int8_t *w = (int8_t *)malloc(kp);
    for (size_t r = 0; r < n; r++) {
        lbt_tk_unpack_row(packed + r * rb, kp, w);
        int32_t s = 0;
        for (size_t c = 0; c < kp; c++) s += (int32_t)w[c] * (int32_t)q[c];
        out[r] = s;
    }
    free(w);
}

/* ternary-kernels/src/reference.rs:18-28 */
void lbt_linear_f64_reference(const int8_t *t, size_t n, size_t k, float dequant, const int8_t *q,
                              float a_scale, double *out) {
    for (size_t r = 0; r < n; r++) {
        double s = 0.0;
        for (size_t c = 0; c < k; c++)
            s += ((double)q[c] / (double)a_scale) * ((double)t[r * k + c] * (double)dequant);
        out[r] = s;
    }
}

/* gemm.rs:141,150 (decode) and gemm.rs:158,178 (prefill): inv = 1/(s_a*s_w) in f32, then
 * one f32 multiply of the converted integer. */
void lbt_ternary_gemm(const uint8_t *packed, size_t rows, size_t cols, float wscale,
                      const int8_t *q, const float *scale, const int32_t *sum, size_t m,
                      float *out) {
    int32_t *ints = (int32_t *)malloc(sizeof(int32_t) * (m * rows + 1));
    lbt_ternary_gemm_i32(packed, rows, cols, q, sum, m, ints);
    for (size_t t = 0; t < m; t++) {
        float inv = 1.0f / (scale[t] * wscale);
        for (size_t r = 0; r < rows; r++) out[t * rows + r] = (float)ints[t * rows + r] * inv;
    }
    free(ints);
}

static float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* bf16.rs:38-51 */
static float bf16_dot_scalar(const uint16_t *w, const float *x, size_t n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    size_t n8 = n / 8 * 8;
    for (size_t i = 0; i < n8; i += 8)
        for (size_t l = 0; l < 8; l++) acc[l] += bf16_to_f32(w[i + l]) * x[i + l];
    float s = 0.0f; /* Rust's f32 `sum()` folds from 0.0 left to right */
    for (size_t l = 0; l < 8; l++) s += acc[l];
    for (size_t i = n8; i < n; i++) s += bf16_to_f32(w[i]) * x[i];
    return s;
}

/* bf16.rs:14-27 */
void lbt_bf16_gemv(const uint16_t *w, size_t rows, size_t cols, const float *x, float *out) {
    for (size_t r = 0; r < rows; r++) out[r] = bf16_dot_scalar(w + r * cols, x, cols);
}

/* sample.rs:17-25 */
uint32_t lbt_argmax(const float *logits, size_t n) {
    size_t best = 0;
    for (size_t i = 0; i < n; i++)
        if (logits[i] > logits[best]) best = i;
    return (uint32_t)best;
}
