/*
 * Timed CPU baseline: a C restatement ("port") of the reference's SIMD kernels for the
 * packed ternary x int8 matmul, threaded over row chunks with OpenMP the way the
 * reference threads them with rayon. TEST/BENCH INFRASTRUCTURE ONLY: it is the thing a
 * GPU number is reported beside, never part of the product path.
 *
 * Follows crates/lb-ternary/src/gemm.rs:
 *   decode256 / block_avx2 / codes_dot_avx2       gemm.rs:364-407
 *   decode512 / xpair / codes_dot_avx512vnni      gemm.rs:412-431,553-588
 *   row-chunk tasking (chunk_rows, 8 tasks/thread) gemm.rs:204-209
 *   decode branch (m == 1) / prefill branch        gemm.rs:137-194
 *   2-row x 4-token register tile idea             gemm.rs:478-550 (here on vpdpbusd)
 * The integers it produces must equal the scalar oracle's (tested).
 *
 * Build: gcc -O3 -fopenmp -fno-fast-math -ffp-contract=off -fPIC -shared.
 * ISA-specific functions carry target attributes; the best kernel is chosen at run time.
 */
#include <immintrin.h>
#include <omp.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define BLOCK 128
#define BLOCK_BYTES 32

enum { K_SCALAR = 0, K_AVX2 = 1, K_VNNI = 2 };

int lbt_simd_best_kernel(void) {
    __builtin_cpu_init();
    if (__builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") &&
        __builtin_cpu_supports("avx512vnni"))
        return K_VNNI;
    if (__builtin_cpu_supports("avx2")) return K_AVX2;
    return K_SCALAR;
}

const char *lbt_simd_kernel_name(int k) {
    return k == K_VNNI ? "avx512vnni" : k == K_AVX2 ? "avx2" : "scalar";
}

int lbt_simd_max_threads(void) { return omp_get_max_threads(); }

/* ---- scalar (gemm.rs:329-343), one token ---- */
static int32_t codes_dot_scalar1(const uint8_t *row, size_t nb, const int8_t *x) {
    int32_t acc = 0;
    for (size_t b = 0; b < nb; b++)
        for (size_t k = 0; k < 4; k++)
            for (size_t j = 0; j < BLOCK_BYTES; j++)
                acc += (int32_t)((row[b * BLOCK_BYTES + j] >> (2 * k)) & 3) *
                       (int32_t)x[b * BLOCK + k * 32 + j];
    return acc;
}

/* ---- AVX2 (gemm.rs:352-407) ---- */
__attribute__((target("avx2"))) static inline int32_t hsum256(__m256i v) {
    __m128i s = _mm_add_epi32(_mm256_castsi256_si128(v), _mm256_extracti128_si256(v, 1));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4e));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0xb1));
    return _mm_cvtsi128_si32(s);
}

__attribute__((target("avx2"))) static inline __m256i block_avx2(const uint8_t *p, const int8_t *xb) {
    const __m256i mask = _mm256_set1_epi8(3);
    __m256i v = _mm256_loadu_si256((const __m256i *)p);
    __m256i c0 = _mm256_and_si256(v, mask);
    __m256i c1 = _mm256_and_si256(_mm256_srli_epi16(v, 2), mask);
    __m256i c2 = _mm256_and_si256(_mm256_srli_epi16(v, 4), mask);
    __m256i c3 = _mm256_and_si256(_mm256_srli_epi16(v, 6), mask);
    __m256i s0 = _mm256_maddubs_epi16(c0, _mm256_loadu_si256((const __m256i *)xb));
    __m256i s1 = _mm256_maddubs_epi16(c1, _mm256_loadu_si256((const __m256i *)(xb + 32)));
    __m256i s2 = _mm256_maddubs_epi16(c2, _mm256_loadu_si256((const __m256i *)(xb + 64)));
    __m256i s3 = _mm256_maddubs_epi16(c3, _mm256_loadu_si256((const __m256i *)(xb + 96)));
    __m256i s = _mm256_add_epi16(_mm256_add_epi16(s0, s1), _mm256_add_epi16(s2, s3));
    return _mm256_madd_epi16(s, _mm256_set1_epi16(1));
}

__attribute__((target("avx2"))) static int32_t codes_dot_avx2_1(const uint8_t *row, size_t nb,
                                                               const int8_t *x) {
    __m256i a = _mm256_setzero_si256();
    for (size_t b = 0; b < nb; b++)
        a = _mm256_add_epi32(a, block_avx2(row + b * BLOCK_BYTES, x + b * BLOCK));
    return hsum256(a);
}

/* ---- AVX-512 VNNI (gemm.rs:412-431, 553-588) ---- */
#define VNNI_TARGET __attribute__((target("avx512f,avx512bw,avx512vnni,avx2")))

VNNI_TARGET static inline __m512i xpair(const int8_t *xb, int k) {
    __m256i lo = _mm256_loadu_si256((const __m256i *)(xb + k * 32));
    __m256i hi = _mm256_loadu_si256((const __m256i *)(xb + BLOCK + k * 32));
    return _mm512_inserti64x4(_mm512_castsi256_si512(lo), hi, 1);
}

/* R rows x T tokens over whole block pairs; the odd last block goes through block_avx2. */
#define DEF_TILE(R, T)                                                                            \
    VNNI_TARGET static void tile_vnni_##R##x##T(const uint8_t *const *rws, size_t nb,             \
                                                 const int8_t *x, size_t stride, int32_t *acc) { \
        const __m512i mask = _mm512_set1_epi8(3);                                                 \
        __m512i a[R][T];                                                                          \
        for (int r = 0; r < R; r++)                                                               \
            for (int t = 0; t < T; t++) a[r][t] = _mm512_setzero_si512();                         \
        size_t pairs = nb / 2;                                                                    \
        for (size_t bb = 0; bb < pairs; bb++) {                                                   \
            __m512i raw[R];                                                                       \
            for (int r = 0; r < R; r++)                                                           \
                raw[r] = _mm512_loadu_si512((const void *)(rws[r] + bb * 2 * BLOCK_BYTES));       \
            for (int k = 0; k < 4; k++) {                                                         \
                __m512i c[R];                                                                     \
                for (int r = 0; r < R; r++)                                                       \
                    c[r] = _mm512_and_si512(_mm512_srli_epi16(raw[r], 2 * k), mask);              \
                for (int t = 0; t < T; t++) {                                                     \
                    __m512i xv = xpair(x + t * stride + bb * 2 * BLOCK, k);                       \
                    for (int r = 0; r < R; r++) a[r][t] = _mm512_dpbusd_epi32(a[r][t], c[r], xv); \
                }                                                                                 \
            }                                                                                     \
        }                                                                                         \
        for (int r = 0; r < R; r++)                                                               \
            for (int t = 0; t < T; t++) {                                                         \
                int32_t v = _mm512_reduce_add_epi32(a[r][t]);                                     \
                if (nb & 1)                                                                       \
                    v += hsum256(block_avx2(rws[r] + (nb - 1) * BLOCK_BYTES,                      \
                                            x + t * stride + (nb - 1) * BLOCK));                  \
                acc[r * 4 + t] = v;                                                               \
            }                                                                                     \
    }
DEF_TILE(1, 1)
DEF_TILE(1, 2)
DEF_TILE(1, 3)
DEF_TILE(1, 4)
DEF_TILE(2, 1)
DEF_TILE(2, 2)
DEF_TILE(2, 3)
DEF_TILE(2, 4)

typedef void (*tile_fn)(const uint8_t *const *, size_t, const int8_t *, size_t, int32_t *);
static const tile_fn TILES[2][4] = {
    {tile_vnni_1x1, tile_vnni_1x2, tile_vnni_1x3, tile_vnni_1x4},
    {tile_vnni_2x1, tile_vnni_2x2, tile_vnni_2x3, tile_vnni_2x4},
};

/* Code dots (before the -sum correction) of rows r..r+rr-1 against tokens t..t+tt-1. */
static void tile_any(int kernel, const uint8_t *const *rws, int rr, size_t nb, const int8_t *x,
                     size_t stride, int tt, int32_t *acc /* [2][4] */) {
    if (kernel == K_VNNI) {
        TILES[rr - 1][tt - 1](rws, nb, x, stride, acc);
        return;
    }
    for (int r = 0; r < rr; r++)
        for (int t = 0; t < tt; t++)
            acc[r * 4 + t] = kernel == K_AVX2 ? codes_dot_avx2_1(rws[r], nb, x + t * stride)
                                              : codes_dot_scalar1(rws[r], nb, x + t * stride);
}

/* gemm.rs:204-209 */
static size_t chunk_rows(size_t n, int threads) {
    size_t c = (n + (size_t)threads * 8 - 1) / ((size_t)threads * 8);
    return c < 8 ? 8 : c;
}

/*
 * Several matrices sharing one quantised input (gemm.rs:128-195). Matrix i is
 * packed[i] = [rows[i], kp/4]; outs[i] (f32 [m, rows[i]]) and/or iouts[i] (i32 [m, rows[i]])
 * may be NULL. threads <= 0 means all.
 */
void lbt_simd_gemm_multi(int kernel, int threads, size_t nmat, const uint8_t *const *packed,
                         const size_t *rows, const float *wscale, size_t kp, const int8_t *q,
                         const float *ascale, const int32_t *asum, size_t m, float *const *outs,
                         int32_t *const *iouts) {
    if (threads <= 0) threads = omp_get_max_threads();
    size_t rb = kp / 4, nb = kp / BLOCK;
    size_t total = 0;
    for (size_t i = 0; i < nmat; i++) total += rows[i];
    size_t chunk = chunk_rows(total, threads);
    size_t ntasks = 0;
    for (size_t i = 0; i < nmat; i++) ntasks += (rows[i] + chunk - 1) / chunk;
    /* task table: (matrix, first row) */
    size_t *tm = (size_t *)malloc(sizeof(size_t) * 2 * (ntasks ? ntasks : 1));
    size_t n = 0;
    for (size_t i = 0; i < nmat; i++)
        for (size_t r0 = 0; r0 < rows[i]; r0 += chunk) {
            tm[2 * n] = i;
            tm[2 * n + 1] = r0;
            n++;
        }
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
    for (size_t task = 0; task < ntasks; task++) {
        size_t mi = tm[2 * task], r0 = tm[2 * task + 1];
        size_t r1 = r0 + chunk < rows[mi] ? r0 + chunk : rows[mi];
        const uint8_t *base = packed[mi];
        /* token tile outer so its activations stay in L1 (gemm.rs:245-268) */
        for (size_t t = 0; t < m; t += 4) {
            int tt = (int)(m - t < 4 ? m - t : 4);
            for (size_t r = r0; r < r1; r += 2) {
                int rr = (int)(r1 - r < 2 ? r1 - r : 2);
                const uint8_t *rws[2] = {base + r * rb, base + (r + rr - 1) * rb};
                int32_t acc[8];
                tile_any(kernel, rws, rr, nb, q + t * kp, kp, tt, acc);
                for (int i = 0; i < rr; i++)
                    for (int j = 0; j < tt; j++) {
                        int32_t d = acc[i * 4 + j] - asum[t + j];
                        size_t o = (t + j) * rows[mi] + r + i;
                        if (iouts && iouts[mi]) iouts[mi][o] = d;
                        if (outs && outs[mi])
                            outs[mi][o] = (float)d * (1.0f / (ascale[t + j] * wscale[mi]));
                    }
            }
        }
    }
    free(tm);
}

/* Threaded quantize_acts (quant.rs:45-75), scalar per row definition, rows in parallel. */
void lbt_quantize_row_scalar(const float *x, size_t n, int8_t *q, float *scale, int32_t *sum);
void lbt_simd_quantize_acts(int threads, const float *x, size_t m, size_t k, size_t kp, int8_t *q,
                            float *scale, int32_t *sum) {
    if (threads <= 0) threads = omp_get_max_threads();
    memset(q, 0, m * kp);
#pragma omp parallel for schedule(static) num_threads(threads) if (m > 1 && m * k >= 16384)
    for (size_t i = 0; i < m; i++) lbt_quantize_row_scalar(x + i * k, k, q + i * kp, &scale[i], &sum[i]);
}
