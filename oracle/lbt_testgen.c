/*
 * Seeded input generators used by the reference's own tests, restated so the parity tests
 * can run the same cases (test infrastructure only).
 *   xorshift64 + unit float     crates/lb-ternary/tests/golden.rs:12-23
 *   golden `case` inputs        crates/lb-ternary/tests/golden.rs:25-35
 *   xorshift64* + ternary/unit  crates/lb-ternary-gpu/tests/gpu_matches_scalar.rs:8-24,28-31
 */
#include <stddef.h>
#include <stdint.h>

static uint64_t xs_next(uint64_t *s) {
    *s ^= *s << 13;
    *s ^= *s >> 7;
    *s ^= *s << 17;
    return *s;
}

/* (next >> 11) as f32 / 2^53 as f32 * 2 - 1, all in f32 */
static float xs_f(uint64_t *s) {
    float u = (float)(xs_next(s) >> 11);
    return u / 9007199254740992.0f * 2.0f - 1.0f;
}

uint64_t lbt_gen_xorshift_next(uint64_t *state) { return xs_next(state); }
float lbt_gen_xorshift_f(uint64_t *state) { return xs_f(state); }

/* golden.rs:28: latent weights (f+f+f)*0.02, rows*cols of them; state advances. */
void lbt_gen_golden_weights(uint64_t *state, size_t n, float *out) {
    for (size_t i = 0; i < n; i++) {
        float a = xs_f(state);
        float b = xs_f(state);
        float c = xs_f(state);
        out[i] = (a + b + c) * 0.02f;
    }
}

/* golden.rs:32-34: activations with an outlier (x20) where i % period == phase. */
void lbt_gen_golden_acts(uint64_t *state, size_t n, size_t period, size_t phase, float gain,
                         float *out) {
    for (size_t i = 0; i < n; i++) {
        float v = xs_f(state);
        out[i] = (i % period == phase) ? v * gain : v;
    }
}

/* golden.rs:138: (next % 3) as i8 - 1 */
void lbt_gen_xorshift_ternary(uint64_t *state, size_t n, int8_t *out) {
    for (size_t i = 0; i < n; i++) out[i] = (int8_t)(xs_next(state) % 3) - 1;
}

static uint64_t xss_next(uint64_t *s) {
    *s ^= *s >> 12;
    *s ^= *s << 25;
    *s ^= *s >> 27;
    return *s * 0x2545F4914F6CDD1DULL;
}

/* gpu_matches_scalar.rs:17-19 */
void lbt_gen_xss_ternary(uint64_t *state, size_t n, int8_t *out) {
    for (size_t i = 0; i < n; i++) out[i] = (int8_t)(xss_next(state) % 3) - 1;
}

/* gpu_matches_scalar.rs:20-22,31: unit() * 4.0 */
void lbt_gen_xss_acts(uint64_t *state, size_t n, float *out) {
    for (size_t i = 0; i < n; i++) {
        float u = (float)(xss_next(state) >> 40) / 16777216.0f * 2.0f - 1.0f;
        out[i] = u * 4.0f;
    }
}
