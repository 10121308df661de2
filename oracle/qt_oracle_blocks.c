/*
 * qt_oracle_blocks.c - TEST INFRASTRUCTURE ONLY (CPU restatement used as the parity checker; never shipped, never
 * called by the product). The block-scaled projection of Q2_0 models: Q8_0 activation blocks against velurex weights with
 * one scale per 64 weights, in the floating-point order of llama.cpp's Q2_0 x Q8_0 dot product.
 *
 * Parity pins (tests/test_oracle_blocks.py): the two formulations below (from planar bytes, from plain trits) agree bit
 * for bit on the shape grid of the reference's own test (rust/crates/quintrit-core/src/block_scaled.rs:1051-1063); the
 * quantiser's known answers (zero block -> codes 0 and scale 0, the largest value maps to +-127, reconstruction within
 * half a step: rust/crates/quintrit-runtime/tests/model_ops_tests.rs:51-70).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>

#include "qt_oracle.h"

uint16_t qto_f32_to_f16(float f);
float qto_f16_to_f32(uint16_t h);
int qto_fast_available(void);
float qto_fast_block_scaled_dot_row(const uint8_t* row, const float* w_scales, const int8_t* acts, const int16_t* act_pairs, const float* a_scales,
                                    size_t cols);

/* rust/crates/quintrit-runtime/src/ops.rs:898-910 (quantize_q8_0_scalar): per block of 32 values amax (NaN ignored),
 * d = f16(amax / 127) returned as f32, codes round_ties_even(x * (127 / amax)) clamped to [-128, 127]; NaN gives 0. */
void qto_quantize_q8_0(const float* x, size_t n, int8_t* qs, float* d) {
    for (size_t b = 0; b < n / 32; ++b) {
        const float* xb = x + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) {
            const float v = fabsf(xb[i]);
            if (v > amax) amax = v; /* f32::max ignores a NaN operand */
        }
        d[b] = qto_f16_to_f32(qto_f32_to_f16(amax / 127.0f));
        const float id = amax != 0.0f ? 127.0f / amax : 0.0f;
        for (int i = 0; i < 32; ++i) {
            const float r = nearbyintf(xb[i] * id); /* round-to-nearest-even in the default rounding mode */
            int q = 0;
            if (r == r) q = r >= 2147483648.0f ? 2147483647 : (r <= -2147483648.0f ? (-2147483647 - 1) : (int)r);
            qs[b * 32 + i] = (int8_t)(q < -128 ? -128 : (q > 127 ? 127 : q));
        }
    }
}

/* ((l0+l4) + (l2+l6)) + ((l1+l5) + (l3+l7)): rust/crates/quintrit-core/src/block_scaled.rs:140-145 (hsum8) */
static float hsum8(const float l[8]) {
    const float r0 = l[4] + l[0], r1 = l[5] + l[1], r2 = l[6] + l[2], r3 = l[7] + l[3];
    return (r0 + r2) + (r1 + r3);
}

/* rust/crates/quintrit-core/src/block_scaled.rs:175-202 (dot_row_scalar): activation block s is plane s % 5 of the
 * 160-trit block s / 5; eight integer lane sums of four products each; lane = fma(w_scale[s/2] * a_scale[s], sum, lane)
 * into the accumulator of the 64-weight block's parity; the two accumulators are added lane by lane, then hsum8. */
float qto_block_scaled_dot_row(const uint8_t* row, const float* w_scales, const int8_t* acts, const float* a_scales, size_t cols) {
    float acc[2][8] = {{0}};
    for (size_t s = 0; s < cols / 32; ++s) {
        const uint8_t* block = row + (s / 5) * 32;
        const int plane = (int)(s % 5);
        const int8_t* a = acts + s * 32;
        const float d = w_scales[s / 2] * a_scales[s];
        float* chain = acc[(s / 2) & 1];
        for (int j = 0; j < 8; ++j) {
            int32_t p = 0;
            for (int k = 4 * j; k < 4 * j + 4; ++k) {
                int8_t t[5];
                qto_byte_to_trits(block[k], t);
                p += (int32_t)t[plane] * (int32_t)a[k];
            }
            chain[j] = fmaf(d, (float)p, chain[j]);
        }
    }
    float l[8];
    for (int j = 0; j < 8; ++j) l[j] = acc[0][j] + acc[1][j];
    return hsum8(l);
}

/* The same value from one byte per trit (the definition the reference's test checks its kernels against,
 * rust/crates/quintrit-core/src/block_scaled.rs:1036-1049). */
float qto_block_scaled_dot_trits(const int8_t* trits, const float* w_scales, const int8_t* acts, const float* a_scales, size_t cols) {
    float acc[2][8] = {{0}};
    for (size_t s = 0; s < cols / 32; ++s) {
        const float d = w_scales[s / 2] * a_scales[s];
        for (int j = 0; j < 8; ++j) {
            int32_t p = 0;
            for (int k = 0; k < 4; ++k) p += (int32_t)trits[s * 32 + 4 * j + k] * (int32_t)acts[s * 32 + 4 * j + k];
            acc[(s / 2) & 1][j] = fmaf(d, (float)p, acc[(s / 2) & 1][j]);
        }
    }
    float l[8];
    for (int j = 0; j < 8; ++j) l[j] = acc[0][j] + acc[1][j];
    return ((l[4] + l[0]) + (l[6] + l[2])) + ((l[5] + l[1]) + (l[7] + l[3]));
}

/* Row-by-row GEMV (rust/crates/quintrit-core/src/block_scaled.rs:206-260): planar rows of ceil(cols/160)*32 bytes,
 * cols/64 weight scales per row, one activation scale per 32 activations. Rows are independent. */
void qto_gemv_block_scaled(const uint8_t* planar, const float* w_scales, const int8_t* acts, const float* a_scales, size_t rows, size_t cols,
                           float* out) {
    const size_t rb = qto_planar_row_bytes(cols), sb = cols / 64;
    if (qto_fast_available() && cols % 32 == 0) { /* the same lanes, eight at a time (qt_oracle_fast.c) */
        int16_t* pairs = (int16_t*)malloc(cols / 2 * sizeof(int16_t) + 64);
        for (size_t k = 0; k < cols / 2; ++k) pairs[k] = (int16_t)((int)acts[2 * k] + (int)acts[2 * k + 1]);
#pragma omp parallel for schedule(static)
        for (long r = 0; r < (long)rows; ++r)
            out[r] = qto_fast_block_scaled_dot_row(planar + (size_t)r * rb, w_scales + (size_t)r * sb, acts, pairs, a_scales, cols);
        free(pairs);
        return;
    }
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; ++r) out[r] = qto_block_scaled_dot_row(planar + (size_t)r * rb, w_scales + (size_t)r * sb, acts, a_scales, cols);
}
