/*
 * qt_oracle_fast.c - TEST INFRASTRUCTURE ONLY (see qt_oracle.h): AVX2 + FMA + F16C forms of the oracle's inner loops.
 *
 * The portable loops of qt_oracle_model.c / qt_oracle_blocks.c are written lane by lane in exactly the order of the
 * reference's AVX2 code (rust/crates/quintrit-runtime/src/ops.rs:970-1014 ggml_vec_dot_f16, :565-595 _f16_f32,
 * :688-712 _bf16, :1254-1347 vec_mad_f16 / vec_scale_f16; rust/crates/quintrit-core/src/block_scaled.rs:175-202), so
 * running eight of those lanes in one 256-bit register changes no bit: every lane still sees the same operations in
 * the same order, conversions are the hardware's round-to-nearest-even (ops.rs:2086-2109 holds the soft conversion to
 * the same bits for all 65536 halves), and -ffp-contract=off keeps multiplies and adds apart where the reference
 * keeps them apart. tests/test_oracle_fast.py holds every function here to its portable twin bit for bit.
 *
 * They exist so that the CPU side of the full-size parity fixtures (1536 tokens of a 40-layer model at a context of a
 * thousand positions) takes minutes instead of hours. The portable code stays the definition: the environment
 * variable QTO_PORTABLE=1 (read once) switches these off.
 */
#include "qt_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#if defined(__x86_64__)
#include <immintrin.h>
#define QTO_X86 1
#else
#define QTO_X86 0
#endif

static int g_fast_state = -1; /* -1: not decided yet */

/* Tests switch the vector forms off and on to compare the two (0 = portable only, 1 = vector forms where the CPU has them). */
void qto_fast_enable(int on) {
#if QTO_X86
    g_fast_state = on && __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma") && __builtin_cpu_supports("f16c");
#else
    (void)on;
    g_fast_state = 0;
#endif
}

int qto_fast_available(void) {
    if (g_fast_state < 0) {
        const char* off = getenv("QTO_PORTABLE");
        qto_fast_enable(!(off && off[0] == '1'));
    }
    return g_fast_state;
}

#if QTO_X86
#define FAST __attribute__((target("avx2,fma,f16c")))

FAST static inline __m256 load_h8(const uint16_t* p) { return _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)p)); }
FAST static inline void store_h8(uint16_t* p, __m256 v) {
    _mm_storeu_si128((__m128i*)p, _mm256_cvtps_ph(v, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
}
FAST static inline __m256 load_bf8(const uint16_t* p) {
    return _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_cvtepu16_epi32(_mm_loadu_si128((const __m128i*)p)), 16));
}

/* the four accumulators of whole groups of 32, as floats acc[j][l] */
FAST void qto_fast_dot_f16_groups(const uint16_t* x, const uint16_t* y, size_t n32, float acc[4][8]) {
    __m256 a0 = _mm256_setzero_ps(), a1 = a0, a2 = a0, a3 = a0;
    for (size_t i = 0; i < n32; i += 32) {
        a0 = _mm256_fmadd_ps(load_h8(x + i), load_h8(y + i), a0);
        a1 = _mm256_fmadd_ps(load_h8(x + i + 8), load_h8(y + i + 8), a1);
        a2 = _mm256_fmadd_ps(load_h8(x + i + 16), load_h8(y + i + 16), a2);
        a3 = _mm256_fmadd_ps(load_h8(x + i + 24), load_h8(y + i + 24), a3);
    }
    _mm256_storeu_ps(acc[0], a0), _mm256_storeu_ps(acc[1], a1), _mm256_storeu_ps(acc[2], a2), _mm256_storeu_ps(acc[3], a3);
}

FAST void qto_fast_dot_f16_f32_groups(const uint16_t* x, const float* y, size_t n32, float acc[4][8]) {
    __m256 a0 = _mm256_setzero_ps(), a1 = a0, a2 = a0, a3 = a0;
    for (size_t i = 0; i < n32; i += 32) {
        a0 = _mm256_fmadd_ps(load_h8(x + i), _mm256_loadu_ps(y + i), a0);
        a1 = _mm256_fmadd_ps(load_h8(x + i + 8), _mm256_loadu_ps(y + i + 8), a1);
        a2 = _mm256_fmadd_ps(load_h8(x + i + 16), _mm256_loadu_ps(y + i + 16), a2);
        a3 = _mm256_fmadd_ps(load_h8(x + i + 24), _mm256_loadu_ps(y + i + 24), a3);
    }
    _mm256_storeu_ps(acc[0], a0), _mm256_storeu_ps(acc[1], a1), _mm256_storeu_ps(acc[2], a2), _mm256_storeu_ps(acc[3], a3);
}

/* product and sum rounded separately */
FAST void qto_fast_dot_bf16_groups(const uint16_t* x, const uint16_t* y, size_t n32, float acc[4][8]) {
    __m256 a0 = _mm256_setzero_ps(), a1 = a0, a2 = a0, a3 = a0;
    for (size_t i = 0; i < n32; i += 32) {
        a0 = _mm256_add_ps(a0, _mm256_mul_ps(load_bf8(x + i), load_bf8(y + i)));
        a1 = _mm256_add_ps(a1, _mm256_mul_ps(load_bf8(x + i + 8), load_bf8(y + i + 8)));
        a2 = _mm256_add_ps(a2, _mm256_mul_ps(load_bf8(x + i + 16), load_bf8(y + i + 16)));
        a3 = _mm256_add_ps(a3, _mm256_mul_ps(load_bf8(x + i + 24), load_bf8(y + i + 24)));
    }
    _mm256_storeu_ps(acc[0], a0), _mm256_storeu_ps(acc[1], a1), _mm256_storeu_ps(acc[2], a2), _mm256_storeu_ps(acc[3], a3);
}

/* y[i] = f16(fma(f16(x[i]), v, f16(y[i]))) for whole groups of 8 (per element: the group size does not matter) */
FAST void qto_fast_mad_f16(uint16_t* y, const uint16_t* x, size_t n8, float v) {
    const __m256 vv = _mm256_set1_ps(v);
    for (size_t i = 0; i < n8; i += 8) store_h8(y + i, _mm256_fmadd_ps(load_h8(x + i), vv, load_h8(y + i)));
}
FAST void qto_fast_scale_f16(uint16_t* y, size_t n8, float v) {
    const __m256 vv = _mm256_set1_ps(v);
    for (size_t i = 0; i < n8; i += 8) store_h8(y + i, _mm256_mul_ps(load_h8(y + i), vv));
}
/* acc[i] = fma(f16(x[i]), v, acc[i]) */
FAST void qto_fast_mad_f16_f32(float* acc, const uint16_t* x, size_t n8, float v) {
    const __m256 vv = _mm256_set1_ps(v);
    for (size_t i = 0; i < n8; i += 8) _mm256_storeu_ps(acc + i, _mm256_fmadd_ps(load_h8(x + i), vv, _mm256_loadu_ps(acc + i)));
}
FAST void qto_fast_scale_f32(float* acc, size_t n8, float v) {
    const __m256 vv = _mm256_set1_ps(v);
    for (size_t i = 0; i < n8; i += 8) _mm256_storeu_ps(acc + i, _mm256_mul_ps(_mm256_loadu_ps(acc + i), vv));
}

/*
 * The block-scaled row dot (block_scaled.rs:175-202) for one planar row. The five digit planes of a 32-byte block are
 * taken apart arithmetically (byte = d0 + 3 d1 + 9 d2 + 28 d3 + 84 d4; bytes the packer never writes give zero trits,
 * as BYTE_TO_TRITS does), lane j of plane s is the exact integer sum of its four products, and the float chain is the
 * portable one: lane = fma(w_scale * a_scale, sum, lane) into the accumulator picked by the parity of s / 2.
 * act_pairs holds the sums of neighbouring activations (a[2k] + a[2k+1]) that turn digit products into trit products.
 */
FAST static inline __m256i digits_div(__m256i v, int mul) {
    /* floor(v * mul / 65536) on bytes, through 16-bit lanes */
    const __m256i z = _mm256_setzero_si256(), m = _mm256_set1_epi16((short)mul);
    const __m256i lo = _mm256_mulhi_epu16(_mm256_unpacklo_epi8(v, z), m), hi = _mm256_mulhi_epu16(_mm256_unpackhi_epi8(v, z), m);
    return _mm256_packus_epi16(lo, hi);
}

FAST float qto_fast_block_scaled_dot_row(const uint8_t* row, const float* w_scales, const int8_t* acts, const int16_t* act_pairs,
                                        const float* a_scales, size_t cols) {
    const size_t ns = cols / 32;
    __m256 acc0 = _mm256_setzero_ps(), acc1 = acc0;
    const __m256i one8 = _mm256_set1_epi8(1), one16 = _mm256_set1_epi16(1);
    /* digit tables for pshufb: index U = d3 + 3 d4 (0..8) and M = d0 + 3 d1 (0..8) */
    const __m256i t_mod3 = _mm256_setr_epi8(0, 1, 2, 0, 1, 2, 0, 1, 2, 0, 0, 0, 0, 0, 0, 0, 0, 1, 2, 0, 1, 2, 0, 1, 2, 0, 0, 0, 0, 0, 0, 0);
    const __m256i t_div3 = _mm256_setr_epi8(0, 0, 0, 1, 1, 1, 2, 2, 2, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 1, 1, 1, 2, 2, 2, 0, 0, 0, 0, 0, 0, 0);
    for (size_t g = 0; g * 5 < ns; ++g) {
        const __m256i b = _mm256_loadu_si256((const __m256i*)(row + g * 32));
        const __m256i U = digits_div(b, 2341);                                       /* floor(b / 28) for b <= 255 */
        /* 28 U = 32 U - 4 U per byte, modulo 256 (the 16-bit shifts spill only into bits that the masks clear) */
        const __m256i U4 = _mm256_and_si256(_mm256_slli_epi16(U, 2), _mm256_set1_epi8((char)0xFC));
        const __m256i U32 = _mm256_and_si256(_mm256_slli_epi16(U, 5), _mm256_set1_epi8((char)0xE0));
        const __m256i Lb = _mm256_sub_epi8(b, _mm256_sub_epi8(U32, U4));             /* b - 28 U, 0..27 (0..31 for junk bytes) */
        /* bytes that are no velurex code: L = 27 (the gap after every 27 values), or b > 250 (U = 8 with L > 26, U = 9) */
        const __m256i bad = _mm256_or_si256(_mm256_cmpgt_epi8(Lb, _mm256_set1_epi8(26)), _mm256_cmpgt_epi8(U, _mm256_set1_epi8(8)));
        const __m256i d2 = _mm256_sub_epi8(_mm256_setzero_si256(),
                                           _mm256_add_epi8(_mm256_cmpgt_epi8(Lb, _mm256_set1_epi8(8)), _mm256_cmpgt_epi8(Lb, _mm256_set1_epi8(17))));
        const __m256i d2x9 = _mm256_add_epi8(_mm256_and_si256(_mm256_slli_epi16(d2, 3), _mm256_set1_epi8((char)0xF8)), d2);
        const __m256i M = _mm256_and_si256(_mm256_sub_epi8(Lb, d2x9), _mm256_set1_epi8(15));
        __m256i dig[5];
        dig[0] = _mm256_shuffle_epi8(t_mod3, M);
        dig[1] = _mm256_shuffle_epi8(t_div3, M);
        dig[2] = d2;
        const __m256i Um = _mm256_and_si256(U, _mm256_set1_epi8(15));
        dig[3] = _mm256_shuffle_epi8(t_mod3, Um);
        dig[4] = _mm256_shuffle_epi8(t_div3, Um);
        for (int p = 0; p < 5; ++p) {
            const size_t s = g * 5 + (size_t)p;
            if (s >= ns) break;
            /* a junk byte decodes to five zero trits: digit 1 */
            const __m256i d = _mm256_blendv_epi8(dig[p], one8, bad);
            const __m256i a = _mm256_loadu_si256((const __m256i*)(acts + s * 32));
            /* sum over pairs of digit * act, minus the pair sums of act = sum over pairs of trit * act (|.| <= 256: exact in 16 bits) */
            const __m256i pr = _mm256_sub_epi16(_mm256_maddubs_epi16(d, a), _mm256_loadu_si256((const __m256i*)(act_pairs + s * 16)));
            const __m256i lanes = _mm256_madd_epi16(pr, one16);  /* eight sums of four consecutive products, in order */
            const __m256 dd = _mm256_set1_ps(w_scales[s / 2] * a_scales[s]);
            if ((s / 2) & 1)
                acc1 = _mm256_fmadd_ps(dd, _mm256_cvtepi32_ps(lanes), acc1);
            else
                acc0 = _mm256_fmadd_ps(dd, _mm256_cvtepi32_ps(lanes), acc0);
        }
    }
    float l[8];
    _mm256_storeu_ps(l, _mm256_add_ps(acc0, acc1));
    const float r0 = l[4] + l[0], r1 = l[5] + l[1], r2 = l[6] + l[2], r3 = l[7] + l[3];
    return (r0 + r2) + (r1 + r3);
}
#else
void qto_fast_dot_f16_groups(const uint16_t* x, const uint16_t* y, size_t n32, float acc[4][8]) { (void)x, (void)y, (void)n32, (void)acc; }
void qto_fast_dot_f16_f32_groups(const uint16_t* x, const float* y, size_t n32, float acc[4][8]) { (void)x, (void)y, (void)n32, (void)acc; }
void qto_fast_dot_bf16_groups(const uint16_t* x, const uint16_t* y, size_t n32, float acc[4][8]) { (void)x, (void)y, (void)n32, (void)acc; }
void qto_fast_mad_f16(uint16_t* y, const uint16_t* x, size_t n8, float v) { (void)y, (void)x, (void)n8, (void)v; }
void qto_fast_scale_f16(uint16_t* y, size_t n8, float v) { (void)y, (void)n8, (void)v; }
void qto_fast_mad_f16_f32(float* acc, const uint16_t* x, size_t n8, float v) { (void)acc, (void)x, (void)n8, (void)v; }
void qto_fast_scale_f32(float* acc, size_t n8, float v) { (void)acc, (void)n8, (void)v; }
float qto_fast_block_scaled_dot_row(const uint8_t* row, const float* w_scales, const int8_t* acts, const int16_t* act_pairs,
                                    const float* a_scales, size_t cols) {
    (void)row, (void)w_scales, (void)acts, (void)act_pairs, (void)a_scales, (void)cols;
    return 0.0f;
}
#endif
