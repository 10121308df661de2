/*
 * qt_oracle_model.c - CPU restatement of the reference's float decode primitives and of its whole-token forward pass.
 * TEST INFRASTRUCTURE ONLY (see qt_oracle.h): the shipped library never calls into this file.
 *
 * Everything follows rust/crates/quintrit-runtime/src/{ops.rs, attention.rs, model.rs, kv_cache.rs}; the lines are
 * cited at each function. Transcendentals (expf, cosf, sinf, powf) are the host libm's, exactly as the reference
 * (Rust f32::exp/cos/sin/powf call the platform libm). Parity: the primitives are pinned by the reference's own unit
 * vectors where it has some (tests/test_oracle_model.py); the whole-token forward has NO stored vectors in the
 * reference (its CPU and GPU builds are only compared with each other at run time), so that level is "parity unpinned".
 */
#include "qt_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* AVX2 + FMA + F16C forms of the inner loops (qt_oracle_fast.c): the same lanes, eight at a time. */
int qto_fast_available(void);
void qto_fast_dot_f16_groups(const uint16_t* x, const uint16_t* y, size_t n32, float acc[4][8]);
void qto_fast_dot_f16_f32_groups(const uint16_t* x, const float* y, size_t n32, float acc[4][8]);
void qto_fast_dot_bf16_groups(const uint16_t* x, const uint16_t* y, size_t n32, float acc[4][8]);
void qto_fast_mad_f16(uint16_t* y, const uint16_t* x, size_t n8, float v);
void qto_fast_scale_f16(uint16_t* y, size_t n8, float v);
void qto_fast_mad_f16_f32(float* acc, const uint16_t* x, size_t n8, float v);
void qto_fast_scale_f32(float* acc, size_t n8, float v);

/* ---- half / bfloat conversions ---------------------------------------------------------------------------------- */

float qto_f16_to_f32(uint16_t h) { return qto_half_to_f32(h); } /* ops.rs:512-539 (exact) */

uint16_t qto_f32_to_f16(float f) {
    /* ops.rs:935-955 f32_to_f16_soft: round to nearest even, the same bits as F16C */
    uint32_t w;
    memcpy(&w, &f, 4);
    const float scale_to_inf = 0x1.0p+112f, scale_to_zero = 0x1.0p-110f; /* bits 0x77800000, 0x08800000 */
    float base = (fabsf(f) * scale_to_inf) * scale_to_zero;
    const uint32_t shl1_w = w + w, sign = w & 0x80000000u;
    uint32_t bias = shl1_w & 0xFF000000u;
    if (bias < 0x71000000u) bias = 0x71000000u;
    const uint32_t bb = (bias >> 1) + 0x07800000u;
    float fb;
    memcpy(&fb, &bb, 4);
    base = fb + base;
    uint32_t bits;
    memcpy(&bits, &base, 4);
    const uint32_t exp_bits = (bits >> 13) & 0x00007C00u, mant = bits & 0x00000FFFu;
    const uint32_t nonsign = exp_bits + mant;
    return (uint16_t)((sign >> 16) | (shl1_w > 0xFF000000u ? 0x7E00u : nonsign));
}

uint16_t qto_f32_to_bf16(float f) {
    /* ops.rs:652-660: round to nearest even on the upper 16 bits; a NaN keeps a quiet bit */
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 64);
    return (uint16_t)((u + (0x7FFFu + ((u >> 16) & 1u))) >> 16);
}

float qto_bf16_to_f32(uint16_t h) {
    const uint32_t u = (uint32_t)h << 16; /* ops.rs:662-664 */
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* ---- RMSNorm: ops.rs:44-57, 62-96 --------------------------------------------------------------------------------- */

void qto_rms_norm(const float* x, const float* w, size_t n, float eps, float* out) {
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) {
        const float sq = x[i] * x[i]; /* rounded to f32 first */
        sum += (double)sq;
    }
    const float mean = (float)(sum / (double)n);
    const float inv = 1.0f / sqrtf(mean + eps);
    for (size_t i = 0; i < n; ++i) {
        const float t = x[i] * inv; /* two roundings, no fusion */
        out[i] = t * w[i];
    }
}

/* ---- RoPE: ops.rs:121-141 (plain: freq_scale 1, ext_factor 0, attn_factor 1), 160-221 ----------------------------- */

void qto_rope_cache(size_t pos, size_t n_dims, float freq_base, float* cache) {
    const float theta_scale = powf(freq_base, -2.0f / (float)n_dims);
    float theta = (float)pos;
    for (size_t i0 = 0; i0 < n_dims; i0 += 2) {
        const float ti = 1.0f * theta; /* freq_scale * theta_extrap */
        cache[i0] = cosf(ti) * 1.0f;
        cache[i0 + 1] = sinf(ti) * 1.0f;
        theta *= theta_scale;
    }
}

/* mode 0 = Normal (pairs 2i, 2i+1), 1 = Neox (pairs i, i + n_dims/2) */
void qto_rope_apply(float* x, size_t heads, size_t head_dim, int mode, const float* cache, size_t n_dims) {
    const size_t offset = mode == 0 ? 1 : n_dims / 2, stride = mode == 0 ? 2 : 1;
    for (size_t h = 0; h < heads; ++h) {
        float* head = x + h * head_dim;
        for (size_t i = 0; i < n_dims / 2; ++i) {
            const float c = cache[2 * i], s = cache[2 * i + 1];
            const size_t a = i * stride;
            const float x0 = head[a], x1 = head[a + offset];
            head[a] = fmaf(x0, c, -(x1 * s));
            head[a + offset] = fmaf(x0, s, x1 * c);
        }
    }
}

/* ---- half dot products -------------------------------------------------------------------------------------------- */

float qto_vec_dot_f16(const uint16_t* x, const uint16_t* y, size_t n) {
    /* ops.rs:970-1014 (AVX2 order), model ops.rs:2010-2034: 4 accumulators x 8 lanes, (s0+s2)+(s1+s3), fold the upper
     * four lanes onto the lower four, two horizontal adds, scalar tail with separate multiply and add */
    float acc[4][8];
    memset(acc, 0, sizeof acc);
    size_t i = 0;
    if (qto_fast_available()) {
        i = n / 32 * 32;
        qto_fast_dot_f16_groups(x, y, i, acc);
    }
    for (; i + 32 <= n; i += 32)
        for (int j = 0; j < 4; ++j)
            for (int l = 0; l < 8; ++l) {
                const size_t k = i + 8 * (size_t)j + (size_t)l;
                acc[j][l] = fmaf(qto_f16_to_f32(x[k]), qto_f16_to_f32(y[k]), acc[j][l]);
            }
    float red[8], t0[4];
    for (int l = 0; l < 8; ++l) red[l] = (acc[0][l] + acc[2][l]) + (acc[1][l] + acc[3][l]);
    for (int l = 0; l < 4; ++l) t0[l] = red[l] + red[l + 4];
    float sum = (t0[0] + t0[1]) + (t0[2] + t0[3]);
    for (; i < n; ++i) {
        const float p = qto_f16_to_f32(x[i]) * qto_f16_to_f32(y[i]);
        sum += p;
    }
    return sum;
}

float qto_vec_dot_f16_f32(const uint16_t* x, const float* y, size_t n) {
    /* ops.rs:565-595: groups of 32 into 4 x 8 lanes, a further group of 8 into accumulator 0, (a0+a1)+(a2+a3),
     * lanes ((l0+l4)+(l2+l6)) + ((l1+l5)+(l3+l7)), tail in double */
    float acc[4][8];
    memset(acc, 0, sizeof acc);
    size_t i = 0;
    if (qto_fast_available()) {
        i = n / 32 * 32;
        qto_fast_dot_f16_f32_groups(x, y, i, acc);
    }
    for (; i + 32 <= n; i += 32)
        for (int j = 0; j < 4; ++j)
            for (int l = 0; l < 8; ++l) {
                const size_t k = i + 8 * (size_t)j + (size_t)l;
                acc[j][l] = fmaf(qto_f16_to_f32(x[k]), y[k], acc[j][l]);
            }
    for (; i + 8 <= n; i += 8)
        for (int l = 0; l < 8; ++l) acc[0][l] = fmaf(qto_f16_to_f32(x[i + (size_t)l]), y[i + (size_t)l], acc[0][l]);
    float a[8], r[4];
    for (int l = 0; l < 8; ++l) a[l] = (acc[0][l] + acc[1][l]) + (acc[2][l] + acc[3][l]);
    for (int l = 0; l < 4; ++l) r[l] = a[l] + a[l + 4];
    double sum = (double)((r[0] + r[2]) + (r[1] + r[3]));
    for (; i < n; ++i) {
        const float p = qto_f16_to_f32(x[i]) * y[i];
        sum += (double)p;
    }
    return (float)sum;
}

/* ---- activations -------------------------------------------------------------------------------------------------- */

static float from_bits(uint32_t u) {
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static uint32_t to_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}

/* One lane of ops.rs:316-387 (ggml's vector expf): the branches select per lane, so a lane's value does not depend on
 * its neighbours. */
float qto_ggml_expf_lane(float x) {
    const float r = from_bits(0x4b400000u);
    const float z = fmaf(x, from_bits(0x3fb8aa3bu), r);
    const float n = z - r;
    const float b = fmaf(-n, from_bits(0x35bfbe8eu), fmaf(-n, from_bits(0x3f317200u), x));
    const uint32_t e = to_bits(z) << 23;
    const float k = from_bits(e + to_bits(1.0f));
    const int c = fabsf(n) > 126.0f;
    const float u = b * b;
    const float j = fmaf(fmaf(fmaf(from_bits(0x3c072010u), b, from_bits(0x3d2b9f17u)), u,
                              fmaf(from_bits(0x3e2aaf33u), b, from_bits(0x3efffedbu))),
                         u, from_bits(0x3f7ffff6u) * b);
    if (!c) return fmaf(j, k, k);
    const uint32_t g = (n <= 0.0f) ? 0x82000000u : 0u;
    const float s1 = from_bits(g + 0x7f000000u);
    const float s2 = from_bits(e - g);
    const int d = fabsf(n) > 192.0f;
    if (d) return s1 * s1;
    return fmaf(s2, j, s2) * s1;
}

float qto_silu(float x) {
    /* ops.rs:389-399: x / (1 + expf(-x)) with the polynomial expf and a true division */
    const float neg = 0.0f - x;
    return x / (1.0f + qto_ggml_expf_lane(neg));
}

void qto_swiglu(const float* gate, const float* up, size_t n, float* out) {
    /* ops.rs:427-464; vector body for whole groups of 8, libm for the remainder */
    size_t i = 0;
    for (; i + 8 <= n; i += 8)
        for (size_t l = 0; l < 8; ++l) out[i + l] = qto_silu(gate[i + l]) * up[i + l];
    for (; i < n; ++i) {
        const float v = gate[i];
        out[i] = (v / (1.0f + expf(-v))) * up[i];
    }
}

void qto_relu2_mul(const float* gate, const float* up, size_t n, float* out) {
    /* ops.rs:301-308 + 467-473 */
    for (size_t i = 0; i < n; ++i) {
        const float p = gate[i] > 0.0f ? gate[i] : 0.0f;
        const float sq = p * p;
        out[i] = sq * up[i];
    }
}

/* The expf the device uses, restated on the CPU so that it can be checked against the host libm bit for bit:
 * glibc's single-precision exp (the published table algorithm: N = 32 entries of 2^(i/N), a cubic in double). */
static uint64_t g_exp2_tab[32];
static int g_exp2_ready = 0;
static void exp2_tab_init(void) {
    if (g_exp2_ready) return;
    for (int i = 0; i < 32; ++i) {
        const double v = exp2((double)i / 32.0);
        uint64_t b;
        memcpy(&b, &v, 8);
        g_exp2_tab[i] = b - ((uint64_t)i << 47);
    }
    g_exp2_ready = 1;
}
const uint64_t* qto_exp2_table(void) {
    exp2_tab_init();
    return g_exp2_tab;
}
float qto_expf_restated(float x) {
    exp2_tab_init();
    const double inv_ln2_n = 0x1.71547652b82fep0 * 32.0, shift = 0x1.8p52;
    const double c0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0, c1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0, c2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    const uint32_t ix = to_bits(x), abstop = (ix >> 20) & 0x7ff;
    if (abstop >= 0x42b) {
        if (ix == 0xff800000u) return 0.0f;
        if (abstop >= 0x7f8) return x + x;
        if (x > 0x1.62e42ep6f) return INFINITY;
        if (x < -0x1.9fe368p6f) return 0.0f;
    }
    const double xd = (double)x;
    const double z0 = inv_ln2_n * xd;
    double kd = z0 + shift;
    uint64_t ki;
    memcpy(&ki, &kd, 8);
    kd -= shift;
    const double r = z0 - kd;
    const uint64_t t = g_exp2_tab[ki % 32] + (ki << 47);
    double s;
    memcpy(&s, &t, 8);
    const double z = fma(c0, r, c1);
    const double r2 = r * r;
    double y = fma(c2, r, 1.0);
    y = fma(z, r2, y);
    y = y * s;
    return (float)y;
}

/* ---- half-precision value accumulation: ops.rs:1254-1298 (fused for whole groups of 32, separate for the tail),
 *      ops.rs:1304-1347, ops.rs:1502-1525 ------------------------------------------------------------------------- */

static void vec_mad_f16(uint16_t* y, const uint16_t* x, size_t n, float v) {
    size_t i = 0;
    if (qto_fast_available()) {
        i = n / 32 * 32;
        qto_fast_mad_f16(y, x, i, v);
    }
    for (; i + 32 <= n; i += 32)
        for (size_t l = 0; l < 32; ++l) y[i + l] = qto_f32_to_f16(fmaf(qto_f16_to_f32(x[i + l]), v, qto_f16_to_f32(y[i + l])));
    for (; i < n; ++i) {
        const float p = qto_f16_to_f32(x[i]) * v;
        y[i] = qto_f32_to_f16(qto_f16_to_f32(y[i]) + p);
    }
}
static void vec_scale_f16(uint16_t* y, size_t n, float v) {
    size_t i = 0;
    if (qto_fast_available()) {
        i = n / 8 * 8;
        qto_fast_scale_f16(y, i, v);
    }
    for (; i < n; ++i) y[i] = qto_f32_to_f16(qto_f16_to_f32(y[i]) * v);
}

/* attention.rs:438-469 attend_range: online softmax over [p0, p1) with an F16 accumulator. K and V rows are `stride`
 * halves apart (the cache holds [pos][kv_head][head_dim]). Returns M and S. */
static void attend_range_f16(const uint16_t* q16, const uint16_t* k, const uint16_t* v, size_t stride, size_t p0, size_t p1, size_t hd,
                             float scale, uint16_t* vkq16, float* m_out, float* s_out) {
    float s_sum = 0.0f, max_score = -INFINITY;
    memset(vkq16, 0, hd * 2);
    for (size_t p = p0; p < p1; ++p) {
        const float score = qto_vec_dot_f16(q16, k + p * stride, hd) * scale;
        const float m_old = max_score;
        float ms = 1.0f, vs = 1.0f;
        if (score > max_score) {
            max_score = score;
            ms = expf(m_old - max_score);
            vec_scale_f16(vkq16, hd, ms);
        } else {
            vs = expf(score - max_score);
        }
        vec_mad_f16(vkq16, v + p * stride, hd, vs);
        s_sum = fmaf(s_sum, ms, vs);
    }
    *m_out = max_score;
    *s_out = s_sum;
}

/* attention.rs:402-434 attend_range_f32 */
static void attend_range_f32(const float* q, const uint16_t* k, const uint16_t* v, size_t stride, size_t p0, size_t p1, size_t hd,
                             float scale, float* vkq, float* m_out, float* s_out) {
    float s_sum = 0.0f, max_score = -INFINITY;
    memset(vkq, 0, hd * 4);
    for (size_t p = p0; p < p1; ++p) {
        const float score = qto_vec_dot_f16_f32(k + p * stride, q, hd) * scale;
        const float m_old = max_score;
        float ms = 1.0f, vs = 1.0f;
        if (score > max_score) {
            max_score = score;
            ms = expf(m_old - max_score);
            size_t d = 0;
            if (qto_fast_available()) {
                d = hd / 8 * 8;
                qto_fast_scale_f32(vkq, d, ms);
            }
            for (; d < hd; ++d) vkq[d] *= ms;
        } else {
            vs = expf(score - max_score);
        }
        size_t d = 0;
        if (qto_fast_available()) {
            d = hd / 8 * 8;
            qto_fast_mad_f16_f32(vkq, v + p * stride, d, vs);
        }
        for (; d < hd; ++d) vkq[d] = fmaf(qto_f16_to_f32(v[p * stride + d]), vs, vkq[d]);
        s_sum = fmaf(s_sum, ms, vs);
    }
    *m_out = max_score;
    *s_out = s_sum;
}

/*
 * attention.rs:483-596 attend_head / attend_head_f32. k and v point at the head's first row (position 0); rows are
 * `stride` halves apart; max_seq_len is the allocated cache length. f32_values selects the llama.cpp arithmetic.
 */
void qto_attend_head(const float* q, const uint16_t* k, const uint16_t* v, size_t stride, size_t seq_len, size_t max_seq_len, size_t hd,
                     float scale, int f32_values, float* out) {
    size_t n_kv = (seq_len + 255) / 256 * 256;
    if (n_kv < 256) n_kv = 256;
    if (n_kv > max_seq_len) n_kv = max_seq_len;
    uint16_t* q16 = (uint16_t*)malloc(hd * 2);
    uint16_t* vkq16 = (uint16_t*)malloc(hd * 2);
    float* part = (float*)malloc(hd * 4);
    float* acc = (float*)malloc(hd * 4);
    for (size_t d = 0; d < hd; ++d) q16[d] = qto_f32_to_f16(q[d]);
    float m, s;
    if (n_kv < 512) {
        if (f32_values) {
            attend_range_f32(q, k, v, stride, 0, seq_len, hd, scale, out, &m, &s);
            const float s_inv = s == 0.0f ? 0.0f : 1.0f / s;
            for (size_t d = 0; d < hd; ++d) out[d] *= s_inv;
        } else {
            attend_range_f16(q16, k, v, stride, 0, seq_len, hd, scale, vkq16, &m, &s);
            const float s_inv = s == 0.0f ? 0.0f : 1.0f / s;
            for (size_t d = 0; d < hd; ++d) out[d] = qto_f16_to_f32(vkq16[d]) * s_inv;
        }
    } else {
        const size_t chunk = (n_kv + 3) / 4;
        float m_final = -INFINITY, s_final = 0.0f;
        memset(acc, 0, hd * 4);
        for (size_t c = 0; c < 4; ++c) {
            const size_t start = c * chunk;
            size_t end = start + chunk;
            if (end > n_kv) end = n_kv;
            if (end > seq_len) end = seq_len;
            if (start >= end) continue;
            if (f32_values) {
                attend_range_f32(q, k, v, stride, start, end, hd, scale, part, &m, &s);
            } else {
                attend_range_f16(q16, k, v, stride, start, end, hd, scale, vkq16, &m, &s);
                for (size_t d = 0; d < hd; ++d) part[d] = qto_f16_to_f32(vkq16[d]);
            }
            if (s == 0.0f) continue;
            const float m_new = m_final > m ? m_final : m;
            const float scale_old = expf(m_final - m_new), scale_new = expf(m - m_new);
            for (size_t d = 0; d < hd; ++d) {
                const float pn = part[d] * scale_new;
                acc[d] = fmaf(acc[d], scale_old, pn);
            }
            const float sn = s * scale_new;
            s_final = fmaf(s_final, scale_old, sn);
            m_final = m_new;
        }
        if (s_final != 0.0f) {
            const float s_inv = 1.0f / s_final;
            for (size_t d = 0; d < hd; ++d) out[d] = acc[d] * s_inv;
        } else {
            memcpy(out, acc, hd * 4);
        }
    }
    free(q16);
    free(vkq16);
    free(part);
    free(acc);
}

/* rust/crates/quintrit-runtime/src/ops.rs:688-712 (ggml_vec_dot_bf16_scalar): four accumulators of eight lanes take
 * acc + x*y with the product and the sum rounded separately (no FMA); (a0+a2)+(a1+a3); g_l = a_{l+4} + a_l;
 * (g0+g2)+(g1+g3); the tail beyond whole groups of 32 is added in double precision. */
float qto_vec_dot_bf16(const uint16_t* x, const uint16_t* y, size_t n) {
    float acc[4][8] = {{0}};
    size_t i = 0;
    if (qto_fast_available()) {
        i = n / 32 * 32;
        qto_fast_dot_bf16_groups(x, y, i, acc);
    }
    for (; i + 32 <= n; i += 32)
        for (int j = 0; j < 4; ++j)
            for (int l = 0; l < 8; ++l) {
                const size_t k = i + 8 * (size_t)j + (size_t)l;
                const float prod = qto_bf16_to_f32(x[k]) * qto_bf16_to_f32(y[k]);
                acc[j][l] = acc[j][l] + prod;
            }
    float a[8];
    for (int l = 0; l < 8; ++l) a[l] = (acc[0][l] + acc[2][l]) + (acc[1][l] + acc[3][l]);
    const float g0 = a[4] + a[0], g1 = a[5] + a[1], g2 = a[6] + a[2], g3 = a[7] + a[3];
    double sum = (double)((g0 + g2) + (g1 + g3));
    for (; i < n; ++i) sum += (double)(qto_bf16_to_f32(x[i]) * qto_bf16_to_f32(y[i]));
    return (float)sum;
}

/* rust/crates/quintrit-runtime/src/sampler.rs:73-83: first index of the strict maximum; NaN never wins */
uint32_t qto_argmax(const float* logits, size_t n) {
    size_t best = 0;
    float bv = -INFINITY;
    for (size_t i = 0; i < n; ++i)
        if (logits[i] > bv) {
            bv = logits[i];
            best = i;
        }
    return (uint32_t)best;
}

/* ---- whole-token forward: model.rs:64-203, 282-377; attention.rs:115-260 ------------------------------------------ */

void qto_quantize_q8_0(const float* x, size_t n, int8_t* qs, float* d);
void qto_gemv_block_scaled(const uint8_t* planar, const float* w_scales, const int8_t* acts, const float* a_scales, size_t rows, size_t cols,
                           float* out);

typedef struct qto_model {
    int arch;     /* 0 = llama / falcon3 (interleaved RoPE, SwiGLU), 1 = bitnet (NEOX RoPE, relu^2, sub-norms), 2 = qwen2 / qwen3 (NEOX RoPE, SwiGLU; config.rs:464-467) */
    int f32_values; /* attention accumulators: 0 = F16 (I2_S files), 1 = F32 (TQ1_0 / TQ2_0 files) */
    int hidden, inter, layers, q_heads, kv_heads, head_dim, vocab, ctx, rope_dims;
    float eps, rope_theta;
    const uint16_t* embed;   /* F16 [vocab][hidden] */
    const uint16_t* lm_head; /* F16 [vocab][hidden], NULL = tied to embed */
    const float* out_norm;
    const uint8_t** w;       /* layers * 7 planar matrices: q, k, v, o, gate, up, down */
    const float* scales;     /* layers * 7 weight scales */
    const float** norms;     /* layers * 4: attn_norm, ffn_norm, attn_sub_norm, ffn_sub_norm (the last two NULL for arch 0) */
    uint16_t *kc, *vc;       /* [layer][pos][kv_head][head_dim] */
    uint8_t** w64;           /* 64-row tiled copies for the AVX-512 GEMV (same integers, only faster), or NULL */
    int bf16_tables;         /* embedding and output head are BF16 instead of F16 (qto_model_set_bf16_tables) */
    const float** block_scales; /* layers * 7 arrays of rows * cols / 64 weight scales: Q2_0 projections (qto_model_set_block_scales) */
    const float** qk_norms;  /* layers * 2 arrays of head_dim weights: RMSNorm of every query and key head before RoPE (qto_model_set_qk_norms), or NULL */
} qto_model_t;

qto_model_t* qto_model_create(int arch, int f32_values, int hidden, int inter, int layers, int q_heads, int kv_heads, int head_dim,
                              int vocab, int ctx, int rope_dims, float eps, float rope_theta, const uint16_t* embed,
                              const uint16_t* lm_head, const float* out_norm, const uint8_t** w, const float* scales, const float** norms) {
    qto_model_t* m = (qto_model_t*)calloc(1, sizeof *m);
    m->arch = arch, m->f32_values = f32_values, m->hidden = hidden, m->inter = inter, m->layers = layers, m->q_heads = q_heads;
    m->kv_heads = kv_heads, m->head_dim = head_dim, m->vocab = vocab, m->ctx = ctx, m->rope_dims = rope_dims, m->eps = eps;
    m->rope_theta = rope_theta, m->embed = embed, m->lm_head = lm_head, m->out_norm = out_norm, m->w = w, m->scales = scales, m->norms = norms;
    const size_t n = (size_t)layers * ctx * kv_heads * head_dim;
    m->kc = (uint16_t*)calloc(n, 2);
    m->vc = (uint16_t*)calloc(n, 2);
    if (qto_cpu_has_avx512_vbmi()) {
        const size_t H = (size_t)hidden, I = (size_t)inter, qd = (size_t)q_heads * head_dim, kvd = (size_t)kv_heads * head_dim;
        const size_t shp[7][2] = {{qd, H}, {kvd, H}, {kvd, H}, {H, qd}, {I, H}, {I, H}, {H, I}};
        m->w64 = (uint8_t**)calloc((size_t)layers * 7, sizeof(uint8_t*));
        for (int i = 0; i < layers * 7; ++i) {
            m->w64[i] = (uint8_t*)malloc(qto_tile64_bytes(shp[i % 7][0], shp[i % 7][1]));
            qto_tile64(w[i], shp[i % 7][0], shp[i % 7][1], m->w64[i]);
        }
    }
    return m;
}
void qto_model_set_bf16_tables(qto_model_t* m, int on) { m->bf16_tables = on != 0; }
/* Q2_0 models: every projection is block-scaled (attention.rs:262-344, model.rs:209-229); the tensor scales are unused */
void qto_model_set_block_scales(qto_model_t* m, const float** scales) { m->block_scales = scales; }
/* query/key-norm models (attention.rs:282-294: the block-scaled path normalises every query and key head before RoPE) */
void qto_model_set_qk_norms(qto_model_t* m, const float** norms) { m->qk_norms = norms; }

void qto_model_free(qto_model_t* m) {
    if (!m) return;
    free(m->kc);
    free(m->vc);
    if (m->w64) {
        for (int i = 0; i < m->layers * 7; ++i) free(m->w64[i]);
        free(m->w64);
    }
    free(m);
}

/* layer.rs:123-177: quantised input -> exact integers -> one multiply by weight_scale / act_scale */
static void project(const qto_model_t* m, int layer, int which, size_t rows, size_t cols, const int8_t* act, float act_scale, float* out) {
    int32_t* acc = (int32_t*)malloc(rows * 4);
    int nt = 1;
#ifdef _OPENMP
    nt = omp_get_max_threads();
#endif
    if (m->w64)
        qto_cpu_gemv_avx512(m->w64[layer * 7 + which], rows, cols, act, acc, nt);
    else
        qto_cpu_gemv_portable(m->w[layer * 7 + which], rows, cols, act, acc, nt);
    qto_rescale(acc, rows, m->scales[layer * 7 + which], act_scale, out);
    free(acc);
}

/* attention.rs:276-280, 342-343; model.rs:211-228: the input quantised to Q8_0 blocks, then the Q2_0 x Q8_0 dot of every row */
static void project_q8(const qto_model_t* m, int layer, int which, size_t rows, size_t cols, const int8_t* qs, const float* d, float* out) {
    qto_gemv_block_scaled(m->w[layer * 7 + which], m->block_scales[layer * 7 + which], qs, d, rows, cols, out);
}

void qto_model_forward(qto_model_t* m, uint32_t token, size_t pos, float* logits) {
    const size_t H = (size_t)m->hidden, I = (size_t)m->inter, hd = (size_t)m->head_dim;
    const size_t qd = (size_t)m->q_heads * hd, kvd = (size_t)m->kv_heads * hd;
    const size_t big = I > qd ? I : qd;
    float* x = (float*)malloc(H * 4);
    float* xn = (float*)malloc((big > H ? big : H) * 4);
    float* q = (float*)malloc(qd * 4);
    float* k = (float*)malloc(kvd * 4);
    float* v = (float*)malloc(kvd * 4);
    float* att = (float*)malloc((qd > H ? qd : H) * 4);
    float* gate = (float*)malloc(I * 4);
    float* up = (float*)malloc(I * 4);
    float* inter = (float*)malloc(I * 4);
    float* delta = (float*)malloc(H * 4);
    int8_t* a8 = (int8_t*)malloc(big > H ? big : H);
    float* d8 = (float*)malloc(((big > H ? big : H) / 32 + 1) * 4); /* Q8_0 block scales */
    const int bs = m->block_scales != NULL;
    float* cache = (float*)malloc((size_t)m->rope_dims * 4);
    const float scale = 1.0f / sqrtf((float)m->head_dim); /* attention.rs:46 */

    /* model.rs:308-317; BF16 tables: hybrid.rs:364-367 (bf16_to_f32 of the row) */
    for (size_t i = 0; i < H; ++i) x[i] = m->bf16_tables ? qto_bf16_to_f32(m->embed[(size_t)token * H + i]) : qto_f16_to_f32(m->embed[(size_t)token * H + i]);
    for (int l = 0; l < m->layers; ++l) {
        const float** nw = m->norms + l * 4;
        qto_rms_norm(x, nw[0], H, m->eps, xn);
        float s = 0.0f;
        if (bs) {
            qto_quantize_q8_0(xn, H, a8, d8);
            project_q8(m, l, 0, qd, H, a8, d8, q);
            project_q8(m, l, 1, kvd, H, a8, d8, k);
            project_q8(m, l, 2, kvd, H, a8, d8, v);
        } else {
            s = qto_quantize_int8(xn, H, a8);
            project(m, l, 0, qd, H, a8, s, q);
            project(m, l, 1, kvd, H, a8, s, k);
            project(m, l, 2, kvd, H, a8, s, v);
        }
        if (m->qk_norms != NULL && m->qk_norms[l * 2] != NULL && m->qk_norms[l * 2 + 1] != NULL) { /* attention.rs:282-294 */
            float head[4096];
            for (size_t h = 0; h < (size_t)m->q_heads; ++h) {
                memcpy(head, q + h * hd, hd * 4);
                qto_rms_norm(head, m->qk_norms[l * 2], hd, m->eps, q + h * hd);
            }
            for (size_t h = 0; h < (size_t)m->kv_heads; ++h) {
                memcpy(head, k + h * hd, hd * 4);
                qto_rms_norm(head, m->qk_norms[l * 2 + 1], hd, m->eps, k + h * hd);
            }
        }
        qto_rope_cache(pos, (size_t)m->rope_dims, m->rope_theta, cache);
        qto_rope_apply(q, (size_t)m->q_heads, hd, m->arch != 0, cache, (size_t)m->rope_dims);
        qto_rope_apply(k, (size_t)m->kv_heads, hd, m->arch != 0, cache, (size_t)m->rope_dims);
        uint16_t* kc = m->kc + ((size_t)l * m->ctx) * kvd;
        uint16_t* vc = m->vc + ((size_t)l * m->ctx) * kvd;
        for (size_t i = 0; i < kvd; ++i) {
            kc[pos * kvd + i] = qto_f32_to_f16(k[i]);
            vc[pos * kvd + i] = qto_f32_to_f16(v[i]);
        }
        const size_t gqa = (size_t)(m->q_heads / m->kv_heads);
#pragma omp parallel for schedule(dynamic, 1) /* heads are independent (attention.rs:205-232) */
        for (long hh = 0; hh < (long)m->q_heads; ++hh) {
            const size_t h = (size_t)hh, kvh = h / gqa;
            qto_attend_head(q + h * hd, kc + kvh * hd, vc + kvh * hd, kvd, pos + 1, (size_t)m->ctx, hd, scale, m->f32_values, att + h * hd);
        }
        const float* o_in = att;
        if (nw[2]) { /* attention.rs:234-246 sub-norm (BitNet) */
            qto_rms_norm(att, nw[2], qd, m->eps, xn);
            o_in = xn;
        }
        if (bs) {
            qto_quantize_q8_0(o_in, qd, a8, d8);
            project_q8(m, l, 3, H, qd, a8, d8, delta);
        } else {
            s = qto_quantize_int8(o_in, qd, a8);
            project(m, l, 3, H, qd, a8, s, delta);
        }
        for (size_t i = 0; i < H; ++i) x[i] += delta[i]; /* model.rs:85 */
        qto_rms_norm(x, nw[1], H, m->eps, xn);
        if (bs) {
            qto_quantize_q8_0(xn, H, a8, d8);
            project_q8(m, l, 4, I, H, a8, d8, gate);
            project_q8(m, l, 5, I, H, a8, d8, up);
        } else {
            s = qto_quantize_int8(xn, H, a8);
            project(m, l, 4, I, H, a8, s, gate);
            project(m, l, 5, I, H, a8, s, up);
        }
        if (m->arch == 1)
            qto_relu2_mul(gate, up, I, inter);
        else
            qto_swiglu(gate, up, I, inter);
        const float* down_in = inter;
        if (nw[3]) {
            qto_rms_norm(inter, nw[3], I, m->eps, xn);
            down_in = xn;
        }
        if (bs) {
            qto_quantize_q8_0(down_in, I, a8, d8);
            project_q8(m, l, 6, H, I, a8, d8, delta);
        } else {
            s = qto_quantize_int8(down_in, I, a8);
            project(m, l, 6, H, I, a8, s, delta);
        }
        for (size_t i = 0; i < H; ++i) x[i] += delta[i];
    }
    qto_rms_norm(x, m->out_norm, H, m->eps, xn); /* model.rs:326-331 */
    uint16_t* x16 = (uint16_t*)malloc(H * 2);
    for (size_t i = 0; i < H; ++i) x16[i] = m->bf16_tables ? qto_f32_to_bf16(xn[i]) : qto_f32_to_f16(xn[i]); /* hybrid.rs:327-333 for BF16 */
    const uint16_t* head = m->lm_head ? m->lm_head : m->embed;
#pragma omp parallel for schedule(static)
    for (long t = 0; t < (long)m->vocab; ++t) /* model.rs:346-375 */
        logits[t] = m->bf16_tables ? qto_vec_dot_bf16(x16, head + (size_t)t * H, H) : qto_vec_dot_f16(x16, head + (size_t)t * H, H);
    free(x16), free(x), free(xn), free(q), free(k), free(v), free(att), free(gate), free(up), free(inter), free(delta), free(a8), free(d8), free(cache);
}
