/*
 * qt_oracle.c - CPU restatement of the reference's velurex packing, exact GEMV, activation quantiser and GGUF ternary
 * decoders. TEST INFRASTRUCTURE ONLY (see qt_oracle.h): the shipped library never calls into this file.
 *
 * Parity pins: tests/test_oracle_pack.py, tests/test_oracle_gemv.py and tests/test_oracle_decoders.py check this file
 * against the known answers held by the reference's own unit tests (cited there).
 */
#include "qt_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------------------------------------ */
/* velurex byte, planar layout (quintrit-core/src/pack.rs)                                                            */
/* ------------------------------------------------------------------------------------------------------------------ */

uint8_t qto_pack_5trits(const int8_t t[5]) {
    /* pack.rs:28-36 */
    return (uint8_t)((t[0] + 1) + 3 * (t[1] + 1) + 9 * (t[2] + 1) + 28 * (t[3] + 1) + 84 * (t[4] + 1));
}

static int8_t g_byte_to_trits[256][5];
static int g_table_ready = 0;

/* Built when the library is loaded, so that threaded callers never race on it. */
__attribute__((constructor)) static void init_table(void) {
    /* pack.rs:43-58: enumerate the 243 states, everything else stays zero */
    if (g_table_ready) return;
    memset(g_byte_to_trits, 0, sizeof g_byte_to_trits);
    for (int s = 0; s < 243; ++s) {
        int8_t t[5] = {(int8_t)(s % 3 - 1), (int8_t)((s / 3) % 3 - 1), (int8_t)((s / 9) % 3 - 1), (int8_t)((s / 27) % 3 - 1),
                       (int8_t)((s / 81) % 3 - 1)};
        memcpy(g_byte_to_trits[qto_pack_5trits(t)], t, 5);
    }
    g_table_ready = 1;
}

void qto_byte_to_trits(uint8_t byte, int8_t out[5]) {
    init_table();
    memcpy(out, g_byte_to_trits[byte], 5);
}

size_t qto_planar_row_bytes(size_t cols) { return (cols + QTO_BLOCK_TRITS - 1) / QTO_BLOCK_TRITS * QTO_BLOCK_BYTES; }

void qto_pack_planar(const int8_t* trits, size_t rows, size_t cols, uint8_t* out) {
    /* pack.rs:84-131: byte j of block b holds the trits at block offsets j, 32+j, 64+j, 96+j, 128+j; a short last
     * block is filled with zero trits. */
    const size_t bpr = (cols + QTO_BLOCK_TRITS - 1) / QTO_BLOCK_TRITS;
    for (size_t r = 0; r < rows; ++r) {
        const int8_t* row = trits + r * cols;
        uint8_t* dst = out + r * bpr * QTO_BLOCK_BYTES;
        for (size_t b = 0; b < bpr; ++b) {
            for (size_t j = 0; j < QTO_BLOCK_BYTES; ++j) {
                int8_t t[5];
                for (size_t p = 0; p < 5; ++p) {
                    const size_t c = b * QTO_BLOCK_TRITS + p * QTO_BLOCK_BYTES + j;
                    t[p] = c < cols ? row[c] : 0;
                }
                dst[b * QTO_BLOCK_BYTES + j] = qto_pack_5trits(t);
            }
        }
    }
}

void qto_unpack_planar(const uint8_t* packed, size_t rows, size_t cols, int8_t* trits) {
    /* pack.rs:134-162 */
    init_table();
    const size_t bpr = (cols + QTO_BLOCK_TRITS - 1) / QTO_BLOCK_TRITS;
    for (size_t r = 0; r < rows; ++r) {
        for (size_t b = 0; b < bpr; ++b) {
            for (size_t j = 0; j < QTO_BLOCK_BYTES; ++j) {
                const int8_t* d = g_byte_to_trits[packed[(r * bpr + b) * QTO_BLOCK_BYTES + j]];
                for (size_t p = 0; p < 5; ++p) {
                    const size_t c = b * QTO_BLOCK_TRITS + p * QTO_BLOCK_BYTES + j;
                    if (c < cols) trits[r * cols + c] = d[p];
                }
            }
        }
    }
}

static size_t tile_full_columns(size_t cols) { return cols / QTO_BLOCK_TRITS * QTO_BLOCK_BYTES; } /* pack.rs:209-212 */

size_t qto_tile_row_bytes(size_t cols) {
    /* pack.rs:223-227: full blocks + the partial block packed five to a byte, rounded up to an even count */
    const size_t tail = (cols % QTO_BLOCK_TRITS + 4) / 5;
    return tile_full_columns(cols) + tail + (tail & 1);
}

size_t qto_column_activation_index(size_t cols, size_t c, size_t p) {
    /* pack.rs:231-239 */
    const size_t full = tile_full_columns(cols);
    if (c < full) return c / QTO_BLOCK_BYTES * QTO_BLOCK_TRITS + p * QTO_BLOCK_BYTES + c % QTO_BLOCK_BYTES;
    return cols / QTO_BLOCK_TRITS * QTO_BLOCK_TRITS + 5 * (c - full) + p;
}

static uint8_t tile_byte(const uint8_t* src_row, size_t cols, size_t c) {
    /* pack.rs:243-258 */
    const size_t full = tile_full_columns(cols);
    if (c < full) return src_row[c];
    const size_t rem = cols % QTO_BLOCK_TRITS;
    int8_t t[5] = {0, 0, 0, 0, 0};
    for (size_t k = 0; k < 5; ++k) {
        const size_t q = 5 * (c - full) + k;
        if (q < rem) t[k] = g_byte_to_trits[src_row[full + q % QTO_BLOCK_BYTES]][q / QTO_BLOCK_BYTES];
    }
    return qto_pack_5trits(t);
}

void qto_tile32(const uint8_t* planar, size_t rows, size_t cols, uint8_t* tiled) {
    /* pack.rs:266-279 + lut.rs:129-154: byte-column c of a tile holds byte c of its 32 rows */
    init_table();
    const size_t src_rb = qto_planar_row_bytes(cols), rb = qto_tile_row_bytes(cols);
    for (size_t b = 0; b < rows / 32; ++b)
        for (size_t r = 0; r < 32; ++r)
            for (size_t c = 0; c < rb; ++c) tiled[b * 32 * rb + c * 32 + r] = tile_byte(planar + (b * 32 + r) * src_rb, cols, c);
}

/* ------------------------------------------------------------------------------------------------------------------ */
/* GEMV integers                                                                                                      */
/* ------------------------------------------------------------------------------------------------------------------ */

void qto_gemv_bruteforce(const int8_t* trits, size_t rows, size_t cols, const int8_t* act, int64_t* out) {
    /* quintrit-cuda/src/pack.rs:92-96 */
    for (size_t r = 0; r < rows; ++r) {
        int64_t s = 0;
        for (size_t c = 0; c < cols; ++c) s += (int64_t)trits[r * cols + c] * (int64_t)act[c];
        out[r] = s;
    }
}

void qto_gemv_planar(const uint8_t* planar, size_t rows, size_t cols, const int8_t* act, int32_t* out) {
    init_table();
    const size_t bpr = (cols + QTO_BLOCK_TRITS - 1) / QTO_BLOCK_TRITS;
    for (size_t r = 0; r < rows; ++r) {
        int64_t s = 0;
        for (size_t b = 0; b < bpr; ++b)
            for (size_t j = 0; j < QTO_BLOCK_BYTES; ++j) {
                const int8_t* d = g_byte_to_trits[planar[(r * bpr + b) * QTO_BLOCK_BYTES + j]];
                for (size_t p = 0; p < 5; ++p) {
                    const size_t c = b * QTO_BLOCK_TRITS + p * QTO_BLOCK_BYTES + j;
                    if (c < cols) s += (int64_t)d[p] * act[c];
                }
            }
        out[r] = (int32_t)s;
    }
}

/* lut.rs:29-71 */
static const int8_t MAP_34[16][2] = {{-1, -1}, {0, -1}, {1, -1}, {-1, 0}, {0, 0}, {1, 0}, {-1, 1}, {0, 1},
                                     {1, 1},   {0, 0},  {0, 0},  {0, 0},  {0, 0}, {0, 0}, {0, 0},  {0, 0}};
static const int8_t MAP_01[16][2] = {{-1, -1}, {0, 0}, {0, -1}, {1, -1}, {1, -1}, {-1, 0}, {-1, 0}, {0, 0},
                                     {0, 0},   {1, 0}, {-1, 1}, {-1, 1}, {0, 1},  {0, 1},  {1, 1},  {0, 0}};

static int8_t clamp_i8(int v) { return (int8_t)(v < -128 ? -128 : (v > 127 ? 127 : v)); }

/* lut.rs:298-358 build_activation_lut_into (portable branch): 64 bytes per tile column + the a2 array */
static void build_lut(const int8_t* act, size_t cols, int8_t* qlut) {
    const size_t rb = qto_tile_row_bytes(cols);
    const size_t a2_off = rb * 64;
    const size_t total = a2_off + (rb + 31) / 32 * 32;
    for (size_t c = 0; c < rb; ++c) {
        int a[5];
        for (size_t p = 0; p < 5; ++p) {
            const size_t idx = qto_column_activation_index(cols, c, p);
            a[p] = idx < cols ? act[idx] : 0;
        }
        int8_t* base = qlut + c * 64;
        for (int s = 0; s < 16; ++s) {
            base[s] = base[16 + s] = clamp_i8(MAP_34[s][0] * a[3] + MAP_34[s][1] * a[4]);
            base[32 + s] = base[48 + s] = clamp_i8(MAP_01[s][0] * a[0] + MAP_01[s][1] * a[1]);
        }
        qlut[a2_off + c] = (int8_t)a[2];
    }
    memset(qlut + a2_off + rb, 0, total - a2_off - rb);
}

/* simd/scalar.rs:11-64 for one 32-row tile, int32 result */
static void block32_scalar(const uint8_t* w, const int8_t* qlut, size_t rb, int32_t* out32) {
    const int8_t* a2p = qlut + rb * 64;
    for (size_t r = 0; r < 32; ++r) {
        int32_t acc = 0;
        for (size_t c = 0; c < rb; ++c) {
            const uint8_t x = w[c * 32 + r];
            const uint8_t v11 = (uint8_t)((x >> 2) & 0x3F);
            const uint8_t v15 = (uint8_t)((v11 >> 3) & 0x1F);
            const uint8_t v17 = (uint8_t)(((unsigned)v11 + v15 + 1) >> 1);
            const unsigned h34 = (v17 >> 2) & 0x0F;
            const int p34 = qlut[c * 64 + h34];
            const uint8_t w2 = (uint8_t)(x + x);
            const uint8_t diff2 = (uint8_t)((uint8_t)(w2 - v11) - (uint8_t)h34);
            const unsigned h01 = diff2 & 0x0F;
            const int p01 = qlut[c * 64 + 32 + h01];
            const uint8_t xm1 = (uint8_t)(x - 1);
            const uint8_t u = (uint8_t)((((unsigned)xm1 + v17 + 1) >> 1) & 0x0F);
            const int t2 = u < 5 ? -1 : (u > 9 ? 1 : 0);
            const int a2 = a2p[c];
            acc += p34 + p01 + t2 * a2;
        }
        out32[r] = acc;
    }
}

void qto_gemv_lut_wide(const uint8_t* tiled, size_t rows, size_t cols, const int8_t* act, int32_t* out) {
    const size_t rb = qto_tile_row_bytes(cols);
    const size_t single = rb * 64 + (rb + 31) / 32 * 32;
    int8_t* hi = (int8_t*)malloc(cols ? cols : 1);
    int8_t* lo = (int8_t*)malloc(cols ? cols : 1);
    int8_t* qlo = (int8_t*)malloc(single ? single : 1);
    int8_t* qhi = (int8_t*)malloc(single ? single : 1);
    /* lut.rs:380-388 split_activations_hi_lo */
    for (size_t i = 0; i < cols; ++i) {
        const int x = act[i];
        const int l = ((x + 8) & 15) - 8;
        lo[i] = (int8_t)l;
        hi[i] = (int8_t)((x - l) >> 4);
    }
    build_lut(lo, cols, qlo);
    build_lut(hi, cols, qhi);
    for (size_t b = 0; b < rows / 32; ++b) {
        int32_t olo[32], ohi[32];
        block32_scalar(tiled + b * 32 * rb, qlo, rb, olo);
        block32_scalar(tiled + b * 32 * rb, qhi, rb, ohi);
        for (int r = 0; r < 32; ++r) out[b * 32 + r] = olo[r] + 16 * ohi[r]; /* lut.rs:552-556 */
    }
    free(hi);
    free(lo);
    free(qlo);
    free(qhi);
}

void qto_rescale(const int32_t* acc, size_t rows, float weight_scale, float act_scale, float* out) {
    /* layer.rs:143-150: the kernels return the integer as f32, then one multiply by weight_scale / act_scale */
    if (act_scale > 0.0f) {
        const float post = weight_scale / act_scale;
        for (size_t i = 0; i < rows; ++i) out[i] = (float)acc[i] * post;
    } else {
        for (size_t i = 0; i < rows; ++i) out[i] = 0.0f;
    }
}

/* ------------------------------------------------------------------------------------------------------------------ */
/* int8 absmax quantiser (quintrit-runtime/src/ops.rs:241-267, levels = 127)                                          */
/* ------------------------------------------------------------------------------------------------------------------ */

float qto_quantize_int8(const float* x, size_t n, int8_t* out) {
    float max_abs = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        const float a = fabsf(x[i]);
        if (a > max_abs) max_abs = a;
    }
    if (!(max_abs > 0.0f)) {
        memset(out, 0, n);
        return 0.0f;
    }
    const float s = 127.0f / max_abs;
    for (size_t i = 0; i < n; ++i) {
        float q = roundf(x[i] * s); /* f32::round: half away from zero */
        if (q != q) {
            out[i] = 0; /* `NaN as i8` is 0 in Rust */
            continue;
        }
        if (q < -128.0f) q = -128.0f;
        if (q > 127.0f) q = 127.0f;
        out[i] = (int8_t)q;
    }
    return s;
}

/* ------------------------------------------------------------------------------------------------------------------ */
/* GGUF ternary decoders                                                                                              */
/* ------------------------------------------------------------------------------------------------------------------ */

static int8_t trit_of(unsigned code) { return code == 3 ? 0 : (int8_t)((int)code - 1); } /* unpack.rs:49-52 */

/* unpack.rs:55-66 decode_portable: groups of 32 bytes -> 4 planes of 32 trits */
static void decode_2bit_planes(const uint8_t* src, size_t src_len, int8_t* out, int high_first) {
    for (size_t g = 0; g < src_len / 32; ++g)
        for (size_t p = 0; p < 4; ++p) {
            const unsigned shift = (unsigned)(high_first ? 6 - 2 * p : 2 * p);
            for (size_t m = 0; m < 32; ++m) out[g * 128 + p * 32 + m] = trit_of((src[g * 32 + m] >> shift) & 3u);
        }
}

int qto_decode_i2_s(const uint8_t* data, size_t data_len, size_t rows, size_t cols, int8_t* trits) {
    /* i2_s.rs:50-66: cols a multiple of 128, rows * cols / 4 bytes, plane 0 in the high bits */
    if (cols % 128 != 0 || data_len != rows * cols / 4) return -1;
    for (size_t r = 0; r < rows; ++r) decode_2bit_planes(data + r * cols / 4, cols / 4, trits + r * cols, 1);
    return 0;
}

int qto_encode_i2_s(const int8_t* trits, size_t rows, size_t cols, uint8_t* out) {
    /* i2_s.rs:20-40 */
    if (cols % 128 != 0) return -1;
    memset(out, 0, rows * cols / 4);
    for (size_t r = 0; r < rows; ++r)
        for (size_t b = 0; b < cols / 128; ++b)
            for (size_t j = 0; j < 128; ++j) {
                const int8_t w = trits[r * cols + b * 128 + j];
                const unsigned code = w == -1 ? 0u : (w == 1 ? 2u : 1u);
                out[r * cols / 4 + b * 32 + j % 32] |= (uint8_t)(code << (6 - 2 * (j / 32)));
            }
    return 0;
}

int qto_decode_tq2_0(const uint8_t* data, size_t data_len, size_t rows, size_t cols, int8_t* trits) {
    /* tq2_0.rs:48-88: blocks of 256 weights = 64 code bytes (two groups of 32, plane 0 in the low bits) + f16 scale */
    const size_t n = rows * cols;
    if (n % 256 != 0 || data_len < n / 256 * 66) return -1;
    for (size_t b = 0; b < n / 256; ++b) decode_2bit_planes(data + b * 66, 64, trits + b * 256, 0);
    return 0;
}

static int8_t tq1_digit(uint8_t byte, unsigned n) {
    /* tq1_0.rs:77-81 */
    static const unsigned POW3[5] = {1, 3, 9, 27, 81};
    const unsigned q = (byte * POW3[n]) & 0xFFu;
    return (int8_t)((int)((q * 3) >> 8) - 1);
}

int qto_decode_tq1_0(const uint8_t* data, size_t data_len, size_t rows, size_t cols, int8_t* trits) {
    /* tq1_0.rs:51-122: block = 48 qs + 4 qh + f16 scale; 32 bytes -> 5 planes of 32, 16 bytes -> 5 planes of 16,
     * 4 bytes -> 4 planes of 4 */
    const size_t n = rows * cols;
    if (n % 256 != 0 || data_len < n / 256 * 54) return -1;
    for (size_t b = 0; b < n / 256; ++b) {
        const uint8_t* qs = data + b * 54;
        const uint8_t* qh = qs + 48;
        int8_t* o = trits + b * 256;
        for (unsigned p = 0; p < 5; ++p)
            for (size_t m = 0; m < 32; ++m) o[p * 32 + m] = tq1_digit(qs[m], p);
        for (unsigned p = 0; p < 5; ++p)
            for (size_t m = 0; m < 16; ++m) o[160 + p * 16 + m] = tq1_digit(qs[32 + m], p);
        for (unsigned p = 0; p < 4; ++p)
            for (size_t j = 0; j < 4; ++j) o[240 + p * 4 + j] = tq1_digit(qh[j], p);
    }
    return 0;
}

float qto_half_to_f32(uint16_t h) {
    /* decoders/mod.rs:91-118 */
    const uint32_t sign = (h >> 15) & 1u, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign << 31;
        } else {
            uint32_t e = 127 - 15 + 1, m = man;
            while ((m & 0x400u) == 0) {
                m <<= 1;
                e -= 1;
            }
            bits = (sign << 31) | (e << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (exp == 0x1F) {
        bits = (sign << 31) | (0xFFu << 23) | (man << 13);
    } else {
        bits = (sign << 31) | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

long qto_decode_q2_0(const uint8_t* data, size_t data_len, size_t rows, size_t cols, int8_t* trits, float* scales) {
    /* q2_0.rs:19-56, 66-101 with 64-weight blocks of 18 bytes */
    if (cols == 0 || cols % 64 != 0) return -1;
    const size_t n = rows * cols;
    if (data_len != n / 64 * 18) return -1;
    for (size_t b = 0; b < n / 64; ++b) {
        const uint8_t* blk = data + b * 18;
        scales[b] = qto_half_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        for (size_t j = 0; j < 16; ++j)
            for (unsigned k = 0; k < 4; ++k) {
                const unsigned code = (blk[2 + j] >> (2 * k)) & 3u;
                if (code == 3) return -(long)(b * 64 + 4 * j + k + 1);
                trits[b * 64 + 4 * j + k] = (int8_t)((int)code - 1);
            }
    }
    return 0;
}

int qto_uniform_block_scale(int ggml_type, const uint8_t* data, size_t data_len, float* scale) {
    /* decoders/mod.rs:121-138; type ids gguf.rs (TQ1_0 = 34, TQ2_0 = 35) */
    size_t block_bytes, off;
    if (ggml_type == 34) {
        block_bytes = 54;
        off = 52;
    } else if (ggml_type == 35) {
        block_bytes = 66;
        off = 64;
    } else {
        return 0;
    }
    if (data_len == 0 || data_len % block_bytes != 0) return 0;
    const uint16_t first = (uint16_t)(data[off] | (data[off + 1] << 8));
    for (size_t b = 1; b < data_len / block_bytes; ++b) {
        const uint8_t* p = data + b * block_bytes + off;
        if ((uint16_t)(p[0] | (p[1] << 8)) != first) return 0;
    }
    *scale = qto_half_to_f32(first);
    return 1;
}

/* ---- seeded synthetic weights (benchmark and fixture input, not part of the reference) ----------------------------
 * The counter-based SplitMix64 stream of quintrit_b200/synth.py (the numpy code there is the definition;
 * tests/test_synth.py holds this copy to it): value i = mix(seed + (i + 1) * GAMMA), u = its high 32 bits,
 * u < 0.3 * 2^32 -> -1, u < 0.6 * 2^32 -> +1, else 0. Writes rows [row0, row0 + rows) of the rows x cols matrix as planar
 * velurex bytes; threaded over rows so that the 9.5 G weights of a Falcon3-10B-shape model take seconds on the host. */
static inline uint32_t synth_u32(uint64_t seed, uint64_t i) {
    uint64_t z = seed + (i + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (uint32_t)(z >> 32);
}

void qto_synth_planar(uint64_t seed, size_t rows, size_t cols, size_t row0, uint8_t* out) {
    const size_t bpr = (cols + QTO_BLOCK_TRITS - 1) / QTO_BLOCK_TRITS;
#pragma omp parallel for schedule(static)
    for (long rr = 0; rr < (long)rows; ++rr) {
        const size_t r = (size_t)rr;
        uint8_t* dst = out + r * bpr * QTO_BLOCK_BYTES;
        const uint64_t base = (uint64_t)(row0 + r) * cols;
        for (size_t b = 0; b < bpr; ++b)
            for (size_t j = 0; j < QTO_BLOCK_BYTES; ++j) {
                int8_t t[5];
                for (size_t p = 0; p < 5; ++p) {
                    const size_t c = b * QTO_BLOCK_TRITS + p * QTO_BLOCK_BYTES + j;
                    int8_t v = 0;
                    if (c < cols) {
                        const uint32_t u = synth_u32(seed, base + c);
                        v = u < 1288490188u ? -1 : (u < 2576980377u ? 1 : 0);
                    }
                    t[p] = v;
                }
                dst[b * QTO_BLOCK_BYTES + j] = qto_pack_5trits(t);
            }
    }
}

uint16_t qto_f32_to_f16(float f);
uint16_t qto_f32_to_bf16(float f);

/* Dense-table values of quintrit_b200/synth.py (table_bits_np is the definition): (u0 + u1 + u2 + u3 - 2^33) * gain with
 * four consecutive uniforms, one double multiply, rounded to float and then to F16 or BF16 bit patterns. */
void qto_synth_table(uint64_t seed, size_t n, size_t start, int bf16, uint16_t* out) {
    const double gain = 0.02 * 1.7320508075688772 / 4294967296.0;
#pragma omp parallel for schedule(static)
    for (long ii = 0; ii < (long)n; ++ii) {
        const uint64_t i = (uint64_t)ii + start;
        const int64_t s = (int64_t)synth_u32(seed, 4 * i) + synth_u32(seed, 4 * i + 1) + synth_u32(seed, 4 * i + 2) + synth_u32(seed, 4 * i + 3);
        const float x = (float)((double)(s - ((int64_t)1 << 33)) * gain);
        out[ii] = bf16 ? qto_f32_to_bf16(x) : qto_f32_to_f16(x);
    }
}

/* Q2_0 block scales of quintrit_b200/synth.py (block_scales_np): 0.5 + 1.5 u / 2^32, to float, to F16 and back. */
float qto_f16_to_f32(uint16_t h);
void qto_synth_block_scales(uint64_t seed, size_t n, size_t start, float* out) {
#pragma omp parallel for schedule(static)
    for (long ii = 0; ii < (long)n; ++ii) {
        const double v = 0.5 + 1.5 * (double)synth_u32(seed, (uint64_t)ii + start) / 4294967296.0;
        out[ii] = qto_f16_to_f32(qto_f32_to_f16((float)v));
    }
}
