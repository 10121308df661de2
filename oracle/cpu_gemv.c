/*
 * cpu_gemv.c - the CPU GEMV that is timed beside the GPU numbers. TEST / BENCHMARK INFRASTRUCTURE ONLY: the shipped
 * library never calls into this file.
 *
 * It restates the reference's production x86 kernel for hosts with AVX-512 VBMI
 * (rust/crates/quintrit-core/src/simd/avx512.rs):
 *   - 64-row tiles: byte-column c of a tile = the 64 bytes of its rows (avx512.rs:53-80, tail repacked as in
 *     quintrit-core/src/pack.rs:241-279);
 *   - per byte-column one compact 64-byte table per activation half (x = 16 hi + lo): the nine (t3,t4) sums at
 *     indices 0..8 and the 27 (t0,t1,t2) sums at 9..35 (avx512.rs:930-953, 1204-1247);
 *   - decode of 64 weight bytes: w >> 2 indexes two 64-entry byte tables holding floor(i/7) and 28 floor(i/7) - 9
 *     (avx512.rs:1256-1292);
 *   - two byte-permute lookups per half, up to three columns summed in int8, lo + 16 hi formed with a multiply-add
 *     by the byte pair (1,16) into int16, 45 columns per int16 chunk, then widened to int32 (avx512.rs:1526-1605);
 *   - three 64-row blocks share every table load (avx512.rs:1107-1119), threads split the rows in whole tiles
 *     (avx512.rs:1141-1169).
 * The integers it returns equal the brute-force product; tests/test_oracle_gemv.py checks that.
 */
#include "qt_oracle.h"

#include <stdlib.h>
#include <string.h>

#if defined(__x86_64__)
#include <immintrin.h>
#endif
#ifdef _OPENMP
#include <omp.h>
#endif

int qto_cpu_has_avx512_vbmi(void) {
#if defined(__x86_64__)
    return __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") && __builtin_cpu_supports("avx512vbmi");
#else
    return 0;
#endif
}

size_t qto_tile64_bytes(size_t rows, size_t cols) { return (rows + 63) / 64 * 64 * qto_tile_row_bytes(cols); }

void qto_tile64(const uint8_t* planar, size_t rows, size_t cols, uint8_t* tiled) {
    /* rows are padded to a multiple of 64 with zero trits (byte 125 = five digits 1) */
    const size_t rb = qto_tile_row_bytes(cols), prb = qto_planar_row_bytes(cols);
    const size_t full = cols / QTO_BLOCK_TRITS * QTO_BLOCK_BYTES, rem = cols % QTO_BLOCK_TRITS;
    const size_t nb = (rows + 63) / 64;
#pragma omp parallel for schedule(static)
    for (long b = 0; b < (long)nb; ++b) {
        for (size_t r = 0; r < 64; ++r) {
            const size_t row = (size_t)b * 64 + r;
            for (size_t c = 0; c < rb; ++c) {
                uint8_t v = 125;
                if (row < rows) {
                    const uint8_t* src = planar + row * prb;
                    if (c < full) {
                        v = src[c];
                    } else {
                        int8_t t[5] = {0, 0, 0, 0, 0}, d[5];
                        for (size_t k = 0; k < 5; ++k) {
                            const size_t q = 5 * (c - full) + k;
                            if (q < rem) {
                                qto_byte_to_trits(src[full + q % QTO_BLOCK_BYTES], d);
                                t[k] = d[q / QTO_BLOCK_BYTES];
                            }
                        }
                        v = qto_pack_5trits(t);
                    }
                }
                tiled[(size_t)b * 64 * rb + c * 64 + r] = v;
            }
        }
    }
}

/* compact [lo | hi] tables: entry U (0..8) = t3 a3 + t4 a4, entry 9 + L (0..26) = t0 a0 + t1 a1 + t2 a2 */
static void build_compact_wide(const int8_t* act, size_t cols, int8_t* lo_tab, int8_t* hi_tab) {
    const size_t rb = qto_tile_row_bytes(cols);
    memset(lo_tab, 0, rb * 64);
    memset(hi_tab, 0, rb * 64);
    for (size_t c = 0; c < rb; ++c) {
        int lo[5], hi[5];
        for (size_t p = 0; p < 5; ++p) {
            const size_t idx = qto_column_activation_index(cols, c, p);
            const int x = idx < cols ? act[idx] : 0;
            const int l = ((x + 8) & 15) - 8;
            lo[p] = l;
            hi[p] = (x - l) >> 4;
        }
        for (int u = 0; u < 9; ++u) {
            const int t3 = u % 3 - 1, t4 = u / 3 - 1;
            lo_tab[c * 64 + u] = (int8_t)(t3 * lo[3] + t4 * lo[4]);
            hi_tab[c * 64 + u] = (int8_t)(t3 * hi[3] + t4 * hi[4]);
        }
        for (int l = 0; l < 27; ++l) {
            const int t0 = l % 3 - 1, t1 = (l / 3) % 3 - 1, t2 = l / 9 - 1;
            lo_tab[c * 64 + 9 + l] = (int8_t)(t0 * lo[0] + t1 * lo[1] + t2 * lo[2]);
            hi_tab[c * 64 + 9 + l] = (int8_t)(t0 * hi[0] + t1 * hi[1] + t2 * hi[2]);
        }
    }
}

#if defined(__x86_64__)
#define NBMAX 3

__attribute__((target("avx512f,avx512bw,avx512vbmi"))) static void blocks_avx512(const uint8_t* w, size_t nb, size_t stride,
                                                                                  const int8_t* lo, const int8_t* hi, size_t rb,
                                                                                  int32_t* out) {
    uint8_t h34_tab[64], m28_tab[64];
    for (int i = 0; i < 64; ++i) {
        h34_tab[i] = (uint8_t)(i / 7);
        m28_tab[i] = (uint8_t)(28 * (i / 7) - 9);
    }
    const __m512i th = _mm512_loadu_si512(h34_tab), tm = _mm512_loadu_si512(m28_tab);
    const __m512i one_sixteen = _mm512_set1_epi16(0x1001);
    __m512i a0[NBMAX], a1[NBMAX], b0[NBMAX], b1[NBMAX];
    for (size_t k = 0; k < nb; ++k) a0[k] = a1[k] = b0[k] = b1[k] = _mm512_setzero_si512();

    for (size_t c0 = 0; c0 < rb; c0 += 45) {
        const size_t clen = rb - c0 < 45 ? rb - c0 : 45;
        __m512i sa[NBMAX], sb[NBMAX];
        for (size_t k = 0; k < nb; ++k) sa[k] = sb[k] = _mm512_setzero_si512();
        for (size_t ci = 0; ci < clen; ci += 3) {
            const size_t n = clen - ci < 3 ? clen - ci : 3;
            __m512i slo[NBMAX], shi[NBMAX];
            for (size_t j = 0; j < n; ++j) {
                const size_t col = c0 + ci + j;
                const __m512i tl = _mm512_loadu_si512(lo + col * 64), thi = _mm512_loadu_si512(hi + col * 64);
                for (size_t k = 0; k < nb; ++k) {
                    const uint8_t* p = w + k * stride + col * 64;
                    _mm_prefetch((const char*)(p + 4096), _MM_HINT_T0);
                    const __m512i wv = _mm512_loadu_si512(p);
                    const __m512i idx = _mm512_srli_epi16(wv, 2);
                    const __m512i u = _mm512_permutexvar_epi8(idx, th);
                    const __m512i l9 = _mm512_sub_epi8(wv, _mm512_permutexvar_epi8(idx, tm));
                    const __m512i l = _mm512_add_epi8(_mm512_permutexvar_epi8(u, tl), _mm512_permutexvar_epi8(l9, tl));
                    const __m512i h = _mm512_add_epi8(_mm512_permutexvar_epi8(u, thi), _mm512_permutexvar_epi8(l9, thi));
                    slo[k] = j == 0 ? l : _mm512_add_epi8(slo[k], l);
                    shi[k] = j == 0 ? h : _mm512_add_epi8(shi[k], h);
                }
            }
            for (size_t k = 0; k < nb; ++k) {
                sa[k] = _mm512_add_epi16(sa[k], _mm512_maddubs_epi16(one_sixteen, _mm512_unpacklo_epi8(slo[k], shi[k])));
                sb[k] = _mm512_add_epi16(sb[k], _mm512_maddubs_epi16(one_sixteen, _mm512_unpackhi_epi8(slo[k], shi[k])));
            }
        }
        for (size_t k = 0; k < nb; ++k) {
            a0[k] = _mm512_add_epi32(a0[k], _mm512_cvtepi16_epi32(_mm512_castsi512_si256(sa[k])));
            a1[k] = _mm512_add_epi32(a1[k], _mm512_cvtepi16_epi32(_mm512_extracti64x4_epi64(sa[k], 1)));
            b0[k] = _mm512_add_epi32(b0[k], _mm512_cvtepi16_epi32(_mm512_castsi512_si256(sb[k])));
            b1[k] = _mm512_add_epi32(b1[k], _mm512_cvtepi16_epi32(_mm512_extracti64x4_epi64(sb[k], 1)));
        }
    }
    /* unpacklo/hi work per 128-bit lane: a0 = rows 0..7 | 16..23, b0 = 8..15 | 24..31, a1 = 32..39 | 48..55, b1 = 40..47 | 56..63 */
    for (size_t k = 0; k < nb; ++k) {
        int32_t t[16];
        int32_t* o = out + k * 64;
        _mm512_storeu_si512(t, a0[k]);
        memcpy(o, t, 32), memcpy(o + 16, t + 8, 32);
        _mm512_storeu_si512(t, b0[k]);
        memcpy(o + 8, t, 32), memcpy(o + 24, t + 8, 32);
        _mm512_storeu_si512(t, a1[k]);
        memcpy(o + 32, t, 32), memcpy(o + 48, t + 8, 32);
        _mm512_storeu_si512(t, b1[k]);
        memcpy(o + 40, t, 32), memcpy(o + 56, t + 8, 32);
    }
}
#endif

int qto_cpu_gemv_avx512(const uint8_t* tiled64, size_t rows, size_t cols, const int8_t* act, int32_t* out, int threads) {
#if defined(__x86_64__)
    if (!qto_cpu_has_avx512_vbmi()) return -1;
    const size_t rb = qto_tile_row_bytes(cols), nblocks = (rows + 63) / 64, stride = 64 * rb;
    int8_t* tabs = (int8_t*)aligned_alloc(64, 2 * rb * 64 + 64);
    build_compact_wide(act, cols, tabs, tabs + rb * 64);
    const size_t groups = (nblocks + NBMAX - 1) / NBMAX;
    if (threads < 1) threads = 1;
#pragma omp parallel for schedule(static) num_threads(threads)
    for (long g = 0; g < (long)groups; ++g) {
        const size_t b = (size_t)g * NBMAX;
        const size_t nb = nblocks - b < NBMAX ? nblocks - b : NBMAX;
        int32_t tmp[NBMAX * 64];
        blocks_avx512(tiled64 + b * stride, nb, stride, tabs, tabs + rb * 64, rb, tmp);
        for (size_t i = 0; i < nb * 64; ++i)
            if (b * 64 + i < rows) out[b * 64 + i] = tmp[i];
    }
    free(tabs);
    return 0;
#else
    (void)tiled64, (void)rows, (void)cols, (void)act, (void)out, (void)threads;
    return -1;
#endif
}

void qto_cpu_gemv_portable(const uint8_t* planar, size_t rows, size_t cols, const int8_t* act, int32_t* out, int threads) {
    if (threads < 1) threads = 1;
    const size_t chunk = 64;
#pragma omp parallel for schedule(static) num_threads(threads)
    for (long r0 = 0; r0 < (long)rows; r0 += (long)chunk) {
        const size_t n = rows - (size_t)r0 < chunk ? rows - (size_t)r0 : chunk;
        qto_gemv_planar(planar + (size_t)r0 * qto_planar_row_bytes(cols), n, cols, act, out + r0);
    }
}

/* Read-only streaming rate of the host in GB/s: every thread sums its share of `bytes` bytes with 64-bit loads, best of
 * `reps` passes (the reference measures its memory ceiling the same way: a 1 GiB buffer read 21 times,
 * docs/benchmarks.md:144-146). The sum is returned through *sink so that the loads cannot be dropped. */
double qto_stream_read_gbs(const uint8_t* buf, size_t bytes, int threads, int reps, uint64_t* sink) {
    double best = 0.0;
    uint64_t total = 0;
    const size_t words = bytes / 8;
    for (int r = 0; r < reps; ++r) {
        uint64_t sum = 0;
#ifdef _OPENMP
        const double t0 = omp_get_wtime();
#pragma omp parallel for schedule(static) reduction(+ : sum) num_threads(threads)
#endif
        for (long c = 0; c < (long)(words / 512); ++c) {
            const uint64_t* p = (const uint64_t*)buf + (size_t)c * 512;
            uint64_t s0 = 0, s1 = 0, s2 = 0, s3 = 0;
            for (int i = 0; i < 512; i += 4) s0 += p[i], s1 += p[i + 1], s2 += p[i + 2], s3 += p[i + 3];
            sum += (s0 + s1) + (s2 + s3);
        }
#ifdef _OPENMP
        const double dt = omp_get_wtime() - t0;
        if (dt > 0.0 && (double)bytes / dt / 1e9 > best) best = (double)bytes / dt / 1e9;
#else
        (void)threads;
#endif
        total += sum;
    }
    if (sink) *sink = total;
    return best;
}
