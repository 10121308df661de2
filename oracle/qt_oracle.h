/*
 * qt_oracle.h - CPU restatement of the reference's ternary decode arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the shipped library links, loads or calls this code; it exists so that the
 * tests, the smoke check and the CPU-baseline leg of the benchmark can compare the CUDA path with the reference's
 * algorithm on the same inputs. Each function names the reference file (path inside the quintrit project) and the
 * lines it follows. The reference is Rust and cannot be built where this runs, so the restatement is pinned by the
 * known answers the reference's own tests hold (see tests/test_oracle_*.py).
 *
 * Plain C99, no dependencies beyond libc/libm.
 */
#ifndef QT_ORACLE_H
#define QT_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- velurex byte and planar layout: rust/crates/quintrit-core/src/pack.rs ---- */

#define QTO_BLOCK_TRITS 160 /* pack.rs:19 QK_5 */
#define QTO_BLOCK_BYTES 32  /* pack.rs:22 BLOCK_BYTES_5 */

/* pack.rs:28-36 pack_5trits: d = t + 1, byte = d0 + 3 d1 + 9 d2 + 28 d3 + 84 d4 (0..250). */
uint8_t qto_pack_5trits(const int8_t t[5]);
/* pack.rs:41-58 BYTE_TO_TRITS: byte -> five trits; bytes that the packer never produces decode to zeros. */
void qto_byte_to_trits(uint8_t byte, int8_t out[5]);
/* pack.rs:103-131 row size of the planar layout: ceil(cols / 160) * 32. */
size_t qto_planar_row_bytes(size_t cols);
/* pack.rs:84-131 pack_matrix / pack_row / pack_block: rows x cols trits -> planar bytes (tail padded with zero trits). */
void qto_pack_planar(const int8_t* trits, size_t rows, size_t cols, uint8_t* out);
/* pack.rs:134-162 unpack_matrix. */
void qto_unpack_planar(const uint8_t* packed, size_t rows, size_t cols, int8_t* trits);
/* pack.rs:209-227 tile_full_columns / tile_row_bytes. */
size_t qto_tile_row_bytes(size_t cols);
/* pack.rs:229-239 column_activation_index. */
size_t qto_column_activation_index(size_t cols, size_t c, size_t p);
/* pack.rs:241-279 tile_byte + tile_rows_into for R = 32: planar rows -> 32-row tiles (rows must be a multiple of 32). */
void qto_tile32(const uint8_t* planar, size_t rows, size_t cols, uint8_t* tiled);

/* ---- GEMV integers ---- */

/* rust/crates/quintrit-cuda/src/pack.rs:92-96 reference_gemv: brute-force sum of trit * act in 64 bits. */
void qto_gemv_bruteforce(const int8_t* trits, size_t rows, size_t cols, const int8_t* act, int64_t* out);
/* Same sum taken from planar bytes through qto_byte_to_trits (decode-then-multiply; no tables). */
void qto_gemv_planar(const uint8_t* planar, size_t rows, size_t cols, const int8_t* act, int32_t* out);
/*
 * The reference CPU kernel's own algebra: split x = 16 hi + lo (quintrit-core/src/lut.rs:380-388), build the dual-hash
 * tables per half (lut.rs:298-358 with MAP_34 / MAP_01, lut.rs:29-71), run the portable 32-row block kernel on each
 * half (quintrit-core/src/simd/scalar.rs:11-64) and recombine lo + 16 hi (lut.rs:545-560). `tiled` is the 32-row tile
 * layout of qto_tile32; rows must be a multiple of 32.
 */
void qto_gemv_lut_wide(const uint8_t* tiled, size_t rows, size_t cols, const int8_t* act, int32_t* out);
/* quintrit-runtime/src/layer.rs:143-150: out = acc * (weight_scale / act_scale), zeros if act_scale <= 0. */
void qto_rescale(const int32_t* acc, size_t rows, float weight_scale, float act_scale, float* out);

/* ---- activation quantiser: rust/crates/quintrit-runtime/src/ops.rs:241-267 ---- */
float qto_quantize_int8(const float* x, size_t n, int8_t* out);

/* ---- GGUF ternary decoders -> trits ---- */

/* quintrit-format/src/decoders/i2_s.rs:43-67 + quintrit-core/src/unpack.rs:55-74 (plane 0 in bits 6-7, code 3 -> 0). */
int qto_decode_i2_s(const uint8_t* data, size_t data_len, size_t rows, size_t cols, int8_t* trits);
/* i2_s.rs:20-40 pack_gguf_i2_s (used to make fixtures). */
int qto_encode_i2_s(const int8_t* trits, size_t rows, size_t cols, uint8_t* out);
/* decoders/tq2_0.rs:48-88 (66-byte blocks of 256: 64 code bytes, plane 0 in bits 0-1, then the f16 scale). */
int qto_decode_tq2_0(const uint8_t* data, size_t data_len, size_t rows, size_t cols, int8_t* trits);
/* decoders/tq1_0.rs:51-122 (54-byte blocks of 256: 48 + 4 digit bytes, then the f16 scale). */
int qto_decode_tq1_0(const uint8_t* data, size_t data_len, size_t rows, size_t cols, int8_t* trits);
/*
 * decoders/q2_0.rs:34-101 with block_size 64: f16 scale + 16 code bytes, lowest bits first; a code 3 is an error
 * (returns -(index + 1) of the first offending weight). scales receives rows * cols / 64 floats.
 */
long qto_decode_q2_0(const uint8_t* data, size_t data_len, size_t rows, size_t cols, int8_t* trits, float* scales);
/* decoders/mod.rs:121-138 uniform_block_scale: 1 and *scale set if every block of a TQ tensor has the same f16 scale. */
int qto_uniform_block_scale(int ggml_type, const uint8_t* data, size_t data_len, float* scale);
/* decoders/mod.rs:85-118 half_to_f32. */
float qto_half_to_f32(uint16_t h);

/* Seeded synthetic ternary matrix (the stream of quintrit_b200/synth.py) as planar bytes, rows [row0, row0 + rows). */
void qto_synth_planar(uint64_t seed, size_t rows, size_t cols, size_t row0, uint8_t* out);

/* ---- timed CPU baseline (oracle/cpu_gemv.c) ---- */

/*
 * Multi-threaded exact GEMV over 64-row tiles with byte-permute table lookups (AVX-512 VBMI), the shape of the
 * reference's production x86 kernel (quintrit-core/src/simd/avx512.rs:982-1169, 1256-1292). Returns 0 on success, -1
 * if the CPU lacks AVX-512 VBMI (callers then use qto_cpu_gemv_portable).
 */
int qto_cpu_has_avx512_vbmi(void);
size_t qto_tile64_bytes(size_t rows, size_t cols);
void qto_tile64(const uint8_t* planar, size_t rows, size_t cols, uint8_t* tiled);
int qto_cpu_gemv_avx512(const uint8_t* tiled64, size_t rows, size_t cols, const int8_t* act, int32_t* out, int threads);
void qto_cpu_gemv_portable(const uint8_t* planar, size_t rows, size_t cols, const int8_t* act, int32_t* out, int threads);

#ifdef __cplusplus
}
#endif
#endif
