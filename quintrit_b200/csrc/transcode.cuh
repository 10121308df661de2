// One-time on-device transcoder: GGUF ternary payloads (I2_S, TQ1_0, TQ2_0) or planar velurex bytes -> the stream
// layout of gemv_lut.cuh, and back to planar bytes.
//
// Reference behaviour reproduced (all on the host there): the decoders of
// rust/crates/quintrit-format/src/decoders/{i2_s.rs:43-67, tq1_0.rs:51-122, tq2_0.rs:48-88} followed by
// quintrit-format/src/transcoder.rs:165-200 (decode, then quintrit-core/src/pack.rs:103-131). The planar bytes this
// produces (read back with stream_to_planar_kernel) are byte-identical to pack_matrix's.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "gemv_lut.cuh"

namespace qtb {

enum Source : int { kSrcPlanar = 0, kSrcTq1 = 34, kSrcTq2 = 35, kSrcI2S = 36 };

// Trit of element (r, c) of a rows x cols tensor stored in `src` with encoding SRC.
template <int SRC>
__device__ __forceinline__ int source_trit(const uint8_t* __restrict__ src, size_t r, size_t c, size_t cols) {
    if (SRC == kSrcI2S) {
        // 128 trits per 32 bytes, element j of a block in byte j % 32 at bits 6 - 2 (j / 32); code 3 reads as 0
        const size_t j = c % 128;
        const unsigned code = (src[r * (cols / 4) + (c / 128) * 32 + j % 32] >> (6 - 2 * (j / 32))) & 3u;
        return code == 3 ? 0 : static_cast<int>(code) - 1;
    } else if (SRC == kSrcTq2) {
        // 66-byte blocks of 256 consecutive elements: two groups of 32 bytes, plane l of a group in bits 2l..2l+1
        const size_t e = r * cols + c, i = e % 256;
        const unsigned code = (src[(e / 256) * 66 + (i / 128) * 32 + i % 32] >> (2 * ((i % 128) / 32))) & 3u;
        return code == 3 ? 0 : static_cast<int>(code) - 1;
    } else {
        // TQ1_0: 54-byte blocks of 256: 32 bytes x 5 digits, 16 bytes x 5 digits, 4 bytes x 4 digits;
        // digit n of a byte = ((byte * 3^n mod 256) * 3) >> 8
        const size_t e = r * cols + c, i = e % 256;
        const uint8_t* blk = src + (e / 256) * 54;
        unsigned byte, n;
        if (i < 160) {
            n = static_cast<unsigned>(i / 32);
            byte = blk[i % 32];
        } else if (i < 240) {
            n = static_cast<unsigned>((i - 160) / 16);
            byte = blk[32 + (i - 160) % 16];
        } else {
            n = static_cast<unsigned>((i - 240) / 4);
            byte = blk[48 + (i - 240) % 4];
        }
        const unsigned pow3 = n == 0 ? 1u : n == 1 ? 3u : n == 2 ? 9u : n == 3 ? 27u : 81u;
        return static_cast<int>((((byte * pow3) & 0xFFu) * 3u) >> 8) - 1;
    }
}

// One thread per 16 output bytes: (block g, tile t, half h, lane l).
template <int SRC>
__global__ void to_stream_kernel(const uint8_t* __restrict__ src, uint4* __restrict__ dst, size_t rows, size_t cols, size_t blocks,
                                 size_t tiles) {
    const size_t n = blocks * tiles * 64;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t l = i % 32, h = (i / 32) % 2, t = (i / 64) % tiles, g = i / (64 * tiles);
        const size_t r = t * kTileRows + l;
        uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const size_t j = (l + 16 * h + k) % 32;
            unsigned byte = 125;  // five zero trits
            if (r < rows) {
                if (SRC == kSrcPlanar) {
                    byte = src[(r * blocks + g) * kBlockBytes + j];
                } else {
                    unsigned b = 0, radix = 1;
#pragma unroll
                    for (int p = 0; p < 5; ++p) {
                        const size_t c = g * kBlockTrits + p * kBlockBytes + j;
                        const int tr = c < cols ? source_trit<SRC>(src, r, c, cols) : 0;
                        b += radix * static_cast<unsigned>(tr + 1);
                        radix = p == 2 ? 28u : radix * 3u;  // 1, 3, 9, 28, 84
                    }
                    byte = b;
                }
            }
            out[k / 4] |= byte << (8 * (k % 4));
        }
        dst[i] = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// Inverse layout change: stream -> planar bytes (rows * blocks * 32).
__global__ void stream_to_planar_kernel(const uint8_t* __restrict__ stream, uint8_t* __restrict__ planar, size_t rows, size_t blocks,
                                        size_t tiles) {
    const size_t n = rows * blocks * kBlockBytes;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t j = i % kBlockBytes, g = (i / kBlockBytes) % blocks, r = i / (kBlockBytes * blocks);
        const size_t t = r / kTileRows, l = r % kTileRows;
        const size_t s = (j + 32 - l) % 32;  // step at which lane l meets column j
        planar[i] = stream[((g * tiles + t) * 2 + s / 16) * 512 + l * 16 + s % 16];
    }
}

// Adds a scale: out_f32[i] = float(acc[i]) * scale.
__global__ void scale_kernel(const int32_t* __restrict__ acc, float* __restrict__ out, size_t n, float scale) {
    const size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (i < n) out[i] = static_cast<float>(acc[i]) * scale;
}

}  // namespace qtb
