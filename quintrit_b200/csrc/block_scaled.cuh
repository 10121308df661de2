// Block-scaled projection of Q2_0 models on the device: one-time transcode of a Q2_0 payload to planar velurex bytes plus
// one f32 scale per 64 weights, the Q8_0 activation quantiser, and the GEMV in the floating-point order of llama.cpp's
// Q2_0 x Q8_0 dot product.
//
// Reference behaviour reproduced: rust/crates/quintrit-format/src/decoders/q2_0.rs:34-101 (decode, code 3 rejected, one
// scale per 64 weights) + quintrit-core/src/pack.rs:103-131 (planar rows); rust/crates/quintrit-runtime/src/ops.rs:898-910
// (quantize_q8_0_scalar); rust/crates/quintrit-core/src/block_scaled.rs:175-202 (dot_row_scalar) and :140-145 (hsum8).
// The reference runs this path on the CPU only.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "gemv_lut.cuh"

namespace qtb {

constexpr int kSrcQ2 = 42;  // GGML type id of Q2_0 (blocks of 64 weights: f16 scale + 16 code bytes)

// One thread per planar output byte (row, block b, byte j): the five trits of columns b*160 + p*32 + j, p = 0..4, from the
// Q2_0 codes (four per byte, lowest bits first; weight = code - 1). A code 3 raises *bad (the first offending weight wins).
__global__ void q2_0_to_planar_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ planar, size_t rows, size_t cols, size_t blocks,
                                      unsigned long long* __restrict__ bad) {
    const size_t n = rows * blocks * 32;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t j = i % 32, b = (i / 32) % blocks, r = i / (32 * blocks);
        const uint8_t* row = src + r * (cols / 64) * 18;
        unsigned d[5];
#pragma unroll
        for (int p = 0; p < 5; ++p) {
            const size_t c = b * kBlockTrits + p * kBlockBytes + j;
            unsigned code = 1;  // padding columns are zero trits
            if (c < cols) {
                code = (row[(c / 64) * 18 + 2 + (c % 64) / 4] >> (2 * (c % 4))) & 3u;
                if (code == 3) {
                    atomicMin(bad, static_cast<unsigned long long>(r * cols + c));
                    code = 1;
                }
            }
            d[p] = code;
        }
        planar[i] = static_cast<uint8_t>(d[0] + 3 * d[1] + 9 * d[2] + 28 * d[3] + 84 * d[4]);
    }
}

// One thread per 64-weight block: its f16 scale widened to f32.
__global__ void q2_0_scales_kernel(const uint8_t* __restrict__ src, float* __restrict__ scales, size_t nblocks) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nblocks; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const unsigned short bits = static_cast<unsigned short>(src[i * 18] | (src[i * 18 + 1] << 8));
        scales[i] = __half2float(__ushort_as_half(bits));
    }
}

// Q8_0 quantiser: one warp per block of 32 values. amax ignores NaN (fmaxf does), d = f16(amax / 127) as f32,
// code = round-to-nearest-even(x * (127 / amax)) clamped to [-128, 127], NaN -> 0.
__global__ void quantize_q8_0_kernel(const float* __restrict__ x, size_t n, int8_t* __restrict__ qs, float* __restrict__ d) {
    const size_t warp = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) / 32, lane = threadIdx.x & 31;
    const size_t nwarps = static_cast<size_t>(gridDim.x) * blockDim.x / 32;
    for (size_t b = warp; b < n / 32; b += nwarps) {
        const float v = x[b * 32 + lane];
        float amax = fabsf(v);
        if (amax != amax) amax = 0.0f;
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (lane == 0) d[b] = __half2float(__float2half_rn(__fdiv_rn(amax, 127.0f)));
        const float id = amax != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
        const float r = rintf(__fmul_rn(v, id));
        int q = 0;
        if (r == r) q = static_cast<int>(fminf(fmaxf(r, -128.0f), 127.0f));
        qs[b * 32 + lane] = static_cast<int8_t>(q);
    }
}

// Trit tables in shared memory: for every byte value the trits of planes 0-3 as four int8 in one word, and plane 4 (in
// the low byte of a word). Each table holds kBsCopies interleaved copies (entry b of copy c at index b * kBsCopies + c):
// the 32 lanes of a warp look up unrelated bytes at the same time, and a lane that reads copy lane % kBsCopies meets at
// most a quarter of the other lanes in its banks.
constexpr int kBsCopies = 8;
__device__ __forceinline__ void build_trit_tables(uint32_t* t0123, uint32_t* t4) {
    for (int b = threadIdx.x; b < 256; b += blockDim.x) {
        int t[5] = {0, 0, 0, 0, 0};
        const bool valid = b <= 250 && b % 28 != 27;
        if (valid) {
            int r = b;
            const int d4 = r / 84;
            r -= 84 * d4;
            const int d3 = r / 28;
            r -= 28 * d3;
            const int d2 = r / 9;
            r -= 9 * d2;
            const int d1 = r / 3, d0 = r - 3 * d1;
            t[0] = d0 - 1, t[1] = d1 - 1, t[2] = d2 - 1, t[3] = d3 - 1, t[4] = d4 - 1;
        }
        const uint32_t w = (static_cast<uint32_t>(t[0]) & 0xFFu) | ((static_cast<uint32_t>(t[1]) & 0xFFu) << 8) | ((static_cast<uint32_t>(t[2]) & 0xFFu) << 16) |
                           ((static_cast<uint32_t>(t[3]) & 0xFFu) << 24);
        for (int c = 0; c < kBsCopies; ++c) {
            t0123[b * kBsCopies + c] = w;
            t4[b * kBsCopies + c] = static_cast<uint32_t>(t[4]) & 0xFFu;
        }
    }
}

constexpr int kBsTableBytes = 2 * 256 * kBsCopies * 4;  // the two trit tables
constexpr int kBsThreads = 256;                       // eight warps, one row per warp at a time
constexpr int kBsWarps = kBsThreads / 32;
constexpr int kBsChunkBlocks = 32;                    // 160-trit blocks a warp decodes at once (one per lane)
constexpr int kBsChunkActs = kBsChunkBlocks * 5;      // activation blocks of such a chunk
constexpr int kBsLaneStride = 9;                      // floats per activation block in the scratch (8 lane sums + 1: no bank conflicts)
constexpr int kBsWarpScratch = kBsChunkActs * kBsLaneStride + kBsChunkActs;  // floats: lane sums, then the scale products

// Block-scaled GEMV, one row per warp, in two steps per chunk of 32 weight blocks (160 activation blocks):
//  1. lane l decodes block l of the chunk (its 32 bytes: two 16-byte loads), forms for each of its five planes the eight
//     exact integer lane sums (dp4a of four trits with four activation codes) and the product w_scale[s/2] * a_scale[s],
//     and leaves them in the warp's scratch - this part is order-free, so it runs 32 blocks wide;
//  2. sixteen lanes (two accumulators x eight lanes of the reference's dot product) run the multiply-add chains over the
//     chunk strictly in the order of s: lane = fma(product, sum, lane), blocks of 64 weights alternating between the two
//     accumulators (block_scaled.rs:175-202).
// At the end the two accumulators are added and the eight lanes reduced as ((l0+l4) + (l2+l6)) + ((l1+l5) + (l3+l7)).
// Activations (int8 codes and block scales) are staged in shared memory once per CTA.
__global__ void __launch_bounds__(kBsThreads) gemv_block_scaled_kernel(const uint8_t* __restrict__ planar, const float* __restrict__ w_scales,
                                                                        const int8_t* __restrict__ qs, const float* __restrict__ a_scales, size_t rows,
                                                                        size_t cols, float* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char bs_smem[];
    uint32_t* t0123 = reinterpret_cast<uint32_t*>(bs_smem);                    // 256 x kBsCopies words
    uint32_t* t4 = t0123 + 256 * kBsCopies;                                    // likewise
    float* s_as = reinterpret_cast<float*>(bs_smem + kBsTableBytes);           // cols / 32 floats
    int8_t* s_q = reinterpret_cast<int8_t*>(s_as + cols / 32);          // cols codes (offset is a multiple of 4)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* pf = reinterpret_cast<float*>(bs_smem + ((kBsTableBytes + (cols / 32) * 4 + cols + 15) / 16) * 16) + warp * kBsWarpScratch;
    float* dd = pf + kBsChunkActs * kBsLaneStride;
    build_trit_tables(t0123, t4);
    for (size_t i = threadIdx.x; i < cols / 32; i += kBsThreads) s_as[i] = a_scales[i];
    for (size_t i = threadIdx.x; i < cols / 4; i += kBsThreads) reinterpret_cast<uint32_t*>(s_q)[i] = reinterpret_cast<const uint32_t*>(qs)[i];
    __syncthreads();
    const size_t row_bytes = (cols + kBlockTrits - 1) / kBlockTrits * kBlockBytes, sb = cols / 64, nact = cols / 32;
    const size_t nblocks = (nact + 4) / 5;
    const int chain_c = (lane >> 3) & 1, chain_j = lane & 7;  // lanes 0-15: accumulator and lane of the dot product
    for (size_t r = static_cast<size_t>(blockIdx.x) * kBsWarps + warp; r < rows; r += static_cast<size_t>(gridDim.x) * kBsWarps) {
        const uint8_t* row = planar + r * row_bytes;
        const float* ws = w_scales + r * sb;
        float acc = 0.0f;
        for (size_t c0 = 0; c0 < nblocks; c0 += kBsChunkBlocks) {
            const size_t b = c0 + lane;
            if (b < nblocks) {
                const uint4 lo = __ldg(reinterpret_cast<const uint4*>(row + b * kBlockBytes));
                const uint4 hi = __ldg(reinterpret_cast<const uint4*>(row + b * kBlockBytes) + 1);
                const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                for (int p = 0; p < 5; ++p) {
                    const size_t s = b * 5 + p;
                    if (s < nact) dd[lane * 5 + p] = __fmul_rn(__ldg(ws + s / 2), s_as[s]);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t w = words[j];
                    const uint32_t b0 = w & 0xFFu, b1 = (w >> 8) & 0xFFu, b2 = (w >> 16) & 0xFFu, b3 = w >> 24;
                    const int cp = lane & (kBsCopies - 1);
                    const uint32_t x0 = t0123[b0 * kBsCopies + cp], x1 = t0123[b1 * kBsCopies + cp], x2 = t0123[b2 * kBsCopies + cp], x3 = t0123[b3 * kBsCopies + cp];
                    // transpose the 4 x 4 bytes: word p = the trits of plane p of the four weights
                    const uint32_t lo01 = __byte_perm(x0, x1, 0x5140), hi01 = __byte_perm(x0, x1, 0x7362);
                    const uint32_t lo23 = __byte_perm(x2, x3, 0x5140), hi23 = __byte_perm(x2, x3, 0x7362);
                    uint32_t plane[5];
                    plane[0] = __byte_perm(lo01, lo23, 0x5410);
                    plane[1] = __byte_perm(lo01, lo23, 0x7632);
                    plane[2] = __byte_perm(hi01, hi23, 0x5410);
                    plane[3] = __byte_perm(hi01, hi23, 0x7632);
                    plane[4] = t4[b0 * kBsCopies + cp] | (t4[b1 * kBsCopies + cp] << 8) | (t4[b2 * kBsCopies + cp] << 16) | (t4[b3 * kBsCopies + cp] << 24);
#pragma unroll
                    for (int p = 0; p < 5; ++p) {
                        const size_t s = b * 5 + p;
                        if (s < nact) {
                            const int a4 = *reinterpret_cast<const int*>(s_q + s * 32 + 4 * j);
                            pf[(lane * 5 + p) * kBsLaneStride + j] = static_cast<float>(__dp4a(static_cast<int>(plane[p]), a4, 0));
                        }
                    }
                }
            }
            __syncwarp();
            // the chains: activation blocks 4m + 2c and 4m + 2c + 1 of the chunk belong to accumulator c (the chunk starts
            // on a multiple of 160 activation blocks, so the pattern of the whole row is the pattern inside the chunk)
            const int n_s = static_cast<int>(min(static_cast<size_t>(kBsChunkActs), nact - c0 * 5));
            if (lane < 16) {
#pragma unroll 4
                for (int s0 = 2 * chain_c; s0 < n_s; s0 += 4) {
                    acc = __fmaf_rn(dd[s0], pf[s0 * kBsLaneStride + chain_j], acc);
                    if (s0 + 1 < n_s) acc = __fmaf_rn(dd[s0 + 1], pf[(s0 + 1) * kBsLaneStride + chain_j], acc);
                }
            }
            __syncwarp();  // the scratch is rewritten by the next chunk
        }
        // lanes 0-7 hold accumulator 0, lanes 8-15 accumulator 1
        float l = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 8));
        const float up4 = __shfl_down_sync(0xffffffffu, l, 4);
        l = __fadd_rn(up4, l);  // r_j = l[j + 4] + l[j]
        const float up2 = __shfl_down_sync(0xffffffffu, l, 2);
        l = __fadd_rn(l, up2);  // (r0 + r2), (r1 + r3)
        const float up1 = __shfl_down_sync(0xffffffffu, l, 1);
        l = __fadd_rn(l, up1);
        if (lane == 0) out[r] = l;
    }
}

__host__ __device__ constexpr size_t block_scaled_smem_bytes(size_t cols) {
    return ((kBsTableBytes + (cols / 32) * 4 + cols + 15) / 16) * 16 + static_cast<size_t>(kBsWarps) * kBsWarpScratch * 4;
}
// CTAs of a launch: eight rows per CTA at a time, a few CTAs per SM.
inline int block_scaled_grid(size_t rows, int sm_count) {
    const size_t want = (rows + kBsWarps - 1) / kBsWarps, cap = static_cast<size_t>(sm_count) * 3;
    return static_cast<int>(want < cap ? want : cap);
}

}  // namespace qtb
