// Block-scaled projection of Q2_0 models on the device: one-time transcode of a Q2_0 payload to planar velurex bytes plus
// one f32 scale per 64 weights, the Q8_0 activation quantiser, and the GEMV in the floating-point order of llama.cpp's
// Q2_0 x Q8_0 dot product.
//
// Reference behaviour reproduced: rust/crates/quintrit-format/src/decoders/q2_0.rs:34-101 (decode, code 3 rejected, one
// scale per 64 weights) + quintrit-core/src/pack.rs:103-131 (planar rows); rust/crates/quintrit-runtime/src/ops.rs:898-910
// (quantize_q8_0_scalar); rust/crates/quintrit-core/src/block_scaled.rs:175-202 (dot_row_scalar) and :140-145 (hsum8).
// The reference runs this path on the CPU only.
#pragma once
#include <algorithm>
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

// Trit table in shared memory: for every byte value the trits of planes 0-3 as four int8 in one word (.x) and the trit of
// plane 4 in the low byte of a second word (.y). The table holds 32 copies, entry b of copy c at index b * 32 + c: lane l
// of a warp reads copy l, so the 32 lanes hit different banks whatever bytes they look up.
constexpr int kBsCopies = 32;
__device__ __forceinline__ void build_trit_table(uint2* tab) {
    for (int b = threadIdx.x; b < 256; b += blockDim.x) {  // the entry of a byte value is computed once and written 32 times
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
        const uint2 e = make_uint2(w, static_cast<uint32_t>(t[4]) & 0xFFu);
#pragma unroll 8
        for (int c = 0; c < kBsCopies; ++c) tab[b * kBsCopies + ((c + b) & (kBsCopies - 1))] = e;  // (rotated: the threads of a warp write different banks)
    }
}

constexpr int kBsTableBytes = 256 * kBsCopies * 8;  // 64 KiB
constexpr int kBsThreads = 256;                      // eight warps of four rows each
constexpr int kBsRowsPerCta = kBsThreads / 8;        // a row belongs to eight threads, one per lane of the reference's dot product

// Look-up of byte K of `w`: the entry address is table base + byte * 256 + lane * 8, formed with one byte permute and one add.
template <int K>
__device__ __forceinline__ uint2 bs_lookup(uint32_t w, uint32_t tab_lane_addr) {
    uint32_t off;
    asm("prmt.b32 %0, %1, 0, %2;" : "=r"(off) : "r"(w), "n"(0x4404 | (K << 4)));  // byte K of w into bits 8-15
    uint2 e;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(e.x), "=r"(e.y) : "r"(tab_lane_addr + off));
    return e;
}

// Four 160-trit blocks = twenty activation blocks s0 .. s0 + 19 of one thread's bytes. FULL: all twenty exist.
template <bool FULL>
__device__ __forceinline__ void bs_group(const uint32_t (&w)[4], uint32_t tab_lane_addr, const int4* __restrict__ q4, const float4* __restrict__ as, float ws_a, float ws_b, int s0,
                                         int nact, float& acc0, float& acc1) {
    float wsc[10], asc[20];
    int qv[20];
#pragma unroll
    for (int k = 0; k < 10; ++k) wsc[k] = __shfl_sync(0xffffffffu, k < 8 ? ws_a : ws_b, k & 7, 8);  // lane k (k - 8) of the row's eight holds scale k (zero past the end)
#pragma unroll
    for (int t = 0; t < 5; ++t) {  // the group's twenty activation scales and this lane's twenty code words: five 16-byte loads each (zeros past the end)
        const float4 a4 = as[t];
        const int4 c4 = q4[t];
        asc[4 * t] = a4.x, asc[4 * t + 1] = a4.y, asc[4 * t + 2] = a4.z, asc[4 * t + 3] = a4.w;
        qv[4 * t] = c4.x, qv[4 * t + 1] = c4.y, qv[4 * t + 2] = c4.z, qv[4 * t + 3] = c4.w;
    }
#pragma unroll
    for (int bi = 0; bi < 4; ++bi) {
        const uint2 e0 = bs_lookup<0>(w[bi], tab_lane_addr), e1 = bs_lookup<1>(w[bi], tab_lane_addr), e2 = bs_lookup<2>(w[bi], tab_lane_addr), e3 = bs_lookup<3>(w[bi], tab_lane_addr);
        // transpose the 4 x 4 bytes: word p = the trits of plane p of the four weights
        const uint32_t lo01 = __byte_perm(e0.x, e1.x, 0x5140), hi01 = __byte_perm(e0.x, e1.x, 0x7362);
        const uint32_t lo23 = __byte_perm(e2.x, e3.x, 0x5140), hi23 = __byte_perm(e2.x, e3.x, 0x7362);
        uint32_t plane[5];
        plane[0] = __byte_perm(lo01, lo23, 0x5410);
        plane[1] = __byte_perm(lo01, lo23, 0x7632);
        plane[2] = __byte_perm(hi01, hi23, 0x5410);
        plane[3] = __byte_perm(hi01, hi23, 0x7632);
        plane[4] = __byte_perm(__byte_perm(e0.y, e1.y, 0x3340), __byte_perm(e2.y, e3.y, 0x3340), 0x5410);
#pragma unroll
        for (int p = 0; p < 5; ++p) {
            const int i = bi * 5 + p;
            if (FULL || s0 + i < nact) {
                const float sum = static_cast<float>(__dp4a(static_cast<int>(plane[p]), qv[i], 0));
                const float dd = __fmul_rn(wsc[i >> 1], asc[i]);
                if ((i >> 1) & 1)
                    acc1 = __fmaf_rn(dd, sum, acc1);
                else
                    acc0 = __fmaf_rn(dd, sum, acc0);
            }
        }
    }
}

// Block-scaled GEMV (block_scaled.rs:175-202). Eight threads own a row: thread j holds the two accumulators of lane j of the
// reference's eight-lane dot product and walks the row's 160-trit blocks in order. Per block it reads its four bytes (the
// planar bytes 4j .. 4j + 3, one 32-bit word), looks each byte up, transposes the 4 x 4 trits into one int8x4 word per plane
// and forms, for each of the block's five activation blocks s = 5 b + p, the exact integer lane sum (dp4a with four activation
// codes) and the step acc[(s / 2) & 1] = fma(w_scale[s / 2] * a_scale[s], sum, acc). Four blocks are unrolled together: twenty
// activation blocks is the period after which the pattern of accumulators repeats, so the choice is made at compile time.
// At the end the two accumulators are added and the eight lanes reduced as ((l0+l4) + (l2+l6)) + ((l1+l5) + (l3+l7)).
// Activations (int8 codes and block scales) are staged in shared memory once per CTA; CTAs walk the rows with a grid stride.
// A launch serves up to three matrices that take the same activation vector (q | k | v, gate | up): their groups of 32 rows are
// numbered one after the other and the CTAs walk that numbering.
struct BsMatrices {
    const uint8_t* planar[3];
    const float* w_scales[3];
    float* out[3];
    unsigned rows[3];
    unsigned group_end[3];  // groups of 32 rows up to and including matrix i
    int count;
};
inline BsMatrices bs_one_matrix(const uint8_t* planar, const float* w_scales, size_t rows, float* out) {
    BsMatrices m{};
    m.planar[0] = planar, m.w_scales[0] = w_scales, m.out[0] = out, m.rows[0] = static_cast<unsigned>(rows);
    m.group_end[0] = m.group_end[1] = m.group_end[2] = static_cast<unsigned>((rows + 31) / 32);
    m.count = 1;
    return m;
}

// ROOMY: a launch whose CTAs do not fill the multiprocessors three deep anyway (few rows, or long rows whose activations take
// the shared memory) is compiled without the register ceiling that three resident CTAs need.
template <bool ROOMY>
__global__ void __launch_bounds__(kBsThreads, ROOMY ? 1 : 3) gemv_block_scaled_kernel(BsMatrices m, const int8_t* __restrict__ qs, const float* __restrict__ a_scales, size_t cols) {
    extern __shared__ __align__(16) unsigned char bs_smem[];
    uint2* tab = reinterpret_cast<uint2*>(bs_smem);
    const int nact = static_cast<int>(cols / 32), nblocks = (nact + 4) / 5, ngroups = (nblocks + 3) / 4;
    // Activations, staged once per CTA in the order the walk reads them: twenty scales per group of four blocks, and per group
    // and lane j the twenty code words (activation block s, bytes 4j .. 4j + 3) side by side - so a walk step fetches each with
    // five 16-byte loads, the eight lanes of a row from eight different bank groups. Zeros past the end of the row.
    float* s_as = reinterpret_cast<float*>(bs_smem + kBsTableBytes);  // ngroups * 20 floats
    int* s_q4 = reinterpret_cast<int*>(s_as + ngroups * 20);         // ngroups * 8 * 20 words
    {   // The first row group's planar rows and scales (two contiguous ranges) are requested into L2 as a whole while the table is built.
        const unsigned grp = blockIdx.x;
        if (grp < m.group_end[2]) {
            const int which = grp < m.group_end[0] ? 0 : (grp < m.group_end[1] ? 1 : 2);
            const unsigned grp0 = which == 0 ? 0u : (which == 1 ? m.group_end[0] : m.group_end[1]);
            const size_t rows = which == 0 ? m.rows[0] : (which == 1 ? m.rows[1] : m.rows[2]);
            const size_t r0 = static_cast<size_t>(grp - grp0) * kBsRowsPerCta, nr = min(static_cast<size_t>(kBsRowsPerCta), rows - r0);
            const size_t row_bytes = static_cast<size_t>(nblocks) * 32, scale_bytes = (cols / 64) * 4;
            const char* pw = reinterpret_cast<const char*>(which == 0 ? m.planar[0] : (which == 1 ? m.planar[1] : m.planar[2])) + r0 * row_bytes;
            const char* ps = reinterpret_cast<const char*>(which == 0 ? m.w_scales[0] : (which == 1 ? m.w_scales[1] : m.w_scales[2])) + r0 * scale_bytes;
            for (size_t off = static_cast<size_t>(threadIdx.x) * 128; off < nr * row_bytes; off += static_cast<size_t>(kBsThreads) * 128)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(pw + off));
            for (size_t off = static_cast<size_t>(threadIdx.x) * 128; off < nr * scale_bytes; off += static_cast<size_t>(kBsThreads) * 128)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(ps + off));
        }
    }
    build_trit_table(tab);
    for (int i = threadIdx.x; i < ngroups * 20; i += kBsThreads) s_as[i] = i < nact ? a_scales[i] : 0.0f;
    for (int i = threadIdx.x; i < ngroups * 160; i += kBsThreads) {
        const int s = i >> 3, jj = i & 7;  // word jj of activation block s: read in the order of the codes, stored transposed
        s_q4[((s / 20) * 8 + jj) * 20 + s % 20] = s < nact ? reinterpret_cast<const int*>(qs)[i] : 0;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, j = lane & 7;
    const size_t row_words = static_cast<size_t>(nblocks) * 8, sb = cols / 64;
    const uint32_t tab_lane_addr = static_cast<uint32_t>(__cvta_generic_to_shared(tab)) + lane * 8;
    for (unsigned grp = blockIdx.x; grp < m.group_end[2]; grp += gridDim.x) {
        const int which = grp < m.group_end[0] ? 0 : (grp < m.group_end[1] ? 1 : 2);
        const unsigned grp0 = which == 0 ? 0u : (which == 1 ? m.group_end[0] : m.group_end[1]);
        const uint8_t* __restrict__ planar = which == 0 ? m.planar[0] : (which == 1 ? m.planar[1] : m.planar[2]);
        const float* __restrict__ w_scales = which == 0 ? m.w_scales[0] : (which == 1 ? m.w_scales[1] : m.w_scales[2]);
        float* __restrict__ out = which == 0 ? m.out[0] : (which == 1 ? m.out[1] : m.out[2]);
        const size_t rows = which == 0 ? m.rows[0] : (which == 1 ? m.rows[1] : m.rows[2]);
        const size_t r = static_cast<size_t>(grp - grp0) * kBsRowsPerCta + (threadIdx.x >> 3);
        const bool valid = r < rows;
        const size_t rr = valid ? r : rows - 1;  // threads beyond the last row walk it once more and store nothing
        const uint32_t* roww = reinterpret_cast<const uint32_t*>(planar) + rr * row_words + j;
        const float* ws = w_scales + rr * sb;
        float acc0 = 0.0f, acc1 = 0.0f;
        // What a group needs from memory - the lane's four words and the row's ten weight scales, of which lane j fetches
        // scale j and lanes 0 and 1 also scales 8 and 9 - is requested two groups ahead and held in registers meanwhile.
        uint32_t n1[4], n2[4];
        float a1, b1, a2, b2;
        auto fetch = [&](int g, uint32_t (&nw)[4], float& sa, float& sb2) {
#pragma unroll
            for (int bi = 0; bi < 4; ++bi) nw[bi] = g * 4 + bi < nblocks ? __ldg(roww + (g * 4 + bi) * 8) : 0x7D7D7D7Du;  // byte 125: five zero trits
            sa = g * 10 + j < static_cast<int>(sb) ? __ldg(ws + g * 10 + j) : 0.0f;
            sb2 = (j < 2 && g * 10 + 8 + j < static_cast<int>(sb)) ? __ldg(ws + g * 10 + 8 + j) : 0.0f;
        };
        fetch(0, n1, a1, b1);
        fetch(1, n2, a2, b2);
        // Two groups per turn, the two register sets taking turns: a set is copied out only once its own loads (two groups old)
        // are back, and never waits for the other set's younger ones. (Four sets, four groups ahead, measured slower.)
        auto step = [&](int g, uint32_t (&nw)[4], float& sa, float& sb2) {
            uint32_t w[4];
#pragma unroll
            for (int bi = 0; bi < 4; ++bi) w[bi] = nw[bi];
            const float wa = sa, wb = sb2;
            fetch(g + 2, nw, sa, sb2);
            const int s0 = g * 20;
            if (s0 + 20 <= nact)
                bs_group<true>(w, tab_lane_addr, reinterpret_cast<const int4*>(s_q4) + (g * 8 + j) * 5, reinterpret_cast<const float4*>(s_as) + g * 5, wa, wb, s0, nact, acc0, acc1);
            else
                bs_group<false>(w, tab_lane_addr, reinterpret_cast<const int4*>(s_q4) + (g * 8 + j) * 5, reinterpret_cast<const float4*>(s_as) + g * 5, wa, wb, s0, nact, acc0, acc1);
        };
        for (int g = 0; g < ngroups; g += 2) {
            step(g, n1, a1, b1);
            if (g + 1 < ngroups) step(g + 1, n2, a2, b2);
        }
        float l = __fadd_rn(acc0, acc1);
        const float up4 = __shfl_down_sync(0xffffffffu, l, 4, 8);
        l = __fadd_rn(up4, l);  // r_j = l[j + 4] + l[j]
        const float up2 = __shfl_down_sync(0xffffffffu, l, 2, 8);
        l = __fadd_rn(l, up2);  // (r0 + r2), (r1 + r3)
        const float up1 = __shfl_down_sync(0xffffffffu, l, 1, 8);
        l = __fadd_rn(l, up1);
        if (j == 0 && valid) out[r] = l;
    }
}

__host__ __device__ constexpr size_t block_scaled_groups(size_t cols) { return ((cols / 32 + 4) / 5 + 3) / 4; }  // groups of four 160-trit blocks in a row
__host__ __device__ constexpr size_t block_scaled_smem_bytes(size_t cols) { return kBsTableBytes + block_scaled_groups(cols) * (20 * 4 + 160 * 4); }
// CTAs of a launch: 32 rows per CTA at a time, as many CTAs as fit the shared memory of the multiprocessors (all resident: what a
// multiprocessor has to issue is the sum over its CTAs, and the CTAs that walk one row group more are spread over all of them).
inline int block_scaled_grid(size_t rows, int sm_count, size_t cols = 0) {
    const size_t per_sm = std::max<size_t>(1, std::min<size_t>(3, (227 * 1024) / (block_scaled_smem_bytes(cols) + 1024)));
    const size_t want = (rows + kBsRowsPerCta - 1) / kBsRowsPerCta, cap = static_cast<size_t>(sm_count) * per_sm;
    return static_cast<int>(want < cap ? want : cap);
}

// Lets both forms of the kernel use the shared memory of a multiprocessor.
inline cudaError_t block_scaled_allow_smem() {
    const int most = static_cast<int>(block_scaled_smem_bytes(131072));
    cudaError_t e = cudaFuncSetAttribute(gemv_block_scaled_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_block_scaled_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    return e;
}
// The launch for the matrices of `m` (all of `cols` columns, over the activation blocks qs / a_scales).
inline void block_scaled_launch(const BsMatrices& m, const int8_t* qs, const float* a_scales, size_t cols, int sm_count, cudaStream_t stream) {
    const int grid = block_scaled_grid(static_cast<size_t>(m.group_end[2]) * kBsRowsPerCta, sm_count, cols);
    if (grid <= 2 * sm_count)
        gemv_block_scaled_kernel<true><<<grid, kBsThreads, block_scaled_smem_bytes(cols), stream>>>(m, qs, a_scales, cols);
    else
        gemv_block_scaled_kernel<false><<<grid, kBsThreads, block_scaled_smem_bytes(cols), stream>>>(m, qs, a_scales, cols);
}

}  // namespace qtb
