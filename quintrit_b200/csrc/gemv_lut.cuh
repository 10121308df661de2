// Exact int32 GEMV of a velurex-encoded ternary matrix with an int8 activation vector, for sm_100a.
//
// What it computes: out[n] = sum_k trit[n][k] * act[k], the integers of the reference's CPU table kernels
// (rust/crates/quintrit-core/src/simd/scalar.rs:11-64, quintrit-core/src/lut.rs:492-562) and of its CUDA projection
// kernel (rust/crates/quintrit-cuda/kernels/gemv.cu:65-138).
//
// How, and why this shape on a B200. The HBM stream is 0.2 bytes per weight, so at ~6.5 TB/s the chip has about three
// issue slots per weight BYTE; decoding a byte into digits arithmetically costs more than that. The byte is therefore
// used directly as the index of a per-byte-column table in shared memory that already holds the finished partial sum
// t0*a0 + t1*a1 + t2*a2 + t3*a3 + t4*a4 of that column's five activations (the reference's activation tables taken one
// step further: its (t0,t1,t2) and (t3,t4) tables merged, int32 entries, so the x = 16 hi + lo split that keeps its
// int8 entries exact is not needed and the integers are the same). Per weight byte the inner loop is one byte-permute
// that forms the table address, one shared-memory load and half a three-input add.
//
// Bank conflicts: a lane owns a ROW and walks the 32 byte-columns of a 160-trit block diagonally (lane l reads column
// (l + s) mod 32 at step s), the table is laid out [byte value][column] with 4-byte entries, so the 32 lanes of a warp
// always hit 32 different banks whatever the weight bytes are. The device weight layout stores every row's 32 block
// bytes pre-rotated by its lane so that step s uses a fixed register byte.
//
// Layout in HBM ("stream" layout): for block g (160 trits), row tile t (32 rows), half h, lane l: 16 bytes at
// ((g * tiles + t) * 2 + h) * 512 + l * 16, byte k of which is planar byte (l + 16 h + k) mod 32 of block g of row
// 32 t + l. Rows beyond the matrix hold byte 125 (five zero trits).
//
// Work decomposition: an item is (block pair, range of row tiles). A CTA builds the 64 KB table of the pair (256 byte
// values x 2 blocks x 32 columns x int32), then its 8 warps stream the tiles; every lane adds its row's partial sum to
// the output with one red.global.add (the K dimension is split over items, so the output is cleared beforehand).
// The kernel is persistent: CTAs take items from a global counter until none is left, three CTAs per SM.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace qtb {

constexpr int kTileRows = 32;
constexpr int kBlockTrits = 160;
constexpr int kBlockBytes = 32;
constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kTableBytes = 256 * 2 * 32 * 4;  // 64 KiB
constexpr int kCtasPerSm = 3;

struct GemvItem {
    unsigned long long w_off;  // offset in uint4 units of block A, tile `tile0`, from the weight base of the problem
    unsigned long long w2_off; // same for block B (unused when nblk == 1)
    unsigned int problem;      // index into the problem table
    int col0;                  // first column (trit index) of block A
    int tile0, ntiles;
    int nblk;                  // 1 or 2
    int pad;
};

struct GemvProblem {
    const uint4* w;            // stream-layout weights
    unsigned long long act_off; // offset of the activation vector in the activation buffer (bytes)
    unsigned long long out_off; // offset of the result vector in the result buffer (int32 elements)
    int rows, cols;
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

__device__ __forceinline__ int lds32(uint32_t addr) {
    int v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Table address of step S for a weight word `w` (byte S % 4 of it) and the lane's column word `c`:
// result byte 0 = column byte ((lane + S) mod 32) * 4 taken from c, byte 1 = the weight byte, bytes 2 and 3 = the
// replicated sign bit of the column byte, which is 0 because the column byte is below 128.
template <int J>
__device__ __forceinline__ uint32_t table_offset(uint32_t w, uint32_t c) {
    constexpr uint32_t sel = (4u + J) | (uint32_t(J) << 4) | ((0xCu + J) << 8) | ((0xCu + J) << 12);
    return prmt(w, c, sel);
}

template <int J>
__device__ __forceinline__ void lookup2(int& acc, uint32_t wa, uint32_t wb, uint32_t c, uint32_t tbase) {
    const int va = lds32(tbase + table_offset<J>(wa, c));
    const int vb = lds32(tbase + 128u + table_offset<J>(wb, c));
    acc += va + vb;
}

template <int J>
__device__ __forceinline__ void lookup1(int& acc, uint32_t wa, uint32_t c, uint32_t tbase) {
    acc += lds32(tbase + table_offset<J>(wa, c));
}

__device__ __forceinline__ void word2(int& acc, uint32_t wa, uint32_t wb, uint32_t c, uint32_t tbase) {
    lookup2<0>(acc, wa, wb, c, tbase);
    lookup2<1>(acc, wa, wb, c, tbase);
    lookup2<2>(acc, wa, wb, c, tbase);
    lookup2<3>(acc, wa, wb, c, tbase);
}

__device__ __forceinline__ void word1(int& acc, uint32_t wa, uint32_t c, uint32_t tbase) {
    lookup1<0>(acc, wa, c, tbase);
    lookup1<1>(acc, wa, c, tbase);
    lookup1<2>(acc, wa, c, tbase);
    lookup1<3>(acc, wa, c, tbase);
}

// Fills the table of one block pair. Thread -> (column = tid & 63, part = tid >> 6); a part writes the byte values
// 28 U + L for U in {part, part + 4, part + 8} and all 27 L. Consecutive threads write consecutive words: no conflicts.
__device__ __forceinline__ void fill_table(int* tab, const int8_t* __restrict__ act, int cols, int col0, int nblk, int tid) {
    const int col = tid & 63, gb = col >> 5, j = col & 31, part = tid >> 6;
    int a[5];
#pragma unroll
    for (int p = 0; p < 5; ++p) {
        const int c = col0 + gb * kBlockTrits + p * kBlockBytes + j;
        a[p] = (gb < nblk && c < cols) ? static_cast<int>(__ldg(act + c)) : 0;
    }
#pragma unroll
    for (int ui = 0; ui < 3; ++ui) {
        const int u = part + 4 * ui;
        if (u > 8) break;
        const int d3 = u % 3, d4 = u / 3;
        const int tu = (d3 - 1) * a[3] + (d4 - 1) * a[4];
        int* dst = tab + (28 * u) * 64 + col;
#pragma unroll
        for (int l = 0; l < 27; ++l) {
            const int t0 = l % 3 - 1, t1 = (l / 3) % 3 - 1, t2 = l / 9 - 1;
            dst[l * 64] = tu + t0 * a[0] + t1 * a[1] + t2 * a[2];
        }
    }
}

__global__ void __launch_bounds__(kGemvThreads, kCtasPerSm)
gemv_lut_kernel(const GemvItem* __restrict__ items, int n_items, const GemvProblem* __restrict__ problems,
                const int8_t* __restrict__ act_base, int32_t* __restrict__ out_base, unsigned int* __restrict__ counters) {
    extern __shared__ __align__(1024) int tab[];
    __shared__ int s_item;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t tbase = static_cast<uint32_t>(__cvta_generic_to_shared(tab));

    // Byte values the packer never produces (the gap after every 27 values and 251..255) read as zero.
    for (int i = tid; i < 13 * 64; i += kGemvThreads) {
        const int k = i >> 6;  // 27, 55, ..., 251, then 252..255
        const int idx = k < 9 ? 28 * k + 27 : 243 + k;
        tab[idx * 64 + (i & 63)] = 0;
    }

    // Column bytes of the diagonal walk: word q, byte j -> ((lane + 4 q + j) mod 32) * 4.
    uint32_t creg[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        uint32_t v = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) v |= static_cast<uint32_t>(((lane + 4 * q + j) & 31) * 4) << (8 * j);
        creg[q] = v;
    }

    while (true) {
        if (tid == 0) s_item = static_cast<int>(atomicAdd(&counters[0], 1u));
        __syncthreads();
        const int it = s_item;
        if (it >= n_items) break;
        const GemvItem item = items[it];
        const GemvProblem pr = problems[item.problem];
        fill_table(tab, act_base + pr.act_off, pr.cols, item.col0, item.nblk, tid);
        __syncthreads();

        int32_t* out = out_base + pr.out_off;
        const uint4* wa = pr.w + item.w_off + lane;
        const uint4* wb = pr.w + item.w2_off + lane;
        if (item.nblk == 2) {
            int t = warp;
            uint4 a0, a1, b0, b1;
            if (t < item.ntiles) {
                a0 = ldg_stream(wa + t * 64);
                a1 = ldg_stream(wa + t * 64 + 32);
                b0 = ldg_stream(wb + t * 64);
                b1 = ldg_stream(wb + t * 64 + 32);
            }
            while (t < item.ntiles) {
                const int tn = t + kGemvWarps;
                uint4 na0 = a0, na1 = a1, nb0 = b0, nb1 = b1;
                if (tn < item.ntiles) {
                    na0 = ldg_stream(wa + tn * 64);
                    na1 = ldg_stream(wa + tn * 64 + 32);
                    nb0 = ldg_stream(wb + tn * 64);
                    nb1 = ldg_stream(wb + tn * 64 + 32);
                }
                int acc = 0;
                word2(acc, a0.x, b0.x, creg[0], tbase);
                word2(acc, a0.y, b0.y, creg[1], tbase);
                word2(acc, a0.z, b0.z, creg[2], tbase);
                word2(acc, a0.w, b0.w, creg[3], tbase);
                word2(acc, a1.x, b1.x, creg[4], tbase);
                word2(acc, a1.y, b1.y, creg[5], tbase);
                word2(acc, a1.z, b1.z, creg[6], tbase);
                word2(acc, a1.w, b1.w, creg[7], tbase);
                const int row = (item.tile0 + t) * kTileRows + lane;
                if (row < pr.rows) atomicAdd(out + row, acc);
                a0 = na0, a1 = na1, b0 = nb0, b1 = nb1;
                t = tn;
            }
        } else {
            for (int t = warp; t < item.ntiles; t += kGemvWarps) {
                const uint4 a0 = ldg_stream(wa + t * 64), a1 = ldg_stream(wa + t * 64 + 32);
                int acc = 0;
                word1(acc, a0.x, creg[0], tbase);
                word1(acc, a0.y, creg[1], tbase);
                word1(acc, a0.z, creg[2], tbase);
                word1(acc, a0.w, creg[3], tbase);
                word1(acc, a1.x, creg[4], tbase);
                word1(acc, a1.y, creg[5], tbase);
                word1(acc, a1.z, creg[6], tbase);
                word1(acc, a1.w, creg[7], tbase);
                const int row = (item.tile0 + t) * kTileRows + lane;
                if (row < pr.rows) atomicAdd(out + row, acc);
            }
        }
        __syncthreads();  // the table and s_item are rewritten next
    }

    // The last CTA to leave re-arms the counters for the next launch.
    if (tid == 0) {
        __threadfence();
        const unsigned int done = atomicAdd(&counters[1], 1u);
        if (done == gridDim.x - 1) {
            counters[0] = 0;
            counters[1] = 0;
            __threadfence();
        }
    }
}

}  // namespace qtb
