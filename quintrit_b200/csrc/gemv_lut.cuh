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
#ifndef QTB_GEMV_THREADS
#define QTB_GEMV_THREADS 256
#endif
#ifndef QTB_GEMV_CTAS
#define QTB_GEMV_CTAS 3
#endif
#ifndef QTB_GEMV_DEPTH
#define QTB_GEMV_DEPTH 2
#endif
constexpr int kGemvThreads = QTB_GEMV_THREADS;  // a multiple of 64 (the table fill maps 64 columns x parts)
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kGemvDepth = QTB_GEMV_DEPTH;      // row tiles a warp keeps in flight in registers
constexpr int kTableBytes = 256 * 2 * 32 * 4;  // 64 KiB
constexpr int kGemvSmemBytes = kTableBytes + 4 * 64 + 16;  // table, four item descriptors, four item indices
constexpr int kCtasPerSm = QTB_GEMV_CTAS;
constexpr int kGemvMaxRegs = (65536 / (kGemvThreads * kCtasPerSm)) / 8 * 8;  // registers per thread that still fit kCtasPerSm CTAs

// One unit of work, self-contained so that a CTA needs a single 64-byte fetch to start on it.
struct __align__(16) GemvItem {
    const uint4* wa;            // block A of the pair, first tile of the item (stream layout)
    const uint4* wb;            // block B (equal to wa when nblk == 1)
    unsigned long long act_off; // offset of the activation vector in the activation buffer (bytes)
    unsigned long long out_off; // offset of the result vector in the result buffer (int32 elements)
    int rows, cols;             // shape of the matrix
    int col0;                   // first column (trit index) of block A
    int tile0, ntiles;          // row tiles of the item
    int nblk;                   // 1 or 2
    int pad[2];
};
static_assert(sizeof(GemvItem) == 64, "GemvItem is fetched as four 16-byte pieces");

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// Shared-memory load at register + compile-time offset: the table base is a template constant so that the address
// formed by the byte permute is used as it is (no add per lookup).
template <uint32_t OFF>
__device__ __forceinline__ int lds32(uint32_t addr) {
    int v;
    asm volatile("ld.shared.b32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
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

template <uint32_t BASE, int J>
__device__ __forceinline__ void lookup2(int& acc, uint32_t wa, uint32_t wb, uint32_t c) {
    const int va = lds32<BASE>(table_offset<J>(wa, c));
    const int vb = lds32<BASE + 128u>(table_offset<J>(wb, c));
    acc += va + vb;
}

template <uint32_t BASE, int J>
__device__ __forceinline__ void lookup1(int& acc, uint32_t wa, uint32_t c) {
    acc += lds32<BASE>(table_offset<J>(wa, c));
}

template <uint32_t BASE>
__device__ __forceinline__ void word2(int& acc, uint32_t wa, uint32_t wb, uint32_t c) {
    lookup2<BASE, 0>(acc, wa, wb, c);
    lookup2<BASE, 1>(acc, wa, wb, c);
    lookup2<BASE, 2>(acc, wa, wb, c);
    lookup2<BASE, 3>(acc, wa, wb, c);
}

template <uint32_t BASE>
__device__ __forceinline__ void word1(int& acc, uint32_t wa, uint32_t c) {
    lookup1<BASE, 0>(acc, wa, c);
    lookup1<BASE, 1>(acc, wa, c);
    lookup1<BASE, 2>(acc, wa, c);
    lookup1<BASE, 3>(acc, wa, c);
}

// The five activations (planes 0..4) of the byte-column this thread fills, or zeros beyond the matrix.
__device__ __forceinline__ void load_column_acts(int a[5], const int8_t* __restrict__ act, int cols, int col0, int nblk, int tid) {
    const int col = tid & 63, gb = col >> 5, j = col & 31;
#pragma unroll
    for (int p = 0; p < 5; ++p) {
        const int c = col0 + gb * kBlockTrits + p * kBlockBytes + j;
        a[p] = (gb < nblk && c < cols) ? static_cast<int>(__ldg(act + c)) : 0;
    }
}

// Fills the table of one block pair. Thread -> (column = tid & 63, part = tid >> 6); a part writes the byte values
// 28 U + L for U in {part, part + parts, ...} and all 27 L. Consecutive threads write consecutive words: no conflicts.
__device__ __forceinline__ void fill_table(int* tab, const int a[5], int tid) {
    constexpr int parts = kGemvThreads / 64;
    const int col = tid & 63, part = tid >> 6;
#pragma unroll
    for (int ui = 0; ui < (9 + parts - 1) / parts; ++ui) {
        const int u = part + parts * ui;
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

// One row tile of a block pair in registers: 64 weight bytes per lane.
struct TileRegs {
    uint4 a0, a1, b0, b1;
};

template <uint32_t BASE>
__device__ __forceinline__ int tile_sum(const TileRegs& r, int nblk, const uint32_t (&creg)[8]) {
    int acc = 0;
    if (nblk == 2) {
        word2<BASE>(acc, r.a0.x, r.b0.x, creg[0]);
        word2<BASE>(acc, r.a0.y, r.b0.y, creg[1]);
        word2<BASE>(acc, r.a0.z, r.b0.z, creg[2]);
        word2<BASE>(acc, r.a0.w, r.b0.w, creg[3]);
        word2<BASE>(acc, r.a1.x, r.b1.x, creg[4]);
        word2<BASE>(acc, r.a1.y, r.b1.y, creg[5]);
        word2<BASE>(acc, r.a1.z, r.b1.z, creg[6]);
        word2<BASE>(acc, r.a1.w, r.b1.w, creg[7]);
    } else {
        word1<BASE>(acc, r.a0.x, creg[0]);
        word1<BASE>(acc, r.a0.y, creg[1]);
        word1<BASE>(acc, r.a0.z, creg[2]);
        word1<BASE>(acc, r.a0.w, creg[3]);
        word1<BASE>(acc, r.a1.x, creg[4]);
        word1<BASE>(acc, r.a1.y, creg[5]);
        word1<BASE>(acc, r.a1.z, creg[6]);
        word1<BASE>(acc, r.a1.w, creg[7]);
    }
    return acc;
}

__device__ __forceinline__ void load_tile(TileRegs& r, const uint4* wa, const uint4* wb, int nblk, int t, int lane) {
    const uint4* pa = wa + t * 64 + lane;
    r.a0 = ldg_stream(pa);
    r.a1 = ldg_stream(pa + 32);
    if (nblk == 2) {
        const uint4* pb = wb + t * 64 + lane;
        r.b0 = ldg_stream(pb);
        r.b1 = ldg_stream(pb + 32);
    }
}

// What a warp needs of the current item while it streams, boiled down to a few registers.
struct ItemRegs {
    const uint4* wa;  // block A, tile 0 of the item, this lane
    const uint4* wb;  // block B, likewise
    int32_t* out;     // result of the lane's row in tile 0 of the item
    int rows_left;    // rows of the matrix from that row on (<= 0: the lane's rows do not exist)
    int ntiles, nblk;
};

// Loads the tile this warp will need after tile `t` of the current item (iteration index i): tile t_next of the same
// item, or else the warp's first tile of the next item, whose descriptor is already in shared memory. `tag` receives
// the iteration index of the item the tile belongs to, or -1 if there is no such tile yet.
__device__ __forceinline__ void preload(TileRegs& r, int& tag, int i, int t_next, const ItemRegs& item, const GemvItem* s_items,
                                        const int* s_idx, int n_items, int warp, int lane) {
    if (t_next < item.ntiles) {
        load_tile(r, item.wa, item.wb, item.nblk, t_next, 0);
        tag = i;
    } else {
        const int nx = (i + 1) & 3;
        if (s_idx[nx] < n_items && warp < s_items[nx].ntiles) {
            load_tile(r, s_items[nx].wa, s_items[nx].wb, s_items[nx].nblk, warp, lane);
            tag = i + 1;
        } else {
            tag = -1;
        }
    }
}

// Five int8 activations of a table column, packed into two registers while they wait for their item.
struct PackedActs {
    uint32_t lo, hi;
};
__device__ __forceinline__ PackedActs pack_acts(const int a[5]) {
    PackedActs p;
    p.lo = (a[0] & 0xFF) | ((a[1] & 0xFF) << 8) | ((a[2] & 0xFF) << 16) | (static_cast<uint32_t>(a[3]) << 24);
    p.hi = static_cast<uint32_t>(a[4]);
    return p;
}
__device__ __forceinline__ void unpack_acts(const PackedActs& p, int a[5]) {
    a[0] = static_cast<int8_t>(p.lo & 0xFF);
    a[1] = static_cast<int8_t>((p.lo >> 8) & 0xFF);
    a[2] = static_cast<int8_t>((p.lo >> 16) & 0xFF);
    a[3] = static_cast<int>(p.lo) >> 24;
    a[4] = static_cast<int>(p.hi);
}

// Persistent kernel. Neither the fetch of work nor the weight stream waits on global memory between two items:
//  * while item i streams, the index of item i + 3 is being fetched from the counter, the descriptor of item i + 2 is
//    being copied into shared memory (cp.async) and the activations of item i + 1 are being loaded into registers;
//  * every warp loads its next row tile one tile ahead, and at the end of an item that next tile is the warp's first
//    tile of item i + 1, which is therefore already on its way while the table of item i + 1 is built.
//
// BASE is the shared-window address of the kernel's dynamic shared memory. It is a property of the toolchain and
// driver, not of the launch, so the host measures it once with smem_base_kernel and picks the matching instantiation;
// the kernel checks it and reports a mismatch through counters[2] instead of computing with a wrong table.
template <uint32_t BASE>
__global__ void __launch_bounds__(kGemvThreads, kCtasPerSm)
gemv_lut_kernel(const GemvItem* __restrict__ items, int n_items, const int8_t* __restrict__ act_base, int32_t* __restrict__ out_base,
                unsigned int* __restrict__ counters) {
    extern __shared__ __align__(1024) int tab[];
    GemvItem* s_items = reinterpret_cast<GemvItem*>(reinterpret_cast<char*>(tab) + kTableBytes);
    int* s_idx = reinterpret_cast<int*>(reinterpret_cast<char*>(tab) + kTableBytes + 4 * sizeof(GemvItem));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (static_cast<uint32_t>(__cvta_generic_to_shared(tab)) != BASE) {
        if (tid == 0) atomicExch(&counters[2], 1u);
        return;
    }

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
        // Opaque to the optimiser: otherwise it recomputes these words from `lane` at every use (about one extra
        // instruction per lookup) instead of keeping eight registers.
        asm volatile("mov.b32 %0, %1;" : "=r"(creg[q]) : "r"(v));
    }

    // Prologue: indices of the first three items, descriptors of the first two, activations of the first.
    if (tid < 3) s_idx[tid] = static_cast<int>(atomicAdd(&counters[0], 1u));
    __syncthreads();
    if (tid < 8) {
        const int k = tid >> 2, idx = s_idx[k];
        if (idx < n_items) reinterpret_cast<uint4*>(&s_items[k])[tid & 3] = reinterpret_cast<const uint4*>(items + idx)[tid & 3];
    }
    __syncthreads();
    PackedActs acts_cur{0, 0};
    if (s_idx[0] < n_items) {
        int a[5];
        load_column_acts(a, act_base + s_items[0].act_off, s_items[0].cols, s_items[0].col0, s_items[0].nblk, tid);
        acts_cur = pack_acts(a);
    }

    TileRegs ra, rb;     // ping-pong: the tile being looked up and the tile on its way
    int tag_a = -1, tag_b;

    for (int i = 0;; ++i) {
        const int cur = i & 3;
        if (s_idx[cur] >= n_items) break;
        ItemRegs item;  // a register copy: the loops must not re-read the descriptor from shared memory
        {
            const GemvItem& d = s_items[cur];
            item.wa = d.wa + lane;
            item.wb = d.wb + lane;
            item.out = out_base + d.out_off + d.tile0 * kTileRows + lane;
            item.rows_left = d.rows - d.tile0 * kTileRows - lane;
            item.ntiles = d.ntiles;
            item.nblk = d.nblk;
        }
        // The warp's first tile of this item is normally on its way already (loaded at the end of the previous item);
        // it is fetched here only at the very start or after items too small to give this warp a tile.
        if (tag_a < 0) preload(ra, tag_a, i, warp, item, s_items, s_idx, n_items, warp, lane);
        // index of item i + 3 (kept in a register until the end of the iteration so that nothing waits on it here)
        unsigned int fetched = 0;
        if (tid == 0) fetched = atomicAdd(&counters[0], 1u);
        // descriptor of item i + 2
        const int idx2 = s_idx[(i + 2) & 3];
        if (tid < 4 && idx2 < n_items) {
            const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(reinterpret_cast<uint4*>(&s_items[(i + 2) & 3]) + tid));
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(reinterpret_cast<const uint4*>(items + idx2) + tid) : "memory");
        }
        // activations of item i + 1
        PackedActs acts_next{0, 0};
        {
            const int nxt = (i + 1) & 3;
            if (s_idx[nxt] < n_items) {
                int a[5];
                load_column_acts(a, act_base + s_items[nxt].act_off, s_items[nxt].cols, s_items[nxt].col0, s_items[nxt].nblk, tid);
                acts_next = pack_acts(a);
            }
        }
        {
            int a[5];
            unpack_acts(acts_cur, a);
            fill_table(tab, a, tid);
        }
        __syncthreads();

        int t = warp;
        while (tag_a == i) {
            preload(rb, tag_b, i, t + kGemvWarps, item, s_items, s_idx, n_items, warp, lane);
            {
                const int acc = tile_sum<BASE>(ra, item.nblk, creg);
                if (t * kTileRows < item.rows_left) atomicAdd(item.out + t * kTileRows, acc);
            }
            t += kGemvWarps;
            if (tag_b != i) {  // rb holds a tile of the next item (or nothing): hand it over and leave
                ra = rb;
                tag_a = tag_b;
                break;
            }
            preload(ra, tag_a, i, t + kGemvWarps, item, s_items, s_idx, n_items, warp, lane);
            {
                const int acc = tile_sum<BASE>(rb, item.nblk, creg);
                if (t * kTileRows < item.rows_left) atomicAdd(item.out + t * kTileRows, acc);
            }
            t += kGemvWarps;
        }
        if (tid == 0) s_idx[(i + 3) & 3] = static_cast<int>(fetched);
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();  // the table, s_idx and s_items are rewritten next
        acts_cur = acts_next;
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

// Reports the shared-window address of dynamic shared memory for a kernel without static shared memory.
__global__ void smem_base_kernel(unsigned int* out) {
    extern __shared__ __align__(1024) int tab[];
    if (threadIdx.x == 0) out[0] = static_cast<unsigned int>(__cvta_generic_to_shared(tab));
}

}  // namespace qtb
