// Batched projection on the 5th-generation tensor cores: out[b][n] = sum_k trit[n][k] * act[b][k] for a batch of int8 activation
// vectors (prompt ingestion, batched decoding), the same integers as the batch-1 kernel of gemv_lut.cuh gives vector by vector.
//
// The reference has no batched path: its CPU runtime and its GPU decoder run a prompt token by token (quintrit-runtime/src/engine.rs
// forward_token, quintrit-runtime/src/gpu.rs:459-493), each token with its own activation scale. What is restated is the projection's
// definition (quintrit-runtime/src/layer.rs:123-177: the exact int32 sum, scaled afterwards), so a batch of B tokens gives B results
// that are bit-identical to B single-token projections.
//
// Shape on a B200. The batch-1 kernel streams velurex bytes (0.2 bytes per weight); turning those into int8 operands costs a table lookup and
// a byte transposition per weight byte, which would leave the tensor pipe waiting. This kernel therefore reads its own copy of the weights,
// made on the device the first time a matrix is used here: two bits per trit (0.25 bytes per weight), four consecutive columns per byte, so
// that one lookup turns a byte into four int8 operands that are already in K order. The product runs as tcgen05.mma.kind::i8 with the
// accumulator in tensor memory:
//   * a work item is 128 weight rows (the M of the instruction) times a range of 128-column blocks (K); the batch is the N (16..256);
//   * warps 2..17 decode, in four groups that take the blocks round-robin: a thread takes a row's 32 bytes of a block from shared memory,
//     looks every byte up in a 256-entry table of int8x4 words (32 copies, one per shared-memory bank, so lookups never collide) and
//     writes the row's 128 int8 operands into its lane of TENSOR MEMORY with tcgen05.st (32 columns a group). Operands that threads
//     store to shared memory need a proxy fence before the tensor cores may read them, and that fence was measured at more than a
//     thousand cycles a block; operands in tensor memory need none;
//   * two loader threads (warp 0 and the last warp) fetch, per block, the tile's 4096 weight bytes (one bulk copy) and the matching four
//     32-byte-wide slices of the activation matrix (one 3-D TMA box, 32-byte swizzle, in place from the caller's vectors where their
//     pitch allows it), both completing on one mbarrier;
//   * one thread of warp 1 issues four MMAs (128 x N x 32, A from tensor memory, B from shared memory) per block and releases the stage
//     and the group's operand columns with tcgen05.commit; a ring of 3 to 8 stages (as many as fit beside the batch) keeps the loads ahead;
//   * the kernel is persistent: a CTA takes items round-robin;
//   * at the end of an item the decode warps read the accumulator with tcgen05.ld (a row per thread, the column chunks shared between the
//     four warps of a lane quarter) and write out[b][row] (when K was split over several items, so that matrices with few rows still fill
//     the chip, each part writes its partial sums and a small second kernel adds the parts: exact integers in any order).
// Every wait on an mbarrier is bounded: after `spin_limit` polls the thread raises an abort flag that the other roles see, the kernel
// sets its status word, waits (bounded) for its own copies in flight, frees its tensor memory and returns.
//
// Weight copy ("two-bit block-major"): byte j of block g of row r at (g * rows_padded + r) * 32 + j holds the columns g * 128 + 4 j + i,
// i = 0..3, as (trit + 1) << 2 i; rows are padded to 128 and columns to whole blocks with code 1 (trit 0).
#pragma once
#include <cstdint>

#include <cuda.h>
#include <cuda_runtime.h>

#include "gemv_lut.cuh"

namespace qtb {

constexpr int kGemmM = 128;
constexpr int kGemmDecodeWarps = 16;
constexpr int kGemmGroups = 4;  // the decode warps work in groups of four; group g decodes the blocks it, it + 4, ... of the CTA's sequence on its own
constexpr int kGemmThreads = 64 + 32 * kGemmDecodeWarps + 32;  // weight loader warp, MMA warp, decode warps, activation loader warp
constexpr int kGemmMaxStages = 8;
constexpr int kGemmMaxN = 256;  // 256 accumulator columns + 4 x 32 operand columns fit the 512 columns of tensor memory
constexpr int kGemmBlockCols = 128;           // columns (K) of one block of the two-bit copy: 32 bytes a row
constexpr int kGemmLutBytes = 256 * 32 * 4;  // 32 copies of the byte -> int8x4 table, one per shared-memory bank: lookups never collide
constexpr unsigned int kGemmStatusTimeout = 4;

struct GemmArgs {
    const uint8_t* w;      // two-bit block-major weights
    int32_t* out;          // [batch][rows]; with K split over several items: the partial sums [part][batch][rows] that gemm_reduce_parts_kernel adds up
    unsigned int* status;  // set to kGemmStatusTimeout when a wait ran out
    int rows, rows_padded, blocks;
    int ldo;               // elements between the results of consecutive vectors in `out` (rows, or more when the results go into a wider row)
    int n;                 // instruction N: the batch rounded up to a multiple of 16
    int batch;             // activation vectors actually present (columns of the accumulator that are written out)
    int blocks_per_cta;    // blocks of one work item (a row tile x a K part)
    int stages;
    unsigned int spin_limit;
};

// Stages that fit the shared memory of an SM for a batch of n: as many as possible (at most kGemmMaxStages), because the blocks in flight have to
// cover the latency of the weight bytes from HBM.
inline int gemm_stages_for(int n, size_t smem_limit) {
    const size_t fixed = kGemmLutBytes + 256 + 1024, stage = size_t(n) * kGemmBlockCols + kGemmM * 32;
    const size_t fit = smem_limit > fixed ? (smem_limit - fixed) / stage : 0;
    return static_cast<int>(fit < size_t(kGemmMaxStages) ? fit : size_t(kGemmMaxStages));
}
inline size_t gemm_smem_bytes(int n, int stages) {
    return size_t(stages) * (size_t(n) * kGemmBlockCols + kGemmM * 32) + kGemmLutBytes + 256 + 1024;  // + barriers + alignment slack
}

// stream layout (gemv_lut.cuh) -> two-bit block-major; `blocks` counts 128-column blocks here, `vblocks` the 160-trit velurex blocks of a row
// The copy may be one of several matrices stacked row-wise into one (q | k | v, gate | up): its rows start at row_off of rows_total.
__global__ void stream_to_two_bit_kernel(const uint4* __restrict__ stream, uint8_t* __restrict__ out, size_t rows, size_t cols, size_t rows_padded, size_t blocks, size_t vblocks,
                                         size_t tiles, size_t row_off, size_t rows_total) {
    const size_t total = blocks * rows_padded * 32;
    const uint8_t* s = reinterpret_cast<const uint8_t*>(stream);
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
        const size_t g = i / (rows_padded * 32), rem = i % (rows_padded * 32), r = rem / 32, j = rem % 32;
        unsigned int byte = 0;
        for (int q = 0; q < 4; ++q) {
            const size_t col = g * 128 + j * 4 + q;
            unsigned int code = 1;  // trit 0 beyond the matrix
            if (r < rows && col < cols) {
                const size_t vb = col / 160, p = (col % 160) / 32, jj = col % 32, t = r / 32, l = r % 32, pos = (jj + 32 - l) % 32;  // planar byte jj sits at position pos of the rotated row
                const unsigned int v = s[((vb * tiles + t) * 2 + pos / 16) * 512 + l * 16 + pos % 16];
                const unsigned int d4 = v / 84, r4 = v - 84 * d4, d3 = r4 / 28, r3 = r4 - 28 * d3, d2 = r3 / 9, r2 = r3 - 9 * d2, d1 = r2 / 3, d0 = r2 - 3 * d1;
                const unsigned int digits[5] = {d0, d1, d2, d3, d4};
                code = v <= 250 ? digits[p] : 1;
            }
            byte |= code << (2 * q);
        }
        out[(g * rows_total + row_off + r) * 32 + j] = static_cast<uint8_t>(byte);
    }
}

// out[i] = sum over the K parts of partial[part][i] (i over batch * rows): the second step of a projection whose K was split over several items
// (partial rows are dense, `rows` apart; the results of a vector are `ldo` apart in out)
__global__ void gemm_reduce_parts_kernel(const int32_t* __restrict__ partial, int32_t* __restrict__ out, size_t count, int parts, int rows, int ldo) {
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < count; i += size_t(gridDim.x) * blockDim.x) {
        int32_t sum = 0;
        for (int p = 0; p < parts; ++p) sum += partial[size_t(p) * count + i];
        out[(i / rows) * ldo + i % rows] = sum;
    }
}

// int8 activation vectors [batch][cols] -> the zero-padded matrix [n][blocks * 128] the TMA reads
__global__ void gemm_pad_activations_kernel(const int8_t* __restrict__ act, int8_t* __restrict__ padded, int batch, int n, int cols, int k_pad) {
    const size_t total = size_t(n) * k_pad;
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
        const int b = static_cast<int>(i / k_pad), c = static_cast<int>(i % k_pad);
        padded[i] = (b < batch && c < cols) ? act[size_t(b) * cols + c] : int8_t(0);
    }
}

namespace gemm_detail {

#ifdef QTB_GEMM_TRACE
// Debug build only: cycle stamps of CTA 0, role `who` (0 loader, 1 MMA thread, 2 decode warp 0), event `ev`, block `k` < 16, at status + 64 + ...
#define QTB_GEMM_STAMP(who, ev, k)                                                                                              \
    do {                                                                                                                        \
        if (blockIdx.x == 0 && (k) < 16) reinterpret_cast<long long*>(a.status + 64)[((who) * 4 + (ev)) * 16 + (k)] = clock64(); \
    } while (0)
#else
#define QTB_GEMM_STAMP(who, ev, k) do { } while (0)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"  // the last operand: how long the hardware may park the thread per try
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(20000u)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out or another role already gave up (the abort flag is then set).
// `heed_abort` false: keep waiting up to the limit although another role gave up (the wait for one's own copies in flight).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile unsigned int* abort_flag, unsigned int limit, bool heed_abort = true) {
    for (unsigned int i = 0; i < limit; ++i) {
        if (mbar_try(bar, parity)) return true;
        if (heed_abort && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
// Plain bulk copy (no tensor map): `bytes` contiguous bytes, a multiple of 16, both addresses 16-byte aligned.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst), "l"(map), "r"(x), "r"(y),
                 "r"(z), "r"(bar)
                 : "memory");
}
// Shared-memory matrix descriptor of the tensor-core instruction (64 bits): start address, leading and stride byte offsets in
// 16-byte units, descriptor version 1 at bit 46, layout type in bits 61..63 (0 no swizzle, 6 32-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    return uint64_t((addr & 0x3FFFFu) >> 4) | (uint64_t(lbo_bytes >> 4) << 16) | (uint64_t(sbo_bytes >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(layout) << 61);
}
// Instruction descriptor for kind::i8: S32 accumulator (2 at bit 4), signed 8-bit A and B (1 at bits 7 and 10), both K-major,
// N / 8 at bit 17, M / 16 at bit 24.
__device__ __forceinline__ uint32_t instr_desc_i8(int m, int n) { return (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24); }
__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    const uint32_t zero = 0;  // no output lane is disabled
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(zero)
        : "memory");
}
// The same instruction with the A operand in tensor memory (128 lanes = rows, 32-bit columns of four consecutive K elements).
__device__ __forceinline__ void mma_i8_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    const uint32_t zero = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(zero)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

}  // namespace gemm_detail

__global__ void __launch_bounds__(kGemmThreads, 1) gemm_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap act_map, GemmArgs a) {
    using namespace gemm_detail;
    extern __shared__ unsigned char gemm_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023) & ~uintptr_t(1023));
    const int S = a.stages, n = a.n;
    unsigned char* b_tiles = smem;                                        // S stages of four n * 32-byte activation tiles
    unsigned char* raw_tiles = b_tiles + size_t(S) * n * kGemmBlockCols;  // S stages of the 128 x 32 weight bytes of a block, as they lie in memory
    uint32_t* lut = reinterpret_cast<uint32_t*>(raw_tiles + size_t(S) * kGemmM * 32);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(lut) + kGemmLutBytes);
    // barriers: loaded[S] (weight bytes and activations of a stage have landed), empty[S] (the MMAs that read the stage are done);
    // a_full[G], a_empty[G] (the int8 operand of group g in tensor memory is written / its MMAs are done); acc_full, acc_empty (the accumulator)
    const uint32_t bar0 = smem_u32(bars);
    auto loaded = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kGemmMaxStages + s); };
    auto a_full = [&](int g) { return bar0 + 8u * (2 * kGemmMaxStages + g); };
    auto a_empty = [&](int g) { return bar0 + 8u * (2 * kGemmMaxStages + kGemmGroups + g); };
    const uint32_t acc_full = bar0 + 8u * (2 * kGemmMaxStages + 2 * kGemmGroups), acc_empty = acc_full + 8u;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * kGemmMaxStages + 2 * kGemmGroups + 2);  // 26 barriers, then these two words
    volatile unsigned int* abort_flag = reinterpret_cast<volatile unsigned int*>(bars + 2 * kGemmMaxStages + 2 * kGemmGroups + 3);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // work items: (row tile, K part), taken round-robin by the CTAs; an item is `per` blocks of one tile
    const int per = a.blocks_per_cta, parts = (a.blocks + per - 1) / per, items = (a.rows_padded / kGemmM) * parts;
    // tensor memory: the accumulator in columns [0, n), then the int8 operand of each decode group (128 rows x 128 K = 32 columns of four bytes)
    uint32_t tmem_cols = 32;
    while (tmem_cols < static_cast<uint32_t>(n) + 32u * kGemmGroups) tmem_cols <<= 1;

    // ---- set-up: byte -> int8x4 table, barriers, tensor memory ----
    for (int v = tid; v < 256; v += kGemmThreads) {
        uint32_t word = 0;
        for (int q = 0; q < 4; ++q) {
            const int code = (v >> (2 * q)) & 3;
            word |= uint32_t(uint8_t(code == 3 ? 0 : code - 1)) << (8 * q);  // code 3 does not occur; it reads as trit 0
        }
        for (int copy = 0; copy < 32; ++copy) lut[v * 32 + ((copy + v) & 31)] = word;  // entry v of copy c at v * 128 + c * 4 (rotated fill: no bank conflicts here)
    }
    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(loaded(s), 2);  // the expect_tx arrivals of the two loader threads
            mbar_init(empty(s), 1);   // tcgen05.commit
        }
        for (int g = 0; g < kGemmGroups; ++g) {
            mbar_init(a_full(g), kGemmDecodeWarps / kGemmGroups);  // one arrival per warp of the group
            mbar_init(a_empty(g), 1);                              // tcgen05.commit
        }
        mbar_init(acc_full, 1);                  // tcgen05.commit after the last MMA of an item
        mbar_init(acc_empty, kGemmDecodeWarps);  // every epilogue warp has read its part
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t*>(tmem_slot))), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 || warp == 2 + kGemmDecodeWarps) {
        // ---- loads, by two threads so that neither's fixed cost per block bounds the pipe: warp 0 fetches the weight bytes of a block (one bulk
        // copy of the tile's 4096 bytes), the last warp its activations (one TMA box: 32 bytes x n vectors x four K tiles) ----
        if (lane == 0) {
            const bool weights = warp == 0;
            int it = 0, s = 0;
            uint32_t ph = 0;  // stage and phase of the ring, advanced by hand (S is a run-time value)
            bool okay = true;
            const uint32_t b_base = smem_u32(b_tiles), raw_base = smem_u32(raw_tiles);
            for (int item = blockIdx.x; item < items && okay; item += gridDim.x) {
                const int row0 = (item / parts) * kGemmM, kb0 = (item % parts) * per, nkb = min(per, a.blocks - kb0);
                const uint8_t* src = a.w + (size_t(kb0) * a.rows_padded + row0) * 32;
                const size_t pitch = size_t(a.rows_padded) * 32;
                for (int k = 0; k < nkb; ++k, ++it) {
                    QTB_GEMM_STAMP(0, 0, it);
                    if (!(okay = mbar_wait(empty(s), ph ^ 1, abort_flag, a.spin_limit))) break;
                    QTB_GEMM_STAMP(0, 1, it);
                    if (weights) {
                        mbar_expect_tx(loaded(s), kGemmM * 32u);
                        bulk_load(raw_base + s * (kGemmM * 32), src, kGemmM * 32, loaded(s));
                        src += pitch;
                    } else {
                        mbar_expect_tx(loaded(s), 4u * n * 32u);
                        tma_load_3d(b_base + s * n * kGemmBlockCols, &act_map, 0, 0, (kb0 + k) * 4, loaded(s));
                    }
                    QTB_GEMM_STAMP(0, 2, it);
                    if (++s == S) s = 0, ph ^= 1;
                }
            }
            // its own copies in flight land before the CTA leaves: the last min(it, S) uses of the ring, newest first
            for (int back = 0; back < min(it, S); ++back) {
                if (--s < 0) s = S - 1, ph ^= 1;
                mbar_wait(loaded(s), ph, abort_flag, a.spin_limit, false);
            }
        }
    } else if (warp == 1) {
        // ---- tensor cores: four MMAs per block (A from tensor memory, B from shared memory), all issued by one thread ----
        if (lane == 0) {
            const uint32_t idesc = instr_desc_i8(kGemmM, n);
            int j = 0, s = 0, it = 0;
            uint32_t ph = 0;
            bool okay = true;
            // descriptor of stage 0, K tile 0; a stage or a tile further on only moves the start address field (16-byte units)
            const uint64_t b_desc0 = smem_desc(smem_u32(b_tiles), 16, 256, 6);
            const uint32_t b_stage16 = uint32_t(n * kGemmBlockCols) >> 4, b_tile16 = uint32_t(n * 32) >> 4;
            for (int item = blockIdx.x; item < items && okay; item += gridDim.x, ++j) {
                const int kb0 = (item % parts) * per, nkb = min(per, a.blocks - kb0);
                if (!(okay = mbar_wait(acc_empty, (j & 1) ^ 1, abort_flag, a.spin_limit))) break;  // the epilogue of the previous item has drained the accumulator
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int k = 0; k < nkb; ++k, ++it) {
                    const int g = it & (kGemmGroups - 1);
                    QTB_GEMM_STAMP(1, 0, k + 100 * j);
                    // the group's arrival also stands for the stage's loads: the group waited for them before it decoded
                    if (!(okay = mbar_wait(a_full(g), (it / kGemmGroups) & 1, abort_flag, a.spin_limit))) break;
                    QTB_GEMM_STAMP(1, 1, k + 100 * j);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t b_desc = b_desc0 + uint64_t(s * b_stage16);
                    const uint32_t a_tmem = tmem_base + uint32_t(n + 32 * g);
#pragma unroll
                    for (int p = 0; p < 4; ++p) mma_i8_ts(tmem_base, a_tmem + 8 * p, b_desc + uint64_t(p * b_tile16), idesc, (k | p) != 0 ? 1u : 0u);
                    mma_commit(empty(s));     // the stage may be loaded again ...
                    mma_commit(a_empty(g));   // ... and the group may write its next operand, once these MMAs are done
                    QTB_GEMM_STAMP(1, 2, k + 100 * j);
                    if (++s == S) s = 0, ph ^= 1;
                }
                mma_commit(acc_full);  // arrives when every MMA issued so far has finished (also on the way out after a failed wait)
            }
        }
    } else {
        // ---- decode warps: a weight row (32 bytes of a block = 128 int8 operands) per thread, in groups of four warps ----
        // Group g takes the blocks g, g + 4, ... of the CTA's block sequence. A warp owns the 32 lanes of tensor memory that its index modulo 4
        // selects, so thread (warp, lane) takes row 32 (warp & 3) + lane of the tile and writes the row's operand into that lane with tcgen05.st:
        // no shared-memory store, so no proxy fence between the decode and the tensor cores.
        const int group = (warp - 2) >> 2, quarter = warp & 3, r = quarter * 32 + lane;
        const uint32_t* lut_lane = lut + lane;  // this lane's copy of the table: entry v at lut_lane[v * 32]
        const unsigned char* raw_mine = raw_tiles + r * 32;
        const uint32_t a_tmem = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(n + 32 * group);
        bool okay = true;
        int j = 0, it = 0, s = group % S, use = 0;  // stage and phase of this group's next block (block `group` of the sequence); its count of blocks so far
        uint32_t ph = (group / S) & 1;
        for (int item = blockIdx.x; item < items && okay; item += gridDim.x, ++j) {
            const int row0 = (item / parts) * kGemmM, nkb = min(per, a.blocks - (item % parts) * per);
            for (int k = 0; k < nkb && okay; ++k, ++it) {
                if ((it & (kGemmGroups - 1)) != group) continue;
                if (warp == 2) QTB_GEMM_STAMP(2, 0, k + 100 * j);
                // The block's bytes have landed and the MMAs of this group's previous operand are done. With fewer stages than groups a group can be a
                // whole use of the stage ahead of the loader; a parity wait only tells the last two phases apart, so the previous use is waited for first.
                if (lane == 0)
                    okay = (S >= kGemmGroups || it < S || mbar_wait(loaded(s), ph ^ 1, abort_flag, a.spin_limit)) && mbar_wait(loaded(s), ph, abort_flag, a.spin_limit) &&
                           mbar_wait(a_empty(group), (use & 1) ^ 1, abort_flag, a.spin_limit);
                okay = __shfl_sync(0xffffffffu, okay ? 1 : 0, 0) != 0;
                if (!okay) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (warp == 2) QTB_GEMM_STAMP(2, 1, k + 100 * j);
                const uint4* raw = reinterpret_cast<const uint4*>(raw_mine + s * (kGemmM * 32));
                const uint4 lo = raw[0], hi = raw[1];
                const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {  // K tile t: input words 2 t and 2 t + 1 become eight columns of four operands
                    uint32_t v[8];
#pragma unroll
                    for (int m = 0; m < 2; ++m) {
                        const uint32_t w = words[2 * t + m];
                        v[4 * m + 0] = lut_lane[(w & 0xffu) << 5];
                        v[4 * m + 1] = lut_lane[((w >> 8) & 0xffu) << 5];
                        v[4 * m + 2] = lut_lane[((w >> 16) & 0xffu) << 5];
                        v[4 * m + 3] = lut_lane[(w >> 24) << 5];
                    }
                    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(a_tmem + 8 * t), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
                                 "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                                 : "memory");
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                if (warp == 2) QTB_GEMM_STAMP(2, 2, k + 100 * j);
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(a_full(group));
                if (warp == 2) QTB_GEMM_STAMP(2, 3, k + 100 * j);
                ++use;
                s += kGemmGroups;  // this group's next block is four uses of the ring further on
                while (s >= S) s -= S, ph ^= 1;
            }
            if (!okay) break;
            // ---- epilogue of the item: accumulator row -> out[b][row] ----
            if (lane == 0) okay = mbar_wait(acc_full, j & 1, abort_flag, a.spin_limit);
            okay = __shfl_sync(0xffffffffu, okay ? 1 : 0, 0) != 0;
            if (!okay) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = row0 + r;
            for (int c0 = group * 16; c0 < n; c0 += 16 * kGemmGroups) {  // the four warps that share a lane quarter alternate over the column chunks
                uint32_t v[16];
                const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(c0);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]),
                      "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < a.rows) {
                    int32_t* dst = a.out + (size_t(item % parts) * a.batch + c0) * a.ldo + row;
                    const int valid = min(16, a.batch - c0);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        if (i < valid) *dst = static_cast<int32_t>(v[i]);
                        dst += a.ldo;
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
        }
    }
    // ---- leave: everyone is past its last use of tensor memory ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && *abort_flag) atomicExch(a.status, kGemmStatusTimeout);
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

}  // namespace qtb
