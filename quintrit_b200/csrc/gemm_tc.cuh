// Batched projection on the 5th-generation tensor cores: out[b][n] = sum_k trit[n][k] * act[b][k] for a batch of int8 activation
// vectors (prompt ingestion, batched decoding), the same integers as the batch-1 kernel of gemv_lut.cuh gives vector by vector.
//
// The reference has no batched path: its CPU runtime and its GPU decoder run a prompt token by token (quintrit-runtime/src/engine.rs
// forward_token, quintrit-runtime/src/gpu.rs:459-493), each token with its own activation scale. What is restated is the projection's
// definition (quintrit-runtime/src/layer.rs:123-177: the exact int32 sum, scaled afterwards), so a batch of B tokens gives B results
// that are bit-identical to B single-token projections.
//
// Shape on a B200. The weights stay velurex bytes in HBM (0.2 bytes per weight) and are decoded into int8 trits on the way into shared
// memory; the product runs as tcgen05.mma.kind::i8 with the accumulator in tensor memory:
//   * a CTA owns 128 weight rows (the M of the instruction) and a range of 160-trit blocks (K); the batch is the N (16..256);
//   * warps 2..9 decode: a thread loads half of a row's 32 bytes of a block (16-byte loads, contiguous over the warp thanks
//     to the block-major copy of the weights described below), looks every byte up in a 256-entry table of its five trits (16 copies, one per bank pair), transposes
//     by byte permutes and stores five 128 x 32 int8 tiles (one per plane of the block) in the K-major layout without swizzle that
//     the instruction reads (8-row x 16-byte core matrices; leading-dimension offset 128 bytes, stride offset 256 bytes);
//   * one thread of warp 0 fetches the matching five 32-byte-wide slices of the activation matrix with TMA (cp.async.bulk.tensor,
//     32-byte swizzle, completion on an mbarrier): plane p of block g multiplies the columns g * 160 + p * 32 .. + 31, which are
//     contiguous in an activation vector, so a slice is a plain 2-D box;
//   * one thread of warp 1 issues five MMAs (128 x N x 32) per block into one accumulator of N tensor-memory columns and releases
//     the stage with tcgen05.commit; a ring of 3 or 4 stages keeps decode, TMA and the tensor pipe overlapped;
//   * the kernel is persistent: a CTA takes items (row tile, K part) round-robin, with two accumulators in tensor memory so that the MMAs of
//     the next item start while the previous one is written out;
//   * at the end of an item the decode warps read the accumulator with tcgen05.ld (a row per thread, the column chunks shared between the two warps of a lane quarter) and write out[b][row] (plain stores, or
//     red.global.add when K was split over several CTAs so that matrices with few rows still fill the chip).
// Every wait on an mbarrier is bounded: after `spin_limit` polls the thread raises an abort flag that the other roles see, the kernel
// sets its status word, waits (bounded) for its own copies in flight, frees its tensor memory and returns.
//
// Weight copy for this kernel ("block-major planar"): byte j of block g of row r at (g * rows_padded + r) * 32 + j, rows padded to
// 128 with byte 125 (five zero trits). Made on the device from the stream layout the first time a matrix is used here.
#pragma once
#include <cstdint>

#include <cuda.h>
#include <cuda_runtime.h>

#include "gemv_lut.cuh"

namespace qtb {

constexpr int kGemmM = 128;
constexpr int kGemmDecodeWarps = 8;
constexpr int kGemmThreads = 64 + 32 * kGemmDecodeWarps;
constexpr int kGemmMaxStages = 4;
constexpr int kGemmMaxN = 256;
constexpr int kGemmAStage = 5 * kGemmM * 32;  // five plane tiles of 128 rows x 32 bytes
constexpr int kGemmLutBytes = 256 * 16 * 8;  // 16 copies of the trit table, one per pair of shared-memory banks: lookups never collide
constexpr unsigned int kGemmStatusTimeout = 4;

struct GemmArgs {
    const uint8_t* w;      // block-major planar weights
    int32_t* out;          // [batch][rows]
    unsigned int* status;  // set to kGemmStatusTimeout when a wait ran out
    int rows, rows_padded, blocks;
    int n;                 // instruction N: the batch rounded up to a multiple of 16
    int batch;             // activation vectors actually present (columns of the accumulator that are written out)
    int blocks_per_cta;    // blocks of one work item (a row tile x a K part); parts of a tile add their results with red.global.add
    int stages;
    unsigned int spin_limit;
};

inline size_t gemm_smem_bytes(int n, int stages) {
    return size_t(stages) * (kGemmAStage + size_t(n) * 160) + kGemmLutBytes + 256 + 1024;  // + barriers + alignment slack
}

// stream layout -> block-major planar (see the top of this file and of gemv_lut.cuh)
__global__ void stream_to_block_major_kernel(const uint4* __restrict__ stream, uint8_t* __restrict__ out, size_t rows, size_t rows_padded, size_t blocks, size_t tiles) {
    const size_t total = blocks * rows_padded * 2;  // 16-byte pieces
    const uint8_t* s = reinterpret_cast<const uint8_t*>(stream);
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
        const size_t g = i / (rows_padded * 2), rem = i % (rows_padded * 2), r = rem / 2, c = rem % 2;
        uint8_t piece[16];
        if (r < rows) {
            const size_t t = r / 32, l = r % 32;
            for (int k = 0; k < 16; ++k) {
                const size_t j = c * 16 + k, q = (j + 32 - l) % 32;  // planar byte j sits at position q of the rotated row
                piece[k] = s[((g * tiles + t) * 2 + q / 16) * 512 + l * 16 + q % 16];
            }
        } else {
            for (int k = 0; k < 16; ++k) piece[k] = 125;
        }
        *reinterpret_cast<uint4*>(out + (g * rows_padded + r) * 32 + c * 16) = *reinterpret_cast<const uint4*>(piece);
    }
}

// int8 activation vectors [batch][cols] -> the zero-padded matrix [n][blocks * 160] the TMA reads
__global__ void gemm_pad_activations_kernel(const int8_t* __restrict__ act, int8_t* __restrict__ padded, int batch, int n, int cols, int k_pad) {
    const size_t total = size_t(n) * k_pad;
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
        const int b = static_cast<int>(i / k_pad), c = static_cast<int>(i % k_pad);
        padded[i] = (b < batch && c < cols) ? act[size_t(b) * cols + c] : int8_t(0);
    }
}

namespace gemm_detail {

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
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(map), "r"(x), "r"(y),
                 "r"(bar)
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
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

}  // namespace gemm_detail

__global__ void __launch_bounds__(kGemmThreads, 1) gemm_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap act_map, GemmArgs a) {
    using namespace gemm_detail;
    extern __shared__ unsigned char gemm_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023) & ~uintptr_t(1023));
    const int S = a.stages, n = a.n;
    unsigned char* a_tiles = smem;                                      // S stages of five 4096-byte tiles
    unsigned char* b_tiles = smem + size_t(S) * kGemmAStage;            // S stages of five n * 32-byte tiles
    uint2* lut = reinterpret_cast<uint2*>(b_tiles + size_t(S) * n * 160);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(lut) + kGemmLutBytes);
    // barriers: full_a[S], full_b[S], empty[S] of the stage ring; acc_full[2], acc_empty[2] of the two accumulators in tensor memory
    const uint32_t bar0 = smem_u32(bars);
    auto full_a = [&](int s) { return bar0 + 8u * s; };
    auto full_b = [&](int s) { return bar0 + 8u * (kGemmMaxStages + s); };
    auto empty = [&](int s) { return bar0 + 8u * (2 * kGemmMaxStages + s); };
    auto acc_full = [&](int b) { return bar0 + 8u * (3 * kGemmMaxStages + b); };
    auto acc_empty = [&](int b) { return bar0 + 8u * (3 * kGemmMaxStages + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 3 * kGemmMaxStages + 4);
    volatile unsigned int* abort_flag = reinterpret_cast<volatile unsigned int*>(bars + 3 * kGemmMaxStages + 5);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // work items: (row tile, K part), taken round-robin by the CTAs; an item is `per` blocks of one tile
    const int per = a.blocks_per_cta, parts = (a.blocks + per - 1) / per, items = (a.rows_padded / kGemmM) * parts;
    uint32_t tmem_cols = 32;
    while (tmem_cols < 2u * static_cast<uint32_t>(n)) tmem_cols <<= 1;  // two accumulators of n columns

    // ---- set-up: trit table, barriers, tensor memory ----
    for (int v = tid; v < 256; v += kGemmThreads) {
        uint32_t lo = 0, hi = 0;
        if (v <= 250) {
            const int d4 = v / 84, r4 = v - 84 * d4, d3 = r4 / 28, r3 = r4 - 28 * d3, d2 = r3 / 9, r2 = r3 - 9 * d2, d1 = r2 / 3, d0 = r2 - 3 * d1;
            if (d0 <= 2 && d1 <= 2 && d2 <= 2 && d3 <= 2 && d4 <= 2) {
                lo = uint32_t(uint8_t(d0 - 1)) | (uint32_t(uint8_t(d1 - 1)) << 8) | (uint32_t(uint8_t(d2 - 1)) << 16) | (uint32_t(uint8_t(d3 - 1)) << 24);
                hi = uint32_t(uint8_t(d4 - 1));
            }
        }
        for (int copy = 0; copy < 16; ++copy) lut[v * 16 + copy] = make_uint2(lo, hi);  // entry v of copy c at v * 128 + c * 8
    }
    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full_a(s), kGemmDecodeWarps);  // one arrival per decode warp
            mbar_init(full_b(s), 1);                 // the TMA thread's expect_tx arrival
            mbar_init(empty(s), 1);                  // tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);                   // tcgen05.commit after the last MMA of an item
            mbar_init(acc_empty(b), kGemmDecodeWarps);   // every epilogue warp has read its part
        }
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

    if (warp == 0) {
        // ---- activations: five TMA boxes of 32 bytes x n rows per block ----
        if (lane == 0) {
            int it = 0, s = 0;
            uint32_t ph = 0;  // stage and phase of the ring, advanced by hand (S is a run-time value)
            bool okay = true;
            const uint32_t b_base = smem_u32(b_tiles);
            for (int item = blockIdx.x; item < items && okay; item += gridDim.x) {
                const int kb0 = (item % parts) * per, nkb = min(per, a.blocks - kb0);
                for (int k = 0; k < nkb; ++k, ++it) {
                    if (!(okay = mbar_wait(empty(s), ph ^ 1, abort_flag, a.spin_limit))) break;
                    mbar_expect_tx(full_b(s), 5u * n * 32u);
                    const uint32_t dst = b_base + s * n * 160;
                    for (int p = 0; p < 5; ++p) tma_load_2d(dst + p * n * 32, &act_map, (kb0 + k) * 160 + p * 32, 0, full_b(s));
                    if (++s == S) s = 0, ph ^= 1;
                }
            }
            // its own copies in flight land before the CTA leaves: the last min(it, S) uses of the ring, newest first
            for (int back = 0; back < min(it, S); ++back) {
                if (--s < 0) s = S - 1, ph ^= 1;
                mbar_wait(full_b(s), ph, abort_flag, a.spin_limit, false);
            }
        }
    } else if (warp == 1) {
        // ---- tensor cores: five MMAs per block, all issued by one thread ----
        if (lane == 0) {
            const uint32_t idesc = instr_desc_i8(kGemmM, n);
            int j = 0, s = 0;
            uint32_t ph = 0;
            bool okay = true;
            const uint32_t a_tiles_u32 = smem_u32(a_tiles), b_tiles_u32 = smem_u32(b_tiles);
            for (int item = blockIdx.x; item < items && okay; item += gridDim.x, ++j) {
                const int kb0 = (item % parts) * per, nkb = min(per, a.blocks - kb0), buf = j & 1;
                if (!(okay = mbar_wait(acc_empty(buf), ((j >> 1) & 1) ^ 1, abort_flag, a.spin_limit))) break;  // the epilogue has drained this accumulator
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + uint32_t(buf * n);
                for (int k = 0; k < nkb; ++k) {
                    if (!(okay = mbar_wait(full_a(s), ph, abort_flag, a.spin_limit) && mbar_wait(full_b(s), ph, abort_flag, a.spin_limit))) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_base = a_tiles_u32 + s * kGemmAStage, b_base = b_tiles_u32 + s * n * 160;
                    for (int p = 0; p < 5; ++p)
                        mma_i8(tmem_d, smem_desc(a_base + p * 4096, 128, 256, 0), smem_desc(b_base + p * n * 32, 16, 256, 6), idesc, (k | p) != 0 ? 1u : 0u);
                    mma_commit(empty(s));
                    if (++s == S) s = 0, ph ^= 1;
                }
                mma_commit(acc_full(buf));  // arrives when every MMA issued so far has finished (also on the way out after a failed wait)
            }
        }
    } else {
        // ---- decode warps: half a weight row (16 bytes of a block) per thread ----
        // Thread d of the 256: lanes 0..7 of every group of 16 take the first halves of 8 consecutive rows, lanes 8..15 the second halves, so a
        // warp reads 512 contiguous bytes and its 16-byte stores fall on 128 contiguous bytes per quarter-warp.
        const int d = tid - 64;
        const int r = (d & 7) + 8 * (d >> 4), c = (d >> 3) & 1;
        const uint32_t lut_base = smem_u32(lut) + (lane & 15) * 8;  // this lane's copy of the table (a 64-bit load serves 16 lanes per cycle)
        const uint32_t row_off = (r >> 3) * 256 + c * 128 + (r & 7) * 16;
        const int quarter = warp & 3;  // a warp reads the 32 lanes of tensor memory that its index modulo 4 selects
        bool okay = true;
        int j = 0, s = 0;
        uint32_t ph = 0;
        const uint32_t a_tiles_u32 = smem_u32(a_tiles) + row_off;
        const size_t block_pitch = size_t(a.rows_padded) * 32;
        for (int item = blockIdx.x; item < items && okay; item += gridDim.x, ++j) {
            const int row0 = (item / parts) * kGemmM, kb0 = (item % parts) * per, nkb = min(per, a.blocks - kb0), buf = j & 1;
            const uint8_t* src = a.w + (size_t(kb0) * a.rows_padded + row0 + r) * 32 + c * 16;
            uint4 next = __ldg(reinterpret_cast<const uint4*>(src));
            for (int k = 0; k < nkb && okay; ++k) {
                const uint4 cur = next;
                src += block_pitch;
                if (k + 1 < nkb) next = __ldg(reinterpret_cast<const uint4*>(src));
                const uint32_t words[4] = {cur.x, cur.y, cur.z, cur.w};
                uint32_t plane[5][4];
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) {
                    uint2 e[4];
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint32_t addr = lut_base + (((words[wi] >> (8 * kk)) & 0xffu) << 7);
                        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(e[kk].x), "=r"(e[kk].y) : "r"(addr));
                    }
                    const uint32_t t01l = prmt(e[0].x, e[1].x, 0x5140), t01h = prmt(e[0].x, e[1].x, 0x7362);
                    const uint32_t t23l = prmt(e[2].x, e[3].x, 0x5140), t23h = prmt(e[2].x, e[3].x, 0x7362);
                    plane[0][wi] = prmt(t01l, t23l, 0x5410);
                    plane[1][wi] = prmt(t01l, t23l, 0x7632);
                    plane[2][wi] = prmt(t01h, t23h, 0x5410);
                    plane[3][wi] = prmt(t01h, t23h, 0x7632);
                    plane[4][wi] = prmt(prmt(e[0].y, e[1].y, 0x0040), prmt(e[2].y, e[3].y, 0x0040), 0x5410);
                }
                // the trits are ready; now the stage must be free
                if (lane == 0) okay = mbar_wait(empty(s), ph ^ 1, abort_flag, a.spin_limit);
                okay = __shfl_sync(0xffffffffu, okay ? 1 : 0, 0) != 0;
                if (!okay) break;
                const uint32_t tile = a_tiles_u32 + s * kGemmAStage;
#pragma unroll
                for (int p = 0; p < 5; ++p)
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(tile + p * 4096), "r"(plane[p][0]), "r"(plane[p][1]), "r"(plane[p][2]), "r"(plane[p][3]) : "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the stores above are read by the tensor cores (async proxy)
                __syncwarp();
                if (lane == 0) mbar_arrive(full_a(s));
                if (++s == S) s = 0, ph ^= 1;
            }
            if (!okay) break;
            // ---- epilogue of the item: accumulator row -> out[b][row] (the tensor pipe works on while the next item is decoded) ----
            if (lane == 0) okay = mbar_wait(acc_full(buf), (j >> 1) & 1, abort_flag, a.spin_limit);
            okay = __shfl_sync(0xffffffffu, okay ? 1 : 0, 0) != 0;
            if (!okay) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = row0 + quarter * 32 + lane;
            for (int c0 = ((warp - 2) >> 2) * 16; c0 < n; c0 += 16 * (kGemmDecodeWarps / 4)) {  // the warps that share a quarter alternate over the column chunks
                uint32_t v[16];
                const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(buf * n + c0);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]),
                      "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < a.rows) {
                    int32_t* dst = a.out + size_t(c0) * a.rows + row;
                    const int valid = min(16, a.batch - c0);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        if (i < valid) {
                            if (parts == 1) *dst = static_cast<int32_t>(v[i]);
                            else atomicAdd(dst, static_cast<int32_t>(v[i]));
                        }
                        dst += a.rows;
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(buf));
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
