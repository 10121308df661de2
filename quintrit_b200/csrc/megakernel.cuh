// One decoded token as ONE cooperative persistent kernel (one CTA per SM), for the LLaMA / Falcon3 architecture.
//
// Why: at batch 1 a B200 streams a whole layer's weights in about 7 us, less than the cost of the 9 kernel boundaries a
// layer has when every step is a launch of its own (the reference's graph has 363 nodes per token,
// rust/crates/quintrit-runtime/src/gpu.rs:410-452). Here a layer is six phases separated by grid-wide barriers:
//   A  x += down(prev) ; RMSNorm ; int8 quantise (every CTA, redundantly) ; q|k|v GEMV (split over CTAs)
//   C  attention: RoPE of q and of the new k on the fly, KV append, one (head, KV chunk) per CTA
//   D  chunk combine + int8 quantise (every CTA) ; o GEMV
//   E  x += o ; RMSNorm ; quantise (every CTA) ; gate|up GEMV
//   F1 SwiGLU on a slice per CTA, maximum through atomicMax
//   F2 down GEMV, quantising its activations on the fly in the table fill
// and the token ends with the final norm, the output head (rows split over CTAs), the greedy choice and pos += 1.
// All arithmetic is the device functions of decode.cuh / gemv_lut.cuh, so the bits equal the per-kernel path and the
// reference CPU runtime. Every wait is bounded: a barrier that does not complete sets status and the kernel returns.
#pragma once
#include <cooperative_groups.h>

#include "decode.cuh"
#include "gemv_lut.cuh"

namespace qtb {

constexpr int kMegaThreads = 512;
constexpr int kMegaWarps = kMegaThreads / 32;
constexpr int kMegaMaxHeads = 64;
constexpr unsigned int kBarrierSpinLimit = 1u << 21;  // polls of one L2 round trip each (~0.7 us): about 1.5 s, then the kernel gives up

struct MegaLayer {
    int first[4], count[4];   // work items of the q|k|v, o, gate|up and down launches (indices into MegaArgs::items)
    const float* attn_norm;
    const float* ffn_norm;
    const float* attn_sub_norm;  // BitNet: RMSNorm of the attention output before o (q_dim weights), else nullptr
    const float* ffn_sub_norm;   // BitNet: RMSNorm of the gated activations before down (inter weights), else nullptr
    float ws[7];
    __half* kc;               // [ctx][kv_dim]
    __half* vc;
    const unsigned char* wbase[7];  // the seven weight matrices of the layer in the stream layout, for the L2 prefetches
    unsigned int wbytes[7];
};

struct MegaArgs {
    const MegaLayer* layers;
    const GemvItem* items;
    int n_layers, hidden, inter, q_heads, kv_heads, head_dim, vocab, ctx, rope_dims, f32_values;
    float eps, attn_scale;
    const __half* embed;
    const __half* lm_head;
    const float* out_norm;
    const float* cos_sin;
    float* xa;                // residual stream at layer starts
    float* xb;                // residual stream after the attention block
    int32_t *acc_qkv, *acc_o, *acc_gu, *acc_down;
    float* v_inter;           // SwiGLU output (inter)
    unsigned int* amax_bits;  // two slots, alternating by layer
    float* scores;            // [q_heads][ctx] attention scores of the current token
    float* part_acc;
    float* part_ms;
    unsigned int attn_region; // bytes of shared memory before the activation vector (mega_attn_region)
    float* logits;
    float* best_val;          // per-CTA greedy candidates
    unsigned int* best_idx;
    uint32_t* token;
    uint32_t* pos;
    uint32_t* history;
    unsigned int* bar;        // grid barrier counter, cleared by the host before every launch
    unsigned int* status;     // 0 = fine, 1 = wrong shared-memory base, 2 = a barrier timed out
    unsigned long long* trace; // optional: CTA 0 stores the global timer at every phase boundary (14 per layer + 3)
    // Tensor parallelism over tp_world GPUs (1 = none). q_heads, kv_heads, inter and vocab above are this rank's shares; the
    // vectors that every rank needs whole (o and down results, attention output, SwiGLU output) live in a "box" of which
    // every rank has one; ranks write their slices straight into the boxes of all ranks over NVLink as (value, sequence
    // number) pairs that the readers poll.
    int attn_v2;               // attention second half by (KV head, 8 coordinates) units that also combine the chunks
    float* attn_out;           // their result: the attention output before the o projection's quantiser (q_dim floats)
    // Softmax factors of the current token, computed once per (head, chunk) by the CTAs that have no values unit and read by
    // every unit of the head's group: rows of fac_stride floats, ms rows of all (head, chunk slot) first, then the vs rows;
    // one word of move flags per (head, chunk slot, group of eight positions); the maximum of every (head, chunk slot);
    // fac_done[kv head] counts the (head, chunk) tasks finished since the token began.
    float* fac;
    unsigned int* fac_flags;
    float* fac_M;
    unsigned int* fac_done;
    int fac_stride;
    int l2_prefetch;           // request the weights of later phases into L2 ahead of their streams (QUINTRIT_B200_L2_PREFETCH=0 switches it off)
    int bf16_tables;           // embedding and output head hold BF16 instead of F16 bit patterns
    int neox;                  // BitNet: RoPE pairs (i, i + rope_dims / 2) instead of (2i, 2i + 1) (config.rs:464-467)
    int relu2;                 // BitNet: relu(gate)^2 * up instead of SwiGLU (ops.rs:301-308)
    double* sumsq_part;        // BitNet FFN sub-norm: one partial sum of squares per CTA
    int tp_rank, tp_world;
    int attn_replicated;       // tensor parallelism with every head on every rank: the attention output needs no exchange
    unsigned char* tp_box[8];  // the boxes as mapped into this process, own box at [tp_rank]
    unsigned int* tp_seq;      // exchanges completed by earlier launches (the same on every rank)
    unsigned long long tp_wait_ns;  // how long a reader waits for a peer's pair before it gives up (kTpWaitLimitNs by default)
    unsigned int box_acc_o, box_acc_down, box_y, box_v, box_amax, box_best;  // byte offsets inside a box (pair buffers; box_v: plain floats)
    int q_dim_full, inter_full, vocab_base, h_slice;  // whole attention width and FFN width, first vocabulary row and hidden / world
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Optional fine-grained stamps for investigations (-DQTB_FINE_TRACE): CTA 0 stores the global timer in one of 32 extra slots
// behind the phase stamps (every layer overwrites them, so the last layer's remain). Compiled out otherwise.
#ifdef QTB_FINE_TRACE
#define QTB_FINE(a, k)                                                                         \
    do {                                                                                       \
        if ((a).trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0 && (k) < 32)           \
            (a).trace[(a).n_layers * 14 + 4 + (k)] = static_cast<unsigned long long>(clock64());  \
    } while (0)
#else
#define QTB_FINE(a, k) \
    do {               \
    } while (0)
#endif

// Grid-wide barrier with a bounded wait. Returns false (in every thread of the CTA) if it gave up or if any thread of the
// grid reported a failure. The barrier counter doubles as the failure signal: whoever gives up (here or in an exchange
// between GPUs) sets the bit kBarFail in it, which releases every waiter at once and is recognised by its size, so the
// polling loop reads one word only. Setting a bit is idempotent: however many threads report, the flag stays set (an add
// per reporting thread would wrap the word back to a legitimate count once 4 x 2^30 has been added). The host clears the
// counter before every launch; legitimate counts stay far below kBarFail, so arrivals after a failure leave the bit alone.
constexpr unsigned int kBarFail = 1u << 30;

__device__ __forceinline__ void report_failure(unsigned int* bar, unsigned int* status, unsigned int code) {
    atomicMax(status, code);
    atomicOr(bar, kBarFail);
}

// `round` counts the barriers of the launch from 1; the barrier is complete once the counter holds round * gridDim.x.
// (Spreading the arrivals over several counters of one sector, polled with two 16-byte loads, measured slower than this
// single word polled with one acquire load: about 2.0 us against 1.4 us per barrier.)
__device__ __forceinline__ bool grid_barrier(unsigned int* bar, unsigned int round, unsigned int* status, int* s_flag,
                                             unsigned int spin_limit = kBarrierSpinLimit) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(bar, 1u);
        int okay = 1;
        const unsigned int target = round * gridDim.x;
        for (unsigned int spins = 0;; ++spins) {
            unsigned int v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(bar));
            if (v >= kBarFail) {
                okay = 0;
                break;
            }
            if (v >= target) break;
            if (spins > spin_limit) {
                report_failure(bar, status, 2u);
                okay = 0;
                break;
            }
        }
        *s_flag = okay;
    }
    __syncthreads();
    return *s_flag != 0;
}

// ---- exchanges between the GPUs of a tensor-parallel group ------------------------------------------------------------
// Every exchanged 32-bit value travels as an 8-byte pair (value, sequence number of the exchange) written with one store
// into the destination rank's box; the reader polls the pair until it carries the number it waits for. An aligned 8-byte
// store arrives as a unit, so no fence and no separate flag are needed and the latency is one NVLink hop. (The same idea
// as the low-latency protocol of collective libraries.) Sequence numbers grow from launch to launch, and a buffer is
// rewritten four exchanges later at the earliest, after the writer has seen results that depend on the reader having
// finished with it.
constexpr unsigned long long kTpWaitLimitNs = 2000000000ull;  // default: a peer that does not show up within 2 s is given up on

__device__ __forceinline__ void ll_store(uint2* p, uint32_t value, uint32_t seq) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(value), "r"(seq) : "memory");
}

// Value of a pair once it carries `seq`. Bounded: after MegaArgs::tp_wait_ns the kernel's status becomes 3, the failure
// bit of the barrier counter is set (the next grid barrier ends the kernel) and 0 is returned. Once the bit is set, by this
// thread or any other, every later wait of the launch returns at once: a kernel whose peer is silent runs out its patience
// once, not once per exchange.
__device__ __forceinline__ uint32_t ll_load(const uint2* p, uint32_t seq, const MegaArgs& a) {
    uint32_t value, got;
    unsigned long long t0 = 0;
    for (unsigned int spins = 0;; ++spins) {
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(value), "=r"(got) : "l"(p) : "memory");
        if (got == seq) return value;
        if ((spins & 63u) == 63u) {
            if (*reinterpret_cast<volatile unsigned int*>(a.bar) >= kBarFail) return 0u;  // somebody gave up already
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > a.tp_wait_ns) {
                report_failure(a.bar, a.status, 3u);
                return 0u;
            }
        }
    }
}

// After a grid barrier, CTA p < tp_world: sends this rank's slice [tp_rank * n, + n) of the local 32-bit vector `src` to
// rank p's pair buffer at byte offset `off` of its box.
__device__ __noinline__ void tp_push_slice(const MegaArgs& a, const uint32_t* src, unsigned int off, int n, unsigned int seq) {
    uint2* dst = reinterpret_cast<uint2*>(a.tp_box[blockIdx.x] + off) + a.tp_rank * n;
    src += a.tp_rank * n;
    for (int i = threadIdx.x; i < n; i += kMegaThreads) ll_store(dst + i, __ldcg(src + i), seq);
}

// Table fill for any block size that is a multiple of 64: thread -> (column = tid & 63, part = tid >> 6).
template <int THREADS>
__device__ __forceinline__ void fill_table_n(int* tab, const int a[5], int tid) {
    constexpr int parts = THREADS / 64;
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

__device__ __forceinline__ int quantize_code(float y, float s) {
    float q = roundf(__fmul_rn(y, s));
    q = q != q ? 0.0f : fminf(fmaxf(q, -128.0f), 127.0f);
    return static_cast<int>(q);
}

// The GEMV share of this CTA in one phase: items first + blockIdx.x, + gridDim.x, ... Activations come either from
// shared memory as int8 codes (act_s) or from global memory as floats that are quantised here with scale `qs`.
// Column bytes of the diagonal walk: word q, byte j -> ((lane + 4 q + j) mod 32) * 4 (see gemv_lut_kernel).
__device__ __forceinline__ void make_column_words(uint32_t (&creg)[8], int lane) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        uint32_t v = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) v |= static_cast<uint32_t>(((lane + 4 * q + j) & 31) * 4) << (8 * j);
        asm volatile("mov.b32 %0, %1;" : "=r"(creg[q]) : "r"(v));
    }
}

// Not inlined: each phase gets its own register allocation instead of competing inside one huge function.
template <uint32_t BASE>
__device__ __noinline__ void mega_gemv(const GemvItem* __restrict__ items, int first, int count, int* tab, const int8_t* act_s,
                                       const float* __restrict__ act_f, float qs, int32_t* __restrict__ out_base) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t creg[8];
    make_column_words(creg, lane);
    for (int k = blockIdx.x; k < count; k += gridDim.x) {
        const GemvItem it = items[first + k];
        // the first three row tiles of this warp do not depend on the table: they are requested before it is built
        const uint4* wa = it.wa + lane;
        const uint4* wb = it.wb + lane;
        TileRegs ra, rb, rc;
        const int n = it.ntiles, W = kMegaWarps;
        int t = warp;
        if (t < n) load_tile(ra, wa, wb, it.nblk, t, 0);
        if (t + W < n) load_tile(rb, wa, wb, it.nblk, t + W, 0);
        if (t + 2 * W < n) load_tile(rc, wa, wb, it.nblk, t + 2 * W, 0);
        {
            const int col = tid & 63, gb = col >> 5, j = col & 31;
            int a[5];
#pragma unroll
            for (int p = 0; p < 5; ++p) {
                const int c = it.col0 + gb * kBlockTrits + p * kBlockBytes + j;
                int v = 0;
                if (gb < it.nblk && c < it.cols) v = act_s != nullptr ? static_cast<int>(act_s[c]) : (qs > 0.0f ? quantize_code(act_f[c], qs) : 0);
                a[p] = v;
            }
            fill_table_n<kMegaThreads>(tab, a, tid);
        }
        __syncthreads();
        int32_t* out = out_base + it.out_off + it.tile0 * kTileRows + lane;
        const int rows_left = it.rows - it.tile0 * kTileRows - lane;
        while (t < n) {  // three row tiles in flight per warp
            {
                const int acc = tile_sum<BASE>(ra, it.nblk, creg);
                if (t * kTileRows < rows_left) atomicAdd(out + t * kTileRows, acc);
            }
            if (t + 3 * W < n) load_tile(ra, wa, wb, it.nblk, t + 3 * W, 0);
            if (t + W >= n) break;
            {
                const int acc = tile_sum<BASE>(rb, it.nblk, creg);
                if ((t + W) * kTileRows < rows_left) atomicAdd(out + (t + W) * kTileRows, acc);
            }
            if (t + 4 * W < n) load_tile(rb, wa, wb, it.nblk, t + 4 * W, 0);
            if (t + 2 * W >= n) break;
            {
                const int acc = tile_sum<BASE>(rc, it.nblk, creg);
                if ((t + 2 * W) * kTileRows < rows_left) atomicAdd(out + (t + 2 * W) * kTileRows, acc);
            }
            if (t + 5 * W < n) load_tile(rc, wa, wb, it.nblk, t + 5 * W, 0);
            t += 3 * W;
        }
        __syncthreads();  // the table is rewritten by the next item
    }
}

// RMSNorm + int8 quantisation of n values held in y_s (overwritten with the normalised values); every thread returns the
// activation scale. Same arithmetic as norm_quant_kernel.
__device__ __forceinline__ float mega_norm_quant(float* y_s, const float* norm_w, int n, float eps, int8_t* a8, double* sh_d,
                                                 float* sh_f, const MegaArgs* ta = nullptr) {
    (void)ta;
    const int tid = threadIdx.x;
    double sum = 0.0;
    for (int i = tid; i < n; i += kMegaThreads) sum += static_cast<double>(__fmul_rn(y_s[i], y_s[i]));
    sum = block_sum_f64(sum, sh_d);
#ifdef QTB_FINE_TRACE
    if (ta) QTB_FINE(*ta, 18);
#endif
    const float mean = __double2float_rn(sum / static_cast<double>(n));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    float amax = 0.0f;
    for (int i = tid; i < n; i += kMegaThreads) {
        const float y = __fmul_rn(__fmul_rn(y_s[i], inv), norm_w[i]);
        y_s[i] = y;
        amax = fmaxf(amax, fabsf(y));
    }
    amax = block_max_f32(amax, sh_f);
#ifdef QTB_FINE_TRACE
    if (ta) QTB_FINE(*ta, 19);
#endif
    const float s = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    if (a8 != nullptr)
        for (int i = tid; i < n; i += kMegaThreads) a8[i] = static_cast<int8_t>(amax > 0.0f ? quantize_code(y_s[i], s) : 0);
    __syncthreads();
    return s;
}

// 16-byte asynchronous copy global -> shared (bypasses registers; completion through cp.async.wait_group).
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gsrc) : "memory");
}
// Requests the n norm weights that the next norm needs (one copy group); they land while other phases run.
__device__ __forceinline__ void request_norm_weights(float* w_s, const float* __restrict__ w, int n) {
    for (int i = threadIdx.x; i < n; i += kMegaThreads) cp_async4(w_s + i, w + i);
    cp_async_commit();
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Asks the copy engine to bring `bytes` (a multiple of 16, from a 16-byte boundary of this GPU's own memory) into L2; nothing
// waits for it. A decode step leaves HBM idle most of the time (the dependent phases between two weight streams take longer
// than the streams), while a layer's weights fit L2 several times: every CTA therefore requests its share of the weights of a
// later phase while an earlier phase runs, and the GEMV phases then read L2 instead of starting a cold HBM stream after
// every grid barrier.
__device__ __forceinline__ void l2_prefetch_bulk(const void* p, unsigned int bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
constexpr unsigned int kPrefetchPiece = 8192;  // bytes per request
// This CTA's share of matrix `which` of layer `ly` (shares are whole pieces; the last CTAs may have none).
__device__ __forceinline__ void prefetch_weights(const MegaLayer& ly, int which) {
    const unsigned int bytes = ly.wbytes[which];
    const unsigned int pieces = (bytes + kPrefetchPiece - 1) / kPrefetchPiece, per = (pieces + gridDim.x - 1) / gridDim.x;
    const unsigned int p0 = blockIdx.x * per, p1 = min(p0 + per, pieces);
    for (unsigned int q = p0 + threadIdx.x; q < p1; q += kMegaThreads) {
        const unsigned int off = q * kPrefetchPiece;
        l2_prefetch_bulk(ly.wbase[which] + off, min(kPrefetchPiece, bytes - off));
    }
}

// y_s[i] = x[i] + acc[i] * post (the rescaled projection added to the residual stream), all loads of a thread issued
// before the first use. acc was accumulated with atomics by other SMs: it is read from L2 (ld.cg).
__device__ __forceinline__ void residual_add(float* y_s, const float* x, const int32_t* acc, float post, bool live, int n) {
    constexpr int kPer = 8;
    for (int i0 = threadIdx.x; i0 < n; i0 += kPer * kMegaThreads) {
        int av[kPer];
        float xv[kPer];
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            const int i = i0 + k * kMegaThreads;
            av[k] = i < n ? __ldcg(acc + i) : 0;
            xv[k] = i < n ? __ldcg(x + i) : 0.0f;
        }
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            const int i = i0 + k * kMegaThreads;
            if (i < n) y_s[i] = __fadd_rn(xv[k], live ? __fmul_rn(static_cast<float>(av[k]), post) : 0.0f);
        }
    }
}

// One try at a pair: the value and whether it carries `seq` yet.
__device__ __forceinline__ uint2 ll_peek(const uint2* p) {
    uint2 r;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p) : "memory");
    return r;
}

// residual_add whose projection results arrive as (value, sequence) pairs from every rank of a tensor-parallel group.
// All pairs of a thread are requested before the first is examined; only those that have not arrived yet are polled.
__device__ __forceinline__ void residual_add_ll(float* y_s, const float* x, const uint2* acc, unsigned int seq, const MegaArgs& a, float post,
                                                bool live, int n) {
    constexpr int kPer = 8;
    for (int i0 = threadIdx.x; i0 < n; i0 += kPer * kMegaThreads) {
        uint2 pr[kPer];
        float xv[kPer];
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            const int i = i0 + k * kMegaThreads;
            pr[k] = i < n ? ll_peek(acc + i) : make_uint2(0u, seq);
            xv[k] = i < n ? __ldcg(x + i) : 0.0f;
        }
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            const int i = i0 + k * kMegaThreads;
            if (i >= n) continue;
            const int av = static_cast<int>(pr[k].y == seq ? pr[k].x : ll_load(acc + i, seq, a));
            y_s[i] = __fadd_rn(xv[k], live ? __fmul_rn(static_cast<float>(av), post) : 0.0f);
        }
    }
}

constexpr int kAttnBlockPos = 128;                          // positions staged in shared memory at a time
constexpr int kAttnBlockBytes = kAttnBlockPos * 256 * 2;    // one staged block (head_dim <= 256 halves per row)

// Byte offset of 16-byte piece `c` of row `r` inside a staged block. The pieces of a row are permuted by the low three
// bits of the row number, so that 8 threads reading the same piece of 8 consecutive rows, or one row's consecutive
// pieces, always touch 8 different 16-byte bank groups (head_dim >= 64, i.e. at least 8 pieces per row).
__device__ __forceinline__ int staged_offset(int r, int c, int row_bytes) { return r * row_bytes + ((c ^ (r & 7)) << 4); }

// Copies rows [p0, p0 + 128) of a KV chunk (head_dim halves each, row stride kvd halves) into a staged block with
// asynchronous 16-byte copies; rows at or beyond `len` are skipped (the row of the current position is patched in from
// shared memory by the consumer).
__device__ __forceinline__ void stage_rows(unsigned char* dst, const __half* src, int p0, int len, int hd, int kvd) {
    const int shift = 31 - __clz(hd >> 3);  // head_dim is a power of two: pieces per row = 1 << shift
    const int row_bytes = hd * 2;
    for (int v = threadIdx.x; v < (kAttnBlockPos << shift); v += kMegaThreads) {
        const int r = v >> shift, c = v & ((1 << shift) - 1);
        if (p0 + r < len) cp_async16(dst + staged_offset(r, c, row_bytes), src + static_cast<size_t>(p0 + r) * kvd + c * 8);
    }
}

// Score of one staged key row against the query, by ONE thread: the 32 accumulator lanes of the reference's dot product
// (ggml_vec_dot_f16: element e goes to lane e mod 32, lanes are summed by a fixed tree) live in 32 registers, so the
// 32 chains run interleaved and the tree needs no shuffles.
template <bool F32>
__device__ __forceinline__ float key_score(const unsigned char* buf, int r, int hd, const float* s_q) {
    float acc[32];
#pragma unroll
    for (int l = 0; l < 32; ++l) acc[l] = 0.0f;
    const int row_bytes = hd * 2;
    const unsigned char* row = buf + r * row_bytes;
    const int sw = r & 7;
    for (int i = 0; i < hd; i += 32) {
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            const uint4 kk = *reinterpret_cast<const uint4*>(row + ((((i >> 3) + cc) ^ sw) << 4));
            const float4 q0 = *reinterpret_cast<const float4*>(s_q + i + 8 * cc), q1 = *reinterpret_cast<const float4*>(s_q + i + 8 * cc + 4);
            const __half2 h0 = *reinterpret_cast<const __half2*>(&kk.x), h1 = *reinterpret_cast<const __half2*>(&kk.y);
            const __half2 h2 = *reinterpret_cast<const __half2*>(&kk.z), h3 = *reinterpret_cast<const __half2*>(&kk.w);
            acc[8 * cc + 0] = __fmaf_rn(__low2float(h0), q0.x, acc[8 * cc + 0]);
            acc[8 * cc + 1] = __fmaf_rn(__high2float(h0), q0.y, acc[8 * cc + 1]);
            acc[8 * cc + 2] = __fmaf_rn(__low2float(h1), q0.z, acc[8 * cc + 2]);
            acc[8 * cc + 3] = __fmaf_rn(__high2float(h1), q0.w, acc[8 * cc + 3]);
            acc[8 * cc + 4] = __fmaf_rn(__low2float(h2), q1.x, acc[8 * cc + 4]);
            acc[8 * cc + 5] = __fmaf_rn(__high2float(h2), q1.y, acc[8 * cc + 5]);
            acc[8 * cc + 6] = __fmaf_rn(__low2float(h3), q1.z, acc[8 * cc + 6]);
            acc[8 * cc + 7] = __fmaf_rn(__high2float(h3), q1.w, acc[8 * cc + 7]);
        }
    }
    if (F32) {  // ggml_vec_dot_f16 summed as (a0+a1)+(a2+a3), then ((l0+l4)+(l2+l6))+((l1+l5)+(l3+l7)): dot_lane_reduce_f16_f32
#pragma unroll
        for (int l = 0; l < 8; ++l) acc[l] = __fadd_rn(__fadd_rn(acc[l], acc[l + 8]), __fadd_rn(acc[l + 16], acc[l + 24]));
    } else {    // (a0+a2)+(a1+a3): dot_lane_reduce_f16
#pragma unroll
        for (int l = 0; l < 8; ++l) acc[l] = __fadd_rn(__fadd_rn(acc[l], acc[l + 16]), __fadd_rn(acc[l + 8], acc[l + 24]));
    }
#pragma unroll
    for (int l = 0; l < 4; ++l) acc[l] = __fadd_rn(acc[l], acc[l + 4]);
    if (F32) return __fadd_rn(__fadd_rn(acc[0], acc[2]), __fadd_rn(acc[1], acc[3]));
    return __fadd_rn(__fadd_rn(acc[0], acc[1]), __fadd_rn(acc[2], acc[3]));
}

// One staged run of the value accumulation for one coordinate (attention.rs:448-470): n positions in order (n starts on a
// multiple of 8 positions of the chunk), the value of position r at col[r * stride], factors ms[r] / vs[r]. The running
// sum is rounded to half precision after every operation unless F32. Arguments are byte offsets into the dynamic shared
// memory. Kept small on purpose: the registers of a call chain (kernel + phase + unit + this) add up, and beyond the
// budget of 128 every function of the kernel starts to spill.
// The dynamic shared memory of the CTA as the compiler knows it (shared state space, 32-bit addressing): loads through a
// pointer that came in as a function argument are generic loads, which cost registers and latency in the chains below.
__device__ __forceinline__ unsigned char* dyn_smem() {
    extern __shared__ __align__(1024) unsigned char dyn_smem_base[];
    return dyn_smem_base;
}

template <bool F32>
__device__ __noinline__ float value_chain(uint32_t col_off, int stride, uint32_t ms_off, uint32_t vs_off, uint32_t next_off, int g0, int n, float acc) {
    auto rnd = [](float x) { return F32 ? x : __half2float(__float2half_rn(x)); };
    unsigned char* base = dyn_smem();
    const __half* col = reinterpret_cast<const __half*>(base + col_off);
    const float* ms = reinterpret_cast<const float*>(base + ms_off);
    const float* vs = reinterpret_cast<const float*>(base + vs_off);
    const unsigned short* next = reinterpret_cast<const unsigned short*>(base + next_off);
    // `next` holds, for every group of 8 positions from the first one of this run, the index (relative to the chunk's first
    // group, like g0) of the first group at or after it whose running maximum moved. Up to there the loop is branch-free,
    // so the loads of later groups overlap the dependent steps of earlier ones.
    const int full = n >> 3;
    int grp = 0;
    while (grp < full) {
        const int e = min(static_cast<int>(next[grp]) - g0, full);
        for (; grp < e; ++grp) {
            float w[8], v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                w[j] = vs[grp * 8 + j];
                v[j] = __half2float(col[(grp * 8 + j) * stride]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = rnd(__fmaf_rn(v[j], w[j], acc));
        }
        if (grp < full) {  // ms = 1 leaves the sum unchanged bit for bit, so the reference's test for it needs no branch
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                acc = rnd(__fmul_rn(acc, ms[grp * 8 + j]));
                acc = rnd(__fmaf_rn(__half2float(col[(grp * 8 + j) * stride]), vs[grp * 8 + j], acc));
            }
            ++grp;
        }
    }
    for (int r = full * 8; r < n; ++r) {
        acc = rnd(__fmul_rn(acc, ms[r]));
        acc = rnd(__fmaf_rn(__half2float(col[r * stride]), vs[r], acc));
    }
    return acc;
}

// KV geometry of the current token (attention.rs:392-396, 483-542): the padded KV axis and the chunk split.
struct KvSplit {
    int pos, seq_len, n_kv, chunk;  // chunk = positions per chunk (n_kv when there is a single chunk)
    bool split;
};
__device__ __forceinline__ KvSplit kv_split(const MegaArgs& a) {
    KvSplit s;
    s.pos = static_cast<int>(a.pos[0]);
    s.seq_len = s.pos + 1;
    s.n_kv = (s.seq_len + 255) / 256 * 256;
    if (s.n_kv < 256) s.n_kv = 256;
    if (s.n_kv > a.ctx) s.n_kv = a.ctx;
    s.split = s.n_kv >= 512;
    s.chunk = s.split ? (s.n_kv + 3) / 4 : s.n_kv;
    return s;
}

// Attention, first half: the scores of `rows` consecutive positions from r0 of one KV head against the query heads that
// share it (rope_kv_kernel + phase A of attention_kernel). The key rows are staged once in shared memory (asynchronous
// 16-byte copies) and used by every query head of the group; the unit that holds the current position computes the new
// key and value rows, appends them to the cache and scores the new key from shared memory. Scores go to
// a.scores[head][position]. `smem` is the CTA's dynamic shared memory from its start: the staged block overlays the GEMV
// table, whose zero rows are restored before returning.
__device__ __noinline__ void mega_scores_unit(const MegaArgs& a, const MegaLayer& ly, int kvh, int r0, int rows, float s_in, unsigned char* smem) {
    const int tid = threadIdx.x;
    const int hd = a.head_dim, gqa = a.q_heads / a.kv_heads;
    const int qd = a.q_heads * hd, kvd = a.kv_heads * hd, row_bytes = hd * 2;
    unsigned char* blk = smem;                                               // kAttnBlockBytes
    float* s_q = reinterpret_cast<float*>(smem + kAttnBlockBytes);           // gqa x head_dim floats
    __half* s_kcur = reinterpret_cast<__half*>(s_q + gqa * hd);              // head_dim halves
    __half* s_vcur = s_kcur + hd;
    const bool f32v = a.f32_values != 0;
    const float attn_scale = a.attn_scale;
    const int pos = static_cast<int>(a.pos[0]);
    const bool has_cur = pos >= r0 && pos < r0 + rows;
    const int len_old = has_cur ? pos - r0 : rows;  // rows that come from the cache
    const __half* kbase = ly.kc + static_cast<size_t>(kvh) * hd + static_cast<size_t>(r0) * kvd;
    const bool live = s_in > 0.0f;
    const float pq = live ? __fdiv_rn(ly.ws[0], s_in) : 0.0f, pk = live ? __fdiv_rn(ly.ws[1], s_in) : 0.0f, pv = live ? __fdiv_rn(ly.ws[2], s_in) : 0.0f;
    const float* cs = a.cos_sin + static_cast<size_t>(pos) * a.rope_dims;
    const int half = hd / 2, hr = a.rope_dims / 2;
    const int n_pairs = (gqa + (has_cur ? 1 : 0)) * half;
    // Pair idx of the rotated, rescaled query heads (and of the new key / value rows): head g, pair p. Its two elements are
    // (2p, 2p + 1), or with NEOX pairing (p, p + rope_dims / 2) inside the rotated part and plain neighbours behind it
    // (ops.rs:160-221).
    struct Pair {
        int g, p, e0, e1, i0, i1, j0, j1;
    };
    auto fetch = [&](int idx) {
        Pair r;
        r.g = idx / half, r.p = idx - r.g * half;
        r.e0 = 2 * r.p, r.e1 = 2 * r.p + 1;
        if (a.neox) {
            r.e0 = r.p < hr ? r.p : a.rope_dims + 2 * (r.p - hr);
            r.e1 = r.p < hr ? r.p + hr : r.e0 + 1;
        }
        const bool is_q = r.g < gqa;
        const int base = is_q ? (kvh * gqa + r.g) * hd : qd + kvh * hd;
        r.i0 = __ldcg(a.acc_qkv + base + r.e0), r.i1 = __ldcg(a.acc_qkv + base + r.e1);
        r.j0 = 0, r.j1 = 0;
        if (!is_q) {
            r.j0 = __ldcg(a.acc_qkv + base + kvd + r.e0);
            r.j1 = __ldcg(a.acc_qkv + base + kvd + r.e1);
        }
        return r;
    };
    // the integer results of this thread's first pair are requested before the key rows are staged (the copies below keep
    // the load/store unit busy for most of a microsecond)
    Pair first{};
    if (tid < n_pairs) first = fetch(tid);
    QTB_FINE(a, 25);
    __syncthreads();  // every thread is done with the table the block overlays
    stage_rows(blk, kbase, 0, len_old, hd, kvd);
    cp_async_commit();
    for (int idx = tid; idx < n_pairs; idx += kMegaThreads) {
        const Pair pr = idx == tid ? first : fetch(idx);
        const int g = pr.g, p = pr.p, e0 = pr.e0, e1 = pr.e1, i0 = pr.i0, i1 = pr.i1, j0 = pr.j0, j1 = pr.j1;
        const bool is_q = g < gqa;
        const bool rot = p < hr;
        float c0 = 1.0f, sn = 0.0f;
        if (rot) {
            c0 = cs[2 * p];
            sn = cs[2 * p + 1];
        }
        const float post = is_q ? pq : pk;
        float x0 = live ? __fmul_rn(static_cast<float>(i0), post) : 0.0f, x1 = live ? __fmul_rn(static_cast<float>(i1), post) : 0.0f;
        if (rot) {
            const float y0 = __fmaf_rn(x0, c0, -__fmul_rn(x1, sn)), y1 = __fmaf_rn(x0, sn, __fmul_rn(x1, c0));
            x0 = y0;
            x1 = y1;
        }
        if (is_q) {
            s_q[g * hd + e0] = f32v ? x0 : __half2float(__float2half_rn(x0));
            s_q[g * hd + e1] = f32v ? x1 : __half2float(__float2half_rn(x1));
        } else {
            s_kcur[e0] = __float2half_rn(x0);
            s_kcur[e1] = __float2half_rn(x1);
            s_vcur[e0] = __float2half_rn(live ? __fmul_rn(static_cast<float>(j0), pv) : 0.0f);
            s_vcur[e1] = __float2half_rn(live ? __fmul_rn(static_cast<float>(j1), pv) : 0.0f);
        }
    }
    __syncthreads();
    if (has_cur && tid < hd) {  // append to the cache (kv_cache.rs:124-138) and put the new key into the staged block
        const size_t at = static_cast<size_t>(pos) * kvd + static_cast<size_t>(kvh) * hd + tid;
        ly.kc[at] = s_kcur[tid];
        ly.vc[at] = s_vcur[tid];
        *reinterpret_cast<__half*>(blk + staged_offset(pos - r0, tid >> 3, row_bytes) + (tid & 7) * 2) = s_kcur[tid];
    }
    QTB_FINE(a, 26);
    cp_async_wait<0>();
    __syncthreads();
    QTB_FINE(a, 27);
    for (int t = tid; t < rows * gqa; t += kMegaThreads) {
        const int g = t / rows, r = t - g * rows;
        const float sc = f32v ? key_score<true>(blk, r, hd, s_q + g * hd) : key_score<false>(blk, r, hd, s_q + g * hd);
        a.scores[static_cast<size_t>(kvh * gqa + g) * a.ctx + r0 + r] = __fmul_rn(sc, attn_scale);
    }
    __syncthreads();
    QTB_FINE(a, 28);
    for (int i = tid; i < 13 * 64; i += kMegaThreads) {  // the zero rows of the table (byte values that are no velurex code)
        const int k = i >> 6;
        reinterpret_cast<int*>(smem)[(k < 9 ? 28 * k + 27 : 243 + k) * 64 + (i & 63)] = 0;
    }
    __syncthreads();
}

constexpr int kAttnSlice = 32;  // coordinates of a head that one values unit accumulates (one warp per query head)

// Shared memory a values unit needs for chunks of `len` positions and `gqa` query heads per KV head.
__host__ __device__ constexpr size_t values_unit_bytes(int len, int gqa) {
    return (static_cast<size_t>(len) * kAttnSlice * 2 + 15) / 16 * 16 + static_cast<size_t>(2) * gqa * len * 4 + (kMegaWarps + 16) * 4 +
           (static_cast<size_t>(gqa) * ((len + 7) / 8 + 1) * 3 + 15) / 16 * 16;
}

// Attention, second half: for one KV head, one chunk of positions and one slice of 32 coordinates, the softmax factors of
// every query head of the group (phase B of attention_kernel, recomputed by every slice) and the value accumulation
// (phase C). The V slice of the whole chunk is staged in shared memory in four copy groups; warp g runs the chains of
// query head g, one coordinate per lane, strictly in position order. Slice 0 also produces M and S of each head.
__device__ __noinline__ void mega_values_unit(const MegaArgs& a, const MegaLayer& ly, int kvh, int c, int slice, unsigned char* smem) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hd = a.head_dim, gqa = a.q_heads / a.kv_heads, kvd = a.kv_heads * hd;
    const bool f32v = a.f32_values != 0;
    const KvSplit ks = kv_split(a);
    int start = 0, end = ks.seq_len;
    if (ks.split) {
        start = c * ks.chunk;
        end = min(min(start + ks.chunk, ks.n_kv), ks.seq_len);
    } else if (c > 0) {
        start = end;
    }
    const int len = end - start;
    if (len <= 0) {
        if (slice == 0 && tid < gqa) {
            float* my_ms = a.part_ms + (static_cast<size_t>(kvh * gqa + tid) * 4 + c) * 2;
            my_ms[0] = -INFINITY;
            my_ms[1] = 0.0f;
        }
        return;
    }
    __half* vbuf = reinterpret_cast<__half*>(smem);                                   // [len][32] halves
    float* f_ms = reinterpret_cast<float*>(smem + (static_cast<size_t>(len) * kAttnSlice * 2 + 15) / 16 * 16);  // [gqa][len]
    float* f_vs = f_ms + gqa * len;                                                   // [gqa][len]: scores, then vs
    float* s_tm = f_vs + gqa * len;                                                   // kMegaWarps floats
    float* s_M = s_tm + kMegaWarps;                                                   // up to 16 heads
    const int ngroups = (len + 7) / 8;
    unsigned short* s_next = reinterpret_cast<unsigned short*>(s_M + 16);             // [gqa][ngroups + 1]: first group >= g whose maximum moved
    unsigned char* s_moved = reinterpret_cast<unsigned char*>(s_next + gqa * (ngroups + 1));  // [gqa][ngroups]: any ms != 1 in the group of 8
    __syncthreads();  // every thread is done with the table the slice overlays
    {
        // the V slice in four groups of rows, so that the chain can start when the first quarter has landed
        const __half* vsrc = ly.vc + static_cast<size_t>(start) * kvd + static_cast<size_t>(kvh) * hd + slice * kAttnSlice;
        const int q_rows = (len + 3) / 4;
        for (int q = 0; q < 4; ++q) {
            const int ra = min(q * q_rows, len), rb = min(ra + q_rows, len);
            for (int v = ra * 4 + tid; v < rb * 4; v += kMegaThreads) {
                const int r = v >> 2, pc = v & 3;
                cp_async16(vbuf + r * kAttnSlice + pc * 8, vsrc + static_cast<size_t>(r) * kvd + pc * 8);
            }
            cp_async_commit();
        }
    }
    for (int idx = tid; idx < gqa * len; idx += kMegaThreads) {
        const int g = idx / len, p = idx - g * len;
        f_vs[idx] = __ldcg(a.scores + static_cast<size_t>(kvh * gqa + g) * a.ctx + start + p);
    }
    __syncthreads();
    QTB_FINE(a, 2);
    // softmax factors: four groups of 128 threads take one head each; running maximum in position order by a scan over
    // the group's threads (attention.rs:448-462)
    for (int g0 = 0; g0 < gqa; g0 += 4) {
        const int g = g0 + (tid >> 7), gt = tid & 127, gw = gt >> 5;  // head, thread and warp inside the group
        const bool active = g < gqa;
        const int per = (len + 127) / 128;
        const int p0 = min(gt * per, len), p1 = min(p0 + per, len);
        float* sc_g = f_vs + (active ? g : 0) * len;
        float* ms_g = f_ms + (active ? g : 0) * len;
        float m = -INFINITY;
        if (active)
            for (int p = p0; p < p1; ++p) m = fmaxf(m, sc_g[p]);
        float incl = m;
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl = fmaxf(incl, t);
        }
        if (lane == 31) s_tm[warp] = incl;
        __syncthreads();
        float run = __shfl_up_sync(0xffffffffu, incl, 1);
        if (lane == 0) run = -INFINITY;
        for (int w = 0; w < gw; ++w) run = fmaxf(run, s_tm[(warp - gw) + w]);
        if (active) {
            for (int p = p0; p < p1; ++p) {
                const float sc = sc_g[p];
                const float m_old = run;
                float ms = 1.0f, vs = 1.0f;
                if (sc > run) {
                    run = sc;
                    ms = device_expf(__fsub_rn(m_old, run));
                } else {
                    vs = device_expf(__fsub_rn(sc, run));
                }
                ms_g[p] = ms;
                sc_g[p] = vs;
            }
            if (gt == 0) s_M[g] = fmaxf(fmaxf(s_tm[warp], s_tm[warp + 1]), fmaxf(s_tm[warp + 2], s_tm[warp + 3]));
        }
        __syncthreads();
    }
    {
        // one flag per head and group of 8 positions: does any rescale factor of the group differ from 1?
        for (int idx = tid; idx < gqa * ngroups; idx += kMegaThreads) {
            const int g = idx / ngroups, p0 = (idx - g * ngroups) * 8;
            bool any = false;
#pragma unroll
            for (int j = 0; j < 8; ++j) any |= p0 + j < len && f_ms[g * len + p0 + j] != 1.0f;
            s_moved[idx] = any ? 1 : 0;
        }
        __syncthreads();
        // For every group the first group at or after it whose maximum moved (the chain runs branch-free up to there): a
        // suffix minimum, one warp per head, 32 groups at a time from the end with the carry of the later groups.
        for (int g = warp; g < gqa; g += kMegaWarps) {
            int carry = ngroups;
            if (lane == 0) s_next[g * (ngroups + 1) + ngroups] = static_cast<unsigned short>(ngroups);
            for (int hi = ngroups; hi > 0; hi -= 32) {
                const int grp = hi - 32 + lane;  // lanes cover [hi - 32, hi); lanes below 0 idle
                int v = (grp >= 0 && s_moved[g * ngroups + grp]) ? grp : ngroups;
                for (int o = 1; o < 32; o <<= 1) {
                    const int t = __shfl_down_sync(0xffffffffu, v, o);
                    if (lane + o < 32) v = min(v, t);
                }
                v = min(v, carry);
                if (grp >= 0) s_next[g * (ngroups + 1) + grp] = static_cast<unsigned short>(v);
                carry = __shfl_sync(0xffffffffu, v, max(0, 32 - hi));  // the lowest covered group's value
            }
        }
        __syncthreads();
    }
    QTB_FINE(a, 3);
    // values: warp g < gqa runs head g (heads beyond the warp count take further rounds); with slice 0, lane 0 of warp
    // kMegaWarps - 1 - g accumulates S of head g over the same positions meanwhile
    const int q_rows = ((len + 3) / 4 + 7) / 8 * 8;  // chain quarters start on multiples of 8 positions, like the flags
    for (int g0 = 0; g0 < gqa; g0 += kMegaWarps / 2) {
        const int g = g0 + warp;
        const bool chain = warp < kMegaWarps / 2 && g < gqa;
        const int gs = g0 + (kMegaWarps - 1 - warp);
        const bool sums = slice == 0 && warp >= kMegaWarps / 2 && gs < gqa && lane == 0;
        float acc = 0.0f, S = 0.0f;
        for (int q = 0; q < 4; ++q) {
            if (g0 == 0) {
                // the copy groups hold ceil(len / 4) rows each, a chain quarter up to 7 more: the first quarter needs two
                // groups, the others everything
                if (q == 0) cp_async_wait<2>();
                if (q == 1) cp_async_wait<0>();
                if (q <= 1) __syncthreads();
            }
            const int ra = min(q * q_rows, len), rb = min(ra + q_rows, len);
            if (chain) {
                const uint32_t o_col = static_cast<uint32_t>(reinterpret_cast<const unsigned char*>(vbuf + ra * kAttnSlice + lane) - smem);
                const uint32_t o_ms = static_cast<uint32_t>(reinterpret_cast<const unsigned char*>(f_ms + g * len + ra) - smem);
                const uint32_t o_vs = static_cast<uint32_t>(reinterpret_cast<const unsigned char*>(f_vs + g * len + ra) - smem);
                const uint32_t o_nx = static_cast<uint32_t>(reinterpret_cast<const unsigned char*>(s_next + g * (ngroups + 1) + (ra >> 3)) - smem);
                acc = f32v ? value_chain<true>(o_col, kAttnSlice, o_ms, o_vs, o_nx, ra >> 3, rb - ra, acc)
                           : value_chain<false>(o_col, kAttnSlice, o_ms, o_vs, o_nx, ra >> 3, rb - ra, acc);
            } else if (sums) {
#pragma unroll 8
                for (int p = ra; p < rb; ++p) S = __fmaf_rn(S, f_ms[gs * len + p], f_vs[gs * len + p]);  // attention.rs:466
            }
        }
        QTB_FINE(a, 12);
        if (chain) a.part_acc[(static_cast<size_t>(kvh * gqa + g) * 4 + c) * hd + slice * kAttnSlice + lane] = acc;
        if (sums) {
            float* my_ms = a.part_ms + (static_cast<size_t>(kvh * gqa + gs) * 4 + c) * 2;
            my_ms[0] = s_M[gs];
            my_ms[1] = S;
        }
    }
    __syncthreads();
    for (int i = tid; i < 13 * 64; i += kMegaThreads) {  // the zero rows of the table (byte values that are no velurex code)
        const int k = i >> 6;
        reinterpret_cast<int*>(smem)[(k < 9 ? 28 * k + 27 : 243 + k) * 64 + (i & 63)] = 0;
    }
    __syncthreads();
}

// ---- attention, second half, second form: one unit per (KV head, 8 coordinates) -----------------------------------------
// The value accumulation is a chain of one dependent step per position (about 16 cycles: multiply-add, round to half,
// widen), so its length, not the work, sets the time. A unit therefore takes ALL chunks of its coordinates at once: lane
// (chunk, coordinate) of warp g runs the chain of query head g for that chunk, the four chunks of the reference's split
// (attention.rs:510-533) side by side, and the unit also combines them (attention.rs:497-541) and contributes to the
// maximum that the quantiser of the o projection needs. What is left after the next grid barrier is a load and a rounding.
// Staging is asynchronous copies only (no registers, everything in flight at once): the unit's 16-byte piece of every
// cached V row into [chunk][position][8 halves], the scores of its heads into one row per (head, chunk). The softmax
// factors (attention.rs:448-462) are computed by all threads, eight consecutive positions each: maxima of the groups, a
// barrier, the maximum before the group from the earlier groups' maxima, then one exponential per position. A word per
// head and group of eight positions tells whether any chunk's running maximum moved there; groups without a move run
// branch-free.
constexpr int kV2Dims = 16;      // coordinates per unit: two warps of eight coordinates x four chunks per query head
constexpr int kV2WarpsPerHead = kV2Dims / 8;
constexpr int kV2MaxCtx = 4096;
constexpr int kV2MaxGqa = 7;     // chain warps (two per head) + the warp of the sum chains must fit the 16 warps of the CTA

// Row length (floats) of the factor rows for chunks of `chunk` positions: a multiple of 8, at least `chunk`.
__host__ __device__ constexpr int values2_clp(int chunk) { return (chunk + 7) / 8 * 8; }
// Positions per chunk in the staged V block: odd, so that the 32-byte pieces the four chunks' lanes read at one step fall into
// four different bank groups.
__host__ __device__ constexpr int values2_clr(int chunk) { return values2_clp(chunk) + 1; }
__host__ __device__ constexpr size_t values2_bytes(int ctx, int gqa) {
    const int nch = ctx >= 512 ? 4 : 1, chunk = ctx >= 512 ? (ctx + 3) / 4 : ctx, clp = values2_clp(chunk);
    return static_cast<size_t>(nch) * values2_clr(chunk) * kV2Dims * 2 + static_cast<size_t>(2) * gqa * nch * clp * 4 + static_cast<size_t>(gqa) * (clp / 8) * 4 +
           static_cast<size_t>(gqa) * 8 * 4 + static_cast<size_t>(gqa) * nch * 8 + 64;
}

template <bool F32>
__device__ __forceinline__ float v2_round(float x) {
    return F32 ? x : __half2float(__float2half_rn(x));
}

// The chain of one lane: `ngr` groups of eight positions in order; values (one half every 32 bytes), factors vs and ms and
// the table of next groups with a move (16 bits per group) at byte offsets into the dynamic shared memory. The operands of the next group are
// loaded while this group's eight dependent steps run. One chain per lane and more warps, rather than several chains per
// lane: a warp issues an instruction every three to four cycles here, so the instructions per step, not the latency of a
// step (16 cycles), set the pace. Rounded to half precision after every operation unless F32 (attention.rs:448-470).
template <bool F32>
__device__ __noinline__ float v2_chain(uint32_t v_off, uint32_t w_off, uint32_t m_off, uint32_t f_off, int ngr) {
    unsigned char* base = dyn_smem();
    const unsigned char* vrow = base + v_off;
    const float* wrow = reinterpret_cast<const float*>(base + w_off);
    const float* mrow = reinterpret_cast<const float*>(base + m_off);
    const unsigned char* fl = base + f_off;
    float acc = 0.0f;
    // The group after the last one is loaded too and not used: it lies in the padding or in the arrays behind the rows.
    __half vn[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) vn[j] = *reinterpret_cast<const __half*>(vrow + j * (kV2Dims * 2));
    float4 w0n = *reinterpret_cast<const float4*>(wrow), w1n = *reinterpret_cast<const float4*>(wrow + 4);
    // `nx[g]` is the first group at or after g in which some chunk's running maximum moved (ngr if none). Up to there the loop
    // has no branch but its own, so the compiler overlaps the loads of the next group with the eight dependent steps.
    const unsigned short* nx = reinterpret_cast<const unsigned short*>(fl);
    int grp = 0;
    while (grp < ngr) {
        const int stop = min(static_cast<int>(nx[grp]), ngr);
        for (; grp < stop; ++grp) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __half2float(vn[j]);
            const float w[8] = {w0n.x, w0n.y, w0n.z, w0n.w, w1n.x, w1n.y, w1n.z, w1n.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) vn[j] = *reinterpret_cast<const __half*>(vrow + (8 * (grp + 1) + j) * (kV2Dims * 2));
            w0n = *reinterpret_cast<const float4*>(wrow + 8 * (grp + 1));
            w1n = *reinterpret_cast<const float4*>(wrow + 8 * (grp + 1) + 4);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = v2_round<F32>(__fmaf_rn(v[j], w[j], acc));
        }
        if (grp < ngr) {
            // a group with a move: its rescale factors are loaded once; the multiply of a position is skipped where this lane's
            // chunk did not move (a factor of one would change nothing, but cost a step's latency)
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __half2float(vn[j]);
            const float w[8] = {w0n.x, w0n.y, w0n.z, w0n.w, w1n.x, w1n.y, w1n.z, w1n.w};
            const float4 m0 = *reinterpret_cast<const float4*>(mrow + grp * 8), m1 = *reinterpret_cast<const float4*>(mrow + grp * 8 + 4);
            const float m[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) vn[j] = *reinterpret_cast<const __half*>(vrow + (8 * (grp + 1) + j) * (kV2Dims * 2));
            w0n = *reinterpret_cast<const float4*>(wrow + 8 * (grp + 1));
            w1n = *reinterpret_cast<const float4*>(wrow + 8 * (grp + 1) + 4);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (m[j] != 1.0f) acc = v2_round<F32>(__fmul_rn(acc, m[j]));
                acc = v2_round<F32>(__fmaf_rn(v[j], w[j], acc));
            }
            ++grp;
        }
    }
    return acc;
}

// S of one (head, chunk): S = fma(S, ms, vs) over its positions in order (attention.rs:466), operands one group ahead.
__device__ __noinline__ float v2_sum_chain(uint32_t m_off, uint32_t w_off, int len) {
    unsigned char* base = dyn_smem();
    const float* ms_row = reinterpret_cast<const float*>(base + m_off);
    const float* vs_row = reinterpret_cast<const float*>(base + w_off);
    float S = 0.0f;
    const int full = len >> 3;
    // The group after the last one is loaded too and not used: it lies in the row's padding or in the arrays behind it.
    float4 m0 = *reinterpret_cast<const float4*>(ms_row), m1 = *reinterpret_cast<const float4*>(ms_row + 4);
    float4 v0 = *reinterpret_cast<const float4*>(vs_row), v1 = *reinterpret_cast<const float4*>(vs_row + 4);
    for (int g = 0; g < full; ++g) {
        const float4 n0 = *reinterpret_cast<const float4*>(ms_row + 8 * g + 8), n1 = *reinterpret_cast<const float4*>(ms_row + 8 * g + 12);
        const float4 u0 = *reinterpret_cast<const float4*>(vs_row + 8 * g + 8), u1 = *reinterpret_cast<const float4*>(vs_row + 8 * g + 12);
        S = __fmaf_rn(S, m0.x, v0.x);
        S = __fmaf_rn(S, m0.y, v0.y);
        S = __fmaf_rn(S, m0.z, v0.z);
        S = __fmaf_rn(S, m0.w, v0.w);
        S = __fmaf_rn(S, m1.x, v1.x);
        S = __fmaf_rn(S, m1.y, v1.y);
        S = __fmaf_rn(S, m1.z, v1.z);
        S = __fmaf_rn(S, m1.w, v1.w);
        m0 = n0, m1 = n1, v0 = u0, v1 = u1;
    }
    for (int p = full * 8; p < len; ++p) S = __fmaf_rn(S, ms_row[p], vs_row[p]);
    return S;
}

// One helper task of the values phase: the softmax factors of head `h`, chunk `c` (attention.rs:448-462), two consecutive
// positions per thread. The running maximum before a position comes from a scan over the block; then one exponential per
// position: ms = exp(m_before - score), vs = 1 where the score exceeds the maximum so far, else ms = 1, vs = exp(score -
// m_before). Positions behind the chunk's end up to the common chain length get vs = 0, ms = 1: such a step leaves a sum
// unchanged bit for bit. Rows, move flags (bit j of a word: the maximum moved at position 8 group + j, and by a factor other
// than one) and the chunk's maximum go to global memory; the count of finished tasks of the KV head is raised last.
__device__ __noinline__ void v2_factors_task(const MegaArgs& a, int h, int c, unsigned char* smem) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const KvSplit ks = kv_split(a);
    const int nch = ks.split ? 4 : 1, CL = ks.chunk, seq = ks.seq_len;
    auto chunk_len = [&](int cc) {
        if (!ks.split) return cc == 0 ? seq : 0;
        const int start = cc * CL;
        return max(0, min(min(start + CL, ks.n_kv), seq) - start);
    };
    int ngr = 0;
    for (int cc = 0; cc < nch; ++cc) ngr = max(ngr, (chunk_len(cc) + 7) / 8);
    const int len = chunk_len(c), slot = h * 4 + c;
    const float* src = a.scores + static_cast<size_t>(h) * a.ctx + c * CL;
    float* ms_out = a.fac + static_cast<size_t>(slot) * a.fac_stride;
    float* vs_out = a.fac + static_cast<size_t>(a.q_heads * 4 + slot) * a.fac_stride;
    unsigned int* fl_out = a.fac_flags + static_cast<size_t>(slot) * (a.fac_stride / 8);
    float* s_wt = reinterpret_cast<float*>(smem);  // one maximum per warp
    // chunks of up to 512 positions: one position per thread; up to 1024: two consecutive ones
    const bool two = ngr * 8 > kMegaThreads;
    const int p0 = two ? 2 * tid : tid, p1 = p0 + 1;
    const float s0 = p0 < len ? __ldcg(src + p0) : -INFINITY, s1 = two && p1 < len ? __ldcg(src + p1) : -INFINITY;
    float incl = fmaxf(s0, s1);
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl = fmaxf(incl, t);
    }
    float before = __shfl_up_sync(0xffffffffu, incl, 1);
    if (lane == 0) before = -INFINITY;
    __syncthreads();  // the table region is free
    if (lane == 31) s_wt[warp] = incl;
    __syncthreads();
    float total = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMegaWarps; ++w) {
        const float t = s_wt[w];
        if (w < warp) before = fmaxf(before, t);
        total = fmaxf(total, t);
    }
    auto factor = [&](int p, float sc, float m_before, float& ms, float& vs) {
        ms = 1.0f, vs = 0.0f;
        bool moved = false;
        if (p < len) {
            vs = 1.0f;
            if (sc > m_before) {
                ms = device_expf(__fsub_rn(m_before, sc));
                moved = ms != 1.0f;  // exp(0) = 1: a maximum that moved by nothing needs no rescale
            } else {
                vs = device_expf(__fsub_rn(sc, m_before));
            }
        }
        return moved;
    };
    float ms0, vs0, ms1 = 1.0f, vs1 = 0.0f;
    const bool mv0 = factor(p0, s0, before, ms0, vs0);
    bool mv1 = false;
    if (two) mv1 = factor(p1, s1, fmaxf(before, s0), ms1, vs1);
    const unsigned int b0 = __ballot_sync(0xffffffffu, mv0), b1 = __ballot_sync(0xffffffffu, mv1);
    if (two) {
        if (p0 < ngr * 8) {
            *reinterpret_cast<float2*>(ms_out + p0) = make_float2(ms0, ms1);
            *reinterpret_cast<float2*>(vs_out + p0) = make_float2(vs0, vs1);
        }
        if ((lane & 3) == 0) {  // four lanes = eight positions = one group
            unsigned int bits = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) bits |= (((b0 >> (lane + i)) & 1u) << (2 * i)) | (((b1 >> (lane + i)) & 1u) << (2 * i + 1));
            const int grp = warp * 8 + (lane >> 2);
            if (grp < ngr) fl_out[grp] = bits;
        }
    } else {
        if (p0 < ngr * 8) {
            ms_out[p0] = ms0;
            vs_out[p0] = vs0;
        }
        if ((lane & 7) == 0) {  // eight lanes = one group
            const int grp = warp * 4 + (lane >> 3);
            if (grp < ngr) fl_out[grp] = (b0 >> lane) & 0xFFu;
        }
    }
    if (tid == 0) a.fac_M[slot] = total;
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        atomicAdd(a.fac_done + h / (a.q_heads / a.kv_heads), 1u);
    }
}

#ifdef QTB_DEBUG_V2
__device__ long long g_v2_clock[16];
#define QTB_V2_CLOCK(k)                                  \
    do {                                                 \
        if (threadIdx.x == 0 && blockIdx.x == 0) g_v2_clock[k] = clock64(); \
    } while (0)
#else
#define QTB_V2_CLOCK(k) \
    do {                \
    } while (0)
#endif

template <bool F32>
__device__ __noinline__ void mega_values2_unit(const MegaArgs& a, const MegaLayer& ly, int l, int kvh, int slice, unsigned char* smem) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hd = a.head_dim, gqa = a.q_heads / a.kv_heads, kvd = a.kv_heads * hd;
    const KvSplit ks = kv_split(a);
    const int nch = ks.split ? 4 : 1, CL = ks.chunk, clp = values2_clp(CL), clr = values2_clr(CL), seq = ks.seq_len;
    const int ngr8 = clp / 8, npairs = gqa * nch;
    constexpr int kPiece = kV2Dims * 2;                                                  // bytes of a cached row a unit takes
    unsigned char* Vr = smem;                                                            // [nch][clr][16 halves]
    float* f_ms = reinterpret_cast<float*>(smem + static_cast<size_t>(nch) * clr * kPiece);  // [gqa][nch][clp]
    float* f_vs = f_ms + npairs * clp;                                                   // scores, then vs
    unsigned short* s_next = reinterpret_cast<unsigned short*>(f_vs + npairs * clp);     // [gqa][ngr8 + 2]: next group with a move
    float* s_scale = reinterpret_cast<float*>(s_next + gqa * (ngr8 + 2) + ((gqa * (ngr8 + 2)) & 1));  // [gqa][4][2]: chunk-combine factors
    float* s_MS = s_scale + gqa * 8;                                                     // [gqa][nch][2]: M, S
    int* s_ok = reinterpret_cast<int*>(s_MS + npairs * 2);
    auto chunk_len = [&](int c) {
        if (!ks.split) return c == 0 ? seq : 0;
        const int start = c * CL;
        return max(0, min(min(start + CL, ks.n_kv), seq) - start);
    };
    int ngr = 0;  // groups of eight positions of the longest chunk: the length of every chain of this unit
    for (int cc = 0; cc < nch; ++cc) ngr = max(ngr, (chunk_len(cc) + 7) / 8);
    __syncthreads();  // every thread is done with the table the arrays overlay
    QTB_FINE(a, 8);
    QTB_V2_CLOCK(0);
    {
        const __half* vsrc = ly.vc + static_cast<size_t>(kvh) * hd + slice * kV2Dims;
        for (int i = tid; i < seq * 2; i += kMegaThreads) {  // two 16-byte copies per cached row
            const int p = i >> 1, h = i & 1, c = ks.split ? p / CL : 0;
            cp_async16(Vr + static_cast<size_t>(c * clr + (p - c * CL)) * kPiece + h * 16, vsrc + static_cast<size_t>(p) * kvd + h * 8);
        }
        cp_async_commit();
        // zero values behind a chunk's end up to the common chain length (the last chunk, mostly)
        for (int c = 0; c < nch; ++c)
            for (int i = chunk_len(c) * 2 + tid; i < ngr * 16; i += kMegaThreads) *reinterpret_cast<uint4*>(Vr + static_cast<size_t>(c * clr) * kPiece + i * 16) = make_uint4(0u, 0u, 0u, 0u);
        // The factors of this group's heads come from the helper CTAs of this phase (v2_factors_task): wait, bounded, until
        // all (head, chunk) tasks of the KV head have been counted.
        if (tid == 0) {
            const unsigned int target = static_cast<unsigned int>(l + 1) * static_cast<unsigned int>(npairs);
            int okay = 1;
            for (unsigned int spins = 0;; ++spins) {
                unsigned int v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a.fac_done + kvh));
                if (v >= target) break;
                if (spins > kBarrierSpinLimit || *reinterpret_cast<volatile unsigned int*>(a.bar) >= kBarFail) {
                    report_failure(a.bar, a.status, 2u);
                    okay = 0;
                    break;
                }
            }
            *s_ok = okay;
        }
    }
    __syncthreads();
    if (*s_ok == 0) return;  // the grid barrier that follows ends the kernel
    QTB_FINE(a, 2);
    QTB_V2_CLOCK(1);
    {
        const int rows4 = a.q_heads * 4, fl_stride = a.fac_stride / 8;
        for (int pair = warp; pair < npairs; pair += kMegaWarps) {
            const int g = pair / nch, c = pair - g * nch, slot = (kvh * gqa + g) * 4 + c;
            const float* ms_src = a.fac + static_cast<size_t>(slot) * a.fac_stride;
            const float* vs_src = a.fac + static_cast<size_t>(rows4 + slot) * a.fac_stride;
            for (int q = lane; q < ngr * 2; q += 32) {
                cp_async16(f_ms + pair * clp + q * 4, ms_src + q * 4);
                cp_async16(f_vs + pair * clp + q * 4, vs_src + q * 4);
            }
        }
        cp_async_commit();
        // For every head and group the first group at or after it in which any chunk moved (the chain runs branch-free up to
        // there): one warp per head, 32 groups at a time from the end with the carry of the later groups.
        for (int g = warp; g < gqa; g += kMegaWarps) {
            unsigned short* nx = s_next + g * (ngr8 + 2);
            int carry = ngr;
            if (lane == 0) nx[ngr] = static_cast<unsigned short>(ngr);
            for (int hi = (ngr + 31) / 32 * 32; hi > 0; hi -= 32) {
                const int grp = hi - 32 + lane;
                unsigned int bits = 0;
                if (grp < ngr)
                    for (int c = 0; c < nch; ++c) bits |= __ldcg(a.fac_flags + static_cast<size_t>((kvh * gqa + g) * 4 + c) * fl_stride + grp);
                const unsigned int any = __ballot_sync(0xffffffffu, bits != 0u);
                const unsigned int later = any >> lane;  // bit 0: this group
                const int nxt = later ? hi - 32 + lane + (__ffs(later) - 1) : carry;
                if (grp < ngr) nx[grp] = static_cast<unsigned short>(nxt);
                carry = __shfl_sync(0xffffffffu, nxt, 0);
            }
        }
        if (tid < npairs) s_MS[tid * 2] = __ldcg(a.fac_M + (kvh * gqa + tid / nch) * 4 + tid % nch);
        if (ks.split && tid < gqa * 8) {
            // The factors that fold chunk c into the running result (attention.rs:510-541): the maximum before the chunk is
            // that of the earlier non-empty chunks, so the eight exponentials of a head are independent: one thread each.
            const int g = tid >> 3, c = (tid >> 1) & 3, which = tid & 1;
            const float* Mg = a.fac_M + (kvh * gqa + g) * 4;
            float m_before = -INFINITY;
            for (int k = 0; k < c; ++k)
                if (chunk_len(k) > 0) m_before = fmaxf(m_before, __ldcg(Mg + k));
            const float M = __ldcg(Mg + c), m_new = fmaxf(m_before, M);
            s_scale[tid] = device_expf(__fsub_rn(which == 0 ? m_before : M, m_new));
        }
        cp_async_wait<0>();
    }
    __syncthreads();
    QTB_FINE(a, 3);
    QTB_V2_CLOCK(3);
    float acc = 0.0f;
    const int head = warp / kV2WarpsPerHead, part8 = warp % kV2WarpsPerHead;  // chain warps: (query head, eight of the unit's coordinates)
    if (warp < gqa * kV2WarpsPerHead) {
        // lane -> (chunk, coordinate)
        const int c = lane >> 3, d = lane & 7;
        const int row = c < nch ? c : 0;  // lanes without a chunk repeat chunk 0; their sums are not used
        const uint32_t v_off = static_cast<uint32_t>(row * clr * kPiece + (part8 * 8 + d) * 2);
        const uint32_t w_off = static_cast<uint32_t>(reinterpret_cast<const unsigned char*>(f_vs + (head * nch + row) * clp) - smem);
        const uint32_t m_off = static_cast<uint32_t>(reinterpret_cast<const unsigned char*>(f_ms + (head * nch + row) * clp) - smem);
        const uint32_t f_off = static_cast<uint32_t>(reinterpret_cast<const unsigned char*>(s_next + head * (ngr8 + 2)) - smem);
        acc = v2_chain<F32>(v_off, w_off, m_off, f_off, ngr);
        QTB_FINE(a, 9);
        QTB_V2_CLOCK(4);
    } else {
        // S of every (head, chunk), one thread each, meanwhile
        const int pair = (warp - gqa * kV2WarpsPerHead) * 32 + lane;
        if (pair < npairs)
            s_MS[pair * 2 + 1] = v2_sum_chain(static_cast<uint32_t>(reinterpret_cast<const unsigned char*>(f_ms + pair * clp) - smem),
                                              static_cast<uint32_t>(reinterpret_cast<const unsigned char*>(f_vs + pair * clp) - smem), chunk_len(pair % nch));
    }
    __syncthreads();
    QTB_FINE(a, 12);
    QTB_V2_CLOCK(5);
    if (warp < gqa * kV2WarpsPerHead) {
        // combine the chunks (attention.rs:497-541); every lane of a coordinate computes the same value
        const int d = lane & 7;
        float part[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) part[c] = __shfl_sync(0xffffffffu, acc, (c * 8 + d) & 31);
        const float* MS = s_MS + head * nch * 2;
        float out;
        if (!ks.split) {
            const float S = MS[1];
            out = __fmul_rn(part[0], S == 0.0f ? 0.0f : __fdiv_rn(1.0f, S));
        } else {
            // A chunk is skipped when its S is zero (attention.rs:519), which happens exactly when it is empty; the factors in
            // s_scale were computed on that assumption. Should an S ever be zero otherwise, the factors are recomputed here.
            bool regular = true;
#pragma unroll
            for (int c = 0; c < 4; ++c) regular &= (MS[2 * c + 1] == 0.0f) == (chunk_len(c) == 0);
            float m_final = -INFINITY, s_final = 0.0f, sum = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float M = MS[2 * c], S = MS[2 * c + 1];
                if (S == 0.0f) continue;
                const float m_new = fmaxf(m_final, M);
                float scale_old = s_scale[head * 8 + 2 * c], scale_new = s_scale[head * 8 + 2 * c + 1];
                if (!regular) {
                    scale_old = device_expf(__fsub_rn(m_final, m_new));
                    scale_new = device_expf(__fsub_rn(M, m_new));
                }
                sum = __fmaf_rn(sum, scale_old, __fmul_rn(part[c], scale_new));
                s_final = __fmaf_rn(s_final, scale_old, __fmul_rn(S, scale_new));
                m_final = m_new;
            }
            out = s_final != 0.0f ? __fmul_rn(sum, __fdiv_rn(1.0f, s_final)) : sum;
        }
        if (lane < 8) a.attn_out[(kvh * gqa + head) * hd + slice * kV2Dims + part8 * 8 + lane] = out;
        float m = lane < 8 ? fabsf(out) : 0.0f;
        for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0 && m > 0.0f) atomicMax(a.amax_bits + 2 + (l & 1), __float_as_uint(m));  // non-negative floats order like their bits
    }
    __syncthreads();
    for (int i = tid; i < 13 * 64; i += kMegaThreads) {  // the zero rows of the table (byte values that are no velurex code)
        const int k = i >> 6;
        reinterpret_cast<int*>(smem)[(k < 9 ? 28 * k + 27 : 243 + k) * 64 + (i & 63)] = 0;
    }
    __syncthreads();
}

// Shared-memory plan of the token kernel (bytes from the dynamic base): attention region (its first 64 KiB double as the
// GEMV table) | y (floats) | a8 | small. The attention region holds whichever is largest: a scores unit (staged key block,
// the group's queries, the new key/value rows), a values unit for the longest chunk, or the lm_head rings.
__host__ __device__ constexpr size_t mega_attn_region(int ctx, int gqa, int head_dim, bool v2) {
    const int len_max = ctx < 512 ? ctx : (ctx + 3) / 4;
    size_t need = static_cast<size_t>(kAttnBlockBytes) + static_cast<size_t>(gqa) * head_dim * 4 + static_cast<size_t>(head_dim) * 4 + 64;
    const size_t vals = v2 ? values2_bytes(ctx, gqa) : values_unit_bytes(len_max, gqa), head = static_cast<size_t>(kMegaWarps) * 4 * 1024 * 2 + 1024;
    if (vals > need) need = vals;
    if (head > need) need = head;
    return (need + 1023) / 1024 * 1024;
}
// After the small arrays: the norm weights of the next norm (hidden floats) and a copy of every layer's descriptor.
__host__ __device__ constexpr size_t mega_smem_bytes(size_t attn_region, int maxvec, int hidden, int layers) {
    return attn_region + static_cast<size_t>(maxvec) * 4 + (static_cast<size_t>(maxvec) + 15) / 16 * 16 + 4096 +
           (static_cast<size_t>(hidden) * 4 + 15) / 16 * 16 + static_cast<size_t>(layers) * sizeof(MegaLayer);
}

// ---- the token kernel ---------------------------------------------------------------------------------------------------
// Every phase is its own non-inlined function and the kernel body keeps almost nothing alive across the calls (scalars
// that outlive a phase sit in shared memory), so each phase gets the whole register file to itself.

// Views into the dynamic shared memory; recomputed inside every phase from the kernel arguments.
struct MegaSmem {
    int* tab;
    float* y;        // activation vector (max(hidden, q_dim) floats)
    int8_t* a8;      // its int8 codes
    double* sh_d;    // 32 doubles
    float* sh_f;     // 32 floats
    float* pair;     // chunk-combine factors: q_heads * (4 * 2 + 4) floats (q_heads <= kMegaMaxHeads)
    float* scale;    // [0] attention-input scale, [1] o-input scale, [2] ffn-input scale, [3] down-input scale (previous layer)
    int* flag;
    float* w;        // weights of the next norm
    MegaLayer* layers;
};
__device__ __forceinline__ MegaSmem mega_smem_views(unsigned char* smem, const MegaArgs& a) {
    MegaSmem v;
    const int maxvec = max(a.hidden, a.q_dim_full);
    v.tab = reinterpret_cast<int*>(smem);
    v.y = reinterpret_cast<float*>(smem + a.attn_region);
    v.a8 = reinterpret_cast<int8_t*>(v.y + maxvec);
    unsigned char* small = reinterpret_cast<unsigned char*>(v.a8) + (maxvec + 15) / 16 * 16;
    v.sh_d = reinterpret_cast<double*>(small);
    v.sh_f = reinterpret_cast<float*>(small + 256);
    v.pair = reinterpret_cast<float*>(small + 384);
    v.scale = reinterpret_cast<float*>(small + 3968);
    v.flag = reinterpret_cast<int*>(small + 4000);
    v.w = reinterpret_cast<float*>(small + 4096);
    v.layers = reinterpret_cast<MegaLayer*>(small + 4096 + (static_cast<size_t>(a.hidden) * 4 + 15) / 16 * 16);
    return v;
}

__device__ __forceinline__ void prefetch_items(const MegaArgs& a, const MegaLayer& ly, int k) {
    const int tid = threadIdx.x, G = gridDim.x, cta = blockIdx.x;
    if (tid < 2 && cta + tid * G < ly.count[k]) prefetch_l2(a.items + ly.first[k] + cta + tid * G);
}

// Phase A (which = 0) and phase E (which = 1): residual (or embedding), RMSNorm, int8 codes for the projection that follows.
// One block-wide reduction with a single barrier: lane 0 of every warp deposits its warp's value, everybody reads all of
// them. `sh` must not have been read since the last __syncthreads of every thread (the phases alternate the buffers).
__device__ __forceinline__ double block_sum_f64_once(double v, double* sh) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    double t0 = 0.0, t1 = 0.0;
#pragma unroll
    for (int i = 0; i < kMegaWarps; i += 2) {  // two interleaved chains, the same order in every thread
        t0 += sh[i];
        t1 += sh[i + 1];
    }
    return t0 + t1;
}
__device__ __forceinline__ float block_max_f32_once(float v, float* sh) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < kMegaWarps; ++i) t = fmaxf(t, sh[i]);
    return t;
}

constexpr int kNormPer = 8;  // elements of the residual stream a thread keeps in registers: hidden <= 8 * 512

// Phase A (which = 0) and phase E (which = 1) for one GPU and hidden <= 4096: the vector never leaves the registers. Every
// thread owns the elements tid + 512 k; all loads (projection sums and residual stream from L2, norm weights from shared
// memory) are issued before the first use, and the two block-wide reductions (sum of squares in double, maximum) cost
// one barrier each. Same arithmetic as mega_norm_quant.
__device__ __forceinline__ void phase_norm_regs(const MegaArgs& a, const MegaSmem& v, int l, int which) {
    const int tid = threadIdx.x, cta = blockIdx.x, G = gridDim.x, H = a.hidden;
    const MegaLayer& ly = v.layers[l];
    const bool embed = which == 0 && l == 0;
    const float s_prev = which == 0 ? v.scale[3] : v.scale[1];
    const float ws_prev = which == 0 ? (l > 0 ? v.layers[l - 1].ws[6] : 0.0f) : ly.ws[3];
    const bool live = s_prev > 0.0f;
    const float post = live ? __fdiv_rn(ws_prev, s_prev) : 0.0f;
    const int32_t* acc = which == 0 ? a.acc_down : a.acc_o;
    const float* x = which == 0 ? a.xb : a.xa;
    int av[kNormPer];
    float y[kNormPer];
    if (embed) {
        const size_t base = static_cast<size_t>(a.token[0]) * H;
#pragma unroll
        for (int k = 0; k < kNormPer; ++k) {
            const int i = tid + k * kMegaThreads;
            y[k] = i < H ? table_to_float(a.embed[base + i], a.bf16_tables != 0) : 0.0f;
        }
    } else {
#pragma unroll
        for (int k = 0; k < kNormPer; ++k) {
            const int i = tid + k * kMegaThreads;
            av[k] = i < H ? __ldcg(acc + i) : 0;
            y[k] = i < H ? __ldcg(x + i) : 0.0f;
        }
#pragma unroll
        for (int k = 0; k < kNormPer; ++k) y[k] = __fadd_rn(y[k], live ? __fmul_rn(static_cast<float>(av[k]), post) : 0.0f);
    }
    cp_async_wait<0>();  // the norm weights requested one phase ago
    __syncthreads();
    if (which == 1) QTB_FINE(a, 17);
    if (cta == 0) {
        float* keep = which == 0 ? a.xa : a.xb;
#pragma unroll
        for (int k = 0; k < kNormPer; ++k)
            if (tid + k * kMegaThreads < H) keep[tid + k * kMegaThreads] = y[k];
    }
    if (which == 1 && cta == G - 1) {
        const int n = (a.q_heads + 2 * a.kv_heads) * a.head_dim;
        for (int i = tid; i < n; i += kMegaThreads) a.acc_qkv[i] = 0;  // consumed by the scores phase
    }
    double sum = 0.0;
#pragma unroll
    for (int k = 0; k < kNormPer; ++k) sum += static_cast<double>(__fmul_rn(y[k], y[k]));  // elements beyond H are zero
    sum = block_sum_f64_once(sum, v.sh_d);
    if (which == 1) QTB_FINE(a, 18);
    const float mean = __double2float_rn(sum / static_cast<double>(H));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, a.eps)));
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < kNormPer; ++k) {
        const int i = tid + k * kMegaThreads;
        y[k] = i < H ? __fmul_rn(__fmul_rn(y[k], inv), v.w[i]) : 0.0f;
        amax = fmaxf(amax, fabsf(y[k]));
    }
    amax = block_max_f32_once(amax, v.sh_f);
    if (which == 1) QTB_FINE(a, 19);
    const float s = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
#pragma unroll
    for (int k = 0; k < kNormPer; ++k) {
        const int i = tid + k * kMegaThreads;
        if (i < H) v.a8[i] = static_cast<int8_t>(amax > 0.0f ? quantize_code(y[k], s) : 0);
    }
    if (tid == 0) v.scale[which == 0 ? 0 : 2] = s;
    __syncthreads();  // the norm weights are rewritten next
}

// Phase A (which = 0) and phase E (which = 1): residual (or embedding), RMSNorm, int8 codes for the projection that follows.
__device__ __noinline__ bool phase_norm(const MegaArgs& a, int l, int which, unsigned int seq_base, unsigned char* smem) {
    const MegaSmem v = mega_smem_views(smem, a);
    const int tid = threadIdx.x, cta = blockIdx.x, G = gridDim.x, H = a.hidden;
    const MegaLayer& ly = v.layers[l];
    prefetch_items(a, ly, which == 0 ? 0 : 2);
    if (which == 1) QTB_FINE(a, 16);

    if (a.tp_world == 1 && H <= kNormPer * kMegaThreads) {
        phase_norm_regs(a, v, l, which);
    } else {
        if (which == 0) {
            if (l == 0) {
                const size_t base = static_cast<size_t>(a.token[0]) * H;
                for (int i = tid; i < H; i += kMegaThreads) v.y[i] = table_to_float(a.embed[base + i], a.bf16_tables != 0);
            } else {
                const float s_prev = v.scale[3];
                const float post = s_prev > 0.0f ? __fdiv_rn(v.layers[l - 1].ws[6], s_prev) : 0.0f;
                if (a.tp_world > 1)  // the down results of the previous layer, from every rank
                    residual_add_ll(v.y, a.xb, reinterpret_cast<const uint2*>(a.tp_box[a.tp_rank] + a.box_acc_down), seq_base + 4u * l, a, post,
                                    s_prev > 0.0f, H);
                else
                    residual_add(v.y, a.xb, a.acc_down, post, s_prev > 0.0f, H);
            }
        } else {
            const float s_q = v.scale[1];
            const float post = s_q > 0.0f ? __fdiv_rn(ly.ws[3], s_q) : 0.0f;
            if (a.tp_world > 1)  // the o results of this layer, from every rank
                residual_add_ll(v.y, a.xa, reinterpret_cast<const uint2*>(a.tp_box[a.tp_rank] + a.box_acc_o), seq_base + 4u * l + 2u, a, post,
                                s_q > 0.0f, H);
            else
                residual_add(v.y, a.xa, a.acc_o, post, s_q > 0.0f, H);
        }
        cp_async_wait<0>();  // the norm weights requested one phase ago
        __syncthreads();
        if (which == 1) QTB_FINE(a, 17);
        if (cta == 0) {
            float* keep = which == 0 ? a.xa : a.xb;
            for (int i = tid; i < H; i += kMegaThreads) keep[i] = v.y[i];
        }
        if (which == 1 && cta == G - 1) {
            const int n = (a.q_heads + 2 * a.kv_heads) * a.head_dim;
            for (int i = tid; i < n; i += kMegaThreads) a.acc_qkv[i] = 0;  // consumed by the scores phase
        }
        const float s = mega_norm_quant(v.y, v.w, H, a.eps, v.a8, v.sh_d, v.sh_f, which == 1 ? &a : nullptr);
        if (tid == 0) v.scale[which == 0 ? 0 : 2] = s;
    }
    if (which == 1) QTB_FINE(a, 20);
    if (which == 0)
        request_norm_weights(v.w, ly.ffn_norm, H);
    else
        request_norm_weights(v.w, l + 1 < a.n_layers ? v.layers[l + 1].attn_norm : a.out_norm, H);
    prefetch_items(a, ly, which == 0 ? 1 : 3);
    __syncthreads();
    return true;
}

// Phase C1: scores, key rows shared out evenly over the CTAs; a spare CTA clears buffers that are idle now.
__device__ __noinline__ void phase_scores(const MegaArgs& a, int l, unsigned char* smem) {
    const MegaSmem v = mega_smem_views(smem, a);
    const int tid = threadIdx.x, cta = blockIdx.x, G = gridDim.x;
    const MegaLayer& ly = v.layers[l];
    const KvSplit ks = kv_split(a);
    int R = (a.kv_heads * ks.seq_len + G - 1) / G;
    R = max(16, min(R, kAttnBlockPos));
    const int per_head = (ks.seq_len + R - 1) / R;
    const float s_h = v.scale[0];
    for (int u = cta; u < a.kv_heads * per_head; u += G) {
        const int kvh = u / per_head, r0 = (u - kvh * per_head) * R;
        mega_scores_unit(a, ly, kvh, r0, min(R, ks.seq_len - r0), s_h, smem);
    }
    if (cta == G - 1) {
        for (int i = tid; i < a.hidden; i += kMegaThreads) a.acc_down[i] = 0;  // read by every CTA in phase A, rewritten by down
        if (tid == 0) {
            a.amax_bits[(l + 1) & 1] = 0u;
            a.amax_bits[2 + ((l + 1) & 1)] = 0u;  // the attention output's maximum of the next layer
        }
    }
}

// Phase C2: softmax factors and value accumulation per (KV head, chunk, 32-coordinate slice).
__device__ __noinline__ void phase_values(const MegaArgs& a, int l, unsigned char* smem) {
    const MegaSmem v = mega_smem_views(smem, a);
    const int cta = blockIdx.x, G = gridDim.x;
    const KvSplit ks = kv_split(a);
    const int nchunks = ks.split ? 4 : 1, slices = a.head_dim / kAttnSlice;
    // The value chains are pure latency (one dependent step per position) and leave the memory system idle: the o, gate, up
    // and down weights of this layer are requested into L2 now.
    if (a.l2_prefetch)
        for (int k = 3; k < 7; ++k) prefetch_weights(v.layers[l], k);
    for (int u = cta; u < a.kv_heads * nchunks * slices; u += G) {
        const int slice = u % slices, c = (u / slices) % nchunks, kvh = u / (slices * nchunks);
        mega_values_unit(a, v.layers[l], kvh, c, slice, smem);
    }
}

// Phase C2, second form: one unit per (KV head, 8 coordinates); see mega_values2_unit.
__device__ __noinline__ void phase_values2(const MegaArgs& a, int l, unsigned char* smem) {
    const MegaSmem v = mega_smem_views(smem, a);
    const int slices = a.head_dim / kV2Dims, units = a.kv_heads * slices, G = gridDim.x, cta = blockIdx.x;
    if (cta < units) {  // the host chose this form only if units < gridDim.x
        if (a.f32_values)
            mega_values2_unit<true>(a, v.layers[l], l, cta / slices, cta % slices, smem);
        else
            mega_values2_unit<false>(a, v.layers[l], l, cta / slices, cta % slices, smem);
        return;
    }
    // helpers: the factor tasks, interleaved over the KV heads so that every head's first tasks start at once
    const KvSplit ks = kv_split(a);
    const int nch = ks.split ? 4 : 1, tasks = a.q_heads * nch;
    int done = 0;
    for (int t = cta - units; t < tasks; t += G - units) {
        v2_factors_task(a, t / nch, t % nch, smem);
        ++done;
    }
    if (done) {
        __syncthreads();
        for (int i = threadIdx.x; i < 13 * 64; i += kMegaThreads) {  // the zero rows of the table the tasks wrote over
            const int k = i >> 6;
            reinterpret_cast<int*>(smem)[(k < 9 ? 28 * k + 27 : 243 + k) * 64 + (i & 63)] = 0;
        }
        __syncthreads();
    }
}

// Phase D after phase_values2: the attention output is complete in a.attn_out and, without a sub-norm, so is its maximum;
// every CTA loads the vector into registers, normalises it if the model has an attention sub-norm (attention.rs:234-246)
// and writes the int8 codes of the o projection's input.
__device__ __noinline__ void phase_combine2(const MegaArgs& a, int l, unsigned char* smem) {
    const MegaSmem v = mega_smem_views(smem, a);
    const int tid = threadIdx.x, qd = a.q_heads * a.head_dim;
    QTB_FINE(a, 21);
    float y[kNormPer];
#pragma unroll
    for (int k = 0; k < kNormPer; ++k) {
        const int i = tid + k * kMegaThreads;
        y[k] = i < qd ? __ldcg(a.attn_out + i) : 0.0f;
    }
    float amax;
    if (const float* sub_w = v.layers[l].attn_sub_norm) {
        float w[kNormPer];
#pragma unroll
        for (int k = 0; k < kNormPer; ++k) w[k] = tid + k * kMegaThreads < qd ? __ldg(sub_w + tid + k * kMegaThreads) : 0.0f;
        double sum = 0.0;
#pragma unroll
        for (int k = 0; k < kNormPer; ++k) sum += static_cast<double>(__fmul_rn(y[k], y[k]));
        sum = block_sum_f64_once(sum, v.sh_d);
        const float mean = __double2float_rn(sum / static_cast<double>(qd));
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, a.eps)));
        amax = 0.0f;
#pragma unroll
        for (int k = 0; k < kNormPer; ++k) {
            y[k] = __fmul_rn(__fmul_rn(y[k], inv), w[k]);
            amax = fmaxf(amax, fabsf(y[k]));
        }
        amax = block_max_f32_once(amax, v.sh_f);
    } else {
        amax = __uint_as_float(__ldcg(a.amax_bits + 2 + (l & 1)));
    }
    QTB_FINE(a, 23);
    const float s_q = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
#pragma unroll
    for (int k = 0; k < kNormPer; ++k) {
        const int i = tid + k * kMegaThreads;
        if (i < qd) v.a8[i] = static_cast<int8_t>(amax > 0.0f ? quantize_code(y[k], s_q) : 0);
    }
    if (tid == 0) v.scale[1] = s_q;
    __syncthreads();
    QTB_FINE(a, 24);
}

// Phase D: combine the chunks of every head (attention.rs:497-541), int8 codes for the o projection.
__device__ __noinline__ bool phase_combine(const MegaArgs& a, int l, unsigned int seq, unsigned char* smem) {
    const MegaSmem v = mega_smem_views(smem, a);
    const int tid = threadIdx.x, hd = a.head_dim, qd = a.q_heads * hd;
    float* s_pair = v.pair;
    const KvSplit ks = kv_split(a);
    QTB_FINE(a, 21);
    // every chunk value of a thread's coordinates is requested before the factors are needed
    float amax = 0.0f;
    for (int base = 0; base < qd; base += 4 * kMegaThreads) {  // uniform trip count: the loop holds a barrier
        const int i0 = base + tid;
        float pv[4][4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = i0 + k * kMegaThreads;
            const int h = i / hd, d = i - h * hd;
            const float* pa = a.part_acc + static_cast<size_t>(h) * 4 * hd + d;
#pragma unroll
            for (int c = 0; c < 4; ++c) pv[k][c] = (i < qd && (c == 0 || ks.split)) ? __ldcg(pa + c * hd) : 0.0f;
        }
        if (base == 0) {
            // Per head: the factors of every chunk in the order of attention.rs:510-541 (computed after the loads above were
            // issued, so that the two round trips to L2 overlap). The running maximum before chunk c is the maximum of the
            // earlier non-empty chunks, so the eight exponentials of a head are independent: one thread each.
            if (!ks.split) {
                if (tid < a.q_heads) {
                    const float S = __ldcg(a.part_ms + static_cast<size_t>(tid) * 8 + 1);
                    s_pair[tid * 8] = S == 0.0f ? 0.0f : __fdiv_rn(1.0f, S);
                }
            } else if (tid < a.q_heads * 8) {
                const int h = tid >> 3, c = (tid >> 1) & 3, which = tid & 1;
                float pm[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) pm[k] = __ldcg(a.part_ms + static_cast<size_t>(h) * 8 + k);
                float m_before = -INFINITY;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if (k < c && pm[2 * k + 1] != 0.0f) m_before = fmaxf(m_before, pm[2 * k]);
                const float m_chunk = pm[2 * c], s_chunk = pm[2 * c + 1];
                const float m_new = fmaxf(m_before, m_chunk);
                float f = device_expf(__fsub_rn(which == 0 ? m_before : m_chunk, m_new));
                if (s_chunk == 0.0f) f = which == 0 ? -1.0f : 0.0f;  // a negative scale_old marks a skipped chunk
                s_pair[h * 8 + 2 * c + which] = f;                    // [c][0] = scale_old, [c][1] = scale_new
                if (which == 0) s_pair[a.q_heads * 8 + h * 4 + c] = s_chunk;
            }
            __syncthreads();  // the factors are written
            QTB_FINE(a, 22);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = i0 + k * kMegaThreads;
            if (i >= qd) continue;
            const int h = i / hd;
            const float* pr = s_pair + h * 8;
            float out;
            if (!ks.split) {
                out = __fmul_rn(pv[k][0], pr[0]);
            } else {
                float acc = 0.0f, s_final = 0.0f;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (pr[2 * c] < 0.0f) continue;
                    acc = __fmaf_rn(acc, pr[2 * c], __fmul_rn(pv[k][c], pr[2 * c + 1]));
                    s_final = __fmaf_rn(s_final, pr[2 * c], __fmul_rn(s_pair[a.q_heads * 8 + h * 4 + c], pr[2 * c + 1]));
                }
                out = s_final != 0.0f ? __fmul_rn(acc, __fdiv_rn(1.0f, s_final)) : acc;
            }
            v.y[i] = out;
            amax = fmaxf(amax, fabsf(out));
        }
    }
    QTB_FINE(a, 23);
    int n_all = qd;
    if (a.tp_world > 1 && !a.attn_replicated) {
        // this rank's heads are a slice of the attention output: CTA p sends it to rank p, then every CTA takes the whole
        // vector from the own box as the pairs arrive
        __syncthreads();
        if (blockIdx.x < a.tp_world) {
            uint2* dst = reinterpret_cast<uint2*>(a.tp_box[blockIdx.x] + a.box_y) + a.tp_rank * qd;
            for (int i = tid; i < qd; i += kMegaThreads) ll_store(dst + i, __float_as_uint(v.y[i]), seq);
        }
        __syncthreads();
        n_all = a.q_dim_full;
        const uint2* all = reinterpret_cast<const uint2*>(a.tp_box[a.tp_rank] + a.box_y);
        amax = 0.0f;
        for (int i0 = tid; i0 < n_all; i0 += 8 * kMegaThreads) {
            uint2 pr[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) pr[k] = i0 + k * kMegaThreads < n_all ? ll_peek(all + i0 + k * kMegaThreads) : make_uint2(0u, seq);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int i = i0 + k * kMegaThreads;
                if (i >= n_all) continue;
                const float y = __uint_as_float(pr[k].y == seq ? pr[k].x : ll_load(all + i, seq, a));
                v.y[i] = y;
                amax = fmaxf(amax, fabsf(y));
            }
        }
    }
    if (const float* sub_w = v.layers[l].attn_sub_norm) {  // BitNet: RMSNorm of the attention output (attention.rs:234-246)
        double sum = 0.0;
        for (int i = tid; i < n_all; i += kMegaThreads) sum += static_cast<double>(__fmul_rn(v.y[i], v.y[i]));
        sum = block_sum_f64(sum, v.sh_d);
        const float mean = __double2float_rn(sum / static_cast<double>(n_all));
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, a.eps)));
        amax = 0.0f;
        for (int i = tid; i < n_all; i += kMegaThreads) {
            const float y = __fmul_rn(__fmul_rn(v.y[i], inv), __ldg(sub_w + i));
            v.y[i] = y;
            amax = fmaxf(amax, fabsf(y));
        }
    }
    amax = block_max_f32(amax, v.sh_f);
    const float s_q = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    for (int i = tid; i < n_all; i += kMegaThreads) v.a8[i] = static_cast<int8_t>(amax > 0.0f ? quantize_code(v.y[i], s_q) : 0);
    if (tid == 0) v.scale[1] = s_q;
    __syncthreads();
    QTB_FINE(a, 24);
    return true;
}

// Phase F1: SwiGLU on this CTA's slice of the intermediate vector, maximum of |v| for the down projection's scale.
__device__ __noinline__ void phase_swiglu(const MegaArgs& a, int l, unsigned char* smem) {
    const MegaSmem v = mega_smem_views(smem, a);
    const int tid = threadIdx.x, cta = blockIdx.x, G = gridDim.x, I = a.inter;
    const MegaLayer& ly = v.layers[l];
    const float s_f = v.scale[2];
    const float pg = s_f > 0.0f ? __fdiv_rn(ly.ws[4], s_f) : 0.0f, pu = s_f > 0.0f ? __fdiv_rn(ly.ws[5], s_f) : 0.0f;
    float m = 0.0f;
    // with tensor parallelism this rank's slice of the intermediate vector goes into the box of every rank
    const int first = a.tp_world > 1 ? a.tp_rank * I : 0;
    auto store = [&](int i, float x) {
        if (a.tp_world > 1) {
            for (int p = 0; p < a.tp_world; ++p) reinterpret_cast<float*>(a.tp_box[p] + a.box_v)[first + i] = x;
        } else {
            a.v_inter[i] = x;
        }
    };
    const bool relu2 = a.relu2 != 0;
    auto act = [&](float g, float u) {  // SwiGLU (ops.rs:427-464) or relu(gate)^2 * up (ops.rs:301-308, 467-473)
        if (!relu2) return __fmul_rn(ggml_silu(g), u);
        const float r = g > 0.0f ? g : 0.0f;
        return __fmul_rn(__fmul_rn(r, r), u);
    };
    double sq = 0.0;  // BitNet FFN sub-norm: this thread's share of the sum of squares
    for (int i0 = cta * kMegaThreads + tid; i0 < I; i0 += 2 * G * kMegaThreads) {
        const int i1 = i0 + G * kMegaThreads;
        const int g0 = __ldcg(a.acc_gu + i0), u0 = __ldcg(a.acc_gu + I + i0);
        const int g1 = i1 < I ? __ldcg(a.acc_gu + i1) : 0, u1 = i1 < I ? __ldcg(a.acc_gu + I + i1) : 0;
        {
            const float g = s_f > 0.0f ? __fmul_rn(static_cast<float>(g0), pg) : 0.0f, u = s_f > 0.0f ? __fmul_rn(static_cast<float>(u0), pu) : 0.0f;
            const float x = act(g, u);
            store(i0, x);
            m = fmaxf(m, fabsf(x));
            sq += static_cast<double>(__fmul_rn(x, x));
        }
        if (i1 < I) {
            const float g = s_f > 0.0f ? __fmul_rn(static_cast<float>(g1), pg) : 0.0f, u = s_f > 0.0f ? __fmul_rn(static_cast<float>(u1), pu) : 0.0f;
            const float x = act(g, u);
            store(i1, x);
            m = fmaxf(m, fabsf(x));
            sq += static_cast<double>(__fmul_rn(x, x));
        }
    }
    if (a.tp_world > 1) __threadfence_system();  // the stores to the other boxes precede the barrier that follows
    if (ly.ffn_sub_norm != nullptr) {  // the maximum is taken after the sub-norm (phase_ffn_sub_norm); here only the partial sum
        sq = block_sum_f64(sq, v.sh_d);
        if (tid == 0) a.sumsq_part[cta] = sq;
    } else {
        m = block_max_f32(m, v.sh_f);
        if (tid == 0 && m > 0.0f) atomicMax(a.amax_bits + (l & 1), __float_as_uint(m));  // non-negative floats order like their bits
    }
    if (cta == G - 1)
        for (int i = tid; i < a.hidden; i += kMegaThreads) a.acc_o[i] = 0;  // consumed in phase E
}

// BitNet, after phase_swiglu and a grid barrier: RMSNorm of the gated activations (model.rs:219-224). Every CTA adds the
// per-CTA sums of squares in the same order, normalises its own slice in place and contributes to the maximum.
__device__ __noinline__ void phase_ffn_sub_norm(const MegaArgs& a, int l, unsigned char* smem) {
    const MegaSmem v = mega_smem_views(smem, a);
    const int tid = threadIdx.x, cta = blockIdx.x, G = gridDim.x, I = a.inter;
    const float* w = v.layers[l].ffn_sub_norm;
    // the per-CTA partial sums: fetched by one thread each (one L2 round trip in all), then added by every thread in the
    // same fixed order (four interleaved chains)
    double* s_part = reinterpret_cast<double*>(v.y);  // the activation vector is not in use between SwiGLU and down
    for (int c = tid; c < G; c += kMegaThreads) s_part[c] = __ldcg(a.sumsq_part + c);
    __syncthreads();
    double p0 = 0.0, p1 = 0.0, p2 = 0.0, p3 = 0.0;
    int c = 0;
    for (; c + 4 <= G; c += 4) {
        p0 += s_part[c];
        p1 += s_part[c + 1];
        p2 += s_part[c + 2];
        p3 += s_part[c + 3];
    }
    for (; c < G; ++c) p0 += s_part[c];
    const double sum = (p0 + p1) + (p2 + p3);
    const float mean = __double2float_rn(sum / static_cast<double>(I));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, a.eps)));
    float m = 0.0f;
    for (int i = cta * kMegaThreads + tid; i < I; i += G * kMegaThreads) {
        const float y = __fmul_rn(__fmul_rn(a.v_inter[i], inv), __ldg(w + i));
        a.v_inter[i] = y;
        m = fmaxf(m, fabsf(y));
    }
    m = block_max_f32(m, v.sh_f);
    if (tid == 0 && m > 0.0f) atomicMax(a.amax_bits + (l & 1), __float_as_uint(m));
}

// Final norm (model.rs:326-331), output head, greedy candidate of this CTA.
__device__ __noinline__ bool phase_head(const MegaArgs& a, unsigned int seq_base, unsigned char* smem) {
    const MegaSmem v = mega_smem_views(smem, a);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, cta = blockIdx.x, G = gridDim.x, H = a.hidden;
    float* y_s = v.y;
    {
        const float s_prev = v.scale[3];
        const float post = s_prev > 0.0f ? __fdiv_rn(v.layers[a.n_layers - 1].ws[6], s_prev) : 0.0f;
        if (a.tp_world > 1)  // the last layer's down results, from every rank
            residual_add_ll(y_s, a.xb, reinterpret_cast<const uint2*>(a.tp_box[a.tp_rank] + a.box_acc_down), seq_base + 4u * a.n_layers, a, post,
                            s_prev > 0.0f, H);
        else
            residual_add(y_s, a.xb, a.acc_down, post, s_prev > 0.0f, H);
    }
    cp_async_wait<0>();
    __syncthreads();
    mega_norm_quant(y_s, v.w, H, a.eps, nullptr, v.sh_d, v.sh_f);
    const bool bf16 = a.bf16_tables != 0;
    for (int i = tid; i < H; i += kMegaThreads)  // model.rs:347-349; BF16 tables: hybrid.rs:327-333
        y_s[i] = bf16 ? bf16_bits_to_float(float_to_bf16_bits(y_s[i])) : __half2float(__float2half_rn(y_s[i]));
    __syncthreads();
    float bv = -INFINITY;
    unsigned int bi = 0xFFFFFFFFu;
    const int np = H & ~31;
    // Every warp walks its rows in segments of kHeadSeg halves that arrive through a private ring of shared-memory
    // buffers (asynchronous copies, three segments ahead); the table is not needed any more and gives up its space.
    constexpr int kHeadSeg = 1024, kHeadStages = 4;
    __half* ring = reinterpret_cast<__half*>(smem) + warp * kHeadStages * kHeadSeg;
    const int nseg = (np + kHeadSeg - 1) / kHeadSeg;
    const int first_row = cta * kMegaWarps + warp, row_stride = G * kMegaWarps;
    const int nrows = first_row < a.vocab ? (a.vocab - first_row + row_stride - 1) / row_stride : 0;
    const int total = nrows * nseg;
    auto issue = [&](int q) {
        if (q < total) {
            const int row = first_row + (q / nseg) * row_stride, sg = q % nseg;
            const __half* src = a.lm_head + static_cast<size_t>(row) * H + sg * kHeadSeg;
            __half* dst = ring + (q % kHeadStages) * kHeadSeg;
            const int nvec = min(kHeadSeg, np - sg * kHeadSeg) / 8;
            for (int x = lane; x < nvec; x += 32) cp_async16(dst + x * 8, src + x * 8);
        }
        cp_async_commit();
    };
    for (int q = 0; q < kHeadStages - 1; ++q) issue(q);
    float acc = 0.0f;
    for (int q = 0; q < total; ++q) {
        issue(q + kHeadStages - 1);
        cp_async_wait<kHeadStages - 1>();
        __syncwarp();
        const int sg = q % nseg;
        const __half* buf = ring + (q % kHeadStages) * kHeadSeg;
        const float* xs = y_s + sg * kHeadSeg;
        const int cnt = min(kHeadSeg, np - sg * kHeadSeg);
        if (bf16) {  // ggml_vec_dot_bf16: product and sum rounded separately
#pragma unroll 8
            for (int i = 0; i < cnt; i += 32) acc = __fadd_rn(acc, __fmul_rn(xs[i + lane], bf16_bits_to_float(__half_as_ushort(buf[i + lane]))));
        } else {
#pragma unroll 8
            for (int i = 0; i < cnt; i += 32) acc = __fmaf_rn(xs[i + lane], __half2float(buf[i + lane]), acc);
        }
        if (sg == nseg - 1) {
            const int row = first_row + (q / nseg) * row_stride;
            const float sum = bf16 ? dot_lane_reduce_bf16(acc) : dot_lane_reduce_f16(acc);  // hidden is a multiple of 32: no tail
            if (lane == 0) {
                a.logits[row] = sum;
                argmax_merge(bv, bi, sum, static_cast<unsigned int>(row + a.vocab_base));
            }
            acc = 0.0f;
        }
        __syncwarp();  // the buffer is refilled three segments later
    }
    cp_async_wait<0>();
    __syncthreads();
    if (a.l2_prefetch && a.n_layers > 0)  // the next token starts with the first layer's attention projections
        for (int k = 0; k < 3; ++k) prefetch_weights(v.layers[0], k);
    float* s_bv = v.sh_f;  // 32 floats: one candidate per warp
    unsigned int* s_bi = reinterpret_cast<unsigned int*>(v.sh_d);
    if (lane == 0) {
        s_bv[warp] = bv;
        s_bi[warp] = bi;
    }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < kMegaWarps; ++w) argmax_merge(bv, bi, s_bv[w], s_bi[w]);
        a.best_val[cta] = bv;
        a.best_idx[cta] = bi;
    }
    return true;
}

// Last step, CTA 0 after the final barrier: the greedy token (lowest index among equal maxima), position advance, clean-up.
// With tensor parallelism every rank first tells every other rank the best row of its vocabulary slice.
__device__ __noinline__ void phase_finish(const MegaArgs& a, unsigned int seq_base, unsigned char* smem) {
    const MegaSmem v = mega_smem_views(smem, a);
    const int tid = threadIdx.x, G = gridDim.x;
    // no static shared memory anywhere in this kernel: it would move the dynamic base the table addresses are built on
    float& s_best_v = v.sh_f[0];
    unsigned int& s_best_i = reinterpret_cast<unsigned int*>(v.sh_f)[1];
    for (int i = tid; i < a.hidden; i += kMegaThreads) a.acc_down[i] = 0;
    if (tid == 0) {
        float bv = -INFINITY;
        unsigned int bi = 0xFFFFFFFFu;
        for (int c = 0; c < G; ++c) argmax_merge(bv, bi, __ldcg(a.best_val + c), __ldcg(a.best_idx + c));
        s_best_v = bv;
        s_best_i = bi;
    }
    if (a.tp_world > 1) {
        const unsigned int seq = seq_base + 4u * a.n_layers + 1u;
        __syncthreads();
        if (tid < a.tp_world) {
            uint2* dst = reinterpret_cast<uint2*>(a.tp_box[tid] + a.box_best) + 2 * a.tp_rank;
            ll_store(dst, __float_as_uint(s_best_v), seq);
            ll_store(dst + 1, s_best_i, seq);
        }
        __syncthreads();
        if (tid == 0) {
            const uint2* all = reinterpret_cast<const uint2*>(a.tp_box[a.tp_rank] + a.box_best);
            float bv = -INFINITY;
            unsigned int bi = 0xFFFFFFFFu;
            for (int r = 0; r < a.tp_world; ++r) {
                const float rv = __uint_as_float(ll_load(all + 2 * r, seq, a));
                argmax_merge(bv, bi, rv, ll_load(all + 2 * r + 1, seq, a));
            }
            s_best_v = bv;
            s_best_i = bi;
            *a.tp_seq = seq;
        }
    }
    if (tid == 0) {
        const unsigned int bi = s_best_i;
        const uint32_t tok = bi == 0xFFFFFFFFu ? 0u : bi;
        a.token[0] = tok;
        a.history[a.pos[0]] = tok;
        a.pos[0] += 1;
        a.amax_bits[0] = 0u;
        a.amax_bits[1] = 0u;
        a.amax_bits[2] = 0u;
        a.amax_bits[3] = 0u;
        if (a.attn_v2)
            for (int k = 0; k < a.kv_heads; ++k) a.fac_done[k] = 0u;
    }
}

template <uint32_t BASE>
__global__ void __launch_bounds__(kMegaThreads, 1) decode_token_kernel(const __grid_constant__ MegaArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, cta = blockIdx.x, G = gridDim.x;
    if (static_cast<uint32_t>(__cvta_generic_to_shared(smem)) != BASE) {
        if (tid == 0) atomicMax(a.status, 1u);
        return;
    }
    {
        const MegaSmem v = mega_smem_views(smem, a);
        for (int i = tid; i < 13 * 64; i += kMegaThreads) {  // byte values that are no velurex code look up zero
            const int k = i >> 6;
            v.tab[(k < 9 ? 28 * k + 27 : 243 + k) * 64 + (i & 63)] = 0;
        }
        request_norm_weights(v.w, a.n_layers > 0 ? a.layers[0].attn_norm : a.out_norm, a.hidden);
        for (int i = tid; i < a.n_layers * static_cast<int>(sizeof(MegaLayer) / 4); i += kMegaThreads)
            reinterpret_cast<uint32_t*>(v.layers)[i] = reinterpret_cast<const uint32_t*>(a.layers)[i];
        if (tid < 4) v.scale[tid] = 0.0f;
        __syncthreads();
        if (a.l2_prefetch && a.n_layers > 0)
            for (int k = 0; k < 3; ++k) prefetch_weights(v.layers[0], k);  // the first layer's q, k and v
    }
    unsigned int bar_round = 0;
#define MEGA_BARRIER()                                                                                   \
    do {                                                                                                 \
        if (!grid_barrier(a.bar, ++bar_round, a.status, mega_smem_views(smem, a).flag)) return;          \
    } while (0)
    int trace_n = 0;
#define MEGA_TRACE()                                                                            \
    do {                                                                                        \
        if (a.trace != nullptr && cta == 0 && tid == 0) a.trace[trace_n++] = static_cast<unsigned long long>(clock64()); \
    } while (0)
#define MEGA_GEMV(k, acts, actf, qs, out)                                                                                        \
    do {                                                                                                                         \
        const MegaSmem v = mega_smem_views(smem, a);                                                                             \
        mega_gemv<BASE>(a.items, v.layers[l].first[k], v.layers[l].count[k], v.tab, acts, actf, qs, out);                         \
    } while (0)
    // Stamps are the SM's cycle counter (reading it costs a few cycles; the global timer costs most of a microsecond per
    // read); the global timer is read once at either end so that the host can convert cycles to nanoseconds.
    if (a.trace != nullptr && cta == 0 && tid == 0) a.trace[a.n_layers * 14 + 4 + 32] = global_timer_ns();
    MEGA_TRACE();
    const bool tp = a.tp_world > 1;
    const unsigned int seq_base = tp ? __ldcg(a.tp_seq) : 0u;  // exchange numbers of this launch: seq_base + 4 l + 1..4, then + 4 L + 1
    for (int l = 0; l < a.n_layers; ++l) {
        if (!phase_norm(a, l, 0, seq_base, smem)) return;
        MEGA_TRACE();  // 1: norm done
        MEGA_GEMV(0, v.a8, nullptr, 0.0f, a.acc_qkv);
        MEGA_TRACE();  // 2: q|k|v streamed (this CTA)
        MEGA_BARRIER();
        MEGA_TRACE();  // 3
        phase_scores(a, l, smem);
        MEGA_TRACE();  // 4: scores done (this CTA)
        MEGA_BARRIER();
        if (a.attn_v2) {
            phase_values2(a, l, smem);
            MEGA_TRACE();  // 5: values and chunk combine done (this CTA)
            MEGA_BARRIER();
            MEGA_TRACE();  // 6
            phase_combine2(a, l, smem);
        } else {
            phase_values(a, l, smem);
            MEGA_TRACE();  // 5: values done (this CTA)
            MEGA_BARRIER();
            MEGA_TRACE();  // 6
            if (!phase_combine(a, l, seq_base + 4u * l + 1u, smem)) return;
        }
        MEGA_TRACE();  // 7: combine + quantise done
        MEGA_GEMV(1, v.a8, nullptr, 0.0f, a.acc_o);
        MEGA_BARRIER();
        if (tp && cta < a.tp_world) tp_push_slice(a, reinterpret_cast<const uint32_t*>(a.acc_o), a.box_acc_o, a.h_slice, seq_base + 4u * l + 2u);
        MEGA_TRACE();  // 8
        if (!phase_norm(a, l, 1, seq_base, smem)) return;
        MEGA_TRACE();  // 9: norm done
        MEGA_GEMV(2, v.a8, nullptr, 0.0f, a.acc_gu);
        MEGA_TRACE();  // 10: gate|up streamed (this CTA)
        MEGA_BARRIER();
        MEGA_TRACE();  // 11
        phase_swiglu(a, l, smem);
        MEGA_BARRIER();
        if (a.relu2 != 0 && a.sumsq_part != nullptr && mega_smem_views(smem, a).layers[l].ffn_sub_norm != nullptr) {
            phase_ffn_sub_norm(a, l, smem);
            MEGA_BARRIER();
        }
        MEGA_TRACE();  // 12
        {
            // down, quantising v on the fly with the scale from the maximum every CTA contributed to
            float vmax = __uint_as_float(__ldcg(a.amax_bits + (l & 1)));
            if (tp) {
                // every rank tells every other rank the maximum of its slice; the scale comes from the maximum of all
                const unsigned int seq = seq_base + 4u * l + 3u;
                if (cta < a.tp_world && tid == 0) __threadfence_system();  // behind the SwiGLU stores of every CTA of this rank
                if (cta < a.tp_world && tid == 0) ll_store(reinterpret_cast<uint2*>(a.tp_box[cta] + a.box_amax) + a.tp_rank, __float_as_uint(vmax), seq);
                const uint2* all = reinterpret_cast<const uint2*>(a.tp_box[a.tp_rank] + a.box_amax);
                vmax = 0.0f;
                for (int r = 0; r < a.tp_world; ++r) vmax = fmaxf(vmax, __uint_as_float(ll_load(all + r, seq, a)));
            }
            const float s_down = vmax > 0.0f ? __fdiv_rn(127.0f, vmax) : 0.0f;
            if (tid == 0) mega_smem_views(smem, a).scale[3] = s_down;
            if (a.l2_prefetch && l + 1 < a.n_layers)  // the next layer's q, k and v while down streams from L2
                for (int k = 0; k < 3; ++k) prefetch_weights(mega_smem_views(smem, a).layers[l + 1], k);
            MEGA_GEMV(3, nullptr, a.v_inter, s_down, a.acc_down);
            MEGA_TRACE();  // 13: down streamed (this CTA)
            for (int i = cta * kMegaThreads + tid; i < 2 * a.inter; i += G * kMegaThreads) a.acc_gu[i] = 0;  // consumed by SwiGLU
        }
        MEGA_BARRIER();
        if (tp && cta < a.tp_world) tp_push_slice(a, reinterpret_cast<const uint32_t*>(a.acc_down), a.box_acc_down, a.h_slice, seq_base + 4u * l + 4u);
        MEGA_TRACE();  // 14 = 0 of the next layer
    }
    if (!phase_head(a, seq_base, smem)) return;
    MEGA_TRACE();  // head done (this CTA)
    MEGA_BARRIER();
    MEGA_TRACE();
    if (a.trace != nullptr && cta == 0 && tid == 0) a.trace[a.n_layers * 14 + 4 + 33] = global_timer_ns();
    if (cta == 0) phase_finish(a, seq_base, smem);
#undef MEGA_GEMV
#undef MEGA_BARRIER
#undef MEGA_TRACE
}

// Self-test of the barrier's give-up path (quintrit_b200_selftest_barrier): a few CTAs, all resident, wait at a barrier
// whose target is twice the arrivals the grid can deliver, with a short poll limit. The wait runs out, status becomes
// 2, the failure bit releases the other waiters, and a second barrier returns false at once. out[cta] = 1 for every CTA
// whose two barriers both reported the failure. Nothing faults and nothing spins beyond the limit.
__global__ void barrier_selftest_kernel(unsigned int* bar, unsigned int* status, unsigned int spin_limit, unsigned int* out) {
    __shared__ int s_flag;
    const bool first = grid_barrier(bar, 2u, status, &s_flag, spin_limit);   // the first barrier asks for twice the arrivals there are
    const bool second = grid_barrier(bar, 4u, status, &s_flag, spin_limit);
    if (threadIdx.x == 0) out[blockIdx.x] = (!first && !second) ? 1u : 0u;
}

}  // namespace qtb
