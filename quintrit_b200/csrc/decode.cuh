// Float kernels of one decoded token (everything around the ternary GEMVs), written so that every value equals the
// reference CPU runtime's bit for bit: rust/crates/quintrit-runtime/src/{ops.rs, attention.rs, model.rs}. The existing
// sm_80 GPU twins in the reference are rust/crates/quintrit-cuda/kernels/layer.cu:21-580.
//
// Rules that keep the bits: no fused multiply-add unless the reference has one (explicit __fmaf_rn / __fmul_rn /
// __fadd_rn / __fdiv_rn / __fsqrt_rn everywhere), the reference's reduction orders for the half dot products, the host
// libm's cos/sin/pow through a table built on the host, glibc's expf restated in double (device_expf), F16 rounding
// after every step of the attention accumulator.
#pragma once
#include <cooperative_groups.h>
#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace qtb {

constexpr int kRowThreads = 1024;  // one block walks a whole activation vector

// ---- block reductions (all threads get the result) ------------------------------------------------------------------
__device__ __forceinline__ double block_sum_f64(double v, double* sh) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[w] = v;
    __syncthreads();
    double t = 0.0;
    for (int i = 0; i < nw; ++i) t += sh[i];
    return t;
}
__device__ __forceinline__ float block_max_f32(float v, float* sh) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[w] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < nw; ++i) t = fmaxf(t, sh[i]);
    return t;
}

// ---- glibc expf (ops: attention.rs:423-428 call f32::exp = the platform libm) ---------------------------------------
// The published table algorithm of glibc's single-precision exp: N = 32 entries of 2^(i/N) (bits, minus i << 47), a
// cubic evaluated in double. The table is filled by the host (exp2_table_bits) so that no constant list is copied.
__device__ __constant__ unsigned long long c_exp2_tab[32];

__device__ __forceinline__ float device_expf(float x) {
    const double inv_ln2_n = 0x1.71547652b82fep0 * 32.0, shift = 0x1.8p52;
    const double c0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0, c1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0, c2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    const uint32_t ix = __float_as_uint(x), abstop = (ix >> 20) & 0x7ffu;
    if (abstop >= 0x42bu) {
        if (ix == 0xff800000u) return 0.0f;
        if (abstop >= 0x7f8u) return __fadd_rn(x, x);
        if (x > 0x1.62e42ep6f) return __uint_as_float(0x7f800000u);
        if (x < -0x1.9fe368p6f) return 0.0f;
    }
    const double xd = static_cast<double>(x);
    const double z0 = __dmul_rn(inv_ln2_n, xd);
    double kd = __dadd_rn(z0, shift);
    const unsigned long long ki = static_cast<unsigned long long>(__double_as_longlong(kd));
    kd = __dsub_rn(kd, shift);
    const double r = __dsub_rn(z0, kd);
    const unsigned long long t = c_exp2_tab[ki & 31ull] + (ki << 47);
    const double s = __longlong_as_double(static_cast<long long>(t));
    const double z = __fma_rn(c0, r, c1);
    const double r2 = __dmul_rn(r, r);
    double y = __fma_rn(c2, r, 1.0);
    y = __fma_rn(z, r2, y);
    y = __dmul_rn(y, s);
    return __double2float_rn(y);
}

// ---- ggml's vector expf, one lane (ops.rs:316-387), and SiLU (ops.rs:389-399) ---------------------------------------
__device__ __forceinline__ float ggml_expf_lane(float x) {
    const float r = __uint_as_float(0x4b400000u);
    const float z = __fmaf_rn(x, __uint_as_float(0x3fb8aa3bu), r);
    const float n = __fsub_rn(z, r);
    const float b = __fmaf_rn(-n, __uint_as_float(0x35bfbe8eu), __fmaf_rn(-n, __uint_as_float(0x3f317200u), x));
    const uint32_t e = __float_as_uint(z) << 23;
    const float k = __uint_as_float(e + 0x3f800000u);
    const bool c = fabsf(n) > 126.0f;
    const float u = __fmul_rn(b, b);
    const float j = __fmaf_rn(__fmaf_rn(__fmaf_rn(__uint_as_float(0x3c072010u), b, __uint_as_float(0x3d2b9f17u)), u,
                                        __fmaf_rn(__uint_as_float(0x3e2aaf33u), b, __uint_as_float(0x3efffedbu))),
                              u, __fmul_rn(__uint_as_float(0x3f7ffff6u), b));
    if (!c) return __fmaf_rn(j, k, k);
    const uint32_t g = (n <= 0.0f) ? 0x82000000u : 0u;
    const float s1 = __uint_as_float(g + 0x7f000000u);
    const float s2 = __uint_as_float(e - g);
    if (fabsf(n) > 192.0f) return __fmul_rn(s1, s1);
    return __fmul_rn(__fmaf_rn(s2, j, s2), s1);
}
__device__ __forceinline__ float ggml_silu(float x) {
    return __fdiv_rn(x, __fadd_rn(1.0f, ggml_expf_lane(__fsub_rn(0.0f, x))));
}

// ---- BF16 tables (ops.rs:650-664): widening is a shift; narrowing rounds to nearest even and keeps a NaN quiet --------
__device__ __forceinline__ float bf16_bits_to_float(unsigned short h) { return __uint_as_float(static_cast<uint32_t>(h) << 16); }
__device__ __forceinline__ unsigned short float_to_bf16_bits(float f) {
    const uint32_t u = __float_as_uint(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return static_cast<unsigned short>((u >> 16) | 64u);
    return static_cast<unsigned short>((u + (0x7FFFu + ((u >> 16) & 1u))) >> 16);
}
// A table entry (F16 or BF16 bit pattern) as float.
__device__ __forceinline__ float table_to_float(__half h, bool bf16) { return bf16 ? bf16_bits_to_float(__half_as_ushort(h)) : __half2float(h); }
// ggml_vec_dot_bf16's reduction of the 32 lanes (ops.rs:702-708): (a0+a2)+(a1+a3), g_l = a_{l+4}+a_l, (g0+g2)+(g1+g3).
__device__ __forceinline__ float dot_lane_reduce_bf16(float v) {
    v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 16));
    v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 8));
    v = __fadd_rn(__shfl_down_sync(0xffffffffu, v, 4), v);
    v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 2));
    v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 1));
    return v;  // lane 0
}

// ---- quantisation of a vector held in shared memory, for the projection that follows -------------------------------------
// q8_d == nullptr: per-tensor absmax int8 (ops.rs:241-267), scale to scale_out[0]. Otherwise Q8_0 blocks for a block-scaled
// (Q2_0) projection (ops.rs:898-910): one warp per block of 32 values, d = f16(amax / 127) to q8_d[block], codes rounded to
// nearest even. `amax` is the thread's partial maximum of |y| (used by the per-tensor form only). n is a multiple of 32 in
// the block form. All threads of the block must call it.
// One Q8_0 block (ops.rs:898-910) by one warp: lane i holds value i of block b.
__device__ __forceinline__ void quantize_q8_0_block(float v, int b, int lane, int8_t* q_out, float* q8_d) {
    float m = fabsf(v);
    if (m != m) m = 0.0f;  // f32::max ignores a NaN
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) q8_d[b] = __half2float(__float2half_rn(__fdiv_rn(m, 127.0f)));
    const float id = m != 0.0f ? __fdiv_rn(127.0f, m) : 0.0f;
    const float r = rintf(__fmul_rn(v, id));
    int q = 0;
    if (r == r) q = static_cast<int>(fminf(fmaxf(r, -128.0f), 127.0f));
    q_out[b * 32 + lane] = static_cast<int8_t>(q);
}

__device__ __forceinline__ void quantize_vector(const float* y_s, int n, float amax, int8_t* q_out, float* scale_out, float* q8_d, float* sh_f) {
    const int tid = threadIdx.x, nthreads = blockDim.x;
    if (q8_d != nullptr) {
        const int lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
        for (int b = warp; b < n / 32; b += nwarps) quantize_q8_0_block(y_s[b * 32 + lane], b, lane, q_out, q8_d);
        return;
    }
    amax = block_max_f32(amax, sh_f);
    const float s = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    for (int i = tid; i < n; i += nthreads) {
        float q = 0.0f;
        if (amax > 0.0f) {
            q = roundf(__fmul_rn(y_s[i], s));
            q = q != q ? 0.0f : fminf(fmaxf(q, -128.0f), 127.0f);
        }
        q_out[i] = static_cast<int8_t>(q);
    }
    if (tid == 0) scale_out[0] = s;
}

// ---- several sequences in one launch -------------------------------------------------------------------------------------
// The kernels below take a token index in blockIdx.z. For a prompt chunk, token z sits at position pos[0] + z of the one
// KV cache. For a step of several independent sequences (seq.pos_stride = 1), token z belongs to the sequence
// s = slot[z] (or z without a slot list), sits at position pos[s] and uses the KV cache at cache + s * cache_stride.
struct SeqIndex {
    const uint32_t* slot;     // sequence of token z, or nullptr: z itself
    int pos_stride;           // 0: one sequence, consecutive positions; 1: one position word per sequence
    size_t cache_stride;      // elements between the caches of two sequences (this layer's cache of sequence s = base + s * stride)
};
__device__ __forceinline__ uint32_t seq_of(const SeqIndex& q, unsigned int z) { return q.slot != nullptr ? q.slot[z] : z; }
__device__ __forceinline__ uint32_t seq_position(const SeqIndex& q, const uint32_t* pos, unsigned int z) {
    return q.pos_stride != 0 ? pos[seq_of(q, z)] : pos[0] + z;
}
__device__ __forceinline__ size_t seq_cache_offset(const SeqIndex& q, unsigned int z) {
    return q.pos_stride != 0 ? static_cast<size_t>(seq_of(q, z)) * q.cache_stride : 0;
}

// The int32 sums of a batched projection whose K dimension was split over several blocks: `parts` partial results, part k
// of token z at base + k * part_stride + z * ld. The kernel that consumes the sums adds the parts (integer addition: any
// order gives the same sum) instead of a pass of its own that would. parts = 1 describes sums that are already complete.
struct AccView {
    const int32_t* base;      // nullptr: the consumer reads its plain pointer instead
    int parts;
    size_t part_stride;
    int ld;
};
__device__ __forceinline__ int32_t acc_view_read(const AccView& v, size_t z, int i) {
    const int32_t* p = v.base + z * v.ld + i;
    int32_t sum = p[0];
    for (int k = 1; k < v.parts; ++k) sum += p[static_cast<size_t>(k) * v.part_stride];
    return sum;
}

// ---- embedding row: model.rs:308-317 ---------------------------------------------------------------------------------
// A batch of tokens (prompt ingestion) runs as gridDim.y rows: token[y] -> x[y][hidden].
__global__ void embed_kernel(const __half* __restrict__ table, const uint32_t* __restrict__ token, int hidden, float* __restrict__ x, bool bf16) {
    const size_t base = static_cast<size_t>(token[blockIdx.y]) * hidden;
    x += static_cast<size_t>(blockIdx.y) * hidden;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden; i += gridDim.x * blockDim.x) x[i] = table_to_float(table[base + i], bf16);
}

// Arguments of the fused "finish the previous projection, normalise, quantise" kernel.
struct NormQuantArgs {
    float* x;                 // residual stream (hidden), updated in place when acc_prev != nullptr
    const int32_t* acc_prev;  // int32 sums of the previous o / down projection (hidden), or nullptr
    const float* scale_prev;  // activation scale that projection was fed with
    float ws_prev;            // its weight scale
    const float* norm_w;      // RMSNorm weights (hidden)
    float eps;
    int n;
    int8_t* q_out;            // int8 codes (n), or nullptr: then the normalised vector is written to y_out as F16 bits (final norm)
    float* scale_out;         // activation scale of q_out
    __half* y16_out;          // F16 (or BF16 bits, y16_bf16) of the normalised vector (final norm before the output head)
    bool y16_bf16;
    int32_t* zero_a;          // result buffers of the next projections, cleared here (the GEMV adds into them)
    int zero_a_n;
    int32_t* zero_b;
    int zero_b_n;
    // block-scaled (Q2_0) models: acc_prev holds the previous projection's F32 results, added as they are (model.rs:85,
    // attention.rs:343), and the codes are Q8_0 blocks with their scales in q8_d
    int block_scaled;
    float* q8_d;
    // A batch of tokens (prompt ingestion): token blockIdx.z uses x + z * b_x, acc_prev + z * b_acc, q_out + z * b_q, scale_prev + z and
    // scale_out + z when b_scale is set. All zero for the single-token launches.
    int b_x, b_acc, b_q, b_scale;
    int b_y16;                // stride of y16_out between tokens
    AccView v_prev;           // the previous projection's sums as parts (then acc_prev only marks that there is a previous projection)
};

// x += acc * (ws / s)  (model.rs:85, 202 after layer.rs:143-147), y = rms_norm(x) (ops.rs:62-96), codes = quantise(y)
// (ops.rs:241-267). One block.
__global__ void __launch_bounds__(kRowThreads) norm_quant_kernel(NormQuantArgs a) {
    __shared__ double sh_d[32];
    __shared__ float sh_f[32];
    extern __shared__ float y_s[];  // n floats
    const int tid = threadIdx.x;
    if (blockIdx.z != 0) {
        const size_t z = blockIdx.z;
        a.x += z * a.b_x;
        if (a.acc_prev != nullptr) a.acc_prev += z * a.b_acc;
        if (a.q_out != nullptr) a.q_out += z * a.b_q;
        if (a.y16_out != nullptr) a.y16_out += z * a.b_y16;
        if (a.b_scale) {
            if (a.scale_prev != nullptr) a.scale_prev += z;
            if (a.scale_out != nullptr) a.scale_out += z;
        }
    }
    for (int i = tid; i < a.zero_a_n; i += kRowThreads) a.zero_a[i] = 0;
    for (int i = tid; i < a.zero_b_n; i += kRowThreads) a.zero_b[i] = 0;
    float post = 0.0f;
    bool has_prev = a.acc_prev != nullptr;
    if (has_prev && !a.block_scaled) {
        const float s = a.scale_prev[0];
        post = s > 0.0f ? __fdiv_rn(a.ws_prev, s) : 0.0f;
        if (!(s > 0.0f)) has_prev = false;  // layer.rs:148-150: a zero activation scale gives a zero projection
    }
    float w_early[4];  // the norm weights of this thread's first four elements, requested before the sum instead of after it
#pragma unroll
    for (int k = 0; k < 4; ++k) w_early[k] = tid + k * kRowThreads < a.n ? a.norm_w[tid + k * kRowThreads] : 0.0f;
    double sum = 0.0;
    for (int i = tid; i < a.n; i += kRowThreads) {
        float v = a.x[i];
        if (a.acc_prev != nullptr) {
            const float d = a.block_scaled ? reinterpret_cast<const float*>(a.acc_prev)[i]
                                           : (has_prev ? __fmul_rn(static_cast<float>(a.v_prev.base != nullptr ? acc_view_read(a.v_prev, blockIdx.z, i) : a.acc_prev[i]), post) : 0.0f);
            v = __fadd_rn(v, d);
            a.x[i] = v;
        }
        y_s[i] = v;
        sum += static_cast<double>(__fmul_rn(v, v));
    }
    sum = block_sum_f64(sum, sh_d);
    const float mean = __double2float_rn(sum / static_cast<double>(a.n));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, a.eps)));
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = tid + k * kRowThreads;
        if (i < a.n) {
            const float y = __fmul_rn(__fmul_rn(y_s[i], inv), w_early[k]);
            y_s[i] = y;
            amax = fmaxf(amax, fabsf(y));
        }
    }
    for (int i = tid + 4 * kRowThreads; i < a.n; i += kRowThreads) {
        const float y = __fmul_rn(__fmul_rn(y_s[i], inv), a.norm_w[i]);
        y_s[i] = y;
        amax = fmaxf(amax, fabsf(y));
    }
    if (a.q_out == nullptr) {
        for (int i = tid; i < a.n; i += kRowThreads) a.y16_out[i] = a.y16_bf16 ? __ushort_as_half(float_to_bf16_bits(y_s[i])) : __float2half_rn(y_s[i]);
        return;
    }
    __syncthreads();
    quantize_vector(y_s, a.n, amax, a.q_out, a.scale_out, a.block_scaled ? a.q8_d : nullptr, sh_f);
}

// ---- query/key-norm (attention.rs:282-294): RMSNorm (ops.rs:62-96) of every query head and every key head before RoPE -------
// One warp per head, in place on the projection results (floats: the block-scaled path, the only one that has this step in the
// reference). Heads 0 .. q_heads - 1 are query heads (weights q_w), the rest key heads (k_w); the value rows behind them are left.
__global__ void qk_norm_kernel(float* __restrict__ qkv, int q_heads, int kv_heads, int head_dim, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps) {
    const int head = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (head >= q_heads + kv_heads) return;
    float* x = qkv + static_cast<size_t>(head) * head_dim;  // the key heads follow the query heads in the stacked row
    const float* w = head < q_heads ? q_w : k_w;
    double sum = 0.0;
    for (int i = lane; i < head_dim; i += 32) sum += static_cast<double>(__fmul_rn(x[i], x[i]));
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = __double2float_rn(sum / static_cast<double>(head_dim));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    for (int i = lane; i < head_dim; i += 32) x[i] = __fmul_rn(__fmul_rn(x[i], inv), w[i]);
}

// ---- q/k/v finish: post-scale, RoPE, KV append (attention.rs:171-203, ops.rs:160-221) --------------------------------
struct RopeKvArgs {
    const int32_t* acc;       // stacked q | k | v sums (q_dim + 2 kv_dim)
    const float* act_scale;
    float ws_q, ws_k, ws_v;
    const float* cos_sin;     // [ctx][rope_dims]: cos at 2i, sin at 2i+1, built on the host with the host libm
    const uint32_t* pos;
    int q_dim, kv_dim, head_dim, rope_dims, neox;
    float* q_out;             // rotated query, F32 (q_dim)
    __half* k_cache;          // [ctx][kv_dim] of this layer
    __half* v_cache;
    int block_scaled;         // acc holds the F32 results of block-scaled projections: used as they are
    int b_acc, b_q, b_scale;  // batch of tokens: token blockIdx.z reads acc + z * b_acc and act_scale + z, writes q_out + z * b_q
    SeqIndex seq;             // its position and KV cache
    AccView v_q, v_k, v_v;    // the three projections' sums as parts (v_q.base != nullptr), instead of the stacked acc
};

// Element idx of the stacked q | k | v sums of token z.
__device__ __forceinline__ int32_t rope_acc(const RopeKvArgs& a, int idx) {
    if (a.v_q.base == nullptr) return a.acc[idx];
    if (idx < a.q_dim) return acc_view_read(a.v_q, blockIdx.z, idx);
    if (idx < a.q_dim + a.kv_dim) return acc_view_read(a.v_k, blockIdx.z, idx - a.q_dim);
    return acc_view_read(a.v_v, blockIdx.z, idx - a.q_dim - a.kv_dim);
}

__global__ void rope_kv_kernel(RopeKvArgs a) {
    if (blockIdx.z != 0) {
        const size_t z = blockIdx.z;
        a.acc += z * a.b_acc;
        a.q_out += z * a.b_q;
        if (a.b_scale) a.act_scale += z;
    }
    const float s = a.block_scaled ? 1.0f : a.act_scale[0];
    const bool live = s > 0.0f;
    const float pq = live ? __fdiv_rn(a.ws_q, s) : 0.0f, pk = live ? __fdiv_rn(a.ws_k, s) : 0.0f, pv = live ? __fdiv_rn(a.ws_v, s) : 0.0f;
    const uint32_t pos = seq_position(a.seq, a.pos, blockIdx.z);
    a.k_cache += seq_cache_offset(a.seq, blockIdx.z);
    a.v_cache += seq_cache_offset(a.seq, blockIdx.z);
    const float* cs = a.cos_sin + static_cast<size_t>(pos) * a.rope_dims;
    const int half_pairs = a.rope_dims / 2;
    const int total_pairs = (a.q_dim + a.kv_dim) / 2;
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < total_pairs + a.kv_dim; t += gridDim.x * blockDim.x) {
        if (t >= total_pairs) {  // a value element: scale and append
            const int i = t - total_pairs;
            const float v = a.block_scaled ? reinterpret_cast<const float*>(a.acc)[a.q_dim + a.kv_dim + i]
                                           : (live ? __fmul_rn(static_cast<float>(rope_acc(a, a.q_dim + a.kv_dim + i)), pv) : 0.0f);
            a.v_cache[static_cast<size_t>(pos) * a.kv_dim + i] = __float2half_rn(v);
            continue;
        }
        // pair index within q|k: head h, pair p of head_dim / 2
        const int pairs_per_head = a.head_dim / 2;
        const int h = t / pairs_per_head, p = t % pairs_per_head;
        const bool is_q = h * a.head_dim < a.q_dim;
        const int base = h * a.head_dim;  // offset inside q|k
        int i0, i1;
        bool rot;
        if (a.neox) {  // pairs (i, i + n_dims/2) for i < n_dims/2; the rest passes through in pairs of its own
            if (p < half_pairs) {
                i0 = p;
                i1 = p + half_pairs;
                rot = true;
            } else {
                i0 = a.rope_dims + 2 * (p - half_pairs);
                i1 = i0 + 1;
                rot = false;
            }
        } else {
            i0 = 2 * p;
            i1 = i0 + 1;
            rot = p < half_pairs;
        }
        const float post = is_q ? pq : pk;
        float x0 = a.block_scaled ? reinterpret_cast<const float*>(a.acc)[base + i0] : (live ? __fmul_rn(static_cast<float>(rope_acc(a, base + i0)), post) : 0.0f);
        float x1 = a.block_scaled ? reinterpret_cast<const float*>(a.acc)[base + i1] : (live ? __fmul_rn(static_cast<float>(rope_acc(a, base + i1)), post) : 0.0f);
        if (rot) {
            const int ci = a.neox ? p : p;
            const float c = cs[2 * ci], sn = cs[2 * ci + 1];
            const float r0 = __fmaf_rn(x0, c, -__fmul_rn(x1, sn));
            const float r1 = __fmaf_rn(x0, sn, __fmul_rn(x1, c));
            x0 = r0;
            x1 = r1;
        }
        if (is_q) {
            a.q_out[base + i0] = x0;
            a.q_out[base + i1] = x1;
        } else {
            const size_t at = static_cast<size_t>(pos) * a.kv_dim + (base - a.q_dim);
            a.k_cache[at + i0] = __float2half_rn(x0);
            a.k_cache[at + i1] = __float2half_rn(x1);
        }
    }
}

// ---- attention of one query head over one chunk of the KV axis (attention.rs:402-469) --------------------------------
// Grid (q_heads, chunks), 256 threads. Phase A: scores in the reference's dot-product order (one warp per position,
// lane = accumulator lane). Phase B: running maximum, then ms / vs per position and the S chain. Phase C: the value
// accumulator, one thread per coordinate, strictly in position order (F16 after every step, or F32 for llama.cpp files).
struct AttnArgs {
    const float* q;           // F32 queries (q_dim)
    const __half* k_cache;    // [ctx][kv_dim]
    const __half* v_cache;
    const uint32_t* pos;
    int head_dim, kv_dim, gqa, ctx, f32_values;
    float scale;
    float* part_acc;          // [q_heads][4][head_dim] chunk accumulators (as F32; the F16 ones are widened exactly)
    float* part_ms;           // [q_heads][4][2]: M and S per chunk (S = 0 marks an empty chunk)
    int b_q, b_acc, b_ms;     // batch of tokens: token blockIdx.z uses q + z * b_q, part_acc + z * b_acc, part_ms + z * b_ms
    SeqIndex seq;             // its position and KV cache
};

constexpr int kAttnThreads = 1024;
constexpr int kAttnMaxChunk = 2048;  // positions per chunk held in shared memory (context <= 8192)
constexpr int kAttnTileRows = 32, kAttnTileStages = 6;  // the ring of key / value rows of attention_kernel
__host__ __device__ constexpr size_t attention_smem(int head_dim) { return static_cast<size_t>(kAttnTileStages) * kAttnTileRows * head_dim * 2; }

__device__ __forceinline__ float dot_lane_reduce_f16(float v) {  // (a0+a2)+(a1+a3), fold 4, two horizontal adds
    v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 16));
    v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 8));
    v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 4));
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
    v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 2));
    return v;  // lane 0
}
__device__ __forceinline__ float dot_lane_reduce_f16_f32(float v) {  // (a0+a1)+(a2+a3), lanes ((l0+l4)+(l2+l6))+((l1+l5)+(l3+l7))
    v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 8));
    v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 16));
    v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 4));
    v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 2));
    v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, 1));
    return v;  // lane 0
}

__device__ __forceinline__ void attn_cp16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void attn_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void attn_cp_wait_all_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// Requests tile t (32 rows, those below len) of a chunk's key or value rows into its stage of the ring; always closes a copy
// group, so every thread counts the same groups.
__device__ __forceinline__ void attn_tile_issue(__half* ring, const __half* rows, int t, int len, int hd, int kv_dim, int tid) {
    const int row0 = t * kAttnTileRows;
    if (row0 < len) {
        __half* stage = ring + static_cast<size_t>(t % kAttnTileStages) * kAttnTileRows * hd;
        const int pieces = hd >> 3, n = min(kAttnTileRows, len - row0) * pieces;  // 16-byte pieces
        for (int i = tid; i < n; i += kAttnThreads) {
            const int r = i / pieces, c = i - r * pieces;
            attn_cp16(stage + r * hd + c * 8, rows + static_cast<size_t>(row0 + r) * kv_dim + c * 8);
        }
    }
    attn_cp_commit();
}
__device__ __forceinline__ void attn_tile_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(kAttnTileStages - 2) : "memory"); }

// One query head and one of the four KV chunks per block (attention.rs:402-469), grid (q_heads, 4, tokens), 1024 threads.
// A block waits for memory, not for arithmetic: a chunk of a long context is a few hundred KB of rows read once. So the key
// rows (phase A) and then the value rows (phase C) stream through a ring of six 32-row tiles in shared memory, requested
// five tiles ahead by all threads with 16-byte asynchronous copies: about 80 KB in flight per block.
//  A. warp w forms the score of row w of the tile (the lane order of ggml_vec_dot_f16 / _f16_f32);
//  B. a scan over the scores gives every position its running maximum and from it the factors ms (rescale of what came
//     before) and vs (weight of this row) - the running maximum is a prefix maximum, so the scan gives the sequential values;
//  C. thread d < head_dim runs the chain of coordinate d over the tile's rows, in position order; meanwhile the first lane
//     of the last warp runs the chain of the sum S over the same positions.
// Dynamic shared memory: attention_smem(head_dim).
__global__ void __launch_bounds__(kAttnThreads) attention_kernel(AttnArgs a) {
    __shared__ float s_score[kAttnMaxChunk];  // scores, then vs
    __shared__ float s_ms[kAttnMaxChunk];     // ms
    __shared__ float s_q[256];
    __shared__ float s_tm[kAttnThreads / 32];
    extern __shared__ __align__(16) unsigned char attn_ring_raw[];
    __half* ring = reinterpret_cast<__half*>(attn_ring_raw);
    const int h = blockIdx.x, c = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hd = a.head_dim, kvh = h / a.gqa;
    if (blockIdx.z != 0) {
        const size_t z = blockIdx.z;
        a.q += z * a.b_q;
        a.part_acc += z * a.b_acc;
        a.part_ms += z * a.b_ms;
    }
    const int seq_len = static_cast<int>(seq_position(a.seq, a.pos, blockIdx.z)) + 1;
    a.k_cache += seq_cache_offset(a.seq, blockIdx.z);
    a.v_cache += seq_cache_offset(a.seq, blockIdx.z);
    int n_kv = (seq_len + 255) / 256 * 256;
    if (n_kv < 256) n_kv = 256;
    if (n_kv > a.ctx) n_kv = a.ctx;
    int start = 0, end = seq_len;
    if (n_kv >= 512) {
        const int chunk = (n_kv + 3) / 4;
        start = c * chunk;
        end = min(min(start + chunk, n_kv), seq_len);
    } else if (c > 0) {
        start = end;  // single-chunk case: chunks 1..3 are empty
    }
    float* my_acc = a.part_acc + (static_cast<size_t>(h) * 4 + c) * hd;
    float* my_ms = a.part_ms + (static_cast<size_t>(h) * 4 + c) * 2;
    const int len = end - start;
    if (len <= 0) {
        if (tid == 0) {
            my_ms[0] = -INFINITY;
            my_ms[1] = 0.0f;
        }
        return;
    }
    const __half* krows = a.k_cache + static_cast<size_t>(kvh) * hd + static_cast<size_t>(start) * a.kv_dim;
    const __half* vrows = a.v_cache + static_cast<size_t>(kvh) * hd + static_cast<size_t>(start) * a.kv_dim;
    const int tiles = (len + kAttnTileRows - 1) / kAttnTileRows;
    for (int t = 0; t < kAttnTileStages - 1; ++t) attn_tile_issue(ring, krows, t, len, hd, a.kv_dim, tid);
    // the query: F16-rounded for bitnet.cpp numerics (attention.rs:212-214), F32 for llama.cpp numerics
    if (tid < hd) {
        const float qv = a.q[h * hd + tid];
        s_q[tid] = a.f32_values ? qv : __half2float(__float2half_rn(qv));
    }
    // Phase A
    for (int t = 0; t < tiles; ++t) {
        attn_tile_wait();
        __syncthreads();  // tile t has arrived for every thread, and every warp is done with tile t - 1, whose stage the next request reuses
        attn_tile_issue(ring, krows, t + kAttnTileStages - 1, len, hd, a.kv_dim, tid);
        const int p = t * kAttnTileRows + warp;
        if (p < len) {
            const __half* kr = ring + (static_cast<size_t>(t % kAttnTileStages) * kAttnTileRows + warp) * hd;
            float acc = 0.0f;
            for (int i = 0; i + 32 <= hd; i += 32) acc = __fmaf_rn(__half2float(kr[i + lane]), s_q[i + lane], acc);
            const float sc = a.f32_values ? dot_lane_reduce_f16_f32(acc) : dot_lane_reduce_f16(acc);
            if (lane == 0) s_score[p] = __fmul_rn(sc, a.scale);
        }
    }
    __syncthreads();  // all scores are written and every stage is free
    for (int t = 0; t < kAttnTileStages - 1; ++t) attn_tile_issue(ring, vrows, t, len, hd, a.kv_dim, tid);  // the value rows travel during phase B
    // Phase B: thread tid owns positions p0 .. p1; the maximum of everything before p0 comes from a scan in position order
    {
        const int per = (len + kAttnThreads - 1) / kAttnThreads;
        const int p0 = min(tid * per, len), p1 = min(p0 + per, len);
        float m = -INFINITY;
        for (int p = p0; p < p1; ++p) m = fmaxf(m, s_score[p]);
        float incl = m;
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl = fmaxf(incl, up);
        }
        float before = __shfl_up_sync(0xffffffffu, incl, 1);
        if (lane == 0) before = -INFINITY;
        if (lane == 31) s_tm[warp] = incl;
        __syncthreads();
        for (int w = 0; w < warp; ++w) before = fmaxf(before, s_tm[w]);
        float run = before;
        for (int p = p0; p < p1; ++p) {
            const float sc = s_score[p];
            const float m_old = run;
            float ms = 1.0f, vs = 1.0f;
            if (sc > run) {
                run = sc;
                ms = device_expf(__fsub_rn(m_old, run));
            } else {
                vs = device_expf(__fsub_rn(sc, run));
            }
            s_ms[p] = ms;
            s_score[p] = vs;
        }
    }
    // Phase C (the barrier of its first tile also publishes the factors of phase B)
    float acc = 0.0f, S = 0.0f;
    const bool sum_lane = tid == kAttnThreads - 32;
    for (int t = 0; t < tiles; ++t) {
        attn_tile_wait();
        __syncthreads();
        attn_tile_issue(ring, vrows, t + kAttnTileStages - 1, len, hd, a.kv_dim, tid);
        const int p_lo = t * kAttnTileRows, rows = min(kAttnTileRows, len - p_lo);
        if (tid < hd) {
            const __half* vr = ring + static_cast<size_t>(t % kAttnTileStages) * kAttnTileRows * hd + tid;
            if (a.f32_values) {
                for (int r = 0; r < rows; ++r) {
                    const float ms = s_ms[p_lo + r];
                    if (ms != 1.0f) acc = __fmul_rn(acc, ms);
                    acc = __fmaf_rn(__half2float(vr[r * hd]), s_score[p_lo + r], acc);
                }
            } else {  // the accumulator is an F16 after every operation
                for (int r = 0; r < rows; ++r) {
                    const float ms = s_ms[p_lo + r];
                    if (ms != 1.0f) acc = __half2float(__float2half_rn(__fmul_rn(acc, ms)));
                    acc = __half2float(__float2half_rn(__fmaf_rn(__half2float(vr[r * hd]), s_score[p_lo + r], acc)));
                }
            }
        } else if (sum_lane) {
            for (int r = 0; r < rows; ++r) S = __fmaf_rn(S, s_ms[p_lo + r], s_score[p_lo + r]);  // attention.rs:466
        }
    }
    if (tid < hd) my_acc[tid] = acc;
    if (sum_lane) {
        float M = -INFINITY;
        for (int w = 0; w < kAttnThreads / 32; ++w) M = fmaxf(M, s_tm[w]);
        my_ms[0] = M;
        my_ms[1] = S;
    }
}

// ---- the same attention for all query heads of a KV head at once --------------------------------------------------------
// Grid (kv_heads, chunks, tokens), 288 threads: the G query heads that share a KV head (grouped-query attention) share one
// pass over its keys and values. The arithmetic per head is attention_kernel's, operation for operation (the reference's
// order: attention.rs:402-469); what changes is who does it and how the rows arrive:
//  A. a warp takes a position and forms the G dot products from one copy of the key row;
//  B. warp g turns head g's scores into the running maximum and the factors ms / vs with a warp scan over blocks of 32
//     positions (the running maximum is a prefix maximum, so the scan gives exactly the sequential values);
//  C. thread d < head_dim runs the G value chains of coordinate d side by side, while the ninth warp runs the G chains of
//     the sums S.
// Key rows (phase A) and value rows (phase C) stream through a ring of three 16-row stages in shared memory filled by
// asynchronous copies two stages ahead, so a block waits for HBM once, not once per row. Per position the factors vs of
// the G heads and a bit mask "ms != 1 for head g" sit in one record that phase C reads with a single shared-memory load.
// Dynamic shared memory: attention_gqa_smem(G, head_dim, context).
constexpr int kAttnGqaThreads = 288;
constexpr int kAttnRingRows = 16, kAttnRingStages = 3;
__host__ __device__ constexpr int attn_gqa_record_words(int g) { return g <= 3 ? 4 : 8; }
__host__ __device__ constexpr int attn_gqa_chunk_max(int ctx) { return ((ctx + 3) / 4 + 31) / 32 * 32 > 256 ? ((ctx + 3) / 4 + 31) / 32 * 32 : 256; }
__host__ __device__ constexpr size_t attention_gqa_smem(int g, int head_dim, int ctx) {
    return static_cast<size_t>(kAttnRingStages) * kAttnRingRows * head_dim * 2 + static_cast<size_t>(attn_gqa_chunk_max(ctx)) * (attn_gqa_record_words(g) + g) * 4 +
           static_cast<size_t>(g) * head_dim * 4 + 64;
}

template <bool F32>
__device__ __forceinline__ float value_round(float x) {  // the accumulator is an F16 after every operation (bitnet.cpp numerics) or stays F32
    return F32 ? x : __half2float(__float2half_rn(x));
}


// Requests rows row0 .. row0 + 15 (those below len) of a chunk into a stage; always closes a copy group, so every thread counts the same groups.
__device__ __forceinline__ void attn_ring_issue(__half* stage, const __half* rows, int row0, int len, int hd, int kv_dim, int tid) {
    const int pieces = hd >> 3, n = min(kAttnRingRows, len - row0) * pieces;  // 16-byte pieces
    for (int i = tid; i < n; i += kAttnGqaThreads) {
        const int r = i / pieces, c = i - r * pieces;
        attn_cp16(stage + r * hd + c * 8, rows + static_cast<size_t>(row0 + r) * kv_dim + c * 8);
    }
    attn_cp_commit();
}

template <int G, bool F32>
__global__ void __launch_bounds__(kAttnGqaThreads) attention_gqa_kernel(AttnArgs a) {
    constexpr int W = attn_gqa_record_words(G);
    extern __shared__ __align__(16) unsigned char gqa_smem[];
    const int kvh = blockIdx.x, c = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hd = a.head_dim, cmax = attn_gqa_chunk_max(a.ctx);
    __half* s_ring = reinterpret_cast<__half*>(gqa_smem);                                        // [3][16][hd]
    float* s_rec = reinterpret_cast<float*>(gqa_smem + static_cast<size_t>(kAttnRingStages) * kAttnRingRows * hd * 2);  // [cmax][W]: vs of head g at word g, the mask at word W - 1
    float* s_ms = s_rec + static_cast<size_t>(cmax) * W;       // [G][cmax]: scores, then ms
    float* s_q = s_ms + static_cast<size_t>(G) * cmax;         // [G][hd]
    float* s_M = s_q + static_cast<size_t>(G) * hd;            // [G]: the chunk's maximum per head
    const int stage_halves = kAttnRingRows * hd;
    if (blockIdx.z != 0) {
        const size_t z = blockIdx.z;
        a.q += z * a.b_q;
        a.part_acc += z * a.b_acc;
        a.part_ms += z * a.b_ms;
    }
    const int seq_len = static_cast<int>(seq_position(a.seq, a.pos, blockIdx.z)) + 1;
    a.k_cache += seq_cache_offset(a.seq, blockIdx.z);
    a.v_cache += seq_cache_offset(a.seq, blockIdx.z);
    int n_kv = (seq_len + 255) / 256 * 256;
    if (n_kv < 256) n_kv = 256;
    if (n_kv > a.ctx) n_kv = a.ctx;
    int start = 0, end = seq_len;
    if (n_kv >= 512) {
        const int chunk = (n_kv + 3) / 4;
        start = c * chunk;
        end = min(min(start + chunk, n_kv), seq_len);
    } else if (c > 0) {
        start = end;  // single-chunk case: chunks 1..3 are empty
    }
    const int h0 = kvh * G;
    const int len = min(end - start, cmax);  // (a chunk never exceeds cmax: n_kv <= ctx)
    if (len <= 0) {
        if (tid < G) {
            float* my_ms = a.part_ms + (static_cast<size_t>(h0 + tid) * 4 + c) * 2;
            my_ms[0] = -INFINITY;
            my_ms[1] = 0.0f;
        }
        return;
    }
    const __half* kbase = a.k_cache + static_cast<size_t>(kvh) * hd + static_cast<size_t>(start) * a.kv_dim;
    const __half* vbase = a.v_cache + static_cast<size_t>(kvh) * hd + static_cast<size_t>(start) * a.kv_dim;
    const int nblk = (len + kAttnRingRows - 1) / kAttnRingRows;
    attn_ring_issue(s_ring, kbase, 0, len, hd, a.kv_dim, tid);
    attn_ring_issue(s_ring + stage_halves, kbase, kAttnRingRows, len, hd, a.kv_dim, tid);
    for (int i = tid; i < G * hd; i += kAttnGqaThreads) {
        const float qv = a.q[h0 * hd + i];
        s_q[i] = F32 ? qv : __half2float(__float2half_rn(qv));
    }
    for (int i = tid; i < len; i += kAttnGqaThreads) reinterpret_cast<uint32_t*>(s_rec)[static_cast<size_t>(i) * W + W - 1] = 0u;
    __syncthreads();
    // Phase A: lane l owns the elements 32 i + l of a row, added in the order of i (ggml_vec_dot_f16 / _f16_f32), then the lanes are reduced.
    // Warps 0-7 take two rows of a stage each.
    {
        const int nq = hd >> 5;  // <= 8
        float qr[G][8];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int i = 0; i < 8; ++i) qr[g][i] = i < nq ? s_q[g * hd + i * 32 + lane] : 0.0f;
        for (int blk = 0; blk < nblk; ++blk) {
            attn_cp_wait_all_but_one();
            __syncthreads();
            attn_ring_issue(s_ring + ((blk + 2) % kAttnRingStages) * stage_halves, kbase, (blk + 2) * kAttnRingRows, len, hd, a.kv_dim, tid);
            const __half* st = s_ring + (blk % kAttnRingStages) * stage_halves;
            const int r1 = 2 * warp, r2 = r1 + 1, p1 = blk * kAttnRingRows + r1, p2 = p1 + 1;
            if (warp < 8 && p1 < len) {
                const bool two = p2 < len;
                const __half* k1 = st + r1 * hd + lane;
                const __half* k2 = st + (two ? r2 : r1) * hd + lane;
                float acc1[G], acc2[G];
#pragma unroll
                for (int g = 0; g < G; ++g) acc1[g] = 0.0f, acc2[g] = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (i < nq) {
                        const float x1 = __half2float(k1[i * 32]), x2 = __half2float(k2[i * 32]);
#pragma unroll
                        for (int g = 0; g < G; ++g) {
                            acc1[g] = __fmaf_rn(x1, qr[g][i], acc1[g]);
                            acc2[g] = __fmaf_rn(x2, qr[g][i], acc2[g]);
                        }
                    }
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float sc1 = F32 ? dot_lane_reduce_f16_f32(acc1[g]) : dot_lane_reduce_f16(acc1[g]);
                    const float sc2 = F32 ? dot_lane_reduce_f16_f32(acc2[g]) : dot_lane_reduce_f16(acc2[g]);
                    if (lane == 0) {
                        s_ms[g * cmax + p1] = __fmul_rn(sc1, a.scale);
                        if (two) s_ms[g * cmax + p2] = __fmul_rn(sc2, a.scale);
                    }
                }
            }
        }
    }
    __syncthreads();  // every score is written, every key stage is read
    attn_ring_issue(s_ring, vbase, 0, len, hd, a.kv_dim, tid);  // the first value rows arrive while phase B runs
    attn_ring_issue(s_ring + stage_halves, vbase, kAttnRingRows, len, hd, a.kv_dim, tid);
    // Phase B: warp g, head g
    if (warp < G) {
        const int g = warp;
        float* sc_g = s_ms + g * cmax;
        float carry = -INFINITY;  // the maximum of all earlier positions
        for (int base = 0; base < len; base += 32) {
            const int p = base + lane;
            const float sc = p < len ? sc_g[p] : -INFINITY;
            float incl = sc;  // inclusive prefix maximum over the block
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl = fmaxf(incl, up);
            }
            float excl = __shfl_up_sync(0xffffffffu, incl, 1);
            if (lane == 0) excl = -INFINITY;
            const float m_old = fmaxf(carry, excl);
            if (p < len) {
                float ms = 1.0f, vs = 1.0f;
                if (sc > m_old) {
                    ms = device_expf(__fsub_rn(m_old, sc));
                } else {
                    vs = device_expf(__fsub_rn(sc, m_old));
                }
                sc_g[p] = ms;
                s_rec[static_cast<size_t>(p) * W + g] = vs;
                if (ms != 1.0f) atomicOr(reinterpret_cast<unsigned int*>(s_rec) + static_cast<size_t>(p) * W + W - 1, 1u << g);
            }
            carry = fmaxf(carry, __shfl_sync(0xffffffffu, incl, 31));
        }
        if (lane == 0) s_M[g] = carry;
    }
    // Phase C: threads below head_dim run the value chains of their coordinate, lanes below G of the last warp the sums
    // S = fma(S, ms, vs) (attention.rs:466), stage by stage in position order.
    const bool sum_lane = warp == kAttnGqaThreads / 32 - 1 && lane < G;
    const bool chain_thread = warp < kAttnGqaThreads / 32 - 1 && tid < hd;
    float acc[G];
#pragma unroll
    for (int g = 0; g < G; ++g) acc[g] = 0.0f;
    float S = 0.0f;
    for (int blk = 0; blk < nblk; ++blk) {
        attn_cp_wait_all_but_one();
        __syncthreads();  // (the first one also publishes phase B's records)
        attn_ring_issue(s_ring + ((blk + 2) % kAttnRingStages) * stage_halves, vbase, (blk + 2) * kAttnRingRows, len, hd, a.kv_dim, tid);
        const int p0 = blk * kAttnRingRows, rows = min(kAttnRingRows, len - p0);
        if (chain_thread) {
            const __half* st = s_ring + (blk % kAttnRingStages) * stage_halves + tid;
#pragma unroll 4
            for (int r = 0; r < rows; ++r) {
                const int p = p0 + r;
                float rec[W];
                if constexpr (W == 4) {
                    const float4 q4 = *reinterpret_cast<const float4*>(s_rec + static_cast<size_t>(p) * 4);
                    rec[0] = q4.x, rec[1] = q4.y, rec[2] = q4.z, rec[3] = q4.w;
                } else {
                    const float4 q0 = *reinterpret_cast<const float4*>(s_rec + static_cast<size_t>(p) * 8);
                    const float4 q1 = *reinterpret_cast<const float4*>(s_rec + static_cast<size_t>(p) * 8 + 4);
                    rec[0] = q0.x, rec[1] = q0.y, rec[2] = q0.z, rec[3] = q0.w, rec[4] = q1.x, rec[5] = q1.y, rec[6] = q1.z, rec[7] = q1.w;
                }
                const unsigned int mask = __float_as_uint(rec[W - 1]);
                if (mask != 0u) {
#pragma unroll
                    for (int g = 0; g < G; ++g)
                        if ((mask >> g) & 1u) acc[g] = value_round<F32>(__fmul_rn(acc[g], s_ms[g * cmax + p]));
                }
                const float vf = __half2float(st[r * hd]);
#pragma unroll
                for (int g = 0; g < G; ++g) acc[g] = value_round<F32>(__fmaf_rn(vf, rec[g], acc[g]));
            }
        } else if (sum_lane) {
            const float* ms_g = s_ms + lane * cmax;
            for (int r = 0; r < rows; ++r) S = __fmaf_rn(S, ms_g[p0 + r], s_rec[static_cast<size_t>(p0 + r) * W + lane]);
        }
    }
    if (chain_thread) {
#pragma unroll
        for (int g = 0; g < G; ++g) a.part_acc[(static_cast<size_t>(h0 + g) * 4 + c) * hd + tid] = acc[g];
    } else if (sum_lane) {
        float* my_ms = a.part_ms + (static_cast<size_t>(h0 + lane) * 4 + c) * 2;
        my_ms[0] = s_M[lane];
        my_ms[1] = S;
    }
}

using AttnGqaKernel = void (*)(AttnArgs);
// The instantiation for a group size and numerics, or nullptr: then attention_kernel runs one query head per block.
inline AttnGqaKernel attention_gqa_for(int gqa, bool f32_values) {
    switch (gqa) {
        case 1: return f32_values ? attention_gqa_kernel<1, true> : attention_gqa_kernel<1, false>;
        case 2: return f32_values ? attention_gqa_kernel<2, true> : attention_gqa_kernel<2, false>;
        case 3: return f32_values ? attention_gqa_kernel<3, true> : attention_gqa_kernel<3, false>;
        case 4: return f32_values ? attention_gqa_kernel<4, true> : attention_gqa_kernel<4, false>;
        default: return nullptr;
    }
}

// ---- combine the KV chunks (attention.rs:497-541), optional sub-norm, quantise for the o projection -------------------
struct AttnFinishArgs {
    const float* part_acc;    // [q_heads][4][head_dim]
    const float* part_ms;     // [q_heads][4][2]
    const uint32_t* pos;
    int q_heads, head_dim, ctx;
    const float* sub_norm_w;  // BitNet attn_sub_norm (q_dim) or nullptr
    float eps;
    int8_t* q_out;
    float* scale_out;
    int32_t* zero_a;          // result buffer of the o projection
    int zero_a_n;
    float* q8_d;              // block-scaled models: Q8_0 block scales of q_out (else nullptr: per-tensor int8)
    int b_acc, b_ms, b_q, b_scale;  // batch of tokens: per-token strides of part_acc, part_ms, q_out; scale_out + z when b_scale is set
    SeqIndex seq;             // the token's position
};

// Coordinate d of head h from the four chunks' accumulators and their (M, S) pairs (attention.rs:497-541).
__device__ __forceinline__ float attn_combine_chunks(const float* part_acc, const float* part_ms, int h, int d, int hd, int n_kv) {
    const float* pa = part_acc + static_cast<size_t>(h) * 4 * hd + d;
    const float* pm = part_ms + static_cast<size_t>(h) * 8;
    if (n_kv < 512) {
        const float S = pm[1];
        const float s_inv = S == 0.0f ? 0.0f : __fdiv_rn(1.0f, S);
        return __fmul_rn(pa[0], s_inv);
    }
    float m_final = -INFINITY, s_final = 0.0f, acc = 0.0f;
    for (int c = 0; c < 4; ++c) {
        const float m_chunk = pm[2 * c], s_chunk = pm[2 * c + 1];
        if (s_chunk == 0.0f) continue;  // empty or fully masked chunk
        const float m_new = fmaxf(m_final, m_chunk);
        const float scale_old = device_expf(__fsub_rn(m_final, m_new));
        const float scale_new = device_expf(__fsub_rn(m_chunk, m_new));
        acc = __fmaf_rn(acc, scale_old, __fmul_rn(pa[c * hd], scale_new));
        s_final = __fmaf_rn(s_final, scale_old, __fmul_rn(s_chunk, scale_new));
        m_final = m_new;
    }
    return s_final != 0.0f ? __fmul_rn(acc, __fdiv_rn(1.0f, s_final)) : acc;
}

// Block-scaled models without a sub-norm: a Q8_0 block of 32 values needs nothing from the rest of the vector, so one warp
// combines and quantises one block and the vector spreads over as many blocks of threads as it has blocks of eight. One token.
constexpr int kQ8BlockThreads = 256;
__global__ void __launch_bounds__(kQ8BlockThreads) attn_finish_q8_kernel(AttnFinishArgs a) {
    const int lane = threadIdx.x & 31, b = blockIdx.x * (kQ8BlockThreads / 32) + (threadIdx.x >> 5), hd = a.head_dim;
    if (b >= a.q_heads * hd / 32) return;
    const int seq_len = static_cast<int>(seq_position(a.seq, a.pos, 0)) + 1;
    int n_kv = (seq_len + 255) / 256 * 256;
    if (n_kv < 256) n_kv = 256;
    if (n_kv > a.ctx) n_kv = a.ctx;
    const int i = b * 32 + lane;
    quantize_q8_0_block(attn_combine_chunks(a.part_acc, a.part_ms, i / hd, i % hd, hd, n_kv), b, lane, a.q_out, a.q8_d);
}

__global__ void __launch_bounds__(kRowThreads) attn_finish_kernel(AttnFinishArgs a) {
    __shared__ double sh_d[32];
    __shared__ float sh_f[32];
    extern __shared__ float y_s[];  // q_dim floats
    const int tid = threadIdx.x, hd = a.head_dim, n = a.q_heads * hd;
    if (blockIdx.z != 0) {
        const size_t z = blockIdx.z;
        a.part_acc += z * a.b_acc;
        a.part_ms += z * a.b_ms;
        a.q_out += z * a.b_q;
        if (a.b_scale) a.scale_out += z;
    }
    for (int i = tid; i < a.zero_a_n; i += kRowThreads) a.zero_a[i] = 0;
    const int seq_len = static_cast<int>(seq_position(a.seq, a.pos, blockIdx.z)) + 1;
    int n_kv = (seq_len + 255) / 256 * 256;
    if (n_kv < 256) n_kv = 256;
    if (n_kv > a.ctx) n_kv = a.ctx;
    for (int i = tid; i < n; i += kRowThreads) y_s[i] = attn_combine_chunks(a.part_acc, a.part_ms, i / hd, i % hd, hd, n_kv);
    __syncthreads();
    if (a.sub_norm_w != nullptr) {
        double sum = 0.0;
        for (int i = tid; i < n; i += kRowThreads) sum += static_cast<double>(__fmul_rn(y_s[i], y_s[i]));
        sum = block_sum_f64(sum, sh_d);
        const float mean = __double2float_rn(sum / static_cast<double>(n));
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, a.eps)));
        for (int i = tid; i < n; i += kRowThreads) y_s[i] = __fmul_rn(__fmul_rn(y_s[i], inv), a.sub_norm_w[i]);
    }
    float amax = 0.0f;
    for (int i = tid; i < n; i += kRowThreads) amax = fmaxf(amax, fabsf(y_s[i]));
    __syncthreads();
    quantize_vector(y_s, n, amax, a.q_out, a.scale_out, a.q8_d, sh_f);
}

// ---- gate / up finish: post-scale, SwiGLU or relu^2 * up, optional sub-norm, quantise for the down projection ---------
// (model.rs:150-193; ops.rs:301-308, 427-473)
struct ActQuantArgs {
    const int32_t* acc_gate;
    const int32_t* acc_up;
    const float* act_scale;
    float ws_gate, ws_up;
    int n, relu2;
    const float* sub_norm_w;  // BitNet ffn_sub_norm (n) or nullptr
    float eps;
    int8_t* q_out;
    float* scale_out;
    int32_t* zero_a;          // result buffer of the down projection
    int zero_a_n;
    int block_scaled;         // acc_gate / acc_up hold F32 results of block-scaled projections; codes are Q8_0 blocks
    float* q8_d;
    int b_acc, b_q, b_scale;  // batch of tokens: per-token strides of acc_gate / acc_up and of q_out; act_scale + z and scale_out + z when b_scale is set
    AccView v_gate, v_up;     // the two projections' sums as parts (v_gate.base != nullptr), instead of acc_gate / acc_up
};

// The same for block-scaled models without an FFN sub-norm: one warp per Q8_0 block of the gated vector. One token.
__global__ void __launch_bounds__(kQ8BlockThreads) act_quant_q8_kernel(ActQuantArgs a) {
    const int lane = threadIdx.x & 31, b = blockIdx.x * (kQ8BlockThreads / 32) + (threadIdx.x >> 5);
    if (b >= a.n / 32) return;
    const int i = b * 32 + lane;
    const float g = reinterpret_cast<const float*>(a.acc_gate)[i], u = reinterpret_cast<const float*>(a.acc_up)[i];
    float v;
    if (a.relu2) {
        const float p = g > 0.0f ? g : 0.0f;
        v = __fmul_rn(__fmul_rn(p, p), u);
    } else {
        v = __fmul_rn(ggml_silu(g), u);
    }
    quantize_q8_0_block(v, b, lane, a.q_out, a.q8_d);
}

__global__ void __launch_bounds__(kRowThreads) act_quant_kernel(ActQuantArgs a) {
    __shared__ double sh_d[32];
    __shared__ float sh_f[32];
    extern __shared__ float y_s[];  // n floats
    const int tid = threadIdx.x;
    if (blockIdx.z != 0) {
        const size_t z = blockIdx.z;
        a.acc_gate += z * a.b_acc;
        a.acc_up += z * a.b_acc;
        a.q_out += z * a.b_q;
        if (a.b_scale) {
            a.act_scale += z;
            a.scale_out += z;
        }
    }
    for (int i = tid; i < a.zero_a_n; i += kRowThreads) a.zero_a[i] = 0;
    const float s_in = a.block_scaled ? 1.0f : a.act_scale[0];
    const bool live = s_in > 0.0f;
    const float pg = live ? __fdiv_rn(a.ws_gate, s_in) : 0.0f, pu = live ? __fdiv_rn(a.ws_up, s_in) : 0.0f;
    for (int i = tid; i < a.n; i += kRowThreads) {
        const float g = a.block_scaled ? reinterpret_cast<const float*>(a.acc_gate)[i] : (live ? __fmul_rn(static_cast<float>(a.v_gate.base != nullptr ? acc_view_read(a.v_gate, blockIdx.z, i) : a.acc_gate[i]), pg) : 0.0f);
        const float u = a.block_scaled ? reinterpret_cast<const float*>(a.acc_up)[i] : (live ? __fmul_rn(static_cast<float>(a.v_up.base != nullptr ? acc_view_read(a.v_up, blockIdx.z, i) : a.acc_up[i]), pu) : 0.0f);
        float v;
        if (a.relu2) {
            const float p = g > 0.0f ? g : 0.0f;
            v = __fmul_rn(__fmul_rn(p, p), u);
        } else {
            v = __fmul_rn(ggml_silu(g), u);
        }
        y_s[i] = v;
    }
    __syncthreads();
    if (a.sub_norm_w != nullptr) {
        double sum = 0.0;
        for (int i = tid; i < a.n; i += kRowThreads) sum += static_cast<double>(__fmul_rn(y_s[i], y_s[i]));
        sum = block_sum_f64(sum, sh_d);
        const float mean = __double2float_rn(sum / static_cast<double>(a.n));
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, a.eps)));
        for (int i = tid; i < a.n; i += kRowThreads) y_s[i] = __fmul_rn(__fmul_rn(y_s[i], inv), a.sub_norm_w[i]);
    }
    float amax = 0.0f;
    for (int i = tid; i < a.n; i += kRowThreads) amax = fmaxf(amax, fabsf(y_s[i]));
    __syncthreads();
    quantize_vector(y_s, a.n, amax, a.q_out, a.scale_out, a.block_scaled ? a.q8_d : nullptr, sh_f);
}

// The same step for the batched paths, one token spread over a cluster of eight blocks: a block computes, normalises and
// quantises an eighth of the vector; the two block-wide reductions (sum of squares for the sub-norm, maximum for the
// scale) become cluster-wide by reading the other blocks' partial results through distributed shared memory, in rank
// order. Grid (8, 1, tokens). Per-tensor int8 codes only (block-scaled models do not take the batched paths).
constexpr int kActClusterSize = 8, kActClusterThreads = 512;
__host__ __device__ constexpr int act_cluster_slice(int n) { return (n + kActClusterSize - 1) / kActClusterSize; }

__global__ void __cluster_dims__(kActClusterSize, 1, 1) __launch_bounds__(kActClusterThreads) act_quant_cluster_kernel(ActQuantArgs a) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ double sh_d[32];
    __shared__ float sh_f[32];
    __shared__ double x_sum;
    __shared__ float x_max;
    extern __shared__ float y_s[];  // this block's slice
    const int tid = threadIdx.x, rank = static_cast<int>(cluster.block_rank());
    if (blockIdx.z != 0) {
        const size_t z = blockIdx.z;
        a.acc_gate += z * a.b_acc;
        a.acc_up += z * a.b_acc;
        a.q_out += z * a.b_q;
        if (a.b_scale) {
            a.act_scale += z;
            a.scale_out += z;
        }
    }
    const int per = act_cluster_slice(a.n), i0 = min(a.n, rank * per), m = min(a.n, i0 + per) - i0;
    const float s_in = a.act_scale[0];
    const bool live = s_in > 0.0f;
    const float pg = live ? __fdiv_rn(a.ws_gate, s_in) : 0.0f, pu = live ? __fdiv_rn(a.ws_up, s_in) : 0.0f;
    for (int i = tid; i < m; i += kActClusterThreads) {
        const int gi = i0 + i;
        const float g = live ? __fmul_rn(static_cast<float>(a.v_gate.base != nullptr ? acc_view_read(a.v_gate, blockIdx.z, gi) : a.acc_gate[gi]), pg) : 0.0f;
        const float u = live ? __fmul_rn(static_cast<float>(a.v_up.base != nullptr ? acc_view_read(a.v_up, blockIdx.z, gi) : a.acc_up[gi]), pu) : 0.0f;
        float v;
        if (a.relu2) {
            const float p = g > 0.0f ? g : 0.0f;
            v = __fmul_rn(__fmul_rn(p, p), u);
        } else {
            v = __fmul_rn(ggml_silu(g), u);
        }
        y_s[i] = v;
    }
    __syncthreads();
    if (a.sub_norm_w != nullptr) {
        double sum = 0.0;
        for (int i = tid; i < m; i += kActClusterThreads) sum += static_cast<double>(__fmul_rn(y_s[i], y_s[i]));
        sum = block_sum_f64(sum, sh_d);
        if (tid == 0) x_sum = sum;
        cluster.sync();
        double total = 0.0;
        for (int r = 0; r < kActClusterSize; ++r) total += *cluster.map_shared_rank(&x_sum, r);
        const float mean = __double2float_rn(total / static_cast<double>(a.n));
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, a.eps)));
        for (int i = tid; i < m; i += kActClusterThreads) y_s[i] = __fmul_rn(__fmul_rn(y_s[i], inv), a.sub_norm_w[i0 + i]);
        __syncthreads();
    }
    float amax = 0.0f;
    for (int i = tid; i < m; i += kActClusterThreads) amax = fmaxf(amax, fabsf(y_s[i]));
    amax = block_max_f32(amax, sh_f);
    if (tid == 0) x_max = amax;
    cluster.sync();
    amax = 0.0f;
    for (int r = 0; r < kActClusterSize; ++r) amax = fmaxf(amax, *cluster.map_shared_rank(&x_max, r));
    const float s = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    for (int i = tid; i < m; i += kActClusterThreads) {
        float q = 0.0f;
        if (amax > 0.0f) {
            q = roundf(__fmul_rn(y_s[i], s));
            q = q != q ? 0.0f : fminf(fmaxf(q, -128.0f), 127.0f);
        }
        a.q_out[i0 + i] = static_cast<int8_t>(q);
    }
    if (rank == 0 && tid == 0) a.scale_out[0] = s;
    cluster.sync();  // no block leaves while its partial results may still be read
}

// ---- output head: one warp per vocabulary row, ggml_vec_dot_f16 order (model.rs:346-375, ops.rs:970-1014) --------------
__global__ void __launch_bounds__(256) lm_head_kernel(const __half* __restrict__ w, const __half* __restrict__ x16, int hidden, int vocab,
                                                      float* __restrict__ logits, bool bf16) {
    extern __shared__ float x_s[];  // hidden floats
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) x_s[i] = table_to_float(x16[i], bf16);
    __syncthreads();
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int np = hidden & ~31;  // hidden is a multiple of 32 (checked at creation): no scalar tail
    for (int row = blockIdx.x * warps + (threadIdx.x >> 5); row < vocab; row += gridDim.x * warps) {
        const __half* wr = w + static_cast<size_t>(row) * hidden;
        float acc = 0.0f;
        if (bf16) {  // ggml_vec_dot_bf16: product and sum rounded separately (ops.rs:694-700)
#pragma unroll 8
            for (int i = 0; i < np; i += 32) acc = __fadd_rn(acc, __fmul_rn(x_s[i + lane], bf16_bits_to_float(__half_as_ushort(wr[i + lane]))));
        } else {
#pragma unroll 8
            for (int i = 0; i < np; i += 32) acc = __fmaf_rn(x_s[i + lane], __half2float(wr[i + lane]), acc);
        }
        const float sum = bf16 ? dot_lane_reduce_bf16(acc) : dot_lane_reduce_f16(acc);
        if (lane == 0) logits[row] = sum;
    }
}

// ---- output head for several tokens at once ------------------------------------------------------------------------------
// The same dot products as lm_head_kernel (lane l of a warp owns the elements 32 i + l of a row and adds them in the order of
// i, then the lanes are reduced), for up to kHeadTokens tokens against kHeadRows vocabulary rows per warp at a time: a row
// element is read from HBM once per token group instead of once per token, and an activation read from shared memory serves
// kHeadRows rows. The activations sit in shared memory as F32, laid out so that a lane reads its elements of four consecutive
// steps with one 16-byte load: float4 index (t * hidden / 128 + k) * 32 + lane holds steps 4k .. 4k + 3.
constexpr int kHeadTokens = 16, kHeadRows = 4, kHeadThreads = 256;
__host__ __device__ constexpr size_t lm_head_batch_smem(int hidden) { return static_cast<size_t>(kHeadTokens) * hidden * sizeof(float); }

__global__ void __launch_bounds__(kHeadThreads, 1) lm_head_batch_kernel(const __half* __restrict__ w, const __half* __restrict__ x16, int hidden, int vocab, int n,
                                                                         float* __restrict__ logits, bool bf16) {
    extern __shared__ float4 x4[];
    float* xs = reinterpret_cast<float*>(x4);
    const int t0 = blockIdx.y * kHeadTokens, nt = min(kHeadTokens, n - t0), k4 = hidden / 128;
    for (int idx = threadIdx.x; idx < kHeadTokens * hidden; idx += kHeadThreads) {
        const int t = idx / hidden, e = idx - t * hidden, step = e >> 5, l = e & 31;
        const float v = t < nt ? table_to_float(x16[static_cast<size_t>(t0 + t) * hidden + e], bf16) : 0.0f;
        xs[((static_cast<size_t>(t) * k4 + (step >> 2)) * 32 + l) * 4 + (step & 3)] = v;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warps = kHeadThreads / 32;
    for (int row0 = (blockIdx.x * warps + (threadIdx.x >> 5)) * kHeadRows; row0 < vocab; row0 += gridDim.x * warps * kHeadRows) {
        const __half* wr[kHeadRows];
#pragma unroll
        for (int r = 0; r < kHeadRows; ++r) wr[r] = w + static_cast<size_t>(min(row0 + r, vocab - 1)) * hidden + lane;
        float acc[kHeadTokens][kHeadRows];
#pragma unroll
        for (int t = 0; t < kHeadTokens; ++t)
#pragma unroll
            for (int r = 0; r < kHeadRows; ++r) acc[t][r] = 0.0f;
        unsigned short raw[kHeadRows][4];
#pragma unroll
        for (int r = 0; r < kHeadRows; ++r)
#pragma unroll
            for (int j = 0; j < 4; ++j) raw[r][j] = __half_as_ushort(wr[r][j * 32]);
        for (int k = 0; k < k4; ++k) {
            float wv[kHeadRows][4];
#pragma unroll
            for (int r = 0; r < kHeadRows; ++r)
#pragma unroll
                for (int j = 0; j < 4; ++j) wv[r][j] = table_to_float(__ushort_as_half(raw[r][j]), bf16);
            if (k + 1 < k4) {  // the next steps' row elements are requested before this step's arithmetic
#pragma unroll
                for (int r = 0; r < kHeadRows; ++r)
#pragma unroll
                    for (int j = 0; j < 4; ++j) raw[r][j] = __half_as_ushort(wr[r][(4 * (k + 1) + j) * 32]);
            }
            const float4* xk = x4 + static_cast<size_t>(k) * 32 + lane;
            if (bf16) {  // ggml_vec_dot_bf16: product and sum rounded separately (ops.rs:694-700)
#pragma unroll
                for (int t = 0; t < kHeadTokens; ++t) {
                    const float4 x = xk[static_cast<size_t>(t) * k4 * 32];
                    const float xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int r = 0; r < kHeadRows; ++r) acc[t][r] = __fadd_rn(acc[t][r], __fmul_rn(xv[j], wv[r][j]));
                }
            } else {
#pragma unroll
                for (int t = 0; t < kHeadTokens; ++t) {
                    const float4 x = xk[static_cast<size_t>(t) * k4 * 32];
                    const float xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int r = 0; r < kHeadRows; ++r) acc[t][r] = __fmaf_rn(xv[j], wv[r][j], acc[t][r]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < kHeadTokens; ++t)
#pragma unroll
            for (int r = 0; r < kHeadRows; ++r) {
                const float sum = bf16 ? dot_lane_reduce_bf16(acc[t][r]) : dot_lane_reduce_f16(acc[t][r]);
                if (lane == 0 && t < nt && row0 + r < vocab) logits[static_cast<size_t>(t0 + t) * vocab + row0 + r] = sum;
            }
    }
}

// ---- greedy sampler: first index of the strict maximum, NaN never wins (sampler.rs:73-83) ------------------------------
__device__ __forceinline__ void argmax_merge(float& bv, unsigned int& bi, float v, unsigned int i) {
    if (v > bv || (v == bv && i < bi)) {
        bv = v;
        bi = i;
    }
}
// Block b takes the row logits + b * n and writes out_token[b] (one block for a single token).
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int n, uint32_t* __restrict__ out_token) {
    __shared__ float sv[32];
    __shared__ unsigned int si[32];
    logits += static_cast<size_t>(blockIdx.x) * n;
    out_token += blockIdx.x;
    float bv = -INFINITY;
    unsigned int bi = 0xFFFFFFFFu;
    int done = 0;
    if (n % 4 == 0) {  // rows start on 16-byte boundaries: four values per load, four loads in flight, indices ascending per thread
        const float4* l4 = reinterpret_cast<const float4*>(logits);
        const int n4 = n / 4;
#pragma unroll 4
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 v = l4[i];
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (e[k] > bv) {  // strict: the earlier index stays on ties
                    bv = e[k];
                    bi = static_cast<unsigned int>(i * 4 + k);
                }
        }
        done = n;
    }
    for (int i = done + threadIdx.x; i < n; i += blockDim.x) {
        const float v = logits[i];
        if (v > bv) {
            bv = v;
            bi = static_cast<unsigned int>(i);
        }
    }
    for (int o = 16; o > 0; o >>= 1) argmax_merge(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = bv;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 32; ++w) argmax_merge(bv, bi, sv[w], si[w]);
        out_token[0] = bi == 0xFFFFFFFFu ? 0u : bi;  // all NaN / -inf: index 0, as the reference's loop leaves it
    }
}

// ---- temperature / top-k / top-p sampling on the device (sampler.rs:59-143) ----------------------------------------------
// One block of 1024 threads, for 1 <= top_k <= 1024 and top_k < n. The reference scales the logits by 1 / temperature, sorts the
// candidates (stable, descending in the total order of floats), keeps top_k, takes exp(x - max) with the float libm
// exponential, sums in double in candidate order, cuts the nucleus with a float running sum, normalises again and walks
// the cumulative sum up to a number from its xorshift64 stream. Here: the k-th largest key is found by a three-pass radix
// select over the keys of all n candidates (where more keys equal the k-th than are wanted, thread t counts and takes
// those of a contiguous range, so they are taken in index order after one block-wide scan); the k survivors are ordered by counting, and thread 0 then performs the sequential
// arithmetic exactly as written there. The chosen id replaces *token; *rng is the generator's state.
constexpr int kSampleThreads = 1024, kSampleMaxK = 1024;

__device__ __forceinline__ uint32_t sample_key(float v) {  // ascending unsigned order = f32::total_cmp order
    const int32_t b = static_cast<int32_t>(__float_as_uint(v));
    return static_cast<uint32_t>(b ^ static_cast<int32_t>(static_cast<uint32_t>(b >> 31) >> 1)) ^ 0x80000000u;
}

__global__ void __launch_bounds__(kSampleThreads) sample_topk_kernel(const float* __restrict__ logits, int n, float temperature, int top_k, float top_p,
                                                                     unsigned long long* __restrict__ rng, uint32_t* __restrict__ token) {
    __shared__ unsigned int hist[2048];
    __shared__ unsigned int s_prefix, s_need, s_count, s_equal;
    __shared__ unsigned int scan[kSampleThreads];
    __shared__ uint32_t c_key[kSampleMaxK], c_idx[kSampleMaxK], o_idx[kSampleMaxK];
    __shared__ float o_val[kSampleMaxK];
    const int tid = threadIdx.x;
    const float inv_temp = __fdiv_rn(1.0f, temperature);
    // Radix select in three passes over digits of 11, 11 and 10 bits: after a pass the keys that carry the chosen digits contain the
    // k-th largest. The passes read the logits with a stride of the block (neighbouring threads, neighbouring addresses), four at a time.
    unsigned int prefix = 0, need = static_cast<unsigned int>(top_k);
    for (int pass = 0; pass < 3; ++pass) {
        const int shift = pass == 0 ? 21 : pass == 1 ? 10 : 0, width = pass == 2 ? 10 : 11;
        const unsigned int above = pass == 0 ? 0u : 0xFFFFFFFFu << (shift + width);  // the digits chosen so far
        for (int i = tid; i < 2048; i += kSampleThreads) hist[i] = 0;
        __syncthreads();
        for (int base = 0; base < n; base += 4 * kSampleThreads) {  // (a uniform trip count: the lanes of a warp vote below)
            float v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = base + u * kSampleThreads + tid;
                v[u] = i < n ? logits[i] : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = base + u * kSampleThreads + tid;
                unsigned int bucket = 2048u;  // no key, or a key outside the chosen digits
                if (i < n) {
                    const uint32_t k = sample_key(__fmul_rn(v[u], inv_temp));
                    if ((k & above) == prefix) bucket = (k >> shift) & ((1u << width) - 1u);
                }
                if (pass == 0) {
                    // the logits of one token share most of their leading bits: the lanes that hit the same bucket send one addition
                    const unsigned int peers = __match_any_sync(0xffffffffu, bucket);
                    if (bucket < 2048u && (tid & 31) == __ffs(peers) - 1) atomicAdd(&hist[bucket], static_cast<unsigned int>(__popc(peers)));
                } else if (bucket < 2048u) {
                    atomicAdd(&hist[bucket], 1u);
                }
            }
        }
        __syncthreads();
        if (tid < 32) {
            // the bucket in which the count from the top reaches `need`: lane L sums buckets 64 L .. 64 L + 63, the lanes' sums are
            // accumulated from the top, and the lane where the target falls walks its 64 buckets
            unsigned int sum = 0;
            for (int i = 0; i < 64; ++i) sum += hist[tid * 64 + i];
            unsigned int from_here = sum;  // buckets of this lane and of all higher lanes
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned int up = __shfl_down_sync(0xffffffffu, from_here, o);
                if (tid + o < 32) from_here += up;
            }
            const unsigned int reach = __ballot_sync(0xffffffffu, from_here >= need);  // lanes 0 .. L*: bit 0 is always set (need <= n)
            const int lane_star = 31 - __clz(static_cast<int>(reach));
            if (tid == lane_star) {
                unsigned int left = need - (from_here - sum);
                int bkt = tid * 64 + 63;
                for (; bkt > tid * 64; --bkt) {
                    if (hist[bkt] >= left) break;
                    left -= hist[bkt];
                }
                s_prefix = prefix | (static_cast<unsigned int>(bkt) << shift);
                s_need = left;          // how many keys of the chosen bucket are still wanted
                s_equal = hist[bkt];    // (after the last pass: how many keys equal the k-th)
                s_count = 0;
            }
        }
        __syncthreads();
        prefix = s_prefix, need = s_need;
        __syncthreads();
    }
    // Every key above the k-th is a candidate. Of the keys equal to it the `need` lowest indices are: all of them in the usual case, which
    // one more strided pass collects; otherwise thread t counts and takes the equal keys of a contiguous range, in index order, after a scan.
    const bool all_equal_taken = s_equal == need;
    for (int base = 0; base < n; base += 4 * kSampleThreads) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = base + u * kSampleThreads + tid;
            v[u] = i < n ? logits[i] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = base + u * kSampleThreads + tid;
            if (i >= n) continue;
            const uint32_t k = sample_key(__fmul_rn(v[u], inv_temp));
            if (k > prefix || (all_equal_taken && k == prefix)) {
                const unsigned int at = atomicAdd(&s_count, 1u);
                if (at < static_cast<unsigned int>(kSampleMaxK)) c_key[at] = k, c_idx[at] = static_cast<uint32_t>(i);
            }
        }
    }
    if (!all_equal_taken) {  // (uniform over the block)
        const int per = (n + kSampleThreads - 1) / kSampleThreads, i0 = min(n, tid * per), i1 = min(n, i0 + per);
        unsigned int mine_eq = 0;
        for (int i = i0; i < i1; ++i) mine_eq += sample_key(__fmul_rn(logits[i], inv_temp)) == prefix ? 1u : 0u;
        scan[tid] = mine_eq;
        __syncthreads();
        for (int o = 1; o < kSampleThreads; o <<= 1) {  // inclusive scan
            const unsigned int add = tid >= o ? scan[tid - o] : 0u;
            __syncthreads();
            scan[tid] += add;
            __syncthreads();
        }
        unsigned int eq_rank = scan[tid] - mine_eq;  // equal keys in the ranges before this thread's
        for (int i = i0; i < i1 && eq_rank < need; ++i) {
            if (sample_key(__fmul_rn(logits[i], inv_temp)) != prefix) continue;
            ++eq_rank;
            const unsigned int at = atomicAdd(&s_count, 1u);
            if (at < static_cast<unsigned int>(kSampleMaxK)) c_key[at] = prefix, c_idx[at] = static_cast<uint32_t>(i);
        }
    }
    __syncthreads();
    const int m = min(static_cast<int>(s_count), top_k);  // = top_k
    // order by counting: descending key, ascending index among equal keys (the stable sort's order)
    if (tid < m) {
        const uint32_t k = c_key[tid], ix = c_idx[tid];
        int rank = 0;
        for (int j = 0; j < m; ++j) rank += (c_key[j] > k || (c_key[j] == k && c_idx[j] < ix)) ? 1 : 0;
        o_idx[rank] = ix;
        o_val[rank] = __fmul_rn(logits[ix], inv_temp);
    }
    __syncthreads();
    __shared__ float s_mx;
    if (tid == 0) {
        float mx = o_val[0];
        for (int i = 0; i < m; ++i)
            if (o_val[i] > mx) mx = o_val[i];
        s_mx = mx;
    }
    __syncthreads();
    if (tid < m) o_val[tid] = device_expf(__fsub_rn(o_val[tid], s_mx));  // every exponential on its own; the sums below stay in candidate order
    __syncthreads();
    if (tid != 0) return;
    double sum = 0.0;
    for (int i = 0; i < m; ++i) sum += static_cast<double>(o_val[i]);
    if (sum > 0.0) {
        const float inv = __double2float_rn(1.0 / sum);
        for (int i = 0; i < m; ++i) o_val[i] = __fmul_rn(o_val[i], inv);
    }
    int cutoff = m;
    if (top_p < 1.0f) {
        float cum = 0.0f;
        for (int i = 0; i < m; ++i) {
            cum = __fadd_rn(cum, o_val[i]);
            if (cum >= top_p) {
                cutoff = i + 1;
                break;
            }
        }
    }
    float psum = 0.0f;
    for (int i = 0; i < cutoff; ++i) psum = __fadd_rn(psum, o_val[i]);
    if (psum > 0.0f) {
        const float inv = __fdiv_rn(1.0f, psum);
        for (int i = 0; i < cutoff; ++i) o_val[i] = __fmul_rn(o_val[i], inv);
    }
    unsigned long long x = *rng;
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    *rng = x;
    const float r = __fdiv_rn(__ull2float_rn(x), 18446744073709551616.0f);
    float acc = 0.0f;
    uint32_t chosen = o_idx[0];
    for (int i = 0; i < cutoff; ++i) {
        acc = __fadd_rn(acc, o_val[i]);
        if (r <= acc || i + 1 == cutoff) {
            chosen = o_idx[i];
            break;
        }
    }
    *token = chosen;
}

// next position (the generation loop runs on the device: the token comes from argmax_kernel, the position from here)
__global__ void advance_kernel(uint32_t* pos, uint32_t* history, const uint32_t* token) {
    history[pos[0]] = token[0];
    pos[0] += 1;
}
// the same for a step of several sequences: token z of the step belongs to sequence slot[z] (or z)
__global__ void advance_batch_kernel(uint32_t* pos, uint32_t* last, const uint32_t* chosen, const uint32_t* slot, int n) {
    const int z = blockIdx.x * blockDim.x + threadIdx.x;
    if (z >= n) return;
    const uint32_t s = slot != nullptr ? slot[z] : static_cast<uint32_t>(z);
    last[s] = chosen[z];
    pos[s] += 1;
}
// tokens of a step: the given ones, or the last chosen token of every listed sequence
__global__ void gather_tokens_kernel(uint32_t* tokens, const uint32_t* last, const uint32_t* slot, int n) {
    const int z = blockIdx.x * blockDim.x + threadIdx.x;
    if (z < n) tokens[z] = last[slot != nullptr ? slot[z] : static_cast<uint32_t>(z)];
}

}  // namespace qtb
