// A mixture-of-experts feed-forward block on the device: softmax router over BF16 rows, top-k experts, every expert a ternary SwiGLU
// FFN with int8 absmax activations, the weighted outputs added in selection order. Included by capi.cu.
//
// The reference has no block of this kind (its `Moe` is Nemotron-H's: sigmoid router with a bias, squared-ReLU experts, a shared
// expert, rust/crates/quintrit-runtime/src/hybrid.rs:798-869); the block is composed of the reference's pieces, each computed as the
// reference computes it: the router as a BF16 projection (hybrid.rs:327-333), softmax (ops.rs:274-298), experts by descending
// probability as std::sort leaves them (hybrid.rs:828-831), their probabilities divided by their sum (hybrid.rs:833-839), an
// expert as the dense model's FFN (layer.rs:123-177, ops.rs:241-267, 427-464), the weighted outputs added in selection order
// (hybrid.rs:847-858).
//
// Launch sequence for a batch of tokens: prepare (BF16 bits and int8 codes of every token), router (every expert row against all
// tokens), select (softmax, ranking, weights), items (the work list of the chosen experts' gate | up and down projections, built on
// the device from the chosen ids), the GEMV kernel over the gate | up items, activation (SwiGLU and int8 codes per chosen expert),
// the GEMV kernel over the down items, combine. Two persistent GEMV launches serve all (token, expert) pairs of the batch.
#pragma once
#include "decode.cuh"
#include "gemv_lut.cuh"

namespace qtb {

struct MoeExpertRef {
    const uint4* w_gu;    // stream-layout weights of the expert's gate rows followed by its up rows (2 * inter x hidden)
    const uint4* w_down;  // hidden x inter
    float ws_gate, ws_up, ws_down;
    int pad;
};

// One block per token: the BF16 bit patterns of x (the router's input, ops.rs:656-664) and its int8 absmax codes (the experts' input).
__global__ void __launch_bounds__(kRowThreads) moe_prepare_kernel(const float* __restrict__ x, int hidden, __half* __restrict__ x16, int8_t* __restrict__ a8,
                                                                  float* __restrict__ s_x) {
    __shared__ float sh_f[32];
    extern __shared__ float y_s[];
    const size_t b = blockIdx.x;
    float amax = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += kRowThreads) {
        const float v = x[b * hidden + i];
        y_s[i] = v;
        x16[b * hidden + i] = __ushort_as_half(float_to_bf16_bits(v));
        amax = fmaxf(amax, fabsf(v));
    }
    __syncthreads();
    quantize_vector(y_s, hidden, amax, a8 + b * hidden, s_x + b, nullptr, sh_f);
}

// Router logits: one warp per expert row and group of four tokens. The dot product is ggml_vec_dot_bf16's (ops.rs:688-712): lane l owns the
// elements 32 i + l, product and sum rounded separately in the order of i, then the lanes are reduced (dot_lane_reduce_bf16), which is what
// lm_head_kernel does for BF16 tables; a few hundred rows against a handful of tokens are latency, not bandwidth, so the rows are spread
// over many small blocks instead of the head kernel's few large ones.
__global__ void __launch_bounds__(128) moe_router_kernel(const __half* __restrict__ router, const __half* __restrict__ x16, int hidden, int n_experts, int batch,
                                                         float* __restrict__ logits) {
    // grid (rows / 4, tokens / 4): a warp takes one expert row and four tokens; the elements of eight steps are requested together
    const int lane = threadIdx.x & 31, row = blockIdx.x * 4 + (threadIdx.x >> 5), b0 = blockIdx.y * 4;
    if (row >= n_experts) return;
    const __half* w = router + static_cast<size_t>(row) * hidden + lane;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const __half* x[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) x[t] = x16 + static_cast<size_t>(min(b0 + t, batch - 1)) * hidden + lane;
    for (int i0 = 0; i0 < hidden; i0 += 256) {
        unsigned short wr[8], xr[4][8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int i = i0 + 32 * k;
            wr[k] = i < hidden ? __half_as_ushort(w[i]) : 0;
#pragma unroll
            for (int t = 0; t < 4; ++t) xr[t][k] = i < hidden ? __half_as_ushort(x[t][i]) : 0;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (i0 + 32 * k < hidden) {
                const float wv = bf16_bits_to_float(wr[k]);
#pragma unroll
                for (int t = 0; t < 4; ++t) acc[t] = __fadd_rn(acc[t], __fmul_rn(bf16_bits_to_float(xr[t][k]), wv));
            }
        }
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const float sum = dot_lane_reduce_bf16(acc[t]);
        if (lane == 0 && b0 + t < batch) logits[static_cast<size_t>(b0 + t) * n_experts + row] = sum;
    }
}

// One block per token: softmax of the router logits as ops.rs:274-298 writes it (one thread, in order), every expert's rank by
// counting (descending probability; equal probabilities by lower id, and the token is flagged: std::sort decides such ties by its
// algorithm, which the host then runs), the first top_k chosen, their probabilities divided by their sum.
__global__ void __launch_bounds__(256) moe_select_kernel(const float* __restrict__ logits, int n_experts, int top_k, float* __restrict__ probs,
                                                         uint32_t* __restrict__ chosen, float* __restrict__ weights, unsigned int* __restrict__ tie) {
    extern __shared__ float p_s[];  // n_experts probabilities, then top_k selected ones
    float* w_s = p_s + n_experts;
    const size_t b = blockIdx.x;
    const int tid = threadIdx.x;
    for (int i = tid; i < n_experts; i += 256) p_s[i] = logits[b * n_experts + i];
    if (tid == 0) tie[b] = 0u;
    __syncthreads();
    __shared__ float s_mx, s_inv;
    if (tid == 0) {
        float mx = p_s[0];
        for (int i = 1; i < n_experts; ++i)
            if (p_s[i] > mx) mx = p_s[i];
        s_mx = mx;
    }
    __syncthreads();
    for (int i = tid; i < n_experts; i += 256) p_s[i] = device_expf(__fsub_rn(p_s[i], s_mx));  // (every exponential on its own: any thread may take it)
    __syncthreads();
    if (tid == 0) {
        double sum = 0.0;
        for (int i = 0; i < n_experts; ++i) sum += static_cast<double>(p_s[i]);  // in the order of the experts, as the reference adds them
        s_inv = sum > 0.0 ? __double2float_rn(1.0 / sum) : 1.0f;
    }
    __syncthreads();
    for (int i = tid; i < n_experts; i += 256) p_s[i] = __fmul_rn(p_s[i], s_inv);  // (a sum of zero leaves the values as they are: times 1)
    __syncthreads();
    for (int i = tid; i < n_experts; i += 256) {
        const float p = p_s[i];
        probs[b * n_experts + i] = p;
        int rank = 0;
        bool tied = false;
        for (int j = 0; j < n_experts; ++j) {
            const float q = p_s[j];
            rank += (q > p || (q == p && j < i)) ? 1 : 0;
            tied |= q == p && j != i;
        }
        if (tied) atomicOr(tie + b, 1u);
        if (rank < top_k) {
            chosen[b * top_k + rank] = static_cast<uint32_t>(i);
            w_s[rank] = p;
        }
    }
    __syncthreads();
    if (tid == 0) {
        double sum = 0.0;
        for (int i = 0; i < top_k; ++i) sum += static_cast<double>(w_s[i]);
        const float s = fmaxf(__double2float_rn(sum), 6.103515625e-5f);
        for (int i = 0; i < top_k; ++i) weights[b * top_k + i] = __fdiv_rn(w_s[i], s);
    }
}

// The work lists of the two GEMV launches, one thread per item: for pair z = (token, selection slot) the chosen expert's gate | up
// projection (block pairs over the hidden columns, all row tiles in one item) and its down projection (block pairs over the
// intermediate columns, the row tiles in `chunks_down` ranges). Same decomposition as build_items on the host.
// `local_z` lists the n_z pairs whose expert this GPU holds (all pairs on one GPU; a share of them under expert parallelism).
__global__ void moe_items_kernel(const MoeExpertRef* __restrict__ experts, const uint32_t* __restrict__ chosen, const uint32_t* __restrict__ local_z, int n_z, int top_k, int hidden,
                                 int inter, int inter_pad, int chunks_down, GemvItem* __restrict__ gu_items, GemvItem* __restrict__ down_items) {
    const int blocks_gu = (hidden + kBlockTrits - 1) / kBlockTrits, pairs_gu = (blocks_gu + 1) / 2, tiles_gu = (2 * inter + kTileRows - 1) / kTileRows;
    const int blocks_d = (inter + kBlockTrits - 1) / kBlockTrits, pairs_d = (blocks_d + 1) / 2, tiles_d = (hidden + kTileRows - 1) / kTileRows;
    const int n_gu = n_z * pairs_gu, n_d = n_z * pairs_d * chunks_down;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_gu + n_d; i += gridDim.x * blockDim.x) {
        GemvItem it{};
        if (i < n_gu) {
            const int z = static_cast<int>(local_z[i / pairs_gu]), g = 2 * (i % pairs_gu);
            const MoeExpertRef& e = experts[chosen[z]];
            it.wa = e.w_gu + static_cast<size_t>(g) * tiles_gu * 64;
            it.nblk = g + 1 < blocks_gu ? 2 : 1;
            it.wb = it.nblk == 2 ? e.w_gu + static_cast<size_t>(g + 1) * tiles_gu * 64 : it.wa;
            it.act_off = static_cast<unsigned long long>(z / top_k) * hidden;
            it.out_off = static_cast<unsigned long long>(z) * 2 * inter;
            it.rows = 2 * inter, it.cols = hidden, it.col0 = g * kBlockTrits, it.tile0 = 0, it.ntiles = tiles_gu;
            gu_items[i] = it;
        } else {
            const int k = i - n_gu, c = k % chunks_down, p = (k / chunks_down) % pairs_d, z = static_cast<int>(local_z[k / (chunks_down * pairs_d)]), g = 2 * p;
            const MoeExpertRef& e = experts[chosen[z]];
            const int t0 = tiles_d * c / chunks_down, t1 = tiles_d * (c + 1) / chunks_down;
            it.wa = e.w_down + (static_cast<size_t>(g) * tiles_d + t0) * 64;
            it.nblk = g + 1 < blocks_d ? 2 : 1;
            it.wb = it.nblk == 2 ? e.w_down + (static_cast<size_t>(g + 1) * tiles_d + t0) * 64 : it.wa;
            it.act_off = static_cast<unsigned long long>(z) * inter_pad;
            it.out_off = static_cast<unsigned long long>(z) * hidden;
            it.rows = hidden, it.cols = inter, it.col0 = g * kBlockTrits, it.tile0 = t0, it.ntiles = t1 - t0;
            down_items[k] = it;
        }
    }
}

// One block per pair z: gate and up sums to floats (one multiply by weight_scale / act_scale each, layer.rs:143-147), SwiGLU
// (ops.rs:427-464), int8 absmax codes of the result for the down projection.
__global__ void __launch_bounds__(kRowThreads) moe_act_quant_kernel(const int32_t* __restrict__ acc_gu, const MoeExpertRef* __restrict__ experts, const uint32_t* __restrict__ chosen,
                                                                    const uint32_t* __restrict__ local_z, const float* __restrict__ s_x, int top_k, int inter, int inter_pad,
                                                                    int8_t* __restrict__ a8_i, float* __restrict__ s_i) {
    __shared__ float sh_f[32];
    extern __shared__ float y_s[];
    const size_t z = local_z[blockIdx.x];
    const MoeExpertRef& e = experts[chosen[z]];
    const float s_in = s_x[z / top_k];
    const bool live = s_in > 0.0f;
    const float pg = live ? __fdiv_rn(e.ws_gate, s_in) : 0.0f, pu = live ? __fdiv_rn(e.ws_up, s_in) : 0.0f;
    const int32_t* acc = acc_gu + z * 2 * inter;
    float amax = 0.0f;
    for (int i = threadIdx.x; i < inter; i += kRowThreads) {
        const float g = live ? __fmul_rn(static_cast<float>(acc[i]), pg) : 0.0f;
        const float u = live ? __fmul_rn(static_cast<float>(acc[inter + i]), pu) : 0.0f;
        const float v = __fmul_rn(ggml_silu(g), u);
        y_s[i] = v;
        amax = fmaxf(amax, fabsf(v));
    }
    __syncthreads();
    quantize_vector(y_s, inter, amax, a8_i + z * inter_pad, s_i + z, nullptr, sh_f);
}

// pairs[z][h] = the down result of pair z as floats: one multiply by weight_scale / act_scale, zero for a zero activation scale
// (layer.rs:143-150) and for a pair whose expert another GPU holds (that GPU writes the value; the exchange adds the shares, of which
// exactly one is not zero).
__global__ void moe_scale_pairs_kernel(const int32_t* __restrict__ acc_down, const MoeExpertRef* __restrict__ experts, const uint32_t* __restrict__ chosen,
                                       const float* __restrict__ s_i, int hidden, float* __restrict__ pairs) {
    const size_t z = blockIdx.y;
    const MoeExpertRef& e = experts[chosen[z]];
    const float s = s_i[z];
    const bool live = e.w_down != nullptr && s > 0.0f;
    const float post = live ? __fdiv_rn(e.ws_down, s) : 0.0f;
    for (int h = blockIdx.x * blockDim.x + threadIdx.x; h < hidden; h += gridDim.x * blockDim.x)
        pairs[z * hidden + h] = live ? __fmul_rn(static_cast<float>(acc_down[z * hidden + h]), post) : 0.0f;
}

// out[token][h] = the pairs' results weighted and added in selection order, the first one assigned (hybrid.rs:853-857).
__global__ void moe_combine_kernel(const float* __restrict__ pairs, const float* __restrict__ weights, int top_k, int hidden, float* __restrict__ out) {
    const size_t b = blockIdx.y;
    for (int h = blockIdx.x * blockDim.x + threadIdx.x; h < hidden; h += gridDim.x * blockDim.x) {
        float o = 0.0f;
        for (int i = 0; i < top_k; ++i) {
            const size_t z = b * top_k + i;
            const float v = __fmul_rn(pairs[z * hidden + h], weights[z]);
            o = i == 0 ? v : __fadd_rn(o, v);
        }
        out[b * hidden + h] = o;
    }
}

}  // namespace qtb
