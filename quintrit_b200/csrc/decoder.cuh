// Whole-token decoder on the device: buffers, launch sequence, CUDA graph, greedy generation loop. Included by capi.cu.
// Host-side counterpart in the reference: rust/crates/quintrit-runtime/src/gpu.rs (GpuModel::load :183-260, new_session
// :289-339, enqueue :389-453, forward :459-493, time_token :346-370).
#pragma once
#include <cmath>
#include <cstring>
#include <vector>

#include "capi_common.cuh"
#include "decode.cuh"
#include "gemv_lut.cuh"
#include "megakernel.cuh"

struct quintrit_b200_matrix;
void qtb_release_stacked(quintrit_b200_matrix* m);  // capi.cu: deletes the host object of a stacked matrix

struct quintrit_b200_decoder {
    uint32_t magic;
    int device, sm_count;
    int arch, f32_values;
    int hidden, inter, layers, q_heads, kv_heads, head_dim, vocab, ctx, rope_dims;
    int q_dim, kv_dim;
    float eps, rope_theta;
    std::vector<float> scales;  // layers * 7
    // device memory
    std::vector<void*> allocs;
    std::vector<void*> owned_matrices;  // matrix handles created by the GGUF loader; released with the decoder
    __half *embed, *lm_head, *kc, *vc, *x16;
    float *out_norm, *cos_sin, *x, *q, *part_acc, *part_ms, *logits;
    float* scores = nullptr;  // single-kernel path: attention scores of the current token, [q_heads][ctx]
    std::vector<float*> norms;  // layers * 4 (device)
    std::vector<float*> qk_norms;  // layers * 2 (device): query and key head norms, empty for models without them
    int8_t *a8_h, *a8_q, *a8_i;
    float *s_h, *s_q, *s_i;
    int32_t *acc_qkv, *acc_o, *acc_gu, *acc_down;
    uint32_t *d_token, *d_pos, *d_history;
    unsigned long long* d_rng = nullptr;       // state of the sampler's xorshift64 generator (runtime level, sampling on the device)
    unsigned int* d_counters;
    qtb::GemvItem* d_items;
    std::vector<int> item_first, item_count;  // layers * 4 launches: qkv, o, gate+up, down
    // single-kernel path (LLaMA / Falcon3 architecture)
    bool use_mega;
    qtb::MegaArgs mega;
    void (*mega_kernel)(qtb::MegaArgs);
    size_t mega_smem;
    float *xa, *xb, *v_inter, *best_val;
    unsigned int *amax_bits, *best_idx, *bar;
    bool attn_v2 = false;
    qtb::AttnGqaKernel attn_gqa = nullptr;     // one-launch-per-step and batched paths: the grouped attention kernel, if this model's shape has one
    size_t attn_gqa_smem = 0;
    size_t attn_gqa_pad = 0;                   // experiments: extra shared memory per block, which lowers the number of resident blocks
    float* attn_out = nullptr;
    float *fac = nullptr, *fac_M = nullptr;
    unsigned int *fac_flags = nullptr, *fac_done = nullptr;
    unsigned long long* trace;  // phase timestamps of the last traced step (13 per layer + 3)
    cudaStream_t stream;
    cudaGraphExec_t graph_step;               // one token: embed ... argmax (token and position read from device memory)
    bool graph_ready;
    uint32_t host_pos;                         // tokens in the KV cache
    // tensor parallelism: this rank's share of a model split over tp_world GPUs (1 = none)
    bool block_scaled = false;                 // every projection is a block-scaled (Q2_0) matrix: Q8_0 activations, F32 results
    std::vector<const quintrit_b200_matrix*> mats;  // the projections (layers * 7), for the block-scaled launches
    float* q8_d = nullptr;                     // Q8_0 block scales of the current projection input
    bool bf16_tables = false;                  // embedding and output head hold BF16 instead of F16 bit patterns
    int tp_rank = 0, tp_world = 1;
    bool attn_replicated = false;              // tensor parallelism with every head on every rank (the ranks do not divide the KV heads)
    int q_dim_full = 0, inter_full = 0, vocab_full = 0;
    unsigned char* tp_box = nullptr;           // the exchange box of this rank (one allocation, shared with the peers)
    size_t tp_box_bytes = 0;
    unsigned int* tp_seq = nullptr;
    bool tp_attached = false;
    void* tp_peer[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};  // peer boxes opened through IPC
    // prompt ingestion in chunks of up to kPrefillMax tokens (batched projections on the tensor cores): per-token rows of the step buffers, made on first use
    struct Prefill {
        uint32_t* tokens = nullptr;
        uint32_t* pos = nullptr;
        float *x = nullptr, *q = nullptr, *part_acc = nullptr, *part_ms = nullptr, *s_h = nullptr, *s_q = nullptr, *s_i = nullptr;
        int8_t *a8_h = nullptr, *a8_q = nullptr, *a8_i = nullptr;
        int32_t *acc_qkv = nullptr, *acc_o = nullptr, *acc_gu = nullptr, *acc_down = nullptr;
        bool warm = false, graph_ready = false;  // a full chunk ran once (lazy allocations done); the graph of a full chunk exists
        cudaGraphExec_t graph = nullptr;
        // batched products: per layer the row-wise stacks q | k | v and gate | up (nullptr: separate launches), and the buffers for the partial
        // sums of split products, one per projection kind (q, k, v, o, gate, up, down; a stack uses the first of its kind)
        bool gemm_ready = false;
        std::vector<quintrit_b200_matrix*> stack;            // layers * 2
        std::vector<quintrit_b200_matrix*> stacked_objects;  // owned: released with the decoder (their device memory is in `allocs`)
        int32_t* parts[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    } pf;
};

namespace qtb {

constexpr uint32_t kMagicDecoder = 0x51544244u;  // "QTBD"

inline int check_decoder(const quintrit_b200_decoder* d) {
    if (d == nullptr || d->magic != kMagicDecoder) return fail(QUINTRIT_ERR_INVALID_HANDLE, "decoder handle is NULL, freed or of the wrong type");
    return QUINTRIT_OK;
}

template <typename T>
int dev_alloc(quintrit_b200_decoder* d, T** p, size_t count, bool zero = true) {
    void* q = nullptr;
    const size_t bytes = std::max<size_t>(count * sizeof(T), 16);
    cudaError_t e = cudaMalloc(&q, bytes);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(decoder buffer)");
    d->allocs.push_back(q);
    if (zero && (e = cudaMemset(q, 0, bytes)) != cudaSuccess) return cuda_fail(e, "cudaMemset(decoder buffer)");
    *p = static_cast<T*>(q);
    return QUINTRIT_OK;
}
template <typename T>
int dev_upload(quintrit_b200_decoder* d, T** p, const void* host, size_t count) {
    int rc = dev_alloc(d, p, count, false);
    if (rc != QUINTRIT_OK) return rc;
    QTB_CUDA(cudaMemcpy(*p, host, count * sizeof(T), cudaMemcpyHostToDevice));
    return QUINTRIT_OK;
}

inline void destroy_decoder(quintrit_b200_decoder* d) {
    if (d == nullptr) return;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(d->device);
    for (void* q : d->tp_peer)
        if (q != nullptr) cudaIpcCloseMemHandle(q);
    if (d->graph_ready) cudaGraphExecDestroy(d->graph_step);
    if (d->pf.graph_ready) cudaGraphExecDestroy(d->pf.graph);
    for (quintrit_b200_matrix* m : d->pf.stacked_objects) qtb_release_stacked(m);
    if (d->stream) cudaStreamDestroy(d->stream);
    for (void* p : d->allocs) cudaFree(p);
    if (prev >= 0) cudaSetDevice(prev);
    d->magic = 0;
    delete d;
}

// Enqueues one GEMV launch (its items were built at creation) on the decoder's stream.
inline int decoder_gemv(quintrit_b200_decoder* d, int layer, int which, const int8_t* act, int32_t* out) {
    const int k = layer * 4 + which;
    return launch_gemv(d->d_items + d->item_first[k], d->item_count[k], act, out, d->d_counters, d->sm_count, d->stream);
}

// Block-scaled projection `which` (0..6) of a layer: out (F32) = W x for Q8_0 blocks (codes, d->q8_d).
// Block-scaled projections `first` .. `first + count - 1` of a layer (at most three, all over the activation codes `codes`) in one
// launch; their results go to `out` one after the other.
inline int decoder_gemv_bs(quintrit_b200_decoder* d, int layer, int first, const int8_t* codes, float* out, int count = 1) {
    BsMatrices bm{};
    size_t rows_all = 0;
    unsigned groups = 0;
    const quintrit_b200_matrix* m0 = d->mats[static_cast<size_t>(layer) * 7 + first];
    for (int i = 0; i < 3; ++i) {
        if (i < count) {
            const quintrit_b200_matrix* m = d->mats[static_cast<size_t>(layer) * 7 + first + i];
            bm.planar[i] = m->d_planar, bm.w_scales[i] = m->d_wscales, bm.out[i] = out + rows_all, bm.rows[i] = static_cast<unsigned>(m->rows);
            rows_all += m->rows;
            groups += static_cast<unsigned>((m->rows + kBsRowsPerCta - 1) / kBsRowsPerCta);
        }
        bm.group_end[i] = groups;
    }
    bm.count = count;
    block_scaled_launch(bm, codes, d->q8_d, m0->cols, d->sm_count, d->stream);
    ++g_launches;
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "block-scaled GEMV launch");
    return QUINTRIT_OK;
}

// Attention of n tokens: all query heads of a KV head in one block where an instantiation exists, else one query head per block.
inline void launch_attention(quintrit_b200_decoder* d, const AttnArgs& at, int n, cudaStream_t s) {
    // several tokens: the query heads of a KV head share one pass over its rows; one token: more, wider blocks pull the rows faster
    if (d->attn_gqa != nullptr && n > 1)
        d->attn_gqa<<<dim3(d->kv_heads, 4, n), kAttnGqaThreads, d->attn_gqa_smem + d->attn_gqa_pad, s>>>(at);
    else
        attention_kernel<<<dim3(d->q_heads, 4, n), kAttnThreads, attention_smem(d->head_dim), s>>>(at);
}

#define QTB_LAUNCH_CHECK()                                   \
    do {                                                     \
        ++g_launches;                                        \
        cudaError_t qtb_e_ = cudaGetLastError();             \
        if (qtb_e_ != cudaSuccess) return cuda_fail(qtb_e_, "kernel launch"); \
    } while (0)

// The launch sequence of one token (gpu.rs:389-453 reshaped: 4 GEMV launches and 5 float kernels per layer).
inline int enqueue_token(quintrit_b200_decoder* d, bool with_head) {
    cudaStream_t s = d->stream;
    const int H = d->hidden, I = d->inter, qd = d->q_dim, kvd = d->kv_dim;
    const bool bs = d->block_scaled;  // Q2_0 model: the int32 result buffers hold F32 results, activations are Q8_0 blocks
    embed_kernel<<<(H + 255) / 256, 256, 0, s>>>(d->embed, d->d_token, H, d->x, d->bf16_tables);
    QTB_LAUNCH_CHECK();
    for (int l = 0; l < d->layers; ++l) {
        const float* sc = d->scales.data() + l * 7;
        NormQuantArgs n1{};
        n1.x = d->x;
        if (l > 0) {
            n1.acc_prev = d->acc_down;
            n1.scale_prev = d->s_i;
            n1.ws_prev = d->scales[(l - 1) * 7 + 6];
        }
        n1.norm_w = d->norms[l * 4 + 0];
        n1.eps = d->eps;
        n1.n = H;
        n1.q_out = d->a8_h;
        n1.scale_out = d->s_h;
        n1.zero_a = d->acc_qkv;
        n1.zero_a_n = bs ? 0 : qd + 2 * kvd;
        n1.block_scaled = bs, n1.q8_d = d->q8_d;
        norm_quant_kernel<<<1, kRowThreads, H * sizeof(float), s>>>(n1);
        QTB_LAUNCH_CHECK();
        int rc;
        if (bs) {
            float* f = reinterpret_cast<float*>(d->acc_qkv);
            if ((rc = decoder_gemv_bs(d, l, 0, d->a8_h, f, 3)) != QUINTRIT_OK) return rc;  // q | k | v
        } else if ((rc = decoder_gemv(d, l, 0, d->a8_h, d->acc_qkv)) != QUINTRIT_OK) {
            return rc;
        }
        if (!d->qk_norms.empty() && d->qk_norms[l * 2] != nullptr) {  // query/key-norm (block-scaled models: acc_qkv holds floats)
            const int heads = d->q_heads + d->kv_heads;
            qk_norm_kernel<<<(heads + 3) / 4, 128, 0, s>>>(reinterpret_cast<float*>(d->acc_qkv), d->q_heads, d->kv_heads, d->head_dim, d->qk_norms[l * 2], d->qk_norms[l * 2 + 1], d->eps);
            QTB_LAUNCH_CHECK();
        }
        RopeKvArgs rk{};
        rk.acc = d->acc_qkv;
        rk.act_scale = d->s_h;
        rk.ws_q = sc[0], rk.ws_k = sc[1], rk.ws_v = sc[2];
        rk.cos_sin = d->cos_sin;
        rk.pos = d->d_pos;
        rk.q_dim = qd, rk.kv_dim = kvd, rk.head_dim = d->head_dim, rk.rope_dims = d->rope_dims, rk.neox = d->arch != QUINTRIT_B200_ARCH_LLAMA;
        rk.q_out = d->q;
        rk.k_cache = d->kc + static_cast<size_t>(l) * d->ctx * kvd;
        rk.v_cache = d->vc + static_cast<size_t>(l) * d->ctx * kvd;
        rk.block_scaled = bs;
        rope_kv_kernel<<<((qd + kvd) / 2 + kvd + 255) / 256, 256, 0, s>>>(rk);
        QTB_LAUNCH_CHECK();
        AttnArgs at{};
        at.q = d->q;
        at.k_cache = rk.k_cache;
        at.v_cache = rk.v_cache;
        at.pos = d->d_pos;
        at.head_dim = d->head_dim, at.kv_dim = kvd, at.gqa = d->q_heads / d->kv_heads, at.ctx = d->ctx, at.f32_values = d->f32_values;
        at.scale = 1.0f / std::sqrt(static_cast<float>(d->head_dim));  // attention.rs:46
        at.part_acc = d->part_acc;
        at.part_ms = d->part_ms;
        launch_attention(d, at, 1, s);
        QTB_LAUNCH_CHECK();
        AttnFinishArgs af{};
        af.part_acc = d->part_acc;
        af.part_ms = d->part_ms;
        af.pos = d->d_pos;
        af.q_heads = d->q_heads, af.head_dim = d->head_dim, af.ctx = d->ctx;
        af.sub_norm_w = d->norms[l * 4 + 2];
        af.eps = d->eps;
        af.q_out = d->a8_q;
        af.scale_out = d->s_q;
        af.zero_a = d->acc_o;
        af.zero_a_n = bs ? 0 : H;
        af.q8_d = bs ? d->q8_d : nullptr;
        if (bs && af.sub_norm_w == nullptr)
            attn_finish_q8_kernel<<<(qd / 32 + kQ8BlockThreads / 32 - 1) / (kQ8BlockThreads / 32), kQ8BlockThreads, 0, s>>>(af);
        else
            attn_finish_kernel<<<1, kRowThreads, qd * sizeof(float), s>>>(af);
        QTB_LAUNCH_CHECK();
        rc = bs ? decoder_gemv_bs(d, l, 3, d->a8_q, reinterpret_cast<float*>(d->acc_o)) : decoder_gemv(d, l, 1, d->a8_q, d->acc_o);
        if (rc != QUINTRIT_OK) return rc;
        NormQuantArgs n2{};
        n2.x = d->x;
        n2.acc_prev = d->acc_o;
        n2.scale_prev = d->s_q;
        n2.ws_prev = sc[3];
        n2.norm_w = d->norms[l * 4 + 1];
        n2.eps = d->eps;
        n2.n = H;
        n2.q_out = d->a8_h;
        n2.scale_out = d->s_h;
        n2.zero_a = d->acc_gu;
        n2.zero_a_n = bs ? 0 : 2 * I;
        n2.block_scaled = bs, n2.q8_d = d->q8_d;
        norm_quant_kernel<<<1, kRowThreads, H * sizeof(float), s>>>(n2);
        QTB_LAUNCH_CHECK();
        if (bs) {
            float* f = reinterpret_cast<float*>(d->acc_gu);
            if ((rc = decoder_gemv_bs(d, l, 4, d->a8_h, f, 2)) != QUINTRIT_OK) return rc;  // gate | up
        } else if ((rc = decoder_gemv(d, l, 2, d->a8_h, d->acc_gu)) != QUINTRIT_OK) {
            return rc;
        }
        ActQuantArgs aq{};
        aq.acc_gate = d->acc_gu;
        aq.acc_up = d->acc_gu + I;
        aq.act_scale = d->s_h;
        aq.ws_gate = sc[4], aq.ws_up = sc[5];
        aq.n = I, aq.relu2 = d->arch == QUINTRIT_B200_ARCH_BITNET;
        aq.sub_norm_w = d->norms[l * 4 + 3];
        aq.eps = d->eps;
        aq.q_out = d->a8_i;
        aq.scale_out = d->s_i;
        aq.zero_a = d->acc_down;
        aq.zero_a_n = bs ? 0 : H;
        aq.block_scaled = bs, aq.q8_d = d->q8_d;
        if (bs && aq.sub_norm_w == nullptr)
            act_quant_q8_kernel<<<(I / 32 + kQ8BlockThreads / 32 - 1) / (kQ8BlockThreads / 32), kQ8BlockThreads, 0, s>>>(aq);
        else
            act_quant_kernel<<<1, kRowThreads, I * sizeof(float), s>>>(aq);
        QTB_LAUNCH_CHECK();
        rc = bs ? decoder_gemv_bs(d, l, 6, d->a8_i, reinterpret_cast<float*>(d->acc_down)) : decoder_gemv(d, l, 3, d->a8_i, d->acc_down);
        if (rc != QUINTRIT_OK) return rc;
    }
    if (with_head) {
        NormQuantArgs nf{};
        nf.x = d->x;
        nf.acc_prev = d->acc_down;
        nf.scale_prev = d->s_i;
        nf.ws_prev = d->scales[(d->layers - 1) * 7 + 6];
        nf.norm_w = d->out_norm;
        nf.eps = d->eps;
        nf.n = H;
        nf.y16_out = d->x16;
        nf.y16_bf16 = d->bf16_tables;
        nf.block_scaled = bs;
        norm_quant_kernel<<<1, kRowThreads, H * sizeof(float), s>>>(nf);
        QTB_LAUNCH_CHECK();
        lm_head_kernel<<<d->sm_count * 8, 256, H * sizeof(float), s>>>(d->lm_head, d->x16, H, d->vocab, d->logits, d->bf16_tables);
        QTB_LAUNCH_CHECK();
        argmax_kernel<<<1, 1024, 0, s>>>(d->logits, d->vocab, d->d_token);
        QTB_LAUNCH_CHECK();
    }
    return QUINTRIT_OK;
}

// Sets the device-side position and token from host values.
inline int decoder_set(quintrit_b200_decoder* d, uint32_t token, uint32_t pos) {
    QTB_CUDA(cudaMemcpyAsync(d->d_token, &token, sizeof token, cudaMemcpyHostToDevice, d->stream));
    QTB_CUDA(cudaMemcpyAsync(d->d_pos, &pos, sizeof pos, cudaMemcpyHostToDevice, d->stream));
    return QUINTRIT_OK;
}

// Captures [one token + advance] into a graph the first time it is needed.
inline int decoder_graph(quintrit_b200_decoder* d) {
    if (d->graph_ready) return QUINTRIT_OK;
    cudaGraph_t g = nullptr;
    QTB_CUDA(cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal));
    int rc = enqueue_token(d, true);
    if (rc == QUINTRIT_OK) {
        advance_kernel<<<1, 1, 0, d->stream>>>(d->d_pos, d->d_history, d->d_token);
        ++g_launches;
    }
    cudaError_t e = cudaStreamEndCapture(d->stream, &g);
    if (rc != QUINTRIT_OK) {
        if (g) cudaGraphDestroy(g);
        return rc;
    }
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture");
    e = cudaGraphInstantiate(&d->graph_step, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
    d->graph_ready = true;
    return QUINTRIT_OK;
}

}  // namespace qtb
