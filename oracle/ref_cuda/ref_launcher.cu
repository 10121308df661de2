// Test infrastructure: host launchers for the REFERENCE's own CUDA kernels (rust/crates/quintrit-cuda/kernels/gemv.cu and layer.cu), so that the
// oracle and the library can be compared on a GPU with the code they restate and replace. The kernel sources are not part of this repository: the
// build (Makefile beside this file) passes their paths as QTREF_GEMV_CU / QTREF_LAYER_CU and they are compiled where they lie, with the reference's own
// compiler options (-std=c++17 -O3; quintrit-cuda/build.rs:93) for sm_100a. Launch geometry, shared-memory sizes and argument order follow the
// reference's Rust launchers: quintrit-cuda/src/gemv.rs:115-175 (grid = rows / (R * W), 32 * W threads, (staged + 256) * 8 bytes), src/layer.rs:78-85,
// 183-256, 335-380 (attention: grid (heads, 4), 384 threads, ((2 * chunk + 3) & ~3) * 4 + 128 * head_dim bytes), src/pack.rs:73-84 (permuted
// activations). Every entry takes host buffers unless its name ends in _device; every entry returns 0 or a cudaError_t.
//
// Only tests and the benchmark's reference arm use this library; nothing of the product links against it.
#include <cstdint>
#include <cstring>
#include <vector>

#include QTREF_GEMV_CU
#include QTREF_LAYER_CU

namespace {

struct Cfg {
    int r, w;
    bool act_from_global;
    void (*plain)(const uint32_t*, const uint2*, const int*, int*, int, EpArgs);
    void (*gated)(const uint32_t*, const uint2*, const int*, int*, int, EpArgs);
    void (*rope)(const uint32_t*, const uint2*, const int*, int*, int, EpArgs);
    const char* tag;
};
// the order of ALL_CONFIGS (quintrit-cuda/src/profile.rs:73)
const Cfg kCfg[6] = {
    {4, 8, false, gemv_r4_w8_pf_plain, gemv_r4_w8_pf_gated, gemv_r4_w8_pf_rope, "r4_w8_pf"},
    {4, 8, true, gemv_r4_w8_g_plain, gemv_r4_w8_g_gated, gemv_r4_w8_g_rope, "r4_w8_g"},
    {2, 4, true, gemv_r2_w4_g_d4_plain, gemv_r2_w4_g_d4_gated, gemv_r2_w4_g_d4_rope, "r2_w4_g_d4"},
    {4, 4, true, gemv_r4_w4_g_d4_plain, gemv_r4_w4_g_d4_gated, gemv_r4_w4_g_d4_rope, "r4_w4_g_d4"},
    {2, 2, true, gemv_r2_w2_g_d4_plain, gemv_r2_w2_g_d4_gated, gemv_r2_w2_g_d4_rope, "r2_w2_g_d4"},
    {2, 1, true, gemv_r2_w1_g_d4_plain, gemv_r2_w1_g_d4_gated, gemv_r2_w1_g_d4_rope, "r2_w1_g_d4"},
};
constexpr int kSharedLimit = 96 * 1024;  // SHARED_LIMIT of the reference's launchers

int blocks_per_row(int cols) { return (cols + 159) / 160; }
int act_entries(int cols) { return blocks_per_row(cols) * 32 + 16; }
size_t gemv_shared(const Cfg& c, int cols) {
    const int n = blocks_per_row(cols) * 32;
    const size_t staged = c.act_from_global ? 0 : size_t(n + (n >> 2)) + 1;
    return (staged + 256) * 8;
}
// entry b * 32 + j holds the activations of the columns b * 160 + p * 32 + j, p = 0..4, in its first five bytes
std::vector<int8_t> permute(const int8_t* act, int cols, int* sum) {
    std::vector<int8_t> out(size_t(act_entries(cols)) * 8, 0);
    int s = 0;
    for (int c = 0; c < cols; ++c) {
        const int b = c / 160, rem = c % 160;
        out[(size_t(b) * 32 + rem % 32) * 8 + rem / 32] = act[c];
        s += act[c];
    }
    *sum = s;
    return out;
}

struct Dev {  // device allocations of one call, freed together
    std::vector<void*> ptrs;
    cudaError_t err = cudaSuccess;
    template <typename T>
    T* alloc(size_t n, const void* host = nullptr) {
        void* p = nullptr;
        if (err == cudaSuccess) err = cudaMalloc(&p, std::max<size_t>(n * sizeof(T), 16));
        if (err == cudaSuccess) ptrs.push_back(p);
        if (err == cudaSuccess) err = host ? cudaMemcpy(p, host, n * sizeof(T), cudaMemcpyHostToDevice) : cudaMemset(p, 0, std::max<size_t>(n * sizeof(T), 16));
        return static_cast<T*>(p);
    }
    template <typename T>
    void fetch(T* host, const T* dev, size_t n) {
        if (err == cudaSuccess) err = cudaDeviceSynchronize();
        if (err == cudaSuccess) err = cudaMemcpy(host, dev, n * sizeof(T), cudaMemcpyDeviceToHost);
    }
    void launched() {
        if (err == cudaSuccess) err = cudaGetLastError();
    }
    ~Dev() {
        for (void* p : ptrs) cudaFree(p);
    }
};

template <typename K>
cudaError_t allow_shared(K kernel) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSharedLimit);
}

}  // namespace

extern "C" int qtref_config_count(void) { return 6; }
extern "C" const char* qtref_config_tag(int cfg) { return cfg >= 0 && cfg < 6 ? kCfg[cfg].tag : nullptr; }
extern "C" int qtref_config_rows_per_block(int cfg) { return cfg >= 0 && cfg < 6 ? kCfg[cfg].r * kCfg[cfg].w : 0; }
// The configuration the reference's profile table picks on a device with many multiprocessors and a large L2 (profile "24sm_24mib" is the nearest to a
// B200 by the rule of profile.rs:150-165): role 0 output, 1 down, 2 qkv, 3 gate|up.
extern "C" int qtref_profile_config(int role) {
    static const int by_role[4] = {0, 1, 2, 0};
    return role >= 0 && role < 4 ? by_role[role] : -1;
}

// out[r] = sum_k trit[r, k] * act[k] through gemv_<tag>_plain. planar: rows * blocks_per_row(cols) * 32 bytes; rows a multiple of the configuration's rows per block.
extern "C" int qtref_gemv_plain(int cfg, const uint8_t* planar, int rows, int cols, const int8_t* act, int32_t* out) {
    if (cfg < 0 || cfg >= 6 || rows <= 0 || rows % (kCfg[cfg].r * kCfg[cfg].w) != 0) return cudaErrorInvalidValue;
    const Cfg& c = kCfg[cfg];
    int sum = 0;
    const std::vector<int8_t> perm = permute(act, cols, &sum);
    Dev d;
    const auto* w = d.alloc<uint8_t>(size_t(rows) * blocks_per_row(cols) * 32, planar);
    const auto* a = d.alloc<int8_t>(perm.size(), perm.data());
    const auto* s = d.alloc<int>(1, &sum);
    auto* o = d.alloc<int32_t>(rows);
    if (d.err == cudaSuccess) d.err = allow_shared(c.plain);
    if (d.err == cudaSuccess) {
        EpArgs ep;
        std::memset(&ep, 0, sizeof ep);
        c.plain<<<rows / (c.r * c.w), 32 * c.w, gemv_shared(c, cols)>>>(reinterpret_cast<const uint32_t*>(w), reinterpret_cast<const uint2*>(a), s, o, blocks_per_row(cols), ep);
        d.launched();
    }
    d.fetch(out, o, rows);
    return d.err;
}

// The same launch on buffers that are already on the device (for timing): d_act_perm holds act_entries(cols) * 8 bytes in the permuted layout.
extern "C" int qtref_gemv_plain_device(int cfg, const void* d_planar, int rows, int cols, const void* d_act_perm, const int* d_act_sum, int32_t* d_out, void* stream) {
    if (cfg < 0 || cfg >= 6 || rows <= 0 || rows % (kCfg[cfg].r * kCfg[cfg].w) != 0) return cudaErrorInvalidValue;
    const Cfg& c = kCfg[cfg];
    static bool allowed[6] = {false, false, false, false, false, false};
    if (!allowed[cfg]) {
        const cudaError_t e = allow_shared(c.plain);
        if (e != cudaSuccess) return e;
        allowed[cfg] = true;
    }
    EpArgs ep;
    std::memset(&ep, 0, sizeof ep);
    c.plain<<<rows / (c.r * c.w), 32 * c.w, gemv_shared(c, cols), static_cast<cudaStream_t>(stream)>>>(static_cast<const uint32_t*>(d_planar), static_cast<const uint2*>(d_act_perm),
                                                                                                      d_act_sum, d_out, blocks_per_row(cols), ep);
    return cudaGetLastError();
}
extern "C" int qtref_permute_activations(const int8_t* act, int cols, int8_t* out_perm, size_t out_capacity, int* out_sum) {
    const std::vector<int8_t> p = permute(act, cols, out_sum);
    if (out_capacity < p.size()) return cudaErrorInvalidValue;
    std::memcpy(out_perm, p.data(), p.size());
    return 0;
}
extern "C" size_t qtref_act_perm_bytes(int cols) { return size_t(act_entries(cols)) * 8; }

// Gated epilogue: `interleaved` holds gate row i and up row i as rows 2i and 2i + 1 (pairs of them: rows = 2 * n). v[i] = act(gate_i) * up_i with the post-scales
// ws / act_scale; *out_amax = max |v| as the kernel collects it. activation: 0 SiLU, 1 squared ReLU.
extern "C" int qtref_gemv_gated(int cfg, const uint8_t* interleaved, int rows, int cols, const int8_t* act, float act_scale, float ws_gate, float ws_up, int activation,
                                float* out_v, float* out_amax) {
    if (cfg < 0 || cfg >= 6 || rows <= 0 || rows % (kCfg[cfg].r * kCfg[cfg].w) != 0) return cudaErrorInvalidValue;
    const Cfg& c = kCfg[cfg];
    int sum = 0;
    const std::vector<int8_t> perm = permute(act, cols, &sum);
    Dev d;
    const auto* w = d.alloc<uint8_t>(size_t(rows) * blocks_per_row(cols) * 32, interleaved);
    const auto* a = d.alloc<int8_t>(perm.size(), perm.data());
    const auto* s = d.alloc<int>(1, &sum);
    const auto* sc = d.alloc<float>(1, &act_scale);
    auto* v = d.alloc<float>(rows / 2);
    auto* cells = d.alloc<int>(2);
    auto* sum_out = d.alloc<int>(1);
    if (d.err == cudaSuccess) d.err = allow_shared(c.gated);
    if (d.err == cudaSuccess) {
        EpArgs ep;
        std::memset(&ep, 0, sizeof ep);
        ep.act_scale = sc, ep.ws_gate = ws_gate, ep.ws_up = ws_up, ep.v = v, ep.cells = cells, ep.par = 0, ep.activation = activation, ep.sum_out = sum_out;
        c.gated<<<rows / (c.r * c.w), 32 * c.w, gemv_shared(c, cols)>>>(reinterpret_cast<const uint32_t*>(w), reinterpret_cast<const uint2*>(a), s, nullptr, blocks_per_row(cols), ep);
        d.launched();
    }
    d.fetch(out_v, v, rows / 2);
    int bits[2] = {0, 0};
    d.fetch(bits, cells, 2);
    std::memcpy(out_amax, &bits[0], 4);
    return d.err;
}

// rms_quant_p<6|8|14>: y = rmsnorm(x) * gamma (norm != 0) or y = x, quantised to int8 with s = 127 / max|y|. Outputs: the int8 values in column order (taken back out
// of the permuted layout), the scale, the activation sum.
extern "C" int qtref_rms_quant(const float* x, const float* gamma, int cols, float eps, int norm, int8_t* out_q, float* out_scale, int* out_sum) {
    Dev d;
    auto* dx = d.alloc<float>(cols, x);
    const auto* g = d.alloc<float>(cols, gamma);
    auto* perm = d.alloc<int8_t>(size_t(act_entries(cols)) * 8);
    auto* sum = d.alloc<int>(1);
    auto* scale = d.alloc<float>(1);
    if (size_t(cols) * 4 > size_t(kSharedLimit)) return cudaErrorInvalidValue;
    const int threads = norm ? 512 : 1024;
    auto kernel = cols <= 512 * 6 ? rms_quant_p6 : (cols <= 512 * 8 ? rms_quant_p8 : rms_quant_p14);
    if (norm && cols > 512 * 14) return cudaErrorInvalidValue;
    if (d.err == cudaSuccess) d.err = allow_shared(kernel);
    if (d.err == cudaSuccess) {
        kernel<<<1, threads, size_t(cols) * 4>>>(dx, g, reinterpret_cast<uint2*>(perm), sum, scale, cols, eps, norm, nullptr, 0.0f, nullptr, 0, 0, 0);
        d.launched();
    }
    std::vector<int8_t> host(size_t(act_entries(cols)) * 8);
    d.fetch(host.data(), perm, host.size());
    d.fetch(out_scale, scale, 1);
    d.fetch(out_sum, sum, 1);
    if (d.err == cudaSuccess)
        for (int c = 0; c < cols; ++c) out_q[c] = host[(size_t(c / 160) * 32 + c % 160 % 32) * 8 + c % 160 / 32];
    return d.err;
}

// final_norm followed by lm_head: logits of an F16 head [vocab][cols] for the hidden state h.
extern "C" int qtref_head(const float* h, const float* norm_w, const uint16_t* head_f16, int vocab, int cols, float eps, float* out_normed, float* out_logits) {
    Dev d;
    const auto* dh = d.alloc<float>(cols, h);
    const auto* w = d.alloc<float>(cols, norm_w);
    const auto* W = d.alloc<uint16_t>(size_t(vocab) * cols, head_f16);
    auto* x = d.alloc<float>(cols);
    auto* logits = d.alloc<float>(vocab);
    if (d.err == cudaSuccess) {
        final_norm<<<1, 1024>>>(dh, w, x, cols, eps);
        lm_head<<<(vocab + 7) / 8, 256>>>(reinterpret_cast<const __half*>(W), x, logits, vocab, cols);
        d.launched();
    }
    if (out_normed) d.fetch(out_normed, x, cols);
    d.fetch(out_logits, logits, vocab);
    return d.err;
}

// rope_kv on the int32 result of a stacked q | k | v projection: q_out receives the rotated query; k_row / v_row the F16 row written at position pos of every KV head
// ([kv_heads][head_dim] each).
extern "C" int qtref_rope_kv(const int32_t* qkv, float act_scale, float ws_q, float ws_k, float ws_v, const float* cos_sin, int pos, int q_heads, int kv_heads, int head_dim,
                             int rope_dims, int neox, float* out_q, uint16_t* out_k_row, uint16_t* out_v_row) {
    const int cache_len = pos + 1;
    Dev d;
    const auto* in = d.alloc<int32_t>(size_t(q_heads + 2 * kv_heads) * head_dim, qkv);
    const auto* sc = d.alloc<float>(1, &act_scale);
    const auto* cs = d.alloc<float>(size_t(cache_len) * rope_dims, cos_sin);
    const auto* dpos = d.alloc<int>(1, &pos);
    auto* q = d.alloc<float>(size_t(q_heads) * head_dim);
    auto* K = d.alloc<uint16_t>(size_t(kv_heads) * cache_len * head_dim);
    auto* V = d.alloc<uint16_t>(size_t(kv_heads) * cache_len * head_dim);
    if (d.err == cudaSuccess) {
        rope_kv<<<1, 256>>>(in, sc, ws_q, ws_k, ws_v, cs, dpos, q, reinterpret_cast<__half*>(K), reinterpret_cast<__half*>(V), q_heads, kv_heads, head_dim, rope_dims, neox, cache_len);
        d.launched();
    }
    d.fetch(out_q, q, size_t(q_heads) * head_dim);
    for (int h = 0; h < kv_heads; ++h) {
        d.fetch(out_k_row + size_t(h) * head_dim, K + (size_t(h) * cache_len + pos) * head_dim, head_dim);
        d.fetch(out_v_row + size_t(h) * head_dim, V + (size_t(h) * cache_len + pos) * head_dim, head_dim);
    }
    return d.err;
}

// attention_h<32|64|128|256> for the token at position pos (L = pos + 1 attended positions). K, V: [kv_heads][cache_len][head_dim] F16; q, out: [q_heads][head_dim].
extern "C" int qtref_attention(const uint16_t* K, const uint16_t* V, const float* q, int q_heads, int kv_heads, int head_dim, int cache_len, int pos, float scale, float* out) {
    if (kv_heads <= 0 || q_heads % kv_heads != 0 || pos < 0 || pos >= cache_len || cache_len > 7936) return cudaErrorInvalidValue;
    const int max_len = cache_len;
    const int padded = std::min(cache_len, std::max((max_len + 255) / 256 * 256, 256));
    const int chunk = std::max(std::min(max_len, 511), (padded + 3) / 4);
    const size_t shared = size_t((2 * chunk + 3) & ~3) * 4 + size_t(128) * head_dim;
    if (shared > size_t(kSharedLimit)) return cudaErrorInvalidValue;
    Dev d;
    const size_t cache = size_t(kv_heads) * cache_len * head_dim;
    const auto* dK = d.alloc<uint16_t>(cache, K);
    const auto* dV = d.alloc<uint16_t>(cache, V);
    const auto* dq = d.alloc<float>(size_t(q_heads) * head_dim, q);
    const auto* dpos = d.alloc<int>(1, &pos);
    auto* o = d.alloc<float>(size_t(q_heads) * head_dim);
    auto* part = d.alloc<float>(size_t(q_heads) * 4 * (head_dim + 2));
    auto* arrivals = d.alloc<unsigned>(q_heads);
    auto kernel = head_dim == 32 ? attention_h32 : head_dim == 64 ? attention_h64 : head_dim == 128 ? attention_h128 : head_dim == 256 ? attention_h256 : nullptr;
    if (kernel == nullptr) return cudaErrorInvalidValue;
    if (d.err == cudaSuccess) d.err = allow_shared(kernel);
    if (d.err == cudaSuccess) {
        kernel<<<dim3(q_heads, 4), 384, shared>>>(reinterpret_cast<const __half*>(dK), reinterpret_cast<const __half*>(dV), dq, o, part, arrivals, q_heads / kv_heads, cache_len, scale,
                                                  dpos, chunk);
        d.launched();
    }
    d.fetch(out, o, size_t(q_heads) * head_dim);
    return d.err;
}
