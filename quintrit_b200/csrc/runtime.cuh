// The symbols of the reference's C API (rust/crates/quintrit-c/include/quintrit.h, ABI version 1) served by this library, so
// that a program written against quintrit.h links against libquintrit_b200.so and runs its GPU path here.
//
//  * runtime level (quintrit.h:322-473, 515-530; quintrit-c/src/runtime.rs): models opened with quintrit_model_open_gpu,
//    sessions, tokenizer, text generation with stop sequences and a streaming callback, sampling; plus the token-id entry
//    points quintrit_session_feed_tokens / _logits / _generate_tokens declared in quintrit_b200.h;
//  * format level (quintrit.h:226-306; quintrit-c/src/gguf.rs): opening and listing GGUF files on the host; tensor conversion
//    for the device layout (kernel id QUINTRIT_KERNEL_B200) through the on-device transcoder;
//  * kernel level (quintrit.h:112-224; quintrit-c/src/tiles.rs): the device GEMV under the kernel id QUINTRIT_KERNEL_B200, to
//    which QUINTRIT_KERNEL_AUTO resolves; the CPU kernels (scalar, simd32, avx512) return QUINTRIT_ERR_UNSUPPORTED with a
//    message, as the reference's build without GPU support does for its GPU entry points (quintrit-c/src/cuda.rs:57-60):
//    this library has no CPU path. quintrit_model_open with the kernel AUTO (or B200) therefore loads the model onto GPU 0.
// Handle rules (quintrit-c/src/runtime.rs:162-220, 573-586; util.rs:163-183): a magic word at the start ("QTGG", "QTMD",
// "QTSS"), zeroed on free; NULL or a foreign pointer gives QUINTRIT_ERR_INVALID_HANDLE; a session keeps its model alive; a
// session in use by another thread gives QUINTRIT_ERR_BUSY.
//
// Included at the end of capi.cu (one translation unit: the helpers of the decoder are file-local there).
#pragma once
#include <cmath>
#include <memory>
#include <mutex>

#include "tokenizer.hpp"

#include "../../include/quintrit_b200_runtime.h"

struct RtModelInner {
    GgufModel data;
    qtb::BpeTokenizer tok;
    std::string tok_error;  // why the file's tokenizer cannot be used (empty: it can)
    std::string arch;       // "bitnet", "falcon3", "qwen3" or "llama" (quintrit-c/src/runtime.rs:222-231)
    uint32_t max_ctx = 0;
    uint32_t threads = 0;   // what quintrit_model_open / _set_threads were given: reported back, used for nothing
    int32_t kernel = QUINTRIT_KERNEL_AUTO;
    std::mutex lock;
    quintrit_b200_decoder* spare = nullptr;  // the decoder made at load time; the first session takes it
    ~RtModelInner() {
        if (spare) destroy_decoder(spare);
    }
};
struct quintrit_model {
    uint32_t magic;
    std::shared_ptr<RtModelInner> inner;
};
struct quintrit_session {
    uint32_t magic;
    std::shared_ptr<RtModelInner> model;
    quintrit_b200_decoder* dec = nullptr;
    std::mutex lock;
    uint32_t ctx = 0;
    std::vector<float> logits;  // of the last position fed, when they were fetched
    bool logits_valid = false;
    // The tokens whose keys and values sit at positions 0 .. cached.size() - 1, as far as the host knows them: a new prompt that begins
    // with the same tokens is ingested from the first difference on (quintrit-runtime/src/engine.rs:700-727). The record is trusted
    // only while its length equals the decoder's position; calls that run the loop on the device clear it.
    std::vector<uint32_t> cached;
    uint32_t last_reused = 0;   // prompt tokens the last text generation found cached
};
struct quintrit_gguf {
    uint32_t magic;
    GgufFile file;
    std::vector<std::string> names;  // NUL-terminated copies handed out by quintrit_gguf_tensor_at
};
struct quintrit_b200_tokenizer {
    uint32_t magic;
    qtb::BpeTokenizer tok;
};

namespace {

constexpr uint32_t kMagicTokenizer = 0x5154544Bu, kMagicGguf = 0x51544747u, kMagicModel = 0x51544d44u, kMagicSession = 0x51545353u;

template <typename H>
int rt_check(const H* h, uint32_t magic, const char* what) {
    if (h == nullptr || h->magic != magic) return fail(QUINTRIT_ERR_INVALID_HANDLE, "%s handle is NULL, freed or of the wrong type", what);
    return QUINTRIT_OK;
}
// A versioned struct is accepted if its leading struct_size is at least the size this library knows (util.rs:126-160).
template <typename S>
int rt_struct(const S* s, const char* what) {
    if (s == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "%s is NULL", what);
    if (reinterpret_cast<uintptr_t>(s) % alignof(S) != 0) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "%s is misaligned", what);
    if (s->struct_size < sizeof(S)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "%s.struct_size is %u, this library needs at least %zu", what, s->struct_size, sizeof(S));
    return QUINTRIT_OK;
}
int rt_text(const char* p, size_t len, const char* what, std::string* out) {
    if (p == nullptr && len != 0) return fail(QUINTRIT_ERR_NULL_POINTER, "%s is NULL", what);
    out->assign(p ? p : "", len);
    if (!qtb::utf8_valid(*out)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "%s is not valid UTF-8", what);
    return QUINTRIT_OK;
}
int rt_cstr(const char* p, const char* what, std::string* out) {
    if (p == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "%s is NULL", what);
    out->assign(p);
    if (!qtb::utf8_valid(*out)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "%s is not valid UTF-8", what);
    return QUINTRIT_OK;
}
// snprintf-style copy: truncated at a character boundary, NUL-terminated whenever capacity > 0 (runtime.rs:541-554).
void rt_write_text(char* buf, size_t cap, const std::string& s) {
    if (buf == nullptr || cap == 0) return;
    size_t n = std::min(s.size(), cap - 1);
    while (n > 0 && n < s.size() && (static_cast<unsigned char>(s[n]) & 0xC0) == 0x80) --n;
    std::memcpy(buf, s.data(), n);
    buf[n] = 0;
}
int rt_unsupported_cpu(const char* what) {
    return fail(QUINTRIT_ERR_UNSUPPORTED, "%s needs the CPU path, which this library does not have: it runs ternary models on NVIDIA B200 GPUs only (use the kernel id QUINTRIT_KERNEL_B200 / QUINTRIT_KERNEL_AUTO and quintrit_model_open_gpu)", what);
}
bool rt_device_kernel(int32_t kernel) { return kernel == QUINTRIT_KERNEL_AUTO || kernel == QUINTRIT_KERNEL_B200; }
int rt_kernel(int32_t kernel, const char* what) {
    if (rt_device_kernel(kernel)) return QUINTRIT_OK;
    if (kernel == QUINTRIT_KERNEL_SCALAR || kernel == QUINTRIT_KERNEL_SIMD32 || kernel == QUINTRIT_KERNEL_AVX512) return rt_unsupported_cpu(what);
    return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "unknown kernel id %d", kernel);
}

// The sampler of the reference runtime (quintrit-runtime/src/sampler.rs:38-143): greedy when temperature <= 0 or top_k == 1,
// else temperature, stable descending order, top-k, softmax (ops.rs:274-298: float exponentials summed in double), nucleus
// cut, renormalisation and one draw from its xorshift64 stream.
struct RtSampler {
    float temperature, top_p;
    size_t top_k;
    uint64_t state;
    RtSampler(float t, uint32_t k, float p, uint64_t seed) : temperature(t), top_p(p), top_k(k), state(seed == 0 ? 0x5EEDC0DE12345678ull : seed) {}
    bool greedy() const { return !(temperature > 0.0f) || top_k == 1; }
    float next_f32() {
        uint64_t x = state;
        x ^= x << 13;
        x ^= x >> 7;
        x ^= x << 17;
        state = x;
        return static_cast<float>(x) / 18446744073709551616.0f;  // u64::MAX as f32 is 2^64
    }
    static int32_t total_key(float v) {  // f32::total_cmp
        int32_t b;
        std::memcpy(&b, &v, 4);
        return b ^ static_cast<int32_t>(static_cast<uint32_t>(b >> 31) >> 1);
    }
    uint32_t sample(const std::vector<float>& logits) {
        const size_t n = logits.size();
        if (greedy()) {
            size_t best = 0;
            float bv = logits[0];
            for (size_t i = 1; i < n; ++i)
                if (logits[i] > bv) bv = logits[i], best = i;
            return static_cast<uint32_t>(best);
        }
        const float inv_temp = 1.0f / temperature;
        std::vector<std::pair<uint32_t, float>> cand(n);
        for (size_t i = 0; i < n; ++i) cand[i] = {static_cast<uint32_t>(i), logits[i] * inv_temp};
        const bool truncate_k = top_k > 0 && top_k < n;
        if (truncate_k || top_p < 1.0f)
            std::stable_sort(cand.begin(), cand.end(), [](const auto& a, const auto& b) { return total_key(b.second) < total_key(a.second); });
        if (truncate_k) cand.resize(top_k);
        std::vector<float> probs(cand.size());
        float mx = cand[0].second;
        for (const auto& c : cand)
            if (c.second > mx) mx = c.second;
        double sum = 0.0;
        for (size_t i = 0; i < cand.size(); ++i) {
            probs[i] = std::exp(cand[i].second - mx);  // the float libm exponential, as f32::exp
            sum += static_cast<double>(probs[i]);
        }
        if (sum > 0.0) {
            const float inv = static_cast<float>(1.0 / sum);
            for (float& p : probs) p *= inv;
        }
        size_t cutoff = probs.size();
        if (top_p < 1.0f) {
            float cum = 0.0f;
            for (size_t i = 0; i < probs.size(); ++i) {
                cum += probs[i];
                if (cum >= top_p) {
                    cutoff = i + 1;
                    break;
                }
            }
        }
        probs.resize(cutoff);
        float psum = 0.0f;
        for (float p : probs) psum += p;
        if (psum > 0.0f) {
            const float inv = 1.0f / psum;
            for (float& p : probs) p *= inv;
        }
        const float r = next_f32();
        float acc = 0.0f;
        for (size_t i = 0; i < probs.size(); ++i) {
            acc += probs[i];
            if (r <= acc || i + 1 == probs.size()) return cand[i].first;
        }
        return cand[0].first;
    }
};

// One position through the decoder of a session; the logits are fetched only when asked for.
// `on_device`: the device already holds this token and position (the token it chose itself at the position it advanced to).
// Sampling on the device (sample_topk_kernel): the parameters of one generation call, or nullptr for the greedy choice / host sampling.
struct RtDeviceSampling {
    float temperature, top_p;
    int top_k;
};
int rt_enqueue_sample(quintrit_b200_decoder* d, const RtDeviceSampling* sp) {
    if (sp == nullptr) return QUINTRIT_OK;
    sample_topk_kernel<<<1, kSampleThreads, 0, d->stream>>>(d->logits, d->vocab, sp->temperature, sp->top_k, sp->top_p, d->d_rng, d->d_token);
    QTB_LAUNCH_CHECK();
    return QUINTRIT_OK;
}

int rt_forward(quintrit_session* s, uint32_t token, uint32_t pos, bool want_logits, uint32_t* greedy, bool on_device = false, const RtDeviceSampling* sample = nullptr) {
    quintrit_b200_decoder* d = s->dec;
    int rc;
    if (!on_device && (rc = decoder_set(d, token, pos)) != QUINTRIT_OK) return rc;
    if ((rc = decoder_step(d)) != QUINTRIT_OK) return rc;
    if ((rc = rt_enqueue_sample(d, sample)) != QUINTRIT_OK) return rc;  // replaces the greedy choice in d_token by the sampled one
    if (want_logits) QTB_CUDA(cudaMemcpyAsync(s->logits.data(), d->logits, size_t(d->vocab) * sizeof(float), cudaMemcpyDeviceToHost, d->stream));
    if (greedy) QTB_CUDA(cudaMemcpyAsync(greedy, d->d_token, sizeof(uint32_t), cudaMemcpyDeviceToHost, d->stream));
    if ((rc = decoder_check_status(d)) != QUINTRIT_OK) return rc;
    if (s->cached.size() >= pos) {
        s->cached.resize(pos);
        s->cached.push_back(token);
    } else {
        s->cached.clear();
    }
    d->host_pos = pos + 1;
    s->logits_valid = want_logits;
    return QUINTRIT_OK;
}

// Feeds tokens from position pos0 without waiting between them; only the last position's logits / greedy token are read back.
int rt_feed(quintrit_session* s, const uint32_t* ids, size_t n, uint32_t pos0, bool want_logits, uint32_t* greedy, const RtDeviceSampling* sample = nullptr) {
    quintrit_b200_decoder* d = s->dec;
    DeviceGuard g(d->device);
    if (n >= 8 && prefill_available(d) && std::getenv("QUINTRIT_B200_NO_PREFILL") == nullptr) {
        // a prompt goes in chunks of up to 256 tokens with the projections on the tensor cores; the result is that of n single steps
        int rc = decoder_prefill(d, ids, n, pos0);
        if (rc != QUINTRIT_OK) return rc;
        if ((rc = rt_enqueue_sample(d, sample)) != QUINTRIT_OK) return rc;
        if (want_logits) QTB_CUDA(cudaMemcpyAsync(s->logits.data(), d->logits, size_t(d->vocab) * sizeof(float), cudaMemcpyDeviceToHost, d->stream));
        if (greedy) QTB_CUDA(cudaMemcpyAsync(greedy, d->d_token, sizeof(uint32_t), cudaMemcpyDeviceToHost, d->stream));
        if ((rc = decoder_check_status(d)) != QUINTRIT_OK) return rc;
        if (s->cached.size() >= pos0) {
            s->cached.resize(pos0);
            s->cached.insert(s->cached.end(), ids, ids + n);
        } else {
            s->cached.clear();
        }
        d->host_pos = pos0 + static_cast<uint32_t>(n);
        s->logits_valid = want_logits;
        return QUINTRIT_OK;
    }
    for (size_t i = 0; i + 1 < n; ++i) {
        int rc;
        if ((rc = decoder_set(d, ids[i], pos0 + static_cast<uint32_t>(i))) != QUINTRIT_OK || (rc = decoder_step(d)) != QUINTRIT_OK) return rc;
    }
    if (s->cached.size() >= pos0) {
        s->cached.resize(pos0);
        s->cached.insert(s->cached.end(), ids, ids + n - 1);
    } else {
        s->cached.clear();
    }
    return rt_forward(s, ids[n - 1], pos0 + static_cast<uint32_t>(n - 1), want_logits, greedy, false, sample);
}

// engine.rs:869-879: the first index of `pending` from which the rest could still be the beginning of a stop sequence.
size_t rt_safe_flush(const std::string& pending, const std::vector<std::string>& stops) {
    for (size_t idx = 0; idx < pending.size(); ++idx) {
        if ((static_cast<unsigned char>(pending[idx]) & 0xC0) == 0x80) continue;  // character boundaries only
        const size_t len = pending.size() - idx;
        for (const std::string& stop : stops)
            if (stop.size() >= len && stop.compare(0, len, pending, idx, len) == 0) return idx;
    }
    return pending.size();
}

// engine.rs:34-121
std::string rt_format_chat(const std::vector<std::pair<std::string, std::string>>& msgs, const std::string& arch) {
    auto role_of = [](std::string r) {
        size_t a = 0, b = r.size();
        while (a < b && (r[a] == ' ' || r[a] == '\t' || r[a] == '\n' || r[a] == '\r')) ++a;
        while (b > a && (r[b - 1] == ' ' || r[b - 1] == '\t' || r[b - 1] == '\n' || r[b - 1] == '\r')) --b;
        r = r.substr(a, b - a);
        for (char& c : r)
            if (c >= 'A' && c <= 'Z') c = static_cast<char>(c + 32);
        return r;
    };
    std::string p;
    if (arch == "falcon3") {
        for (size_t i = 0; i < msgs.size(); ++i) {
            const std::string role = role_of(msgs[i].first);
            if (role == "system") {
                p += "<|system|>\n" + msgs[i].second + "\n";
            } else if (role == "assistant") {
                p += "<|assistant|>\n" + msgs[i].second + "<|endoftext|>";
                if (i + 1 != msgs.size()) p += "\n";
            } else {
                p += "<|user|>\n" + msgs[i].second + "\n";
            }
        }
        return p + "<|assistant|>\n";
    }
    if (arch == "qwen3") {  // ChatML with an empty thinking block (engine.rs:70-87)
        for (const auto& m : msgs) {
            const std::string role = role_of(m.first);
            p += "<|im_start|>" + std::string(role == "system" || role == "assistant" ? role : "user") + "\n" + m.second + "<|im_end|>\n";
        }
        return p + "<|im_start|>assistant\n<think>\n\n</think>\n\n";
    }
    for (const auto& m : msgs) {
        const std::string role = role_of(m.first);
        p += role == "system" ? "### System:\n" : (role == "assistant" ? "### Assistant:\n" : "### User:\n");
        p += m.second + "\n\n";
    }
    return p + "### Assistant:\n";
}

// The tokenizer of a GGUF file with BOS / EOS as ModelConfig::from_gguf resolves them (config.rs:376-415). Returns why it
// cannot be used, or an empty string.
std::string rt_build_tokenizer(const GgufFile& g, qtb::BpeTokenizer* tok) {
    const std::string tok_model = meta_str(g, "tokenizer.ggml.model", "");
    const GgufValue* pre_v = g.find("tokenizer.ggml.pre");
    const std::string pre = pre_v != nullptr && pre_v->type == 8 ? pre_v->s : std::string();
    bool add_bos;
    if (const GgufValue* v = g.find("tokenizer.ggml.add_bos_token"); v != nullptr && v->type == 7) {
        add_bos = v->u != 0;
    } else {
        static const char* const with_bos[] = {"llama3", "llama-v3", "llama-bpe", "falcon3", "falcon-h1", "pixtral", "midm-2.0", "lfm2", "tekken", "jina-v5-nano"};
        add_bos = false;
        for (const char* n : with_bos) add_bos |= pre == n;
    }
    int64_t bos = -1, eos = -1;
    if (add_bos) {
        if (const GgufValue* v = g.find("tokenizer.ggml.bos_token_id"); v != nullptr && v->is_int() && v->type != 9) bos = static_cast<int64_t>(v->u);
        else if (tok_model == "gpt2") bos = 11;
    }
    if (const GgufValue* v = g.find("tokenizer.ggml.eos_token_id"); v != nullptr && v->is_int() && v->type != 9) eos = static_cast<int64_t>(v->u);
    const GgufValue* toks = g.find("tokenizer.ggml.tokens");
    if (toks == nullptr || toks->type != 9 || toks->elem_type != 8 || toks->strs.empty()) {
        tok->build({}, {}, {}, nullptr, bos, eos);
        return "the model file carries no tokenizer (tokenizer.ggml.tokens): use the token-id entry points";
    }
    const GgufValue* merges = g.find("tokenizer.ggml.merges");
    const GgufValue* types = g.find("tokenizer.ggml.token_type");
    return tok->build(toks->strs, merges != nullptr ? merges->strs : std::vector<std::string>(), types != nullptr ? types->ints : std::vector<int64_t>(),
                      pre_v != nullptr && pre_v->type == 8 ? pre.c_str() : nullptr, bos, eos);
}

int rt_open_gpu(const char* path, const quintrit_gpu_options_t* options, quintrit_model** out) {
    uint32_t device = 0, want_ctx = 0;
    if (options != nullptr) {
        int rc = rt_struct(options, "options");
        if (rc != QUINTRIT_OK) return rc;
        if (options->flags & ~uint32_t(QUINTRIT_MODEL_OPEN_VERBOSE)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "options.flags has unknown bits set: 0x%x", options->flags);
        device = options->device_index, want_ctx = options->context_length;  // the library never prints: VERBOSE changes nothing
    }
    auto inner = std::make_shared<RtModelInner>();
    int rc = load_gguf_model(path, device, &inner->data);
    if (rc != QUINTRIT_OK) return rc;
    const GgufFile& g = inner->data.file;
    const GgufModelShape& m = inner->data.shape;
    inner->max_ctx = inner->data.context_for(want_ctx);
    if (inner->max_ctx == 0) return fail(QUINTRIT_ERR_MODEL, "the context window of the model is empty");
    {
        std::string name = meta_str(g, "general.name", ""), base = meta_str(g, "general.basename", "");
        for (char& c : name) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
        for (char& c : base) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
        inner->arch = m.arch_id == QUINTRIT_B200_ARCH_BITNET ? "bitnet"
                      : m.arch == "qwen3" ? "qwen3"
                      : (m.arch == "falcon3" || name.find("falcon") != std::string::npos || base.find("falcon") != std::string::npos) ? "falcon3" : "llama";
    }
    inner->tok_error = rt_build_tokenizer(g, &inner->tok);
    // the weights are on the device; one decoder is made now so that device errors surface here, as in GpuModel::load
    if ((rc = decoder_from_model(inner->data, inner->max_ctx, &inner->spare)) != QUINTRIT_OK) return rc;
    inner->max_ctx = static_cast<uint32_t>(inner->spare->ctx);
    quintrit_model* h = new quintrit_model();
    h->magic = kMagicModel;
    h->inner = std::move(inner);
    *out = h;
    return QUINTRIT_OK;
}

int rt_need_tokenizer(const RtModelInner& m) {
    if (!m.tok_error.empty()) return fail(QUINTRIT_ERR_UNSUPPORTED, "%s", m.tok_error.c_str());
    return QUINTRIT_OK;
}

struct RtSessionLock {  // try_lock: a session in use by another thread is QUINTRIT_ERR_BUSY (runtime.rs:214-220)
    std::unique_lock<std::mutex> hold;
    explicit RtSessionLock(quintrit_session* s) : hold(s->lock, std::try_to_lock) {}
    int check() const { return hold.owns_lock() ? QUINTRIT_OK : fail(QUINTRIT_ERR_BUSY, "the session is in use by another thread"); }
};

const char* rt_type_name(uint32_t t) {
    switch (t) {
        case kGgmlF32: return "F32";
        case kGgmlF16: return "F16";
        case kGgmlQ8_0: return "Q8_0";
        case kGgmlBF16: return "BF16";
        case kGgmlTq1: return "TQ1_0";
        case kGgmlTq2: return "TQ2_0";
        case kGgmlI2S: return "I2_S";
        case kGgmlVelurex: return "VELUREX";
        case kGgmlQ2: return "Q2_0";
        default: return "UNKNOWN";
    }
}
void rt_fill_tensor(const quintrit_gguf* h, size_t index, quintrit_tensor_info_t* out) {
    const GgufTensor& t = h->file.tensors.at(h->file.order[index]);
    out->struct_size = sizeof *out;
    out->ggml_type = static_cast<int32_t>(t.type);
    out->n_dims = static_cast<uint32_t>(t.shape.size());
    out->is_ternary = t.type == kGgmlI2S || t.type == kGgmlTq1 || t.type == kGgmlTq2 ? 1 : 0;
    for (size_t d = 0; d < QUINTRIT_MAX_DIMS; ++d) out->shape[d] = d < t.shape.size() ? t.shape[d] : 0;
    out->num_elements = t.elements();
    out->offset = t.offset;
    out->data_bytes = h->file.data(t) != nullptr ? t.byte_len() : 0;
    out->name = h->names[index].c_str();
    out->type_name = rt_type_name(t.type);
}
void rt_layout(size_t rows, size_t cols, quintrit_tiled_layout_t* out) {
    out->struct_size = sizeof *out;
    out->kernel = QUINTRIT_KERNEL_B200;
    out->tile_rows = 1;  // planar rows: no row padding
    out->rows = rows, out->cols = cols, out->padded_rows = rows;
    out->bytes_per_row = quintrit_b200_planar_row_bytes(cols);
    out->total_bytes = rows * out->bytes_per_row;
}
// The five trits of a velurex byte (quintrit-core/src/pack.rs:41-58); bytes the packer never writes are an error here.
bool rt_byte_trits(uint8_t b, int8_t out[5]) {
    const int u = b / 28, l = b % 28;
    if (b > 250 || l > 26) return false;
    out[0] = static_cast<int8_t>(l % 3 - 1), out[1] = static_cast<int8_t>(l / 3 % 3 - 1), out[2] = static_cast<int8_t>(l / 9 - 1);
    out[3] = static_cast<int8_t>(u % 3 - 1), out[4] = static_cast<int8_t>(u / 3 - 1);
    return true;
}
int rt_shape(size_t rows, size_t cols) {
    if (rows == 0 || cols == 0 || rows > (size_t(1) << 31) || cols > (size_t(1) << 31)) return fail(QUINTRIT_ERR_INVALID_SHAPE, "rows and cols must be in [1, 2^31]");
    return QUINTRIT_OK;
}
// A ternary tensor of a GGUF file as a device matrix (transcoded there), with its scale.
int rt_tensor_matrix(const quintrit_gguf* h, const char* name, quintrit_b200_matrix_t** out, float* scale, size_t* rows, size_t* cols) {
    std::string nm;
    int rc = rt_cstr(name, "name", &nm);
    if (rc != QUINTRIT_OK) return rc;
    const GgufTensor* t = h->file.tensor(nm);
    if (t == nullptr) return fail(QUINTRIT_ERR_NOT_FOUND, "no tensor named '%s'", nm.c_str());
    if (t->type != kGgmlI2S && t->type != kGgmlTq1 && t->type != kGgmlTq2) return fail(QUINTRIT_ERR_FORMAT, "tensor '%s' is not an I2_S, TQ1_0 or TQ2_0 tensor", nm.c_str());
    if (t->shape.size() != 2) return fail(QUINTRIT_ERR_FORMAT, "tensor '%s' is not a matrix", nm.c_str());
    *cols = static_cast<size_t>(t->shape[0]), *rows = static_cast<size_t>(t->shape[1]);
    const uint8_t* data = nullptr;
    uint64_t len = 0;
    int32_t source = 0;
    float s = 0.0f;
    if ((rc = projection(h->file, nm, *rows, *cols, &data, &len, &source, &s)) != QUINTRIT_OK) return rc;
    if (scale) *scale = s;
    if (out == nullptr) return QUINTRIT_OK;
    return quintrit_b200_matrix_upload(0, source, data, len, *rows, *cols, out);
}

}  // namespace

// ---- version ------------------------------------------------------------------------------------------------------------------
extern "C" const char* quintrit_version(void) { return "0.2.0"; }  // the API level of quintrit.h:49-52 this library serves
extern "C" uint32_t quintrit_abi_version(void) { return 1; }      // quintrit.h:55

// ---- CPU and kernel queries -----------------------------------------------------------------------------------------------------
extern "C" int quintrit_cpu_features(uint64_t* out_mask) {
    return guard([&]() -> int {
        if (out_mask == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_mask is NULL");
        uint64_t m = 0;
#if defined(__x86_64__)
        if (__builtin_cpu_supports("avx2")) m |= 1u << 0;
        if (__builtin_cpu_supports("avx512f")) m |= 1u << 1;
        if (__builtin_cpu_supports("avx512bw")) m |= 1u << 2;
        if (__builtin_cpu_supports("avx512vbmi")) m |= 1u << 3;
        if (__builtin_cpu_supports("avx512vnni")) m |= 1u << 4;
#endif
        *out_mask = m;
        return ok();
    });
}
extern "C" int quintrit_kernel_supported(int32_t kernel, int32_t* out_supported) {
    return guard([&]() -> int {
        if (out_supported == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_supported is NULL");
        if (kernel < 0 || (kernel > QUINTRIT_KERNEL_AVX512 && kernel != QUINTRIT_KERNEL_B200)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "unknown kernel id %d", kernel);
        int supported = 0;
        if (rt_device_kernel(kernel)) {
            int n = 0;
            if (cudaGetDeviceCount(&n) != cudaSuccess) n = 0, (void)cudaGetLastError();
            for (int i = 0; i < n && !supported; ++i) {
                cudaDeviceProp p;
                if (cudaGetDeviceProperties(&p, i) == cudaSuccess && p.major == 10) supported = 1;
            }
        }
        *out_supported = supported;
        return ok();
    });
}
extern "C" int quintrit_kernel_resolve(int32_t kernel, int32_t* out_kernel) {
    return guard([&]() -> int {
        if (out_kernel == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_kernel is NULL");
        if (kernel < 0 || (kernel > QUINTRIT_KERNEL_AVX512 && kernel != QUINTRIT_KERNEL_B200)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "unknown kernel id %d", kernel);
        *out_kernel = kernel == QUINTRIT_KERNEL_AUTO ? QUINTRIT_KERNEL_B200 : kernel;
        return ok();
    });
}
extern "C" const char* quintrit_kernel_name(int32_t kernel) {
    switch (kernel) {
        case QUINTRIT_KERNEL_AUTO: return "auto";
        case QUINTRIT_KERNEL_SCALAR: return "scalar";
        case QUINTRIT_KERNEL_SIMD32: return "simd32";
        case QUINTRIT_KERNEL_AVX512: return "avx512";
        case QUINTRIT_KERNEL_B200: return "b200";
        default: return nullptr;
    }
}
extern "C" int quintrit_kernel_tile_rows(int32_t kernel, size_t* out_tile_rows) {
    return guard([&]() -> int {
        if (out_tile_rows == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_tile_rows is NULL");
        int rc = rt_kernel(kernel, "the tile layout of a CPU kernel");
        if (rc != QUINTRIT_OK) return rc;
        *out_tile_rows = 1;
        return ok();
    });
}
extern "C" int quintrit_supported_kernels(int32_t* out, size_t capacity, size_t* out_count) {
    return guard([&]() -> int {
        if (out_count == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_count is NULL");
        *out_count = 1;
        if (out == nullptr || capacity < 1) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "1 kernel does not fit into a buffer of %zu", capacity);
        out[0] = QUINTRIT_KERNEL_B200;
        return ok();
    });
}
extern "C" int quintrit_default_threads(uint32_t* out_threads) {
    return guard([&]() -> int {
        if (out_threads == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_threads is NULL");
        *out_threads = 1;  // the host side of a call is one thread; the work runs on the GPU
        return ok();
    });
}

// ---- kernel level -------------------------------------------------------------------------------------------------------------
extern "C" int quintrit_tiled_layout(int32_t kernel, size_t rows, size_t cols, quintrit_tiled_layout_t* out_layout) {
    return guard([&]() -> int {
        int rc = rt_struct(out_layout, "out_layout");
        if (rc != QUINTRIT_OK || (rc = rt_kernel(kernel, "the tiled layout of a CPU kernel")) != QUINTRIT_OK || (rc = rt_shape(rows, cols)) != QUINTRIT_OK) return rc;
        rt_layout(rows, cols, out_layout);
        return ok();
    });
}
extern "C" int quintrit_tiled_size(int32_t kernel, size_t rows, size_t cols, size_t* out_bytes) {
    return guard([&]() -> int {
        if (out_bytes == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_bytes is NULL");
        int rc = rt_kernel(kernel, "the tiled layout of a CPU kernel");
        if (rc != QUINTRIT_OK || (rc = rt_shape(rows, cols)) != QUINTRIT_OK) return rc;
        *out_bytes = rows * quintrit_b200_planar_row_bytes(cols);
        return ok();
    });
}
extern "C" int quintrit_pack_matrix(int32_t kernel, const int8_t* trits, size_t trits_len, size_t rows, size_t cols, uint8_t* out, size_t out_capacity) {
    return guard([&]() -> int {
        int rc = rt_kernel(kernel, "packing for a CPU kernel");
        if (rc != QUINTRIT_OK || (rc = rt_shape(rows, cols)) != QUINTRIT_OK) return rc;
        return quintrit_b200_pack_planar(trits, trits_len, rows, cols, out, out_capacity);
    });
}
extern "C" int quintrit_unpack_matrix(int32_t kernel, const uint8_t* tiled, size_t tiled_len, size_t rows, size_t cols, int8_t* out, size_t out_capacity) {
    return guard([&]() -> int {
        int rc = rt_kernel(kernel, "unpacking the layout of a CPU kernel");
        if (rc != QUINTRIT_OK || (rc = rt_shape(rows, cols)) != QUINTRIT_OK) return rc;
        if (tiled == nullptr || out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "a buffer is NULL");
        const size_t rb = quintrit_b200_planar_row_bytes(cols);
        if (tiled_len < rows * rb) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "the packed buffer holds %zu bytes, %zu are needed", tiled_len, rows * rb);
        if (out_capacity < rows * cols) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out holds %zu trits, %zu are needed", out_capacity, rows * cols);
        for (size_t r = 0; r < rows; ++r)
            for (size_t b = 0; b < rb; ++b) {
                int8_t t[5];
                if (!rt_byte_trits(tiled[r * rb + b], t)) return fail(QUINTRIT_ERR_INVALID_VALUE, "byte %zu of row %zu is %u, not a velurex code", b, r, tiled[r * rb + b]);
                const size_t block = b / kBlockBytes, j = b % kBlockBytes;
                for (size_t p = 0; p < 5; ++p) {
                    const size_t c = block * kBlockTrits + p * kBlockBytes + j;
                    if (c < cols) out[r * cols + c] = t[p];
                }
            }
        return ok();
    });
}
namespace {
int rt_gemv(int32_t kernel, const uint8_t* weights, size_t weights_len, size_t rows, size_t cols, const int8_t* acts, size_t acts_len, void* out, size_t out_cap,
            uint32_t threads, bool as_float, float scale) {
    int rc = rt_kernel(kernel, "the GEMV of a CPU kernel");
    if (rc != QUINTRIT_OK || (rc = rt_shape(rows, cols)) != QUINTRIT_OK) return rc;
    if (threads > 256) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "num_threads %u exceeds 256", threads);
    if (weights == nullptr || acts == nullptr || out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "a buffer is NULL");
    if (cols > 131072) return fail(QUINTRIT_ERR_INVALID_SHAPE, "cols %zu exceeds 131072", cols);
    const size_t need = rows * quintrit_b200_planar_row_bytes(cols);
    if (weights_len < need) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "weights hold %zu bytes, %zu are needed", weights_len, need);
    // the weights live in host memory at this level: every call places them on the device, multiplies and frees them
    quintrit_b200_matrix_t* m = nullptr;
    if ((rc = quintrit_b200_matrix_upload(0, QUINTRIT_B200_SRC_PLANAR, weights, need, rows, cols, &m)) != QUINTRIT_OK) return rc;
    rc = as_float ? quintrit_b200_gemv_f32(m, acts, acts_len, scale, static_cast<float*>(out), out_cap) : quintrit_b200_gemv_i32(m, acts, acts_len, static_cast<int32_t*>(out), out_cap);
    const LastError keep = last_error();
    quintrit_b200_matrix_free(m);
    if (rc != QUINTRIT_OK) last_error() = keep;
    return rc;
}
}  // namespace
extern "C" int quintrit_gemv_i32(int32_t kernel, const uint8_t* weights, size_t weights_len, size_t rows, size_t cols, const int8_t* activations, size_t activations_len,
                                 int32_t* out, size_t out_capacity, uint32_t num_threads) {
    return guard([&]() -> int { return rt_gemv(kernel, weights, weights_len, rows, cols, activations, activations_len, out, out_capacity, num_threads, false, 1.0f); });
}
extern "C" int quintrit_gemv_f32(int32_t kernel, const uint8_t* weights, size_t weights_len, size_t rows, size_t cols, const int8_t* activations, size_t activations_len,
                                 float scale, float* out, size_t out_capacity, uint32_t num_threads) {
    return guard([&]() -> int { return rt_gemv(kernel, weights, weights_len, rows, cols, activations, activations_len, out, out_capacity, num_threads, true, scale); });
}

// ---- format level -------------------------------------------------------------------------------------------------------------
extern "C" int quintrit_gguf_open(const char* path, quintrit_gguf_t** out_gguf) {
    return guard([&]() -> int {
        if (out_gguf == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_gguf is NULL");
        *out_gguf = nullptr;
        std::string p;
        int rc = rt_cstr(path, "path", &p);
        if (rc != QUINTRIT_OK) return rc;
        std::unique_ptr<quintrit_gguf> h(new quintrit_gguf());
        std::string why;
        const int st = h->file.open(p.c_str(), why);
        if (st == 1) return fail(QUINTRIT_ERR_IO, "%s", why.c_str());
        if (st != 0) return fail(QUINTRIT_ERR_FORMAT, "%s", why.c_str());
        h->names = h->file.order;
        h->magic = kMagicGguf;
        *out_gguf = h.release();
        return ok();
    });
}
extern "C" int quintrit_gguf_close(quintrit_gguf_t* gguf) {
    return guard([&]() -> int {
        if (gguf == nullptr) return ok();
        int rc = rt_check(gguf, kMagicGguf, "gguf");
        if (rc != QUINTRIT_OK) return rc;
        gguf->magic = 0;
        delete gguf;
        return ok();
    });
}
extern "C" int quintrit_gguf_info(const quintrit_gguf_t* gguf, quintrit_gguf_info_t* out_info) {
    return guard([&]() -> int {
        int rc = rt_check(gguf, kMagicGguf, "gguf");
        if (rc != QUINTRIT_OK || (rc = rt_struct(out_info, "out_info")) != QUINTRIT_OK) return rc;
        out_info->struct_size = sizeof *out_info;
        out_info->version = gguf->file.version;
        out_info->tensor_count = gguf->file.order.size();
        out_info->metadata_count = gguf->file.metadata.size();
        out_info->data_offset = gguf->file.data_start();
        return ok();
    });
}
extern "C" int quintrit_gguf_tensor_at(const quintrit_gguf_t* gguf, size_t index, quintrit_tensor_info_t* out_info) {
    return guard([&]() -> int {
        int rc = rt_check(gguf, kMagicGguf, "gguf");
        if (rc != QUINTRIT_OK || (rc = rt_struct(out_info, "out_info")) != QUINTRIT_OK) return rc;
        if (index >= gguf->file.order.size()) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "tensor index %zu is not below the tensor count %zu", index, gguf->file.order.size());
        rt_fill_tensor(gguf, index, out_info);
        return ok();
    });
}
extern "C" int quintrit_gguf_tensor_find(const quintrit_gguf_t* gguf, const char* name, quintrit_tensor_info_t* out_info) {
    return guard([&]() -> int {
        int rc = rt_check(gguf, kMagicGguf, "gguf");
        if (rc != QUINTRIT_OK || (rc = rt_struct(out_info, "out_info")) != QUINTRIT_OK) return rc;
        std::string nm;
        if ((rc = rt_cstr(name, "name", &nm)) != QUINTRIT_OK) return rc;
        for (size_t i = 0; i < gguf->file.order.size(); ++i)
            if (gguf->file.order[i] == nm) {
                rt_fill_tensor(gguf, i, out_info);
                return ok();
            }
        return fail(QUINTRIT_ERR_NOT_FOUND, "no tensor named '%s'", nm.c_str());
    });
}
extern "C" int quintrit_gguf_metadata_string(const quintrit_gguf_t* gguf, const char* key, char* buffer, size_t capacity, size_t* out_len) {
    return guard([&]() -> int {
        int rc = rt_check(gguf, kMagicGguf, "gguf");
        if (rc != QUINTRIT_OK) return rc;
        if (out_len == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_len is NULL");
        std::string k;
        if ((rc = rt_cstr(key, "key", &k)) != QUINTRIT_OK) return rc;
        const GgufValue* v = gguf->file.find(k);
        if (v == nullptr) return fail(QUINTRIT_ERR_NOT_FOUND, "no metadata key '%s'", k.c_str());
        if (v->type != 8) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "metadata '%s' is not a string", k.c_str());
        *out_len = v->s.size();
        if (buffer == nullptr || capacity <= v->s.size()) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "the value needs %zu bytes including the NUL, buffer holds %zu", v->s.size() + 1, capacity);
        std::memcpy(buffer, v->s.c_str(), v->s.size() + 1);
        return ok();
    });
}
extern "C" int quintrit_gguf_metadata_u64(const quintrit_gguf_t* gguf, const char* key, uint64_t* out_value) {
    return guard([&]() -> int {
        int rc = rt_check(gguf, kMagicGguf, "gguf");
        if (rc != QUINTRIT_OK) return rc;
        if (out_value == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_value is NULL");
        std::string k;
        if ((rc = rt_cstr(key, "key", &k)) != QUINTRIT_OK) return rc;
        const GgufValue* v = gguf->file.find(k);
        if (v == nullptr) return fail(QUINTRIT_ERR_NOT_FOUND, "no metadata key '%s'", k.c_str());
        if (v->type == 9 || !v->is_int() || static_cast<int64_t>(v->u) < 0) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "metadata '%s' is not a non-negative integer", k.c_str());
        *out_value = v->u;
        return ok();
    });
}
extern "C" int quintrit_gguf_tensor_data(const quintrit_gguf_t* gguf, const char* name, const uint8_t** out_data, size_t* out_len) {
    return guard([&]() -> int {
        int rc = rt_check(gguf, kMagicGguf, "gguf");
        if (rc != QUINTRIT_OK) return rc;
        if (out_data == nullptr || out_len == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "an out pointer is NULL");
        std::string nm;
        if ((rc = rt_cstr(name, "name", &nm)) != QUINTRIT_OK) return rc;
        const GgufTensor* t = gguf->file.tensor(nm);
        if (t == nullptr) return fail(QUINTRIT_ERR_NOT_FOUND, "no tensor named '%s'", nm.c_str());
        uint64_t len = 0;
        const uint8_t* p = gguf->file.data(*t, &len);
        if (p == nullptr) return fail(QUINTRIT_ERR_FORMAT, "the payload of '%s' cannot be read (unknown type or outside the file)", nm.c_str());
        *out_data = p, *out_len = static_cast<size_t>(len);
        return ok();
    });
}
extern "C" int quintrit_gguf_tensor_layout(const quintrit_gguf_t* gguf, const char* name, int32_t kernel, quintrit_tiled_layout_t* out_layout, float* out_scale) {
    return guard([&]() -> int {
        int rc = rt_check(gguf, kMagicGguf, "gguf");
        if (rc != QUINTRIT_OK || (rc = rt_kernel(kernel, "the tiled layout of a CPU kernel")) != QUINTRIT_OK) return rc;
        if (out_layout != nullptr && (rc = rt_struct(out_layout, "out_layout")) != QUINTRIT_OK) return rc;
        size_t rows = 0, cols = 0;
        if ((rc = rt_tensor_matrix(gguf, name, nullptr, out_scale, &rows, &cols)) != QUINTRIT_OK) return rc;
        if (out_layout) rt_layout(rows, cols, out_layout);
        return ok();
    });
}
extern "C" int quintrit_gguf_convert_tensor(const quintrit_gguf_t* gguf, const char* name, int32_t kernel, uint8_t* out, size_t out_capacity,
                                            quintrit_tiled_layout_t* out_layout, float* out_scale) {
    return guard([&]() -> int {
        int rc = rt_check(gguf, kMagicGguf, "gguf");
        if (rc != QUINTRIT_OK || (rc = rt_kernel(kernel, "conversion for a CPU kernel")) != QUINTRIT_OK) return rc;
        if (out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out is NULL");
        if (out_layout != nullptr && (rc = rt_struct(out_layout, "out_layout")) != QUINTRIT_OK) return rc;
        size_t rows = 0, cols = 0;
        quintrit_b200_matrix_t* m = nullptr;  // transcoded on the device, read back as planar bytes
        if ((rc = rt_tensor_matrix(gguf, name, &m, out_scale, &rows, &cols)) != QUINTRIT_OK) return rc;
        rc = quintrit_b200_matrix_download_planar(m, out, out_capacity);
        const LastError keep = last_error();
        quintrit_b200_matrix_free(m);
        if (rc != QUINTRIT_OK) {
            last_error() = keep;
            return rc;
        }
        if (out_layout) rt_layout(rows, cols, out_layout);
        return ok();
    });
}

// ---- runtime level: models ------------------------------------------------------------------------------------------------------
extern "C" int quintrit_model_open(const char* path, const quintrit_model_options_t* options, quintrit_model_t** out_model) {
    return guard([&]() -> int {
        if (out_model == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_model is NULL");
        *out_model = nullptr;
        std::string p;
        int rc = rt_cstr(path, "path", &p);
        if (rc != QUINTRIT_OK) return rc;
        uint32_t threads = 1;
        if (options != nullptr) {
            if ((rc = rt_struct(options, "options")) != QUINTRIT_OK || (rc = rt_kernel(options->kernel, "quintrit_model_open with a CPU kernel")) != QUINTRIT_OK) return rc;
            if (options->flags & ~uint32_t(QUINTRIT_MODEL_OPEN_VERBOSE)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "options.flags has unknown bits set: 0x%x", options->flags);
            if (options->num_threads > 256) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "num_threads %u exceeds 256", options->num_threads);
            if (options->num_threads != 0) threads = options->num_threads;
        }
        // the only engine of this library is the GPU: AUTO resolves to it, on device 0 with the default context
        quintrit_model* h = nullptr;
        if ((rc = rt_open_gpu(p.c_str(), nullptr, &h)) != QUINTRIT_OK) return rc;
        h->inner->threads = threads, h->inner->kernel = QUINTRIT_KERNEL_B200;
        *out_model = h;
        return ok();
    });
}
extern "C" int quintrit_model_open_gpu(const char* path, const quintrit_gpu_options_t* options, quintrit_model_t** out_model) {
    return guard([&]() -> int {
        if (out_model == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_model is NULL");
        *out_model = nullptr;
        std::string p;
        int rc = rt_cstr(path, "path", &p);
        if (rc != QUINTRIT_OK) return rc;
        quintrit_model* h = nullptr;
        if ((rc = rt_open_gpu(p.c_str(), options, &h)) != QUINTRIT_OK) return rc;
        *out_model = h;
        return ok();
    });
}
extern "C" int quintrit_model_free(quintrit_model_t* model) {
    return guard([&]() -> int {
        if (model == nullptr) return ok();
        int rc = rt_check(model, kMagicModel, "model");
        if (rc != QUINTRIT_OK) return rc;
        model->magic = 0;
        delete model;  // sessions hold the weights through their own reference
        return ok();
    });
}
extern "C" int quintrit_model_info(const quintrit_model_t* model, quintrit_model_info_t* out_info) {
    return guard([&]() -> int {
        int rc = rt_check(model, kMagicModel, "model");
        if (rc != QUINTRIT_OK || (rc = rt_struct(out_info, "out_info")) != QUINTRIT_OK) return rc;
        const RtModelInner& m = *model->inner;
        const GgufModelShape& s = m.data.shape;
        std::memset(out_info, 0, sizeof *out_info);
        out_info->struct_size = sizeof *out_info;
        out_info->kernel = m.kernel, out_info->num_threads = m.threads;  // AUTO and 0 for a model of quintrit_model_open_gpu (quintrit.h:523)
        out_info->num_layers = static_cast<uint32_t>(s.layers), out_info->hidden_size = static_cast<uint32_t>(s.hidden);
        out_info->num_heads = static_cast<uint32_t>(s.heads), out_info->num_kv_heads = static_cast<uint32_t>(s.kv_heads), out_info->head_dim = static_cast<uint32_t>(s.head_dim);
        out_info->vocab_size = s.vocab, out_info->context_length = s.ctx_train;
        out_info->bos_token_id = m.tok.bos(), out_info->eos_token_id = m.tok.eos();
        std::strncpy(out_info->architecture, m.arch.c_str(), sizeof out_info->architecture - 1);
        return ok();
    });
}
extern "C" int quintrit_model_set_threads(quintrit_model_t* model, uint32_t num_threads) {
    return guard([&]() -> int {
        int rc = rt_check(model, kMagicModel, "model");
        if (rc != QUINTRIT_OK) return rc;
        if (num_threads > 256) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "num_threads %u exceeds 256", num_threads);
        if (model->inner.use_count() > 1) return fail(QUINTRIT_ERR_BUSY, "the model has live sessions; free them before changing the thread count");
        if (model->inner->kernel != QUINTRIT_KERNEL_AUTO) model->inner->threads = num_threads != 0 ? num_threads : 1;  // recorded; the work runs on the GPU
        return ok();
    });
}
extern "C" int quintrit_model_device(const quintrit_model_t* model, int32_t* out_device, uint32_t* out_index) {
    return guard([&]() -> int {
        int rc = rt_check(model, kMagicModel, "model");
        if (rc != QUINTRIT_OK) return rc;
        if (out_device == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_device is NULL");
        *out_device = QUINTRIT_DEVICE_CUDA;
        if (out_index) *out_index = model->inner->data.device;
        return ok();
    });
}
extern "C" int quintrit_model_tokenize(const quintrit_model_t* model, const char* text, size_t text_len, uint32_t flags, uint32_t* out, size_t capacity, size_t* out_count) {
    return guard([&]() -> int {
        int rc = rt_check(model, kMagicModel, "model");
        if (rc != QUINTRIT_OK) return rc;
        std::string s;
        if ((rc = rt_text(text, text_len, "text", &s)) != QUINTRIT_OK) return rc;
        if (flags & ~uint32_t(QUINTRIT_TOKENIZE_ADD_BOS)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "unknown flags 0x%x", flags);
        if (out_count == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_count is NULL");
        const RtModelInner& m = *model->inner;
        if ((rc = rt_need_tokenizer(m)) != QUINTRIT_OK) return rc;
        std::vector<uint32_t> ids = m.tok.encode(s);
        if ((flags & QUINTRIT_TOKENIZE_ADD_BOS) && m.tok.bos() >= 0 && (ids.empty() || ids[0] != static_cast<uint32_t>(m.tok.bos()))) ids.insert(ids.begin(), static_cast<uint32_t>(m.tok.bos()));
        *out_count = ids.size();
        if (out == nullptr && capacity != 0) return fail(QUINTRIT_ERR_NULL_POINTER, "out is NULL");
        if (capacity < ids.size()) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "%zu tokens do not fit into a buffer of %zu", ids.size(), capacity);
        std::copy(ids.begin(), ids.end(), out);
        return ok();
    });
}
extern "C" int quintrit_model_detokenize(const quintrit_model_t* model, const uint32_t* tokens, size_t count, char* out, size_t capacity, size_t* out_len) {
    return guard([&]() -> int {
        int rc = rt_check(model, kMagicModel, "model");
        if (rc != QUINTRIT_OK) return rc;
        if (tokens == nullptr && count != 0) return fail(QUINTRIT_ERR_NULL_POINTER, "tokens is NULL");
        if (out_len == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_len is NULL");
        const RtModelInner& m = *model->inner;
        if ((rc = rt_need_tokenizer(m)) != QUINTRIT_OK) return rc;
        for (size_t i = 0; i < count; ++i)
            if (tokens[i] >= m.data.shape.vocab) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "token id %u is outside the vocabulary of %llu", tokens[i], static_cast<unsigned long long>(m.data.shape.vocab));
        const std::string s = m.tok.decode(tokens, count);
        *out_len = s.size();
        if (out == nullptr || capacity <= s.size()) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "the text needs %zu bytes including the NUL, buffer holds %zu", s.size() + 1, capacity);
        std::memcpy(out, s.c_str(), s.size() + 1);
        return ok();
    });
}
extern "C" int quintrit_model_format_chat(const quintrit_model_t* model, const quintrit_chat_message_t* messages, size_t count, char* out, size_t capacity, size_t* out_len) {
    return guard([&]() -> int {
        int rc = rt_check(model, kMagicModel, "model");
        if (rc != QUINTRIT_OK) return rc;
        if (messages == nullptr && count != 0) return fail(QUINTRIT_ERR_NULL_POINTER, "messages is NULL");
        if (out_len == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_len is NULL");
        std::vector<std::pair<std::string, std::string>> msgs(count);
        for (size_t i = 0; i < count; ++i)
            if ((rc = rt_cstr(messages[i].role, "messages[i].role", &msgs[i].first)) != QUINTRIT_OK || (rc = rt_cstr(messages[i].content, "messages[i].content", &msgs[i].second)) != QUINTRIT_OK) return rc;
        const std::string s = rt_format_chat(msgs, model->inner->arch);
        *out_len = s.size();
        if (out == nullptr || capacity <= s.size()) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "the prompt needs %zu bytes including the NUL, buffer holds %zu", s.size() + 1, capacity);
        std::memcpy(out, s.c_str(), s.size() + 1);
        return ok();
    });
}

// ---- runtime level: sessions ------------------------------------------------------------------------------------------------------
extern "C" int quintrit_session_create(const quintrit_model_t* model, const quintrit_session_options_t* options, quintrit_session_t** out_session) {
    return guard([&]() -> int {
        int rc = rt_check(model, kMagicModel, "model");
        if (rc != QUINTRIT_OK) return rc;
        if (options != nullptr && (rc = rt_struct(options, "options")) != QUINTRIT_OK) return rc;
        if (out_session == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_session is NULL");
        *out_session = nullptr;
        const std::shared_ptr<RtModelInner>& m = model->inner;
        uint32_t ctx = options != nullptr ? options->context_length : 0;
        if (ctx == 0) ctx = m->max_ctx;
        if (ctx > m->max_ctx) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "context_length %u exceeds the GPU context of the model (%u)", ctx, m->max_ctx);
        ctx = ctx >= 256 ? ctx / 256 * 256 : ctx;
        std::unique_ptr<quintrit_session> s(new quintrit_session());
        {
            std::lock_guard<std::mutex> hold(m->lock);
            if (m->spare != nullptr && static_cast<uint32_t>(m->spare->ctx) == ctx) {
                s->dec = m->spare;
                m->spare = nullptr;
            }
        }
        if (s->dec == nullptr && (rc = decoder_from_model(m->data, ctx, &s->dec)) != QUINTRIT_OK) return rc;
        s->ctx = static_cast<uint32_t>(s->dec->ctx);
        s->model = m;
        s->logits.assign(static_cast<size_t>(s->dec->vocab), 0.0f);
        s->magic = kMagicSession;
        *out_session = s.release();
        return ok();
    });
}
extern "C" int quintrit_session_free(quintrit_session_t* session) {
    return guard([&]() -> int {
        if (session == nullptr) return ok();
        int rc = rt_check(session, kMagicSession, "session");
        if (rc != QUINTRIT_OK) return rc;
        session->magic = 0;
        destroy_decoder(session->dec);
        delete session;
        return ok();
    });
}
extern "C" int quintrit_session_reset(quintrit_session_t* session) {
    return guard([&]() -> int {
        int rc = rt_check(session, kMagicSession, "session");
        if (rc != QUINTRIT_OK) return rc;
        RtSessionLock lk(session);
        if ((rc = lk.check()) != QUINTRIT_OK) return rc;
        session->dec->host_pos = 0;  // positions are rewritten from 0 on; nothing of the old conversation is read again
        session->cached.clear();
        session->logits_valid = false;
        return ok();
    });
}
extern "C" int quintrit_session_info(const quintrit_session_t* session, quintrit_session_info_t* out_info) {
    return guard([&]() -> int {
        int rc = rt_check(session, kMagicSession, "session");
        if (rc != QUINTRIT_OK || (rc = rt_struct(out_info, "out_info")) != QUINTRIT_OK) return rc;
        RtSessionLock lk(const_cast<quintrit_session*>(session));
        if ((rc = lk.check()) != QUINTRIT_OK) return rc;
        out_info->struct_size = sizeof *out_info, out_info->reserved = 0;
        out_info->context_length = session->ctx, out_info->position = session->dec->host_pos;
        return ok();
    });
}
extern "C" int quintrit_generate_params_default(quintrit_generate_params_t* params) {
    return guard([&]() -> int {
        if (params == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "params is NULL");
        std::memset(params, 0, sizeof *params);
        params->struct_size = sizeof *params, params->max_tokens = 128, params->top_k = 1, params->temperature = 0.0f, params->top_p = 1.0f;
        return ok();
    });
}

namespace {
// The generation loop of quintrit-c/src/runtime.rs:382-520 over a decoder on the device. Greedy decoding reads back only the
// token the device chose; sampling reads the logits of every step and samples on the host with the reference's sampler.
int rt_generate(quintrit_session* s, const std::string& prompt, const quintrit_generate_params_t& prm, const std::vector<std::string>& stops, quintrit_token_callback cb,
                void* user, std::string* full_out, quintrit_generate_result_t* res) {
    const RtModelInner& m = *s->model;
    const qtb::BpeTokenizer& tk = m.tok;
    const bool keep = prm.flags & QUINTRIT_GENERATE_KEEP_CONTEXT;
    std::vector<uint32_t> tokens = tk.encode(prompt);
    if (!keep && tk.bos() >= 0 && (tokens.empty() || tokens[0] != static_cast<uint32_t>(tk.bos()))) tokens.insert(tokens.begin(), static_cast<uint32_t>(tk.bos()));
    if (tokens.empty()) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "the prompt produced no tokens");
    for (uint32_t t : tokens)
        if (t >= m.data.shape.vocab) return fail(QUINTRIT_ERR_MODEL, "tokenizer produced token %u outside the vocabulary of %llu", t, static_cast<unsigned long long>(m.data.shape.vocab));
    const uint32_t base = keep ? s->dec->host_pos : 0;
    if (size_t(base) + tokens.size() > s->ctx)
        return fail(QUINTRIT_ERR_CONTEXT_OVERFLOW, "%zu prompt tokens do not fit: the context window holds %u tokens and %u are already used", tokens.size(), s->ctx, base);
    // A prompt that begins like the cached conversation is ingested from the first difference on; at least its last token is computed
    // again, because its logits start the generation (engine.rs:700-727).
    size_t common = 0;
    if (!keep && s->cached.size() == s->dec->host_pos && std::getenv("QUINTRIT_B200_NO_PREFIX_REUSE") == nullptr)
        while (common < s->cached.size() && common + 1 < tokens.size() && s->cached[common] == tokens[common]) ++common;
    s->last_reused = static_cast<uint32_t>(common);
    const uint32_t pos0 = keep ? base : static_cast<uint32_t>(common);
    if (!keep) {
        s->dec->host_pos = pos0;
        s->cached.resize(common);
    }
    RtSampler sampler(prm.temperature, prm.top_k, prm.top_p, prm.seed);
    // Sampling runs on the device where the candidates are cut to at most 1024 (top_k): the logits then never leave the GPU and the
    // sampled token is the next step's input there, as the greedy choice is. Other settings sample on the host from the logits.
    RtDeviceSampling dev_sampling{prm.temperature, prm.top_p, static_cast<int>(prm.top_k)};
    const bool on_device_sampling = !sampler.greedy() && prm.top_k >= 1 && prm.top_k <= static_cast<uint32_t>(kSampleMaxK) && prm.top_k < m.data.shape.vocab &&
                                    s->dec->tp_world == 1 && std::getenv("QUINTRIT_B200_HOST_SAMPLER") == nullptr;
    const RtDeviceSampling* dsp = on_device_sampling ? &dev_sampling : nullptr;
    if (on_device_sampling) {
        DeviceGuard dg(s->dec->device);
        if (s->dec->d_rng == nullptr) {
            int rc0 = dev_alloc(s->dec, &s->dec->d_rng, 1);
            if (rc0 != QUINTRIT_OK) return rc0;
        }
        QTB_CUDA(cudaMemcpyAsync(s->dec->d_rng, &sampler.state, sizeof sampler.state, cudaMemcpyHostToDevice, s->dec->stream));
        QTB_CUDA(cudaStreamSynchronize(s->dec->stream));  // (the state is a local of this call)
    }
    const bool greedy = sampler.greedy() || on_device_sampling;  // the device chooses: only the token comes back
    const bool llama_like = m.arch == "bitnet" || m.arch == "llama";
    uint32_t device_choice = 0;
    int rc = rt_feed(s, tokens.data() + common, tokens.size() - common, pos0, !greedy, &device_choice, dsp);
    if (rc != QUINTRIT_OK) return rc;
    uint32_t pos = base + static_cast<uint32_t>(tokens.size());
    std::string full, pending;
    uint32_t generated = 0;
    int reason = QUINTRIT_FINISH_LENGTH;
    bool stopped = false;
    auto emit = [&](const std::string& text) {  // true once the callback has asked to stop
        if (stopped || text.empty()) return stopped;
        if (cb != nullptr && cb(text.data(), text.size(), user) != 0) stopped = true;
        return stopped;
    };
    auto find_stop = [&](const std::string& text) {
        size_t best = std::string::npos;
        for (const std::string& st : stops) best = std::min(best, text.find(st));
        return best;
    };
    qtb::StreamDecoder sd;
    DeviceGuard g(s->dec->device);
    for (uint32_t step = 0; step < prm.max_tokens; ++step) {
        const uint32_t next = greedy ? device_choice : sampler.sample(s->logits);
        if ((tk.eos() >= 0 && next == static_cast<uint32_t>(tk.eos())) || (llama_like && next == 128009)) {
            reason = QUINTRIT_FINISH_EOS;
            break;
        }
        const std::string piece = sd.push(tk, next);
        full += piece;
        ++generated;
        bool halt = false;
        if (stops.empty()) {
            if (emit(piece)) reason = QUINTRIT_FINISH_CALLBACK, halt = true;
        } else {
            pending += piece;
            const size_t idx = find_stop(pending);
            if (idx != std::string::npos) {
                const bool cb_stop = emit(pending.substr(0, idx));
                full.resize(full.size() - (pending.size() - idx));
                pending.clear();
                reason = cb_stop ? QUINTRIT_FINISH_CALLBACK : QUINTRIT_FINISH_STOP_SEQUENCE;
                break;
            }
            const size_t safe = rt_safe_flush(pending, stops);
            if (safe > 0) {
                if (emit(pending.substr(0, safe))) reason = QUINTRIT_FINISH_CALLBACK, halt = true;
                pending.erase(0, safe);
            }
        }
        if (pos >= s->ctx) {
            if (!halt) reason = QUINTRIT_FINISH_CONTEXT_FULL;
            break;
        }
        // feed the token (also after a callback stop, so that the cache matches the text the caller has seen)
        if ((rc = rt_forward(s, next, pos, !greedy, &device_choice, greedy, dsp)) != QUINTRIT_OK) return rc;
        ++pos;
        if (halt) break;
    }
    if (reason != QUINTRIT_FINISH_STOP_SEQUENCE && reason != QUINTRIT_FINISH_CALLBACK) {
        const std::string rest = sd.finish(tk);  // an incomplete character at the very end
        full += rest;
        if (stops.empty()) {
            emit(rest);
        } else {
            pending += rest;
            const size_t idx = find_stop(pending);
            if (idx != std::string::npos) {
                emit(pending.substr(0, idx));
                full.resize(full.size() - (pending.size() - idx));
                pending.clear();
                reason = QUINTRIT_FINISH_STOP_SEQUENCE;
            }
        }
    }
    if (!pending.empty()) emit(pending);
    if (res != nullptr) {
        res->struct_size = sizeof *res;
        res->finish_reason = reason, res->prompt_tokens = static_cast<uint32_t>(tokens.size()), res->generated_tokens = generated, res->text_bytes = full.size();
    }
    *full_out = std::move(full);
    return QUINTRIT_OK;
}
}  // namespace

extern "C" int quintrit_session_generate(quintrit_session_t* session, const char* prompt, size_t prompt_len, const quintrit_generate_params_t* params, quintrit_token_callback callback,
                                         void* user_data, char* out, size_t out_capacity, size_t* out_len, quintrit_generate_result_t* result) {
    return guard([&]() -> int {
        int rc = rt_check(session, kMagicSession, "session");
        if (rc != QUINTRIT_OK) return rc;
        std::string text;
        if ((rc = rt_text(prompt, prompt_len, "prompt", &text)) != QUINTRIT_OK) return rc;
        quintrit_generate_params_t prm;
        quintrit_generate_params_default(&prm);
        if (params != nullptr) {
            if ((rc = rt_struct(params, "params")) != QUINTRIT_OK) return rc;
            prm = *params;
        }
        if (prm.flags & ~uint32_t(QUINTRIT_GENERATE_KEEP_CONTEXT)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "params.flags has unknown bits set: 0x%x", prm.flags);
        if (!(prm.temperature >= 0.0f) || !std::isfinite(prm.temperature)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "temperature must be finite and not negative");
        if (!(prm.top_p > 0.0f && prm.top_p <= 1.0f)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "top_p must be in (0, 1]");
        if (prm.stop_count > 64) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "at most 64 stop sequences");
        if (prm.stop_count != 0 && prm.stop_sequences == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "stop_sequences is NULL");
        std::vector<std::string> stops;
        for (size_t i = 0; i < prm.stop_count; ++i) {
            std::string st;
            if ((rc = rt_cstr(prm.stop_sequences[i], "stop_sequences[i]", &st)) != QUINTRIT_OK) return rc;
            if (!st.empty()) stops.push_back(std::move(st));
        }
        if (result != nullptr && (rc = rt_struct(result, "result")) != QUINTRIT_OK) return rc;
        if (out == nullptr && out_capacity != 0) return fail(QUINTRIT_ERR_NULL_POINTER, "out is NULL");
        if ((rc = rt_need_tokenizer(*session->model)) != QUINTRIT_OK) return rc;
        RtSessionLock lk(session);
        if ((rc = lk.check()) != QUINTRIT_OK) return rc;
        std::string full;
        if ((rc = rt_generate(session, text, prm, stops, callback, user_data, &full, result)) != QUINTRIT_OK) return rc;
        rt_write_text(out, out_capacity, full);
        if (out_len) *out_len = full.size();
        return ok();
    });
}

// ---- token-id entry points (declared in quintrit_b200.h) -----------------------------------------------------------------------------
extern "C" int quintrit_session_feed_tokens(quintrit_session_t* session, const uint32_t* tokens, size_t count, uint32_t flags) {
    return guard([&]() -> int {
        int rc = rt_check(session, kMagicSession, "session");
        if (rc != QUINTRIT_OK) return rc;
        if (tokens == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "tokens is NULL");
        if (count == 0) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "no tokens to feed");
        if (flags & ~uint32_t(QUINTRIT_GENERATE_KEEP_CONTEXT)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "unknown flags 0x%x", flags);
        RtSessionLock lk(session);
        if ((rc = lk.check()) != QUINTRIT_OK) return rc;
        const uint32_t pos0 = (flags & QUINTRIT_GENERATE_KEEP_CONTEXT) ? session->dec->host_pos : 0;
        for (size_t i = 0; i < count; ++i)
            if (tokens[i] >= static_cast<uint32_t>(session->dec->vocab_full)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "token id %u is outside the vocabulary of %d", tokens[i], session->dec->vocab_full);
        if (size_t(pos0) + count > session->ctx) return fail(QUINTRIT_ERR_CONTEXT_OVERFLOW, "%zu tokens do not fit: the context window holds %u tokens and %u are already used", count, session->ctx, pos0);
        if (pos0 == 0) session->dec->host_pos = 0;
        if ((rc = rt_feed(session, tokens, count, pos0, true, nullptr)) != QUINTRIT_OK) return rc;
        return ok();
    });
}
extern "C" int quintrit_session_logits(quintrit_session_t* session, float* out, size_t capacity) {
    return guard([&]() -> int {
        int rc = rt_check(session, kMagicSession, "session");
        if (rc != QUINTRIT_OK) return rc;
        if (out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out is NULL");
        RtSessionLock lk(session);
        if ((rc = lk.check()) != QUINTRIT_OK) return rc;
        if (!session->logits_valid) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "the session holds no logits: feed tokens first (quintrit_session_feed_tokens)");
        if (capacity < session->logits.size()) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out holds %zu values, the vocabulary has %zu", capacity, session->logits.size());
        std::copy(session->logits.begin(), session->logits.end(), out);
        return ok();
    });
}
extern "C" int quintrit_session_generate_tokens(quintrit_session_t* session, const uint32_t* prompt, size_t prompt_len, size_t max_new, uint32_t* out, size_t out_capacity, size_t* out_count) {
    return guard([&]() -> int {
        int rc = rt_check(session, kMagicSession, "session");
        if (rc != QUINTRIT_OK) return rc;
        if (out_count == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_count is NULL");
        *out_count = 0;
        RtSessionLock lk(session);
        if ((rc = lk.check()) != QUINTRIT_OK) return rc;
        // greedy, without leaving the device between tokens; the session restarts from position 0
        if ((rc = quintrit_b200_decoder_generate(session->dec, prompt, prompt_len, max_new, out, out_capacity)) != QUINTRIT_OK) return rc;
        session->cached.clear();  // the loop ran on the device: the host has no record of what the cache holds now
        session->logits_valid = false;
        *out_count = max_new;
        return ok();
    });
}

extern "C" int quintrit_b200_session_reused_tokens(const struct quintrit_session* session, uint32_t* out_reused) {
    return guard([&]() -> int {
        int rc = rt_check(session, kMagicSession, "session");
        if (rc != QUINTRIT_OK) return rc;
        if (out_reused == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_reused is NULL");
        *out_reused = session->last_reused;
        return ok();
    });
}

// ---- the tokenizer alone, on a host without a GPU (declared in quintrit_b200.h) ---------------------------------------------
extern "C" int quintrit_b200_tokenizer_open(const char* path, quintrit_b200_tokenizer_t** out_tokenizer) {
    return guard([&]() -> int {
        if (out_tokenizer == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_tokenizer is NULL");
        *out_tokenizer = nullptr;
        std::string p;
        int rc = rt_cstr(path, "path", &p);
        if (rc != QUINTRIT_OK) return rc;
        GgufFile g;
        std::string why;
        const int st = g.open(p.c_str(), why);
        if (st == 1) return fail(QUINTRIT_ERR_IO, "%s", why.c_str());
        if (st != 0) return fail(QUINTRIT_ERR_FORMAT, "%s", why.c_str());
        std::unique_ptr<quintrit_b200_tokenizer> h(new quintrit_b200_tokenizer());
        why = rt_build_tokenizer(g, &h->tok);
        if (!why.empty()) return fail(QUINTRIT_ERR_UNSUPPORTED, "%s", why.c_str());
        h->magic = kMagicTokenizer;
        *out_tokenizer = h.release();
        return ok();
    });
}
extern "C" int quintrit_b200_tokenizer_free(quintrit_b200_tokenizer_t* tokenizer) {
    return guard([&]() -> int {
        if (tokenizer == nullptr) return ok();
        int rc = rt_check(tokenizer, kMagicTokenizer, "tokenizer");
        if (rc != QUINTRIT_OK) return rc;
        tokenizer->magic = 0;
        delete tokenizer;
        return ok();
    });
}
extern "C" int quintrit_b200_tokenizer_info(const quintrit_b200_tokenizer_t* tokenizer, uint64_t* out_vocab, int64_t* out_bos, int64_t* out_eos) {
    return guard([&]() -> int {
        int rc = rt_check(tokenizer, kMagicTokenizer, "tokenizer");
        if (rc != QUINTRIT_OK) return rc;
        if (out_vocab) *out_vocab = tokenizer->tok.vocab_size();
        if (out_bos) *out_bos = tokenizer->tok.bos();
        if (out_eos) *out_eos = tokenizer->tok.eos();
        return ok();
    });
}
extern "C" int quintrit_b200_tokenizer_encode(const quintrit_b200_tokenizer_t* tokenizer, const char* text, size_t text_len, uint32_t flags, uint32_t* out, size_t capacity,
                                              size_t* out_count) {
    return guard([&]() -> int {
        int rc = rt_check(tokenizer, kMagicTokenizer, "tokenizer");
        if (rc != QUINTRIT_OK) return rc;
        std::string s;
        if ((rc = rt_text(text, text_len, "text", &s)) != QUINTRIT_OK) return rc;
        if (flags & ~uint32_t(QUINTRIT_TOKENIZE_ADD_BOS)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "unknown flags 0x%x", flags);
        if (out_count == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_count is NULL");
        const qtb::BpeTokenizer& tk = tokenizer->tok;
        std::vector<uint32_t> ids = tk.encode(s);
        if ((flags & QUINTRIT_TOKENIZE_ADD_BOS) && tk.bos() >= 0 && (ids.empty() || ids[0] != static_cast<uint32_t>(tk.bos()))) ids.insert(ids.begin(), static_cast<uint32_t>(tk.bos()));
        *out_count = ids.size();
        if (out == nullptr && capacity != 0) return fail(QUINTRIT_ERR_NULL_POINTER, "out is NULL");
        if (capacity < ids.size()) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "%zu tokens do not fit into a buffer of %zu", ids.size(), capacity);
        std::copy(ids.begin(), ids.end(), out);
        return ok();
    });
}
// `streaming` != 0 decodes the ids one by one the way the generation loop emits text (characters are never split: a token that
// ends inside a character adds nothing until the character is complete) and, with out_piece_ends, reports the text length after
// every token plus the final flush (count + 1 values).
extern "C" int quintrit_b200_tokenizer_decode(const quintrit_b200_tokenizer_t* tokenizer, const uint32_t* tokens, size_t count, int streaming, char* out, size_t capacity,
                                              size_t* out_len, size_t* out_piece_ends) {
    return guard([&]() -> int {
        int rc = rt_check(tokenizer, kMagicTokenizer, "tokenizer");
        if (rc != QUINTRIT_OK) return rc;
        if (tokens == nullptr && count != 0) return fail(QUINTRIT_ERR_NULL_POINTER, "tokens is NULL");
        if (out_len == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_len is NULL");
        const qtb::BpeTokenizer& tk = tokenizer->tok;
        for (size_t i = 0; i < count; ++i)
            if (tokens[i] >= tk.vocab_size()) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "token id %u is outside the vocabulary of %zu", tokens[i], tk.vocab_size());
        std::string s;
        if (streaming) {
            qtb::StreamDecoder sd;
            for (size_t i = 0; i < count; ++i) {
                s += sd.push(tk, tokens[i]);
                if (out_piece_ends) out_piece_ends[i] = s.size();
            }
            s += sd.finish(tk);
            if (out_piece_ends) out_piece_ends[count] = s.size();
        } else {
            s = tk.decode(tokens, count);
        }
        *out_len = s.size();
        if (out == nullptr || capacity <= s.size()) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "the text needs %zu bytes including the NUL, buffer holds %zu", s.size() + 1, capacity);
        std::memcpy(out, s.c_str(), s.size() + 1);
        return ok();
    });
}
