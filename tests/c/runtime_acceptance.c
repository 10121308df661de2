/*
 * Acceptance program for the runtime and format levels of the C API as libquintrit_b200.so serves them, in plain C99
 * against include/quintrit_b200_runtime.h. argv[1] is a GGUF model with a byte-level tokenizer; the program walks one
 * tensor through the format level (convert, unpack, GEMV against a direct sum), then drives a GPU model through
 * tokenizing, sessions and generation, and prints facts for the harness to compare with the CPU oracle:
 *   PROMPT_IDS=<ids>   GREEDY_HEX=<text, hex>   SAMPLED_HEX=<text, hex>   STOP_HEX=...   KEEP_HEX=...
 * Exit code 0 = every check held. Needs a B200.
 */
#include "quintrit_b200_runtime.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static int bad = 0;
#define EXPECT(cond)                                                                                                   \
    do {                                                                                                               \
        if (!(cond)) {                                                                                                 \
            fprintf(stderr, "line %d: expected %s (last error %d: %s)\n", __LINE__, #cond, quintrit_last_error_code(), \
                    quintrit_last_error_message());                                                                    \
            ++bad;                                                                                                     \
        }                                                                                                              \
    } while (0)
#define STATUS(call, want) EXPECT((call) == (want))

struct sink {
    char text[8192];
    size_t len;
    int pieces, stop_after;
};

static int on_piece(const char* text, size_t len, void* user) {
    struct sink* s = (struct sink*)user;
    if (s->len + len < sizeof s->text) {
        memcpy(s->text + s->len, text, len);
        s->len += len;
    }
    s->pieces++;
    return s->stop_after > 0 && s->pieces >= s->stop_after;
}

static void hex(const char* label, const char* data, size_t len) {
    size_t i;
    printf("%s=", label);
    for (i = 0; i < len; ++i) printf("%02x", (unsigned)(unsigned char)data[i]);
    printf("\n");
}

static void format_level(const char* path) {
    quintrit_gguf_t* g = NULL;
    quintrit_gguf_info_t gi;
    quintrit_tensor_info_t ti;
    quintrit_tiled_layout_t lay;
    char first[256] = "";
    char arch[32];
    size_t i, r, len = 0;
    float scale = 0.0f, scale2 = 0.0f;

    STATUS(quintrit_gguf_open(path, &g), QUINTRIT_OK);
    if (g == NULL) return;
    memset(&gi, 0, sizeof gi);
    gi.struct_size = sizeof gi;
    STATUS(quintrit_gguf_info(g, &gi), QUINTRIT_OK);
    EXPECT(gi.version >= 2 && gi.tensor_count > 0 && gi.data_offset % 32 == 0);
    memset(&ti, 0, sizeof ti);
    ti.struct_size = sizeof ti;
    for (i = 0; i < gi.tensor_count; ++i) {
        STATUS(quintrit_gguf_tensor_at(g, i, &ti), QUINTRIT_OK);
        if (ti.is_ternary && first[0] == '\0' && strlen(ti.name) < sizeof first) strcpy(first, ti.name);
    }
    STATUS(quintrit_gguf_tensor_at(g, (size_t)gi.tensor_count, &ti), QUINTRIT_ERR_INVALID_ARGUMENT);
    STATUS(quintrit_gguf_tensor_find(g, "no.such.tensor", &ti), QUINTRIT_ERR_NOT_FOUND);
    STATUS(quintrit_gguf_metadata_string(g, "general.architecture", arch, sizeof arch, &len), QUINTRIT_OK);
    EXPECT(len == strlen(arch));
    STATUS(quintrit_gguf_metadata_string(g, "general.architecture", arch, 2, &len), QUINTRIT_ERR_BUFFER_TOO_SMALL);
    EXPECT(first[0] != '\0');
    if (first[0] != '\0') {
        uint8_t* planar;
        int8_t *trits, *acts;
        int32_t* got;
        float* gotf;
        size_t rows, cols;
        memset(&lay, 0, sizeof lay);
        lay.struct_size = sizeof lay;
        STATUS(quintrit_gguf_tensor_layout(g, first, QUINTRIT_KERNEL_AUTO, &lay, &scale), QUINTRIT_OK);
        EXPECT(lay.kernel == QUINTRIT_KERNEL_B200 && lay.tile_rows == 1 && lay.total_bytes == lay.rows * lay.bytes_per_row);
        rows = (size_t)lay.rows, cols = (size_t)lay.cols;
        planar = (uint8_t*)malloc((size_t)lay.total_bytes);
        trits = (int8_t*)malloc(rows * cols);
        acts = (int8_t*)malloc(cols);
        got = (int32_t*)malloc(rows * sizeof *got);
        gotf = (float*)malloc(rows * sizeof *gotf);
        STATUS(quintrit_gguf_convert_tensor(g, first, lay.kernel, planar, (size_t)lay.total_bytes - 1, &lay, &scale2), QUINTRIT_ERR_BUFFER_TOO_SMALL);
        STATUS(quintrit_gguf_convert_tensor(g, first, lay.kernel, planar, (size_t)lay.total_bytes, &lay, &scale2), QUINTRIT_OK);
        EXPECT(scale == scale2 && scale > 0.0f);
        STATUS(quintrit_unpack_matrix(lay.kernel, planar, (size_t)lay.total_bytes, rows, cols, trits, rows * cols), QUINTRIT_OK);
        for (i = 0; i < cols; ++i) acts[i] = (int8_t)((int)((i * 53 + 11) % 255) - 127);
        STATUS(quintrit_gemv_i32(lay.kernel, planar, (size_t)lay.total_bytes, rows, cols, acts, cols, got, rows, 0), QUINTRIT_OK);
        STATUS(quintrit_gemv_f32(lay.kernel, planar, (size_t)lay.total_bytes, rows, cols, acts, cols, 0.25f, gotf, rows, 0), QUINTRIT_OK);
        for (r = 0; r < rows; ++r) {
            long long sum = 0;
            for (i = 0; i < cols; ++i) sum += (long long)trits[r * cols + i] * acts[i];
            if (sum != got[r] || (float)sum * 0.25f != gotf[r]) {
                fprintf(stderr, "row %lu: %lld expected, %d / %g computed\n", (unsigned long)r, sum, got[r], gotf[r]);
                ++bad;
                break;
            }
        }
        {   /* the host packer gives the bytes the device transcoder gave */
            uint8_t* again = (uint8_t*)malloc((size_t)lay.total_bytes);
            STATUS(quintrit_pack_matrix(QUINTRIT_KERNEL_AUTO, trits, rows * cols, rows, cols, again, (size_t)lay.total_bytes), QUINTRIT_OK);
            EXPECT(memcmp(again, planar, (size_t)lay.total_bytes) == 0);
            free(again);
        }
        STATUS(quintrit_gemv_i32(QUINTRIT_KERNEL_SIMD32, planar, (size_t)lay.total_bytes, rows, cols, acts, cols, got, rows, 0), QUINTRIT_ERR_UNSUPPORTED);
        printf("format level: '%s' %lu x %lu, scale %g\n", first, (unsigned long)rows, (unsigned long)cols, scale);
        free(planar), free(trits), free(acts), free(got), free(gotf);
    }
    STATUS(quintrit_gguf_close(g), QUINTRIT_OK);
}

static void runtime_level(const char* path, const char* prompt) {
    quintrit_gpu_options_t opt;
    quintrit_model_t* model = NULL;
    quintrit_model_info_t mi;
    quintrit_session_t *s = NULL, *s2 = NULL;
    quintrit_session_options_t so;
    quintrit_session_info_t si;
    quintrit_generate_params_t p;
    quintrit_generate_result_t res;
    struct sink sink;
    static char out[8192], again[8192], text[8192];
    uint32_t ids[512];
    size_t n = 0, out_len = 0, again_len = 0, text_len = 0, i;
    int32_t dev = -1;
    uint32_t dev_index = 99;
    const char* stops[2];
    uint64_t after_first;

    memset(&opt, 0, sizeof opt);
    opt.struct_size = sizeof opt;
    STATUS(quintrit_model_open_gpu("no-such-file.gguf", &opt, &model), QUINTRIT_ERR_IO);
    EXPECT(model == NULL);
    opt.flags = 0x80;
    STATUS(quintrit_model_open_gpu(path, &opt, &model), QUINTRIT_ERR_INVALID_ARGUMENT);
    opt.flags = 0;
    STATUS(quintrit_model_open_gpu(path, &opt, &model), QUINTRIT_OK);
    if (model == NULL) return;
    memset(&mi, 0, sizeof mi);
    mi.struct_size = sizeof mi;
    STATUS(quintrit_model_info(model, &mi), QUINTRIT_OK);
    EXPECT(mi.kernel == QUINTRIT_KERNEL_AUTO && mi.num_threads == 0 && mi.vocab_size > 0 && mi.num_layers > 0);
    printf("model: %s, %u layers, hidden %u, %u/%u heads of %u, vocab %lu, context %lu, bos %ld, eos %ld\n", mi.architecture, mi.num_layers, mi.hidden_size,
           mi.num_heads, mi.num_kv_heads, mi.head_dim, (unsigned long)mi.vocab_size, (unsigned long)mi.context_length, (long)mi.bos_token_id, (long)mi.eos_token_id);
    STATUS(quintrit_model_device(model, &dev, &dev_index), QUINTRIT_OK);
    EXPECT(dev == QUINTRIT_DEVICE_CUDA && dev_index == 0);

    /* tokenizer: size query, fill, round trip */
    STATUS(quintrit_model_tokenize(model, prompt, strlen(prompt), QUINTRIT_TOKENIZE_ADD_BOS, NULL, 0, &n), QUINTRIT_ERR_BUFFER_TOO_SMALL);
    EXPECT(n > 0 && n <= 512);
    STATUS(quintrit_model_tokenize(model, prompt, strlen(prompt), QUINTRIT_TOKENIZE_ADD_BOS, ids, 512, &n), QUINTRIT_OK);
    printf("PROMPT_IDS=");
    for (i = 0; i < n; ++i) printf("%s%u", i ? "," : "", (unsigned)ids[i]);
    printf("\n");
    {   /* without BOS the ids decode to the prompt; with it, one more id stands in front */
        uint32_t plain[512];
        size_t m = 0;
        STATUS(quintrit_model_tokenize(model, prompt, strlen(prompt), 0, plain, 512, &m), QUINTRIT_OK);
        EXPECT(m == n || (m + 1 == n && memcmp(plain, ids + 1, m * sizeof plain[0]) == 0 && (int64_t)ids[0] == mi.bos_token_id));
        STATUS(quintrit_model_detokenize(model, plain, m, text, sizeof text, &text_len), QUINTRIT_OK);
        EXPECT(text_len == strlen(prompt) && memcmp(text, prompt, text_len) == 0);
    }
    STATUS(quintrit_model_detokenize(model, ids, n, text, 2, &text_len), QUINTRIT_ERR_BUFFER_TOO_SMALL);
    STATUS(quintrit_model_tokenize(model, "\xff\xfe", 2, 0, ids, 512, &n), QUINTRIT_ERR_INVALID_ARGUMENT); /* not UTF-8 */

    memset(&so, 0, sizeof so);
    so.struct_size = sizeof so;
    so.context_length = (uint32_t)mi.context_length + 256;
    STATUS(quintrit_session_create(model, &so, &s), QUINTRIT_ERR_INVALID_ARGUMENT);
    so.context_length = 0;
    STATUS(quintrit_session_create(model, &so, &s), QUINTRIT_OK);
    STATUS(quintrit_session_create(model, NULL, &s2), QUINTRIT_OK);
    if (s == NULL || s2 == NULL) return;
    STATUS(quintrit_model_set_threads(model, 3), QUINTRIT_ERR_BUSY); /* live sessions */

    /* greedy: callback pieces and buffer agree; a second call and a second session give the same text */
    STATUS(quintrit_generate_params_default(&p), QUINTRIT_OK);
    EXPECT(p.struct_size == sizeof p && p.top_k == 1 && p.temperature == 0.0f && p.top_p == 1.0f && p.max_tokens == 128);
    p.max_tokens = 10;
    memset(&sink, 0, sizeof sink);
    memset(&res, 0, sizeof res);
    res.struct_size = sizeof res;
    STATUS(quintrit_session_generate(s, prompt, strlen(prompt), &p, on_piece, &sink, out, sizeof out, &out_len, &res), QUINTRIT_OK);
    EXPECT(out_len == sink.len && memcmp(out, sink.text, out_len) == 0 && out[out_len] == '\0' && res.text_bytes == out_len);
    EXPECT(res.generated_tokens > 0 && res.generated_tokens <= 10 && res.prompt_tokens > 0);
    hex("GREEDY_HEX", out, out_len);
    printf("GREEDY_TOKENS=%u reason %d\n", (unsigned)res.generated_tokens, (int)res.finish_reason);
    STATUS(quintrit_session_generate(s, prompt, strlen(prompt), &p, NULL, NULL, again, sizeof again, &again_len, NULL), QUINTRIT_OK);
    EXPECT(again_len == out_len && memcmp(out, again, out_len) == 0);
    STATUS(quintrit_session_generate(s2, prompt, strlen(prompt), &p, NULL, NULL, again, sizeof again, &again_len, NULL), QUINTRIT_OK);
    EXPECT(again_len == out_len && memcmp(out, again, out_len) == 0);
    /* a small buffer truncates at a character boundary, NUL-terminated, and still reports the full length */
    STATUS(quintrit_session_generate(s2, prompt, strlen(prompt), &p, NULL, NULL, again, 4, &again_len, NULL), QUINTRIT_OK);
    EXPECT(again_len == out_len && strlen(again) <= 3 && memcmp(again, out, strlen(again)) == 0);

    /* seeded sampling: the same seed gives the same text */
    p.temperature = 0.8f, p.top_k = 40, p.top_p = 0.9f, p.seed = 3;
    STATUS(quintrit_session_generate(s, prompt, strlen(prompt), &p, NULL, NULL, out, sizeof out, &out_len, &res), QUINTRIT_OK);
    STATUS(quintrit_session_generate(s2, prompt, strlen(prompt), &p, NULL, NULL, again, sizeof again, &again_len, NULL), QUINTRIT_OK);
    EXPECT(again_len == out_len && memcmp(out, again, out_len) == 0);
    hex("SAMPLED_HEX", out, out_len);
    STATUS(quintrit_generate_params_default(&p), QUINTRIT_OK);

    /* the callback stops the generation; the position counts what was fed */
    p.max_tokens = 10;
    memset(&sink, 0, sizeof sink);
    sink.stop_after = 2;
    STATUS(quintrit_session_generate(s, prompt, strlen(prompt), &p, on_piece, &sink, NULL, 0, NULL, &res), QUINTRIT_OK);
    EXPECT(res.finish_reason == QUINTRIT_FINISH_CALLBACK && sink.pieces == 2 && res.generated_tokens >= 2 && res.generated_tokens < 10);
    memset(&si, 0, sizeof si);
    si.struct_size = sizeof si;
    STATUS(quintrit_session_info(s, &si), QUINTRIT_OK);
    EXPECT(si.position == res.prompt_tokens + res.generated_tokens && si.context_length <= mi.context_length);
    after_first = si.position;

    /* KEEP_CONTEXT continues behind the cached tokens without BOS */
    p.flags = QUINTRIT_GENERATE_KEEP_CONTEXT;
    p.max_tokens = 3;
    STATUS(quintrit_session_generate(s, " and", 4, &p, NULL, NULL, out, sizeof out, &out_len, &res), QUINTRIT_OK);
    STATUS(quintrit_session_info(s, &si), QUINTRIT_OK);
    EXPECT(si.position > after_first && si.position <= after_first + res.prompt_tokens + 3);
    hex("KEEP_HEX", out, out_len);
    p.flags = 0x40;
    STATUS(quintrit_session_generate(s, prompt, strlen(prompt), &p, NULL, NULL, NULL, 0, NULL, NULL), QUINTRIT_ERR_INVALID_ARGUMENT);
    p.flags = 0;
    STATUS(quintrit_session_reset(s), QUINTRIT_OK);
    STATUS(quintrit_session_info(s, &si), QUINTRIT_OK);
    EXPECT(si.position == 0);

    /* stop sequences: the text ends before the first match; an empty one is ignored */
    p.max_tokens = 10;
    STATUS(quintrit_session_generate(s, prompt, strlen(prompt), &p, NULL, NULL, out, sizeof out, &out_len, &res), QUINTRIT_OK);
    if (out_len >= 3) {
        char marker[8];
        size_t cut = out_len / 2, mlen;
        while (cut > 0 && ((unsigned char)out[cut] & 0xC0) == 0x80) --cut; /* a character boundary */
        mlen = 1;
        while (cut + mlen < out_len && ((unsigned char)out[cut + mlen] & 0xC0) == 0x80) ++mlen;
        memcpy(marker, out + cut, mlen);
        marker[mlen] = '\0';
        stops[0] = "";
        stops[1] = marker;
        p.stop_sequences = stops;
        p.stop_count = 2;
        memset(&sink, 0, sizeof sink);
        STATUS(quintrit_session_generate(s, prompt, strlen(prompt), &p, on_piece, &sink, again, sizeof again, &again_len, &res), QUINTRIT_OK);
        EXPECT(res.finish_reason == QUINTRIT_FINISH_STOP_SEQUENCE && strstr(again, marker) == NULL);
        EXPECT(again_len <= cut && memcmp(again, out, again_len) == 0 && sink.len == again_len && memcmp(sink.text, again, again_len) == 0);
        hex("STOP_HEX", again, again_len);
        p.stop_sequences = NULL;
        p.stop_count = 0;
    }

    /* errors, not crashes */
    {
        char* huge = (char*)malloc(20000);
        memset(huge, 'x', 20000);
        STATUS(quintrit_session_generate(s, huge, 20000, &p, NULL, NULL, NULL, 0, NULL, NULL), QUINTRIT_ERR_CONTEXT_OVERFLOW);
        free(huge);
    }
    p.top_p = 0.0f;
    STATUS(quintrit_session_generate(s, prompt, strlen(prompt), &p, NULL, NULL, NULL, 0, NULL, NULL), QUINTRIT_ERR_INVALID_ARGUMENT);
    p.top_p = 1.0f;
    STATUS(quintrit_session_generate(NULL, prompt, strlen(prompt), &p, NULL, NULL, NULL, 0, NULL, NULL), QUINTRIT_ERR_INVALID_HANDLE);
    STATUS(quintrit_session_generate((quintrit_session_t*)model, prompt, strlen(prompt), &p, NULL, NULL, NULL, 0, NULL, NULL), QUINTRIT_ERR_INVALID_HANDLE);

    /* a session keeps its model alive */
    STATUS(quintrit_session_free(s2), QUINTRIT_OK);
    STATUS(quintrit_model_free(model), QUINTRIT_OK);
    p.max_tokens = 10;
    STATUS(quintrit_session_generate(s, prompt, strlen(prompt), &p, NULL, NULL, again, sizeof again, &again_len, NULL), QUINTRIT_OK);
    EXPECT(again_len == out_len && memcmp(out, again, out_len) == 0);
    STATUS(quintrit_session_free(s), QUINTRIT_OK);
    STATUS(quintrit_session_free(NULL), QUINTRIT_OK);
    STATUS(quintrit_model_free(NULL), QUINTRIT_OK);
}

int main(int argc, char** argv) {
    if (argc < 2) {
        fprintf(stderr, "usage: %s model.gguf [prompt]\n", argv[0]);
        return 2;
    }
    EXPECT(quintrit_abi_version() == QUINTRIT_ABI_VERSION && strcmp(quintrit_version(), QUINTRIT_VERSION_STRING) == 0);
    format_level(argv[1]);
    runtime_level(argv[1], argc > 2 ? argv[2] : "the cat sat on the mat");
    if (bad != 0) {
        fprintf(stderr, "%d check(s) failed\n", bad);
        return 1;
    }
    printf("runtime acceptance passed\n");
    return 0;
}
