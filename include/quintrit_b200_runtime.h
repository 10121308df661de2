/*
 * quintrit_b200_runtime.h - the functions of the reference's C API that libquintrit_b200.so exports under their own
 * names, for a program that has no copy of the reference's header.
 *
 * The library exports every function of rust/crates/quintrit-c/include/quintrit.h (ABI version 1) with that header's
 * names, argument order, struct layouts, status codes and buffer rules, so a program compiled against quintrit.h links
 * against this library unchanged. Such a program keeps including quintrit.h; this header declares the same items for
 * everyone else and is skipped when quintrit.h was included before it (its guard QUINTRIT_H is honoured and set).
 *
 * What differs from the reference library, by design (this library has no CPU engine):
 *   - QUINTRIT_KERNEL_AUTO resolves to QUINTRIT_KERNEL_B200 (quintrit_b200.h): planar rows, tile_rows 1. The kernel ids
 *     1..3 (scalar, simd32, avx512) give QUINTRIT_ERR_UNSUPPORTED wherever they would compute or lay out data.
 *   - quintrit_gemv_i32 / _f32 take host buffers, as in the reference, and therefore move the weights to the GPU on
 *     every call; resident weights are quintrit_b200_matrix_* (quintrit_b200.h).
 *   - quintrit_model_open loads the model onto GPU 0 (kernel AUTO or B200; num_threads is recorded and reported, and
 *     used for nothing); quintrit_model_open_gpu is the reference's own GPU entry (quintrit.h:515-527).
 *   - quintrit_cuda_device_info reports `supported` = 1 for compute capability 10.0 only.
 * Everything else follows the reference: quintrit-c/src/{tiles,gguf,runtime,cuda}.rs.
 */
#ifndef QUINTRIT_B200_RUNTIME_H
#define QUINTRIT_B200_RUNTIME_H

#include "quintrit_b200.h"

#ifndef QUINTRIT_H
#define QUINTRIT_H

#ifdef __cplusplus
extern "C" {
#endif

/* ---- version and host queries (quintrit.h:107-161) ---- */
#define QUINTRIT_VERSION_STRING "0.2.0"
#define QUINTRIT_ABI_VERSION 1
const char* quintrit_version(void);
uint32_t quintrit_abi_version(void);

#define QUINTRIT_CPU_AVX2 ((uint64_t)1 << 0)
#define QUINTRIT_CPU_AVX512F ((uint64_t)1 << 1)
#define QUINTRIT_CPU_AVX512BW ((uint64_t)1 << 2)
#define QUINTRIT_CPU_AVX512VBMI ((uint64_t)1 << 3)
#define QUINTRIT_CPU_AVX512VNNI ((uint64_t)1 << 4)
int quintrit_cpu_features(uint64_t* out_mask); /* of the host; informational */

#define QUINTRIT_KERNEL_AUTO 0
#define QUINTRIT_KERNEL_SCALAR 1
#define QUINTRIT_KERNEL_SIMD32 2
#define QUINTRIT_KERNEL_AVX512 3
#define QUINTRIT_MAX_THREADS 256
int quintrit_kernel_supported(int32_t kernel, int32_t* out_supported); /* B200/AUTO: 1 if a compute-capability-10.0 GPU is present */
int quintrit_kernel_resolve(int32_t kernel, int32_t* out_kernel);
const char* quintrit_kernel_name(int32_t kernel); /* "auto", "scalar", "simd32", "avx512", "b200"; NULL for an unknown id */
int quintrit_kernel_tile_rows(int32_t kernel, size_t* out_tile_rows);
int quintrit_supported_kernels(int32_t* out, size_t capacity, size_t* out_count);
int quintrit_default_threads(uint32_t* out_threads);

/* ---- kernel level (quintrit.h:163-224; quintrit-c/src/tiles.rs) ---- */
typedef struct quintrit_tiled_layout {
    uint32_t struct_size; /* sizeof(quintrit_tiled_layout_t), set by the caller */
    int32_t kernel;
    uint64_t tile_rows;
    uint64_t rows;
    uint64_t cols;
    uint64_t padded_rows;
    uint64_t bytes_per_row;
    uint64_t total_bytes;
} quintrit_tiled_layout_t;
int quintrit_tiled_layout(int32_t kernel, size_t rows, size_t cols, quintrit_tiled_layout_t* out_layout);
int quintrit_tiled_size(int32_t kernel, size_t rows, size_t cols, size_t* out_bytes);
int quintrit_pack_matrix(int32_t kernel, const int8_t* trits, size_t trits_len, size_t rows, size_t cols, uint8_t* out, size_t out_capacity);
int quintrit_unpack_matrix(int32_t kernel, const uint8_t* tiled, size_t tiled_len, size_t rows, size_t cols, int8_t* out, size_t out_capacity);
int quintrit_gemv_i32(int32_t kernel, const uint8_t* weights, size_t weights_len, size_t rows, size_t cols, const int8_t* activations,
                      size_t activations_len, int32_t* out, size_t out_capacity, uint32_t num_threads);
int quintrit_gemv_f32(int32_t kernel, const uint8_t* weights, size_t weights_len, size_t rows, size_t cols, const int8_t* activations,
                      size_t activations_len, float scale, float* out, size_t out_capacity, uint32_t num_threads);

/* ---- format level (quintrit.h:226-306; quintrit-c/src/gguf.rs) ---- */
typedef struct quintrit_gguf quintrit_gguf_t;
#define QUINTRIT_MAX_DIMS 8
#define QUINTRIT_GGML_F32 0
#define QUINTRIT_GGML_F16 1
#define QUINTRIT_GGML_Q8_0 8
#define QUINTRIT_GGML_BF16 30
#define QUINTRIT_GGML_TQ1_0 34
#define QUINTRIT_GGML_TQ2_0 35
#define QUINTRIT_GGML_I2_S 36
typedef struct quintrit_gguf_info {
    uint32_t struct_size;
    uint32_t version;
    uint64_t tensor_count;
    uint64_t metadata_count;
    uint64_t data_offset;
} quintrit_gguf_info_t;
typedef struct quintrit_tensor_info {
    uint32_t struct_size;
    int32_t ggml_type;
    uint32_t n_dims;
    int32_t is_ternary;
    uint64_t shape[QUINTRIT_MAX_DIMS]; /* innermost first: a weight matrix is [cols, rows] */
    uint64_t num_elements;
    uint64_t offset;
    uint64_t data_bytes;
    const char* name;      /* valid until quintrit_gguf_close */
    const char* type_name; /* static */
} quintrit_tensor_info_t;
int quintrit_gguf_open(const char* path, quintrit_gguf_t** out_gguf);
int quintrit_gguf_close(quintrit_gguf_t* gguf);
int quintrit_gguf_info(const quintrit_gguf_t* gguf, quintrit_gguf_info_t* out_info);
int quintrit_gguf_tensor_at(const quintrit_gguf_t* gguf, size_t index, quintrit_tensor_info_t* out_info);
int quintrit_gguf_tensor_find(const quintrit_gguf_t* gguf, const char* name, quintrit_tensor_info_t* out_info);
int quintrit_gguf_metadata_string(const quintrit_gguf_t* gguf, const char* key, char* buffer, size_t capacity, size_t* out_len);
int quintrit_gguf_metadata_u64(const quintrit_gguf_t* gguf, const char* key, uint64_t* out_value);
int quintrit_gguf_tensor_data(const quintrit_gguf_t* gguf, const char* name, const uint8_t** out_data, size_t* out_len);
int quintrit_gguf_tensor_layout(const quintrit_gguf_t* gguf, const char* name, int32_t kernel, quintrit_tiled_layout_t* out_layout, float* out_scale);
int quintrit_gguf_convert_tensor(const quintrit_gguf_t* gguf, const char* name, int32_t kernel, uint8_t* out, size_t out_capacity,
                                 quintrit_tiled_layout_t* out_layout, float* out_scale); /* transcoded on the GPU, read back as planar bytes */

/* ---- runtime level (quintrit.h:308-473, 515-530; quintrit-c/src/runtime.rs) ---- */
typedef struct quintrit_model quintrit_model_t;
typedef struct quintrit_session quintrit_session_t;
typedef struct quintrit_model_options {
    uint32_t struct_size;
    uint32_t num_threads;
    int32_t kernel;
    uint32_t flags;
} quintrit_model_options_t;
typedef struct quintrit_model_info {
    uint32_t struct_size;
    int32_t kernel;
    uint32_t num_threads;
    uint32_t num_layers;
    uint32_t hidden_size;
    uint32_t num_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint64_t vocab_size;
    uint64_t context_length;
    int64_t bos_token_id; /* -1: none */
    int64_t eos_token_id; /* -1: none */
    char architecture[16]; /* "bitnet", "falcon3" or "llama" */
} quintrit_model_info_t;
typedef struct quintrit_session_options {
    uint32_t struct_size;
    uint32_t context_length; /* 0 = the model's GPU context */
} quintrit_session_options_t;
typedef struct quintrit_session_info {
    uint32_t struct_size;
    uint32_t reserved;
    uint64_t context_length;
    uint64_t position;
} quintrit_session_info_t;
#define QUINTRIT_MODEL_OPEN_VERBOSE 1
#define QUINTRIT_TOKENIZE_ADD_BOS 1
#define QUINTRIT_GENERATE_KEEP_CONTEXT 1
#define QUINTRIT_FINISH_LENGTH 0
#define QUINTRIT_FINISH_EOS 1
#define QUINTRIT_FINISH_STOP_SEQUENCE 2
#define QUINTRIT_FINISH_CALLBACK 3
#define QUINTRIT_FINISH_CONTEXT_FULL 4
typedef struct quintrit_generate_params {
    uint32_t struct_size;
    uint32_t flags;
    uint32_t max_tokens;
    uint32_t top_k;    /* 0 = off, 1 = greedy */
    float temperature; /* 0 = greedy */
    float top_p;       /* (0, 1] */
    uint64_t seed;
    const char* const* stop_sequences;
    size_t stop_count; /* at most 64 */
} quintrit_generate_params_t;
typedef struct quintrit_generate_result {
    uint32_t struct_size;
    int32_t finish_reason;
    uint32_t prompt_tokens;
    uint32_t generated_tokens;
    uint64_t text_bytes;
} quintrit_generate_result_t;
typedef struct quintrit_chat_message {
    const char* role;
    const char* content;
} quintrit_chat_message_t;
typedef int (*quintrit_token_callback)(const char* text, size_t len, void* user_data); /* non-zero return stops the generation */

int quintrit_model_open(const char* path, const quintrit_model_options_t* options, quintrit_model_t** out_model);
int quintrit_model_free(quintrit_model_t* model);
int quintrit_model_info(const quintrit_model_t* model, quintrit_model_info_t* out_info);
int quintrit_model_set_threads(quintrit_model_t* model, uint32_t num_threads);
int quintrit_model_tokenize(const quintrit_model_t* model, const char* text, size_t text_len, uint32_t flags, uint32_t* out, size_t capacity, size_t* out_count);
int quintrit_model_detokenize(const quintrit_model_t* model, const uint32_t* tokens, size_t count, char* out, size_t capacity, size_t* out_len);
int quintrit_model_format_chat(const quintrit_model_t* model, const quintrit_chat_message_t* messages, size_t count, char* out, size_t capacity, size_t* out_len);
int quintrit_session_create(const quintrit_model_t* model, const quintrit_session_options_t* options, quintrit_session_t** out_session);
int quintrit_session_free(quintrit_session_t* session);
int quintrit_session_reset(quintrit_session_t* session);
int quintrit_session_info(const quintrit_session_t* session, quintrit_session_info_t* out_info);
int quintrit_generate_params_default(quintrit_generate_params_t* params);
int quintrit_session_generate(quintrit_session_t* session, const char* prompt, size_t prompt_len, const quintrit_generate_params_t* params,
                              quintrit_token_callback callback, void* user_data, char* out, size_t out_capacity, size_t* out_len,
                              quintrit_generate_result_t* result);

#define QUINTRIT_DEVICE_CPU 0
#define QUINTRIT_DEVICE_CUDA 1
int quintrit_model_open_gpu(const char* path, const quintrit_gpu_options_t* options, quintrit_model_t** out_model);
int quintrit_model_device(const quintrit_model_t* model, int32_t* out_device, uint32_t* out_index);

#ifdef __cplusplus
}
#endif
#endif /* QUINTRIT_H */
#endif
