/*
 * quintrit_b200.h - C ABI of libquintrit_b200.so, the B200 (sm_100a) device for quintrit's ternary decode path.
 *
 * Conventions are those of the reference's C API (rust/crates/quintrit-c/include/quintrit.h:10-33): every fallible
 * function returns an int status (0 = QUINTRIT_OK, the same numeric codes as quintrit.h:73-88), results go through
 * out-parameters, the last error message is kept per thread, versioned structs start with a uint32_t struct_size,
 * handles are opaque, tagged with a magic word and released by the matching *_free (NULL allowed). No function
 * throws, aborts or prints. There is no CPU fallback: without a usable CUDA device every compute entry returns
 * QUINTRIT_ERR_DEVICE or QUINTRIT_ERR_UNSUPPORTED.
 *
 * Plain C99: pointers and sizes only.
 *
 * The library also exports every function of quintrit.h itself (see quintrit_b200_runtime.h). A program that includes
 * the reference's quintrit.h includes it BEFORE this header: the declarations both share are then taken from there.
 */
#ifndef QUINTRIT_B200_H
#define QUINTRIT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef QUINTRIT_OK /* the codes of quintrit.h:73-88, repeated so that this header stands alone */
#define QUINTRIT_OK 0
#define QUINTRIT_ERR_NULL_POINTER 1
#define QUINTRIT_ERR_INVALID_ARGUMENT 2
#define QUINTRIT_ERR_INVALID_SHAPE 3
#define QUINTRIT_ERR_BUFFER_TOO_SMALL 4
#define QUINTRIT_ERR_INVALID_VALUE 5
#define QUINTRIT_ERR_UNSUPPORTED 6
#define QUINTRIT_ERR_IO 7
#define QUINTRIT_ERR_FORMAT 8
#define QUINTRIT_ERR_NOT_FOUND 9
#define QUINTRIT_ERR_MODEL 10
#define QUINTRIT_ERR_CONTEXT_OVERFLOW 11
#define QUINTRIT_ERR_BUSY 12
#define QUINTRIT_ERR_INTERNAL 13
#define QUINTRIT_ERR_INVALID_HANDLE 14
#define QUINTRIT_ERR_DEVICE 15
#endif

#define QUINTRIT_B200_ABI_VERSION 1

/* Kernel id of this library's device GEMV for the kernel-level functions of quintrit.h:112-224 (planar rows, tile_rows 1).
 * QUINTRIT_KERNEL_AUTO (0) resolves to it; the reference's ids 1..3 are its CPU kernels, which this library does not have. */
#define QUINTRIT_KERNEL_B200 16

/* ---- errors and version: replaces quintrit.h:91-110 (quintrit-c/src/error.rs:64-81, 149-157) ---- */
#ifndef QUINTRIT_H
const char* quintrit_status_string(int status);
int quintrit_last_error_code(void);
const char* quintrit_last_error_message(void);
#endif
const char* quintrit_b200_version(void);
uint32_t quintrit_b200_abi_version(void);

/* ---- devices: same names, struct and meaning as quintrit.h:490-513 (quintrit-c/src/cuda.rs:20-104), except that
 * `supported` is 1 only for compute capability 10.0 (the kernels are built for sm_100a alone). ---- */
#ifndef QUINTRIT_H
typedef struct quintrit_cuda_device_info {
    uint32_t struct_size;
    uint32_t index;
    int32_t compute_major;
    int32_t compute_minor;
    uint32_t sm_count;
    uint32_t supported;
    uint64_t total_memory;
    uint64_t l2_cache_bytes;
    char name[64];
} quintrit_cuda_device_info_t;

int quintrit_cuda_device_count(uint32_t* out_count);
int quintrit_cuda_device_info(uint32_t index, quintrit_cuda_device_info_t* out_info);
#endif

/* ---- host-side layout helpers: replace quintrit-cuda/src/pack.rs:24-48 (blocks_per_row, row_bytes, pack_planar),
 * i.e. quintrit-core/src/pack.rs:103-131. A trit outside {-1,0,1} gives QUINTRIT_ERR_INVALID_VALUE (as
 * quintrit_pack_matrix, quintrit.h:196-202). ---- */
size_t quintrit_b200_planar_row_bytes(size_t cols);
int quintrit_b200_pack_planar(const int8_t* trits, size_t trits_len, size_t rows, size_t cols, uint8_t* out, size_t out_capacity);

/* ---- a ternary matrix resident in HBM ---- */
typedef struct quintrit_b200_matrix quintrit_b200_matrix_t;

/* Source encodings accepted by quintrit_b200_matrix_upload; the numbers are the GGML type ids of
 * quintrit-format/src/gguf.rs (I2_S 36, TQ1_0 34, TQ2_0 35, Q2_0 42), 0 stands for planar velurex bytes. */
#define QUINTRIT_B200_SRC_PLANAR 0
#define QUINTRIT_B200_SRC_TQ1_0 34
#define QUINTRIT_B200_SRC_TQ2_0 35
#define QUINTRIT_B200_SRC_I2_S 36
#define QUINTRIT_B200_SRC_Q2_0 42 /* blocks of 64 weights: f16 scale + 16 code bytes; gives a block-scaled matrix (below) */

/*
 * Copies an encoded rows x cols ternary matrix from host memory to the device and transcodes it THERE into the
 * streaming velurex layout the GEMV kernel reads (still five trits per byte, 1.60 bits per weight). Replaces the host
 * transcode + upload of quintrit-runtime/src/gpu.rs:120-138, 212-219 (quintrit-format/src/transcoder.rs:165-200 then
 * Device::upload). `data` holds the tensor payload exactly as the GGUF file stores it (for I2_S without the trailing
 * scale, for TQ1_0 / TQ2_0 with the per-block f16 scales, which are ignored here) or planar bytes of
 * quintrit_b200_planar_row_bytes(cols) per row. On failure *out_matrix is NULL.
 */
int quintrit_b200_matrix_upload(uint32_t device_index, int32_t source, const uint8_t* data, size_t data_len, size_t rows,
                                size_t cols, quintrit_b200_matrix_t** out_matrix);
int quintrit_b200_matrix_free(quintrit_b200_matrix_t* matrix);
/* rows, cols and the bytes the matrix occupies in HBM (padding included). Any out pointer may be NULL. */
int quintrit_b200_matrix_info(const quintrit_b200_matrix_t* matrix, size_t* out_rows, size_t* out_cols, size_t* out_device_bytes);
/* Reads the matrix back as planar bytes (inverse of the device transcode; for tests and round trips). */
int quintrit_b200_matrix_download_planar(const quintrit_b200_matrix_t* matrix, uint8_t* out, size_t out_capacity);

/*
 * Block-scaled matrices (source QUINTRIT_B200_SRC_Q2_0). Replaces BlockScaledLayer::from_q2_0 / forward_q8 of
 * quintrit-runtime/src/layer.rs:420-507 (decode_q2_0_packed of quintrit-format/src/decoders/q2_0.rs:34-101, then
 * quintrit-core/src/block_scaled.rs:175-260), which the reference runs on the CPU only. The upload transcodes the payload
 * on the device to planar velurex bytes and keeps one f32 scale per 64 weights; a weight with the code 3 gives
 * QUINTRIT_ERR_FORMAT. Such a matrix is served by the entry points below (and by matrix_free / matrix_info /
 * matrix_download_planar); the integer GEMV entry points return QUINTRIT_ERR_UNSUPPORTED for it.
 */
/* The rows * cols / 64 weight scales, row-major (q2_0.rs:83-101). */
int quintrit_b200_matrix_scales(const quintrit_b200_matrix_t* matrix, float* out, size_t out_capacity);
/* Q8_0 activation blocks on the device: codes and one scale per 32 values, as quantize_q8_0 of
 * quintrit-runtime/src/ops.rs:879-910 (d = f16(amax / 127), round to nearest even). n must be a multiple of 32. */
int quintrit_b200_quantize_q8_0(uint32_t device_index, const float* x, size_t n, int8_t* out_codes, float* out_scales);
/* out = W x for f32 activations: Q8_0 quantisation followed by the Q2_0 x Q8_0 dot product of every row, bit for bit the
 * floats of quantize_q8_0 + BlockScaledLayer::forward_q8 (host buffers; copies and waits). */
int quintrit_b200_gemv_block_scaled(const quintrit_b200_matrix_t* matrix, const float* x, size_t x_len, float* out, size_t out_capacity);
/* The same for activations that are Q8_0 blocks already: BlockScaledLayer::forward_q8 (layer.rs:476-487). */
int quintrit_b200_gemv_block_scaled_q8(const quintrit_b200_matrix_t* matrix, const int8_t* codes, size_t codes_len, const float* scales,
                                       size_t scales_len, float* out, size_t out_capacity);

/*
 * Exact integer GEMV with host buffers: out[i] = sum_j W[i][j] * activations[j]. Replaces quintrit_gemv_i32
 * (quintrit.h:214-216) for a device matrix and Gemv::plain + upload/download of the reference's GPU launcher
 * (quintrit-cuda/src/gemv.rs:191-226). Copies the activations to the device, runs the kernel, copies the int32 sums
 * back and waits. The full int8 range is exact; cols must not exceed 131072 (quintrit.h:211).
 */
int quintrit_b200_gemv_i32(const quintrit_b200_matrix_t* matrix, const int8_t* activations, size_t activations_len,
                           int32_t* out, size_t out_capacity);
/* As above with out[i] = scale * sum (quintrit_gemv_f32, quintrit.h:222-224; quintrit-runtime/src/layer.rs:143-150:
 * pass weight_scale / act_scale). */
int quintrit_b200_gemv_f32(const quintrit_b200_matrix_t* matrix, const int8_t* activations, size_t activations_len,
                           float scale, float* out, size_t out_capacity);
/*
 * The same GEMV on device pointers, enqueued on `stream` (a cudaStream_t, NULL = default stream) without waiting:
 * the device seam of quintrit-cuda/src/gemv.rs:191-226 (Gemv::plain). d_activations: cols int8; d_out: rows int32.
 */
int quintrit_b200_gemv_i32_device(const quintrit_b200_matrix_t* matrix, const int8_t* d_activations, int32_t* d_out, void* stream);

/*
 * quintrit_b200_gemv_i32_device for callers that must not allocate. It has no counterpart in the reference.
 *
 * Who needs it: code that runs where device-memory allocation is forbidden or unaffordable - inside a region that is
 * being captured into a CUDA graph, in a serving loop whose memory was carved up front by a pool with nothing left
 * for cudaMalloc, or in a latency-critical thread that may not take the allocator's lock. The kernel's scratch (its
 * work list and counters) lives in a static device array of 262400 bytes that the library carries on every GPU that
 * loads it, instead of the buffers quintrit_b200_matrix_upload allocated for the handle. The call allocates nothing
 * (no cudaMalloc, cudaFree or allocating library routine); inputs and outputs are the caller's: the matrix handle
 * (its weights were placed in HBM earlier, by code that was allowed to allocate), cols int8 activations and rows int32
 * results in device memory.
 *
 * Limits and rules: a matrix that needs more than 4096 work items is rejected with QUINTRIT_ERR_INVALID_SHAPE (none of
 * the model shapes of this project comes near). All calls on one GPU share the one array: the array keeps the last
 * call's contents, the words that must start at zero are cleared by every call, and two calls that overlap on the GPU
 * (different streams, or threads) race - issue them in one stream or order them yourself. The first call on a device
 * looks up the array's device address and measures the shared-memory base with a tiny kernel and a 4-byte read-back
 * (under a lock, so first calls from several host threads are safe); make that first call outside any stream capture.
 * Because the call never waits, it does not read back the kernel's status word (the kernel's check that its table sits
 * at the measured shared-memory base): the kernel instantiation was chosen from that measurement at set-up, and a
 * mismatch, which would leave d_out all zero, is reported only by the entry points that wait (quintrit_b200_gemv_i32).
 * The 4096-item limit is a guard: with cols <= 131072 no shape reaches it on a 148-multiprocessor device.
 */
int quintrit_b200_gemv_i32_noalloc(const quintrit_b200_matrix_t* matrix, const int8_t* d_activations, int32_t* d_out, void* stream);

/* ---- a list of GEMVs executed as one persistent launch (one decode step's projections) ---- */
typedef struct quintrit_b200_plan quintrit_b200_plan_t;

/*
 * Builds a launch plan over `count` matrices of one device. Problem i multiplies matrices[i] with its own activation
 * vector. The plan owns one device buffer for all activation vectors (concatenated, each padded to a multiple of 16
 * bytes) and one for all int32 results (concatenated, each padded to a multiple of 4 values); the matrices must
 * outlive the plan. There is no counterpart in the reference, which launches one kernel per projection
 * (quintrit-runtime/src/gpu.rs:410-452); the plan exists because a B200 finishes a small projection faster than a
 * launch can be issued.
 */
int quintrit_b200_plan_create(const quintrit_b200_matrix_t* const* matrices, size_t count, quintrit_b200_plan_t** out_plan);
int quintrit_b200_plan_free(quintrit_b200_plan_t* plan);
/* Offsets (in elements) of problem `index` inside the concatenated activation and result buffers, and their totals. */
int quintrit_b200_plan_layout(const quintrit_b200_plan_t* plan, size_t index, size_t* out_act_offset, size_t* out_out_offset,
                              size_t* out_act_total, size_t* out_out_total);
/* Device pointers of the plan's activation (int8) and result (int32) buffers, for callers that fill them on the device. */
int quintrit_b200_plan_buffers(const quintrit_b200_plan_t* plan, int8_t** out_d_activations, int32_t** out_d_results);
/* Enqueues result clearing and the persistent GEMV kernel on `stream` (NULL = default); does not wait. */
int quintrit_b200_plan_launch(quintrit_b200_plan_t* plan, void* stream);
/* Host-buffer form: copies `activations` (act_total bytes) in, launches, copies out_total int32 back and waits. */
int quintrit_b200_plan_run(quintrit_b200_plan_t* plan, const int8_t* activations, size_t activations_len, int32_t* out,
                           size_t out_capacity);
/* ---- whole-token decoder: the device seam of the runtime ---- */
typedef struct quintrit_b200_decoder quintrit_b200_decoder_t;

#define QUINTRIT_B200_ARCH_LLAMA 0  /* LLaMA / Falcon3: interleaved RoPE pairs, SwiGLU (quintrit-runtime/src/config.rs:284-288, 464-467) */
#define QUINTRIT_B200_ARCH_BITNET 1 /* BitNet b1.58: NEOX RoPE pairs, squared ReLU, attention and FFN sub-norms (config.rs:419-422) */
#define QUINTRIT_B200_ARCH_QWEN 2   /* Qwen2 / Qwen3: NEOX RoPE pairs (config.rs:464-467), SwiGLU; Qwen3 adds query/key-norm (desc.qk_norms) */

/*
 * Description of a model whose ternary projections are already on the device. It plays the part of GpuModel::load
 * (quintrit-runtime/src/gpu.rs:183-260) after the GGUF has been read: dense tables are given as host pointers and copied.
 * matrices: layers * 7 handles in the order q, k, v, o, gate, up, down; scales: their weight scales (layers * 7);
 * norms: layers * 4 host pointers to F32 weights in the order attn_norm, ffn_norm, attn_sub_norm, ffn_sub_norm (the
 * last two NULL unless arch is BITNET). embed / lm_head: F16 bit patterns [vocab][hidden]; lm_head NULL = tied
 * (quintrit-runtime/src/model.rs:353). f32_values selects the attention arithmetic of files without I2_S tensors
 * (FP32 value accumulators, quintrit-runtime/src/config.rs:425-429), 0 the FP16 accumulators of I2_S files.
 * context_length is rounded down to a multiple of 256 (gpu.rs:141-146); head_dim must be a multiple of 32.
 */
typedef struct quintrit_b200_decoder_desc {
    uint32_t struct_size;
    uint32_t device_index;
    int32_t arch;
    int32_t f32_values;
    uint32_t hidden_size, intermediate_size, num_layers, num_heads, num_kv_heads, head_dim, vocab_size, context_length, rope_dims;
    float rms_norm_eps, rope_theta;
    const uint16_t* embed;
    const uint16_t* lm_head;
    const float* output_norm;
    const quintrit_b200_matrix_t* const* matrices;
    const float* scales;
    const float* const* norms;
    /* Tensor parallelism (fields added after the first version of the struct; a smaller struct_size means one GPU).
     * tp_world in {1, 2, 4, 8} ranks, one process and one GPU each, share the model: the dimensions above stay those of
     * the whole model, and this rank supplies its rows of every projection - q / k / v for its num_heads / tp_world query
     * heads and num_kv_heads / tp_world KV heads, rows [tp_rank * n / tp_world, (tp_rank + 1) * n / tp_world) of o, gate,
     * up and down - and, if lm_head is not NULL, its vocab_size / tp_world rows of the head (embed stays whole). Where
     * tp_world does not divide num_kv_heads, every rank supplies the whole q, k and v instead: attention is replicated on
     * every rank and only o, gate, up, down and the head are split. After creation the ranks exchange
     * quintrit_b200_decoder_tp_handle and call quintrit_b200_decoder_tp_attach. */
    uint32_t tp_rank, tp_world;
    /* 0: embed / lm_head hold F16 bit patterns (the reference's dense path, quintrit-runtime/src/model.rs:308-375);
     * 1: BF16 bit patterns, with the reference's BF16 projection arithmetic (quintrit-runtime/src/hybrid.rs:327-333, 364-367:
     * the row widened with bf16_to_f32, the normalised vector rounded with f32_to_bf16, rows through ggml_vec_dot_bf16,
     * ops.rs:650-712). The hidden size must be a multiple of 32 either way. */
    uint32_t table_dtype;
    /* Query/key-norm (quintrit-runtime/src/attention.rs:282-294): num_layers * 2 arrays of head_dim weights - the RMSNorm of every query
     * head and of every key head before RoPE - or NULL. The reference has this step on its block-scaled path only, and so has this
     * library: with per-tensor projections it gives QUINTRIT_ERR_UNSUPPORTED. */
    const float* const* qk_norms;
} quintrit_b200_decoder_desc_t;

int quintrit_b200_decoder_create(const quintrit_b200_decoder_desc_t* desc, quintrit_b200_decoder_t** out_decoder);
int quintrit_b200_decoder_free(quintrit_b200_decoder_t* decoder);

/*
 * Tensor-parallel group set-up (no counterpart in the reference, whose GPU decoder runs on one GPU): every rank's decoder
 * owns an exchange box in device memory into which the other ranks' kernels write their slices of the vectors every rank
 * needs whole (attention output, o and down results, SwiGLU output, greedy candidates) over NVLink peer stores.
 * quintrit_b200_decoder_tp_handle writes the 64-byte inter-process handle of this rank's box; the caller gathers the
 * handles of all ranks in rank order (any host transport: the benchmark uses torch.distributed) and passes the
 * tp_world * 64 bytes to quintrit_b200_decoder_tp_attach, which maps the peers' boxes. All ranks must then make the same
 * sequence of forward / generate / time_token calls; a rank that does not show up within two seconds makes the others
 * return QUINTRIT_ERR_DEVICE instead of waiting forever. quintrit_b200_decoder_forward returns this rank's
 * vocab_size / tp_world logits (rows tp_rank * vocab_size / tp_world onward); the greedy token is the global one.
 */
#define QUINTRIT_B200_TP_HANDLE_BYTES 64
int quintrit_b200_decoder_tp_handle(const quintrit_b200_decoder_t* decoder, uint8_t* out_handle, size_t out_capacity);
int quintrit_b200_decoder_tp_attach(quintrit_b200_decoder_t* decoder, const uint8_t* handles, size_t handles_len);
/* The same for a group whose decoders all live in this process (one thread per GPU, or several ranks on one GPU for
 * tests): `group` holds the tp_world decoders in rank order, this decoder among them; peer access between their devices is
 * enabled as needed. The environment variable QUINTRIT_B200_TP_WAIT_MS (read at creation) replaces the two seconds a
 * rank waits for a silent peer. */
int quintrit_b200_decoder_tp_attach_local(quintrit_b200_decoder_t* decoder, quintrit_b200_decoder_t* const* group, size_t group_len);

/* Options of quintrit_b200_decoder_open_gguf: the struct of quintrit.h:502-507 (same fields and meaning; no flag is
 * defined here, so flags must be 0; the context is capped at 8192 instead of 7936). */
#ifndef QUINTRIT_H
typedef struct quintrit_gpu_options {
    uint32_t struct_size;    /* set to sizeof(quintrit_gpu_options_t) */
    uint32_t device_index;   /* GPU to use (quintrit_cuda_device_info_t::index) */
    uint32_t context_length; /* largest context window in tokens; 0 = min(4096, the model's maximum); at most 7936 */
    uint32_t flags;          /* 0, or QUINTRIT_MODEL_OPEN_VERBOSE (accepted, no effect: the library never prints) */
} quintrit_gpu_options_t;
#endif

/*
 * Loads a GGUF model onto a GPU and returns a decoder for it: the device half of quintrit_model_open_gpu
 * (quintrit.h:515-527; quintrit-c/src/runtime.rs, GpuModel::load quintrit-runtime/src/gpu.rs:183-260) without the
 * tokenizer - prompts are token ids. The hyperparameters are derived like ModelConfig::from_gguf
 * (quintrit-runtime/src/config.rs:257-455); the ternary payloads (I2_S, TQ1_0, TQ2_0) are copied as the file stores
 * them and transcoded on the device; files without I2_S tensors use the FP32-accumulator attention. `options` may be
 * NULL (GPU 0, default context). A path that is not a regular file gives QUINTRIT_ERR_IO, a malformed file
 * QUINTRIT_ERR_FORMAT, a missing or mis-shaped tensor QUINTRIT_ERR_MODEL, and mixture-of-experts, hybrid and
 * query/key-norm models QUINTRIT_ERR_UNSUPPORTED (a file whose projections are all Q2_0 runs through the block-scaled kernels). On failure *out_decoder is NULL. The decoder owns the weights.
 */
int quintrit_b200_decoder_open_gguf(const char* path, const quintrit_gpu_options_t* options, quintrit_b200_decoder_t** out_decoder);

/* Shape of a decoder (the part of quintrit_model_info, quintrit.h:410-420, that concerns the device). */
typedef struct quintrit_b200_decoder_info {
    uint32_t struct_size; /* set to sizeof(quintrit_b200_decoder_info_t) before the call */
    int32_t arch;
    int32_t f32_values;
    uint32_t hidden_size, intermediate_size, num_layers, num_heads, num_kv_heads, head_dim, vocab_size, context_length, rope_dims;
    uint32_t device_index;
    uint32_t single_kernel; /* 1 if tokens are decoded by the one-kernel-per-token path */
    uint32_t table_dtype;   /* 0 = F16 embedding and head, 1 = BF16 */
} quintrit_b200_decoder_info_t;
int quintrit_b200_decoder_info(const quintrit_b200_decoder_t* decoder, quintrit_b200_decoder_info_t* out_info);

/*
 * The directory of a GGUF file as text, read on the host only (no GPU needed): "version", the hyperparameters one per
 * line as quintrit_b200_decoder_open_gguf derives them, then "tensor <name> type=<ggml id> shape=<d0>x<d1>.. bytes=<n>"
 * per tensor in file order. *out_needed receives the length including the final NUL (also with
 * QUINTRIT_ERR_BUFFER_TOO_SMALL, e.g. when out is NULL). The reference's counterpart is GgufFile::open
 * (quintrit-format/src/gguf.rs:190-313) as used by the `inspect` tools.
 */
int quintrit_b200_gguf_describe(const char* path, char* out, size_t out_capacity, size_t* out_needed);
/*
 * One token at position `pos` (positions are fed in order; an earlier position restarts from that prefix), as
 * GpuSession::forward (quintrit-runtime/src/gpu.rs:459-493) but from a token id: the embedding row is looked up on the
 * device. logits (vocab_size floats) may be NULL; out_token (may be NULL) receives the greedy choice
 * (quintrit-runtime/src/sampler.rs:73-83), computed on the device.
 */
int quintrit_b200_decoder_forward(quintrit_b200_decoder_t* decoder, uint32_t token, uint32_t pos, float* logits, size_t logits_capacity,
                                  uint32_t* out_token);
/*
 * Feeds `prompt_len` tokens from position 0 and then decodes `max_new` tokens greedily without leaving the device
 * (token and position live in device memory, one CUDA graph replay per token). out_tokens receives max_new ids.
 * The generate loop of the reference is quintrit-runtime/src/engine.rs:626-700 with the CPU sampler.
 */
int quintrit_b200_decoder_generate(quintrit_b200_decoder_t* decoder, const uint32_t* prompt, size_t prompt_len, size_t max_new,
                                   uint32_t* out_tokens, size_t out_capacity);
/* Device time of one decode step in milliseconds: minimum over `blocks` blocks of `iters` graph replays, as
 * GpuSession::time_token (quintrit-runtime/src/gpu.rs:346-370). Every replay decodes token 0 at the first free
 * position, so the cached prefix is not disturbed and the context length is the number of cached tokens plus one. */
int quintrit_b200_decoder_time_token(quintrit_b200_decoder_t* decoder, uint32_t blocks, uint32_t iters, float* out_ms);

/*
 * Profiling aid (the reference's counterpart is its ATTN_STOP phase cut, quintrit-cuda/kernels/layer.cu:296-297): runs one
 * decode step like quintrit_b200_decoder_time_token and returns the device's global timer (ns) as sampled by CTA 0 at
 * every phase boundary of the single-kernel path: 14 stamps per layer (norm, q|k|v, barrier, scores, barrier + values,
 * barrier, combine, o + barrier, norm, gate|up, barrier, SwiGLU + barrier, down, barrier) after one at the start, then two
 * around the output head, then 32 slots that stay zero unless the library was built with -DQTB_FINE_TRACE (stamps inside
 * phases). *out_count receives the number of values (also on QUINTRIT_ERR_BUFFER_TOO_SMALL).
 */
int quintrit_b200_decoder_trace_step(quintrit_b200_decoder_t* decoder, uint64_t* out_ns, size_t capacity, size_t* out_count);

/*
 * Self-test of the bounded grid barrier of the single-kernel decode path (failure detection, no counterpart in the
 * reference, which has no device-side waits): `ctas` CTAs, all resident, wait at the barrier for an arrival that cannot
 * come, with `spin_limit` polls of patience (1..2^20). The wait runs out, the kernel sets its status word and the failure
 * bit releases every other waiter; nothing faults and nothing spins beyond the limit. Returns QUINTRIT_ERR_DEVICE with
 * the message a decoder gives for the same condition; *out_released receives the number of CTAs that left through the
 * failure path (expected: ctas). The device stays usable.
 */
int quintrit_b200_selftest_barrier(uint32_t device_index, uint32_t ctas, uint32_t spin_limit, uint32_t* out_released);

/*
 * Prompt ingestion: `count` tokens at positions pos .. pos + count - 1 in chunks of up to 256, every projection of a chunk as one
 * batched product on the tensor cores (quintrit_b200_gemm_i32). The reference ingests a prompt token by token
 * (quintrit-c/src/runtime.rs:430-436); the result here is bit for bit that of `count` calls of quintrit_b200_decoder_forward:
 * the KV cache, the position, and - for the last token - the logits and the greedy choice (logits and out_token may be NULL).
 * Per-tensor ternary models on one GPU; block-scaled (Q2_0) and tensor-parallel decoders give QUINTRIT_ERR_UNSUPPORTED. The
 * text and token entry points of the runtime level use it for prompts of 8 tokens or more.
 */
int quintrit_b200_decoder_prefill(quintrit_b200_decoder_t* decoder, const uint32_t* tokens, size_t count, uint32_t pos, float* logits, size_t logits_capacity,
                                  uint32_t* out_token);

/* ---- mixture-of-experts feed-forward block (the shape of Qwen3-30B-A3B: softmax router, top-k of n experts, ternary SwiGLU experts) ----
 * The reference has no block of this kind (its Moe is Nemotron-H's, quintrit-runtime/src/hybrid.rs:798-869); this one is composed of
 * the reference's pieces, each computed as the reference computes it: the router as a BF16 projection (hybrid.rs:327-333), softmax
 * (ops.rs:274-298), experts by descending probability as std::sort leaves them (hybrid.rs:828-831), their probabilities divided by
 * their sum (hybrid.rs:833-839), an expert as the dense model's FFN (int8 absmax activations, exact integer sums, one multiply by
 * weight_scale / act_scale, SwiGLU: layer.rs:123-177, ops.rs:241-267, 427-464), the weighted outputs added in selection order
 * (hybrid.rs:847-858). One GPU; the experts of a batch run as two persistent GEMV launches whose work lists are built on the device
 * from the chosen ids.
 *
 * router_bf16: n_experts x hidden BF16 bit patterns. gate_up[e]: a matrix of 2 * inter rows (the expert's gate rows, then its up
 * rows) x hidden columns; down[e]: hidden x inter; scales[3 e + 0 / 1 / 2]: the weight scales of expert e's gate, up and down. The
 * matrices stay the caller's and must outlive the block. hidden is a multiple of 128 (at most 3200), inter a multiple of 16. */
typedef struct quintrit_b200_moe quintrit_b200_moe_t;
int quintrit_b200_moe_create(uint32_t device_index, uint32_t hidden, uint32_t inter, uint32_t n_experts, uint32_t top_k, uint32_t max_batch, const uint16_t* router_bf16,
                             const quintrit_b200_matrix_t* const* gate_up, const quintrit_b200_matrix_t* const* down, const float* scales, quintrit_b200_moe_t** out_moe);
void quintrit_b200_moe_free(quintrit_b200_moe_t* moe);
/* batch tokens (x: [batch][hidden] floats in host memory) through the block; out: [batch][hidden]; out_experts / out_weights
 * ([batch][top_k], may be NULL): the chosen experts in selection order and their weights. */
int quintrit_b200_moe_forward(quintrit_b200_moe_t* moe, const float* x, size_t batch, float* out, uint32_t* out_experts, float* out_weights);
/* Device time of the block's launches for the inputs of the last forward call (batch = its batch), averaged over `repeats` back-to-back runs. */
int quintrit_b200_moe_time(quintrit_b200_moe_t* moe, size_t batch, uint32_t repeats, float* out_ms);
/* Expert parallelism: a block that holds experts expert_first .. expert_first + expert_count - 1 only (gate_up, down and scales list those
 * experts; the router stays whole on every GPU). Every GPU routes every token (the same choice everywhere), runs the pairs whose expert it
 * holds, and leaves every pair's result - one row of `hidden` floats per (token, selection slot), zero bits where the expert lives
 * elsewhere - in a device buffer (quintrit_b200_moe_pairs). The caller adds the buffers of all GPUs as 32-bit integers (exactly one share of
 * every value is not zero, so the sum is that share bit for bit; with NCCL: an all-reduce of the buffer viewed as int32) and calls
 * quintrit_b200_moe_finish, which weights and adds the pairs in selection order. The result is the one-GPU result. */
int quintrit_b200_moe_create_shard(uint32_t device_index, uint32_t hidden, uint32_t inter, uint32_t n_experts, uint32_t top_k, uint32_t max_batch, const uint16_t* router_bf16,
                                   uint32_t expert_first, uint32_t expert_count, const quintrit_b200_matrix_t* const* gate_up, const quintrit_b200_matrix_t* const* down,
                                   const float* scales, quintrit_b200_moe_t** out_moe);
int quintrit_b200_moe_forward_partial(quintrit_b200_moe_t* moe, const float* x, size_t batch);
int quintrit_b200_moe_pairs(quintrit_b200_moe_t* moe, void** out_device_pointer, size_t* out_floats);
int quintrit_b200_moe_finish(quintrit_b200_moe_t* moe, size_t batch, float* out, uint32_t* out_experts, float* out_weights);

/* ---- the token sampler on the device (temperature, top-k, nucleus; quintrit-runtime/src/sampler.rs:59-143) ----------------
 * The runtime level (quintrit_session_generate) samples on the device when 1 <= top_k <= 1024: the logits never leave the GPU and
 * the sampled token is the next step's input there. This entry runs the same kernel on `count` logits of the caller's (host
 * memory): the candidates are the top_k largest logits / temperature in the total order of floats (ties by lower id, as the
 * reference's stable sort leaves them), softmax with the float exponential summed in double, nucleus cut at top_p, and a draw
 * with the xorshift64 generator whose state is *state (updated; never zero). The token is the one the reference's sampler
 * returns for the same logits, parameters and state. */
int quintrit_b200_sample_logits(uint32_t device_index, const float* logits, size_t count, float temperature, uint32_t top_k, float top_p, uint64_t* state,
                                uint32_t* out_token);

/* ---- several sequences decoded together (batched decode) ---------------------------------------------------------------
 * The reference decodes one sequence per session, one token per step (quintrit-runtime/src/engine.rs:282, 626-631); nothing in
 * it batches sequences. Here up to 256 independent sequences share one pass over the weights per step: the projections of a
 * step are batched products on the tensor cores (quintrit_b200_gemm_i32: every token keeps its own activation scale, the
 * integers are those of the batch-1 kernel), attention runs per sequence over that sequence's own KV cache at its own
 * position, the output head reads every vocabulary row once for all tokens. Every sequence's logits and greedy tokens are
 * bit for bit those of the same sequence decoded alone with quintrit_b200_decoder_forward.
 *
 * A batch belongs to a decoder (per-tensor ternary model on one GPU; else QUINTRIT_ERR_UNSUPPORTED): it holds one KV cache of
 * the decoder's context length per sequence and uses the decoder's weights, stream and per-token buffers, so the decoder
 * and its batches are used by one thread at a time, and a batch is freed before its decoder. */
typedef struct quintrit_b200_batch quintrit_b200_batch_t;

int quintrit_b200_batch_create(quintrit_b200_decoder_t* decoder, uint32_t sequences, quintrit_b200_batch_t** out_batch);
void quintrit_b200_batch_free(quintrit_b200_batch_t* batch);
/* Number of sequences, context length, tokens cached per sequence (any pointer may be NULL). */
int quintrit_b200_batch_info(const quintrit_b200_batch_t* batch, uint32_t* out_sequences, uint32_t* out_context, uint32_t* out_positions, size_t positions_capacity);
/* Drops the cached tokens of one sequence from `position` on (0 = start a new sequence in that slot). */
int quintrit_b200_batch_rewind(quintrit_b200_batch_t* batch, uint32_t sequence, uint32_t position);
/* Appends `count` prompt tokens to one sequence, in chunks on the tensor cores as quintrit_b200_decoder_prefill does; the last
 * token's logits and greedy choice are returned (both may be NULL) and the choice is kept as the sequence's next input. */
int quintrit_b200_batch_prefill(quintrit_b200_batch_t* batch, uint32_t sequence, const uint32_t* tokens, size_t count, float* logits, size_t logits_capacity,
                                uint32_t* out_token);
/* One step of `count` sequences: sequences[z] (distinct; NULL = all sequences in order) is fed tokens[z] (NULL = the token
 * the sequence chose last) at its own position. out_tokens[z] receives the greedy choice, logits ([count][vocab], may be NULL)
 * the logits; every listed sequence advances by one position. */
int quintrit_b200_batch_step(quintrit_b200_batch_t* batch, const uint32_t* sequences, size_t count, const uint32_t* tokens, uint32_t* out_tokens, float* logits,
                             size_t logits_capacity);

/* ---- batched projection on the tensor cores: out[b][n] = sum_k trit[n][k] * act[b][k] for `batch` int8 activation vectors
 * ([batch][cols], row-major), the integers quintrit_b200_gemv_i32 gives vector by vector (so every vector may carry its own
 * activation scale, as the tokens of a prompt do: quintrit-runtime/src/layer.rs:123-177 per token). out is [batch][rows]. The
 * kernel is tcgen05.mma.kind::i8 with the accumulator in tensor memory and the activations fetched by TMA; the first call on a
 * matrix makes a second device copy of its weights with two bits per trit in the order this kernel reads (0.25 bytes per weight
 * more), from which int8 operands are made with one table lookup per four weights. Per-tensor matrices only (not Q2_0). The _device form takes device pointers and enqueues on `stream` without
 * waiting; its status is reported by the next host-buffer call on the matrix. ---- */
int quintrit_b200_gemm_i32(quintrit_b200_matrix_t* matrix, const int8_t* activations, size_t activations_len, size_t batch, int32_t* out, size_t out_capacity);
int quintrit_b200_gemm_i32_device(quintrit_b200_matrix_t* matrix, const int8_t* d_activations, size_t batch, int32_t* d_out, void* stream);

/* ---- token-id entry points on a session of the runtime level (quintrit_model_open_gpu -> quintrit_session_create; the
 * handles are those of quintrit.h / quintrit_b200_runtime.h). They are what a server that tokenizes elsewhere binds, and what
 * the parity tests drive: the same decoder as quintrit_session_generate, without text. ---- */
struct quintrit_session;
/* Feeds `count` token ids (each below the vocabulary size); flags: 0 restarts the session at position 0,
 * QUINTRIT_GENERATE_KEEP_CONTEXT (1) continues after the cached tokens. The logits of the last position are kept for
 * quintrit_session_logits. QUINTRIT_ERR_CONTEXT_OVERFLOW if the tokens do not fit, QUINTRIT_ERR_BUSY if another thread
 * uses the session. */
int quintrit_session_feed_tokens(struct quintrit_session* session, const uint32_t* tokens, size_t count, uint32_t flags);
/* Copies the logits of the last position fed (vocab_size floats); QUINTRIT_ERR_INVALID_ARGUMENT if there are none. */
int quintrit_session_logits(struct quintrit_session* session, float* out, size_t capacity);
/* Greedy decoding from position 0 without leaving the device between tokens (quintrit_b200_decoder_generate on the
 * session's decoder): out receives max_new ids, *out_count their number. */
int quintrit_session_generate_tokens(struct quintrit_session* session, const uint32_t* prompt, size_t prompt_len, size_t max_new, uint32_t* out,
                                     size_t out_capacity, size_t* out_count);

/* Prompt tokens that the last quintrit_session_generate call of this session found in the KV cache and did not compute again: a prompt
 * that begins like the conversation the session holds is ingested from the first differing token on (the reference's
 * InferenceEngine::reusable_prefix, quintrit-runtime/src/engine.rs:700-727; at least the last prompt token is always computed). */
int quintrit_b200_session_reused_tokens(const struct quintrit_session* session, uint32_t* out_reused);

/* ---- the tokenizer of a GGUF file on its own (byte-level BPE as quintrit-runtime/src/tokenizer.rs builds it; no GPU needed):
 * for a front end that tokenizes on another host and for tests. The runtime level uses the same object. ---- */
typedef struct quintrit_b200_tokenizer quintrit_b200_tokenizer_t;
int quintrit_b200_tokenizer_open(const char* path, quintrit_b200_tokenizer_t** out_tokenizer);
int quintrit_b200_tokenizer_free(quintrit_b200_tokenizer_t* tokenizer);
int quintrit_b200_tokenizer_info(const quintrit_b200_tokenizer_t* tokenizer, uint64_t* out_vocab, int64_t* out_bos, int64_t* out_eos);
/* As quintrit_model_tokenize (quintrit.h:433-437): flags 0 or QUINTRIT_TOKENIZE_ADD_BOS (1); *out_count always receives the count. */
int quintrit_b200_tokenizer_encode(const quintrit_b200_tokenizer_t* tokenizer, const char* text, size_t text_len, uint32_t flags, uint32_t* out,
                                   size_t capacity, size_t* out_count);
/* As quintrit_model_detokenize (quintrit.h:439-443). streaming != 0 decodes token by token as the generation loop emits text
 * (a token that ends inside a UTF-8 character adds nothing until the character is complete); out_piece_ends, if not NULL,
 * receives the text length after every token and after the final flush (count + 1 values). */
int quintrit_b200_tokenizer_decode(const quintrit_b200_tokenizer_t* tokenizer, const uint32_t* tokens, size_t count, int streaming, char* out,
                                   size_t capacity, size_t* out_len, size_t* out_piece_ends);

/* Kernel launches issued by this library on the calling thread since the last call with reset != 0 (counting aid). */
uint64_t quintrit_b200_launch_count(int reset);

#ifdef __cplusplus
}
#endif
#endif
