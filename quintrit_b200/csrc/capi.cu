// C ABI of libquintrit_b200.so (declared in include/quintrit_b200.h): device queries, on-device transcode of ternary
// matrices into the stream layout, the exact GEMV with host or device buffers, and the persistent multi-GEMV plan.
// Host code is C++ over the CUDA runtime API; the reference's host side for the same seam is
// rust/crates/quintrit-cuda/src/{device.rs,gemv.rs,pack.rs} and rust/crates/quintrit-c/src/cuda.rs.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <mutex>
#include <new>
#include <vector>

#include "capi_common.cuh"
#include "gemv_lut.cuh"
#include "transcode.cuh"
#include "gemm_tc.cuh"
#include "block_scaled.cuh"

using namespace qtb;

struct quintrit_b200_matrix {
    uint32_t magic;
    int device;
    int sm_count;
    size_t rows, cols, blocks, tiles;
    uint4* d_w;
    size_t w_bytes;
    // single-matrix launch state
    GemvItem* d_items;
    int n_items;
    unsigned int* d_counters;
    int8_t* d_act;
    int32_t* d_out;
    float* d_outf;
    // block-scaled (Q2_0) matrices: planar bytes and one f32 scale per 64 weights instead of the stream layout
    bool block_scaled = false;
    uint8_t* d_planar = nullptr;
    float* d_wscales = nullptr;
    float* d_x = nullptr;    // cols floats: activations of one call
    float* d_as = nullptr;   // cols / 32 activation block scales
    // batched projection on the tensor cores (gemm_tc.cuh): two-bit block-major copy of the weights and call buffers, made on first use
    uint8_t* d_gemm_w = nullptr;
    size_t gemm_rows_padded = 0;
    int8_t* d_gemm_act = nullptr;     // kGemmMaxN x whole 128-column blocks, zero padded
    int8_t* d_gemm_in = nullptr;      // host-call staging: kGemmMaxN x cols
    int32_t* d_gemm_out = nullptr;    // host-call staging: kGemmMaxN x rows
    unsigned int* d_gemm_status = nullptr;
    int32_t* d_gemm_parts = nullptr;  // partial sums of a projection whose K is split: kGemmMaxParts x kGemmMaxN x rows
};

void qtb_release_stacked(quintrit_b200_matrix* m) {
    if (m != nullptr) {
        m->magic = 0;
        delete m;
    }
}

struct quintrit_b200_plan {
    uint32_t magic;
    int device;
    int sm_count;
    size_t count;
    std::vector<size_t> act_off, out_off, rows, cols;
    size_t act_total, out_total;
    GemvItem* d_items;
    int n_items;
    unsigned int* d_counters;
    int8_t* d_act;
    int32_t* d_out;
    // plan_run with host buffers works in up to four segments of consecutive matrices: the activations of the next segments go up and the
    // results of the finished ones come down (on streams of their own) while a segment's kernel runs
    struct Segment {
        int item0, items;
        size_t act0, act_bytes, out0, out_count;
        cudaEvent_t up = nullptr, done = nullptr;
    };
    std::vector<Segment> segments;
    cudaStream_t s_run = nullptr, s_copy = nullptr;
};

namespace {

const char* kVersion = "0.1.0";

int check_matrix(const quintrit_b200_matrix* m, bool any_kind = false) {
    if (m == nullptr || m->magic != kMagicMatrix) return fail(QUINTRIT_ERR_INVALID_HANDLE, "matrix handle is NULL, freed or of the wrong type");
    if (m->block_scaled && !any_kind)
        return fail(QUINTRIT_ERR_UNSUPPORTED, "a block-scaled (Q2_0) matrix is not supported by this call: use quintrit_b200_gemv_block_scaled");
    return QUINTRIT_OK;
}
int check_plan(const quintrit_b200_plan* p) {
    if (p == nullptr || p->magic != kMagicPlan) return fail(QUINTRIT_ERR_INVALID_HANDLE, "plan handle is NULL, freed or of the wrong type");
    return QUINTRIT_OK;
}

int device_props(int index, cudaDeviceProp* prop) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) return fail(QUINTRIT_ERR_DEVICE, "no usable CUDA device: %s", cudaGetErrorString(e));
    if (index < 0 || index >= n) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "GPU index %d does not exist (%d devices)", index, n);
    QTB_CUDA(cudaGetDeviceProperties(prop, index));
    return QUINTRIT_OK;
}

int require_b200(int index, cudaDeviceProp* prop) {
    int rc = device_props(index, prop);
    if (rc != QUINTRIT_OK) return rc;
    if (prop->major != 10)
        return fail(QUINTRIT_ERR_UNSUPPORTED, "GPU %d (%s, compute capability %d.%d) is not supported: the kernels are built for sm_100a only", index,
                    prop->name, prop->major, prop->minor);
    return QUINTRIT_OK;
}

// Tiles per work item. A table fill costs about as much shared-memory time as streaming 8 row tiles, so items are
// kept well above that; the environment variable is an experiment knob.
int item_tiles_override() {
    const char* s = std::getenv("QUINTRIT_B200_ITEM_TILES");
    if (s == nullptr) return 0;
    const int v = std::atoi(s);
    return v > 0 ? v : 0;
}

void build_items(std::vector<GemvItem>& items, const uint4* w, size_t act_off, size_t out_off, size_t rows, size_t cols, size_t blocks,
                 size_t tiles, size_t tiles_per_item) {
    const size_t pairs = (blocks + 1) / 2;
    const size_t chunks = std::max<size_t>(1, (tiles + tiles_per_item - 1) / tiles_per_item);
    for (size_t p = 0; p < pairs; ++p) {
        for (size_t c = 0; c < chunks; ++c) {
            const size_t t0 = tiles * c / chunks, t1 = tiles * (c + 1) / chunks;
            if (t1 == t0) continue;
            GemvItem it{};
            const size_t g = 2 * p;
            it.wa = w + (g * tiles + t0) * 64;
            it.nblk = g + 1 < blocks ? 2 : 1;
            it.wb = it.nblk == 2 ? w + ((g + 1) * tiles + t0) * 64 : it.wa;
            it.act_off = act_off;
            it.out_off = out_off;
            it.rows = static_cast<int>(rows);
            it.cols = static_cast<int>(cols);
            it.col0 = static_cast<int>(g * kBlockTrits);
            it.tile0 = static_cast<int>(t0);
            it.ntiles = static_cast<int>(t1 - t0);
            items.push_back(it);
        }
    }
}

using GemvKernel = void (*)(const GemvItem*, int, const int8_t*, int32_t*, unsigned int*);

// Picks the kernel instantiation whose table-base constant equals the shared-window address this device gives to
// dynamic shared memory (measured once per device with smem_base_kernel).
int gemv_kernel_for_device(int dev, GemvKernel* out) {
    static GemvKernel chosen[64] = {};
    static std::mutex lock;  // first calls on a device from several host threads must not race on the cache
    if (dev < 0 || dev >= 64) return fail(QUINTRIT_ERR_DEVICE, "device index %d out of range", dev);
    std::lock_guard<std::mutex> hold(lock);
    if (chosen[dev] == nullptr) {
        unsigned int* d_base = nullptr;
        unsigned int base = 0xFFFFFFFFu;
        QTB_CUDA(cudaMalloc(&d_base, sizeof(unsigned int)));
        smem_base_kernel<<<1, 32, 1024>>>(d_base);
        cudaError_t e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaMemcpy(&base, d_base, sizeof base, cudaMemcpyDeviceToHost);
        cudaFree(d_base);
        if (e != cudaSuccess) return cuda_fail(e, "smem_base_kernel");
        GemvKernel k = nullptr;
        switch (base) {
            case 0: k = gemv_lut_kernel<0>; break;
            case 1024: k = gemv_lut_kernel<1024>; break;
            case 2048: k = gemv_lut_kernel<2048>; break;
            case 3072: k = gemv_lut_kernel<3072>; break;
            case 4096: k = gemv_lut_kernel<4096>; break;
            default: return fail(QUINTRIT_ERR_DEVICE, "unexpected shared-memory base %u on CUDA device %d: no kernel was built for it", base, dev);
        }
        QTB_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemBytes));
        chosen[dev] = k;
    }
    *out = chosen[dev];
    return QUINTRIT_OK;
}

int launch_gemv(const GemvItem* d_items, int n_items, const int8_t* d_act, int32_t* d_out, unsigned int* d_counters, int sm_count,
                cudaStream_t stream) {
    int dev = 0;
    QTB_CUDA(cudaGetDevice(&dev));
    GemvKernel k = nullptr;
    int rc = gemv_kernel_for_device(dev, &k);
    if (rc != QUINTRIT_OK) return rc;
    const int grid = std::max(1, std::min(n_items, sm_count * kCtasPerSm));
    k<<<grid, kGemvThreads, kGemvSmemBytes, stream>>>(d_items, n_items, d_act, d_out, d_counters);
    ++g_launches;
    QTB_CUDA(cudaGetLastError());
    return QUINTRIT_OK;
}

// After a synchronisation: did the kernel refuse to run because its table-base constant was wrong?
int check_kernel_status(unsigned int* d_counters) {
    unsigned int flag = 0;
    QTB_CUDA(cudaMemcpy(&flag, d_counters + 2, sizeof flag, cudaMemcpyDeviceToHost));
    if (flag != 0) return fail(QUINTRIT_ERR_DEVICE, "GEMV kernel on the CUDA device found its shared-memory table at an unexpected address");
    return QUINTRIT_OK;
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

}  // namespace

#include "decoder.cuh"
#include "moe.cuh"
#include "gguf.hpp"

// ---------------------------------------------------------------------------------------------------------------------
// errors, version, devices
// ---------------------------------------------------------------------------------------------------------------------

extern "C" const char* quintrit_status_string(int status) {
    static const char* names[] = {"success", "a required pointer is NULL", "invalid argument", "invalid shape", "buffer too small",
                                  "invalid value", "unsupported", "I/O error", "format error", "not found", "model error",
                                  "context overflow", "busy", "internal error", "invalid handle", "device error"};
    return status >= 0 && status <= 15 ? names[status] : "unknown status";
}
extern "C" int quintrit_last_error_code(void) { return last_error().code; }
extern "C" const char* quintrit_last_error_message(void) { return last_error().message.c_str(); }
extern "C" const char* quintrit_b200_version(void) { return kVersion; }
extern "C" uint32_t quintrit_b200_abi_version(void) { return QUINTRIT_B200_ABI_VERSION; }

extern "C" int quintrit_cuda_device_count(uint32_t* out_count) {
    return guard([&]() -> int {
        if (out_count == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_count is NULL");
        int n = 0;
        // A machine without a driver reports zero devices (quintrit.h:510).
        if (cudaGetDeviceCount(&n) != cudaSuccess) {
            cudaGetLastError();
            n = 0;
        }
        *out_count = static_cast<uint32_t>(n);
        return ok();
    });
}

extern "C" int quintrit_cuda_device_info(uint32_t index, quintrit_cuda_device_info_t* out_info) {
    return guard([&]() -> int {
        if (out_info == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_info is NULL");
        if (out_info->struct_size < sizeof(quintrit_cuda_device_info_t))
            return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "struct_size %u is smaller than quintrit_cuda_device_info_t (%zu)", out_info->struct_size,
                        sizeof(quintrit_cuda_device_info_t));
        cudaDeviceProp prop;
        int rc = device_props(static_cast<int>(index), &prop);
        if (rc != QUINTRIT_OK) return rc;
        const uint32_t size = out_info->struct_size;
        std::memset(out_info, 0, sizeof(quintrit_cuda_device_info_t));
        out_info->struct_size = size;
        out_info->index = index;
        out_info->compute_major = prop.major;
        out_info->compute_minor = prop.minor;
        out_info->sm_count = static_cast<uint32_t>(prop.multiProcessorCount);
        out_info->supported = prop.major == 10 ? 1u : 0u;
        out_info->total_memory = prop.totalGlobalMem;
        out_info->l2_cache_bytes = static_cast<uint64_t>(prop.l2CacheSize);
        std::strncpy(out_info->name, prop.name, sizeof(out_info->name) - 1);
        return ok();
    });
}

// ---------------------------------------------------------------------------------------------------------------------
// host-side layout helpers
// ---------------------------------------------------------------------------------------------------------------------

extern "C" size_t quintrit_b200_planar_row_bytes(size_t cols) { return (cols + kBlockTrits - 1) / kBlockTrits * kBlockBytes; }

extern "C" int quintrit_b200_pack_planar(const int8_t* trits, size_t trits_len, size_t rows, size_t cols, uint8_t* out, size_t out_capacity) {
    return guard([&]() -> int {
        if (trits == nullptr || out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "trits or out is NULL");
        if (rows == 0 || cols == 0 || rows > (size_t(1) << 31) || cols > (size_t(1) << 31))
            return fail(QUINTRIT_ERR_INVALID_SHAPE, "rows and cols must be in [1, 2^31]");
        if (trits_len < rows * cols) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "trits hold %zu values, %zu are needed", trits_len, rows * cols);
        const size_t blocks = (cols + kBlockTrits - 1) / kBlockTrits, need = rows * blocks * kBlockBytes;
        if (out_capacity < need) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out holds %zu bytes, %zu are needed", out_capacity, need);
        static const unsigned radix[5] = {1, 3, 9, 28, 84};
        for (size_t r = 0; r < rows; ++r) {
            const int8_t* row = trits + r * cols;
            for (size_t b = 0; b < blocks; ++b)
                for (size_t j = 0; j < kBlockBytes; ++j) {
                    unsigned byte = 0;
                    for (size_t p = 0; p < 5; ++p) {
                        const size_t c = b * kBlockTrits + p * kBlockBytes + j;
                        const int t = c < cols ? row[c] : 0;
                        if (t < -1 || t > 1) return fail(QUINTRIT_ERR_INVALID_VALUE, "trit %d at row %zu, column %zu is outside {-1, 0, 1}", t, r, c);
                        byte += radix[p] * static_cast<unsigned>(t + 1);
                    }
                    out[(r * blocks + b) * kBlockBytes + j] = static_cast<uint8_t>(byte);
                }
        }
        return ok();
    });
}

// ---------------------------------------------------------------------------------------------------------------------
// matrices
// ---------------------------------------------------------------------------------------------------------------------

namespace {

void destroy_matrix(quintrit_b200_matrix* m) {
    if (m == nullptr) return;
    DeviceGuard g(m->device);
    cudaFree(m->d_w);
    cudaFree(m->d_items);
    cudaFree(m->d_counters);
    cudaFree(m->d_act);
    cudaFree(m->d_out);
    cudaFree(m->d_outf);
    cudaFree(m->d_planar);
    cudaFree(m->d_wscales);
    cudaFree(m->d_x);
    cudaFree(m->d_as);
    cudaFree(m->d_gemm_w);
    cudaFree(m->d_gemm_act);
    cudaFree(m->d_gemm_in);
    cudaFree(m->d_gemm_out);
    cudaFree(m->d_gemm_status);
    cudaFree(m->d_gemm_parts);
    m->magic = 0;
    delete m;
}

size_t source_bytes(int32_t source, size_t rows, size_t cols) {
    switch (source) {
        case kSrcPlanar: return rows * quintrit_b200_planar_row_bytes(cols);
        case kSrcI2S: return rows * cols / 4;
        case kSrcTq2: return rows * cols / 256 * 66;
        case kSrcTq1: return rows * cols / 256 * 54;
        case kSrcQ2: return rows * cols / 64 * 18;
        default: return 0;
    }
}

}  // namespace

extern "C" int quintrit_b200_matrix_upload(uint32_t device_index, int32_t source, const uint8_t* data, size_t data_len, size_t rows, size_t cols,
                                           quintrit_b200_matrix_t** out_matrix) {
    return guard([&]() -> int {
        if (out_matrix == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_matrix is NULL");
        *out_matrix = nullptr;
        if (data == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "data is NULL");
        if (rows == 0 || cols == 0 || rows > (size_t(1) << 31)) return fail(QUINTRIT_ERR_INVALID_SHAPE, "rows and cols must be at least 1");
        if (cols > 131072) return fail(QUINTRIT_ERR_INVALID_SHAPE, "cols %zu exceeds 131072", cols);
        if (source != kSrcPlanar && source != kSrcI2S && source != kSrcTq1 && source != kSrcTq2 && source != kSrcQ2)
            return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "unknown source encoding %d", source);
        if (source == kSrcQ2 && cols % 64 != 0) return fail(QUINTRIT_ERR_FORMAT, "a Q2_0 row of %zu weights is not a multiple of the block size 64", cols);
        if (source == kSrcI2S && cols % 128 != 0) return fail(QUINTRIT_ERR_FORMAT, "an I2_S row of %zu weights is not a multiple of 128", cols);
        if ((source == kSrcTq1 || source == kSrcTq2) && (rows * cols) % 256 != 0)
            return fail(QUINTRIT_ERR_FORMAT, "a TQ tensor of %zu weights is not a multiple of 256", rows * cols);
        const size_t need = source_bytes(source, rows, cols);
        if (data_len < need) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "data holds %zu bytes, a %zu x %zu tensor needs %zu", data_len, rows, cols, need);
        cudaDeviceProp prop;
        int rc = require_b200(static_cast<int>(device_index), &prop);
        if (rc != QUINTRIT_OK) return rc;
        DeviceGuard g(static_cast<int>(device_index));

        quintrit_b200_matrix* m = new quintrit_b200_matrix();
        m->magic = kMagicMatrix;
        m->device = static_cast<int>(device_index);
        m->sm_count = prop.multiProcessorCount;
        m->rows = rows;
        m->cols = cols;
        m->blocks = (cols + kBlockTrits - 1) / kBlockTrits;
        m->tiles = (rows + kTileRows - 1) / kTileRows;
        m->w_bytes = m->blocks * m->tiles * 1024;
        auto bail = [&](cudaError_t e, const char* what) {
            destroy_matrix(m);
            return cuda_fail(e, what);
        };
        cudaError_t e;
        uint8_t* d_src = nullptr;
        if (source == kSrcQ2) {
            // block-scaled matrix: planar velurex bytes + one f32 scale per 64 weights (q2_0.rs:34-101, pack.rs:103-131)
            m->block_scaled = true;
            m->w_bytes = rows * m->blocks * kBlockBytes + rows * (cols / 64) * sizeof(float);
            unsigned long long* d_bad = nullptr;
            unsigned long long bad = ~0ull;
            if ((e = cudaMalloc(&m->d_planar, rows * m->blocks * kBlockBytes)) != cudaSuccess) return bail(e, "cudaMalloc(planar weights)");
            if ((e = cudaMalloc(&m->d_wscales, rows * (cols / 64) * sizeof(float))) != cudaSuccess) return bail(e, "cudaMalloc(weight scales)");
            if ((e = cudaMalloc(&m->d_x, cols * sizeof(float))) != cudaSuccess) return bail(e, "cudaMalloc(activations)");
            if ((e = cudaMalloc(&m->d_as, cols / 32 * sizeof(float))) != cudaSuccess) return bail(e, "cudaMalloc(activation scales)");
            if ((e = cudaMalloc(&m->d_act, cols)) != cudaSuccess) return bail(e, "cudaMalloc(activation codes)");
            if ((e = cudaMalloc(&m->d_outf, rows * sizeof(float))) != cudaSuccess) return bail(e, "cudaMalloc(results f32)");
            if ((e = cudaMalloc(&d_src, need)) != cudaSuccess) return bail(e, "cudaMalloc(staging)");
            if ((e = cudaMalloc(&d_bad, sizeof bad)) != cudaSuccess) {
                cudaFree(d_src);
                return bail(e, "cudaMalloc(flag)");
            }
            e = cudaMemcpy(d_src, data, need, cudaMemcpyHostToDevice);
            if (e == cudaSuccess) e = cudaMemcpy(d_bad, &bad, sizeof bad, cudaMemcpyHostToDevice);
            if (e == cudaSuccess) {
                const size_t nb = rows * m->blocks * kBlockBytes, ns = rows * (cols / 64);
                q2_0_to_planar_kernel<<<static_cast<int>(std::min<size_t>((nb + 255) / 256, 148 * 16)), 256>>>(d_src, m->d_planar, rows, cols, m->blocks, d_bad);
                q2_0_scales_kernel<<<static_cast<int>(std::min<size_t>((ns + 255) / 256, 148 * 16)), 256>>>(d_src, m->d_wscales, ns);
                g_launches += 2;
                e = cudaGetLastError();
            }
            if (e == cudaSuccess) e = cudaMemcpy(&bad, d_bad, sizeof bad, cudaMemcpyDeviceToHost);
            cudaFree(d_src);
            cudaFree(d_bad);
            if (e != cudaSuccess) return bail(e, "Q2_0 transcode");
            if (bad != ~0ull) {
                destroy_matrix(m);
                return fail(QUINTRIT_ERR_FORMAT, "Q2_0 weight %llu uses code 3 (+2), which is not ternary", bad);
            }
            QTB_CUDA(block_scaled_allow_smem());
            *out_matrix = m;
            return ok();
        }
        if ((e = cudaMalloc(&m->d_w, m->w_bytes)) != cudaSuccess) return bail(e, "cudaMalloc(weights)");
        if ((e = cudaMalloc(&d_src, need)) != cudaSuccess) return bail(e, "cudaMalloc(staging)");
        if ((e = cudaMemcpy(d_src, data, need, cudaMemcpyHostToDevice)) != cudaSuccess) {
            cudaFree(d_src);
            return bail(e, "cudaMemcpy(source)");
        }
        const size_t n16 = m->blocks * m->tiles * 64;
        const int grid = static_cast<int>(std::min<size_t>((n16 + 255) / 256, 148 * 16));
        switch (source) {
            case kSrcPlanar: to_stream_kernel<kSrcPlanar><<<grid, 256>>>(d_src, m->d_w, rows, cols, m->blocks, m->tiles); break;
            case kSrcI2S: to_stream_kernel<kSrcI2S><<<grid, 256>>>(d_src, m->d_w, rows, cols, m->blocks, m->tiles); break;
            case kSrcTq2: to_stream_kernel<kSrcTq2><<<grid, 256>>>(d_src, m->d_w, rows, cols, m->blocks, m->tiles); break;
            default: to_stream_kernel<kSrcTq1><<<grid, 256>>>(d_src, m->d_w, rows, cols, m->blocks, m->tiles); break;
        }
        ++g_launches;
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        cudaFree(d_src);
        if (e != cudaSuccess) return bail(e, "transcode kernel");

        // launch state for single-matrix calls: enough items to occupy every CTA slot, but no item below 16 tiles
        std::vector<GemvItem> items;
        const size_t pairs = (m->blocks + 1) / 2, slots = static_cast<size_t>(m->sm_count) * kCtasPerSm;
        size_t tiles_per_item = item_tiles_override();
        if (tiles_per_item == 0) {
            const size_t chunks = std::max<size_t>(1, (slots + pairs - 1) / pairs);
            tiles_per_item = std::max<size_t>(16, (m->tiles + chunks - 1) / chunks);
        }
        build_items(items, m->d_w, 0, 0, rows, cols, m->blocks, m->tiles, tiles_per_item);
        m->n_items = static_cast<int>(items.size());
        if ((e = cudaMalloc(&m->d_items, items.size() * sizeof(GemvItem))) != cudaSuccess) return bail(e, "cudaMalloc(items)");
        if ((e = cudaMalloc(&m->d_counters, 4 * sizeof(unsigned int))) != cudaSuccess) return bail(e, "cudaMalloc(counters)");
        if ((e = cudaMalloc(&m->d_act, (cols + 15) / 16 * 16)) != cudaSuccess) return bail(e, "cudaMalloc(activations)");
        if ((e = cudaMalloc(&m->d_out, rows * sizeof(int32_t))) != cudaSuccess) return bail(e, "cudaMalloc(results)");
        if ((e = cudaMalloc(&m->d_outf, rows * sizeof(float))) != cudaSuccess) return bail(e, "cudaMalloc(results f32)");
        if ((e = cudaMemcpy(m->d_items, items.data(), items.size() * sizeof(GemvItem), cudaMemcpyHostToDevice)) != cudaSuccess) return bail(e, "cudaMemcpy(items)");
        if ((e = cudaMemset(m->d_counters, 0, 4 * sizeof(unsigned int))) != cudaSuccess) return bail(e, "cudaMemset(counters)");
        *out_matrix = m;
        return ok();
    });
}

extern "C" int quintrit_b200_matrix_free(quintrit_b200_matrix_t* matrix) {
    return guard([&]() -> int {
        if (matrix == nullptr) return ok();
        int rc = check_matrix(matrix, true);
        if (rc != QUINTRIT_OK) return rc;
        destroy_matrix(matrix);
        return ok();
    });
}

extern "C" int quintrit_b200_matrix_info(const quintrit_b200_matrix_t* matrix, size_t* out_rows, size_t* out_cols, size_t* out_device_bytes) {
    return guard([&]() -> int {
        int rc = check_matrix(matrix, true);
        if (rc != QUINTRIT_OK) return rc;
        if (out_rows) *out_rows = matrix->rows;
        if (out_cols) *out_cols = matrix->cols;
        if (out_device_bytes) *out_device_bytes = matrix->w_bytes;
        return ok();
    });
}

extern "C" int quintrit_b200_matrix_download_planar(const quintrit_b200_matrix_t* matrix, uint8_t* out, size_t out_capacity) {
    return guard([&]() -> int {
        int rc = check_matrix(matrix, true);
        if (rc != QUINTRIT_OK) return rc;
        if (out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out is NULL");
        const size_t need = matrix->rows * matrix->blocks * kBlockBytes;
        if (out_capacity < need) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out holds %zu bytes, %zu are needed", out_capacity, need);
        DeviceGuard g(matrix->device);
        if (matrix->block_scaled) {
            QTB_CUDA(cudaMemcpy(out, matrix->d_planar, need, cudaMemcpyDeviceToHost));
            return ok();
        }
        uint8_t* d_planar = nullptr;
        QTB_CUDA(cudaMalloc(&d_planar, need));
        const int grid = static_cast<int>(std::min<size_t>((need + 255) / 256, 148 * 16));
        stream_to_planar_kernel<<<grid, 256>>>(reinterpret_cast<const uint8_t*>(matrix->d_w), d_planar, matrix->rows, matrix->blocks, matrix->tiles);
        ++g_launches;
        cudaError_t e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaMemcpy(out, d_planar, need, cudaMemcpyDeviceToHost);
        cudaFree(d_planar);
        if (e != cudaSuccess) return cuda_fail(e, "download");
        return ok();
    });
}

// ---------------------------------------------------------------------------------------------------------------------
// GEMV
// ---------------------------------------------------------------------------------------------------------------------

extern "C" int quintrit_b200_gemv_i32_device(const quintrit_b200_matrix_t* matrix, const int8_t* d_activations, int32_t* d_out, void* stream) {
    return guard([&]() -> int {
        int rc = check_matrix(matrix);
        if (rc != QUINTRIT_OK) return rc;
        if (d_activations == nullptr || d_out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "a device pointer is NULL");
        DeviceGuard g(matrix->device);
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        QTB_CUDA(cudaMemsetAsync(d_out, 0, matrix->rows * sizeof(int32_t), s));
        rc = launch_gemv(matrix->d_items, matrix->n_items, d_activations, d_out, matrix->d_counters, matrix->sm_count, s);
        return rc == QUINTRIT_OK ? ok() : rc;
    });
}

namespace {
int gemv_host(const quintrit_b200_matrix* m, const int8_t* act, size_t act_len, void* out, size_t out_cap, bool as_float, float scale) {
    int rc = check_matrix(m);
    if (rc != QUINTRIT_OK) return rc;
    if (act == nullptr || out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "activations or out is NULL");
    if (act_len < m->cols) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "activations hold %zu values, the matrix has %zu columns", act_len, m->cols);
    if (out_cap < m->rows) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out holds %zu values, the matrix has %zu rows", out_cap, m->rows);
    DeviceGuard g(m->device);
    QTB_CUDA(cudaMemcpyAsync(m->d_act, act, m->cols, cudaMemcpyHostToDevice, 0));
    QTB_CUDA(cudaMemsetAsync(m->d_out, 0, m->rows * sizeof(int32_t), 0));
    rc = launch_gemv(m->d_items, m->n_items, m->d_act, m->d_out, m->d_counters, m->sm_count, 0);
    if (rc != QUINTRIT_OK) return rc;
    if (as_float) {
        scale_kernel<<<static_cast<unsigned>((m->rows + 255) / 256), 256>>>(m->d_out, m->d_outf, m->rows, scale);
        ++g_launches;
        QTB_CUDA(cudaGetLastError());
        QTB_CUDA(cudaMemcpyAsync(out, m->d_outf, m->rows * sizeof(float), cudaMemcpyDeviceToHost, 0));
    } else {
        QTB_CUDA(cudaMemcpyAsync(out, m->d_out, m->rows * sizeof(int32_t), cudaMemcpyDeviceToHost, 0));
    }
    QTB_CUDA(cudaStreamSynchronize(0));
    rc = check_kernel_status(m->d_counters);
    return rc == QUINTRIT_OK ? ok() : rc;
}
}  // namespace

extern "C" int quintrit_b200_gemv_i32(const quintrit_b200_matrix_t* matrix, const int8_t* activations, size_t activations_len, int32_t* out,
                                      size_t out_capacity) {
    return guard([&]() -> int { return gemv_host(matrix, activations, activations_len, out, out_capacity, false, 1.0f); });
}

extern "C" int quintrit_b200_gemv_f32(const quintrit_b200_matrix_t* matrix, const int8_t* activations, size_t activations_len, float scale,
                                      float* out, size_t out_capacity) {
    return guard([&]() -> int { return gemv_host(matrix, activations, activations_len, out, out_capacity, true, scale); });
}

// ---------------------------------------------------------------------------------------------------------------------
// block-scaled (Q2_0 x Q8_0) projection
// ---------------------------------------------------------------------------------------------------------------------

namespace {
int check_block_scaled(const quintrit_b200_matrix* m) {
    int rc = check_matrix(m, true);
    if (rc != QUINTRIT_OK) return rc;
    if (!m->block_scaled) return fail(QUINTRIT_ERR_UNSUPPORTED, "the matrix was not uploaded from a Q2_0 payload: it has no block scales");
    return QUINTRIT_OK;
}
int launch_block_scaled(const quintrit_b200_matrix* m) {
    block_scaled_launch(bs_one_matrix(m->d_planar, m->d_wscales, m->rows, m->d_outf), m->d_act, m->d_as, m->cols, m->sm_count, nullptr);
    ++g_launches;
    QTB_CUDA(cudaGetLastError());
    return QUINTRIT_OK;
}
}  // namespace

extern "C" int quintrit_b200_matrix_scales(const quintrit_b200_matrix_t* matrix, float* out, size_t out_capacity) {
    return guard([&]() -> int {
        int rc = check_block_scaled(matrix);
        if (rc != QUINTRIT_OK) return rc;
        if (out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out is NULL");
        const size_t need = matrix->rows * (matrix->cols / 64);
        if (out_capacity < need) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out holds %zu values, %zu are needed", out_capacity, need);
        DeviceGuard g(matrix->device);
        QTB_CUDA(cudaMemcpy(out, matrix->d_wscales, need * sizeof(float), cudaMemcpyDeviceToHost));
        return ok();
    });
}

extern "C" int quintrit_b200_quantize_q8_0(uint32_t device_index, const float* x, size_t n, int8_t* out_codes, float* out_scales) {
    return guard([&]() -> int {
        if (x == nullptr || out_codes == nullptr || out_scales == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "a pointer is NULL");
        if (n == 0 || n % 32 != 0) return fail(QUINTRIT_ERR_INVALID_SHAPE, "Q8_0 quantization needs whole blocks of 32 values, got %zu", n);
        cudaDeviceProp prop;
        int rc = require_b200(static_cast<int>(device_index), &prop);
        if (rc != QUINTRIT_OK) return rc;
        DeviceGuard g(static_cast<int>(device_index));
        float *d_x = nullptr, *d_d = nullptr;
        int8_t* d_q = nullptr;
        cudaError_t e = cudaMalloc(&d_x, n * sizeof(float));
        if (e == cudaSuccess) e = cudaMalloc(&d_d, n / 32 * sizeof(float));
        if (e == cudaSuccess) e = cudaMalloc(&d_q, n);
        if (e == cudaSuccess) e = cudaMemcpy(d_x, x, n * sizeof(float), cudaMemcpyHostToDevice);
        if (e == cudaSuccess) {
            quantize_q8_0_kernel<<<static_cast<int>(std::min<size_t>((n / 32 + 7) / 8, 148 * 8)), 256>>>(d_x, n, d_q, d_d);
            ++g_launches;
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaMemcpy(out_codes, d_q, n, cudaMemcpyDeviceToHost);
        if (e == cudaSuccess) e = cudaMemcpy(out_scales, d_d, n / 32 * sizeof(float), cudaMemcpyDeviceToHost);
        cudaFree(d_x);
        cudaFree(d_d);
        cudaFree(d_q);
        if (e != cudaSuccess) return cuda_fail(e, "quantize_q8_0");
        return ok();
    });
}

extern "C" int quintrit_b200_gemv_block_scaled(const quintrit_b200_matrix_t* matrix, const float* x, size_t x_len, float* out, size_t out_capacity) {
    return guard([&]() -> int {
        int rc = check_block_scaled(matrix);
        if (rc != QUINTRIT_OK) return rc;
        if (x == nullptr || out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "a pointer is NULL");
        if (x_len != matrix->cols) return fail(QUINTRIT_ERR_INVALID_SHAPE, "%zu activations for %zu columns", x_len, matrix->cols);
        if (out_capacity < matrix->rows) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out holds %zu values, %zu are needed", out_capacity, matrix->rows);
        DeviceGuard g(matrix->device);
        QTB_CUDA(cudaMemcpy(matrix->d_x, x, x_len * sizeof(float), cudaMemcpyHostToDevice));
        quantize_q8_0_kernel<<<static_cast<int>(std::min<size_t>((x_len / 32 + 7) / 8, 148 * 8)), 256>>>(matrix->d_x, x_len, matrix->d_act, matrix->d_as);
        ++g_launches;
        QTB_CUDA(cudaGetLastError());
        if ((rc = launch_block_scaled(matrix)) != QUINTRIT_OK) return rc;
        QTB_CUDA(cudaMemcpy(out, matrix->d_outf, matrix->rows * sizeof(float), cudaMemcpyDeviceToHost));
        return ok();
    });
}

extern "C" int quintrit_b200_gemv_block_scaled_q8(const quintrit_b200_matrix_t* matrix, const int8_t* codes, size_t codes_len, const float* scales,
                                                  size_t scales_len, float* out, size_t out_capacity) {
    return guard([&]() -> int {
        int rc = check_block_scaled(matrix);
        if (rc != QUINTRIT_OK) return rc;
        if (codes == nullptr || scales == nullptr || out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "a pointer is NULL");
        if (codes_len != matrix->cols) return fail(QUINTRIT_ERR_INVALID_SHAPE, "%zu activation codes for %zu columns", codes_len, matrix->cols);
        if (scales_len != matrix->cols / 32) return fail(QUINTRIT_ERR_INVALID_SHAPE, "%zu activation scales, %zu are needed", scales_len, matrix->cols / 32);
        if (out_capacity < matrix->rows) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out holds %zu values, %zu are needed", out_capacity, matrix->rows);
        DeviceGuard g(matrix->device);
        QTB_CUDA(cudaMemcpy(matrix->d_act, codes, codes_len, cudaMemcpyHostToDevice));
        QTB_CUDA(cudaMemcpy(matrix->d_as, scales, scales_len * sizeof(float), cudaMemcpyHostToDevice));
        if ((rc = launch_block_scaled(matrix)) != QUINTRIT_OK) return rc;
        QTB_CUDA(cudaMemcpy(out, matrix->d_outf, matrix->rows * sizeof(float), cudaMemcpyDeviceToHost));
        return ok();
    });
}

// ---------------------------------------------------------------------------------------------------------------------
// plans
// ---------------------------------------------------------------------------------------------------------------------

namespace {
void destroy_plan(quintrit_b200_plan* p) {
    if (p == nullptr) return;
    DeviceGuard g(p->device);
    for (auto& sg : p->segments) {
        if (sg.up) cudaEventDestroy(sg.up);
        if (sg.done) cudaEventDestroy(sg.done);
    }
    if (p->s_run) cudaStreamDestroy(p->s_run);
    if (p->s_copy) cudaStreamDestroy(p->s_copy);
    cudaFree(p->d_items);
    cudaFree(p->d_counters);
    cudaFree(p->d_act);
    cudaFree(p->d_out);
    p->magic = 0;
    delete p;
}
}  // namespace

extern "C" int quintrit_b200_plan_create(const quintrit_b200_matrix_t* const* matrices, size_t count, quintrit_b200_plan_t** out_plan) {
    return guard([&]() -> int {
        if (out_plan == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_plan is NULL");
        *out_plan = nullptr;
        if (matrices == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "matrices is NULL");
        if (count == 0 || count > (1u << 20)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "a plan needs between 1 and 2^20 matrices");
        for (size_t i = 0; i < count; ++i) {
            int rc = check_matrix(matrices[i]);
            if (rc != QUINTRIT_OK) return rc;
            if (matrices[i]->device != matrices[0]->device) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "matrix %zu lives on another device", i);
        }
        quintrit_b200_plan* p = new quintrit_b200_plan();
        p->magic = kMagicPlan;
        p->device = matrices[0]->device;
        p->sm_count = matrices[0]->sm_count;
        p->count = count;
        DeviceGuard g(p->device);
        std::vector<GemvItem> items;
        size_t act = 0, out = 0;
        size_t tiles_per_item = item_tiles_override();
        if (tiles_per_item == 0) {
            // Measured on the 280 projections of the Falcon3-10B shape: items of 48 and 64 row tiles 21 300, 96 tiles 22 360, 128 tiles 22 130, 192 tiles
            // 22 070 Gweights/s (fewer table builds against a longer tail). A small plan keeps 64, so that every CTA slot still gets several items.
            size_t pair_tiles = 0;
            for (size_t i = 0; i < count; ++i) pair_tiles += (matrices[i]->blocks + 1) / 2 * matrices[i]->tiles;
            tiles_per_item = pair_tiles / 96 >= size_t(8) * p->sm_count * kCtasPerSm ? 96 : 64;
        }
        std::vector<size_t> item_at(count + 1), weights_before(count + 1);
        size_t weights = 0;
        for (size_t i = 0; i < count; ++i) {
            const quintrit_b200_matrix* m = matrices[i];
            item_at[i] = items.size(), weights_before[i] = weights;
            p->act_off.push_back(act);
            p->out_off.push_back(out);
            p->rows.push_back(m->rows);
            p->cols.push_back(m->cols);
            build_items(items, m->d_w, act, out, m->rows, m->cols, m->blocks, m->tiles, tiles_per_item);
            act += (m->cols + 15) / 16 * 16;
            out += (m->rows + 3) / 4 * 4;
            weights += m->rows * m->cols;
        }
        item_at[count] = items.size(), weights_before[count] = weights;
        p->act_total = act;
        p->out_total = out;
        p->n_items = static_cast<int>(items.size());
        {
            // segments of about equal weight counts, cut between matrices; small plans run as one
            int want = 1;
            if (const char* v = std::getenv("QUINTRIT_B200_PLAN_SEGMENTS")) want = std::max(1, std::min(16, std::atoi(v)));
            else if (count >= 16 && weights >= (size_t(1) << 30)) want = 4;
            size_t first = 0;
            for (int sgi = 0; sgi < want && first < count; ++sgi) {
                size_t last = count;  // exclusive
                if (sgi + 1 < want) {
                    const size_t target = weights * (sgi + 1) / want;
                    last = first + 1;
                    while (last < count && weights_before[last] < target) ++last;
                }
                quintrit_b200_plan::Segment sg;
                sg.item0 = static_cast<int>(item_at[first]), sg.items = static_cast<int>(item_at[last] - item_at[first]);
                sg.act0 = p->act_off[first], sg.act_bytes = (last < count ? p->act_off[last] : act) - sg.act0;
                sg.out0 = p->out_off[first], sg.out_count = (last < count ? p->out_off[last] : out) - sg.out0;
                p->segments.push_back(sg);
                first = last;
            }
        }
        auto bail = [&](cudaError_t e, const char* what) {
            destroy_plan(p);
            return cuda_fail(e, what);
        };
        cudaError_t e;
        if ((e = cudaMalloc(&p->d_items, items.size() * sizeof(GemvItem))) != cudaSuccess) return bail(e, "cudaMalloc(items)");
        if ((e = cudaMalloc(&p->d_counters, 4 * sizeof(unsigned int))) != cudaSuccess) return bail(e, "cudaMalloc(counters)");
        if ((e = cudaMalloc(&p->d_act, act)) != cudaSuccess) return bail(e, "cudaMalloc(activations)");
        if ((e = cudaMalloc(&p->d_out, out * sizeof(int32_t))) != cudaSuccess) return bail(e, "cudaMalloc(results)");
        if ((e = cudaMemcpy(p->d_items, items.data(), items.size() * sizeof(GemvItem), cudaMemcpyHostToDevice)) != cudaSuccess) return bail(e, "cudaMemcpy(items)");
        if ((e = cudaMemset(p->d_counters, 0, 4 * sizeof(unsigned int))) != cudaSuccess) return bail(e, "cudaMemset(counters)");
        if ((e = cudaMemset(p->d_act, 0, act)) != cudaSuccess) return bail(e, "cudaMemset(activations)");
        if ((e = cudaStreamCreateWithFlags(&p->s_run, cudaStreamNonBlocking)) != cudaSuccess) return bail(e, "cudaStreamCreate");
        if ((e = cudaStreamCreateWithFlags(&p->s_copy, cudaStreamNonBlocking)) != cudaSuccess) return bail(e, "cudaStreamCreate");
        for (auto& sg : p->segments)
            if ((e = cudaEventCreateWithFlags(&sg.up, cudaEventDisableTiming)) != cudaSuccess || (e = cudaEventCreateWithFlags(&sg.done, cudaEventDisableTiming)) != cudaSuccess)
                return bail(e, "cudaEventCreate");
        *out_plan = p;
        return ok();
    });
}

extern "C" int quintrit_b200_plan_free(quintrit_b200_plan_t* plan) {
    return guard([&]() -> int {
        if (plan == nullptr) return ok();
        int rc = check_plan(plan);
        if (rc != QUINTRIT_OK) return rc;
        destroy_plan(plan);
        return ok();
    });
}

extern "C" int quintrit_b200_plan_layout(const quintrit_b200_plan_t* plan, size_t index, size_t* out_act_offset, size_t* out_out_offset,
                                         size_t* out_act_total, size_t* out_out_total) {
    return guard([&]() -> int {
        int rc = check_plan(plan);
        if (rc != QUINTRIT_OK) return rc;
        if (index >= plan->count) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "problem %zu does not exist (%zu problems)", index, plan->count);
        if (out_act_offset) *out_act_offset = plan->act_off[index];
        if (out_out_offset) *out_out_offset = plan->out_off[index];
        if (out_act_total) *out_act_total = plan->act_total;
        if (out_out_total) *out_out_total = plan->out_total;
        return ok();
    });
}

extern "C" int quintrit_b200_plan_buffers(const quintrit_b200_plan_t* plan, int8_t** out_d_activations, int32_t** out_d_results) {
    return guard([&]() -> int {
        int rc = check_plan(plan);
        if (rc != QUINTRIT_OK) return rc;
        if (out_d_activations) *out_d_activations = plan->d_act;
        if (out_d_results) *out_d_results = plan->d_out;
        return ok();
    });
}

extern "C" int quintrit_b200_plan_launch(quintrit_b200_plan_t* plan, void* stream) {
    return guard([&]() -> int {
        int rc = check_plan(plan);
        if (rc != QUINTRIT_OK) return rc;
        DeviceGuard g(plan->device);
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        QTB_CUDA(cudaMemsetAsync(plan->d_out, 0, plan->out_total * sizeof(int32_t), s));
        rc = launch_gemv(plan->d_items, plan->n_items, plan->d_act, plan->d_out, plan->d_counters, plan->sm_count, s);
        return rc == QUINTRIT_OK ? ok() : rc;
    });
}

extern "C" int quintrit_b200_plan_run(quintrit_b200_plan_t* plan, const int8_t* activations, size_t activations_len, int32_t* out,
                                      size_t out_capacity) {
    return guard([&]() -> int {
        int rc = check_plan(plan);
        if (rc != QUINTRIT_OK) return rc;
        if (activations == nullptr || out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "activations or out is NULL");
        if (activations_len < plan->act_total) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "activations hold %zu bytes, %zu are needed", activations_len, plan->act_total);
        if (out_capacity < plan->out_total) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out holds %zu values, %zu are needed", out_capacity, plan->out_total);
        DeviceGuard g(plan->device);
        // Segment by segment: the copy stream brings the activations up (all of them, in segment order) and takes each segment's results down as
        // soon as its kernel is done; the run stream clears the results and runs the kernels. With pinned host buffers the copies of one segment
        // overlap the kernel of another; with pageable ones the runtime serialises them and the result is the same.
        QTB_CUDA(cudaDeviceSynchronize());  // launches the caller made on streams of its own (plan_launch) use the same buffers: they come first
        QTB_CUDA(cudaMemsetAsync(plan->d_out, 0, plan->out_total * sizeof(int32_t), plan->s_run));
        for (auto& sg : plan->segments) {
            QTB_CUDA(cudaMemcpyAsync(plan->d_act + sg.act0, activations + sg.act0, sg.act_bytes, cudaMemcpyHostToDevice, plan->s_copy));
            QTB_CUDA(cudaEventRecord(sg.up, plan->s_copy));
        }
        for (auto& sg : plan->segments) {
            QTB_CUDA(cudaStreamWaitEvent(plan->s_run, sg.up, 0));
            rc = launch_gemv(plan->d_items + sg.item0, sg.items, plan->d_act, plan->d_out, plan->d_counters, plan->sm_count, plan->s_run);
            if (rc != QUINTRIT_OK) return rc;
            QTB_CUDA(cudaEventRecord(sg.done, plan->s_run));
            QTB_CUDA(cudaStreamWaitEvent(plan->s_copy, sg.done, 0));
            QTB_CUDA(cudaMemcpyAsync(out + sg.out0, plan->d_out + sg.out0, sg.out_count * sizeof(int32_t), cudaMemcpyDeviceToHost, plan->s_copy));
        }
        unsigned int flag = 0;
        QTB_CUDA(cudaMemcpyAsync(&flag, plan->d_counters + 2, sizeof flag, cudaMemcpyDeviceToHost, plan->s_copy));
        QTB_CUDA(cudaStreamSynchronize(plan->s_copy));
        QTB_CUDA(cudaStreamSynchronize(plan->s_run));
        if (flag != 0) return fail(QUINTRIT_ERR_DEVICE, "GEMV kernel on the CUDA device found its shared-memory table at an unexpected address");
        return ok();
    });
}

extern "C" uint64_t quintrit_b200_launch_count(int reset) {
    const uint64_t n = g_launches;
    if (reset) g_launches = 0;
    return n;
}

// ---------------------------------------------------------------------------------------------------------------------
// decoder
// ---------------------------------------------------------------------------------------------------------------------

namespace {

// Tiles per item for a launch over `tile_pairs` (sum over its problems of row tiles x block pairs): enough items to give
// every CTA slot one, but no item below 8 row tiles (a table build costs about as much as streaming 8 tiles).
size_t decoder_item_tiles(size_t tile_pairs, size_t slots) {
    const size_t override = item_tiles_override();
    if (override) return override;
    return std::max<size_t>(8, (tile_pairs + slots - 1) / slots);
}

int mega_setup(quintrit_b200_decoder* d, const quintrit_b200_decoder_desc_t* desc);

// The table of device_expf on the current device: glibc's 2^(i/32), correctly rounded (the host libm's exp2), minus i << 47.
int upload_exp2_table() {
    unsigned long long tab[32];
    for (int i = 0; i < 32; ++i) {
        const double v = std::exp2(static_cast<double>(i) / 32.0);
        unsigned long long b;
        std::memcpy(&b, &v, 8);
        tab[i] = b - (static_cast<unsigned long long>(i) << 47);
    }
    QTB_CUDA(cudaMemcpyToSymbol(c_exp2_tab, tab, sizeof tab));
    return QUINTRIT_OK;
}

// Lets a kernel use all the shared memory the device offers a block beyond the kernel's own static arrays.
template <typename K>
int allow_max_dynamic_smem(K kernel, int smem_optin) {
    cudaFuncAttributes fa{};
    QTB_CUDA(cudaFuncGetAttributes(&fa, kernel));
    QTB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin - static_cast<int>(fa.sharedSizeBytes)));
    return QUINTRIT_OK;
}

int decoder_create_impl(const quintrit_b200_decoder_desc_t* desc, quintrit_b200_decoder** out) {
    if (desc->struct_size < sizeof(quintrit_b200_decoder_desc_t))
        return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "struct_size %u is smaller than quintrit_b200_decoder_desc_t (%zu)", desc->struct_size,
                    sizeof(quintrit_b200_decoder_desc_t));
    if (!desc->embed || !desc->output_norm || !desc->matrices || !desc->scales || !desc->norms)
        return fail(QUINTRIT_ERR_NULL_POINTER, "a required pointer of the decoder description is NULL");
    if (desc->arch != QUINTRIT_B200_ARCH_LLAMA && desc->arch != QUINTRIT_B200_ARCH_BITNET && desc->arch != QUINTRIT_B200_ARCH_QWEN)
        return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "unknown architecture %d", desc->arch);
    // tensor parallelism: the fields exist only in descriptions of the newer size
    uint32_t tp_rank = 0, tp_world = 1;
    if (desc->struct_size >= offsetof(quintrit_b200_decoder_desc_t, tp_world) + sizeof(uint32_t) && desc->tp_world != 0) {
        tp_rank = desc->tp_rank, tp_world = desc->tp_world;
    }
    if (tp_world != 1 && tp_world != 2 && tp_world != 4 && tp_world != 8) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "tp_world %u must be 1, 2, 4 or 8", tp_world);
    if (tp_rank >= tp_world) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "tp_rank %u is not below tp_world %u", tp_rank, tp_world);
    uint32_t table_dtype = 0;
    if (desc->struct_size >= offsetof(quintrit_b200_decoder_desc_t, table_dtype) + sizeof(uint32_t)) table_dtype = desc->table_dtype;
    if (table_dtype > 1) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "table_dtype %u is not 0 (F16) or 1 (BF16)", table_dtype);
    const uint32_t H = desc->hidden_size, I_full = desc->intermediate_size, L = desc->num_layers, hd = desc->head_dim;
    if (!H || !I_full || !L || !desc->num_heads || !desc->num_kv_heads || !hd || !desc->vocab_size)
        return fail(QUINTRIT_ERR_MODEL, "a model dimension is zero");
    if (tp_world > 1) {
        if (desc->arch != QUINTRIT_B200_ARCH_LLAMA) return fail(QUINTRIT_ERR_UNSUPPORTED, "tensor parallelism is available for the LLaMA / Falcon3 architecture only");
        if (H % tp_world || I_full % tp_world || desc->vocab_size % tp_world)
            return fail(QUINTRIT_ERR_UNSUPPORTED, "tp_world %u must divide the hidden size, the FFN size and the vocabulary", tp_world);
    }
    // Where the ranks do not divide the KV heads (Falcon3's 4 KV heads on 8 GPUs) attention is replicated: every rank holds the whole q, k and v
    // projections and the whole KV cache and computes every head, so the attention output needs no exchange; o, gate, up, down and the output
    // head stay split as before.
    const bool attn_replicated = tp_world > 1 && desc->num_kv_heads % tp_world != 0;
    const uint32_t head_split = attn_replicated ? 1u : tp_world;
    const uint32_t I = I_full / tp_world;  // this rank's rows of gate and up
    if (hd % 32 != 0 || hd > 256) return fail(QUINTRIT_ERR_UNSUPPORTED, "head_dim %u is not supported (a multiple of 32, at most 256)", hd);
    if (H % 32 != 0) return fail(QUINTRIT_ERR_UNSUPPORTED, "the hidden size %u must be a multiple of 32", H);  // as gpu.rs:171-173
    if (desc->num_heads % desc->num_kv_heads != 0) return fail(QUINTRIT_ERR_MODEL, "num_heads is not a multiple of num_kv_heads");
    if (desc->rope_dims == 0 || desc->rope_dims % 2 != 0 || desc->rope_dims > hd)
        return fail(QUINTRIT_ERR_MODEL, "rope_dims %u must be even and at most the head dimension %u", desc->rope_dims, hd);
    // gpu.rs:141-146: rounded down to a multiple of 256 from 256 on; a smaller window is kept as it is (a multiple of 8 here)
    const uint32_t ctx = desc->context_length >= 256 ? desc->context_length / 256 * 256 : desc->context_length;
    if (ctx == 0 || ctx > 8192 || ctx % 8 != 0)
        return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "context_length %u must be a multiple of 8 below 256, or give 256..8192 after rounding down to a multiple of 256", desc->context_length);
    const size_t qd_full = size_t(desc->num_heads) * hd;
    const size_t qd = qd_full / head_split, kvd = size_t(desc->num_kv_heads) * hd / head_split;  // this rank's query and KV widths
    const uint32_t vocab_local = desc->vocab_size / tp_world;
    if (std::max<size_t>({H, I_full, qd_full}) * sizeof(float) > 200 * 1024) return fail(QUINTRIT_ERR_UNSUPPORTED, "a vector of the model does not fit the shared memory of one block");
    cudaDeviceProp prop;
    int rc = require_b200(static_cast<int>(desc->device_index), &prop);
    if (rc != QUINTRIT_OK) return rc;
    const size_t shapes[7][2] = {{qd, H}, {kvd, H}, {kvd, H}, {H / tp_world, qd_full}, {I, H}, {I, H}, {H / tp_world, I_full}};
    // A model of Q2_0 projections: every matrix is block-scaled (attention.rs:262-344, model.rs:209-229); mixtures are refused.
    bool block_scaled = false;
    if (desc->matrices[0] != nullptr && check_matrix(desc->matrices[0], true) == QUINTRIT_OK) block_scaled = desc->matrices[0]->block_scaled;
    if (block_scaled && tp_world > 1) return fail(QUINTRIT_ERR_UNSUPPORTED, "tensor parallelism is not available for block-scaled (Q2_0) models");
    for (size_t i = 0; i < size_t(L) * 7; ++i) {
        const quintrit_b200_matrix* m = desc->matrices[i];
        rc = check_matrix(m, true);
        if (rc != QUINTRIT_OK) return rc;
        if (m->block_scaled != block_scaled) return fail(QUINTRIT_ERR_UNSUPPORTED, "matrix %zu: block-scaled (Q2_0) and per-tensor projections cannot be mixed in one model", i);
        if (m->device != static_cast<int>(desc->device_index)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "matrix %zu lives on another device", i);
        if (m->rows != shapes[i % 7][0] || m->cols != shapes[i % 7][1])
            return fail(QUINTRIT_ERR_MODEL, "matrix %zu is %zu x %zu, the model needs %zu x %zu", i, m->rows, m->cols, shapes[i % 7][0], shapes[i % 7][1]);
    }
    DeviceGuard guard(static_cast<int>(desc->device_index));
    quintrit_b200_decoder* d = new quintrit_b200_decoder();
    *out = d;  // the caller destroys it on failure
    d->magic = kMagicDecoder;
    d->device = static_cast<int>(desc->device_index);
    d->sm_count = prop.multiProcessorCount;
    d->arch = desc->arch, d->f32_values = desc->f32_values != 0;
    d->hidden = H, d->inter = I, d->layers = L, d->q_heads = desc->num_heads / head_split, d->kv_heads = desc->num_kv_heads / head_split, d->head_dim = hd;
    d->attn_replicated = attn_replicated;
    d->tp_rank = static_cast<int>(tp_rank), d->tp_world = static_cast<int>(tp_world);
    d->bf16_tables = table_dtype == 1;
    const float* const* qk_norms = nullptr;
    if (desc->struct_size >= offsetof(quintrit_b200_decoder_desc_t, qk_norms) + sizeof(void*)) qk_norms = desc->qk_norms;
    if (qk_norms != nullptr) {
        if (!block_scaled) return fail(QUINTRIT_ERR_UNSUPPORTED, "query/key-norm is available for block-scaled (Q2_0) models only, as in the reference");
        d->qk_norms.assign(size_t(L) * 2, nullptr);
        for (size_t i = 0; i < size_t(L) * 2; ++i) {
            if (qk_norms[i] == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "qk_norms[%zu] is NULL", i);
            if ((rc = dev_upload(d, &d->qk_norms[i], qk_norms[i], hd)) != QUINTRIT_OK) return rc;
        }
    }
    d->block_scaled = block_scaled;
    d->mats.assign(desc->matrices, desc->matrices + size_t(L) * 7);
    d->q_dim_full = static_cast<int>(qd_full), d->inter_full = static_cast<int>(I_full), d->vocab_full = static_cast<int>(desc->vocab_size);
    d->vocab = vocab_local, d->ctx = ctx, d->rope_dims = desc->rope_dims, d->q_dim = static_cast<int>(qd), d->kv_dim = static_cast<int>(kvd);
    d->eps = desc->rms_norm_eps, d->rope_theta = desc->rope_theta;
    d->scales.assign(desc->scales, desc->scales + size_t(L) * 7);
    d->graph_ready = false;
    d->stream = nullptr;
    d->host_pos = 0;
    QTB_CUDA(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));

    if ((rc = upload_exp2_table()) != QUINTRIT_OK) return rc;
    // cos / sin of every position with the host libm, chained as ops.rs:121-141 (freq_scale 1, no YaRN)
    {
        std::vector<float> cs(size_t(ctx) * desc->rope_dims);
        const float theta_scale = std::pow(desc->rope_theta, -2.0f / static_cast<float>(desc->rope_dims));
        for (uint32_t p = 0; p < ctx; ++p) {
            float theta = static_cast<float>(p);
            for (uint32_t i0 = 0; i0 < desc->rope_dims; i0 += 2) {
                cs[size_t(p) * desc->rope_dims + i0] = std::cos(theta);
                cs[size_t(p) * desc->rope_dims + i0 + 1] = std::sin(theta);
                theta *= theta_scale;
            }
        }
        if ((rc = dev_upload(d, &d->cos_sin, cs.data(), cs.size())) != QUINTRIT_OK) return rc;
    }
    if ((rc = dev_upload(d, &d->embed, desc->embed, size_t(desc->vocab_size) * H)) != QUINTRIT_OK) return rc;
    d->lm_head = d->embed + size_t(tp_rank) * vocab_local * H;  // tied head: this rank's rows of the embedding
    if (desc->lm_head && (rc = dev_upload(d, &d->lm_head, desc->lm_head, size_t(vocab_local) * H)) != QUINTRIT_OK) return rc;
    if ((rc = dev_upload(d, &d->out_norm, desc->output_norm, H)) != QUINTRIT_OK) return rc;
    d->norms.assign(size_t(L) * 4, nullptr);
    for (size_t i = 0; i < size_t(L) * 4; ++i) {
        const size_t n = (i % 4 == 2) ? qd : (i % 4 == 3 ? I : H);
        if (desc->norms[i] == nullptr) {
            if (i % 4 < 2) return fail(QUINTRIT_ERR_NULL_POINTER, "norm weights %zu are NULL", i);
            if (desc->arch == QUINTRIT_B200_ARCH_BITNET) return fail(QUINTRIT_ERR_MODEL, "a BitNet model needs its sub-norm weights (%zu)", i);
            continue;
        }
        if ((rc = dev_upload(d, &d->norms[i], desc->norms[i], n)) != QUINTRIT_OK) return rc;
    }
    const size_t kv_elems = size_t(L) * ctx * kvd;
    if ((rc = dev_alloc(d, &d->kc, kv_elems)) != QUINTRIT_OK) return rc;  // zero-initialised like kv_cache.rs:24-46
    if ((rc = dev_alloc(d, &d->vc, kv_elems)) != QUINTRIT_OK) return rc;
    if ((rc = dev_alloc(d, &d->x, H)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->q, qd)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->x16, H)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->part_acc, size_t(d->q_heads) * 4 * hd)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->part_ms, size_t(d->q_heads) * 8)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->logits, d->vocab)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->a8_h, H + 16)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->a8_q, qd + 16)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->a8_i, I + 16)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->s_h, 4)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->s_q, 4)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->s_i, 4)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->acc_qkv, qd + 2 * kvd)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->acc_o, H)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->acc_gu, 2 * size_t(I))) != QUINTRIT_OK || (rc = dev_alloc(d, &d->acc_down, H)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->d_token, 4)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->d_pos, 4)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->d_history, ctx + 1)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->d_counters, 4)) != QUINTRIT_OK)
        return rc;

    if ((rc = dev_alloc(d, &d->q8_d, std::max<size_t>({H, I, qd}) / 32 + 1)) != QUINTRIT_OK) return rc;
    if (block_scaled) {  // no work items: the block-scaled projections are plain launches; one kernel per step
        QTB_CUDA(block_scaled_allow_smem());
        const int big_bs = static_cast<int>(std::max<size_t>({H, I, qd}) * sizeof(float));
        QTB_CUDA(cudaFuncSetAttribute(norm_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, big_bs));
        QTB_CUDA(cudaFuncSetAttribute(attn_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, big_bs));
        QTB_CUDA(cudaFuncSetAttribute(act_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, big_bs));
        QTB_CUDA(cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, big_bs));
        QTB_CUDA(cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(attention_smem(256))));
        d->use_mega = false;
        QTB_CUDA(cudaDeviceSynchronize());
        return QUINTRIT_OK;
    }
    // work items of the four GEMV launches of every layer
    std::vector<GemvItem> items;
    const size_t slots = size_t(d->sm_count) * kCtasPerSm;
    auto tiles_of = [](const quintrit_b200_matrix* m) { return m->tiles * ((m->blocks + 1) / 2); };
    for (uint32_t l = 0; l < L; ++l) {
        const quintrit_b200_matrix* const* m = desc->matrices + size_t(l) * 7;
        auto begin = [&]() { d->item_first.push_back(static_cast<int>(items.size())); };
        auto end = [&]() { d->item_count.push_back(static_cast<int>(items.size()) - d->item_first.back()); };
        begin();  // q | k | v share the activations and stack their results
        size_t t = decoder_item_tiles(tiles_of(m[0]) + tiles_of(m[1]) + tiles_of(m[2]), slots);
        build_items(items, m[0]->d_w, 0, 0, m[0]->rows, m[0]->cols, m[0]->blocks, m[0]->tiles, t);
        build_items(items, m[1]->d_w, 0, qd, m[1]->rows, m[1]->cols, m[1]->blocks, m[1]->tiles, t);
        build_items(items, m[2]->d_w, 0, qd + kvd, m[2]->rows, m[2]->cols, m[2]->blocks, m[2]->tiles, t);
        end();
        begin();
        build_items(items, m[3]->d_w, 0, 0, m[3]->rows, m[3]->cols, m[3]->blocks, m[3]->tiles, decoder_item_tiles(tiles_of(m[3]), slots));
        end();
        begin();  // gate | up
        t = decoder_item_tiles(tiles_of(m[4]) + tiles_of(m[5]), slots);
        build_items(items, m[4]->d_w, 0, 0, m[4]->rows, m[4]->cols, m[4]->blocks, m[4]->tiles, t);
        build_items(items, m[5]->d_w, 0, I, m[5]->rows, m[5]->cols, m[5]->blocks, m[5]->tiles, t);
        end();
        begin();
        build_items(items, m[6]->d_w, 0, 0, m[6]->rows, m[6]->cols, m[6]->blocks, m[6]->tiles, decoder_item_tiles(tiles_of(m[6]), slots));
        end();
    }
    if ((rc = dev_upload(d, &d->d_items, items.data(), items.size())) != QUINTRIT_OK) return rc;

    // one-time kernel set-up, before any stream capture
    GemvKernel k = nullptr;
    if ((rc = gemv_kernel_for_device(d->device, &k)) != QUINTRIT_OK) return rc;
    // The limit is a property of the kernel, shared by every decoder of the process: it is set to the most the device allows, so that a
    // later, smaller model does not lower it under an earlier, larger one.
    int smem_optin = 0;
    QTB_CUDA(cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, d->device));
    const size_t big = std::max<size_t>({H, I, qd}) * sizeof(float);
    if (big + 1024 > static_cast<size_t>(smem_optin)) return fail(QUINTRIT_ERR_UNSUPPORTED, "a vector of %zu bytes does not fit the shared memory of a multiprocessor (%d bytes)", big, smem_optin);
    if ((rc = allow_max_dynamic_smem(norm_quant_kernel, smem_optin)) != QUINTRIT_OK) return rc;
    if ((rc = allow_max_dynamic_smem(attn_finish_kernel, smem_optin)) != QUINTRIT_OK) return rc;
    if ((rc = allow_max_dynamic_smem(act_quant_kernel, smem_optin)) != QUINTRIT_OK) return rc;
    if ((rc = allow_max_dynamic_smem(lm_head_kernel, smem_optin)) != QUINTRIT_OK) return rc;
    if ((rc = allow_max_dynamic_smem(lm_head_batch_kernel, smem_optin)) != QUINTRIT_OK) return rc;
    if ((rc = allow_max_dynamic_smem(attention_kernel, smem_optin)) != QUINTRIT_OK) return rc;
    // attention for all query heads of a KV head at once, where the group size and the head size allow it
    d->attn_gqa = nullptr, d->attn_gqa_smem = 0;
    if (hd % 32 == 0 && hd <= 256 && std::getenv("QUINTRIT_B200_ATTN_GQA_OFF") == nullptr) {
        const int group = d->q_heads / d->kv_heads;
        AttnGqaKernel kq = attention_gqa_for(group, d->f32_values != 0);
        const size_t bytes = kq != nullptr ? attention_gqa_smem(group, static_cast<int>(hd), d->ctx) : 0;
        if (kq != nullptr && bytes + 1024 <= static_cast<size_t>(smem_optin)) {
            if ((rc = allow_max_dynamic_smem(kq, smem_optin)) != QUINTRIT_OK) return rc;
            d->attn_gqa = kq, d->attn_gqa_smem = bytes;
            if (const char* pad = std::getenv("QUINTRIT_B200_ATTN_SMEM_PAD")) d->attn_gqa_pad = std::min<size_t>(static_cast<size_t>(std::atoi(pad)), smem_optin - 1024 - bytes);
        }
    }
    d->use_mega = false;
    const char* mode = std::getenv("QUINTRIT_B200_DECODE");  // "kernels" keeps the one-launch-per-step path (experiments)
    // the single-kernel path stages KV rows with a piece permutation that needs a power-of-two head_dim of at least 64
    // and one values unit of the longest chunk must fit the shared memory of an SM next to the activation vectors
    const int gqa_n = d->q_heads / d->kv_heads;
    // the second form of the attention's second half (units that take all chunks of 8 coordinates) where its arrays fit
    d->attn_v2 = tp_world == 1 && d->ctx <= static_cast<uint32_t>(kV2MaxCtx) && gqa_n <= kV2MaxGqa && qd_full <= size_t(kNormPer) * kMegaThreads && hd % kV2Dims == 0 &&
                 d->kv_heads * (hd / kV2Dims) < static_cast<uint32_t>(d->sm_count);  // some CTAs must stay free to compute the softmax factors
    if (const char* v2 = std::getenv("QUINTRIT_B200_ATTN_V2")) d->attn_v2 = d->attn_v2 && v2[0] != '0';  // experiments: "0" keeps the first form
    auto bytes_for = [&](bool v2) {
        return mega_smem_bytes(mega_attn_region(d->ctx, gqa_n, hd, v2), static_cast<int>(std::max<size_t>(H, qd_full)), static_cast<int>(H), static_cast<int>(L));
    };
    if (d->attn_v2 && bytes_for(true) > static_cast<size_t>(smem_optin)) d->attn_v2 = false;
    const size_t mega_bytes = bytes_for(d->attn_v2);
    const bool staged_ok = hd >= 64 && (hd & (hd - 1)) == 0 && gqa_n <= 16 && mega_bytes <= static_cast<size_t>(smem_optin);
    if (staged_ok && d->q_heads <= kMegaMaxHeads && !(mode && std::strcmp(mode, "kernels") == 0)) {
        if ((rc = mega_setup(d, desc)) != QUINTRIT_OK) return rc;
        d->use_mega = true;
    }
    if (tp_world > 1 && !d->use_mega) return fail(QUINTRIT_ERR_UNSUPPORTED, "tensor parallelism needs the single-kernel decode path, which does not take this model");
    QTB_CUDA(cudaDeviceSynchronize());
    return QUINTRIT_OK;
}

// Work items of one GEMV phase of the single-kernel path: one round over `ctas` CTAs. The launch's problems share their
// column count; the chunks of row tiles are shared out in proportion to the problems' row tiles.
void mega_phase_items(std::vector<GemvItem>& items, const quintrit_b200_matrix* const* ms, const size_t* out_offs, int n, size_t ctas) {
    const size_t pairs = (ms[0]->blocks + 1) / 2;
    size_t total_tiles = 0;
    for (int i = 0; i < n; ++i) total_tiles += ms[i]->tiles;
    const size_t chunks_total = std::max<size_t>(n, ctas / pairs);
    for (int i = 0; i < n; ++i) {
        size_t chunks = std::max<size_t>(1, chunks_total * ms[i]->tiles / total_tiles);
        chunks = std::min(chunks, ms[i]->tiles);
        const size_t tiles_per_item = (ms[i]->tiles + chunks - 1) / chunks;
        build_items(items, ms[i]->d_w, 0, out_offs[i], ms[i]->rows, ms[i]->cols, ms[i]->blocks, ms[i]->tiles, tiles_per_item);
    }
}

template <uint32_t BASE>
int mega_bind(quintrit_b200_decoder* d) {
    d->mega_kernel = decode_token_kernel<BASE>;
    QTB_CUDA(cudaFuncSetAttribute(decode_token_kernel<BASE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(d->mega_smem)));
    int per_sm = 0;
    QTB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_token_kernel<BASE>, kMegaThreads, d->mega_smem));
    if (per_sm < 1) return fail(QUINTRIT_ERR_DEVICE, "the decode kernel does not fit one CTA per multiprocessor on this CUDA device");
    return QUINTRIT_OK;
}

// Builds the arguments of the single-kernel path (after all buffers exist).
int mega_setup(quintrit_b200_decoder* d, const quintrit_b200_decoder_desc_t* desc) {
    const int L = d->layers, H = d->hidden, I = d->inter, qd = d->q_dim, kvd = d->kv_dim;
    int rc;
    // Tensor parallelism: the vectors every rank needs whole live in one allocation (the "box") that the peers map.
    const auto up256 = [](size_t n) { return (n + 255) / 256 * 256; };
    // pair buffers (8 bytes per value) for the o and down results, the attention output, the partial maxima and the greedy
    // candidates; the SwiGLU output travels as plain floats
    const size_t off_acc_o = 0, off_acc_down = up256(off_acc_o + size_t(H) * 8), off_y = up256(off_acc_down + size_t(H) * 8),
                 off_v = up256(off_y + size_t(d->q_dim_full) * 8), off_amax = up256(off_v + size_t(d->inter_full) * 4), off_best = off_amax + 256,
                 box_bytes = off_best + 256;
    if (d->tp_world > 1) {
        if ((rc = dev_alloc(d, &d->tp_box, box_bytes)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->tp_seq, 4)) != QUINTRIT_OK) return rc;
        d->tp_box_bytes = box_bytes;
    }
    const size_t slice_off = size_t(d->tp_rank) * (H / d->tp_world);  // first row of this rank in the o and down results
    if ((rc = dev_alloc(d, &d->xa, H)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->xb, H)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->v_inter, I)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->amax_bits, 4)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->best_val, d->sm_count)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->best_idx, d->sm_count)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->bar, 16)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->trace, size_t(L) * 14 + 4 + 32 + 2)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->scores, size_t(d->q_heads) * d->ctx)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->attn_out, size_t(qd))) != QUINTRIT_OK)
        return rc;
    const int fac_stride = values2_clp(d->ctx >= 512 ? (d->ctx + 3) / 4 : d->ctx);
    if (d->attn_v2 && ((rc = dev_alloc(d, &d->fac, size_t(2) * d->q_heads * 4 * fac_stride)) != QUINTRIT_OK ||
                       (rc = dev_alloc(d, &d->fac_flags, size_t(d->q_heads) * 4 * (fac_stride / 8))) != QUINTRIT_OK ||
                       (rc = dev_alloc(d, &d->fac_M, size_t(d->q_heads) * 4)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->fac_done, size_t(d->kv_heads))) != QUINTRIT_OK))
        return rc;
    std::vector<GemvItem> items;
    std::vector<MegaLayer> layers(L);
    for (int l = 0; l < L; ++l) {
        const quintrit_b200_matrix* const* m = desc->matrices + size_t(l) * 7;
        MegaLayer& ly = layers[l];
        const size_t o_qkv[3] = {0, size_t(qd), size_t(qd + kvd)}, o_zero[1] = {slice_off}, o_gu[2] = {0, size_t(I)};
        auto phase = [&](int k, const quintrit_b200_matrix* const* ms, const size_t* offs, int n) {
            ly.first[k] = static_cast<int>(items.size());
            mega_phase_items(items, ms, offs, n, d->sm_count);
            ly.count[k] = static_cast<int>(items.size()) - ly.first[k];
        };
        phase(0, m, o_qkv, 3);
        phase(1, m + 3, o_zero, 1);
        phase(2, m + 4, o_gu, 2);
        phase(3, m + 6, o_zero, 1);
        ly.attn_norm = d->norms[l * 4 + 0];
        ly.ffn_norm = d->norms[l * 4 + 1];
        ly.attn_sub_norm = d->norms[l * 4 + 2];  // nullptr unless the model has sub-norms (BitNet)
        ly.ffn_sub_norm = d->norms[l * 4 + 3];
        for (int k = 0; k < 7; ++k) ly.ws[k] = d->scales[l * 7 + k];
        ly.kc = d->kc + size_t(l) * d->ctx * kvd;
        ly.vc = d->vc + size_t(l) * d->ctx * kvd;
        for (int k = 0; k < 7; ++k) {
            ly.wbase[k] = reinterpret_cast<const unsigned char*>(m[k]->d_w);
            ly.wbytes[k] = static_cast<unsigned int>(m[k]->w_bytes);
        }
    }
    GemvItem* d_items = nullptr;
    MegaLayer* d_layers = nullptr;
    if ((rc = dev_upload(d, &d_items, items.data(), items.size())) != QUINTRIT_OK) return rc;
    if ((rc = dev_upload(d, &d_layers, layers.data(), layers.size())) != QUINTRIT_OK) return rc;
    MegaArgs& a = d->mega;
    a.layers = d_layers, a.items = d_items;
    a.n_layers = L, a.hidden = H, a.inter = I, a.q_heads = d->q_heads, a.kv_heads = d->kv_heads, a.head_dim = d->head_dim;
    a.vocab = d->vocab, a.ctx = d->ctx, a.rope_dims = d->rope_dims, a.f32_values = d->f32_values;
    a.eps = d->eps, a.attn_scale = 1.0f / std::sqrt(static_cast<float>(d->head_dim));
    a.embed = d->embed, a.lm_head = d->lm_head, a.out_norm = d->out_norm, a.cos_sin = d->cos_sin;
    a.xa = d->xa, a.xb = d->xb;
    a.acc_qkv = d->acc_qkv, a.acc_o = d->acc_o, a.acc_gu = d->acc_gu, a.acc_down = d->acc_down;
    a.v_inter = d->v_inter, a.amax_bits = d->amax_bits, a.part_acc = d->part_acc, a.part_ms = d->part_ms, a.logits = d->logits;
    a.scores = d->scores, a.attn_region = static_cast<unsigned int>(mega_attn_region(d->ctx, d->q_heads / d->kv_heads, d->head_dim, d->attn_v2));
    a.attn_v2 = d->attn_v2 ? 1 : 0, a.attn_out = d->attn_out;
    a.fac = d->fac, a.fac_flags = d->fac_flags, a.fac_M = d->fac_M, a.fac_done = d->fac_done, a.fac_stride = fac_stride;
    a.bf16_tables = d->bf16_tables ? 1 : 0;
    a.l2_prefetch = 1;
    if (const char* pf = std::getenv("QUINTRIT_B200_L2_PREFETCH")) a.l2_prefetch = pf[0] != '0';  // experiments: "0" keeps the cold streams
    a.neox = d->arch != QUINTRIT_B200_ARCH_LLAMA, a.relu2 = d->arch == QUINTRIT_B200_ARCH_BITNET;
    a.sumsq_part = nullptr;
    if (d->arch == QUINTRIT_B200_ARCH_BITNET) {
        double* part = nullptr;
        if ((rc = dev_alloc(d, &part, static_cast<size_t>(d->sm_count))) != QUINTRIT_OK) return rc;
        a.sumsq_part = part;
    }
    a.tp_rank = d->tp_rank, a.tp_world = d->tp_world, a.tp_seq = d->tp_seq, a.attn_replicated = d->attn_replicated ? 1 : 0;
    a.tp_wait_ns = kTpWaitLimitNs;
    if (const char* ms = std::getenv("QUINTRIT_B200_TP_WAIT_MS")) {  // shorter or longer patience with a silent peer, in milliseconds
        const long v = std::strtol(ms, nullptr, 10);
        if (v >= 1 && v <= 10000) a.tp_wait_ns = static_cast<unsigned long long>(v) * 1000000ull;
    }
    for (int p = 0; p < 8; ++p) a.tp_box[p] = nullptr;
    a.tp_box[d->tp_rank] = d->tp_box;
    a.box_acc_o = static_cast<unsigned int>(off_acc_o), a.box_acc_down = static_cast<unsigned int>(off_acc_down), a.box_y = static_cast<unsigned int>(off_y);
    a.box_v = static_cast<unsigned int>(off_v), a.box_amax = static_cast<unsigned int>(off_amax), a.box_best = static_cast<unsigned int>(off_best);
    a.q_dim_full = d->q_dim_full, a.inter_full = d->inter_full, a.vocab_base = d->tp_rank * d->vocab, a.h_slice = H / d->tp_world;
    if (d->tp_world > 1) a.v_inter = reinterpret_cast<float*>(d->tp_box + off_v);
    a.best_val = d->best_val, a.best_idx = d->best_idx, a.token = d->d_token, a.pos = d->d_pos, a.history = d->d_history;
    a.bar = d->bar, a.status = d->d_counters + 2, a.trace = nullptr;
    d->mega_smem = mega_smem_bytes(a.attn_region, std::max(H, d->q_dim_full), H, L);
    // the table-base constant: measured once per device like the GEMV kernel's
    unsigned int base = 0xFFFFFFFFu;
    smem_base_kernel<<<1, 32, 1024>>>(reinterpret_cast<unsigned int*>(d->bar));
    QTB_CUDA(cudaGetLastError());
    QTB_CUDA(cudaMemcpy(&base, d->bar, sizeof base, cudaMemcpyDeviceToHost));
    QTB_CUDA(cudaMemset(d->bar, 0, 64));
    switch (base) {
        case 0: return mega_bind<0>(d);
        case 1024: return mega_bind<1024>(d);
        case 2048: return mega_bind<2048>(d);
        case 3072: return mega_bind<3072>(d);
        case 4096: return mega_bind<4096>(d);
        default: return fail(QUINTRIT_ERR_DEVICE, "unexpected shared-memory base %u on CUDA device %d: no kernel was built for it", base, d->device);
    }
}

int decoder_step(quintrit_b200_decoder* d) {
    if (d->tp_world > 1 && !d->tp_attached) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "the tensor-parallel group is not attached yet (quintrit_b200_decoder_tp_attach)");
    if (d->use_mega) {
        QTB_CUDA(cudaMemsetAsync(d->bar, 0, 16 * sizeof(unsigned int), d->stream));
        void* args[] = {&d->mega};
        QTB_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(d->mega_kernel), dim3(d->sm_count), dim3(kMegaThreads), args, d->mega_smem, d->stream));
        ++g_launches;
        return QUINTRIT_OK;
    }
    int rc = decoder_graph(d);
    if (rc != QUINTRIT_OK) return rc;
    QTB_CUDA(cudaGraphLaunch(d->graph_step, d->stream));
    return QUINTRIT_OK;
}

// The status word of the decode kernel as an error of the C ABI.
int kernel_status_error(unsigned int flag) {
    if (flag == kGemmStatusTimeout) return fail(QUINTRIT_ERR_DEVICE, "the batched projection kernel on the CUDA device gave up waiting at a barrier");
    if (flag == 3) return fail(QUINTRIT_ERR_DEVICE, "the decode kernel on the CUDA device gave up waiting for another rank of the tensor-parallel group");
    if (flag == 2) return fail(QUINTRIT_ERR_DEVICE, "the decode kernel on the CUDA device gave up waiting at a grid barrier");
    if (flag != 0) return fail(QUINTRIT_ERR_DEVICE, "a kernel on the CUDA device found its shared-memory table at an unexpected address");
    return QUINTRIT_OK;
}

int decoder_check_status(quintrit_b200_decoder* d) {
    unsigned int flag = 0;
    QTB_CUDA(cudaMemcpyAsync(&flag, d->d_counters + 2, sizeof flag, cudaMemcpyDeviceToHost, d->stream));
    QTB_CUDA(cudaStreamSynchronize(d->stream));
    if (flag != 0) {  // the word is sticky on the device: clear it so that the decoder stays usable after the error
        cudaMemsetAsync(d->d_counters + 2, 0, sizeof(unsigned int), d->stream);
        return kernel_status_error(flag);
    }
    return QUINTRIT_OK;
}

}  // namespace

extern "C" int quintrit_b200_decoder_create(const quintrit_b200_decoder_desc_t* desc, quintrit_b200_decoder_t** out_decoder) {
    return guard([&]() -> int {
        if (out_decoder == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_decoder is NULL");
        *out_decoder = nullptr;
        if (desc == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "desc is NULL");
        quintrit_b200_decoder* d = nullptr;
        int rc = decoder_create_impl(desc, &d);
        if (rc != QUINTRIT_OK) {
            destroy_decoder(d);
            return rc;
        }
        *out_decoder = d;
        return ok();
    });
}

// ---- decoder from a GGUF file ---------------------------------------------------------------------------------------------
namespace {

struct GgufModelShape {
    std::string arch;
    int arch_id = QUINTRIT_B200_ARCH_LLAMA;
    uint64_t vocab = 0, hidden = 0, inter = 0, layers = 0, heads = 0, kv_heads = 0, head_dim = 0, ctx_train = 0, rope_dims = 0;
    float eps = 1e-5f, theta = 500000.0f;
    bool has_i2s = false, has_q2 = false, tied = false;
    bool qk_norm = false;  // Qwen3: every query and key head is RMS-normalised before RoPE (blk.N.attn_q_norm / attn_k_norm)
};

uint64_t meta_usize(const GgufFile& g, const std::string& key, uint64_t fallback, bool allow_array_max = false) {
    const GgufValue* v = g.find(key);
    if (v == nullptr) return fallback;
    if (v->type == 9) return allow_array_max && v->count > 0 ? v->max_u : fallback;
    return v->is_int() ? v->u : fallback;
}
float meta_f32(const GgufFile& g, const std::string& key, float fallback) {
    const GgufValue* v = g.find(key);
    if (v == nullptr) return fallback;
    if (v->type == 6 || v->type == 12) return static_cast<float>(v->f);
    return fallback;
}
std::string meta_str(const GgufFile& g, const std::string& key, const char* fallback) {
    const GgufValue* v = g.find(key);
    return v != nullptr && v->type == 8 ? v->s : std::string(fallback);
}
// The hyperparameters as ModelConfig::from_gguf derives them (quintrit-runtime/src/config.rs:257-455): keys are prefixed
// with general.architecture, missing ones take the reference's defaults, head_dim = attention.key_length or hidden / heads.
int read_shape(const GgufFile& g, GgufModelShape* out) {
    GgufModelShape& m = *out;
    m.arch = meta_str(g, "general.architecture", "bitnet-b1.58");
    const std::string a = m.arch;
    if (a == "qwen35" || a == "nemotron_h_moe")
        return fail(QUINTRIT_ERR_UNSUPPORTED, "architecture '%s' is not supported by the GPU decoder (hybrid and mixture-of-experts models run on the CPU only)", a.c_str());
    // config.rs:276-290, 419-424, 464-467: BitNet (NEOX RoPE, squared ReLU, sub-norms); Qwen2 / Qwen3 (NEOX RoPE; Qwen3 with query/key-norm); else LLaMA
    m.arch_id = (a == "bitnet-b1.58" || a == "bitnet") ? QUINTRIT_B200_ARCH_BITNET : (a == "qwen2" || a == "qwen3") ? QUINTRIT_B200_ARCH_QWEN : QUINTRIT_B200_ARCH_LLAMA;
    m.qk_norm = a == "qwen3";
    const GgufTensor* embd = g.tensor("token_embd.weight");
    uint64_t vocab_fallback = 128256;
    if (embd != nullptr && embd->shape.size() >= 2) vocab_fallback = embd->shape[1];
    else if (const GgufValue* toks = g.find("tokenizer.ggml.tokens"); toks != nullptr && toks->type == 9) vocab_fallback = toks->count;  // config.rs:293-304
    m.vocab = meta_usize(g, a + ".vocab_size", vocab_fallback);
    m.hidden = meta_usize(g, a + ".embedding_length", 2560);
    m.inter = meta_usize(g, a + ".feed_forward_length", 6912, true);
    m.layers = meta_usize(g, a + ".block_count", 30);
    m.heads = meta_usize(g, a + ".attention.head_count", 20, true);
    m.kv_heads = meta_usize(g, a + ".attention.head_count_kv", 5, true);
    m.eps = meta_f32(g, a + ".attention.layer_norm_rms_epsilon", 1e-5f);
    m.theta = meta_f32(g, a + ".rope.freq_base", 500000.0f);
    m.ctx_train = meta_usize(g, a + ".context_length", 4096);
    if (!m.vocab || !m.hidden || !m.inter || !m.layers || !m.heads || !m.kv_heads || !m.ctx_train || m.vocab > (1u << 24) || m.hidden > (1u << 20) ||
        m.inter > (1u << 22) || m.layers > 4096 || m.heads > 4096)
        return fail(QUINTRIT_ERR_MODEL, "the hyperparameters of the file are zero or implausibly large");
    m.head_dim = meta_usize(g, a + ".attention.key_length", m.hidden / m.heads);
    if (m.head_dim == 0 || m.head_dim % 2 != 0 || m.head_dim > 4096)
        return fail(QUINTRIT_ERR_MODEL, "metadata '%s.attention.key_length' = %llu must be even and in 2..=4096", a.c_str(), static_cast<unsigned long long>(m.head_dim));
    m.rope_dims = meta_usize(g, a + ".rope.dimension_count", m.head_dim);
    if (m.rope_dims == 0 || m.rope_dims % 2 != 0 || m.rope_dims > m.head_dim)
        return fail(QUINTRIT_ERR_MODEL, "metadata '%s.rope.dimension_count' = %llu must be even and at most the head dimension %llu", a.c_str(),
                    static_cast<unsigned long long>(m.rope_dims), static_cast<unsigned long long>(m.head_dim));
    const std::string scaling = meta_str(g, a + ".rope.scaling.type", "none");
    if (scaling != "none") return fail(QUINTRIT_ERR_UNSUPPORTED, "RoPE scaling '%s' is not supported by the GPU decoder", scaling.c_str());
    for (const auto& kv : g.tensors) {
        m.has_i2s |= kv.second.type == kGgmlI2S;
        m.has_q2 |= kv.second.type == kGgmlQ2;
    }
    // a pre-transcoded container records which attention numerics its source file selected (config.rs:425-429 decides by tensor type)
    if (const GgufValue* v = g.find("quintrit_b200.f32_values"))
        if (v->is_int()) m.has_i2s = v->u == 0;
    m.tied = g.tensor("output.weight") == nullptr;
    return QUINTRIT_OK;
}

// One ternary projection: payload view, GGML type and per-tensor scale (gguf.rs:343-358: the f32 behind an I2_S payload, or
// the f16 scale every TQ block repeats - quintrit-format/src/decoders/mod.rs:121-138 rejects a tensor whose blocks differ).
int projection(const GgufFile& g, const std::string& name, uint64_t rows, uint64_t cols, const uint8_t** data, uint64_t* len, int32_t* source,
               float* scale) {
    const GgufTensor* t = g.tensor(name);
    if (t == nullptr) return fail(QUINTRIT_ERR_MODEL, "Missing %s", name.c_str());
    if (t->type != kGgmlI2S && t->type != kGgmlTq1 && t->type != kGgmlTq2 && t->type != kGgmlQ2 && t->type != kGgmlVelurex)
        return fail(QUINTRIT_ERR_UNSUPPORTED, "%s has GGML type %u; the GPU decoder needs I2_S, TQ1_0, TQ2_0 or Q2_0 projections", name.c_str(), t->type);
    if (t->shape.size() != 2 || t->shape[0] != cols || t->shape[1] != rows)
        return fail(QUINTRIT_ERR_MODEL, "%s does not have the shape %llu x %llu", name.c_str(), static_cast<unsigned long long>(rows), static_cast<unsigned long long>(cols));
    *data = g.data(*t, len);
    if (*data == nullptr) return fail(QUINTRIT_ERR_FORMAT, "the payload of %s does not lie inside the file", name.c_str());
    *source = static_cast<int32_t>(t->type);
    if (t->type == kGgmlVelurex) {  // the container's planar velurex rows: nothing to decode, the scale sits behind the payload as I2_S has it
        *source = kSrcPlanar;
        if (!g.trailing_scale(*t, scale)) return fail(QUINTRIT_ERR_FORMAT, "the scale of %s does not lie inside the file", name.c_str());
        return QUINTRIT_OK;
    }
    if (t->type == kGgmlQ2) {  // one scale per 64 weights inside the payload: no tensor scale
        *scale = 1.0f;
        return QUINTRIT_OK;
    }
    if (t->type == kGgmlI2S) {
        if (!g.trailing_scale(*t, scale)) return fail(QUINTRIT_ERR_FORMAT, "the scale of %s does not lie inside the file", name.c_str());
        return QUINTRIT_OK;
    }
    const size_t block = t->type == kGgmlTq1 ? 54 : 66, at = block - 2;
    uint16_t first = 0;
    std::memcpy(&first, *data + at, 2);
    for (uint64_t b = 1; b < *len / block; ++b) {
        uint16_t h = 0;
        std::memcpy(&h, *data + b * block + at, 2);
        if (h != first) return fail(QUINTRIT_ERR_UNSUPPORTED, "%s has block scales that differ; only tensors with one scale are ternary projections", name.c_str());
    }
    *scale = __half2float(__ushort_as_half(first));
    return QUINTRIT_OK;
}

// A model file as the decoder needs it: the mapped file, the hyperparameters, the ternary projections transcoded on the
// device (owned here), their scales, and views of the dense tensors inside the mapping.
struct GgufModel {
    GgufFile file;
    GgufModelShape shape;
    uint32_t device = 0;
    std::vector<quintrit_b200_matrix*> mats;
    std::vector<float> scales;
    std::vector<std::vector<float>> f32_store;
    std::vector<const float*> norms;
    std::vector<const float*> qk_norms;  // layers * 2 (query, key) when the architecture has them, else empty
    const uint16_t* embed = nullptr;
    const uint16_t* head = nullptr;
    const float* out_norm = nullptr;
    uint32_t table_type = kGgmlF16;
    GgufModel() = default;
    GgufModel(const GgufModel&) = delete;
    GgufModel& operator=(const GgufModel&) = delete;
    ~GgufModel() {
        for (quintrit_b200_matrix* x : mats) destroy_matrix(x);
    }
    // Largest context a decoder of this model may have: the model's maximum, at most `limit` (0: 4096) and 7936, rounded down to
    // a multiple of 256 when it reaches 256 (gpu.rs:141-146).
    uint32_t context_for(uint32_t limit) const {
        uint64_t want = std::min<uint64_t>(shape.ctx_train, limit != 0 ? limit : 4096);
        want = std::min<uint64_t>(want, 7936);
        return static_cast<uint32_t>(want >= 256 ? want / 256 * 256 : want);
    }
};

// Reads the file, checks what the decoder needs and places the ternary projections on GPU `device` (the loading half of
// GpuModel::load, gpu.rs:183-260).
int load_gguf_model(const char* path, uint32_t device, GgufModel* out) {
    GgufModel& md = *out;
    GgufFile& g = md.file;
    GgufModelShape& m = md.shape;
    md.device = device;
    std::string why;
    const int rc_open = g.open(path, why);
    if (rc_open == 1) return fail(QUINTRIT_ERR_IO, "%s", why.c_str());
    if (rc_open != 0) return fail(QUINTRIT_ERR_FORMAT, "%s", why.c_str());
    int rc = read_shape(g, &m);
    if (rc != QUINTRIT_OK) return rc;
    const uint64_t qd = m.heads * m.head_dim, kvd = m.kv_heads * m.head_dim;

    if (const GgufTensor* e = g.tensor("token_embd.weight"))
        if (e->type == kGgmlBF16) md.table_type = kGgmlBF16;
    const uint32_t table_type = md.table_type;
    auto dense_f16 = [&](const char* name, uint64_t n, const uint16_t** outp) -> int {
        const GgufTensor* t = g.tensor(name);
        if (t == nullptr) return fail(QUINTRIT_ERR_MODEL, "Missing %s tensor", name);
        if (t->type != table_type) return fail(QUINTRIT_ERR_UNSUPPORTED, "%s is not %s; the GPU decoder needs an embedding and a head that are both F16 or both BF16", name, table_type == kGgmlF16 ? "F16" : "BF16");
        uint64_t len = 0;
        const uint8_t* p = g.data(*t, &len);
        if (p == nullptr || len != n * 2) return fail(QUINTRIT_ERR_MODEL, "%s has %llu values, expected %llu", name, static_cast<unsigned long long>(len / 2), static_cast<unsigned long long>(n));
        *outp = reinterpret_cast<const uint16_t*>(p);
        return QUINTRIT_OK;
    };
    auto dense_f32 = [&](const std::string& name, uint64_t n, const float** outp) -> int {
        const GgufTensor* t = g.tensor(name);
        if (t == nullptr || t->type != kGgmlF32) return fail(QUINTRIT_ERR_MODEL, "Missing %s", name.c_str());
        uint64_t len = 0;
        const uint8_t* p = g.data(*t, &len);
        if (p == nullptr || len != n * 4) return fail(QUINTRIT_ERR_MODEL, "%s does not hold %llu values", name.c_str(), static_cast<unsigned long long>(n));
        md.f32_store.emplace_back(n);
        std::memcpy(md.f32_store.back().data(), p, n * 4);  // tensor payloads are not necessarily 4-byte aligned in memory
        *outp = md.f32_store.back().data();
        return QUINTRIT_OK;
    };

    const char* proj_names[7] = {"attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"};
    const uint64_t shapes[7][2] = {{qd, m.hidden}, {kvd, m.hidden}, {kvd, m.hidden}, {m.hidden, qd}, {m.inter, m.hidden}, {m.inter, m.hidden}, {m.hidden, m.inter}};
    md.f32_store.reserve(m.layers * 6 + 1);
    for (uint64_t l = 0; l < m.layers && rc == QUINTRIT_OK; ++l) {
        const std::string prefix = "blk." + std::to_string(l) + ".";
        for (int k = 0; k < 7 && rc == QUINTRIT_OK; ++k) {
            const uint8_t* data = nullptr;
            uint64_t len = 0;
            int32_t source = 0;
            float scale = 0.0f;
            rc = projection(g, prefix + proj_names[k] + ".weight", shapes[k][0], shapes[k][1], &data, &len, &source, &scale);
            if (rc != QUINTRIT_OK) break;
            quintrit_b200_matrix_t* h = nullptr;
            rc = quintrit_b200_matrix_upload(device, source, data, len, shapes[k][0], shapes[k][1], &h);
            if (rc != QUINTRIT_OK) break;
            md.mats.push_back(h);
            md.scales.push_back(scale);
        }
        const char* norm_names[4] = {"attn_norm", "ffn_norm", "attn_sub_norm", "ffn_sub_norm"};
        const uint64_t norm_len[4] = {m.hidden, m.hidden, m.hidden, m.inter};
        for (int k = 0; k < 4 && rc == QUINTRIT_OK; ++k) {
            const float* p = nullptr;
            if (k < 2 || m.arch_id == QUINTRIT_B200_ARCH_BITNET) rc = dense_f32(prefix + norm_names[k] + ".weight", norm_len[k], &p);
            md.norms.push_back(p);
        }
        const char* head_norms[2] = {"attn_q_norm", "attn_k_norm"};  // engine.rs:480, validate.rs:250-251: head_dim F32 values each
        for (int k = 0; k < 2 && rc == QUINTRIT_OK && m.qk_norm; ++k) {
            const float* p = nullptr;
            rc = dense_f32(prefix + head_norms[k] + ".weight", m.head_dim, &p);
            md.qk_norms.push_back(p);
        }
    }
    if (rc == QUINTRIT_OK) rc = dense_f16("token_embd.weight", m.vocab * m.hidden, &md.embed);
    if (rc == QUINTRIT_OK && !m.tied) rc = dense_f16("output.weight", m.vocab * m.hidden, &md.head);
    if (rc == QUINTRIT_OK) rc = dense_f32("output_norm.weight", m.hidden, &md.out_norm);
    return rc;
}

// A decoder (KV cache, buffers, copies of the dense tables) over a loaded model; the model keeps the projections.
int decoder_from_model(const GgufModel& md, uint32_t ctx, quintrit_b200_decoder** out) {
    const GgufModelShape& m = md.shape;
    quintrit_b200_decoder_desc_t desc;
    std::memset(&desc, 0, sizeof desc);
    desc.struct_size = sizeof desc;
    desc.device_index = md.device;
    desc.arch = m.arch_id;
    desc.f32_values = m.has_i2s ? 0 : 1;  // config.rs:425-429: files with I2_S tensors use the F16-accumulator attention
    desc.hidden_size = static_cast<uint32_t>(m.hidden), desc.intermediate_size = static_cast<uint32_t>(m.inter);
    desc.num_layers = static_cast<uint32_t>(m.layers), desc.num_heads = static_cast<uint32_t>(m.heads), desc.num_kv_heads = static_cast<uint32_t>(m.kv_heads);
    desc.head_dim = static_cast<uint32_t>(m.head_dim), desc.vocab_size = static_cast<uint32_t>(m.vocab), desc.context_length = ctx;
    desc.rope_dims = static_cast<uint32_t>(m.rope_dims), desc.rms_norm_eps = m.eps, desc.rope_theta = m.theta;
    desc.embed = md.embed, desc.lm_head = md.head, desc.output_norm = md.out_norm;
    desc.table_dtype = md.table_type == kGgmlBF16 ? 1u : 0u;
    desc.matrices = reinterpret_cast<const quintrit_b200_matrix_t* const*>(md.mats.data());
    desc.scales = md.scales.data();
    desc.norms = md.norms.data();
    desc.qk_norms = md.qk_norms.empty() ? nullptr : md.qk_norms.data();
    quintrit_b200_decoder* d = nullptr;
    const int rc = decoder_create_impl(&desc, &d);
    if (rc != QUINTRIT_OK) {
        destroy_decoder(d);
        return rc;
    }
    *out = d;
    return QUINTRIT_OK;
}

int open_gguf_impl(const char* path, const quintrit_gpu_options_t* options, quintrit_b200_decoder** out) {
    uint32_t device = 0, want_ctx = 0;
    if (options != nullptr) {
        if (options->struct_size < sizeof(quintrit_gpu_options_t))
            return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "struct_size %u is smaller than quintrit_gpu_options_t (%zu)", options->struct_size, sizeof(quintrit_gpu_options_t));
        if (options->flags & ~1u) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "unknown flag bits 0x%x", options->flags);
        device = options->device_index;
        want_ctx = options->context_length;
    }
    GgufModel md;
    int rc = load_gguf_model(path, device, &md);
    if (rc != QUINTRIT_OK) return rc;
    const uint32_t ctx = md.context_for(want_ctx);
    if (ctx == 0) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "the context window of the model is empty");
    quintrit_b200_decoder* d = nullptr;
    if ((rc = decoder_from_model(md, ctx, &d)) != QUINTRIT_OK) return rc;
    for (quintrit_b200_matrix* x : md.mats) d->owned_matrices.push_back(x);  // the decoder takes the projections over
    md.mats.clear();
    *out = d;
    return QUINTRIT_OK;
}

}  // namespace

extern "C" int quintrit_b200_decoder_open_gguf(const char* path, const quintrit_gpu_options_t* options, quintrit_b200_decoder_t** out_decoder) {
    return guard([&]() -> int {
        if (out_decoder == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_decoder is NULL");
        *out_decoder = nullptr;
        if (path == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "path is NULL");
        quintrit_b200_decoder* d = nullptr;
        const int rc = open_gguf_impl(path, options, &d);
        if (rc != QUINTRIT_OK) return rc;
        *out_decoder = d;
        return ok();
    });
}

extern "C" int quintrit_b200_decoder_info(const quintrit_b200_decoder_t* decoder, quintrit_b200_decoder_info_t* out_info) {
    return guard([&]() -> int {
        int rc = check_decoder(decoder);
        if (rc != QUINTRIT_OK) return rc;
        if (out_info == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_info is NULL");
        if (out_info->struct_size < sizeof(quintrit_b200_decoder_info_t))
            return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "struct_size %u is smaller than quintrit_b200_decoder_info_t (%zu)", out_info->struct_size, sizeof(quintrit_b200_decoder_info_t));
        const quintrit_b200_decoder* d = decoder;
        out_info->arch = d->arch, out_info->f32_values = d->f32_values ? 1 : 0;
        out_info->hidden_size = d->hidden, out_info->intermediate_size = d->inter, out_info->num_layers = d->layers;
        out_info->num_heads = d->q_heads, out_info->num_kv_heads = d->kv_heads, out_info->head_dim = d->head_dim;
        out_info->vocab_size = d->vocab_full, out_info->context_length = d->ctx, out_info->rope_dims = d->rope_dims;
        out_info->device_index = static_cast<uint32_t>(d->device), out_info->single_kernel = d->use_mega ? 1 : 0;
        out_info->table_dtype = d->bf16_tables ? 1 : 0;
        return ok();
    });
}

// A GGUF file's directory as text, without touching a GPU: one line per hyperparameter, then one line per tensor
// ("tensor <name> type=<id> shape=<d0>x<d1>... bytes=<n>"). *out_needed receives the length including the final NUL.
extern "C" int quintrit_b200_gguf_describe(const char* path, char* out, size_t out_capacity, size_t* out_needed) {
    return guard([&]() -> int {
        if (path == nullptr || out_needed == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "a pointer is NULL");
        GgufFile g;
        std::string why;
        const int rc_open = g.open(path, why);
        if (rc_open == 1) return fail(QUINTRIT_ERR_IO, "%s", why.c_str());
        if (rc_open != 0) return fail(QUINTRIT_ERR_FORMAT, "%s", why.c_str());
        GgufModelShape m;
        int rc = read_shape(g, &m);
        if (rc != QUINTRIT_OK) return rc;
        std::string text = "version " + std::to_string(g.version) + "\narchitecture " + m.arch + "\nvocab_size " + std::to_string(m.vocab) + "\nhidden_size " +
                           std::to_string(m.hidden) + "\nintermediate_size " + std::to_string(m.inter) + "\nnum_layers " + std::to_string(m.layers) + "\nnum_heads " +
                           std::to_string(m.heads) + "\nnum_kv_heads " + std::to_string(m.kv_heads) + "\nhead_dim " + std::to_string(m.head_dim) + "\nrope_dims " +
                           std::to_string(m.rope_dims) + "\ncontext_length " + std::to_string(m.ctx_train) + "\ntied " + (m.tied ? "1" : "0") + "\nf32_values " +
                           (m.has_i2s ? "0" : "1") + "\n";
        char num[64];
        std::snprintf(num, sizeof num, "rms_norm_eps %.9g\nrope_theta %.9g\n", static_cast<double>(m.eps), static_cast<double>(m.theta));
        text += num;
        for (const std::string& name : g.order) {
            const GgufTensor& t = g.tensors.at(name);
            text += "tensor " + name + " type=" + std::to_string(t.type) + " shape=";
            for (size_t i = 0; i < t.shape.size(); ++i) text += (i ? "x" : "") + std::to_string(t.shape[i]);
            text += " bytes=" + std::to_string(t.byte_len()) + (g.data(t) != nullptr ? "" : " outside-file") + "\n";
        }
        *out_needed = text.size() + 1;
        if (out == nullptr || out_capacity < text.size() + 1) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out holds %zu bytes, %zu are needed", out_capacity, text.size() + 1);
        std::memcpy(out, text.c_str(), text.size() + 1);
        return ok();
    });
}

extern "C" int quintrit_b200_decoder_tp_handle(const quintrit_b200_decoder_t* decoder, uint8_t* out_handle, size_t out_capacity) {
    return guard([&]() -> int {
        int rc = check_decoder(decoder);
        if (rc != QUINTRIT_OK) return rc;
        if (out_handle == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_handle is NULL");
        if (out_capacity < QUINTRIT_B200_TP_HANDLE_BYTES) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out_handle holds %zu bytes, %d are needed", out_capacity, QUINTRIT_B200_TP_HANDLE_BYTES);
        if (decoder->tp_world <= 1) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "the decoder was not created as a rank of a tensor-parallel group");
        static_assert(sizeof(cudaIpcMemHandle_t) == QUINTRIT_B200_TP_HANDLE_BYTES, "handle size");
        DeviceGuard g(decoder->device);
        cudaIpcMemHandle_t h;
        QTB_CUDA(cudaIpcGetMemHandle(&h, decoder->tp_box));
        std::memcpy(out_handle, &h, sizeof h);
        return ok();
    });
}

extern "C" int quintrit_b200_decoder_tp_attach(quintrit_b200_decoder_t* decoder, const uint8_t* handles, size_t handles_len) {
    return guard([&]() -> int {
        int rc = check_decoder(decoder);
        if (rc != QUINTRIT_OK) return rc;
        quintrit_b200_decoder* d = decoder;
        if (handles == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "handles is NULL");
        if (d->tp_world <= 1) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "the decoder was not created as a rank of a tensor-parallel group");
        if (handles_len != size_t(d->tp_world) * QUINTRIT_B200_TP_HANDLE_BYTES)
            return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "%zu handle bytes for %d ranks (%d each)", handles_len, d->tp_world, QUINTRIT_B200_TP_HANDLE_BYTES);
        if (d->tp_attached) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "the tensor-parallel group is attached already");
        DeviceGuard g(d->device);
        for (int p = 0; p < d->tp_world; ++p) {
            if (p == d->tp_rank) continue;
            cudaIpcMemHandle_t h;
            std::memcpy(&h, handles + size_t(p) * QUINTRIT_B200_TP_HANDLE_BYTES, sizeof h);
            void* ptr = nullptr;
            const cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                for (void*& q : d->tp_peer)
                    if (q != nullptr) {
                        cudaIpcCloseMemHandle(q);
                        q = nullptr;
                    }
                return cuda_fail(e, "cudaIpcOpenMemHandle(peer box)");
            }
            d->tp_peer[p] = ptr;
            d->mega.tp_box[p] = static_cast<unsigned char*>(ptr);
        }
        d->tp_attached = true;
        return ok();
    });
}

extern "C" int quintrit_b200_decoder_tp_attach_local(quintrit_b200_decoder_t* decoder, quintrit_b200_decoder_t* const* group, size_t group_len) {
    return guard([&]() -> int {
        int rc = check_decoder(decoder);
        if (rc != QUINTRIT_OK) return rc;
        quintrit_b200_decoder* d = decoder;
        if (group == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "group is NULL");
        if (d->tp_world <= 1) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "the decoder was not created as a rank of a tensor-parallel group");
        if (group_len != static_cast<size_t>(d->tp_world)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "%zu decoders for %d ranks", group_len, d->tp_world);
        if (d->tp_attached) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "the tensor-parallel group is attached already");
        for (int p = 0; p < d->tp_world; ++p) {
            rc = check_decoder(group[p]);
            if (rc != QUINTRIT_OK) return rc;
            if (group[p]->tp_world != d->tp_world || group[p]->tp_rank != p || group[p]->tp_box_bytes != d->tp_box_bytes)
                return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "decoder %d of the group is not rank %d of the same %d-rank model", p, p, d->tp_world);
        }
        if (group[d->tp_rank] != d) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "the decoder is not at its own rank in the group");
        DeviceGuard g(d->device);
        for (int p = 0; p < d->tp_world; ++p) {
            if (p == d->tp_rank) continue;
            if (group[p]->device != d->device) {
                int can = 0;
                QTB_CUDA(cudaDeviceCanAccessPeer(&can, d->device, group[p]->device));
                if (!can) return fail(QUINTRIT_ERR_DEVICE, "CUDA device %d cannot access the memory of device %d", d->device, group[p]->device);
                const cudaError_t e = cudaDeviceEnablePeerAccess(group[p]->device, 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return cuda_fail(e, "cudaDeviceEnablePeerAccess");
                (void)cudaGetLastError();
            }
            d->mega.tp_box[p] = group[p]->tp_box;
        }
        d->tp_attached = true;
        return ok();
    });
}

extern "C" int quintrit_b200_decoder_free(quintrit_b200_decoder_t* decoder) {
    return guard([&]() -> int {
        if (decoder == nullptr) return ok();
        int rc = check_decoder(decoder);
        if (rc != QUINTRIT_OK) return rc;
        const std::vector<void*> owned = decoder->owned_matrices;
        destroy_decoder(decoder);
        for (void* m : owned) destroy_matrix(static_cast<quintrit_b200_matrix*>(m));
        return ok();
    });
}

extern "C" int quintrit_b200_decoder_forward(quintrit_b200_decoder_t* decoder, uint32_t token, uint32_t pos, float* logits, size_t logits_capacity,
                                             uint32_t* out_token) {
    return guard([&]() -> int {
        int rc = check_decoder(decoder);
        if (rc != QUINTRIT_OK) return rc;
        quintrit_b200_decoder* d = decoder;
        if (token >= static_cast<uint32_t>(d->vocab_full)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "token id %u is not below the vocabulary size %d", token, d->vocab_full);
        if (pos >= static_cast<uint32_t>(d->ctx)) return fail(QUINTRIT_ERR_CONTEXT_OVERFLOW, "position %u does not fit the context window of %d tokens", pos, d->ctx);
        if (pos > d->host_pos) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "position %u skips positions: %u tokens are cached", pos, d->host_pos);
        if (logits != nullptr && logits_capacity < static_cast<size_t>(d->vocab)) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "logits hold %zu values, the vocabulary has %d", logits_capacity, d->vocab);
        DeviceGuard g(d->device);
        if ((rc = decoder_set(d, token, pos)) != QUINTRIT_OK || (rc = decoder_step(d)) != QUINTRIT_OK) return rc;
        if (logits) QTB_CUDA(cudaMemcpyAsync(logits, d->logits, size_t(d->vocab) * sizeof(float), cudaMemcpyDeviceToHost, d->stream));
        if (out_token) QTB_CUDA(cudaMemcpyAsync(out_token, d->d_token, sizeof(uint32_t), cudaMemcpyDeviceToHost, d->stream));
        if ((rc = decoder_check_status(d)) != QUINTRIT_OK) return rc;
        d->host_pos = pos + 1;
        return ok();
    });
}

extern "C" int quintrit_b200_decoder_generate(quintrit_b200_decoder_t* decoder, const uint32_t* prompt, size_t prompt_len, size_t max_new,
                                              uint32_t* out_tokens, size_t out_capacity) {
    return guard([&]() -> int {
        int rc = check_decoder(decoder);
        if (rc != QUINTRIT_OK) return rc;
        quintrit_b200_decoder* d = decoder;
        if (prompt == nullptr || out_tokens == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "prompt or out_tokens is NULL");
        if (prompt_len == 0 || max_new == 0) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "the prompt and the number of new tokens must not be empty");
        if (out_capacity < max_new) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out_tokens hold %zu ids, %zu are needed", out_capacity, max_new);
        if (prompt_len + max_new - 1 > static_cast<size_t>(d->ctx))
            return fail(QUINTRIT_ERR_CONTEXT_OVERFLOW, "%zu prompt tokens and %zu new tokens do not fit the context window of %d tokens", prompt_len, max_new, d->ctx);
        for (size_t i = 0; i < prompt_len; ++i)
            if (prompt[i] >= static_cast<uint32_t>(d->vocab_full)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "token id %u is not below the vocabulary size %d", prompt[i], d->vocab_full);
        DeviceGuard g(d->device);
        uint32_t* d_prompt = nullptr;
        QTB_CUDA(cudaMalloc(&d_prompt, prompt_len * sizeof(uint32_t)));
        cudaError_t e = cudaMemcpyAsync(d_prompt, prompt, prompt_len * sizeof(uint32_t), cudaMemcpyHostToDevice, d->stream);
        if (e == cudaSuccess) rc = decoder_set(d, prompt[0], 0);
        for (size_t i = 0; e == cudaSuccess && rc == QUINTRIT_OK && i < prompt_len; ++i) {
            rc = decoder_step(d);
            if (rc == QUINTRIT_OK && i + 1 < prompt_len)  // the next prompt token replaces the prediction
                e = cudaMemcpyAsync(d->d_token, d_prompt + i + 1, sizeof(uint32_t), cudaMemcpyDeviceToDevice, d->stream);
        }
        for (size_t j = 1; e == cudaSuccess && rc == QUINTRIT_OK && j < max_new; ++j) rc = decoder_step(d);
        if (e == cudaSuccess && rc == QUINTRIT_OK)
            e = cudaMemcpyAsync(out_tokens, d->d_history + (prompt_len - 1), max_new * sizeof(uint32_t), cudaMemcpyDeviceToHost, d->stream);
        if (e == cudaSuccess && rc == QUINTRIT_OK) rc = decoder_check_status(d);
        cudaStreamSynchronize(d->stream);
        cudaFree(d_prompt);
        if (e != cudaSuccess) return cuda_fail(e, "generate");
        if (rc != QUINTRIT_OK) return rc;
        d->host_pos = static_cast<uint32_t>(prompt_len + max_new - 1);
        return ok();
    });
}

extern "C" int quintrit_b200_decoder_time_token(quintrit_b200_decoder_t* decoder, uint32_t blocks, uint32_t iters, float* out_ms) {
    return guard([&]() -> int {
        int rc = check_decoder(decoder);
        if (rc != QUINTRIT_OK) return rc;
        quintrit_b200_decoder* d = decoder;
        if (out_ms == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_ms is NULL");
        if (blocks == 0 || iters == 0) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "blocks and iters must be at least 1");
        if (d->host_pos >= static_cast<uint32_t>(d->ctx)) return fail(QUINTRIT_ERR_CONTEXT_OVERFLOW, "the context window is full: no position left to time a step at");
        DeviceGuard g(d->device);
        // The timed step decodes token 0 at the first free position: the cached prefix stays as it is, and the scratch
        // entry it writes is overwritten by the next real token.
        const uint32_t pos = d->host_pos, token = 0;
        cudaEvent_t e0, e1;
        QTB_CUDA(cudaEventCreate(&e0));
        QTB_CUDA(cudaEventCreate(&e1));
        float best = 1e30f;
        if (!d->use_mega && (rc = decoder_graph(d)) != QUINTRIT_OK) return rc;
        for (uint32_t b = 0; b < blocks; ++b) {
            cudaEventRecord(e0, d->stream);
            for (uint32_t i = 0; i < iters; ++i) {
                decoder_set(d, token, pos);  // every step decodes the same position: the context length stays fixed
                if ((rc = decoder_step(d)) != QUINTRIT_OK) return rc;
            }
            cudaEventRecord(e1, d->stream);
            cudaEventSynchronize(e1);
            float ms = 0;
            cudaEventElapsedTime(&ms, e0, e1);
            best = std::min(best, ms / iters);
        }
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        QTB_CUDA(cudaGetLastError());
        *out_ms = best;
        return ok();
    });
}

// ---------------------------------------------------------------------------------------------------------------------
// GEMV without any allocation
// ---------------------------------------------------------------------------------------------------------------------

namespace {

constexpr int kNoAllocMaxItems = 4096;
constexpr size_t kNoAllocHeaderBytes = 256;
constexpr size_t kNoAllocScratchBytes = kNoAllocHeaderBytes + size_t(kNoAllocMaxItems) * sizeof(GemvItem);  // 262400 bytes

// Work list and counters of quintrit_b200_gemv_i32_noalloc. Every GPU that loads the library holds these 256.25 KiB
// until the process exits. Layout: four 32-bit words (next item, CTAs done, kernel status, measured shared-memory
// base) padded to 256 bytes, then up to kNoAllocMaxItems descriptors of 64 bytes.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// Writes the work list of one matrix into the scratch array and clears the words that must start at zero: the same
// decomposition as build_items (block pairs x ranges of row tiles), computed on the device so that nothing is staged.
__global__ void noalloc_prepare_kernel(unsigned char* scratch, const uint4* w, int rows, int cols, int blocks, int tiles, int chunks,
                                       int n_items) {
    unsigned int* words = reinterpret_cast<unsigned int*>(scratch);
    GemvItem* items = reinterpret_cast<GemvItem*>(scratch + kNoAllocHeaderBytes);
    if (blockIdx.x == 0 && threadIdx.x < 3) words[threadIdx.x] = 0;  // next item, CTAs done, kernel status
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_items; i += gridDim.x * blockDim.x) {
        const int p = i / chunks, c = i % chunks;
        const long long t0 = static_cast<long long>(tiles) * c / chunks, t1 = static_cast<long long>(tiles) * (c + 1) / chunks;
        const int g = 2 * p;
        GemvItem it{};
        it.wa = w + (static_cast<size_t>(g) * tiles + t0) * 64;
        it.nblk = g + 1 < blocks ? 2 : 1;
        it.wb = it.nblk == 2 ? w + (static_cast<size_t>(g + 1) * tiles + t0) * 64 : it.wa;
        it.act_off = 0;
        it.out_off = 0;
        it.rows = rows;
        it.cols = cols;
        it.col0 = g * kBlockTrits;
        it.tile0 = static_cast<int>(t0);
        it.ntiles = static_cast<int>(t1 - t0);
        items[i] = it;
    }
}

struct NoAllocDevice {
    bool ready = false;
    unsigned char* scratch = nullptr;  // device address of g_noalloc_scratch on this device
    GemvKernel kernel = nullptr;
};
NoAllocDevice g_noalloc[64];
std::mutex g_noalloc_lock;  // two host threads may make the first call on a device at the same time

// Per-device set-up, run by the first call on that device (with that device current): the device address of the
// static array, and the kernel instantiation that matches this device's shared-memory base. Allocates nothing: the
// base is measured into the array's fourth word.
int noalloc_setup(int dev, NoAllocDevice** out) {
    if (dev < 0 || dev >= 64) return fail(QUINTRIT_ERR_DEVICE, "device index %d out of range", dev);
    NoAllocDevice& s = g_noalloc[dev];
    std::lock_guard<std::mutex> hold(g_noalloc_lock);
    if (!s.ready) {
        unsigned char* ptr = nullptr;
        // In host code the array's name is only a handle for the symbol; the address a kernel can use comes from here.
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_noalloc_scratch)");
        unsigned int base = 0xFFFFFFFFu;
        smem_base_kernel<<<1, 32, 1024>>>(reinterpret_cast<unsigned int*>(ptr) + 3);
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaMemcpy(&base, ptr + 12, sizeof base, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return cuda_fail(e, "smem_base_kernel");
        switch (base) {
            case 0: s.kernel = gemv_lut_kernel<0>; break;
            case 1024: s.kernel = gemv_lut_kernel<1024>; break;
            case 2048: s.kernel = gemv_lut_kernel<2048>; break;
            case 3072: s.kernel = gemv_lut_kernel<3072>; break;
            case 4096: s.kernel = gemv_lut_kernel<4096>; break;
            default: return fail(QUINTRIT_ERR_DEVICE, "unexpected shared-memory base %u on CUDA device %d: no kernel was built for it", base, dev);
        }
        QTB_CUDA(cudaFuncSetAttribute(s.kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemBytes));
        s.scratch = ptr;
        s.ready = true;
    }
    *out = &s;
    return QUINTRIT_OK;
}

}  // namespace

extern "C" int quintrit_b200_gemv_i32_noalloc(const quintrit_b200_matrix_t* matrix, const int8_t* d_activations, int32_t* d_out, void* stream) {
    return guard([&]() -> int {
        int rc = check_matrix(matrix);
        if (rc != QUINTRIT_OK) return rc;
        if (d_activations == nullptr || d_out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "a device pointer is NULL");
        const size_t pairs = (matrix->blocks + 1) / 2, slots = static_cast<size_t>(matrix->sm_count) * kCtasPerSm;
        const size_t want_chunks = std::max<size_t>(1, (slots + pairs - 1) / pairs);
        const size_t tiles_per_item = std::max<size_t>(16, (matrix->tiles + want_chunks - 1) / want_chunks);
        const size_t chunks = std::max<size_t>(1, (matrix->tiles + tiles_per_item - 1) / tiles_per_item);
        const size_t n_items = pairs * chunks;
        if (n_items > static_cast<size_t>(kNoAllocMaxItems))
            return fail(QUINTRIT_ERR_INVALID_SHAPE,
                        "a %zu x %zu matrix needs %zu work items, the static scratch of the no-allocation entry point holds %d (%zu bytes)",
                        matrix->rows, matrix->cols, n_items, kNoAllocMaxItems, kNoAllocScratchBytes);
        DeviceGuard g(matrix->device);
        NoAllocDevice* s = nullptr;
        if ((rc = noalloc_setup(matrix->device, &s)) != QUINTRIT_OK) return rc;
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        QTB_CUDA(cudaMemsetAsync(d_out, 0, matrix->rows * sizeof(int32_t), st));
        noalloc_prepare_kernel<<<static_cast<unsigned>((n_items + 255) / 256), 256, 0, st>>>(
            s->scratch, matrix->d_w, static_cast<int>(matrix->rows), static_cast<int>(matrix->cols), static_cast<int>(matrix->blocks),
            static_cast<int>(matrix->tiles), static_cast<int>(chunks), static_cast<int>(n_items));
        ++g_launches;
        QTB_CUDA(cudaGetLastError());
        const int grid = static_cast<int>(std::max<size_t>(1, std::min(n_items, slots)));
        s->kernel<<<grid, kGemvThreads, kGemvSmemBytes, st>>>(reinterpret_cast<const GemvItem*>(s->scratch + kNoAllocHeaderBytes),
                                                             static_cast<int>(n_items), d_activations, d_out,
                                                             reinterpret_cast<unsigned int*>(s->scratch));
        ++g_launches;
        QTB_CUDA(cudaGetLastError());
        return ok();
    });
}

// Runs the barrier self-test kernel: `ctas` co-resident CTAs (at most one per multiprocessor) wait for an arrival that
// never comes, with `spin_limit` polls of patience. Expected outcome: QUINTRIT_ERR_DEVICE ("gave up waiting at a grid
// barrier") and *out_released == ctas, i.e. every CTA saw the failure at both of its barriers and returned.
extern "C" int quintrit_b200_selftest_barrier(uint32_t device_index, uint32_t ctas, uint32_t spin_limit, uint32_t* out_released) {
    return guard([&]() -> int {
        if (out_released == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_released is NULL");
        *out_released = 0;
        cudaDeviceProp prop;
        int rc = require_b200(static_cast<int>(device_index), &prop);
        if (rc != QUINTRIT_OK) return rc;
        if (ctas == 0 || ctas > static_cast<uint32_t>(prop.multiProcessorCount)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "ctas must be 1..%d (every CTA has to be resident)", prop.multiProcessorCount);
        if (spin_limit == 0 || spin_limit > (1u << 20)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "spin_limit must be 1..2^20 polls");
        DeviceGuard g(static_cast<int>(device_index));
        unsigned int* d_words = nullptr;  // [0..15] barrier counters, [16] status, [17..] one flag per CTA
        QTB_CUDA(cudaMalloc(&d_words, (17 + ctas) * sizeof(unsigned int)));
        cudaError_t e = cudaMemset(d_words, 0, (17 + ctas) * sizeof(unsigned int));
        if (e == cudaSuccess) {
            barrier_selftest_kernel<<<ctas, 128>>>(d_words, d_words + 16, spin_limit, d_words + 17);
            ++g_launches;
            e = cudaGetLastError();
        }
        std::vector<unsigned int> host(17 + ctas, 0u);
        if (e == cudaSuccess) e = cudaMemcpy(host.data(), d_words, host.size() * sizeof(unsigned int), cudaMemcpyDeviceToHost);
        cudaFree(d_words);
        if (e != cudaSuccess) return cuda_fail(e, "barrier self-test");
        for (uint32_t i = 0; i < ctas; ++i) *out_released += host[17 + i];
        rc = kernel_status_error(host[16]);
        return rc == QUINTRIT_OK ? ok() : rc;
    });
}

extern "C" int quintrit_b200_decoder_trace_step(quintrit_b200_decoder_t* decoder, uint64_t* out_ns, size_t capacity, size_t* out_count) {
    return guard([&]() -> int {
        int rc = check_decoder(decoder);
        if (rc != QUINTRIT_OK) return rc;
        quintrit_b200_decoder* d = decoder;
        if (out_count == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_count is NULL");
        if (!d->use_mega) return fail(QUINTRIT_ERR_UNSUPPORTED, "phase tracing is available for the single-kernel decode path only");
        const size_t n = size_t(d->layers) * 14 + 4 + 32;  // phase stamps, then 32 optional fine stamps (zero unless built with QTB_FINE_TRACE)
        *out_count = n;
        if (out_ns == nullptr || capacity < n) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out_ns holds %zu values, %zu are needed", capacity, n);
        if (d->host_pos >= static_cast<uint32_t>(d->ctx)) return fail(QUINTRIT_ERR_CONTEXT_OVERFLOW, "the context window is full");
        DeviceGuard g(d->device);
        QTB_CUDA(cudaMemsetAsync(d->trace, 0, (n + 2) * sizeof(uint64_t), d->stream));
        d->mega.trace = d->trace;
        rc = decoder_set(d, 0, d->host_pos);
        if (rc == QUINTRIT_OK) rc = decoder_step(d);
        d->mega.trace = nullptr;
        if (rc != QUINTRIT_OK) return rc;
        // The kernel stamps the SM's cycle counter and reads the global timer once at either end: cycles become nanoseconds
        // by the ratio of the two spans. Slot layers * 14 + 3 receives the SM clock in kHz.
        std::vector<uint64_t> raw(n + 2);
        QTB_CUDA(cudaMemcpyAsync(raw.data(), d->trace, (n + 2) * sizeof(uint64_t), cudaMemcpyDeviceToHost, d->stream));
        if ((rc = decoder_check_status(d)) != QUINTRIT_OK) return rc;
        const size_t last = size_t(d->layers) * 14 + 2;
        const double span_ns = static_cast<double>(raw[n + 1] - raw[n]), span_cyc = static_cast<double>(raw[last] - raw[0]);
        const double ns_per_cycle = span_cyc > 0 ? span_ns / span_cyc : 0.0;
        for (size_t i = 0; i < n; ++i) out_ns[i] = raw[i] == 0 ? 0 : raw[n] + static_cast<uint64_t>(static_cast<double>(raw[i] - raw[0]) * ns_per_cycle);
        out_ns[last + 1] = ns_per_cycle > 0 ? static_cast<uint64_t>(1e6 / ns_per_cycle) : 0;
        return ok();
    });
}

// ---- batched projection on the tensor cores (gemm_tc.cuh) ------------------------------------------------------------------------
namespace {

std::mutex g_gemm_lock;
constexpr int kGemmMaxParts = 8;
constexpr size_t kGemmSmemLimit = 227 * 1024;  // dynamic shared memory a CTA may ask for on this device
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                      CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, fetched at run time so that the library loads on a machine without a driver.
int tensor_map_encoder(TensorMapEncodeFn* out) {
    static TensorMapEncodeFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) return fail(QUINTRIT_ERR_DEVICE, "the CUDA driver does not provide cuTensorMapEncodeTiled");
        fn = reinterpret_cast<TensorMapEncodeFn>(p);
    }
    *out = fn;
    return QUINTRIT_OK;
}

// Makes the two-bit copy of the weights and the call buffers of a matrix the first time it is used by the batched projection.
int gemm_prepare(quintrit_b200_matrix* m) {
    std::lock_guard<std::mutex> hold(g_gemm_lock);
    if (m->d_gemm_w != nullptr) return QUINTRIT_OK;
    if (m->block_scaled) return fail(QUINTRIT_ERR_UNSUPPORTED, "the batched projection takes per-tensor ternary matrices, not block-scaled (Q2_0) ones");
    const size_t rows_padded = (m->rows + kGemmM - 1) / kGemmM * kGemmM, gblocks = (m->cols + kGemmBlockCols - 1) / kGemmBlockCols, k_pad = gblocks * kGemmBlockCols;
    uint8_t* w = nullptr;
    QTB_CUDA(cudaMalloc(&w, gblocks * rows_padded * 32));
    const size_t bytes = gblocks * rows_padded * 32;
    stream_to_two_bit_kernel<<<static_cast<int>(std::min<size_t>((bytes + 255) / 256, 148 * 32)), 256>>>(m->d_w, w, m->rows, m->cols, rows_padded, gblocks, m->blocks, m->tiles, 0, rows_padded);
    ++g_launches;
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMalloc(&m->d_gemm_act, size_t(kGemmMaxN) * k_pad);
    if (e == cudaSuccess) e = cudaMalloc(&m->d_gemm_status, 4096);  // the status word; the rest is used by debug builds only
    if (e == cudaSuccess) e = cudaMemset(m->d_gemm_status, 0, 4096);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_i8_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kGemmSmemLimit));
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(w);
        return cuda_fail(e, "set-up of the batched projection");
    }
    m->gemm_rows_padded = rows_padded;
    m->d_gemm_w = w;
    return QUINTRIT_OK;
}

// One launch for up to kGemmMaxN activation vectors that are on the device ([batch][cols]); d_out is [batch][rows].
// With `defer`, a product whose K dimension is split leaves its parts where they are and describes them in *defer for the kernel that consumes the
// sums (which adds them); otherwise a second kernel adds the parts into d_out.
// `status` is the word a time-out is reported in: the matrix's own by default, a decoder's for the launches a decoder makes (one read-back per call).
// `parts` is the buffer for the partial sums of a split K dimension (kGemmMaxParts x kGemmMaxN x rows values): the matrix's own, made on first need, by default.
int gemm_launch(quintrit_b200_matrix* m, const int8_t* d_act, int batch, int32_t* d_out, cudaStream_t stream, int ldo = 0, AccView* defer = nullptr, unsigned int* status = nullptr,
                int32_t* parts = nullptr) {
    if (ldo == 0) ldo = static_cast<int>(m->rows);
    if (defer != nullptr) *defer = AccView{d_out, 1, 0, ldo};
    TensorMapEncodeFn encode = nullptr;
    int rc = tensor_map_encoder(&encode);
    if (rc != QUINTRIT_OK) return rc;
    const int gblocks = static_cast<int>((m->cols + kGemmBlockCols - 1) / kGemmBlockCols);
    const int n = std::max(16, (batch + 15) / 16 * 16), k_pad = gblocks * kGemmBlockCols;
    // The TMA reads the caller's vectors in place when their pitch and address allow it (columns and vectors beyond the matrix read as zeros);
    // otherwise they are first copied into a zero-padded matrix with a pitch of whole blocks.
    const bool in_place = m->cols % 32 == 0 && reinterpret_cast<uintptr_t>(d_act) % 16 == 0;
    const void* base = d_act;
    cuuint64_t pitch = m->cols, vectors = static_cast<cuuint64_t>(batch);
    if (!in_place) {
        gemm_pad_activations_kernel<<<std::min((n * k_pad + 255) / 256, 148 * 8), 256, 0, stream>>>(d_act, m->d_gemm_act, batch, n, static_cast<int>(m->cols), k_pad);
        ++g_launches;
        base = m->d_gemm_act, pitch = static_cast<cuuint64_t>(k_pad), vectors = static_cast<cuuint64_t>(n);
    }
    // the activations as a 3-D tensor: 32 bytes of a K tile, the vectors, the K tiles of a vector; a box is 32 x n x 4 (the four tiles of a block)
    CUtensorMap map;
    const cuuint64_t dims[3] = {32, vectors, pitch / 32};
    const cuuint64_t strides[2] = {pitch, 32};  // bytes between vectors and between K tiles: multiples of 16
    const cuuint32_t box[3] = {32, static_cast<cuuint32_t>(n), 4}, elem[3] = {1, 1, 1};
    const CUresult cr = encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(QUINTRIT_ERR_DEVICE, "cuTensorMapEncodeTiled failed with CUDA driver error %d", static_cast<int>(cr));
    GemmArgs a;
    a.w = m->d_gemm_w, a.out = d_out, a.status = status != nullptr ? status : m->d_gemm_status;
    a.rows = static_cast<int>(m->rows), a.rows_padded = static_cast<int>(m->gemm_rows_padded), a.blocks = gblocks;
    a.n = n, a.batch = batch, a.ldo = ldo;
    a.stages = gemm_stages_for(n, kGemmSmemLimit);
    if (const char* v = std::getenv("QUINTRIT_B200_GEMM_STAGES")) a.stages = std::max(2, std::min(std::atoi(v), a.stages));  // experiments: fewer stages (at least two: see the decode groups)
    a.spin_limit = 1u << 16;  // polls of up to 20 us each: about a second before a wait gives up
    // Work items are (row tile, K part); K is split (at least four blocks a part, at most kGemmMaxParts parts) where the items of whole tiles would
    // leave SMs idle: the cost of a split is the largest number of items an SM gets times the blocks of an item plus about one block for its
    // epilogue, plus the pass that adds the parts (its bytes at about 3 TB/s against 0.4 us a block).
    const int m_tiles = a.rows_padded / kGemmM;
    int ksplit = 1;
    long best = -1;
    for (int ks = 1; ks <= std::min(kGemmMaxParts, std::max(1, a.blocks / 4)); ++ks) {
        const int per = (a.blocks + ks - 1) / ks, parts = (a.blocks + per - 1) / per;
        const long waves = (long(m_tiles) * parts + m->sm_count - 1) / m->sm_count;
        const long add_pass = parts > 1 ? long((parts + 1) * double(batch) * double(m->rows) * 4.0 / 1.2e6) + 3 : 0;  // bytes the second kernel moves, in units of a block's time
        const long cost = waves * (per + 1) + add_pass;
        if (best < 0 || cost < best) best = cost, ksplit = parts;
    }
    if (const char* v = std::getenv("QUINTRIT_B200_GEMM_KSPLIT")) ksplit = std::max(1, std::min({std::atoi(v), a.blocks, kGemmMaxParts}));
    a.blocks_per_cta = (a.blocks + ksplit - 1) / ksplit;
    ksplit = (a.blocks + a.blocks_per_cta - 1) / a.blocks_per_cta;
    if (ksplit > 1) {
        if (parts == nullptr) {
            if (m->d_gemm_parts == nullptr) {
                std::lock_guard<std::mutex> hold(g_gemm_lock);
                if (m->d_gemm_parts == nullptr) QTB_CUDA(cudaMalloc(&m->d_gemm_parts, size_t(kGemmMaxParts) * kGemmMaxN * m->rows * sizeof(int32_t)));
            }
            parts = m->d_gemm_parts;
        }
        a.out = parts, a.ldo = static_cast<int>(m->rows);
    }
    gemm_i8_tcgen05_kernel<<<std::min(m_tiles * ksplit, m->sm_count), kGemmThreads, gemm_smem_bytes(n, a.stages), stream>>>(map, a);
    ++g_launches;
    if (ksplit > 1 && defer != nullptr) {
        *defer = AccView{parts, ksplit, size_t(batch) * m->rows, static_cast<int>(m->rows)};
    } else if (ksplit > 1) {
        const size_t count = size_t(batch) * m->rows;
        gemm_reduce_parts_kernel<<<static_cast<int>(std::min<size_t>((count + 255) / 256, size_t(m->sm_count) * 8)), 256, 0, stream>>>(parts, d_out, count, ksplit, static_cast<int>(m->rows), ldo);
        ++g_launches;
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "batched projection launch");
    return QUINTRIT_OK;
}

int gemm_check_status(quintrit_b200_matrix* m, cudaStream_t stream) {
    unsigned int flag = 0;
    QTB_CUDA(cudaMemcpyAsync(&flag, m->d_gemm_status, sizeof flag, cudaMemcpyDeviceToHost, stream));
    QTB_CUDA(cudaStreamSynchronize(stream));
    if (flag != 0) {
        cudaMemsetAsync(m->d_gemm_status, 0, sizeof flag, stream);
        return fail(QUINTRIT_ERR_DEVICE, "the batched projection kernel on the CUDA device gave up waiting at a barrier");
    }
    return QUINTRIT_OK;
}

}  // namespace

extern "C" int quintrit_b200_gemm_i32_device(quintrit_b200_matrix_t* matrix, const int8_t* d_activations, size_t batch, int32_t* d_out, void* stream) {
    return guard([&]() -> int {
        int rc = check_matrix(matrix, true);
        if (rc != QUINTRIT_OK) return rc;
        if (d_activations == nullptr || d_out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "a device pointer is NULL");
        if (batch == 0 || batch > (size_t(1) << 20)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "batch must be in [1, 2^20]");
        DeviceGuard g(matrix->device);
        if ((rc = gemm_prepare(matrix)) != QUINTRIT_OK) return rc;
        for (size_t b0 = 0; b0 < batch; b0 += kGemmMaxN) {
            const int nb = static_cast<int>(std::min<size_t>(kGemmMaxN, batch - b0));
            if ((rc = gemm_launch(matrix, d_activations + b0 * matrix->cols, nb, d_out + b0 * matrix->rows, static_cast<cudaStream_t>(stream))) != QUINTRIT_OK) return rc;
        }
        return ok();
    });
}

extern "C" int quintrit_b200_gemm_i32(quintrit_b200_matrix_t* matrix, const int8_t* activations, size_t activations_len, size_t batch, int32_t* out, size_t out_capacity) {
    return guard([&]() -> int {
        int rc = check_matrix(matrix, true);
        if (rc != QUINTRIT_OK) return rc;
        if (activations == nullptr || out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "activations or out is NULL");
        if (batch == 0 || batch > (size_t(1) << 20)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "batch must be in [1, 2^20]");
        if (activations_len < batch * matrix->cols) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "activations hold %zu values, %zu x %zu are needed", activations_len, batch, matrix->cols);
        if (out_capacity < batch * matrix->rows) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out holds %zu values, %zu x %zu are needed", out_capacity, batch, matrix->rows);
        DeviceGuard g(matrix->device);
        if ((rc = gemm_prepare(matrix)) != QUINTRIT_OK) return rc;
        if (matrix->d_gemm_in == nullptr) {  // staging of host-buffer calls, made when the first one comes
            std::lock_guard<std::mutex> hold(g_gemm_lock);
            if (matrix->d_gemm_in == nullptr) {
                int32_t* o = nullptr;
                int8_t* in = nullptr;
                QTB_CUDA(cudaMalloc(&o, size_t(kGemmMaxN) * matrix->rows * sizeof(int32_t)));
                const cudaError_t e = cudaMalloc(&in, size_t(kGemmMaxN) * matrix->cols);
                if (e != cudaSuccess) {
                    cudaFree(o);
                    return cuda_fail(e, "cudaMalloc(batched projection staging)");
                }
                matrix->d_gemm_out = o, matrix->d_gemm_in = in;
            }
        }
        for (size_t b0 = 0; b0 < batch; b0 += kGemmMaxN) {
            const int nb = static_cast<int>(std::min<size_t>(kGemmMaxN, batch - b0));
            QTB_CUDA(cudaMemcpyAsync(matrix->d_gemm_in, activations + b0 * matrix->cols, size_t(nb) * matrix->cols, cudaMemcpyHostToDevice, nullptr));
            if ((rc = gemm_launch(matrix, matrix->d_gemm_in, nb, matrix->d_gemm_out, nullptr)) != QUINTRIT_OK) return rc;
            QTB_CUDA(cudaMemcpyAsync(out + b0 * matrix->rows, matrix->d_gemm_out, size_t(nb) * matrix->rows * sizeof(int32_t), cudaMemcpyDeviceToHost, nullptr));
            if ((rc = gemm_check_status(matrix, nullptr)) != QUINTRIT_OK) return rc;
        }
        return ok();
    });
}

// ---- prompt ingestion: a chunk of tokens per pass, projections on the tensor cores -------------------------------------------------
namespace {

constexpr int kPrefillMax = kGemmMaxN;

// The batched products of a decoder: q | k | v and gate | up of a layer are stacked row-wise into one matrix each where their row counts are whole
// tiles (one launch instead of three or two, and no launch too small to fill the device); o and down keep their own two-bit copies. The partial
// sums of split products go to four buffers of the decoder, one per kind of product, shared by all layers.
int decoder_gemm_prepare(quintrit_b200_decoder* d) {
    if (d->pf.gemm_ready) return QUINTRIT_OK;
    auto mat = [&](int l, int k) { return const_cast<quintrit_b200_matrix*>(d->mats[size_t(l) * 7 + k]); };
    const bool stack_off = std::getenv("QUINTRIT_B200_GEMM_STACK_OFF") != nullptr;
    int rc;
    d->pf.stack.assign(size_t(d->layers) * 2, nullptr);
    auto stack = [&](int l, int first, int count, quintrit_b200_matrix** out) -> int {
        size_t rows = 0;
        for (int k = first; k < first + count; ++k) {
            const quintrit_b200_matrix* m = mat(l, k);
            if (m->rows % kGemmM != 0 || m->cols != mat(l, first)->cols || m->block_scaled) return QUINTRIT_OK;  // not stackable: separate launches
            rows += m->rows;
        }
        const quintrit_b200_matrix* m0 = mat(l, first);
        const size_t gblocks = (m0->cols + kGemmBlockCols - 1) / kGemmBlockCols;
        uint8_t* w = nullptr;
        int r = dev_alloc(d, &w, gblocks * rows * 32, false);
        if (r != QUINTRIT_OK) return r;
        size_t off = 0;
        for (int k = first; k < first + count; ++k) {
            const quintrit_b200_matrix* m = mat(l, k);
            const size_t bytes = gblocks * m->rows * 32;
            stream_to_two_bit_kernel<<<static_cast<int>(std::min<size_t>((bytes + 255) / 256, 148 * 32)), 256>>>(m->d_w, w, m->rows, m->cols, m->rows, gblocks, m->blocks, m->tiles, off, rows);
            ++g_launches;
            off += m->rows;
        }
        QTB_CUDA(cudaGetLastError());
        quintrit_b200_matrix* sm = new quintrit_b200_matrix();
        sm->magic = kMagicMatrix, sm->device = d->device, sm->sm_count = d->sm_count;
        sm->rows = rows, sm->cols = m0->cols, sm->blocks = m0->blocks, sm->tiles = 0;
        sm->d_w = nullptr, sm->w_bytes = 0, sm->d_items = nullptr, sm->n_items = 0, sm->d_counters = nullptr, sm->d_act = nullptr, sm->d_out = nullptr, sm->d_outf = nullptr;
        sm->d_gemm_w = w, sm->gemm_rows_padded = rows;
        d->pf.stacked_objects.push_back(sm);
        *out = sm;
        return QUINTRIT_OK;
    };
    size_t rows_kind[4] = {0, 0, 0, 0};  // qkv, o, gate|up, down
    for (int l = 0; l < d->layers; ++l) {
        quintrit_b200_matrix *sq = nullptr, *sg = nullptr;
        if (!stack_off && ((rc = stack(l, 0, 3, &sq)) != QUINTRIT_OK || (rc = stack(l, 4, 2, &sg)) != QUINTRIT_OK)) return rc;
        d->pf.stack[size_t(l) * 2] = sq, d->pf.stack[size_t(l) * 2 + 1] = sg;
        for (int k = 0; k < 7; ++k) {
            const bool stacked = (k < 3 && sq != nullptr) || ((k == 4 || k == 5) && sg != nullptr);
            if (!stacked && (rc = gemm_prepare(mat(l, k))) != QUINTRIT_OK) return rc;
        }
        rows_kind[0] = std::max(rows_kind[0], sq != nullptr ? sq->rows : std::max({mat(l, 0)->rows, mat(l, 1)->rows, mat(l, 2)->rows}));
        rows_kind[1] = std::max(rows_kind[1], mat(l, 3)->rows);
        rows_kind[2] = std::max(rows_kind[2], sg != nullptr ? sg->rows : std::max(mat(l, 4)->rows, mat(l, 5)->rows));
        rows_kind[3] = std::max(rows_kind[3], mat(l, 6)->rows);
    }
    // one buffer per product that can be in flight with deferred parts at the same time: q, k, v (or the stack), o, gate, up (or the stack), down
    for (int k = 0; k < 7; ++k) {
        const int kind = k < 3 ? 0 : k == 3 ? 1 : k < 6 ? 2 : 3;
        const bool second_of_stack = (k == 1 || k == 2 || k == 5);
        bool all_stacked = true;
        for (int l = 0; l < d->layers; ++l) all_stacked = all_stacked && d->pf.stack[size_t(l) * 2 + (kind == 0 ? 0 : 1)] != nullptr;
        if (second_of_stack && all_stacked && (kind == 0 || kind == 2)) continue;  // the stack's one buffer is parts[first of the kind]
        if ((rc = dev_alloc(d, &d->pf.parts[k], size_t(kGemmMaxParts) * kGemmMaxN * rows_kind[kind], false)) != QUINTRIT_OK) return rc;
    }
    QTB_CUDA(cudaFuncSetAttribute(gemm_i8_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kGemmSmemLimit)));
    QTB_CUDA(cudaDeviceSynchronize());
    d->pf.gemm_ready = true;
    return QUINTRIT_OK;
}

int prefill_buffers(quintrit_b200_decoder* d) {
    if (d->pf.x != nullptr) return QUINTRIT_OK;
    const size_t B = kPrefillMax, H = d->hidden, I = d->inter, qd = d->q_dim, kvd = d->kv_dim, hd = d->head_dim;
    int rc;
    if ((rc = dev_alloc(d, &d->pf.tokens, B)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->pf.pos, 4)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->pf.x, B * H)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->pf.q, B * qd)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->pf.part_acc, B * d->q_heads * 4 * hd)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->pf.part_ms, B * d->q_heads * 8)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->pf.s_h, B)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->pf.s_q, B)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->pf.s_i, B)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->pf.a8_h, B * H)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->pf.a8_q, B * qd)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->pf.a8_i, B * I)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->pf.acc_qkv, B * (qd + 2 * kvd))) != QUINTRIT_OK || (rc = dev_alloc(d, &d->pf.acc_o, B * H)) != QUINTRIT_OK ||
        (rc = dev_alloc(d, &d->pf.acc_gu, B * 2 * I)) != QUINTRIT_OK || (rc = dev_alloc(d, &d->pf.acc_down, B * H)) != QUINTRIT_OK)
        return rc;
    return QUINTRIT_OK;
}

// One chunk of n <= kPrefillMax tokens (already in d->pf.tokens) at positions pos0 .. pos0 + n - 1: the launch sequence of enqueue_token with a token
// index in gridDim.z, the projections as batched products (every token keeps its own activation scale; the integers are those of the batch-1
// kernel). With `with_head` the last token's logits and greedy choice land in d->logits / d->d_token as after a single step.
// Where the tokens of a batched pass sit: the KV cache they append to and read, their positions, and (for a step of several sequences) the
// sequence of every token. The default is the decoder's own cache with consecutive positions from pf.pos[0] (a prompt chunk).
struct BatchTarget {
    __half *kc = nullptr, *vc = nullptr;  // [layers][ctx][kv_dim] of the first sequence
    const uint32_t* pos = nullptr;
    SeqIndex seq{nullptr, 0, 0};
    bool own = true;                      // the decoder's own cache: a full chunk may be replayed as the captured graph
};
BatchTarget own_target(quintrit_b200_decoder* d) {
    BatchTarget t;
    t.kc = d->kc, t.vc = d->vc, t.pos = d->pf.pos;
    return t;
}

int prefill_layers(quintrit_b200_decoder* d, int n, const BatchTarget& tg) {
    cudaStream_t s = d->stream;
    const int H = d->hidden, I = d->inter, qd = d->q_dim, kvd = d->kv_dim, hd = d->head_dim, qkv = qd + 2 * kvd;
    embed_kernel<<<dim3((H + 255) / 256, n), 256, 0, s>>>(d->embed, d->pf.tokens, H, d->pf.x, d->bf16_tables);
    QTB_LAUNCH_CHECK();
    auto mat = [&](int l, int k) { return const_cast<quintrit_b200_matrix*>(d->mats[size_t(l) * 7 + k]); };
    int rc;
    // Projections whose K dimension is split leave their parts to the kernel that consumes the sums (AccView); only the last layer's down
    // projection is completed by a pass of its own, because the final norm of a later launch reads it.
    const bool defer = std::getenv("QUINTRIT_B200_GEMM_DEFER_OFF") == nullptr;
    AccView v_q{}, v_k{}, v_v{}, v_o{}, v_gate{}, v_up{}, v_down{};
    auto view = [&](AccView* v) { return defer ? v : nullptr; };
    unsigned int* st = d->d_counters + 2;  // the decoder's status word: a time-out in a batched product is read back with the decoder's other failures
    for (int l = 0; l < d->layers; ++l) {
        const float* sc = d->scales.data() + l * 7;
        NormQuantArgs n1{};
        n1.x = d->pf.x, n1.b_x = H;
        if (l > 0) n1.acc_prev = d->pf.acc_down, n1.b_acc = H, n1.scale_prev = d->pf.s_i, n1.ws_prev = d->scales[(l - 1) * 7 + 6];
        n1.norm_w = d->norms[l * 4 + 0], n1.eps = d->eps, n1.n = H;
        n1.q_out = d->pf.a8_h, n1.b_q = H, n1.scale_out = d->pf.s_h, n1.b_scale = 1;
        if (l > 0) n1.v_prev = v_down;
        norm_quant_kernel<<<dim3(1, 1, n), kRowThreads, H * sizeof(float), s>>>(n1);
        QTB_LAUNCH_CHECK();
        if (quintrit_b200_matrix* sq = d->pf.stack[size_t(l) * 2]) {  // q | k | v as one product
            if ((rc = gemm_launch(sq, d->pf.a8_h, n, d->pf.acc_qkv, s, qkv, &v_q, st, d->pf.parts[0])) != QUINTRIT_OK) return rc;
            v_k = v_q, v_k.base += qd;
            v_v = v_q, v_v.base += qd + kvd;
        } else if ((rc = gemm_launch(mat(l, 0), d->pf.a8_h, n, d->pf.acc_qkv, s, qkv, view(&v_q), st, d->pf.parts[0])) != QUINTRIT_OK ||
                   (rc = gemm_launch(mat(l, 1), d->pf.a8_h, n, d->pf.acc_qkv + qd, s, qkv, view(&v_k), st, d->pf.parts[1])) != QUINTRIT_OK ||
                   (rc = gemm_launch(mat(l, 2), d->pf.a8_h, n, d->pf.acc_qkv + qd + kvd, s, qkv, view(&v_v), st, d->pf.parts[2])) != QUINTRIT_OK) {
            return rc;
        }
        const bool qkv_views = defer || d->pf.stack[size_t(l) * 2] != nullptr;
        RopeKvArgs rk{};
        rk.acc = d->pf.acc_qkv, rk.b_acc = qkv, rk.act_scale = d->pf.s_h, rk.b_scale = 1;
        rk.ws_q = sc[0], rk.ws_k = sc[1], rk.ws_v = sc[2];
        rk.cos_sin = d->cos_sin, rk.pos = tg.pos, rk.seq = tg.seq;
        rk.q_dim = qd, rk.kv_dim = kvd, rk.head_dim = hd, rk.rope_dims = d->rope_dims, rk.neox = d->arch != QUINTRIT_B200_ARCH_LLAMA;
        rk.q_out = d->pf.q, rk.b_q = qd;
        if (qkv_views) rk.v_q = v_q, rk.v_k = v_k, rk.v_v = v_v;
        rk.k_cache = tg.kc + static_cast<size_t>(l) * d->ctx * kvd;
        rk.v_cache = tg.vc + static_cast<size_t>(l) * d->ctx * kvd;
        rope_kv_kernel<<<dim3(((qd + kvd) / 2 + kvd + 255) / 256, 1, n), 256, 0, s>>>(rk);
        QTB_LAUNCH_CHECK();
        AttnArgs at{};
        at.q = d->pf.q, at.b_q = qd;
        at.k_cache = rk.k_cache, at.v_cache = rk.v_cache, at.pos = tg.pos, at.seq = tg.seq;
        at.head_dim = hd, at.kv_dim = kvd, at.gqa = d->q_heads / d->kv_heads, at.ctx = d->ctx, at.f32_values = d->f32_values;
        at.scale = 1.0f / std::sqrt(static_cast<float>(hd));
        at.part_acc = d->pf.part_acc, at.b_acc = d->q_heads * 4 * hd, at.part_ms = d->pf.part_ms, at.b_ms = d->q_heads * 8;
        launch_attention(d, at, n, s);
        QTB_LAUNCH_CHECK();
        AttnFinishArgs af{};
        af.part_acc = d->pf.part_acc, af.b_acc = d->q_heads * 4 * hd, af.part_ms = d->pf.part_ms, af.b_ms = d->q_heads * 8, af.pos = tg.pos, af.seq = tg.seq;
        af.q_heads = d->q_heads, af.head_dim = hd, af.ctx = d->ctx;
        af.sub_norm_w = d->norms[l * 4 + 2], af.eps = d->eps;
        af.q_out = d->pf.a8_q, af.b_q = qd, af.scale_out = d->pf.s_q, af.b_scale = 1;
        attn_finish_kernel<<<dim3(1, 1, n), kRowThreads, qd * sizeof(float), s>>>(af);
        QTB_LAUNCH_CHECK();
        if ((rc = gemm_launch(mat(l, 3), d->pf.a8_q, n, d->pf.acc_o, s, 0, view(&v_o), st, d->pf.parts[3])) != QUINTRIT_OK) return rc;
        NormQuantArgs n2{};
        n2.x = d->pf.x, n2.b_x = H, n2.acc_prev = d->pf.acc_o, n2.b_acc = H, n2.scale_prev = d->pf.s_q, n2.ws_prev = sc[3];
        n2.norm_w = d->norms[l * 4 + 1], n2.eps = d->eps, n2.n = H;
        n2.q_out = d->pf.a8_h, n2.b_q = H, n2.scale_out = d->pf.s_h, n2.b_scale = 1;
        if (defer) n2.v_prev = v_o;
        norm_quant_kernel<<<dim3(1, 1, n), kRowThreads, H * sizeof(float), s>>>(n2);
        QTB_LAUNCH_CHECK();
        if (quintrit_b200_matrix* sg = d->pf.stack[size_t(l) * 2 + 1]) {  // gate | up as one product
            if ((rc = gemm_launch(sg, d->pf.a8_h, n, d->pf.acc_gu, s, 2 * I, &v_gate, st, d->pf.parts[4])) != QUINTRIT_OK) return rc;
            v_up = v_gate, v_up.base += I;
        } else if ((rc = gemm_launch(mat(l, 4), d->pf.a8_h, n, d->pf.acc_gu, s, 2 * I, view(&v_gate), st, d->pf.parts[4])) != QUINTRIT_OK ||
                   (rc = gemm_launch(mat(l, 5), d->pf.a8_h, n, d->pf.acc_gu + I, s, 2 * I, view(&v_up), st, d->pf.parts[5])) != QUINTRIT_OK) {
            return rc;
        }
        const bool gu_views = defer || d->pf.stack[size_t(l) * 2 + 1] != nullptr;
        ActQuantArgs aq{};
        aq.acc_gate = d->pf.acc_gu, aq.acc_up = d->pf.acc_gu + I, aq.b_acc = 2 * I, aq.act_scale = d->pf.s_h, aq.b_scale = 1;
        aq.ws_gate = sc[4], aq.ws_up = sc[5];
        aq.n = I, aq.relu2 = d->arch == QUINTRIT_B200_ARCH_BITNET;
        aq.sub_norm_w = d->norms[l * 4 + 3], aq.eps = d->eps;
        aq.q_out = d->pf.a8_i, aq.b_q = I, aq.scale_out = d->pf.s_i;
        if (gu_views) aq.v_gate = v_gate, aq.v_up = v_up;
        if (std::getenv("QUINTRIT_B200_ACT_CLUSTER_OFF") == nullptr)
            act_quant_cluster_kernel<<<dim3(kActClusterSize, 1, n), kActClusterThreads, act_cluster_slice(I) * sizeof(float), s>>>(aq);
        else
            act_quant_kernel<<<dim3(1, 1, n), kRowThreads, I * sizeof(float), s>>>(aq);
        QTB_LAUNCH_CHECK();
        if ((rc = gemm_launch(mat(l, 6), d->pf.a8_i, n, d->pf.acc_down, s, 0, l + 1 < d->layers ? view(&v_down) : nullptr, st, d->pf.parts[6])) != QUINTRIT_OK) return rc;
    }
    return QUINTRIT_OK;
}

int enqueue_prefill_chunk(quintrit_b200_decoder* d, int n, uint32_t pos0, bool with_head, const BatchTarget& tg) {
    cudaStream_t s = d->stream;
    const int H = d->hidden;
    QTB_CUDA(cudaMemcpyAsync(d->pf.pos, &pos0, sizeof pos0, cudaMemcpyHostToDevice, s));
    int rc;
    // A full chunk is about 1200 launches; from the third full chunk on they are replayed as one CUDA graph (the first runs as it is and makes
    // every lazy allocation, the second is captured). The position and the tokens are read from device memory, so one graph serves every chunk.
    if (n == kPrefillMax && tg.own && d->pf.graph_ready) {
        QTB_CUDA(cudaGraphLaunch(d->pf.graph, s));
    } else if (n == kPrefillMax && tg.own && d->pf.warm && std::getenv("QUINTRIT_B200_PREFILL_GRAPH_OFF") == nullptr) {
        cudaGraph_t g = nullptr;
        QTB_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
        rc = prefill_layers(d, n, tg);
        const cudaError_t e = cudaStreamEndCapture(s, &g);
        if (rc != QUINTRIT_OK) {
            if (g) cudaGraphDestroy(g);
            return rc;
        }
        if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture(prompt chunk)");
        const cudaError_t ei = cudaGraphInstantiate(&d->pf.graph, g, 0);
        cudaGraphDestroy(g);
        if (ei != cudaSuccess) return cuda_fail(ei, "cudaGraphInstantiate(prompt chunk)");
        d->pf.graph_ready = true;
        QTB_CUDA(cudaGraphLaunch(d->pf.graph, s));
    } else {
        if ((rc = prefill_layers(d, n, tg)) != QUINTRIT_OK) return rc;
        if (n == kPrefillMax) d->pf.warm = true;
    }
    if (with_head) {  // the last token of the chunk: final norm, output head, greedy choice, as a single step ends
        const size_t last = static_cast<size_t>(n - 1);
        NormQuantArgs nf{};
        nf.x = d->pf.x + last * H, nf.acc_prev = d->pf.acc_down + last * H, nf.scale_prev = d->pf.s_i + last;
        nf.ws_prev = d->scales[(d->layers - 1) * 7 + 6], nf.norm_w = d->out_norm, nf.eps = d->eps, nf.n = H;
        nf.y16_out = d->x16, nf.y16_bf16 = d->bf16_tables;
        norm_quant_kernel<<<1, kRowThreads, H * sizeof(float), s>>>(nf);
        QTB_LAUNCH_CHECK();
        lm_head_kernel<<<d->sm_count * 8, 256, H * sizeof(float), s>>>(d->lm_head, d->x16, H, d->vocab, d->logits, d->bf16_tables);
        QTB_LAUNCH_CHECK();
        argmax_kernel<<<1, 1024, 0, s>>>(d->logits, d->vocab, d->d_token);
        QTB_LAUNCH_CHECK();
    }
    return QUINTRIT_OK;
}

// Whether a decoder can ingest prompts in chunks: per-tensor ternary projections on one GPU (the block-scaled and tensor-parallel decoders
// take their prompts token by token).
bool prefill_available(const quintrit_b200_decoder* d) { return !d->block_scaled && d->tp_world == 1 && d->hidden % 32 == 0 && d->inter % 32 == 0 && d->q_dim % 32 == 0; }

// Tokens at positions pos0 .. pos0 + count - 1, chunk by chunk; ends like a single step of the last token (logits, greedy token, position).
int decoder_prefill(quintrit_b200_decoder* d, const uint32_t* tokens, size_t count, uint32_t pos0, const BatchTarget* target = nullptr) {
    int rc = prefill_buffers(d);
    if (rc != QUINTRIT_OK) return rc;
    if ((rc = decoder_gemm_prepare(d)) != QUINTRIT_OK) return rc;
    const BatchTarget tg = target != nullptr ? *target : own_target(d);
    for (size_t c0 = 0; c0 < count; c0 += kPrefillMax) {
        const int n = static_cast<int>(std::min<size_t>(kPrefillMax, count - c0));
        QTB_CUDA(cudaMemcpyAsync(d->pf.tokens, tokens + c0, size_t(n) * sizeof(uint32_t), cudaMemcpyHostToDevice, d->stream));
        if (tg.own) QTB_CUDA(cudaMemcpyAsync(d->d_history + pos0 + c0, d->pf.tokens, size_t(n) * sizeof(uint32_t), cudaMemcpyDeviceToDevice, d->stream));
        if ((rc = enqueue_prefill_chunk(d, n, pos0 + static_cast<uint32_t>(c0), c0 + n == count, tg)) != QUINTRIT_OK) return rc;
    }
    if (tg.own) {
        const uint32_t next = pos0 + static_cast<uint32_t>(count);  // the device-side position as after `count` single steps
        QTB_CUDA(cudaMemcpyAsync(d->d_pos, &next, sizeof next, cudaMemcpyHostToDevice, d->stream));
    }
    return QUINTRIT_OK;
}

}  // namespace

extern "C" int quintrit_b200_decoder_prefill(quintrit_b200_decoder_t* decoder, const uint32_t* tokens, size_t count, uint32_t pos, float* logits, size_t logits_capacity,
                                             uint32_t* out_token) {
    return guard([&]() -> int {
        int rc = check_decoder(decoder);
        if (rc != QUINTRIT_OK) return rc;
        quintrit_b200_decoder* d = decoder;
        if (tokens == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "tokens is NULL");
        if (count == 0) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "no tokens to ingest");
        if (!prefill_available(d)) return fail(QUINTRIT_ERR_UNSUPPORTED, "this decoder takes its prompt token by token (block-scaled or tensor-parallel model)");
        if (size_t(pos) + count > static_cast<size_t>(d->ctx)) return fail(QUINTRIT_ERR_CONTEXT_OVERFLOW, "%zu tokens from position %u do not fit the context window of %d tokens", count, pos, d->ctx);
        if (pos > d->host_pos) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "position %u skips positions: %u tokens are cached", pos, d->host_pos);
        for (size_t i = 0; i < count; ++i)
            if (tokens[i] >= static_cast<uint32_t>(d->vocab_full)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "token id %u is not below the vocabulary size %d", tokens[i], d->vocab_full);
        if (logits != nullptr && logits_capacity < static_cast<size_t>(d->vocab)) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "logits hold %zu values, the vocabulary has %d", logits_capacity, d->vocab);
        DeviceGuard g(d->device);
        std::vector<uint32_t> pinned(tokens, tokens + count);  // the copies below are asynchronous: keep the ids alive until the synchronisation
        if ((rc = decoder_prefill(d, pinned.data(), count, pos)) != QUINTRIT_OK) return rc;
        if (logits) QTB_CUDA(cudaMemcpyAsync(logits, d->logits, size_t(d->vocab) * sizeof(float), cudaMemcpyDeviceToHost, d->stream));
        if (out_token) QTB_CUDA(cudaMemcpyAsync(out_token, d->d_token, sizeof(uint32_t), cudaMemcpyDeviceToHost, d->stream));
        if ((rc = decoder_check_status(d)) != QUINTRIT_OK) return rc;  // (the batched projections report a time-out through the same word)
        d->host_pos = pos + static_cast<uint32_t>(count);
        return ok();
    });
}

// ---- mixture-of-experts feed-forward block ------------------------------------------------------------------------------------------
struct quintrit_b200_moe {
    uint32_t magic;
    int device, sm_count;
    int hidden, inter, inter_pad, n_experts, top_k, max_batch, chunks_down;
    std::vector<void*> allocs;
    __half *router = nullptr, *x16 = nullptr;
    MoeExpertRef* experts = nullptr;
    float *x = nullptr, *s_x = nullptr, *logits = nullptr, *probs = nullptr, *weights = nullptr, *s_i = nullptr, *out = nullptr;
    int8_t *a8_x = nullptr, *a8_i = nullptr;
    uint32_t *chosen = nullptr, *local_z = nullptr;
    unsigned int *tie = nullptr, *counters = nullptr;
    int32_t *acc_gu = nullptr, *acc_down = nullptr;
    float* pairs = nullptr;      // [max_batch * top_k][hidden]: every pair's down result as floats (zeros for pairs of experts held elsewhere)
    int expert_first = 0, expert_count = 0, n_local = 0, last_batch = 0;  // this GPU's experts; the local pairs of the last forward
    GemvItem *gu_items = nullptr, *down_items = nullptr;
    cudaStream_t stream = nullptr;
};

namespace {

constexpr uint32_t kMagicMoe = 0x51544258u;  // "QTBX"

int check_moe(const quintrit_b200_moe* m) {
    if (m == nullptr || m->magic != kMagicMoe) return fail(QUINTRIT_ERR_INVALID_HANDLE, "mixture-of-experts handle is NULL, freed or of the wrong type");
    return QUINTRIT_OK;
}

void destroy_moe(quintrit_b200_moe* m) {
    if (m == nullptr) return;
    DeviceGuard g(m->device);
    if (m->stream) cudaStreamDestroy(m->stream);
    for (void* p : m->allocs) cudaFree(p);
    m->magic = 0;
    delete m;
}

template <typename T>
int moe_alloc(quintrit_b200_moe* m, T** p, size_t count) {
    void* q = nullptr;
    const size_t bytes = std::max<size_t>(count * sizeof(T), 16);
    cudaError_t e = cudaMalloc(&q, bytes);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(mixture-of-experts buffer)");
    m->allocs.push_back(q);
    if ((e = cudaMemset(q, 0, bytes)) != cudaSuccess) return cuda_fail(e, "cudaMemset(mixture-of-experts buffer)");
    *p = static_cast<T*>(q);
    return QUINTRIT_OK;
}

// The launches of one batch on the block's stream; x is on the device in m->x, the result lands in m->out.
int moe_enqueue(quintrit_b200_moe* m, int batch) {
    cudaStream_t s = m->stream;
    const int H = m->hidden, I = m->inter, E = m->n_experts, K = m->top_k, nz = batch * K;
    moe_prepare_kernel<<<batch, kRowThreads, H * sizeof(float), s>>>(m->x, H, m->x16, m->a8_x, m->s_x);
    QTB_LAUNCH_CHECK();
    moe_router_kernel<<<dim3((E + 3) / 4, (batch + 3) / 4), 128, 0, s>>>(m->router, m->x16, H, E, batch, m->logits);
    QTB_LAUNCH_CHECK();
    moe_select_kernel<<<batch, 256, (E + K) * sizeof(float), s>>>(m->logits, E, K, m->probs, m->chosen, m->weights, m->tie);
    QTB_LAUNCH_CHECK();
    return QUINTRIT_OK;
}
// The experts of the local pairs (m->local_z, m->n_local: set by the caller from the chosen ids) up to every pair's down result as floats.
int moe_enqueue_experts(quintrit_b200_moe* m, int batch) {
    cudaStream_t s = m->stream;
    const int H = m->hidden, I = m->inter, K = m->top_k, nz = batch * K, nl = m->n_local;
    const int pairs_gu = ((H + kBlockTrits - 1) / kBlockTrits + 1) / 2, pairs_d = ((I + kBlockTrits - 1) / kBlockTrits + 1) / 2;
    const int n_gu = nl * pairs_gu, n_d = nl * pairs_d * m->chunks_down;
    QTB_CUDA(cudaMemsetAsync(m->acc_down, 0, size_t(nz) * H * sizeof(int32_t), s));
    if (nl > 0) {
        moe_items_kernel<<<(n_gu + n_d + 255) / 256, 256, 0, s>>>(m->experts, m->chosen, m->local_z, nl, K, H, I, m->inter_pad, m->chunks_down, m->gu_items, m->down_items);
        QTB_LAUNCH_CHECK();
        QTB_CUDA(cudaMemsetAsync(m->acc_gu, 0, size_t(nz) * 2 * I * sizeof(int32_t), s));
        int rc = launch_gemv(m->gu_items, n_gu, m->a8_x, m->acc_gu, m->counters, m->sm_count, s);
        if (rc != QUINTRIT_OK) return rc;
        moe_act_quant_kernel<<<nl, kRowThreads, I * sizeof(float), s>>>(m->acc_gu, m->experts, m->chosen, m->local_z, m->s_x, K, I, m->inter_pad, m->a8_i, m->s_i);
        QTB_LAUNCH_CHECK();
        if ((rc = launch_gemv(m->down_items, n_d, m->a8_i, m->acc_down, m->counters, m->sm_count, s)) != QUINTRIT_OK) return rc;
    }
    moe_scale_pairs_kernel<<<dim3((H + 255) / 256, nz), 256, 0, s>>>(m->acc_down, m->experts, m->chosen, m->s_i, H, m->pairs);
    QTB_LAUNCH_CHECK();
    return QUINTRIT_OK;
}
int moe_enqueue_combine(quintrit_b200_moe* m, int batch) {
    moe_combine_kernel<<<dim3((m->hidden + 255) / 256, batch), 256, 0, m->stream>>>(m->pairs, m->weights, m->top_k, m->hidden, m->out);
    QTB_LAUNCH_CHECK();
    return QUINTRIT_OK;
}

// Router, selection (with the host's std::sort for tokens with equal probabilities), the list of local pairs, the local experts: everything up
// to the pairs' results, then a synchronisation.
int moe_partial(quintrit_b200_moe* m, const float* x, size_t batch) {
    cudaStream_t s = m->stream;
    const int B = static_cast<int>(batch), K = m->top_k, E = m->n_experts;
    QTB_CUDA(cudaMemcpyAsync(m->x, x, batch * m->hidden * sizeof(float), cudaMemcpyHostToDevice, s));
    int rc = moe_enqueue(m, B);
    if (rc != QUINTRIT_OK) return rc;
    // Experts with exactly equal probabilities: std::sort (the reference's choice, hybrid.rs:828-831) orders them by its algorithm. The
    // device ranks such ties by id and flags the token; the host then sorts that token's experts with the standard library's std::sort
    // and replaces the device's choice and weights.
    std::vector<unsigned int> tie(batch);
    std::vector<uint32_t> chosen(batch * K);
    QTB_CUDA(cudaMemcpyAsync(tie.data(), m->tie, batch * sizeof(unsigned int), cudaMemcpyDeviceToHost, s));
    QTB_CUDA(cudaMemcpyAsync(chosen.data(), m->chosen, batch * K * sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    QTB_CUDA(cudaStreamSynchronize(s));
    for (int b = 0; b < B; ++b) {
        if (tie[b] == 0) continue;
        std::vector<float> p(E);
        QTB_CUDA(cudaMemcpy(p.data(), m->probs + size_t(b) * E, E * sizeof(float), cudaMemcpyDeviceToHost));
        std::vector<uint32_t> order(E);
        for (int i = 0; i < E; ++i) order[i] = static_cast<uint32_t>(i);
        std::sort(order.begin(), order.end(), [&](uint32_t a, uint32_t c) { return p[a] > p[c]; });
        std::vector<float> w(K);
        double sum = 0.0;
        for (int i = 0; i < K; ++i) w[i] = p[order[i]], sum += static_cast<double>(w[i]);
        const float sc = std::max(static_cast<float>(sum), 6.103515625e-5f);
        for (int i = 0; i < K; ++i) w[i] /= sc, chosen[size_t(b) * K + i] = order[i];
        QTB_CUDA(cudaMemcpy(m->chosen + size_t(b) * K, order.data(), K * sizeof(uint32_t), cudaMemcpyHostToDevice));
        QTB_CUDA(cudaMemcpy(m->weights + size_t(b) * K, w.data(), K * sizeof(float), cudaMemcpyHostToDevice));
    }
    std::vector<uint32_t> local;
    for (size_t z = 0; z < chosen.size(); ++z)
        if (chosen[z] >= static_cast<uint32_t>(m->expert_first) && chosen[z] < static_cast<uint32_t>(m->expert_first + m->expert_count)) local.push_back(static_cast<uint32_t>(z));
    m->n_local = static_cast<int>(local.size()), m->last_batch = B;
    if (!local.empty()) QTB_CUDA(cudaMemcpyAsync(m->local_z, local.data(), local.size() * sizeof(uint32_t), cudaMemcpyHostToDevice, s));
    if ((rc = moe_enqueue_experts(m, B)) != QUINTRIT_OK) return rc;
    unsigned int flag = 0;
    QTB_CUDA(cudaMemcpyAsync(&flag, m->counters + 2, sizeof flag, cudaMemcpyDeviceToHost, s));
    QTB_CUDA(cudaStreamSynchronize(s));  // (also keeps `local` alive until its copy is done)
    if (flag != 0) return fail(QUINTRIT_ERR_DEVICE, "GEMV kernel on the CUDA device found its shared-memory table at an unexpected address");
    return QUINTRIT_OK;
}

int moe_finish(quintrit_b200_moe* m, size_t batch, float* out, uint32_t* out_experts, float* out_weights) {
    cudaStream_t s = m->stream;
    int rc = moe_enqueue_combine(m, static_cast<int>(batch));
    if (rc != QUINTRIT_OK) return rc;
    QTB_CUDA(cudaMemcpyAsync(out, m->out, batch * m->hidden * sizeof(float), cudaMemcpyDeviceToHost, s));
    if (out_experts) QTB_CUDA(cudaMemcpyAsync(out_experts, m->chosen, batch * m->top_k * sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    if (out_weights) QTB_CUDA(cudaMemcpyAsync(out_weights, m->weights, batch * m->top_k * sizeof(float), cudaMemcpyDeviceToHost, s));
    QTB_CUDA(cudaStreamSynchronize(s));
    return QUINTRIT_OK;
}

}  // namespace

extern "C" int quintrit_b200_moe_create_shard(uint32_t device_index, uint32_t hidden, uint32_t inter, uint32_t n_experts, uint32_t top_k, uint32_t max_batch,
                                              const uint16_t* router_bf16, uint32_t expert_first, uint32_t expert_count, const quintrit_b200_matrix_t* const* gate_up,
                                              const quintrit_b200_matrix_t* const* down, const float* scales, quintrit_b200_moe_t** out_moe) {
    return guard([&]() -> int {
        if (out_moe == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_moe is NULL");
        *out_moe = nullptr;
        if (router_bf16 == nullptr || gate_up == nullptr || down == nullptr || scales == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "router_bf16, gate_up, down or scales is NULL");
        if (hidden == 0 || hidden % 128 != 0 || lm_head_batch_smem(static_cast<int>(hidden)) > 200 * 1024)
            return fail(QUINTRIT_ERR_UNSUPPORTED, "the hidden size %u must be a multiple of 128, at most 3200", hidden);
        if (inter == 0 || inter % 16 != 0 || inter > 49152) return fail(QUINTRIT_ERR_UNSUPPORTED, "the expert width %u must be a multiple of 16, at most 49152", inter);
        if (n_experts == 0 || n_experts > 1024 || top_k == 0 || top_k > n_experts || top_k > 64) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "%u experts with top-%u routing are not supported (at most 1024 experts, top-64)", n_experts, top_k);
        if (max_batch == 0 || max_batch > 256) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "max_batch must be in [1, 256]");
        cudaDeviceProp prop;
        int rc = require_b200(static_cast<int>(device_index), &prop);
        if (rc != QUINTRIT_OK) return rc;
        if (expert_count == 0 || expert_first > n_experts || expert_count > n_experts - expert_first)
            return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "experts %u .. %u + %u do not lie inside the %u experts of the block", expert_first, expert_first, expert_count, n_experts);
        std::vector<MoeExpertRef> refs(n_experts, MoeExpertRef{nullptr, nullptr, 0.0f, 0.0f, 0.0f, 0});  // experts held elsewhere keep null weights
        for (uint32_t e = 0; e < expert_count; ++e) {
            if ((rc = check_matrix(gate_up[e])) != QUINTRIT_OK || (rc = check_matrix(down[e])) != QUINTRIT_OK) return rc;
            if (gate_up[e]->device != static_cast<int>(device_index) || down[e]->device != static_cast<int>(device_index)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "expert %u lives on another device", e);
            if (gate_up[e]->rows != size_t(2) * inter || gate_up[e]->cols != hidden)
                return fail(QUINTRIT_ERR_INVALID_SHAPE, "gate_up of expert %u is %zu x %zu, the block needs %u x %u (gate rows, then up rows)", e, gate_up[e]->rows, gate_up[e]->cols, 2 * inter, hidden);
            if (down[e]->rows != hidden || down[e]->cols != inter) return fail(QUINTRIT_ERR_INVALID_SHAPE, "down of expert %u is %zu x %zu, the block needs %u x %u", e, down[e]->rows, down[e]->cols, hidden, inter);
            refs[expert_first + e] = MoeExpertRef{gate_up[e]->d_w, down[e]->d_w, scales[3 * e], scales[3 * e + 1], scales[3 * e + 2], 0};
        }
        DeviceGuard g(static_cast<int>(device_index));
        if ((rc = upload_exp2_table()) != QUINTRIT_OK) return rc;
        GemvKernel k = nullptr;
        if ((rc = gemv_kernel_for_device(static_cast<int>(device_index), &k)) != QUINTRIT_OK) return rc;
        int smem_optin = 0;
        QTB_CUDA(cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, static_cast<int>(device_index)));
        if ((rc = allow_max_dynamic_smem(lm_head_batch_kernel, smem_optin)) != QUINTRIT_OK || (rc = allow_max_dynamic_smem(moe_prepare_kernel, smem_optin)) != QUINTRIT_OK ||
            (rc = allow_max_dynamic_smem(moe_act_quant_kernel, smem_optin)) != QUINTRIT_OK)
            return rc;
        quintrit_b200_moe* m = new quintrit_b200_moe();
        m->magic = kMagicMoe, m->device = static_cast<int>(device_index), m->sm_count = prop.multiProcessorCount;
        m->hidden = static_cast<int>(hidden), m->inter = static_cast<int>(inter), m->inter_pad = static_cast<int>((inter + 15) / 16 * 16);
        m->n_experts = static_cast<int>(n_experts), m->top_k = static_cast<int>(top_k), m->max_batch = static_cast<int>(max_batch);
        m->expert_first = static_cast<int>(expert_first), m->expert_count = static_cast<int>(expert_count);
        const int tiles_d = (m->hidden + kTileRows - 1) / kTileRows;
        m->chunks_down = std::max(1, tiles_d / 32);  // down items of about 32 row tiles
        const size_t B = max_batch, Z = B * top_k, H = hidden, I = inter, E = n_experts;
        const size_t pairs_gu = ((H + kBlockTrits - 1) / kBlockTrits + 1) / 2, pairs_d = ((I + kBlockTrits - 1) / kBlockTrits + 1) / 2;
        auto bail = [&](int code) {
            destroy_moe(m);
            return code;
        };
        if ((rc = moe_alloc(m, &m->router, E * H)) != QUINTRIT_OK || (rc = moe_alloc(m, &m->experts, E)) != QUINTRIT_OK || (rc = moe_alloc(m, &m->x, B * H)) != QUINTRIT_OK ||
            (rc = moe_alloc(m, &m->x16, B * H)) != QUINTRIT_OK || (rc = moe_alloc(m, &m->a8_x, B * H + 256)) != QUINTRIT_OK || (rc = moe_alloc(m, &m->s_x, B)) != QUINTRIT_OK ||
            (rc = moe_alloc(m, &m->logits, B * E)) != QUINTRIT_OK || (rc = moe_alloc(m, &m->probs, B * E)) != QUINTRIT_OK || (rc = moe_alloc(m, &m->chosen, Z)) != QUINTRIT_OK ||
            (rc = moe_alloc(m, &m->weights, Z)) != QUINTRIT_OK || (rc = moe_alloc(m, &m->tie, B)) != QUINTRIT_OK || (rc = moe_alloc(m, &m->counters, 4)) != QUINTRIT_OK ||
            (rc = moe_alloc(m, &m->acc_gu, Z * 2 * I)) != QUINTRIT_OK || (rc = moe_alloc(m, &m->a8_i, Z * m->inter_pad + 256)) != QUINTRIT_OK || (rc = moe_alloc(m, &m->s_i, Z)) != QUINTRIT_OK ||
            (rc = moe_alloc(m, &m->acc_down, Z * H)) != QUINTRIT_OK || (rc = moe_alloc(m, &m->out, B * H)) != QUINTRIT_OK || (rc = moe_alloc(m, &m->gu_items, Z * pairs_gu)) != QUINTRIT_OK ||
            (rc = moe_alloc(m, &m->down_items, Z * pairs_d * m->chunks_down)) != QUINTRIT_OK || (rc = moe_alloc(m, &m->local_z, Z)) != QUINTRIT_OK ||
            (rc = moe_alloc(m, &m->pairs, Z * H)) != QUINTRIT_OK)
            return bail(rc);
        cudaError_t e = cudaMemcpy(m->router, router_bf16, E * H * sizeof(uint16_t), cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaMemcpy(m->experts, refs.data(), E * sizeof(MoeExpertRef), cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            destroy_moe(m);
            return cuda_fail(e, "set-up of the mixture-of-experts block");
        }
        *out_moe = m;
        return ok();
    });
}

extern "C" void quintrit_b200_moe_free(quintrit_b200_moe_t* moe) {
    if (moe == nullptr || moe->magic != kMagicMoe) return;
    destroy_moe(moe);
}

extern "C" int quintrit_b200_moe_create(uint32_t device_index, uint32_t hidden, uint32_t inter, uint32_t n_experts, uint32_t top_k, uint32_t max_batch, const uint16_t* router_bf16,
                                        const quintrit_b200_matrix_t* const* gate_up, const quintrit_b200_matrix_t* const* down, const float* scales,
                                        quintrit_b200_moe_t** out_moe) {
    return quintrit_b200_moe_create_shard(device_index, hidden, inter, n_experts, top_k, max_batch, router_bf16, 0, n_experts, gate_up, down, scales, out_moe);
}

namespace {
int moe_check_batch(quintrit_b200_moe* m, size_t batch) {
    if (batch == 0 || batch > static_cast<size_t>(m->max_batch)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "a batch of %zu tokens (the block was made for 1 to %d)", batch, m->max_batch);
    return QUINTRIT_OK;
}
}  // namespace

extern "C" int quintrit_b200_moe_forward(quintrit_b200_moe_t* moe, const float* x, size_t batch, float* out, uint32_t* out_experts, float* out_weights) {
    return guard([&]() -> int {
        int rc = check_moe(moe);
        if (rc != QUINTRIT_OK) return rc;
        if (x == nullptr || out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "x or out is NULL");
        if ((rc = moe_check_batch(moe, batch)) != QUINTRIT_OK) return rc;
        if (moe->expert_count != moe->n_experts) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "this block holds experts %d .. %d of %d: run quintrit_b200_moe_forward_partial, add the pairs of all GPUs, then quintrit_b200_moe_finish", moe->expert_first, moe->expert_first + moe->expert_count, moe->n_experts);
        DeviceGuard g(moe->device);
        if ((rc = moe_partial(moe, x, batch)) != QUINTRIT_OK) return rc;
        if ((rc = moe_finish(moe, batch, out, out_experts, out_weights)) != QUINTRIT_OK) return rc;
        return ok();
    });
}

extern "C" int quintrit_b200_moe_forward_partial(quintrit_b200_moe_t* moe, const float* x, size_t batch) {
    return guard([&]() -> int {
        int rc = check_moe(moe);
        if (rc != QUINTRIT_OK) return rc;
        if (x == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "x is NULL");
        if ((rc = moe_check_batch(moe, batch)) != QUINTRIT_OK) return rc;
        DeviceGuard g(moe->device);
        if ((rc = moe_partial(moe, x, batch)) != QUINTRIT_OK) return rc;
        return ok();
    });
}

extern "C" int quintrit_b200_moe_pairs(quintrit_b200_moe_t* moe, void** out_device_pointer, size_t* out_floats) {
    return guard([&]() -> int {
        int rc = check_moe(moe);
        if (rc != QUINTRIT_OK) return rc;
        if (out_device_pointer == nullptr || out_floats == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_device_pointer or out_floats is NULL");
        *out_device_pointer = moe->pairs;
        *out_floats = size_t(moe->last_batch) * moe->top_k * moe->hidden;
        return ok();
    });
}

extern "C" int quintrit_b200_moe_finish(quintrit_b200_moe_t* moe, size_t batch, float* out, uint32_t* out_experts, float* out_weights) {
    return guard([&]() -> int {
        int rc = check_moe(moe);
        if (rc != QUINTRIT_OK) return rc;
        if (out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out is NULL");
        if (batch == 0 || batch != static_cast<size_t>(moe->last_batch)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "the last partial forward held %d tokens, not %zu", moe->last_batch, batch);
        DeviceGuard g(moe->device);
        if ((rc = moe_finish(moe, batch, out, out_experts, out_weights)) != QUINTRIT_OK) return rc;
        return ok();
    });
}

extern "C" int quintrit_b200_moe_time(quintrit_b200_moe_t* moe, size_t batch, uint32_t repeats, float* out_ms) {
    return guard([&]() -> int {
        int rc = check_moe(moe);
        if (rc != QUINTRIT_OK) return rc;
        quintrit_b200_moe* m = moe;
        if (out_ms == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_ms is NULL");
        if (repeats == 0 || batch == 0 || batch != static_cast<size_t>(m->last_batch)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "the block is timed on the batch of its last forward (%d tokens), at least once", m->last_batch);
        DeviceGuard g(m->device);
        cudaEvent_t e0, e1;
        QTB_CUDA(cudaEventCreate(&e0));
        QTB_CUDA(cudaEventCreate(&e1));
        QTB_CUDA(cudaEventRecord(e0, m->stream));
        for (uint32_t r = 0; r < repeats && rc == QUINTRIT_OK; ++r) {
            rc = moe_enqueue(m, static_cast<int>(batch));
            if (rc == QUINTRIT_OK) rc = moe_enqueue_experts(m, static_cast<int>(batch));
            if (rc == QUINTRIT_OK) rc = moe_enqueue_combine(m, static_cast<int>(batch));
        }
        cudaEventRecord(e1, m->stream);
        cudaError_t e = cudaStreamSynchronize(m->stream);
        float ms = 0.0f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        if (rc != QUINTRIT_OK) return rc;
        if (e != cudaSuccess) return cuda_fail(e, "timing of the mixture-of-experts block");
        *out_ms = ms / static_cast<float>(repeats);
        return ok();
    });
}

// ---- the device sampler on logits the caller holds -----------------------------------------------------------------------------------
extern "C" int quintrit_b200_sample_logits(uint32_t device_index, const float* logits, size_t count, float temperature, uint32_t top_k, float top_p, uint64_t* state,
                                           uint32_t* out_token) {
    return guard([&]() -> int {
        if (logits == nullptr || state == nullptr || out_token == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "logits, state or out_token is NULL");
        if (!(temperature > 0.0f) || !std::isfinite(temperature)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "temperature must be finite and positive");
        if (!(top_p > 0.0f && top_p <= 1.0f)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "top_p must be in (0, 1]");
        if (top_k < 1 || top_k > static_cast<uint32_t>(kSampleMaxK) || top_k >= count)
            return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "top_k %u must be in [1, %d] and below the number of logits (%zu)", top_k, kSampleMaxK, count);
        if (count > (size_t(1) << 24)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "at most 2^24 logits");
        if (*state == 0) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "the generator state must not be zero (a zero state never leaves zero)");
        cudaDeviceProp prop;
        int rc = require_b200(static_cast<int>(device_index), &prop);
        if (rc != QUINTRIT_OK) return rc;
        DeviceGuard g(static_cast<int>(device_index));
        if ((rc = upload_exp2_table()) != QUINTRIT_OK) return rc;
        unsigned char* buf = nullptr;
        QTB_CUDA(cudaMalloc(&buf, count * sizeof(float) + 16));
        float* d_logits = reinterpret_cast<float*>(buf + 16);
        unsigned long long* d_rng = reinterpret_cast<unsigned long long*>(buf);
        uint32_t* d_tok = reinterpret_cast<uint32_t*>(buf + 8);
        cudaError_t e = cudaMemcpy(d_logits, logits, count * sizeof(float), cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaMemcpy(d_rng, state, sizeof(uint64_t), cudaMemcpyHostToDevice);
        if (e == cudaSuccess) {
            sample_topk_kernel<<<1, kSampleThreads>>>(d_logits, static_cast<int>(count), temperature, static_cast<int>(top_k), top_p, d_rng, d_tok);
            ++g_launches;
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaMemcpy(state, d_rng, sizeof(uint64_t), cudaMemcpyDeviceToHost);
        if (e == cudaSuccess) e = cudaMemcpy(out_token, d_tok, sizeof(uint32_t), cudaMemcpyDeviceToHost);
        cudaFree(buf);
        if (e != cudaSuccess) return cuda_fail(e, "device sampler");
        return ok();
    });
}

// ---- several sequences decoded together: one pass of the batched projections per step ----------------------------------------------
struct quintrit_b200_batch {
    uint32_t magic;
    quintrit_b200_decoder* d;              // weights, stream and the per-token buffers of the batched pass are the decoder's
    int device;                            // (kept here too: releasing the batch must not read a decoder that was freed first)
    int n_seq;
    __half *kc = nullptr, *vc = nullptr;   // [n_seq][layers][ctx][kv_dim]
    uint32_t *d_pos = nullptr, *d_last = nullptr, *d_slot = nullptr, *d_chosen = nullptr;
    float* logits = nullptr;               // [n_seq][vocab] of the last step
    __half* x16 = nullptr;                 // [n_seq][hidden]: the final norm's output
    std::vector<uint32_t> host_pos;        // tokens cached per sequence
    std::vector<uint32_t> staged;          // host copy of the ids given to an asynchronous copy
    std::vector<void*> allocs;
    // The launches of a step of n tokens (about 500 for 40 layers) are replayed as one CUDA graph from the third step of that size on: tokens,
    // sequence list and positions are read from device memory, so the graph of a size serves every step of that size.
    std::vector<cudaGraphExec_t> graph;    // [n_seq + 1], nullptr until captured
    std::vector<char> warm;                // a step of that size has run as plain launches (lazy allocations done)
};

namespace {

constexpr uint32_t kMagicBatch = 0x51544242u;  // "QTBB"

int check_batch(const quintrit_b200_batch* b) {
    if (b == nullptr || b->magic != kMagicBatch) return fail(QUINTRIT_ERR_INVALID_HANDLE, "batch handle is NULL, freed or of the wrong type");
    return check_decoder(b->d);
}

void destroy_batch(quintrit_b200_batch* b) {
    if (b == nullptr) return;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(b->device);
    for (cudaGraphExec_t g : b->graph)
        if (g != nullptr) cudaGraphExecDestroy(g);
    for (void* p : b->allocs) cudaFree(p);
    if (prev >= 0) cudaSetDevice(prev);
    b->magic = 0;
    delete b;
}

template <typename T>
int batch_alloc(quintrit_b200_batch* b, T** p, size_t count) {
    void* q = nullptr;
    const size_t bytes = std::max<size_t>(count * sizeof(T), 16);
    cudaError_t e = cudaMalloc(&q, bytes);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(batch buffer)");
    b->allocs.push_back(q);
    if ((e = cudaMemset(q, 0, bytes)) != cudaSuccess) return cuda_fail(e, "cudaMemset(batch buffer)");
    *p = static_cast<T*>(q);
    return QUINTRIT_OK;
}

size_t batch_cache_stride(const quintrit_b200_decoder* d) { return static_cast<size_t>(d->layers) * d->ctx * d->kv_dim; }

// The output head for the n tokens of a step: final norm per token, then every vocabulary row against all tokens, then the greedy choice per token.
int batch_head(quintrit_b200_batch* b, int n) {
    quintrit_b200_decoder* d = b->d;
    cudaStream_t s = d->stream;
    const int H = d->hidden;
    NormQuantArgs nf{};
    nf.x = d->pf.x, nf.b_x = H, nf.acc_prev = d->pf.acc_down, nf.b_acc = H, nf.scale_prev = d->pf.s_i, nf.b_scale = 1;
    nf.ws_prev = d->scales[(d->layers - 1) * 7 + 6], nf.norm_w = d->out_norm, nf.eps = d->eps, nf.n = H;
    nf.y16_out = b->x16, nf.b_y16 = H, nf.y16_bf16 = d->bf16_tables;
    norm_quant_kernel<<<dim3(1, 1, n), kRowThreads, H * sizeof(float), s>>>(nf);
    QTB_LAUNCH_CHECK();
    if (H % 128 == 0 && lm_head_batch_smem(H) <= 200 * 1024) {
        lm_head_batch_kernel<<<dim3(d->sm_count, (n + kHeadTokens - 1) / kHeadTokens), kHeadThreads, lm_head_batch_smem(H), s>>>(d->lm_head, b->x16, H, d->vocab, n, b->logits,
                                                                                                                                  d->bf16_tables);
        QTB_LAUNCH_CHECK();
    } else {  // a hidden size the grouped kernel does not take: token by token
        for (int t = 0; t < n; ++t) {
            lm_head_kernel<<<d->sm_count * 8, 256, H * sizeof(float), s>>>(d->lm_head, b->x16 + size_t(t) * H, H, d->vocab, b->logits + size_t(t) * d->vocab, d->bf16_tables);
            QTB_LAUNCH_CHECK();
        }
    }
    argmax_kernel<<<n, 1024, 0, s>>>(b->logits, d->vocab, b->d_chosen);
    QTB_LAUNCH_CHECK();
    return QUINTRIT_OK;
}

}  // namespace

extern "C" int quintrit_b200_batch_create(quintrit_b200_decoder_t* decoder, uint32_t sequences, quintrit_b200_batch_t** out_batch) {
    return guard([&]() -> int {
        if (out_batch == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out_batch is NULL");
        *out_batch = nullptr;
        int rc = check_decoder(decoder);
        if (rc != QUINTRIT_OK) return rc;
        quintrit_b200_decoder* d = decoder;
        if (sequences == 0 || sequences > static_cast<uint32_t>(kPrefillMax)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "sequences must be in [1, %d], got %u", kPrefillMax, sequences);
        if (!prefill_available(d)) return fail(QUINTRIT_ERR_UNSUPPORTED, "this decoder has no batched pass (block-scaled or tensor-parallel model)");
        DeviceGuard g(d->device);
        if ((rc = prefill_buffers(d)) != QUINTRIT_OK) return rc;
        if ((rc = decoder_gemm_prepare(d)) != QUINTRIT_OK) return rc;
        quintrit_b200_batch* b = new quintrit_b200_batch();
        b->magic = kMagicBatch, b->d = d, b->device = d->device, b->n_seq = static_cast<int>(sequences);
        b->host_pos.assign(sequences, 0);
        b->graph.assign(sequences + 1, nullptr);
        b->warm.assign(sequences + 1, 0);
        const size_t n = sequences;
        if ((rc = batch_alloc(b, &b->kc, n * batch_cache_stride(d))) != QUINTRIT_OK || (rc = batch_alloc(b, &b->vc, n * batch_cache_stride(d))) != QUINTRIT_OK ||
            (rc = batch_alloc(b, &b->d_pos, n)) != QUINTRIT_OK || (rc = batch_alloc(b, &b->d_last, n)) != QUINTRIT_OK || (rc = batch_alloc(b, &b->d_slot, n)) != QUINTRIT_OK ||
            (rc = batch_alloc(b, &b->d_chosen, n)) != QUINTRIT_OK || (rc = batch_alloc(b, &b->logits, n * d->vocab)) != QUINTRIT_OK ||
            (rc = batch_alloc(b, &b->x16, n * d->hidden)) != QUINTRIT_OK) {
            destroy_batch(b);
            return rc;
        }
        *out_batch = b;
        return ok();
    });
}

extern "C" void quintrit_b200_batch_free(quintrit_b200_batch_t* batch) {
    if (batch == nullptr || batch->magic != kMagicBatch) return;
    destroy_batch(batch);
}

extern "C" int quintrit_b200_batch_info(const quintrit_b200_batch_t* batch, uint32_t* out_sequences, uint32_t* out_context, uint32_t* out_positions, size_t positions_capacity) {
    return guard([&]() -> int {
        int rc = check_batch(batch);
        if (rc != QUINTRIT_OK) return rc;
        if (out_sequences) *out_sequences = static_cast<uint32_t>(batch->n_seq);
        if (out_context) *out_context = static_cast<uint32_t>(batch->d->ctx);
        if (out_positions != nullptr) {
            if (positions_capacity < static_cast<size_t>(batch->n_seq)) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "positions hold %zu values, the batch has %d sequences", positions_capacity, batch->n_seq);
            std::copy(batch->host_pos.begin(), batch->host_pos.end(), out_positions);
        }
        return ok();
    });
}

extern "C" int quintrit_b200_batch_rewind(quintrit_b200_batch_t* batch, uint32_t sequence, uint32_t position) {
    return guard([&]() -> int {
        int rc = check_batch(batch);
        if (rc != QUINTRIT_OK) return rc;
        if (sequence >= static_cast<uint32_t>(batch->n_seq)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "sequence %u of %d", sequence, batch->n_seq);
        if (position > batch->host_pos[sequence]) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "position %u skips positions: %u tokens are cached", position, batch->host_pos[sequence]);
        DeviceGuard g(batch->d->device);
        QTB_CUDA(cudaMemcpyAsync(batch->d_pos + sequence, &position, sizeof position, cudaMemcpyHostToDevice, batch->d->stream));
        QTB_CUDA(cudaStreamSynchronize(batch->d->stream));
        batch->host_pos[sequence] = position;
        return ok();
    });
}

extern "C" int quintrit_b200_batch_prefill(quintrit_b200_batch_t* batch, uint32_t sequence, const uint32_t* tokens, size_t count, float* logits, size_t logits_capacity,
                                           uint32_t* out_token) {
    return guard([&]() -> int {
        int rc = check_batch(batch);
        if (rc != QUINTRIT_OK) return rc;
        quintrit_b200_batch* b = batch;
        quintrit_b200_decoder* d = b->d;
        if (tokens == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "tokens is NULL");
        if (count == 0) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "no tokens to ingest");
        if (sequence >= static_cast<uint32_t>(b->n_seq)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "sequence %u of %d", sequence, b->n_seq);
        const uint32_t pos = b->host_pos[sequence];
        if (size_t(pos) + count > static_cast<size_t>(d->ctx)) return fail(QUINTRIT_ERR_CONTEXT_OVERFLOW, "%zu tokens from position %u do not fit the context window of %d tokens", count, pos, d->ctx);
        for (size_t i = 0; i < count; ++i)
            if (tokens[i] >= static_cast<uint32_t>(d->vocab_full)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "token id %u is not below the vocabulary size %d", tokens[i], d->vocab_full);
        if (logits != nullptr && logits_capacity < static_cast<size_t>(d->vocab)) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "logits hold %zu values, the vocabulary has %d", logits_capacity, d->vocab);
        DeviceGuard g(d->device);
        b->staged.assign(tokens, tokens + count);
        BatchTarget tg;
        tg.kc = b->kc + sequence * batch_cache_stride(d), tg.vc = b->vc + sequence * batch_cache_stride(d), tg.pos = d->pf.pos, tg.own = false;
        if ((rc = decoder_prefill(d, b->staged.data(), count, pos, &tg)) != QUINTRIT_OK) return rc;
        const uint32_t next = pos + static_cast<uint32_t>(count);
        QTB_CUDA(cudaMemcpyAsync(b->d_pos + sequence, &next, sizeof next, cudaMemcpyHostToDevice, d->stream));
        QTB_CUDA(cudaMemcpyAsync(b->d_last + sequence, d->d_token, sizeof(uint32_t), cudaMemcpyDeviceToDevice, d->stream));
        if (logits) QTB_CUDA(cudaMemcpyAsync(logits, d->logits, size_t(d->vocab) * sizeof(float), cudaMemcpyDeviceToHost, d->stream));
        if (out_token) QTB_CUDA(cudaMemcpyAsync(out_token, d->d_token, sizeof(uint32_t), cudaMemcpyDeviceToHost, d->stream));
        if ((rc = decoder_check_status(d)) != QUINTRIT_OK) return rc;
        b->host_pos[sequence] = next;
        return ok();
    });
}

extern "C" int quintrit_b200_batch_step(quintrit_b200_batch_t* batch, const uint32_t* sequences, size_t count, const uint32_t* tokens, uint32_t* out_tokens, float* logits,
                                        size_t logits_capacity) {
    return guard([&]() -> int {
        int rc = check_batch(batch);
        if (rc != QUINTRIT_OK) return rc;
        quintrit_b200_batch* b = batch;
        quintrit_b200_decoder* d = b->d;
        if (sequences == nullptr) count = static_cast<size_t>(b->n_seq);
        if (count == 0 || count > static_cast<size_t>(b->n_seq)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "a step takes 1 to %d sequences, got %zu", b->n_seq, count);
        const int n = static_cast<int>(count);
        std::vector<char> seen(static_cast<size_t>(b->n_seq), 0);
        for (int z = 0; z < n; ++z) {
            const uint32_t sq = sequences != nullptr ? sequences[z] : static_cast<uint32_t>(z);
            if (sq >= static_cast<uint32_t>(b->n_seq)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "sequence %u of %d", sq, b->n_seq);
            if (seen[sq]) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "sequence %u is listed twice", sq);
            seen[sq] = 1;
            if (b->host_pos[sq] >= static_cast<uint32_t>(d->ctx)) return fail(QUINTRIT_ERR_CONTEXT_OVERFLOW, "sequence %u has filled the context window of %d tokens", sq, d->ctx);
            if (tokens == nullptr && b->host_pos[sq] == 0) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "sequence %u has no previous token to continue from", sq);
            if (tokens != nullptr && tokens[z] >= static_cast<uint32_t>(d->vocab_full)) return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "token id %u is not below the vocabulary size %d", tokens[z], d->vocab_full);
        }
        if (logits != nullptr && logits_capacity < count * static_cast<size_t>(d->vocab)) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "logits hold %zu values, %zu are needed", logits_capacity, count * static_cast<size_t>(d->vocab));
        DeviceGuard g(d->device);
        cudaStream_t s = d->stream;
        // the ids of both copies below, complete before the first copy is enqueued; the sequence list is always read from device memory (one
        // graph per step size), so "all sequences in order" is written out
        // Inside the step the tokens are ordered by the length of their sequences, longest first: the attention blocks of a launch are handed to the
        // multiprocessors in order, and with that order every multiprocessor gets long and short ones alike. order[k] = the caller's index z.
        std::vector<uint32_t> order(count);
        for (size_t z = 0; z < count; ++z) order[z] = static_cast<uint32_t>(z);
        auto seq_at = [&](uint32_t z) { return sequences != nullptr ? sequences[z] : z; };
        std::stable_sort(order.begin(), order.end(), [&](uint32_t x, uint32_t y) { return b->host_pos[seq_at(x)] > b->host_pos[seq_at(y)]; });
        b->staged.resize(count * (tokens != nullptr ? 2 : 1));
        for (size_t k = 0; k < count; ++k) {
            b->staged[k] = seq_at(order[k]);
            if (tokens != nullptr) b->staged[count + k] = tokens[order[k]];
        }
        const uint32_t* slot = b->d_slot;
        QTB_CUDA(cudaMemcpyAsync(b->d_slot, b->staged.data(), count * sizeof(uint32_t), cudaMemcpyHostToDevice, s));
        if (tokens != nullptr) {
            QTB_CUDA(cudaMemcpyAsync(d->pf.tokens, b->staged.data() + count, count * sizeof(uint32_t), cudaMemcpyHostToDevice, s));
        } else {
            gather_tokens_kernel<<<(n + 255) / 256, 256, 0, s>>>(d->pf.tokens, b->d_last, slot, n);
            QTB_LAUNCH_CHECK();
        }
        BatchTarget tg;
        tg.kc = b->kc, tg.vc = b->vc, tg.pos = b->d_pos, tg.own = false;
        tg.seq.slot = slot, tg.seq.pos_stride = 1, tg.seq.cache_stride = batch_cache_stride(d);
        auto enqueue = [&]() -> int {
            int r = prefill_layers(d, n, tg);
            if (r == QUINTRIT_OK) r = batch_head(b, n);
            if (r != QUINTRIT_OK) return r;
            advance_batch_kernel<<<(n + 255) / 256, 256, 0, s>>>(b->d_pos, b->d_last, b->d_chosen, slot, n);
            QTB_LAUNCH_CHECK();
            return QUINTRIT_OK;
        };
        if (b->graph[n] != nullptr) {
            QTB_CUDA(cudaGraphLaunch(b->graph[n], s));
        } else if (b->warm[n] && std::getenv("QUINTRIT_B200_BATCH_GRAPH_OFF") == nullptr) {
            cudaGraph_t g = nullptr;
            QTB_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
            rc = enqueue();
            const cudaError_t e = cudaStreamEndCapture(s, &g);
            if (rc != QUINTRIT_OK) {
                if (g) cudaGraphDestroy(g);
                return rc;
            }
            if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture(batch step)");
            const cudaError_t ei = cudaGraphInstantiate(&b->graph[n], g, 0);
            cudaGraphDestroy(g);
            if (ei != cudaSuccess) {
                b->graph[n] = nullptr;
                return cuda_fail(ei, "cudaGraphInstantiate(batch step)");
            }
            QTB_CUDA(cudaGraphLaunch(b->graph[n], s));
        } else {
            if ((rc = enqueue()) != QUINTRIT_OK) return rc;
            b->warm[n] = 1;
        }
        std::vector<uint32_t> chosen(out_tokens != nullptr ? count : 0);
        if (out_tokens) QTB_CUDA(cudaMemcpyAsync(chosen.data(), b->d_chosen, count * sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
        if (logits)
            for (size_t k = 0; k < count; ++k)
                QTB_CUDA(cudaMemcpyAsync(logits + size_t(order[k]) * d->vocab, b->logits + k * d->vocab, size_t(d->vocab) * sizeof(float), cudaMemcpyDeviceToHost, s));
        if ((rc = decoder_check_status(d)) != QUINTRIT_OK) return rc;  // (waits for the stream)
        if (out_tokens)
            for (size_t k = 0; k < count; ++k) out_tokens[order[k]] = chosen[k];
        for (int z = 0; z < n; ++z) b->host_pos[sequences != nullptr ? sequences[z] : static_cast<uint32_t>(z)] += 1;
        return ok();
    });
}

#ifdef QTB_GEMM_TRACE
extern "C" int quintrit_b200_debug_gemm_trace(quintrit_b200_matrix_t* m, long long* out) {  // debug builds: 4 roles x 4 events x 16 blocks of cycle stamps
    cudaDeviceSynchronize();
    return cudaMemcpy(out, m->d_gemm_status + 64, 4 * 4 * 16 * sizeof(long long), cudaMemcpyDeviceToHost);
}
#endif

#include "runtime.cuh"
