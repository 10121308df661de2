// C ABI of libquintrit_b200.so (declared in include/quintrit_b200.h): device queries, on-device transcode of ternary
// matrices into the stream layout, the exact GEMV with host or device buffers, and the persistent multi-GEMV plan.
// Host code is C++ over the CUDA runtime API; the reference's host side for the same seam is
// rust/crates/quintrit-cuda/src/{device.rs,gemv.rs,pack.rs} and rust/crates/quintrit-c/src/cuda.rs.
#include <algorithm>
#include <cstdlib>
#include <new>
#include <vector>

#include "capi_common.cuh"
#include "gemv_lut.cuh"
#include "transcode.cuh"

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
};

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
};

namespace {

const char* kVersion = "0.1.0";

int check_matrix(const quintrit_b200_matrix* m) {
    if (m == nullptr || m->magic != kMagicMatrix) return fail(QUINTRIT_ERR_INVALID_HANDLE, "matrix handle is NULL, freed or of the wrong type");
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
    if (dev < 0 || dev >= 64) return fail(QUINTRIT_ERR_DEVICE, "device index %d out of range", dev);
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
    m->magic = 0;
    delete m;
}

size_t source_bytes(int32_t source, size_t rows, size_t cols) {
    switch (source) {
        case kSrcPlanar: return rows * quintrit_b200_planar_row_bytes(cols);
        case kSrcI2S: return rows * cols / 4;
        case kSrcTq2: return rows * cols / 256 * 66;
        case kSrcTq1: return rows * cols / 256 * 54;
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
        if (source != kSrcPlanar && source != kSrcI2S && source != kSrcTq1 && source != kSrcTq2)
            return fail(QUINTRIT_ERR_INVALID_ARGUMENT, "unknown source encoding %d", source);
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
        int rc = check_matrix(matrix);
        if (rc != QUINTRIT_OK) return rc;
        destroy_matrix(matrix);
        return ok();
    });
}

extern "C" int quintrit_b200_matrix_info(const quintrit_b200_matrix_t* matrix, size_t* out_rows, size_t* out_cols, size_t* out_device_bytes) {
    return guard([&]() -> int {
        int rc = check_matrix(matrix);
        if (rc != QUINTRIT_OK) return rc;
        if (out_rows) *out_rows = matrix->rows;
        if (out_cols) *out_cols = matrix->cols;
        if (out_device_bytes) *out_device_bytes = matrix->w_bytes;
        return ok();
    });
}

extern "C" int quintrit_b200_matrix_download_planar(const quintrit_b200_matrix_t* matrix, uint8_t* out, size_t out_capacity) {
    return guard([&]() -> int {
        int rc = check_matrix(matrix);
        if (rc != QUINTRIT_OK) return rc;
        if (out == nullptr) return fail(QUINTRIT_ERR_NULL_POINTER, "out is NULL");
        const size_t need = matrix->rows * matrix->blocks * kBlockBytes;
        if (out_capacity < need) return fail(QUINTRIT_ERR_BUFFER_TOO_SMALL, "out holds %zu bytes, %zu are needed", out_capacity, need);
        DeviceGuard g(matrix->device);
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
// plans
// ---------------------------------------------------------------------------------------------------------------------

namespace {
void destroy_plan(quintrit_b200_plan* p) {
    if (p == nullptr) return;
    DeviceGuard g(p->device);
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
        if (tiles_per_item == 0) tiles_per_item = 64;
        for (size_t i = 0; i < count; ++i) {
            const quintrit_b200_matrix* m = matrices[i];
            p->act_off.push_back(act);
            p->out_off.push_back(out);
            p->rows.push_back(m->rows);
            p->cols.push_back(m->cols);
            build_items(items, m->d_w, act, out, m->rows, m->cols, m->blocks, m->tiles, tiles_per_item);
            act += (m->cols + 15) / 16 * 16;
            out += (m->rows + 3) / 4 * 4;
        }
        p->act_total = act;
        p->out_total = out;
        p->n_items = static_cast<int>(items.size());
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
        QTB_CUDA(cudaMemcpyAsync(plan->d_act, activations, plan->act_total, cudaMemcpyHostToDevice, 0));
        QTB_CUDA(cudaMemsetAsync(plan->d_out, 0, plan->out_total * sizeof(int32_t), 0));
        rc = launch_gemv(plan->d_items, plan->n_items, plan->d_act, plan->d_out, plan->d_counters, plan->sm_count, 0);
        if (rc != QUINTRIT_OK) return rc;
        QTB_CUDA(cudaMemcpyAsync(out, plan->d_out, plan->out_total * sizeof(int32_t), cudaMemcpyDeviceToHost, 0));
        unsigned int flag = 0;
        QTB_CUDA(cudaMemcpyAsync(&flag, plan->d_counters + 2, sizeof flag, cudaMemcpyDeviceToHost, 0));
        QTB_CUDA(cudaStreamSynchronize(0));
        if (flag != 0) return fail(QUINTRIT_ERR_DEVICE, "GEMV kernel on the CUDA device found its shared-memory table at an unexpected address");
        return ok();
    });
}

extern "C" uint64_t quintrit_b200_launch_count(int reset) {
    const uint64_t n = g_launches;
    if (reset) g_launches = 0;
    return n;
}
