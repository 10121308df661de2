// Error reporting, argument checks and handle tags shared by the C ABI entry points. The rules are those of the
// reference's C layer: thread-local last error (rust/crates/quintrit-c/src/error.rs:64-81, 149-157), nothing thrown
// across the ABI (error.rs:95-108), struct_size / NULL / handle-magic checks (quintrit-c/src/util.rs:10-183).
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>

#include <cuda_runtime.h>

#include "../../include/quintrit_b200.h"

namespace qtb {

struct LastError {
    int code = 0;
    std::string message;
};
inline LastError& last_error() {
    static thread_local LastError e;
    return e;
}
inline int ok() {
    LastError& e = last_error();
    e.code = 0;
    e.message.clear();
    return QUINTRIT_OK;
}
inline int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    LastError& e = last_error();
    e.code = code;
    e.message = buf;
    return code;
}
inline int cuda_fail(cudaError_t err, const char* what) {
    return fail(QUINTRIT_ERR_DEVICE, "CUDA device error in %s: %s", what, cudaGetErrorString(err));
}

#define QTB_CUDA(call)                                      \
    do {                                                    \
        cudaError_t qtb_err_ = (call);                      \
        if (qtb_err_ != cudaSuccess) return cuda_fail(qtb_err_, #call); \
    } while (0)

// Runs `body` and turns any C++ exception into QUINTRIT_ERR_INTERNAL (the guard of quintrit-c/src/error.rs:95-108).
template <typename F>
inline int guard(F&& body) {
    try {
        return body();
    } catch (const std::bad_alloc&) {
        return fail(QUINTRIT_ERR_INTERNAL, "out of host memory");
    } catch (const std::exception& e) {
        return fail(QUINTRIT_ERR_INTERNAL, "internal error: %s", e.what());
    } catch (...) {
        return fail(QUINTRIT_ERR_INTERNAL, "internal error");
    }
}

constexpr uint32_t kMagicMatrix = 0x5154424Du;  // "QTBM"
constexpr uint32_t kMagicPlan = 0x51544250u;    // "QTBP"

thread_local inline uint64_t g_launches = 0;

}  // namespace qtb
