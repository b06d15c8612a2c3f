// Host-side glue shared by every exported op: error reporting, a plain view of a
// tensor handle (read only through the consumer's accessors), stream and
// workspace lookup. Plays the role that impl/cuda/helper.hpp (DiopiTensor,
// getStream, DIOPI_CALL) plays in the reference's no-ATen demo backend.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <exception>
#include <string>

#include "diopi_b200.h"

#define B200_EXPORT extern "C" __attribute__((visibility("default")))

namespace b200 {

constexpr int kMaxDims = 8;

// Thrown inside an op; the guard turns it into a return code plus a message.
struct OpError : public std::exception {
    diopiError_t code;
    std::string msg;
    OpError(diopiError_t c, std::string m) : code(c), msg(std::move(m)) {}
    const char* what() const noexcept override { return msg.c_str(); }
};

[[noreturn]] void fail(diopiError_t code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

// Process-wide switches. Each starts from its environment variable, read once when the first op runs, and can be
// changed afterwards with diopiB200SetOption; no op reads the environment on its call path.
//   log                   DIOPI_B200_LOG                   one line per call on stderr
//   fuse_token_attention  DIOPI_B200_FUSE_TOKEN_ATTENTION  run the unfused pair of decode calls as the fused kernel
//   decode_plain          DIOPI_B200_DECODE_PLAIN          decode ops on the one-CTA-per-(request, head) kernel, no split-KV
//   prefill_simt          DIOPI_B200_PREFILL_SIMT          prefill on the SIMT kernel, not on the tensor-core one
struct Options {
    int log = 0, fuse_token_attention = 0, decode_plain = 0, prefill_simt = 0;
};
Options& options();
// Returns false when `name` is not one of the switches above.
bool set_option(const char* name, int64_t value);
void set_last_error(const std::string& msg);
bool log_enabled();
void logf(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

#define B200_REQUIRE(cond, ...)                                   \
    do {                                                          \
        if (!(cond)) ::b200::fail(diopiErrorOccurred, __VA_ARGS__); \
    } while (0)

#define B200_CUDA(expr)                                                                                   \
    do {                                                                                                  \
        cudaError_t e__ = (expr);                                                                         \
        if (e__ != cudaSuccess) ::b200::fail(diopiErrorOccurred, "cuda error: %s (%s)", cudaGetErrorString(e__), #expr); \
    } while (0)

struct TensorView {
    void* data = nullptr;
    diopiDtype_t dtype = diopi_dtype_unsupported;
    int ndim = 0;
    int64_t shape[kMaxDims] = {0};
    int64_t stride[kMaxDims] = {0};
    int64_t numel = 0;
    bool defined = false;

    int64_t size(int i) const { return shape[i < 0 ? i + ndim : i]; }
    int64_t str(int i) const { return stride[i < 0 ? i + ndim : i]; }
    bool contiguous() const;
    // True when the trailing `n` dims are laid out densely (row-major).
    bool inner_contiguous(int n) const;
    int64_t elem_size() const;
};

// Reads shape/stride/dtype/data of a handle. `name` is only used in messages.
// A null handle gives an undefined view when `optional` is set, else an error.
TensorView view_of(diopiConstTensorHandle_t h, const char* name, bool optional = false);

bool is_float_dtype(diopiDtype_t dt);
bool is_index_dtype(diopiDtype_t dt);
const char* dtype_name(diopiDtype_t dt);
int64_t dtype_size(diopiDtype_t dt);

cudaStream_t stream_of(diopiContextHandle_t ctx);

// Device scratch owned by the context (diopiRequireBuffer when the consumer has it,
// else a 1-D int8 diopiRequireTensor). Never freed by the library.
void* workspace(diopiContextHandle_t ctx, int64_t bytes);

struct DeviceInfo {
    int device = 0;
    int sm_count = 0;
    int max_smem_optin = 0;
};
// Properties of the current device, looked up once per device.
const DeviceInfo& device_info();

// One word per device in mapped pinned host memory that kernels write when they meet something they
// must refuse (an index outside the pool, a wait that ran out). Every op takes the word of the current
// device (reads and clears it, at no cost) when it is entered, runs its body, and only then reports a
// status it took, once, as its return code: a status left by an earlier kernel never keeps a later call
// from running (in a tensor-parallel layer a skipped call on one rank would leave its peers waiting),
// and a call never reports its own kernel, which may still be running.
int* async_status_device_ptr();
// The same word if an earlier call already set the block up, else null (kernels accept null). Never allocates.
int* async_status_device_ptr_if_ready();
int take_async_status();              // reads and clears the current device's status
void restore_async_status(int v);     // puts a taken status back (the op failed for a reason of its own)
[[noreturn]] void fail_with_async_status(int v);
int drop_handled_status(int taken);   // 0 when the op's body declared that status handled (clear_async_status_if), else `taken`
// Drops the current device's status when it is `code`: for an op that reports the same event through its own error.
void clear_async_status_if(int code);

// Runs `body`, mapping exceptions to return codes; nothing escapes the C boundary.
// `report_status` = false for housekeeping calls (options, context release): they must not use up a kernel's status, which
// belongs to the next op call.
template <typename F>
diopiError_t guard(const char* op, F&& body, bool report_status = true) noexcept {
    void* rec = nullptr;
    if (diopiRecordStart) diopiRecordStart(op, &rec);
    diopiError_t rc = diopiSuccess;
    int stale = 0;
    try {
        if (report_status) stale = take_async_status();
        body();
        if (stale != 0) {
            const int v = stale;
            stale = 0;
            fail_with_async_status(v);   // after the launch: see the comment at async_status_device_ptr
        }
    } catch (const OpError& e) {
        set_last_error(std::string(op) + ": " + e.msg);
        rc = e.code;
    } catch (const std::exception& e) {
        set_last_error(std::string(op) + ": " + e.what());
        rc = diopiErrorOccurred;
    } catch (...) {
        set_last_error(std::string(op) + ": unknown exception");
        rc = diopiErrorOccurred;
    }
    stale = drop_handled_status(stale);
    if (stale != 0) restore_async_status(stale);   // the body failed on its own: the status waits for the next call
    if (diopiRecordEnd && rec) diopiRecordEnd(&rec);
    return rc;
}

}  // namespace b200
