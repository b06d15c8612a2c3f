#include "common.hpp"

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace b200 {

namespace {
std::mutex g_err_mu;
char g_err_buf[4096] = "";

std::mutex g_dev_mu;
DeviceInfo g_dev[64];
bool g_dev_ready[64] = {false};

std::atomic<int*> g_status_host{nullptr};
std::mutex g_status_mu;
}  // namespace

void set_last_error(const std::string& msg) {
    std::lock_guard<std::mutex> lock(g_err_mu);
    std::snprintf(g_err_buf, sizeof(g_err_buf), "%s", msg.c_str());
    if (log_enabled()) std::fprintf(stderr, "[diopi_b200] error: %s\n", g_err_buf);
}

const char* last_error_cstr() {
    // The buffer is static; a reader racing with a writer sees a torn but terminated string.
    return g_err_buf;
}

void fail(diopiError_t code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    std::vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    throw OpError(code, buf);
}

Options& options() {
    static Options o = [] {
        auto on = [](const char* name) {
            const char* v = std::getenv(name);
            return (v && v[0] && v[0] != '0') ? 1 : 0;
        };
        Options x;
        x.log = on("DIOPI_B200_LOG");
        x.fuse_token_attention = on("DIOPI_B200_FUSE_TOKEN_ATTENTION");
        x.decode_plain = on("DIOPI_B200_DECODE_PLAIN");
        x.prefill_simt = on("DIOPI_B200_PREFILL_SIMT");
        return x;
    }();
    return o;
}

bool set_option(const char* name, int64_t value) {
    if (name == nullptr) return false;
    Options& o = options();
    const int v = value != 0 ? 1 : 0;
    if (std::strcmp(name, "log") == 0) o.log = v;
    else if (std::strcmp(name, "fuse_token_attention") == 0) o.fuse_token_attention = v;
    else if (std::strcmp(name, "decode_plain") == 0) o.decode_plain = v;
    else if (std::strcmp(name, "prefill_simt") == 0) o.prefill_simt = v;
    else return false;
    return true;
}

bool log_enabled() { return options().log != 0; }

void logf(const char* fmt, ...) {
    if (!log_enabled()) return;
    va_list ap;
    va_start(ap, fmt);
    std::fputs("[diopi_b200] ", stderr);
    std::vfprintf(stderr, fmt, ap);
    std::fputc('\n', stderr);
    va_end(ap);
}

bool TensorView::contiguous() const { return inner_contiguous(ndim); }

bool TensorView::inner_contiguous(int n) const {
    int64_t expect = 1;
    for (int i = ndim - 1; i >= ndim - n && i >= 0; --i) {
        if (shape[i] != 1 && stride[i] != expect) return false;
        expect *= shape[i];
    }
    return true;
}

int64_t TensorView::elem_size() const { return dtype_size(dtype); }

int64_t dtype_size(diopiDtype_t dt) {
    switch (dt) {
        case diopi_dtype_int8:
        case diopi_dtype_uint8:
        case diopi_dtype_bool: return 1;
        case diopi_dtype_int16:
        case diopi_dtype_uint16:
        case diopi_dtype_float16:
        case diopi_dtype_bfloat16: return 2;
        case diopi_dtype_int32:
        case diopi_dtype_uint32:
        case diopi_dtype_float32: return 4;
        case diopi_dtype_int64:
        case diopi_dtype_uint64:
        case diopi_dtype_float64: return 8;
        default: return 0;
    }
}

bool is_float_dtype(diopiDtype_t dt) {
    return dt == diopi_dtype_float16 || dt == diopi_dtype_bfloat16 || dt == diopi_dtype_float32 || dt == diopi_dtype_float64;
}

bool is_index_dtype(diopiDtype_t dt) { return dt == diopi_dtype_int32 || dt == diopi_dtype_int64; }

const char* dtype_name(diopiDtype_t dt) {
    switch (dt) {
        case diopi_dtype_int8: return "int8";
        case diopi_dtype_uint8: return "uint8";
        case diopi_dtype_int16: return "int16";
        case diopi_dtype_uint16: return "uint16";
        case diopi_dtype_int32: return "int32";
        case diopi_dtype_uint32: return "uint32";
        case diopi_dtype_int64: return "int64";
        case diopi_dtype_uint64: return "uint64";
        case diopi_dtype_float16: return "float16";
        case diopi_dtype_float32: return "float32";
        case diopi_dtype_float64: return "float64";
        case diopi_dtype_bool: return "bool";
        case diopi_dtype_bfloat16: return "bfloat16";
        default: return "unsupported";
    }
}

TensorView view_of(diopiConstTensorHandle_t h, const char* name, bool optional) {
    TensorView tv;
    if (h == nullptr) {
        if (optional) return tv;
        fail(diopiErrorOccurred, "tensor '%s' is a null handle", name);
    }
    diopiSize_t shape{nullptr, 0}, stride{nullptr, 0};
    if (diopiGetTensorShape(h, &shape) != diopiSuccess) fail(diopiErrorOccurred, "cannot read the shape of '%s'", name);
    if (diopiGetTensorStride(h, &stride) != diopiSuccess) fail(diopiErrorOccurred, "cannot read the strides of '%s'", name);
    if (diopiGetTensorDtype(h, &tv.dtype) != diopiSuccess) fail(diopiErrorOccurred, "cannot read the dtype of '%s'", name);
    if (shape.len > kMaxDims || shape.len < 0) fail(diopiErrorOccurred, "'%s' has %ld dims; at most %d are supported", name, (long)shape.len, kMaxDims);
    if (stride.len != shape.len) fail(diopiErrorOccurred, "'%s': %ld strides for %ld dims", name, (long)stride.len, (long)shape.len);
    tv.ndim = static_cast<int>(shape.len);
    tv.numel = 1;
    for (int i = 0; i < tv.ndim; ++i) {
        tv.shape[i] = shape.data[i];
        tv.stride[i] = stride.data[i];
        if (tv.shape[i] < 0) fail(diopiErrorOccurred, "'%s' has a negative extent", name);
        tv.numel *= tv.shape[i];
    }
    const void* p = nullptr;
    if (diopiGetTensorDataConst(h, &p) != diopiSuccess) fail(diopiErrorOccurred, "cannot read the data pointer of '%s'", name);
    tv.data = const_cast<void*>(p);
    if (tv.numel > 0 && tv.data == nullptr) fail(diopiErrorOccurred, "'%s' has %ld elements but a null data pointer", name, (long)tv.numel);
    if (diopiGetTensorDevice) {
        diopiDevice_t dev = diopi_device;
        if (diopiGetTensorDevice(h, &dev) == diopiSuccess && dev != diopi_device && tv.numel > 0)
            fail(diopiErrorOccurred, "'%s' lives in host memory; this backend takes device tensors only", name);
    }
    tv.defined = true;
    return tv;
}

cudaStream_t stream_of(diopiContextHandle_t ctx) {
    if (ctx == nullptr) fail(diopiErrorOccurred, "null context handle");
    diopiStreamHandle_t s = nullptr;
    if (diopiGetStream(ctx, &s) != diopiSuccess) fail(diopiErrorOccurred, "diopiGetStream failed");
    return static_cast<cudaStream_t>(s);
}

void* workspace(diopiContextHandle_t ctx, int64_t bytes) {
    diopiTensorHandle_t t = nullptr;
    diopiError_t rc;
    if (diopiRequireBuffer) {
        rc = diopiRequireBuffer(ctx, &t, bytes, diopi_device);
    } else {
        diopiSize_t size{&bytes, 1};
        rc = diopiRequireTensor(ctx, &t, &size, nullptr, diopi_dtype_int8, diopi_device);
    }
    if (rc != diopiSuccess || t == nullptr) fail(diopiErrorOccurred, "the consumer could not provide %ld bytes of device scratch", (long)bytes);
    void* p = nullptr;
    if (diopiGetTensorData(t, &p) != diopiSuccess || p == nullptr) fail(diopiErrorOccurred, "scratch tensor has no data pointer");
    return p;
}

const DeviceInfo& device_info() {
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) fail(diopiErrorOccurred, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_dev_mu);
    if (!g_dev_ready[dev]) {
        DeviceInfo di;
        di.device = dev;
        B200_CUDA(cudaDeviceGetAttribute(&di.sm_count, cudaDevAttrMultiProcessorCount, dev));
        B200_CUDA(cudaDeviceGetAttribute(&di.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        int major = 0;
        B200_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        if (major != 10) fail(diopiErrorOccurred, "this library holds sm_100a code only; device %d has compute capability %d.x", dev, major);
        g_dev[dev] = di;
        g_dev_ready[dev] = true;
    }
    return g_dev[dev];
}

// One 64-byte line per device, so that a status is attributed to the device whose kernel raised it.
constexpr int kStatusStrideInts = 16;
constexpr int kStatusDevices = 64;

int current_device_index() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStatusDevices) return 0;
    return dev;
}

int* async_status_device_ptr() {
    int* h = g_status_host.load(std::memory_order_acquire);
    if (!h) {
        std::lock_guard<std::mutex> lock(g_status_mu);
        h = g_status_host.load(std::memory_order_relaxed);
        if (!h) {
            // Portable + mapped: under unified addressing every device may store to the same pointer.
            const size_t bytes = static_cast<size_t>(kStatusDevices) * kStatusStrideInts * sizeof(int);
            B200_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&h), bytes, cudaHostAllocPortable | cudaHostAllocMapped));
            std::memset(h, 0, bytes);
            g_status_host.store(h, std::memory_order_release);
        }
    }
    return h + current_device_index() * kStatusStrideInts;
}

int* async_status_device_ptr_if_ready() {
    int* h = g_status_host.load(std::memory_order_acquire);
    return h ? h + current_device_index() * kStatusStrideInts : nullptr;
}

namespace {
thread_local int t_handled_code = 0;
}

// An op that fails with an error of its own for the very event a status stands for (a group refused because a kernel gave
// up) says so: neither the status its guard took nor one still in the word is reported a second time.
void clear_async_status_if(int code) {
    t_handled_code = code;
    int* h = async_status_device_ptr_if_ready();
    if (h && *reinterpret_cast<volatile int*>(h) == code) *reinterpret_cast<volatile int*>(h) = 0;
}

int drop_handled_status(int taken) {
    const int handled = t_handled_code;
    t_handled_code = 0;
    return taken == handled ? 0 : taken;
}

int take_async_status() {
    int* h = async_status_device_ptr_if_ready();
    if (!h) return 0;
    const int v = *reinterpret_cast<volatile int*>(h);
    if (v != 0) *reinterpret_cast<volatile int*>(h) = 0;
    return v;
}

void restore_async_status(int v) {
    int* h = async_status_device_ptr_if_ready();
    if (h && v != 0 && *reinterpret_cast<volatile int*>(h) == 0) *reinterpret_cast<volatile int*>(h) = v;
}

void fail_with_async_status(int v) {
    const char* what = "unknown";
    switch (v) {
        case 1: what = "a pool slot index read from b_loc or dest_loc was outside the pool; that row was skipped"; break;
        case 2: what = "a token id passed to diopiApplyPenalty was outside the vocabulary; that entry was skipped"; break;
        case 3: what = "a kernel gave up a bounded wait (its own memory pipeline, or the rows of a tensor-parallel peer)"; break;
        default: break;
    }
    fail(diopiErrorOccurred, "an earlier kernel of this library reported status %d: %s (this call itself was launched)", v, what);
}

}  // namespace b200
