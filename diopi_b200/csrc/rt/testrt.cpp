// A small consumer-side DIOPI run time, used by the tests and the benchmark to
// drive libdiopi_impl.so the way a framework would. It plays the part that
// diopi_test/diopi_stub/csrc/litert.cpp plays for the reference's conformance
// suite: it defines the accessor functions the backend imports
// (diopiGetTensorData, diopiGetStream, diopiRequireTensor, ...) and adds a few C
// helpers so that Python can wrap memory it already owns (a torch CUDA tensor's
// data_ptr, or a numpy array for host-only validation tests) in a tensor handle
// without a copy.
//
// Temporaries handed out through diopiRequireTensor/diopiRequireBuffer come from a
// per-context cache of device blocks: a block is reused once the context has been
// told (b200rt_context_release) that the work using it was enqueued; reuse is safe
// because all work of a context goes to one stream.
#include <cuda_runtime_api.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "diopi_b200.h"

#define RT_EXPORT extern "C" __attribute__((visibility("default")))

struct diopiTensor {
    std::vector<int64_t> shape;
    std::vector<int64_t> stride;
    diopiDtype_t dtype = diopi_dtype_float32;
    diopiDevice_t device = diopi_device;
    void* data = nullptr;
    int64_t numel = 0;
};

namespace {

struct Block {
    void* ptr = nullptr;
    int64_t bytes = 0;
    bool in_use = false;
    bool on_device = true;
};

int64_t elem_size(diopiDtype_t dt) {
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
        case diopi_dtype_float32:
        case diopi_dtype_tfloat32:
        case diopi_dtype_complex32: return 4;
        case diopi_dtype_int64:
        case diopi_dtype_uint64:
        case diopi_dtype_float64:
        case diopi_dtype_complex64: return 8;
        case diopi_dtype_complex128: return 16;
        default: return 0;
    }
}

}  // namespace

struct diopiContext {
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    bool stream_ready = false;
    std::vector<Block> blocks;
    std::vector<diopiTensor*> temps;
    int64_t n_require_calls = 0;
    int64_t n_device_allocs = 0;
    std::mutex mu;
};

// ---------------------------------------------------------------------------
// The accessors the backend imports.
// ---------------------------------------------------------------------------
RT_EXPORT diopiError_t diopiGetTensorData(diopiTensorHandle_t th, void** data) {
    if (!th || !data) return diopiErrorOccurred;
    *data = th->data;
    return diopiSuccess;
}
RT_EXPORT diopiError_t diopiGetTensorDataConst(diopiConstTensorHandle_t th, const void** data) {
    if (!th || !data) return diopiErrorOccurred;
    *data = th->data;
    return diopiSuccess;
}
RT_EXPORT diopiError_t diopiGetTensorShape(diopiConstTensorHandle_t th, diopiSize_t* size) {
    if (!th || !size) return diopiErrorOccurred;
    size->data = th->shape.data();
    size->len = static_cast<int64_t>(th->shape.size());
    return diopiSuccess;
}
RT_EXPORT diopiError_t diopiGetTensorStride(diopiConstTensorHandle_t th, diopiSize_t* stride) {
    if (!th || !stride) return diopiErrorOccurred;
    stride->data = th->stride.data();
    stride->len = static_cast<int64_t>(th->stride.size());
    return diopiSuccess;
}
RT_EXPORT diopiError_t diopiGetTensorDtype(diopiConstTensorHandle_t th, diopiDtype_t* dtype) {
    if (!th || !dtype) return diopiErrorOccurred;
    *dtype = th->dtype;
    return diopiSuccess;
}
RT_EXPORT diopiError_t diopiGetTensorDevice(diopiConstTensorHandle_t th, diopiDevice_t* device) {
    if (!th || !device) return diopiErrorOccurred;
    *device = th->device;
    return diopiSuccess;
}
RT_EXPORT diopiError_t diopiGetTensorNumel(diopiConstTensorHandle_t th, int64_t* numel) {
    if (!th || !numel) return diopiErrorOccurred;
    *numel = th->numel;
    return diopiSuccess;
}
RT_EXPORT diopiError_t diopiGetTensorElemSize(diopiConstTensorHandle_t th, int64_t* itemsize) {
    if (!th || !itemsize) return diopiErrorOccurred;
    *itemsize = elem_size(th->dtype);
    return diopiSuccess;
}

RT_EXPORT diopiError_t diopiGetStream(diopiContextHandle_t ctx, diopiStreamHandle_t* stream) {
    if (!ctx || !stream) return diopiErrorOccurred;
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (!ctx->stream_ready) {
        // A context made without a stream creates one lazily, on first use.
        if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) return diopiErrorOccurred;
        ctx->own_stream = true;
        ctx->stream_ready = true;
    }
    *stream = ctx->stream;
    return diopiSuccess;
}

static diopiError_t require_bytes(diopiContextHandle_t ctx, int64_t bytes, diopiDevice_t device, void** out) {
    ctx->n_require_calls++;
    const bool on_device = (device == diopi_device);
    Block* best = nullptr;
    for (auto& b : ctx->blocks) {
        if (!b.in_use && b.on_device == on_device && b.bytes >= bytes && (!best || b.bytes < best->bytes)) best = &b;
    }
    if (!best) {
        Block nb;
        nb.bytes = std::max<int64_t>(bytes, 256);
        nb.on_device = on_device;
        if (on_device) {
            if (cudaMalloc(&nb.ptr, nb.bytes) != cudaSuccess) return diopiErrorOccurred;
            ctx->n_device_allocs++;
        } else {
            nb.ptr = ::operator new(static_cast<size_t>(nb.bytes));
        }
        ctx->blocks.push_back(nb);
        best = &ctx->blocks.back();
    }
    best->in_use = true;
    *out = best->ptr;
    return diopiSuccess;
}

RT_EXPORT diopiError_t diopiRequireTensor(diopiContextHandle_t ctx, diopiTensorHandle_t* tensor, const diopiSize_t* size, const diopiSize_t* stride,
                                          const diopiDtype_t dtype, const diopiDevice_t device) {
    if (!ctx || !tensor || !size) return diopiErrorOccurred;
    std::lock_guard<std::mutex> lock(ctx->mu);
    auto* t = new diopiTensor();
    t->dtype = dtype;
    t->device = device;
    t->shape.assign(size->data, size->data + size->len);
    t->numel = 1;
    for (auto s : t->shape) t->numel *= s;
    if (stride && stride->data && stride->len == size->len) {
        t->stride.assign(stride->data, stride->data + stride->len);
    } else {
        t->stride.resize(t->shape.size());
        int64_t acc = 1;
        for (int i = static_cast<int>(t->shape.size()) - 1; i >= 0; --i) {
            t->stride[i] = acc;
            acc *= t->shape[i];
        }
    }
    // Storage must cover the furthest element the strides can reach.
    int64_t span = t->numel > 0 ? 1 : 0;
    if (t->numel > 0)
        for (size_t i = 0; i < t->shape.size(); ++i) span += (t->shape[i] - 1) * t->stride[i];
    diopiError_t err = require_bytes(ctx, span * elem_size(dtype), device, &t->data);
    if (err != diopiSuccess) {
        delete t;
        return err;
    }
    ctx->temps.push_back(t);
    *tensor = t;
    return diopiSuccess;
}

RT_EXPORT diopiError_t diopiRequireBuffer(diopiContextHandle_t ctx, diopiTensorHandle_t* tensor, int64_t num_bytes, diopiDevice_t device) {
    diopiSize_t size{&num_bytes, 1};
    return diopiRequireTensor(ctx, tensor, &size, nullptr, diopi_dtype_int8, device);
}

RT_EXPORT const char* diopiGetVersion() { return "DIOPI 1.0.0 (b200 test run time)"; }

// ---------------------------------------------------------------------------
// Helpers for the Python side (ctypes).
// ---------------------------------------------------------------------------

// Wrap caller-owned memory. stride may be null (contiguous). The handle does not own data.
RT_EXPORT diopiTensorHandle_t b200rt_tensor_create(void* data, int ndim, const int64_t* shape, const int64_t* stride, int dtype, int device) {
    auto* t = new diopiTensor();
    t->data = data;
    t->dtype = static_cast<diopiDtype_t>(dtype);
    t->device = static_cast<diopiDevice_t>(device);
    t->shape.assign(shape, shape + ndim);
    t->numel = 1;
    for (auto s : t->shape) t->numel *= s;
    if (stride) {
        t->stride.assign(stride, stride + ndim);
    } else {
        t->stride.resize(ndim);
        int64_t acc = 1;
        for (int i = ndim - 1; i >= 0; --i) {
            t->stride[i] = acc;
            acc *= t->shape[i];
        }
    }
    return t;
}

RT_EXPORT void b200rt_tensor_destroy(diopiTensorHandle_t t) { delete t; }

// stream == nullptr and lazy != 0: the context creates its own stream at first use.
// stream == nullptr and lazy == 0: the legacy default stream is used.
RT_EXPORT diopiContextHandle_t b200rt_context_create(void* stream, int lazy) {
    auto* c = new diopiContext();
    if (stream || !lazy) {
        c->stream = static_cast<cudaStream_t>(stream);
        c->stream_ready = true;
    }
    return c;
}

RT_EXPORT void b200rt_context_set_stream(diopiContextHandle_t ctx, void* stream) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    ctx->own_stream = false;
    ctx->stream = static_cast<cudaStream_t>(stream);
    ctx->stream_ready = true;
}

// Marks every temporary of the context reusable. Call after the ops that used them were enqueued.
RT_EXPORT void b200rt_context_release(diopiContextHandle_t ctx) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    for (auto* t : ctx->temps) delete t;
    ctx->temps.clear();
    for (auto& b : ctx->blocks) b.in_use = false;
}

RT_EXPORT int b200rt_context_synchronize(diopiContextHandle_t ctx) {
    if (!ctx->stream_ready) return 0;
    return static_cast<int>(cudaStreamSynchronize(ctx->stream));
}

RT_EXPORT void b200rt_context_destroy(diopiContextHandle_t ctx) {
    if (!ctx) return;
    if (ctx->stream_ready) cudaStreamSynchronize(ctx->stream);
    b200rt_context_release(ctx);
    for (auto& b : ctx->blocks) {
        if (b.on_device)
            cudaFree(b.ptr);
        else
            ::operator delete(b.ptr);
    }
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

// Counters the tests read: [0] require calls, [1] device allocations, [2] cached blocks, [3] cached bytes.
RT_EXPORT void b200rt_context_stats(diopiContextHandle_t ctx, int64_t* out4) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    out4[0] = ctx->n_require_calls;
    out4[1] = ctx->n_device_allocs;
    out4[2] = static_cast<int64_t>(ctx->blocks.size());
    int64_t total = 0;
    for (auto& b : ctx->blocks) total += b.bytes;
    out4[3] = total;
}
