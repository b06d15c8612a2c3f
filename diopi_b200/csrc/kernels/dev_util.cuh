// Device-side helpers shared by the kernels: index loads for int32/int64 tensors,
// conversions between the storage types and fp32, 16-byte vector unpacking.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>

#include "kernels.hpp"

namespace b200 {
namespace k {

__device__ __forceinline__ int64_t load_index(const void* p, int64_t off, int is64) {
    return is64 ? reinterpret_cast<const int64_t*>(p)[off] : static_cast<int64_t>(reinterpret_cast<const int32_t*>(p)[off]);
}

__device__ __forceinline__ int64_t load_index(const IndexArg& a, int64_t i) { return load_index(a.ptr, i * a.s0, a.is64); }
__device__ __forceinline__ int64_t load_index(const IndexArg& a, int64_t i, int64_t j) { return load_index(a.ptr, i * a.s0 + j * a.s1, a.is64); }

// First status wins; the word lives in mapped host memory, so it is visible without a copy.
__device__ __forceinline__ void report_status(int* status, int code) {
    if (status) atomicCAS_system(status, 0, code);
}

template <typename T>
struct Cvt;
template <>
struct Cvt<__half> {
    static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f(float f) { return __float2half_rn(f); }
};
template <>
struct Cvt<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float f) { return __float2bfloat16_rn(f); }
};
template <>
struct Cvt<float> {
    static __device__ __forceinline__ float to_f(float v) { return v; }
    static __device__ __forceinline__ float from_f(float f) { return f; }
};

// Elements held by one 16-byte vector.
template <typename T>
struct Vec16 {
    static constexpr int N = 16 / sizeof(T);
};

// Unpack a 16-byte vector into fp32.
template <typename T>
__device__ __forceinline__ void unpack16(const uint4& v, float (&f)[Vec16<T>::N]);

template <>
__device__ __forceinline__ void unpack16<__half>(const uint4& v, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
template <>
__device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void unpack16<float>(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
}

// Pack fp32 values into a 16-byte vector, rounding to nearest even.
template <typename T>
__device__ __forceinline__ uint4 pack16(const float (&f)[Vec16<T>::N]);

template <>
__device__ __forceinline__ uint4 pack16<__half>(const float (&f)[8]) {
    uint4 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return v;
}
template <>
__device__ __forceinline__ uint4 pack16<__nv_bfloat16>(const float (&f)[8]) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
}
template <>
__device__ __forceinline__ uint4 pack16<float>(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}

__device__ __forceinline__ int64_t imin64(int64_t a, int64_t b) { return a < b ? a : b; }
__device__ __forceinline__ int64_t imax64(int64_t a, int64_t b) { return a > b ? a : b; }

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace k
}  // namespace b200
