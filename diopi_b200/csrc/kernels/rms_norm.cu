// RMSNorm forward: inv_rms[r] = 1/sqrt(mean(x[r,:]^2) + eps); out = weight * (x * inv_rms) (+ bias).
// Replaces cuApplyRMSNorm / HostApplyRMSNorm of
// impl/torch/functions/functions_ext/layer_norm_cuda_kernel.cu:322-378,735-743 and the separate
// bias add of impl/torch/functions/functions_ext.cpp:75-78. Arithmetic follows the golden function
// (diopi_test/python/conformance/customized_test.py:392-403): everything in fp32 with one rounding
// to the storage type at the end.
//
// HBM-bound: 2*n1*n2*e bytes + n1*4 (inv_rms) + n2*e (weight). The reference kernel reads every
// row twice (reduce, then apply); here a row is read once with 16-byte loads and stays in
// registers between the two phases:
//   * row kernel: one CTA per row, each thread keeps up to 8 vectors;
//   * warp kernel: one warp per row for short rows, several rows per CTA;
//   * scalar kernel: any n2/alignment/fp64, two passes (the second one hits L2).
#include "dev_util.cuh"

namespace b200 {
namespace k {

namespace {

template <typename T>
__device__ __forceinline__ void store_inv(void* inv_rms, Dt inv_dt, int64_t row, float v) {
    if (inv_dt == Dt::F32)
        static_cast<float*>(inv_rms)[row] = v;
    else
        static_cast<T*>(inv_rms)[row] = Cvt<T>::from_f(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// out = w * (x * inv) (+ b) with the roundings of the golden function: no contraction into an fma.
__device__ __forceinline__ float norm_one(float x, float inv, float w, float b, bool has_bias) {
    const float y = __fmul_rn(w, __fmul_rn(x, inv));
    return has_bias ? __fadd_rn(y, b) : y;
}

// One CTA per row; thread t holds vectors t, t+THREADS, ... (VPT of them).
template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS) rms_row_kernel(RmsNormArgs a, int n_vec) {
    constexpr int N = Vec16<T>::N;
    __shared__ float s_part[THREADS / 32];
    const int64_t row = blockIdx.x;
    const uint4* x = reinterpret_cast<const uint4*>(static_cast<const T*>(a.x) + row * a.n2);
    const uint4* w4 = reinterpret_cast<const uint4*>(a.weight);
    uint4 raw[VPT], wraw[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int idx = threadIdx.x + v * THREADS;
        raw[v] = idx < n_vec ? __ldcs(x + idx) : make_uint4(0, 0, 0, 0);
    }
    // the weights are asked for now, so that their latency (an L2 hit) passes during the reduction instead of after it
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int idx = threadIdx.x + v * THREADS;
        wraw[v] = idx < n_vec ? __ldg(w4 + idx) : make_uint4(0, 0, 0, 0);
    }
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        float f[N];
        unpack16<T>(raw[v], f);
#pragma unroll
        for (int e = 0; e < N; ++e) ss = fmaf(f[e], f[e], ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) tot += s_part[w];
    const float inv = 1.0f / sqrtf(tot / static_cast<float>(a.n2) + static_cast<float>(a.eps));
    if (threadIdx.x == 0) store_inv<T>(a.inv_rms, a.inv_dt, row, inv);

    const uint4* b4 = reinterpret_cast<const uint4*>(a.bias);
    uint4* o = reinterpret_cast<uint4*>(static_cast<T*>(a.out) + row * a.n2);
    const bool has_bias = a.bias != nullptr;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int idx = threadIdx.x + v * THREADS;
        if (idx < n_vec) {
            float f[N], wf[N], bf[N];
            unpack16<T>(raw[v], f);
            unpack16<T>(wraw[v], wf);
            if (has_bias) unpack16<T>(__ldg(b4 + idx), bf);
#pragma unroll
            for (int e = 0; e < N; ++e) f[e] = norm_one(f[e], inv, wf[e], has_bias ? bf[e] : 0.f, has_bias);
            __stcs(o + idx, pack16<T>(f));
        }
    }
}

// One warp per row, VPT vectors per lane.
template <typename T, int VPT>
__global__ void __launch_bounds__(256) rms_warp_kernel(RmsNormArgs a, int n_vec) {
    constexpr int N = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= a.n1) return;
    const uint4* x = reinterpret_cast<const uint4*>(static_cast<const T*>(a.x) + row * a.n2);
    uint4 raw[VPT];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int idx = lane + v * 32;
        raw[v] = idx < n_vec ? __ldcs(x + idx) : make_uint4(0, 0, 0, 0);
        float f[N];
        unpack16<T>(raw[v], f);
#pragma unroll
        for (int e = 0; e < N; ++e) ss = fmaf(f[e], f[e], ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / static_cast<float>(a.n2) + static_cast<float>(a.eps));
    if (lane == 0) store_inv<T>(a.inv_rms, a.inv_dt, row, inv);
    const uint4* w4 = reinterpret_cast<const uint4*>(a.weight);
    const uint4* b4 = reinterpret_cast<const uint4*>(a.bias);
    uint4* o = reinterpret_cast<uint4*>(static_cast<T*>(a.out) + row * a.n2);
    const bool has_bias = a.bias != nullptr;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int idx = lane + v * 32;
        if (idx < n_vec) {
            float f[N], wf[N], bf[N];
            unpack16<T>(raw[v], f);
            unpack16<T>(__ldg(w4 + idx), wf);
            if (has_bias) unpack16<T>(__ldg(b4 + idx), bf);
#pragma unroll
            for (int e = 0; e < N; ++e) f[e] = norm_one(f[e], inv, wf[e], has_bias ? bf[e] : 0.f, has_bias);
            __stcs(o + idx, pack16<T>(f));
        }
    }
}

// Any width and alignment; one warp per row, two passes. ACC is the arithmetic type.
template <typename T, typename ACC>
struct ScalarIo {
    static __device__ __forceinline__ ACC ld(const T* p) { return static_cast<ACC>(Cvt<T>::to_f(*p)); }
    static __device__ __forceinline__ void st(T* p, ACC v) { *p = Cvt<T>::from_f(static_cast<float>(v)); }
};
template <>
struct ScalarIo<double, double> {
    static __device__ __forceinline__ double ld(const double* p) { return *p; }
    static __device__ __forceinline__ void st(double* p, double v) { *p = v; }
};

__device__ __forceinline__ float mul_rn(float x, float y) { return __fmul_rn(x, y); }
__device__ __forceinline__ double mul_rn(double x, double y) { return __dmul_rn(x, y); }
__device__ __forceinline__ float add_rn(float x, float y) { return __fadd_rn(x, y); }
__device__ __forceinline__ double add_rn(double x, double y) { return __dadd_rn(x, y); }

template <typename T, typename ACC>
__global__ void __launch_bounds__(256) rms_scalar_kernel(RmsNormArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= a.n1) return;
    const T* x = static_cast<const T*>(a.x) + row * a.n2;
    ACC ss = 0;
    for (int64_t c = lane; c < a.n2; c += 32) {
        const ACC v = ScalarIo<T, ACC>::ld(x + c);
        ss += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const ACC inv = static_cast<ACC>(1) / sqrt(ss / static_cast<ACC>(a.n2) + static_cast<ACC>(a.eps));
    if (lane == 0) {
        if (a.inv_dt == Dt::F64)
            static_cast<double*>(a.inv_rms)[row] = static_cast<double>(inv);
        else if (a.inv_dt == Dt::F32)
            static_cast<float*>(a.inv_rms)[row] = static_cast<float>(inv);
        else
            ScalarIo<T, ACC>::st(static_cast<T*>(a.inv_rms) + row, inv);
    }
    const T* w = static_cast<const T*>(a.weight);
    const T* b = static_cast<const T*>(a.bias);
    T* o = static_cast<T*>(a.out) + row * a.n2;
    for (int64_t c = lane; c < a.n2; c += 32) {
        ACC y = mul_rn(ScalarIo<T, ACC>::ld(x + c), inv);
        y = mul_rn(ScalarIo<T, ACC>::ld(w + c), y);
        if (b) y = add_rn(y, ScalarIo<T, ACC>::ld(b + c));
        ScalarIo<T, ACC>::st(o + c, y);
    }
}

template <typename T>
void launch_typed(const RmsNormArgs& a, cudaStream_t st) {
    constexpr int N = Vec16<T>::N;
    const bool aligned = a.n2 % N == 0 && reinterpret_cast<uintptr_t>(a.x) % 16 == 0 && reinterpret_cast<uintptr_t>(a.out) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(a.weight) % 16 == 0 && (a.bias == nullptr || reinterpret_cast<uintptr_t>(a.bias) % 16 == 0);
    const int64_t n_vec64 = a.n2 / N;
    if (aligned && n_vec64 <= 8192 && a.n1 < (1ll << 31)) {
        const int n_vec = static_cast<int>(n_vec64);
        const unsigned rows = static_cast<unsigned>(a.n1);
        if (n_vec <= 32) {
            rms_warp_kernel<T, 1><<<(rows + 7) / 8, 256, 0, st>>>(a, n_vec);
        } else if (n_vec <= 64) {
            rms_warp_kernel<T, 2><<<(rows + 7) / 8, 256, 0, st>>>(a, n_vec);
        } else if (n_vec <= 128) {
            rms_row_kernel<T, 128, 1><<<rows, 128, 0, st>>>(a, n_vec);
        } else if (n_vec <= 256) {
            rms_row_kernel<T, 128, 2><<<rows, 128, 0, st>>>(a, n_vec);
        } else if (n_vec <= 512) {
            rms_row_kernel<T, 128, 4><<<rows, 128, 0, st>>>(a, n_vec);
        } else if (n_vec <= 1024) {
            rms_row_kernel<T, 256, 4><<<rows, 256, 0, st>>>(a, n_vec);
        } else if (n_vec <= 2048) {
            rms_row_kernel<T, 256, 8><<<rows, 256, 0, st>>>(a, n_vec);
        } else if (n_vec <= 4096) {
            rms_row_kernel<T, 512, 8><<<rows, 512, 0, st>>>(a, n_vec);
        } else {
            rms_row_kernel<T, 1024, 8><<<rows, 1024, 0, st>>>(a, n_vec);
        }
        return;
    }
    const unsigned blocks = static_cast<unsigned>((a.n1 + 7) / 8);
    rms_scalar_kernel<T, float><<<blocks, 256, 0, st>>>(a);
}

}  // namespace

void launch_rms_norm(const RmsNormArgs& a, int /*sm_count*/, cudaStream_t st) {
    if (a.n1 == 0 || a.n2 == 0) return;
    switch (a.dt) {
        case Dt::F16: launch_typed<__half>(a, st); break;
        case Dt::BF16: launch_typed<__nv_bfloat16>(a, st); break;
        case Dt::F32: launch_typed<float>(a, st); break;
        case Dt::F64: {
            const unsigned blocks = static_cast<unsigned>((a.n1 + 7) / 8);
            rms_scalar_kernel<double, double><<<blocks, 256, 0, st>>>(a);
            break;
        }
    }
}

}  // namespace k
}  // namespace b200
