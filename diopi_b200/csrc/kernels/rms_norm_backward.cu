// RMSNorm backward. With r = inv_rms[row], gw = grad_output * weight (all in fp32):
//   grad_input  = r * gw - x * r^3 * mean(gw * x)          (mean over the normalised row)
//   grad_weight = sum over rows of grad_output * x * r
//   grad_bias   = sum over rows of grad_output
// Replaces cuComputeGradInput / cuComputePartGradGammaBeta / cuComputeGradGammaBeta as used for the RMS case in
// impl/torch/functions/functions_ext/layer_norm_cuda_kernel.cu:452-717 (entered from
// impl/torch/functions/functions_ext.cpp, diopiRMSNormBackward). The arithmetic is the derivative of the golden
// forward function (diopi_test/python/conformance/customized_test.py:392-403) taken in fp32 with one rounding at the
// end; inv_rms is the tensor the forward call saved.
//
// HBM-bound: reads grad_output and x once, writes grad_input once (3*n1*n2*e bytes) + n1 inv_rms values.
//   * rows kernel: a persistent grid of CTAs walks the rows; a thread keeps its 16-byte vectors of x and
//     grad_output in registers between the row reduction and the store, and adds its columns' terms of
//     grad_weight / grad_bias into registers over all its rows. Each CTA then writes one fp32 partial row.
//   * colsum kernel: adds the partial rows in a fixed order (deterministic) and rounds to the storage type.
//   * scalar kernels: any width, alignment or fp64.
#include "dev_util.cuh"

namespace b200 {
namespace k {

namespace {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename T>
__device__ __forceinline__ float load_inv(const void* inv_rms, Dt inv_dt, int64_t row) {
    if (inv_dt == Dt::F32) return __ldg(static_cast<const float*>(inv_rms) + row);
    return Cvt<T>::to_f(static_cast<const T*>(inv_rms)[row]);
}

template <typename T, int THREADS, int VPT, bool HAS_DB>
__global__ void __launch_bounds__(THREADS, (THREADS * VPT * Vec16<T>::N <= 4096 && THREADS == 512) ? 2 : 1) rms_bwd_rows_kernel(RmsNormBwdArgs a, int n_vec) {
    constexpr int N = Vec16<T>::N;
    constexpr int W = THREADS / 32;
    __shared__ float s_part[2][W];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    float wf[VPT][N], dw[VPT][N], db[HAS_DB ? VPT : 1][N];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int idx = threadIdx.x + v * THREADS;
        const uint4 raw = idx < n_vec ? __ldg(reinterpret_cast<const uint4*>(a.weight) + idx) : make_uint4(0, 0, 0, 0);
        unpack16<T>(raw, wf[v]);
#pragma unroll
        for (int e = 0; e < N; ++e) {
            dw[v][e] = 0.f;
            if constexpr (HAS_DB) db[v][e] = 0.f;
        }
    }
    const float inv_n2 = 1.0f / static_cast<float>(a.n2);
    int buf = 0;
    // The next row's vectors are requested before this row's reduction, so that loads stay in flight throughout.
    uint4 xnext[VPT], gnext[VPT];
    auto fetch = [&](int64_t row) {
        const uint4* x4 = reinterpret_cast<const uint4*>(static_cast<const T*>(a.x) + row * a.n2);
        const uint4* g4 = reinterpret_cast<const uint4*>(static_cast<const T*>(a.g) + row * a.n2);
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int idx = threadIdx.x + v * THREADS;
            xnext[v] = idx < n_vec ? __ldcs(x4 + idx) : make_uint4(0, 0, 0, 0);
            gnext[v] = idx < n_vec ? __ldcs(g4 + idx) : make_uint4(0, 0, 0, 0);
        }
    };
    if (blockIdx.x < a.n1) fetch(blockIdx.x);
    for (int64_t row = blockIdx.x; row < a.n1; row += gridDim.x) {
        uint4 xraw[VPT], graw[VPT];
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            xraw[v] = xnext[v];
            graw[v] = gnext[v];
        }
        if (row + gridDim.x < a.n1) fetch(row + gridDim.x);
        const float inv = load_inv<T>(a.inv_rms, a.inv_dt, row);
        float c = 0.f;
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            float xf[N], gf[N];
            unpack16<T>(xraw[v], xf);
            unpack16<T>(graw[v], gf);
#pragma unroll
            for (int e = 0; e < N; ++e) c = fmaf(gf[e] * wf[v][e], xf[e], c);
        }
        c = warp_sum_f(c);
        if (lane == 0) s_part[buf][warp] = c;
        __syncthreads();
        // every warp adds the W partials in the same fixed order: one shared-memory load per lane and a butterfly,
        // instead of W loads and adds per thread
        float tot = lane < W ? s_part[buf][lane] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
        buf ^= 1;  // the next row writes the other half: no second barrier per row
        const float coef = tot * inv_n2 * inv * inv * inv;
        uint4* o4 = reinterpret_cast<uint4*>(static_cast<T*>(a.dx) + row * a.n2);
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int idx = threadIdx.x + v * THREADS;
            float xf[N], gf[N], of[N];
            unpack16<T>(xraw[v], xf);
            unpack16<T>(graw[v], gf);
#pragma unroll
            for (int e = 0; e < N; ++e) {
                of[e] = fmaf(inv, gf[e] * wf[v][e], -xf[e] * coef);
                dw[v][e] = fmaf(gf[e] * xf[e], inv, dw[v][e]);
                if constexpr (HAS_DB) db[v][e] += gf[e];
            }
            if (idx < n_vec) __stcs(o4 + idx, pack16<T>(of));
        }
    }
    float* pw = a.ws + static_cast<size_t>(blockIdx.x) * a.n2;
    float* pb = a.ws + (static_cast<size_t>(gridDim.x) + blockIdx.x) * a.n2;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int idx = threadIdx.x + v * THREADS;
        if (idx < n_vec) {
#pragma unroll
            for (int e = 0; e < N; e += 4) {
                *reinterpret_cast<float4*>(pw + static_cast<size_t>(idx) * N + e) = make_float4(dw[v][e], dw[v][e + 1], dw[v][e + 2], dw[v][e + 3]);
                if constexpr (HAS_DB)
                    *reinterpret_cast<float4*>(pb + static_cast<size_t>(idx) * N + e) = make_float4(db[v][e], db[v][e + 1], db[v][e + 2], db[v][e + 3]);
            }
        }
    }
}

// grad_weight (blockIdx.y == 0) or grad_bias (1): column sums of the `parts` partial rows, added in a fixed order.
// A CTA covers 32 columns; its 8 warps take the partial rows round-robin and meet in shared memory.
template <typename T>
__global__ void __launch_bounds__(256) rms_bwd_colsum_kernel(RmsNormBwdArgs a, int parts) {
    __shared__ float s[8][33];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t col = static_cast<int64_t>(blockIdx.x) * 32 + lane;
    const float* src = a.ws + static_cast<size_t>(blockIdx.y) * parts * a.n2;
    float acc = 0.f;
    asm volatile("griddepcontrol.wait;" ::: "memory");  // no-op for a plain launch
    if (col < a.n2) {
#pragma unroll 4
        for (int p = warp; p < parts; p += 8) acc += src[static_cast<size_t>(p) * a.n2 + col];
    }
    s[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && col < a.n2) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) tot += s[w][lane];
        T* dst = static_cast<T*>(blockIdx.y == 0 ? a.dw : a.db);
        dst[col] = Cvt<T>::from_f(tot);
    }
}

// ---- any width / alignment / fp64 -------------------------------------------------------------
template <typename T, typename ACC>
struct BwdIo {
    static __device__ __forceinline__ ACC ld(const T* p) { return static_cast<ACC>(Cvt<T>::to_f(*p)); }
    static __device__ __forceinline__ void st(T* p, ACC v) { *p = Cvt<T>::from_f(static_cast<float>(v)); }
};
template <>
struct BwdIo<double, double> {
    static __device__ __forceinline__ double ld(const double* p) { return *p; }
    static __device__ __forceinline__ void st(double* p, double v) { *p = v; }
};

template <typename T, typename ACC>
__device__ __forceinline__ ACC load_inv_any(const void* inv_rms, Dt inv_dt, int64_t row) {
    if (inv_dt == Dt::F64) return static_cast<ACC>(static_cast<const double*>(inv_rms)[row]);
    if (inv_dt == Dt::F32) return static_cast<ACC>(static_cast<const float*>(inv_rms)[row]);
    return BwdIo<T, ACC>::ld(static_cast<const T*>(inv_rms) + row);
}

// grad_input: one warp per row, two passes (the second one hits L2).
template <typename T, typename ACC>
__global__ void __launch_bounds__(256) rms_bwd_dx_scalar_kernel(RmsNormBwdArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= a.n1) return;
    const T* x = static_cast<const T*>(a.x) + row * a.n2;
    const T* g = static_cast<const T*>(a.g) + row * a.n2;
    const T* w = static_cast<const T*>(a.weight);
    ACC c = 0;
    for (int64_t j = lane; j < a.n2; j += 32) c += BwdIo<T, ACC>::ld(g + j) * BwdIo<T, ACC>::ld(w + j) * BwdIo<T, ACC>::ld(x + j);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    const ACC inv = load_inv_any<T, ACC>(a.inv_rms, a.inv_dt, row);
    const ACC coef = c / static_cast<ACC>(a.n2) * inv * inv * inv;
    T* o = static_cast<T*>(a.dx) + row * a.n2;
    for (int64_t j = lane; j < a.n2; j += 32)
        BwdIo<T, ACC>::st(o + j, inv * (BwdIo<T, ACC>::ld(g + j) * BwdIo<T, ACC>::ld(w + j)) - BwdIo<T, ACC>::ld(x + j) * coef);
}

// grad_weight / grad_bias: one thread per column walks the rows (coalesced across the warp).
template <typename T, typename ACC>
__global__ void __launch_bounds__(128) rms_bwd_cols_scalar_kernel(RmsNormBwdArgs a) {
    const int64_t col = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (col >= a.n2) return;
    ACC sw = 0, sb = 0;
    for (int64_t row = 0; row < a.n1; ++row) {
        const ACC gv = BwdIo<T, ACC>::ld(static_cast<const T*>(a.g) + row * a.n2 + col);
        const ACC xv = BwdIo<T, ACC>::ld(static_cast<const T*>(a.x) + row * a.n2 + col);
        sw += gv * xv * load_inv_any<T, ACC>(a.inv_rms, a.inv_dt, row);
        sb += gv;
    }
    BwdIo<T, ACC>::st(static_cast<T*>(a.dw) + col, sw);
    if (a.db) BwdIo<T, ACC>::st(static_cast<T*>(a.db) + col, sb);
}

struct RowsConfig {
    int threads, vpt;
};
using RowsKernel = void (*)(RmsNormBwdArgs, int);

// Threads per CTA and 16-byte vectors per thread for a row of n_vec vectors. A thread keeps 2 * VPT * N fp32 column
// sums besides its row data, so 8 elements per thread is the comfortable size and 16 the limit (one CTA per SM).
template <typename T>
bool rows_config(const RmsNormBwdArgs& a, RowsConfig& c) {
    constexpr int N = Vec16<T>::N;
    auto al = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    if (a.n2 % N != 0 || !al(a.x) || !al(a.g) || !al(a.dx) || !al(a.weight)) return false;
    if (a.inv_dt == Dt::F64) return false;
    const int64_t n_vec = a.n2 / N;
    if (n_vec <= 128) c = {128, 1};
    else if (n_vec <= 256) c = {256, 1};
    else if (N == 8) {
        if (n_vec <= 512) c = {512, 1};
        else if (n_vec <= 1024) c = {512, 2};
        else return false;
    } else {
        if (n_vec <= 512) c = {256, 2};
        else if (n_vec <= 1024) c = {256, 4};
        else if (n_vec <= 2048) c = {512, 4};
        else return false;
    }
    return true;
}

template <typename T, bool HAS_DB>
RowsKernel rows_kernel_db(const RowsConfig& c) {
    constexpr int N = Vec16<T>::N;
    if (c.threads == 128) return rms_bwd_rows_kernel<T, 128, 1, HAS_DB>;
    if (c.threads == 256 && c.vpt == 1) return rms_bwd_rows_kernel<T, 256, 1, HAS_DB>;
    if constexpr (N == 8) {
        if (c.vpt == 1) return rms_bwd_rows_kernel<T, 512, 1, HAS_DB>;
        return rms_bwd_rows_kernel<T, 512, 2, HAS_DB>;
    } else {
        if (c.threads == 256 && c.vpt == 2) return rms_bwd_rows_kernel<T, 256, 2, HAS_DB>;
        if (c.threads == 256) return rms_bwd_rows_kernel<T, 256, 4, HAS_DB>;
        return rms_bwd_rows_kernel<T, 512, 4, HAS_DB>;
    }
}

template <typename T>
RowsKernel rows_kernel(const RowsConfig& c, bool has_db) {
    return has_db ? rows_kernel_db<T, true>(c) : rows_kernel_db<T, false>(c);
}

template <typename T>
int parts_typed(const RmsNormBwdArgs& a, int sm_count) {
    RowsConfig c;
    if (!rows_config<T>(a, c)) return 0;
    int per_sm = 0;  // resident CTAs per SM, by the kernel's register use
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rows_kernel<T>(c, a.db != nullptr), c.threads, 0) != cudaSuccess || per_sm < 1) {
        (void)cudaGetLastError();
        per_sm = 1;
    }
    per_sm = std::min(per_sm, 4);
    return static_cast<int>(std::min<int64_t>(a.n1, static_cast<int64_t>(sm_count) * per_sm));
}

template <typename T>
void launch_typed(const RmsNormBwdArgs& a, cudaStream_t st) {
    RowsConfig c;
    if (a.parts > 0 && a.ws != nullptr && rows_config<T>(a, c)) {
        const int n_vec = static_cast<int>(a.n2 / Vec16<T>::N);
        rows_kernel<T>(c, a.db != nullptr)<<<a.parts, c.threads, 0, st>>>(a, n_vec);
        // Programmatic dependent launch: the column-sum kernel's launch overlaps the rows kernel; it waits for the
        // rows kernel's writes before its first load.
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>((a.n2 + 31) / 32), a.db ? 2 : 1);
        cfg.blockDim = dim3(256);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaLaunchKernelEx(&cfg, rms_bwd_colsum_kernel<T>, a, a.parts);
        return;
    }
    rms_bwd_dx_scalar_kernel<T, float><<<static_cast<unsigned>((a.n1 + 7) / 8), 256, 0, st>>>(a);
    rms_bwd_cols_scalar_kernel<T, float><<<static_cast<unsigned>((a.n2 + 127) / 128), 128, 0, st>>>(a);
}

}  // namespace

int rms_norm_bwd_parts(const RmsNormBwdArgs& a, int sm_count) {
    if (a.n1 <= 0 || a.n2 <= 0 || a.n1 >= (1ll << 31)) return 0;
    switch (a.dt) {
        case Dt::F16: return parts_typed<__half>(a, sm_count);
        case Dt::BF16: return parts_typed<__nv_bfloat16>(a, sm_count);
        case Dt::F32: return parts_typed<float>(a, sm_count);
        default: return 0;
    }
}

void launch_rms_norm_bwd(const RmsNormBwdArgs& a, cudaStream_t st) {
    if (a.n2 == 0) return;
    if (a.n1 == 0) {  // no rows: the column sums are empty sums
        const size_t e = a.dt == Dt::F64 ? 8 : (a.dt == Dt::F32 ? 4 : 2);
        cudaMemsetAsync(a.dw, 0, static_cast<size_t>(a.n2) * e, st);
        if (a.db) cudaMemsetAsync(a.db, 0, static_cast<size_t>(a.n2) * e, st);
        return;
    }
    switch (a.dt) {
        case Dt::F16: launch_typed<__half>(a, st); break;
        case Dt::BF16: launch_typed<__nv_bfloat16>(a, st); break;
        case Dt::F32: launch_typed<float>(a, st); break;
        case Dt::F64:
            rms_bwd_dx_scalar_kernel<double, double><<<static_cast<unsigned>((a.n1 + 7) / 8), 256, 0, st>>>(a);
            rms_bwd_cols_scalar_kernel<double, double><<<static_cast<unsigned>((a.n2 + 127) / 128), 128, 0, st>>>(a);
            break;
    }
}

}  // namespace k
}  // namespace b200
