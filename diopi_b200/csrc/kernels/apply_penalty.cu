// ApplyPenalty: for request i and entries e in [cum[i], cum[i+1]):
//   logits[i, ids[e]] = logits[i, ids[e]] - counts[e] * frequency[i] - presence[i]
// Replaces the per-request host loop (two device->host reads, index_select, mul, sub, sub,
// index_put_ per request) of impl/torch/functions/functions_lightllm.cpp:28-51. Golden:
// diopi_test/python/conformance/customized_test.py:667-692.
//
// Bit-exact by construction: the three operations are rounded one by one in the dtype of logits,
// exactly as the tensor expression above evaluates them. For fp16/bf16 each operation is carried
// out in fp32 and rounded to the storage type (what the torch CPU kernels do); for fp32 the
// intrinsics keep the compiler from contracting mul+sub into an fma.
//
// Latency-bound scatter: E entries, each a 4-byte (or 2-byte) read-modify-write; one thread per
// entry, the request found by binary search in the prefix sums. Entries of one request must not
// repeat a token id (the result would depend on thread order); the reference's own result for
// repeated ids is "last one wins, computed from the original value".
#include "dev_util.cuh"

namespace b200 {
namespace k {

namespace {

template <typename T>
__device__ __forceinline__ T penalise(T logit, int64_t count, T freq, T pres);

template <>
__device__ __forceinline__ float penalise<float>(float logit, int64_t count, float freq, float pres) {
    const float prod = __fmul_rn(static_cast<float>(count), freq);
    return __fsub_rn(__fsub_rn(logit, prod), pres);
}
template <>
__device__ __forceinline__ __half penalise<__half>(__half logit, int64_t count, __half freq, __half pres) {
    const __half c = __float2half_rn(static_cast<float>(count));
    const __half prod = __float2half_rn(__fmul_rn(__half2float(c), __half2float(freq)));
    const __half d = __float2half_rn(__fsub_rn(__half2float(logit), __half2float(prod)));
    return __float2half_rn(__fsub_rn(__half2float(d), __half2float(pres)));
}
template <>
__device__ __forceinline__ __nv_bfloat16 penalise<__nv_bfloat16>(__nv_bfloat16 logit, int64_t count, __nv_bfloat16 freq, __nv_bfloat16 pres) {
    const __nv_bfloat16 c = __float2bfloat16_rn(static_cast<float>(count));
    const __nv_bfloat16 prod = __float2bfloat16_rn(__fmul_rn(__bfloat162float(c), __bfloat162float(freq)));
    const __nv_bfloat16 d = __float2bfloat16_rn(__fsub_rn(__bfloat162float(logit), __bfloat162float(prod)));
    return __float2bfloat16_rn(__fsub_rn(__bfloat162float(d), __bfloat162float(pres)));
}
template <>
__device__ __forceinline__ double penalise<double>(double logit, int64_t count, double freq, double pres) {
    const double prod = __dmul_rn(static_cast<double>(count), freq);
    return __dsub_rn(__dsub_rn(logit, prod), pres);
}

template <typename T>
__global__ void __launch_bounds__(256) penalty_kernel(PenaltyArgs a) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < a.E; e += stride) {
        // request i with cum[i] <= e < cum[i+1]
        int64_t lo = 0, hi = a.B;  // smallest i with cum[i+1] > e
        while (lo < hi) {
            const int64_t mid = (lo + hi) >> 1;
            if (load_index(a.cum, mid + 1) > e)
                hi = mid;
            else
                lo = mid + 1;
        }
        const int64_t i = lo;
        if (i >= a.B || load_index(a.cum, i) > e) continue;  // entry outside every request
        int64_t id = load_index(a.ids, e);
        if (id < 0) id += a.V;
        if (id < 0 || id >= a.V) {
            report_status(a.status, 2);
            continue;
        }
        const int64_t cnt = load_index(a.counts, e);
        T* p = static_cast<T*>(a.logits) + i * a.l_s0 + id * a.l_s1;
        const T f = static_cast<const T*>(a.frequency)[i * a.f_s];
        const T pr = static_cast<const T*>(a.presence)[i * a.p_s];
        *p = penalise<T>(*p, cnt, f, pr);
    }
}

// V2 (diopi_test/python/conformance/customized_test.py:823-841): entries index the flattened logits, every entry
// has its own penalties, and a repetition penalty comes first: x > 0 ? x / r : x * r, then - count * f - p.
// Each operation is rounded on its own in the dtype of logits, as the golden tensor expression does.
template <typename T>
struct Rnd;
template <>
struct Rnd<float> {
    static __device__ __forceinline__ float ld(const void* p, int64_t i) { return static_cast<const float*>(p)[i]; }
    static __device__ __forceinline__ float r(float v) { return v; }
    static __device__ __forceinline__ void st(void* p, int64_t i, float v) { static_cast<float*>(p)[i] = v; }
};
template <>
struct Rnd<__half> {
    static __device__ __forceinline__ float ld(const void* p, int64_t i) { return __half2float(static_cast<const __half*>(p)[i]); }
    static __device__ __forceinline__ float r(float v) { return __half2float(__float2half_rn(v)); }
    static __device__ __forceinline__ void st(void* p, int64_t i, float v) { static_cast<__half*>(p)[i] = __float2half_rn(v); }
};
template <>
struct Rnd<__nv_bfloat16> {
    static __device__ __forceinline__ float ld(const void* p, int64_t i) { return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]); }
    static __device__ __forceinline__ float r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
    static __device__ __forceinline__ void st(void* p, int64_t i, float v) { static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); }
};

template <typename T>
__global__ void __launch_bounds__(256) penalty_v2_kernel(PenaltyV2Args a) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < a.E; e += stride) {
        int64_t id = load_index(a.ids, e);
        if (id < 0) id += a.numel;
        if (id < 0 || id >= a.numel) {
            report_status(a.status, 2);
            continue;
        }
        const float x = Rnd<T>::ld(a.logits, id);
        const float rp = Rnd<T>::ld(a.repetition, e * a.r_s);
        const float f = Rnd<T>::ld(a.frequency, e * a.f_s);
        const float pr = Rnd<T>::ld(a.presence, e * a.p_s);
        const float cnt = Rnd<T>::r(static_cast<float>(load_index(a.counts, e)));
        const float rep = Rnd<T>::r(x > 0.f ? __fdiv_rn(x, rp) : __fmul_rn(x, rp));
        const float prod = Rnd<T>::r(__fmul_rn(cnt, f));
        const float d = Rnd<T>::r(__fsub_rn(rep, prod));
        Rnd<T>::st(a.logits, id, __fsub_rn(d, pr));
    }
}

__global__ void __launch_bounds__(256) penalty_v2_f64_kernel(PenaltyV2Args a) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t e = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < a.E; e += stride) {
        int64_t id = load_index(a.ids, e);
        if (id < 0) id += a.numel;
        if (id < 0 || id >= a.numel) {
            report_status(a.status, 2);
            continue;
        }
        double* lg = static_cast<double*>(a.logits);
        const double x = lg[id];
        const double rp = static_cast<const double*>(a.repetition)[e * a.r_s];
        const double rep = x > 0.0 ? __ddiv_rn(x, rp) : __dmul_rn(x, rp);
        const double prod = __dmul_rn(static_cast<double>(load_index(a.counts, e)), static_cast<const double*>(a.frequency)[e * a.f_s]);
        lg[id] = __dsub_rn(__dsub_rn(rep, prod), static_cast<const double*>(a.presence)[e * a.p_s]);
    }
}

}  // namespace

void launch_apply_penalty_v2(const PenaltyV2Args& a, cudaStream_t st) {
    if (a.E == 0 || a.numel == 0) return;
    const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((a.E + 255) / 256, 148ll * 32));
    switch (a.dt) {
        case Dt::F16: penalty_v2_kernel<__half><<<blocks, 256, 0, st>>>(a); break;
        case Dt::BF16: penalty_v2_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(a); break;
        case Dt::F32: penalty_v2_kernel<float><<<blocks, 256, 0, st>>>(a); break;
        case Dt::F64: penalty_v2_f64_kernel<<<blocks, 256, 0, st>>>(a); break;
    }
}

void launch_apply_penalty(const PenaltyArgs& a, cudaStream_t st) {
    if (a.E == 0 || a.B == 0) return;
    const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((a.E + 255) / 256, 148ll * 32));
    switch (a.dt) {
        case Dt::F16: penalty_kernel<__half><<<blocks, 256, 0, st>>>(a); break;
        case Dt::BF16: penalty_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(a); break;
        case Dt::F32: penalty_kernel<float><<<blocks, 256, 0, st>>>(a); break;
        case Dt::F64: penalty_kernel<double><<<blocks, 256, 0, st>>>(a); break;
    }
}

}  // namespace k
}  // namespace b200
