// Rotary embedding on the two halves (x1, x2) of the last dimension:
//   forward:  o1 = x1*cos - x2*sin,  o2 = x1*sin + x2*cos
//   conj:     o1 = x1*cos + x2*sin,  o2 = -x1*sin + x2*cos
// Replaces the TensorIterator kernel of impl/torch/functions/functions_ext/rotary.cu:14-46; the
// arithmetic (fp32, each product and the sum rounded on its own, one final rounding to the storage
// type) follows diopi_test/python/conformance/customized_test.py:374-390.
//
// HBM-bound: 2*numel(x)*e bytes + the cos/sin tables (re-read from L2 for every head).
// cos/sin broadcast over x's leading dims; the host turns that into one stride per collapsed leading
// dim (0 where broadcast), so the kernel only does a short div/mod chain per vector.
#include "dev_util.cuh"

namespace b200 {
namespace k {

namespace {

template <typename IDX>
struct Offsets {
    IDX x, o, c, s;
};

// IDX = uint32_t when every extent and the element count fit 32 bits (the usual case): 32-bit
// division is several times cheaper than 64-bit, and this chain is most of the kernel's arithmetic.
template <typename IDX>
__device__ __forceinline__ Offsets<IDX> lead_offsets(const RopeArgs& a, IDX lead) {
    Offsets<IDX> r{0, 0, 0, 0};
#pragma unroll
    for (int d = kRopeMaxDims - 1; d >= 0; --d) {
        if (d < a.nd) {
            const IDX sz = static_cast<IDX>(a.size[d]);
            const IDX q = lead / sz;
            const IDX i = lead - q * sz;
            lead = q;
            r.x += i * static_cast<IDX>(a.xs[d]);
            r.o += i * static_cast<IDX>(a.os[d]);
            r.c += i * static_cast<IDX>(a.cs[d]);
            r.s += i * static_cast<IDX>(a.ss[d]);
        }
    }
    return r;
}

// Same result as rotate() for fp16/bf16 inputs with one instruction less per output: the product of two such
// values is exact in fp32, so fma(x1, c, -(x2*s)) rounds exactly once, like the subtraction of the two products.
__device__ __forceinline__ void rotate16(float x1, float x2, float c, float s, bool conj, float& o1, float& o2) {
    const float b = x2 * s, e = x2 * c;
    if (!conj) {
        o1 = fmaf(x1, c, -b);
        o2 = fmaf(x1, s, e);
    } else {
        o1 = fmaf(x1, c, b);
        o2 = fmaf(-x1, s, e);
    }
}

__device__ __forceinline__ void rotate(float x1, float x2, float c, float s, bool conj, float& o1, float& o2) {
    const float a = __fmul_rn(x1, c), b = __fmul_rn(x2, s), d = __fmul_rn(x1, s), e = __fmul_rn(x2, c);
    if (!conj) {
        o1 = __fsub_rn(a, b);
        o2 = __fadd_rn(d, e);
    } else {
        o1 = __fadd_rn(a, b);
        o2 = __fadd_rn(-d, e);
    }
}

// One thread per 16-byte vector of x1 (and the matching vector of x2). Last dims dense and aligned.
template <typename T, typename IDX>
__global__ void __launch_bounds__(256) rope_vec_kernel(RopeArgs a, int vec_per_half, int64_t total_vec) {
    constexpr int N = Vec16<T>::N;
    const IDX stride = static_cast<IDX>(gridDim.x) * blockDim.x;
    const IDX total = static_cast<IDX>(total_vec);
    for (IDX i = static_cast<IDX>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const IDX lead = i / static_cast<IDX>(vec_per_half);
        const int v = static_cast<int>(i - lead * static_cast<IDX>(vec_per_half));
        const Offsets<IDX> of = lead_offsets<IDX>(a, lead);
        const T* x = static_cast<const T*>(a.x) + of.x;
        T* o = static_cast<T*>(a.out) + of.o;
        const uint4 r1 = __ldcs(reinterpret_cast<const uint4*>(x) + v);
        const uint4 r2 = __ldcs(reinterpret_cast<const uint4*>(x + a.half) + v);
        const uint4 rc = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(a.cos) + of.c) + v);
        const uint4 rs = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(a.sin) + of.s) + v);
        float x1[N], x2[N], c[N], s[N], o1[N], o2[N];
        unpack16<T>(r1, x1);
        unpack16<T>(r2, x2);
        unpack16<T>(rc, c);
        unpack16<T>(rs, s);
#pragma unroll
        for (int e = 0; e < N; ++e) {
            if (sizeof(T) == 2)
                rotate16(x1[e], x2[e], c[e], s[e], a.conj, o1[e], o2[e]);
            else
                rotate(x1[e], x2[e], c[e], s[e], a.conj, o1[e], o2[e]);
        }
        __stcs(reinterpret_cast<uint4*>(o) + v, pack16<T>(o1));
        __stcs(reinterpret_cast<uint4*>(o + a.half) + v, pack16<T>(o2));
    }
}

// The same, for tables that are broadcast over the last leading dim (one cos/sin row per token, shared by its heads):
// a thread takes vector v of HP neighbouring heads, loads its cos/sin vectors once and keeps 2 * HP loads of x in
// flight; the offset chain and the unpacking of the tables are paid once per HP head-vectors instead of once each.
template <typename T, typename IDX, int HP>
__global__ void __launch_bounds__(256) rope_vec_heads_kernel(RopeArgs a, int vec_per_half, int64_t total_vec) {
    constexpr int N = Vec16<T>::N;
    const IDX stride = static_cast<IDX>(gridDim.x) * blockDim.x;
    const IDX total = static_cast<IDX>(total_vec);
    const IDX heads = static_cast<IDX>(a.size[a.nd - 1]);
    const IDX groups = heads / HP;
    const IDX x_hs = static_cast<IDX>(a.xs[a.nd - 1]), o_hs = static_cast<IDX>(a.os[a.nd - 1]);
    for (IDX i = static_cast<IDX>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const IDX lg = i / static_cast<IDX>(vec_per_half);
        const int v = static_cast<int>(i - lg * static_cast<IDX>(vec_per_half));
        const IDX outer = lg / groups;
        const IDX lead = outer * heads + (lg - outer * groups) * HP;
        const Offsets<IDX> of = lead_offsets<IDX>(a, lead);
        const T* x = static_cast<const T*>(a.x) + of.x;
        T* o = static_cast<T*>(a.out) + of.o;
        uint4 r1[HP], r2[HP];
#pragma unroll
        for (int hp = 0; hp < HP; ++hp) {
            r1[hp] = __ldcs(reinterpret_cast<const uint4*>(x + hp * x_hs) + v);
            r2[hp] = __ldcs(reinterpret_cast<const uint4*>(x + hp * x_hs + a.half) + v);
        }
        const uint4 rc = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(a.cos) + of.c) + v);
        const uint4 rs = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(a.sin) + of.s) + v);
        float c[N], s[N];
        unpack16<T>(rc, c);
        unpack16<T>(rs, s);
#pragma unroll
        for (int hp = 0; hp < HP; ++hp) {
            float x1[N], x2[N], o1[N], o2[N];
            unpack16<T>(r1[hp], x1);
            unpack16<T>(r2[hp], x2);
#pragma unroll
            for (int e = 0; e < N; ++e) {
                if (sizeof(T) == 2)
                    rotate16(x1[e], x2[e], c[e], s[e], a.conj, o1[e], o2[e]);
                else
                    rotate(x1[e], x2[e], c[e], s[e], a.conj, o1[e], o2[e]);
            }
            __stcs(reinterpret_cast<uint4*>(o + hp * o_hs) + v, pack16<T>(o1));
            __stcs(reinterpret_cast<uint4*>(o + hp * o_hs + a.half) + v, pack16<T>(o2));
        }
    }
}

template <typename T>
struct Io {
    static __device__ __forceinline__ float ld(const T* p) { return Cvt<T>::to_f(*p); }
    static __device__ __forceinline__ void st(T* p, float v) { *p = Cvt<T>::from_f(v); }
};

// One thread per (x1, x2) pair; any strides.
template <typename T>
__global__ void __launch_bounds__(256) rope_scalar_kernel(RopeArgs a, int64_t total) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t lead = i / a.half;
        const int64_t j = i - lead * a.half;
        const Offsets<int64_t> of = lead_offsets<int64_t>(a, lead);
        const T* x = static_cast<const T*>(a.x) + of.x;
        T* o = static_cast<T*>(a.out) + of.o;
        const float c = Io<T>::ld(static_cast<const T*>(a.cos) + of.c + j * a.c_ls);
        const float s = Io<T>::ld(static_cast<const T*>(a.sin) + of.s + j * a.s_ls);
        float o1, o2;
        rotate(Io<T>::ld(x + j * a.x_ls), Io<T>::ld(x + (j + a.half) * a.x_ls), c, s, a.conj, o1, o2);
        Io<T>::st(o + j * a.o_ls, o1);
        Io<T>::st(o + (j + a.half) * a.o_ls, o2);
    }
}

__global__ void __launch_bounds__(256) rope_scalar_f64_kernel(RopeArgs a, int64_t total) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t lead = i / a.half;
        const int64_t j = i - lead * a.half;
        const Offsets<int64_t> of = lead_offsets<int64_t>(a, lead);
        const double* x = static_cast<const double*>(a.x) + of.x;
        double* o = static_cast<double*>(a.out) + of.o;
        const double c = static_cast<const double*>(a.cos)[of.c + j * a.c_ls];
        const double s = static_cast<const double*>(a.sin)[of.s + j * a.s_ls];
        const double x1 = x[j * a.x_ls], x2 = x[(j + a.half) * a.x_ls];
        const double p = __dmul_rn(x1, c), q = __dmul_rn(x2, s), r = __dmul_rn(x1, s), t = __dmul_rn(x2, c);
        o[j * a.o_ls] = a.conj ? __dadd_rn(p, q) : __dsub_rn(p, q);
        o[(j + a.half) * a.o_ls] = a.conj ? __dadd_rn(-r, t) : __dadd_rn(r, t);
    }
}

template <typename T>
void launch_typed(const RopeArgs& a, cudaStream_t st) {
    constexpr int N = Vec16<T>::N;
    const int e = static_cast<int>(sizeof(T));
    auto al = [&](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    bool vec = a.half % N == 0 && a.x_ls == 1 && a.o_ls == 1 && a.c_ls == 1 && a.s_ls == 1 && al(a.x) && al(a.out) && al(a.cos) && al(a.sin);
    for (int d = 0; d < a.nd && vec; ++d)
        vec = (a.xs[d] * e) % 16 == 0 && (a.os[d] * e) % 16 == 0 && (a.cs[d] * e) % 16 == 0 && (a.ss[d] * e) % 16 == 0;
    if (vec) {
        const int vph = static_cast<int>(a.half / N);
        const int64_t total = a.n_lead * vph;
        const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 148ll * 64));
        // 32-bit index arithmetic when every element offset of the four tensors fits
        int64_t span = a.half * 2;
        for (int d = 0; d < a.nd; ++d) span += (a.size[d] - 1) * std::max(std::max(a.xs[d], a.os[d]), std::max(a.cs[d], a.ss[d]));
        constexpr int HP = 4;
        const bool shared_rows = a.nd >= 1 && a.cs[a.nd - 1] == 0 && a.ss[a.nd - 1] == 0 && a.size[a.nd - 1] % HP == 0;   // one table row per token, for all its heads
        const bool idx32 = total < (1ll << 31) && span < (1ll << 31);
        if (shared_rows) {
            const int64_t total_h = total / HP;
            const unsigned blocks_h = static_cast<unsigned>(std::min<int64_t>((total_h + 255) / 256, 148ll * 64));
            if (idx32)
                rope_vec_heads_kernel<T, uint32_t, HP><<<blocks_h, 256, 0, st>>>(a, vph, total_h);
            else
                rope_vec_heads_kernel<T, int64_t, HP><<<blocks_h, 256, 0, st>>>(a, vph, total_h);
        } else if (idx32) {
            rope_vec_kernel<T, uint32_t><<<blocks, 256, 0, st>>>(a, vph, total);
        } else {
            rope_vec_kernel<T, int64_t><<<blocks, 256, 0, st>>>(a, vph, total);
        }
    } else {
        const int64_t total = a.n_lead * a.half;
        const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 148ll * 64));
        rope_scalar_kernel<T><<<blocks, 256, 0, st>>>(a, total);
    }
}

// V2 (diopi_test/python/conformance/customized_test.py:843-852): query and key [T, H*dim] are rotated in place,
// x = x * cos + rotate_half(x) * sin with rotate_half(x) = (-x2, x1) and cos/sin as wide as the head. The golden
// works in the dtype of the tensors: both products and the sum are each rounded to that dtype.
template <typename T>
struct RtT {
    static __device__ __forceinline__ float r(float v) { return Cvt<T>::to_f(Cvt<T>::from_f(v)); }
};
template <>
struct RtT<float> {
    static __device__ __forceinline__ float r(float v) { return v; }
};

template <typename T>
__global__ void __launch_bounds__(256) rope_v2_kernel(RopeV2Args a, int64_t total) {
    const int64_t half = a.dim / 2;
    const int64_t heads = a.q_heads + a.k_heads;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t j = i % half;
        const int64_t th = i / half;
        const int64_t hh = th % heads;
        const int64_t t = th / heads;
        const bool is_q = hh < a.q_heads;
        const int64_t h = is_q ? hh : hh - a.q_heads;
        T* x = (is_q ? static_cast<T*>(a.q) + t * a.q_s0 : static_cast<T*>(a.kk) + t * a.k_s0) + h * a.dim;
        const T* c = static_cast<const T*>(a.cos) + t * a.c_st + h * a.c_sh;
        const T* s = static_cast<const T*>(a.sin) + t * a.s_st + h * a.s_sh;
        const float x1 = Cvt<T>::to_f(x[j]), x2 = Cvt<T>::to_f(x[j + half]);
        const float o1 = RtT<T>::r(__fadd_rn(RtT<T>::r(__fmul_rn(x1, Cvt<T>::to_f(c[j]))), RtT<T>::r(__fmul_rn(-x2, Cvt<T>::to_f(s[j])))));
        const float o2 = RtT<T>::r(__fadd_rn(RtT<T>::r(__fmul_rn(x2, Cvt<T>::to_f(c[j + half]))), RtT<T>::r(__fmul_rn(x1, Cvt<T>::to_f(s[j + half])))));
        x[j] = Cvt<T>::from_f(o1);
        x[j + half] = Cvt<T>::from_f(o2);
    }
}

__global__ void __launch_bounds__(256) rope_v2_f64_kernel(RopeV2Args a, int64_t total) {
    const int64_t half = a.dim / 2;
    const int64_t heads = a.q_heads + a.k_heads;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t j = i % half;
        const int64_t th = i / half;
        const int64_t hh = th % heads;
        const int64_t t = th / heads;
        const bool is_q = hh < a.q_heads;
        const int64_t h = is_q ? hh : hh - a.q_heads;
        double* x = (is_q ? static_cast<double*>(a.q) + t * a.q_s0 : static_cast<double*>(a.kk) + t * a.k_s0) + h * a.dim;
        const double* c = static_cast<const double*>(a.cos) + t * a.c_st + h * a.c_sh;
        const double* s = static_cast<const double*>(a.sin) + t * a.s_st + h * a.s_sh;
        const double x1 = x[j], x2 = x[j + half];
        x[j] = __dadd_rn(__dmul_rn(x1, c[j]), __dmul_rn(-x2, s[j]));
        x[j + half] = __dadd_rn(__dmul_rn(x2, c[j + half]), __dmul_rn(x1, s[j + half]));
    }
}

// The step in front of decode attention in one launch: q_out = rope(q); k_pool[dest_loc[t]] = rope(k[t]);
// v_pool[dest_loc[t]] = v[t]. The same arithmetic as rope_vec_kernel and the same slot rule as the row scatter
// (negative slots count from the end, out-of-range slots are reported and skipped), so the result equals the
// four separate calls bit for bit; the rotated key is never written to a tensor of its own.
// One thread per 16-byte vector pair (q, k) or per 16-byte vector (v). (Four heads per thread, as in
// rope_vec_heads_kernel, measured slower here: 4.95 against 5.34 TB/s; the scattered pool rows gain nothing from it.)
template <typename T>
__global__ void __launch_bounds__(256) rope_store_kv_kernel(RopeStoreArgs a, uint32_t vph, uint32_t per_token, uint32_t total) {
    constexpr int N = Vec16<T>::N;
    const uint32_t wq = static_cast<uint32_t>(a.Hq) * vph, wk = static_cast<uint32_t>(a.Hk) * vph;
    const uint32_t stride = gridDim.x * blockDim.x;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint32_t t = i / per_token;
        uint32_t r = i - t * per_token;
        const T* src;
        T* dst;
        if (r < wq) {
            const uint32_t h = r / vph;
            r -= h * vph;
            src = static_cast<const T*>(a.q) + static_cast<int64_t>(t) * a.q_s0 + static_cast<int64_t>(h) * a.D;
            dst = static_cast<T*>(a.q_out) + static_cast<int64_t>(t) * a.qo_s0 + static_cast<int64_t>(h) * a.D;
        } else {
            int64_t slot = load_index(a.dest, t);
            if (slot < 0) slot += a.slots;
            if (slot < 0 || slot >= a.slots) {
                if (r == wq) report_status(a.status, 1);
                continue;
            }
            r -= wq;
            if (r >= wk) {  // a vector of the value row: plain copy
                r -= wk;
                const uint4* vs = reinterpret_cast<const uint4*>(static_cast<const T*>(a.v) + static_cast<int64_t>(t) * a.v_s0) + r;
                uint4* vd = reinterpret_cast<uint4*>(static_cast<T*>(a.v_pool) + slot * a.vp_s0) + r;
                *vd = __ldcs(vs);
                continue;
            }
            const uint32_t h = r / vph;
            r -= h * vph;
            src = static_cast<const T*>(a.k) + static_cast<int64_t>(t) * a.k_s0 + static_cast<int64_t>(h) * a.D;
            dst = static_cast<T*>(a.k_pool) + slot * a.kp_s0 + static_cast<int64_t>(h) * a.D;
        }
        const int64_t half = a.D / 2;
        const uint4 r1 = __ldcs(reinterpret_cast<const uint4*>(src) + r);
        const uint4 r2 = __ldcs(reinterpret_cast<const uint4*>(src + half) + r);
        const uint4 rc = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(a.cos) + static_cast<int64_t>(t) * a.c_s0) + r);
        const uint4 rs = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(a.sin) + static_cast<int64_t>(t) * a.s_s0) + r);
        float x1[N], x2[N], c[N], sn[N], o1[N], o2[N];
        unpack16<T>(r1, x1);
        unpack16<T>(r2, x2);
        unpack16<T>(rc, c);
        unpack16<T>(rs, sn);
#pragma unroll
        for (int e = 0; e < N; ++e) {
            if (sizeof(T) == 2)
                rotate16(x1[e], x2[e], c[e], sn[e], a.conj, o1[e], o2[e]);
            else
                rotate(x1[e], x2[e], c[e], sn[e], a.conj, o1[e], o2[e]);
        }
        *(reinterpret_cast<uint4*>(dst) + r) = pack16<T>(o1);
        *(reinterpret_cast<uint4*>(dst + half) + r) = pack16<T>(o2);
    }
}

template <typename T>
bool launch_store_typed(const RopeStoreArgs& a, cudaStream_t st) {
    constexpr int N = Vec16<T>::N;
    const int e = static_cast<int>(sizeof(T));
    if (a.D % (2 * N) != 0) return false;
    auto al = [&](const void* p, int64_t s0) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) % 16 == 0 && (s0 * e) % 16 == 0); };
    if (!al(a.q, a.q_s0) || !al(a.q_out, a.qo_s0) || !al(a.k, a.k_s0) || !al(a.k_pool, a.kp_s0) || !al(a.v, a.v_s0) || !al(a.v_pool, a.vp_s0) ||
        !al(a.cos, a.c_s0) || !al(a.sin, a.s_s0))
        return false;
    const int64_t vph = a.D / 2 / N;
    const int64_t per_token = (a.Hq + a.Hk) * vph + (a.v ? a.Hk * 2 * vph : 0);
    const int64_t total = a.T * per_token;
    if (total >= (1ll << 31)) return false;
    const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 148ll * 64));
    rope_store_kv_kernel<T><<<blocks, 256, 0, st>>>(a, static_cast<uint32_t>(vph), static_cast<uint32_t>(per_token), static_cast<uint32_t>(total));
    return true;
}

}  // namespace

void launch_rope_v2(const RopeV2Args& a, cudaStream_t st) {
    const int64_t total = a.T * (a.q_heads + a.k_heads) * (a.dim / 2);
    if (total == 0) return;
    const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 148ll * 64));
    switch (a.dt) {
        case Dt::F16: rope_v2_kernel<__half><<<blocks, 256, 0, st>>>(a, total); break;
        case Dt::BF16: rope_v2_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(a, total); break;
        case Dt::F32: rope_v2_kernel<float><<<blocks, 256, 0, st>>>(a, total); break;
        case Dt::F64: rope_v2_f64_kernel<<<blocks, 256, 0, st>>>(a, total); break;
    }
}

bool launch_rope_store_kv(const RopeStoreArgs& a, cudaStream_t st) {
    if (a.T == 0 || a.D == 0) return true;
    switch (a.dt) {
        case Dt::F16: return launch_store_typed<__half>(a, st);
        case Dt::BF16: return launch_store_typed<__nv_bfloat16>(a, st);
        case Dt::F32: return launch_store_typed<float>(a, st);
        default: return false;
    }
}

void launch_rope(const RopeArgs& a, cudaStream_t st) {
    if (a.n_lead == 0 || a.half == 0) return;
    switch (a.dt) {
        case Dt::F16: launch_typed<__half>(a, st); break;
        case Dt::BF16: launch_typed<__nv_bfloat16>(a, st); break;
        case Dt::F32: launch_typed<float>(a, st); break;
        case Dt::F64: {
            const int64_t total = a.n_lead * a.half;
            const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 148ll * 64));
            rope_scalar_f64_kernel<<<blocks, 256, 0, st>>>(a, total);
            break;
        }
    }
}

}  // namespace k
}  // namespace b200
