// Causal prefill over a packed ragged batch (diopiContextAttentionInference).
// Replaces the per-request host loop and the materialised [1,H,L,L] mask/score tensors of
// impl/torch/functions/functions_lightllm.cpp:109-147; golden:
// diopi_test/python/conformance/customized_test.py:8-33,735-749.
// For query row r of request i (r relative to the request) and head h:
//   out[r] = sum_{j<=r} softmax_j(q[r].k[j] / sqrt(D)) * v[j]
// The additive mask of the reference is {+1 allowed, -1e8 masked}; the +1 cancels inside the
// softmax and exp(-1e8 - max) is exactly 0 in fp32, so skipping masked keys is identical.
//
// This file holds the blockwise SIMT kernel: any dtype (fp16/bf16/fp32), any D up to 256, never
// more than two K/V tiles of 32 keys in shared memory, fp32 arithmetic with an online softmax. It
// is the path for shapes the tensor-core kernel does not take (fp32, head dims other than 64, 128, 256, unaligned rows).
#include "dev_util.cuh"

namespace b200 {
namespace k {

void launch_prefill_tc(const PrefillArgs& a, int sm_count, int max_smem, cudaStream_t st, bool* taken);

namespace {

constexpr int kRowsPerCta = 8;  // one warp per query row
constexpr int kKeysPerTile = 32;
constexpr float kLog2e = 1.4426950408889634f;

template <typename T>
__global__ void __launch_bounds__(kRowsPerCta * 32) prefill_simt_kernel(const PrefillArgs a) {
    constexpr int R = 8;  // D <= 256
    extern __shared__ __align__(16) unsigned char smem[];
    const int D = a.D;
    const int kpad = D + (sizeof(T) == 2 ? 2 : 1);  // odd number of 32-bit words per K row: no bank conflicts
    T* sK = reinterpret_cast<T*>(smem);
    T* sV = sK + kKeysPerTile * kpad;
    float* sQ = reinterpret_cast<float*>(sV + kKeysPerTile * D);  // 32*(kpad+D) elements: a multiple of 4 bytes

    // The host does not know the lengths, so the grid is sized for the worst case
    // (sum of ceil(L_i/8) <= total_rows/8 + B); find which request and row tile this CTA is.
    const int h = blockIdx.y;
    const int hkv = h / a.kv_group;   // grouped-query attention: several query heads share one K/V head
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int req = -1;
    int64_t L = 0, start = 0, r0 = 0;
    {
        int64_t tiles_before = 0;
        const int64_t flat = blockIdx.x;
        for (int i = 0; i < a.B; ++i) {
            int64_t Li = a.uniform_len > 0 ? a.uniform_len : load_index(a.b_len, i);
            const int64_t si = a.uniform_len > 0 ? i * a.uniform_len : load_index(a.b_start, i);
            if (Li <= 0 || si < 0 || si >= a.total_rows) continue;
            Li = imin64(Li, a.total_rows - si);
            const int64_t nt = (Li + kRowsPerCta - 1) / kRowsPerCta;
            if (flat < tiles_before + nt) {
                req = i;
                L = Li;
                start = si;
                r0 = (flat - tiles_before) * kRowsPerCta;
                break;
            }
            tiles_before += nt;
        }
    }
    if (req < 0) return;
    const int64_t r = r0 + warp;  // my query row (relative)
    const bool row_ok = r < L;
    const float scale = kLog2e / sqrtf(static_cast<float>(D));

    float* myq = sQ + warp * D;
    for (int d = lane; d < D; d += 32)
        myq[d] = row_ok ? Cvt<T>::to_f(static_cast<const T*>(a.q)[(start + r) * a.q_s0 + static_cast<int64_t>(h) * a.q_s1 + d]) * scale : 0.f;

    float acc[R];
#pragma unroll
    for (int x = 0; x < R; ++x) acc[x] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int64_t last_key = imin64(L - 1, r0 + kRowsPerCta - 1);  // keys this CTA needs: [0, last_key]
    for (int64_t j0 = 0; j0 <= last_key; j0 += kKeysPerTile) {
        __syncthreads();
        const int nk = static_cast<int>(imin64(kKeysPerTile, last_key + 1 - j0));
        for (int idx = threadIdx.x; idx < nk * D; idx += blockDim.x) {
            const int jj = idx / D, d = idx - jj * D;
            sK[jj * kpad + d] = static_cast<const T*>(a.kmat)[(start + j0 + jj) * a.k_s0 + static_cast<int64_t>(hkv) * a.k_s1 + d];
            sV[jj * D + d] = static_cast<const T*>(a.vmat)[(start + j0 + jj) * a.v_s0 + static_cast<int64_t>(hkv) * a.v_s1 + d];
        }
        __syncthreads();
        if (!row_ok) continue;
        // lane = key: full dot product per lane
        const int64_t j = j0 + lane;
        float s = -INFINITY;
        if (lane < nk && j <= r) {
            float dot = 0.f;
            const T* kr = sK + lane * kpad;
            for (int d = 0; d < D; ++d) dot = fmaf(myq[d], Cvt<T>::to_f(kr[d]), dot);
            s = dot;
        }
        float tmax = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
        if (tmax == -INFINITY) continue;  // whole tile masked for this row
        const float m_new = fmaxf(m, tmax);
        const float alpha = exp2f(m - m_new);
        const float p = exp2f(s - m_new);  // 0 for masked lanes
        float psum = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
        l = l * alpha + psum;
#pragma unroll
        for (int x = 0; x < R; ++x) acc[x] *= alpha;
        for (int jj = 0; jj < nk; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            if (pj != 0.f) {
#pragma unroll
                for (int x = 0; x < R; ++x) {
                    const int d = lane + 32 * x;
                    if (d < D) acc[x] = fmaf(pj, Cvt<T>::to_f(sV[jj * D + d]), acc[x]);
                }
            }
        }
        m = m_new;
    }
    if (!row_ok) return;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* o = static_cast<T*>(a.out) + (start + r) * a.o_s0 + static_cast<int64_t>(h) * a.o_s1;
#pragma unroll
    for (int x = 0; x < R; ++x) {
        const int d = lane + 32 * x;
        if (d < D) o[d] = Cvt<T>::from_f(acc[x] * inv);
    }
}

template <typename T>
void launch_simt(const PrefillArgs& a, cudaStream_t st) {
    const int kpad = a.D + (sizeof(T) == 2 ? 2 : 1);
    const size_t smem = static_cast<size_t>(kKeysPerTile) * (kpad + a.D) * sizeof(T) + 16 + static_cast<size_t>(kRowsPerCta) * a.D * sizeof(float);
    const int64_t row_tiles = a.total_rows / kRowsPerCta + a.B;
    auto kern = prefill_simt_kernel<T>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    dim3 grid(static_cast<unsigned>(row_tiles), a.H, 1);
    kern<<<grid, kRowsPerCta * 32, smem, st>>>(a);
}

}  // namespace

const char* launch_prefill(const PrefillArgs& a, int sm_count, int max_smem, cudaStream_t st) {
    if (a.B <= 0 || a.H <= 0 || a.D <= 0 || a.total_rows <= 0) return "none";
    bool taken = false;
    launch_prefill_tc(a, sm_count, max_smem, st, &taken);
    if (taken) return "tensor-core";
    switch (a.dt) {
        case Dt::F16: launch_simt<__half>(a, st); break;
        case Dt::BF16: launch_simt<__nv_bfloat16>(a, st); break;
        case Dt::F32: launch_simt<float>(a, st); break;
        default: break;
    }
    return "simt";
}

}  // namespace k
}  // namespace b200
