// Device code shared by the decode kernels (token_decode.cu: one query head per K/V head; token_decode_gqa.cu:
// several query heads per K/V head): mbarrier and bulk-copy wrappers with bounded waits, the walk over a CTA's range
// of the flattened (request, token) pairs, slot lookup for both addressing forms, and the kernel that merges the
// split-KV partials. Each .cu file includes this inside its own translation unit.
#pragma once

#include <cfloat>

#include "dev_util.cuh"

namespace b200 {
namespace k {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // a wait longer than this is given up

// ---------------------------------------------------------------------------
// PTX wrappers: mbarrier + bulk copy.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Waits for the phase with the given parity. Gives up after kWaitLimitNs or as soon as another
// thread of the CTA has given up; returns false then.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* give_up) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0xffu) == 0) {
            if (*give_up) return false;
            if (global_ns() - t0 > kWaitLimitNs) {
                *give_up = 1;
                return false;
            }
        }
    }
    return true;
}
// One contiguous global -> shared copy; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar)
                 : "memory");
}

// 2^x by the special-function unit alone (ex2.approx.ftz): -inf gives 0, tiny results flush to 0, and there is no
// range fix-up code around it as there is around exp2f. Used in the streaming loop only.
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---------------------------------------------------------------------------
// Walks the stages of one CTA's token range. Producer and consumers run the same
// walk, so nothing but the data itself has to be handed over.
// ---------------------------------------------------------------------------
struct StageWalk {
    const int* pre;  // pre[i] = first flattened token of request i; pre[B] = total
    int t, t1, i;

    __device__ void init(const int* pre_, int B, int t0_, int t1_) {
        pre = pre_;
        t = t0_;
        t1 = t1_;
        int lo = 0, hi = B;  // smallest i with pre[i+1] > t
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (pre[mid + 1] > t)
                hi = mid;
            else
                lo = mid + 1;
        }
        i = lo;
    }
    // Next stage: tokens [j0, j0+cnt) of request req; last = the request's part in this CTA ends here.
    __device__ bool next(int TT, int& req, int& j0, int& cnt, bool& last) {
        if (t >= t1) return false;
        const int req_end = min(pre[i + 1], t1);
        cnt = min(TT, req_end - t);
        req = i;
        j0 = t - pre[i];
        t += cnt;
        last = (t == req_end);
        if (t == pre[i + 1] && t < t1) {
            do {
                ++i;
            } while (pre[i + 1] == t);
        }
        return true;
    }
};

// Pool row of token j of request r (L = clamped length of the request).
__device__ __forceinline__ int64_t token_slot(const DecodeArgs& a, int r, int L, int64_t j) {
    if (a.block_size > 0) {
        const int64_t blk = load_index(a.b_loc, r, j / a.block_size);
        return blk < 0 ? -1 : blk * a.block_size + j % a.block_size;
    }
    return load_index(a.b_loc, r, static_cast<int64_t>(a.max_input_len) - L + j);
}

// Clamped request length: never negative, never beyond the window b_loc holds.
__device__ __forceinline__ int request_len(const DecodeArgs& a, int i) {
    int64_t L = load_index(a.b_len, i);
    L = L < 0 ? 0 : L;
    L = L > a.max_input_len ? a.max_input_len : L;
    return static_cast<int>(L);
}

// Merges the partials of one (request, head) and writes out[i,h,:]. One warp each.
template <typename T>
__global__ void __launch_bounds__(128) decode_combine_kernel(const DecodeArgs a, int n_cta, const float* __restrict__ ws_acc,
                                                              const float* __restrict__ ws_ml, int64_t out_pass, int64_t ws_pass_acc,
                                                              int64_t ws_pass_ml) {
    __shared__ int s_part[4][2];
    ws_acc += blockIdx.z * ws_pass_acc;   // blockIdx.z: the pass (query head inside its group of K/V sharers)
    ws_ml += blockIdx.z * ws_pass_ml;
    const int i = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // start = sum of the lengths before request i, total = sum of all lengths
    int before = 0, all = 0;
    for (int r = threadIdx.x; r < a.B; r += blockDim.x) {
        const int L = request_len(a, r);
        all += L;
        if (r < i) before += L;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        before += __shfl_xor_sync(0xffffffffu, before, o);
        all += __shfl_xor_sync(0xffffffffu, all, o);
    }
    if (lane == 0) {
        s_part[warp][0] = before;
        s_part[warp][1] = all;
    }
    __syncthreads();
    before = s_part[0][0] + s_part[1][0] + s_part[2][0] + s_part[3][0];
    all = s_part[0][1] + s_part[1][1] + s_part[2][1] + s_part[3][1];

    // Which CTAs of the split kernel hold a part of request i: token range [first_token(c), first_token(c + 1)) each.
    const int h = blockIdx.y * 4 + warp;
    const int L = request_len(a, i);
    int c_first = 0, c_last = -1;
    auto first_token = [&](int c) { return static_cast<int>(static_cast<int64_t>(all) * c / n_cta); };
    if (L > 0) {
        // largest c with first_token(c) <= t: all * c / n_cta < t + 1, i.e. c <= ((t + 1) * n_cta - 1) / all. One division
        // each (a binary search over first_token cost eight 64-bit divisions per bound, microseconds of serial integer work).
        auto cta_of = [&](int t) {
            const int64_t c = ((static_cast<int64_t>(t) + 1) * n_cta - 1) / all;
            return static_cast<int>(c < n_cta - 1 ? c : n_cta - 1);
        };
        c_first = cta_of(before);
        c_last = cta_of(before + L - 1);
    }

    // Bit c - c_first of `live` = CTA c's range is not empty (an empty range wrote nothing); a request spans few CTAs.
    uint64_t live = 0;
    {
        int lo = first_token(c_first);
        for (int c = c_first; c <= c_last; ++c) {
            const int hi = first_token(c + 1);
            if (hi != lo && c - c_first < 64) live |= 1ull << (c - c_first);
            lo = hi;
        }
    }
    auto is_live = [&](int c) { return c - c_first < 64 ? ((live >> (c - c_first)) & 1ull) != 0 : first_token(c) != first_token(c + 1); };

    // Everything above read only the caller's inputs. The partials are written by the split kernel, which may
    // still be running when this kernel was launched early: wait for it to finish (no-op for a plain launch).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (h >= a.H) return;
    constexpr int R = 8;  // D <= 256 on this path
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    // Two passes with independent loads (one memory latency each): the maximum over the parts, then the weighted sum.
    float M = -INFINITY, Lsum = 0.f;
    for (int c = c_first; c <= c_last; ++c) {
        if (!is_live(c)) continue;
        M = fmaxf(M, ws_ml[((static_cast<int64_t>(c) + i) * a.H + h) * 2]);
    }
    const float Mr = (M == -INFINITY) ? 0.f : M;
    for (int c = c_first; c <= c_last; ++c) {
        if (!is_live(c)) continue;
        const int64_t slot_id = static_cast<int64_t>(c) + i;
        const float2 ml = *reinterpret_cast<const float2*>(ws_ml + (slot_id * a.H + h) * 2);
        const float w = exp2f(ml.x - Mr);
        Lsum = fmaf(ml.y, w, Lsum);
        const float* src = ws_acc + (slot_id * a.H + h) * a.D;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int d = lane + 32 * r;
            if (d < a.D) acc[r] = fmaf(src[d], w, acc[r]);
        }
    }
    const float inv = Lsum > 0.f ? 1.f / Lsum : 0.f;
    T* o = static_cast<T*>(a.out) + blockIdx.z * out_pass + static_cast<int64_t>(i) * a.out_s0 + static_cast<int64_t>(h) * a.out_s1;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = lane + 32 * r;
        if (d < a.D) o[d * a.out_s2] = Cvt<T>::from_f(acc[r] * inv);
    }
}

}  // namespace
}  // namespace k
}  // namespace b200
