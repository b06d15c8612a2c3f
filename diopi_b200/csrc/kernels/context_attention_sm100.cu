// Tensor-core causal prefill for sm_100a: tcgen05.mma with accumulators in TMEM, operands staged by TMA.
// Path of diopiContextAttentionInference for fp16/bf16, head_dim 128, dense 16-byte aligned rows; every
// other shape runs on the blockwise SIMT kernel. Replaces the per-request matmul/mask/softmax/matmul
// chain of impl/torch/functions/functions_lightllm.cpp:109-147.
//
// One CTA = one tile of 128 query rows of one (request, head); two CTAs share an SM so that one CTA's
// soft-max overlaps the other's MMAs. Per CTA, for key blocks of 64 up to the causal limit:
//   warp 0 (one lane)  TMA: Q once (two 64-wide boxes, 128-byte swizzle), then K_j and V_j into a 2-stage ring
//   warp 1 (one lane)  issues both products, each as soon as its inputs are ready (probing the barriers, never
//                      blocking on one while the other could go):
//                        S_j = Q K_j^T  tcgen05.mma M128 N64 K16 x 8, both operands K-major from shared memory,
//                                       into TMEM buffer S[j%2] once P V of block j - 2 has released it
//                        O  += P_j V_j  tcgen05.mma M128 N128 K16 x 4, A = P_j read from TMEM, B = V_j MN-major
//   warps 2-5          thread = query row: tcgen05.ld of its S row, causal/length mask, online soft-max in base 2
//                      (scale and maximum folded into one fma + ex2.approx per score; the reference maximum is
//                      only raised when the row maximum grew by more than 2^8, and only then is O in TMEM
//                      rescaled), P_j packed to 16 bit and written over the S cells just read
// The L x L score and mask tensors of the reference never exist; FLOPs counted = 4*D*L*(L+1)/2 per head.
//
// All waits are bounded (2 s); a wait that runs out sets a flag, every role leaves its loop, TMEM is
// freed and the status word is written. No TMA multicast is used.
#include <cuda.h>

#include <mutex>

#include <type_traits>

#include "dev_util.cuh"
#include "sm100_ptx.cuh"

namespace b200 {
namespace k {

namespace {

using namespace sm100;  // NOLINT

constexpr int BM = 128;      // query rows per CTA
constexpr int BN = 64;       // keys per block
constexpr int HD = 128;      // head dim
constexpr int kStages = 2;   // K/V ring
constexpr int kDefaultPolyEvery = 8;  // share of the exponentials computed on the fma pipe (see prefill_tc_kernel)
constexpr int kThreads = 192;
constexpr float kLog2e = 1.4426950408889634f;

// shared memory map (bytes); every operand tile starts on a 1024-byte boundary (128-byte swizzle atoms)
constexpr int kQBytes = BM * HD * 2;            // 32 KB: two [128 x 64] blocks
constexpr int kKStage = BN * HD * 2;            // 16 KB: two [64 x 64] blocks
constexpr int kVStage = BN * HD * 2;            // 16 KB
constexpr int kOffQ = 0;
constexpr int kOffK = kOffQ + kQBytes;
constexpr int kOffV = kOffK + kStages * kKStage;
constexpr int kOffBar = kOffV + kStages * kVStage;   // 96 KB
constexpr int kNumBars = 15;
constexpr int kOffTmemSlot = kOffBar + kNumBars * 8;
constexpr int kOffFlag = kOffTmemSlot + 8;
constexpr int kSmemBytes = kOffFlag + 8;          // two CTAs per SM: 2 * (96.2 KB + 1 KB reserved) of the SM's 228 KB

// TMEM columns (fp32 cells): S[0] 0..63, S[1] 64..127 (P_j overwrites the first 32 cells of S[j%2]), O 128..255
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS0 = 0, kColO = 128;

enum Bar { Q_FULL = 0, K_FULL = 1, V_FULL = 3, K_EMPTY = 5, V_EMPTY = 7, S_FULL = 9, S_EMPTY = 11, P_FULL = 13, O_FULL = 14 };

struct TcParams {
    IndexArg b_start, b_len;
    int B, H;
    int64_t total_rows;
    void* out;
    int64_t o_s0, o_s1;
    int n_tiles_max;
    float scale_log2;
    int* status;
    int64_t uniform_len;   // > 0: request i owns rows [i * uniform_len, (i + 1) * uniform_len)
    int kv_group;          // query heads per K/V head
};

// 2^x by the special-function unit alone (ex2.approx.ftz): -inf gives 0, no range fix-up code around it.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two fp32 operations per instruction (fma.rn.f32x2 / add.rn.f32x2 on 64-bit register pairs): the soft-max warps are
// bound by instruction issue next to the special-function unit, and these halve the scale-and-shift and row-sum work.
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b, float c) {
    uint64_t ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %1};" : "=l"(rb) : "f"(b));
    asm("mov.b64 %0, {%1, %1};" : "=l"(rc) : "f"(c));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(rd));
}
__device__ __forceinline__ void fadd2(float& d0, float& d1, float a0, float a1) {
    uint64_t ra, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rd) : "f"(d0), "f"(d1));
    asm("add.rn.f32x2 %0, %0, %1;" : "+l"(rd) : "l"(ra));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(rd));
}
// 2^x for a pair of values on the fma pipe (no special-function unit): x = j + f with j = round(x), f in
// [-0.5, 0.5]; 2^f by a cubic (relative error 7.5e-5, a third of the rounding step of an fp16 probability), 2^j by
// adding j to the exponent field. The special-function unit does 16 ex2 per clock and SM, which for head_dim 128 takes
// as long as the two matrix products of a tile; moving part of the exponentials here shortens the longest stage.
// x <= -125 (masked scores are -inf) gives 2^-125, which is nothing in the row sum and packs to 0.
__device__ __forceinline__ void poly_exp2_pair(float& a, float& b) {
    constexpr float kMagic = 12582912.f;  // 1.5 * 2^23: the low mantissa bits of x + kMagic hold round(x)
    uint64_t x, t, j, f, pz, cm, cnm, c1, c2, c3, c0;
    const float xa = fmaxf(a, -125.f), xb = fmaxf(b, -125.f);
    asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(xa), "f"(xb));
    asm("mov.b64 %0, {%1, %1};" : "=l"(cm) : "f"(kMagic));
    asm("mov.b64 %0, {%1, %1};" : "=l"(cnm) : "f"(-kMagic));
    asm("mov.b64 %0, {%1, %1};" : "=l"(c0) : "f"(0.9999280571937561f));
    asm("mov.b64 %0, {%1, %1};" : "=l"(c1) : "f"(0.6932609677314758f));
    asm("mov.b64 %0, {%1, %1};" : "=l"(c2) : "f"(0.2426111251115799f));
    asm("mov.b64 %0, {%1, %1};" : "=l"(c3) : "f"(0.0551716648042202f));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(t) : "l"(x), "l"(cm));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(j) : "l"(t), "l"(cnm));
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(f) : "l"(x), "l"(j));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(pz) : "l"(c3), "l"(f), "l"(c2));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(pz) : "l"(pz), "l"(f), "l"(c1));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(pz) : "l"(pz), "l"(f), "l"(c0));
    float pa, pb, ta, tb;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(pa), "=f"(pb) : "l"(pz));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(ta), "=f"(tb) : "l"(t));
    a = __int_as_float(__float_as_int(pa) + (__float_as_int(ta) << 23));
    b = __int_as_float(__float_as_int(pb) + (__float_as_int(tb) << 23));
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    if (BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// kPolyEvery: of every kPolyEvery groups of four scores, one computes two of its exponentials on the fma pipe
// (1: half of all exponentials, 2: a quarter, 4: an eighth, 8: a sixteenth, 0: none).
template <bool BF16, int kPolyEvery>
__global__ void __launch_bounds__(kThreads, 2) prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                                                   const __grid_constant__ CUtensorMap map_v, const TcParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffTmemSlot);
    volatile int* give_up = reinterpret_cast<volatile int*>(smem + kOffFlag);
    auto bar = [&](int i) { return smem_u32(&bars[i]); };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y;
    const int hkv = h / p.kv_group;   // grouped-query attention: several query heads share one K/V head

    // ---- which (request, row tile) is this CTA? Heaviest tiles (late rows) are handed out first. ----
    int req = -1;
    int64_t L = 0, start = 0, r0 = 0;
    {
        const int64_t flat = static_cast<int64_t>(p.n_tiles_max) - 1 - blockIdx.x;
        int64_t before = 0;
        for (int i = 0; i < p.B; ++i) {
            int64_t Li = p.uniform_len > 0 ? p.uniform_len : load_index(p.b_len, i);
            const int64_t si = p.uniform_len > 0 ? i * p.uniform_len : load_index(p.b_start, i);
            if (Li <= 0 || si < 0 || si >= p.total_rows) continue;
            Li = imin64(Li, p.total_rows - si);
            const int64_t nt = (Li + BM - 1) / BM;
            if (flat < before + nt) {
                req = i;
                L = Li;
                start = si;
                r0 = (flat - before) * BM;
                break;
            }
            before += nt;
        }
    }
    if (req < 0) return;  // the whole CTA leaves together, before any barrier or TMEM use
    const int nblk = static_cast<int>((imin64(L, r0 + BM) + BN - 1) / BN);

    if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte aligned base; refuse rather than compute garbage
        if (tid == 0) report_status(p.status, 3);
        return;
    }
    if (tid == 0) {
        mbar_init(bar(Q_FULL), 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar(K_FULL + s), 1);
            mbar_init(bar(V_FULL + s), 1);
            mbar_init(bar(K_EMPTY + s), 1);
            mbar_init(bar(V_EMPTY + s), 1);
            mbar_init(bar(S_FULL + s), 1);
            mbar_init(bar(S_EMPTY + s), 1);   // freed by the commit that follows P V of the block that used the buffer
        }
        mbar_init(bar(P_FULL), 4);
        mbar_init(bar(O_FULL), 1);
        *give_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ================================ TMA producer =================================
        if (lane == 0) {
            const int row0 = static_cast<int>(start + r0);
            mbar_expect_tx(bar(Q_FULL), kQBytes);
            tma_load_3d(smem_u32(smem + kOffQ), &map_q, 0, h, row0, bar(Q_FULL));
            tma_load_3d(smem_u32(smem + kOffQ + BM * 128), &map_q, 64, h, row0, bar(Q_FULL));
            for (int j = 0; j < nblk; ++j) {
                const int s = j % kStages;
                const uint32_t ph = static_cast<uint32_t>((j / kStages) & 1);
                const int krow = static_cast<int>(start + static_cast<int64_t>(j) * BN);
                if (!mbar_wait(bar(K_EMPTY + s), ph ^ 1u, give_up)) break;
                mbar_expect_tx(bar(K_FULL + s), kKStage);
                tma_load_3d(smem_u32(smem + kOffK + s * kKStage), &map_k, 0, hkv, krow, bar(K_FULL + s));
                tma_load_3d(smem_u32(smem + kOffK + s * kKStage + BN * 128), &map_k, 64, hkv, krow, bar(K_FULL + s));
                if (!mbar_wait(bar(V_EMPTY + s), ph ^ 1u, give_up)) break;
                mbar_expect_tx(bar(V_FULL + s), kVStage);
                tma_load_3d(smem_u32(smem + kOffV + s * kVStage), &map_v, 0, hkv, krow, bar(V_FULL + s));
                tma_load_3d(smem_u32(smem + kOffV + s * kVStage + BN * 128), &map_v, 64, hkv, krow, bar(V_FULL + s));
            }
        }
    } else if (warp == 1) {
        // ================================ MMA issuer ===================================
        if (lane == 0) {
            const uint32_t idesc_qk = make_idesc(BM, BN, BF16 ? 1 : 0, 0);
            const uint32_t idesc_pv = make_idesc(BM, HD, BF16 ? 1 : 0, 1);
            const uint32_t q_addr = smem_u32(smem + kOffQ);
            bool ok = mbar_wait(bar(Q_FULL), 0, give_up);
            // Event driven: Q K^T of the next block and P V of the oldest finished soft-max are issued in whatever
            // order their inputs become ready, so a ready P never queues behind a Q K^T that still waits for its
            // S buffer, and the other way round.
            int nqk = 0, npv = 0;
            unsigned long long idle_since = 0;
            while (ok && npv < nblk) {
                bool progressed = false;
                if (npv < nqk) {
                    const int i = npv;
                    const int s = i % kStages;
                    if (mbar_test(bar(P_FULL), static_cast<uint32_t>(i & 1)) && mbar_test(bar(V_FULL + s), static_cast<uint32_t>((i / kStages) & 1))) {
                        tc_fence_after();
                        const uint32_t v_addr = smem_u32(smem + kOffV + s * kVStage);
#pragma unroll
                        for (int t = 0; t < BN / 16; ++t) {
                            // B = V [64 keys x 128 d], MN-major: 16 keys = 16 rows of 128 bytes; the second 64-wide d block is 8 KB further
                            const uint64_t bd = make_desc(v_addr + t * 16 * 128, BN * 128, 1024);
                            // A = P in TMEM: 16 keys = 8 cells of the S buffer the soft-max threads overwrote
                            umma_ts(tmem_base + kColO, tmem_base + kColS0 + s * BN + t * 8, bd, idesc_pv, (i > 0 || t > 0) ? 1u : 0u);
                        }
                        umma_commit(bar(S_EMPTY + s));   // the S/P buffer may be overwritten by Q K^T of block i + 2
                        umma_commit(bar(V_EMPTY + s));
                        umma_commit(bar(O_FULL));
                        ++npv;
                        progressed = true;
                    }
                }
                if (nqk < nblk) {
                    const int s = nqk % kStages;
                    const uint32_t ph = static_cast<uint32_t>((nqk / kStages) & 1);
                    if (mbar_test(bar(K_FULL + s), ph) && mbar_test(bar(S_EMPTY + s), ph ^ 1u)) {
                        tc_fence_after();
                        const uint32_t k_addr = smem_u32(smem + kOffK + s * kKStage);
#pragma unroll
                        for (int t = 0; t < HD / 16; ++t) {
                            // both operands K-major; d block t/4 (64 wide), 16 d = 32 bytes inside the swizzled row
                            const uint64_t ad = make_desc(q_addr + (t / 4) * (BM * 128) + (t % 4) * 32, 0, 1024);
                            const uint64_t bd = make_desc(k_addr + (t / 4) * (BN * 128) + (t % 4) * 32, 0, 1024);
                            umma(tmem_base + kColS0 + s * BN, ad, bd, idesc_qk, t > 0 ? 1u : 0u);
                        }
                        umma_commit(bar(S_FULL + s));
                        umma_commit(bar(K_EMPTY + s));
                        ++nqk;
                        progressed = true;
                    }
                }
                if (progressed) {
                    idle_since = 0;
                } else {
                    if (*give_up) break;
                    const unsigned long long now = global_ns();
                    if (idle_since == 0) idle_since = now;
                    if (now - idle_since > kWaitLimitNs) {
                        *give_up = 1;
                        break;
                    }
                }
            }
        }
    } else {
        // ================================ soft-max warps: thread = query row ==========================
        const int quarter = warp & 3;                 // the TMEM lane quarter this warp may touch
        const int row = quarter * 32 + lane;          // row inside the tile
        const int64_t rr = r0 + row;                  // row inside the request
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < nblk; ++j) {
            const int s = j % kStages;
            const uint32_t ph = static_cast<uint32_t>((j / kStages) & 1);
            if (!warp_wait(bar(S_FULL + s), ph, give_up)) {
                ok = false;
                break;
            }
            tc_fence_after();
            uint32_t u0[32], u1[32];
            tmem_ld32(lane_base + kColS0 + s * BN, u0);
            tmem_ld32(lane_base + kColS0 + s * BN + 32, u1);
            tmem_wait_ld();

            // Raw scores stay in the registers the TMEM load filled; scale and maximum are folded into the
            // exponent: p = 2^(s * scale - m) is one fma and one ex2 per element.
            float sc[BN];
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                sc[c] = __uint_as_float(u0[c]);
                sc[c + 32] = __uint_as_float(u1[c]);
            }
            const int64_t key0 = static_cast<int64_t>(j) * BN;
            if ((key0 + BN - 1 > r0) || (key0 + BN > L)) {  // block touches the diagonal or the request's end
                const int64_t lim = imin64(rr, L - 1) - key0;  // last allowed column of this row inside the block
#pragma unroll
                for (int c = 0; c < BN; ++c)
                    if (c > lim) sc[c] = -INFINITY;
            }
            // three-input maximum: 32 instructions for 64 values, in four independent chains
            float mx0 = fmaxf(sc[0], sc[1]), mx1 = fmaxf(sc[2], sc[3]), mx2 = fmaxf(sc[4], sc[5]), mx3 = fmaxf(sc[6], sc[7]);
#pragma unroll
            for (int c = 8; c < BN; c += 8) {
                mx0 = fmax3(mx0, sc[c], sc[c + 1]);
                mx1 = fmax3(mx1, sc[c + 2], sc[c + 3]);
                mx2 = fmax3(mx2, sc[c + 4], sc[c + 5]);
                mx3 = fmax3(mx3, sc[c + 6], sc[c + 7]);
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;  // scale > 0: max commutes with it
            // Lazy maximum: keep the old reference while the new maximum is within 2^8 of it.
            const float m_new = fmaxf(m_used, mx);
            const bool need = (m_new > m_used + 8.0f) || (m_used == -INFINITY && m_new != -INFINITY);
            if (__any_sync(0xffffffffu, need)) {
                const float m_next = need ? m_new : m_used;
                const float alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_next);
                if (j > 0) {
                    if (!warp_wait(bar(O_FULL), static_cast<uint32_t>((j - 1) & 1), give_up)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int c4 = 0; c4 < HD / 32; ++c4) {
                        uint32_t o[32];
                        tmem_ld32(lane_base + kColO + c4 * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                        tmem_st32(lane_base + kColO + c4 * 32, o);
                    }
                    tmem_wait_st();
                }
                l *= alpha;
                m_used = m_next;
            }
            const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
            float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
#pragma unroll
            for (int c = 0; c < BN; c += 4) {
                ffma2(sc[c], sc[c + 1], sc[c], sc[c + 1], p.scale_log2, neg_m);
                ffma2(sc[c + 2], sc[c + 3], sc[c + 2], sc[c + 3], p.scale_log2, neg_m);
                sc[c] = fast_exp2(sc[c]);
                sc[c + 1] = fast_exp2(sc[c + 1]);
                if (kPolyEvery > 0 && (c / 4) % (kPolyEvery > 0 ? kPolyEvery : 1) == 0) {
                    poly_exp2_pair(sc[c + 2], sc[c + 3]);
                } else {
                    sc[c + 2] = fast_exp2(sc[c + 2]);
                    sc[c + 3] = fast_exp2(sc[c + 3]);
                }
                fadd2(rs0, rs1, sc[c], sc[c + 1]);
                fadd2(rs2, rs3, sc[c + 2], sc[c + 3]);
            }
            l += (rs0 + rs1) + (rs2 + rs3);
            // P_j over the S cells this thread just consumed: cell c holds keys 2c (low half) and 2c + 1
            uint32_t pk[32];
#pragma unroll
            for (int c = 0; c < 32; ++c) pk[c] = pack2<BF16>(sc[2 * c], sc[2 * c + 1]);
            tmem_st32(lane_base + kColS0 + s * BN, pk);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(P_FULL));
        }
        // The last two P V products may both still be in flight here (a finished S_j only proves that P V of block
        // j - 2 is done), and a parity wait can only tell neighbouring phases apart: wait for them one by one.
        if (ok && nblk >= 2) ok = warp_wait(bar(O_FULL), static_cast<uint32_t>((nblk - 2) & 1), give_up);
        if (ok && warp_wait(bar(O_FULL), static_cast<uint32_t>((nblk - 1) & 1), give_up)) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const bool store = rr < L;
            unsigned char* dst = static_cast<unsigned char*>(p.out) + ((start + rr) * p.o_s0 + static_cast<int64_t>(h) * p.o_s1) * 2;
#pragma unroll
            for (int c4 = 0; c4 < HD / 32; ++c4) {
                uint32_t o[32];
                tmem_ld32(lane_base + kColO + c4 * 32, o);
                tmem_wait_ld();
                if (store) {
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        uint4 v;
                        v.x = pack2<BF16>(__uint_as_float(o[ch * 8 + 0]) * inv, __uint_as_float(o[ch * 8 + 1]) * inv);
                        v.y = pack2<BF16>(__uint_as_float(o[ch * 8 + 2]) * inv, __uint_as_float(o[ch * 8 + 3]) * inv);
                        v.z = pack2<BF16>(__uint_as_float(o[ch * 8 + 4]) * inv, __uint_as_float(o[ch * 8 + 5]) * inv);
                        v.w = pack2<BF16>(__uint_as_float(o[ch * 8 + 6]) * inv, __uint_as_float(o[ch * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c4 * 64 + ch * 16) = v;
                    }
                }
            }
        }
    }

    // ---- common exit: everybody arrives, TMEM is returned by the warp that took it ----
    tc_fence_before();
    __syncthreads();
    if (*give_up) {
        if (tid == 0) report_status(p.status, 3);
        const unsigned long long t_begin = global_ns();
        while (global_ns() - t_begin < 2000000ull) __nanosleep(1000);  // let copies/MMAs still in flight finish
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(ptr);
    });
    return fn;
}

// 3-D view [D, H, rows] of a packed [rows, H, D] tensor; box = 64 elements x 1 head x `box_rows` rows, 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* base, int64_t rows, int H, int64_t s0, int64_t s1, int box_rows, bool bf16) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(HD), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(s1) * 2, static_cast<cuuint64_t>(s0) * 2};
    const cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace

void launch_prefill_tc(const PrefillArgs& a, int /*sm_count*/, int max_smem, cudaStream_t st, bool* taken) {
    *taken = false;
    if (a.force_simt) return;
    if (a.dt != Dt::F16 && a.dt != Dt::BF16) return;
    if (a.D != HD || a.H > 65535 || kSmemBytes > max_smem) return;
    if (a.total_rows >= (1ll << 31) - BM) return;
    auto ok = [](const void* p, int64_t s0, int64_t s1) {
        return reinterpret_cast<uintptr_t>(p) % 16 == 0 && (s0 * 2) % 16 == 0 && (s1 * 2) % 16 == 0 && s0 > 0 && s1 > 0;
    };
    if (!ok(a.q, a.q_s0, a.q_s1) || !ok(a.kmat, a.k_s0, a.k_s1) || !ok(a.vmat, a.v_s0, a.v_s1) || !ok(a.out, a.o_s0, a.o_s1)) return;
    const bool bf16 = a.dt == Dt::BF16;
    CUtensorMap mq, mk, mv;
    if (!make_map(&mq, a.q, a.total_rows, a.H, a.q_s0, a.q_s1, BM, bf16)) return;
    if (!make_map(&mk, a.kmat, a.total_rows, a.H / a.kv_group, a.k_s0, a.k_s1, BN, bf16)) return;
    if (!make_map(&mv, a.vmat, a.total_rows, a.H / a.kv_group, a.v_s0, a.v_s1, BN, bf16)) return;

    TcParams p;
    p.b_start = a.b_start;
    p.b_len = a.b_len;
    p.B = a.B;
    p.H = a.H;
    p.total_rows = a.total_rows;
    p.out = a.out;
    p.o_s0 = a.o_s0;
    p.o_s1 = a.o_s1;
    p.n_tiles_max = static_cast<int>(a.total_rows / BM + a.B);
    p.scale_log2 = kLog2e / sqrtf(static_cast<float>(HD));
    p.status = nullptr;
    p.uniform_len = a.uniform_len;
    p.kv_group = a.kv_group;
    dim3 grid(p.n_tiles_max, a.H, 1);
    const int poly = kDefaultPolyEvery;
    auto go = [&](auto kern) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        kern<<<grid, kThreads, kSmemBytes, st>>>(mq, mk, mv, p);
    };
    auto pick = [&](auto bf) {
        constexpr bool B = decltype(bf)::value;
        switch (poly) {
            case 1: go(prefill_tc_kernel<B, 1>); break;
            case 2: go(prefill_tc_kernel<B, 2>); break;
            case 4: go(prefill_tc_kernel<B, 4>); break;
            case 8: go(prefill_tc_kernel<B, 8>); break;
            default: go(prefill_tc_kernel<B, 0>); break;
        }
    };
    if (bf16)
        pick(std::true_type{});
    else
        pick(std::false_type{});
    *taken = true;
}

}  // namespace k
}  // namespace b200
