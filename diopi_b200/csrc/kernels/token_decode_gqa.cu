// Paged-KV decode attention with grouped K/V heads: kv_group query heads read one K/V head
// (diopiPagedAttention with num_kv_heads < num_heads, proto/include/diopi/functions_ext.h:616-618; golden function
// diopi_test/python/conformance/customized_test.py:785-821, which repeats every K/V head kv_group times).
//
// One pass over the rows: a K/V row lands in shared memory once and every query head of its group consumes it there.
// Doing that with scalar FMAs would cost kv_group times the arithmetic of the one-to-one kernel per byte (at group 8
// the FMA pipe, not HBM, would be the limit), so the two small products run on the tensor cores with the query heads
// of a group as the M extent of mma.sync m16n8k16 (fp16/bf16 in, fp32 accumulate):
//     S [16 heads x 16 tokens] = Q_g [16 x D] K^T      (rows beyond kv_group are zero padding)
//     O [16 heads x D]        += P [16 x 16] V
// with the online softmax on the accumulator fragment in between, exactly the layout trick of blocked attention: the
// accumulator fragment of S is the A fragment of the second product. Tried and dropped: blocks of 8 tokens (m16n8k8 for the
// second product, six 33 KB stages instead of three 66 KB ones): 107 us where this form takes 97 us on 64 query heads
// over 8 K/V heads, the per-stage hand-over costs more than the shorter chain wins; a 128-register cap, so that the
// merge kernel's CTAs become resident beside this kernel's: 101 us; separate accumulators for even and odd k steps of
// Q K^T (shorter dependent chains): no change. Per stage the kernel pays about 0.24 us of hand-over on top of the bytes.
//
// Work split: the flattened (request, token) pairs are cut into equal ranges, one per CTA (as in token_decode.cu).
// Per CTA four producer warps look up slots and issue one bulk copy per row part (the K/V heads of this CTA:
// hg * D * 2 bytes) into a ring of shared-memory stages; rows are stored with a pitch of row bytes + 16, so that the
// eight rows an ldmatrix reads fall into different banks. Eight consumer warps: warp = (token block g, M tile, K/V head hl),
// one M tile of 16 query heads for groups up to 16 and 2, 4 or 8 tiles for groups up to 128 (they read the same rows in
// shared memory); a stage holds G = 8 / (hg * M tiles) blocks of 16 tokens. Every consumer warp keeps (m, l, O) of its (head, token block) in
// registers; at the end of a request's part the G token blocks are merged through shared memory and one partial per
// (CTA, request, query head) goes to scratch, in the layout decode_combine_kernel reads.
//
// Algorithmic bytes: 2 * sumL * Hkv * D * e (K and V, once) + 2 * B * Hq * D * e + index loads.
#include <type_traits>

#include "decode_common.cuh"
#include "token_decode_gqa.hpp"

namespace b200 {
namespace k {

namespace {

constexpr int kGqaConsumerWarps = 8;
constexpr int kGqaProducerWarps = 4;
constexpr int kGqaThreads = 32 * (kGqaConsumerWarps + kGqaProducerWarps);
constexpr int kGqaMaxStages = 16;
constexpr int kGqaMaxB = 2048;
constexpr int kBlockTokens = 16;   // tokens one warp step covers: the K extent of the second product

struct GqaPlan {
    int hg;           // K/V heads per CTA (1, 2, 4 or 8)
    int n_hg;         // CTAs along the head axis
    int MT;           // M tiles of 16 query heads per group: 1 for groups up to 16, 2, 4 or 8 for wider ones
    int G;            // token blocks per stage = consumer warps / (hg * MT)
    int TT;           // tokens per stage = 16 * G
    int pitch;        // bytes between rows of a stage: hg * D * 2 + 16
    int stage_bytes;  // K rows then V rows: 2 * TT * pitch
    int nstages;
    int n_cta;        // CTAs along the flattened token axis
    int smem_bytes;
    int off_bars, off_pre, off_red, off_flag;
    int red_floats_per_warp;   // rows a warp holds (kv_group, at most 16) * (D + 2)
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (std::is_same<T, __half>::value) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}
template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if constexpr (std::is_same<T, __half>::value) {
        __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    } else {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
}

template <typename T, int HD>
__global__ void __launch_bounds__(kGqaThreads, 1) decode_gqa_kernel(const DecodeArgs a, const GqaPlan p, float* __restrict__ ws_acc,
                                                                    float* __restrict__ ws_ml) {
    constexpr int KS = HD / 16;   // k steps of Q K^T
    constexpr int DN = HD / 8;    // n tiles of P V
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.off_bars);  // full[nstages], empty[nstages], red[2]
    int* pre = reinterpret_cast<int*>(smem + p.off_pre);
    float* red = reinterpret_cast<float*>(smem + p.off_red);
    volatile int* give_up = reinterpret_cast<volatile int*>(smem + p.off_flag);

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the merge kernel may become resident early

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    const int R = a.kv_group;
    const int Hkv = a.H / R;
    const int hg0 = blockIdx.y * p.hg;                 // first K/V head of this CTA
    const int heads_here = min(p.hg, Hkv - hg0);
    const uint32_t row_bytes = static_cast<uint32_t>(heads_here) * HD * 2u;

    if (tid == 0) {
        for (int s = 0; s < p.nstages; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[p.nstages + s]), kGqaConsumerWarps);
        }
        mbar_init(smem_u32(&bars[2 * p.nstages]), kGqaConsumerWarps);
        mbar_init(smem_u32(&bars[2 * p.nstages + 1]), kGqaConsumerWarps);
        *give_up = 0;
        pre[0] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < a.B; i += static_cast<int>(blockDim.x)) pre[i + 1] = request_len(a, i);
    __syncthreads();
    if (warp == 0) {
        int carry = 0;
        for (int base = 0; base < a.B; base += 32) {
            const int idx = base + lane;
            int v = idx < a.B ? pre[idx + 1] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int u = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += u;
            }
            if (idx < a.B) pre[idx + 1] = v + carry;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();

    const int total = pre[a.B];
    const int t0 = static_cast<int>(static_cast<int64_t>(total) * cta / p.n_cta);
    const int t1 = static_cast<int>(static_cast<int64_t>(total) * (cta + 1) / p.n_cta);
    const int TT = p.TT;
    const uint32_t v_off = static_cast<uint32_t>(TT) * static_cast<uint32_t>(p.pitch);

    if (warp >= kGqaConsumerWarps) {
        // =========================== producer warps ==============================
        // A stage's tokens are dealt out to the four warps (token pw + 4 i to warp pw), so a stage occupies only
        // TT / 4 lanes of each; the other lanes work on the stages after it: a warp looks up the slots of a batch of
        // 32 / (TT / 4) stages with one load per lane, and the batch after that is requested before the copies of this
        // one are issued. (With one stage of lookahead the slot load's latency, a microsecond under load, set the
        // time per stage.) Warp 0 also announces the bytes of each stage; a copy of another warp may land before the
        // announcement: the phase cannot complete before the announcing arrive, so the early bytes are only booked ahead.
        const int pw = warp - kGqaConsumerWarps;
        const int LPS = TT / kGqaProducerWarps;   // lanes per stage: 2, 4, 8 or 16
        const int NB = 32 / LPS;                  // stages per batch
        const int sb = lane / LPS;                // this lane's stage inside a batch
        const int my_tok = pw + kGqaProducerWarps * (lane % LPS);
        const char* kbase = static_cast<const char*>(a.kmat) + static_cast<int64_t>(hg0) * a.k_s1 * 2;
        const char* vbase = static_cast<const char*>(a.vmat) + static_cast<int64_t>(hg0) * a.v_s1 * 2;
        const int64_t k_row = a.k_s0 * 2, v_row = a.v_s0 * 2;
        StageWalk walk;
        walk.init(pre, a.B, t0, t1);
        // Walks the next batch: returns its number of stages; this lane keeps the token count of its stage and the slot of its token.
        auto load_batch = [&](int& my_cnt, int64_t& my_slot) -> int {
            int n = 0, req = 0, j0 = 0, cnt = 0, my_req = 0, my_j = 0;
            bool last;
            my_cnt = 0;
            my_slot = 0;
            for (; n < NB; ++n) {
                if (!walk.next(TT, req, j0, cnt, last)) break;
                if (n == sb) {
                    my_req = req;
                    my_j = j0;
                    my_cnt = cnt;
                }
            }
            if (my_tok < my_cnt) {
                const int L = pre[my_req + 1] - pre[my_req];
                int64_t sl = token_slot(a, my_req, L, static_cast<int64_t>(my_j) + my_tok);
                if (sl < 0 || sl >= a.slots) {
                    report_status(a.status, 1);
                    sl = 0;  // keep the byte count of the stage intact
                }
                my_slot = sl;
            }
            return n;
        };
        int cur_cnt, nxt_cnt;
        int64_t cur_slot, nxt_slot;
        int n_cur = load_batch(cur_cnt, cur_slot);
        int ring = 0;
        uint32_t ring_phase = 0;
        bool ok = true;
        while (ok && n_cur > 0) {
            const int n_nxt = load_batch(nxt_cnt, nxt_slot);   // in flight while this batch's copies are issued
            for (int s = 0; s < n_cur; ++s) {
                const int cnt_s = __shfl_sync(0xffffffffu, cur_cnt, s * LPS);
                if (lane == 0) {
                    ok = mbar_wait(smem_u32(&bars[p.nstages + ring]), ring_phase ^ 1u, give_up);
                    if (ok && pw == 0) mbar_arrive_expect_tx(smem_u32(&bars[ring]), static_cast<uint32_t>(cnt_s) * row_bytes * 2u);
                }
                ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
                if (!ok) break;
                if (sb == s && my_tok < cur_cnt) {
                    const uint32_t full = smem_u32(&bars[ring]);
                    const uint32_t dst = smem_u32(smem + static_cast<size_t>(ring) * p.stage_bytes) + static_cast<uint32_t>(my_tok) * static_cast<uint32_t>(p.pitch);
                    bulk_g2s(dst, kbase + cur_slot * k_row, row_bytes, full);
                    bulk_g2s(dst + v_off, vbase + cur_slot * v_row, row_bytes, full);
                }
                if (++ring == p.nstages) {
                    ring = 0;
                    ring_phase ^= 1u;
                }
            }
            n_cur = n_nxt;
            cur_cnt = nxt_cnt;
            cur_slot = nxt_slot;
        }
    } else {
        // =========================== consumer warps ==============================
        const int hl = warp % p.hg;                 // K/V head inside this CTA's group
        const int mtile = (warp / p.hg) % p.MT;     // which 16 query heads of the group (groups wider than 16)
        const int g = warp / (p.hg * p.MT);         // token block inside a stage
        const bool active = hl < heads_here;
        const int hkv = hg0 + hl;
        const int rb = mtile * 16;                  // first query head of this warp's M tile
        const int r0 = rb + (lane >> 2);            // the two accumulator rows (query heads of the group) this thread holds
        const int r1 = r0 + 8;
        const int cq = (lane & 3) * 2;     // first of its two accumulator columns inside an 8-wide tile
        const float scale_log2 = kLog2e / sqrtf(static_cast<float>(HD));

        // ldmatrix row addresses inside a stage, relative to the stage start:
        //   K (not transposed): lanes 0-7 give the rows of matrix 0, 8-15 of matrix 1, ...: token (lane & 7), d offset 8 * (lane >> 3)
        //   V (transposed):     token (lane & 7) + 8 * ((lane >> 3) & 1), d offset 8 * (lane >> 4)
        const uint32_t k_lane_off = static_cast<uint32_t>(g * kBlockTokens + (lane & 7)) * p.pitch + static_cast<uint32_t>(hl * HD + 8 * (lane >> 3)) * 2u;
        const uint32_t v_lane_off =
            v_off + static_cast<uint32_t>(g * kBlockTokens + (lane & 7) + 8 * ((lane >> 3) & 1)) * p.pitch + static_cast<uint32_t>(hl * HD + 8 * (lane >> 4)) * 2u;
        const uint32_t k_tile1 = 8u * static_cast<uint32_t>(p.pitch);   // tokens 8-15 of the block

        uint32_t qf[KS][4];
        float o[DN][4];
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
        int cur_req = -1;
        uint32_t red_phase = 0;

        StageWalk walk;
        walk.init(pre, a.B, t0, t1);
        int req, j0, cnt;
        bool last;
        int ring = 0;
        uint32_t ring_phase = 0;
        while (walk.next(TT, req, j0, cnt, last)) {
            if (req != cur_req) {
                cur_req = req;
                m0 = m1 = -INFINITY;
                l0 = l1 = 0.f;
#pragma unroll
                for (int n = 0; n < DN; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
                // A fragments of Q_g: a0 = (r0, k), a1 = (r1, k), a2 = (r0, k + 8), a3 = (r1, k + 8), k = 16 ks + cq
                const char* qb = static_cast<const char*>(a.q) + (static_cast<int64_t>(req) * a.q_s0 + static_cast<int64_t>(hkv) * R * a.q_s1) * 2;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    const int col = ks * 16 + cq;
                    qf[ks][0] = qf[ks][1] = qf[ks][2] = qf[ks][3] = 0u;
                    if (active && r0 < R) {
                        const char* q0 = qb + (static_cast<int64_t>(r0) * a.q_s1 + col) * 2;
                        qf[ks][0] = *reinterpret_cast<const uint32_t*>(q0);
                        qf[ks][2] = *reinterpret_cast<const uint32_t*>(q0 + 16);
                    }
                    if (active && r1 < R) {
                        const char* q1 = qb + (static_cast<int64_t>(r1) * a.q_s1 + col) * 2;
                        qf[ks][1] = *reinterpret_cast<const uint32_t*>(q1);
                        qf[ks][3] = *reinterpret_cast<const uint32_t*>(q1 + 16);
                    }
                }
            }
            const uint32_t stage = smem_u32(smem + static_cast<size_t>(ring) * p.stage_bytes);
            const uint32_t empty_bar = smem_u32(&bars[p.nstages + ring]);
            const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars[ring]), ring_phase, give_up) ? 1 : 0) != 0;
            if (++ring == p.nstages) {
                ring = 0;
                ring_phase ^= 1u;
            }
            if (!ok) break;
            const int valid = cnt - g * kBlockTokens;   // tokens of this warp's block that exist
            if (active && valid > 0) {
                // ---- S = Q K^T over the block's 16 tokens: two 8-token tiles ----
                float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int ks = 0; ks < KS; ks += 2) {
                    uint32_t b[4], c[4];
                    ldsm_x4(stage + k_lane_off + ks * 32, b);             // tokens 0-7:  (d 16ks..+7), (+8..15), (16(ks+1)..), (+8..)
                    ldsm_x4(stage + k_lane_off + k_tile1 + ks * 32, c);   // tokens 8-15
                    mma16816<T>(s0, qf[ks], b[0], b[1]);
                    mma16816<T>(s1, qf[ks], c[0], c[1]);
                    mma16816<T>(s0, qf[ks + 1], b[2], b[3]);
                    mma16816<T>(s1, qf[ks + 1], c[2], c[3]);
                }
                // ---- online softmax in base 2 on the accumulator fragment ----
                // s0[0], s0[1]: row r0, tokens cq, cq + 1;  s0[2], s0[3]: row r1;  s1[*]: the same for tokens + 8
                const bool full = valid >= kBlockTokens;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int tok = cq + (i & 1);
                    s0[i] = (full || tok < valid) ? s0[i] * scale_log2 : -INFINITY;
                    s1[i] = (full || tok + 8 < valid) ? s1[i] * scale_log2 : -INFINITY;
                }
                float mx0 = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
                float mx1 = fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);   // finite: every block holds at least one token
                const float al0 = ex2_fast(m0 - mn0), al1 = ex2_fast(m1 - mn1);
                m0 = mn0;
                m1 = mn1;
                float pr0[4], pr1[4];
                pr0[0] = ex2_fast(s0[0] - mn0);
                pr0[1] = ex2_fast(s0[1] - mn0);
                pr0[2] = ex2_fast(s0[2] - mn1);
                pr0[3] = ex2_fast(s0[3] - mn1);
                pr1[0] = ex2_fast(s1[0] - mn0);
                pr1[1] = ex2_fast(s1[1] - mn0);
                pr1[2] = ex2_fast(s1[2] - mn1);
                pr1[3] = ex2_fast(s1[3] - mn1);
                l0 = l0 * al0 + (pr0[0] + pr0[1]) + (pr1[0] + pr1[1]);   // this thread's share of the row sums; the quad is added at the end
                l1 = l1 * al1 + (pr0[2] + pr0[3]) + (pr1[2] + pr1[3]);
#pragma unroll
                for (int n = 0; n < DN; ++n) {
                    o[n][0] *= al0;
                    o[n][1] *= al0;
                    o[n][2] *= al1;
                    o[n][3] *= al1;
                }
                // the accumulator fragment of S is the A fragment of P V: a0 = (r0, tok cq..), a1 = (r1, ..), a2 = (r0, tok + 8), a3 = (r1, tok + 8)
                uint32_t pa[4];
                pa[0] = pack2<T>(pr0[0], pr0[1]);
                pa[1] = pack2<T>(pr0[2], pr0[3]);
                pa[2] = pack2<T>(pr1[0], pr1[1]);
                pa[3] = pack2<T>(pr1[2], pr1[3]);
                // ---- O += P V: B fragments by transposed loads, b0 = tokens (cq, cq + 1), b1 = tokens + 8, column d = lane / 4 ----
                // Rows of tokens that do not exist hold whatever the ring held before (their weight is 0, but 0 * inf
                // or 0 * nan would poison the sum): their halves of the fragments are cleared.
                uint32_t keep0 = 0xffffffffu, keep1 = 0xffffffffu;
                if (!full) {
                    keep0 = (cq < valid ? 0x0000ffffu : 0u) | (cq + 1 < valid ? 0xffff0000u : 0u);
                    keep1 = (cq + 8 < valid ? 0x0000ffffu : 0u) | (cq + 9 < valid ? 0xffff0000u : 0u);
                }
#pragma unroll
                for (int n = 0; n < DN; n += 2) {
                    uint32_t b[4];
                    ldsm_x4_trans(stage + v_lane_off + n * 16, b);   // (tok 0-7, d 8n..), (tok 8-15, d 8n..), (tok 0-7, d 8(n+1)..), (tok 8-15, ..)
                    mma16816<T>(o[n], pa, b[0] & keep0, b[1] & keep1);
                    mma16816<T>(o[n + 1], pa, b[2] & keep0, b[3] & keep1);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar);

            if (last) {
                // The request's part in this CTA is done: add the row sums over the quad, merge the G token blocks,
                // store one partial per query head.
                l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
                l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
                l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
                l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
                const int64_t slot_id = static_cast<int64_t>(cta) + req;
                if (p.G == 1) {
                    if (active) {
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            const int r = half ? r1 : r0;
                            if (r < R) {
                                const int64_t hq = static_cast<int64_t>(hkv) * R + r;
                                float* dst = ws_acc + (slot_id * a.H + hq) * HD + cq;
#pragma unroll
                                for (int n = 0; n < DN; ++n) *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2 * half], o[n][2 * half + 1]);
                                if ((lane & 3) == 0) *reinterpret_cast<float2*>(ws_ml + (slot_id * a.H + hq) * 2) = make_float2(half ? m1 : m0, half ? l1 : l0);
                            }
                        }
                    }
                } else {
                    // every warp leaves (m, l, O) of its rows in shared memory: red[warp][r][HD + 2]
                    float* mine = red + static_cast<size_t>(warp) * p.red_floats_per_warp;
                    if (active) {
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            const int r = half ? r1 : r0;
                            if (r < R) {
                                float* dst = mine + (r - rb) * (HD + 2);
                                if ((lane & 3) == 0) {
                                    dst[0] = half ? m1 : m0;
                                    dst[1] = half ? l1 : l0;
                                }
#pragma unroll
                                for (int n = 0; n < DN; ++n) *reinterpret_cast<float2*>(dst + 2 + n * 8 + cq) = make_float2(o[n][2 * half], o[n][2 * half + 1]);
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars[2 * p.nstages]));
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars[2 * p.nstages]), red_phase, give_up) ? 1 : 0)) break;
                    // warp (g, M tile, hl) merges rows g, g + G, ... of its M tile over the G token blocks; a lane owns 4 columns (HD = 128) or 2 (HD = 64)
                    if (active) {
                        constexpr int CPL = HD / 32;   // columns per lane
                        const int rows_here = min(16, R - rb);
                        for (int rl = g; rl < rows_here; rl += p.G) {
                            const int r = rb + rl;
                            float M = -INFINITY;
                            for (int gg = 0; gg < p.G; ++gg)
                                M = fmaxf(M, red[static_cast<size_t>((gg * p.MT + mtile) * p.hg + hl) * p.red_floats_per_warp + rl * (HD + 2)]);
                            const float Mr = (M == -INFINITY) ? 0.f : M;
                            float L = 0.f, acc[CPL];
#pragma unroll
                            for (int e = 0; e < CPL; ++e) acc[e] = 0.f;
                            for (int gg = 0; gg < p.G; ++gg) {
                                const float* src = red + static_cast<size_t>((gg * p.MT + mtile) * p.hg + hl) * p.red_floats_per_warp + rl * (HD + 2);
                                const float w = exp2f(src[0] - Mr);   // a block that saw no token left m = -inf, l = 0, O = 0
                                L = fmaf(src[1], w, L);
#pragma unroll
                                for (int e = 0; e < CPL; ++e) acc[e] = fmaf(src[2 + lane * CPL + e], w, acc[e]);
                            }
                            const int64_t hq = static_cast<int64_t>(hkv) * R + r;
                            float* dst = ws_acc + (slot_id * a.H + hq) * HD + lane * CPL;
#pragma unroll
                            for (int e = 0; e < CPL; ++e) dst[e] = acc[e];
                            if (lane == 0) *reinterpret_cast<float2*>(ws_ml + (slot_id * a.H + hq) * 2) = make_float2(M, L);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars[2 * p.nstages + 1]));
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars[2 * p.nstages + 1]), red_phase, give_up) ? 1 : 0)) break;
                    red_phase ^= 1u;
                }
            }
        }
    }

    // A thread that gave up a wait reports it; copies that might still be in flight get time to land
    // before the shared memory of the CTA is released.
    if (*give_up) {
        if (lane == 0) report_status(a.status, 3);
        const unsigned long long t_begin = global_ns();
        while (global_ns() - t_begin < 2000000ull) __nanosleep(1000);
    }
}

bool make_gqa_plan(const DecodeArgs& a, int sm_count, int max_smem, GqaPlan& p) {
    if (a.force_plain || a.mode != DecodeMode::FUSED) return false;
    if (a.dt != Dt::F16 && a.dt != Dt::BF16) return false;
    if (a.kv_group < 2 || a.kv_group > 128 || a.H % a.kv_group != 0) return false;
    if (a.D != 64 && a.D != 128) return false;
    if (a.B > kGqaMaxB || a.B <= 0) return false;
    if (static_cast<int64_t>(a.B) * a.max_input_len >= (1ll << 31)) return false;
    const int Hkv = a.H / a.kv_group;
    auto rows_ok = [&](const void* ptr, int64_t s0, int64_t s1, int64_t s2) {
        return s2 == 1 && (Hkv == 1 || s1 == a.D) && (s0 * 2) % 16 == 0 && reinterpret_cast<uintptr_t>(ptr) % 16 == 0;
    };
    if (!rows_ok(a.kmat, a.k_s0, a.k_s1, a.k_s2) || !rows_ok(a.vmat, a.v_s0, a.v_s1, a.v_s2)) return false;
    // q is read with 32-bit loads
    if (a.q_s2 != 1 || a.q_s0 % 2 != 0 || a.q_s1 % 2 != 0 || reinterpret_cast<uintptr_t>(a.q) % 4 != 0) return false;

    int mt = 1;
    while (mt * 16 < a.kv_group) mt *= 2;   // 1, 2, 4 or 8 tiles of 16 query heads
    p.MT = mt;
    int hg = 1;
    while (hg * 2 <= std::min(Hkv, kGqaConsumerWarps / mt)) hg *= 2;
    p.hg = hg;
    p.n_hg = (Hkv + hg - 1) / hg;
    p.G = kGqaConsumerWarps / (hg * mt);
    p.TT = kBlockTokens * p.G;
    p.pitch = hg * a.D * 2 + 16;
    p.stage_bytes = 2 * p.TT * p.pitch;
    p.red_floats_per_warp = std::min(a.kv_group, 16) * (a.D + 2);
    const int red_bytes = p.G > 1 ? kGqaConsumerWarps * p.red_floats_per_warp * 4 : 0;
    int off = 0;
    auto take = [&](int bytes, int align) {
        off = (off + align - 1) / align * align;
        const int at = off;
        off += bytes;
        return at;
    };
    take((2 * kGqaMaxStages + 2) * 8, 8);
    take((a.B + 1) * 4, 4);
    take(red_bytes, 16);
    take(4, 4);
    const int fixed = off + 128;
    int nst = std::min((max_smem - fixed) / p.stage_bytes, kGqaMaxStages);
    if (nst < 2) return false;
    p.nstages = nst;
    off = nst * p.stage_bytes;
    p.off_bars = take((2 * kGqaMaxStages + 2) * 8, 8);
    p.off_pre = take((a.B + 1) * 4, 4);
    p.off_red = take(red_bytes, 16);
    p.off_flag = take(4, 4);
    p.smem_bytes = off;

    int n_cta = std::max(1, sm_count / p.n_hg);
    const int64_t max_tokens = static_cast<int64_t>(a.B) * a.max_input_len;
    const int64_t useful = std::max<int64_t>(1, (max_tokens + 2 * p.TT - 1) / (2 * p.TT));
    p.n_cta = static_cast<int>(std::min<int64_t>(n_cta, useful));
    return true;
}

int64_t gqa_ws_floats_acc(const DecodeArgs& a, const GqaPlan& p) { return static_cast<int64_t>(p.n_cta + a.B) * a.H * a.D; }
int64_t gqa_ws_floats_ml(const DecodeArgs& a, const GqaPlan& p) { return static_cast<int64_t>(p.n_cta + a.B) * a.H * 2; }

template <typename T>
void launch_gqa_t(const DecodeArgs& a, const GqaPlan& p, float* ws_acc, float* ws_ml, cudaStream_t st) {
    dim3 grid(p.n_cta, p.n_hg);
    if (a.D == 128) {
        auto kern = decode_gqa_kernel<T, 128>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, p.smem_bytes);
        kern<<<grid, kGqaThreads, p.smem_bytes, st>>>(a, p, ws_acc, ws_ml);
    } else {
        auto kern = decode_gqa_kernel<T, 64>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, p.smem_bytes);
        kern<<<grid, kGqaThreads, p.smem_bytes, st>>>(a, p, ws_acc, ws_ml);
    }
    // the merge kernel as a programmatic dependent: its launch latency and set-up overlap this kernel's tail
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.B, (a.H + 3) / 4, 1);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const float* acc_c = ws_acc;
    const float* ml_c = ws_ml;
    const int64_t zero = 0;
    cudaLaunchKernelEx(&cfg, decode_combine_kernel<T>, a, p.n_cta, acc_c, ml_c, zero, zero, zero);
}

}  // namespace

int64_t decode_gqa_workspace_bytes(const DecodeArgs& a, int sm_count, int max_smem) {
    GqaPlan p;
    if (!make_gqa_plan(a, sm_count, max_smem, p)) return 0;
    return (gqa_ws_floats_acc(a, p) + gqa_ws_floats_ml(a, p)) * 4 + 256;
}

bool launch_decode_gqa(const DecodeArgs& a, void* ws, int sm_count, int max_smem, cudaStream_t st) {
    GqaPlan p;
    if (!make_gqa_plan(a, sm_count, max_smem, p)) return false;
    const uintptr_t base = (reinterpret_cast<uintptr_t>(ws) + 255) & ~static_cast<uintptr_t>(255);
    float* ws_acc = reinterpret_cast<float*>(base);
    float* ws_ml = ws_acc + gqa_ws_floats_acc(a, p);
    if (a.dt == Dt::F16)
        launch_gqa_t<__half>(a, p, ws_acc, ws_ml, st);
    else
        launch_gqa_t<__nv_bfloat16>(a, p, ws_acc, ws_ml, st);
    return true;
}

}  // namespace k
}  // namespace b200
