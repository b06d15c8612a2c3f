// Paged-KV decode attention: one query token per request against the K/V rows that
// b_loc names in the pool.
//
//   QK    mode = diopiTokenAttentionInference       (functions_lightllm.cpp:53-80)
//   PV    mode = diopiTokenSoftmaxReduceVInference  (functions_lightllm.cpp:82-107)
//   FUSED mode = both in one pass; the logits stay in registers.
//
// The reference walks the requests on the host, copies each request's rows out of
// the pool and calls a batched GEMV. Here everything is read on the device and each
// K/V byte is read once.
//
// Split path (the fast one). The (request, token) pairs are flattened in request
// order and cut into equal ranges, one per CTA, so every CTA streams the same number of
// bytes whatever the mix of request lengths. Inside a CTA one producer warp looks up the
// pool slots and issues one bulk asynchronous copy (cp.async.bulk, completion on an
// mbarrier) per row: the row of a token is contiguous over heads, H*D*e bytes (8 KB at
// 32 x 128 x fp16). Rows land in a ring of shared-memory stages; 16 consumer warps
// take 16 bytes of every row each, so one head is spread over D*e/16 neighbouring lanes,
// the dot product finishes with warp shuffles, and max/sum/accumulator of the online
// softmax stay in fp32 registers. A CTA writes one partial (m, l, acc[D]) per request
// it touched into scratch; a second small kernel merges the partials of a request.
// Scratch slot of (CTA c, request i) is c + i: both only grow along the flattened
// order, so the sum is unique and at most n_cta + B slots are needed.
//
// Algorithmic bytes, fused: 2*sumL*H*D*e (K and V) + 2*B*H*D*e (q, out) + index loads.
// The scratch traffic, (n_cta + B)*H*(D+2)*4 bytes written and read once, is overhead.
//
// Plain path: one CTA per (request, head), any strides, any D up to 512. Used when the
// rows are not 16-byte aligned/dense or D*e/16 is not 8, 16 or 32.
#include <cfloat>
#include <type_traits>
#include <mutex>

#include "decode_common.cuh"
#include "token_decode_gqa.hpp"

namespace b200 {
namespace k {

namespace {

constexpr int kConsumerWarps = 16;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kMaxProducerWarps = 4;             // short rows need more copy instructions per byte than one warp can issue
constexpr int kThreads = kConsumerThreads + 32 * kMaxProducerWarps;   // launch bound; the launch uses 512 + 32 * plan.producer_warps
constexpr int kMaxB = 2048;                      // request prefix sums live in shared memory
constexpr int kMaxG = 32;                        // token groups per CTA
constexpr int kMaxStages = 32;

struct SplitPlan {
    int lph;          // lanes (16-byte chunks) per head
    int hg;           // heads per CTA
    int n_hg;         // CTAs along the head axis
    int C;            // chunks per row for a full head group = hg * lph
    int G;            // token groups: consumer thread = g * C + chunk
    int TT;           // tokens per stage = G * tpg
    int tpg;          // tokens per group per stage
    int nmat;         // matrices streamed: 2 when fused
    int stage_bytes;  // one ring slot: ups * G tokens, K rows then V rows = ups * G * C * 16 * nmat bytes
    int nstages;      // ring slots
    int n_cta;        // CTAs along the flattened token axis
    int smem_bytes;
    int off_bars, off_pre, off_red, off_flag;
    int ups;           // token groups per ring slot (1, 2 or 4): a tile of TPG groups spans TPG / ups ring slots
    int pdl;           // launch the merge kernel as a programmatic dependent
    int producer_warps;
    // Grouped K/V heads: `passes` query heads per K/V head. CTA x of the grid works on token range x / passes for
    // pass x % passes, so the CTAs that stream the same rows run side by side and all but the first find them in L2.
    int passes;
    int64_t q_pass, out_pass;          // element offset of a pass inside q and out
    int64_t ws_pass_acc, ws_pass_ml;   // float offset of a pass inside the two scratch blocks
};

// Sums v[u] over the LPH lanes of a head (lanes lih = 0..LPH-1, LPH-aligned in the warp). On return lane lih holds
// the total of token group lih % TPG. Recursive halving: each step hands half of the values to the partner lane, so
// TPG - 1 + log2(LPH / TPG) shuffles do what TPG butterflies of log2(LPH) steps would.
template <int TPG, int LPH>
__device__ __forceinline__ float head_reduce_scatter(float (&v)[TPG], int lih) {
    static_assert(LPH >= TPG, "a head has at least as many lanes as a tile has token groups");
#pragma unroll
    for (int o = TPG >> 1; o > 0; o >>= 1) {  // bit o of the lane picks the half it keeps
        const bool upper = (lih & o) != 0;
#pragma unroll
        for (int i = 0; i < o; ++i) {
            const float send = upper ? v[i] : v[i + o];
            const float keep = upper ? v[i + o] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
    }
    float r = v[0];
#pragma unroll
    for (int o = TPG; o < LPH; o <<= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

template <typename T, int LPH, int MODE, int TPG>
__global__ void __launch_bounds__(kThreads, 1) decode_split_kernel(const DecodeArgs a, const SplitPlan p, float* __restrict__ ws_acc,
                                                                    float* __restrict__ ws_ml) {
    constexpr int EPC = Vec16<T>::N;  // elements per 16-byte chunk
    constexpr bool kHasK = (MODE != static_cast<int>(DecodeMode::PV));
    constexpr bool kHasV = (MODE != static_cast<int>(DecodeMode::QK));
    constexpr bool kFused = (MODE == static_cast<int>(DecodeMode::FUSED));

    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.off_bars);  // full[nstages], empty[nstages], red[2]
    int* pre = reinterpret_cast<int*>(smem + p.off_pre);
    float* red = reinterpret_cast<float*>(smem + p.off_red);
    volatile int* give_up = reinterpret_cast<volatile int*>(smem + p.off_flag);

    // Let the merge kernel (launched with programmatic stream serialization) become resident early; it
    // does its own set-up and then blocks in griddepcontrol.wait until this whole grid has finished.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int pass = p.passes > 1 ? static_cast<int>(blockIdx.x) % p.passes : 0;
    const int cta = p.passes > 1 ? static_cast<int>(blockIdx.x) / p.passes : static_cast<int>(blockIdx.x);
    ws_acc += pass * p.ws_pass_acc;
    ws_ml += pass * p.ws_pass_ml;
    const int hg0 = blockIdx.y * p.hg;               // first head of this CTA
    const int heads_here = min(p.hg, a.H - hg0);
    const int C_eff = heads_here * LPH;               // chunks per row actually copied
    const uint32_t row_bytes = static_cast<uint32_t>(C_eff) * 16u;

    // ---- set-up: barriers and the prefix sums of the request lengths -------------
    if (tid == 0) {
        for (int s = 0; s < p.nstages; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);                            // full: the producer's arrive + bytes
            mbar_init(smem_u32(&bars[p.nstages + s]), kConsumerWarps);   // empty: one arrive per consumer warp
        }
        mbar_init(smem_u32(&bars[2 * p.nstages]), kConsumerWarps);
        mbar_init(smem_u32(&bars[2 * p.nstages + 1]), kConsumerWarps);
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

    // A tile = TT = G * TPG tokens = TPG token groups. It occupies TPG / ups consecutive ring slots of
    // ups * G tokens each (K rows, then V rows). ups = TPG (one 64 KB slot per tile) measured fastest: every
    // extra mbarrier round trip per token costs more than the finer refill granularity wins.
    if (warp >= kConsumerWarps) {
        // =========================== producer warps ==============================
        // Producer warp pw issues the copies of the tokens whose index has (t / 8) % producer_warps == pw; warp 0
        // also announces the bytes of each ring slot. A copy of the other warp may land before that announcement:
        // the slot's phase cannot complete before the announcing arrive, so the early bytes are only booked ahead.
        const int pw = warp - kConsumerWarps;
        const char* kbase = kHasK ? static_cast<const char*>(a.kmat) + static_cast<int64_t>(hg0) * a.k_s1 * sizeof(T) : nullptr;
        const char* vbase = kHasV ? static_cast<const char*>(a.vmat) + static_cast<int64_t>(hg0) * a.v_s1 * sizeof(T) : nullptr;
        const int64_t k_row = a.k_s0 * static_cast<int64_t>(sizeof(T));
        const int64_t v_row = a.v_s0 * static_cast<int64_t>(sizeof(T));
        const int tps = p.ups * p.G;      // tokens per ring slot
        const int spt = TPG / p.ups;      // ring slots per tile
        const uint32_t v_off = kFused ? static_cast<uint32_t>(tps) * static_cast<uint32_t>(p.C) * 16u : 0u;

        StageWalk walk;
        walk.init(pre, a.B, t0, t1);
        int req, j0, cnt;
        bool last;
        bool have = walk.next(TT, req, j0, cnt, last);
        int64_t slot[TPG];  // tokens lane, lane+32, ... of the tile
        auto fetch_slots = [&](int r, int j, int n, int64_t (&out)[TPG]) {
            const int L = pre[r + 1] - pre[r];
#pragma unroll
            for (int u = 0; u < TPG; ++u) {
                const int t = lane + 32 * u;
                out[u] = 0;
                if (t < n) {
                    int64_t sl = token_slot(a, r, L, static_cast<int64_t>(j) + t);
                    if (sl < 0 || sl >= a.slots) {
                        report_status(a.status, 1);
                        sl = 0;  // keep the byte count of the slot intact
                    }
                    out[u] = sl;
                }
            }
        };
        if (have) fetch_slots(req, j0, cnt, slot);
        int ring = 0;          // ring slot of the tile's first token group
        uint32_t ring_phase = 0;
        while (have) {
            const int cur_cnt = cnt;
            int64_t cur_slot[TPG];
#pragma unroll
            for (int u = 0; u < TPG; ++u) cur_slot[u] = slot[u];
            // Look up the next tile's pool slots before blocking, so that load overlaps the waits.
            have = walk.next(TT, req, j0, cnt, last);
            if (have) fetch_slots(req, j0, cnt, slot);
            // Lane u < spt owns ring slot u of this tile: waits until it is free and announces its bytes.
            bool mine_ok = true;
            if (lane < spt) {  // every producer warp waits for the slots to be free; only warp 0 announces bytes
                int s = ring + lane;
                uint32_t parity = ring_phase;
                if (s >= p.nstages) {
                    s -= p.nstages;
                    parity ^= 1u;
                }
                mine_ok = mbar_wait(smem_u32(&bars[p.nstages + s]), parity ^ 1u, give_up);
                if (mine_ok && pw == 0) {
                    const int here = min(max(cur_cnt - lane * tps, 0), tps);  // tokens of the tile that fall into this ring slot
                    mbar_arrive_expect_tx(smem_u32(&bars[s]), static_cast<uint32_t>(here) * row_bytes * static_cast<uint32_t>(p.nmat));
                }
            }
            if (!__all_sync(0xffffffffu, mine_ok ? 1 : 0)) break;
            // Then every lane issues the copies of its tokens (token t lives in ring slot t / tps at position t % tps).
#pragma unroll
            for (int u = 0; u < TPG; ++u) {
                const int t = lane + 32 * u;
                if (t < cur_cnt && ((t >> 3) % p.producer_warps) == pw) {
                    const int su = t / tps;
                    int s = ring + su;
                    if (s >= p.nstages) s -= p.nstages;
                    const uint32_t full = smem_u32(&bars[s]);
                    const uint32_t dst = smem_u32(smem + static_cast<size_t>(s) * p.stage_bytes) + static_cast<uint32_t>(t - su * tps) * row_bytes;
                    if (kHasK) bulk_g2s(dst, kbase + cur_slot[u] * k_row, row_bytes, full);
                    if (kHasV) bulk_g2s(dst + v_off, vbase + cur_slot[u] * v_row, row_bytes, full);
                }
            }
            ring += spt;
            if (ring >= p.nstages) {
                ring -= p.nstages;
                ring_phase ^= 1u;
            }
        }
    } else {
        // =========================== consumer warps ==============================
        const int GC = p.G * p.C;
        int g = tid / p.C;
        int c = tid - g * p.C;
        const bool real = (tid < GC) && (c < C_eff);
        if (!real) {  // shadow threads mirror group 0 so that shuffles stay full-warp; they never store
            g = 0;
            c = c % LPH;
        }
        const int hl = c / LPH;    // head within this CTA's group
        const int lih = c % LPH;   // lane within the head
        const int h = hg0 + hl;
        const int ups_mask = p.ups - 1;   // ups is 1, 2 or 4
        const uint32_t v_off = kFused ? static_cast<uint32_t>(p.ups * p.G) * static_cast<uint32_t>(p.C) * 16u : 0u;
        const uint32_t my_off = static_cast<uint32_t>(g) * row_bytes + static_cast<uint32_t>(c) * 16u;  // my 16 bytes of token group 0 of a ring slot
        const uint32_t group_step = static_cast<uint32_t>(p.G) * row_bytes;                              // next token group inside the slot
        const float sqrt_d = sqrtf(static_cast<float>(a.D));
        const float qscale = kLog2e / sqrt_d;  // softmax runs in base 2

        float qreg[EPC];
        float acc[EPC];
        float m = -INFINITY, l = 0.f;
        int cur_req = -1;
        int64_t att_col0 = 0;
        uint32_t red_phase = 0;

        // PV mode reads the stored logits in groups of four tiles (a request's next 4 * TT tokens), one group ahead
        // of their use: under a saturated memory system an ordinary load queues behind the bulk copies for several
        // microseconds, more than one tile lasts. Entry i = 8 * tile + token group of a group is loaded by lane
        // i % LPH of the head into register i / LPH, and handed round with a shuffle when its tile comes up.
        constexpr int kLgTiles = 4;
        constexpr int kLgRegs = kLgTiles * TPG / LPH > 0 ? kLgTiles * TPG / LPH : 1;
        StageWalk ahead;
        float lg_cur[kLgRegs], lg_nxt[kLgRegs];
        int lg_nxt_cnt = 0, lg_left = 0, lg_k = 0, lg_cur_req = -1;
        int64_t lg_col0 = 0;
        auto fetch_logits = [&]() {
            int r, j, n;
            bool l_;
            lg_nxt_cnt = 0;
#pragma unroll
            for (int i = 0; i < kLgRegs; ++i) lg_nxt[i] = -INFINITY;
            if (!ahead.next(kLgTiles * TT, r, j, n, l_)) return;
            lg_nxt_cnt = n;
            if (r != lg_cur_req) {
                lg_cur_req = r;
                lg_col0 = load_index(a.b_start, r);
            }
#pragma unroll
            for (int i = 0; i < kLgRegs; ++i) {
                const int e = lih + i * LPH;                          // entry of the group
                const int off = (e >> 3) * TT + g + (e & 7) * p.G;    // its token, counted from the group's first
                const int64_t col = lg_col0 + j + off;
                if (e < kLgTiles * TPG && off < n && col >= 0 && col < a.att_cols)
                    lg_nxt[i] = Cvt<T>::to_f(static_cast<const T*>(a.att)[static_cast<int64_t>(h) * a.att_s0 + col * a.att_s1]) * kLog2e;
            }
        };
        if (!kHasK) {
            static_assert(kHasK || TPG == 8, "the logits groups assume eight token groups per tile");
            ahead.init(pre, a.B, t0, t1);
            fetch_logits();
        }

        StageWalk walk;
        walk.init(pre, a.B, t0, t1);
        int req, j0, cnt;
        bool last;
        int ring = 0;          // next ring slot to consume (kept incrementally: no division in the loop)
        uint32_t ring_phase = 0;
        bool ok = true;
        while (ok && walk.next(TT, req, j0, cnt, last)) {
            if (req != cur_req) {
                cur_req = req;
                m = -INFINITY;
                l = 0.f;
#pragma unroll
                for (int e = 0; e < EPC; ++e) acc[e] = 0.f;
                if (kHasK) {
                    const T* qp = static_cast<const T*>(a.q) + pass * p.q_pass + static_cast<int64_t>(req) * a.q_s0 + static_cast<int64_t>(h) * a.q_s1 + lih * EPC;
                    if (MODE == static_cast<int>(DecodeMode::QK)) {
                        // The reference divides the finished dot product by sqrt(D); do the same at the store.
#pragma unroll
                        for (int e = 0; e < EPC; ++e) qreg[e] = Cvt<T>::to_f(qp[e]);
                    } else {
#pragma unroll
                        for (int e = 0; e < EPC; ++e) qreg[e] = Cvt<T>::to_f(qp[e]) * qscale;
                    }
                }
                if (MODE == static_cast<int>(DecodeMode::QK)) att_col0 = load_index(a.b_start, req);
            }

            float sc[TPG];
            if (!kHasK) {
                // Stored logits: when a group of tiles is used up, the group loaded meanwhile takes its place and the
                // load of the one after it starts.
                if (lg_left == 0) {
#pragma unroll
                    for (int i = 0; i < kLgRegs; ++i) lg_cur[i] = lg_nxt[i];
                    lg_left = (lg_nxt_cnt + TT - 1) / TT;
                    lg_k = 0;
                    fetch_logits();
                }
                const int e0 = lg_k * TPG;  // first entry of this tile; all its entries sit in register e0 / LPH
                float mine = lg_cur[0];
#pragma unroll
                for (int i = 1; i < kLgRegs; ++i)
                    if (i == e0 / LPH) mine = lg_cur[i];
#pragma unroll
                for (int u = 0; u < TPG; ++u) sc[u] = __shfl_sync(0xffffffffu, mine, (lane & ~(LPH - 1)) + ((e0 + u) & (LPH - 1)));
                ++lg_k;
                --lg_left;
            }
            // token group u sits in ring slot u / ups; a slot is waited for right before its first use
            const unsigned char* slot_ptr[TPG];
            uint32_t empty_bar[TPG];
            const bool full_tile = cnt == TT;  // every token group of the tile holds a token (all but a request's last tile)
            // K: this thread's 16 bytes of each row against its 16 bytes of q. A full tile has no per-token test,
            // so the TPG loads and dot products are independent straight-line code.
            auto dots = [&](auto full_c) {
                constexpr bool kFull = decltype(full_c)::value;
#pragma unroll
                for (int u = 0; u < TPG; ++u) {
                    if ((u & ups_mask) == 0) {
                        const int s = ring;
                        const uint32_t parity = ring_phase;
                        if (++ring == p.nstages) {
                            ring = 0;
                            ring_phase ^= 1u;
                        }
                        slot_ptr[u] = smem + static_cast<size_t>(s) * p.stage_bytes + my_off;
                        empty_bar[u] = smem_u32(&bars[p.nstages + s]);
                        if (ok && !mbar_wait(smem_u32(&bars[s]), parity, give_up)) ok = false;
                    } else {
                        slot_ptr[u] = slot_ptr[u - 1] + group_step;
                        empty_bar[u] = empty_bar[u - 1];
                    }
                    if (kHasK) {
                        float part = 0.f;
                        if (kFull || (ok && g + u * p.G < cnt)) {
                            const uint4 kv = *reinterpret_cast<const uint4*>(slot_ptr[u]);
                            float f[EPC];
                            unpack16<T>(kv, f);
#pragma unroll
                            for (int e = 0; e < EPC; ++e) part = fmaf(qreg[e], f[e], part);
                        }
                        sc[u] = part;
                    }
                }
            };
            if (full_tile) dots(std::true_type{}); else dots(std::false_type{});
            ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;  // the whole warp leaves together
            if (!ok) break;

            if (kHasK) {
                // lane lih of a head now holds the finished sum of token group lih % TPG
                const float mine = head_reduce_scatter<TPG, LPH>(sc, lih);
                if (MODE == static_cast<int>(DecodeMode::QK)) {
                    // the TPG stores of a head are one instruction, and with one token group per tile one run of columns
                    if (real && lih < TPG) {
                        const int t = g + lih * p.G;
                        const int64_t col = att_col0 + j0 + t;
                        if (t < cnt && col >= 0 && col < a.att_cols)
                            static_cast<T*>(a.att)[static_cast<int64_t>(h) * a.att_s0 + col * a.att_s1] = Cvt<T>::from_f(mine / sqrt_d);
                    }
                    __syncwarp();
                    if (lane == 0) {
#pragma unroll
                        for (int u = 0; u < TPG; ++u)
                            if ((u & ups_mask) == ups_mask) mbar_arrive(empty_bar[u]);
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < TPG; ++u) {
                        const float all = __shfl_sync(0xffffffffu, mine, (lane & ~(LPH - 1)) + u);
                        sc[u] = (full_tile || g + u * p.G < cnt) ? all : -INFINITY;
                    }
                }
            }
            if (kHasV) {
                float m_new = m;
#pragma unroll
                for (int u = 0; u < TPG; ++u) m_new = fmaxf(m_new, sc[u]);
                const float m_ref = (m_new == -INFINITY) ? 0.f : m_new;
                const float alpha = ex2_fast(m - m_ref);
                l *= alpha;
#pragma unroll
                for (int e = 0; e < EPC; ++e) acc[e] *= alpha;
                auto weighted_v = [&](auto full_c) {
                    constexpr bool kFull = decltype(full_c)::value;
#pragma unroll
                    for (int u = 0; u < TPG; ++u) {
                        if (kFull || g + u * p.G < cnt) {
                            const float pr = ex2_fast(sc[u] - m_ref);
                            l += pr;
                            const uint4 vv = *reinterpret_cast<const uint4*>(slot_ptr[u] + v_off);
                            float f[EPC];
                            unpack16<T>(vv, f);
#pragma unroll
                            for (int e = 0; e < EPC; ++e) acc[e] = fmaf(pr, f[e], acc[e]);
                        }
                        // last token group of a ring slot: the slot is done for the whole warp, hand it back
                        if ((u & ups_mask) == ups_mask) {
                            __syncwarp();
                            if (lane == 0) mbar_arrive(empty_bar[u]);
                        }
                    }
                };
                if (full_tile) weighted_v(std::true_type{}); else weighted_v(std::false_type{});
                m = m_new;
            }

            if (last && kHasV) {
                // The request's part in this CTA is done: merge the token groups, then store the partial.
                if (p.G > 1) {
                    if (tid < GC) {
                        red[tid * (EPC + 2) + 0] = m;
                        red[tid * (EPC + 2) + 1] = l;
#pragma unroll
                        for (int e = 0; e < EPC; ++e) red[tid * (EPC + 2) + 2 + e] = acc[e];
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars[2 * p.nstages]));
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars[2 * p.nstages]), red_phase, give_up) ? 1 : 0)) break;
                    if (real && g == 0) {
                        float M = m;
                        for (int gg = 1; gg < p.G; ++gg) M = fmaxf(M, red[(gg * p.C + c) * (EPC + 2)]);
                        const float Mr = (M == -INFINITY) ? 0.f : M;
                        const float w0 = exp2f(m - Mr);
                        l *= w0;
#pragma unroll
                        for (int e = 0; e < EPC; ++e) acc[e] *= w0;
                        for (int gg = 1; gg < p.G; ++gg) {
                            const float* r = &red[(gg * p.C + c) * (EPC + 2)];
                            const float w = exp2f(r[0] - Mr);
                            l = fmaf(r[1], w, l);
#pragma unroll
                            for (int e = 0; e < EPC; ++e) acc[e] = fmaf(r[2 + e], w, acc[e]);
                        }
                        m = M;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars[2 * p.nstages + 1]));
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars[2 * p.nstages + 1]), red_phase, give_up) ? 1 : 0)) break;
                    red_phase ^= 1u;
                }
                if (real && g == 0) {
                    const int64_t slot_id = static_cast<int64_t>(cta) + req;
                    float* dst = ws_acc + (slot_id * a.H + h) * a.D + lih * EPC;
#pragma unroll
                    for (int e = 0; e < EPC; e += 4) *reinterpret_cast<float4*>(dst + e) = make_float4(acc[e], acc[e + 1], acc[e + 2], acc[e + 3]);
                    if (lih == 0) *reinterpret_cast<float2*>(ws_ml + (slot_id * a.H + h) * 2) = make_float2(m, l);
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

// ---------------------------------------------------------------------------
// Plain path: one CTA of 4 warps per (request, head); warps stride over the tokens,
// lanes over D. No scratch, any strides.
// ---------------------------------------------------------------------------
template <typename T, int MODE>
__global__ void __launch_bounds__(128) decode_plain_kernel(const DecodeArgs a) {
    constexpr int R = 16;  // D <= 512
    constexpr bool kHasK = (MODE != static_cast<int>(DecodeMode::PV));
    constexpr bool kHasV = (MODE != static_cast<int>(DecodeMode::QK));
    __shared__ float s_m[4], s_l[4];
    __shared__ float s_acc[4][512];
    const int i = blockIdx.x, h = blockIdx.y;
    const int hkv = a.kv_group > 1 ? h / a.kv_group : h;   // grouped-query attention: the K/V head this query head reads
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int L = request_len(a, i);
    const int64_t col0 = (MODE == static_cast<int>(DecodeMode::FUSED)) ? 0 : load_index(a.b_start, i);
    const float inv_sqrt_d = 1.0f / sqrtf(static_cast<float>(a.D));

    float qf[R], acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        acc[r] = 0.f;
        qf[r] = 0.f;
        const int d = lane + 32 * r;
        if (kHasK && d < a.D) qf[r] = Cvt<T>::to_f(static_cast<const T*>(a.q)[static_cast<int64_t>(i) * a.q_s0 + static_cast<int64_t>(h) * a.q_s1 + d * a.q_s2]);
    }
    float m = -INFINITY, l = 0.f;
    for (int j = warp; j < L; j += 4) {
        int64_t slot = token_slot(a, i, L, j);
        if (slot < 0 || slot >= a.slots) {
            if (lane == 0) report_status(a.status, 1);
            continue;
        }
        const int64_t col = col0 + j;
        float sc;
        if (kHasK) {
            const T* kp = static_cast<const T*>(a.kmat) + slot * a.k_s0 + static_cast<int64_t>(hkv) * a.k_s1;
            float part = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int d = lane + 32 * r;
                if (d < a.D) part = fmaf(qf[r], Cvt<T>::to_f(kp[d * a.k_s2]), part);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            sc = part * inv_sqrt_d;
            if (MODE == static_cast<int>(DecodeMode::QK)) {
                if (lane == 0 && col >= 0 && col < a.att_cols) static_cast<T*>(a.att)[static_cast<int64_t>(h) * a.att_s0 + col * a.att_s1] = Cvt<T>::from_f(sc);
                continue;
            }
        } else {
            if (col < 0 || col >= a.att_cols) continue;
            sc = Cvt<T>::to_f(static_cast<const T*>(a.att)[static_cast<int64_t>(h) * a.att_s0 + col * a.att_s1]);
        }
        if (kHasV) {
            sc *= kLog2e;
            const float m_new = fmaxf(m, sc);
            const float alpha = exp2f(m - m_new), pr = exp2f(sc - m_new);
            l = l * alpha + pr;
            const T* vp = static_cast<const T*>(a.vmat) + slot * a.v_s0 + static_cast<int64_t>(hkv) * a.v_s1;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int d = lane + 32 * r;
                if (d < a.D) acc[r] = fmaf(pr, Cvt<T>::to_f(vp[d * a.v_s2]), acc[r] * alpha);
            }
            m = m_new;
        }
    }
    if (!kHasV) return;
    if (lane == 0) {
        s_m[warp] = m;
        s_l[warp] = l;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int d = lane + 32 * r;
        if (d < a.D) s_acc[warp][d] = acc[r];
    }
    __syncthreads();
    if (warp == 0) {
        const float M = fmaxf(fmaxf(s_m[0], s_m[1]), fmaxf(s_m[2], s_m[3]));
        const float Mr = (M == -INFINITY) ? 0.f : M;
        float w[4], Ls = 0.f;
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            w[x] = exp2f(s_m[x] - Mr);
            Ls += s_l[x] * w[x];
        }
        const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
        T* o = static_cast<T*>(a.out) + static_cast<int64_t>(i) * a.out_s0 + static_cast<int64_t>(h) * a.out_s1;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int d = lane + 32 * r;
            if (d < a.D) {
                const float v = s_acc[0][d] * w[0] + s_acc[1][d] * w[1] + s_acc[2][d] * w[2] + s_acc[3][d] * w[3];
                o[d * a.out_s2] = Cvt<T>::from_f(v * inv);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Host side: path choice and launch.
// ---------------------------------------------------------------------------
int elem_bytes(Dt dt) { return dt == Dt::F32 ? 4 : 2; }

// Fills `p` when the arguments qualify for the split path.
bool make_split_plan(const DecodeArgs& a, int sm_count, int max_smem, SplitPlan& p) {
    if (a.dt == Dt::F64) return false;
    if (a.kv_group > 1) return false;  // a K/V row shared by several query heads: plain path
    if (a.force_plain) return false;
    const int e = elem_bytes(a.dt);
    const bool has_k = a.mode != DecodeMode::PV, has_v = a.mode != DecodeMode::QK;
    if ((a.D * e) % 16 != 0) return false;
    const int lph = a.D * e / 16;
    if (lph != 8 && lph != 16 && lph != 32) return false;
    if (a.B > kMaxB || a.B <= 0) return false;
    if (static_cast<int64_t>(a.B) * a.max_input_len >= (1ll << 31)) return false;
    auto rows_ok = [&](const void* ptr, int64_t s0, int64_t s1, int64_t s2) {
        return (a.D == 1 || s2 == 1) && (a.H == 1 || s1 == a.D) && (s0 * e) % 16 == 0 && reinterpret_cast<uintptr_t>(ptr) % 16 == 0;
    };
    if (has_k && !rows_ok(a.kmat, a.k_s0, a.k_s1, a.k_s2)) return false;
    if (has_v && !rows_ok(a.vmat, a.v_s0, a.v_s1, a.v_s2)) return false;
    if (has_k && a.q_s2 != 1 && a.D != 1) return false;

    p.lph = lph;
    p.hg = std::min(a.H, kConsumerThreads / lph);
    p.n_hg = (a.H + p.hg - 1) / p.hg;
    p.C = p.hg * lph;
    p.G = std::min(kConsumerThreads / p.C, kMaxG);
    p.tpg = a.mode == DecodeMode::FUSED ? 4 : 8;   // a tile is 64 KB either way (two matrices or one)
    p.TT = p.G * p.tpg;
    p.nmat = (has_k && has_v) ? 2 : 1;
    // Settled by sweeps: dependent launch of the merge kernel, four producer warps, one ring slot per tile, one CTA per SM,
    // as many ring slots as fit.
    p.pdl = 1;
    p.producer_warps = kMaxProducerWarps;
    p.ups = p.tpg;
    p.stage_bytes = p.ups * p.G * p.C * 16 * p.nmat;
    const int ctas_per_sm = 1;

    const int red_bytes = (p.G > 1 && has_v) ? kConsumerThreads * (16 / e + 2) * 4 : 0;
    int off = 0;
    auto take = [&](int bytes, int align) {
        off = (off + align - 1) / align * align;
        const int at = off;
        off += bytes;
        return at;
    };
    const int budget = max_smem / ctas_per_sm - (ctas_per_sm > 1 ? 1024 : 0);
    // everything but the stages
    int fixed = 0;
    {
        off = 0;
        take((2 * kMaxStages + 2) * 8, 8);
        take((a.B + 1) * 4, 4);
        take(red_bytes, 16);
        take(4, 4);
        fixed = off + 128;
    }
    int nst = (budget - fixed) / p.stage_bytes;
    nst = std::min(nst, kMaxStages);
    if (nst < p.tpg / p.ups + 1) return false;  // a tile holds tpg/ups ring slots at once; one more must be in flight
    p.nstages = nst;
    off = nst * p.stage_bytes;
    p.off_bars = take((2 * kMaxStages + 2) * 8, 8);
    p.off_pre = take((a.B + 1) * 4, 4);
    p.off_red = take(red_bytes, 16);
    p.off_flag = take(4, 4);
    p.smem_bytes = off;
    p.passes = 1;
    p.q_pass = p.out_pass = p.ws_pass_acc = p.ws_pass_ml = 0;

    // One CTA per SM (times ctas_per_sm) over the head groups, but no more CTAs than there can be work for.
    int n_cta = std::max(1, sm_count * ctas_per_sm / p.n_hg);
    const int64_t max_tokens = static_cast<int64_t>(a.B) * a.max_input_len;
    const int64_t useful = std::max<int64_t>(1, (max_tokens + 2 * p.TT - 1) / (2 * p.TT));
    n_cta = static_cast<int>(std::min<int64_t>(n_cta, useful));
    p.n_cta = n_cta;
    return true;
}

template <typename T, int LPH, int MODE>
void launch_split_t(const DecodeArgs& a, const SplitPlan& p, float* ws_acc, float* ws_ml, cudaStream_t st) {
    dim3 grid(p.n_cta * p.passes, p.n_hg);
    constexpr bool fused = MODE == static_cast<int>(DecodeMode::FUSED);
    // fused: 4 token groups per tile; one matrix only: 8, so that a tile is 64 KB either way
    {
        auto kern = decode_split_kernel<T, LPH, MODE, (fused ? 4 : 8)>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, p.smem_bytes);
        kern<<<grid, kConsumerThreads + 32 * p.producer_warps, p.smem_bytes, st>>>(a, p, ws_acc, ws_ml);
    }
    if (MODE != static_cast<int>(DecodeMode::QK)) {
        // Programmatic dependent launch: the merge kernel's launch latency and set-up overlap the split kernel.
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(a.B, (a.H + 3) / 4, p.passes);
        cfg.blockDim = dim3(128);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = p.pdl ? 1 : 0;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const float* acc_c = ws_acc;
        const float* ml_c = ws_ml;
        cudaLaunchKernelEx(&cfg, decode_combine_kernel<T>, a, p.n_cta, acc_c, ml_c, p.out_pass, p.ws_pass_acc, p.ws_pass_ml);
    }
}

template <typename T, int MODE>
void launch_split_lph(const DecodeArgs& a, const SplitPlan& p, float* ws_acc, float* ws_ml, cudaStream_t st) {
    switch (p.lph) {
        case 8: launch_split_t<T, 8, MODE>(a, p, ws_acc, ws_ml, st); break;
        case 16: launch_split_t<T, 16, MODE>(a, p, ws_acc, ws_ml, st); break;
        default: launch_split_t<T, 32, MODE>(a, p, ws_acc, ws_ml, st); break;
    }
}

template <typename T>
void launch_split_mode(const DecodeArgs& a, const SplitPlan& p, float* ws_acc, float* ws_ml, cudaStream_t st) {
    switch (a.mode) {
        case DecodeMode::QK: launch_split_lph<T, 0>(a, p, ws_acc, ws_ml, st); break;
        case DecodeMode::PV: launch_split_lph<T, 1>(a, p, ws_acc, ws_ml, st); break;
        default: launch_split_lph<T, 2>(a, p, ws_acc, ws_ml, st); break;
    }
}

template <typename T>
void launch_plain_mode(const DecodeArgs& a, cudaStream_t st) {
    dim3 grid(a.B, a.H);
    switch (a.mode) {
        case DecodeMode::QK: decode_plain_kernel<T, 0><<<grid, 128, 0, st>>>(a); break;
        case DecodeMode::PV: decode_plain_kernel<T, 1><<<grid, 128, 0, st>>>(a); break;
        default: decode_plain_kernel<T, 2><<<grid, 128, 0, st>>>(a); break;
    }
}

int64_t split_ws_floats_acc(const DecodeArgs& a, const SplitPlan& p) { return static_cast<int64_t>(p.n_cta + a.B) * a.H * a.D; }
int64_t split_ws_floats_ml(const DecodeArgs& a, const SplitPlan& p) { return static_cast<int64_t>(p.n_cta + a.B) * a.H * 2; }

// ---------------------------------------------------------------------------
// Built-in scratch for callers that cannot provide any.
//
// The fused decode kernel needs a few MB for its split-KV partials. The regular entry point asks the
// caller's context for them. A serving engine that gives all free HBM to its KV pool at start-up and
// then runs its decode loop without an allocator has nothing to answer that request with, so a second
// entry point runs the same kernels on this fixed array instead. The array is part of the library's
// device image: every GPU that loads the library holds kStaticScratchBytes of it until the process ends.
// All calls on a device share it; nothing in it has to start at zero (each partial the merge kernel
// reads was written earlier in the same call), but two calls that run on the GPU at the same time
// (different streams) would overwrite each other's partials.
// ---------------------------------------------------------------------------
constexpr int64_t kStaticScratchBytes = 8ll << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the run time, not an address a kernel may use:
// the device address is looked up once per device (with that device current) and cached.
cudaError_t static_scratch_address(void** out) {
    static std::mutex mu;
    static void* cached[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        cached[dev] = p;
    }
    *out = cached[dev];
    return cudaSuccess;
}

}  // namespace

// Grouped K/V heads (kv_group query heads read one K/V head) whose shape the single-pass kernel of token_decode_gqa.cu
// does not take (fp32, head dims other than 64 and 128, groups wider than 128): the call is run as kv_group passes,
// pass s taking query head s of every group. Each pass is an ordinary problem with as many query heads as K/V heads
// (q and out are addressed with the group's stride), so the streaming kernel serves it unchanged. The K/V rows are
// read once per pass; the plain kernel, which reads them once per query head with one CTA per (request, head),
// measured 62 GB/s on a 64-over-8-head batch where this form reaches the streaming rate on every pass.
DecodeArgs group_pass(const DecodeArgs& a, int s) {
    DecodeArgs b = a;
    const int64_t e = elem_bytes(a.dt);
    b.H = a.H / a.kv_group;
    b.kv_group = 1;
    b.q = static_cast<const char*>(a.q) + static_cast<int64_t>(s) * a.q_s1 * e;
    b.out = static_cast<char*>(a.out) + static_cast<int64_t>(s) * a.out_s1 * e;
    b.q_s1 = a.q_s1 * a.kv_group;
    b.out_s1 = a.out_s1 * a.kv_group;
    return b;
}
bool grouped_on_split_path(const DecodeArgs& a, int sm_count, int max_smem) {
    if (a.kv_group <= 1 || a.mode != DecodeMode::FUSED || a.H % a.kv_group != 0) return false;
    SplitPlan p;
    return make_split_plan(group_pass(a, 0), sm_count, max_smem, p);
}

// The passes of a grouped call in ONE launch: sm_count / kv_group token ranges, kv_group CTAs (one per pass) on each,
// neighbours in the grid, so that the K/V rows one of them brings in are L2 hits for the others.
bool side_by_side_plan(const DecodeArgs& a, int sm_count, int max_smem, SplitPlan& p) {
    if (sm_count / a.kv_group < 1) return false;
    const DecodeArgs b = group_pass(a, 0);
    if (!make_split_plan(b, sm_count / a.kv_group, max_smem, p)) return false;
    p.passes = a.kv_group;
    p.q_pass = a.q_s1;
    p.out_pass = a.out_s1;
    p.ws_pass_acc = split_ws_floats_acc(b, p);
    p.ws_pass_ml = split_ws_floats_ml(b, p);
    return true;
}

int64_t decode_workspace_bytes(const DecodeArgs& a, int sm_count, int max_smem) {
    if (a.kv_group > 1) {
        const int64_t gqa = decode_gqa_workspace_bytes(a, sm_count, max_smem);   // the single-pass kernel when the shape qualifies
        if (gqa > 0) return gqa;
    }
    if (grouped_on_split_path(a, sm_count, max_smem)) {
        int64_t need = decode_workspace_bytes(group_pass(a, 0), sm_count, max_smem);
        SplitPlan p;
        if (side_by_side_plan(a, sm_count, max_smem, p)) need = std::max<int64_t>(need, (p.ws_pass_acc + p.ws_pass_ml) * p.passes * 4 + 256);
        return need;
    }
    SplitPlan p;
    if (a.mode == DecodeMode::QK) return 0;
    if (!make_split_plan(a, sm_count, max_smem, p)) return 0;
    return (split_ws_floats_acc(a, p) + split_ws_floats_ml(a, p)) * 4 + 256;
}

void launch_decode(const DecodeArgs& a, void* ws, int sm_count, int max_smem, cudaStream_t st) {
    if (a.B <= 0 || a.H <= 0 || a.D <= 0) return;
    if (a.kv_group > 1 && launch_decode_gqa(a, ws, sm_count, max_smem, st)) return;
    if (grouped_on_split_path(a, sm_count, max_smem)) {
        SplitPlan gp;
        if (side_by_side_plan(a, sm_count, max_smem, gp)) {
            const DecodeArgs b = group_pass(a, 0);
            uintptr_t base = (reinterpret_cast<uintptr_t>(ws) + 255) & ~static_cast<uintptr_t>(255);
            float* ws_acc = reinterpret_cast<float*>(base);
            float* ws_ml = ws_acc + gp.ws_pass_acc * gp.passes;
            switch (b.dt) {
                case Dt::F16: launch_split_mode<__half>(b, gp, ws_acc, ws_ml, st); break;
                case Dt::BF16: launch_split_mode<__nv_bfloat16>(b, gp, ws_acc, ws_ml, st); break;
                default: launch_split_mode<float>(b, gp, ws_acc, ws_ml, st); break;
            }
            return;
        }
        // else the passes one after the other; they share the scratch
        for (int s = 0; s < a.kv_group; ++s) launch_decode(group_pass(a, s), ws, sm_count, max_smem, st);
        return;
    }
    SplitPlan p;
    if (make_split_plan(a, sm_count, max_smem, p)) {
        float* ws_acc = nullptr;
        float* ws_ml = nullptr;
        if (a.mode != DecodeMode::QK) {
            // 256-byte aligned start, acc block first (its size is a multiple of 16 bytes)
            uintptr_t base = (reinterpret_cast<uintptr_t>(ws) + 255) & ~static_cast<uintptr_t>(255);
            ws_acc = reinterpret_cast<float*>(base);
            ws_ml = ws_acc + split_ws_floats_acc(a, p);
        }
        switch (a.dt) {
            case Dt::F16: launch_split_mode<__half>(a, p, ws_acc, ws_ml, st); break;
            case Dt::BF16: launch_split_mode<__nv_bfloat16>(a, p, ws_acc, ws_ml, st); break;
            default: launch_split_mode<float>(a, p, ws_acc, ws_ml, st); break;
        }
        return;
    }
    switch (a.dt) {
        case Dt::F16: launch_plain_mode<__half>(a, st); break;
        case Dt::BF16: launch_plain_mode<__nv_bfloat16>(a, st); break;
        case Dt::F32: launch_plain_mode<float>(a, st); break;
        default: break;  // fp64 is refused by the caller
    }
}

int64_t decode_static_scratch_capacity() { return kStaticScratchBytes; }

cudaError_t launch_decode_static_scratch(const DecodeArgs& a, int sm_count, int max_smem, cudaStream_t st, int64_t* needed) {
    *needed = decode_workspace_bytes(a, sm_count, max_smem);
    if (*needed > kStaticScratchBytes) return cudaErrorMemoryAllocation;  // the caller turns this into its own message
    void* ws = nullptr;
    if (*needed > 0) {
        cudaError_t e = static_scratch_address(&ws);
        if (e != cudaSuccess) return e;
    }
    launch_decode(a, ws, sm_count, max_smem, st);
    return cudaSuccess;
}

}  // namespace k
}  // namespace b200
