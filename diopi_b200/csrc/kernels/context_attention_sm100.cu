// Tensor-core causal prefill for sm_100a: tcgen05.mma with accumulators in TMEM, operands staged by TMA.
// Path of diopiContextAttentionInference (and of diopiPromptFlashAttention) for fp16/bf16, head_dim 64, 128 or 256,
// dense 16-byte aligned rows; every other shape runs on the blockwise SIMT kernel. Replaces the per-request
// matmul/mask/softmax/matmul chain of impl/torch/functions/functions_lightllm.cpp:109-147.
//
// One CTA per SM works on NT tiles of 128 query rows of one (request, head) that share every K/V block they read
// (key blocks of 64; head_dim 64 and 128: two tiles, head_dim 256: one), with two score buffers per tile:
//   warp 0 (one lane)  TMA: the Q tiles once (64-wide boxes, 128-byte swizzle), then K_j and V_j into a ring of 4 (2) stages
//   warp 1 (warp 2)    one lane issues every product of tile 0 (tile 1) as soon as its inputs are ready (probing the
//                      barriers, never blocking on one while another could go):
//                        S_t = Q_t K_j^T  tcgen05.mma M128 N64 K16, both operands K-major from shared memory
//                        O_t += P_t V_j   tcgen05.mma M128 N<HD> K16, A = P_t read from TMEM, B = V_j MN-major
//   warps 4-7 (8-11)   soft-max of tile 0 (tile 1), thread = query row: tcgen05.ld of its S row, causal/length mask,
//                      online soft-max in base 2 (scale and maximum folded into one fma + ex2 per score; the reference
//                      maximum is only raised when the row maximum grew by more than 2^8, and only then is O in TMEM
//                      rescaled), P packed to 16 bit and written over the S cells just read
// While the soft-max of block j reads one score buffer of a tile, Q_t K_{j+1}^T fills the other. A K/V block is fetched
// and held in shared memory once for both tiles. TMEM columns (512 allocated): score buffers at 64 * (2 t + j % 2),
// O_t at 256 + t * HD.
// What the measurements taught (benchmark config: 8 requests of 1024..8192 rows, 32 heads, D 128, fp16):
//   one tile per CTA, two CTAs per SM, own K/V copies: 873 TFLOP/s; this form: 950 to 980 TFLOP/s. On the way: one
//   thread issuing for both tiles was the limit (1.30 of the time of one issuing warp per tile with descriptors made
//   once). What bounds this form is the tensor pipe's instruction rate, not the soft-max: issued by itself, a
//   tcgen05.mma M128 K16 takes about 98 cycles when it accumulates onto the one before it and about 72 when two chains
//   alternate, whatever N <= 128 is (only N = 256 runs at the nominal 4096 MAC per cycle), so the products of a pair of
//   64-key blocks (two Q K^T of 8 steps at N 64, two P V of 4 steps) take 1670 to 1830 cycles alone and the loop takes
//   2010 per pair. That is why nothing done to the soft-max moved the time: more or fewer exponentials on the fma pipe,
//   the two warps of a scheduler taking turns at the special-function unit (16 ex2 per cycle and SM, 1060 cycles per pair
//   of blocks), 224 registers for the soft-max threads by setmaxnreg. Key blocks of 128 halve the Q K^T instructions,
//   but TMEM (512 columns: 2 x 128 for O) then holds one score buffer per tile: with P written over the scores 754 to
//   795 TFLOP/s (Q K^T, soft-max and P V of a tile in series), with P handed over through shared memory (the buffer is
//   free once the scores are in registers) 900 against 952 for this form in the same run: the soft-max threads then
//   wait for the shared P piece and run 1800 cycles per 64 keys. A CTA spends 3.5 us before its first scores, 47 us
//   in the loop and 1.9 us storing O on average; the SMs are busy 94 % of the kernel's span.
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

constexpr int BM = 128;      // query rows per tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 256;

enum Bar { Q_FULL = 0, K_FULL = 1, V_FULL = 5, K_EMPTY = 9, V_EMPTY = 13, O_FULL = 17, S_FULL = 19, S_EMPTY = 23, P_FULL = 27, kNumBars = 31 };   // up to four ring stages and four score buffers

// Shared-memory map and sizes of one configuration; every operand tile starts on a 1024-byte boundary (swizzle atoms).
template <int HD, int BN, int NT>
struct Cfg {
    static_assert(HD % 64 == 0 && HD <= 256 && BN == 64 && (NT == 1 || NT == 2), "unsupported tile shape");
    static_assert(NT * HD <= 256, "the O tiles take TMEM columns 256..511");
    // score buffers per tile: as many as fit TMEM columns 0..255, two at most (a second one lets Q K^T of block j + 1 run
    // while the soft-max of block j reads the first)
    static constexpr int kSlotsPerTile = 256 / (NT * BN) >= 2 ? 2 : 1;
    static_assert(NT * BN * kSlotsPerTile <= 256, "score buffers take TMEM columns 0..255");
    static constexpr int kThreads = 128 + 128 * NT;   // warp group 0: TMA warp, MMA warp, two idle warps; then one soft-max warp group per tile
    static constexpr int kDBlocks = HD / 64;          // 64-wide column blocks of a row
    static constexpr int kQTile = BM * HD * 2;
    static constexpr int kKStage = BN * HD * 2;
    // K/V ring: four stages where they fit beside the Q tiles (64-key blocks at head_dim <= 128), else two
    static constexpr int kStages = (NT * BM * HD * 2 + 8 * BN * HD * 2 <= 200 * 1024) ? 4 : 2;
    static constexpr int kOffQ = 0;
    static constexpr int kOffK = kOffQ + NT * kQTile;
    static constexpr int kOffV = kOffK + kStages * kKStage;
    static constexpr int kOffBar = kOffV + kStages * kKStage;
    static constexpr int kOffTmemSlot = kOffBar + kNumBars * 8;
    static constexpr int kOffFlag = kOffTmemSlot + 8;
    static constexpr int kUsedBytes = kOffFlag + 8;
    // at least 120 KB, so that never two CTAs share an SM: each allocates all 512 TMEM columns
    static constexpr int kSmemBytes = kUsedBytes > 120 * 1024 ? kUsedBytes : 120 * 1024;
};

struct TcParams {
    IndexArg b_start, b_len;
    int B, H;
    int64_t total_rows;
    void* out;
    int64_t o_s0, o_s1;
    int n_groups_max;      // upper bound of the number of groups of NT tiles over all requests
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

// Share of the exponentials computed on the fma pipe, per head dim (see prefill_tc_kernel).
constexpr int kPolyEvery64 = 2, kPolyEvery128 = 8, kPolyEvery256 = 8;

// kPolyEvery: of every kPolyEvery groups of four scores, one computes two of its exponentials on the fma pipe
// (1: half of all exponentials, 2: a quarter, 4: an eighth, 8: a sixteenth, 0: none).
template <bool BF16, int HD, int BN, int NT, int kPolyEvery>
__global__ void __launch_bounds__(Cfg<HD, BN, NT>::kThreads, 1)
    prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const TcParams p) {
    using C = Cfg<HD, BN, NT>;
    constexpr int kStages = C::kStages;
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::kOffTmemSlot);
    volatile int* give_up = reinterpret_cast<volatile int*>(smem + C::kOffFlag);
    auto bar = [&](int i) { return smem_u32(&bars[i]); };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y;
    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
    }
    const int hkv = h / p.kv_group;   // grouped-query attention: several query heads share one K/V head

    // ---- which (request, group of NT row tiles) is this CTA? Heaviest groups (late rows) are handed out first. ----
    int req = -1;
    int64_t L = 0, start = 0, r0 = 0;
    {
        // Every warp does the same search, 32 requests at a time: lane i loads request i's length and start (one round of
        // loads in flight instead of a chain of dependent ones), a warp scan gives the groups before it.
        const int64_t flat = static_cast<int64_t>(p.n_groups_max) - 1 - blockIdx.x;
        int64_t before = 0;
        for (int base = 0; base < p.B && req < 0; base += 32) {
            const int i = base + lane;
            int64_t Li = 0, si = 0;
            if (i < p.B) {
                Li = p.uniform_len > 0 ? p.uniform_len : load_index(p.b_len, i);
                si = p.uniform_len > 0 ? i * p.uniform_len : load_index(p.b_start, i);
                if (Li <= 0 || si < 0 || si >= p.total_rows) Li = 0;
                else Li = imin64(Li, p.total_rows - si);
            }
            const int ng = static_cast<int>((Li + BM * NT - 1) / (BM * NT));
            int incl = ng;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += up;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, ng > 0 && flat < before + incl);
            if (hit != 0) {
                const int src = __ffs(hit) - 1;
                req = base + src;
                L = __shfl_sync(0xffffffffu, Li, src);
                start = __shfl_sync(0xffffffffu, si, src);
                r0 = (flat - before - __shfl_sync(0xffffffffu, incl - ng, src)) * (BM * NT);
            } else {
                before += __shfl_sync(0xffffffffu, incl, 31);
            }
        }
    }
    if (req < 0) return;  // the whole CTA leaves together, before any barrier or TMEM use
    // key blocks tile t reads: up to its last row's diagonal; a tile that starts beyond the request has none
    int nblk[NT];
    int nblk_max = 0;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const int64_t rt = r0 + static_cast<int64_t>(t) * BM;
        nblk[t] = rt < L ? static_cast<int>((imin64(L, rt + BM) + BN - 1) / BN) : 0;
        nblk_max = nblk[t] > nblk_max ? nblk[t] : nblk_max;
    }

    if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte aligned base; refuse rather than compute garbage
        if (tid == 0) report_status(p.status, 3);
        return;
    }
    if (tid == 0) {
        mbar_init(bar(Q_FULL), 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar(K_FULL + s), 1);
            mbar_init(bar(V_FULL + s), 1);
            mbar_init(bar(K_EMPTY + s), NT);   // one arrival per tile: the commit after its product, or a plain arrive for a tile that skips the block
            mbar_init(bar(V_EMPTY + s), NT);
        }
        mbar_init(bar(O_FULL), 1);
        mbar_init(bar(O_FULL + 1), 1);
        for (int s = 0; s < 4; ++s) {
            mbar_init(bar(S_FULL + s), 1);
            mbar_init(bar(S_EMPTY + s), 1);    // freed by the commit that follows the P V that read the buffer
            mbar_init(bar(P_FULL + s), 4);     // the four warps of a soft-max group
        }
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

    // Score buffer of (tile t, block j) and how many times it was used before: a tile's buffers take turns.
    constexpr int SPT = C::kSlotsPerTile;
    auto slot_of = [](int t, int j) { return t * SPT + (j % SPT); };
    auto use_of = [](int j) { return j / SPT; };

    if (warp == 0) {
        // ================================ TMA producer =================================
        if (lane == 0) {
            const int row0 = static_cast<int>(start + r0);
            mbar_expect_tx(bar(Q_FULL), NT * C::kQTile);
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int d = 0; d < C::kDBlocks; ++d)
                    tma_load_3d(smem_u32(smem + C::kOffQ + t * C::kQTile + d * (BM * 128)), &map_q, d * 64, h, row0 + t * BM, bar(Q_FULL));
            for (int j = 0; j < nblk_max; ++j) {
                const int s = j % kStages;
                const uint32_t ph = static_cast<uint32_t>((j / kStages) & 1);
                const int krow = static_cast<int>(start + static_cast<int64_t>(j) * BN);
                if (!mbar_wait(bar(K_EMPTY + s), ph ^ 1u, give_up)) break;
                mbar_expect_tx(bar(K_FULL + s), C::kKStage);
#pragma unroll
                for (int d = 0; d < C::kDBlocks; ++d)
                    tma_load_3d(smem_u32(smem + C::kOffK + s * C::kKStage + d * (BN * 128)), &map_k, d * 64, hkv, krow, bar(K_FULL + s));
                if (!mbar_wait(bar(V_EMPTY + s), ph ^ 1u, give_up)) break;
                mbar_expect_tx(bar(V_FULL + s), C::kKStage);
#pragma unroll
                for (int d = 0; d < C::kDBlocks; ++d)
                    tma_load_3d(smem_u32(smem + C::kOffV + s * C::kKStage + d * (BN * 128)), &map_v, d * 64, hkv, krow, bar(V_FULL + s));
            }
        }
    } else if (warp == 1 || (NT == 2 && warp == 2)) {
        // ================================ MMA issuers: one warp (one lane) per tile ===================================
        const int t = warp - 1;
        if (lane == 0 && nblk[t] == 0) {
            // A tile beyond the request's end reads no block: its share of the K/V hand-backs is given as soon as each
            // block has landed (an arrival must not fall into an earlier phase of the barrier).
            bool ok = true;
            for (int j = 0; ok && j < nblk_max; ++j) {
                const int s = j % kStages;
                const uint32_t ph = static_cast<uint32_t>((j / kStages) & 1);
                ok = mbar_wait(bar(K_FULL + s), ph, give_up) && mbar_wait(bar(V_FULL + s), ph, give_up);
                if (ok) {
                    mbar_arrive(bar(K_EMPTY + s));
                    mbar_arrive(bar(V_EMPTY + s));
                }
            }
        } else if (lane == 0) {
            const uint32_t idesc_qk = make_idesc(BM, BN, BF16 ? 1 : 0, 0);
            const uint32_t idesc_pv = make_idesc(BM, HD, BF16 ? 1 : 0, 1);
            // Descriptors are made once; a product adds the (compile-time) offset of its 16-wide k step to the address field.
            const uint64_t q_desc = make_desc(smem_u32(smem + C::kOffQ + t * C::kQTile), 0, 1024);
            const uint64_t k_desc0 = make_desc(smem_u32(smem + C::kOffK), 0, 1024);          // stage s: + s * stage bytes in the address field
            const uint64_t v_desc0 = make_desc(smem_u32(smem + C::kOffV), BN * 128, 1024);
            const int my_blocks = nblk[t];
            bool ok = mbar_wait(bar(Q_FULL), 0, give_up);
            // Event driven: the next Q K^T and the P V of the oldest finished soft-max are issued in whatever order their
            // inputs become ready; P V first, because it is what frees a score buffer.
            int nqk = 0, npv = 0;
            unsigned long long idle_since = 0;
            uint32_t idle_probes = 0;
            while (ok && npv < my_blocks) {
                bool progressed = false;
                if (npv < nqk) {
                    const int j = npv;
                    const int s = j % kStages, sl = slot_of(t, j);
                    if (mbar_test(bar(P_FULL + sl), static_cast<uint32_t>(use_of(j) & 1)) && mbar_test(bar(V_FULL + s), static_cast<uint32_t>((j / kStages) & 1))) {
                        tc_fence_after();
                        const uint64_t vd = v_desc0 + static_cast<uint64_t>(s) * (C::kKStage >> 4);
#pragma unroll
                        for (int kk = 0; kk < BN / 16; ++kk) {
                            // B = V [BN keys x HD], MN-major: 16 keys = 16 rows of 128 bytes; the next 64-wide column block is BN * 128 bytes further.
                            // A = P in TMEM: 16 keys = 8 cells of the score buffer the soft-max threads overwrote.
                            umma_ts(tmem_base + kColO + t * HD, tmem_base + sl * BN + kk * 8, vd + static_cast<uint64_t>((kk * 16 * 128) >> 4), idesc_pv,
                                    (j > 0 || kk > 0) ? 1u : 0u);
                        }
                        umma_commit(bar(S_EMPTY + sl));
                        umma_commit(bar(V_EMPTY + s));
                        umma_commit(bar(O_FULL + t));
                        ++npv;
                        progressed = true;
                    }
                }
                if (nqk < my_blocks) {
                    const int j = nqk;
                    const int s = j % kStages, sl = slot_of(t, j);
                    if (mbar_test(bar(K_FULL + s), static_cast<uint32_t>((j / kStages) & 1)) &&
                        mbar_test(bar(S_EMPTY + sl), static_cast<uint32_t>((use_of(j) & 1) ^ 1))) {
                        tc_fence_after();
                        const uint64_t kd = k_desc0 + static_cast<uint64_t>(s) * (C::kKStage >> 4);
#pragma unroll
                        for (int kk = 0; kk < HD / 16; ++kk) {
                            // both operands K-major; column block kk / 4 (64 wide), 16 columns = 32 bytes inside the swizzled row
                            const uint64_t ad = q_desc + static_cast<uint64_t>(((kk / 4) * (BM * 128) + (kk % 4) * 32) >> 4);
                            const uint64_t bd = kd + static_cast<uint64_t>(((kk / 4) * (BN * 128) + (kk % 4) * 32) >> 4);
                            umma(tmem_base + sl * BN, ad, bd, idesc_qk, kk > 0 ? 1u : 0u);
                        }
                        umma_commit(bar(S_FULL + sl));
                        umma_commit(bar(K_EMPTY + s));
                        ++nqk;
                        progressed = true;
                    }
                }
                if (progressed) {
                    idle_since = 0;
                    idle_probes = 0;
                } else if ((++idle_probes & 0xffu) == 0) {
                    // The clock and the flag are looked at once in 256 idle rounds (a round is a handful of barrier probes).
                    if (*give_up) break;
                    const unsigned long long now = global_ns();
                    if (idle_since == 0) idle_since = now;
                    if (now - idle_since > kWaitLimitNs) {
                        *give_up = 1;
                        ok = false;
                    }
                }
            }
            // blocks beyond this tile's diagonal that the other tile still reads: hand them back as they land
            for (int j = my_blocks; ok && j < nblk_max; ++j) {
                const int s = j % kStages;
                const uint32_t ph = static_cast<uint32_t>((j / kStages) & 1);
                ok = mbar_wait(bar(K_FULL + s), ph, give_up) && mbar_wait(bar(V_FULL + s), ph, give_up);
                if (ok) {
                    mbar_arrive(bar(K_EMPTY + s));
                    mbar_arrive(bar(V_EMPTY + s));
                }
            }
        }
    } else if (warp >= 4) {
        // ================================ soft-max warps: thread = query row ==========================
        const int t = NT == 2 ? ((warp - 4) >> 2) : 0;   // the tile of this warp group
        const int quarter = warp & 3;                    // the TMEM lane quarter this warp may touch
        const int row = quarter * 32 + lane;             // row inside the tile
        const int64_t rt0 = r0 + static_cast<int64_t>(t) * BM;   // first row of the tile inside the request
        const int64_t rr = rt0 + row;                    // this thread's row inside the request
        const int my_blocks = nblk[t];
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const uint32_t o_col = kColO + t * HD;
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < my_blocks; ++j) {
            const int sl = slot_of(t, j);
            const uint32_t ph = static_cast<uint32_t>(use_of(j) & 1);
            if (!warp_wait(bar(S_FULL + sl), ph, give_up)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const int64_t key0 = static_cast<int64_t>(j) * BN;
            const bool edge = (key0 + BN - 1 > rt0) || (key0 + BN > L);   // block touches the tile's diagonal or the request's end
            const int lim = edge ? static_cast<int>(imin64(imin64(rr, L - 1) - key0, BN)) : BN;   // last allowed column of this row inside the block
            {
                // 64 scores fit in registers: one trip to TMEM, the row maximum and the exponentials on the same registers.
                // Two copies of the code, with and without the mask, so that a block away from the diagonal executes no
                // masking instruction at all (merged, the compiler turns the mask into 64 predicated selects every block).
                auto block64 = [&](auto edge_c) -> bool {
                    constexpr bool kEdge = decltype(edge_c)::value;
                    uint32_t ua[32], ub[32];
                    tmem_ld32(lane_base + sl * BN, ua);
                    tmem_ld32(lane_base + sl * BN + 32, ub);
                    tmem_wait_ld();
                    float sc[64];
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        sc[c] = __uint_as_float(ua[c]);
                        sc[c + 32] = __uint_as_float(ub[c]);
                    }
                    if constexpr (kEdge) {
#pragma unroll
                        for (int c = 0; c < 64; ++c)
                            if (c > lim) sc[c] = -INFINITY;
                    }
                    float mx0 = fmaxf(sc[0], sc[1]), mx1 = fmaxf(sc[2], sc[3]), mx2 = fmaxf(sc[4], sc[5]), mx3 = fmaxf(sc[6], sc[7]);
#pragma unroll
                    for (int c = 8; c < 64; c += 8) {
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
                            if (!warp_wait(bar(O_FULL + t), static_cast<uint32_t>((j - 1) & 1), give_up)) return false;
                            tc_fence_after();
#pragma unroll
                            for (int c4 = 0; c4 < HD / 32; ++c4) {
                                uint32_t o[32];
                                tmem_ld32(lane_base + o_col + c4 * 32, o);
                                tmem_wait_ld();
#pragma unroll
                                for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                                tmem_st32(lane_base + o_col + c4 * 32, o);
                            }
                            tmem_wait_st();
                        }
                        l *= alpha;
                        m_used = m_next;
                    }
                    const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
                    float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
                    if constexpr (kPolyEvery == 0) {
                        // plain scalar form: one fma, one ex2, one add per score
#pragma unroll
                        for (int c = 0; c < 64; c += 4) {
                            sc[c] = fast_exp2(fmaf(sc[c], p.scale_log2, neg_m));
                            sc[c + 1] = fast_exp2(fmaf(sc[c + 1], p.scale_log2, neg_m));
                            sc[c + 2] = fast_exp2(fmaf(sc[c + 2], p.scale_log2, neg_m));
                            sc[c + 3] = fast_exp2(fmaf(sc[c + 3], p.scale_log2, neg_m));
                            rs0 += sc[c];
                            rs1 += sc[c + 1];
                            rs2 += sc[c + 2];
                            rs3 += sc[c + 3];
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < 64; c += 4) {
                            ffma2(sc[c], sc[c + 1], sc[c], sc[c + 1], p.scale_log2, neg_m);
                            ffma2(sc[c + 2], sc[c + 3], sc[c + 2], sc[c + 3], p.scale_log2, neg_m);
                            sc[c] = fast_exp2(sc[c]);
                            sc[c + 1] = fast_exp2(sc[c + 1]);
                            if ((c / 4) % (kPolyEvery > 0 ? kPolyEvery : 1) == 0) {
                                poly_exp2_pair(sc[c + 2], sc[c + 3]);
                            } else {
                                sc[c + 2] = fast_exp2(sc[c + 2]);
                                sc[c + 3] = fast_exp2(sc[c + 3]);
                            }
                            fadd2(rs0, rs1, sc[c], sc[c + 1]);
                            fadd2(rs2, rs3, sc[c + 2], sc[c + 3]);
                        }
                    }
                    l += (rs0 + rs1) + (rs2 + rs3);
                    uint32_t pk[32];
#pragma unroll
                    for (int c = 0; c < 32; ++c) pk[c] = pack2<BF16>(sc[2 * c], sc[2 * c + 1]);   // cell c: keys 2c (low half) and 2c + 1
                    tmem_st32(lane_base + sl * BN, pk);
                    return true;
                };
                const bool fine = edge ? block64(std::true_type{}) : block64(std::false_type{});
                if (!fine) {
                    ok = false;
                    break;
                }
            }
            tmem_wait_st();
            tc_fence_before();
            // A parity wait tells n finished products from n + 1, not from n + 2. Inside the loop that is enough: at the
            // start of block j between j - 1 and j products of this tile are finished (Q K_j^T needed the buffer P V_{j-2}
            // read; P V_j is not issued yet). After the last hand-over it would not be (n - 2, n - 1 or n): so the last
            // block sees P V_{n-2} finished before it hands P over, which leaves n - 1 or n for the wait after the loop.
            if (j > 0 && j == my_blocks - 1 && !warp_wait(bar(O_FULL + t), static_cast<uint32_t>((j - 1) & 1), give_up)) {
                ok = false;
                break;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(P_FULL + sl));
        }
        // All products but the last are known to be finished (see the loop): one wait for the last one.
        if (ok && my_blocks >= 1 && warp_wait(bar(O_FULL + t), static_cast<uint32_t>((my_blocks - 1) & 1), give_up)) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const bool store = rr < L;
            unsigned char* dst = static_cast<unsigned char*>(p.out) + ((start + rr) * p.o_s0 + static_cast<int64_t>(h) * p.o_s1) * 2;
#pragma unroll
            for (int c4 = 0; c4 < HD / 32; ++c4) {
                uint32_t o[32];
                tmem_ld32(lane_base + o_col + c4 * 32, o);
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
bool make_map(CUtensorMap* map, const void* base, int D, int64_t rows, int H, int64_t s0, int64_t s1, int box_rows, bool bf16) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(s1) * 2, static_cast<cuuint64_t>(s0) * 2};
    const cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int HD, int BN, int NT, int kPolyEvery>
bool launch_cfg(const PrefillArgs& a, int max_smem, cudaStream_t st) {
    using C = Cfg<HD, BN, NT>;
    if (C::kSmemBytes > max_smem) return false;
    const bool bf16 = a.dt == Dt::BF16;
    CUtensorMap mq, mk, mv;
    if (!make_map(&mq, a.q, HD, a.total_rows, a.H, a.q_s0, a.q_s1, BM, bf16)) return false;
    if (!make_map(&mk, a.kmat, HD, a.total_rows, a.H / a.kv_group, a.k_s0, a.k_s1, BN, bf16)) return false;
    if (!make_map(&mv, a.vmat, HD, a.total_rows, a.H / a.kv_group, a.v_s0, a.v_s1, BN, bf16)) return false;
    TcParams p;
    p.b_start = a.b_start;
    p.b_len = a.b_len;
    p.B = a.B;
    p.H = a.H;
    p.total_rows = a.total_rows;
    p.out = a.out;
    p.o_s0 = a.o_s0;
    p.o_s1 = a.o_s1;
    p.n_groups_max = static_cast<int>(a.total_rows / (BM * NT) + a.B);
    p.scale_log2 = kLog2e / sqrtf(static_cast<float>(HD));
    p.status = nullptr;
    p.uniform_len = a.uniform_len;
    p.kv_group = a.kv_group;
    dim3 grid(p.n_groups_max, a.H, 1);
    auto go = [&](auto kern) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        kern<<<grid, C::kThreads, C::kSmemBytes, st>>>(mq, mk, mv, p);
    };
    if (bf16)
        go(prefill_tc_kernel<true, HD, BN, NT, kPolyEvery>);
    else
        go(prefill_tc_kernel<false, HD, BN, NT, kPolyEvery>);
    return true;
}

}  // namespace

void launch_prefill_tc(const PrefillArgs& a, int /*sm_count*/, int max_smem, cudaStream_t st, bool* taken) {
    *taken = false;
    if (a.force_simt) return;
    if (a.dt != Dt::F16 && a.dt != Dt::BF16) return;
    if ((a.D != 64 && a.D != 128 && a.D != 256) || a.H > 65535) return;
    if (a.total_rows >= (1ll << 31) - 2 * BM) return;
    auto ok = [](const void* p, int64_t s0, int64_t s1) {
        return reinterpret_cast<uintptr_t>(p) % 16 == 0 && (s0 * 2) % 16 == 0 && (s1 * 2) % 16 == 0 && s0 > 0 && s1 > 0;
    };
    if (!ok(a.q, a.q_s0, a.q_s1) || !ok(a.kmat, a.k_s0, a.k_s1) || !ok(a.vmat, a.v_s0, a.v_s1) || !ok(a.out, a.o_s0, a.o_s1)) return;
    switch (a.D) {
        case 64: *taken = launch_cfg<64, 64, 2, kPolyEvery64>(a, max_smem, st); break;
        case 128: *taken = launch_cfg<128, 64, 2, kPolyEvery128>(a, max_smem, st); break;
        default: *taken = launch_cfg<256, 64, 1, kPolyEvery256>(a, max_smem, st); break;
    }
}

}  // namespace k
}  // namespace b200
