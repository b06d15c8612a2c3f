// diopiMatmulAllReduce: out = sum over the ranks of a group of (x1_r @ x2_r + bias_r), the row-parallel linear layer
// that follows attention in a head-sharded model, as ONE kernel per rank. The reference forwards this call to the
// vendor's aclnnMatmulAllReduce (impl/ascend/functions_ext/matmul_all_reduce.cpp:13-17,
// impl/ascend_npu/diopi_impl/functions_ext/matmul_all_reduce.cpp:12-17; signature proto/include/diopi/functions_ext.h:664-665);
// there is no NVIDIA implementation to replace.
//
// Per rank, a persistent grid (one CTA per SM at most) walks the 128 x TN output tiles (TN = 128; 64 or 32 for outputs of
// few rows, so that enough CTAs stream the weights):
//   warp 0 (one lane)  TMA: x1 tile [128 x 64] and x2 tile [64 x TN] (or [TN x 64] when x2 is given K-major) into a
//                      ring of 4 to 6 stages, 128-byte swizzle, no multicast
//   warp 1 (one lane)  tcgen05.mma M128 N<TN> K16, fp32 accumulators in TMEM (two accumulator buffers, so the epilogue
//                      of one tile overlaps the products of the next)
//   warps 2-5          epilogue: TMEM -> registers -> shared memory (transpose to whole rows) -> (+ bias) -> 16-byte stores
//                      of the fp32 partial rows into EVERY rank's staging area over NVLink (peer pointers, this rank's
//                      own copy included). Every 64-bit word stored is (call number << 32 | payload): the data is its
//                      own arrival mark, there is no flag to write after it and no fence to wait for.
// Once a CTA has sent all its tiles, the same warps read, for each of those tiles, the partial rows of all ranks from
// this rank's own staging area (re-reading a row until every word carries this call's number, bounded by a time limit),
// add them in rank order in fp32 and write the tile of `out` once. Every rank adds the same numbers in the same
// order: all ranks get identical bits.
// That is the one-shot form (each rank receives world x the output): right for decode-sized outputs, where latency
// counts. In the two-shot form a tile's partials go only to its owner (rank tile % world), which adds them up and
// writes the finished 16-bit rows (marked the same way) into every rank's result area; every rank then copies the
// tiles it does not own from its result area to `out`: 1 / world of the one-shot bytes for the partials at the price
// of a second hop. The staging area fixes the largest output (tiles) a group can take.
//
// Waiting on another rank's kernel: the marks are the call's sequence number (kept in device memory, no reset between
// calls, nothing per call from the host: a captured launch can be replayed) and the staging
// area is double-buffered; a rank cannot run two calls ahead of a peer, because it needs that peer's rows of the
// call in between. A wait that runs out (a peer that never calls; the limit is a property of the group, 2 s unless
// set otherwise) raises the status word (code 3), the kernel returns with TMEM freed, and the group is poisoned on
// every rank (word 2 of each rank's control words): the ranks' call numbers may no longer agree, so no later call
// may trust a mark. Kernels launched on a poisoned group leave at once; the host refuses them until the group is
// destroyed and created again.
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "dev_util.cuh"
#include "sm100_ptx.cuh"

namespace b200 {
namespace k {

namespace {

using namespace sm100;  // NOLINT

constexpr int TM = 128, TK = 64;              // rows of an output tile, K step of one ring stage
constexpr int kTileCap = 128;                 // widest tile; a group's capacity is counted in 128 x 128 tiles
constexpr int kMaxStages = 10;
constexpr int kThreads = 192;
constexpr int kRingBytes = 128 * 1024;        // stages of (x1 tile, x2 tile): 4 x 32 KB ... 10 x 12 KB
constexpr int kRowPadMax = kTileCap + 4;      // floats per row of the transpose buffer (16-byte stores without bank conflicts)
constexpr int kOffRing = 0;
constexpr int kOffT = kOffRing + kRingBytes;  // transpose buffer: 4 warps x 32 rows x (TN + 4) floats
constexpr int kTBytes = 4 * 32 * kRowPadMax * 4;
constexpr int kOffBar = kOffT + kTBytes;
enum Bar { FULL = 0, EMPTY = kMaxStages, ACC_FULL = 2 * kMaxStages, ACC_EMPTY = 2 * kMaxStages + 2, kNumBars = 2 * kMaxStages + 4 };
constexpr int kOffTmemSlot = kOffBar + kNumBars * 8;
constexpr int kOffFlag = kOffTmemSlot + 8;
constexpr int kSmemBytes = kOffFlag + 8;
constexpr uint32_t kTmemCols = 256;           // two accumulators of up to 128 fp32 columns

// Narrow tiles (TN = 64, 32) exist for outputs of few rows: the product is then bound by streaming the weights, and
// 128-wide tiles would leave most SMs without work (N = 4096: 32 CTAs at TN = 128, 128 CTAs at TN = 32).
// AM = rows of x1 a stage holds: 128, or 64 when the whole product has at most 64 rows. The MMA still reads 128 rows
// of shared memory; what it finds behind the 64 loaded ones only reaches accumulator rows that are never read. Halving
// the x1 tile leaves room for more stages, i.e. more weight bytes in flight per CTA.
template <int TN, int AM = 128>
struct Tile {
    static constexpr int kABytes = AM * TK * 2;
    static constexpr int kBBytes = TN * TK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = kRingBytes / kStageBytes < kMaxStages ? kRingBytes / kStageBytes : kMaxStages;   // 4 ... 10
    static constexpr int kRowPad = TN + 4;
    static constexpr int kLanesPerRow = TN / 4;                     // a lane owns 4 columns
    static constexpr int kRowsPerInstr = 32 / kLanesPerRow;         // rows one warp-wide access covers: 1, 2, 4
    static constexpr size_t kPartialRowBytes = TN * 8;   // fp32 payload + mark per value
    static constexpr size_t kResultRowBytes = TN * 4;    // 16-bit payload pairs + mark
};
constexpr size_t kPartialCapBytes = static_cast<size_t>(TM) * kTileCap * 8;   // room of one 128 x 128 tile of partials
constexpr size_t kResultCapBytes = static_cast<size_t>(TM) * kTileCap * 4;

// Data that carries its own arrival mark: a 64-bit word = (call number << 32) | 32 bits of payload, written and read
// with single 64-bit accesses (two per 16-byte vector access), which are atomic: a reader that finds this call's number
// in the upper half has the payload of this call in the lower half. No flag after the data, no fence before a flag:
// a row is usable the moment it lands. Costs twice the bytes, which at these sizes is cheaper than a fence round trip.
__device__ __forceinline__ void st_pair(unsigned char* p, uint32_t a, uint32_t b, uint32_t epoch) {
    const uint64_t hi = static_cast<uint64_t>(epoch) << 32;
    asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(hi | a), "l"(hi | b) : "memory");
}
__device__ __forceinline__ bool ld_pair(const unsigned char* p, uint32_t epoch, uint32_t& a, uint32_t& b) {
    uint64_t x, y;
    asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(x), "=l"(y) : "l"(p) : "memory");
    a = static_cast<uint32_t>(x);
    b = static_cast<uint32_t>(y);
    return static_cast<uint32_t>(x >> 32) == epoch && static_cast<uint32_t>(y >> 32) == epoch;
}
// Between two polls: starts the clock at the first miss, gives up after the time limit or when another role did.
__device__ __forceinline__ bool poll_again(unsigned long long& t0, volatile int* give_up, unsigned long long limit_ns) {
    const unsigned long long now = global_ns();
    if (t0 == 0) t0 = now;
    if (*give_up || now - t0 > limit_ns) {
        *give_up = 1;
        return false;
    }
    return true;
}

// Byte offsets inside one rank's area. A partial row holds words (x, y) of the lane that owns columns 4c .. 4c+3 at
// 16 c and its words (z, w) at TN * 4 + 16 c, so that each of a warp's two stores covers whole 512-byte runs. Tiles of
// any width are packed into regions sized for max_tiles tiles of 128 x 128.
template <int TN>
__device__ __forceinline__ size_t partial_slot(int buf, int world, int src, int max_tiles, int tile) {
    return (static_cast<size_t>(buf) * world + src) * max_tiles * kPartialCapBytes + static_cast<size_t>(tile) * TM * Tile<TN>::kPartialRowBytes;
}
template <int TN>
__device__ __forceinline__ size_t result_slot(int buf, int max_tiles, int tile) {
    return static_cast<size_t>(buf) * max_tiles * kResultCapBytes + static_cast<size_t>(tile) * TM * Tile<TN>::kResultRowBytes;
}

template <bool BF16, bool B_KMAJOR, int TN, int AM>
__global__ void __launch_bounds__(kThreads, 1) matmul_allreduce_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                                        const MatmulAllReduceArgs a) {
    using TL = Tile<TN, AM>;
    constexpr int kStages = TL::kStages;
    constexpr int kABytes = TL::kABytes;
    static_assert(B_KMAJOR || TN >= 64, "an MN-major x2 tile is made of 64-column boxes");
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffTmemSlot);
    volatile int* give_up = reinterpret_cast<volatile int*>(smem + kOffFlag);
    auto bar = [&](int i) { return smem_u32(&bars[i]); };
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_n = (a.N + TN - 1) / TN;
    const int n_tiles = ((a.M + TM - 1) / TM) * tiles_n;
    const int kblocks = (a.K + TK - 1) / TK;
    // Split-K (groups of one rank only): S CTAs share an output tile, each with a slice of the k blocks; the slices meet in
    // the staging area like the partials of S ranks would. Virtual tile vt = tile * S + slice; S = 1 is the plain form.
    const int S = a.k_splits > 1 ? a.k_splits : 1;
    const int n_vt = n_tiles * S;
    const int W = a.world * S;            // sources of partial rows per tile
    const int mt = a.max_tiles / S;       // tiles the staging area holds when every rank brings S sources
    // The call's sequence number lives in device memory (the number of calls this group has finished, plus one) and is
    // advanced by the last CTA to leave: the host passes nothing that changes from call to call, so a captured launch
    // can be replayed. Every CTA reads it here, before any CTA of this launch can have left.
    const uint32_t epoch = *reinterpret_cast<volatile const uint32_t*>(a.ctrl) + 1u;
    const int buf = static_cast<int>(epoch & 1u);   // which half of the staging area this call uses
    // A group in which any rank ever gave up a wait is poisoned for good: the ranks' call numbers may no longer agree,
    // and a stale partial row of the abandoned call would pass for a fresh one. Every CTA reads the word here, before
    // anything is allocated or sent, and leaves; the host refuses further calls until the group is made anew.
    if (__syncthreads_or(*reinterpret_cast<volatile const uint32_t*>(a.ctrl + 2) != 0u ? 1 : 0)) {   // one answer per CTA
        if (tid == 0 && blockIdx.x == 0) {
            report_status(a.status, 3);
            if (a.poison_host) *reinterpret_cast<volatile int*>(a.poison_host) = 1;
        }
        return;
    }
    // The waits inside the CTA (ring, accumulators) last as long as the epilogue warps wait for a peer: give them
    // twice the peer limit, so that the peer wait is the one that runs out first and names the cause.
    const unsigned long long pipe_limit = 2ull * a.wait_limit_ns;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar(FULL + s), 1);
            mbar_init(bar(EMPTY + s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar(ACC_FULL + s), 1);
            mbar_init(bar(ACC_EMPTY + s), 4);   // one arrive per epilogue warp
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

    if (warp == 0) {
        // ================================ TMA producer =================================
        if (lane == 0) {
            int it = 0;  // ring position, counted over all tiles of this CTA
            for (int vt = blockIdx.x; vt < n_vt; vt += gridDim.x) {
                const int tile = vt / S, slice = vt - tile * S;
                const int m0 = (tile / tiles_n) * TM, n0 = (tile % tiles_n) * TN;
                const int kb0 = slice * kblocks / S, kb1 = (slice + 1) * kblocks / S;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = static_cast<uint32_t>((it / kStages) & 1);
                    if (!mbar_wait(bar(EMPTY + s), ph ^ 1u, give_up, pipe_limit)) goto producer_done;
                    mbar_expect_tx(bar(FULL + s), TL::kStageBytes);
                    const uint32_t a_dst = smem_u32(smem + kOffRing + s * TL::kStageBytes), b_dst = a_dst + kABytes;
                    tma_load_2d(a_dst, &map_a, kb * TK, m0, bar(FULL + s));
                    if (B_KMAJOR) {
                        tma_load_2d(b_dst, &map_b, kb * TK, n0, bar(FULL + s));          // [TN rows of x2^T x 64 k]
                    } else {
#pragma unroll
                        for (int nb = 0; nb < TN / 64; ++nb)                              // boxes of 64 columns x 64 k
                            tma_load_2d(b_dst + nb * TK * 128, &map_b, n0 + nb * 64, kb * TK, bar(FULL + s));
                    }
                }
            }
        producer_done:;
        }
    } else if (warp == 1) {
        // ================================ MMA issuer ===================================
        if (lane == 0) {
            const uint32_t idesc = make_idesc(TM, TN, BF16 ? 1 : 0, B_KMAJOR ? 0 : 1);
            int it = 0, nt = 0;
            for (int vt = blockIdx.x; vt < n_vt; vt += gridDim.x, ++nt) {
                const int slice = vt % S;
                const int kb0 = slice * kblocks / S, kb1 = (slice + 1) * kblocks / S;
                const int acc = nt & 1;
                if (!mbar_wait(bar(ACC_EMPTY + acc), static_cast<uint32_t>(((nt >> 1) & 1) ^ 1), give_up, pipe_limit)) break;
                tc_fence_after();
                bool ok = true;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(bar(FULL + s), static_cast<uint32_t>((it / kStages) & 1), give_up, pipe_limit)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + kOffRing + s * TL::kStageBytes), b_addr = a_addr + kABytes;
#pragma unroll
                    for (int t = 0; t < TK / 16; ++t) {
                        const uint64_t ad = make_desc(a_addr + t * 32, 0, 1024);   // K-major: 16 k = 32 bytes inside the swizzled row
                        const uint64_t bd = B_KMAJOR ? make_desc(b_addr + t * 32, 0, 1024)
                                                     : make_desc(b_addr + t * 16 * 128, TK * 128, 1024);  // MN-major: 16 k = 16 rows; next 64 columns 8 KB on
                        umma(tmem_base + acc * kTileCap, ad, bd, idesc, (kb > kb0 || t > 0) ? 1u : 0u);
                    }
                    umma_commit(bar(EMPTY + s));
                }
                if (!ok) break;
                umma_commit(bar(ACC_FULL + acc));
            }
        }
    } else {
        // ================================ epilogue warps ================================
        constexpr int LPR = TL::kLanesPerRow, RPI = TL::kRowsPerInstr;
        const int quarter = warp & 3;                    // the TMEM lane quarter this warp may touch
        const int sub = lane / LPR, cl = lane % LPR;     // row inside one warp-wide access, 4-column group inside the row
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        float* tbuf = reinterpret_cast<float*>(smem + kOffT) + quarter * 32 * kRowPadMax;
        bool ok = true;
        int nt = 0;
        // ---- first pass: every tile of this CTA, product -> partial rows into the staging areas -----------------------
        for (int vt = blockIdx.x; ok && vt < n_vt; vt += gridDim.x, ++nt) {
            const int tile = vt / S, slice = vt - tile * S;
            const int acc = nt & 1;
            const int m0 = (tile / tiles_n) * TM, n0 = (tile % tiles_n) * TN;
            if (!warp_wait(bar(ACC_FULL + acc), static_cast<uint32_t>((nt >> 1) & 1), give_up, pipe_limit)) {
                ok = false;
                break;
            }
            tc_fence_after();
#pragma unroll
            for (int c4 = 0; c4 < TN / 32; ++c4) {
                uint32_t u[32];
                tmem_ld32(lane_base + acc * kTileCap + c4 * 32, u);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; c += 4) {
                    float4 v = make_float4(__uint_as_float(u[c]), __uint_as_float(u[c + 1]), __uint_as_float(u[c + 2]), __uint_as_float(u[c + 3]));
                    *reinterpret_cast<float4*>(tbuf + lane * TL::kRowPad + c4 * 32 + c) = v;   // thread = row of the tile
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(ACC_EMPTY + acc));   // the accumulator may be overwritten by the tile after next
            // whole rows now: a lane owns columns 4 cl .. 4 cl + 3 of the rows sub, sub + RPI, ... of this warp's slab
            const int col = n0 + 4 * cl;
            float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (a.bias != nullptr && col < a.N && slice == 0) {   // the bias once per rank: with the first slice of K
                if (BF16) {
                    const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(a.bias) + col;
                    bias4 = make_float4(__bfloat162float(b[0]), __bfloat162float(b[1]), __bfloat162float(b[2]), __bfloat162float(b[3]));
                } else {
                    const __half* b = static_cast<const __half*>(a.bias) + col;
                    bias4 = make_float4(__half2float(b[0]), __half2float(b[1]), __half2float(b[2]), __half2float(b[3]));
                }
            }
            const int rows_here = min(32, a.M - (m0 + quarter * 32));   // rows of this warp's slab that exist
            const size_t slot = partial_slot<TN>(buf, W, a.rank * S + slice, mt, tile);
            const int owner = tile % a.world;
            if (col < a.N) {
                for (int rr = sub; rr < rows_here; rr += RPI) {
                    float4 v = *reinterpret_cast<const float4*>(tbuf + rr * TL::kRowPad + 4 * cl);
                    v.x += bias4.x;
                    v.y += bias4.y;
                    v.z += bias4.z;
                    v.w += bias4.w;
                    const size_t off = slot + static_cast<size_t>(quarter * 32 + rr) * TL::kPartialRowBytes + 16 * cl;
                    if (a.two_shot) {
                        st_pair(a.peer_stage[owner] + off, __float_as_uint(v.x), __float_as_uint(v.y), epoch);
                        st_pair(a.peer_stage[owner] + off + TN * 4, __float_as_uint(v.z), __float_as_uint(v.w), epoch);
                    } else {
                        for (int p = 0; p < a.world; ++p) {
                            st_pair(a.peer_stage[p] + off, __float_as_uint(v.x), __float_as_uint(v.y), epoch);
                            st_pair(a.peer_stage[p] + off + TN * 4, __float_as_uint(v.z), __float_as_uint(v.w), epoch);
                        }
                    }
                }
            }
            __syncwarp();   // the transpose buffer is rewritten by the next tile
        }

        // ---- second pass: add the partials of all ranks in rank order (two-shot: only for the tiles this rank owns) ----
        // The rows of a tile are dealt out to the four warps: warp q takes rows q, q + 4, q + 8, ...; entry e of that
        // list is row q + 4 e, and one warp-wide access covers RPI consecutive entries.
        const unsigned char* my_stage = a.peer_stage[a.rank];
        constexpr int RB = 8;   // accesses in flight per warp
        for (int vt = blockIdx.x; ok && vt < n_vt; vt += gridDim.x) {
            const int tile = vt / S;
            if (vt - tile * S != 0) continue;   // the CTA with the first slice of a tile adds the sources up (sharing the adding among the S CTAs measured no faster)
            if (a.two_shot && tile % a.world != a.rank) continue;
            const int m0 = (tile / tiles_n) * TM, n0 = (tile % tiles_n) * TN;
            const int col = n0 + 4 * cl;
            const int rows_valid = min(TM, a.M - m0);
            for (int e0 = 0; ok && quarter + 4 * e0 < rows_valid; e0 += RB * RPI) {
                float4 sum[RB];
#pragma unroll
                for (int i = 0; i < RB; ++i) sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int r = 0; ok && r < W; ++r) {
                    const unsigned char* src = my_stage + partial_slot<TN>(buf, W, r, mt, tile) + 16 * cl;
                    uint32_t w[RB][4];
                    unsigned long long t0 = 0;
                    for (;;) {   // until every word of the batch carries this call's number
                        bool here = true;
                        if (col < a.N) {
#pragma unroll
                            for (int i = 0; i < RB; ++i) {
                                const int row = quarter + 4 * (e0 + i * RPI + sub);
                                if (row < rows_valid) {
                                    const unsigned char* q = src + static_cast<size_t>(row) * TL::kPartialRowBytes;
                                    here &= ld_pair(q, epoch, w[i][0], w[i][1]);
                                    here &= ld_pair(q + TN * 4, epoch, w[i][2], w[i][3]);
                                }
                            }
                        }
                        if (__all_sync(0xffffffffu, here ? 1 : 0)) break;
                        if (!__all_sync(0xffffffffu, poll_again(t0, give_up, a.wait_limit_ns) ? 1 : 0)) {   // the warp stops as one
                            ok = false;
                            break;
                        }
                    }
                    if (!ok) break;
#pragma unroll
                    for (int i = 0; i < RB; ++i) {
                        if (quarter + 4 * (e0 + i * RPI + sub) < rows_valid) {
                            sum[i].x += __uint_as_float(w[i][0]);
                            sum[i].y += __uint_as_float(w[i][1]);
                            sum[i].z += __uint_as_float(w[i][2]);
                            sum[i].w += __uint_as_float(w[i][3]);
                        }
                    }
                }
                if (!ok || col >= a.N) continue;
#pragma unroll
                for (int i = 0; i < RB; ++i) {
                    const int row = quarter + 4 * (e0 + i * RPI + sub);
                    if (row < rows_valid) {
                        uint2 packed;
                        if (BF16) {
                            __nv_bfloat162 lo = __floats2bfloat162_rn(sum[i].x, sum[i].y), hi = __floats2bfloat162_rn(sum[i].z, sum[i].w);
                            packed.x = *reinterpret_cast<uint32_t*>(&lo);
                            packed.y = *reinterpret_cast<uint32_t*>(&hi);
                        } else {
                            __half2 lo = __floats2half2_rn(sum[i].x, sum[i].y), hi = __floats2half2_rn(sum[i].z, sum[i].w);
                            packed.x = *reinterpret_cast<uint32_t*>(&lo);
                            packed.y = *reinterpret_cast<uint32_t*>(&hi);
                        }
                        *reinterpret_cast<uint2*>(static_cast<unsigned char*>(a.out) + (static_cast<int64_t>(m0 + row) * a.out_s0 + col) * 2) = packed;
                        if (a.two_shot) {   // and the finished rows to every other rank's result area
                            const size_t roff = result_slot<TN>(buf, a.max_tiles, tile) + static_cast<size_t>(row) * TL::kResultRowBytes + 16 * cl;
                            for (int p = 0; p < a.world; ++p)
                                if (p != a.rank) st_pair(a.peer_result[p] + roff, packed.x, packed.y, epoch);
                        }
                    }
                }
            }
        }

        // ---- two-shot only, third pass: the tiles other ranks added up arrive in this rank's result area -----------
        if (a.two_shot) {
            const unsigned char* my_result = a.peer_result[a.rank];
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                if (tile % a.world == a.rank) continue;   // written straight to out above
                const int m0 = (tile / tiles_n) * TM, n0 = (tile % tiles_n) * TN;
                const int col = n0 + 4 * cl;
                const int rows_valid = min(TM, a.M - m0);
                const unsigned char* src = my_result + result_slot<TN>(buf, a.max_tiles, tile) + 16 * cl;
                for (int e0 = 0; ok && quarter + 4 * e0 < rows_valid; e0 += RB * RPI) {
                    uint32_t w[RB][2];
                    unsigned long long t0 = 0;
                    for (;;) {
                        bool here = true;
                        if (col < a.N) {
#pragma unroll
                            for (int i = 0; i < RB; ++i) {
                                const int row = quarter + 4 * (e0 + i * RPI + sub);
                                if (row < rows_valid) here &= ld_pair(src + static_cast<size_t>(row) * TL::kResultRowBytes, epoch, w[i][0], w[i][1]);
                            }
                        }
                        if (__all_sync(0xffffffffu, here ? 1 : 0)) break;
                        if (!__all_sync(0xffffffffu, poll_again(t0, give_up, a.wait_limit_ns) ? 1 : 0)) {
                            ok = false;
                            break;
                        }
                    }
                    if (!ok || col >= a.N) continue;
#pragma unroll
                    for (int i = 0; i < RB; ++i) {
                        const int row = quarter + 4 * (e0 + i * RPI + sub);
                        if (row < rows_valid)
                            *reinterpret_cast<uint2*>(static_cast<unsigned char*>(a.out) + (static_cast<int64_t>(m0 + row) * a.out_s0 + col) * 2) =
                                make_uint2(w[i][0], w[i][1]);
                    }
                }
            }
        }
    }

    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(a.ctrl + 1, 1u) == gridDim.x - 1) {   // the last CTA of this launch
            a.ctrl[1] = 0;
            *reinterpret_cast<volatile uint32_t*>(a.ctrl) = epoch;
            __threadfence();
        }
    }
    if (*give_up) {
        if (tid == 0) {
            report_status(a.status, 3);
            // Make the give-up sticky on every rank: a plain store into each peer's control words (and the own ones).
            for (int p = 0; p < a.world; ++p) *reinterpret_cast<volatile uint32_t*>(a.peer_ctrl[p] + 2) = 1u;
            if (a.poison_host) *reinterpret_cast<volatile int*>(a.poison_host) = 1;
            __threadfence_system();
        }
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

// 2-D view [inner, outer] of a row-major matrix with `ld` elements between rows; box = 64 inner elements x box_outer rows.
bool make_map_2d(CUtensorMap* map, const void* base, int64_t inner, int64_t outer, int64_t ld, int box_outer, bool bf16) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_outer)};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace

// Capacity is counted in 128 x 128 tiles whatever width the kernel then picks.
int matmul_allreduce_tiles(int64_t M, int64_t N) { return static_cast<int>(((M + TM - 1) / TM) * ((N + kTileCap - 1) / kTileCap)); }

// One rank's area: partial tiles [2 halves][world sources][max_tiles] (fp32 with arrival marks, 128 KB each), finished
// tiles [2][max_tiles] (16-bit with arrival marks, 64 KB each, two-shot form) and four control words (calls finished,
// CTAs of the running call that have left, poisoned, spare).
MarLayout matmul_allreduce_layout(int world, int max_tiles) {
    MarLayout l;
    size_t off = 0;
    l.stage_off = off;
    off += static_cast<size_t>(2) * world * max_tiles * kPartialCapBytes;
    l.result_off = off;
    off += static_cast<size_t>(2) * max_tiles * kResultCapBytes;
    l.ctrl_off = off;
    off += 4 * sizeof(uint32_t);
    l.bytes = (off + 255) / 256 * 256;
    return l;
}

const char* launch_matmul_allreduce(const MatmulAllReduceArgs& a, int sm_count, int max_smem, cudaStream_t st) {
    if (a.M == 0 || a.N == 0) return nullptr;
    if (kSmemBytes > max_smem) return "not enough shared memory per block on this device";
    if (a.dt != Dt::F16 && a.dt != Dt::BF16) return "x1 and x2 must be float16 or bfloat16";
    if (a.M >= (1ll << 31) || a.N >= (1ll << 31) || a.K >= (1ll << 31)) return "matrix extents must fit 31 bits";
    if (a.N % 4 != 0) return "the output width must be a multiple of 4";
    auto al = [](const void* p, int64_t ld) { return reinterpret_cast<uintptr_t>(p) % 16 == 0 && (ld * 2) % 16 == 0; };
    if (!al(a.x1, a.x1_ld) || !al(a.x2, a.x2_ld) || !al(a.out, a.out_s0 * 1) || (a.out_s0 * 2) % 8 != 0)
        return "x1, x2 and out need 16-byte aligned bases and row pitches that are multiples of 16 bytes";
    const bool bf16 = a.dt == Dt::BF16;
    // Tile width: 128 when there are enough 128-wide tiles to occupy the SMs; else narrower, so that more CTAs stream
    // the weights (32 needs x2 K-major: an MN-major tile is made of 64-column boxes). force_tile_width overrides the choice.
    const int64_t row_tiles = (a.M + TM - 1) / TM;
    int tn = 128;
    if (row_tiles * ((a.N + 127) / 128) * 2 <= sm_count) tn = (a.x2_kmajor && row_tiles * ((a.N + 63) / 64) * 2 <= sm_count * 2) ? 32 : 64;
    {
        const int f = a.force_tile_width;
        if (f == 128 || f == 64 || (f == 32 && a.x2_kmajor)) tn = f;
    }
    // Split-K, for a group of one rank (a plain product) whose output has too few 128-wide tiles for the SMs: instead of
    // narrower tiles (every CTA then re-reads all of x1 from L2: 128 CTAs x 512 KB at M 64, K 4096) several CTAs share a
    // 128-wide tile and a slice of K each; the slices are added in the staging area like the partials of ranks.
    int splits = 1;
    if (a.world == 1 && a.force_tile_width == 0) {
        const int64_t tiles128 = row_tiles * ((a.N + 127) / 128);
        const int64_t kblocks = (a.K + TK - 1) / TK;
        int64_t sp = std::min<int64_t>(std::min<int64_t>(sm_count / std::max<int64_t>(tiles128, 1), kblocks / 4), std::min<int64_t>(a.max_tiles / std::max<int64_t>(tiles128, 1), 8));
        if (tiles128 * 2 <= sm_count && sp >= 2) {
            splits = static_cast<int>(sp);
            tn = 128;
        }
    }
    const int am = ((tn < 128 || splits > 1) && a.M <= 64) ? 64 : 128;   // rows of x1 a ring stage holds
    CUtensorMap ma, mb;
    if (!make_map_2d(&ma, a.x1, a.K, a.M, a.x1_ld, am, bf16)) return "cuTensorMapEncodeTiled failed for x1";
    const bool okb = a.x2_kmajor ? make_map_2d(&mb, a.x2, a.K, a.N, a.x2_ld, tn, bf16) : make_map_2d(&mb, a.x2, a.N, a.K, a.x2_ld, TK, bf16);
    if (!okb) return "cuTensorMapEncodeTiled failed for x2";
    const int n_tiles = static_cast<int>(row_tiles * ((a.N + tn - 1) / tn));
    const int grid = std::min(n_tiles * splits, sm_count);
    MatmulAllReduceArgs b = a;
    b.k_splits = splits;
    auto go = [&](auto kern) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        kern<<<grid, kThreads, kSmemBytes, st>>>(ma, mb, b);
    };
    auto pick = [&](auto bf) {
        constexpr bool B = decltype(bf)::value;
        if (a.x2_kmajor) {
            if (tn == 128) { if (am == 64) go(matmul_allreduce_kernel<B, true, 128, 64>); else go(matmul_allreduce_kernel<B, true, 128, 128>); }
            else if (tn == 64) { if (am == 64) go(matmul_allreduce_kernel<B, true, 64, 64>); else go(matmul_allreduce_kernel<B, true, 64, 128>); }
            else { if (am == 64) go(matmul_allreduce_kernel<B, true, 32, 64>); else go(matmul_allreduce_kernel<B, true, 32, 128>); }
        } else {
            if (tn == 128) { if (am == 64) go(matmul_allreduce_kernel<B, false, 128, 64>); else go(matmul_allreduce_kernel<B, false, 128, 128>); }
            else if (am == 64) go(matmul_allreduce_kernel<B, false, 64, 64>);
            else go(matmul_allreduce_kernel<B, false, 64, 128>);
        }
    };
    if (bf16)
        pick(std::true_type{});
    else
        pick(std::false_type{});
    return nullptr;
}

}  // namespace k
}  // namespace b200
