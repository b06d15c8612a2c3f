// diopiMatmulAllReduce: out = sum over the ranks of a group of (x1_r @ x2_r + bias_r), the row-parallel linear layer
// that follows attention in a head-sharded model, as ONE kernel per rank. The reference forwards this call to the
// vendor's aclnnMatmulAllReduce (impl/ascend/functions_ext/matmul_all_reduce.cpp:13-17,
// impl/ascend_npu/diopi_impl/functions_ext/matmul_all_reduce.cpp:12-17; signature proto/include/diopi/functions_ext.h:664-665);
// there is no NVIDIA implementation to replace.
//
// Per rank, a persistent grid (one CTA per SM at most) walks the 128 x 128 output tiles:
//   warp 0 (one lane)  TMA: x1 tile [128 x 64] and x2 tile [64 x 128] (or [128 x 64] when x2 is given K-major) into a
//                      4-stage ring, 128-byte swizzle, no multicast
//   warp 1 (one lane)  tcgen05.mma M128 N128 K16, fp32 accumulators in TMEM (two accumulator buffers, so the epilogue
//                      of one tile overlaps the products of the next)
//   warps 2-5          epilogue: TMEM -> registers (+ bias) -> shared memory (transpose to whole rows) -> plain 16-byte
//                      stores of the fp32 partial tile into EVERY rank's staging area over NVLink (peer pointers, this
//                      rank's own copy included), then one release-store of a flag per destination and warp
// and, once a CTA has sent all its tiles, the same warps wait for the flags of all ranks for each of those tiles
// (acquire loads of this rank's own memory, bounded by a time limit), add the partials in rank order in fp32 and
// write the tile of `out` once. Every rank adds the same numbers in the same order: all ranks get identical bits.
// This is the one-shot form (each rank receives world x the output in fp32): right for decode-sized outputs, where
// latency counts; the staging area fixes the largest output (tiles) a group can take.
//
// Waiting on another rank's kernel: flags carry the call's sequence number (kept in device memory, no reset between
// calls, nothing per call from the host: a captured launch can be replayed) and the staging
// area is double-buffered; a rank cannot run two calls ahead of a peer, because it needs that peer's flags of the
// call in between. A wait that runs out (a peer that never calls) raises the status word (code 3) and the kernel
// returns with TMEM freed.
#include <cuda.h>

#include <mutex>

#include "dev_util.cuh"
#include "sm100_ptx.cuh"

namespace b200 {
namespace k {

namespace {

using namespace sm100;  // NOLINT

constexpr int TM = 128, TN = 128, TK = 64;   // tile of the output, K step of one ring stage
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr int kABytes = TM * TK * 2;          // 16 KB
constexpr int kBBytes = TN * TK * 2;          // 16 KB
constexpr int kRowPad = TN + 4;               // floats per row of the transpose buffer (16-byte stores without bank conflicts)
constexpr int kOffA = 0;
constexpr int kOffB = kOffA + kStages * kABytes;
constexpr int kOffT = kOffB + kStages * kBBytes;               // transpose buffer: 4 warps x 32 rows x kRowPad floats
constexpr int kTBytes = 4 * 32 * kRowPad * 4;
constexpr int kOffBar = kOffT + kTBytes;
enum Bar { FULL = 0, EMPTY = kStages, ACC_FULL = 2 * kStages, ACC_EMPTY = 2 * kStages + 2, kNumBars = 2 * kStages + 4 };
constexpr int kOffTmemSlot = kOffBar + kNumBars * 8;
constexpr int kOffFlag = kOffTmemSlot + 8;
constexpr int kSmemBytes = kOffFlag + 8;
constexpr uint32_t kTmemCols = 256;           // two accumulators of 128 fp32 columns

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <bool BF16, bool B_KMAJOR>
__global__ void __launch_bounds__(kThreads, 1) matmul_allreduce_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                                        const MatmulAllReduceArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffTmemSlot);
    volatile int* give_up = reinterpret_cast<volatile int*>(smem + kOffFlag);
    auto bar = [&](int i) { return smem_u32(&bars[i]); };
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_n = (a.N + TN - 1) / TN;
    const int n_tiles = ((a.M + TM - 1) / TM) * tiles_n;
    const int kblocks = (a.K + TK - 1) / TK;
    // The call's sequence number lives in device memory (the number of calls this group has finished, plus one) and is
    // advanced by the last CTA to leave: the host passes nothing that changes from call to call, so a captured launch
    // can be replayed. Every CTA reads it here, before any CTA of this launch can have left.
    const uint32_t epoch = *reinterpret_cast<volatile const uint32_t*>(a.ctrl) + 1u;
    const int buf = static_cast<int>(epoch & 1u);   // which half of the staging area this call uses

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
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                const int m0 = (tile / tiles_n) * TM, n0 = (tile % tiles_n) * TN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = static_cast<uint32_t>((it / kStages) & 1);
                    if (!mbar_wait(bar(EMPTY + s), ph ^ 1u, give_up)) goto producer_done;
                    mbar_expect_tx(bar(FULL + s), kABytes + kBBytes);
                    tma_load_2d(smem_u32(smem + kOffA + s * kABytes), &map_a, kb * TK, m0, bar(FULL + s));
                    if (B_KMAJOR) {
                        tma_load_2d(smem_u32(smem + kOffB + s * kBBytes), &map_b, kb * TK, n0, bar(FULL + s));
                    } else {  // two boxes of 64 columns x 64 k
                        tma_load_2d(smem_u32(smem + kOffB + s * kBBytes), &map_b, n0, kb * TK, bar(FULL + s));
                        tma_load_2d(smem_u32(smem + kOffB + s * kBBytes + TK * 128), &map_b, n0 + 64, kb * TK, bar(FULL + s));
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
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++nt) {
                const int acc = nt & 1;
                if (!mbar_wait(bar(ACC_EMPTY + acc), static_cast<uint32_t>(((nt >> 1) & 1) ^ 1), give_up)) break;
                tc_fence_after();
                bool ok = true;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(bar(FULL + s), static_cast<uint32_t>((it / kStages) & 1), give_up)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + kOffA + s * kABytes), b_addr = smem_u32(smem + kOffB + s * kBBytes);
#pragma unroll
                    for (int t = 0; t < TK / 16; ++t) {
                        const uint64_t ad = make_desc(a_addr + t * 32, 0, 1024);   // K-major: 16 k = 32 bytes inside the swizzled row
                        const uint64_t bd = B_KMAJOR ? make_desc(b_addr + t * 32, 0, 1024)
                                                     : make_desc(b_addr + t * 16 * 128, TK * 128, 1024);  // MN-major: 16 k = 16 rows; next 64 columns 8 KB on
                        umma(tmem_base + acc * TN, ad, bd, idesc, (kb > 0 || t > 0) ? 1u : 0u);
                    }
                    umma_commit(bar(EMPTY + s));
                }
                if (!ok) break;
                umma_commit(bar(ACC_FULL + acc));
            }
        }
    } else {
        // ================================ epilogue warps ================================
        const int quarter = warp & 3;                    // the TMEM lane quarter this warp may touch
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        float* tbuf = reinterpret_cast<float*>(smem + kOffT) + quarter * 32 * kRowPad;
        const size_t tile_floats = static_cast<size_t>(TM) * TN;
        const size_t src_off = (static_cast<size_t>(buf) * a.world + a.rank) * a.max_tiles; // tile slots of (buf, src = this rank)
        bool ok = true;
        int nt = 0;
        for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++nt) {
            const int acc = nt & 1;
            const int m0 = (tile / tiles_n) * TM, n0 = (tile % tiles_n) * TN;
            if (!warp_wait(bar(ACC_FULL + acc), static_cast<uint32_t>((nt >> 1) & 1), give_up)) {
                ok = false;
                break;
            }
            tc_fence_after();
#pragma unroll
            for (int c4 = 0; c4 < TN / 32; ++c4) {
                uint32_t u[32];
                tmem_ld32(lane_base + acc * TN + c4 * 32, u);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; c += 4) {
                    float4 v = make_float4(__uint_as_float(u[c]), __uint_as_float(u[c + 1]), __uint_as_float(u[c + 2]), __uint_as_float(u[c + 3]));
                    *reinterpret_cast<float4*>(tbuf + lane * kRowPad + c4 * 32 + c) = v;   // thread = row of the tile
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(ACC_EMPTY + acc));   // the accumulator may be overwritten by the tile after next
            // whole rows now: lane l owns columns 4l .. 4l+3 of each of this warp's 32 rows
            const int col = n0 + 4 * lane;
            float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (a.bias != nullptr && col < a.N) {
                if (BF16) {
                    const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(a.bias) + col;
                    bias4 = make_float4(__bfloat162float(b[0]), __bfloat162float(b[1]), __bfloat162float(b[2]), __bfloat162float(b[3]));
                } else {
                    const __half* b = static_cast<const __half*>(a.bias) + col;
                    bias4 = make_float4(__half2float(b[0]), __half2float(b[1]), __half2float(b[2]), __half2float(b[3]));
                }
            }
            const int rows_here = min(32, a.M - (m0 + quarter * 32));   // rows of this warp's slab that exist
            for (int rr = 0; rr < rows_here; ++rr) {
                float4 v = *reinterpret_cast<const float4*>(tbuf + rr * kRowPad + 4 * lane);
                v.x += bias4.x;
                v.y += bias4.y;
                v.z += bias4.z;
                v.w += bias4.w;
                const size_t off = (src_off + tile) * tile_floats + static_cast<size_t>(quarter * 32 + rr) * TN + 4 * lane;
                if (col < a.N) {
                    for (int p = 0; p < a.world; ++p) *reinterpret_cast<float4*>(a.peer_stage[p] + off) = v;
                }
            }
            // This warp's 32 rows are on their way: one flag per destination says "rows 32q .. 32q+31 of tile `tile` from
            // rank `rank` are there". A flag per warp, not per tile, so that no warp ever waits for another here.
            __threadfence_system();
            __syncwarp();
            if (lane < a.world)
                st_release_sys(a.peer_flag[lane] + ((static_cast<size_t>(buf) * a.world + a.rank) * a.max_tiles + tile) * 4 + quarter, epoch);
        }

        // ---- second pass over this CTA's tiles: add the partials of all ranks, write out ------------------------
        const float* my_stage = a.peer_stage[a.rank];
        const uint32_t* my_flag = a.peer_flag[a.rank];
        for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
            const int m0 = (tile / tiles_n) * TM, n0 = (tile % tiles_n) * TN;
            // The rows of a tile are dealt out to the four warps whatever quarter sent them, so every warp waits for all
            // the flags of the tile: lane 4r + q for quarter q of rank r.
            bool mine = true;
            if (lane < 4 * a.world) {
                const uint32_t* f = my_flag + ((static_cast<size_t>(buf) * a.world + (lane >> 2)) * a.max_tiles + tile) * 4 + (lane & 3);
                if (ld_acquire_sys(f) != epoch) {
                    const unsigned long long t0 = global_ns();
                    uint32_t spins = 0;
                    while (ld_acquire_sys(f) != epoch) {
                        if ((++spins & 0x3fu) == 0) {
                            if (*give_up || global_ns() - t0 > kWaitLimitNs) {
                                *give_up = 1;
                                mine = false;
                                break;
                            }
                        }
                    }
                }
            }
            if (!__all_sync(0xffffffffu, mine ? 1 : 0)) {
                ok = false;
                break;
            }
            const int col = n0 + 4 * lane;
            const int rows_valid = min(TM, a.M - m0);
            if (col < a.N) {
                constexpr int RB = 8;   // rows in flight per warp: 8 independent 16-byte loads per rank
                for (int row0 = quarter; row0 < rows_valid; row0 += 4 * RB) {
                    float4 sum[RB];
#pragma unroll
                    for (int i = 0; i < RB; ++i) sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int r = 0; r < a.world; ++r) {
                        const float* src = my_stage + ((static_cast<size_t>(buf) * a.world + r) * a.max_tiles + tile) * tile_floats + 4 * lane;
                        float4 v[RB];
#pragma unroll
                        for (int i = 0; i < RB; ++i) {
                            const int row = row0 + 4 * i;
                            v[i] = row < rows_valid ? __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(row) * TN)) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                        for (int i = 0; i < RB; ++i) {
                            sum[i].x += v[i].x;
                            sum[i].y += v[i].y;
                            sum[i].z += v[i].z;
                            sum[i].w += v[i].w;
                        }
                    }
#pragma unroll
                    for (int i = 0; i < RB; ++i) {
                        const int row = row0 + 4 * i;
                        if (row < rows_valid) {
                            unsigned char* dst = static_cast<unsigned char*>(a.out) + (static_cast<int64_t>(m0 + row) * a.out_s0 + col) * 2;
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
                            *reinterpret_cast<uint2*>(dst) = packed;
                        }
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
        if (tid == 0) report_status(a.status, 3);
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

int matmul_allreduce_tiles(int64_t M, int64_t N) { return static_cast<int>(((M + TM - 1) / TM) * ((N + TN - 1) / TN)); }

size_t matmul_allreduce_stage_bytes(int world, int max_tiles) {
    return static_cast<size_t>(2) * world * max_tiles * TM * TN * sizeof(float);
}
// flag words of the two staging halves, then two control words (calls finished, CTAs of the running call that left)
size_t matmul_allreduce_flag_words(int world, int max_tiles) { return static_cast<size_t>(2) * world * max_tiles * 4; }
size_t matmul_allreduce_flag_bytes(int world, int max_tiles) { return (matmul_allreduce_flag_words(world, max_tiles) + 2) * sizeof(uint32_t); }

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
    CUtensorMap ma, mb;
    if (!make_map_2d(&ma, a.x1, a.K, a.M, a.x1_ld, TM, bf16)) return "cuTensorMapEncodeTiled failed for x1";
    const bool okb = a.x2_kmajor ? make_map_2d(&mb, a.x2, a.K, a.N, a.x2_ld, TN, bf16) : make_map_2d(&mb, a.x2, a.N, a.K, a.x2_ld, TK, bf16);
    if (!okb) return "cuTensorMapEncodeTiled failed for x2";
    const int n_tiles = matmul_allreduce_tiles(a.M, a.N);
    const int grid = std::min(n_tiles, sm_count);
    auto go = [&](auto kern) {
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        kern<<<grid, kThreads, kSmemBytes, st>>>(ma, mb, a);
    };
    if (bf16) {
        if (a.x2_kmajor) go(matmul_allreduce_kernel<true, true>); else go(matmul_allreduce_kernel<true, false>);
    } else {
        if (a.x2_kmajor) go(matmul_allreduce_kernel<false, true>); else go(matmul_allreduce_kernel<false, false>);
    }
    return nullptr;
}

}  // namespace k
}  // namespace b200
