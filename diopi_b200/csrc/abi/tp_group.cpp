// Tensor-parallel groups and diopiMatmulAllReduce.
//
// The reference's diopiMatmulAllReduce names its communicator by a string (an HCCL group created elsewhere by the
// Ascend run time; proto/include/diopi/functions_ext.h:653-665). Here a group is a set of ranks, one process and one
// GPU each, whose staging areas are mapped into each other's address space through CUDA IPC, so that the kernel can
// store its partial tiles straight into the peers' memory over NVLink. The consumer creates the group once:
//   diopiB200GroupCreate(name, rank, world, max_tiles, handle_out)   on every rank: allocates and exports the local area
//   (exchange the 64-byte handles by any means: torch.distributed, MPI, a file)
//   diopiB200GroupConnect(name, all_handles)                         on every rank: maps the peers' areas
// and then calls diopiMatmulAllReduce(..., group = name, ...) like the reference's backend does. The set-up entry
// points have no counterpart in the reference.
//
// Recovery rule. Every wait of the kernel on a peer is bounded (diopiB200GroupSetWaitLimit, 2 s by default). When one
// runs out on any rank (a peer that never made the call, or died), that rank reports status 3 and marks the group
// unusable on every rank; from then on diopiMatmulAllReduce on that group returns an error without launching on the
// rank that gave up, and on the others as soon as one of their kernels has seen the mark. The consumer then calls
// diopiB200GroupDestroy on every rank and sets the group up again.
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include "../kernels/kernels.hpp"
#include "common.hpp"

using namespace b200;  // NOLINT

namespace {

struct Group {
    int rank = 0, world = 1, max_tiles = 0, device = 0;
    bool connected = false;
    void* local = nullptr;                       // partial tiles, finished tiles, control words
    void* mapped[k::kMaxGroupRanks] = {nullptr}; // peers' areas as opened here (null for the own rank)
    unsigned char* stage[k::kMaxGroupRanks] = {nullptr};
    unsigned char* result[k::kMaxGroupRanks] = {nullptr};
    uint32_t* ctrl[k::kMaxGroupRanks] = {nullptr};
    int* poison = nullptr;                       // mapped pinned host word: a kernel of this rank found or made the group unusable
    unsigned long long wait_limit_ns = 2000000000ull;
    int form = 0;         // 0: chosen per call; 1: one-shot; 2: two-shot
    int tile_width = 0;   // 0: chosen per call; 128, 64, 32
};

std::mutex g_mu;
std::map<std::string, Group> g_groups;

void set_pointers(Group& g, int r, void* base) {
    const k::MarLayout l = k::matmul_allreduce_layout(g.world, g.max_tiles);
    char* b = static_cast<char*>(base);
    g.stage[r] = reinterpret_cast<unsigned char*>(b + l.stage_off);
    g.result[r] = reinterpret_cast<unsigned char*>(b + l.result_off);
    g.ctrl[r] = reinterpret_cast<uint32_t*>(b + l.ctrl_off);
}

void release(Group& g) {
    for (int r = 0; r < g.world; ++r)
        if (g.mapped[r]) cudaIpcCloseMemHandle(g.mapped[r]);
    if (g.local) cudaFree(g.local);
    if (g.poison) cudaFreeHost(g.poison);
    g = Group{};
}

bool sum_op(const char* s) {
    if (s == nullptr) return false;
    const char* want = "sum";
    for (int i = 0; i < 4; ++i) {
        const char c = static_cast<char>(s[i] >= 'A' && s[i] <= 'Z' ? s[i] - 'A' + 'a' : s[i]);
        if (c != want[i]) return false;
        if (c == '\0') break;
    }
    return true;
}

}  // namespace

static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the exported handle is documented as 64 bytes");

B200_EXPORT diopiError_t diopiB200GroupCreate(const char* group, int rank, int world, int64_t max_tiles, void* local_handle) {
    return guard("diopiB200GroupCreate", [&] {
        B200_REQUIRE(group != nullptr && group[0] != '\0', "the group needs a name");
        B200_REQUIRE(world >= 1 && world <= k::kMaxGroupRanks, "a group has 1 to %d ranks, got %d", k::kMaxGroupRanks, world);
        B200_REQUIRE(rank >= 0 && rank < world, "rank %d is outside a group of %d", rank, world);
        B200_REQUIRE(max_tiles >= 1 && max_tiles <= 65536, "max_tiles (128 x 128 output tiles per call) must be between 1 and 65536");
        B200_REQUIRE(local_handle != nullptr || world == 1, "local_handle must point to 64 bytes");
        std::lock_guard<std::mutex> lock(g_mu);
        B200_REQUIRE(g_groups.find(group) == g_groups.end(), "group '%s' exists already", group);
        Group g;
        g.rank = rank;
        g.world = world;
        g.max_tiles = static_cast<int>(max_tiles);
        B200_CUDA(cudaGetDevice(&g.device));
        const size_t bytes = k::matmul_allreduce_layout(world, g.max_tiles).bytes;
        B200_CUDA(cudaMalloc(&g.local, bytes));
        cudaError_t e = cudaMemset(g.local, 0, bytes);
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        if (e == cudaSuccess && local_handle != nullptr) {
            cudaIpcMemHandle_t h;
            e = cudaIpcGetMemHandle(&h, g.local);
            if (e == cudaSuccess) std::memcpy(local_handle, &h, sizeof(h));
        }
        if (e == cudaSuccess) {
            e = cudaHostAlloc(reinterpret_cast<void**>(&g.poison), 64, cudaHostAllocMapped);
            if (e == cudaSuccess) std::memset(g.poison, 0, 64);
        }
        if (e != cudaSuccess) {
            cudaFree(g.local);
            fail(diopiErrorOccurred, "cuda error while creating group '%s': %s", group, cudaGetErrorString(e));
        }
        set_pointers(g, rank, g.local);
        g.connected = world == 1;
        g_groups[group] = g;
    });
}

B200_EXPORT diopiError_t diopiB200GroupConnect(const char* group, const void* handles) {
    return guard("diopiB200GroupConnect", [&] {
        B200_REQUIRE(group != nullptr && handles != nullptr, "group and handles must not be null");
        std::lock_guard<std::mutex> lock(g_mu);
        auto it = g_groups.find(group);
        B200_REQUIRE(it != g_groups.end(), "no group named '%s'", group);
        Group& g = it->second;
        B200_REQUIRE(!g.connected, "group '%s' is connected already", group);
        B200_CUDA(cudaSetDevice(g.device));
        for (int r = 0; r < g.world; ++r) {
            if (r == g.rank) continue;
            cudaIpcMemHandle_t h;
            std::memcpy(&h, static_cast<const char*>(handles) + static_cast<size_t>(r) * sizeof(h), sizeof(h));
            void* p = nullptr;
            const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) fail(diopiErrorOccurred, "cannot map the staging area of rank %d of group '%s': %s", r, group, cudaGetErrorString(e));
            g.mapped[r] = p;
            set_pointers(g, r, p);
        }
        g.connected = true;
    });
}

B200_EXPORT diopiError_t diopiB200GroupSetOption(const char* group, const char* option, int64_t value) {
    return guard("diopiB200GroupSetOption", [&] {
        B200_REQUIRE(group != nullptr && option != nullptr, "group and option must not be null");
        std::lock_guard<std::mutex> lock(g_mu);
        auto it = g_groups.find(group);
        B200_REQUIRE(it != g_groups.end(), "no group named '%s'", group);
        Group& g = it->second;
        if (std::strcmp(option, "wait_limit_ms") == 0) {
            B200_REQUIRE(value >= 1 && value <= 600000, "wait_limit_ms must be between 1 and 600000 (10 min), got %ld", (long)value);
            g.wait_limit_ns = static_cast<unsigned long long>(value) * 1000000ull;
        } else if (std::strcmp(option, "form") == 0) {
            B200_REQUIRE(value >= 0 && value <= 2, "form must be 0 (chosen per call), 1 (one-shot) or 2 (two-shot), got %ld", (long)value);
            g.form = static_cast<int>(value);
        } else if (std::strcmp(option, "tile_width") == 0) {
            B200_REQUIRE(value == 0 || value == 128 || value == 64 || value == 32, "tile_width must be 0 (chosen per call), 128, 64 or 32, got %ld", (long)value);
            g.tile_width = static_cast<int>(value);
        } else {
            fail(diopiErrorOccurred, "unknown group option '%s'; known: wait_limit_ms, form, tile_width", option);
        }
    });
}

B200_EXPORT diopiError_t diopiB200GroupDestroy(const char* group) {
    return guard("diopiB200GroupDestroy", [&] {
        B200_REQUIRE(group != nullptr, "group must not be null");
        std::lock_guard<std::mutex> lock(g_mu);
        auto it = g_groups.find(group);
        B200_REQUIRE(it != g_groups.end(), "no group named '%s'", group);
        cudaDeviceSynchronize();
        release(it->second);
        g_groups.erase(it);
    });
}

// proto/include/diopi/functions_ext.h:664-665. out [.., N] = sum over the group's ranks of (x1 [.., K] @ x2 [K, N] + bias [N]).
// reduce_op must be "sum"; comm_turn and stream_mode are tuning knobs of the vendor's library and are not read.
B200_EXPORT diopiError_t diopiMatmulAllReduce(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t x1, diopiConstTensorHandle_t x2,
                                              diopiConstTensorHandle_t bias, const char* group, const char* reduce_op, int64_t /*comm_turn*/,
                                              int64_t /*stream_mode*/) {
    return guard("diopiMatmulAllReduce", [&] {
        TensorView o = view_of(out, "out"), av = view_of(x1, "x1"), bv = view_of(x2, "x2");
        TensorView cv = view_of(bias, "bias", /*optional=*/true);
        if (!sum_op(reduce_op)) fail(diopiNoImplement, "reduce_op '%s' is not implemented; only \"sum\" is", reduce_op ? reduce_op : "(null)");
        k::MatmulAllReduceArgs a{};
        if (av.dtype == diopi_dtype_float16)
            a.dt = k::Dt::F16;
        else if (av.dtype == diopi_dtype_bfloat16)
            a.dt = k::Dt::BF16;
        else
            fail(diopiDtypeNotSupported, "'x1' has dtype %s; supported: float16, bfloat16", dtype_name(av.dtype));
        B200_REQUIRE(bv.dtype == av.dtype && o.dtype == av.dtype && (!cv.defined || cv.dtype == av.dtype), "x1, x2, bias and out must share a dtype");
        B200_REQUIRE(av.ndim >= 2 && av.ndim <= 3 && bv.ndim == 2 && o.ndim == av.ndim, "x1 and out must have 2 or 3 dims, x2 two");
        const int64_t K = av.shape[av.ndim - 1], N = bv.shape[1];
        int64_t M = 1;
        for (int i = 0; i < av.ndim - 1; ++i) {
            B200_REQUIRE(o.shape[i] == av.shape[i], "'out' must have the leading dims of 'x1'");
            M *= av.shape[i];
        }
        B200_REQUIRE(K > 0, "the contraction length must not be 0");
        B200_REQUIRE(bv.shape[0] == K, "'x2' is [%ld, %ld] but 'x1' has %ld columns", (long)bv.shape[0], (long)bv.shape[1], (long)K);
        B200_REQUIRE(o.shape[o.ndim - 1] == N, "'out' must have %ld columns", (long)N);
        if (cv.defined) B200_REQUIRE(cv.numel == N && cv.contiguous(), "'bias' must be a dense vector of %ld elements", (long)N);
        // rows of x1 and out: dense last dim; a 3-D tensor must collapse to rows with one pitch
        auto row_pitch = [&](const TensorView& t, const char* name) -> int64_t {
            B200_REQUIRE(t.shape[t.ndim - 1] == 1 || t.stride[t.ndim - 1] == 1, "the last dim of '%s' must be dense", name);
            const int64_t p = t.stride[t.ndim - 2];
            if (t.ndim == 3) B200_REQUIRE(t.shape[0] == 1 || t.stride[0] == p * t.shape[1], "'%s' must be a stack of rows with one pitch", name);
            return p;
        };
        a.x1_ld = row_pitch(av, "x1");
        a.out_s0 = row_pitch(o, "out");
        if (bv.stride[1] == 1 || N == 1) {
            a.x2_kmajor = false;
            a.x2_ld = bv.stride[0];
        } else if (bv.stride[0] == 1) {
            a.x2_kmajor = true;   // a transposed view of a [N, K] weight
            a.x2_ld = bv.stride[1];
        } else {
            fail(diopiErrorOccurred, "'x2' must be dense along one of its dims");
        }
        B200_REQUIRE(group != nullptr, "group must not be null");
        cudaStream_t st = stream_of(ctx);
        const DeviceInfo& di = device_info();
        {
            std::lock_guard<std::mutex> lock(g_mu);
            auto it = g_groups.find(group);
            B200_REQUIRE(it != g_groups.end(), "no group named '%s': create it with diopiB200GroupCreate / diopiB200GroupConnect first", group);
            Group& g = it->second;
            B200_REQUIRE(g.connected, "group '%s' is not connected yet", group);
            B200_REQUIRE(g.device == di.device, "group '%s' lives on device %d, the current device is %d", group, g.device, di.device);
            if (*reinterpret_cast<volatile int*>(g.poison) != 0) {
                clear_async_status_if(3);   // the same event; this error names it better
                fail(diopiErrorOccurred,
                     "group '%s' is unusable: a kernel of this group gave up waiting for a peer's rows (or a peer did), so the ranks' call "
                     "numbers may no longer agree; destroy the group on every rank and create it again",
                     group);
            }
            if (M == 0 || N == 0) return;
            const int tiles = k::matmul_allreduce_tiles(M, N);
            B200_REQUIRE(tiles <= g.max_tiles, "the output has %d tiles of 128 x 128; group '%s' was created for at most %d", tiles, group, g.max_tiles);
            a.rank = g.rank;
            a.world = g.world;
            a.max_tiles = g.max_tiles;
            a.ctrl = g.ctrl[g.rank];
            a.poison_host = g.poison;
            a.wait_limit_ns = g.wait_limit_ns;
            // One-shot (every rank receives every partial) for groups of two or three and for outputs of fewer tiles than
            // ranks; else two-shot (partials to a tile's owner, finished tiles handed round): the second hop costs a
            // microsecond or two, the one-shot bytes grow with the group. The group option "form" forces one.
            a.two_shot = g.world >= 4 && tiles >= g.world;
            if (g.form == 1) a.two_shot = false;
            if (g.form == 2) a.two_shot = g.world > 1;
            a.force_tile_width = g.tile_width;
            for (int r = 0; r < g.world; ++r) {
                a.peer_stage[r] = g.stage[r];
                a.peer_result[r] = g.result[r];
                a.peer_ctrl[r] = g.ctrl[r];
            }
        }
        a.x1 = av.data;
        a.x2 = bv.data;
        a.bias = cv.defined ? cv.data : nullptr;
        a.out = o.data;
        a.M = static_cast<int>(M);
        a.N = static_cast<int>(N);
        a.K = static_cast<int>(K);
        a.status = async_status_device_ptr();
        const char* why = k::launch_matmul_allreduce(a, di.sm_count, di.max_smem_optin, st);
        if (why) fail(diopiErrorOccurred, "%s", why);
        B200_CUDA(cudaGetLastError());
    });
}
