// Launch interfaces between the exported ops (plain C++) and the CUDA kernels.
// Everything crosses as raw pointers, element strides and sizes.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>

namespace b200 {
namespace k {

enum class Dt : int { F16 = 0, BF16 = 1, F32 = 2, F64 = 3 };

// A 1-D or 2-D tensor of int32/int64 indices read on the device.
struct IndexArg {
    const void* ptr = nullptr;
    int64_t s0 = 0;  // stride of dim 0, in elements
    int64_t s1 = 0;  // stride of dim 1 (2-D only)
    int is64 = 0;
};

// ---- DestIndexCopyKV -------------------------------------------------------
struct CopyKVArgs {
    const void* src;  // [T, H, D]
    void* dst;        // [slots, H, D]
    IndexArg dest;    // [T]
    int64_t T, H, D, slots;
    int64_t src_s0, src_s1, src_s2;
    int64_t dst_s0, dst_s1, dst_s2;
    int elem_bytes;
    int* status;
};
void launch_dest_index_copy(const CopyKVArgs& a, cudaStream_t st);

// ---- decode attention over the paged pool -----------------------------------
enum class DecodeMode : int { QK = 0, PV = 1, FUSED = 2 };

struct DecodeArgs {
    DecodeMode mode;
    Dt dt;
    const void* q;   int64_t q_s0, q_s1, q_s2;          // [B,H,D]          (QK, FUSED)
    const void* kmat; int64_t k_s0, k_s1, k_s2;         // [slots,H,D]      (QK, FUSED)
    const void* vmat; int64_t v_s0, v_s1, v_s2;         // [slots,H,D]      (PV, FUSED)
    void* att;       int64_t att_s0, att_s1;            // [H,sumL] logits: written by QK, read by PV
    void* out;       int64_t out_s0, out_s1, out_s2;    // [B,H,D]          (PV, FUSED)
    IndexArg b_loc, b_start, b_len;
    int B, H, D, max_input_len;
    int64_t slots;       // extent of dim 0 of the pool (bounds check)
    int64_t att_cols;    // extent of dim 1 of att (bounds check)
    int* status;
    int block_size;      // 0: b_loc names one slot per token, right-aligned in its first max_input_len columns;
                         // > 0: b_loc is a block table, token j of request i sits in row b_loc[i, j / block_size] * block_size + j % block_size
    int kv_group;        // query heads per K/V head (0 or 1 = one to one)
    int force_plain;     // non-zero: the one-CTA-per-(request, head) kernel whatever the shape (no split-KV, no scratch)
};

// Size in bytes of the scratch the split-KV path needs for these arguments, 0 if the
// arguments take the plain (no scratch) path.
int64_t decode_workspace_bytes(const DecodeArgs& a, int sm_count, int max_smem);
// `ws` must hold decode_workspace_bytes(); ignored by the plain path.
void launch_decode(const DecodeArgs& a, void* ws, int sm_count, int max_smem, cudaStream_t st);
// Same launch on the library's built-in scratch array. `needed` receives the scratch size of these arguments;
// cudaErrorMemoryAllocation means it exceeds decode_static_scratch_capacity() and nothing was launched.
// The first call on a device looks up the array's device address (cudaGetSymbolAddress). Allocates nothing.
int64_t decode_static_scratch_capacity();
cudaError_t launch_decode_static_scratch(const DecodeArgs& a, int sm_count, int max_smem, cudaStream_t st, int64_t* needed);

// ---- RMSNorm ----------------------------------------------------------------
struct RmsNormArgs {
    Dt dt;
    const void* x;      // [n1, n2] dense
    const void* weight; // [n2]
    const void* bias;   // [n2] or null
    void* out;          // [n1, n2]
    void* inv_rms;      // [n1]
    Dt inv_dt;          // F32, F64, or the input's half type
    int64_t n1, n2;
    double eps;
};
void launch_rms_norm(const RmsNormArgs& a, int sm_count, cudaStream_t st);

struct RmsNormBwdArgs {
    Dt dt;
    const void* g;        // grad_output [n1, n2] dense
    const void* x;        // input       [n1, n2] dense
    const void* weight;   // [n2]
    const void* inv_rms;  // [n1], saved by the forward call
    Dt inv_dt;            // F32, F64, or the input's half type
    void* dx;             // grad_input  [n1, n2]
    void* dw;             // grad_weight [n2]
    void* db;             // grad_bias   [n2] or null
    int64_t n1, n2;
    float* ws;            // 2 * parts * n2 floats of scratch (partial column sums), or null
    int parts;            // CTAs of the rows kernel; 0 = the scalar kernels, which need no scratch
};
// Number of partial rows the vector path wants for these arguments (0: not eligible, no scratch needed).
int rms_norm_bwd_parts(const RmsNormBwdArgs& a, int sm_count);
void launch_rms_norm_bwd(const RmsNormBwdArgs& a, cudaStream_t st);

// ---- rotary embedding -------------------------------------------------------
constexpr int kRopeMaxDims = 6;
struct RopeArgs {
    Dt dt;
    const void* x; void* out; const void* cos; const void* sin;
    int nd;                          // number of leading (collapsed) dims
    int64_t size[kRopeMaxDims];
    int64_t xs[kRopeMaxDims], os[kRopeMaxDims], cs[kRopeMaxDims], ss[kRopeMaxDims];
    int64_t x_ls, o_ls, c_ls, s_ls;  // stride of the last dim
    int64_t half;                    // D / 2
    int64_t n_lead;                  // product of size[]
    bool conj;
};
void launch_rope(const RopeArgs& a, cudaStream_t st);

// rope(q) -> q_out, rope(k) -> k_pool[dest], v -> v_pool[dest] in one launch. Rows are dense ([heads, D] contiguous),
// cos/sin hold one row of D/2 values per token. v and v_pool may both be null.
struct RopeStoreArgs {
    Dt dt;
    const void* q; void* q_out; const void* k; void* k_pool; const void* v; void* v_pool;
    const void* cos; const void* sin;
    IndexArg dest;                 // [T]
    int64_t T, Hq, Hk, D, slots;
    int64_t q_s0, qo_s0, k_s0, kp_s0, v_s0, vp_s0, c_s0, s_s0;  // stride of dim 0, in elements
    bool conj;
    int* status;
};
// Returns false (nothing launched) when the arguments do not qualify for the one-launch kernel.
bool launch_rope_store_kv(const RopeStoreArgs& a, cudaStream_t st);

// In-place rotate-half form on [T, H*dim] query and key with full-width cos/sin (diopiRotaryEmbeddingV2).
struct RopeV2Args {
    Dt dt;
    void* q; int64_t q_s0; int64_t q_heads;     // [T, q_heads*dim], row stride in elements
    void* kk; int64_t k_s0; int64_t k_heads;    // [T, k_heads*dim]
    const void* cos; const void* sin;
    int64_t c_st, c_sh, s_st, s_sh;             // strides of cos/sin over token and head (0 where broadcast)
    int64_t T, dim;
};
void launch_rope_v2(const RopeV2Args& a, cudaStream_t st);

// ---- ApplyPenalty -----------------------------------------------------------
struct PenaltyArgs {
    Dt dt;
    void* logits; int64_t l_s0, l_s1; int64_t B, V;
    const void* presence; int64_t p_s;
    const void* frequency; int64_t f_s;
    IndexArg ids, counts, cum;
    int64_t E;
    int* status;
};
void launch_apply_penalty(const PenaltyArgs& a, cudaStream_t st);

// Flattened form with a repetition penalty and per-entry penalties (diopiApplyPenaltyV2).
struct PenaltyV2Args {
    Dt dt;
    void* logits; int64_t numel;                // contiguous, indexed flat
    const void* presence; const void* frequency; const void* repetition;  // [E]
    int64_t p_s, f_s, r_s;
    IndexArg ids, counts;
    int64_t E;
    int* status;
};
void launch_apply_penalty_v2(const PenaltyV2Args& a, cudaStream_t st);

// ---- causal prefill ---------------------------------------------------------
struct PrefillArgs {
    Dt dt;
    const void* q; const void* kmat; const void* vmat; void* out;   // [sumL, H, D]
    int64_t q_s0, q_s1, k_s0, k_s1, v_s0, v_s1, o_s0, o_s1;          // last dim dense
    IndexArg b_start, b_len;     // ignored when uniform_len > 0
    int B, H, D;
    int64_t total_rows;
    int max_input_len;
    int64_t uniform_len = 0;     // > 0: padded batch, request i owns rows [i * uniform_len, (i + 1) * uniform_len)
    int kv_group = 1;            // query heads per K/V head (grouped-query attention); k/v have H / kv_group heads
    bool force_simt = false;     // the SIMT kernel whatever the shape
};
// Returns the name of the kernel family that took the call ("tensor-core", "simt") or "none" for an empty problem.
const char* launch_prefill(const PrefillArgs& a, int sm_count, int max_smem, cudaStream_t st);

// ---- matmul + all-reduce over a tensor-parallel group --------------------------------------
constexpr int kMaxGroupRanks = 8;
struct MatmulAllReduceArgs {
    Dt dt;                    // F16 or BF16
    const void* x1;           // [M, K] row-major, x1_ld elements between rows
    const void* x2;           // [K, N] row-major (x2_kmajor = false, x2_ld between k rows) or stored as [N, K] (x2_kmajor = true, x2_ld between n rows)
    const void* bias;         // [N] or null
    void* out;                // [M, N], out_s0 elements between rows
    int64_t x1_ld, x2_ld, out_s0;
    bool x2_kmajor;
    int M, N, K;
    int rank, world, max_tiles;
    uint32_t* ctrl;           // this rank's control words: [0] calls finished so far, [1] CTAs of the running call that left, [2] poisoned
    uint32_t* peer_ctrl[kMaxGroupRanks];         // the control words of every rank (own included), as mapped into this process
    int* poison_host;         // mapped host word of this group: set when a kernel of this rank found or made the group unusable
    unsigned long long wait_limit_ns;            // how long a wait for a peer's rows (or for this kernel's own pipeline) may last
    unsigned char* peer_stage[kMaxGroupRanks];   // partial-tile area of every rank (own included), as mapped into this process
    unsigned char* peer_result[kMaxGroupRanks];  // finished-tile area of every rank (two-shot form)
    bool two_shot;            // partials to the tile's owner only, finished tiles handed round
    int force_tile_width;     // 0: the launch picks; 128, 64 or (K-major x2 only) 32: this width
    int k_splits;             // set by the launch: CTAs that share one output tile, each with a slice of K (groups of one only)
    int* status;
};
int matmul_allreduce_tiles(int64_t M, int64_t N);
struct MarLayout {
    size_t stage_off, result_off, ctrl_off, bytes;   // byte offsets inside one rank's area
};
MarLayout matmul_allreduce_layout(int world, int max_tiles);
// Returns null after a launch, else the reason why these arguments cannot run.
const char* launch_matmul_allreduce(const MatmulAllReduceArgs& a, int sm_count, int max_smem, cudaStream_t st);

}  // namespace k
}  // namespace b200
