/*
 * diopi_b200.h — the C ABI of the B200 backend (libdiopi_impl.so).
 *
 * The library is a drop-in DIOPI backend for the LLM-inference hot path. A DIOPI
 * consumer owns tensors, contexts and streams and hands them over as opaque
 * handles; the backend reads them only through the run-time accessors declared
 * in the first half of this file (the consumer defines those), launches its
 * kernels on the stream of the context it was given, and returns without
 * synchronising.
 *
 * Every enum value, struct layout and prototype here is ABI-identical to the
 * DIOPI interface headers it stands in for (proto/include/diopi/diopirt.h,
 * proto/include/diopi/functions.h, proto/include/diopi/functions_ext.h). When the
 * consumer has already included the original diopirt.h, the type block below is
 * skipped and only the prototypes are (re)declared, so a translation unit may
 * include both; a mismatch then fails to compile.
 */
#ifndef DIOPI_B200_H_
#define DIOPI_B200_H_

#include <stddef.h>
#include <stdint.h>
#if !defined(__cplusplus)
#include <stdbool.h>
#endif

#if defined(__cplusplus)
extern "C" {
#endif

/* ------------------------------------------------------------------------- */
/* Run-time types (stand in for proto/include/diopi/diopirt.h:27-112).        */
/* ------------------------------------------------------------------------- */
#ifndef _PROJECT_DIOPERATOR_INTERFACE_RT_H_

/* A borrowed array of int64: shapes, strides, normalized_shape. Passed by value. */
typedef struct {
    const int64_t* data;
    int64_t len;
} diopiSize_t;

/* Return codes. Only the four values the backend can return are spelled out
 * with their own names; the numeric gaps belong to the consumer-side run time. */
typedef enum {
    diopiSuccess = 0,
    diopiErrorOccurred = 1,
    diopiNotInited = 2,
    diopiNoRegisteredStreamCreateFunction = 3,
    diopiNoRegisteredStreamDestoryFunction = 4,
    diopiNoRegisteredStreamSyncFunction = 5,
    diopiNoRegisteredDeviceMemoryMallocFunction = 6,
    diopiNoRegisteredDeviceMemoryFreeFunction = 7,
    diopiNoRegisteredDevice2DdeviceMemoryCopyFunction = 8,
    diopiNoRegisteredDevice2HostMemoryCopyFunction = 9,
    diopiNoRegisteredHost2DeviceMemoryCopyFunction = 10,
    diopiNoRegisteredGetLastErrorFunction = 11,
    diopi5DNotSupported = 12,
    diopiNoImplement = 13,
    diopiForceFallbackToCPU = 14,
    diopiDtypeNotSupported = 1000
} diopiError_t;

typedef enum { diopi_host = 0, diopi_device = 1 } diopiDevice_t;

typedef int8_t diopiDeviceIndex_t;

typedef enum {
    diopi_dtype_int8 = 0,
    diopi_dtype_uint8 = 1,
    diopi_dtype_int16 = 2,
    diopi_dtype_uint16 = 3,
    diopi_dtype_int32 = 4,
    diopi_dtype_uint32 = 5,
    diopi_dtype_int64 = 6,
    diopi_dtype_uint64 = 7,
    diopi_dtype_float16 = 8,
    diopi_dtype_float32 = 9,
    diopi_dtype_float64 = 10,
    diopi_dtype_bool = 11,
    diopi_dtype_bfloat16 = 12,
    diopi_dtype_tfloat32 = 13,
    diopi_dtype_complex32 = 14,
    diopi_dtype_complex64 = 15,
    diopi_dtype_complex128 = 16,
    diopi_dtype_unsupported = 255
} diopiDtype_t;

/* Opaque handles: the backend never looks inside them. */
struct diopiContext;
typedef struct diopiContext* diopiContextHandle_t;
struct diopiTensor;
typedef struct diopiTensor* diopiTensorHandle_t;
typedef const struct diopiTensor* diopiConstTensorHandle_t;
typedef void* diopiStreamHandle_t; /* a cudaStream_t for this backend */

#define DIOPI_B200_OWN_RT_TYPES 1
#endif /* _PROJECT_DIOPERATOR_INTERFACE_RT_H_ */

#define DIOPI_B200_WEAK __attribute__((weak))

/* ------------------------------------------------------------------------- */
/* Run-time accessors the library IMPORTS (the consumer defines them).        */
/* Strong ones (diopirt.h:122-126,129,145,147) must exist; weak ones           */
/* (diopirt.h:127,130,140,149) are used only when the loader resolved them.    */
/* ------------------------------------------------------------------------- */
extern diopiError_t diopiGetTensorData(diopiTensorHandle_t th, void** data);
extern diopiError_t diopiGetTensorDataConst(diopiConstTensorHandle_t th, const void** data);
extern diopiError_t diopiGetTensorShape(diopiConstTensorHandle_t th, diopiSize_t* size);
extern diopiError_t diopiGetTensorStride(diopiConstTensorHandle_t th, diopiSize_t* stride);
extern diopiError_t diopiGetTensorDtype(diopiConstTensorHandle_t th, diopiDtype_t* dtype);
extern diopiError_t diopiGetTensorNumel(diopiConstTensorHandle_t th, int64_t* numel);
extern diopiError_t diopiGetStream(diopiContextHandle_t ctx, diopiStreamHandle_t* stream);
extern diopiError_t diopiRequireTensor(diopiContextHandle_t ctx, diopiTensorHandle_t* tensor, const diopiSize_t* size, const diopiSize_t* stride,
                                       const diopiDtype_t dtype, const diopiDevice_t device);
extern DIOPI_B200_WEAK diopiError_t diopiGetTensorDevice(diopiConstTensorHandle_t th, diopiDevice_t* device);
extern DIOPI_B200_WEAK diopiError_t diopiGetTensorElemSize(diopiConstTensorHandle_t th, int64_t* itemsize);
extern DIOPI_B200_WEAK diopiError_t diopiGetCurrentDeviceIndex(diopiDeviceIndex_t* pDevIndex);
extern DIOPI_B200_WEAK diopiError_t diopiRequireBuffer(diopiContextHandle_t ctx, diopiTensorHandle_t* tensor, int64_t num_bytes, diopiDevice_t device);
extern DIOPI_B200_WEAK diopiError_t diopiRecordStart(const char* record_name, void** record);
extern DIOPI_B200_WEAK diopiError_t diopiRecordEnd(void** record);

/* ------------------------------------------------------------------------- */
/* Symbols the library EXPORTS.                                               */
/* ------------------------------------------------------------------------- */

/* Backend identification and the text of the most recent failure on any thread.
 * Replace proto/include/diopi/functions.h:19-21. The vendor name contains the
 * substring "Device", which the reference's device-info test looks for. */
const char* diopiGetVendorName();
const char* diopiGetImplVersion();
const char* diopiGetLastErrorString();

/* out[dest_loc[t], :, :] = k[t, :, :] — writes new tokens' K (or V) rows into the
 * paged pool. k [T,H,D]; dest_loc [T] int32/int64; out [slots,H,D], same dtype as k.
 * Bit-exact byte copy. Replaces proto/include/diopi/functions_ext.h:563. */
diopiError_t diopiDestIndexCopyKV(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t k, diopiConstTensorHandle_t dest_loc);

/* Decode logits: for request i and j in [0, L_i):
 *   slot = b_loc[i, max_input_len - L_i + j]
 *   token_attention_out[h, b_start_loc[i] + j] = dot(q[i,h,:], k[slot,h,:]) / sqrt(D)
 * q [B,H,D]; k [slots,H,D]; b_loc [B,N>=max_input_len]; b_start_loc, b_seq_len [B];
 * token_attention_out [H, sum(L)]. Replaces functions_ext.h:579-581. */
diopiError_t diopiTokenAttentionInference(diopiContextHandle_t ctx, diopiTensorHandle_t token_attention_out, diopiConstTensorHandle_t q,
                                          diopiConstTensorHandle_t k, diopiConstTensorHandle_t b_loc, diopiConstTensorHandle_t b_start_loc,
                                          diopiConstTensorHandle_t b_seq_len, int max_input_len);

/* Decode output: P = softmax(logics[:, start_i : start_i + L_i]) per head,
 * out[i,h,:] = sum_j P[h,j] * v[slot(i,j),h,:]. A request of length 0 gets zeros.
 * other_kv_index is accepted and ignored, as in the reference.
 * Replaces functions_ext.h:597-599. */
diopiError_t diopiTokenSoftmaxReduceVInference(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t logics,
                                               diopiConstTensorHandle_t v, diopiConstTensorHandle_t b_loc, diopiConstTensorHandle_t b_start_loc,
                                               diopiConstTensorHandle_t b_seq_len, int max_input_len, int other_kv_index);

/* Causal prefill over a packed ragged batch: for request i on rows
 * [b_start_loc[i], b_start_loc[i] + b_seq_len[i]) of q/k/v/out [sum(L),H,D]:
 * out = softmax(q k^T / sqrt(D) + causal mask) v, per head.
 * Replaces functions_ext.h:634-636. */
diopiError_t diopiContextAttentionInference(diopiContextHandle_t ctx, diopiTensorHandle_t context_attention_out, diopiConstTensorHandle_t q,
                                            diopiConstTensorHandle_t k, diopiConstTensorHandle_t v, diopiConstTensorHandle_t b_start_loc,
                                            diopiConstTensorHandle_t b_seq_len, int max_input_len);

/* In-place sampling penalty: for request i and entries e in
 * [p_cumsum_seq_len[i], p_cumsum_seq_len[i+1]):
 *   logits[i, p_token_ids[e]] -= p_token_counts[e] * frequency_penalty[i] + presence_penalty[i]
 * evaluated as three separately rounded operations in the dtype of logits.
 * Replaces functions_ext.h:527-529. */
diopiError_t diopiApplyPenalty(diopiContextHandle_t ctx, diopiTensorHandle_t logits, diopiConstTensorHandle_t presence_penalty,
                               diopiConstTensorHandle_t frequency_penalty, diopiConstTensorHandle_t p_token_ids, diopiConstTensorHandle_t p_token_counts,
                               diopiConstTensorHandle_t p_cumsum_seq_len, int p_max_len_in_batch);

/* Rotary embedding on the two halves of the last dimension; cos/sin broadcast
 * against x's leading dimensions. interleaved=true returns diopiNoImplement, as the
 * reference's NVIDIA backend does. Replaces functions_ext.h:31-32. */
diopiError_t diopiRotaryEmbedding(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t x, diopiConstTensorHandle_t cos,
                                  diopiConstTensorHandle_t sin, const bool conj, const bool interleaved);

/* RMS normalisation over the trailing normalized_shape dims:
 * inv_rms = rsqrt(mean(x^2) + eps) (fp32; fp64 for fp64 input),
 * out = weight * (x * inv_rms) (+ bias), one rounding at the end.
 * Replaces functions_ext.h:45-46. */
diopiError_t diopiRMSNorm(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiTensorHandle_t inv_rms, diopiConstTensorHandle_t input,
                          diopiSize_t normalized_shape, diopiConstTensorHandle_t weight, diopiConstTensorHandle_t bias, double eps);

/* Derivative of diopiRMSNorm given the inv_rms it saved, in fp32 with one rounding at the end:
 * grad_input = inv_rms * (g * weight) - x * inv_rms^3 * mean(g * weight * x),
 * grad_weight = sum over rows of g * x * inv_rms, grad_bias = sum over rows of g (grad_bias may be null).
 * Column sums are added in a fixed order (no atomics). Replaces functions_ext.h:62-65. */
diopiError_t diopiRMSNormBackward(diopiContextHandle_t ctx, diopiTensorHandle_t grad_input, diopiTensorHandle_t grad_weight,
                                  diopiTensorHandle_t grad_bias, diopiConstTensorHandle_t grad_output, diopiConstTensorHandle_t input,
                                  diopiConstTensorHandle_t weight, diopiConstTensorHandle_t bias, diopiConstTensorHandle_t inv_rms,
                                  diopiSize_t normalized_shape, double eps);

/* In-place rotary embedding on query and key [tokens, heads*dim] in the rotate-half form with cos/sin
 * as wide as a head: x = x*cos + (-x2, x1)*sin, each operation rounded in the tensors' dtype.
 * Replaces functions_ext.h:649-650. */
diopiError_t diopiRotaryEmbeddingV2(diopiContextHandle_t ctx, diopiTensorHandle_t query, diopiTensorHandle_t key, diopiConstTensorHandle_t cos,
                                    diopiConstTensorHandle_t sin, int64_t dim);

/* In-place penalty on the flattened logits with one penalty triple per entry:
 * x = logits.flat[id]; x = x > 0 ? x / repetition : x * repetition; x -= count * frequency; x -= presence.
 * Replaces functions_ext.h:547-549. */
diopiError_t diopiApplyPenaltyV2(diopiContextHandle_t ctx, diopiTensorHandle_t logits, diopiConstTensorHandle_t presence_penalty,
                                 diopiConstTensorHandle_t frequency_penalty, diopiConstTensorHandle_t repetition_penalty,
                                 diopiConstTensorHandle_t p_token_ids, diopiConstTensorHandle_t p_token_counts);

/* Causal prefill over a padded batch in BSH layout: request i owns rows [i*max_input_len, (i+1)*max_input_len)
 * of query/out [batch*max_input_len, num_heads*dim] and key/value [.., num_kv_heads*dim]; num_kv_heads may divide
 * num_heads (grouped-query attention). atten_mask is not read (the mask is causal) and actual_seq_lengths gives
 * the batch size only, as in the reference's golden function. Replaces functions_ext.h:684-686. */
diopiError_t diopiPromptFlashAttention(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t query, diopiConstTensorHandle_t key,
                                       diopiConstTensorHandle_t value, diopiConstTensorHandle_t atten_mask, diopiSize_t actual_seq_lengths,
                                       int64_t max_input_len, int64_t num_heads, int64_t num_kv_heads, int64_t dim);

/* Decode attention over a block-paged KV cache, BSH layout: q/out [batch, num_heads*dim], k/v [rows, num_kv_heads*dim],
 * token j of request i in row block_table[i, j/block_size]*block_size + j%block_size, lengths given on the host.
 * atten_mask is not read. Replaces functions_ext.h:616-618. */
diopiError_t diopiPagedAttention(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t q, diopiConstTensorHandle_t k,
                                 diopiConstTensorHandle_t v, diopiConstTensorHandle_t atten_mask, diopiSize_t actual_seq_lengths, int64_t num_heads,
                                 int64_t num_kv_heads, int64_t dim, diopiConstTensorHandle_t block_table, int64_t block_size);

/* Extension (not in the DIOPI headers): the fused decode step. Equivalent to
 * diopiTokenAttentionInference followed by diopiTokenSoftmaxReduceVInference on
 * the same index tensors, but the logits never reach memory: one pass over the
 * gathered K and V rows with an online softmax, fp32 accumulation.
 * It is the composition of functions_ext.h:579-581 and :597-599; out [B,H,D]. */
diopiError_t diopiTokenDecodeAttentionInference(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t q, diopiConstTensorHandle_t k,
                                                diopiConstTensorHandle_t v, diopiConstTensorHandle_t b_loc, diopiConstTensorHandle_t b_start_loc,
                                                diopiConstTensorHandle_t b_seq_len, int max_input_len);

/* Extension (not in the DIOPI headers): the step in front of decode attention as one call. Equivalent, bit for bit, to
 * diopiRotaryEmbedding(q_out, q, cos, sin, conj, false), then diopiRotaryEmbedding into a temporary for k and
 * diopiDestIndexCopyKV(k_pool, temporary, dest_loc), then diopiDestIndexCopyKV(v_pool, v, dest_loc)
 * (functions_ext.h:31-32 and :563). q/q_out [T, heads, D], k/v [T, kv_heads, D], pools [slots, kv_heads, D],
 * cos/sin one row of D/2 per token; v and v_pool may both be null; q_out may be q. */
diopiError_t diopiRotaryEmbeddingCopyKV(diopiContextHandle_t ctx, diopiTensorHandle_t q_out, diopiTensorHandle_t k_pool, diopiTensorHandle_t v_pool,
                                        diopiConstTensorHandle_t q, diopiConstTensorHandle_t k, diopiConstTensorHandle_t v, diopiConstTensorHandle_t cos,
                                        diopiConstTensorHandle_t sin, diopiConstTensorHandle_t dest_loc, bool conj);

/* out [.., N] = sum over the ranks of `group` of (x1 [.., K] @ x2 [K, N] + bias [N]): the row-parallel linear layer of a
 * tensor-parallel model as one kernel per rank (tcgen05 GEMM whose epilogue stores the fp32 partial tiles into every
 * rank's staging area over NVLink; each rank then adds the partials in rank order, so all ranks hold identical bits).
 * float16/bfloat16; x2 row-major or the transposed view of an [N, K] weight; reduce_op "sum"; comm_turn and stream_mode
 * are not read. The group must have been set up with the two calls below. Replaces functions_ext.h:664-665. */
diopiError_t diopiMatmulAllReduce(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t x1, diopiConstTensorHandle_t x2,
                                  diopiConstTensorHandle_t bias, const char* group, const char* reduce_op, int64_t comm_turn, int64_t stream_mode);

/* Extensions with no counterpart in the reference (there the group string names an HCCL communicator made elsewhere):
 * set-up of a tensor-parallel group of up to 8 ranks, one process and one GPU each. Create allocates this rank's staging
 * area for outputs of at most max_tiles tiles of 128 x 128 (2 * world * max_tiles * 64 KiB) and writes its 64-byte CUDA
 * IPC handle to local_handle; the caller exchanges the handles (rank order) and passes all of them to Connect, which
 * maps the peers' areas. A group of one rank is usable after Create. Destroy unmaps and frees. */
diopiError_t diopiB200GroupCreate(const char* group, int rank, int world, int64_t max_tiles, void* local_handle);
diopiError_t diopiB200GroupConnect(const char* group, const void* handles);
diopiError_t diopiB200GroupDestroy(const char* group);
/* Options of one group; no counterpart in the reference.
 *   "wait_limit_ms"  how long a kernel of the group waits for a peer's rows before it gives up (1 .. 600000; 2000 when
 *                    never set). A wait that runs out makes the call that sees it next fail with status 3 and marks the
 *                    group unusable on every rank: later calls on it are refused until every rank has destroyed the
 *                    group and created it again (the ranks' call numbers may no longer agree).
 *   "form"           0 the exchange is chosen per call, 1 one-shot (every rank receives every partial), 2 two-shot
 *                    (partials to a tile's owner, finished tiles handed round). Must be the same on every rank.
 *   "tile_width"     0 chosen per call, or 128 / 64 / 32 output columns per tile. Must be the same on every rank. */
diopiError_t diopiB200GroupSetOption(const char* group, const char* option, int64_t value);

/* Forget a context: launches a decode-logits call that the fuse_token_attention switch has recorded on `ctx` (instead of
 * launching it) and drops the record, which holds raw tensor pointers keyed by the context handle. Call it before a
 * context on which diopiTokenAttentionInference ran with that switch on is destroyed; a no-op otherwise. No counterpart
 * in the reference. */
diopiError_t diopiB200ContextRelease(diopiContextHandle_t ctx);

/* Process-wide switches; no counterpart in the reference. Each starts from an environment variable read once
 * (DIOPI_B200_LOG, DIOPI_B200_FUSE_TOKEN_ATTENTION, DIOPI_B200_DECODE_PLAIN, DIOPI_B200_PREFILL_SIMT) and is changed
 * here by name: "log", "fuse_token_attention", "decode_plain", "prefill_simt"; value 0 switches off, non-zero on. */
diopiError_t diopiB200SetOption(const char* name, int64_t value);

/* Extension with no counterpart in the reference: the same fused decode step for callers that
 * cannot provide scratch memory (an engine whose HBM all went to the KV pool and whose context has
 * no allocator; a harness whose diopiRequireTensor fails). It never calls diopiRequireBuffer /
 * diopiRequireTensor and allocates nothing: the split-KV partials go to a fixed 8 MiB array inside
 * the library's device image, held by every GPU that loads the library. Refuses, with an error,
 * problems whose partials ((148 + batch) * head_num * (head_dim + 2) * 4 bytes) exceed it. The first
 * call on a device looks up the array's address: make it before any stream capture. Calls that may
 * overlap on one GPU share the array and race; keep them on one stream. With the fuse_token_attention
 * switch on, a logits call recorded on `ctx` is NOT launched by this entry point (launching it needs
 * scratch): call diopiB200ContextRelease(ctx) first if one may be pending. */
diopiError_t diopiTokenDecodeAttentionInferenceNoAlloc(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t q,
                                                       diopiConstTensorHandle_t k, diopiConstTensorHandle_t v, diopiConstTensorHandle_t b_loc,
                                                       diopiConstTensorHandle_t b_start_loc, diopiConstTensorHandle_t b_seq_len, int max_input_len);

#if defined(__cplusplus)
}
#endif

#endif /* DIOPI_B200_H_ */
