// The exported C entry points of libdiopi_impl.so: argument validation, then one launch on the
// stream of the caller's context. No host synchronisation, no per-request host loop; lengths,
// start offsets and slot tables are read on the device.
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "../kernels/kernels.hpp"
#include "common.hpp"

namespace b200 {
const char* last_error_cstr();
}

using namespace b200;  // NOLINT

namespace {

k::Dt float_dt(const TensorView& t, const char* name, bool allow_f64) {
    switch (t.dtype) {
        case diopi_dtype_float16: return k::Dt::F16;
        case diopi_dtype_bfloat16: return k::Dt::BF16;
        case diopi_dtype_float32: return k::Dt::F32;
        case diopi_dtype_float64:
            if (allow_f64) return k::Dt::F64;
            break;
        default: break;
    }
    fail(diopiDtypeNotSupported, "'%s' has dtype %s; supported: float16, bfloat16, float32%s", name, dtype_name(t.dtype), allow_f64 ? ", float64" : "");
}

k::IndexArg index_arg(const TensorView& t, const char* name, int ndim) {
    if (!is_index_dtype(t.dtype)) fail(diopiDtypeNotSupported, "'%s' has dtype %s; index tensors must be int32 or int64", name, dtype_name(t.dtype));
    B200_REQUIRE(t.ndim == ndim, "'%s' must have %d dim(s), got %d", name, ndim, t.ndim);
    k::IndexArg a;
    a.ptr = t.data;
    a.s0 = t.stride[0];
    a.s1 = ndim > 1 ? t.stride[1] : 0;
    a.is64 = t.dtype == diopi_dtype_int64;
    return a;
}

void same_dtype(const TensorView& a, const char* an, const TensorView& b, const char* bn) {
    B200_REQUIRE(a.dtype == b.dtype, "'%s' (%s) and '%s' (%s) must share a dtype", an, dtype_name(a.dtype), bn, dtype_name(b.dtype));
}

// Common checks and argument packing of the three decode entry points.
void run_decode(diopiContextHandle_t ctx, k::DecodeMode mode, const TensorView* out, const TensorView* att, const TensorView* q, const TensorView* kmat,
                const TensorView* vmat, const TensorView& b_loc, const TensorView& b_start, const TensorView& b_len, int max_input_len, bool launch = true) {
    k::DecodeArgs a{};
    a.mode = mode;
    a.force_plain = options().decode_plain;
    const TensorView& pool = kmat ? *kmat : *vmat;
    a.dt = float_dt(pool, kmat ? "k" : "v", false);
    B200_REQUIRE(pool.ndim == 3, "the K/V pool must be [slots, head_num, head_dim], got %d dims", pool.ndim);
    a.H = static_cast<int>(pool.shape[1]);
    a.D = static_cast<int>(pool.shape[2]);
    a.slots = pool.shape[0];
    B200_REQUIRE(b_loc.ndim == 2, "'b_loc' must be [batch, N], got %d dims", b_loc.ndim);
    a.B = static_cast<int>(b_loc.shape[0]);
    B200_REQUIRE(max_input_len >= 0, "max_input_len must not be negative (got %d)", max_input_len);
    B200_REQUIRE(b_loc.shape[1] >= max_input_len, "'b_loc' has %ld columns, fewer than max_input_len = %d", (long)b_loc.shape[1], max_input_len);
    a.max_input_len = max_input_len;
    a.b_loc = index_arg(b_loc, "b_loc", 2);
    a.b_start = index_arg(b_start, "b_start_loc", 1);
    a.b_len = index_arg(b_len, "b_seq_len", 1);
    B200_REQUIRE(b_start.shape[0] == a.B && b_len.shape[0] == a.B, "'b_start_loc' and 'b_seq_len' must have batch = %d entries", a.B);
    B200_REQUIRE(a.D <= 512, "head_dim %d is beyond the supported maximum of 512", a.D);

    if (q) {
        same_dtype(*q, "q", pool, "k");
        B200_REQUIRE(q->ndim == 3 && q->shape[0] == a.B && q->shape[1] == a.H && q->shape[2] == a.D, "'q' must be [%d, %d, %d]", a.B, a.H, a.D);
        a.q = q->data;
        a.q_s0 = q->stride[0];
        a.q_s1 = q->stride[1];
        a.q_s2 = q->stride[2];
    }
    if (kmat) {
        a.kmat = kmat->data;
        a.k_s0 = kmat->stride[0];
        a.k_s1 = kmat->stride[1];
        a.k_s2 = kmat->stride[2];
    }
    if (vmat) {
        same_dtype(*vmat, "v", pool, "k");
        B200_REQUIRE(vmat->ndim == 3 && vmat->shape[1] == a.H && vmat->shape[2] == a.D, "'v' must be [slots, %d, %d]", a.H, a.D);
        if (kmat) B200_REQUIRE(vmat->shape[0] == kmat->shape[0], "'k' and 'v' pools differ in slot count");
        a.vmat = vmat->data;
        a.v_s0 = vmat->stride[0];
        a.v_s1 = vmat->stride[1];
        a.v_s2 = vmat->stride[2];
    }
    if (att) {
        same_dtype(*att, "logits", pool, "k/v");
        B200_REQUIRE(att->ndim == 2 && att->shape[0] == a.H, "the logits tensor must be [head_num = %d, sum of lengths]", a.H);
        a.att = att->data;
        a.att_s0 = att->stride[0];
        a.att_s1 = att->stride[1];
        a.att_cols = att->shape[1];
    }
    if (out) {
        same_dtype(*out, "out", pool, "k/v");
        B200_REQUIRE(out->ndim == 3 && out->shape[0] == a.B && out->shape[1] == a.H && out->shape[2] == a.D, "'out' must be [%d, %d, %d]", a.B, a.H, a.D);
        a.out = out->data;
        a.out_s0 = out->stride[0];
        a.out_s1 = out->stride[1];
        a.out_s2 = out->stride[2];
    }
    if (a.B == 0 || a.H == 0 || a.D == 0) return;
    B200_REQUIRE(a.slots > 0 || max_input_len == 0, "the K/V pool has no slots");
    if (!launch) return;  // checks only
    cudaStream_t st = stream_of(ctx);
    if (max_input_len == 0 || a.slots == 0) {
        // Every request is empty: no logits to write, zeros for the attention output.
        if (out && out->numel > 0) {
            B200_REQUIRE(out->contiguous(), "'out' must be contiguous when every request is empty");
            B200_CUDA(cudaMemsetAsync(out->data, 0, static_cast<size_t>(out->numel * out->elem_size()), st));
        }
        return;
    }
    const DeviceInfo& di = device_info();
    a.status = async_status_device_ptr();
    const int64_t ws_bytes = k::decode_workspace_bytes(a, di.sm_count, di.max_smem_optin);
    void* ws = ws_bytes > 0 ? workspace(ctx, ws_bytes) : nullptr;
    logf("decode mode=%d B=%d H=%d D=%d max_input_len=%d scratch=%ld bytes (%s path)", static_cast<int>(mode), a.B, a.H, a.D, max_input_len, (long)ws_bytes,
         (ws_bytes > 0 || mode == k::DecodeMode::QK) ? "split or plain" : "plain");
    k::launch_decode(a, ws, di.sm_count, di.max_smem_optin, st);
    B200_CUDA(cudaGetLastError());
}

// ---- the two-call decode run as one kernel (opt-in) ------------------------------------------------
// With the option fuse_token_attention on (DIOPI_B200_FUSE_TOKEN_ATTENTION=1 at start-up, or diopiB200SetOption),
// diopiTokenAttentionInference checks its arguments and
// records them instead of launching. If the next call of this library on the same context is
// diopiTokenSoftmaxReduceVInference on the same logits tensor and the same index tensors, the pair runs as the
// fused kernel and the logits tensor is never written. Any other call of this library on that context first
// launches the recorded logits kernel, so the logits are in memory whenever this library reads them. What the
// library cannot see is the caller reading the logits itself, or freeing q/k/the index tensors between the two
// calls: hence opt-in. The entry point that allocates nothing does not look at the record.
struct PendingQK {
    TensorView att, q, k, b_loc, b_start, b_len;
    int max_input_len = 0;
};
std::mutex g_pending_mu;
std::unordered_map<diopiContextHandle_t, PendingQK> g_pending;

bool fuse_pair_enabled() { return options().fuse_token_attention != 0; }

bool take_pending(diopiContextHandle_t ctx, PendingQK& out) {
    std::lock_guard<std::mutex> lock(g_pending_mu);
    auto it = g_pending.find(ctx);
    if (it == g_pending.end()) return false;
    out = it->second;
    g_pending.erase(it);
    return true;
}

// Launches the recorded logits kernel of this context, if there is one. Called first by every other entry point.
void flush_pending(diopiContextHandle_t ctx) {
    {
        std::lock_guard<std::mutex> lock(g_pending_mu);
        if (g_pending.empty()) return;
    }
    PendingQK p;
    if (!take_pending(ctx, p)) return;
    run_decode(ctx, k::DecodeMode::QK, nullptr, &p.att, &p.q, &p.k, nullptr, p.b_loc, p.b_start, p.b_len, p.max_input_len);
}

bool same_tensor(const TensorView& a, const TensorView& b) {
    if (a.data != b.data || a.dtype != b.dtype || a.ndim != b.ndim) return false;
    for (int i = 0; i < a.ndim; ++i)
        if (a.shape[i] != b.shape[i] || a.stride[i] != b.stride[i]) return false;
    return true;
}

}  // namespace

// ---------------------------------------------------------------------------------------------
B200_EXPORT const char* diopiGetVendorName() { return "B200Device"; }
B200_EXPORT const char* diopiGetImplVersion() {
    static char buf[160];
    static bool once = [] {
        std::snprintf(buf, sizeof(buf), "diopi_b200 0.1.0 (sm_100a, CUDA runtime %d.%d)", CUDART_VERSION / 1000, (CUDART_VERSION % 1000) / 10);
        return true;
    }();
    (void)once;
    return buf;
}
B200_EXPORT const char* diopiGetLastErrorString() { return last_error_cstr(); }

// Extension: forget a context. With the fuse_token_attention switch on, diopiTokenAttentionInference may have recorded a
// call on this context instead of launching it; the record holds raw tensor pointers and is keyed by the context handle.
// This launches the recorded kernel (the logits get written) and drops the record, so that a context created later at
// the same address cannot inherit it. Call it before destroying a context on which the pair of decode calls was used.
B200_EXPORT diopiError_t diopiB200ContextRelease(diopiContextHandle_t ctx) {
    return guard("diopiB200ContextRelease", [&] {
        B200_REQUIRE(ctx != nullptr, "null context handle");
        flush_pending(ctx);
    }, /*report_status=*/false);
}

// Extension: changes one of the process-wide switches of common.hpp (the environment gives only their start values).
B200_EXPORT diopiError_t diopiB200SetOption(const char* name, int64_t value) {
    return guard("diopiB200SetOption", [&] {
        if (!set_option(name, value))
            fail(diopiErrorOccurred, "unknown option '%s'; known: log, fuse_token_attention, decode_plain, prefill_simt", name ? name : "(null)");
    }, /*report_status=*/false);
}

// ---------------------------------------------------------------------------------------------
B200_EXPORT diopiError_t diopiDestIndexCopyKV(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t kh, diopiConstTensorHandle_t dest_loc) {
    return guard("diopiDestIndexCopyKV", [&] {
        flush_pending(ctx);
        TensorView o = view_of(out, "out"), src = view_of(kh, "k"), d = view_of(dest_loc, "dest_loc");
        same_dtype(o, "out", src, "k");
        B200_REQUIRE(dtype_size(src.dtype) > 0, "'k' has an unsupported dtype");
        B200_REQUIRE(src.ndim == 3 && o.ndim == 3, "'k' and 'out' must be [tokens, head_num, head_dim]");
        B200_REQUIRE(src.shape[1] == o.shape[1] && src.shape[2] == o.shape[2], "'k' is [*, %ld, %ld] but 'out' is [*, %ld, %ld]", (long)src.shape[1],
                     (long)src.shape[2], (long)o.shape[1], (long)o.shape[2]);
        k::CopyKVArgs a{};
        a.dest = index_arg(d, "dest_loc", 1);
        B200_REQUIRE(d.shape[0] == src.shape[0], "'dest_loc' has %ld entries for %ld rows of 'k'", (long)d.shape[0], (long)src.shape[0]);
        a.src = src.data;
        a.dst = o.data;
        a.T = src.shape[0];
        a.H = src.shape[1];
        a.D = src.shape[2];
        a.slots = o.shape[0];
        a.src_s0 = src.stride[0];
        a.src_s1 = src.stride[1];
        a.src_s2 = src.stride[2];
        a.dst_s0 = o.stride[0];
        a.dst_s1 = o.stride[1];
        a.dst_s2 = o.stride[2];
        a.elem_bytes = static_cast<int>(dtype_size(src.dtype));
        if (src.numel == 0) return;
        B200_REQUIRE(a.slots > 0, "'out' has no slots");
        cudaStream_t st = stream_of(ctx);
        a.status = async_status_device_ptr();
        k::launch_dest_index_copy(a, st);
        B200_CUDA(cudaGetLastError());
    });
}

B200_EXPORT diopiError_t diopiTokenAttentionInference(diopiContextHandle_t ctx, diopiTensorHandle_t token_attention_out, diopiConstTensorHandle_t q,
                                                      diopiConstTensorHandle_t kh, diopiConstTensorHandle_t b_loc, diopiConstTensorHandle_t b_start_loc,
                                                      diopiConstTensorHandle_t b_seq_len, int max_input_len) {
    return guard("diopiTokenAttentionInference", [&] {
        TensorView att = view_of(token_attention_out, "token_attention_out"), qv = view_of(q, "q"), kv = view_of(kh, "k");
        TensorView bl = view_of(b_loc, "b_loc"), bs = view_of(b_start_loc, "b_start_loc"), bn = view_of(b_seq_len, "b_seq_len");
        flush_pending(ctx);
        if (fuse_pair_enabled()) {
            run_decode(ctx, k::DecodeMode::QK, nullptr, &att, &qv, &kv, nullptr, bl, bs, bn, max_input_len, /*launch=*/false);
            PendingQK p;
            p.att = att; p.q = qv; p.k = kv; p.b_loc = bl; p.b_start = bs; p.b_len = bn;
            p.max_input_len = max_input_len;
            std::lock_guard<std::mutex> lock(g_pending_mu);
            g_pending[ctx] = p;
            return;
        }
        run_decode(ctx, k::DecodeMode::QK, nullptr, &att, &qv, &kv, nullptr, bl, bs, bn, max_input_len);
    });
}

B200_EXPORT diopiError_t diopiTokenSoftmaxReduceVInference(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t logics,
                                                           diopiConstTensorHandle_t v, diopiConstTensorHandle_t b_loc, diopiConstTensorHandle_t b_start_loc,
                                                           diopiConstTensorHandle_t b_seq_len, int max_input_len, int /*other_kv_index*/) {
    return guard("diopiTokenSoftmaxReduceVInference", [&] {
        TensorView o = view_of(out, "out"), att = view_of(logics, "logics"), vv = view_of(v, "v");
        TensorView bl = view_of(b_loc, "b_loc"), bs = view_of(b_start_loc, "b_start_loc"), bn = view_of(b_seq_len, "b_seq_len");
        PendingQK p;
        if (take_pending(ctx, p)) {
            if (same_tensor(p.att, att) && same_tensor(p.b_loc, bl) && same_tensor(p.b_start, bs) && same_tensor(p.b_len, bn) &&
                p.max_input_len == max_input_len) {
                run_decode(ctx, k::DecodeMode::FUSED, &o, nullptr, &p.q, &p.k, &vv, bl, bs, bn, max_input_len);
                return;
            }
            run_decode(ctx, k::DecodeMode::QK, nullptr, &p.att, &p.q, &p.k, nullptr, p.b_loc, p.b_start, p.b_len, p.max_input_len);
        }
        run_decode(ctx, k::DecodeMode::PV, &o, &att, nullptr, nullptr, &vv, bl, bs, bn, max_input_len);
    });
}

B200_EXPORT diopiError_t diopiTokenDecodeAttentionInference(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t q,
                                                            diopiConstTensorHandle_t kh, diopiConstTensorHandle_t v, diopiConstTensorHandle_t b_loc,
                                                            diopiConstTensorHandle_t b_start_loc, diopiConstTensorHandle_t b_seq_len, int max_input_len) {
    return guard("diopiTokenDecodeAttentionInference", [&] {
        flush_pending(ctx);
        TensorView o = view_of(out, "out"), qv = view_of(q, "q"), kv = view_of(kh, "k"), vv = view_of(v, "v");
        TensorView bl = view_of(b_loc, "b_loc"), bs = view_of(b_start_loc, "b_start_loc"), bn = view_of(b_seq_len, "b_seq_len");
        run_decode(ctx, k::DecodeMode::FUSED, &o, nullptr, &qv, &kv, &vv, bl, bs, bn, max_input_len);
    });
}

B200_EXPORT diopiError_t diopiContextAttentionInference(diopiContextHandle_t ctx, diopiTensorHandle_t context_attention_out, diopiConstTensorHandle_t q,
                                                        diopiConstTensorHandle_t kh, diopiConstTensorHandle_t v, diopiConstTensorHandle_t b_start_loc,
                                                        diopiConstTensorHandle_t b_seq_len, int max_input_len) {
    return guard("diopiContextAttentionInference", [&] {
        flush_pending(ctx);
        TensorView o = view_of(context_attention_out, "context_attention_out"), qv = view_of(q, "q"), kv = view_of(kh, "k"), vv = view_of(v, "v");
        TensorView bs = view_of(b_start_loc, "b_start_loc"), bn = view_of(b_seq_len, "b_seq_len");
        k::PrefillArgs a{};
        a.force_simt = options().prefill_simt != 0;
        a.dt = float_dt(qv, "q", false);
        same_dtype(kv, "k", qv, "q");
        same_dtype(vv, "v", qv, "q");
        same_dtype(o, "context_attention_out", qv, "q");
        B200_REQUIRE(qv.ndim == 3, "'q' must be [sum of lengths, head_num, head_dim]");
        for (const TensorView* t : {&kv, &vv, &o}) {
            B200_REQUIRE(t->ndim == 3 && t->shape[0] == qv.shape[0] && t->shape[1] == qv.shape[1] && t->shape[2] == qv.shape[2],
                         "q, k, v and out must share the shape [%ld, %ld, %ld]", (long)qv.shape[0], (long)qv.shape[1], (long)qv.shape[2]);
            B200_REQUIRE(t->shape[2] == 1 || t->stride[2] == 1, "the last dim of q, k, v and out must be dense");
        }
        B200_REQUIRE(qv.shape[2] == 1 || qv.stride[2] == 1, "the last dim of q, k, v and out must be dense");
        a.total_rows = qv.shape[0];
        a.H = static_cast<int>(qv.shape[1]);
        a.D = static_cast<int>(qv.shape[2]);
        B200_REQUIRE(a.D <= 256, "head_dim %d is beyond the supported maximum of 256", a.D);
        a.b_start = index_arg(bs, "b_start_loc", 1);
        a.b_len = index_arg(bn, "b_seq_len", 1);
        a.B = static_cast<int>(bs.shape[0]);
        B200_REQUIRE(bn.shape[0] == a.B, "'b_start_loc' and 'b_seq_len' differ in length");
        a.max_input_len = max_input_len;
        a.q = qv.data;
        a.kmat = kv.data;
        a.vmat = vv.data;
        a.out = o.data;
        a.q_s0 = qv.stride[0];
        a.q_s1 = qv.stride[1];
        a.k_s0 = kv.stride[0];
        a.k_s1 = kv.stride[1];
        a.v_s0 = vv.stride[0];
        a.v_s1 = vv.stride[1];
        a.o_s0 = o.stride[0];
        a.o_s1 = o.stride[1];
        if (qv.numel == 0 || a.B == 0) return;
        cudaStream_t st = stream_of(ctx);
        const DeviceInfo& di = device_info();
        const char* path = k::launch_prefill(a, di.sm_count, di.max_smem_optin, st);
        logf("prefill B=%d H=%d D=%d rows=%ld kv_group=%d: %s kernel", a.B, a.H, a.D, (long)a.total_rows, a.kv_group, path);
        B200_CUDA(cudaGetLastError());
    });
}

B200_EXPORT diopiError_t diopiApplyPenalty(diopiContextHandle_t ctx, diopiTensorHandle_t logits, diopiConstTensorHandle_t presence_penalty,
                                           diopiConstTensorHandle_t frequency_penalty, diopiConstTensorHandle_t p_token_ids,
                                           diopiConstTensorHandle_t p_token_counts, diopiConstTensorHandle_t p_cumsum_seq_len, int /*p_max_len_in_batch*/) {
    return guard("diopiApplyPenalty", [&] {
        flush_pending(ctx);
        TensorView lg = view_of(logits, "logits"), pp = view_of(presence_penalty, "presence_penalty"), fp = view_of(frequency_penalty, "frequency_penalty");
        TensorView ids = view_of(p_token_ids, "p_token_ids"), cnt = view_of(p_token_counts, "p_token_counts"), cum = view_of(p_cumsum_seq_len, "p_cumsum_seq_len");
        k::PenaltyArgs a{};
        a.dt = float_dt(lg, "logits", true);
        same_dtype(pp, "presence_penalty", lg, "logits");
        same_dtype(fp, "frequency_penalty", lg, "logits");
        B200_REQUIRE(lg.ndim == 2, "'logits' must be [batch, vocab], got %d dims", lg.ndim);
        a.B = lg.shape[0];
        a.V = lg.shape[1];
        B200_REQUIRE(pp.ndim == 1 && fp.ndim == 1 && pp.shape[0] == a.B && fp.shape[0] == a.B, "the penalties must be [batch = %ld]", (long)a.B);
        a.ids = index_arg(ids, "p_token_ids", 1);
        a.counts = index_arg(cnt, "p_token_counts", 1);
        a.cum = index_arg(cum, "p_cumsum_seq_len", 1);
        B200_REQUIRE(ids.shape[0] == cnt.shape[0], "'p_token_ids' and 'p_token_counts' differ in length");
        B200_REQUIRE(cum.shape[0] == a.B + 1, "'p_cumsum_seq_len' must have batch + 1 = %ld entries, got %ld", (long)(a.B + 1), (long)cum.shape[0]);
        a.E = ids.shape[0];
        a.logits = lg.data;
        a.l_s0 = lg.stride[0];
        a.l_s1 = lg.stride[1];
        a.presence = pp.data;
        a.p_s = pp.stride[0];
        a.frequency = fp.data;
        a.f_s = fp.stride[0];
        if (a.E == 0 || a.B == 0 || a.V == 0) return;
        cudaStream_t st = stream_of(ctx);
        a.status = async_status_device_ptr();
        k::launch_apply_penalty(a, st);
        B200_CUDA(cudaGetLastError());
    });
}

B200_EXPORT diopiError_t diopiRotaryEmbedding(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t x, diopiConstTensorHandle_t cos,
                                              diopiConstTensorHandle_t sin, const bool conj, const bool interleaved) {
    return guard("diopiRotaryEmbedding", [&] {
        flush_pending(ctx);
        if (interleaved) fail(diopiNoImplement, "interleaved rotary embedding is not implemented (nor is it in the reference's CUDA backend)");
        TensorView o = view_of(out, "out"), xv = view_of(x, "x"), cv = view_of(cos, "cos"), sv = view_of(sin, "sin");
        k::RopeArgs a{};
        a.dt = float_dt(xv, "x", true);
        same_dtype(o, "out", xv, "x");
        same_dtype(cv, "cos", xv, "x");
        same_dtype(sv, "sin", xv, "x");
        B200_REQUIRE(xv.ndim >= 1, "'x' must have at least one dim");
        B200_REQUIRE(o.ndim == xv.ndim, "'out' must have the shape of 'x'");
        for (int i = 0; i < xv.ndim; ++i) B200_REQUIRE(o.shape[i] == xv.shape[i], "'out' must have the shape of 'x'");
        const int64_t D = xv.shape[xv.ndim - 1];
        B200_REQUIRE(D % 2 == 0, "the last dim of 'x' (%ld) must be even", (long)D);
        a.half = D / 2;
        B200_REQUIRE(cv.ndim >= 1 && sv.ndim >= 1 && cv.ndim <= xv.ndim && sv.ndim <= xv.ndim, "'cos'/'sin' must have between 1 and %d dims", xv.ndim);
        B200_REQUIRE(cv.shape[cv.ndim - 1] == a.half && sv.shape[sv.ndim - 1] == a.half, "the last dim of 'cos'/'sin' must be %ld", (long)a.half);
        if (xv.numel == 0) return;
        // Leading dims of x, with the matching (right-aligned) stride of cos/sin, 0 where they broadcast.
        const int nl = xv.ndim - 1;
        int64_t size[kMaxDims], xs[kMaxDims], os[kMaxDims], cs[kMaxDims], ss[kMaxDims];
        for (int i = 0; i < nl; ++i) {
            size[i] = xv.shape[i];
            xs[i] = xv.stride[i];
            os[i] = o.stride[i];
            auto bstride = [&](const TensorView& t, const char* name) -> int64_t {
                const int ti = i - (xv.ndim - t.ndim);
                if (ti < 0) return 0;
                if (t.shape[ti] == 1) return 0;
                B200_REQUIRE(t.shape[ti] == xv.shape[i], "'%s' dim %d (%ld) does not broadcast against 'x' dim %d (%ld)", name, ti, (long)t.shape[ti], i,
                             (long)xv.shape[i]);
                return t.stride[ti];
            };
            cs[i] = bstride(cv, "cos");
            ss[i] = bstride(sv, "sin");
        }
        // Collapse neighbouring dims that walk memory uniformly in all four tensors; drop dims of extent 1.
        int nd = 0;
        for (int i = 0; i < nl; ++i) {
            if (size[i] == 1) continue;
            if (nd > 0 && xs[nd - 1] == size[i] * xs[i] && os[nd - 1] == size[i] * os[i] && cs[nd - 1] == size[i] * cs[i] && ss[nd - 1] == size[i] * ss[i]) {
                size[nd - 1] *= size[i];
                xs[nd - 1] = xs[i];
                os[nd - 1] = os[i];
                cs[nd - 1] = cs[i];
                ss[nd - 1] = ss[i];
            } else {
                size[nd] = size[i];
                xs[nd] = xs[i];
                os[nd] = os[i];
                cs[nd] = cs[i];
                ss[nd] = ss[i];
                ++nd;
            }
        }
        B200_REQUIRE(nd <= k::kRopeMaxDims, "'x' needs %d independent leading dims; at most %d are supported", nd, k::kRopeMaxDims);
        a.nd = nd;
        a.n_lead = 1;
        for (int i = 0; i < nd; ++i) {
            a.size[i] = size[i];
            a.xs[i] = xs[i];
            a.os[i] = os[i];
            a.cs[i] = cs[i];
            a.ss[i] = ss[i];
            a.n_lead *= size[i];
        }
        a.x = xv.data;
        a.out = o.data;
        a.cos = cv.data;
        a.sin = sv.data;
        a.x_ls = xv.stride[xv.ndim - 1];
        a.o_ls = o.stride[o.ndim - 1];
        a.c_ls = cv.stride[cv.ndim - 1];
        a.s_ls = sv.stride[sv.ndim - 1];
        a.conj = conj;
        cudaStream_t st = stream_of(ctx);
        k::launch_rope(a, st);
        B200_CUDA(cudaGetLastError());
    });
}

B200_EXPORT diopiError_t diopiRMSNorm(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiTensorHandle_t inv_rms, diopiConstTensorHandle_t input,
                                      diopiSize_t normalized_shape, diopiConstTensorHandle_t weight, diopiConstTensorHandle_t bias, double eps) {
    return guard("diopiRMSNorm", [&] {
        flush_pending(ctx);
        TensorView o = view_of(out, "out"), iv = view_of(inv_rms, "inv_rms"), xv = view_of(input, "input"), wv = view_of(weight, "weight");
        TensorView bv = view_of(bias, "bias", /*optional=*/true);
        k::RmsNormArgs a{};
        a.dt = float_dt(xv, "input", true);
        same_dtype(o, "out", xv, "input");
        same_dtype(wv, "weight", xv, "input");
        if (bv.defined) same_dtype(bv, "bias", xv, "input");
        B200_REQUIRE(normalized_shape.len >= 1 && normalized_shape.len <= xv.ndim && normalized_shape.data != nullptr,
                     "normalized_shape must name between 1 and %d trailing dims", xv.ndim);
        int64_t n2 = 1;
        for (int64_t i = 0; i < normalized_shape.len; ++i) {
            const int64_t want = normalized_shape.data[i];
            const int64_t have = xv.shape[xv.ndim - normalized_shape.len + i];
            B200_REQUIRE(want == have, "normalized_shape[%ld] = %ld does not match the input's trailing dim %ld", (long)i, (long)want, (long)have);
            n2 *= want;
        }
        a.n2 = n2;
        a.n1 = n2 > 0 ? xv.numel / n2 : 0;
        B200_REQUIRE(o.numel == xv.numel, "'out' must have the shape of 'input'");
        B200_REQUIRE(wv.numel == n2, "'weight' must have %ld elements (normalized_shape), got %ld", (long)n2, (long)wv.numel);
        if (bv.defined) B200_REQUIRE(bv.numel == n2, "'bias' must have %ld elements (normalized_shape), got %ld", (long)n2, (long)bv.numel);
        if (xv.numel == 0) return;
        B200_REQUIRE(iv.numel == a.n1, "'inv_rms' must have one element per normalised row (%ld), got %ld", (long)a.n1, (long)iv.numel);
        B200_REQUIRE(xv.contiguous() && o.contiguous() && wv.contiguous() && iv.contiguous() && (!bv.defined || bv.contiguous()),
                     "input, out, weight, bias and inv_rms must be contiguous");
        if (iv.dtype == diopi_dtype_float32)
            a.inv_dt = k::Dt::F32;
        else if (iv.dtype == xv.dtype)
            a.inv_dt = a.dt;
        else
            fail(diopiDtypeNotSupported, "'inv_rms' has dtype %s; expected float32 or the input's dtype (%s)", dtype_name(iv.dtype), dtype_name(xv.dtype));
        a.x = xv.data;
        a.weight = wv.data;
        a.bias = bv.defined ? bv.data : nullptr;
        a.out = o.data;
        a.inv_rms = iv.data;
        a.eps = eps;
        cudaStream_t st = stream_of(ctx);
        const DeviceInfo& di = device_info();
        k::launch_rms_norm(a, di.sm_count, st);
        B200_CUDA(cudaGetLastError());
    });
}

// The step in front of decode attention as one call (an addition to the reference's operator set):
//   diopiRotaryEmbedding(q_out, q, cos, sin, conj, false);
//   diopiRotaryEmbedding(tmp, k, cos, sin, conj, false); diopiDestIndexCopyKV(k_pool, tmp, dest_loc);
//   diopiDestIndexCopyKV(v_pool, v, dest_loc);            (skipped when v and v_pool are null)
// with bit-identical results. Dense [tokens, heads, head_dim] rows with one cos/sin row of head_dim/2 per token run
// as one kernel that never materialises the rotated key; anything else runs the calls above on context scratch.
B200_EXPORT diopiError_t diopiRotaryEmbeddingCopyKV(diopiContextHandle_t ctx, diopiTensorHandle_t q_out, diopiTensorHandle_t k_pool, diopiTensorHandle_t v_pool,
                                                    diopiConstTensorHandle_t q, diopiConstTensorHandle_t kh, diopiConstTensorHandle_t vh,
                                                    diopiConstTensorHandle_t cos, diopiConstTensorHandle_t sin, diopiConstTensorHandle_t dest_loc, bool conj) {
    bool composed = false;
    diopiError_t rc = guard("diopiRotaryEmbeddingCopyKV", [&] {
        flush_pending(ctx);
        TensorView qo = view_of(q_out, "q_out"), kp = view_of(k_pool, "k_pool"), qv = view_of(q, "q"), kv = view_of(kh, "k");
        TensorView cv = view_of(cos, "cos"), sv = view_of(sin, "sin"), d = view_of(dest_loc, "dest_loc");
        TensorView vp = view_of(v_pool, "v_pool", /*optional=*/true), vv = view_of(vh, "v", /*optional=*/true);
        B200_REQUIRE(vp.defined == vv.defined, "'v' and 'v_pool' must be given together or both be null");
        k::RopeStoreArgs a{};
        a.dt = float_dt(qv, "q", true);
        same_dtype(qo, "q_out", qv, "q");
        same_dtype(kv, "k", qv, "q");
        same_dtype(kp, "k_pool", qv, "q");
        same_dtype(cv, "cos", qv, "q");
        same_dtype(sv, "sin", qv, "q");
        if (vv.defined) {
            same_dtype(vv, "v", qv, "q");
            same_dtype(vp, "v_pool", qv, "q");
        }
        B200_REQUIRE(qv.ndim == 3 && kv.ndim == 3 && qo.ndim == 3 && kp.ndim == 3, "'q', 'q_out', 'k' and 'k_pool' must be [rows, head_num, head_dim]");
        const int64_t T = qv.shape[0], D = qv.shape[2];
        B200_REQUIRE(kv.shape[0] == T && kv.shape[2] == D && kp.shape[2] == D && kp.shape[1] == kv.shape[1], "'k' must be [%ld, kv_heads, %ld] and 'k_pool' [slots, kv_heads, %ld]",
                     (long)T, (long)D, (long)D);
        for (int i = 0; i < 3; ++i) B200_REQUIRE(qo.shape[i] == qv.shape[i], "'q_out' must have the shape of 'q'");
        if (vv.defined) {
            B200_REQUIRE(vv.ndim == 3 && vp.ndim == 3, "'v' and 'v_pool' must be [rows, head_num, head_dim]");
            for (int i = 0; i < 3; ++i) B200_REQUIRE(vv.shape[i] == kv.shape[i], "'v' must have the shape of 'k'");
            for (int i = 0; i < 3; ++i) B200_REQUIRE(vp.shape[i] == kp.shape[i], "'v_pool' must have the shape of 'k_pool'");
        }
        B200_REQUIRE(D % 2 == 0, "head_dim (%ld) must be even", (long)D);
        a.dest = index_arg(d, "dest_loc", 1);
        B200_REQUIRE(d.shape[0] == T, "'dest_loc' has %ld entries for %ld rows", (long)d.shape[0], (long)T);
        if (T == 0 || D == 0) return;
        B200_REQUIRE(kp.shape[0] > 0, "'k_pool' has no slots");
        auto dense = [](const TensorView& t) { return (t.shape[2] == 1 || t.stride[2] == 1) && (t.shape[1] == 1 || t.stride[1] == t.shape[2]); };
        // cos/sin: exactly one row of D/2 per token ([T, D/2] or [T, 1, D/2]), last dim dense
        auto table = [&](const TensorView& t, int64_t& s0) {
            if (t.numel != T * (D / 2) || t.shape[t.ndim - 1] != D / 2 || t.shape[0] != T) return false;
            if (D / 2 > 1 && t.stride[t.ndim - 1] != 1) return false;
            s0 = t.stride[0];
            return true;
        };
        const bool one_kernel = dense(qv) && dense(qo) && dense(kv) && dense(kp) && (!vv.defined || (dense(vv) && dense(vp))) && table(cv, a.c_s0) &&
                                table(sv, a.s_s0);
        if (one_kernel) {
            a.q = qv.data; a.q_out = qo.data; a.k = kv.data; a.k_pool = kp.data;
            a.v = vv.defined ? vv.data : nullptr;
            a.v_pool = vp.defined ? vp.data : nullptr;
            a.cos = cv.data; a.sin = sv.data;
            a.T = T; a.Hq = qv.shape[1]; a.Hk = kv.shape[1]; a.D = D; a.slots = kp.shape[0];
            a.q_s0 = qv.stride[0]; a.qo_s0 = qo.stride[0]; a.k_s0 = kv.stride[0]; a.kp_s0 = kp.stride[0];
            a.v_s0 = vv.defined ? vv.stride[0] : 0;
            a.vp_s0 = vp.defined ? vp.stride[0] : 0;
            a.conj = conj;
            a.status = async_status_device_ptr();
            cudaStream_t st = stream_of(ctx);
            if (k::launch_rope_store_kv(a, st)) {
                B200_CUDA(cudaGetLastError());
                return;
            }
        }
        composed = true;
    });
    if (rc != diopiSuccess || !composed) return rc;
    // The separate calls, each with its own checks and error text.
    rc = diopiRotaryEmbedding(ctx, q_out, q, cos, sin, conj, false);
    if (rc != diopiSuccess) return rc;
    diopiTensorHandle_t tmp = nullptr;
    diopiSize_t shape{nullptr, 0};
    diopiDtype_t dt;
    if (diopiGetTensorShape(kh, &shape) != diopiSuccess || diopiGetTensorDtype(kh, &dt) != diopiSuccess ||
        diopiRequireTensor(ctx, &tmp, &shape, nullptr, dt, diopi_device) != diopiSuccess || tmp == nullptr)
        return guard("diopiRotaryEmbeddingCopyKV", [&] { fail(diopiErrorOccurred, "the consumer could not provide a scratch tensor for the rotated key"); });
    rc = diopiRotaryEmbedding(ctx, tmp, kh, cos, sin, conj, false);
    if (rc != diopiSuccess) return rc;
    rc = diopiDestIndexCopyKV(ctx, k_pool, tmp, dest_loc);
    if (rc != diopiSuccess || vh == nullptr) return rc;
    return diopiDestIndexCopyKV(ctx, v_pool, vh, dest_loc);
}

// diopiRMSNormBackward (proto/include/diopi/functions_ext.h:62-65). `eps` and `bias` carry no information the
// derivative needs (inv_rms is given); grad_bias may be null when the forward call had no bias.
B200_EXPORT diopiError_t diopiRMSNormBackward(diopiContextHandle_t ctx, diopiTensorHandle_t grad_input, diopiTensorHandle_t grad_weight,
                                              diopiTensorHandle_t grad_bias, diopiConstTensorHandle_t grad_output, diopiConstTensorHandle_t input,
                                              diopiConstTensorHandle_t weight, diopiConstTensorHandle_t bias, diopiConstTensorHandle_t inv_rms,
                                              diopiSize_t normalized_shape, double /*eps*/) {
    return guard("diopiRMSNormBackward", [&] {
        flush_pending(ctx);
        TensorView dx = view_of(grad_input, "grad_input"), dw = view_of(grad_weight, "grad_weight"), gv = view_of(grad_output, "grad_output");
        TensorView xv = view_of(input, "input"), wv = view_of(weight, "weight"), iv = view_of(inv_rms, "inv_rms");
        TensorView db = view_of(grad_bias, "grad_bias", /*optional=*/true), bv = view_of(bias, "bias", /*optional=*/true);
        k::RmsNormBwdArgs a{};
        a.dt = float_dt(xv, "input", true);
        same_dtype(dx, "grad_input", xv, "input");
        same_dtype(gv, "grad_output", xv, "input");
        same_dtype(wv, "weight", xv, "input");
        same_dtype(dw, "grad_weight", xv, "input");
        if (db.defined) same_dtype(db, "grad_bias", xv, "input");
        B200_REQUIRE(normalized_shape.len >= 1 && normalized_shape.len <= xv.ndim && normalized_shape.data != nullptr,
                     "normalized_shape must name between 1 and %d trailing dims", xv.ndim);
        int64_t n2 = 1;
        for (int64_t i = 0; i < normalized_shape.len; ++i) {
            const int64_t want = normalized_shape.data[i];
            const int64_t have = xv.shape[xv.ndim - normalized_shape.len + i];
            B200_REQUIRE(want == have, "normalized_shape[%ld] = %ld does not match the input's trailing dim %ld", (long)i, (long)want, (long)have);
            n2 *= want;
        }
        a.n2 = n2;
        a.n1 = n2 > 0 ? xv.numel / n2 : 0;
        B200_REQUIRE(dx.numel == xv.numel && gv.numel == xv.numel, "'grad_input' and 'grad_output' must have the shape of 'input'");
        B200_REQUIRE(wv.numel == n2 && dw.numel == n2, "'weight' and 'grad_weight' must have %ld elements (normalized_shape)", (long)n2);
        if (db.defined) B200_REQUIRE(db.numel == n2, "'grad_bias' must have %ld elements (normalized_shape), got %ld", (long)n2, (long)db.numel);
        if (bv.defined) B200_REQUIRE(bv.numel == n2, "'bias' must have %ld elements (normalized_shape), got %ld", (long)n2, (long)bv.numel);
        if (n2 == 0) return;
        B200_REQUIRE(iv.numel == a.n1, "'inv_rms' must have one element per normalised row (%ld), got %ld", (long)a.n1, (long)iv.numel);
        B200_REQUIRE(xv.contiguous() && gv.contiguous() && dx.contiguous() && wv.contiguous() && dw.contiguous() && iv.contiguous() &&
                         (!db.defined || db.contiguous()),
                     "grad_input, grad_weight, grad_bias, grad_output, input, weight and inv_rms must be contiguous");
        if (iv.dtype == diopi_dtype_float32)
            a.inv_dt = k::Dt::F32;
        else if (iv.dtype == xv.dtype)
            a.inv_dt = a.dt;
        else
            fail(diopiDtypeNotSupported, "'inv_rms' has dtype %s; expected float32 or the input's dtype (%s)", dtype_name(iv.dtype), dtype_name(xv.dtype));
        a.g = gv.data;
        a.x = xv.data;
        a.weight = wv.data;
        a.inv_rms = iv.data;
        a.dx = dx.data;
        a.dw = dw.data;
        a.db = db.defined ? db.data : nullptr;
        cudaStream_t st = stream_of(ctx);
        const DeviceInfo& di = device_info();
        a.parts = k::rms_norm_bwd_parts(a, di.sm_count);
        if (a.parts > 0) a.ws = static_cast<float*>(workspace(ctx, static_cast<int64_t>(2) * a.parts * a.n2 * static_cast<int64_t>(sizeof(float))));
        k::launch_rms_norm_bwd(a, st);
        B200_CUDA(cudaGetLastError());
    });
}

// ---------------------------------------------------------------------------------------------
// The fused decode step for callers that cannot hand out scratch memory.
//
// diopiTokenDecodeAttentionInference asks the caller's context (diopiRequireBuffer /
// diopiRequireTensor) for the few MB its split-KV partials need. Some callers cannot answer that:
// a serving engine that gave every free byte of HBM to its KV pool at start-up and runs its decode
// loop with no allocator behind the context, or a thin C harness that implements the tensor
// accessors but leaves diopiRequireTensor returning an error. This entry point runs the same
// kernels on a fixed 8 MiB array inside the library's device image instead. It calls no
// cudaMalloc/cudaFree/cudaHostAlloc and never calls back into diopiRequire*.
//
// Limits and rules, all checked or stated here:
//  * (148 + batch) * head_num * (head_dim + 2) * 4 bytes must fit in 8 MiB (e.g. batch <= 356 at
//    32 heads x 128); larger problems are refused with an error that names both numbers. Shapes that
//    the scratch-free plain path serves (odd head_dim, strided rows) have no such limit.
//  * The first call on each device looks up the array's address (cudaGetSymbolAddress); make that
//    first call during start-up, before any stream capture begins.
//  * All calls on a device share the one array. It needs no clearing between calls, but two calls
//    that may run on the GPU at the same time (different streams) race on it: keep them on one stream
//    or order them with events.
//  * Out-of-range slot indices are still skipped, but are only reported through the status word if
//    an earlier ordinary call created that word; this entry point does not create it.
B200_EXPORT diopiError_t diopiTokenDecodeAttentionInferenceNoAlloc(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t q,
                                                                   diopiConstTensorHandle_t kh, diopiConstTensorHandle_t v, diopiConstTensorHandle_t b_loc,
                                                                   diopiConstTensorHandle_t b_start_loc, diopiConstTensorHandle_t b_seq_len,
                                                                   int max_input_len) {
    return guard("diopiTokenDecodeAttentionInferenceNoAlloc", [&] {
        TensorView o = view_of(out, "out"), qv = view_of(q, "q"), kv = view_of(kh, "k"), vv = view_of(v, "v");
        TensorView bl = view_of(b_loc, "b_loc"), bs = view_of(b_start_loc, "b_start_loc"), bn = view_of(b_seq_len, "b_seq_len");
        k::DecodeArgs a{};
        a.mode = k::DecodeMode::FUSED;
        a.force_plain = options().decode_plain;
        a.dt = float_dt(kv, "k", false);
        B200_REQUIRE(kv.ndim == 3 && vv.ndim == 3 && qv.ndim == 3 && o.ndim == 3, "q, k, v and out must have 3 dims");
        a.H = static_cast<int>(kv.shape[1]);
        a.D = static_cast<int>(kv.shape[2]);
        a.slots = kv.shape[0];
        B200_REQUIRE(bl.ndim == 2, "'b_loc' must be [batch, N], got %d dims", bl.ndim);
        a.B = static_cast<int>(bl.shape[0]);
        B200_REQUIRE(max_input_len >= 0 && bl.shape[1] >= max_input_len, "'b_loc' has %ld columns for max_input_len = %d", (long)bl.shape[1], max_input_len);
        a.max_input_len = max_input_len;
        a.b_loc = index_arg(bl, "b_loc", 2);
        a.b_start = index_arg(bs, "b_start_loc", 1);
        a.b_len = index_arg(bn, "b_seq_len", 1);
        B200_REQUIRE(bs.shape[0] == a.B && bn.shape[0] == a.B, "'b_start_loc' and 'b_seq_len' must have batch = %d entries", a.B);
        B200_REQUIRE(a.D <= 512, "head_dim %d is beyond the supported maximum of 512", a.D);
        same_dtype(qv, "q", kv, "k");
        same_dtype(vv, "v", kv, "k");
        same_dtype(o, "out", kv, "k");
        B200_REQUIRE(qv.shape[0] == a.B && qv.shape[1] == a.H && qv.shape[2] == a.D, "'q' must be [%d, %d, %d]", a.B, a.H, a.D);
        B200_REQUIRE(o.shape[0] == a.B && o.shape[1] == a.H && o.shape[2] == a.D, "'out' must be [%d, %d, %d]", a.B, a.H, a.D);
        B200_REQUIRE(vv.shape[0] == kv.shape[0] && vv.shape[1] == a.H && vv.shape[2] == a.D, "'v' must have the shape of 'k'");
        a.q = qv.data;
        a.q_s0 = qv.stride[0];
        a.q_s1 = qv.stride[1];
        a.q_s2 = qv.stride[2];
        a.kmat = kv.data;
        a.k_s0 = kv.stride[0];
        a.k_s1 = kv.stride[1];
        a.k_s2 = kv.stride[2];
        a.vmat = vv.data;
        a.v_s0 = vv.stride[0];
        a.v_s1 = vv.stride[1];
        a.v_s2 = vv.stride[2];
        a.out = o.data;
        a.out_s0 = o.stride[0];
        a.out_s1 = o.stride[1];
        a.out_s2 = o.stride[2];
        if (a.B == 0 || a.H == 0 || a.D == 0) return;
        B200_REQUIRE(a.slots > 0 || max_input_len == 0, "the K/V pool has no slots");
        cudaStream_t st = stream_of(ctx);
        if (max_input_len == 0) {
            B200_REQUIRE(o.contiguous(), "'out' must be contiguous when every request is empty");
            B200_CUDA(cudaMemsetAsync(o.data, 0, static_cast<size_t>(o.numel * o.elem_size()), st));
            return;
        }
        const DeviceInfo& di = device_info();
        a.status = async_status_device_ptr_if_ready();
        int64_t needed = 0;
        cudaError_t e = k::launch_decode_static_scratch(a, di.sm_count, di.max_smem_optin, st, &needed);
        if (e == cudaErrorMemoryAllocation)
            fail(diopiErrorOccurred,
                 "this problem needs %ld bytes of split-KV scratch but the built-in array holds %ld; use diopiTokenDecodeAttentionInference "
                 "(scratch from the context) or a smaller batch",
                 (long)needed, (long)k::decode_static_scratch_capacity());
        B200_CUDA(e);
        B200_CUDA(cudaGetLastError());
    });
}

// ---------------------------------------------------------------------------------------------
// The newer lightllm call forms of rotary embedding and penalty.
B200_EXPORT diopiError_t diopiRotaryEmbeddingV2(diopiContextHandle_t ctx, diopiTensorHandle_t query, diopiTensorHandle_t key, diopiConstTensorHandle_t cos,
                                                diopiConstTensorHandle_t sin, int64_t dim) {
    return guard("diopiRotaryEmbeddingV2", [&] {
        flush_pending(ctx);
        TensorView qv = view_of(query, "query"), kv = view_of(key, "key"), cv = view_of(cos, "cos"), sv = view_of(sin, "sin");
        k::RopeV2Args a{};
        a.dt = float_dt(qv, "query", true);
        same_dtype(kv, "key", qv, "query");
        same_dtype(cv, "cos", qv, "query");
        same_dtype(sv, "sin", qv, "query");
        B200_REQUIRE(dim > 0 && dim % 2 == 0, "dim (%ld) must be positive and even", (long)dim);
        B200_REQUIRE(qv.ndim == 2 && kv.ndim == 2 && qv.shape[0] == kv.shape[0], "'query' and 'key' must be [tokens, heads * dim] with the same tokens");
        B200_REQUIRE(qv.shape[1] % dim == 0 && kv.shape[1] % dim == 0, "the width of 'query'/'key' must be a multiple of dim = %ld", (long)dim);
        B200_REQUIRE((qv.shape[1] == 1 || qv.stride[1] == 1) && (kv.shape[1] == 1 || kv.stride[1] == 1), "rows of 'query' and 'key' must be dense");
        a.T = qv.shape[0];
        a.dim = dim;
        a.q_heads = qv.shape[1] / dim;
        a.k_heads = kv.shape[1] / dim;
        a.q = qv.data;
        a.q_s0 = qv.stride[0];
        a.kk = kv.data;
        a.k_s0 = kv.stride[0];
        // cos/sin: [tokens or 1, (1,) dim]; a middle head dim may be 1 (broadcast) or match both head counts
        auto table = [&](const TensorView& t, const char* name, int64_t& st, int64_t& sh) {
            B200_REQUIRE(t.ndim == 2 || t.ndim == 3, "'%s' must be [tokens, dim] or [tokens, 1, dim]", name);
            B200_REQUIRE(t.shape[t.ndim - 1] == dim && (dim == 1 || t.stride[t.ndim - 1] == 1), "the last dim of '%s' must be dim = %ld and dense", name, (long)dim);
            B200_REQUIRE(t.shape[0] == a.T || t.shape[0] == 1, "'%s' has %ld rows for %ld tokens", name, (long)t.shape[0], (long)a.T);
            st = t.shape[0] == 1 ? 0 : t.stride[0];
            sh = 0;
            if (t.ndim == 3 && t.shape[1] != 1) {
                B200_REQUIRE(t.shape[1] == a.q_heads && t.shape[1] == a.k_heads, "'%s' has %ld heads; expected 1 or the head count of query and key", name,
                             (long)t.shape[1]);
                sh = t.stride[1];
            }
        };
        table(cv, "cos", a.c_st, a.c_sh);
        table(sv, "sin", a.s_st, a.s_sh);
        a.cos = cv.data;
        a.sin = sv.data;
        if (a.T == 0 || (qv.numel == 0 && kv.numel == 0)) return;
        cudaStream_t st = stream_of(ctx);
        k::launch_rope_v2(a, st);
        B200_CUDA(cudaGetLastError());
    });
}

B200_EXPORT diopiError_t diopiApplyPenaltyV2(diopiContextHandle_t ctx, diopiTensorHandle_t logits, diopiConstTensorHandle_t presence_penalty,
                                             diopiConstTensorHandle_t frequency_penalty, diopiConstTensorHandle_t repetition_penalty,
                                             diopiConstTensorHandle_t p_token_ids, diopiConstTensorHandle_t p_token_counts) {
    return guard("diopiApplyPenaltyV2", [&] {
        flush_pending(ctx);
        TensorView lg = view_of(logits, "logits"), pp = view_of(presence_penalty, "presence_penalty"), fp = view_of(frequency_penalty, "frequency_penalty");
        TensorView rp = view_of(repetition_penalty, "repetition_penalty"), ids = view_of(p_token_ids, "p_token_ids"), cnt = view_of(p_token_counts, "p_token_counts");
        k::PenaltyV2Args a{};
        a.dt = float_dt(lg, "logits", true);
        same_dtype(pp, "presence_penalty", lg, "logits");
        same_dtype(fp, "frequency_penalty", lg, "logits");
        same_dtype(rp, "repetition_penalty", lg, "logits");
        a.ids = index_arg(ids, "p_token_ids", 1);
        a.counts = index_arg(cnt, "p_token_counts", 1);
        a.E = ids.shape[0];
        B200_REQUIRE(cnt.shape[0] == a.E, "'p_token_ids' and 'p_token_counts' differ in length");
        for (const TensorView* t : {&pp, &fp, &rp}) B200_REQUIRE(t->ndim == 1 && t->shape[0] == a.E, "the penalties must have one entry per token id (%ld)", (long)a.E);
        B200_REQUIRE(lg.contiguous(), "'logits' must be contiguous (it is indexed as a flat array)");
        a.logits = lg.data;
        a.numel = lg.numel;
        a.presence = pp.data;
        a.p_s = pp.stride[0];
        a.frequency = fp.data;
        a.f_s = fp.stride[0];
        a.repetition = rp.data;
        a.r_s = rp.stride[0];
        if (a.E == 0 || a.numel == 0) return;
        cudaStream_t st = stream_of(ctx);
        a.status = async_status_device_ptr();
        k::launch_apply_penalty_v2(a, st);
        B200_CUDA(cudaGetLastError());
    });
}

// ---------------------------------------------------------------------------------------------
// Causal prefill over a padded batch in BSH layout: request i owns rows [i * max_input_len, (i + 1) * max_input_len)
// of query/key/value [batch * max_input_len, heads * dim]. Same kernels as diopiContextAttentionInference, with
// the request spans computed instead of read, and num_kv_heads < num_heads served as grouped-query attention.
// As in the golden function (customized_test.py:751-783), every one of the max_input_len rows of a request is
// computed under the causal mask; atten_mask is not read and actual_seq_lengths only gives the batch size.
B200_EXPORT diopiError_t diopiPromptFlashAttention(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t query,
                                                   diopiConstTensorHandle_t key, diopiConstTensorHandle_t value, diopiConstTensorHandle_t /*atten_mask*/,
                                                   diopiSize_t actual_seq_lengths, int64_t max_input_len, int64_t num_heads, int64_t num_kv_heads,
                                                   int64_t dim) {
    return guard("diopiPromptFlashAttention", [&] {
        flush_pending(ctx);
        TensorView o = view_of(out, "out"), qv = view_of(query, "query"), kv = view_of(key, "key"), vv = view_of(value, "value");
        k::PrefillArgs a{};
        a.force_simt = options().prefill_simt != 0;
        a.dt = float_dt(qv, "query", false);
        same_dtype(kv, "key", qv, "query");
        same_dtype(vv, "value", qv, "query");
        same_dtype(o, "out", qv, "query");
        B200_REQUIRE(num_heads > 0 && num_kv_heads > 0 && dim > 0 && num_heads % num_kv_heads == 0,
                     "num_heads (%ld) must be a positive multiple of num_kv_heads (%ld)", (long)num_heads, (long)num_kv_heads);
        B200_REQUIRE(dim <= 256, "dim %ld is beyond the supported maximum of 256", (long)dim);
        const int64_t B = actual_seq_lengths.len;
        B200_REQUIRE(B >= 0 && max_input_len >= 0, "batch and max_input_len must not be negative");
        const int64_t rows = B * max_input_len;
        auto rows_of = [&](const TensorView& t, const char* name, int64_t heads, int64_t& row_stride) {
            // [rows, heads*dim] or [batch, max_input_len, heads*dim], last dim dense, rows evenly spaced
            B200_REQUIRE(t.ndim == 2 || t.ndim == 3, "'%s' must be [batch*len, heads*dim] or [batch, len, heads*dim]", name);
            B200_REQUIRE(t.shape[t.ndim - 1] == heads * dim && (heads * dim == 1 || t.stride[t.ndim - 1] == 1), "the last dim of '%s' must be %ld and dense", name,
                         (long)(heads * dim));
            if (t.ndim == 2) {
                B200_REQUIRE(t.shape[0] == rows, "'%s' has %ld rows; expected batch * max_input_len = %ld", name, (long)t.shape[0], (long)rows);
                row_stride = t.stride[0];
            } else {
                B200_REQUIRE(t.shape[0] == B && t.shape[1] == max_input_len, "'%s' must be [%ld, %ld, *]", name, (long)B, (long)max_input_len);
                B200_REQUIRE(B <= 1 || t.stride[0] == t.shape[1] * t.stride[1], "the batch stride of '%s' must equal len * row stride", name);
                row_stride = t.stride[1];
            }
        };
        rows_of(qv, "query", num_heads, a.q_s0);
        rows_of(o, "out", num_heads, a.o_s0);
        rows_of(kv, "key", num_kv_heads, a.k_s0);
        rows_of(vv, "value", num_kv_heads, a.v_s0);
        a.q_s1 = a.k_s1 = a.v_s1 = a.o_s1 = dim;
        a.total_rows = rows;
        a.H = static_cast<int>(num_heads);
        a.D = static_cast<int>(dim);
        a.B = static_cast<int>(B);
        a.max_input_len = static_cast<int>(max_input_len);
        a.uniform_len = max_input_len;
        a.kv_group = static_cast<int>(num_heads / num_kv_heads);
        a.q = qv.data;
        a.kmat = kv.data;
        a.vmat = vv.data;
        a.out = o.data;
        if (rows == 0) return;
        cudaStream_t st = stream_of(ctx);
        const DeviceInfo& di = device_info();
        const char* path = k::launch_prefill(a, di.sm_count, di.max_smem_optin, st);
        logf("prefill B=%d H=%d D=%d rows=%ld kv_group=%d: %s kernel", a.B, a.H, a.D, (long)a.total_rows, a.kv_group, path);
        B200_CUDA(cudaGetLastError());
    });
}

// ---------------------------------------------------------------------------------------------
// Decode attention over a block-paged KV cache in BSH layout: one query token per request, token j of request i
// sits in row block_table[i, j / block_size] * block_size + j % block_size of key/value [rows, num_kv_heads*dim].
// The fused decode kernels do the work (split path when num_kv_heads == num_heads, plain path for grouped heads);
// the host-side lengths are staged into context scratch with one small asynchronous copy. atten_mask is not
// read (a decode token sees its whole prefix), as in the golden function (customized_test.py:785-821).
B200_EXPORT diopiError_t diopiPagedAttention(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t q, diopiConstTensorHandle_t kh,
                                             diopiConstTensorHandle_t v, diopiConstTensorHandle_t /*atten_mask*/, diopiSize_t actual_seq_lengths,
                                             int64_t num_heads, int64_t num_kv_heads, int64_t dim, diopiConstTensorHandle_t block_table,
                                             int64_t block_size) {
    return guard("diopiPagedAttention", [&] {
        flush_pending(ctx);
        TensorView o = view_of(out, "out"), qv = view_of(q, "q"), kv = view_of(kh, "k"), vv = view_of(v, "v"), bt = view_of(block_table, "block_table");
        k::DecodeArgs a{};
        a.mode = k::DecodeMode::FUSED;
        a.force_plain = options().decode_plain;
        a.dt = float_dt(qv, "q", false);
        same_dtype(kv, "k", qv, "q");
        same_dtype(vv, "v", qv, "q");
        same_dtype(o, "out", qv, "q");
        B200_REQUIRE(num_heads > 0 && num_kv_heads > 0 && dim > 0 && num_heads % num_kv_heads == 0,
                     "num_heads (%ld) must be a positive multiple of num_kv_heads (%ld)", (long)num_heads, (long)num_kv_heads);
        B200_REQUIRE(dim <= 512, "dim %ld is beyond the supported maximum of 512", (long)dim);
        B200_REQUIRE(block_size > 0 && block_size < (1ll << 30), "block_size must be positive (got %ld)", (long)block_size);
        const int64_t B = actual_seq_lengths.len;
        auto bsh = [&](const TensorView& t, const char* name, int64_t lead, int64_t heads, int64_t& s0) {
            // [lead, heads*dim] or [lead, 1, heads*dim]
            B200_REQUIRE((t.ndim == 2 || (t.ndim == 3 && t.shape[1] == 1)) && (lead < 0 || t.shape[0] == lead) && t.shape[t.ndim - 1] == heads * dim,
                         "'%s' must be [%s, %ld] (a middle dim of 1 is allowed)", name, lead < 0 ? "rows" : "batch", (long)(heads * dim));
            B200_REQUIRE(heads * dim == 1 || t.stride[t.ndim - 1] == 1, "the last dim of '%s' must be dense", name);
            s0 = t.stride[0];
        };
        bsh(qv, "q", B, num_heads, a.q_s0);
        bsh(o, "out", B, num_heads, a.out_s0);
        bsh(kv, "k", -1, num_kv_heads, a.k_s0);
        bsh(vv, "v", -1, num_kv_heads, a.v_s0);
        B200_REQUIRE(kv.shape[0] == vv.shape[0], "'k' and 'v' differ in row count");
        a.q_s1 = a.k_s1 = a.v_s1 = a.out_s1 = dim;
        a.q_s2 = a.k_s2 = a.v_s2 = a.out_s2 = 1;
        a.q = qv.data;
        a.kmat = kv.data;
        a.vmat = vv.data;
        a.out = o.data;
        a.B = static_cast<int>(B);
        a.H = static_cast<int>(num_heads);
        a.D = static_cast<int>(dim);
        a.slots = kv.shape[0];
        a.block_size = static_cast<int>(block_size);
        a.kv_group = static_cast<int>(num_heads / num_kv_heads);
        a.b_loc = index_arg(bt, "block_table", 2);
        B200_REQUIRE(bt.shape[0] == B, "'block_table' has %ld rows for a batch of %ld", (long)bt.shape[0], (long)B);
        if (B == 0) return;
        B200_REQUIRE(actual_seq_lengths.data != nullptr, "actual_seq_lengths has no data");
        int64_t longest = 0;
        for (int64_t i = 0; i < B; ++i) {
            const int64_t L = actual_seq_lengths.data[i];
            B200_REQUIRE(L >= 0 && L <= bt.shape[1] * block_size, "request %ld has length %ld but its block table covers %ld tokens", (long)i, (long)L,
                         (long)(bt.shape[1] * block_size));
            longest = L > longest ? L : longest;
        }
        B200_REQUIRE(longest < (1ll << 31), "sequence lengths must fit 31 bits");
        a.max_input_len = static_cast<int>(longest);
        cudaStream_t st = stream_of(ctx);
        if (longest == 0 || a.slots == 0) {
            B200_REQUIRE(longest == 0, "the K/V cache has no rows");
            B200_REQUIRE(o.contiguous(), "'out' must be contiguous when every request is empty");
            B200_CUDA(cudaMemsetAsync(o.data, 0, static_cast<size_t>(o.numel * o.elem_size()), st));
            return;
        }
        // lengths: host array -> context scratch (the copy reads the host array before it returns: pageable source)
        void* lens_dev = workspace(ctx, B * static_cast<int64_t>(sizeof(int64_t)));
        B200_CUDA(cudaMemcpyAsync(lens_dev, actual_seq_lengths.data, static_cast<size_t>(B) * sizeof(int64_t), cudaMemcpyHostToDevice, st));
        a.b_len.ptr = lens_dev;
        a.b_len.s0 = 1;
        a.b_len.is64 = 1;
        a.b_start = a.b_len;  // not read in fused mode
        const DeviceInfo& di = device_info();
        a.status = async_status_device_ptr();
        const int64_t ws_bytes = k::decode_workspace_bytes(a, di.sm_count, di.max_smem_optin);
        void* ws = ws_bytes > 0 ? workspace(ctx, ws_bytes) : nullptr;
        k::launch_decode(a, ws, di.sm_count, di.max_smem_optin, st);
        B200_CUDA(cudaGetLastError());
    });
}
