"""Python call forms of the ops, with the names and argument order of the reference's
wrappers (diopi_test/python/conformance/diopi_functions.py: rotary_emb 7030, rms_norm 7040,
apply_penalty 7851, destindex_copy_kv 7896, token_attention 7905, token_softmax_reducev 7914,
context_attention 7942). Each takes torch CUDA tensors, wraps them as DIOPI handles and makes
exactly one call through the C ABI of libdiopi_impl.so on torch's current stream.
"""
from __future__ import annotations

import torch

from . import _lib
from .runtime import Context, Sizes, Tensor, check_returncode, default_context


def _impl():
    return _lib.load().impl


def _t(x, as_device=None):
    if x is None or isinstance(x, Tensor):
        return x
    return Tensor(x, as_device=as_device)


def _h(x):
    return None if x is None else x.handle


def _call(name: str, ctx: Context | None, *args):
    ctx = ctx or default_context()
    rc = getattr(_impl(), name)(ctx.handle, *args)
    check_returncode(name, rc)


def vendor_name() -> str:
    return _impl().diopiGetVendorName().decode()


def impl_version() -> str:
    return _impl().diopiGetImplVersion().decode()


def last_error() -> str:
    return _impl().diopiGetLastErrorString().decode(errors="replace")


def set_option(name: str, value: int) -> None:
    """A process-wide switch of the library: log, fuse_token_attention, decode_plain, prefill_simt."""
    check_returncode("diopiB200SetOption", _impl().diopiB200SetOption(name.encode(), int(value)))


def destindex_copy_kv(k, dest_loc, out, *, ctx=None, as_device=None):
    """out[dest_loc] = k; returns out."""
    tk, td, to = _t(k, as_device), _t(dest_loc, as_device), _t(out, as_device)
    _call("diopiDestIndexCopyKV", ctx, _h(to), _h(tk), _h(td))
    return out


def token_attention(q, k, out, b_loc, b_start_loc, b_seq_len, max_input_len, *, ctx=None, as_device=None):
    """Decode logits into out [H, sum(L)]; returns out."""
    ts = [_t(x, as_device) for x in (out, q, k, b_loc, b_start_loc, b_seq_len)]
    _call("diopiTokenAttentionInference", ctx, *[_h(t) for t in ts], int(max_input_len))
    return out


def token_softmax_reducev(logics, v, out, b_loc, b_start_loc, b_seq_len, max_input_len, other_kv_index, *, ctx=None, as_device=None):
    """softmax(logics) @ v per request into out [B, H, D]; returns out."""
    ts = [_t(x, as_device) for x in (out, logics, v, b_loc, b_start_loc, b_seq_len)]
    _call("diopiTokenSoftmaxReduceVInference", ctx, *[_h(t) for t in ts], int(max_input_len), int(other_kv_index))
    return out


def token_decode_attention(q, k, v, out, b_loc, b_start_loc, b_seq_len, max_input_len, *, ctx=None, as_device=None):
    """The fused decode step (token_attention then token_softmax_reducev in one pass); returns out."""
    ts = [_t(x, as_device) for x in (out, q, k, v, b_loc, b_start_loc, b_seq_len)]
    _call("diopiTokenDecodeAttentionInference", ctx, *[_h(t) for t in ts], int(max_input_len))
    return out


def token_decode_attention_noalloc(q, k, v, out, b_loc, b_start_loc, b_seq_len, max_input_len, *, ctx=None, as_device=None):
    """The fused decode step on the library's built-in scratch array: for callers whose context cannot
    hand out device memory (no allocator behind diopiRequireTensor). Same result as token_decode_attention;
    refuses problems whose split-KV partials exceed the 8 MiB array. Returns out."""
    ts = [_t(x, as_device) for x in (out, q, k, v, b_loc, b_start_loc, b_seq_len)]
    _call("diopiTokenDecodeAttentionInferenceNoAlloc", ctx, *[_h(t) for t in ts], int(max_input_len))
    return out


def context_attention(q, k, v, out, b_start_loc, b_seq_len, max_input_len, *, ctx=None, as_device=None):
    """Causal prefill over the packed ragged batch; returns out."""
    ts = [_t(x, as_device) for x in (out, q, k, v, b_start_loc, b_seq_len)]
    _call("diopiContextAttentionInference", ctx, *[_h(t) for t in ts], int(max_input_len))
    return out


def prompt_flash_attention(query, key, value, attenMask, actualSeqLengths, maxInputLen, numHeads, numKeyValueHeads, dim, *, ctx=None, as_device=None):
    """Causal prefill over a padded BSH batch; returns a new tensor like query (diopi_functions.py:7951)."""
    out = torch.empty_like(query)
    ts = [_t(x, as_device) for x in (out, query, key, value, attenMask)]
    _call("diopiPromptFlashAttention", ctx, *[_h(t) for t in ts], Sizes(list(actualSeqLengths)), int(maxInputLen), int(numHeads),
          int(numKeyValueHeads), int(dim))
    return out


def paged_attention(query, key, value, attenMask, actualSeqLengths, numHeads, numKeyValueHeads, dim, blockTable, blockSize, *, ctx=None, as_device=None):
    """Decode attention over a block-paged KV cache (BSH); returns a new tensor like query (diopi_functions.py:7984)."""
    out = torch.empty_like(query)
    ts = [_t(x, as_device) for x in (out, query, key, value, attenMask)]
    tb = _t(blockTable, as_device)
    _call("diopiPagedAttention", ctx, *[_h(t) for t in ts], Sizes(list(actualSeqLengths)), int(numHeads), int(numKeyValueHeads), int(dim), _h(tb),
          int(blockSize))
    return out


def apply_penalty(logits, presence_penalty, frequency_penalty, p_token_ids, p_token_counts, p_cumsum_seq_len,
                  p_max_len_in_batch, *, ctx=None, as_device=None):
    """In-place presence/frequency penalty; returns logits."""
    ts = [_t(x, as_device) for x in (logits, presence_penalty, frequency_penalty, p_token_ids, p_token_counts, p_cumsum_seq_len)]
    _call("diopiApplyPenalty", ctx, *[_h(t) for t in ts], int(p_max_len_in_batch))
    return logits


def rotary_emb(input, cos, sin, conj, interleaved, *, out=None, ctx=None, as_device=None):
    """Returns a new tensor like input (or fills `out`)."""
    if out is None:
        out = torch.empty_like(input)
    ts = [_t(x, as_device) for x in (out, input, cos, sin)]
    _call("diopiRotaryEmbedding", ctx, *[_h(t) for t in ts], bool(conj), bool(interleaved))
    return out


def rotary_emb_v2(query, key, cos, sin, dim, *, ctx=None, as_device=None):
    """In-place rotate-half rotary embedding on query and key [tokens, heads*dim]; returns (query, key)
    (diopi_functions.py:8051)."""
    ts = [_t(x, as_device) for x in (query, key, cos, sin)]
    _call("diopiRotaryEmbeddingV2", ctx, *[_h(t) for t in ts], int(dim))
    return query, key


def apply_penalty_v2(logits, presence_penalty, frequency_penalty, repetition_penalty, p_token_ids, p_token_counts, *, ctx=None, as_device=None):
    """In-place penalty on flattened logits with per-entry penalties; returns logits (diopi_functions.py:8019)."""
    ts = [_t(x, as_device) for x in (logits, presence_penalty, frequency_penalty, repetition_penalty, p_token_ids, p_token_counts)]
    _call("diopiApplyPenaltyV2", ctx, *[_h(t) for t in ts])
    return logits


def rms_norm(input, normalized_shape, weight, bias, eps, *, return_inv_rms=False, ctx=None, as_device=None):
    """Returns out (and inv_rms when asked). inv_rms is fp32 for fp16/bf16/fp32 input, fp64 for fp64."""
    out = torch.empty_like(input)
    n = len(normalized_shape)
    inv_dtype = torch.float64 if input.dtype == torch.float64 else torch.float32
    inv_rms = torch.empty(tuple(input.shape[: input.dim() - n]), dtype=inv_dtype, device=input.device)
    ts = [_t(x, as_device) for x in (out, inv_rms, input)]
    tw, tb = _t(weight, as_device), _t(bias, as_device)
    _call("diopiRMSNorm", ctx, _h(ts[0]), _h(ts[1]), _h(ts[2]), Sizes(normalized_shape), _h(tw), _h(tb), float(eps))
    return (out, inv_rms) if return_inv_rms else out


def rotary_emb_copy_kv(q, k, v, cos, sin, dest_loc, k_pool, v_pool, conj=False, *, q_out=None, ctx=None, as_device=None):
    """q_out = rope(q); k_pool[dest_loc] = rope(k); v_pool[dest_loc] = v (v and v_pool may be None). Returns q_out."""
    q_out = torch.empty_like(q) if q_out is None else q_out
    ts = [_t(x, as_device) for x in (q_out, k_pool, v_pool, q, k, v, cos, sin, dest_loc)]
    _call("diopiRotaryEmbeddingCopyKV", ctx, *[_h(t) for t in ts], bool(conj))
    return q_out


def rms_norm_backward(grad_output, input, weight, bias, inv_rms, normalized_shape, eps, *, ctx=None, as_device=None):
    """Returns (grad_input, grad_weight, grad_bias or None) from the inv_rms a forward call saved."""
    grad_input = torch.empty_like(input)
    grad_weight = torch.empty_like(weight)
    grad_bias = torch.empty_like(bias) if bias is not None else None
    ts = [_t(x, as_device) for x in (grad_input, grad_weight, grad_bias, grad_output, input, weight, bias, inv_rms)]
    _call("diopiRMSNormBackward", ctx, *[_h(t) for t in ts], Sizes(normalized_shape), float(eps))
    return grad_input, grad_weight, grad_bias


def matmul_all_reduce(x1, x2, bias, group, *, out=None, reduce_op="sum", comm_turn=0, stream_mode=1, ctx=None, as_device=None):
    """out = sum over the ranks of `group` of (x1 @ x2 + bias); `group` is the name given to tp_group.create."""
    if out is None:
        out = torch.empty(tuple(x1.shape[:-1]) + (x2.shape[1],), dtype=x1.dtype, device=x1.device)
    ts = [_t(x, as_device) for x in (out, x1, x2, bias)]
    _call("diopiMatmulAllReduce", ctx, *[_h(t) for t in ts], group.encode(), reduce_op.encode(), int(comm_turn), int(stream_mode))
    return out
