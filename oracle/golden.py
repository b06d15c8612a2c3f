"""CPU restatement of the reference's golden functions for the LLM-inference hot path.

TEST INFRASTRUCTURE ONLY. Nothing in the product (``diopi_b200/``) imports this module; it is
used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline/reference legs of
``bench.py`` as the checker and as the timed CPU baseline, never as a code path of the library.

Each function restates, in plain torch on the tensors' own device (CPU in practice), one golden
function of diopi_test/python/conformance/customized_test.py, keeping its dtype behaviour:
matrix products and divisions run in the input dtype, soft-max of the prefill path in fp32.
Pinning: ``tests/golden/*.npz`` hold inputs and outputs produced by the reference's own functions
(script: tests/golden/make_fixtures.py, run where the reference tree is mounted) together with the
literal known-answer cases of diopi_test/python/configs/diopi_configs.py; tests/test_oracle.py
checks this module against all of them. bfloat16 is not exercised by the reference's own tests
(its Python run time has no bfloat16 mapping), so bf16 parity rests on these functions alone.

Passing ``upcast=True`` evaluates the same formula on fp32 copies of half-precision inputs: that
is the "fp32 accumulation" reference the half-precision tolerances are stated against.
"""
from __future__ import annotations

import math

import torch


def _f32(*ts):
    return [t.float() if (t is not None and t.is_floating_point()) else t for t in ts]


def _slots(b_loc, i, length, max_input_len):
    """Pool slots of request i: b_loc is right-aligned inside its first max_input_len columns
    (customized_test.py:703-707, 720-724)."""
    first = int(max_input_len) - int(length)
    return b_loc[i, first:first + int(length)].long()


def destindex_copy_kv(k, dest_loc, out):
    """out[dest_loc[t]] = k[t] (customized_test.py:694-696; functions_lightllm.cpp:18-26)."""
    out.index_put_((dest_loc.long(),), k)
    return out


def token_attention(q, k, out, b_loc, b_start_loc, b_seq_len, max_input_len, upcast=False):
    """Decode logits (customized_test.py:698-713; functions_lightllm.cpp:53-80):
    out[h, start_i + j] = q[i,h,:] . k[slot(i,j),h,:] / sqrt(D)."""
    if upcast:
        q, k = _f32(q, k)
    batch, dim = b_loc.shape[0], q.shape[2]
    inv = math.sqrt(dim)
    for i in range(batch):
        length = int(b_seq_len[i])
        start = int(b_start_loc[i])
        keys = k[_slots(b_loc, i, length, max_input_len)]          # [L, H, D]
        # per head: a 1 x D row times a D x L matrix, in the input dtype, then the division
        scores = torch.matmul(q[i].unsqueeze(1), keys.permute(1, 2, 0)) / inv   # [H, 1, L]
        out[:, start:start + length] = scores.reshape(q.shape[1], length).to(out.dtype)
    return out


def token_softmax_reducev(logics, v, out, b_loc, b_start_loc, b_seq_len, max_input_len, other_kv_index=0, upcast=False):
    """softmax over each request's logits, then the weighted sum of its V rows
    (customized_test.py:715-733; functions_lightllm.cpp:82-107). other_kv_index is unused there too."""
    if upcast:
        logics, v = _f32(logics, v)
    batch, head = b_loc.shape[0], v.shape[1]
    for i in range(batch):
        length = int(b_seq_len[i])
        start = int(b_start_loc[i])
        probs = logics[:, start:start + length].softmax(-1).reshape(head, 1, length)
        values = v[_slots(b_loc, i, length, max_input_len)].permute(1, 0, 2)    # [H, L, D]
        out[i] = torch.matmul(probs, values).reshape(head, v.shape[2]).to(out.dtype)
    return out


def token_decode_attention(q, k, v, out, b_loc, b_start_loc, b_seq_len, max_input_len, upcast=False):
    """The two decode ops back to back, through a logits tensor of the input dtype — the composition
    the fused kernel replaces."""
    total = int(b_seq_len.sum())
    width = max(total, int((b_start_loc + b_seq_len).max()) if b_seq_len.numel() else 0)
    dt = torch.float32 if upcast else q.dtype
    logits = torch.zeros(q.shape[1], width, dtype=dt, device=q.device)
    token_attention(q, k, logits, b_loc, b_start_loc, b_seq_len, max_input_len, upcast=upcast)
    tmp = torch.zeros(out.shape, dtype=dt, device=out.device)
    token_softmax_reducev(logits, v, tmp, b_loc, b_start_loc, b_seq_len, max_input_len, 0, upcast=upcast)
    out.copy_(tmp)
    return out


def context_attention(q, k, v, out, b_start_loc, b_seq_len, max_input_len=0, upcast=False, row_block=None):
    """Causal prefill per request (customized_test.py:8-33, 735-749; functions_lightllm.cpp:109-147).
    scores = q k^T / sqrt(D) in the input dtype; soft-max of (scores.float() + mask) with the additive
    mask {allowed: 1, masked: -1e8}; probabilities cast back to the input dtype; then P v.
    ``row_block`` evaluates the same rows a block at a time so that long requests fit in memory;
    soft-max is row-wise, so the result is the same."""
    if upcast:
        q, k, v = _f32(q, k, v)
    dim = q.shape[2]
    for i in range(b_start_loc.shape[0]):
        start, length = int(b_start_loc[i]), int(b_seq_len[i])
        if length == 0:
            continue
        qs = q[start:start + length].transpose(0, 1)   # [H, L, D]
        ks = k[start:start + length].transpose(0, 1)
        vs = v[start:start + length].transpose(0, 1)
        step = length if not row_block else int(row_block)
        for r0 in range(0, length, step):
            r1 = min(length, r0 + step)
            scores = torch.matmul(qs[:, r0:r1], ks[:, :r1].transpose(1, 2)) / math.sqrt(dim)   # [H, rows, r1]
            rows = torch.arange(r0, r1, device=q.device).unsqueeze(1)
            cols = torch.arange(0, r1, device=q.device).unsqueeze(0)
            mask = torch.where(cols <= rows, 1.0, -100000000.0).to(torch.float32)
            probs = torch.softmax(scores.float() + mask, dim=-1).to(qs.dtype)
            res = torch.matmul(probs, vs[:, :r1])          # [H, rows, D]
            out[start + r0:start + r1] = res.transpose(0, 1).to(out.dtype)
    return out


def apply_penalty(logits, presence_penalty, frequency_penalty, p_token_ids, p_token_counts, p_cumsum_seq_len, p_max_len_in_batch=0):
    """In place: logits[i, id] = logits[i, id] - count * frequency[i] - presence[i], each operation
    rounded in the dtype of logits (customized_test.py:667-692; functions_lightllm.cpp:28-51)."""
    for i in range(logits.shape[0]):
        lo, hi = int(p_cumsum_seq_len[i]), int(p_cumsum_seq_len[i + 1])
        ids = p_token_ids[lo:hi].long()
        picked = logits[i, ids]
        picked = picked - p_token_counts[lo:hi] * frequency_penalty[i] - presence_penalty[i]
        logits[i, ids] = picked
    return logits


def rotary_emb(input, cos, sin, conj=False, interleaved=False):
    """Rotation of the two halves of the last dim in fp32, one rounding at the end
    (customized_test.py:374-390; the interleaved flag is ignored there as well)."""
    half = input.shape[-1] // 2
    x1, x2 = input[..., :half].float(), input[..., half:].float()
    c, s = cos.float(), sin.float()
    if conj:
        o1, o2 = x1 * c + x2 * s, -x1 * s + x2 * c
    else:
        o1, o2 = x1 * c - x2 * s, x1 * s + x2 * c
    return torch.cat((o1.to(input.dtype), o2.to(input.dtype)), dim=-1)


def rotary_emb_f64(input, cos, sin, conj=False):
    """fp64 variant: the reference's fp32 detour would lose precision that its fp64 test cases keep
    only because their tolerance allows it; the kernel computes fp64 in fp64."""
    half = input.shape[-1] // 2
    x1, x2 = input[..., :half], input[..., half:]
    if conj:
        o1, o2 = x1 * cos + x2 * sin, -x1 * sin + x2 * cos
    else:
        o1, o2 = x1 * cos - x2 * sin, x1 * sin + x2 * cos
    return torch.cat((o1, o2), dim=-1)


def rms_norm(input, normalized_shape, weight, bias=None, eps=1e-6, return_inv_rms=False):
    """inv_rms = rsqrt(mean(x^2 over the trailing dims) + eps) in fp32; out = weight * (x * inv_rms)
    (+ bias), cast once (customized_test.py:392-403)."""
    dims = tuple(range(-1, -len(normalized_shape) - 1, -1)) if normalized_shape is not None else (-1,)
    inv = torch.rsqrt(input.to(torch.float32).pow(2).mean(dims, keepdim=True) + eps)  # fp32 even for fp64 input
    y = weight * (input * inv)
    if bias is not None:
        y = y + bias
    y = y.to(input.dtype)
    if return_inv_rms:
        return y, inv.reshape(input.shape[: input.dim() - len(dims)])
    return y


def rms_norm_backward(grad_output, input, weight, normalized_shape, inv_rms=None, eps=1e-6, with_bias=False):
    """Derivative of rms_norm above in closed form, in fp32 (fp64 for fp64 input) with one rounding at the end:
    gw = g * weight; grad_input = inv * gw - x * inv^3 * mean(gw * x); grad_weight = sum_rows(g * x * inv);
    grad_bias = sum_rows(g). The reference's harness obtains the same quantities by torch.autograd.grad on the golden
    forward function (diopi_test/python/conformance/gen_output.py:172-204); its CUDA path is
    impl/torch/functions/functions_ext/layer_norm_cuda_kernel.cu:452-717. Returns (grad_input, grad_weight, grad_bias|None)."""
    acc = torch.float64 if input.dtype == torch.float64 else torch.float32
    k = len(normalized_shape)
    n2 = 1
    for d in normalized_shape:
        n2 *= int(d)
    x = input.reshape(-1, n2).to(acc)
    g = grad_output.reshape(-1, n2).to(acc)
    w = weight.reshape(1, n2).to(acc)
    if inv_rms is None:
        inv = torch.rsqrt(x.pow(2).mean(1, keepdim=True) + eps)
    else:
        inv = inv_rms.reshape(-1, 1).to(acc)
    gw = g * w
    dx = inv * gw - x * inv.pow(3) * (gw * x).mean(1, keepdim=True)
    dw = (g * x * inv).sum(0)
    db = g.sum(0) if with_bias else None
    shape_w = tuple(input.shape[input.dim() - k:])
    return (dx.reshape(input.shape).to(input.dtype), dw.reshape(shape_w).to(input.dtype),
            db.reshape(shape_w).to(input.dtype) if with_bias else None)


def rotary_emb_v2(query, key, cos, sin, dim):
    """Rotate-half form on [tokens, heads*dim] query and key with cos/sin as wide as a head, in the
    dtype of the tensors (customized_test.py:843-852). Returns new (query, key)."""
    def one(x):
        x3 = x.view(x.shape[0], -1, dim)
        x1, x2 = x3[..., : dim // 2], x3[..., dim // 2:]
        rot = torch.cat((-x2, x1), dim=-1)
        return (x3 * cos + rot * sin).view(x.shape[0], -1)
    return one(query), one(key)


def apply_penalty_v2(logits, presence_penalty, frequency_penalty, repetition_penalty, p_token_ids, p_token_counts):
    """Flattened penalty with a repetition term first (customized_test.py:823-841); in place on logits."""
    flat = logits.view(-1)
    ids = p_token_ids.long()
    cur = flat.index_select(0, ids)
    rep = torch.where(cur > 0, cur / repetition_penalty, cur * repetition_penalty)
    rep = rep - p_token_counts * frequency_penalty - presence_penalty
    flat[ids] = rep
    return logits


def prompt_flash_attention(query, key, value, atten_mask, actual_seq_lengths, max_input_len, num_heads, num_kv_heads, dim, upcast=False):
    """Padded-batch causal prefill in BSH layout (customized_test.py:751-783): every request has max_input_len rows,
    all of them computed under the causal mask; the mask argument and the actual lengths are not used there.
    num_kv_heads < num_heads repeats each K/V head (the reference only runs the equal case)."""
    bs = len(actual_seq_lengths)
    rows = bs * max_input_len
    q = query.reshape(rows, num_heads, dim)
    rep = num_heads // num_kv_heads
    k = key.reshape(rows, num_kv_heads, dim).repeat_interleave(rep, dim=1)
    v = value.reshape(rows, num_kv_heads, dim).repeat_interleave(rep, dim=1)
    start = torch.arange(bs, dtype=torch.int32) * max_input_len
    lens = torch.full((bs,), max_input_len, dtype=torch.int32)
    out = torch.zeros(rows, num_heads, dim, dtype=torch.float32 if upcast else query.dtype)
    context_attention(q, k, v, out, start, lens, max_input_len, upcast=upcast)
    return out.reshape(rows, num_heads * dim)


def paged_attention(query, key, value, atten_mask, actual_seq_lengths, num_heads, num_kv_heads, dim, block_table, block_size, upcast=False):
    """Decode attention over a block-paged cache: token j of request i is row block_table[i, j // bs] * bs + j % bs.
    The reference's golden (customized_test.py:785-821) is written for one request whose block table starts at
    block 0 (rows 0..L-1); this is the same formula for any batch and table, and equals it on that case."""
    B = len(actual_seq_lengths)
    rep = num_heads // num_kv_heads
    k = key.reshape(-1, num_kv_heads, dim).repeat_interleave(rep, dim=1)
    v = value.reshape(-1, num_kv_heads, dim).repeat_interleave(rep, dim=1)
    q = query.reshape(B, num_heads, dim)
    mx = max(int(x) for x in actual_seq_lengths) if B else 0
    b_loc = torch.zeros(B, max(mx, 1), dtype=torch.int64)
    for i, L in enumerate(actual_seq_lengths):
        j = torch.arange(int(L))
        b_loc[i, mx - int(L):mx] = block_table[i].long()[j // block_size] * block_size + j % block_size
    lens = torch.tensor([int(x) for x in actual_seq_lengths], dtype=torch.int32)
    start = torch.cat([torch.zeros(1, dtype=torch.int32), lens.cumsum(0)[:-1].to(torch.int32)]) if B else lens
    out = torch.zeros(B, num_heads, dim, dtype=torch.float32 if upcast else query.dtype)
    token_decode_attention(q, k, v, out, b_loc, start, lens, mx, upcast=upcast)
    return out.reshape(B, num_heads * dim)


def matmul_all_reduce(x1s, x2s, biases=None):
    """out = sum over ranks r of (x1s[r] @ x2s[r] + biases[r]), products and sums in fp32 in rank order, one rounding
    to the input dtype at the end. The reference only forwards diopiMatmulAllReduce to the vendor's
    aclnnMatmulAllReduce (impl/ascend/functions_ext/matmul_all_reduce.cpp:13-17), a closed third-party library (CANN,
    version not pinned in the tree) that is absent here, and holds no golden function, config or test for it: parity
    of this function against the reference is unpinned. The formula is the one the vendor documents for that call
    (matrix product plus bias on every rank, then a sum all-reduce)."""
    total = None
    for r, (a, b) in enumerate(zip(x1s, x2s)):
        part = a.reshape(-1, a.shape[-1]).float() @ b.float()
        if biases is not None and biases[r] is not None:
            part = part + biases[r].float()
        total = part if total is None else total + part
    return total.to(x1s[0].dtype).reshape(tuple(x1s[0].shape[:-1]) + (x2s[0].shape[1],))
