"""Argument validation of every exported op, on CPU: each call must come back with an error code and
a message before any CUDA work is attempted (the tensors here only pretend to live on a device)."""
import pytest
import torch

from diopi_b200.runtime import DTYPE_NOT_SUPPORTED, ERROR_OCCURRED, NO_IMPLEMENT, DiopiError


@pytest.fixture(scope="module")
def F(built_libs):
    from diopi_b200 import functions
    return functions


def fails(code, fn, *args, match=None, **kw):
    with pytest.raises(DiopiError, match=match) as e:
        fn(*args, as_device=True, **kw)
    assert e.value.code == code, e.value
    return e.value


def decode_args(dtype=torch.float16, B=2, H=4, D=64, slots=32, N=8, idx=torch.int32):
    return dict(q=torch.zeros(B, H, D, dtype=dtype), k=torch.zeros(slots, H, D, dtype=dtype), v=torch.zeros(slots, H, D, dtype=dtype),
                out=torch.zeros(B, H, D, dtype=dtype), att=torch.zeros(H, 16, dtype=dtype), b_loc=torch.zeros(B, N, dtype=idx),
                st=torch.zeros(B, dtype=idx), ln=torch.zeros(B, dtype=idx))


def test_decode_validation(F):
    a = decode_args()
    fails(ERROR_OCCURRED, F.token_decode_attention, a["q"], a["k"], a["v"], a["out"], a["b_loc"], a["st"], a["ln"], 9, match="fewer than max_input_len")
    fails(ERROR_OCCURRED, F.token_decode_attention, a["q"], a["k"], a["v"], a["out"], a["b_loc"], a["st"], a["ln"], -1, match="negative")
    fails(ERROR_OCCURRED, F.token_decode_attention, a["q"][:, :2], a["k"], a["v"], a["out"], a["b_loc"], a["st"], a["ln"], 4, match="'q' must be")
    fails(ERROR_OCCURRED, F.token_decode_attention, a["q"], a["k"], a["v"].float(), a["out"], a["b_loc"], a["st"], a["ln"], 4, match="share a dtype")
    fails(ERROR_OCCURRED, F.token_decode_attention, a["q"], a["k"], a["v"][:5], a["out"], a["b_loc"], a["st"], a["ln"], 4, match="slot count")
    fails(DTYPE_NOT_SUPPORTED, F.token_decode_attention, a["q"], a["k"], a["v"], a["out"], a["b_loc"].float(), a["st"], a["ln"], 4, match="int32 or int64")
    fails(ERROR_OCCURRED, F.token_decode_attention, a["q"], a["k"], a["v"], a["out"], a["b_loc"], a["st"][:1], a["ln"], 4, match="batch")
    d = decode_args(dtype=torch.float64)
    fails(DTYPE_NOT_SUPPORTED, F.token_decode_attention, d["q"], d["k"], d["v"], d["out"], d["b_loc"], d["st"], d["ln"], 4, match="float64")
    fails(ERROR_OCCURRED, F.token_attention, a["q"], a["k"], a["att"][:2], a["b_loc"], a["st"], a["ln"], 4, match="logits")
    fails(ERROR_OCCURRED, F.token_softmax_reducev, a["att"], a["v"], a["out"][:1], a["b_loc"], a["st"], a["ln"], 4, 0, match="'out' must be")
    fails(ERROR_OCCURRED, F.token_attention, a["q"], a["k"][0], a["att"], a["b_loc"], a["st"], a["ln"], 4, match="pool must be")


def test_null_handles(F, built_libs):
    import ctypes
    rc = built_libs.impl.diopiDestIndexCopyKV(None, None, None, None)
    assert rc == ERROR_OCCURRED and "null handle" in F.last_error()
    rc = built_libs.impl.diopiRMSNorm(None, None, None, None, built_libs.impl.diopiRMSNorm.argtypes[4](), None, None, ctypes.c_double(1e-6))
    assert rc == ERROR_OCCURRED


def test_host_tensor_is_refused(F):
    a = decode_args()
    with pytest.raises(DiopiError, match="host memory"):
        F.destindex_copy_kv(a["q"], torch.zeros(2, dtype=torch.int32), a["k"], as_device=False)


def test_copy_kv_validation(F):
    k, out, d = torch.zeros(3, 4, 8), torch.zeros(10, 4, 8), torch.zeros(3, dtype=torch.int32)
    fails(ERROR_OCCURRED, F.destindex_copy_kv, k, d, out.half(), match="share a dtype")
    fails(ERROR_OCCURRED, F.destindex_copy_kv, k, d[:2], out, match="entries")
    fails(ERROR_OCCURRED, F.destindex_copy_kv, k, d, out[:, :2], match="but 'out' is")
    fails(DTYPE_NOT_SUPPORTED, F.destindex_copy_kv, k, d.to(torch.int16), out, match="int32 or int64")


def test_rotary_validation(F):
    x, c = torch.zeros(2, 3, 8), torch.zeros(2, 1, 4)
    e = fails(NO_IMPLEMENT, F.rotary_emb, x, c, c, False, True, match="interleaved")
    assert e.code == 13
    fails(ERROR_OCCURRED, F.rotary_emb, torch.zeros(2, 3, 7), c, c, False, False, match="even")
    fails(ERROR_OCCURRED, F.rotary_emb, x, torch.zeros(2, 1, 3), c, False, False, match="last dim of 'cos'")
    fails(ERROR_OCCURRED, F.rotary_emb, x, torch.zeros(5, 1, 4), torch.zeros(5, 1, 4), False, False, match="broadcast")
    fails(ERROR_OCCURRED, F.rotary_emb, x, c.half(), c.half(), False, False, match="share a dtype")
    fails(DTYPE_NOT_SUPPORTED, F.rotary_emb, x.int(), c.int(), c.int(), False, False)


def test_rms_norm_validation(F):
    x, w = torch.zeros(4, 6), torch.zeros(6)
    fails(ERROR_OCCURRED, F.rms_norm, x, (5,), w, None, 1e-6, match="normalized_shape")
    fails(ERROR_OCCURRED, F.rms_norm, x, (6,), torch.zeros(5), None, 1e-6, match="'weight' must have")
    fails(ERROR_OCCURRED, F.rms_norm, x, (6,), w, torch.zeros(3), 1e-6, match="'bias' must have")
    fails(ERROR_OCCURRED, F.rms_norm, x.t()[:6, :4].t(), (6,), w, None, 1e-6, match="contiguous") if False else None
    fails(ERROR_OCCURRED, F.rms_norm, x, (6,), w.half(), None, 1e-6, match="share a dtype")
    fails(ERROR_OCCURRED, F.rms_norm, x, (1, 2, 3), w, None, 1e-6, match="trailing dims")
    xt = torch.zeros(6, 4).t()   # shape [4, 6], not contiguous
    fails(ERROR_OCCURRED, F.rms_norm, xt, (6,), w, None, 1e-6, match="contiguous")


def test_penalty_validation(F):
    lg, p = torch.zeros(3, 10), torch.zeros(3)
    ids, cum = torch.zeros(5, dtype=torch.int32), torch.zeros(4, dtype=torch.int32)
    fails(ERROR_OCCURRED, F.apply_penalty, lg, p[:2], p, ids, ids, cum, 0, match="penalties")
    fails(ERROR_OCCURRED, F.apply_penalty, lg, p, p, ids, ids[:4], cum, 0, match="differ in length")
    fails(ERROR_OCCURRED, F.apply_penalty, lg, p, p, ids, ids, cum[:3], 0, match="batch \\+ 1")
    fails(ERROR_OCCURRED, F.apply_penalty, lg, p.half(), p, ids, ids, cum, 0, match="share a dtype")
    fails(DTYPE_NOT_SUPPORTED, F.apply_penalty, lg.int(), p.int(), p.int(), ids, ids, cum, 0)


def test_v2_validation(F):
    q, k = torch.zeros(4, 64), torch.zeros(4, 32)
    c = torch.zeros(4, 1, 16)
    fails(ERROR_OCCURRED, F.rotary_emb_v2, q, k, c, c, 15, match="even")
    fails(ERROR_OCCURRED, F.rotary_emb_v2, q, k, c, c, 24, match="multiple of dim")
    fails(ERROR_OCCURRED, F.rotary_emb_v2, q, k[:3], c, c, 16, match="same tokens")
    fails(ERROR_OCCURRED, F.rotary_emb_v2, q, k, torch.zeros(4, 1, 8), c, 16, match="last dim of 'cos'")
    fails(ERROR_OCCURRED, F.rotary_emb_v2, q, k, torch.zeros(3, 1, 16), c, 16, match="rows for")
    lg, pen = torch.zeros(3, 10), torch.zeros(5)
    ids = torch.zeros(5, dtype=torch.int32)
    fails(ERROR_OCCURRED, F.apply_penalty_v2, lg, pen[:4], pen, pen, ids, ids, match="one entry per token id")
    fails(ERROR_OCCURRED, F.apply_penalty_v2, lg, pen, pen, pen, ids, ids[:4], match="differ in length")
    fails(ERROR_OCCURRED, F.apply_penalty_v2, lg.t(), pen, pen, pen, ids, ids, match="contiguous")
    fails(ERROR_OCCURRED, F.apply_penalty_v2, lg, pen.half(), pen, pen, ids, ids, match="share a dtype")


def test_prompt_flash_attention_validation(F):
    q = torch.zeros(6, 4 * 16, dtype=torch.float16)
    kv = torch.zeros(6, 2 * 16, dtype=torch.float16)
    fails(ERROR_OCCURRED, F.prompt_flash_attention, q, kv, kv, None, [3, 3], 3, 4, 3, 16, match="multiple of num_kv_heads")
    fails(ERROR_OCCURRED, F.prompt_flash_attention, q, kv, kv, None, [3, 3], 4, 4, 2, 16, match="rows; expected")
    fails(ERROR_OCCURRED, F.prompt_flash_attention, q, kv[:, :16], kv, None, [3, 3], 3, 4, 2, 16, match="last dim of 'key'")
    fails(DTYPE_NOT_SUPPORTED, F.prompt_flash_attention, q.double(), kv.double(), kv.double(), None, [3, 3], 3, 4, 2, 16)


def test_paged_attention_validation(F):
    q = torch.zeros(2, 4 * 16, dtype=torch.float16)
    kv = torch.zeros(64, 4 * 16, dtype=torch.float16)
    tbl = torch.zeros(2, 2, dtype=torch.int32)
    fails(ERROR_OCCURRED, F.paged_attention, q, kv, kv, None, [3, 3], 4, 3, 16, tbl, 16, match="multiple of num_kv_heads")
    fails(ERROR_OCCURRED, F.paged_attention, q, kv, kv, None, [3, 40], 4, 4, 16, tbl, 16, match="block table covers")
    fails(ERROR_OCCURRED, F.paged_attention, q, kv, kv, None, [3, 3], 4, 4, 16, tbl, 0, match="block_size")
    fails(ERROR_OCCURRED, F.paged_attention, q, kv, kv, None, [3, 3, 3], 4, 4, 16, tbl, 16, match="'q' must be")
    fails(DTYPE_NOT_SUPPORTED, F.paged_attention, q, kv, kv, None, [3, 3], 4, 4, 16, tbl.float(), 16, match="int32 or int64")


def test_context_attention_validation(F):
    q = torch.zeros(8, 2, 16, dtype=torch.float16)
    st, ln = torch.zeros(2, dtype=torch.int32), torch.zeros(2, dtype=torch.int32)
    fails(ERROR_OCCURRED, F.context_attention, q, q[:4], q, q.clone(), st, ln, 4, match="share the shape")
    fails(ERROR_OCCURRED, F.context_attention, q, q, q, q.clone(), st, ln[:1], 4, match="differ in length")
    fails(DTYPE_NOT_SUPPORTED, F.context_attention, q.double(), q.double(), q.double(), q.double(), st, ln, 4)
    big = torch.zeros(2, 1, 300, dtype=torch.float16)
    fails(ERROR_OCCURRED, F.context_attention, big, big, big, big.clone(), st, ln, 4, match="maximum of 256")


def test_zero_size_inputs_succeed_without_a_device(F):
    """Empty tensors return success before any launch (diopi_configs.py:9080-9105 for rotary)."""
    e = torch.zeros(0, 4, 8)
    F.destindex_copy_kv(e, torch.zeros(0, dtype=torch.int32), torch.zeros(5, 4, 8), as_device=True)
    F.rotary_emb(torch.zeros(0, 8), torch.zeros(0, 4), torch.zeros(0, 4), False, False, as_device=True)
    F.rms_norm(torch.zeros(0, 8), (8,), torch.zeros(8), None, 1e-6, as_device=True)
    F.apply_penalty(torch.zeros(2, 5), torch.zeros(2), torch.zeros(2), torch.zeros(0, dtype=torch.int32), torch.zeros(0, dtype=torch.int32),
                    torch.zeros(3, dtype=torch.int32), 0, as_device=True)
    F.context_attention(torch.zeros(0, 2, 8), torch.zeros(0, 2, 8), torch.zeros(0, 2, 8), torch.zeros(0, 2, 8), torch.zeros(0, dtype=torch.int32),
                        torch.zeros(0, dtype=torch.int32), 0, as_device=True)
    a = decode_args(B=0)
    F.token_decode_attention(a["q"], a["k"], a["v"], a["out"], a["b_loc"], a["st"], a["ln"], 4, as_device=True)


def test_new_entry_points_validation(F):
    """RMSNorm backward, the rope + copy call and MatmulAllReduce refuse bad arguments before any CUDA work."""
    x = torch.zeros(4, 64, dtype=torch.float16)
    w = torch.zeros(64, dtype=torch.float16)
    inv = torch.zeros(4, dtype=torch.float32)
    fails(ERROR_OCCURRED, F.rms_norm_backward, x, x, w, None, inv, (32,), 1e-6, match="normalized_shape")
    fails(ERROR_OCCURRED, F.rms_norm_backward, x, x, w, None, inv[:3], (64,), 1e-6, match="inv_rms")
    fails(ERROR_OCCURRED, F.rms_norm_backward, x.float(), x, w, None, inv, (64,), 1e-6, match="share a dtype")
    fails(DTYPE_NOT_SUPPORTED, F.rms_norm_backward, x, x, w, None, inv.to(torch.int32), (64,), 1e-6, match="inv_rms")

    q, k = torch.zeros(5, 4, 64, dtype=torch.float16), torch.zeros(5, 2, 64, dtype=torch.float16)
    cs = torch.zeros(5, 1, 32, dtype=torch.float16)
    pool = torch.zeros(40, 2, 64, dtype=torch.float16)
    dest = torch.zeros(5, dtype=torch.int32)
    fails(ERROR_OCCURRED, F.rotary_emb_copy_kv, q, k, k, cs, cs, dest, pool, None, match="given together")
    fails(ERROR_OCCURRED, F.rotary_emb_copy_kv, q, k, None, cs, cs, dest[:3], pool, None, match="dest_loc")
    fails(ERROR_OCCURRED, F.rotary_emb_copy_kv, q, k[:, :, :32], None, cs, cs, dest, pool, None, match="kv_heads")
    fails(DTYPE_NOT_SUPPORTED, F.rotary_emb_copy_kv, q, k, None, cs, cs, dest.float(), pool, None, match="int32 or int64")

    a, b = torch.zeros(8, 64, dtype=torch.float16), torch.zeros(64, 128, dtype=torch.float16)
    fails(NO_IMPLEMENT, F.matmul_all_reduce, a, b, None, "nobody", reduce_op="max", match="only \"sum\"")
    fails(DTYPE_NOT_SUPPORTED, F.matmul_all_reduce, a.float(), b.float(), None, "nobody", match="float16, bfloat16")
    fails(ERROR_OCCURRED, F.matmul_all_reduce, a, b[:32], None, "nobody", match="columns")
    fails(ERROR_OCCURRED, F.matmul_all_reduce, a, b, torch.zeros(5, dtype=torch.float16), "nobody", match="bias")


def test_group_setup_validation(built_libs):
    """The group set-up calls check their arguments first (no CUDA call is reached here)."""
    import ctypes
    from diopi_b200 import _lib
    impl = _lib.load().impl
    buf = ctypes.create_string_buffer(64)
    assert impl.diopiB200GroupCreate(b"g", 0, 9, 4, buf) != 0
    assert b"1 to 8 ranks" in impl.diopiGetLastErrorString()
    assert impl.diopiB200GroupCreate(b"g", 3, 2, 4, buf) != 0
    assert impl.diopiB200GroupCreate(b"", 0, 1, 4, buf) != 0
    assert impl.diopiB200GroupCreate(b"g", 0, 2, 0, buf) != 0
    assert impl.diopiB200GroupConnect(b"missing", buf) != 0
    assert b"no group named" in impl.diopiGetLastErrorString()
    assert impl.diopiB200GroupDestroy(b"missing") != 0


def test_option_entry_points(F, built_libs):
    """The switches are changed by name; unknown names and values out of range come back as errors with the known names."""
    from diopi_b200 import tp_group
    for name in ("log", "fuse_token_attention", "decode_plain", "prefill_simt"):
        F.set_option(name, 1)
        F.set_option(name, 0)
    with pytest.raises(DiopiError, match="unknown option 'warp_speed'.*known: log"):
        F.set_option("warp_speed", 1)
    rc = built_libs.impl.diopiB200SetOption(None, 1)
    assert rc == ERROR_OCCURRED
    # group options: refused for a group that does not exist (creating one needs a device)
    with pytest.raises(DiopiError, match="no group named 'ghost'"):
        tp_group.set_option("ghost", "wait_limit_ms", 50)
