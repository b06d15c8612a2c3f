"""Parity of the CUDA path, called through the C ABI of libdiopi_impl.so, against the reference's
outputs (tests/golden) and the CPU oracle on the same seeded inputs.

Tolerances (stated by the task): bit-exact for DestIndexCopyKV and ApplyPenalty; rtol=atol=1e-3 for
fp32; rtol=atol=1e-2 for fp16/bf16 against the oracle evaluated with fp32 accumulation."""
import threading

import pytest
import torch

from conftest import fixture_names, load_fixture
from oracle import golden

pytestmark = pytest.mark.gpu

TOL32 = dict(rtol=1e-3, atol=1e-3)
TOL16 = dict(rtol=1e-2, atol=1e-2)


def tol(dtype):
    return TOL32 if dtype in (torch.float32, torch.float64) else TOL16


def close(got, want, dtype=None):
    torch.testing.assert_close(got.detach().cpu().double(), want.detach().cpu().double(), **tol(dtype or want.dtype))


@pytest.fixture(scope="module")
def F(built_libs):
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from diopi_b200 import functions
    return functions


def cuda(*ts):
    return [t.cuda() if isinstance(t, torch.Tensor) else t for t in ts]


def full_pool(f, key):
    rows = f[key]
    pool = torch.zeros((f["pool"],) + tuple(rows.shape[1:]), dtype=rows.dtype)
    pool[f["used"].long()] = rows
    return pool


# ------------------------------------------------------------------ DestIndexCopyKV
@pytest.mark.parametrize("name", fixture_names("destindex_copy_kv"))
def test_destindex_copy_kv_fixture(F, name):
    f = load_fixture(name)
    k, d, out = cuda(f["k"], f["dest_loc"], f["out_before"].clone())
    k0, d0 = k.clone(), d.clone()
    F.destindex_copy_kv(k, d, out)
    assert torch.equal(out.cpu(), f["out"])
    assert torch.equal(k, k0) and torch.equal(d, d0)  # inputs untouched


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32, torch.float64])
@pytest.mark.parametrize("idx_dtype", [torch.int32, torch.int64])
def test_destindex_copy_kv_layouts(F, dtype, idx_dtype):
    g = torch.Generator().manual_seed(5)
    T, H, D, slots = 37, 5, 24, 211   # odd sizes: rows of 240/480/960 bytes
    k = torch.randn(T, H, D, generator=g).to(dtype)
    base = torch.randn(slots, H, D, generator=g).to(dtype)
    dest = torch.randperm(slots, generator=g)[:T].to(idx_dtype)
    dest[3] = dest[3] - slots  # a negative index counts from the end, as index_put_ does
    want = golden.destindex_copy_kv(k, dest, base.clone())
    out = base.clone().cuda()
    F.destindex_copy_kv(k.cuda(), dest.cuda(), out)
    assert torch.equal(out.cpu(), want)
    # strided views: a head shard of a wider pool and every other source row (element path)
    wide = torch.randn(slots, 2 * H, D, generator=g).to(dtype).cuda()
    view = wide[:, H:, :]
    src = torch.randn(2 * T, H, D, generator=g).to(dtype).cuda()[::2]
    want2 = golden.destindex_copy_kv(src.cpu(), dest, view.cpu().clone())
    F.destindex_copy_kv(src, dest.cuda(), view)
    assert torch.equal(view.cpu(), want2)
    # 1-byte rows / empty input
    F.destindex_copy_kv(k.cuda()[:0], dest.cuda()[:0], out)
    assert torch.equal(out.cpu(), want)


# ------------------------------------------------------------------ decode: fixtures
@pytest.mark.parametrize("name", fixture_names("token_attention_config"))
def test_token_attention_config(F, name):
    f = load_fixture(name)
    k, v = full_pool(f, "k_rows"), full_pool(f, "v_rows")
    q, bl, bs, bn = f["q"], f["b_loc"], f["b_start_loc"], f["b_seq_len"]
    mx = f["max_input_len"]
    att = torch.zeros_like(f["att"]).cuda()
    F.token_attention(q.cuda(), k.cuda(), att, bl.cuda(), bs.cuda(), bn.cuda(), mx)
    close(att, f["att"])
    red = torch.zeros_like(f["reducev"]).cuda()
    F.token_softmax_reducev(f["logics"].cuda(), v.cuda(), red, bl.cuda(), bs.cuda(), bn.cuda(), mx, 10)
    close(red, f["reducev"])
    fused = torch.zeros_like(f["fused"]).cuda()
    F.token_decode_attention(q.cuda(), k.cuda(), v.cuda(), fused, bl.cuda(), bs.cuda(), bn.cuda(), mx)
    close(fused, f["fused"])


@pytest.mark.parametrize("name", fixture_names("decode_seeded"))
def test_decode_seeded_fixture(F, name):
    f = load_fixture(name)
    q, k, v, bl, bs, bn = cuda(f["q"], f["k"], f["v"], f["b_loc"], f["b_start_loc"], f["b_seq_len"])
    mx = f["max_input_len"]
    att = torch.zeros_like(f["att"]).cuda()
    F.token_attention(q, k, att, bl, bs, bn, mx)
    close(att, f["att"])
    out = torch.full_like(f["out"], 7.0).cuda()
    F.token_softmax_reducev(f["att"].cuda(), v, out, bl, bs, bn, mx, 0)
    close(out, f["out"])
    fused = torch.full_like(f["out"], 7.0).cuda()
    F.token_decode_attention(q, k, v, fused, bl, bs, bn, mx)
    close(fused, f["out"])
    for i in (f["b_seq_len"] == 0).nonzero().flatten().tolist():
        assert torch.count_nonzero(fused[i]) == 0 and torch.count_nonzero(out[i]) == 0


# ------------------------------------------------------------------ decode: the CPU-runnable config, whole step
def test_decode_cfg1_step(F):
    from diopi_b200 import workloads
    w = workloads.decode("cfg1", device="cuda")
    # oracle on CPU copies of the same inputs
    kc, vc = w.k_pool.cpu().clone(), w.v_pool.cpu().clone()
    golden.destindex_copy_kv(w.k_new.cpu(), w.dest_loc.cpu(), kc)
    golden.destindex_copy_kv(w.v_new.cpu(), w.dest_loc.cpu(), vc)
    H = w.q.shape[1]
    att_ref = golden.token_attention(w.q.cpu(), kc, torch.zeros(H, w.sum_len), w.b_loc.cpu(), w.b_start_loc.cpu(), w.b_seq_len.cpu(), w.max_input_len)
    out_ref = golden.token_softmax_reducev(att_ref, vc, torch.zeros_like(w.q.cpu()), w.b_loc.cpu(), w.b_start_loc.cpu(), w.b_seq_len.cpu(), w.max_input_len)
    # device path
    F.destindex_copy_kv(w.k_new, w.dest_loc, w.k_pool)
    F.destindex_copy_kv(w.v_new, w.dest_loc, w.v_pool)
    assert torch.equal(w.k_pool.cpu(), kc) and torch.equal(w.v_pool.cpu(), vc)
    att = torch.zeros(H, w.sum_len, device="cuda")
    F.token_attention(w.q, w.k_pool, att, w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len)
    close(att, att_ref)
    out = torch.empty_like(w.q)
    F.token_softmax_reducev(att, w.v_pool, out, w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len, int(w.b_loc[0, -1]))
    close(out, out_ref)
    fused = torch.empty_like(w.q)
    F.token_decode_attention(w.q, w.k_pool, w.v_pool, fused, w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len)
    close(fused, out_ref)


def make_decode_case(B, H, D, dtype, lens, idx_dtype=torch.int32, extra_cols=0, seed=0, pool_extra=17):
    g = torch.Generator().manual_seed(seed)
    lens = torch.tensor(lens)
    total = int(lens.sum())
    slots = total + pool_extra
    k = (torch.randn(slots, H, D, generator=g) * 0.7).to(dtype)
    v = torch.randn(slots, H, D, generator=g).to(dtype)
    q = torch.randn(B, H, D, generator=g).to(dtype)
    perm = torch.randperm(slots, generator=g)
    mx = int(lens.max()) if B else 0
    bl = torch.zeros(B, mx + extra_cols, dtype=idx_dtype)
    st = torch.zeros(B, dtype=idx_dtype)
    acc = 0
    for i in range(B):
        L = int(lens[i])
        bl[i, mx - L:mx] = perm[acc:acc + L].to(idx_dtype)
        st[i] = acc
        acc += L
    return dict(q=q, k=k, v=v, b_loc=bl, b_start_loc=st, b_seq_len=lens.to(idx_dtype), max_input_len=mx, total=total)


def check_decode_case(F, c, k_dev=None, v_dev=None):
    dtype = c["q"].dtype
    H = c["q"].shape[1]
    args = (c["b_loc"], c["b_start_loc"], c["b_seq_len"], c["max_input_len"])
    att_ref = golden.token_attention(c["q"], c["k"], torch.zeros(H, c["total"]), *args, upcast=True)
    out_ref = golden.token_softmax_reducev(att_ref, c["v"], torch.zeros(c["q"].shape), *args, upcast=True)
    dargs = (c["b_loc"].cuda(), c["b_start_loc"].cuda(), c["b_seq_len"].cuda(), c["max_input_len"])
    kd = c["k"].cuda() if k_dev is None else k_dev
    vd = c["v"].cuda() if v_dev is None else v_dev
    q = c["q"].cuda()
    att = torch.zeros(H, c["total"], dtype=dtype, device="cuda")
    F.token_attention(q, kd, att, *dargs)
    close(att, att_ref, dtype)
    out = torch.full(c["q"].shape, 3.0, dtype=dtype, device="cuda")
    F.token_softmax_reducev(att_ref.to(dtype).cuda(), vd, out, *dargs, 0)
    close(out, out_ref, dtype)
    fused = torch.full(c["q"].shape, 3.0, dtype=dtype, device="cuda")
    F.token_decode_attention(q, kd, vd, fused, *dargs)
    close(fused, out_ref, dtype)
    return fused


DECODE_CASES = [
    # B, H, D, dtype, lens
    (1, 1, 64, torch.float16, [1]),
    (3, 32, 128, torch.float16, [4, 5, 4]),
    (5, 32, 128, torch.float16, [300, 0, 1, 1500, 77]),          # an empty request and a long one
    (4, 32, 128, torch.bfloat16, [129, 513, 2, 64]),
    (7, 8, 64, torch.float32, [16, 128, 33, 1, 0, 90, 128]),     # the CPU-runnable config's shape
    (3, 40, 128, torch.float16, [200, 31, 333]),                 # 40 heads: a full head group of 32 and a part group of 8
    (3, 12, 64, torch.float16, [50, 260, 9]),                    # 8 lanes per head, 5 token groups
    (2, 6, 256, torch.float16, [120, 45]),                       # 32 lanes per head
    (2, 4, 128, torch.float32, [70, 300]),                       # fp32, 32 lanes per head
    (2, 3, 32, torch.float32, [65, 8]),                          # fp32, 8 lanes per head
    (2, 5, 80, torch.float16, [40, 100]),                        # D*e/16 = 10: plain path
    (2, 2, 40, torch.float32, [33, 7]),                          # plain path, fp32
    (2, 64, 128, torch.float16, [700, 256]),                     # 64 heads: two head groups
]


@pytest.mark.parametrize("B,H,D,dtype,lens", DECODE_CASES)
def test_decode_shapes(F, B, H, D, dtype, lens):
    check_decode_case(F, make_decode_case(B, H, D, dtype, lens, seed=B * 131 + H))


def test_decode_all_small_lengths(F):
    """Every length from 0 to 33 in one batch (stage and group tails), both index dtypes, b_loc wider than max_input_len."""
    lens = list(range(0, 34))
    for idx_dtype in (torch.int32, torch.int64):
        check_decode_case(F, make_decode_case(len(lens), 8, 128, torch.float16, lens, idx_dtype=idx_dtype, extra_cols=10, seed=3))


def test_decode_many_requests(F):
    g = torch.Generator().manual_seed(11)
    lens = torch.randint(0, 40, (300,), generator=g).tolist()
    check_decode_case(F, make_decode_case(300, 4, 64, torch.float16, lens, seed=4))


def test_decode_strided_pool(F):
    """Head shard taken as a view of a wider pool (rows not dense over heads -> plain path), and a pool
    whose slot stride is padded (rows dense, stride larger -> split path)."""
    c = make_decode_case(3, 8, 128, torch.float16, [100, 257, 30], seed=9)
    slots = c["k"].shape[0]
    wide_k = torch.zeros(slots, 16, 128, dtype=torch.float16, device="cuda")
    wide_v = torch.zeros_like(wide_k)
    wide_k[:, 4:12] = c["k"].cuda()
    wide_v[:, 4:12] = c["v"].cuda()
    check_decode_case(F, c, wide_k[:, 4:12], wide_v[:, 4:12])
    pad_k = torch.zeros(slots, 8 * 128 + 64, dtype=torch.float16, device="cuda")
    pad_v = torch.zeros_like(pad_k)
    kk = pad_k[:, : 8 * 128].view(slots, 8, 128)   # stride(0) = 1088 elements
    vv = pad_v[:, : 8 * 128].view(slots, 8, 128)
    kk.copy_(c["k"].cuda())
    vv.copy_(c["v"].cuda())
    check_decode_case(F, c, kk, vv)


def test_decode_inputs_not_mutated(F):
    c = make_decode_case(4, 8, 128, torch.float16, [60, 0, 130, 9], seed=21)
    dev = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in c.items()}
    before = {k: v.clone() for k, v in dev.items() if isinstance(v, torch.Tensor)}
    out = torch.empty_like(dev["q"])
    F.token_decode_attention(dev["q"], dev["k"], dev["v"], out, dev["b_loc"], dev["b_start_loc"], dev["b_seq_len"], dev["max_input_len"])
    torch.cuda.synchronize()
    for k, v in before.items():
        assert torch.equal(dev[k], v), k


# ------------------------------------------------------------------ decode at full benchmark size
@pytest.fixture(scope="module")
def cfg2():
    from diopi_b200 import workloads
    return workloads.decode("cfg2", device="cuda")


def compact_oracle(w, reqs, k_pool, v_pool):
    """Oracle output of a few requests of a large workload: their rows are moved into a compact pool."""
    mx = w.max_input_len
    b_loc, lens = w.b_loc.cpu(), w.b_seq_len.cpu()
    rows, new_loc = [], torch.zeros(len(reqs), mx, dtype=torch.int32)
    acc = 0
    for n, i in enumerate(reqs):
        L = int(lens[i])
        rows.append(b_loc[i, mx - L:].long())
        new_loc[n, mx - L:] = torch.arange(acc, acc + L, dtype=torch.int32)
        acc += L
    rows = torch.cat(rows).cuda()
    k, v = k_pool[rows].cpu(), v_pool[rows].cpu()
    q = w.q[reqs].cpu()
    ln = lens[reqs]
    st = torch.cat([torch.zeros(1, dtype=torch.int32), ln.cumsum(0)[:-1].to(torch.int32)])
    out = torch.zeros(q.shape)
    return golden.token_decode_attention(q, k, v, out, new_loc, st, ln, mx, upcast=True)


def test_decode_cfg2_full_size(F, cfg2):
    w = cfg2
    k0 = w.k_pool.clone()
    # DestIndexCopyKV at full size: the touched rows equal the new rows bit for bit, every other row keeps its bits
    F.destindex_copy_kv(w.k_new, w.dest_loc, w.k_pool)
    F.destindex_copy_kv(w.v_new, w.dest_loc, w.v_pool)
    assert torch.equal(w.k_pool[w.dest_loc.long()], w.k_new)
    mask = torch.ones(w.k_pool.shape[0], dtype=torch.bool, device="cuda")
    mask[w.dest_loc.long()] = False
    assert torch.equal(w.k_pool[mask].view(torch.int16), k0[mask].view(torch.int16))
    del k0, mask

    fused = torch.empty_like(w.q)
    F.token_decode_attention(w.q, w.k_pool, w.v_pool, fused, w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len)
    # (1) the two stand-alone ops chained through an fp16 logits tensor agree with the fused kernel
    att = torch.zeros(w.q.shape[1], w.sum_len, dtype=w.q.dtype, device="cuda")
    F.token_attention(w.q, w.k_pool, att, w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len)
    two = torch.empty_like(w.q)
    F.token_softmax_reducev(att, w.v_pool, two, w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len, 0)
    close(two, fused)
    # (2) a sample of requests against the oracle with fp32 accumulation
    reqs = [0, 17, 63, int(w.b_seq_len.argmax()), int(w.b_seq_len.argmin())]
    close(fused[reqs], compact_oracle(w, reqs, w.k_pool, w.v_pool), torch.float16)
    # (3) the output is linear in V: doubling V doubles it (exact but for fp16 subnormals)
    w.v_pool.mul_(2)
    twice = torch.empty_like(w.q)
    F.token_decode_attention(w.q, w.k_pool, w.v_pool, twice, w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len)
    w.v_pool.mul_(0.5)
    assert float((twice.float() - 2 * fused.float()).abs().max()) <= 2.0 ** -23
    # (4) paging invariance: moving every row to another slot and renaming the slots in b_loc changes nothing
    slots = w.k_pool.shape[0]
    perm = torch.randperm(slots, device="cuda")
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(slots, device="cuda")
    k2, v2 = w.k_pool[perm], w.v_pool[perm]          # new slot s holds old row perm[s]
    b2 = inv[w.b_loc.long()].to(torch.int32)         # old slot -> new slot
    moved = torch.empty_like(w.q)
    F.token_decode_attention(w.q, k2, v2, moved, b2, w.b_start_loc, w.b_seq_len, w.max_input_len)
    assert torch.equal(moved, fused)


def test_decode_cfg5_shard_full_size(F):
    """One GPU's share of the 64-head decode config (8 heads, 128 requests, lengths up to 8192): 2 KB rows, i.e. the
    kernel form with several tokens side by side and four copy-issuing warps, at the size the benchmark runs it.
    Same size-independent properties as the 32-head config."""
    from diopi_b200 import workloads
    w = workloads.decode("cfg5", device="cuda", head_range=workloads.shard_heads(64, 8, 0))
    assert tuple(w.q.shape) == (128, 8, 128)
    F.destindex_copy_kv(w.k_new, w.dest_loc, w.k_pool)
    F.destindex_copy_kv(w.v_new, w.dest_loc, w.v_pool)
    assert torch.equal(w.k_pool[w.dest_loc.long()], w.k_new) and torch.equal(w.v_pool[w.dest_loc.long()], w.v_new)
    args = (w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len)
    fused = torch.empty_like(w.q)
    F.token_decode_attention(w.q, w.k_pool, w.v_pool, fused, *args)
    # (1) stand-alone pair through fp16 logits
    att = torch.zeros(w.q.shape[1], w.sum_len, dtype=w.q.dtype, device="cuda")
    F.token_attention(w.q, w.k_pool, att, *args)
    two = torch.empty_like(w.q)
    F.token_softmax_reducev(att, w.v_pool, two, *args, 0)
    close(two, fused)
    # (2) five requests against the oracle with fp32 accumulation
    reqs = [0, 41, 127, int(w.b_seq_len.argmax()), int(w.b_seq_len.argmin())]
    close(fused[reqs], compact_oracle(w, reqs, w.k_pool, w.v_pool), torch.float16)
    # (3) linear in V
    w.v_pool.mul_(2)
    twice = torch.empty_like(w.q)
    F.token_decode_attention(w.q, w.k_pool, w.v_pool, twice, *args)
    w.v_pool.mul_(0.5)
    assert float((twice.float() - 2 * fused.float()).abs().max()) <= 2.0 ** -23
    # (4) re-paging the pool changes nothing
    slots = w.k_pool.shape[0]
    perm = torch.randperm(slots, device="cuda")
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(slots, device="cuda")
    k2, v2 = w.k_pool[perm], w.v_pool[perm]
    b2 = inv[w.b_loc.long()].to(torch.int32)
    moved = torch.empty_like(w.q)
    F.token_decode_attention(w.q, k2, v2, moved, b2, w.b_start_loc, w.b_seq_len, w.max_input_len)
    assert torch.equal(moved, fused)


# ------------------------------------------------------------------ the pair of decode calls run as one kernel (opt-in)
def test_token_attention_pair_runs_fused_when_asked(F, monkeypatch):
    """With DIOPI_B200_FUSE_TOKEN_ATTENTION=1 the logits call is recorded and the softmax-reduce call that follows on
    the same tensors runs the fused kernel: same output as the fused entry point, the logits tensor is not written.
    Any other call in between launches the recorded logits kernel first."""
    c = make_decode_case(5, 8, 128, torch.float16, [300, 17, 0, 1024, 77], seed=77)
    d = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in c.items()}
    idx = (d["b_loc"], d["b_start_loc"], d["b_seq_len"], d["max_input_len"])
    total = int(c["b_seq_len"].sum())
    fused = torch.empty_like(d["q"])
    F.token_decode_attention(d["q"], d["k"], d["v"], fused, *idx)
    plain_att = torch.zeros(8, total, dtype=torch.float16, device="cuda")
    F.token_attention(d["q"], d["k"], plain_att, *idx)
    plain_out = torch.empty_like(d["q"])
    F.token_softmax_reducev(plain_att, d["v"], plain_out, *idx, 0)

    F.set_option("fuse_token_attention", 1)
    att = torch.full((8, total), 7.0, dtype=torch.float16, device="cuda")
    out = torch.empty_like(d["q"])
    F.token_attention(d["q"], d["k"], att, *idx)
    F.token_softmax_reducev(att, d["v"], out, *idx, 0)
    torch.cuda.synchronize()
    assert torch.equal(out, fused)
    assert bool((att == 7.0).all())  # never written
    close(out, plain_out, torch.float16)

    # another op of the library between the two calls: the logits are written before it runs, then the plain second half
    F.token_attention(d["q"], d["k"], att, *idx)
    F.rms_norm(torch.ones(4, 64, device="cuda"), (64,), torch.ones(64, device="cuda"), None, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(att, plain_att)
    F.token_softmax_reducev(att, d["v"], out, *idx, 0)
    assert torch.equal(out, plain_out)

    # the second call names another logits tensor: both halves run on their own
    att2 = torch.zeros_like(att)
    F.token_attention(d["q"], d["k"], att2, *idx)
    F.token_softmax_reducev(plain_att, d["v"], out, *idx, 0)
    torch.cuda.synchronize()
    assert torch.equal(att2, plain_att) and torch.equal(out, plain_out)

    # bad arguments are still refused at the first call
    from diopi_b200.runtime import DiopiError
    with pytest.raises(DiopiError):
        F.token_attention(d["q"][:, :4], d["k"], att, *idx)
    F.set_option("fuse_token_attention", 0)
    F.token_attention(d["q"], d["k"], att2.zero_(), *idx)
    torch.cuda.synchronize()
    assert torch.equal(att2, plain_att)


def test_context_release_flushes_a_recorded_call(F):
    """With the pair fusion on, the logits call is only recorded; releasing the context launches it and drops the
    record, so that nothing stale is left behind for a context created later at the same address."""
    from diopi_b200 import _lib
    from diopi_b200.runtime import Context
    c = make_decode_case(3, 8, 128, torch.float16, [40, 9, 200], seed=5)
    d = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in c.items()}
    idx = (d["b_loc"], d["b_start_loc"], d["b_seq_len"], d["max_input_len"])
    total = int(c["b_seq_len"].sum())
    plain = torch.zeros(8, total, dtype=torch.float16, device="cuda")
    F.token_attention(d["q"], d["k"], plain, *idx)
    ctx = Context()
    att = torch.zeros_like(plain)
    F.set_option("fuse_token_attention", 1)
    try:
        F.token_attention(d["q"], d["k"], att, *idx, ctx=ctx)
        torch.cuda.synchronize()
        assert torch.count_nonzero(att) == 0          # recorded, not launched
        assert _lib.load().impl.diopiB200ContextRelease(ctx.handle) == 0
        torch.cuda.synchronize()
        assert torch.equal(att, plain)                # launched by the release
        att.zero_()
        assert _lib.load().impl.diopiB200ContextRelease(ctx.handle) == 0   # nothing left: a no-op
        torch.cuda.synchronize()
        assert torch.count_nonzero(att) == 0
    finally:
        F.set_option("fuse_token_attention", 0)


# ------------------------------------------------------------------ status word, streams
def test_out_of_range_slot_is_reported(F):
    c = make_decode_case(2, 8, 128, torch.float16, [20, 40], seed=2)
    bad = c["b_loc"].clone()
    bad[1, -3] = c["k"].shape[0] + 5   # beyond the pool: the row is skipped and a status is raised
    out = torch.empty(c["q"].shape, dtype=torch.float16, device="cuda")
    from diopi_b200.runtime import DiopiError
    # The kernel of the first call raises the status; the next call takes it when it is entered and reports it after
    # making its own launch (a call never reports its own kernel).
    F.token_decode_attention(c["q"].cuda(), c["k"].cuda(), c["v"].cuda(), out, bad.cuda(), c["b_start_loc"].cuda(), c["b_seq_len"].cuda(), c["max_input_len"])
    torch.cuda.synchronize()
    good = torch.empty_like(out)
    with pytest.raises(DiopiError, match="outside the pool"):
        F.token_decode_attention(c["q"].cuda(), c["k"].cuda(), c["v"].cuda(), good, c["b_loc"].cuda(), c["b_start_loc"].cuda(), c["b_seq_len"].cuda(), c["max_input_len"])
    torch.cuda.synchronize()
    want = golden.token_decode_attention(c["q"], c["k"], c["v"], torch.zeros(c["q"].shape), c["b_loc"], c["b_start_loc"], c["b_seq_len"], c["max_input_len"], upcast=True)
    close(good, want, torch.float16)   # the call that reported the status did run
    # the status is reported once; the library keeps working
    check_decode_case(F, c)


def test_two_threads_two_contexts(F):
    """Ops are called from two host threads on two contexts/streams (the reference's stream test does
    the same with matmul+sum: diopi_test/python/tests/diopi/test_stream.py:102-108)."""
    from diopi_b200.runtime import Context
    c = make_decode_case(6, 8, 128, torch.float16, [100, 200, 50, 300, 10, 64], seed=31)
    dev = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in c.items()}
    ref = torch.empty_like(dev["q"])
    F.token_decode_attention(dev["q"], dev["k"], dev["v"], ref, dev["b_loc"], dev["b_start_loc"], dev["b_seq_len"], dev["max_input_len"])
    torch.cuda.synchronize()
    results, errors = {}, []

    def worker(n):
        try:
            s = torch.cuda.Stream()
            ctx = Context(s)
            outs = []
            for _ in range(20):
                o = torch.empty_like(dev["q"])
                F.token_decode_attention(dev["q"], dev["k"], dev["v"], o, dev["b_loc"], dev["b_start_loc"], dev["b_seq_len"], dev["max_input_len"], ctx=ctx)
                ctx.release()
                outs.append(o)
            ctx.synchronize()
            results[n] = outs
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    ts = [threading.Thread(target=worker, args=(n,)) for n in range(2)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errors, errors
    for outs in results.values():
        for o in outs:
            assert torch.equal(o, ref)


# ------------------------------------------------------------------ ApplyPenalty
@pytest.mark.parametrize("name", fixture_names("apply_penalty_v2"))
def test_apply_penalty_v2_fixture(F, name):
    f = load_fixture(name)
    lg = f["logits"].clone().cuda()
    F.apply_penalty_v2(lg, *cuda(f["presence"], f["frequency"], f["repetition"], f["ids"], f["counts"]))
    assert torch.equal(lg.cpu(), f["out"])   # bit-exact: every operation is rounded as the golden rounds it
    lg64 = f["logits"].clone().cuda()
    F.apply_penalty_v2(lg64, *cuda(f["presence"], f["frequency"], f["repetition"], f["ids"].long(), f["counts"].long()))
    assert torch.equal(lg64.cpu(), f["out"])


@pytest.mark.parametrize("name", fixture_names("rotary_emb_v2"))
def test_rotary_emb_v2_fixture(F, name):
    f = load_fixture(name)
    q, k = f["query"].clone().cuda(), f["key"].clone().cuda()
    F.rotary_emb_v2(q, k, f["cos"].cuda(), f["sin"].cuda(), f["dim"])
    assert torch.equal(q.cpu(), f["out_query"]) and torch.equal(k.cpu(), f["out_key"])
    # [tokens, dim] tables, bf16, and rows taken from a wider buffer
    g = torch.Generator().manual_seed(3)
    wide = torch.randn(6, 3 * 256, generator=g).to(torch.bfloat16).cuda()
    qv, kv = wide[:, :512], wide[:, 512:]
    c, s_ = torch.randn(6, 64, generator=g).to(torch.bfloat16), torch.randn(6, 64, generator=g).to(torch.bfloat16)
    wq, wk = golden.rotary_emb_v2(qv.cpu().contiguous(), kv.cpu().contiguous(), c.view(6, 1, 64), s_.view(6, 1, 64), 64)
    F.rotary_emb_v2(qv, kv, c.cuda(), s_.cuda(), 64)
    assert torch.equal(qv.cpu(), wq) and torch.equal(kv.cpu(), wk)


@pytest.mark.parametrize("name", [n for n in fixture_names("apply_penalty") if "_v2_" not in n])
def test_apply_penalty_fixture(F, name):
    f = load_fixture(name)
    lg = f["logits"].clone().cuda()
    ins = cuda(f["presence"], f["frequency"], f["ids"], f["counts"], f["cum"])
    keep = [t.clone() for t in ins]
    F.apply_penalty(lg, *ins, 5)
    assert torch.equal(lg.cpu(), f["out"])
    for a, b in zip(ins, keep):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_apply_penalty_cfg5_bit_exact(F, dtype):
    from diopi_b200 import workloads
    p = workloads.penalty(device="cuda", dtype=dtype)
    want = golden.apply_penalty(p["logits"].cpu().clone(), p["presence"].cpu(), p["frequency"].cpu(), p["ids"].cpu(), p["counts"].cpu(), p["cum"].cpu())
    F.apply_penalty(p["logits"], p["presence"], p["frequency"], p["ids"], p["counts"], p["cum"], p["max_len"])
    assert torch.equal(p["logits"].cpu(), want)
    # int64 index tensors give the same bits
    p2 = workloads.penalty(device="cuda", dtype=dtype)
    F.apply_penalty(p2["logits"], p2["presence"], p2["frequency"], p2["ids"].long(), p2["counts"].long(), p2["cum"].long(), p2["max_len"])
    assert torch.equal(p2["logits"].cpu(), want)


# ------------------------------------------------------------------ rotary, RMSNorm
@pytest.mark.parametrize("name", [n for n in fixture_names("rotary_emb") if "_v2_" not in n])
def test_rotary_fixture(F, name):
    f = load_fixture(name)
    x, c, s = cuda(f["x"], f["cos"], f["sin"])
    out = F.rotary_emb(x, c, s, bool(f["conj"]), False)
    close(out, f["out"])
    assert torch.equal(x.cpu(), f["x"])


def test_rotary_misc(F):
    from diopi_b200.runtime import FunctionNotImplementedError
    x = torch.randn(4, 6, 32, device="cuda", dtype=torch.float16)
    c = torch.randn(4, 1, 16, device="cuda", dtype=torch.float16)
    with pytest.raises(FunctionNotImplementedError):
        F.rotary_emb(x, c, c, False, True)
    # empty tensors are a no-op (diopi_configs.py:9080-9105)
    for xs, cs in [((0,), (0,)), ((0, 128), (0, 64)), ((3, 8, 0), (3, 1, 0)), ((1, 0, 16, 32), (0, 1, 16))]:
        e = torch.empty(xs, device="cuda", dtype=torch.float32)
        ce = torch.empty(cs, device="cuda", dtype=torch.float32)
        assert F.rotary_emb(e, ce, ce, False, False).shape == e.shape
    # non-contiguous x (a slice of a fused qkv buffer) and in-place use
    qkv = torch.randn(50, 3, 8, 64, device="cuda", dtype=torch.bfloat16)
    xq = qkv[:, 0]
    cs = torch.randn(50, 1, 32, device="cuda", dtype=torch.bfloat16)
    sn = torch.randn(50, 1, 32, device="cuda", dtype=torch.bfloat16)
    want = golden.rotary_emb(xq.cpu(), cs.cpu(), sn.cpu(), False)
    close(F.rotary_emb(xq, cs, sn, False, False), want)
    F.rotary_emb(xq, cs, sn, False, False, out=xq)
    close(xq, want)


def test_rotary_cfg3(F):
    from diopi_b200 import workloads
    p = workloads.prenorm(device="cuda")
    x = p["k_in"].view(8192, p["heads"], p["head_dim"])
    out = F.rotary_emb(x, p["cos"], p["sin"], False, False)
    want = golden.rotary_emb(x.cpu(), p["cos"].cpu(), p["sin"].cpu(), False)
    close(out, want)
    assert torch.equal(out.cpu(), want)  # same fp32 operations and one rounding: identical bits


def _rope_copy_case(T, Hq, Hk, D, dtype, seed, pool=150):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(T, h, D, generator=g).to(dtype) for h in (Hq, Hk, Hk))
    ang = torch.rand(T, 1, D // 2, generator=g) * 6.28
    cos, sin = ang.cos().to(dtype), ang.sin().to(dtype)
    dest = torch.randperm(pool, generator=g)[:T].to(torch.int32)
    kp, vp = (torch.randn(pool, Hk, D, generator=g).to(dtype) for _ in range(2))
    return q, k, v, cos, sin, dest, kp, vp


def _rope_copy_want(q, k, v, cos, sin, dest, kp, vp, conj):
    want_q = golden.rotary_emb(q, cos, sin, conj)
    want_k = golden.destindex_copy_kv(golden.rotary_emb(k, cos, sin, conj), dest, kp.clone())
    want_v = golden.destindex_copy_kv(v, dest, vp.clone())
    return want_q, want_k, want_v


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("conj", [False, True])
def test_rotary_emb_copy_kv(F, dtype, conj):
    """The one-launch form against the golden rotary_emb and destindex_copy_kv applied one after the other: identical bits."""
    for (T, Hq, Hk, D) in ((37, 8, 2, 128), (5, 4, 4, 64), (64, 32, 32, 128)):
        q, k, v, cos, sin, dest, kp, vp = _rope_copy_case(T, Hq, Hk, D, dtype, seed=T + D)
        want_q, want_k, want_v = _rope_copy_want(q, k, v, cos, sin, dest, kp, vp, conj)
        dq, dk, dv, dc, ds, dd, dkp, dvp = cuda(q, k, v, cos, sin, dest, kp, vp)
        got_q = F.rotary_emb_copy_kv(dq, dk, dv, dc, ds, dd, dkp, dvp, conj)
        assert torch.equal(got_q.cpu(), want_q) and torch.equal(dkp.cpu(), want_k) and torch.equal(dvp.cpu(), want_v)
        assert torch.equal(dq.cpu(), q) and torch.equal(dk.cpu(), k) and torch.equal(dv.cpu(), v)  # inputs untouched
        # without v, in place on q, int64 slots, cos/sin as [T, D/2]
        dkp2, dvp2, dq2 = kp.cuda(), vp.cuda(), q.cuda()
        F.rotary_emb_copy_kv(dq2, dk, None, dc.view(T, D // 2), ds.view(T, D // 2), dd.long(), dkp2, None, conj, q_out=dq2)
        assert torch.equal(dq2.cpu(), want_q) and torch.equal(dkp2.cpu(), want_k) and torch.equal(dvp2.cpu(), vp)


def test_rotary_emb_copy_kv_other_layouts(F):
    """Layouts the one-launch kernel does not take (strided heads, a head_dim that is not a multiple of 16 bytes per
    half, cos/sin shared by all tokens) run as the separate calls, with the same results."""
    q, k, v, cos, sin, dest, kp, vp = _rope_copy_case(19, 4, 2, 128, torch.float16, seed=3)
    want_q, want_k, want_v = _rope_copy_want(q, k, v, cos, sin, dest, kp, vp, False)
    wide = torch.zeros(19, 4, 256, dtype=torch.float16, device="cuda")
    wide[..., :128] = q.cuda()
    dkp, dvp = kp.cuda(), vp.cuda()
    got_q = F.rotary_emb_copy_kv(wide[..., :128], k.cuda(), v.cuda(), cos.cuda(), sin.cuda(), dest.cuda(), dkp, dvp)
    assert torch.equal(got_q.cpu(), want_q) and torch.equal(dkp.cpu(), want_k) and torch.equal(dvp.cpu(), want_v)
    q, k, v, cos, sin, dest, kp, vp = _rope_copy_case(7, 3, 3, 12, torch.float32, seed=4)
    want_q, want_k, want_v = _rope_copy_want(q, k, v, cos, sin, dest, kp, vp, True)
    dkp, dvp = kp.cuda(), vp.cuda()
    got_q = F.rotary_emb_copy_kv(q.cuda(), k.cuda(), v.cuda(), cos.cuda(), sin.cuda(), dest.cuda(), dkp, dvp, True)
    assert torch.equal(got_q.cpu(), want_q) and torch.equal(dkp.cpu(), want_k) and torch.equal(dvp.cpu(), want_v)
    shared_cos, shared_sin = cos[:1], sin[:1]  # [1, 1, D/2]: broadcast over the tokens
    want_q, want_k, want_v = _rope_copy_want(q, k, v, shared_cos, shared_sin, dest, kp, vp, False)
    dkp, dvp = kp.cuda(), vp.cuda()
    got_q = F.rotary_emb_copy_kv(q.cuda(), k.cuda(), v.cuda(), shared_cos.cuda(), shared_sin.cuda(), dest.cuda(), dkp, dvp)
    assert torch.equal(got_q.cpu(), want_q) and torch.equal(dkp.cpu(), want_k) and torch.equal(dvp.cpu(), want_v)


def test_rotary_emb_copy_kv_bad_slot(F):
    from diopi_b200.runtime import DiopiError
    q, k, v, cos, sin, dest, kp, vp = _rope_copy_case(9, 4, 4, 128, torch.float16, seed=8)
    bad = dest.clone()
    bad[4] = 10_000
    dkp, dvp = kp.cuda(), vp.cuda()
    F.rotary_emb_copy_kv(q.cuda(), k.cuda(), v.cuda(), cos.cuda(), sin.cuda(), bad.cuda(), dkp, dvp)
    torch.cuda.synchronize()
    with pytest.raises(DiopiError, match="outside the pool"):
        F.rotary_emb_copy_kv(q.cuda(), k.cuda(), v.cuda(), cos.cuda(), sin.cuda(), dest.cuda(), dkp, dvp)
    want_q, want_k, want_v = _rope_copy_want(q, k, v, cos, sin, dest, kp, vp, False)
    got_q = F.rotary_emb_copy_kv(q.cuda(), k.cuda(), v.cuda(), cos.cuda(), sin.cuda(), dest.cuda(), dkp, dvp)
    assert torch.equal(got_q.cpu(), want_q) and torch.equal(dkp.cpu(), want_k) and torch.equal(dvp.cpu(), want_v)
    with pytest.raises(DiopiError, match="given together"):
        F.rotary_emb_copy_kv(q.cuda(), k.cuda(), v.cuda(), cos.cuda(), sin.cuda(), dest.cuda(), dkp, None)


@pytest.mark.parametrize("name", [n for n in fixture_names("rms_norm") if "_backward_" not in n])
def test_rms_norm_fixture(F, name):
    f = load_fixture(name)
    x, w = cuda(f["x"], f["weight"])
    b = f["bias"].cuda() if "bias" in f else None
    ns = tuple(f["normalized_shape"].tolist())
    out, inv = F.rms_norm(x, ns, w, b, f["eps"], return_inv_rms=True)
    # the reference's own tolerance for rms_norm is 1e-4 (diopi_configs.py:9139-9140); halves get 1e-2
    t = dict(rtol=1e-4, atol=1e-4) if x.dtype in (torch.float32, torch.float64) else TOL16
    torch.testing.assert_close(out.cpu().double(), f["out"].double(), **t)
    _, inv_ref = golden.rms_norm(f["x"], ns, f["weight"], f.get("bias"), f["eps"], return_inv_rms=True)
    torch.testing.assert_close(inv.cpu().double(), inv_ref.double(), rtol=1e-5, atol=1e-6)
    assert inv.dtype == (torch.float64 if x.dtype == torch.float64 else torch.float32)


@pytest.mark.parametrize("n2", [8, 200, 256, 1000, 1024, 4096, 5120, 8192, 16384, 40000, 70000])
def test_rms_norm_widths(F, n2):
    g = torch.Generator().manual_seed(n2)
    for dtype in (torch.bfloat16, torch.float32):
        x = torch.randn(5, n2, generator=g).to(dtype)
        w = (1 + 0.1 * torch.randn(n2, generator=g)).to(dtype)
        b = torch.randn(n2, generator=g).to(dtype)
        want, inv_ref = golden.rms_norm(x, (n2,), w, b, 1e-5, return_inv_rms=True)
        out, inv = F.rms_norm(x.cuda(), (n2,), w.cuda(), b.cuda(), 1e-5, return_inv_rms=True)
        close(out, want)
        torch.testing.assert_close(inv.cpu(), inv_ref, rtol=1e-5, atol=1e-6)


BWD_TOL = {torch.float32: dict(rtol=1e-4, atol=1e-4), torch.float64: dict(rtol=1e-4, atol=1e-4),
           torch.float16: dict(rtol=4e-3, atol=4e-3), torch.bfloat16: dict(rtol=3e-2, atol=3e-2)}


@pytest.mark.parametrize("name", fixture_names("rms_norm_backward"))
def test_rms_norm_backward_fixture(F, name):
    """Against torch.autograd.grad of the reference's golden forward function (the harness's backward golden)."""
    f = load_fixture(name)
    ns = tuple(f["normalized_shape"].tolist())
    x, w = cuda(f["x"], f["weight"])
    b = f["bias"].cuda() if "bias" in f else None
    _, inv = F.rms_norm(x, ns, w, b, f["eps"], return_inv_rms=True)
    t = BWD_TOL[x.dtype]
    for g, pre in ((f["grad_output"], ""), (torch.ones_like(f["x"]), "ones_")):
        before = (x.clone(), w.clone(), inv.clone())
        dx, dw, db = F.rms_norm_backward(g.cuda(), x, w, b, inv, ns, f["eps"])
        torch.testing.assert_close(dx.cpu().double(), f[pre + "grad_input"].double(), **t)
        torch.testing.assert_close(dw.cpu().double(), f[pre + "grad_weight"].double(), **t)
        if b is not None:
            torch.testing.assert_close(db.cpu().double(), f[pre + "grad_bias"].double(), **t)
        assert torch.equal(before[0], x) and torch.equal(before[1], w) and torch.equal(before[2], inv)  # inputs untouched


@pytest.mark.parametrize("n2", [8, 200, 1000, 1024, 2048, 4096, 5120, 8192, 16384, 40000])
def test_rms_norm_backward_widths(F, n2):
    """Every kernel configuration (vectors per thread, scalar path for odd widths) against the closed-form oracle;
    the single-rounding results agree to the last place or so."""
    gen = torch.Generator().manual_seed(n2)
    rows = 301 if n2 <= 4096 else 33
    for dtype in (torch.bfloat16, torch.float32):
        x = torch.randn(rows, n2, generator=gen).to(dtype)
        g = torch.randn(rows, n2, generator=gen).to(dtype)
        w = (1 + 0.1 * torch.randn(n2, generator=gen)).to(dtype)
        b = torch.randn(n2, generator=gen).to(dtype)
        _, inv = F.rms_norm(x.cuda(), (n2,), w.cuda(), b.cuda(), 1e-5, return_inv_rms=True)
        want = golden.rms_norm_backward(g, x, w, (n2,), inv_rms=inv.cpu(), with_bias=True)
        got = F.rms_norm_backward(g.cuda(), x.cuda(), w.cuda(), b.cuda(), inv, (n2,), 1e-5)
        t = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
        for a, e in zip(got, want):
            torch.testing.assert_close(a.cpu().double(), e.double(), **t)
        # no grad_bias asked for
        got2 = F.rms_norm_backward(g.cuda(), x.cuda(), w.cuda(), None, inv, (n2,), 1e-5)
        assert got2[2] is None and torch.equal(got2[0], got[0])
        # the two forms may run with different numbers of partial rows, i.e. add the column sums in another order
        torch.testing.assert_close(got2[1].cpu().double(), got[1].cpu().double(), **t)


def test_rms_norm_backward_cfg3(F):
    from diopi_b200 import workloads
    p = workloads.prenorm(device="cuda")
    x, w = p["x"], p["weight"]
    g = torch.randn(x.shape, generator=torch.Generator(device="cuda").manual_seed(5), device="cuda", dtype=torch.float32).to(x.dtype)
    _, inv = F.rms_norm(x, (4096,), w, None, p["eps"], return_inv_rms=True)
    dx, dw, _ = F.rms_norm_backward(g, x, w, None, inv, (4096,), p["eps"])
    want = golden.rms_norm_backward(g.cpu(), x.cpu(), w.cpu(), (4096,), inv_rms=inv.cpu())
    torch.testing.assert_close(dx.cpu().double(), want[0].double(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(dw.cpu().double(), want[1].double(), rtol=1e-2, atol=2e-1)  # sums of 8192 terms of size ~1, bf16 result
    # run twice: the column sums are added in a fixed order
    dx2, dw2, _ = F.rms_norm_backward(g, x, w, None, inv, (4096,), p["eps"])
    assert torch.equal(dx, dx2) and torch.equal(dw, dw2)


def test_rms_norm_cfg3(F):
    from diopi_b200 import workloads
    p = workloads.prenorm(device="cuda")
    out, inv = F.rms_norm(p["x"], (4096,), p["weight"], None, p["eps"], return_inv_rms=True)
    want, inv_ref = golden.rms_norm(p["x"].cpu(), (4096,), p["weight"].cpu(), None, p["eps"], return_inv_rms=True)
    close(out, want)
    torch.testing.assert_close(inv.cpu(), inv_ref, rtol=1e-5, atol=1e-6)
    # at most one bf16 ulp apart anywhere (the sum of squares is added in another order)
    diff = (out.cpu().float() - want.float()).abs()
    assert float((diff / want.float().abs().clamp_min(1e-3)).max()) < 1e-2


# ------------------------------------------------------------------ prefill
@pytest.mark.parametrize("name", fixture_names("context_attention"))
def test_context_attention_fixture(F, name):
    f = load_fixture(name)
    q, k, v, st, bn = cuda(f["q"], f["k"], f["v"], f["b_start_loc"], f["b_seq_len"])
    out = torch.zeros_like(q)
    F.context_attention(q, k, v, out, st, bn, f["max_input_len"])
    close(out, f["out"])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("H,D,lens", [(4, 128, [1, 130, 7, 257]), (2, 64, [300, 1]), (3, 80, [33, 64]), (2, 128, [128, 256, 0, 384])])
def test_context_attention_ragged(F, dtype, H, D, lens):
    g = torch.Generator().manual_seed(sum(lens) + D)
    total = sum(lens)
    q, k, v = ((torch.randn(total, H, D, generator=g) / D ** 0.5 * 3).to(dtype) for _ in range(3))
    lens_t = torch.tensor(lens, dtype=torch.int32)
    st = torch.cat([torch.zeros(1, dtype=torch.int32), lens_t.cumsum(0)[:-1].to(torch.int32)])
    want = golden.context_attention(q, k, v, torch.zeros(total, H, D), st, lens_t, max(lens), upcast=True)
    out = torch.zeros(total, H, D, dtype=dtype, device="cuda")
    F.context_attention(q.cuda(), k.cuda(), v.cuda(), out, st.cuda(), lens_t.cuda(), max(lens))
    close(out, want, dtype)
    # int64 index tensors, and a max_input_len that understates the lengths (the reference ignores it)
    out2 = torch.zeros_like(out)
    F.context_attention(q.cuda(), k.cuda(), v.cuda(), out2, st.long().cuda(), lens_t.long().cuda(), 1)
    assert torch.equal(out2, out)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("H,D", [(3, 64), (2, 128), (2, 256)])
def test_context_attention_tensor_core_head_dims(F, capfd, dtype, H, D):
    """Head dims 64, 128 and 256 (the reference's own config runs 64 and 256, diopi_configs.py:9339-9381) on the
    tensor-core kernel: the log line proves which kernel took the call; requests that end inside a key block, inside
    a row tile, inside the second tile of a pair, one of a single row and one of several hundred key blocks' worth."""
    g = torch.Generator().manual_seed(D * 3 + H)
    lens = [1, 130, 700, 257, 1029, 128, 256, 383]
    total = sum(lens)
    q, k, v = ((torch.randn(total, H, D, generator=g) / D ** 0.5 * 3).to(dtype) for _ in range(3))
    lens_t = torch.tensor(lens, dtype=torch.int32)
    st = torch.cat([torch.zeros(1, dtype=torch.int32), lens_t.cumsum(0)[:-1].to(torch.int32)])
    want = golden.context_attention(q, k, v, torch.zeros(total, H, D), st, lens_t, max(lens), upcast=True)
    out = torch.zeros(total, H, D, dtype=dtype, device="cuda")
    F.set_option("log", 1)
    try:
        F.context_attention(q.cuda(), k.cuda(), v.cuda(), out, st.cuda(), lens_t.cuda(), max(lens))
        torch.cuda.synchronize()
    finally:
        F.set_option("log", 0)
    assert "tensor-core kernel" in capfd.readouterr().err
    close(out, want, dtype)
    # the SIMT kernel, which shares no code with it, agrees
    F.set_option("prefill_simt", 1)
    try:
        simt = torch.zeros_like(out)
        F.context_attention(q.cuda(), k.cuda(), v.cuda(), simt, st.cuda(), lens_t.cuda(), max(lens))
    finally:
        F.set_option("prefill_simt", 0)
    close(out, simt.float().cpu(), dtype)


def test_context_attention_cfg4_full_size(F):
    """The tensor-core prefill config at the size the benchmark runs it (8 requests of 1024..8192 rows, 32 heads,
    D 128, fp16). Whole (request, head) pairs are compared with the row-blocked oracle evaluated with fp32
    accumulation: the longest request (64 query tiles, several thousand keys per row: lazily raised maximum,
    polynomial exponentials, multi-wave tile order), the shortest, and two neighbours in the packed batch (last rows
    of one request next to the first rows of the other). Then two size-independent properties."""
    from diopi_b200 import workloads
    p = workloads.prefill(device="cuda")
    q, k, v, st, ln, mx = p["q"], p["k"], p["v"], p["b_start_loc"], p["b_seq_len"], p["max_input_len"]
    lens = [int(x) for x in p["lens"]]
    assert max(lens) > 8000 and q.shape[1:] == (32, 128)
    out = torch.zeros_like(q)
    F.context_attention(q, k, v, out, st, ln, mx)
    longest, shortest = lens.index(max(lens)), lens.index(min(lens))
    starts = [int(x) for x in st.cpu()]
    for req, head in [(longest, 0), (longest, 31), (shortest, 5), (0, 17), (1, 17)]:
        s0, L = starts[req], lens[req]
        sl = slice(s0, s0 + L)
        one = lambda t: t[sl, head:head + 1].cpu()
        want = golden.context_attention(one(q), one(k), one(v), torch.zeros(L, 1, 128), torch.zeros(1, dtype=torch.int32),
                                        torch.tensor([L], dtype=torch.int32), L, upcast=True, row_block=1024)
        close(out[sl, head:head + 1], want, torch.float16)
    # (1) run to run identical
    again = torch.zeros_like(q)
    F.context_attention(q, k, v, again, st, ln, mx)
    assert torch.equal(again, out)
    # (2) packing the requests in the reverse order moves their rows and nothing else
    order = list(range(len(lens)))[::-1]
    rows = torch.cat([torch.arange(starts[i], starts[i] + lens[i]) for i in order]).cuda()
    ln2 = torch.tensor([lens[i] for i in order], dtype=torch.int32)
    st2 = torch.cat([torch.zeros(1, dtype=torch.int32), ln2.cumsum(0)[:-1].to(torch.int32)])
    out2 = torch.zeros_like(q)
    F.context_attention(q[rows], k[rows], v[rows], out2, st2.cuda(), ln2.cuda(), mx)
    assert torch.equal(out2, out[rows])


# ------------------------------------------------------------------ padded-batch prefill (BSH) with grouped-query heads
@pytest.mark.parametrize("name", fixture_names("prompt_flash_attention"))
def test_prompt_flash_attention_fixture(F, name):
    f = load_fixture(name)
    bs, mlen, heads = f["batch"], f["max_input_len"], f["heads"]
    q, k, v = cuda(f["query"], f["key"], f["value"])
    out = F.prompt_flash_attention(q, k, v, None, [mlen] * bs, mlen, heads, heads, 128)
    close(out, f["out"])
    out3 = F.prompt_flash_attention(q.view(bs, mlen, -1), k.view(bs, mlen, -1), v.view(bs, mlen, -1), None, [mlen] * bs, mlen, heads, heads, 128)
    assert torch.equal(out3.view_as(out), out)


@pytest.mark.parametrize("dtype,dim", [(torch.float16, 128), (torch.bfloat16, 128), (torch.float32, 64)])
def test_prompt_flash_attention_grouped_heads(F, dtype, dim):
    g = torch.Generator().manual_seed(17)
    bs, mlen, heads, kv_heads = 2, 200, 8, 2
    q = (torch.randn(bs * mlen, heads * dim, generator=g) * 0.3).to(dtype)
    k = (torch.randn(bs * mlen, kv_heads * dim, generator=g) * 0.3).to(dtype)
    v = torch.randn(bs * mlen, kv_heads * dim, generator=g).to(dtype)
    want = golden.prompt_flash_attention(q, k, v, None, [mlen] * bs, mlen, heads, kv_heads, dim, upcast=True)
    out = F.prompt_flash_attention(q.cuda(), k.cuda(), v.cuda(), None, [mlen] * bs, mlen, heads, kv_heads, dim)
    close(out, want, dtype)


# ------------------------------------------------------------------ decode over a block-paged cache (BSH)
@pytest.mark.parametrize("name", fixture_names("paged_attention"))
def test_paged_attention_fixture(F, name):
    f = load_fixture(name)
    heads = f["heads"]
    table = torch.tensor([[0, 1]], dtype=torch.int32).cuda()
    out = F.paged_attention(f["query"].cuda(), f["key"].cuda(), f["value"].cuda(), None, [5], heads, heads, 128, table, 128)
    close(out, f["out"])


@pytest.mark.parametrize("dtype,heads,kv_heads,dim,block", [(torch.float16, 32, 32, 128, 16), (torch.bfloat16, 8, 8, 64, 128), (torch.float16, 8, 2, 128, 16),
                                                            (torch.float32, 4, 1, 64, 7)])
def test_paged_attention_batches(F, dtype, heads, kv_heads, dim, block):
    g = torch.Generator().manual_seed(heads * 7 + block)
    lens = [1, 3 * block, 0, 5 * block + 3, block - 1 if block > 1 else 1]
    B = len(lens)
    nblocks = sum((L + block - 1) // block for L in lens) + 3
    rows = nblocks * block
    k = (torch.randn(rows, kv_heads * dim, generator=g) * 0.5).to(dtype)
    v = torch.randn(rows, kv_heads * dim, generator=g).to(dtype)
    q = torch.randn(B, heads * dim, generator=g).to(dtype)
    perm = torch.randperm(nblocks, generator=g)
    width = max((L + block - 1) // block for L in lens)
    table = torch.zeros(B, width, dtype=torch.int32)
    used = 0
    for i, L in enumerate(lens):
        nb = (L + block - 1) // block
        table[i, :nb] = perm[used:used + nb].to(torch.int32)
        used += nb
    want = golden.paged_attention(q, k, v, None, lens, heads, kv_heads, dim, table, block, upcast=True)
    out = F.paged_attention(q.cuda(), k.cuda(), v.cuda(), None, lens, heads, kv_heads, dim, table.cuda(), block)
    close(out, want, dtype)
    assert torch.count_nonzero(out[2]) == 0   # the empty request
    out64 = F.paged_attention(q.cuda(), k.cuda(), v.cuda(), None, lens, heads, kv_heads, dim, table.long().cuda(), block)
    assert torch.equal(out64, out)


# ------------------------------------------------------------------ grouped K/V heads: the single-pass kernel
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,block", [(16, 8, 128, 16), (32, 8, 128, 16), (64, 8, 128, 16), (16, 1, 128, 16), (12, 3, 128, 8), (40, 5, 64, 32),
                                                      (32, 2, 64, 16), (24, 12, 128, 16), (7, 1, 64, 4), (48, 16, 128, 128),
                                                      (64, 2, 128, 16), (64, 1, 128, 16), (48, 2, 64, 16), (40, 1, 128, 8), (96, 3, 64, 16), (128, 1, 128, 16)])
def test_paged_attention_grouped_heads(F, dtype, heads, kv_heads, dim, block):
    """Query-head groups of 2 to 128 over 1 to 16 K/V heads (powers of two and not), head dims 64 and 128: every
    shape of the tensor-core kernel (K/V heads per CTA 1, 2, 4, 8; 1, 2, 4 or 8 tiles of 16 query heads per group;
    8 to 1 token blocks per stage; a second CTA row for the heads beyond eight), with request lengths that leave
    ragged last blocks, an empty and a one-token request."""
    g = torch.Generator().manual_seed(heads * 131 + kv_heads * 7 + dim)
    lens = [1, 700, 0, 129, 16, 17, 333, 15, 1024, 31]
    B = len(lens)
    nblocks = sum((L + block - 1) // block for L in lens) + 3
    rows = nblocks * block
    k = (torch.randn(rows, kv_heads * dim, generator=g) * 0.5).to(dtype)
    v = torch.randn(rows, kv_heads * dim, generator=g).to(dtype)
    q = torch.randn(B, heads * dim, generator=g).to(dtype)
    perm = torch.randperm(nblocks, generator=g)
    width = max((L + block - 1) // block for L in lens)
    table = torch.zeros(B, width, dtype=torch.int32)
    used = 0
    for i, L in enumerate(lens):
        nb = (L + block - 1) // block
        table[i, :nb] = perm[used:used + nb].to(torch.int32)
        used += nb
    want = golden.paged_attention(q, k, v, None, lens, heads, kv_heads, dim, table, block, upcast=True)
    out = F.paged_attention(q.cuda(), k.cuda(), v.cuda(), None, lens, heads, kv_heads, dim, table.cuda(), block)
    close(out, want, dtype)
    assert torch.count_nonzero(out[2]) == 0   # the empty request
    # same answer from the one-CTA-per-(request, head) kernel, which shares no code with the tensor-core one
    F.set_option("decode_plain", 1)
    try:
        plain = F.paged_attention(q.cuda(), k.cuda(), v.cuda(), None, lens, heads, kv_heads, dim, table.cuda(), block)
    finally:
        F.set_option("decode_plain", 0)
    close(out, plain.float().cpu(), dtype)
    # rows the block table never names may hold anything, infinities and NaNs included: they are never weighted in
    kk, vv = k.clone(), v.clone()
    named = torch.zeros(rows, dtype=torch.bool)
    for i, L in enumerate(lens):
        j = torch.arange(L)
        named[table[i].long()[j // block] * block + j % block] = True
    kk[~named] = float("nan")
    vv[~named] = float("inf")
    out2 = F.paged_attention(q.cuda(), kk.cuda(), vv.cuda(), None, lens, heads, kv_heads, dim, table.cuda(), block)
    assert torch.equal(out2, out)


def test_paged_attention_grouped_full_size(F):
    """64 query heads over 8 K/V heads at the size the benchmark runs (64 requests of 512..4096 tokens): sampled
    requests against the oracle with fp32 accumulation, run-to-run identical bits, and the same result from a cache
    whose blocks were moved to other places."""
    from diopi_b200 import opbench
    c = opbench.paged_case(8)
    args = (c["lens"], c["q_heads"], c["kv_heads"], c["D"])
    out = F.paged_attention(c["q"], c["k"], c["v"], None, *args, c["table"], c["block"])
    again = F.paged_attention(c["q"], c["k"], c["v"], None, *args, c["table"], c["block"])
    assert torch.equal(out, again)
    lens = c["lens"]
    reqs = [0, 31, 63, lens.index(max(lens)), lens.index(min(lens))]
    bs, tab = c["block"], c["table"].cpu()
    for i in reqs:
        nb = (lens[i] + bs - 1) // bs
        blocks = tab[i, :nb].long()
        rows = (blocks[:, None] * bs + torch.arange(bs)[None, :]).reshape(-1).cuda()
        k1, v1 = c["k"][rows].cpu(), c["v"][rows].cpu()
        t1 = torch.arange(nb, dtype=torch.int32).view(1, nb)
        want = golden.paged_attention(c["q"][i:i + 1].cpu(), k1, v1, None, [lens[i]], c["q_heads"], c["kv_heads"], c["D"], t1, bs, upcast=True)
        close(out[i:i + 1], want, torch.float16)
    nblocks = c["k"].shape[0] // bs
    perm = torch.randperm(nblocks, device="cuda")        # new block b holds old block perm[b]
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(nblocks, device="cuda")
    k2 = c["k"].view(nblocks, bs, -1)[perm].reshape(c["k"].shape)
    v2 = c["v"].view(nblocks, bs, -1)[perm].reshape(c["v"].shape)
    t2 = inv[c["table"].long()].to(torch.int32)
    moved = F.paged_attention(c["q"], k2, v2, None, *args, t2, c["block"])
    assert torch.equal(moved, out)
