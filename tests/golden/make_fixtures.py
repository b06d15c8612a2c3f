"""Generates tests/golden/*.npz from the reference's own golden functions.

Run in a container where the reference tree is mounted:
    python tests/golden/make_fixtures.py [/path/to/reference]
It imports diopi_test/python/conformance/customized_test.py unmodified and evaluates
CustomizedTest.<fn> on CPU for (a) the literal known-answer cases of
diopi_test/python/configs/diopi_configs.py (index tensors, shapes and values typed in from
lines 9053-9078, 9137-9337, 9339-9381, 9517-9610; some head counts and leading extents are cut down so
that the files stay small) with seeded random float data where the config draws random data, and (b) small seeded cases of the benchmark's shapes.
context_attention calls ``.cuda()`` on its mask (customized_test.py:16); there is no GPU here, so
``torch.Tensor.cuda`` is patched to the identity for the duration of this script (and, for paged_attention,
``device="cuda"`` arguments of torch.empty/torch.arange are routed to the CPU) — the function bodies
themselves run unchanged, on CPU.
bfloat16 tensors are stored as their uint16 bit patterns (numpy has no bfloat16).
"""
import sys
from pathlib import Path

import numpy as np
import torch

REF = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).resolve().parents[3] / "reference"   # default: a checkout beside this repository
sys.path.insert(0, str(REF / "diopi_test" / "python" / "conformance"))
torch.Tensor.cuda = lambda self, *a, **k: self  # see the module docstring
from customized_test import CustomizedTest as G  # noqa: E402

OUT = Path(__file__).resolve().parent
gen = torch.Generator().manual_seed(20240607)


def randn(*shape, dtype=torch.float32, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).to(dtype)


def to_np(t):
    if isinstance(t, torch.Tensor):
        if t.dtype == torch.bfloat16:
            return t.view(torch.int16).numpy().view(np.uint16)
        return t.numpy()
    return np.asarray(t)


def save(name, **arrays):
    np.savez_compressed(OUT / f"{name}.npz", **{k: to_np(v) for k, v in arrays.items() if v is not None})
    print("wrote", name, {k: tuple(np.shape(to_np(v))) for k, v in arrays.items() if v is not None})


DT = {"f32": torch.float32, "f16": torch.float16}

# ---- apply_penalty: literal values of diopi_configs.py:9265-9312 ------------------------------
for tag, dt in DT.items():
    logits = torch.tensor([[0.1, 0.5, 0.4, 0.3, 0.5], [0.2, 0.4, 0.0, 0.0, 0.0], [0.3, 0.4, 0.5, 0.3, 0.0]], dtype=dt)
    pres = torch.tensor([0.1, 0.8, 1.0], dtype=dt)
    freq = torch.tensor([0.3, 0.5, 0.4], dtype=dt)
    ids = torch.tensor([0, 1, 2, 3, 4, 0, 1, 0, 1, 2, 3], dtype=torch.int32)
    cnt = torch.tensor([3, 3, 2, 2, 1, 3, 3, 3, 3, 2, 2], dtype=torch.int32)
    cum = torch.tensor([0, 5, 7, 11], dtype=torch.int32)
    out = G.apply_penalty(logits.clone(), pres, freq, ids, cnt, cum, 5)
    save(f"apply_penalty_config_{tag}", logits=logits, presence=pres, frequency=freq, ids=ids, counts=cnt, cum=cum, out=out)

# ---- apply_penalty: seeded, ids without repetition inside a request ----------------------------
for tag, dt in DT.items():
    B, V = 6, 997
    logits = randn(B, V, dtype=dt, scale=2.0)
    pres = torch.rand(B, generator=gen).to(dt)
    freq = torch.rand(B, generator=gen).to(dt)
    lens = torch.randint(0, 40, (B,), generator=gen)
    lens[2] = 0
    ids = torch.cat([torch.randperm(V, generator=gen)[: int(n)] for n in lens]).to(torch.int32)
    cnt = torch.randint(1, 9, (int(lens.sum()),), generator=gen).to(torch.int32)
    cum = torch.cat([torch.zeros(1, dtype=torch.int64), lens.cumsum(0)]).to(torch.int32)
    out = G.apply_penalty(logits.clone(), pres, freq, ids, cnt, cum, int(lens.max()))
    save(f"apply_penalty_seeded_{tag}", logits=logits, presence=pres, frequency=freq, ids=ids, counts=cnt, cum=cum, out=out)

# ---- destindex_copy_kv: diopi_configs.py:9314-9337 (heads cut from 32 to 2 to keep the file small)
for tag, dt in DT.items():
    for case, (T, dest) in enumerate([(5, (0, 1, 2, 3, 4)), (4, (14, 15, 16, 17))]):
        k = randn(T, 2, 128, dtype=dt)
        base = randn(120, 2, 128, dtype=dt).round()  # integers compress well; the copy is bit-exact anyway
        d = torch.tensor(dest, dtype=torch.int32)
        out = G.destindex_copy_kv(k, d, base.clone())
        save(f"destindex_copy_kv_config{case}_{tag}", k=k, dest_loc=d, out_before=base, out=out)

# ---- token_attention / token_softmax_reducev: index tensors of diopi_configs.py:9517-9610 ------
b_loc = torch.tensor([[0, 0, 1, 2, 10] + [0] * 10, [3, 4, 5, 6, 11] + [0] * 10, [0, 7, 8, 9, 12] + [0] * 10], dtype=torch.int32)
b_start = torch.tensor([0, 4, 9], dtype=torch.int32)
b_len = torch.tensor([4, 5, 4], dtype=torch.int32)
for tag, dt in DT.items():
    H, D = 8, 128  # heads cut from 32 to 8 to keep the file small
    q = randn(3, H, D, dtype=dt)
    k = randn(100, H, D, dtype=dt)
    v = randn(100, H, D, dtype=dt)
    att = G.token_attention(q, k, torch.zeros(H, 13, dtype=dt), b_loc, b_start, b_len, 5)
    logics = randn(H, 13, dtype=dt)
    red = G.token_softmax_reducev(logics, v, torch.zeros(3, H, D, dtype=dt), b_loc, b_start, b_len, 5, 10)
    fused = G.token_softmax_reducev(att, v, torch.zeros(3, H, D, dtype=dt), b_loc, b_start, b_len, 5, 10)
    # keep only the 13 pool rows that are referenced, at their slots (the rest of the pool is never read)
    used = sorted(set(b_loc[:, :5].flatten().tolist()))
    save(f"token_attention_config_{tag}", q=q, k_rows=k[used], v_rows=v[used], used=np.array(used), pool=np.array(100), b_loc=b_loc,
         b_start_loc=b_start, b_seq_len=b_len, max_input_len=np.array(5), att=att, logics=logics, reducev=red, fused=fused)

# ---- decode, seeded, shape of the CPU-runnable benchmark config (B4 H8 D64, lens in [16,128]) --
for tag, dt in DT.items():
    B, H, D = 4, 8, 64
    lens = torch.randint(8, 49, (B,), generator=gen)  # the benchmark config draws from [16,128]
    lens[1] = 0 if tag == "f32" else lens[1]  # one empty request in the fp32 case
    pool = int(lens.sum()) + 16  # the benchmark config adds 64 spare slots; 16 keep the file small
    k = randn(pool, H, D, dtype=dt)
    v = randn(pool, H, D, dtype=dt)
    q = randn(B, H, D, dtype=dt)
    perm = torch.randperm(pool, generator=gen)
    mx = int(lens.max())
    bl = torch.zeros(B, mx + 3, dtype=torch.int32)
    st = torch.zeros(B, dtype=torch.int32)
    acc = 0
    for i in range(B):
        L = int(lens[i])
        bl[i, mx - L:mx] = perm[acc:acc + L].to(torch.int32)
        st[i] = acc
        acc += L
    bn = lens.to(torch.int32)
    att = G.token_attention(q, k, torch.zeros(H, acc, dtype=dt), bl, st, bn, mx)
    out = G.token_softmax_reducev(att, v, torch.zeros(B, H, D, dtype=dt), bl, st, bn, mx, 0)
    save(f"decode_seeded_{tag}", q=q, k=k, v=v, b_loc=bl, b_start_loc=st, b_seq_len=bn, max_input_len=np.array(mx), att=att, out=out)

# ---- context_attention: ragged layouts of diopi_configs.py:9339-9381 ---------------------------
# heads cut from 32/32/32/64 to 4/4/4/1 to keep the files small
layouts = [((4, 4, 64), (0,), (4,), 4), ((17, 4, 128), (0, 5), (5, 12), 12), ((64, 4, 128), (0, 16, 48), (16, 32, 16), 32),
           ((128, 1, 256), (0, 32, 64), (32, 32, 64), 64)]  # last layout halved as well
for tag, dt in DT.items():
    for case, (shape, starts, lens, mx) in enumerate(layouts):
        q, k, v = (randn(*shape, dtype=dt) for _ in range(3))
        st = torch.tensor(starts, dtype=torch.int32)
        bn = torch.tensor(lens, dtype=torch.int32)
        out = G.context_attention(q, k, v, torch.zeros(shape, dtype=dt), st, bn, mx)
        save(f"context_attention_config{case}_{tag}", q=q, k=k, v=v, b_start_loc=st, b_seq_len=bn, max_input_len=np.array(mx), out=out)

# ---- rotary_emb: shape/broadcast/conj combinations of diopi_configs.py:9053-9078 ---------------
rot = [((12,), (6,), True), ((64,), (32,), False), ((2, 128), (2, 64), False), ((3, 8, 256), (3, 1, 128), False), ((1, 64), (1, 32), True),
       ((3, 5, 12), (3, 5, 6), True), ((1, 25, 4, 64), (25, 1, 32), False), ((2, 16, 4, 32), (16, 1, 16), False), ((3, 20, 2, 64), (20, 1, 32), True)]
for tag, dt in {**DT, "f64": torch.float64}.items():
    for case, (xs, cs, conj) in enumerate(rot):
        x, c, s = randn(*xs, dtype=dt), randn(*cs, dtype=dt), randn(*cs, dtype=dt)
        out = G.rotary_emb(x, c, s, conj, False)
        save(f"rotary_emb_config{case}_{tag}", x=x, cos=c, sin=s, conj=np.array(conj), out=out)

# ---- rms_norm: diopi_configs.py:9137-9263 -------------------------------------------------------
rms = [((16,), (16,), 1e-4, False), ((5, 5), (5,), 1e-6, False), ((7, 25, 32), (32,), 1e-6, True), ((3, 64, 64), (64, 64), 1e-6, False),
       ((1, 8, 8, 64), (8, 64), 1e-6, True), ((3, 2, 4, 7, 8), (7, 8), 1e-2, True), ((5, 5), (5, 5), 1e-4, True), ((3, 4096), (4096,), 1e-6, False)]
for tag, dt in {**DT, "f64": torch.float64, "bf16": torch.bfloat16}.items():
    for case, (xs, ns, eps, with_bias) in enumerate(rms):
        x, w = randn(*xs, dtype=dt), (1 + 0.1 * torch.randn(*ns, generator=gen)).to(dt)
        b = randn(*ns, dtype=dt) if with_bias else None
        out = G.rms_norm(x, ns, w, b, eps)
        save(f"rms_norm_config{case}_{tag}", x=x, weight=w, bias=b, eps=np.array(eps), normalized_shape=np.array(ns), out=out)

# ---- apply_penalty_v2: literal values of diopi_configs.py:9470-9515, plus a seeded case ----------
for tag, dt in DT.items():
    logits = torch.tensor([[0.1, 0.5, 0.4, 0.3, 0.5], [0.2, 0.4, 0.0, 0.0, 0.0], [0.3, 0.4, 0.5, 0.3, 0.0]], dtype=dt)
    pen = torch.tensor([0.1, 0.1, 0.1, 0.1, 0.8, 0.8, 0.8, 0.8, 1.0, 1.0, 1.0], dtype=dt)
    ids = torch.tensor([0, 1, 2, 3, 4, 5, 6, 8, 9, 10, 11], dtype=torch.int32)
    cnt = torch.tensor([3, 3, 2, 2, 1, 3, 3, 3, 3, 2, 2], dtype=torch.int32)
    out = G.apply_penalty_v2(logits.clone(), pen, pen, pen, ids, cnt)
    save(f"apply_penalty_v2_config_{tag}", logits=logits, presence=pen, frequency=pen, repetition=pen, ids=ids, counts=cnt, out=out)
    B, V, E = 7, 501, 300
    logits = randn(B, V, dtype=dt, scale=2.0)
    ids = torch.randperm(B * V, generator=gen)[:E].to(torch.int32)
    cnt = torch.randint(1, 9, (E,), generator=gen).to(torch.int32)
    pres, freq = torch.rand(E, generator=gen).to(dt), torch.rand(E, generator=gen).to(dt)
    rep = (0.5 + torch.rand(E, generator=gen)).to(dt)
    out = G.apply_penalty_v2(logits.clone(), pres, freq, rep, ids, cnt)
    save(f"apply_penalty_v2_seeded_{tag}", logits=logits, presence=pres, frequency=freq, repetition=rep, ids=ids, counts=cnt, out=out)

# ---- rotary_emb_v2: diopi_configs.py:9107-9135 (query/key (8, 4096), cos/sin (8, 1, 128), dim 128) ----
for tag, dt in DT.items():
    q, k = randn(8, 4096, dtype=dt), randn(8, 1024, dtype=dt)
    c, s_ = randn(8, 1, 128, dtype=dt), randn(8, 1, 128, dtype=dt)
    oq, ok = G.rotary_emb_v2(q.clone(), k.clone(), c, s_, 128)
    save(f"rotary_emb_v2_config_{tag}", query=q, key=k, cos=c, sin=s_, dim=np.array(128), out_query=oq, out_key=ok)

# ---- prompt_flash_attention: diopi_configs.py:9383-9421 (maxInputLen 2, two requests, 32 heads x 128; fp16 only there) ----
for tag, dt in DT.items():
    for case, (bs, mlen, heads) in enumerate([(2, 2, 32), (3, 70, 2)]):
        q, k, v = (randn(bs * mlen, heads * 128, dtype=dt) for _ in range(3))
        mask = torch.zeros(bs, mlen, mlen, dtype=torch.bool)
        out = G.prompt_flash_attention(q, k, v, mask, [mlen] * bs, mlen, heads, heads, 128)
        save(f"prompt_flash_attention_config{case}_{tag}", query=q, key=k, value=v, batch=np.array(bs), max_input_len=np.array(mlen), heads=np.array(heads), out=out)

# paged_attention also names device="cuda" in torch.empty/torch.arange; route those to the CPU for this script
def _cpu_device(fn):
    def wrapped(*a, **k):
        if k.get("device") == "cuda":
            k["device"] = "cpu"
        return fn(*a, **k)
    return wrapped


torch.empty = _cpu_device(torch.empty)
torch.arange = _cpu_device(torch.arange)

# ---- paged_attention: diopi_configs.py:9423-9468 (one request of length 5, block table [[0, 1]], block size 128) ----
for tag, dt in DT.items():
    heads = 32 if tag == "f16" else 4
    q = randn(1, heads * 128, dtype=dt)
    k, v = randn(1026, heads * 128, dtype=dt)[:300], randn(1026, heads * 128, dtype=dt)[:300]   # only rows < 256 are addressable
    out = G.paged_attention(q, k, v, torch.zeros(1, 1, 5, dtype=torch.bool), [5], heads, heads, 128, torch.tensor([[0, 1]], dtype=torch.int32), 128)
    save(f"paged_attention_config_{tag}", query=q, key=k[:8], value=v[:8], heads=np.array(heads), out=out)

# ---- rms_norm backward: the conformance harness takes torch.autograd.grad of the golden forward function
# (diopi_test/python/conformance/gen_output.py:172-204) with grad_outputs of ones; a seeded random grad_output is
# stored as well. Shapes follow diopi_configs.py:9137-9263 (leading extents cut down). Own generator, so that the
# files above do not depend on this section.
gen_b = torch.Generator().manual_seed(20240608)
rms_b = [((16,), (16,), 1e-4, False), ((5, 5), (5,), 1e-6, False), ((7, 25, 32), (32,), 1e-6, True), ((3, 64, 64), (64, 64), 1e-6, False),
         ((3, 2, 4, 7, 8), (7, 8), 1e-2, True), ((9, 256), (256,), 1e-6, True), ((2, 2048), (2048,), 1e-6, False)]
for tag, dt in {**DT, "f64": torch.float64, "bf16": torch.bfloat16}.items():
    for case, (xs, ns, eps, with_bias) in enumerate(rms_b):
        def rb(*shape):
            return torch.randn(*shape, generator=gen_b).to(dt)
        x, w = rb(*xs).requires_grad_(True), (1 + 0.1 * torch.randn(*ns, generator=gen_b)).to(dt).requires_grad_(True)
        b = rb(*ns).requires_grad_(True) if with_bias else None
        leaves = [x, w] + ([b] if with_bias else [])
        out = G.rms_norm(x, ns, w, b, eps)
        ones = torch.autograd.grad([out], leaves, [torch.ones_like(out)], retain_graph=True)
        g = rb(*xs)
        rnd = torch.autograd.grad([out], leaves, [g])
        save(f"rms_norm_backward_config{case}_{tag}", x=x.detach(), weight=w.detach(), bias=b.detach() if with_bias else None, eps=np.array(eps),
             normalized_shape=np.array(ns), grad_output=g,
             ones_grad_input=ones[0], ones_grad_weight=ones[1], ones_grad_bias=ones[2] if with_bias else None,
             grad_input=rnd[0], grad_weight=rnd[1], grad_bias=rnd[2] if with_bias else None)
