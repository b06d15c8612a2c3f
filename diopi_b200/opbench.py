"""Per-op micro-benchmark through the C ABI: `python -m diopi_b200.opbench --op <name> [--size full|small]`.

Times one op of the path on its benchmark config with CUDA events and prints one JSON line with the time, the
algorithmic bytes or FLOPs, the achieved rate against the measured peak and the SM clocks sampled while it ran.
bench.py covers the decode step (the headline metric) and calls `run_op` for the other ops on one GPU; the command
line form also gives profiler captures a small, committed command.

Cold-cache discipline: the decode and prefill workloads are many times the L2 size, so launches queued back to back
all stream from DRAM. The ops whose working set is near the L2 size (RMSNorm, rotary, their fusions and backward)
cycle through several buffer sets, so that every launch finds its data cold and launch gaps are not part of the
figure; the two small latency-bound ops (penalty, DestIndexCopyKV) are bracketed one launch at a time after a 512 MB
write has flushed L2.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from . import functions as F
from . import workloads
from .clocks import ClockSampler
from .runtime import Context

ROOT = Path(__file__).resolve().parent.parent

OPS = ["prefill", "rms_norm", "rms_norm_bwd", "rotary", "rope_copy_kv", "penalty", "copy_kv", "qk", "pv", "pair", "decode", "paged"]


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


def time_rotating(fns, rounds, warmup):
    """Average device time of one launch when the launches run back to back and cycle through `fns`, each
    working on its own buffers: with the sets together larger than L2, every launch finds its data cold,
    and launch gaps are not part of the figure the way they are when each launch is timed alone."""
    for _ in range(warmup):
        for fn in fns:
            fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(rounds):
        for fn in fns:
            fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / (rounds * len(fns))


def time_op(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2], times[0]


def _flush_buffer():
    return torch.empty(512 << 20, dtype=torch.uint8, device="cuda")


def paged_case(kv_heads: int, q_heads: int = 64, B: int = 64, D: int = 128, block: int = 16, lo: int = 512, hi: int = 4096, seed: int = 1006,
               dtype=torch.float16):
    """A block-paged decode batch: q_heads query heads over kv_heads K/V heads, lengths U[lo, hi], blocks in random order."""
    gc = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (B,), generator=gc)
    nblk = (lens + block - 1) // block
    blocks = int(nblk.sum()) + 8
    g = torch.Generator(device="cuda").manual_seed(seed)
    k = torch.randn(blocks * block, kv_heads * D, generator=g, device="cuda", dtype=torch.float32).to(dtype)
    v = torch.randn(blocks * block, kv_heads * D, generator=g, device="cuda", dtype=torch.float32).to(dtype)
    q = torch.randn(B, q_heads * D, generator=g, device="cuda", dtype=torch.float32).to(dtype)
    perm = torch.randperm(blocks, generator=gc)
    table = torch.zeros(B, int(nblk.max()), dtype=torch.int32)
    o = 0
    for i in range(B):
        n = int(nblk[i])
        table[i, :n] = perm[o:o + n].to(torch.int32)
        o += n
    return dict(q=q, k=k, v=v, table=table.cuda(), lens=lens.tolist(), sum_len=int(lens.sum()), q_heads=q_heads, kv_heads=kv_heads, D=D, block=block)


def library_prefill(pf, out, fn, rounds):
    """The same prefill batch on attention kernels of libraries that happen to be installed, timed the same way (queued
    back to back) and compared with this library's output: flash_attn's varlen kernel (mma.sync code built for earlier
    GPUs) and torch's scaled_dot_product_attention, one call per request on contiguous copies made beforehand. They are
    yardsticks printed beside the measurement, not part of the library and never on its call path."""
    res = {}
    lens = pf["lens"]
    fn()
    torch.cuda.synchronize()
    try:
        from flash_attn import flash_attn_varlen_func
        cu = torch.cat([torch.zeros(1, dtype=torch.int32), lens.cumsum(0).to(torch.int32)]).cuda()
        mx = int(lens.max())
        fa = lambda: flash_attn_varlen_func(pf["q"], pf["k"], pf["v"], cu, cu, mx, mx, causal=True)  # noqa: E731
        o = fa()
        ms = time_rotating([fa], rounds=rounds, warmup=1)
        res["flash_attn_varlen"] = {"ms": ms, "tflops": pf["flops"] / ms / 1e9, "max_abs_diff": (o.float() - out.float()).abs().max().item()}
    except Exception as e:  # noqa: BLE001
        res["flash_attn_varlen"] = {"error": repr(e)[:200]}
    try:
        import torch.nn.functional as TF
        starts = pf["b_start_loc"].tolist()
        per = []
        for s0, L in zip(starts, lens.tolist()):
            per.append(tuple(t[s0:s0 + L].transpose(0, 1).unsqueeze(0).contiguous() for t in (pf["q"], pf["k"], pf["v"])))
        def sd():
            return [TF.scaled_dot_product_attention(q, k, v, is_causal=True) for q, k, v in per]
        outs = sd()
        ms = time_rotating([sd], rounds=rounds, warmup=1)
        diff = max((o[0].transpose(0, 1).float() - out[s0:s0 + L].float()).abs().max().item() for o, s0, L in zip(outs, starts, lens.tolist()))
        res["torch_sdpa_per_request"] = {"ms": ms, "tflops": pf["flops"] / ms / 1e9, "max_abs_diff": diff, "calls": len(per)}
        # the longest request alone, on both
        i = int(lens.argmax())
        s0, L = starts[i], int(lens[i])
        H, D = pf["q"].shape[1], pf["q"].shape[2]
        fl = H * 4 * D * L * (L + 1) // 2
        q, k, v = per[i]
        one = lambda: TF.scaled_dot_product_attention(q, k, v, is_causal=True)  # noqa: E731
        ms1 = time_rotating([one], rounds=rounds, warmup=1)
        q1, k1, v1 = (t[s0:s0 + L].contiguous() for t in (pf["q"], pf["k"], pf["v"]))
        o1 = torch.empty_like(q1)
        st1 = torch.zeros(1, dtype=torch.int32, device="cuda")
        ln1 = torch.full((1,), L, dtype=torch.int32, device="cuda")
        mine = lambda: F.context_attention(q1, k1, v1, o1, st1, ln1, L)  # noqa: E731
        ms2 = time_rotating([mine], rounds=rounds, warmup=1)
        res["longest_request_alone"] = {"rows": L, "torch_sdpa_ms": ms1, "torch_sdpa_tflops": fl / ms1 / 1e9, "this_library_ms": ms2, "this_library_tflops": fl / ms2 / 1e9}
    except Exception as e:  # noqa: BLE001
        res["torch_sdpa_per_request"] = {"error": repr(e)[:200]}
    return res


def run_op(op: str, size: str = "full", iters: int = 10, warmup: int = 3, kv_heads: int = 8, head_dim: int = 128, ctx: Context | None = None,
           compare: bool = False) -> dict:
    """Runs one op's benchmark on the current device and returns its record (with a `clocks` entry)."""
    hbm, tf_burst, tf_sust, kind = peaks()
    ctx = ctx or Context()
    rec = {"op": op, "size": size, "peak_source": kind}
    sampler = ClockSampler(torch.cuda.current_device())

    if op == "prefill":
        kw = dict(D=head_dim, H=max(1, 4096 // head_dim))   # heads x head_dim = 4096 as at D 128
        pf = workloads.prefill(**kw) if size == "full" else workloads.prefill(B=4, lo=512, hi=2048, **kw)
        out = torch.empty_like(pf["q"])
        fn = lambda: F.context_attention(pf["q"], pf["k"], pf["v"], out, pf["b_start_loc"], pf["b_seq_len"], pf["max_input_len"], ctx=ctx)  # noqa: E731
        with sampler:
            med, best = time_op(fn, iters, warmup, None)
            back = time_rotating([fn], rounds=max(5, iters), warmup=1)
        tf = pf["flops"] / back / 1e9
        rec.update(ms=back, ms_single_launch_median=med, ms_single_launch_best=best, flops=pf["flops"], tflops=tf, frac_of_burst_peak=tf / tf_burst,
                   frac_of_sustained_peak=tf / tf_sust, head_dim=head_dim, heads=kw["H"], lens=pf["lens"].tolist(),
                   unit="TFLOP/s (causal-only FLOPs, fp16)", timing="launches queued back to back, average per call")
        if compare:
            rec["library_comparators"] = library_prefill(pf, out, fn, max(5, iters))
    elif op in ("rms_norm", "rms_norm_bwd", "rotary", "rope_copy_kv"):
        tokens = 8192 if size == "full" else 1024
        p = workloads.prenorm(tokens=tokens)
        from . import _lib
        from .runtime import Sizes, Tensor
        impl = _lib.load().impl
        sets = 6  # 6 x 134 MB of traffic between two uses of the same buffers: well beyond the 126 MB L2
        if op == "rms_norm":
            x = p["x"]
            nbytes = 2 * x.numel() * 2 + tokens * 4 + 4096 * 2
            xs = [Tensor(x.clone()) for _ in range(sets)]
            outs = [Tensor(torch.empty_like(x)) for _ in range(sets)]
            invs = [Tensor(torch.empty(tokens, dtype=torch.float32, device="cuda")) for _ in range(sets)]
            wt, ns = Tensor(p["weight"]), Sizes((4096,))
            fns = [(lambda i=i: impl.diopiRMSNorm(ctx.handle, outs[i].handle, invs[i].handle, xs[i].handle, ns, wt.handle, None, 1e-6)) for i in range(sets)]
        elif op == "rms_norm_bwd":
            x = p["x"]
            nbytes = 3 * x.numel() * 2 + tokens * 4 + 2 * 4096 * 2
            _, inv = F.rms_norm(x, (4096,), p["weight"], None, p["eps"], return_inv_rms=True, ctx=ctx)
            g = torch.randn_like(x)
            ctx.release()
            xs = [Tensor(x.clone()) for _ in range(sets)]
            gs = [Tensor(g.clone()) for _ in range(sets)]
            dxs = [Tensor(torch.empty_like(x)) for _ in range(sets)]
            dws = [Tensor(torch.empty_like(p["weight"])) for _ in range(sets)]
            wt, it, ns = Tensor(p["weight"]), Tensor(inv), Sizes((4096,))

            def bwd(i):
                impl.diopiRMSNormBackward(ctx.handle, dxs[i].handle, dws[i].handle, None, gs[i].handle, xs[i].handle, wt.handle, None, it.handle, ns, 1e-6)
                ctx.release()
            fns = [(lambda i=i: bwd(i)) for i in range(sets)]
        elif op == "rope_copy_kv":
            # prefill-sized pre-attention step: rope(q), rope(k) into the pool, v into the pool, in one launch; the
            # separate calls it replaces move 8 * numel * e bytes (k is written and read once more), this one 6
            H, D = p["heads"], p["head_dim"]
            sets = 3
            q = p["x"].view(tokens, H, D)
            kk = p["k_in"].view(tokens, H, D)
            nbytes = 6 * q.numel() * 2 + 2 * p["cos"].numel() * 2 + tokens * 4
            dest = torch.randperm(tokens, device="cuda").to(torch.int32)
            qs = [Tensor(q.clone()) for _ in range(sets)]
            ks = [Tensor(kk.clone()) for _ in range(sets)]
            vs = [Tensor(kk.clone()) for _ in range(sets)]
            qo = [Tensor(torch.empty_like(q)) for _ in range(sets)]
            kp = [Tensor(torch.empty_like(q)) for _ in range(sets)]
            vp = [Tensor(torch.empty_like(q)) for _ in range(sets)]
            ct, st_, dt_ = Tensor(p["cos"]), Tensor(p["sin"]), Tensor(dest)
            fns = [(lambda i=i: impl.diopiRotaryEmbeddingCopyKV(ctx.handle, qo[i].handle, kp[i].handle, vp[i].handle, qs[i].handle, ks[i].handle, vs[i].handle,
                                                                   ct.handle, st_.handle, dt_.handle, False)) for i in range(sets)]

            def separate(i):
                impl.diopiRotaryEmbedding(ctx.handle, qo[i].handle, qs[i].handle, ct.handle, st_.handle, False, False)
                impl.diopiRotaryEmbedding(ctx.handle, ks[i].handle, ks[i].handle, ct.handle, st_.handle, False, False)
                impl.diopiDestIndexCopyKV(ctx.handle, kp[i].handle, ks[i].handle, dt_.handle)
                impl.diopiDestIndexCopyKV(ctx.handle, vp[i].handle, vs[i].handle, dt_.handle)
            rec["ms_separate_calls"] = time_rotating([(lambda i=i: separate(i)) for i in range(sets)], rounds=10, warmup=1)
        else:
            x = p["k_in"].view(tokens, p["heads"], p["head_dim"])
            nbytes = 2 * x.numel() * 2 + 2 * p["cos"].numel() * 2
            xs = [Tensor(x.clone()) for _ in range(sets)]
            outs = [Tensor(torch.empty_like(x)) for _ in range(sets)]
            ct, st_ = Tensor(p["cos"]), Tensor(p["sin"])
            fns = [(lambda i=i: impl.diopiRotaryEmbedding(ctx.handle, outs[i].handle, xs[i].handle, ct.handle, st_.handle, False, False)) for i in range(sets)]
        with sampler:
            back = time_rotating(fns, rounds=max(10, iters), warmup=max(1, warmup))
        rec.update(ms=back, bytes=nbytes, gbs=nbytes / back / 1e6, frac_of_peak=nbytes / back / 1e6 / hbm, unit="GB/s",
                   timing=f"{sets} buffer sets cycled back to back (cold L2), average per launch")
    elif op == "paged":
        # diopiPagedAttention, 64 query heads x 128 over kv_heads K/V heads, B 64, lengths U[512, 4096], blocks of 16
        c = paged_case(kv_heads) if size == "full" else paged_case(kv_heads, B=16)

        # handles made once and the entry point called directly, as a C++ consumer would: the host side of a call is
        # then a few microseconds and the figure is the device's (a fresh Python wrapper per call costs more than the kernel)
        import time
        from . import _lib
        from .runtime import Sizes, Tensor
        impl = _lib.load().impl
        out = torch.empty_like(c["q"])
        hs = [Tensor(t) for t in (out, c["q"], c["k"], c["v"], c["table"])]
        lens_arg = Sizes(c["lens"])

        def run():
            rc = impl.diopiPagedAttention(ctx.handle, hs[0].handle, hs[1].handle, hs[2].handle, hs[3].handle, None, lens_arg, c["q_heads"], kv_heads, c["D"],
                                          hs[4].handle, c["block"])
            if rc:
                raise RuntimeError(F.last_error())
            ctx.release()
        with sampler:
            back = time_rotating([run], rounds=max(20, iters), warmup=max(2, warmup))
        torch.cuda.synchronize()
        h0 = time.perf_counter()
        for _ in range(200):
            run()
        rec["host_ms_per_call"] = (time.perf_counter() - h0) * 1e3 / 200
        torch.cuda.synchronize()
        nbytes = 2 * c["sum_len"] * kv_heads * c["D"] * 2 + 2 * c["q"].numel() * 2
        rec.update(ms=back, bytes=nbytes, gbs=nbytes / back / 1e6, frac_of_peak=nbytes / back / 1e6 / hbm, unit="GB/s", q_heads=c["q_heads"], kv_heads=kv_heads,
                   sum_len=c["sum_len"], note="bytes = every K/V row once + q + out: the figure a single pass over the rows is bound by",
                   timing="launches queued back to back, average per call")
    elif op == "penalty":
        p = workloads.penalty()
        flush = _flush_buffer()
        with sampler:
            med, best = time_op(lambda: F.apply_penalty(p["logits"], p["presence"], p["frequency"], p["ids"], p["counts"], p["cum"], p["max_len"], ctx=ctx),
                                iters, warmup, flush)
        E = int(p["ids"].numel())
        rec.update(ms=med, ms_best=best, entries=E, bytes=E * (2 * 4 + 2 * 4) + 2 * 128 * 4 + 129 * 4, sector_bytes=E * 2 * 32,
                   unit="ms (latency-bound scatter)", timing="one launch bracketed alone after an L2 flush, median")
    else:
        w = workloads.decode("cfg2" if size == "full" else "cfg2s")
        out = torch.empty_like(w.q)
        att = torch.zeros(w.q.shape[1], w.sum_len, dtype=w.q.dtype, device="cuda")
        fns = {
            "copy_kv": (lambda: F.destindex_copy_kv(w.k_new, w.dest_loc, w.k_pool, ctx=ctx), w.copy_bytes() // 2),
            "qk": (lambda: F.token_attention(w.q, w.k_pool, att, w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len, ctx=ctx), w.fused_bytes() // 2),
            "pv": (lambda: F.token_softmax_reducev(att, w.v_pool, out, w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len, 0, ctx=ctx), w.fused_bytes() // 2),
            # the two calls of the unchanged header one after the other; with DIOPI_B200_FUSE_TOKEN_ATTENTION=1 in the
            # environment they run as the fused kernel (algorithmic bytes of the pair: K, V and the logits both ways)
            "pair": (lambda: (F.token_attention(w.q, w.k_pool, att, w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len, ctx=ctx),
                              F.token_softmax_reducev(att, w.v_pool, out, w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len, 0, ctx=ctx)), w.fused_bytes()),
            "decode": (lambda: F.token_decode_attention(w.q, w.k_pool, w.v_pool, out, w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len, ctx=ctx), w.fused_bytes()),
        }
        fn, nbytes = fns[op]

        def run():
            fn()
            ctx.release()
        if op == "copy_kv":
            flush = _flush_buffer()
            with sampler:
                med, best = time_op(run, iters, warmup, flush)
            rec.update(ms=med, ms_best=best, bytes=nbytes, gbs=nbytes / med / 1e6, frac_of_peak=nbytes / med / 1e6 / hbm, unit="GB/s", sum_len=w.sum_len,
                       timing="one launch bracketed alone after an L2 flush, median (launch-latency bound: 1 MB)")
        else:
            with sampler:
                back = time_rotating([run], rounds=max(20, iters), warmup=max(1, warmup))
            rec.update(ms=back, bytes=nbytes, gbs=nbytes / back / 1e6, frac_of_peak=nbytes / back / 1e6 / hbm, unit="GB/s",
                       sum_len=w.sum_len, timing="launches queued back to back, average per call")
    rec["clocks"] = sampler.summary()
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=OPS)
    ap.add_argument("--size", default="full", choices=["full", "small"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--kv-heads", type=int, default=8, help="paged: K/V heads under 64 query heads")
    ap.add_argument("--head-dim", type=int, default=128, help="prefill: head dimension (heads = 4096 / head_dim)")
    ap.add_argument("--compare", action="store_true", help="prefill: also time installed library attention kernels on the same batch")
    args = ap.parse_args()
    print(json.dumps(run_op(args.op, args.size, args.iters, args.warmup, args.kv_heads, args.head_dim, compare=args.compare)), flush=True)


if __name__ == "__main__":
    sys.exit(main())
