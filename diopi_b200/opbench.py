"""Per-op micro-benchmark through the C ABI: `python -m diopi_b200.opbench --op <name> [--size full|small]`.

Times one op of the path on its benchmark config with CUDA events (L2 flushed between iterations with a
512 MB write for the ops whose working set is near the L2 size) and prints one JSON line with the time, the
algorithmic bytes or FLOPs and the achieved rate against the measured peak. bench.py covers the decode step
(the headline metric); this covers the other ops and gives profiler captures a small, committed command.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from . import functions as F
from . import workloads
from .runtime import Context

ROOT = Path(__file__).resolve().parent.parent


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["prefill", "rms_norm", "rms_norm_bwd", "rotary", "rope_copy_kv", "penalty", "copy_kv", "qk", "pv", "pair", "decode", "paged"])
    ap.add_argument("--size", default="full", choices=["full", "small"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--kv-heads", type=int, default=8, help="paged: K/V heads under 64 query heads")
    args = ap.parse_args()
    hbm, tf_burst, tf_sust, kind = peaks()
    ctx = Context()
    flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
    rec = {"op": args.op, "size": args.size, "peak_source": kind}

    if args.op == "prefill":
        pf = workloads.prefill() if args.size == "full" else workloads.prefill(B=4, lo=512, hi=2048)
        out = torch.empty_like(pf["q"])
        med, best = time_op(lambda: F.context_attention(pf["q"], pf["k"], pf["v"], out, pf["b_start_loc"], pf["b_seq_len"], pf["max_input_len"], ctx=ctx),
                            args.iters, args.warmup, None)
        tf = pf["flops"] / med / 1e9
        rec.update(ms=med, ms_best=best, flops=pf["flops"], tflops=tf, frac_of_burst_peak=tf / tf_burst, frac_of_sustained_peak=tf / tf_sust,
                   lens=pf["lens"].tolist(), unit="TFLOP/s (causal-only FLOPs, fp16)")
    elif args.op in ("rms_norm", "rms_norm_bwd", "rotary", "rope_copy_kv"):
        tokens = 8192 if args.size == "full" else 1024
        p = workloads.prenorm(tokens=tokens)
        from .runtime import Sizes, Tensor
        from . import _lib
        impl = _lib.load().impl
        sets = 6  # 6 x 134 MB of traffic between two uses of the same buffers: well beyond the 126 MB L2
        if args.op == "rms_norm":
            x = p["x"]
            nbytes = 2 * x.numel() * 2 + tokens * 4 + 4096 * 2
            med, best = time_op(lambda: F.rms_norm(x, (4096,), p["weight"], None, p["eps"], ctx=ctx), args.iters, args.warmup, flush)
            xs = [Tensor(x.clone()) for _ in range(sets)]
            outs = [Tensor(torch.empty_like(x)) for _ in range(sets)]
            invs = [Tensor(torch.empty(tokens, dtype=torch.float32, device="cuda")) for _ in range(sets)]
            wt, ns = Tensor(p["weight"]), Sizes((4096,))
            fns = [(lambda i=i: impl.diopiRMSNorm(ctx.handle, outs[i].handle, invs[i].handle, xs[i].handle, ns, wt.handle, None, 1e-6)) for i in range(sets)]
        elif args.op == "rms_norm_bwd":
            x = p["x"]
            nbytes = 3 * x.numel() * 2 + tokens * 4 + 2 * 4096 * 2
            _, inv = F.rms_norm(x, (4096,), p["weight"], None, p["eps"], return_inv_rms=True, ctx=ctx)
            g = torch.randn_like(x)
            med, best = time_op(lambda: F.rms_norm_backward(g, x, p["weight"], None, inv, (4096,), p["eps"], ctx=ctx), args.iters, args.warmup, flush)
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
        elif args.op == "rope_copy_kv":
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
            med = time_rotating(fns[:1], rounds=1, warmup=1)
        else:
            x = p["k_in"].view(tokens, p["heads"], p["head_dim"])
            out = torch.empty_like(x)
            nbytes = 2 * x.numel() * 2 + 2 * p["cos"].numel() * 2
            med, best = time_op(lambda: F.rotary_emb(x, p["cos"], p["sin"], False, False, out=out, ctx=ctx), args.iters, args.warmup, flush)
            xs = [Tensor(x.clone()) for _ in range(sets)]
            outs = [Tensor(torch.empty_like(x)) for _ in range(sets)]
            ct, st_ = Tensor(p["cos"]), Tensor(p["sin"])
            fns = [(lambda i=i: impl.diopiRotaryEmbedding(ctx.handle, outs[i].handle, xs[i].handle, ct.handle, st_.handle, False, False)) for i in range(sets)]
        back = time_rotating(fns, rounds=10, warmup=1)
        rec.update(ms=back, ms_single_launch_with_gap=med, bytes=nbytes, gbs=nbytes / back / 1e6, frac_of_peak=nbytes / back / 1e6 / hbm, unit="GB/s",
                   timing=f"{sets} buffer sets cycled back to back (cold L2), average per launch; ms_single_launch_with_gap brackets one launch alone")
    elif args.op == "paged":
        # diopiPagedAttention, 64 query heads x 128 over --kv-heads K/V heads, B 64, lengths U[512, 4096], blocks of 16
        B, Hq, D, bs, Hkv = 64, 64, 128, 16, args.kv_heads
        gc = torch.Generator().manual_seed(1006)
        lens = torch.randint(512, 4097, (B,), generator=gc)
        nblk = (lens + bs - 1) // bs
        blocks = int(nblk.sum()) + 8
        g = torch.Generator(device="cuda").manual_seed(1006)
        k = torch.randn(blocks * bs, Hkv * D, generator=g, device="cuda", dtype=torch.float32).to(torch.float16)
        v = torch.randn(blocks * bs, Hkv * D, generator=g, device="cuda", dtype=torch.float32).to(torch.float16)
        q = torch.randn(B, Hq * D, generator=g, device="cuda", dtype=torch.float32).to(torch.float16)
        perm = torch.randperm(blocks, generator=gc)
        table = torch.zeros(B, int(nblk.max()), dtype=torch.int32)
        o = 0
        for i in range(B):
            n = int(nblk[i])
            table[i, :n] = perm[o:o + n].to(torch.int32)
            o += n
        table = table.cuda()
        lens_l = lens.tolist()

        def run():
            F.paged_attention(q, k, v, None, lens_l, Hq, Hkv, D, table, bs, ctx=ctx)
            ctx.release()
        back = time_rotating([run], rounds=max(20, args.iters), warmup=2)
        nbytes = 2 * int(lens.sum()) * Hkv * D * 2 + 2 * q.numel() * 2
        rec.update(ms=back, bytes=nbytes, gbs=nbytes / back / 1e6, frac_of_peak=nbytes / back / 1e6 / hbm, unit="GB/s", kv_heads=Hkv, sum_len=int(lens.sum()),
                   note="bytes = every K/V row once + q + out: the figure a single pass over the rows would be bound by")
    elif args.op == "penalty":
        p = workloads.penalty()
        med, best = time_op(lambda: F.apply_penalty(p["logits"], p["presence"], p["frequency"], p["ids"], p["counts"], p["cum"], p["max_len"], ctx=ctx),
                            args.iters, args.warmup, flush)
        E = int(p["ids"].numel())
        rec.update(ms=med, ms_best=best, entries=E, bytes=E * (2 * 4 + 2 * 4) + 2 * 128 * 4 + 129 * 4, sector_bytes=E * 2 * 32, unit="ms (latency-bound)")
    else:
        w = workloads.decode("cfg2" if args.size == "full" else "cfg2s")
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
        fn, nbytes = fns[args.op]

        def run():
            fn()
            ctx.release()
        med, best = time_op(run, args.iters, args.warmup, flush if args.op == "copy_kv" else None)
        if args.op == "copy_kv":
            rec.update(ms=med, ms_best=best, bytes=nbytes, gbs=nbytes / med / 1e6, frac_of_peak=nbytes / med / 1e6 / hbm, unit="GB/s", sum_len=w.sum_len)
        else:
            # the pool is several times the L2 size, so launches queued back to back all stream from DRAM; a launch
            # bracketed alone also counts the host's time between recording the event and launching the kernel
            back = time_rotating([run], rounds=max(20, args.iters), warmup=1)
            rec.update(ms=back, ms_single_launch_with_gap=med, bytes=nbytes, gbs=nbytes / back / 1e6, frac_of_peak=nbytes / back / 1e6 / hbm, unit="GB/s",
                       sum_len=w.sum_len, timing="launches queued back to back, average per call; ms_single_launch_with_gap brackets one call alone")
    print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    sys.exit(main())
