#!/usr/bin/env python
"""Benchmark of the paged-KV decode step (the path BASELINE.json's metric is quoted on).

One step = what a serving engine does per layer for one decode iteration of a batch:
  diopiDestIndexCopyKV (new K rows) + diopiDestIndexCopyKV (new V rows) + diopiTokenDecodeAttentionInference,
all three through the C ABI of libdiopi_impl.so on the rank's GPU.

Workloads (seeded synthetic; there is no dataset behind this path):
  cfg2 (default): LLaMA-7B decode, B64 H32 D128 fp16, lens in [512,4096], pool 64*4096 slots per GPU. With N GPUs
        every rank holds one such 32-head shard of a 32*N-head model (same slot tables on every rank):
        per-GPU work is fixed -> "scaling": "weak". No collective on the data path.
  cfg5: B128 H64 D128 fp16, lens in [1024,8192]; the 64 heads are split over the N ranks -> "strong".

The printed JSON line follows the driver's contract; `value` is whole-job algorithmic GB/s with inputs resident
in HBM, `e2e` is the same step driven from pinned host buffers (H2D of the step's inputs, D2H of the output, a
sync per step); mean, median and best step are all given. After the headline (cfg2) the same line gains, each leg
with the SM clocks sampled while it ran: `strong_cfg5` (the 64-head config split over the N ranks, at every N),
and at N = 1 `l2_warm` (the step on a batch that stays in L2) and `ops` (every other op of the path on its benchmark
config, through diopi_b200.opbench), at N > 1 `matmul_allreduce` (the fused GEMM + all-reduce on the N ranks, with a
parity check). `--impl reference` times the reference's CPU implementation of the step (its golden functions where
a checkout is mounted, else the oracle port) on all host threads instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

METRIC = "token_attn_decode_hbm_gbs"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per token of one decode_split_kernel launch, from the ncu capture
# of the quarter-size case summarised in profiles/decode_split_kernel_cfg2.md (660.0 MB for 40 019 tokens); the
# traffic of a launch grows with its token count, so it is scaled by the workload's tokens.
NCU_TRAFFIC_BYTES_PER_TOKEN = 661.483e6 / 40019


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy bandwidth)"
        except Exception:  # noqa: BLE001
            pass
    return FALLBACK_HBM_GBS, "fallback"


from diopi_b200.clocks import ClockSampler  # noqa: E402


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def workload_description(name, n, heads_here):
    if name == "cfg2s":
        return "a quarter of the LLaMA-7B decode step (16 of 64 requests), for profiler captures"
    if name == "cfg2":
        return (f"LLaMA-7B decode step (configs[1]): B64 H32 D128 fp16 per GPU, lens U[512,4096], pool 64*4096 slots; "
                f"{n} GPU(s) x 32-head shard (a {32 * n}-head model at N>1)")
    return f"64-head decode (configs[4]): B128 H64 D128 fp16, lens U[1024,8192]; {heads_here} heads on each of {n} GPU(s)"


# ------------------------------------------------------------------------------------------------ b200 arm
class StepRunner:
    """One decode step of a workload through the C ABI, with everything that does not change from step to step
    (tensor handles, bound entry points) made once, as a framework's integration would: the per-step host work is
    three foreign calls. `device_step` works on inputs resident in HBM; `e2e_step` first copies the step's inputs
    (q, new K/V rows, slot table, lengths) from ONE pinned host buffer, and copies the output back to pinned host
    memory and waits for it (the caller reads the result)."""

    def __init__(self, w, ctx):
        from diopi_b200 import _lib
        from diopi_b200.runtime import Tensor, check_returncode
        self.w, self.ctx, self.check = w, ctx, check_returncode
        impl = _lib.load().impl
        self.copy_kv, self.decode = impl.diopiDestIndexCopyKV, impl.diopiTokenDecodeAttentionInference
        self.out = torch.empty_like(w.q)
        names = ("q", "k_new", "v_new", "dest_loc", "b_loc", "b_start_loc", "b_seq_len")
        offs, total_in = {}, 0
        for k in names:
            t = getattr(w, k)
            offs[k] = total_in
            total_in += (t.numel() * t.element_size() + 255) // 256 * 256
        self.host_buf = torch.empty(total_in, dtype=torch.uint8).pin_memory()
        self.dev_buf = torch.empty(total_in, dtype=torch.uint8, device="cuda")
        dev_in = {}
        for k in names:
            t = getattr(w, k)
            nb = t.numel() * t.element_size()
            self.host_buf[offs[k]:offs[k] + nb].view(t.dtype).view(t.shape).copy_(t.cpu())
            dev_in[k] = self.dev_buf[offs[k]:offs[k] + nb].view(t.dtype).view(t.shape)
        self.host_out = torch.empty(self.out.shape, dtype=self.out.dtype).pin_memory()
        self.h2d = sum(getattr(w, k).numel() * getattr(w, k).element_size() for k in names)
        self.d2h = self.host_out.numel() * self.host_out.element_size()
        self._keep = [Tensor(getattr(w, k)) for k in names] + [Tensor(v) for v in dev_in.values()] + [Tensor(w.k_pool), Tensor(w.v_pool), Tensor(self.out)]
        n = len(names)
        res = dict(zip(names, self._keep[:n]))
        stg = dict(zip(names, self._keep[n:2 * n]))
        kp, vp, out = self._keep[2 * n:]
        c = ctx.handle
        self._dev_args = ((c, kp.handle, res["k_new"].handle, res["dest_loc"].handle), (c, vp.handle, res["v_new"].handle, res["dest_loc"].handle),
                          (c, out.handle, res["q"].handle, kp.handle, vp.handle, res["b_loc"].handle, res["b_start_loc"].handle, res["b_seq_len"].handle,
                           int(w.max_input_len)))
        self._e2e_args = ((c, kp.handle, stg["k_new"].handle, stg["dest_loc"].handle), (c, vp.handle, stg["v_new"].handle, stg["dest_loc"].handle),
                          (c, out.handle, stg["q"].handle, kp.handle, vp.handle, stg["b_loc"].handle, stg["b_start_loc"].handle, stg["b_seq_len"].handle,
                           int(w.max_input_len)))

    def _calls(self, args, dec_events=None):
        rc = self.copy_kv(*args[0]) or self.copy_kv(*args[1])
        if dec_events is not None:
            dec_events[0].record()
        rc = rc or self.decode(*args[2])
        if dec_events is not None:
            dec_events[1].record()
        if rc:
            self.check("decode step", rc)
        self.ctx.release()

    def device_step(self, dec_events=None):
        self._calls(self._dev_args, dec_events)

    def e2e_step(self):
        self.dev_buf.copy_(self.host_buf, non_blocking=True)
        self._calls(self._e2e_args)
        self.host_out.copy_(self.out, non_blocking=True)
        self.ctx.synchronize()  # the caller reads the result


def timed_steps(runner, K, warmup, barrier, with_decode_events=True):
    """K device steps after `warmup` untimed ones, CUDA events on the launching stream around the region and around
    every step; returns (ms per step [mean over the region], per-step list, decode-call ms mean, clocks)."""
    for _ in range(warmup):
        runner.device_step()
    barrier()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(K + 1)]
    dec = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)] if with_decode_events else None
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    marks[0].record()
    for i in range(K):
        runner.device_step(dec[i] if dec else None)
        marks[i + 1].record()
    barrier()
    sampler.stop()
    per_step = [marks[i].elapsed_time(marks[i + 1]) for i in range(K)]
    dec_ms = (sum(a.elapsed_time(b) for a, b in dec) / K) if dec else None
    return marks[0].elapsed_time(marks[K]) / K, per_step, dec_ms, sampler.summary()


def timed_e2e(runner, K, barrier):
    for _ in range(3):
        runner.e2e_step()
    barrier()
    per_step = []
    t_begin = time.perf_counter()
    for _ in range(K):
        t0 = time.perf_counter()
        runner.e2e_step()
        per_step.append((time.perf_counter() - t0) * 1e3)
    barrier()
    return (time.perf_counter() - t_begin) * 1e3 / K, per_step


def max_over_ranks(values, n):
    if n == 1:
        return list(values)
    import torch.distributed as dist
    t = torch.tensor(list(values), device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def strong_cfg5_leg(n, rank, ctx, barrier, K):
    """The 64-head decode config split by heads over the N ranks (all of it on one GPU at N = 1): the strong-scaling
    figure. Every rank holds [slots, 64/N, 128] shards of the pools and the same slot tables."""
    from diopi_b200 import workloads
    h0, h1 = workloads.shard_heads(64, n, rank)
    w = workloads.decode("cfg5", device="cuda", head_range=(h0, h1))
    runner = StepRunner(w, ctx)
    ms, per_step, dec_ms, clocks = timed_steps(runner, K, 3, barrier)
    e2e_ms, _ = timed_e2e(runner, min(K, 10), barrier)
    ms, dec_ms, e2e_ms = max_over_ranks([ms, dec_ms, e2e_ms], n)
    step_bytes = w.fused_bytes() + w.copy_bytes()
    rec = {"workload": "configs[4]: B128 H64 D128 fp16, lens U[1024,8192], 64 heads split over the ranks", "ms_per_step": ms,
           "ms_per_step_median": statistics.median(per_step), "ms_per_step_best": min(per_step), "decode_call_ms": dec_ms,
           "per_gpu_gbs": step_bytes / (ms * 1e-3) / 1e9, "job_gbs": step_bytes * n / (ms * 1e-3) / 1e9, "heads_per_gpu": h1 - h0, "sum_len": w.sum_len,
           "pool_gb_per_gpu": 2 * w.k_pool.numel() * w.k_pool.element_size() / 1e9, "e2e_ms": e2e_ms, "steps": K, "scaling": "strong", "clocks": clocks}
    del runner, w
    torch.cuda.empty_cache()
    return rec


def l2_warm_leg(ctx, barrier):
    """The same step on a batch whose K/V rows (8 requests x 512 tokens x 2 x 8 KB = 67 MB) stay in the 126 MB L2
    from one step to the next: what the kernels do when DRAM is out of the way."""
    from diopi_b200 import workloads
    w = workloads.decode("cfg2w", device="cuda")
    runner = StepRunner(w, ctx)
    ms, per_step, dec_ms, clocks = timed_steps(runner, 50, 5, barrier)
    b = w.fused_bytes() + w.copy_bytes()
    return {"workload": "B8 H32 D128 fp16, 512 tokens each: K/V rows resident in L2", "ms_per_step": ms, "ms_per_step_median": statistics.median(per_step),
            "ms_per_step_best": min(per_step), "gbs": b / (ms * 1e-3) / 1e9, "bytes": b, "clocks": clocks}


def matmul_allreduce_leg(n, rank):
    """diopiMatmulAllReduce on the N ranks of this run (M 64, N 4096, K 4096 / N per rank, bf16): every rank's result
    against an fp32 torch product of the same inputs all-reduced by NCCL, identical bits on all ranks, and the
    time per call beside torch.matmul + NCCL all-reduce."""
    import torch.distributed as dist
    from diopi_b200 import tp_group, tpbench
    from diopi_b200.runtime import Context
    from diopi_b200 import functions as F
    M, N, K = 64, 4096, 4096 // n
    tp_group.create("bench_tp", max_tiles=((M + 127) // 128) * ((N + 127) // 128))
    rec = {"world": n, "M": M, "N": N, "K_per_rank": K, "dtype": "bf16"}
    try:
        ctx = Context()
        x1, x2, bias = tpbench.inputs(rank, M, K, N, torch.bfloat16, "cuda")
        out = F.matmul_all_reduce(x1, x2, bias, "bench_tp", ctx=ctx)
        torch.cuda.synchronize()
        want = x1.float() @ x2.float()
        if bias is not None:
            want += bias.float()
        dist.all_reduce(want)
        err = float((out.float() - want).abs().max())
        ok = torch.allclose(out.float(), want, rtol=1e-2, atol=1e-2)
        gathered = [torch.empty_like(out) for _ in range(n)]
        dist.all_gather(gathered, out)
        same = all(torch.equal(g, gathered[0]) for g in gathered)
        flag = torch.tensor([int(ok and same)], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        rec.update(parity="ok" if bool(flag.item()) else "MISMATCH", parity_vs="fp32 torch product of the same inputs, all-reduced by NCCL (rtol = atol = 1e-2)",
                   max_abs_err=err, identical_bits=bool(same), form="two-shot" if n >= 4 else "one-shot")
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
        fused_ms, _ = tpbench.timed(lambda: F.matmul_all_reduce(x1, x2, bias, "bench_tp", out=out, ctx=ctx), 50, 5)

        def pair():
            torch.matmul(x1, x2, out=out)
            if bias is not None:
                out.add_(bias)
            dist.all_reduce(out)
        pair_ms, _ = tpbench.timed(pair, 50, 5)
        sampler.stop()
        rec.update(us=fused_ms * 1e3, nccl_pair_us=pair_ms * 1e3, clocks=sampler.summary())
    finally:
        tp_group.destroy("bench_tp")
    return rec


def run_b200(args):
    rank, local_rank, world = dist_env()
    n = world
    if args.gpus != n and rank == 0 and n > 1:
        print(f"[bench] --gpus {args.gpus} but WORLD_SIZE={n}; using {n}", file=sys.stderr)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the library has no CPU path")
    torch.cuda.set_device(local_rank)
    if n > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from diopi_b200 import build, workloads
    from diopi_b200.runtime import Context
    if rank == 0:
        build.build()
    if n > 1:
        dist.barrier()

    name = args.workload
    if name in ("cfg2", "cfg2s"):
        w = workloads.decode(name, device="cuda", float_seed=1002 + 97 * rank)
        scaling = "weak"
    else:
        # --shard-of N on one GPU builds rank 0's shard of an N-way split (to study the per-GPU kernel of a wide split)
        h0, h1 = workloads.shard_heads(64, max(n, args.shard_of), rank)
        w = workloads.decode("cfg5", device="cuda", head_range=(h0, h1))
        scaling = "strong"
    ctx = Context()
    runner = StepRunner(w, ctx)
    out = runner.out

    def barrier():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- timed region: K steps, events on the launching stream; the decode call is bracketed separately ----
    K, W = args.steps, max(args.warmup, 3)
    total_ms_per_step, per_step, dec_ms, clocks = timed_steps(runner, K, W, barrier)
    if args.kernels_only:
        if rank == 0:
            print(json.dumps({"workload": name, "ms_per_step": total_ms_per_step, "decode_ms": dec_ms,
                              "decode_gbs": w.fused_bytes() / (dec_ms * 1e-3) / 1e9, "sum_len": w.sum_len}), flush=True)
        return

    # ---- end to end: the same step driven from pinned host buffers ----
    e2e_ms, e2e_steps = timed_e2e(runner, K, barrier)

    # ---- max over ranks ----
    ms_per_step, dec_ms, e2e_ms = max_over_ranks([total_ms_per_step, dec_ms, e2e_ms], n)
    bytes_local = torch.tensor([float(w.fused_bytes() + w.copy_bytes()), float(w.q.shape[0])], device="cuda", dtype=torch.float64)
    if n > 1:
        dist.all_reduce(bytes_local, op=dist.ReduceOp.SUM)
    job_bytes, job_tokens = bytes_local.tolist()
    if scaling == "strong":
        job_tokens = float(w.q.shape[0])  # every rank serves the same requests
    value = job_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- all-gather of the per-head outputs (only where a caller wants the full tensor): timed apart ----
    gather = None
    if n > 1:
        from diopi_b200 import head_shard
        full = head_shard.allocate_full(out, n) if scaling == "weak" else None
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if full is not None:
            for _ in range(3):
                head_shard.all_gather_heads(out, full)
            barrier()
            g0.record()
            for _ in range(20):
                head_shard.all_gather_heads(out, full)
            g1.record()
            barrier()
            gt = max_over_ranks([g0.elapsed_time(g1) / 20], n)[0]
            gather = {"ms": gt, "bytes_per_rank": out.numel() * out.element_size(), "in_timed_region": False}

    line = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        per_gpu_dec_gbs = w.fused_bytes() / (dec_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": n, "steps": K, "warmup": W,
            "ms_per_step": ms_per_step, "ms_per_step_median": statistics.median(per_step), "ms_per_step_best": min(per_step),
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": bench_config(name, n, w),
            "tokens_per_s": job_tokens / (ms_per_step * 1e-3),
            "pct_of_8tbs_per_gpu": value / n / NOMINAL_HBM_GBS * 100.0,
            "roofline": {"bound": "hbm", "kernel": "decode_split_kernel (+ decode_combine_kernel)", "achieved": per_gpu_dec_gbs, "peak": peak,
                         "unit": "GB/s", "frac": per_gpu_dec_gbs / peak, "peak_source": peak_kind,
                         "algorithmic_bytes_per_launch": w.fused_bytes(), "avg_launch_ms": dec_ms,
                         "traffic": (NCU_TRAFFIC_BYTES_PER_TOKEN * w.sum_len) if name in ("cfg2", "cfg2s") else None},
            "e2e": {"value": job_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms, "ms_per_step_median": statistics.median(e2e_steps),
                    "ms_per_step_best": min(e2e_steps), "h2d_bytes_per_step": runner.h2d, "d2h_bytes_per_step": runner.d2h,
                    "note": "KV pool is device-resident state; per-step inputs come from pinned host memory; one sync per step"},
            "gpu_launches": 4 * K,
            "clocks": clocks,
        }
        if gather:
            line["allgather"] = gather
    cpu_w = w if (n == 1 and not args.no_cpu_baseline) else None
    if cpu_w is not None and rank == 0:
        line["cpu_baseline"] = cpu_baseline(w, budget_s=args.cpu_budget)
    del runner, out, w, cpu_w
    torch.cuda.empty_cache()

    # ---- further legs: every one guarded, so that the headline above is printed whatever happens to them ----
    def guarded(fn, *a):
        try:
            return fn(*a)
        except Exception as e:  # noqa: BLE001
            return {"error": f"{type(e).__name__}: {e}"[:300]}

    if name == "cfg2" and not args.headline_only:
        strong = guarded(strong_cfg5_leg, n, rank, ctx, barrier, min(K, 20))
        if rank == 0:
            line["strong_cfg5"] = strong
        if n == 1:
            line["l2_warm"] = guarded(l2_warm_leg, ctx, barrier)
            from diopi_b200 import opbench
            ops = {}
            for key, op, kw in (("prefill_cfg4", "prefill", {}), ("prefill_d64", "prefill", {"head_dim": 64}), ("prefill_d256", "prefill", {"head_dim": 256}),
                                ("rms_norm_cfg3", "rms_norm", {}), ("rotary_cfg3", "rotary", {}), ("rope_copy_kv", "rope_copy_kv", {}),
                                ("rms_norm_bwd", "rms_norm_bwd", {}), ("penalty_cfg5", "penalty", {}), ("copy_kv", "copy_kv", {}), ("qk", "qk", {}),
                                ("pv", "pv", {}), ("paged_gqa_64q_8kv", "paged", {"kv_heads": 8}), ("paged_mha_64q_64kv", "paged", {"kv_heads": 64})):
                ops[key] = guarded(lambda: opbench.run_op(op, "full", iters=10, warmup=3, ctx=ctx, **kw))
                torch.cuda.empty_cache()
            line["ops"] = ops
        else:
            mar = guarded(matmul_allreduce_leg, n, rank)
            if rank == 0:
                line["matmul_allreduce"] = mar
    if rank == 0:
        print(json.dumps(line), flush=True)
    if n > 1:
        dist.barrier()
        dist.destroy_process_group()


def bench_config(name, n, w):
    """The `config` object of the JSON line; both arms print the same keys."""
    return {"workload": workload_description(name, n, w.q.shape[1]), "batch": int(w.q.shape[0]), "heads_per_gpu": int(w.q.shape[1]),
            "head_dim": int(w.q.shape[2]), "sum_len": w.sum_len, "seed": w.meta["seed"], "pool_slots": w.meta["slots"],
            "l2": "inputs larger than L2: every step streams %.2f GB of K/V per GPU through a 126 MB L2" % (w.fused_bytes() / 1e9),
            "parallelism": f"heads sharded over {n} GPU(s), no collective on the data path"}


# ------------------------------------------------------------------------------------------------ CPU oracle timing
def oracle_step(c):
    from oracle import golden
    golden.destindex_copy_kv(c["k_new"], c["dest_loc"], c["k_pool"])
    golden.destindex_copy_kv(c["v_new"], c["dest_loc"], c["v_pool"])
    att = torch.zeros(c["q"].shape[1], c["width"], dtype=c["q"].dtype)
    golden.token_attention(c["q"], c["k_pool"], att, c["b_loc"], c["b_start_loc"], c["b_seq_len"], c["max_input_len"])
    out = torch.zeros_like(c["q"])
    golden.token_softmax_reducev(att, c["v_pool"], out, c["b_loc"], c["b_start_loc"], c["b_seq_len"], c["max_input_len"], 0)
    return out


def cpu_copy(w, requests=None):
    """Host copy of a workload, optionally restricted to its first `requests` requests (the pool stays whole)."""
    B = w.q.shape[0] if requests is None else requests
    lens = w.b_seq_len[:B].cpu()
    c = dict(q=w.q[:B].cpu(), k_new=w.k_new[:B].cpu(), v_new=w.v_new[:B].cpu(), dest_loc=w.dest_loc[:B].cpu(), k_pool=w.k_pool.cpu(),
             v_pool=w.v_pool.cpu(), b_loc=w.b_loc[:B].cpu(), b_start_loc=w.b_start_loc[:B].cpu(), b_seq_len=lens, max_input_len=w.max_input_len)
    c["width"] = int((c["b_start_loc"] + lens).max())
    H, D, e = w.q.shape[1], w.q.shape[2], w.q.element_size()
    sl = int(lens.sum())
    c["bytes"] = 2 * sl * H * D * e + 2 * B * H * D * e + sl * 4 + 2 * B * 4 + 2 * (2 * B * H * D * e + B * 4)
    c["requests"] = B
    return c


def cpu_baseline(w, budget_s=20.0):
    """The CPU oracle on the same workload, bounded to about budget_s seconds of work, on all host threads."""
    torch.set_num_threads(os.cpu_count() or 1)
    c = cpu_copy(w)
    t0 = time.perf_counter()
    oracle_step(c)
    first = time.perf_counter() - t0
    reps, spent, times = 0, 0.0, []
    while spent < budget_s and reps < 5:
        t0 = time.perf_counter()
        oracle_step(c)
        dt = time.perf_counter() - t0
        times.append(dt)
        spent += dt
        reps += 1
    best = min(times) if times else first
    return {"value": c["bytes"] / best / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port", "ms_per_step": best * 1e3,
            "sample": f"the full step ({c['requests']} requests, {int(c['b_seq_len'].sum())} tokens), best of {max(reps, 1)} after one warm-up; "
                      f"torch {torch.__version__} CPU, os.cpu_count()={os.cpu_count()}"}


# ------------------------------------------------------------------------------------------------ reference arm
def reference_golden():
    """The reference's own golden functions (diopi_test/python/conformance/customized_test.py, class CustomizedTest),
    imported unmodified when a checkout of the reference lies beside this repository; else None."""
    conf = ROOT.parent / "reference" / "diopi_test" / "python" / "conformance"
    if not (conf / "customized_test.py").exists():
        return None
    try:
        sys.path.insert(0, str(conf))
        from customized_test import CustomizedTest
        return CustomizedTest
    except Exception:  # noqa: BLE001
        return None
    finally:
        if str(conf) in sys.path:
            sys.path.remove(str(conf))


def reference_step(G, c):
    """The step through the reference's golden functions: same three calls as oracle_step."""
    G.destindex_copy_kv(c["k_new"], c["dest_loc"].long(), c["k_pool"])
    G.destindex_copy_kv(c["v_new"], c["dest_loc"].long(), c["v_pool"])
    att = torch.zeros(c["q"].shape[1], c["width"], dtype=c["q"].dtype)
    G.token_attention(c["q"], c["k_pool"], att, c["b_loc"], c["b_start_loc"], c["b_seq_len"], c["max_input_len"])
    out = torch.zeros_like(c["q"])
    G.token_softmax_reducev(att, c["v_pool"], out, c["b_loc"], c["b_start_loc"], c["b_seq_len"], c["max_input_len"], 0)
    return out


def run_reference(args):
    """The reference's implementation of this path is Python: torch golden functions evaluated on the host CPU. Where
    a checkout of the reference is mounted they are imported unmodified and timed (kind "reference"); it cannot travel
    to a box without it, so there the oracle port, tested equal to it on the committed fixtures, runs instead (kind
    "port"). Either way on all host threads (a launcher may have set OMP_NUM_THREADS=1 for its ranks), rank 0 only."""
    rank, local_rank, world = dist_env()
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    from diopi_b200 import workloads
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    w = workloads.decode(args.workload, device=dev, float_seed=1002 if args.workload in ("cfg2", "cfg2s") else None)
    G = reference_golden()
    step = (lambda c: reference_step(G, c)) if G is not None else oracle_step
    kind = "reference" if G is not None else "port"
    K, W = args.steps, max(args.warmup, 1)
    c = cpu_copy(w)
    t0 = time.perf_counter()
    step(c)
    first = time.perf_counter() - t0
    # bound the whole run to a few minutes: shrink the sample to the first requests if the full batch is too slow
    budget = 150.0
    if first * (K + W) > budget:
        frac = budget / (first * (K + W))
        c = cpu_copy(w, requests=max(1, int(w.q.shape[0] * frac)))
    for _ in range(W):
        step(c)
    times = []
    for _ in range(K):
        t0 = time.perf_counter()
        step(c)
        times.append(time.perf_counter() - t0)
    sec = sum(times) / K
    value = c["bytes"] / sec / 1e9
    what = "the reference's CustomizedTest golden functions" if G is not None else "CPU oracle port of the golden functions"
    sample = f"{c['requests']} of {w.q.shape[0]} requests per step ({int(c['b_seq_len'].sum())} tokens), {what}, torch {torch.__version__} CPU"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": sec * 1e3, "ms_per_step_median": statistics.median(times) * 1e3, "ms_per_step_best": min(times) * 1e3,
            "higher_is_better": True, "scaling": "weak" if args.workload in ("cfg2", "cfg2s") else "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": bench_config(args.workload, world, w),
            "tokens_per_s": c["requests"] / sec,
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=["cfg2", "cfg2s", "cfg5"])
    ap.add_argument("--kernels-only", action="store_true", help="run warm-up + timed steps only (for profiler captures)")
    ap.add_argument("--shard-of", type=int, default=1, help="cfg5 on one GPU: hold only rank 0's head shard of an N-way split")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--headline-only", action="store_true", help="skip the legs after the headline (strong cfg5, per-op figures, matmul + all-reduce)")
    ap.add_argument("--cpu-budget", type=float, default=20.0)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
