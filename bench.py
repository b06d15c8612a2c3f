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
sync per step). `--impl reference` times the CPU oracle (the restated golden functions, all host threads) on the
same workload instead.
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
    from diopi_b200 import build, functions as F, workloads
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
    out = torch.empty_like(w.q)

    def step():
        F.destindex_copy_kv(w.k_new, w.dest_loc, w.k_pool, ctx=ctx)
        F.destindex_copy_kv(w.v_new, w.dest_loc, w.v_pool, ctx=ctx)
        F.token_decode_attention(w.q, w.k_pool, w.v_pool, out, w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len, ctx=ctx)
        ctx.release()

    def barrier():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    # ---- timed region: K steps, events on the launching stream; the decode call is bracketed separately ----
    K = args.steps
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dec = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    ev0.record()
    for i in range(K):
        F.destindex_copy_kv(w.k_new, w.dest_loc, w.k_pool, ctx=ctx)
        F.destindex_copy_kv(w.v_new, w.dest_loc, w.v_pool, ctx=ctx)
        dec[i][0].record()
        F.token_decode_attention(w.q, w.k_pool, w.v_pool, out, w.b_loc, w.b_start_loc, w.b_seq_len, w.max_input_len, ctx=ctx)
        dec[i][1].record()
        ctx.release()
    ev1.record()
    barrier()
    sampler.stop()
    total_ms = ev0.elapsed_time(ev1)
    dec_ms = sum(a.elapsed_time(b) for a, b in dec) / K
    if args.kernels_only:
        if rank == 0:
            print(json.dumps({"workload": name, "ms_per_step": total_ms / K, "decode_ms": dec_ms,
                              "decode_gbs": w.fused_bytes() / (dec_ms * 1e-3) / 1e9, "sum_len": w.sum_len}), flush=True)
        return

    # ---- end to end: the same step driven from pinned host buffers ----
    # The engine stages the step's inputs (q, new K/V rows, slot tables, lengths) in ONE pinned host buffer and moves
    # them with one H2D copy; tensor handles of the persistent device buffers are made once, as a framework would.
    from diopi_b200.runtime import Tensor
    names = ("q", "k_new", "v_new", "dest_loc", "b_loc", "b_start_loc", "b_seq_len")
    offs, total_in = {}, 0
    for k in names:
        t = getattr(w, k)
        offs[k] = total_in
        total_in += (t.numel() * t.element_size() + 255) // 256 * 256
    host_buf = torch.empty(total_in, dtype=torch.uint8).pin_memory()
    dev_buf = torch.empty(total_in, dtype=torch.uint8, device="cuda")
    dev_in = {}
    for k in names:
        t = getattr(w, k)
        nb = t.numel() * t.element_size()
        host_buf[offs[k]:offs[k] + nb].view(t.dtype).view(t.shape).copy_(t.cpu())
        dev_in[k] = dev_buf[offs[k]:offs[k] + nb].view(t.dtype).view(t.shape)
    host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    h2d = sum(getattr(w, k).numel() * getattr(w, k).element_size() for k in names)
    d2h = host_out.numel() * host_out.element_size()
    hd = {k: Tensor(v) for k, v in dev_in.items()}
    h_kpool, h_vpool, h_out = Tensor(w.k_pool), Tensor(w.v_pool), Tensor(out)

    def e2e_step():
        dev_buf.copy_(host_buf, non_blocking=True)
        F.destindex_copy_kv(hd["k_new"], hd["dest_loc"], h_kpool, ctx=ctx)
        F.destindex_copy_kv(hd["v_new"], hd["dest_loc"], h_vpool, ctx=ctx)
        F.token_decode_attention(hd["q"], h_kpool, h_vpool, h_out, hd["b_loc"], hd["b_start_loc"], hd["b_seq_len"], w.max_input_len, ctx=ctx)
        host_out.copy_(out, non_blocking=True)
        ctx.release()
        torch.cuda.synchronize()  # the caller reads the result

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        e2e_step()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / K

    # ---- max over ranks ----
    stats = torch.tensor([total_ms, dec_ms, e2e_ms], device="cuda", dtype=torch.float64)
    bytes_local = torch.tensor([float(w.fused_bytes() + w.copy_bytes()), float(w.q.shape[0])], device="cuda", dtype=torch.float64)
    if n > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(bytes_local, op=dist.ReduceOp.SUM)
    total_ms, dec_ms, e2e_ms = stats.tolist()
    job_bytes, job_tokens = bytes_local.tolist()
    if scaling == "strong":
        job_tokens = float(w.q.shape[0])  # every rank serves the same requests
    ms_per_step = total_ms / K
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
            gt = torch.tensor([g0.elapsed_time(g1) / 20], device="cuda", dtype=torch.float64)
            dist.all_reduce(gt, op=dist.ReduceOp.MAX)
            gather = {"ms": gt.item(), "bytes_per_rank": out.numel() * out.element_size(), "in_timed_region": False}

    if rank == 0:
        peak, peak_kind = measured_peak()
        per_gpu_dec_gbs = w.fused_bytes() / (dec_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": n, "steps": K, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": workload_description(name, n, w.q.shape[1]), "batch": int(w.q.shape[0]), "heads_per_gpu": int(w.q.shape[1]),
                       "head_dim": int(w.q.shape[2]), "sum_len": w.sum_len, "seed": w.meta["seed"], "pool_slots": w.meta["slots"],
                       "l2": "inputs larger than L2: every step streams %.2f GB of K/V per GPU through a 126 MB L2" % (w.fused_bytes() / 1e9),
                       "parallelism": f"heads sharded over {n} GPU(s), no collective on the data path"},
            "tokens_per_s": job_tokens / (ms_per_step * 1e-3),
            "pct_of_8tbs_per_gpu": value / n / NOMINAL_HBM_GBS * 100.0,
            "roofline": {"bound": "hbm", "kernel": "decode_split_kernel (+ decode_combine_kernel)", "achieved": per_gpu_dec_gbs, "peak": peak,
                         "unit": "GB/s", "frac": per_gpu_dec_gbs / peak, "peak_source": peak_kind,
                         "algorithmic_bytes_per_launch": w.fused_bytes(), "avg_launch_ms": dec_ms,
                         "traffic": (NCU_TRAFFIC_BYTES_PER_TOKEN * w.sum_len) if name in ("cfg2", "cfg2s") else None},
            "e2e": {"value": job_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "note": "KV pool is device-resident state; per-step inputs come from pinned host memory"},
            "gpu_launches": 4 * K,
            "clocks": sampler.summary(),
        }
        if gather:
            line["allgather"] = gather
        if n == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(w, budget_s=args.cpu_budget)
        print(json.dumps(line), flush=True)
    if n > 1:
        dist.barrier()
        dist.destroy_process_group()


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
    """The CPU oracle on the same workload, bounded to about budget_s seconds of work."""
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
def run_reference(args):
    """The reference's own implementation of the path is Python (torch golden functions, evaluated on CPU in the
    reference's CI when no GPU is there); it cannot travel, so the oracle port — tested equal to it on the committed
    fixtures — is what runs here, with all host threads."""
    rank, local_rank, world = dist_env()
    if rank != 0:
        return
    from diopi_b200 import workloads
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    w = workloads.decode(args.workload, device=dev)
    K, W = args.steps, max(args.warmup, 1)
    c = cpu_copy(w)
    t0 = time.perf_counter()
    oracle_step(c)
    first = time.perf_counter() - t0
    # bound the whole run to a few minutes: shrink the sample to the first requests if the full batch is too slow
    budget = 150.0
    if first * (K + W) > budget:
        frac = budget / (first * (K + W))
        c = cpu_copy(w, requests=max(1, int(w.q.shape[0] * frac)))
    for _ in range(W):
        oracle_step(c)
    t0 = time.perf_counter()
    for _ in range(K):
        oracle_step(c)
    sec = (time.perf_counter() - t0) / K
    value = c["bytes"] / sec / 1e9
    sample = f"{c['requests']} of {w.q.shape[0]} requests per step ({int(c['b_seq_len'].sum())} tokens), CPU oracle port of the golden functions"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak" if args.workload == "cfg2" else "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": workload_description(args.workload, world, w.q.shape[1]), "batch": int(w.q.shape[0]),
                       "sum_len": w.sum_len, "seed": w.meta["seed"]},
            "tokens_per_s": c["requests"] / sec,
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
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
    ap.add_argument("--cpu-budget", type=float, default=20.0)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
