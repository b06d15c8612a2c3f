"""diopiMatmulAllReduce on several GPUs, one process each: the body of the multi-rank tests. Start with torchrun:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        tests/mar_ranks.py check   [--form 0|1|2] [--rows 200 --cols 1032 --k-total 4096]
        tests/mar_ranks.py timeout [--limit-ms 50]

check    every rank's result against the sum the CPU oracle forms from all ranks' inputs (inputs are seeded per rank,
         so every rank can rebuild all of them), identical bits on all ranks, over several shapes and calls.
timeout  the failure the bounded wait exists for, made on the host: rank 1 leaves one call out. The kernels of the
         other ranks give up after the group's limit and return; their next call reports status 3; the group then
         refuses calls on every rank that saw the mark; after Destroy + Create on every rank the group works again.
         Nothing traps, nothing waits without a limit, and no rank leaves with a kernel in flight.

Rank 0 prints one JSON line; the exit code is 0 only when every rank passed."""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from diopi_b200 import functions as F, tp_group  # noqa: E402
from diopi_b200.runtime import Context, DiopiError  # noqa: E402
from diopi_b200.tpbench import inputs  # noqa: E402
from oracle import golden  # noqa: E402


def all_ok(flag: bool) -> bool:
    t = torch.tensor([int(flag)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item())


def run_check(args, rank, world):
    dtype = torch.bfloat16
    shapes = [(args.rows, args.k_total // world, args.cols), (64, 4096 // world, 4096), (8, 64, 1024), (300, 128, 520)]
    tiles = max(((m + 127) // 128) * ((n + 127) // 128) for m, _, n in shapes)
    tp_group.create("tp", max_tiles=tiles)
    tp_group.set_option("tp", "form", args.form)
    ctx = Context()
    worst, ok, same = 0.0, True, True
    for (M, K, N) in shapes:
        x1, x2, bias = inputs(rank, M, K, N, dtype, "cuda")
        cpu = [inputs(r, M, K, N, dtype, "cpu") for r in range(world)]
        want = golden.matmul_all_reduce([c[0] for c in cpu], [c[1] for c in cpu], [c[2] for c in cpu])
        for rep in range(3):   # both halves of the staging area, and a mark left from the call before
            out = F.matmul_all_reduce(x1, x2, bias, "tp", ctx=ctx)
            torch.cuda.synchronize()
            worst = max(worst, float((out.cpu().float() - want.float()).abs().max()))
            ok = ok and torch.allclose(out.cpu().float(), want.float(), rtol=1e-2, atol=1e-2)
            gathered = [torch.empty_like(out) for _ in range(world)]
            dist.all_gather(gathered, out)
            same = same and all(torch.equal(g, gathered[0]) for g in gathered)
    passed = all_ok(ok and same)
    tp_group.destroy("tp")
    return passed, {"check": "parity", "world": world, "form": {0: "auto", 1: "one-shot", 2: "two-shot"}[args.form], "shapes": shapes,
                    "parity": "ok" if passed else "MISMATCH", "max_abs_err": worst, "ranks_identical": bool(same)}


def run_timeout(args, rank, world):
    dtype = torch.bfloat16
    M, K, N = 64, 256, 512
    tp_group.create("tp", max_tiles=8, wait_limit_ms=args.limit_ms)
    ctx = Context()
    x1, x2, bias = inputs(rank, M, K, N, dtype, "cuda")
    good = F.matmul_all_reduce(x1, x2, bias, "tp", ctx=ctx).clone()
    torch.cuda.synchronize()
    dist.barrier()
    notes = {}
    # --- the failure: rank 1 leaves this call out ---
    t0 = time.perf_counter()
    if rank != 1:
        F.matmul_all_reduce(x1, x2, bias, "tp", ctx=ctx)   # launches; the kernel gives up after the limit and returns
        torch.cuda.synchronize()
    notes["gave_up_after_ms"] = (time.perf_counter() - t0) * 1e3
    dist.barrier()   # host-side: everybody is between steps, nothing in flight
    # --- the GPU still answers a plain op ---
    alive = float((torch.ones(1024, device="cuda") * 2).sum().item()) == 2048.0
    # --- the next call reports status 3 or is refused: on every rank that gave up, and on rank 1 as soon as one of its kernels saw the mark ---
    refused = False
    msg = ""
    for _ in range(2):
        try:
            F.matmul_all_reduce(x1, x2, bias, "tp", ctx=ctx)
            torch.cuda.synchronize()
        except DiopiError as e:
            refused = True
            msg = str(e)
    within = notes["gave_up_after_ms"] < args.limit_ms * 2 * 4 + 2000   # pipeline waits use twice the limit; generous slack for a shared box
    ok_fail = alive and refused and (rank == 1 or within)
    dist.barrier()
    # --- recovery: destroy on every rank, create again, the group works ---
    tp_group.destroy("tp")
    dist.barrier()
    tp_group.create("tp", max_tiles=8, wait_limit_ms=args.limit_ms)
    again = F.matmul_all_reduce(x1, x2, bias, "tp", ctx=ctx)
    torch.cuda.synchronize()
    recovered = torch.equal(again, good)
    passed = all_ok(ok_fail and recovered)
    tp_group.destroy("tp")
    return passed, {"check": "timeout", "world": world, "limit_ms": args.limit_ms, "gave_up_after_ms": notes["gave_up_after_ms"], "gpu_alive": alive,
                    "refused_afterwards": refused, "message": msg[:160], "recovered_after_recreate": bool(recovered), "result": "ok" if passed else "FAILED"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["check", "timeout"])
    ap.add_argument("--rows", type=int, default=200)
    ap.add_argument("--cols", type=int, default=1032)
    ap.add_argument("--k-total", type=int, default=4096)
    ap.add_argument("--limit-ms", type=int, default=50)
    ap.add_argument("--form", type=int, default=0, choices=[0, 1, 2], help="0 chosen per call, 1 one-shot, 2 two-shot")
    args = ap.parse_args()
    world, rank, local = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    passed, rec = (run_check if args.what == "check" else run_timeout)(args, rank, world)
    if rank == 0:
        print(json.dumps(rec), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if passed else 1


if __name__ == "__main__":
    sys.exit(main())
