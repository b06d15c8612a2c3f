"""diopiMatmulAllReduce on N GPUs, one process each (start with torchrun; a plain `python -m diopi_b200.tpbench` is a
group of one):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m diopi_b200.tpbench [--rows 64 --k-total 4096 --cols 4096] [--check] [--iters 50]

Every rank holds x1 [M, K_total / N] and x2 [K_total / N, n] of a row-parallel linear layer. Rank 0 prints one JSON line:
the time per call of the fused kernel (CUDA events, max over ranks) beside the same product done as torch.matmul
followed by an NCCL all-reduce, and with --check the comparison of every rank's result with the sum the CPU oracle
forms from all ranks' inputs (inputs are seeded per rank, so every rank can rebuild all of them).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent


def inputs(rank, M, K, N, dtype, device):
    g = torch.Generator().manual_seed(4000 + rank)
    x1 = torch.randn(M, K, generator=g).to(dtype)
    x2 = (torch.randn(K, N, generator=g) * (K ** -0.5)).to(dtype)
    bias = torch.randn(N, generator=g).to(dtype) if rank == 0 else None   # as a row-parallel layer does: bias once
    return x1.to(device), x2.to(device), (bias.to(device) if bias is not None else None)


def timed(fn, iters, warmup):
    """(device ms per call, host ms per call spent queueing it): when the two are close, the host is the limit."""
    import time
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    h0 = time.perf_counter()
    for _ in range(iters):
        fn()
    h1 = time.perf_counter()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters, (h1 - h0) * 1e3 / iters], device="cuda")
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0].item()), float(t[1].item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=64)
    ap.add_argument("--k-total", type=int, default=4096)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f16"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--x2", default="rowmajor", choices=["rowmajor", "kmajor"], help="kmajor: x2 is the transposed view of an [N, K] weight")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from . import functions as F
    from . import tp_group
    from .runtime import Context
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    M, N, K = args.rows, args.cols, args.k_total // world
    tiles = ((M + 127) // 128) * ((N + 127) // 128)
    tp_group.create("tp", max_tiles=tiles)
    ctx = Context()
    x1, x2, bias = inputs(rank, M, K, N, dtype, "cuda")
    if args.x2 == "kmajor":
        x2 = x2.t().contiguous().t()   # same values, stored as [N, K]
    out = torch.empty(M, N, dtype=dtype, device="cuda")
    rec = {"op": "matmul_all_reduce", "mode": os.environ.get("DIOPI_B200_MAR_MODE", "auto"), "world": world, "M": M, "N": N, "K_per_rank": K, "dtype": args.dtype, "x2": args.x2}

    # handles made once, the entry point called directly: the host side of a call is then a few microseconds, as it is
    # for a C++ consumer, and the figure is the device's
    from . import _lib
    from .runtime import Tensor, check_returncode
    impl = _lib.load().impl
    t_out, t_x1, t_x2 = Tensor(out), Tensor(x1), Tensor(x2)
    t_bias = Tensor(bias) if bias is not None else None

    def fused():
        rc = impl.diopiMatmulAllReduce(ctx.handle, t_out.handle, t_x1.handle, t_x2.handle, t_bias.handle if t_bias else None, b"tp", b"sum", 0, 1)
        if rc != 0:
            check_returncode("diopiMatmulAllReduce", rc)

    if args.check:
        sys.path.insert(0, str(ROOT))
        from oracle import golden
        fused()
        torch.cuda.synchronize()
        cpu = [inputs(r, M, K, N, dtype, "cpu") for r in range(world)]
        want = golden.matmul_all_reduce([c[0] for c in cpu], [c[1] for c in cpu], [c[2] for c in cpu])
        err = float((out.cpu().float() - want.float()).abs().max())
        ok = torch.allclose(out.cpu().float(), want.float(), rtol=1e-2, atol=1e-2)
        same = True
        if world > 1:
            gathered = [torch.empty_like(out) for _ in range(world)]
            dist.all_gather(gathered, out)
            same = all(torch.equal(g, gathered[0]) for g in gathered)
            flag = torch.tensor([int(ok and same)], device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok = bool(flag.item())
        rec.update(parity="ok" if (ok and same) else "MISMATCH", max_abs_err=err, ranks_identical=bool(same))

    rec["fused_ms"], rec["fused_host_ms"] = timed(fused, args.iters, args.warmup)

    def unfused():
        torch.matmul(x1, x2, out=out)
        if bias is not None:
            out.add_(bias)
        if world > 1:
            dist.all_reduce(out)
    rec["matmul_plus_nccl_allreduce_ms"], rec["matmul_plus_nccl_allreduce_host_ms"] = timed(unfused, args.iters, args.warmup)
    flops = 2.0 * M * N * K
    rec["gemm_tflops_per_rank_in_fused_call"] = flops / rec["fused_ms"] / 1e9
    rec["nvlink_bytes_sent_per_rank"] = (world - 1) * M * N * 4
    if rank == 0:
        print(json.dumps(rec), flush=True)
    tp_group.destroy("tp")
    if world > 1:
        dist.destroy_process_group()
    return 0 if rec.get("parity", "ok") == "ok" else 1


if __name__ == "__main__":
    sys.exit(main())
