"""diopiMatmulAllReduce on N GPUs, one process each (start with torchrun; a plain `python -m diopi_b200.tpbench` is a
group of one):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m diopi_b200.tpbench [--rows 64 --k-total 4096 --cols 4096] [--iters 50]

Every rank holds x1 [M, K_total / N] and x2 [K_total / N, n] of a row-parallel linear layer. Rank 0 prints one JSON line:
the time per call of the fused kernel (CUDA events, max over ranks) beside the same product done as torch.matmul
followed by an NCCL all-reduce, with the SM clocks sampled meanwhile. Inputs are seeded per rank, so every rank can
rebuild all of them (the parity check against the CPU oracle lives with the tests: tests/mar_ranks.py).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


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
    ap.add_argument("--form", type=int, default=0, choices=[0, 1, 2], help="0 chosen per call, 1 one-shot, 2 two-shot")
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
    # a group of one may split K over up to eight CTAs per tile when its staging area has room for the slices
    tp_group.create("tp", max_tiles=tiles * 8 if world == 1 else tiles)
    tp_group.set_option("tp", "form", args.form)
    ctx = Context()
    x1, x2, bias = inputs(rank, M, K, N, dtype, "cuda")
    if args.x2 == "kmajor":
        x2 = x2.t().contiguous().t()   # same values, stored as [N, K]
    out = torch.empty(M, N, dtype=dtype, device="cuda")
    rec = {"op": "matmul_all_reduce", "form": {0: "auto", 1: "one-shot", 2: "two-shot"}[args.form], "world": world, "M": M, "N": N, "K_per_rank": K, "dtype": args.dtype, "x2": args.x2}

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

    from .clocks import ClockSampler
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    rec["fused_ms"], rec["fused_host_ms"] = timed(fused, args.iters, args.warmup)
    sampler.stop()
    rec["clocks"] = sampler.summary()

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
    return 0


if __name__ == "__main__":
    sys.exit(main())
