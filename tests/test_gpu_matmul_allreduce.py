"""diopiMatmulAllReduce through the C ABI. A group of one rank runs the whole kernel (TMA, tcgen05 product, staging,
flags, reduction) on one GPU; the multi-rank test starts one process per GPU and needs at least two."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from oracle import golden

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def F(built_libs):
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from diopi_b200 import functions, tp_group
    tp_group.create("solo", max_tiles=64, rank=0, world=1)
    yield functions
    tp_group.destroy("solo")


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(64, 512, 4096), (5, 72, 136), (300, 256, 520), (128, 64, 128), (129, 1024, 264)])
def test_one_rank_matches_oracle(F, dtype, shape):
    M, K, N = shape
    x1, x2, b = rand((M, K), dtype, 1), rand((K, N), dtype, 2, K ** -0.5), rand((N,), dtype, 3)
    want = golden.matmul_all_reduce([x1], [x2], [b])
    got = F.matmul_all_reduce(x1.cuda(), x2.cuda(), b.cuda(), "solo")
    # fp32 accumulation in both; the products are added in another order, the result is rounded once
    torch.testing.assert_close(got.cpu().float(), want.float(), rtol=1e-2, atol=1e-2)
    got2 = F.matmul_all_reduce(x1.cuda(), x2.cuda(), None, "solo")
    torch.testing.assert_close(got2.cpu().float(), golden.matmul_all_reduce([x1], [x2]).float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("tn", ["128", "64", "32"])
@pytest.mark.parametrize("kmajor", [False, True])
def test_tile_widths(F, tn, kmajor):
    """Every tile width the launch can pick (the group option tile_width forces one; 32 exists only for a K-major x2,
    where the request is ignored otherwise), on shapes with ragged edges in all three extents."""
    from diopi_b200 import tp_group
    tp_group.set_option("solo", "tile_width", int(tn))
    for (M, K, N) in ((64, 512, 1024), (37, 200, 328), (130, 64, 96)):
        x1, b = rand((M, K), torch.bfloat16, 20 + M), rand((N,), torch.bfloat16, 21)
        w = rand((N, K), torch.bfloat16, 22 + N, K ** -0.5)
        x2 = w.t() if kmajor else w.t().contiguous()
        want = golden.matmul_all_reduce([x1], [x2], [b])
        got = F.matmul_all_reduce(x1.cuda(), (w.cuda().t() if kmajor else x2.cuda()), b.cuda(), "solo")
        torch.testing.assert_close(got.cpu().float(), want.float(), rtol=1e-2, atol=1e-2)
    tp_group.set_option("solo", "tile_width", 0)


def test_transposed_weight_and_stacked_rows(F):
    dtype = torch.bfloat16
    x1 = rand((2, 70, 128), dtype, 4)
    w = rand((264, 128), dtype, 5, 128 ** -0.5)          # [N, K] as torch.nn.Linear keeps it
    want = golden.matmul_all_reduce([x1], [w.t()])
    got = F.matmul_all_reduce(x1.cuda(), w.cuda().t(), None, "solo")
    assert got.shape == (2, 70, 264)
    torch.testing.assert_close(got.cpu().float(), want.float(), rtol=1e-2, atol=1e-2)
    same = F.matmul_all_reduce(x1.cuda(), w.t().contiguous().cuda(), None, "solo")
    assert torch.equal(got, same)   # the two layouts of x2 give the same bits


def test_calls_in_a_row_use_both_staging_halves(F):
    x1, x2 = rand((64, 256), torch.float16, 6), rand((256, 512), torch.float16, 7, 1 / 16)
    a, b = x1.cuda(), x2.cuda()
    first = F.matmul_all_reduce(a, b, None, "solo").clone()
    for i in range(5):
        # another product in between, so that a stale staging half would show
        F.matmul_all_reduce(a * 2, b, None, "solo")
        assert torch.equal(F.matmul_all_reduce(a, b, None, "solo"), first)
    torch.testing.assert_close(first.cpu().float(), golden.matmul_all_reduce([x1], [x2]).float(), rtol=1e-2, atol=1e-2)


def test_refusals(F):
    from diopi_b200.runtime import DiopiError, FunctionNotImplementedError
    a, b = torch.zeros(8, 64, dtype=torch.float16, device="cuda"), torch.zeros(64, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(DiopiError, match="no group named"):
        F.matmul_all_reduce(a, b, None, "nobody")
    with pytest.raises(FunctionNotImplementedError):
        F.matmul_all_reduce(a, b, None, "solo", reduce_op="max")
    with pytest.raises(DiopiError, match="tiles"):
        F.matmul_all_reduce(torch.zeros(1024, 64, dtype=torch.float16, device="cuda"), torch.zeros(64, 4096, dtype=torch.float16, device="cuda"), None, "solo")
    with pytest.raises(DiopiError):
        F.matmul_all_reduce(a.float(), b.float(), None, "solo")
    with pytest.raises(DiopiError, match="16 bytes"):   # a row pitch of 132 elements is not a multiple of 16 bytes
        F.matmul_all_reduce(a, torch.zeros(64, 132, dtype=torch.float16, device="cuda"), None, "solo")
    assert F.matmul_all_reduce(a[:0], b, None, "solo").shape == (0, 64)


@pytest.mark.parametrize("kmajor", [False, True])
@pytest.mark.parametrize("shape", [(64, 4096, 4096), (17, 1000, 2048), (64, 520, 640), (128, 2048, 1024)])
def test_split_k_in_a_group_of_one(F, shape, kmajor):
    """A group of one rank whose output has few 128-wide tiles splits K over several CTAs per tile (up to 8 slices, here
    4, 4, 2 and 4); the slices are added in the staging area. Ragged K (the last 64-wide k block partly beyond the
    matrix), bias added once, both layouts of x2, and two calls in a row (both halves of the staging area)."""
    from diopi_b200 import tp_group
    M, K, N = shape
    tp_group.create("wide", max_tiles=256, rank=0, world=1)
    try:
        x1, b = rand((M, K), torch.bfloat16, 40 + M), rand((N,), torch.bfloat16, 41)
        w = rand((N, K), torch.bfloat16, 42 + N, K ** -0.5)
        x2 = w.t() if kmajor else w.t().contiguous()
        want = golden.matmul_all_reduce([x1], [x2], [b])
        x2d = w.cuda().t() if kmajor else x2.cuda()
        got = F.matmul_all_reduce(x1.cuda(), x2d, b.cuda(), "wide")
        torch.testing.assert_close(got.cpu().float(), want.float(), rtol=1e-2, atol=1e-2)
        again = F.matmul_all_reduce(x1.cuda(), x2d, b.cuda(), "wide")
        assert torch.equal(again, got)
        # the narrow-tile form without split-K (forced tile width) gives the same numbers to rounding
        tp_group.set_option("wide", "tile_width", 64)
        narrow = F.matmul_all_reduce(x1.cuda(), x2d, b.cuda(), "wide")
        torch.testing.assert_close(narrow.float(), got.float(), rtol=1e-2, atol=1e-2)
    finally:
        tp_group.destroy("wide")


def test_group_options(F):
    from diopi_b200 import tp_group
    from diopi_b200.runtime import DiopiError
    tp_group.set_option("solo", "wait_limit_ms", 100)
    tp_group.set_option("solo", "form", 2)          # a group of one has nobody to hand tiles to: runs as one-shot
    x1, x2 = rand((64, 128), torch.float16, 31).cuda(), rand((128, 256), torch.float16, 32, 0.1).cuda()
    got = F.matmul_all_reduce(x1, x2, None, "solo")
    torch.testing.assert_close(got.cpu().float(), golden.matmul_all_reduce([x1.cpu()], [x2.cpu()]).float(), rtol=1e-2, atol=1e-2)
    tp_group.set_option("solo", "form", 0)
    tp_group.set_option("solo", "wait_limit_ms", 2000)
    for option, value, msg in (("wait_limit_ms", 0, "between 1 and 600000"), ("form", 3, "form must be"), ("tile_width", 48, "tile_width must be"),
                               ("colour", 1, "unknown group option")):
        with pytest.raises(DiopiError, match=msg):
            tp_group.set_option("solo", option, value)


def run_ranks(world, what, extra=(), port=29617):
    """Runs tests/mar_ranks.py as one process per GPU; NVLS is switched off in NCCL, the kernels use plain peer stores."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           str(ROOT / "tests" / "mar_ranks.py"), what, *extra]
    res = subprocess.run(cmd, cwd=ROOT, env=dict(os.environ, NCCL_NVLS_ENABLE="0"), capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    return json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mode", ["1", "2"])
def test_ranks_match_oracle(world, mode):
    """One process per GPU under torchrun: every rank's result equals the oracle's sum over all ranks, and all ranks
    hold identical bits; in the one-shot form (1) and in the two-shot form (2)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    rec = run_ranks(world, "check", extra=["--form", mode])
    assert rec["parity"] == "ok" and rec["world"] == world and rec["ranks_identical"]


def test_a_missing_rank_runs_the_wait_out_and_the_group_recovers():
    """The bounded wait on a peer, made to run out from the host: rank 1 leaves one call out, the other rank's kernel
    gives up after the group's 50 ms limit and returns (the GPU still answers), later calls are refused with status 3 /
    'unusable', and after Destroy + Create on both ranks the group gives the right result again."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    rec = run_ranks(2, "timeout", extra=["--limit-ms", "50"], port=29618)
    assert rec["result"] == "ok" and rec["gpu_alive"] and rec["refused_afterwards"] and rec["recovered_after_recreate"]
    assert rec["gave_up_after_ms"] < 2500


def test_replay_from_a_cuda_graph(F):
    """Nothing the host passes changes from call to call (the sequence number lives in device memory), so a captured
    call can be replayed."""
    from diopi_b200.runtime import Context
    x1, x2 = rand((64, 256), torch.bfloat16, 8).cuda(), rand((256, 384), torch.bfloat16, 9, 1 / 16).cuda()
    want = F.matmul_all_reduce(x1, x2, None, "solo").clone()
    out = torch.zeros_like(want)
    side = torch.cuda.Stream()
    ctx = Context(stream=side)
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        F.matmul_all_reduce(x1, x2, None, "solo", out=out, ctx=ctx)
    for i in range(4):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want), i
    # and plain calls still line up afterwards
    assert torch.equal(F.matmul_all_reduce(x1, x2, None, "solo"), want)
