"""Head sharding over two ranks on CPU (gloo): the shard rule, the gathers, and that per-shard results of
the path assemble to the unsharded result. The per-shard compute here is the CPU oracle, standing in for
the per-GPU kernels (which the -m gpu tests check); what is tested is the host-side logic around them."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, heads, results):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from diopi_b200 import head_shard
        from oracle import golden
        g = torch.Generator().manual_seed(7)   # same data on every rank
        B, D, lens = 3, 16, [5, 0, 9]
        slots = sum(lens) + 4
        q = torch.randn(B, heads, D, generator=g)
        k = torch.randn(slots, heads, D, generator=g)
        v = torch.randn(slots, heads, D, generator=g)
        mx = max(lens)
        b_loc = torch.zeros(B, mx, dtype=torch.int32)
        start = torch.zeros(B, dtype=torch.int32)
        perm = torch.randperm(slots, generator=g)
        acc = 0
        for i, L in enumerate(lens):
            b_loc[i, mx - L:] = perm[acc:acc + L].to(torch.int32)
            start[i] = acc
            acc += L
        ln = torch.tensor(lens, dtype=torch.int32)
        full_ref = golden.token_decode_attention(q, k, v, torch.zeros(B, heads, D), b_loc, start, ln, mx)
        qs, ks, vs = (head_shard.shard(t, world, rank) for t in (q, k, v))
        h0, h1 = head_shard.shard_heads(heads, world, rank)
        assert qs.shape[1] == h1 - h0 and ks.is_contiguous()
        local = golden.token_decode_attention(qs, ks, vs, torch.zeros_like(qs), b_loc, start, ln, mx)
        if heads % world == 0:
            full = head_shard.all_gather_heads(local, head_shard.allocate_full(local, world))
        else:
            full = head_shard.all_gather_uneven(local, heads)
        ok = torch.allclose(full, full_ref, rtol=1e-6, atol=1e-6)
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("heads", [8, 5])
def test_head_shard_gather_two_ranks(heads):
    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        port = free_port()
        procs = [ctx.Process(target=worker, args=(r, world, port, heads, results)) for r in range(world)]
        [p.start() for p in procs]
        [p.join(120) for p in procs]
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert dict(results) == {0: True, 1: True}


def test_shard_rule_covers_all_heads():
    from diopi_b200.workloads import shard_heads
    for heads in (1, 5, 32, 64, 7):
        for world in (1, 2, 3, 4, 8):
            ranges = [shard_heads(heads, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == heads
            for a, b in zip(ranges, ranges[1:]):
                assert a[1] == b[0]
            sizes = [b - a for a, b in ranges]
            assert max(sizes) - min(sizes) <= 1


def tp_worker(rank, world, port, results):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from diopi_b200 import tp_group
        from oracle import golden
        # the handle exchange of the matmul + all-reduce group: every rank ends with all handles in rank order
        mine = bytes([rank + 1]) * tp_group.HANDLE_BYTES
        allh = tp_group.exchange(mine)
        ok = allh == b"".join(bytes([r + 1]) * tp_group.HANDLE_BYTES for r in range(world))
        try:
            tp_group.exchange(b"short")
            ok = False
        except ValueError:
            pass
        # the arithmetic of the op across ranks, with the oracle standing in for the kernel: every rank's partial
        # product gathered and added in rank order equals the oracle's result for the whole group
        g = torch.Generator().manual_seed(11)
        x1 = [torch.randn(6, 16, generator=g).to(torch.bfloat16) for _ in range(world)]
        x2 = [torch.randn(16, 24, generator=g).to(torch.bfloat16) for _ in range(world)]
        bias = [torch.randn(24, generator=g).to(torch.bfloat16) for _ in range(world)]
        want = golden.matmul_all_reduce(x1, x2, bias)
        part = x1[rank].float() @ x2[rank].float() + bias[rank].float()
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        total = parts[0].clone()
        for p in parts[1:]:
            total += p
        ok = ok and torch.equal(total.to(torch.bfloat16), want)
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_tp_group_exchange_two_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        port = free_port()
        procs = [ctx.Process(target=tp_worker, args=(r, world, port, results)) for r in range(world)]
        [p.start() for p in procs]
        [p.join(120) for p in procs]
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert dict(results) == {0: True, 1: True}
