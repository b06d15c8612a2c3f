"""Head sharding of the decode/prefill ops over the GPUs of one box.

The ops need no exchange: each rank holds q[:, h0:h1], the K/V pool shard [slots, h0:h1, D] and the
(replicated, tiny) index tensors, and produces out[:, h0:h1]. The only collective is optional: an
all-gather of the per-head outputs for a caller that wants the full [B, H, D] tensor on every rank.
Works over any torch.distributed backend (nccl on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .workloads import shard_heads  # noqa: F401  (re-exported: the split rule lives with the workloads)


def shard(t: torch.Tensor, world: int, rank: int, dim: int = 1) -> torch.Tensor:
    """The contiguous head shard of `rank` (a copy, so that rows stay dense for the bulk-copy path)."""
    h0, h1 = shard_heads(t.shape[dim], world, rank)
    return t.narrow(dim, h0, h1 - h0).contiguous()


def allocate_full(local_out: torch.Tensor, world: int) -> torch.Tensor:
    """Full-size output buffer for equal shards: [B, Hs * world, D]."""
    B, Hs, D = local_out.shape
    return torch.empty(B, Hs * world, D, dtype=local_out.dtype, device=local_out.device)


_staging: dict = {}


def all_gather_heads(local_out: torch.Tensor, full: torch.Tensor, group=None) -> torch.Tensor:
    """Gathers equal head shards [B, Hs, D] of all ranks into full [B, Hs*world, D] on every rank.

    One all_gather_into_tensor into a [world, B, Hs, D] staging buffer (kept per shape), then one strided
    copy into the head-major layout. The payload is small (256 KB per rank at B128 x 8 heads x 128 x fp16),
    so the cost is launch latency, not bandwidth."""
    world = dist.get_world_size(group)
    B, Hs, D = local_out.shape
    assert full.shape == (B, Hs * world, D), (tuple(full.shape), (B, Hs * world, D))
    key = (tuple(local_out.shape), local_out.dtype, local_out.device, world)
    st = _staging.get(key)
    if st is None:
        st = _staging[key] = torch.empty(world, B, Hs, D, dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(st.view(-1), local_out.contiguous().view(-1), group=group)
    full.view(B, world, Hs, D).copy_(st.permute(1, 0, 2, 3))
    return full


def all_gather_uneven(local_out: torch.Tensor, heads_total: int, group=None) -> torch.Tensor:
    """Gather for head counts that do not divide evenly: one broadcast-free all_gather of padded shards."""
    world = dist.get_world_size(group)
    B, Hs, D = local_out.shape
    widest = -(-heads_total // world)
    padded = torch.zeros(B, widest, D, dtype=local_out.dtype, device=local_out.device)
    padded[:, :Hs] = local_out
    st = torch.empty(world, B, widest, D, dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(st.view(-1), padded.view(-1), group=group)
    parts = []
    for r in range(world):
        h0, h1 = shard_heads(heads_total, world, r)
        parts.append(st[r, :, : h1 - h0])
    return torch.cat(parts, dim=1)
