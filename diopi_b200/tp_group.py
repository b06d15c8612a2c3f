"""Set-up of a tensor-parallel group for diopiMatmulAllReduce: one process per GPU, handles exchanged through
torch.distributed (any backend; the exchange is 64 bytes per rank and happens once).

    tp_group.create("tp", pg=None, max_tiles=256)   # every rank, after torch.cuda.set_device
    out = functions.matmul_all_reduce(x1, x2, None, "tp")
    tp_group.destroy("tp")

`exchange` is the only part that talks to other ranks; it is separate so that it can be tested on CPU with gloo.
"""
from __future__ import annotations

import ctypes

from . import _lib
from .runtime import check_returncode

HANDLE_BYTES = 64


def exchange(local: bytes, pg=None) -> bytes:
    """All ranks' handles in rank order. `local` is this rank's handle."""
    import torch.distributed as dist
    if len(local) != HANDLE_BYTES:
        raise ValueError(f"a handle has {HANDLE_BYTES} bytes, got {len(local)}")
    world = dist.get_world_size(pg)
    gathered = [None] * world
    dist.all_gather_object(gathered, bytes(local), group=pg)
    for r, h in enumerate(gathered):
        if not isinstance(h, (bytes, bytearray)) or len(h) != HANDLE_BYTES:
            raise RuntimeError(f"rank {r} sent a malformed handle")
    return b"".join(bytes(h) for h in gathered)


def create(name: str, pg=None, max_tiles: int = 256, rank: int | None = None, world: int | None = None, wait_limit_ms: int | None = None) -> None:
    """Creates and connects the group `name` over the ranks of process group `pg` (default: the world group).
    Without torch.distributed (rank and world left None, or world == 1) a group of one rank is made.
    `wait_limit_ms` bounds every wait of a kernel of the group on a peer (2 s when left None)."""
    impl = _lib.load().impl
    if world is None:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            rank, world = dist.get_rank(pg), dist.get_world_size(pg)
        else:
            rank, world = 0, 1
    buf = ctypes.create_string_buffer(HANDLE_BYTES)
    check_returncode("diopiB200GroupCreate", impl.diopiB200GroupCreate(name.encode(), int(rank), int(world), int(max_tiles), buf))
    if wait_limit_ms is not None:
        set_option(name, "wait_limit_ms", wait_limit_ms)
    if world > 1:
        handles = exchange(buf.raw, pg)
        check_returncode("diopiB200GroupConnect", impl.diopiB200GroupConnect(name.encode(), ctypes.c_char_p(handles)))
        import torch.distributed as dist
        dist.barrier(group=pg)   # nobody launches before every rank has mapped every area


def set_option(name: str, option: str, value: int) -> None:
    """wait_limit_ms, form (0 auto, 1 one-shot, 2 two-shot) or tile_width (0 auto, 128, 64, 32) of group `name`;
    form and tile_width must be set alike on every rank."""
    impl = _lib.load().impl
    check_returncode("diopiB200GroupSetOption", impl.diopiB200GroupSetOption(name.encode(), option.encode(), int(value)))


def destroy(name: str) -> None:
    impl = _lib.load().impl
    check_returncode("diopiB200GroupDestroy", impl.diopiB200GroupDestroy(name.encode()))
