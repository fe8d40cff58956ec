"""Joining a tensor-parallel group: one process per GPU, handles exchanged by the caller's transport.

The reference is single-device; this is the host logic of the row-split layer stack. `all_gather`
is any callable that takes one picklable object and returns the list of every rank's object in
rank order (for `torch.distributed`: `all_gather_object` over a gloo group, see `torch_all_gather`).
"""
from __future__ import annotations

from typing import Any, Callable


def join(backend, rank: int, world: int, all_gather: Callable[[Any], list], peer_memory: bool = True) -> None:
    """NCCL group for long vectors, peer-memory inboxes for the short ones a decode step sums."""
    if world < 2:
        return
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a group of {world}")
    ids = all_gather(type(backend).comm_unique_id() if rank == 0 else None)
    if len(ids) != world or ids[0] is None:
        raise ValueError("all_gather must return one entry per rank, rank 0 first")
    backend.comm_init(ids[0], world, rank)
    if peer_memory and world <= 8:
        handles = all_gather(backend.comm_peer_handle())
        if len(handles) != world or any(len(h) != 64 for h in handles):
            raise ValueError("all_gather must return one 64-byte handle per rank")
        backend.comm_attach_peers(handles, rank)


def torch_all_gather(group=None) -> Callable[[Any], list]:
    import torch.distributed as dist

    def gather(obj):
        out = [None] * dist.get_world_size(group)
        dist.all_gather_object(out, obj, group=group)
        return out

    return gather
