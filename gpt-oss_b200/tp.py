"""Process-group plumbing of a tensor-parallel group: one process per GPU, launched by torchrun.

The data path never touches torch.distributed: it is the library's own peer-memory kernels.  The
process group only carries the 192 bytes of CUDA IPC handles each rank exports for its three
symmetric buffers (what the reference's single process gets for free by reading
gpu_transformers[peer]->state.*, getp-csrc/getp_run.cpp:2594, :2965, :3221)."""
from __future__ import annotations

import torch
import torch.distributed as dist


def exchange_blobs(blob: bytes, group=None) -> list[bytes]:
    """All-gathers one equal-sized byte string per rank; returns them in rank order."""
    world = dist.get_world_size(group)
    mine = torch.tensor(list(blob), dtype=torch.uint8)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine, group=group)
    return [bytes(p.tolist()) for p in parts]


def attach_group(blk, rank: int, group=None) -> None:
    """Exports this rank's buffers, exchanges the handles and attaches every peer's."""
    blobs = exchange_blobs(blk.tp_export_all(), group)   # in group-rank order
    for r, b in enumerate(blobs):
        if r != rank:
            blk.tp_attach_all(r, b)
    dist.barrier(group)


def tp_groups(world: int, tp_size: int) -> list[list[int]]:
    """Contiguous partition of the ranks into TP groups (tp_init, getp-csrc/nccl.hpp:73-86)."""
    assert world % tp_size == 0
    return [list(range(g * tp_size, (g + 1) * tp_size)) for g in range(world // tp_size)]
