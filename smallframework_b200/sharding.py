"""Sharding of an inference batch over the GPUs of one node.

Images are independent, so the path has no exchange step: every rank (one process per GPU)
owns a contiguous range of images, runs its own layer chain on them and the results meet
again only on the host ("final host gather").  The only collectives are the ones the
measurement needs: a barrier and a max-reduce of the per-rank time.  They work on any
torch.distributed backend (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(total_images: int, world_size: int, rank: int):
    """Contiguous [begin, end) of `total_images` owned by `rank`; the first
    total % world ranks get one image more."""
    if not (0 <= rank < world_size):
        raise ValueError("rank out of range")
    base, extra = divmod(total_images, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def max_over_ranks(value: float, device="cpu") -> float:
    """The slowest rank's time: the job is done when the last shard is done."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_to_host(local: torch.Tensor, total_images: int, dst: int = 0):
    """Final host gather: every rank sends its [images, features] tensor to `dst`, which returns
    them stacked in image order on the host (others return None).  The tensors travel as they are:
    device tensors over NCCL, host tensors over gloo."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local.cpu()
    world, rank = dist.get_world_size(), dist.get_rank()
    sizes = [shard_range(total_images, world, r) for r in range(world)]
    if rank == dst:
        parts = [torch.empty((e - b,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
                 for b, e in sizes]
        parts[dst] = local
        reqs = [dist.irecv(parts[r], src=r) for r in range(world) if r != dst]
        for q in reqs:
            q.wait()
        return torch.cat([p.cpu() for p in parts], dim=0)
    dist.send(local.contiguous(), dst=dst)
    return None
