"""Process-per-GPU plumbing for multi-GPU runs: rank discovery from the launcher's environment,
batch sharding, reductions of host scalars over ranks and distribution of the tensor-parallel id.
torch.distributed is used for rendezvous and host-side reductions only (gloo on CPU, nccl on GPU);
no tensor of the forward path goes through it.
"""
from __future__ import annotations

import os
from typing import Tuple


def env_ranks() -> Tuple[int, int, int]:
    """(rank, world_size, local_rank) from RANK / WORLD_SIZE / LOCAL_RANK (1 process when absent)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous split of `total` independent units (sequences) over ranks: (start, count).
    The first total % world ranks get one extra unit; ranks beyond `total` get none."""
    if world <= 0 or rank < 0 or rank >= world or total < 0:
        raise ValueError("shard_range: bad rank / world / total")
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def init_process_group(backend: str):
    import torch.distributed as dist
    rank, world, _ = env_ranks()
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return rank, world


def _reduce(value: float, op_name: str, device=None) -> float:
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=getattr(dist.ReduceOp, op_name))
    return float(t.item())


def max_over_ranks(value: float, device=None) -> float:
    return _reduce(value, "MAX", device)


def sum_over_ranks(value: float, device=None) -> float:
    return _reduce(value, "SUM", device)


def barrier():
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def broadcast_bytes(payload: bytes, nbytes: int, src: int = 0, device=None) -> bytes:
    """Rank `src` sends `payload` (nbytes long) to every rank; used for the 128-byte communicator id."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return payload
    if dist.get_rank() == src:
        t = torch.tensor(list(payload), dtype=torch.uint8, device=device or "cpu")
    else:
        t = torch.zeros(nbytes, dtype=torch.uint8, device=device or "cpu")
    dist.broadcast(t, src=src)
    return bytes(t.cpu().tolist())
