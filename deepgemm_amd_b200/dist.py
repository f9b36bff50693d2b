"""Multi-GPU partitioning of the GEMM path: one process per GPU, no collective inside the GEMM.

Dense GEMMs are split column-parallel along N (every rank holds all of A and a slice of B / SFB and
writes its slice of D's columns); grouped GEMMs are split expert-parallel (every rank holds a contiguous
range of experts with their row segments).  NCCL is used only to gather outputs for verification,
as in the reference's helper deep_gemm/utils/dist.py:10-66.
"""
from __future__ import annotations

import os
from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def init_dist(backend: str | None = None) -> Tuple[int, int, int]:
    """Join the process group described by RANK / WORLD_SIZE / MASTER_* (torchrun); returns
    (rank, world_size, local_rank).  A single process without those variables is world size 1."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return rank, world, local_rank


def shard_columns(n: int, world: int, rank: int, multiple: int = 128) -> Tuple[int, int]:
    """[begin, end) of the N slice of `rank`: blocks of `multiple` columns dealt out evenly, the ragged
    last block going to the last rank that owns any."""
    blocks = -(-n // multiple)
    per, extra = divmod(blocks, world)
    first = rank * per + min(rank, extra)
    count = per + (1 if rank < extra else 0)
    return min(first * multiple, n), min((first + count) * multiple, n)


def shard_experts(num_experts: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of the experts owned by `rank` (contiguous ranges, sizes differing by at most one)."""
    per, extra = divmod(num_experts, world)
    first = rank * per + min(rank, extra)
    return first, first + per + (1 if rank < extra else 0)


def expert_rows(aligned_ms: Sequence[int], begin: int, end: int) -> Tuple[int, int]:
    """Row range of experts [begin, end) in the m-grouped contiguous layout."""
    start = sum(aligned_ms[:begin])
    return start, start + sum(aligned_ms[begin:end])


def uneven_all_gather(t: torch.Tensor, dim: int = 0) -> torch.Tensor:
    """all_gather of tensors whose size differs along `dim` (two collectives: sizes, then padded data)."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return t
    world = dist.get_world_size()
    t = t.movedim(dim, 0).contiguous()
    size = torch.tensor([t.size(0)], dtype=torch.int64, device=t.device)
    sizes: List[torch.Tensor] = [torch.zeros_like(size) for _ in range(world)]
    dist.all_gather(sizes, size)
    counts = [int(s.item()) for s in sizes]
    padded = torch.zeros((max(counts),) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    padded[: t.size(0)] = t
    if t.dtype in (torch.float8_e4m3fn,):
        padded = padded.view(torch.uint8)
    bufs = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(bufs, padded)
    out = torch.cat([b[:c] for b, c in zip(bufs, counts)], dim=0)
    if t.dtype in (torch.float8_e4m3fn,):
        out = out.view(t.dtype)
    return out.movedim(0, dim)
