"""Row sharding of GGUF tensors across the GPUs of one machine.

The reference has no multi-GPU path.  Tensors are independent, and inside a
tensor of shape ``(rows, K)`` every row is its own contiguous run of
``K/32 * block_bytes`` packed bytes, so rank ``r`` of ``W`` decodes rows
``[r*rows/W, (r+1)*rows/W)`` from its own pinned staging buffer with no
data-path exchange.  Only a replicated layout needs a collective: an in-place
all-gather of the decoded rows (NCCL over NVLink on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

from typing import Dict, Iterable, Optional, Tuple

import torch

from .gguf_loader import QUANT_INFO, GGUFTensorInfo


def row_range(rows: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Half-open row interval owned by ``rank``; intervals tile ``[0, rows)``."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError(f"bad shard ({rank}, {world_size})")
    return rows * rank // world_size, rows * (rank + 1) // world_size


def shard_extent(info: GGUFTensorInfo, rank: int, world_size: int) -> Tuple[int, int, int, Optional[Tuple[int, int]]]:
    """(byte offset inside the tensor, byte count, element count, rows) of a rank's share.

    Tensors with fewer than two axes are replicated: every rank takes all of them.
    """
    shape = info.shape
    per_block, block_bytes = QUANT_INFO[info.dtype]
    if len(shape) < 2:
        return 0, info.nbytes, info.numel, None
    r0, r1 = row_range(shape[0], rank, world_size)
    row_elems = info.numel // shape[0]
    if row_elems % per_block:
        raise ValueError(f"{info.name}: row length {row_elems} does not cover whole {per_block}-element blocks")
    row_bytes = row_elems // per_block * block_bytes
    return r0 * row_bytes, (r1 - r0) * row_bytes, (r1 - r0) * row_elems, (r0, r1)


def plan(tensors: Dict[str, GGUFTensorInfo], rank: int, world_size: int) -> Dict[str, Tuple[int, int, int, Optional[Tuple[int, int]]]]:
    """Per-tensor share of one rank, in file order."""
    return {name: shard_extent(info, rank, world_size) for name, info in tensors.items()}


def plan_bytes(tensors: Iterable[GGUFTensorInfo], rank: int, world_size: int) -> Tuple[int, int]:
    """(packed bytes, elements) one rank reads for the whole file."""
    b = e = 0
    for info in tensors:
        _, nb, ne, _ = shard_extent(info, rank, world_size)
        b += nb
        e += ne
    return b, e


def all_gather_rows(full: torch.Tensor, group=None, async_op: bool = False) -> list:
    """Completes a replicated tensor in place.

    Every rank has already written its own ``row_range`` slice of ``full``;
    afterwards every rank holds all rows.  Equal shares use one
    ``all_gather_into_tensor`` (on CUDA the rank's own slice is the send buffer:
    NCCL's in-place form, no staging copy); ragged shares fall back to per-rank
    broadcasts.  With ``async_op`` the collectives are only enqueued (behind the
    work already on the current stream) and their handles are returned; the
    caller waits on them before the tensor is used.
    """
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    rows = full.shape[0]
    if world == 1:
        return []
    works = []
    if rows % world == 0:
        r0, r1 = row_range(rows, rank, world)
        mine = full[r0:r1] if full.is_cuda else full[r0:r1].clone()
        works.append(dist.all_gather_into_tensor(full, mine, group=group, async_op=async_op))
    else:
        for src in range(world):
            r0, r1 = row_range(rows, src, world)
            if r1 > r0:
                works.append(dist.broadcast(full[r0:r1], src=dist.get_global_rank(group, src) if group is not None else src,
                                            group=group, async_op=async_op))
    return [w for w in works if w is not None] if async_op else []
