"""The one exchange step of the path: all-gather of a row-sharded, row-wise quantized weight.

A weight [N, K] sharded over ranks by rows (what FSDP2's dim-0 sharding gives) is quantized per row
on each rank, so the gathered int8 rows and scales are bit-identical to quantizing the whole weight
on one device; only int8 + one scale per row cross the link. The collective is NCCL on GPUs (gloo
in the CPU tests); nothing here touches device code.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor


def shard_rows(n_rows: int, rank: int, world: int) -> tuple[int, int]:
    """[start, stop) of the rows owned by `rank` when `n_rows` are split evenly (ceil-sized chunks,
    trailing ranks may own fewer or none) -- torch.chunk's rule, which FSDP2 follows."""
    chunk = -(-n_rows // world)
    start = min(rank * chunk, n_rows)
    return start, min(start + chunk, n_rows)


def all_gather_quantized_rows(q_local: Tensor, scale_local: Tensor, group=None, *, total_rows: int | None = None):
    """Gather (int8 [n_r, K], scale [n_r, 1]) from every rank into ([N, K], [N, 1]).

    Ranks may own different numbers of rows (the last chunks of an uneven split); shards are padded
    to the largest one for the collective and the padding is dropped afterwards."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return q_local, scale_local
    k = q_local.shape[1]
    rows = torch.tensor([q_local.shape[0]], dtype=torch.int64, device=q_local.device)
    all_rows = [torch.zeros_like(rows) for _ in range(world)]
    if total_rows is None:
        dist.all_gather(all_rows, rows, group=group)
        counts = [int(r.item()) for r in all_rows]
    else:
        counts = [shard_rows(total_rows, r, world)[1] - shard_rows(total_rows, r, world)[0] for r in range(world)]
    biggest = max(counts)
    if q_local.shape[0] != biggest:
        q_pad = q_local.new_zeros((biggest, k))
        q_pad[: q_local.shape[0]] = q_local
        s_pad = scale_local.new_zeros((biggest, 1))
        s_pad[: scale_local.shape[0]] = scale_local
        q_local, scale_local = q_pad, s_pad
    q_all = q_local.new_empty((world * biggest, k))
    s_all = scale_local.new_empty((world * biggest, 1))
    dist.all_gather_into_tensor(q_all, q_local.contiguous(), group=group)
    dist.all_gather_into_tensor(s_all, scale_local.contiguous(), group=group)
    if all(c == biggest for c in counts):
        return q_all, s_all
    keep = torch.cat([torch.arange(r * biggest, r * biggest + c, device=q_all.device) for r, c in enumerate(counts)])
    return q_all.index_select(0, keep), s_all.index_select(0, keep)
