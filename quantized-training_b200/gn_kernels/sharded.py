"""The one exchange step of the path: all-gather of a row-sharded, row-wise quantized weight.

A weight [N, K] sharded over ranks by rows (what FSDP2's dim-0 sharding gives) is quantized per row
on each rank, so the gathered int8 rows and scales are bit-identical to quantizing the whole weight
on one device; only int8 + one scale per row cross the link. Two forms: `all_gather_quantized_rows`
hands already quantized shards to the process group's all-gather (NCCL on GPUs, gloo in the CPU tests),
and `SymmetricRowGather` runs quantize and gather as ONE kernel whose stores go straight into every
rank's gathered buffer over NVLink (peer-to-peer stores into a symmetric allocation).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist
from torch import Tensor

from . import _native as nv


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


class SymmetricRowGather:
    """Quantize + all-gather of a row-sharded bf16 weight in one kernel.

    Every rank allocates the same gathered buffers (int8 [total_rows, cols] and scales [total_rows, 1],
    `buffers` of each for double buffering) in symmetric memory, exchanges their addresses once, and
    `quantize_scatter` then runs the row-wise quantize kernel with every rank's buffer as a destination:
    the shard's int8 rows and scales leave the SM as peer-to-peer stores, no collective kernel runs and
    no SM is set aside for one. `fence` is the barrier that orders the readers after every rank's
    kernel: a 4-byte all-reduce on the calling stream (stream order puts it after this rank's kernel, and
    it cannot complete before every rank has reached it). Needs even shards (total_rows % world == 0).
    """

    def __init__(self, total_rows: int, cols: int, group=None, *, device: torch.device, out_dtype=torch.int8,
                 scale_dtype=torch.bfloat16, buffers: int = 2):
        import torch.distributed._symmetric_memory as symm

        # the buffers are only written with plain stores: keep them off NVLink multicast objects
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if total_rows % self.world:
            raise ValueError("SymmetricRowGather needs the rows to split evenly over the ranks")
        if self.world > 16:
            raise ValueError("SymmetricRowGather serves at most 16 ranks (one NVLink domain)")
        self.total_rows, self.cols, self.shard_rows = total_rows, cols, total_rows // self.world
        self.device = device
        self.q, self.scale, self._q_ptrs, self._s_ptrs = [], [], [], []
        ptr_array = ctypes.c_void_p * self.world
        for _ in range(buffers):
            q = symm.empty((total_rows, cols), dtype=out_dtype, device=device)
            s = symm.empty((total_rows, 1), dtype=scale_dtype, device=device)
            hq, hs = symm.rendezvous(q, self.group), symm.rendezvous(s, self.group)
            self.q.append(q)
            self.scale.append(s)
            self._q_ptrs.append(ptr_array(*[int(p) for p in hq.buffer_ptrs]))
            self._s_ptrs.append(ptr_array(*[int(p) for p in hs.buffer_ptrs]))
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)

    def quantize_scatter(self, w_shard: Tensor, buffer: int = 0, *, eps: float = 1e-12) -> None:
        """Quantize this rank's rows [shard_rows, cols] into buffer `buffer` of every rank (current stream)."""
        if w_shard.shape != (self.shard_rows, self.cols) or w_shard.dtype is not torch.bfloat16 or w_shard.stride(1) != 1:
            raise ValueError("quantize_scatter: expected this rank's bf16 shard [shard_rows, cols] with unit inner stride")
        dev = nv.require_cuda(w_shard)
        with nv.on_device(dev):
            nv.check(nv.load().qt_quantize_rowwise_scatter(
                w_shard.data_ptr(), nv.code(w_shard.dtype), self.shard_rows, self.cols, w_shard.stride(0), self.world,
                self._q_ptrs[buffer], self._s_ptrs[buffer], self.rank * self.shard_rows, nv.code(self.q[buffer].dtype),
                nv.code(self.scale[buffer].dtype), float(eps), nv.stream_ptr(dev)))

    def fence(self) -> None:
        """Every rank's scatter issued before this call has landed once this returns control to the stream."""
        dist.all_reduce(self._flag, group=self.group)
