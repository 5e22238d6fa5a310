"""world_size-2 CPU test (gloo) of the path's only exchange step: each rank quantizes its own row
shard of a weight (here with the CPU oracle standing in for the kernel), the shards are gathered,
and the result must equal quantizing the whole weight in one place -- bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import reference_math as om


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, n_rows: int, k: int, fail_rank: int):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    sys.path[:0] = [str(root), str(root / "quantized-training_b200")]
    from gn_kernels.sharded import all_gather_quantized_rows, shard_rows

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(2024)  # same full weight everywhere; each rank looks at its rows only
        w = (torch.randn(n_rows, k) * 0.02).bfloat16()
        lo, hi = shard_rows(n_rows, rank, world)
        q, s = om.quantize_rowwise(w[lo:hi].float().numpy())
        q_t = torch.from_numpy(q)
        s_t = torch.from_numpy(om.f32_to_bf16_bits(s).view(np.int16).copy()).view(torch.bfloat16).reshape(-1, 1)
        q_all, s_all = all_gather_quantized_rows(q_t, s_t, total_rows=n_rows)
        q_ref, s_ref = om.quantize_rowwise(w.float().numpy())
        assert q_all.shape == (n_rows, k) and s_all.shape == (n_rows, 1)
        assert np.array_equal(q_all.numpy(), q_ref)
        assert np.array_equal(s_all.float().numpy(), s_ref)
        # the variant that discovers the row counts with a collective agrees
        q2, s2 = all_gather_quantized_rows(q_t, s_t)
        assert torch.equal(q2, q_all) and torch.equal(s2, s_all)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_rows,k", [(64, 48), (37, 16), (3, 8)])
def test_row_sharded_quantize_then_gather_equals_unsharded(n_rows, k):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), n_rows, k, -1), nprocs=world, join=True)


def test_shard_rows_follows_chunk_rule():
    import sys
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "quantized-training_b200"))
    from gn_kernels.sharded import shard_rows

    for n, world in [(10, 4), (256, 8), (3, 8), (0, 2), (33, 2)]:
        chunks = torch.arange(n).chunk(world) if n else []
        for r in range(world):
            lo, hi = shard_rows(n, r, world)
            want = chunks[r].tolist() if r < len(chunks) else []
            assert list(range(lo, hi)) == want
