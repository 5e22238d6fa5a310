"""FSDP2 with the INT8 weight all-gather on two GPUs (skipped with fewer): every rank holds a row
shard of each Linear weight, `fsdp_pre_all_gather` quantizes the shard row-wise, NCCL gathers int8
rows + bf16 scales, and the forward must equal the unsharded INT8 mixed-precision forward bit for
bit (row-wise quantization commutes with row sharding)."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _build(seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(
        torch.nn.Linear(256, 512, bias=False), torch.nn.GELU(), torch.nn.Linear(512, 384, bias=False)
    ).bfloat16()


def _worker(rank: int, world: int, port: int, out_path: str):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    sys.path[:0] = [str(root), str(root / "quantized-training_b200")]
    import torch.distributed as dist
    from torch.distributed.fsdp import fully_shard

    from subclasses import MixedPrecisionConfig, convert_mixed_precision
    from subclasses.mixed_precision import Int8RowScaledLinearWeight

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        model = _build().cuda()
        convert_mixed_precision(model, config=MixedPrecisionConfig())
        for layer in (model[0], model[2]):
            fully_shard(layer)
        fully_shard(model)
        g = torch.Generator().manual_seed(100)              # same batch on both ranks: grads must agree
        x = torch.randn(64, 256, generator=g).bfloat16().cuda().requires_grad_()
        seen = []
        hook = model[2].register_forward_pre_hook(lambda m, a: seen.append(type(m.weight.data if not hasattr(m.weight, "_local_tensor") else m.weight._local_tensor)))
        y = model(x)
        gathered_types = []
        for layer in (model[0], model[2]):
            state = layer._get_fsdp_state()
            for fp in state._fsdp_param_group.fsdp_params:
                gathered_types.append([t.dtype for t in fp.all_gather_outputs])
        y.float().square().mean().backward()
        hook.remove()
        grads = [p.grad.full_tensor().float().cpu() if hasattr(p.grad, "full_tensor") else p.grad.float().cpu() for p in model.parameters()]
        if rank == 0:
            torch.save({"y": y.detach().float().cpu(), "gx": x.grad.float().cpu(), "grads": grads,
                        "gathered": [[str(d) for d in ds] for ds in gathered_types]}, out_path)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fsdp2_int8_all_gather_matches_unsharded(tmp_path):
    import torch.multiprocessing as mp

    from subclasses import MixedPrecisionConfig, convert_mixed_precision

    out_path = str(tmp_path / "fsdp.pt")
    mp.spawn(_worker, args=(2, _free_port(), out_path), nprocs=2, join=True)
    got = torch.load(out_path)
    # the all-gather moved int8 rows and bf16 scales, not bf16 weights
    assert all(ds == ["torch.int8", "torch.bfloat16"] for ds in got["gathered"]), got["gathered"]

    model = _build().cuda()
    convert_mixed_precision(model, config=MixedPrecisionConfig())
    g = torch.Generator().manual_seed(100)
    x = torch.randn(64, 256, generator=g).bfloat16().cuda().requires_grad_()
    y = model(x)
    y.float().square().mean().backward()
    assert torch.equal(y.detach().float().cpu(), got["y"])                     # forward: bit-exact
    ref_grads = [p.grad.float().cpu() for p in model.parameters()]
    for a, b in zip(got["grads"], ref_grads):                                   # grad_weight: same INT8 matmul
        assert (a - b).norm() / b.norm() < 2e-2
    # grad_input uses the gathered int8 weight (scale folded into dY): within quantization error
    assert (got["gx"] - x.grad.float().cpu()).norm() / x.grad.float().norm().cpu() < 3e-2
