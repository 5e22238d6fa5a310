"""FSDP2 with the INT8 weight all-gather, on one GPU (a process group of one rank: the hooks, the gather
buffers and the backward re-gather all run) and on two (skipped with fewer): every rank holds a row
shard of each Linear weight, `fsdp_pre_all_gather` quantizes the shard, NCCL gathers int8 rows + bf16
scales, and forward, grad-input and grad-weight must equal the unsharded INT8 mixed-precision layer bit
for bit (row-wise quantization commutes with row sharding; the backward gather quantizes along the
output dimension with column maxima agreed by an all-reduce(MAX))."""
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


def _worker(rank: int, world: int, port: int, out_path: str, mode: str = "int8_mp", variant: str = ""):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    sys.path[:0] = [str(root), str(root / "quantized-training_b200")]
    import torch.distributed as dist
    from torch.distributed.fsdp import fully_shard

    from subclasses import MixedPrecisionConfig, MixedPrecisionLinearWeight, convert_bitnet, convert_mixed_precision

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        model = _build().cuda()
        kwargs = {}
        if mode == "bitnet":
            convert_bitnet(model)
        else:
            convert_mixed_precision(model, config=MixedPrecisionConfig(grad_input=variant != "bf16_grad_input"))
            MixedPrecisionLinearWeight.backward_gather = "row" if variant == "row_backward" else "col"
            if variant == "fp32_reduce":
                from torch.distributed.fsdp import MixedPrecisionPolicy

                kwargs["mp_policy"] = MixedPrecisionPolicy(reduce_dtype=torch.float32)
        for layer in (model[0], model[2]):
            fully_shard(layer, **kwargs)
        fully_shard(model, **kwargs)
        g = torch.Generator().manual_seed(100)              # same batch on both ranks: grads must agree
        x = torch.randn(64, 256, generator=g).bfloat16().cuda().requires_grad_()
        y = model(x)
        gathered_types = []
        for layer in (model[0], model[2]):
            state = layer._get_fsdp_state()
            for fp in state._fsdp_param_group.fsdp_params:
                gathered_types.append([t.dtype for t in fp.all_gather_outputs])
        gathered_shapes = [[tuple(t.shape) for t in fp.all_gather_outputs]
                           for layer in (model[0], model[2]) for fp in layer._get_fsdp_state()._fsdp_param_group.fsdp_params]
        y.float().square().mean().backward()
        grads = [p.grad.full_tensor().float().cpu() if hasattr(p.grad, "full_tensor") else p.grad.float().cpu() for p in model.parameters()]
        if rank == 0:
            torch.save({"y": y.detach().float().cpu(), "gx": x.grad.float().cpu(), "grads": grads,
                        "gathered": [[str(d) for d in ds] for ds in gathered_types], "gathered_shapes": gathered_shapes}, out_path)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _unsharded(grad_input=True):
    from subclasses import MixedPrecisionConfig, convert_mixed_precision

    model = _build().cuda()
    convert_mixed_precision(model, config=MixedPrecisionConfig(grad_input=grad_input))
    g = torch.Generator().manual_seed(100)
    x = torch.randn(64, 256, generator=g).bfloat16().cuda().requires_grad_()
    y = model(x)
    y.float().square().mean().backward()
    return y.detach().float().cpu(), x.grad.float().cpu(), [p.grad.float().cpu() for p in model.parameters()]


@pytest.mark.parametrize("world", [1, 2])
def test_fsdp2_int8_all_gather_matches_unsharded(tmp_path, world):
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip("needs two GPUs")
    out_path = str(tmp_path / "fsdp.pt")
    mp.spawn(_worker, args=(world, _free_port(), out_path), nprocs=world, join=True)
    got = torch.load(out_path)
    if world > 1:   # the all-gather moved int8 rows and bf16 scales, not bf16 weights
        assert all(ds == ["torch.int8", "torch.bfloat16"] for ds in got["gathered"]), got["gathered"]
    else:           # one rank: nothing crosses a link, the hook hands FSDP2 the bf16 shard
        assert all(ds == ["torch.bfloat16"] for ds in got["gathered"]), got["gathered"]
    y, gx, grads = _unsharded()
    assert torch.equal(got["y"], y)                       # forward: the gathered rows are the unsharded quantization
    assert torch.equal(got["gx"], gx)                     # grad_input: same for the column-wise backward gather
    for a, b in zip(got["grads"], grads):                 # grad_weight: the same INT8 product on every rank
        assert torch.equal(a, b)


@pytest.mark.parametrize("variant", ["row_backward", "bf16_grad_input", "fp32_reduce"])
def test_fsdp2_int8_all_gather_variants(tmp_path, variant):
    """Two ranks when the box has them, else one. row_backward: the forward's row-wise quantization also serves backward,
    its row scales folded into dY (within quantization error of the reference's product). bf16_grad_input:
    a config that keeps grad-input in bf16 gathers the bf16 weight, so every product is the unsharded one.
    fp32_reduce: gradients are reduce-scattered in fp32 (torch's MixedPrecisionPolicy) with the INT8 gather."""
    import torch.multiprocessing as mp

    world = 2 if torch.cuda.device_count() >= 2 else 1   # with one rank the gather is bf16 and all variants are exact
    out_path = str(tmp_path / "fsdp.pt")
    mp.spawn(_worker, args=(world, _free_port(), out_path, "int8_mp", variant), nprocs=world, join=True)
    got = torch.load(out_path)
    y, gx, grads = _unsharded(grad_input=variant != "bf16_grad_input")
    assert torch.equal(got["y"], y)
    if variant == "bf16_grad_input" or world == 1:
        assert all(ds == ["torch.bfloat16"] for ds in got["gathered"]), got["gathered"]
    folded = variant == "row_backward" and world > 1
    if folded:
        assert (got["gx"] - gx).norm() / gx.norm() < 3e-2
    else:
        assert torch.equal(got["gx"], gx)
    for a, b in zip(got["grads"], grads):
        assert (a - b).norm() / b.norm() < (3e-2 if folded else 1e-6)


@pytest.mark.parametrize("world", [1, 2])
def test_fsdp2_bitnet_2bit_all_gather_matches_unsharded(tmp_path, world):
    """BitNet weights cross NVLink as packed 2-bit ternaries (4 per byte); the tensor-wide abs-mean is
    the average of the two equal-size shards' abs-means, equal to the unsharded one up to fp32 rounding,
    so the forward agrees within a few weights flipping between ternary levels."""
    import torch.multiprocessing as mp

    from subclasses import convert_bitnet

    if torch.cuda.device_count() < world:
        pytest.skip("needs two GPUs")
    out_path = str(tmp_path / "fsdp_bitnet.pt")
    mp.spawn(_worker, args=(world, _free_port(), out_path, "bitnet"), nprocs=world, join=True)
    got = torch.load(out_path)
    assert all(ds == ["torch.int8"] for ds in got["gathered"]), got["gathered"]
    # 512x256 and 384x512 weights, four ternaries per byte
    assert sorted(int(torch.tensor(s[0]).prod()) for s in got["gathered_shapes"]) == sorted([512 * 256 // 4, 384 * 512 // 4])

    model = _build().cuda()
    convert_bitnet(model)
    g = torch.Generator().manual_seed(100)
    x = torch.randn(64, 256, generator=g).bfloat16().cuda().requires_grad_()
    y = model(x)
    y.float().square().mean().backward()
    yr = y.detach().float().cpu()
    assert (got["y"] - yr).norm() / yr.norm() < 2e-2
    for a, p in zip(got["grads"], model.parameters()):
        b = p.grad.float().cpu()
        assert (a - b).norm() / b.norm() < 3e-2
    gx = x.grad.float().cpu()
    assert (got["gx"] - gx).norm() / gx.norm() < 3e-2


def _gather_worker(rank: int, world: int, port: int, out_path: str):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    sys.path[:0] = [str(root), str(root / "quantized-training_b200")]
    import torch.distributed as dist

    import gn_kernels
    from gn_kernels.sharded import SymmetricRowGather, all_gather_quantized_rows

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        rows, cols = 1024, 1536
        g = torch.Generator().manual_seed(7)
        w = (torch.randn(rows, cols, generator=g) * 0.02).bfloat16().to(dev)
        shard = w[rank * rows // world:(rank + 1) * rows // world]
        q_local, s_local = gn_kernels.quantize_rowwise(shard)
        q_nccl, s_nccl = all_gather_quantized_rows(q_local, s_local, total_rows=rows)
        gather = SymmetricRowGather(rows, cols, device=dev)
        ok = True
        for b in (0, 1, 0):                       # both buffers, and a buffer reused
            gather.q[b].fill_(99)
            dist.barrier()                        # nobody's fill may overwrite a peer's rows
            gather.quantize_scatter(shard, b)
            gather.fence()
            ok = ok and torch.equal(gather.q[b], q_nccl) and torch.equal(gather.scale[b], s_nccl)
        q_full, s_full = gn_kernels.quantize_rowwise(w)
        ok = ok and torch.equal(q_nccl, q_full) and torch.equal(s_nccl, s_full)
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            torch.save({"ok": bool(flag.item())}, out_path)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2])
def test_fused_quantize_scatter_equals_quantize_then_all_gather(tmp_path, world):
    """One kernel that quantizes this rank's weight rows and stores them into every rank's gathered buffer
    (peer-to-peer stores into symmetric memory) against quantize + NCCL all-gather: bit-identical, and
    identical to quantizing the whole weight on one GPU."""
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip("needs two GPUs")
    out_path = str(tmp_path / "gather.pt")
    mp.spawn(_gather_worker, args=(world, _free_port(), out_path), nprocs=world, join=True)
    assert torch.load(out_path)["ok"]
