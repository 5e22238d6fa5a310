"""AdamWBF16SR: AdamW with bf16 states, fp32 math and stochastically rounded bf16 weights.

Same constructor, state layout (`step`, `exp_avg`, `exp_avg_sq`) and `lr`-as-tensor convention as the
reference optimizer (other_optim/bf16_sr.py:6-75); the update is a fused sm_100a kernel that covers
many parameter tensors per launch (qt_adamw_bf16_sr_multi) instead of one torch.compile'd Python
function per parameter, and the 16 random bits come from Philox inside the kernel instead of a
materialised int32 `random_()` tensor.
"""
from __future__ import annotations

import torch
from torch import Tensor
from torch.optim.optimizer import Optimizer, ParamsT

from gn_kernels import _native as nv
import ctypes

from gn_kernels.quantize import next_philox_key, reserve_philox_keys


class AdamWBF16SR(Optimizer):
    def __init__(
        self,
        params: ParamsT,
        lr: float = 1e-3,
        betas: tuple[float, float] = (0.9, 0.999),
        eps: float = 1e-8,
        weight_decay: float = 1e-2,
    ) -> None:
        defaults = dict(lr=torch.as_tensor(lr), betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()

        for group in self.param_groups:
            lr = group["lr"]
            if not isinstance(lr, Tensor):
                raise RuntimeError(
                    "lr was changed to a non-Tensor object. If you want to update lr, please use "
                    "optim.param_groups[0]['lr'].fill_(new_lr)"
                )
            beta1, beta2 = group["betas"]
            # parameters that share step count, device and dtypes go to the kernel together
            buckets: dict[tuple, list[tuple[Tensor, Tensor, Tensor, Tensor]]] = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if len(state) == 0:
                    state["step"] = torch.tensor(0.0)
                    state["exp_avg"] = torch.zeros_like(p, dtype=torch.bfloat16)
                    state["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.bfloat16)
                state["step"] += 1
                item = tuple(_local(t) for t in (p, p.grad, state["exp_avg"], state["exp_avg_sq"]))
                k = (float(state["step"]), item[0].device, item[0].dtype, item[1].dtype)
                buckets.setdefault(k, []).append(item)
            for (step, _, p_dtype, _), items in buckets.items():
                adamw_multi([i[0] for i in items], [i[1] for i in items], step, [i[2] for i in items],
                            [i[3] for i in items], lr, beta1, beta2, group["weight_decay"], group["eps"],
                            p_dtype is torch.bfloat16)
        return loss


_bc_cache: dict[tuple[float, float, float], tuple[float, float]] = {}


def _bias_corrections(step: float, beta1: float, beta2: float) -> tuple[float, float]:
    """(1 - beta1^step, sqrt(1 - beta2^step)) formed exactly as the reference does -- fp32 tensor
    arithmetic on the host (bf16_sr.py:91-92,102) -- and remembered per step value, since every
    parameter of a step shares them."""
    k = (step, beta1, beta2)
    hit = _bc_cache.get(k)
    if hit is None:
        if len(_bc_cache) > 64:
            _bc_cache.clear()
        step32 = torch.tensor(step, dtype=torch.float32)
        bc1 = 1 - beta1**step32
        bc2 = 1 - beta2**step32
        hit = (float(bc1), float(bc2.sqrt()))
        _bc_cache[k] = hit
    return hit


def _local(t: Tensor) -> Tensor:
    """The local shard of a DTensor (FSDP2 parameters), or the tensor itself."""
    to_local = getattr(t, "to_local", None)
    t = to_local() if callable(to_local) else t
    inner = getattr(t, "_data", None)  # wrapper subclasses over a plain bf16 tensor
    if isinstance(inner, Tensor):
        return inner
    if type(t) is not Tensor and type(t) is not torch.nn.Parameter and t.data_ptr() == 0:
        # e.g. an INT8 weight-only parameter (subclasses.Int8LinearWeight): its storage is int8 + scales, which
        # this kernel cannot update. The reference's AdamWBF16SR reaches such parameters through their own
        # in-place ops; here they take a stock optimizer, whose add_/addcdiv_ land in the fused INT8 update.
        raise TypeError(
            f"AdamWBF16SR cannot update a {type(t).__name__} parameter: it has no bf16 storage. Use torch.optim.AdamW "
            "(or another stock optimizer) for INT8 weight-only models; its in-place updates run the fused "
            "de-quantize / update / stochastic re-quantize kernel.")
    return t


def adamw(p: Tensor, grad: Tensor, step: Tensor, exp_avg: Tensor, exp_avg_sq: Tensor, lr: Tensor, beta1: float,
          beta2: float, weight_decay: float, eps: float, bf16_sr: bool, *, key: tuple[int, int] | None = None) -> None:
    """One in-place AdamW step on (p, exp_avg, exp_avg_sq); same arguments as the reference's
    `adamw` (other_optim/bf16_sr.py:78-90). `key` = (seed, offset) pins the random bits."""
    p, grad, exp_avg, exp_avg_sq = (_local(t) for t in (p, grad, exp_avg, exp_avg_sq))
    dev = nv.require_cuda(p, grad, exp_avg, exp_avg_sq)
    if not (p.is_contiguous() and grad.is_contiguous() and exp_avg.is_contiguous() and exp_avg_sq.is_contiguous()):
        raise ValueError("adamw: tensors must be contiguous")
    if exp_avg.dtype is not torch.bfloat16 or exp_avg_sq.dtype is not torch.bfloat16:
        raise TypeError("adamw: optimizer states are bfloat16")
    bc1, sqrt_bc2 = _bias_corrections(float(step), beta1, beta2)
    lr32 = float(lr) if lr.device.type == "cpu" else float(lr.detach().to("cpu", torch.float32))
    seed, offset = key if key is not None else (next_philox_key(dev) if bf16_sr else (0, 0))
    with nv.on_device(dev):
        nv.check(nv.load().qt_adamw_bf16_sr(
            p.data_ptr(), nv.code(p.dtype), grad.data_ptr(), nv.code(grad.dtype), exp_avg.data_ptr(), exp_avg_sq.data_ptr(),
            p.numel(), lr32, float(beta1), float(beta2), float(weight_decay), float(eps), bc1,
            sqrt_bc2, int(bool(bf16_sr)), seed, offset, nv.stream_ptr(dev)))


def adamw_multi(params: list[Tensor], grads: list[Tensor], step: float | Tensor, exp_avgs: list[Tensor],
                exp_avg_sqs: list[Tensor], lr: Tensor, beta1: float, beta2: float, weight_decay: float, eps: float,
                bf16_sr: bool, *, key: tuple[int, int] | None = None) -> None:
    """`adamw` for a list of parameters that share step count, device and dtypes, in as few launches
    as the kernel's table allows. Tensor t draws the random bits of `adamw(..., key=(seed, offset + t))`."""
    n = len(params)
    if not (len(grads) == len(exp_avgs) == len(exp_avg_sqs) == n):
        raise ValueError("adamw_multi: lists differ in length")
    if n == 0:
        return
    params, grads, exp_avgs, exp_avg_sqs = ([_local(t) for t in ts] for ts in (params, grads, exp_avgs, exp_avg_sqs))
    dev = nv.require_cuda(*params, *grads, *exp_avgs, *exp_avg_sqs)
    p_dtype, g_dtype = params[0].dtype, grads[0].dtype
    for p, g, m, v in zip(params, grads, exp_avgs, exp_avg_sqs):
        if not (p.is_contiguous() and g.is_contiguous() and m.is_contiguous() and v.is_contiguous()):
            raise ValueError("adamw: tensors must be contiguous")
        if m.dtype is not torch.bfloat16 or v.dtype is not torch.bfloat16:
            raise TypeError("adamw: optimizer states are bfloat16")
        if p.dtype is not p_dtype or g.dtype is not g_dtype:
            raise TypeError("adamw_multi: parameters (and gradients) of one call share a dtype")
        if not (g.numel() == m.numel() == v.numel() == p.numel()):
            raise ValueError("adamw: parameter, gradient and states differ in size")
    bc1, sqrt_bc2 = _bias_corrections(float(step), beta1, beta2)
    lr32 = float(lr) if lr.device.type == "cpu" else float(lr.detach().to("cpu", torch.float32))
    seed, offset = key if key is not None else (reserve_philox_keys(dev, n) if bf16_sr else (0, 0))
    ptrs = ctypes.c_void_p * n
    with nv.on_device(dev):
        nv.check(nv.load().qt_adamw_bf16_sr_multi(
            n, ptrs(*[t.data_ptr() for t in params]), ptrs(*[t.data_ptr() for t in grads]),
            ptrs(*[t.data_ptr() for t in exp_avgs]), ptrs(*[t.data_ptr() for t in exp_avg_sqs]),
            (ctypes.c_int64 * n)(*[t.numel() for t in params]), nv.code(p_dtype), nv.code(g_dtype), lr32, float(beta1),
            float(beta2), float(weight_decay), float(eps), bc1, sqrt_bc2, int(bool(bf16_sr)), seed, offset,
            nv.stream_ptr(dev)))
