"""BitNet b1.58 training: ternary weights (tensor-wise abs-mean scale), INT8 activations, INT8
tensor-core forward; 2-bit packed weights for the FSDP2 all-gather (reference: subclasses/bitnet.py).

Names and semantics follow the reference; the abs-mean reduction, the ternarize(+pack) step, the
unpack and the activation quantize are sm_100a kernels, and `scaled_mm` accepts the 0-dim tensor
scale the reference's call site passes.
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F
import torch.utils._pytree as pytree
from torch import Tensor, nn

from gn_kernels import _native as nv
from gn_kernels import scaled_mm

from .int8 import quantize_int8

aten = torch.ops.aten

_REWRAP_OPS = {
    aten.t.default,
    aten.detach.default,
    aten.empty_like.default,
    aten.new_zeros.default,
    aten.slice.Tensor,
    aten.view.default,
    aten.as_strided.default,
    aten._to_copy.default,
    aten._pin_memory.default,
    aten.split.Tensor,
    aten.clone.default,
}


# ---- kernels behind the helper functions --------------------------------------------------------


def get_bitnet_scale(x: Tensor) -> Tensor:
    """Tensor-wise abs-mean, always fp32, 0-dim (reference: bitnet.py:110-112)."""
    dev = nv.require_cuda(x)
    if x.dtype not in (torch.bfloat16, torch.float32):
        x = x.float()
    x = x.contiguous()
    out = torch.empty((), dtype=torch.float32, device=dev)
    if x.numel() == 0:
        return out.fill_(float("nan"))
    workspace = torch.empty(1024, dtype=torch.float64, device=dev)
    with nv.on_device(dev):
        nv.check(nv.load().qt_abs_mean(x.data_ptr(), nv.code(x.dtype), x.numel(), out.data_ptr(), workspace.data_ptr(),
                                       workspace.numel() * 8, nv.stream_ptr(dev)))
    return out


def _ternarize(w: Tensor, scale: Tensor, eps: float, pack: bool) -> Tensor:
    dev = nv.require_cuda(w, scale)
    if w.dtype not in (torch.bfloat16, torch.float32):
        w = w.float()
    w = w.contiguous()
    scale = scale.detach().to(torch.float32).reshape(1).contiguous()
    if pack:
        assert w.ndim == 2 and w.shape[1] % 4 == 0, "2-bit packing needs the last dim to be a multiple of 4"
        out = torch.empty((w.shape[0], w.shape[1] // 4), dtype=torch.int8, device=dev)
    else:
        out = torch.empty(w.shape, dtype=torch.int8, device=dev)
    with nv.on_device(dev):
        nv.check(nv.load().qt_bitnet_quantize_weight(w.data_ptr(), nv.code(w.dtype), w.numel(), scale.data_ptr(), eps,
                                                     out.data_ptr(), int(pack), nv.stream_ptr(dev)))
    return out


def quantize_bitnet_weight(w: Tensor, scale: Tensor, eps: float = 1e-5) -> Tensor:
    """round(w / clip(scale, eps)) clipped to {-1, 0, 1}, int8 (reference: bitnet.py:115-118)."""
    return _ternarize(w, scale, eps, pack=False)


def _pack_i2_in_i8(x: Tensor) -> Tensor:
    """Pack four 2-bit values per byte along the last dim, first value in the top bits
    (reference: bitnet.py:185-195). Bit arithmetic on an already-quantized int8 tensor."""
    x0 = x[:, ::4] << 6
    x1 = (x[:, 1::4] & 0b11) << 4
    x2 = (x[:, 2::4] & 0b11) << 2
    x3 = x[:, 3::4] & 0b11
    return x0 | x1 | x2 | x3


def _unpack_i2_in_i8(x: Tensor) -> Tensor:
    """Inverse of `_pack_i2_in_i8`, sign-extending each field (reference: bitnet.py:198-201)."""
    dev = nv.require_cuda(x)
    x = x.contiguous()
    out = torch.empty((x.shape[0], x.shape[1] * 4), dtype=torch.int8, device=dev)
    with nv.on_device(dev):
        nv.check(nv.load().qt_unpack_i2(x.data_ptr(), x.numel(), out.data_ptr(), nv.stream_ptr(dev)))
    return out


def quantize_and_pack_bitnet_weight(w: Tensor, scale: Tensor, eps: float = 1e-5) -> Tensor:
    """Ternarize and 2-bit pack in one pass over the weight ([N,K] -> int8 [N,K/4])."""
    return _ternarize(w, scale, eps, pack=True)


# ---- the training subclass ----------------------------------------------------------------------


class BitNetTrainingLinearWeight(Tensor):
    """bf16 master weight whose forward uses its ternary quantization (reference: bitnet.py:16-107)."""

    @staticmethod
    @torch._dynamo.disable
    def __new__(cls, data: Tensor):
        return Tensor._make_wrapper_subclass(cls, data.shape, dtype=data.dtype, device=data.device)

    @torch._dynamo.disable
    def __init__(self, data: Tensor):
        self._data = data

    def __tensor_flatten__(self):
        return ["_data"], []

    @classmethod
    def __tensor_unflatten__(cls, tensor_data_dict, tensor_attributes, outer_size=None, outer_stride=None):
        return cls(tensor_data_dict["_data"], *tensor_attributes)

    def __repr__(self):
        return f"{self.__class__.__name__}(data={self._data})"

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or dict()
        if func is F.linear:
            return _BitNetTrainingLinear.apply(*args, **kwargs)
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs):
        kwargs = kwargs or {}
        out = func(
            *pytree.tree_map_only(cls, lambda x: x._data, args),
            **pytree.tree_map_only(cls, lambda x: x._data, kwargs),
        )
        if func is aten.copy_.default:
            return args[0]
        if func in _REWRAP_OPS:
            return pytree.tree_map_only(Tensor, lambda x: cls(x), out)
        return out

    # FSDP2 all-gather extension (reference: bitnet.py:83-107): the abs-mean is averaged over the
    # ranks, each rank ternarizes + packs its own rows, and 2 bits per weight cross NVLink.
    def fsdp_pre_all_gather(self, mesh, outer_size=None, outer_stride=None, module=None, mp_policy=None):
        scale = get_bitnet_scale(self._data)
        dist.all_reduce(scale, op=dist.ReduceOp.AVG, group=mesh.get_group() if hasattr(mesh, "get_group") else None)
        data_i2 = quantize_and_pack_bitnet_weight(self._data, scale)
        return (data_i2,), (scale,)

    def fsdp_post_all_gather(self, all_gather_outputs: Tuple[Tensor, ...], metadata: Any, param_dtype: torch.dtype, *,
                             out: Optional[Tensor] = None):
        (data_i2,) = all_gather_outputs
        (scale,) = metadata
        scale = scale.to(param_dtype)
        if out is not None:
            assert isinstance(out, BitNetPacked2bitLinearWeight)
            out.scale = scale
            return
        return BitNetPacked2bitLinearWeight(data_i2, scale), all_gather_outputs


def _bitnet_backward(ctx, grad_output, weight_i8):
    """Shared backward of both BitNet linears: bf16 matmuls against the ternary weight and the
    de-quantized int8 activation (reference: bitnet.py:146-168, 290-311)."""
    input_i8, row_scale, tensor_scale = ctx.saved_tensors[0], ctx.saved_tensors[1], ctx.saved_tensors[3]
    grad_input = grad_weight = grad_bias = None
    batch_dims = grad_output.shape[:-1]
    gy = grad_output.reshape(-1, weight_i8.shape[0])
    if ctx.needs_input_grad[0]:
        grad_input = (gy @ weight_i8.to(gy.dtype)) * tensor_scale
        grad_input = grad_input.view(*batch_dims, weight_i8.shape[1])
    if ctx.needs_input_grad[1]:
        grad_weight = gy.T @ (input_i8 * row_scale.view(-1, 1))
    if len(ctx.needs_input_grad) > 2 and ctx.needs_input_grad[2]:
        grad_bias = gy.sum(0)
    return grad_input, grad_weight, grad_bias


class _BitNetTrainingLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input: Tensor, weight: BitNetTrainingLinearWeight, bias: Tensor | None = None):
        batch_dims = input.shape[:-1]
        x2d = input.reshape(-1, weight.shape[1])
        input_i8, row_scale = quantize_int8(x2d, eps=1e-5)

        # fp32 scale for the weight quantize, cast to the weight dtype for the matmul and backward
        tensor_scale = get_bitnet_scale(weight._data)
        weight_i8 = quantize_bitnet_weight(weight._data, tensor_scale)
        tensor_scale = tensor_scale.to(weight.dtype)

        ctx.save_for_backward(input_i8, row_scale, weight_i8, tensor_scale)
        out = scaled_mm(input_i8, weight_i8.T, row_scale, tensor_scale)
        out = out.view(*batch_dims, weight.shape[0])
        return out + bias if bias is not None else out

    @staticmethod
    def backward(ctx, grad_output):
        return _bitnet_backward(ctx, grad_output, ctx.saved_tensors[2])


def convert_bitnet(module: nn.Module):
    """Wrap every nn.Linear weight under `module`; RMSNorm insertion is the caller's job
    (reference: bitnet.py:171-182)."""
    if isinstance(module, nn.Linear):
        module.weight = nn.Parameter(
            BitNetTrainingLinearWeight(module.weight.detach()),
            requires_grad=module.weight.requires_grad,
        )
    else:
        for m in module.children():
            convert_bitnet(m)
    return module


class BitNetPacked2bitLinearWeight(Tensor):
    """Gathered BitNet weight: 2-bit packed ternary values [N, K/4] + a 0-dim scale
    (reference: bitnet.py:206-263). A container for the quantized FSDP all-gather."""

    @staticmethod
    @torch._dynamo.disable
    def __new__(cls, int_data: Tensor, scale: Tensor):
        M, N = int_data.shape
        return Tensor._make_wrapper_subclass(cls, (M, N * 4), dtype=scale.dtype, device=scale.device)

    @torch._dynamo.disable
    def __init__(self, int_data: Tensor, scale: Tensor):
        assert int_data.dtype is torch.int8
        assert scale.shape == ()
        self.int_data = int_data
        self.scale = scale

    def __tensor_flatten__(self):
        return ["int_data", "scale"], []

    @classmethod
    def __tensor_unflatten__(cls, tensor_data_dict, tensor_attributes, outer_size=None, outer_stride=None):
        return cls(tensor_data_dict["int_data"], tensor_data_dict["scale"], *tensor_attributes)

    def __repr__(self):
        return f"{self.__class__.__name__}(data={self.dequantize()})"

    def dequantize(self, out_dtype=None):
        out = _unpack_i2_in_i8(self.int_data) * self.scale
        return out.to(out_dtype) if out_dtype is not None else out

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or dict()
        if func is F.linear:
            return _BitNetPacked2bitLinear.apply(*args, **kwargs)
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs):
        kwargs = kwargs or {}
        if func in (aten.detach.default, aten.clone.default):
            w = args[0]
            return cls(func(w.int_data, *args[1:], **kwargs), func(w.scale, *args[1:], **kwargs))
        if func is aten.as_strided.default:
            return cls(args[0].int_data, args[0].scale)
        raise NotImplementedError(f"{cls.__name__} dispatch: attempting to run {func}, this is not supported")


class _BitNetPacked2bitLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input: Tensor, weight: BitNetPacked2bitLinearWeight, bias: Tensor | None = None):
        batch_dims = input.shape[:-1]
        x2d = input.reshape(-1, weight.shape[1])
        input_i8, row_scale = quantize_int8(x2d, eps=1e-5)
        weight_i2, tensor_scale = weight.int_data, weight.scale
        ctx.save_for_backward(input_i8, row_scale, weight_i2, tensor_scale)

        weight_i8 = _unpack_i2_in_i8(weight_i2)
        out = scaled_mm(input_i8, weight_i8.T, row_scale, tensor_scale)
        out = out.view(*batch_dims, weight.shape[0])
        return out + bias if bias is not None else out

    @staticmethod
    def backward(ctx, grad_output):
        return _bitnet_backward(ctx, grad_output, _unpack_i2_in_i8(ctx.saved_tensors[2]))
