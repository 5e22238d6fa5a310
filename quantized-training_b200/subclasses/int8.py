"""INT8 absmax quantization and the INT8 weight-only training subclass.

Public surface mirrors the reference (subclasses/int8.py): `quantize_int8`, `Int8QTConfig`,
`Int8LinearWeight`, `convert_int8_quantized_training`. The quantize step runs on the sm_100a
kernels (one HBM pass, in-kernel Philox for stochastic rounding); there is no CPU path.
"""
from __future__ import annotations

from typing import Literal, NamedTuple

import torch
import torch.nn.functional as F
from torch import Tensor, nn

import gn_kernels
from gn_kernels import scaled_mm

aten = torch.ops.aten


class _QuantCache:
    """Remembers the last few round-to-nearest quantizations so a tensor that feeds several Linear
    layers (the hidden state into q/k/v, or into gate/up) is quantized once, not once per layer.

    An entry is valid only for the very same tensor object state: same storage address, shape, strides
    and version counter. The entry keeps a reference to its source tensor, so the storage cannot be
    freed and handed to another tensor while the entry lives; an in-place write bumps the version.
    Stochastic rounding is never cached (every use must draw fresh noise). Tensors made under
    torch.inference_mode have no version counter and are never cached.

    What the cache pins is bounded three ways: at most SLOTS entries, at most MAX_BYTES of source plus
    quantized bytes (oldest entries go first), and everything is dropped when a backward pass ends (the
    Linear's backward queues `clear` on the autograd engine)."""

    SLOTS = 4
    MAX_BYTES = 1 << 30

    def __init__(self):
        self.entries: list[tuple[tuple, Tensor, tuple, int]] = []
        self._clear_queued = False

    @staticmethod
    def cacheable(t: Tensor) -> bool:
        # plain tensors only: fake / functional tensors (torch.compile's tracing) have no data pointer, and
        # tensors made under inference_mode no version counter
        return type(t) is Tensor and not t.is_inference()

    @staticmethod
    def key(t: Tensor, eps: float):
        return (t.data_ptr(), t._version, tuple(t.shape), tuple(t.stride()), t.dtype, eps)

    def get(self, t: Tensor, eps: float):
        k = self.key(t, eps)
        for kk, _src, out, _n in self.entries:
            if kk == k:
                return out
        return None

    def put(self, t: Tensor, eps: float, out: tuple):
        nbytes = t.numel() * t.element_size() + sum(o.numel() * o.element_size() for o in out)
        if nbytes > self.MAX_BYTES:
            return
        self.entries.append((self.key(t, eps), t, out, nbytes))
        while len(self.entries) > self.SLOTS or sum(e[3] for e in self.entries) > self.MAX_BYTES:
            self.entries.pop(0)

    def clear(self):
        self.entries.clear()
        self._clear_queued = False

    def clear_after_backward(self):
        """Called from inside a backward function: drop every entry once the running backward pass is over."""
        if torch.compiler.is_compiling() or not self.entries:
            return   # nothing to drop (the cache is not used under tracing, where no backward pass is running either)
        if not self._clear_queued:
            try:
                torch.autograd.Variable._execution_engine.queue_callback(self.clear)
                self._clear_queued = True
            except RuntimeError:   # not inside a backward pass (a backward function being traced): drop now
                self.clear()


_quant_cache = _QuantCache()


def _rows_quantize(t2d: Tensor, stochastic_rounding: bool, eps: float, key=None, col_absmax: Tensor | None = None,
                   cache: bool = False):
    """Quantize each ROW of a 2-D tensor; returns contiguous int8 of t2d's shape and scale [rows,1].

    A transposed view (unit stride along dim 0) is served by the transposing column-wise kernel
    on its base, so `quantize_int8(B.T, dim=1)` never materialises `B.T` in bf16. `cache=True` lets
    repeated round-to-nearest requests for the same activation reuse the first result."""
    use_cache = cache and not stochastic_rounding and not torch.compiler.is_compiling() and _QuantCache.cacheable(t2d)
    if use_cache:
        hit = _quant_cache.get(t2d, eps)
        if hit is not None:
            return hit
    if t2d.shape[0] > 1 and t2d.shape[1] > 1 and t2d.stride(0) == 1 and t2d.stride(1) >= t2d.shape[0]:
        out = gn_kernels.quantize_colwise_t(t2d.T, torch.int8, stochastic_rounding, eps=eps, key=key,
                                            col_absmax_=col_absmax)
    else:
        out = gn_kernels.quantize_rowwise(t2d, torch.int8, stochastic_rounding, eps=eps, key=key)
    if use_cache:
        _quant_cache.put(t2d, eps, out)
    return out


@torch.no_grad()
def quantize_int8(tensor: Tensor, stochastic_rounding: bool = False, *, dim: int = -1, eps: float = 1e-12):
    """Symmetric absmax INT8 quantization along `dim` (reference: subclasses/int8.py:12-26).

    scale = amax(|x|, dim) / 127 in fp32; x / clip(scale, eps); round-half-even, or floor(x + u)
    with u ~ U[0,1) when `stochastic_rounding`; clip to [-128, 127]. Returns (int8 tensor shaped
    like `tensor`, scale with `dim` kept as size 1, in `tensor.dtype`).
    """
    if not tensor.is_cuda:
        raise RuntimeError("quantize_int8 runs on the CUDA kernels only; move the tensor to a B200 first")
    if tensor.dtype not in (torch.bfloat16, torch.float32):
        # fp16 and others: quantize from the exact fp32 values, report the scale in the input dtype
        q, s = quantize_int8(tensor.float(), stochastic_rounding, dim=dim, eps=eps)
        return q, s.to(tensor.dtype)
    nd = tensor.ndim
    if nd == 0:
        raise ValueError("quantize_int8 needs at least one dimension")
    dim = dim % nd
    if nd == 1:
        q, s = _rows_quantize(tensor.view(1, -1), stochastic_rounding, eps)
        return q.view(-1), s.view(1)
    if nd > 2:
        if dim != nd - 1:
            raise NotImplementedError("quantize_int8 on >2-D tensors supports the last dim only")
        flat = tensor.reshape(-1, tensor.shape[-1])
        q, s = _rows_quantize(flat, stochastic_rounding, eps)
        return q.view(tensor.shape), s.view(*tensor.shape[:-1], 1)
    if dim == 1:
        return _rows_quantize(tensor, stochastic_rounding, eps)
    # dim == 0: per-column scales; quantize the rows of the transpose and view the result back
    qt, st = _rows_quantize(tensor.T, stochastic_rounding, eps)
    return qt.T, st.T


class Int8QTConfig(NamedTuple):
    activation: Literal["none", "int8", "int8_sr"] = "none"


class Int8LinearWeight(Tensor):
    """Weight held as int8 rows + one scale per output row (reference: subclasses/int8.py:33-135).

    Behaves as a tensor of the scale's dtype; `F.linear` on it runs `_Int8Linear`; optimizer
    updates (`add_`, `addcdiv_`, `copy_`) de-quantize, apply, and re-quantize with stochastic rounding.
    """

    @staticmethod
    @torch._dynamo.disable
    def __new__(cls, int_data: Tensor, scale: Tensor, config: Int8QTConfig):
        return Tensor._make_wrapper_subclass(cls, int_data.shape, dtype=scale.dtype, device=int_data.device)

    @torch._dynamo.disable
    def __init__(self, int_data: Tensor, scale: Tensor, config: Int8QTConfig):
        assert int_data.dtype is torch.int8
        assert int_data.ndim == 2
        assert scale.ndim == 2
        self.int_data = int_data
        self.scale = scale
        self.config = config

    def __tensor_flatten__(self):
        return ["int_data", "scale"], [self.config]

    @classmethod
    def __tensor_unflatten__(cls, tensor_data_dict, tensor_attributes, outer_size=None, outer_stride=None):
        return cls(tensor_data_dict["int_data"], tensor_data_dict["scale"], *tensor_attributes)

    @classmethod
    def from_float(cls, tensor: Tensor, *, config: Int8QTConfig = Int8QTConfig()):
        int_data, scale = quantize_int8(tensor.detach())
        out = cls(int_data, scale, config)
        out.requires_grad_(tensor.requires_grad)
        return out

    def dequantize(self):
        return self.int_data * self.scale.view(-1, 1)

    def __repr__(self):
        return (
            f"{self.__class__.__name__}(shape={tuple(self.shape)}, config={self.config}, "
            f"dtype={self.dtype}, device={self.device}, requires_grad={self.requires_grad})"
        )

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or dict()
        if func is F.linear:
            return _Int8Linear.apply(*args, **kwargs)
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)

    @classmethod
    def __torch_dispatch__(cls, func, types, args, kwargs):
        kwargs = kwargs or {}
        if func in (aten.detach.default, aten.clone.default):
            w = args[0]
            return cls(func(w.int_data, *args[1:], **kwargs), func(w.scale, *args[1:], **kwargs), w.config)

        if func is aten._to_copy.default:
            w = args[0]
            device, dtype = kwargs.get("device", None), kwargs.get("dtype", None)
            return cls(w.int_data.to(device=device), w.scale.to(device=device, dtype=dtype), w.config)

        # optimizers build their state with zeros_like: hand them a plain tensor
        if func is aten.zeros_like.default:
            w = args[0]
            return torch.zeros(w.shape, dtype=kwargs.get("dtype", w.dtype), device=kwargs.get("device", w.device))

        if func in (aten.sub.Tensor, aten.mul.Tensor):
            plain = [a.dequantize() if isinstance(a, cls) else a for a in args]
            return func(*plain, **kwargs)

        if func is aten.copy_.default:
            dst, src = args[0], args[1]
            if isinstance(dst, cls) and isinstance(src, cls):
                dst.int_data.copy_(src.int_data)
                dst.scale.copy_(src.scale)
            elif isinstance(dst, cls):
                # weight update lands here: re-quantize with stochastic rounding (int8.py:119-122)
                int_data, scale = quantize_int8(src, stochastic_rounding=True)
                dst.int_data.copy_(int_data)
                dst.scale.copy_(scale)
            else:
                dst.copy_(src.dequantize())
            return dst

        # in-place optimizer arithmetic: de-quantize, apply, re-quantize with stochastic rounding
        # (int8.py:124-133) -- one fused kernel when the operands are plain bf16 tensors of the
        # weight's shape, else the three steps through copy_
        if func in (aten.addcdiv_.default, aten.add_.Tensor):
            dst = args[0]
            if isinstance(dst, cls) and not torch.compiler.is_compiling():
                if func is aten.add_.Tensor:
                    operands, value = args[1:2], kwargs.get("alpha", 1)
                else:
                    operands, value = args[1:3], kwargs.get("value", 1)
                if (len(args) == 1 + len(operands) and isinstance(value, (int, float))
                        and gn_kernels.int8_weight_update_supported(dst.int_data, dst.scale, *operands)):
                    gn_kernels.int8_weight_update_(dst.int_data, dst.scale, operands[0],
                                                   operands[1] if len(operands) > 1 else None, value)
                    return dst
            return dst.copy_(func(dst.dequantize(), *args[1:], **kwargs))

        # decoupled weight decay of stock optimizers (param.mul_(1 - lr * wd)): the same three steps. The
        # reference's dispatch has no entry for it, which leaves the weights undecayed there.
        if func in (aten.mul_.Tensor, aten.mul_.Scalar):
            dst = args[0]
            return dst.copy_(dst.dequantize() * args[1])

        raise NotImplementedError(f"{cls.__name__} dispatch: attempting to run {func}, this is not supported")


class _Int8Linear(torch.autograd.Function):
    """F.linear for Int8LinearWeight (reference: subclasses/int8.py:138-180)."""

    @staticmethod
    def forward(ctx, input: Tensor, weight: Int8LinearWeight, bias: Tensor | None = None):
        ctx.save_for_backward(input, weight)
        ctx.bias = bias is not None

        if weight.config.activation == "none":
            # weight-only: bf16 GEMM on the up-cast int8 weight, then the per-output-row scale -- as one
            # tcgen05 GEMM whose epilogue applies the scale (both bf16 roundings kept) where the shapes allow
            x2d = input.reshape(-1, weight.shape[1])
            w_bf16 = weight.int_data.to(input.dtype)            # exact: every int8 value is a bf16 value
            scale = weight.scale.reshape(-1)
            if gn_kernels.bf16_mm_colscale_supported(x2d, w_bf16, scale):
                out = gn_kernels.bf16_mm_colscale(x2d, w_bf16, scale).view(*input.shape[:-1], weight.shape[0])
            else:
                out = (input @ w_bf16.T) * weight.scale.T
        else:
            # dynamic activation quantization + INT8 tensor cores
            batch_dims = input.shape[:-1]
            x2d = input.reshape(-1, weight.shape[1])
            x_i8, x_scale = quantize_int8(x2d, weight.config.activation == "int8_sr")
            out = scaled_mm(x_i8, weight.int_data.T, x_scale, weight.scale.T.contiguous())
            out = out.view(*batch_dims, -1)

        return out + bias if bias is not None else out

    @staticmethod
    def backward(ctx, grad_output):
        input, weight = ctx.saved_tensors
        grad_input = (grad_output * weight.scale.T) @ weight.int_data.to(grad_output.dtype)
        grad_output = grad_output.reshape(-1, weight.shape[0])
        input = input.reshape(-1, weight.shape[1])
        grad_weight = grad_output.T @ input
        grad_bias = grad_output.sum(0) if ctx.bias else None
        return grad_input, grad_weight, grad_bias


def convert_int8_quantized_training(module: nn.Module, *, config: Int8QTConfig = Int8QTConfig()):
    """Swap every nn.Linear weight under `module` for an Int8LinearWeight (int8.py:183-192)."""
    if isinstance(module, nn.Linear):
        module.weight = nn.Parameter(
            Int8LinearWeight.from_float(module.weight, config=config),
            requires_grad=module.weight.requires_grad,
        )
    else:
        for m in module.children():
            convert_int8_quantized_training(m, config=config)
    return module
